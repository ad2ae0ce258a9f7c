"""NVLink peer-store amax exchange for the row-sharded cast.

One fp32 per rank has to cross GPUs between the amax pass and the cast pass, so
latency is everything and bandwidth nothing: instead of a collective launch, the
amax kernel's last CTA stores (sequence number, amax) as one 8-byte word into
every peer's slot buffer, and the cast kernel reads its own buffer.  Set-up maps
the peers' buffers through CUDA IPC once per process group.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _lib

MAX_RANKS = 16


class PeerAmaxExchange:
    """Slot buffers of all ranks of ``group`` mapped into this process.

    Collective constructor: every rank of the group must create it at the same
    point.  The current CUDA device must be this rank's GPU, all ranks must be on
    one node with peer access between their GPUs.
    """

    def __init__(self, group=None):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("torch.distributed must be initialised")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks")
        self.seq = 0
        self._local = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        _lib.call("tnq_exchange_create", ctypes.byref(self._local), handle)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._ptrs = (ctypes.c_void_p * self.world)()
        self._opened = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self._ptrs[r] = self._local.value
            else:
                p = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                _lib.call("tnq_exchange_open", buf, ctypes.byref(p))
                self._ptrs[r] = p.value
                self._opened.append(p.value)
        self._amax = torch.empty(1, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        dist.barrier(group=group)

    def run(self, local_rows, n, in_dt, out_dt, ws, stream, out) -> torch.Tensor:
        """Enqueue amax + publish + wait + cast for one call; returns the device
        tensor that will hold the global amax."""
        self.seq = self.seq % 0xFFFFFFFF + 1
        _lib.call(
            "tnq_fp8_sharded_cast", local_rows.data_ptr(), out.data_ptr(), n, in_dt, out_dt, ws.data_ptr(),
            self._ptrs, self.world, self.rank, self.seq, self._amax.data_ptr(), stream,
        )
        return self._amax

    def global_amax(self, local_rows: torch.Tensor) -> torch.Tensor:
        """Enqueue: amax of this rank's rows, exchange, MAX over ranks.  Returns a new
        one-element fp32 device tensor that will hold the tensor-wide amax."""
        _lib.require_cuda(local_rows, "local_rows")
        if local_rows.dtype not in _lib.IN_DTYPES or not local_rows.is_contiguous():
            raise TypeError("local_rows must be a contiguous bfloat16 / float32 tensor")
        dev = local_rows.device
        out = torch.empty(1, dtype=torch.float32, device=dev)
        self.seq = self.seq % 0xFFFFFFFF + 1
        with torch.cuda.device(dev):
            _lib.call(
                "tnq_sharded_amax", local_rows.data_ptr(), local_rows.numel(), _lib.IN_DTYPES[local_rows.dtype],
                _lib.workspace(dev).data_ptr(), self._ptrs, self.world, self.rank, self.seq, out.data_ptr(),
                _lib.stream_ptr(dev),
            )
        return out

    def status(self) -> int:
        """0, or TNQ_ETIMEOUT if a cast kernel gave up waiting for a peer (synchronises)."""
        v = ctypes.c_uint32(0)
        _lib.call("tnq_exchange_status", self._local, ctypes.byref(v))
        return int(v.value)

    def close(self):
        if self._local.value is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody may still be storing into a buffer that goes away
        for p in self._opened:
            _lib.call("tnq_exchange_close", ctypes.c_void_p(p))
        self._opened = []
        _lib.call("tnq_exchange_destroy", self._local)
        self._local = ctypes.c_void_p()
