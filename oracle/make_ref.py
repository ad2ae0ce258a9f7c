"""Place an UNMODIFIED copy of the reference's Python package under ``oracle/_ref/``.

    python oracle/make_ref.py /path/to/transformer_nuggets-checkout

TEST INFRASTRUCTURE ONLY.  The reference (drisspg/transformer_nuggets) is pure Python, so there is
nothing to compile: "building" it means making its package importable where the checkout itself is
absent (the machine the GPU benchmark runs on).  ``oracle/_ref/`` is ignored by git - the copy never
enters this repository's history - but it travels with the working tree like the built
``libtnq.so``.  Only ``transformer_nuggets/**/*.py`` and the reference's two test files for this path
(``test/test_fp8.py``, ``test/test_mx.py``) are copied; nothing is edited.  The benchmark's reference arm
and CPU-baseline leg import the package through ``oracle/reference.py``; ``tests/test_gpu_reference_suite.py``
runs the two test files against this repository's package; no file of the shipped package touches any of it.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make_ref(ref_root: str) -> str:
    src = os.path.join(ref_root, "transformer_nuggets")
    if not os.path.isfile(os.path.join(src, "fp8", "scaled_quant.py")):
        raise FileNotFoundError(f"{ref_root} does not look like a transformer_nuggets checkout")
    dst = os.path.join(DEST, "transformer_nuggets")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    digest = hashlib.sha256()
    count = 0
    for folder, _dirs, files in sorted(os.walk(src)):
        for name in sorted(files):
            if not name.endswith(".py"):
                continue
            a = os.path.join(folder, name)
            b = os.path.join(dst, os.path.relpath(a, src))
            os.makedirs(os.path.dirname(b), exist_ok=True)
            shutil.copyfile(a, b)
            with open(a, "rb") as f:
                digest.update(os.path.relpath(a, src).encode() + b"\0" + f.read())
            count += 1
    tests_dst = os.path.join(DEST, "test")
    if os.path.isdir(tests_dst):
        shutil.rmtree(tests_dst)
    for name in ("test_fp8.py", "test_mx.py"):  # the reference's own tests of the cast path, unmodified
        a = os.path.join(ref_root, "test", name)
        if os.path.isfile(a):
            os.makedirs(tests_dst, exist_ok=True)
            shutil.copyfile(a, os.path.join(tests_dst, name))
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as f:
        f.write(f"unmodified copy of {count} .py files of the reference package transformer_nuggets\n"
                f"sha256 over (relative path, contents) in sorted order: {digest.hexdigest()}\n")
    return dst


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_ref.py /path/to/transformer_nuggets-checkout")
    print(make_ref(sys.argv[1]))
