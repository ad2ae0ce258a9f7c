"""Import the UNMODIFIED reference package from ``oracle/_ref/`` (put there by ``oracle/make_ref.py``).

TEST INFRASTRUCTURE ONLY: used by the benchmark's reference arm, its CPU-baseline leg and its
same-machine comparator runs, so that what is timed beside this library is the reference's own
code (``kind: "reference"``) rather than a restatement of it.  Nothing in the shipped package
imports this module.
"""

from __future__ import annotations

import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "transformer_nuggets", "fp8", "scaled_quant.py"))


def load(submodule: str):
    """``importlib.import_module("transformer_nuggets." + submodule)`` from the copy under
    ``oracle/_ref``.  Raises ``ImportError`` (with the reason) if the copy is absent or one of the
    reference's own dependencies is missing."""
    if not available():
        raise ImportError("oracle/_ref/transformer_nuggets is absent: run `python oracle/make_ref.py <checkout>`")
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    sys.dont_write_bytecode = True
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    mod = importlib.import_module("transformer_nuggets." + submodule)
    origin = os.path.abspath(getattr(mod, "__file__", ""))
    if not origin.startswith(REF_DIR):
        raise ImportError(f"transformer_nuggets resolved to {origin}, not to the copy under oracle/_ref")
    return mod
