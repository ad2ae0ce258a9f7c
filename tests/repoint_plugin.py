"""pytest plugin for running the reference's own test files against this repository's package: every
``transformer_nuggets...`` module name the tests import resolves to the ``transformer_nuggets_b200`` module of the
same path.  Loaded with ``-p repoint_plugin`` by tests/test_gpu_reference_suite.py in a child process."""

import importlib
import sys


def pytest_configure(config):
    config.addinivalue_line("markers", "slow: the reference marks its GPU tests slow")
    for name in ("", ".fp8", ".fp8.scaled_quant", ".mx", ".mx.to_blocked"):
        sys.modules["transformer_nuggets" + name] = importlib.import_module("transformer_nuggets_b200" + name)
