"""The reference's own tests of the cast path (test/test_fp8.py, test/test_mx.py), unmodified, run against this
repository's package: a child pytest process loads them from the copy that ``oracle/make_ref.py`` places under
``oracle/_ref/test`` with the import name ``transformer_nuggets`` pointed at ``transformer_nuggets_b200``."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TESTS = os.path.join(ROOT, "oracle", "_ref", "test")


@pytest.mark.parametrize("name,n_tests", [("test_fp8.py", 6), ("test_mx.py", 5)])
def test_reference_test_file_passes_against_this_package(name, n_tests):
    path = os.path.join(REF_TESTS, name)
    if not os.path.isfile(path):
        pytest.skip("no copy of the reference's tests under oracle/_ref/test (run oracle/make_ref.py)")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, os.path.join(ROOT, "tests"), os.environ.get("PYTHONPATH", "")]),
               PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run([sys.executable, "-m", "pytest", path, "-q", "-p", "repoint_plugin", "-p", "no:cacheprovider",
                        "--rootdir", REF_TESTS, "-c", os.devnull],
                       capture_output=True, text=True, env=env, cwd=REF_TESTS, timeout=600)
    tail = (r.stdout + r.stderr)[-1500:]
    assert r.returncode == 0, tail
    assert f"{n_tests} passed" in r.stdout and " failed" not in r.stdout and " skipped" not in r.stdout, tail
