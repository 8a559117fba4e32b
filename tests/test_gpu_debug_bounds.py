"""The debug-bounds build of the extension (``rl_engine._C_dbg``, ``-DRLK_DEBUG_BOUNDS=1``) on a GPU: valid small
workloads leave the error word clean, an out-of-range caller index is reported and its access skipped.  The cases run in
a child process because the build is chosen at import time (``RLK_DEBUG_BOUNDS=1``)."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_debug_bounds_build_checks_caller_indices():
    env = dict(os.environ, RLK_DEBUG_BOUNDS="1", PYTHONPATH=ROOT)
    done = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "debug_bounds_cases.py")], env=env, text=True,
                          capture_output=True, timeout=600, check=False)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "DEBUG-BOUNDS OK" in done.stdout
