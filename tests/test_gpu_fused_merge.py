"""GPU: the opt-in merge inside the decode kernels (RK_DECODE_FUSED_MERGE=1 is read once per process, so the decode
parity tests run again in a child process with it set)."""
import os
import pathlib
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_decode_parity_with_the_merge_inside_the_kernel():
    root = pathlib.Path(__file__).resolve().parent.parent
    env = dict(os.environ, RK_DECODE_FUSED_MERGE="1")
    done = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_decode.py", "tests/test_gpu_seqsplit.py", "-x", "-q", "-m", "gpu",
                           "-p", "no:cacheprovider"], cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]
