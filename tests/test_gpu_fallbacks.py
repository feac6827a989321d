"""GPU parity of the kernels that only an environment variable selects.

Each variable is read once per process by the library, so every alternative runs in a child process
(tests/fallback_worker.py) that checks its cases against the oracle.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fallback_worker.py")


@pytest.mark.parametrize("what,var,value", [
    ("streamed", "FB200_GEMM16_STREAMED", "1"),
    ("exact_small", "FB200_EXACT_SMALL_BATCH", "1"),
    ("decode_scalar", "FB200_ATTN_DECODE_TC", "0"),
    ("prefill_mma", "FB200_ATTN_TCGEN05", "0"),
    ("prefill_sequential", "FB200_TC_GROUP", "0"),
    ("q5k_row_copies", "FB200_Q5K_TENSOR_TMA", "0"),
])
def test_alternative_kernel(what, var, value):
    out = subprocess.run([sys.executable, WORKER, what], env=dict(os.environ, **{var: value}),
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert f"done {what}" in out.stdout
