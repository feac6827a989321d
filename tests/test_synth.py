"""The torch encoders of kalosm_b200.synth emit valid GGUF blocks (checked with the oracle's decoder)."""
import numpy as np
import pytest
import torch

import fixtures as F
from kalosm_b200 import synth
from oracle import oracle as O


@pytest.mark.parametrize("ty,tol", [(O.Q4_0, 0.15), (O.Q8_0, 0.01), (O.Q4K, 0.12), (O.Q6K, 0.04)])
def test_blocks_decode_back(ty, tol):
    n, k = 24, 1024
    raw = synth.random_qweights(5, 0.02, n, k, ty).numpy()
    assert raw.size == O.nbytes_for(ty, n * k)
    back = O.dequantize(raw, ty, n * k)
    gen = torch.Generator().manual_seed(5)
    ref = (torch.randn(n, k, generator=gen) * 0.02).numpy().ravel()
    assert np.all(np.isfinite(back))
    assert F.rel_l2(back, ref) < tol
    assert abs(float(np.std(back)) - 0.02) < 0.004
    again = synth.random_qweights(5, 0.02, n, k, ty).numpy()
    assert np.array_equal(raw, again)


@pytest.mark.parametrize("ty,tol", [(O.Q5_0, 0.06), (O.Q5K, 0.06)])
def test_five_bit_encoders_decode_back(ty, tol):
    # the tests' own Q5_0 / Q5_K encoders (fixtures.quantize_q5_0 / quantize_q5k): right byte count,
    # decoded by the oracle to within 5-bit rounding of the values they were given, every bit field used
    n, k = 24, 1024
    w = O.normal(7, 0.02, n * k)
    raw = F.random_q5_weights(7, 0.02, n, k, ty)
    assert raw.dtype == np.uint8 and raw.size == O.nbytes_for(ty, n * k)
    back = O.dequantize(raw, ty, n * k)
    assert np.all(np.isfinite(back))
    assert F.rel_l2(back, w) < tol
    bs, bb = O.BLOCK[ty]
    blocks = raw.reshape(-1, bb)
    qh = blocks[:, 2:6] if ty == O.Q5_0 else blocks[:, 16:48]
    assert 0.3 < np.unpackbits(qh).mean() < 0.7  # the fifth bits are in use
    assert np.array_equal(raw, F.random_q5_weights(7, 0.02, n, k, ty))
