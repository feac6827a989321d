"""The allocation-free product entry point against the regular one (collected last on purpose).

Some hosts of this library cannot call into the CUDA allocator when they need a product (memory
budget frozen after start-up, allocator locks held by the calling thread, allocation forbidden
by the embedding application). fb200_q_mat_mul_noalloc serves them from a fixed scratch array
inside the library. Here it is driven through the C ABI twice in a row per case, with different
inputs, and compared with fb200_q_mat_mul at the tolerance the other product tests use (2e-3
relative L2). For 2..32 rows both entry points run the same fp16 kernel and agree far more
closely; a single row goes to the integer-limb kernel in fb200_q_mat_mul but to the fp16 kernel
here, so that case really compares two kernels. Between the two calls a product of another
shape and row bucket runs through the same shared array, so the second call starts from stale
contents it must overwrite. The documented refusals are checked last.
"""
import numpy as np
import pytest

import fixtures as F
import kalosm_b200 as kb
from gpu_util import TYPES, activations, dev, weights  # noqa: F401
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("m", [1, 7, 16, 32])
def test_noalloc_matches_regular_entry_point_twice(dev, tname, m):
    ty = TYPES[tname]
    n, k = 176, 2048
    raw = weights(41, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    out = dev.empty((m, n))  # allocated before the calls under test
    # another shape (larger K, another row bucket) that shares the scratch array between the calls
    m2 = 20 if m <= 16 else 5
    n2, k2 = 48, 4096
    raw2 = weights(43, n2, k2, ty)
    w2 = kb.QMatrix.from_raw_bytes(dev, (n2, k2), raw2, ty)
    x2 = activations(7 + m, m2, k2)
    out2 = dev.empty((m2, n2))
    for call in range(2):
        x = activations(100 * call + m, m, k)
        xt = dev.tensor(x)
        ref = xt.q_mat_mul(w).as_slice()
        out.fill_bytes(0xCD)  # poison: every output must be written by the call
        got = xt.q_mat_mul_noalloc(w, out).as_slice()
        assert got.shape == (m, n)
        assert np.all(np.isfinite(got))
        assert F.rel_l2(got, ref) < TOL, (tname, m, call, F.rel_l2(got, ref))
        assert F.rel_l2(got, O.q_mat_mul(x, raw, ty, n, k)) < TOL
        if call == 0:
            got2 = dev.tensor(x2).q_mat_mul_noalloc(w2, out2).as_slice()
            assert F.rel_l2(got2, O.q_mat_mul(x2, raw2, ty, n2, k2)) < TOL
    assert dev.status() == 0


def test_noalloc_rejects_what_does_not_fit(dev):
    ty = O.Q4K
    w = kb.QMatrix.from_raw_bytes(dev, (16, 256), weights(1, 16, 256, ty), ty)
    out = dev.empty((33, 16))
    with pytest.raises(kb.FusorError) as e:  # more than 32 rows
        dev.tensor(np.zeros((33, 256), np.float32)).q_mat_mul_noalloc(w, out)
    assert e.value.code == kb.ERR_CAPACITY and "32" in str(e.value)
    # K so large that 32 packed rows exceed the 4 MiB array (136 bytes per element of K)
    big_k = 32768
    wb = kb.QMatrix.from_raw_bytes(dev, (16, big_k), weights(2, 16, big_k, ty), ty)
    with pytest.raises(kb.FusorError) as e:
        dev.tensor(np.zeros((32, big_k), np.float32)).q_mat_mul_noalloc(wb, dev.empty((32, 16)))
    assert e.value.code == kb.ERR_CAPACITY and "scratch" in str(e.value)
    # ... while 8 rows of the same K fit (34 bytes per element)
    x = activations(3, 8, big_k)
    got = dev.tensor(x).q_mat_mul_noalloc(wb, dev.empty((8, 16))).as_slice()
    assert F.rel_l2(got, dev.tensor(x).q_mat_mul(wb).as_slice()) < TOL
    dense = kb.QMatrix.from_raw_bytes(dev, (2, 4), np.arange(8, dtype=np.float32), kb.F32)
    with pytest.raises(kb.FusorError) as e:  # dense weights are outside this entry point
        dev.tensor(np.ones((1, 4), np.float32)).q_mat_mul_noalloc(dense, dev.empty((1, 2)))
    assert e.value.code == kb.ERR_UNSUPPORTED_DTYPE
