"""GPU parity: dequantisation (bit-exact) and q_mat_mul (<= 2e-3 relative L2) against the oracle.

Every test calls the CUDA path through the C ABI (kalosm_b200 is a ctypes binding) on the same
bytes the oracle sees. Tolerance for products: 2e-3 relative L2 of the fp32 oracle.
"""
import numpy as np
import pytest

import fixtures as F
import kalosm_b200 as kb
from gpu_util import TYPES, activations, dev, weights  # noqa: F401
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _b(*parts):
    return np.frombuffer(b"".join(parts), dtype=np.uint8)


X32 = np.arange(1, 33, dtype=np.float32)[None, :]


def test_known_answers(dev):
    # fusor-ml/core/src/quantized/matmul/tests.rs:1305-1423
    cases = [
        (O.Q4_0, _b(F.f16_bytes(1.0), bytes([0x99]) * 16, F.f16_bytes(1.0), bytes([0x77]) * 16)),
        (O.Q5_0, _b(F.f16_bytes(1.0), bytes([0xFF] * 4), bytes([0x11]) * 16,
                    F.f16_bytes(1.0), bytes(4), bytes([0xFF]) * 16)),
        (O.Q8_0, _b(F.f16_bytes(1.0), bytes([1]) * 32, F.f16_bytes(1.0), bytes([0xFF]) * 32)),
    ]
    for ty, raw in cases:
        w = kb.QMatrix.from_raw_bytes(dev, (2, 32), raw, ty)
        y = dev.tensor(X32).q_mat_mul(w).as_slice()
        assert y.shape == (1, 2)
        assert abs(y[0, 0] - 528.0) < 1e-3 and abs(y[0, 1] + 528.0) < 1e-3, (ty, y)
    raw = _b(F.f16_bytes(1.0), F.f16_bytes(0.0), bytes([1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]),
             bytes(32), bytes([0x11]) * 128)
    w = kb.QMatrix.from_raw_bytes(dev, (1, 256), raw, O.Q5K)
    y = dev.tensor(np.arange(1, 257, dtype=np.float32)[None, :]).q_mat_mul(w).as_slice()
    assert abs(y[0, 0] - 32896.0) < 1e-2


@pytest.mark.parametrize("case", F.CONFORMANCE_CASES, ids=lambda c: c[0])
def test_conformance_fixtures(dev, case):
    # dequantize: bit-exact with the oracle; q_mat_mul: the case's absolute tolerance and 2e-3 rel-L2
    name, ty, (n, k), rows, tol, seed = case
    raw = F.GEN[ty]((n, k))
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    assert w.shape == (n, k) and w.ggml_type == ty and w.nbytes == raw.size
    deq = w.dequantize().as_slice()
    ref = O.dequantize(raw, ty, n * k).reshape(n, k)
    assert np.array_equal(deq.view(np.uint32), ref.view(np.uint32)), name
    x = F.uniform_input(rows, k, seed)
    y = dev.tensor(x).q_mat_mul(w).as_slice()
    exp = O.q_mat_mul(x, raw, ty, n, k)
    assert np.max(np.abs(y - exp)) < tol
    assert F.rel_l2(y, exp) < TOL, (name, F.rel_l2(y, exp))


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("shape", [(48, 512), (16, 256), (33, 1024), (4096, 4096)])
def test_dequantize_bit_exact_random(dev, tname, shape):
    ty = TYPES[tname]
    n, k = shape
    raw = weights(11 + n, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    deq = w.dequantize().as_slice()
    ref = O.dequantize(raw, ty, n * k).reshape(n, k)
    assert np.array_equal(deq.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16, 17, 32, 33, 70])
def test_q_mat_mul_batches(dev, tname, m):
    ty = TYPES[tname]
    n, k = 272, 1024
    raw = weights(5, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    x = activations(m, m, k)
    y = dev.tensor(x).q_mat_mul(w).as_slice()
    exp = O.q_mat_mul(x, raw, ty, n, k)
    assert y.shape == (m, n)
    assert F.rel_l2(y, exp) < TOL, F.rel_l2(y, exp)
    # rows are independent: row 0 of a batch agrees with the single-row product of row 0
    # (another kernel: batches go through fp16 weights and activations, 11 bits instead of the 27
    # of the single-row kernel's int8 limbs: compared to a tolerance, not bitwise)
    y0 = dev.tensor(x[:1]).q_mat_mul(w).as_slice()
    assert F.rel_l2(y0[0], y[0]) < (1e-6 if m == 1 else TOL)


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("tile", ["128,1", "256,1", "128,2", "256,2", ""])
def test_prefill_product_tensor_cores(dev, tname, tile, monkeypatch):
    # more than 32 rows: the tcgen05 kernel, every CTA tile shape (activation rows, 128-row weight
    # halves; "" = the cost model's choice), ragged N and M, plain / residual / SwiGLU epilogues
    monkeypatch.setenv("FB200_TC_TILE", tile)
    ty = TYPES[tname]
    f, k = 528, 1024  # 33 row-tiles per part: the last CTA of every tile shape is ragged
    g_raw, u_raw = weights(31, f, k, ty), weights(32, f, k, ty)
    gate = kb.QMatrix.from_raw_bytes(dev, (f, k), g_raw, ty)
    up = kb.QMatrix.from_raw_bytes(dev, (f, k), u_raw, ty)
    gu = kb.QMatrix.concat_rows([gate, up])
    for m in (40, 300):
        x = activations(70 + m, m, k)
        eg, eu = O.q_mat_mul(x, g_raw, ty, f, k), O.q_mat_mul(x, u_raw, ty, f, k)
        both = dev.tensor(x).q_mat_mul(gu).as_slice()
        assert both.shape == (m, 2 * f)
        assert F.rel_l2(both, np.concatenate([eg, eu], axis=1)) < TOL
        h = dev.tensor(x).q_mat_mul(gu, epilogue=kb.EPI_SWIGLU).as_slice()
        assert h.shape == (m, f) and F.rel_l2(h, O.silu_mul(eg, eu)) < TOL
        r1, r2 = activations(80 + m, m, f), activations(90 + m, m, f)
        y = dev.tensor(x).q_mat_mul(gate, epilogue=kb.EPI_RESIDUAL, r1=dev.tensor(r1), r2=dev.tensor(r2)).as_slice()
        assert F.rel_l2(y, (eg + r1) + r2) < TOL
        assert dev.status() == 0
    # repeated launches agree bit for bit (fixed accumulation order in the tensor core)
    xt = dev.tensor(activations(7, 300, k))
    assert np.array_equal(xt.q_mat_mul(gu).as_slice(), xt.q_mat_mul(gu).as_slice())


def _sampled_columns(raw, ty, n, k, cols):
    """Raw GGUF bytes of the rows `cols` of an [n, k] matrix (rows are contiguous block runs)."""
    bs, bb = O.BLOCK[ty]
    row_bytes = k // bs * bb
    return np.concatenate([raw[c * row_bytes:(c + 1) * row_bytes] for c in cols])


@pytest.mark.parametrize("tname,n,k", [("q4_0", 4096, 4096), ("q4k", 4096, 4096), ("q4k", 1024, 4096),
                                        ("q4k", 14336, 4096), ("q4k", 4096, 14336), ("q8_0", 4096, 4096),
                                        ("q8_0", 14336, 4096), ("q8_0", 4096, 14336), ("q6k", 1024, 4096),
                                        ("q6k", 4096, 14336)])
def test_q_mat_mul_llama_shapes(dev, tname, n, k):
    # the projection shapes of a Llama-3-8B layer at every row count of the sweep: one row (integer
    # limb kernel), 8 and 32 rows (fp16 mma kernel), 512 and 2048 rows (tcgen05 kernel). The oracle
    # runs on a sample of output columns (and, for the large row counts, of activation rows: rows
    # are independent) to keep the CPU time bounded.
    ty = TYPES[tname]
    raw = weights(n + k, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    cols = np.sort(np.random.default_rng(1).choice(n, 256, replace=False))
    sub = _sampled_columns(raw, ty, n, k, cols)
    for m in (1, 8, 32, 512, 2048):
        x = activations(m + 3, m, k)
        y = dev.tensor(x).q_mat_mul(w).as_slice()
        assert y.shape == (m, n)
        rows = np.arange(m) if m <= 32 else np.sort(np.random.default_rng(m).choice(m, 16, replace=False))
        exp = O.q_mat_mul(x[rows], sub, ty, len(cols), k)
        err = F.rel_l2(y[np.ix_(rows, cols)], exp)
        assert err < TOL, (tname, n, k, m, err)
    assert dev.status() == 0


def test_q_mat_mul_output_head(dev):
    # the 128256 x 4096 Q6_K output head (the largest matrix of the decoder, 431 MB) stand-alone
    ty, n, k = O.Q6K, 128256, 4096
    raw = weights(99, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    assert w.nbytes == 430940160
    rng = np.random.default_rng(5)
    cols = np.sort(np.concatenate([rng.choice(n, 500, replace=False), [0, 15, 16, n - 17, n - 16, n - 1]]))
    sub = _sampled_columns(raw, ty, n, k, cols)
    for m in (1, 8):
        x = activations(m + 40, m, k)
        y = dev.tensor(x).q_mat_mul(w).as_slice()
        assert y.shape == (m, n) and np.all(np.isfinite(y))
        err = F.rel_l2(y[:, cols], O.q_mat_mul(x, sub, ty, len(cols), k))
        assert err < TOL, (m, err)
    assert dev.status() == 0


def test_repeatable_bitwise(dev):
    # fixed reduction order, no float atomics: repeated launches agree bit for bit
    ty, n, k = O.Q4K, 1024, 2048
    raw = weights(3, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    x = dev.tensor(activations(9, 4, k))
    first = x.q_mat_mul(w).as_slice()
    for _ in range(4):
        assert np.array_equal(first, x.q_mat_mul(w).as_slice())


def test_linearity_property(dev):
    # size-independent property: W(ax + by) ~ a Wx + b Wy
    ty, n, k = O.Q6K, 512, 4096
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), weights(21, n, k, ty), ty)
    x, z = activations(1, 1, k), activations(2, 1, k)
    lhs = dev.tensor(2.0 * x - 0.5 * z).q_mat_mul(w).as_slice()
    rhs = 2.0 * dev.tensor(x).q_mat_mul(w).as_slice() - 0.5 * dev.tensor(z).q_mat_mul(w).as_slice()
    assert F.rel_l2(lhs, rhs) < TOL


def test_activation_range(dev):
    # activations far outside the fp16 range still work (per-row power-of-two scaling)
    ty, n, k = O.Q4K, 64, 512
    raw = weights(8, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    for mag in (1e-9, 1e9):
        x = activations(4, 2, k) * np.float32(mag)
        y = dev.tensor(x).q_mat_mul(w).as_slice()
        assert F.rel_l2(y, O.q_mat_mul(x, raw, ty, n, k)) < TOL


def test_epilogues(dev):
    ty, f, k = O.Q4K, 96, 512
    g_raw, u_raw = weights(1, f, k, ty), weights(2, f, k, ty)
    gate = kb.QMatrix.from_raw_bytes(dev, (f, k), g_raw, ty)
    up = kb.QMatrix.from_raw_bytes(dev, (f, k), u_raw, ty)
    gu = kb.QMatrix.concat_rows([gate, up])
    assert gu is not None and gu.shape == (2 * f, k)
    for m in (1, 6, 20):
        x = activations(m, m, k)
        h = dev.tensor(x).q_mat_mul(gu, epilogue=kb.EPI_SWIGLU).as_slice()
        exp = O.silu_mul(O.q_mat_mul(x, g_raw, ty, f, k), O.q_mat_mul(x, u_raw, ty, f, k))
        assert h.shape == (m, f) and F.rel_l2(h, exp) < TOL
        # concatenated matrix without epilogue = both products side by side
        both = dev.tensor(x).q_mat_mul(gu).as_slice()
        assert F.rel_l2(both[:, :f], O.q_mat_mul(x, g_raw, ty, f, k)) < TOL
        r1, r2 = activations(50 + m, m, f), activations(60 + m, m, f)
        y = dev.tensor(x).q_mat_mul(gate, epilogue=kb.EPI_RESIDUAL, r1=dev.tensor(r1),
                                    r2=dev.tensor(r2)).as_slice()
        assert F.rel_l2(y, (O.q_mat_mul(x, g_raw, ty, f, k) + r1) + r2) < TOL
    # Linear with a bias (fusor-ml/fusor/src/layers/linear.rs:93-121): one [N] row added to every output row,
    # through the single-row, the small-batch and the tensor-core kernels
    bias = activations(77, 1, f)[0]
    for m in (1, 6, 20, 40, 300):
        x = activations(200 + m, m, k)
        y = dev.tensor(x).q_mat_mul(gate, epilogue=kb.EPI_BIAS, r1=dev.tensor(bias)).as_slice()
        assert y.shape == (m, f)
        assert F.rel_l2(y, O.q_mat_mul(x, g_raw, ty, f, k) + bias[None, :]) < TOL, m
    # mismatched parts: None, as QMatrix::concat_rows does
    other = kb.QMatrix.from_raw_bytes(dev, (f, k), weights(3, f, k, O.Q6K), O.Q6K)
    assert kb.QMatrix.concat_rows([gate, other]) is None


def test_host_buffer_entry_point(dev):
    ty, n, k = O.Q8_0, 128, 256
    raw = weights(4, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    x = activations(2, 3, k)
    assert F.rel_l2(w.q_mat_mul_host(x), O.q_mat_mul(x, raw, ty, n, k)) < TOL


def test_error_paths(dev):
    with pytest.raises(kb.FusorError) as e:  # K not a multiple of the block size
        kb.QMatrix.from_raw_bytes(dev, (2, 48), np.zeros(54, np.uint8), O.Q4_0)
    assert e.value.code == kb.ERR_INVALID_SHAPE
    with pytest.raises(kb.FusorError) as e:  # unknown ggml type
        kb.QMatrix.from_raw_bytes(dev, (2, 32), np.zeros(36, np.uint8), 99)
    assert e.value.code == kb.ERR_UNSUPPORTED_DTYPE
    with pytest.raises(kb.FusorError) as e:  # wrong byte count
        kb.QMatrix.from_raw_bytes(dev, (2, 32), np.zeros(35, np.uint8), O.Q4_0)
    assert e.value.code == kb.ERR_INVALID_SHAPE
    w = kb.QMatrix.from_raw_bytes(dev, (2, 32), np.zeros(36, np.uint8), O.Q4_0)
    with pytest.raises(kb.FusorError):  # inner dimensions differ
        dev.tensor(np.zeros((1, 64), np.float32)).q_mat_mul(w)
    # empty and dense inputs
    dense = kb.QMatrix.from_raw_bytes(dev, (2, 4), np.arange(8, dtype=np.float32), kb.F32)
    y = dev.tensor(np.ones((1, 4), np.float32)).q_mat_mul(dense).as_slice()
    assert np.allclose(y, [[6.0, 22.0]])
    h16 = kb.QMatrix.from_raw_bytes(dev, (2, 4), np.arange(8, dtype=np.float16), kb.F16)
    assert np.allclose(h16.dequantize().as_slice(), np.arange(8).reshape(2, 4))


@pytest.mark.parametrize("tname", list(TYPES))
def test_rms_norm_fused_into_product(dev, tname):
    # rms_norm_fused / rms_norm_residual_fused followed by q_mat_mul, one row (fused prologue) and
    # several rows (norm kernel + product)
    ty = TYPES[tname]
    n, k = 160, 1024
    raw = weights(31, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    nw = (1.0 + 0.02 * activations(70, 1, k)[0]).astype(np.float32)
    for m in (1, 5):
        x, r = activations(71 + m, m, k), activations(72 + m, m, k)
        for res in (None, r):
            y = dev.tensor(x).rms_norm_q_mat_mul(dev.tensor(nw), 1e-5, w,
                                                 residual=None if res is None else dev.tensor(res)).as_slice()
            exp = O.q_mat_mul(O.rms_norm(x, nw, 1e-5, residual=res), raw, ty, n, k)
            assert F.rel_l2(y, exp) < TOL, (tname, m, F.rel_l2(y, exp))


def test_single_row_large_k_and_tail_tiles(dev):
    # K large enough for the one-CTA-per-SM configuration; N not a multiple of 16
    for ty, n, k in [(O.Q6K, 40, 14336), (O.Q4K, 1000, 16384), (O.Q4_0, 17, 8192), (O.Q8_0, 250, 2048)]:
        raw = weights(n, n, k, ty)
        w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
        x = activations(k % 97, 1, k)
        y = dev.tensor(x).q_mat_mul(w).as_slice()
        assert F.rel_l2(y, O.q_mat_mul(x, raw, ty, n, k)) < TOL
    assert dev.status() == 0


Q5_TYPES = {"q5_0": O.Q5_0, "q5k": O.Q5K}


@pytest.mark.parametrize("tname", list(Q5_TYPES))
@pytest.mark.parametrize("m", [1, 2, 5, 8, 9, 16, 17, 32, 33, 70])
def test_q5_products(dev, tname, m):
    # Q5_K stays in GGUF byte order and takes a kernel of its own; Q5_0 is widened to Q8_0 tiles
    # when the matrix is built (BlockQ5_0 / BlockQ5K, fusor-ml/gguf/src/lib.rs:1046-1073, 1819-1861).
    # Every row bucket (1, 2..8 / 16 / 32 packed rows, more than 32), N not a multiple of 16, K a
    # multiple of the block size only; dequantize stays bit-exact and the type reported is the file's
    ty = Q5_TYPES[tname]
    n, k = 273, 1024 if ty == O.Q5K else 1056
    raw = F.random_q5_weights(17, 0.02, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    assert w.ggml_type == ty and w.nbytes == raw.size
    assert np.array_equal(w.dequantize().as_slice().view(np.uint32),
                          O.dequantize(raw, ty, n * k).reshape(n, k).view(np.uint32))
    x = activations(200 + m, m, k) + np.float32(0.75)  # a mean far from zero: the offsets of Q5_K matter
    y = dev.tensor(x).q_mat_mul(w).as_slice()
    exp = O.q_mat_mul(x, raw, ty, n, k)
    assert y.shape == (m, n)
    assert F.rel_l2(y, exp) < TOL, F.rel_l2(y, exp)
    assert np.array_equal(y, dev.tensor(x).q_mat_mul(w).as_slice())  # fixed summation order
    assert dev.status() == 0


@pytest.mark.parametrize("tname,n,k", [("q5k", 4096, 4096), ("q5k", 4096, 14336), ("q5_0", 4096, 4096),
                                        ("q5_0", 1024, 4096)])
def test_q5_products_llama_shapes(dev, tname, n, k):
    ty = Q5_TYPES[tname]
    raw = F.random_q5_weights(n + k, 0.02, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    cols = np.sort(np.random.default_rng(2).choice(n, 128, replace=False))
    sub = _sampled_columns(raw, ty, n, k, cols)
    for m in (1, 8, 32):
        x = activations(300 + m, m, k)
        y = dev.tensor(x).q_mat_mul(w).as_slice()
        exp = O.q_mat_mul(x, sub, ty, len(cols), k)
        assert F.rel_l2(y[:, cols], exp) < TOL, (m, F.rel_l2(y[:, cols], exp))


def test_q5_epilogues(dev):
    # bias and residual rows are added by the product kernel; SwiGLU is refused for Q5_K (Q5_0, stored
    # as Q8_0 tiles, takes every epilogue of that type)
    for ty, k in ((O.Q5_0, 512), (O.Q5K, 512)):
        n = 96
        raw = F.random_q5_weights(23, 0.02, n, k, ty)
        w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
        for m in (1, 7, 40):
            x = activations(400 + m, m, k)
            exp = O.q_mat_mul(x, raw, ty, n, k)
            r1, r2 = activations(410 + m, m, n), activations(420 + m, m, n)
            y = dev.tensor(x).q_mat_mul(w, epilogue=kb.EPI_RESIDUAL, r1=dev.tensor(r1), r2=dev.tensor(r2)).as_slice()
            assert F.rel_l2(y, (exp + r1) + r2) < TOL
            bias = activations(430, 1, n)[0]
            y = dev.tensor(x).q_mat_mul(w, epilogue=kb.EPI_BIAS, r1=dev.tensor(bias)).as_slice()
            assert F.rel_l2(y, exp + bias[None, :]) < TOL
        if ty == O.Q5_0:
            x = activations(440, 3, k)
            exp = O.q_mat_mul(x, raw, ty, n, k)
            h = dev.tensor(x).q_mat_mul(w, epilogue=kb.EPI_SWIGLU).as_slice()
            assert F.rel_l2(h, O.silu_mul(exp[:, :n // 2], exp[:, n // 2:])) < TOL
            continue
        with pytest.raises(kb.FusorError) as e:
            dev.tensor(activations(1, 2, k)).q_mat_mul(w, epilogue=kb.EPI_SWIGLU)
        assert e.value.code == kb.ERR_UNSUPPORTED_DTYPE


@pytest.mark.parametrize("tname", ["q4k", "q6k", "q8_0"])
def test_prefill_product_split_k(dev, tname):
    # long rows, few tiles: the tcgen05 product cuts K into ranges (grid.z) and a second kernel adds the
    # partial products in range order, together with the residual or bias rows; ragged N and M
    ty = TYPES[tname]
    n, k = 1000, 8192
    raw = weights(61, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
    for m in (300, 513):
        x = activations(600 + m, m, k)
        exp = O.q_mat_mul(x, raw, ty, n, k)
        xt = dev.tensor(x)
        y = xt.q_mat_mul(w).as_slice()
        assert F.rel_l2(y, exp) < TOL, (tname, m, F.rel_l2(y, exp))
        assert np.array_equal(y, xt.q_mat_mul(w).as_slice())
        r1, r2 = activations(610 + m, m, n), activations(620 + m, m, n)
        y = xt.q_mat_mul(w, epilogue=kb.EPI_RESIDUAL, r1=dev.tensor(r1), r2=dev.tensor(r2)).as_slice()
        assert F.rel_l2(y, (exp + r1) + r2) < TOL
        bias = activations(630, 1, n)[0]
        y = xt.q_mat_mul(w, epilogue=kb.EPI_BIAS, r1=dev.tensor(bias)).as_slice()
        assert F.rel_l2(y, exp + bias[None, :]) < TOL
    assert dev.status() == 0
