"""Pins the CPU oracle against the reference's own known answers (no GPU needed).

Each test names the reference test or fixture it restates.
"""
import numpy as np
import pytest

import fixtures as F
from oracle import oracle as O


def _block_q4_0(scale, packed):
    return F.f16_bytes(scale) + bytes([packed]) * 16


def _block_q5_0(scale, high_bits, low):
    return F.f16_bytes(scale) + bytes(high_bits) + bytes([low]) * 16


def _block_q8_0(scale, value):
    return F.f16_bytes(scale) + bytes([value & 0xFF]) * 32


X32 = np.arange(1, 33, dtype=np.float32)[None, :]


def test_q4_0_qgemv_known_answer():
    # fusor-ml/core/src/quantized/matmul/tests.rs:1336-1366 -> [528, -528]
    raw = np.frombuffer(_block_q4_0(1.0, 0x99) + _block_q4_0(1.0, 0x77), dtype=np.uint8)
    y = O.q_mat_mul(X32, raw, O.Q4_0, 2, 32)
    assert y.shape == (1, 2)
    assert abs(y[0, 0] - 528.0) < 1e-3 and abs(y[0, 1] + 528.0) < 1e-3


def test_q5_0_qgemv_known_answer():
    # tests.rs:1305-1334
    raw = np.frombuffer(_block_q5_0(1.0, [0xFF] * 4, 0x11) + _block_q5_0(1.0, [0] * 4, 0xFF),
                        dtype=np.uint8)
    y = O.q_mat_mul(X32, raw, O.Q5_0, 2, 32)
    assert abs(y[0, 0] - 528.0) < 1e-3 and abs(y[0, 1] + 528.0) < 1e-3


def test_q8_0_qgemv_known_answer():
    # tests.rs:1368-1397
    raw = np.frombuffer(_block_q8_0(1.0, 1) + _block_q8_0(1.0, -1), dtype=np.uint8)
    y = O.q_mat_mul(X32, raw, O.Q8_0, 2, 32)
    assert abs(y[0, 0] - 528.0) < 1e-3 and abs(y[0, 1] + 528.0) < 1e-3


def test_q5k_qgemv_known_answer():
    # tests.rs:1399-1423 -> 32896
    raw = (F.f16_bytes(1.0) + F.f16_bytes(0.0) + bytes([1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1])
           + bytes(32) + bytes([0x11]) * 128)
    x = np.arange(1, 257, dtype=np.float32)[None, :]
    y = O.q_mat_mul(x, np.frombuffer(raw, dtype=np.uint8), O.Q5K, 1, 256)
    assert abs(y[0, 0] - 32896.0) < 1e-2


def test_q5k_dequantize_literals():
    # fusor-ml/gguf/src/lib.rs:2377-2432
    qs = bytes(((i % 16) | (((i + 1) % 16) << 4)) for i in range(128))
    raw = F.f16_bytes(1.0) + F.f16_bytes(0.0) + bytes([1] * 12) + bytes(32) + qs
    d = O.dequantize(np.frombuffer(raw, dtype=np.uint8), O.Q5K, 256)
    assert np.allclose(d[:16], np.arange(16, dtype=np.float32), atol=0.01)
    raw = F.f16_bytes(1.0) + F.f16_bytes(0.0) + bytes([1] * 12) + bytes([0xFF]) * 32 + bytes(128)
    d = O.dequantize(np.frombuffer(raw, dtype=np.uint8), O.Q5K, 256)
    assert np.allclose(d[:32], 16.0, atol=0.01)


def test_q4k_scale_unpack_fixture_golden():
    # Block of fusor-ml/gguf/src/lib.rs:2322-2331; the reference pins its values through code,
    # so the frozen copy under tests/golden/ (made by tests/golden/make_golden.py) is compared
    # and the scale unpacking is also re-derived independently here.
    scales = [8, 16, 24, 32, 40, 48, 56, 64, 72, 80, 88, 96]
    qs = bytes((i * 3) % 256 for i in range(128))
    raw = F.f16_bytes(0.1) + F.f16_bytes(0.05) + bytes(scales) + qs
    d = O.dequantize(np.frombuffer(raw, dtype=np.uint8), O.Q4K, 256)
    dd, dm = np.float32(np.float16(0.1)), np.float32(np.float16(0.05))
    sc, mn = [], []
    for j in range(8):
        if j < 4:
            sc.append(scales[j] & 63)
            mn.append(scales[j + 4] & 63)
        else:
            sc.append((scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4))
            mn.append((scales[j + 4] >> 4) | ((scales[j] >> 6) << 4))
    exp = np.empty(256, dtype=np.float32)
    for j in range(4):
        for l in range(32):
            w = qs[32 * j + l]
            exp[64 * j + l] = np.float32(np.float32(sc[2 * j]) * dd) * np.float32(w & 0xF) \
                - np.float32(np.float32(mn[2 * j]) * dm)
            exp[64 * j + 32 + l] = np.float32(np.float32(sc[2 * j + 1]) * dd) * np.float32(w >> 4) \
                - np.float32(np.float32(mn[2 * j + 1]) * dm)
    assert np.array_equal(d.view(np.uint32), exp.view(np.uint32))
    gold = np.load(F.__file__.replace("fixtures.py", "golden/q4k_scale_fixture.npy"))
    assert np.array_equal(d.view(np.uint32), gold.view(np.uint32))


def test_block_geometry():
    # fusor-ml/gguf/src/lib.rs:99-121; core/src/quantized/mod.rs:578-617
    import ctypes as C
    for ty, (bs, bb) in O.BLOCK.items():
        e, b = C.c_int(), C.c_int()
        assert O.lib().oracle_block_geometry(ty, C.byref(e), C.byref(b)) == 0
        assert (e.value, b.value) == (bs, bb)


@pytest.mark.parametrize("case", F.CONFORMANCE_CASES, ids=lambda c: c[0])
def test_conformance_q_mat_mul_vs_host_matmul(case):
    # conformance/src/common/quantized.rs:120-163: expected = x @ dequantised^T on the host,
    # compared with the case's absolute tolerance.
    name, ty, (n, k), rows, tol, seed = case
    raw = F.GEN[ty]((n, k))
    w = O.dequantize(raw, ty, n * k).reshape(n, k)
    x = F.uniform_input(rows, k, seed)
    y = O.q_mat_mul(x, raw, ty, n, k)
    exp = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.max(np.abs(y - exp)) < tol
    assert F.rel_l2(y, exp) < 1e-5


def test_thread_count_does_not_change_results():
    ty, n, k = O.Q4K, 256, 512
    raw = F.q4k_raw_bytes((n, k))
    x = F.uniform_input(5, k, 1)
    O.set_threads(1)
    a1 = O.q_mat_mul(x[:1], raw, ty, n, k)
    a5 = O.q_mat_mul(x, raw, ty, n, k)
    O.set_threads(3)
    b1 = O.q_mat_mul(x[:1], raw, ty, n, k)
    b5 = O.q_mat_mul(x, raw, ty, n, k)
    O.set_threads(0)
    assert np.array_equal(a1, b1) and np.array_equal(a5, b5)
    assert np.array_equal(a1[0], a5[0])


@pytest.mark.parametrize("ty", [O.Q4_0, O.Q5_0, O.Q8_0, O.Q4K, O.Q5K, O.Q6K])
def test_dequantize_matches_gguf_package(ty):
    # Secondary cross-check with the independent `gguf` Python package where it is installed.
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    qt = {O.Q4_0: gguf.GGMLQuantizationType.Q4_0, O.Q5_0: gguf.GGMLQuantizationType.Q5_0,
          O.Q8_0: gguf.GGMLQuantizationType.Q8_0, O.Q4K: gguf.GGMLQuantizationType.Q4_K,
          O.Q5K: gguf.GGMLQuantizationType.Q5_K, O.Q6K: gguf.GGMLQuantizationType.Q6_K}[ty]
    bs, bb = O.BLOCK[ty]
    shape = (4, 2 * bs if bs == 256 else 8 * bs)
    raw = F.GEN[ty](shape)
    mine = O.dequantize(raw, ty, shape[0] * shape[1])
    theirs = quants.dequantize(raw.reshape(shape[0], -1), qt).reshape(-1)
    assert np.allclose(mine, theirs, rtol=1e-6, atol=1e-7)


def test_quantisers_emit_valid_blocks():
    for ty, tol in [(O.Q4_0, 0.15), (O.Q8_0, 0.01), (O.Q4K, 0.12), (O.Q6K, 0.04)]:
        x = O.normal(7 + ty, 0.02, 64 * 512)
        raw = O.quantize(x, ty)
        back = O.dequantize(raw, ty, x.size)
        assert np.all(np.isfinite(back))
        assert F.rel_l2(back, x) < tol, (ty, F.rel_l2(back, x))
        again = O.random_qweights(11, 0.02, 4096, ty)
        assert np.array_equal(again, O.random_qweights(11, 0.02, 4096, ty))


def test_rope_table_literals():
    # models/kalosm-llama/src/raw/rope.rs:279-329 (head_dim 2, theta 5000, ctx 6)
    cos, sin = O.rope_tables(2, 6, 5000.0)
    exp_cos = np.array([1.0, 0.5403, -0.4161, -0.99, -0.6536, 0.2837], dtype=np.float32)
    exp_sin = np.array([0.0, 0.8415, 0.9093, 0.1411, -0.7568, -0.9589], dtype=np.float32)
    assert np.abs(cos[:, 0] - exp_cos).sum() < 1e-2
    assert np.abs(sin[:, 0] - exp_sin).sum() < 1e-2


def test_rope_matches_host_reference():
    # conformance/src/common/mod.rs:631-653: plain rotation of pairs
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 3, 5, 8)).astype(np.float32)
    cos, sin = O.rope_tables(8, 16, 10000.0)
    for inter in (True, False):
        y = O.rope(x, cos, sin, start_pos=2, interleaved=inter)
        exp = np.empty_like(x)
        for s in range(5):
            c, sn = cos[2 + s], sin[2 + s]
            if inter:
                x0, x1 = x[:, :, s, 0::2], x[:, :, s, 1::2]
                exp[:, :, s, 0::2] = x0 * c - x1 * sn
                exp[:, :, s, 1::2] = x0 * sn + x1 * c
            else:
                x0, x1 = x[:, :, s, :4], x[:, :, s, 4:]
                exp[:, :, s, :4] = x0 * c - x1 * sn
                exp[:, :, s, 4:] = x1 * c + x0 * sn
        assert np.allclose(y, exp, atol=1e-6)


def test_kv_capacity_literals():
    # fusor-ml/fusor/src/cache/tensor_cache.rs:319-333
    assert O.kv_capacity(1, 4096) == 256
    assert O.kv_capacity(64, 4096) == 256
    assert O.kv_capacity(65, 4096) == 256
    assert O.kv_capacity(256, 4096) == 256
    assert O.kv_capacity(257, 4096) == 512
    assert O.kv_capacity(1, 96) == 96
    assert O.kv_capacity(65, 96) == 96
    assert O.kv_capacity(96, 96) == 96


def _attention_numpy(q, k, v, scale, causal):
    b, h, sq, d = q.shape
    hkv, skv = k.shape[1], k.shape[2]
    g = h // hkv
    out = np.empty(q.shape, dtype=np.float64)
    for bi in range(b):
        for hi in range(h):
            s = q[bi, hi].astype(np.float64) @ k[bi, hi // g].astype(np.float64).T * scale
            if causal:
                i = np.arange(sq)[:, None] + (skv - sq)
                s = np.where(np.arange(skv)[None, :] > i, -np.inf, s)
            s = np.exp(s - s.max(axis=1, keepdims=True))
            out[bi, hi] = (s / s.sum(axis=1, keepdims=True)) @ v[bi, hi // g].astype(np.float64)
    return out


@pytest.mark.parametrize("shape", [(1, 4, 2, 7, 7, 16, True), (2, 8, 2, 1, 33, 32, False),
                                   (1, 4, 4, 5, 9, 8, True)])
def test_attention_matches_scalar_reference(shape):
    # scalar attention of fusor-ml/core/tests/attention.rs:25-81 (softmax(q.k*scale [+causal]).v, GQA)
    b, h, hkv, sq, skv, d, causal = shape
    rng = np.random.default_rng(5)
    q = rng.standard_normal((b, h, sq, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, skv, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, skv, d)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    out = O.attention(q, k, v, scale, causal=causal)
    assert F.rel_l2(out, _attention_numpy(q, k, v, scale, causal)) < 1e-5
    if causal and sq == skv:
        mask = np.where(np.arange(skv)[None, :] > np.arange(sq)[:, None], -np.inf, 0.0)
        out2 = O.attention(q, k, v, scale, mask=mask.astype(np.float32), mask_kind=0)
        assert np.array_equal(out, out2)


def test_top_k_tie_rule():
    # fusor-ml/fusor/src/lib.rs:416-453: descending logit, ties -> higher id first, NaN/inf skipped
    logits = np.array([1.0, 3.0, 3.0, np.nan, 2.0, np.inf, 3.0], dtype=np.float32)
    ids, vals = O.top_k(logits, 3)
    assert ids.tolist() == [6, 2, 1] and vals.tolist() == [3.0, 3.0, 3.0]
    ids, _ = O.top_k(logits, 1)
    assert ids.tolist() == [6]


def test_rms_norm_and_silu():
    rng = np.random.default_rng(9)
    x = rng.standard_normal((3, 64)).astype(np.float32)
    r = rng.standard_normal((3, 64)).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    y = O.rms_norm(x, w, 1e-5, residual=r)
    s = (x + r).astype(np.float64)
    exp = s / np.sqrt((s * s).mean(axis=1, keepdims=True) + 1e-5) * w
    assert np.allclose(y, exp, rtol=1e-5, atol=1e-6)
    g = O.silu_mul(x, r)
    assert np.allclose(g, x / (1 + np.exp(-x.astype(np.float64))) * r, rtol=1e-5, atol=1e-6)


def test_frozen_conformance_vectors():
    # tests/golden/conformance_small.npz (made by tests/golden/make_golden.py)
    import os
    gold = np.load(os.path.join(os.path.dirname(F.__file__), "golden", "conformance_small.npz"))
    O.set_threads(1)
    try:
        for name, ty, (n, k), rows, _tol, seed in F.CONFORMANCE_CASES[:6]:
            raw = F.GEN[ty]((n, k))
            assert np.array_equal(O.dequantize(raw, ty, n * k).view(np.uint32),
                                  gold[name + "_deq"].view(np.uint32))
            x = F.deterministic_input((rows, k), seed)
            assert np.array_equal(O.q_mat_mul(x, raw, ty, n, k), gold[name + "_y"])
    finally:
        O.set_threads(0)


def test_sampler_properties_of_the_reference_tests():
    # models/kalosm-llama/src/sampler.rs:372-441 restated on the oracle's samplers (with the
    # counter-based draw in place of rand::StdRng): flat logits reach past the first sorted
    # candidate, top-p 0.5 keeps the first two of four, min-p 0.1 keeps only the leader, and
    # Mirostat's cut-off keeps every candidate when no surprise exceeds mu.
    flat = np.zeros(4, np.float32)
    assert {O.sample(flat, top_k=4, seed=s)[0] for s in range(64)} - {3}
    assert {O.sample(flat, top_k=4, seed=s, strategy=1, mu=10.0)[0] for s in range(64)} - {3}
    assert {O.sample(flat, top_k=4, top_p=0.5, seed=s)[0] for s in range(64)} <= {2, 3}
    assert O.sample(np.array([-5.0, -4.0, -3.0, 0.0], np.float32), top_k=4, min_p=0.1, seed=0)[0] == 3
    # sort order: descending value, ties -> higher id (sampler.rs:252-259); temperature 0 = first
    assert O.sample(np.array([1.0, 2.0, 2.0, 0.5], np.float32), temperature=0.0, top_k=2)[0] == 2
    # repetition penalty (sampler.rs:272-279): positive logits divided, non-positive multiplied
    lg = np.array([2.0, 1.9, -0.1, -0.2], np.float32)
    assert O.sample(lg, temperature=0.0, top_k=4, repetition_penalty=2.0, previous=[0])[0] == 1      # 1.0 < 1.9
    assert O.sample(lg, temperature=0.0, top_k=4, repetition_penalty=2.0, previous=[0, 1])[0] == 0   # 1.0 > 0.95
    assert O.sample(np.array([-0.1, -0.15], np.float32), temperature=0.0, top_k=2, repetition_penalty=2.0,
                    previous=[0])[0] == 1                                                            # -0.2 < -0.15
    assert O.sample(lg, temperature=0.0, top_k=4, repetition_penalty=1.0, previous=[0])[0] == 0      # <= 1: off
    # only the last `range` previous tokens count (sampler.rs:297-303)
    assert O.sample(lg, temperature=0.0, top_k=4, repetition_penalty=2.0, repetition_penalty_range=1,
                    previous=[0, 3])[0] == 0
    assert O.sample(np.full(8, np.nan, np.float32), top_k=4)[0] == 0xFFFFFFFF
