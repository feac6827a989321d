"""GPU parity of the elementwise ops, the KV cache and attention against the oracle."""
import numpy as np
import pytest

import fixtures as F
import kalosm_b200 as kb
from gpu_util import dev, weights  # noqa: F401
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_rms_norm(dev):
    rng = np.random.default_rng(1)
    for rows, n in [(1, 4096), (5, 64), (3, 8192), (2, 100)]:
        x = rng.standard_normal((rows, n)).astype(np.float32)
        r = rng.standard_normal((rows, n)).astype(np.float32)
        w = (1 + 0.02 * rng.standard_normal(n)).astype(np.float32)
        b = rng.standard_normal(n).astype(np.float32)
        y = dev.rms_norm(dev.tensor(x), dev.tensor(w), 1e-5).as_slice()
        assert np.allclose(y, O.rms_norm(x, w, 1e-5), rtol=1e-5, atol=1e-6)
        y = dev.rms_norm(dev.tensor(x), dev.tensor(w), 1e-5, residual=dev.tensor(r),
                         bias=dev.tensor(b)).as_slice()
        assert np.allclose(y, O.rms_norm(x, w, 1e-5, residual=r, bias=b), rtol=1e-5, atol=1e-5)


def test_silu_mul(dev):
    rng = np.random.default_rng(2)
    g = (4 * rng.standard_normal(10000)).astype(np.float32)
    u = rng.standard_normal(10000).astype(np.float32)
    y = dev.silu_mul(dev.tensor(g), dev.tensor(u)).as_slice()
    assert np.allclose(y, O.silu_mul(g, u), rtol=1e-5, atol=1e-6)


def test_rope_tables_and_apply(dev):
    # table literals of models/kalosm-llama/src/raw/rope.rs:279-329
    rc = kb.RopeCache(dev, 2, 6, 5000.0)
    cos, sin = rc.cos.as_slice(), rc.sin.as_slice()
    assert np.abs(cos[:, 0] - [1.0, 0.5403, -0.4161, -0.99, -0.6536, 0.2837]).sum() < 1e-2
    assert np.abs(sin[:, 0] - [0.0, 0.8415, 0.9093, 0.1411, -0.7568, -0.9589]).sum() < 1e-2
    rng = np.random.default_rng(3)
    for scaling in (None, (8.0, 1.0, 4.0, 8192)):
        rc = kb.RopeCache(dev, 128, 64, 500000.0, scaling)
        ocos, osin = O.rope_tables(128, 64, 500000.0, scaling)
        assert np.allclose(rc.cos.as_slice(), ocos, atol=1e-6)
        assert np.allclose(rc.sin.as_slice(), osin, atol=1e-6)
        q = rng.standard_normal((2, 8, 5, 128)).astype(np.float32)
        k = rng.standard_normal((2, 2, 5, 128)).astype(np.float32)
        for inter in (True, False):
            qt, kt = dev.tensor(q), dev.tensor(k)
            rc.forward(qt, kt, start_pos=7, interleaved=inter)
            # tolerance 1e-4 as the reference's RoPE conformance cases (suite/native/rope_ops.rs:170-229)
            assert np.allclose(qt.as_slice(), O.rope(q, ocos, osin, 7, inter), atol=1e-4)
            assert np.allclose(kt.as_slice(), O.rope(k, ocos, osin, 7, inter), atol=1e-4)


def test_argmax_tie_rule(dev):
    # fusor-ml/fusor/src/lib.rs:432-443: ties -> higher id; non-finite skipped
    logits = np.zeros((3, 5000), dtype=np.float32)
    logits[0, [17, 4000, 4999]] = 3.0
    logits[1, 10] = np.inf
    logits[1, 11] = np.nan
    logits[1, 123] = 1.0
    logits[2] = -1.0
    logits[2, 0] = -0.5
    ids, vals = dev.argmax(dev.tensor(logits))
    ids, vals = ids.as_slice(), vals.as_slice()
    for r in range(3):
        oid, oval = O.top_k(logits[r], 1)
        assert ids[r] == oid[0] and vals[r] == oval[0]
    assert ids.tolist() == [4999, 123, 0]
    rng = np.random.default_rng(4)
    big = rng.standard_normal((4, 128256)).astype(np.float32)
    ids, _ = dev.argmax(dev.tensor(big))
    assert ids.as_slice().tolist() == big.argmax(axis=1).tolist()


def test_embedding_lookup(dev):
    for ty in (O.Q4K, O.Q6K, O.Q8_0, O.Q4_0):
        n, k = 100, 512
        raw = weights(ty, n, k, ty)
        w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
        ids = np.array([[0, 99, 17], [5, 5, 64]], dtype=np.uint32)
        out = w.embedding(dev.tensor(ids)).as_slice()
        table = O.dequantize(raw, ty, n * k).reshape(n, k)
        assert np.array_equal(out.view(np.uint32), table[ids].view(np.uint32))


def test_kv_cache_capacity_and_append(dev):
    # capacity literals of fusor-ml/fusor/src/cache/tensor_cache.rs:319-333
    rng = np.random.default_rng(5)
    c = kb.KvCache(dev, 2, 2, 64, 4096)
    k1 = rng.standard_normal((2, 2, 65, 64)).astype(np.float32)
    v1 = rng.standard_normal((2, 2, 65, 64)).astype(np.float32)
    kt, vt, n = c.append(dev.tensor(k1), dev.tensor(v1))
    assert n == 65 and c.capacity == 256
    k2 = rng.standard_normal((2, 2, 192, 64)).astype(np.float32)
    v2 = rng.standard_normal((2, 2, 192, 64)).astype(np.float32)
    kt, vt, n = c.append(dev.tensor(k2), dev.tensor(v2))
    assert n == 257 and c.capacity == 512
    full_k = np.concatenate([k1, k2], axis=2).astype(np.float16)
    assert np.array_equal(kt.as_slice()[:, :, :257], full_k)
    assert np.array_equal(vt.as_slice()[:, :, :257], np.concatenate([v1, v2], axis=2).astype(np.float16))
    small = kb.KvCache(dev, 1, 1, 64, 96)
    small.append(dev.tensor(k1[:1, :1]), dev.tensor(v1[:1, :1]))
    assert small.capacity == 96
    with pytest.raises(kb.FusorError) as e:
        small.append(dev.tensor(k1[:1, :1]), dev.tensor(v1[:1, :1]))
    assert e.value.code == kb.ERR_CAPACITY
    c.reset()
    assert c.current_seq_len == 0


def _attn_case(dev, b, h, hkv, sq, skv, d, causal, seed, tol, repeat=1):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((b, h, sq, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, skv, d)).astype(np.float16)
    v = rng.standard_normal((b, hkv, skv, d)).astype(np.float16)
    scale = float(1.0 / np.sqrt(d))
    exp = O.attention(q, k.astype(np.float32), v.astype(np.float32), scale, causal=causal)
    qt, kt, vt = dev.tensor(q), dev.tensor(k), dev.tensor(v)
    first = None
    for _ in range(repeat):
        out = dev.flash_attention(qt, kt, vt, scale, mask_kind=kb.MASK_CAUSAL if causal else kb.MASK_NONE).as_slice()
        err = np.max(np.abs(out - exp))
        assert err < tol, (b, h, hkv, sq, skv, err)
        assert F.rel_l2(out, exp) < 2e-3
        if first is None:
            first = out
        assert np.array_equal(first, out)


@pytest.mark.parametrize("kv", [129, 192, 256, 257, 384, 511, 512, 569, 1025])
@pytest.mark.parametrize("heads", [(16, 2), (32, 8)])
def test_decode_attention_tile_boundaries(dev, kv, heads):
    # conformance/src/suite/native/flash_attention_ops.rs:305-348: decode at tile-boundary KV
    # lengths, head_dim 128, each repeated 4x; tolerance 1e-3 (5e-3 beyond 1024 keys)
    h, hkv = heads
    _attn_case(dev, 1, h, hkv, 1, kv, 128, False, kv, 5e-3 if kv > 1024 else 1e-3, repeat=4)


@pytest.mark.parametrize("shape", [(1, 4, 4, 7, 7, 64, True), (2, 8, 2, 33, 33, 128, True),
                                   (1, 32, 8, 128, 128, 128, True), (2, 8, 8, 5, 40, 64, False),
                                   (1, 32, 8, 4, 300, 128, True), (8, 32, 8, 1, 1024, 128, False)])
def test_attention_prefill_and_gqa(dev, shape):
    b, h, hkv, sq, skv, d, causal = shape
    # 32 query positions and more run on fp16 tensor cores: wider absolute bound, same 2e-3 relative L2
    _attn_case(dev, b, h, hkv, sq, skv, d, causal, 7, 1e-3 if sq < 32 else 4e-3)


@pytest.mark.parametrize("shape", [(1, 32, 8, 512, 512, 128, True), (2, 8, 2, 100, 100, 64, True),
                                   (1, 8, 8, 96, 300, 128, True), (1, 4, 4, 70, 200, 64, False),
                                   (1, 32, 8, 33, 1000, 128, True), (1, 4, 1, 64, 64, 128, True),
                                   (1, 2, 2, 65, 129, 64, True)])
def test_prefill_attention_tensor_cores(dev, shape):
    # 32 or more query positions, no mask or causal: the tensor-core kernel (fp16 operands, fp32
    # accumulation: 2e-3 relative L2 against the f32 oracle). The cache is larger than the valid
    # length and holds NaN / huge values past it: they must never reach the result.
    b, h, hkv, sq, skv, d, causal = shape
    rng = np.random.default_rng(sq + skv)
    cap = skv + 37
    q = rng.standard_normal((b, h, sq, d)).astype(np.float32)
    k = np.full((b, hkv, cap, d), 1.0e4, np.float16)
    v = np.full((b, hkv, cap, d), np.nan, np.float16)
    k[:, :, :skv] = rng.standard_normal((b, hkv, skv, d))
    v[:, :, :skv] = rng.standard_normal((b, hkv, skv, d))
    scale = float(1.0 / np.sqrt(d))
    exp = O.attention(q, k[:, :, :skv].astype(np.float32), v[:, :, :skv].astype(np.float32), scale, causal=causal)
    qt, kt, vt = dev.tensor(q), dev.tensor(k), dev.tensor(v)
    kind = kb.MASK_CAUSAL if causal else kb.MASK_NONE
    out = dev.flash_attention(qt, kt, vt, scale, skv=skv, mask_kind=kind).as_slice()
    assert np.all(np.isfinite(out))
    assert F.rel_l2(out, exp) < 2e-3, F.rel_l2(out, exp)
    assert np.max(np.abs(out - exp)) < 4e-3
    assert np.array_equal(out, dev.flash_attention(qt, kt, vt, scale, skv=skv, mask_kind=kind).as_slice())


@pytest.mark.parametrize("s", [2048, 8192])
def test_prefill_attention_long_causal(dev, s):
    # causal prefill at the long sequence lengths of the sweep (32 query heads, 8 KV heads, head
    # size 128). Row i of a causal pass is the unmasked attention of that one query over keys
    # 0..i, which is how the oracle checks a sample of rows without an S x S score matrix.
    b, h, hkv, d = 1, 32, 8, 128
    rng = np.random.default_rng(s)
    q = rng.standard_normal((b, h, s, d), dtype=np.float32)
    k = rng.standard_normal((b, hkv, s, d), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((b, hkv, s, d), dtype=np.float32).astype(np.float16)
    scale = float(1.0 / np.sqrt(d))
    out = dev.flash_attention(dev.tensor(q), dev.tensor(k), dev.tensor(v), scale, mask_kind=kb.MASK_CAUSAL).as_slice()
    assert np.all(np.isfinite(out))
    rows = sorted({0, 1, 63, 64, 127, 128, s // 2 - 1, s // 2, s - 65, s - 64, s - 1} | set(rng.choice(s, 12).tolist()))
    for i in rows:
        exp = O.attention(q[:, :, i:i + 1], k[:, :, :i + 1].astype(np.float32), v[:, :, :i + 1].astype(np.float32), scale)
        err = F.rel_l2(out[:, :, i:i + 1], exp)
        assert err < 2e-3, (s, i, err)
    assert dev.status() == 0


@pytest.mark.parametrize("b,l", [(8, 4096), (8, 16384), (32, 4096)])
def test_decode_attention_long_contexts(dev, b, l):
    # one query position per sequence against a long fp16 cache (the split-KV decode kernel)
    h, hkv, d = 32, 8, 128
    rng = np.random.default_rng(b * l)
    q = rng.standard_normal((b, h, 1, d), dtype=np.float32)
    k = rng.standard_normal((b, hkv, l, d), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((b, hkv, l, d), dtype=np.float32).astype(np.float16)
    scale = float(1.0 / np.sqrt(d))
    out = dev.flash_attention(dev.tensor(q), dev.tensor(k), dev.tensor(v), scale).as_slice()
    exp = O.attention(q, k.astype(np.float32), v.astype(np.float32), scale)
    assert F.rel_l2(out, exp) < 2e-3, F.rel_l2(out, exp)
    assert np.max(np.abs(out - exp)) < 5e-3
    assert dev.status() == 0


def test_attention_masks_and_cache_capacity(dev):
    rng = np.random.default_rng(8)
    b, h, hkv, sq, skv, d, cap = 2, 4, 2, 6, 10, 64, 32
    q = rng.standard_normal((b, h, sq, d)).astype(np.float32)
    k = np.zeros((b, hkv, cap, d), np.float16)
    v = np.zeros((b, hkv, cap, d), np.float16)
    k[:, :, :skv] = rng.standard_normal((b, hkv, skv, d))
    v[:, :, :skv] = rng.standard_normal((b, hkv, skv, d))
    k[:, :, skv:] = 100.0  # rows beyond skv must never be read
    scale = 0.125
    kf, vf = k[:, :, :skv].astype(np.float32), v[:, :, :skv].astype(np.float32)
    qk = (rng.standard_normal((sq, skv)) * 2).astype(np.float32)
    out = dev.flash_attention(dev.tensor(q), dev.tensor(k), dev.tensor(v), scale, skv=skv,
                              mask=dev.tensor(qk), mask_kind=kb.MASK_QK).as_slice()
    assert np.max(np.abs(out - O.attention(q, kf, vf, scale, mask=qk, mask_kind=0))) < 1e-3
    bk = np.where(rng.random((b, skv)) < 0.3, -np.inf, 0.0).astype(np.float32)
    bk[:, 0] = 0.0
    out = dev.flash_attention(dev.tensor(q), dev.tensor(k), dev.tensor(v), scale, skv=skv,
                              mask=dev.tensor(bk), mask_kind=kb.MASK_BATCH_KEY).as_slice()
    assert np.max(np.abs(out - O.attention(q, kf, vf, scale, mask=bk, mask_kind=1))) < 1e-3


def test_peer_exchange_wait_is_bounded(dev):
    # a peer that never arrives: the wait gives up after its poll limit, the handle's status word
    # says so, and the GPU keeps working (no trap, no hang); a handle of its own keeps the
    # session handle's status clean. While the word is set every blocking call reports the
    # time-out; clearing the word brings the handle back.
    other = kb.Device(0)
    assert other.status() == 0
    with pytest.raises(kb.FusorError) as e:
        other.exchange_wait_check(4096)
    assert e.value.code == kb.ERR_TIMEOUT
    assert other.status() == kb.ERR_TIMEOUT
    x = other.tensor(np.ones((2, 8), np.float32))
    with pytest.raises(kb.FusorError) as e:  # the read-back is where a failed step surfaces
        x.as_slice()
    assert e.value.code == kb.ERR_TIMEOUT and "status" in str(e.value)
    with pytest.raises(kb.FusorError) as e:
        other.synchronize()
    assert e.value.code == kb.ERR_TIMEOUT
    other.clear_status()
    assert other.status() == 0
    other.synchronize()
    assert np.array_equal(x.as_slice(), np.ones((2, 8), np.float32))
    other.close()
    assert dev.status() == 0


def test_scratch_budget_and_poison(dev):
    # a handle with a scratch budget refuses a product whose packed activations do not fit
    # (instead of allocating), and serves it once the budget is lifted; in poison mode fresh
    # scratch starts as NaN bytes and the result is still exact, i.e. nothing reads scratch it
    # did not write
    other = kb.Device(0)
    ty, n, k = O.Q4K, 64, 8192
    raw = weights(12, n, k, ty)
    w = kb.QMatrix.from_raw_bytes(other, (n, k), raw, ty)
    x = np.random.default_rng(3).standard_normal((8, k)).astype(np.float32)
    other.set_scratch_limit(64 << 10)
    with pytest.raises(kb.FusorError) as e:
        other.tensor(x).q_mat_mul(w)
    assert e.value.code == kb.ERR_CAPACITY and "budget" in str(e.value)
    other.set_scratch_limit(0)
    other.set_poison(True)
    y = other.tensor(x).q_mat_mul(w).as_slice()
    assert F.rel_l2(y, O.q_mat_mul(x, raw, ty, n, k)) < 2e-3
    w.free()
    other.close()
