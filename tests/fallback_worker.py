"""Runs in a child process of tests/test_gpu_fallbacks.py with one kernel-selection variable set.

The library reads those variables once per process, so each alternative kernel gets a process of its
own. Every case is checked against the oracle with the bound of the parity tests proper.
Prints one line "ok <what>" per case; any failure raises.
"""
import sys

import numpy as np

sys.path.insert(0, __file__.rsplit("/", 2)[0])
sys.path.insert(0, __file__.rsplit("/", 1)[0])

import fixtures as F  # noqa: E402
import kalosm_b200 as kb  # noqa: E402
from llama_util import build_models, tiny_cfg  # noqa: E402
from oracle import oracle as O  # noqa: E402

TOL = 2e-3


def products(dev, row_counts):
    """q_mat_mul of 2 .. 32 activation rows: Q4_K, Q6_K, Q8_0 and Q4_0 weights; a K of several
    groups per warp (4096) and a long one (14336 = 56 groups, beyond the K-stationary kernel)."""
    for ty, n, k in [(O.Q4K, 512, 4096), (O.Q6K, 256, 14336), (O.Q8_0, 384, 4096), (O.Q4_0, 256, 2048)]:
        raw = O.random_qweights(11 + ty, 0.02, n * k, ty)
        w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty)
        for m in row_counts:
            x = O.normal(500 + m, 1.0, m * k).reshape(m, k)
            y = dev.tensor(x).q_mat_mul(w).as_slice()
            err = F.rel_l2(y, O.q_mat_mul(x, raw, ty, n, k))
            assert err < TOL, (ty, n, k, m, err)
            print(f"ok product type {ty} {n}x{k} rows {m}: {err:.1e}")


def attention(dev, cases):
    for b, h, hkv, sq, skv, d, causal in cases:
        rng = np.random.default_rng(skv * 7 + sq)
        q = rng.standard_normal((b, h, sq, d)).astype(np.float32)
        k = rng.standard_normal((b, hkv, skv, d)).astype(np.float16)
        v = rng.standard_normal((b, hkv, skv, d)).astype(np.float16)
        scale = float(1.0 / np.sqrt(d))
        exp = O.attention(q, k.astype(np.float32), v.astype(np.float32), scale, causal=causal)
        out = dev.flash_attention(dev.tensor(q), dev.tensor(k), dev.tensor(v), scale,
                                  mask_kind=kb.MASK_CAUSAL if causal else kb.MASK_NONE).as_slice()
        err = F.rel_l2(out, exp)
        assert err < TOL and np.max(np.abs(out - exp)) < 5e-3, (b, h, hkv, sq, skv, err)
        print(f"ok attention b{b} h{h}/{hkv} q{sq} kv{skv} d{d}: {err:.1e}")


def decoder(dev, batch, prompt_len=9):
    """Prompt pass and six steps of a two-layer decoder at `batch` sequences."""
    cfg = tiny_cfg()
    gpu, cpu = build_models(dev, cfg, batch=batch, seed=31)
    prompt = np.random.default_rng(32).integers(0, cfg["vocab"], size=(batch, prompt_len), dtype=np.uint32)
    lg, nxt = gpu.forward(prompt)
    lo = cpu.forward(prompt)
    assert F.rel_l2(lg, lo) < 8e-3
    tok = np.array([O.top_k(lo[i], 1)[0][0] for i in range(batch)], dtype=np.uint32)
    for step in range(6):
        lo = cpu.forward(tok[:, None])
        lg, nxt = gpu.forward(tok[:, None])
        err = F.rel_l2(lg, lo)
        assert err < 4e-3, (step, err)
        tok = np.array([O.top_k(lo[i], 1)[0][0] for i in range(batch)], dtype=np.uint32)
    print(f"ok decoder batch {batch}")


def main(what):
    dev = kb.Device(0)
    if what == "streamed":          # FB200_GEMM16_STREAMED=1: K streamed through shared memory
        products(dev, [2, 8, 9, 16, 17, 32])
        decoder(dev, 4)
    elif what == "exact_small":     # FB200_EXACT_SMALL_BATCH=1: 2 .. 8 rows on the int8 limb kernel
        products(dev, [2, 5, 8])
    elif what == "decode_scalar":   # FB200_ATTN_DECODE_TC=0: decode attention without tensor cores
        attention(dev, [(1, 32, 8, 1, 569, 128, False), (4, 32, 8, 1, 1025, 128, False),
                        (2, 16, 2, 1, 64, 128, False), (3, 8, 8, 1, 300, 64, False)])
        decoder(dev, 4)
    elif what == "prefill_mma":     # FB200_ATTN_TCGEN05=0: prompt attention on the mma.sync kernel
        attention(dev, [(1, 8, 2, 128, 128, 128, True), (1, 8, 8, 200, 200, 128, True),
                        (2, 4, 2, 64, 320, 128, False)])
    elif what == "q5k_row_copies":   # FB200_Q5K_TENSOR_TMA=0: Q5_K stages fetched by 16 row copies
        for n, k in ((273, 1024), (512, 4096)):
            raw = F.random_q5_weights(71, 0.02, n, k, O.Q5K)
            w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, O.Q5K)
            for m in (1, 8, 16, 32, 40):
                x = O.normal(700 + m, 1.0, m * k).reshape(m, k) + np.float32(0.5)
                err = F.rel_l2(dev.tensor(x).q_mat_mul(w).as_slice(), O.q_mat_mul(x, raw, O.Q5K, n, k))
                assert err < TOL, (n, k, m, err)
                print(f"ok Q5_K {n}x{k} rows {m}: {err:.1e}")
    elif what == "prefill_sequential":  # FB200_TC_GROUP=0: q, k, v of a prompt pass one after the other
        decoder(dev, 1, prompt_len=48)
    else:
        raise SystemExit(f"unknown case {what}")
    assert dev.status() == 0
    print("done", what)


if __name__ == "__main__":
    main(sys.argv[1])
