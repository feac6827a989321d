"""Deterministic quantised fixtures used by the reference's conformance suite, restated.

The byte generators follow fusor-ml/conformance/src/common/quantized.rs:165-272 (the formulas
are data definitions: which byte holds which value); the shape list follows :309-335.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def f16_bytes(v: float) -> bytes:
    return np.float16(np.float32(v)).tobytes()


def nib(lo: int, hi: int) -> int:
    return (lo & 0x0F) | ((hi & 0x0F) << 4)


def deterministic_input(shape, seed):
    total = int(np.prod(shape))
    i = np.arange(total, dtype=np.int64)
    v = ((i + seed) % 23).astype(np.float32)
    return ((v - np.float32(11.0)) * np.float32(0.04)).reshape(shape)


def _blocks(shape, bs):
    return shape[0] * shape[1] // bs


def q4_0_raw_bytes(shape):
    out = bytearray()
    for b in range(_blocks(shape, 32)):
        out += f16_bytes(np.float32(0.025) + np.float32(b) * np.float32(0.003))
        out += bytes(nib(10 + ((b + i * 2) % 6), 9 + ((b * 3 + i * 5) % 7)) for i in range(16))
    return np.frombuffer(bytes(out), dtype=np.uint8)


def q5_0_raw_bytes(shape):
    out = bytearray()
    for b in range(_blocks(shape, 32)):
        out += f16_bytes(np.float32(0.02) + np.float32(b) * np.float32(0.0025))
        out += b"\xff" * 4
        out += bytes(nib(4 + ((b + i * 3) % 8), 6 + ((b * 2 + i * 5) % 8)) for i in range(16))
    return np.frombuffer(bytes(out), dtype=np.uint8)


def q8_0_raw_bytes(shape):
    out = bytearray()
    for b in range(_blocks(shape, 32)):
        out += f16_bytes(np.float32(0.01) + np.float32(b) * np.float32(0.0015))
        out += bytes((4 + ((b * 7 + i * 5) % 17)) & 0xFF for i in range(32))
    return np.frombuffer(bytes(out), dtype=np.uint8)


def q4k_raw_bytes(shape):
    out = bytearray()
    for b in range(_blocks(shape, 256)):
        out += f16_bytes(np.float32(0.004) + np.float32(b) * np.float32(0.0005))
        out += f16_bytes(np.float32(0.0005) + np.float32(b) * np.float32(0.0001))
        out += bytes(((b * 5 + i * 3) % 24) + 1 for i in range(12))
        out += bytes(nib(10 + ((b + i * 2) % 6), 11 + ((b * 3 + i) % 5)) for i in range(128))
    return np.frombuffer(bytes(out), dtype=np.uint8)


def q5k_raw_bytes(shape):
    out = bytearray()
    for b in range(_blocks(shape, 256)):
        out += f16_bytes(np.float32(0.0045) + np.float32(b) * np.float32(0.0004))
        out += f16_bytes(np.float32(0.0005) + np.float32(b) * np.float32(0.0001))
        out += bytes(((b * 7 + i * 2) % 24) + 1 for i in range(12))
        out += b"\xff" * 32
        out += bytes(nib(8 + ((b + i * 3) % 8), 9 + ((b * 2 + i * 5) % 7)) for i in range(128))
    return np.frombuffer(bytes(out), dtype=np.uint8)


def q6k_raw_bytes(shape):
    out = bytearray()
    for b in range(_blocks(shape, 256)):
        out += bytes(nib(b * 5 + i * 3 + 1, b * 7 + i * 11 + 2) for i in range(128))
        out += bytes((b * 17 + i * 9 + 0x12) & 0xFF for i in range(64))
        out += bytes((((b * 5 + i * 2) % 7) + 1) & 0xFF for i in range(16))
        out += f16_bytes(np.float32(0.0035) + np.float32(b) * np.float32(0.00035))
    return np.frombuffer(bytes(out), dtype=np.uint8)


GEN = {O.Q4_0: q4_0_raw_bytes, O.Q5_0: q5_0_raw_bytes, O.Q8_0: q8_0_raw_bytes,
       O.Q4K: q4k_raw_bytes, O.Q5K: q5k_raw_bytes, O.Q6K: q6k_raw_bytes}

# (name, type, [N, K], input rows, q_mat_mul abs tolerance, seed)
CONFORMANCE_CASES = [
    ("q4_0", O.Q4_0, (2, 64), 3, 1.0, 800),
    ("q5_0", O.Q5_0, (2, 64), 1, 1.0, 801),
    ("q8_0", O.Q8_0, (2, 64), 1, 0.5, 802),
    ("q4k", O.Q4K, (2, 512), 1, 2.0, 803),
    ("q5k", O.Q5K, (2, 512), 1, 1.0, 804),
    ("q6k", O.Q6K, (2, 512), 1, 1.0, 805),
    ("q5_0_wide", O.Q5_0, (2, 64), 3, 1.0, 810),
    ("q8_0_wide", O.Q8_0, (2, 64), 3, 0.5, 811),
    ("q8_0_single_row_wide_output", O.Q8_0, (96, 64), 1, 0.5, 826),
    ("q4k_wide", O.Q4K, (2, 512), 3, 2.0, 812),
    ("q4k_large_qgemv", O.Q4K, (8192, 512), 1, 2.0, 827),
    ("q4k_mid_qgemv", O.Q4K, (4096, 512), 1, 2.0, 830),
    ("q4k_tall_qgemv", O.Q4K, (128, 4608), 1, 2.0, 828),
    ("q4k_tail_rows_wide_output", O.Q4K, (128, 512), 48, 2.0, 832),
    ("q4k_tail_rows_llama_k", O.Q4K, (128, 4096), 48, 2.0, 833),
    ("q5k_wide", O.Q5K, (2, 512), 3, 1.0, 813),
    ("q6k_wide", O.Q6K, (2, 512), 3, 1.0, 814),
    ("q6k_large_qgemv", O.Q6K, (8192, 512), 1, 1.0, 831),
    ("q6k_tall_qgemv", O.Q6K, (128, 4608), 1, 1.0, 829),
    ("q4_0_tiled", O.Q4_0, (64, 64), 64, 1.0, 820),
    ("q5_0_tiled", O.Q5_0, (64, 64), 64, 1.0, 821),
    ("q8_0_tiled", O.Q8_0, (64, 64), 64, 0.5, 822),
    ("q4k_tiled", O.Q4K, (64, 512), 64, 2.0, 823),
    ("q5k_tiled", O.Q5K, (64, 512), 64, 1.0, 824),
    ("q6k_tiled", O.Q6K, (64, 512), 64, 1.0, 825),
]


def uniform_input(rows, k, seed, lo=-0.25, hi=0.25):
    """Seeded Uniform(-0.25, 0.25) activations (conformance/src/suite/native/quantized_matmul.rs:95-117
    draws from the same distribution; the generator itself is not pinned by the reference)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.uniform(lo, hi, size=(rows, k)).astype(np.float32)


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))


# ---- encoders for the two 5-bit formats -----------------------------------------------------------
# Only the tests need them (seeded weights with realistic statistics); parity is judged on the
# bytes they produce, through the oracle's decoder. Round-to-nearest on a min/max grid.

def quantize_q5_0(x):
    """f32 [..., 32 n] -> Q5_0 bytes: d = (value of largest magnitude) / -16, q = round(x / d) + 16."""
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    idx = np.argmax(np.abs(xb), axis=1)
    d = (xb[np.arange(xb.shape[0]), idx] / np.float32(-16.0)).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0).astype(np.float32)
    q = np.clip(np.floor(xb * inv[:, None] + 16.5), 0, 31).astype(np.uint32)
    lo, hi = q[:, :16], q[:, 16:]
    qs = ((lo & 15) | ((hi & 15) << 4)).astype(np.uint8)
    sh = np.arange(16, dtype=np.uint32)
    qh = (((lo >> 4) << sh).sum(axis=1) | ((hi >> 4) << (sh + 16)).sum(axis=1)).astype(np.uint32)
    out = np.empty((xb.shape[0], 22), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:6] = qh.view(np.uint8).reshape(-1, 4)
    out[:, 6:] = qs
    return out.reshape(-1)


def quantize_q5k(x):
    """f32 [..., 256 n] -> Q5_K bytes: per 32-element sub-block a 6-bit (scale, min) pair against the
    super-block's f16 d / dmin, 5-bit quants; byte layout of BlockQ5K (gguf/src/lib.rs:1819-1861)."""
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 8, 32)
    nb = xb.shape[0]
    mn = np.maximum(-xb.min(axis=2), 0)
    scale = (xb.max(axis=2) + mn) / np.float32(31.0)
    d = (scale.max(axis=1) / np.float32(63.0)).astype(np.float16)
    dmin = (mn.max(axis=1) / np.float32(63.0)).astype(np.float16)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.clip(np.rint(np.divide(scale, df[:, None], out=np.zeros_like(scale), where=df[:, None] > 0)), 0, 63).astype(np.uint32)
    m = np.clip(np.rint(np.divide(mn, dmf[:, None], out=np.zeros_like(mn), where=dmf[:, None] > 0)), 0, 63).astype(np.uint32)
    step = df[:, None] * sc
    q = np.divide(xb + (dmf[:, None] * m)[:, :, None], step[:, :, None], out=np.zeros_like(xb), where=step[:, :, None] > 0)
    q = np.clip(np.rint(q), 0, 31).astype(np.uint32)
    out = np.zeros((nb, 176), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    s = np.zeros((nb, 12), dtype=np.uint32)
    s[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    s[:, 4:8] = (m[:, 0:4] & 63) | ((m[:, 4:8] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:8] & 15) | ((m[:, 4:8] & 15) << 4)
    out[:, 4:16] = s.astype(np.uint8)
    qh = np.zeros((nb, 32), dtype=np.uint32)
    for j in range(8):
        qh |= (q[:, j, :] >> 4) << j
    out[:, 16:48] = qh.astype(np.uint8)
    for c in range(4):
        out[:, 48 + 32 * c:80 + 32 * c] = ((q[:, 2 * c, :] & 15) | ((q[:, 2 * c + 1, :] & 15) << 4)).astype(np.uint8)
    return out.reshape(-1)


def random_q5_weights(seed, sigma, n, k, ty):
    """Seeded N(0, sigma) [n, k] weights in Q5_0 / Q5_K bytes."""
    w = O.normal(seed, sigma, n * k)
    return quantize_q5_0(w) if ty == O.Q5_0 else quantize_q5k(w)
