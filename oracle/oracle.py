"""ctypes binding of the CPU oracle (``libfusor_oracle.so``).

Test infrastructure only: tests, the smoke check and the benchmark's CPU-baseline leg import
this; the product package never does. Arrays are numpy, C-contiguous.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfusor_oracle.so")

# ggml type ids, fusor-ml/gguf/src/lib.rs:35-50
F32, F16, Q4_0, Q5_0, Q8_0, Q4K, Q5K, Q6K = 0, 1, 2, 6, 8, 12, 13, 14
BLOCK = {Q4_0: (32, 18), Q5_0: (32, 22), Q8_0: (32, 34), Q4K: (256, 144), Q5K: (256, 176),
         Q6K: (256, 210)}
TYPE_NAMES = {Q4_0: "Q4_0", Q5_0: "Q5_0", Q8_0: "Q8_0", Q4K: "Q4_K", Q5K: "Q5_K", Q6K: "Q6_K"}


def build(force: bool = False) -> str:
    """Compile the oracle if the shared object is missing or older than its source."""
    src = os.path.join(_HERE, "fusor_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libfusor_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        vp, u8p, f32p, u32p = C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p
        sz, u32, i32, f32, u64 = C.c_size_t, C.c_uint32, C.c_int, C.c_float, C.c_uint64
        sigs = {
            "oracle_set_threads": (None, [i32]),
            "oracle_num_threads": (i32, []),
            "oracle_block_geometry": (i32, [u32, C.POINTER(i32), C.POINTER(i32)]),
            "oracle_f16_to_f32": (f32, [C.c_uint16]),
            "oracle_f32_to_f16": (C.c_uint16, [f32]),
            "oracle_dequantize": (i32, [u8p, u32, sz, f32p]),
            "oracle_q_mat_mul": (i32, [f32p, sz, sz, u8p, u32, sz, f32p]),
            "oracle_rms_norm": (None, [f32p, f32p, f32p, f32p, f32, sz, sz, f32p]),
            "oracle_silu_mul": (None, [f32p, f32p, sz, f32p]),
            "oracle_rope_tables": (None, [i32, i32, f32, f32, f32, f32, i32, f32p, f32p]),
            "oracle_rope": (None, [f32p, i32, i32, i32, i32, f32p, f32p, i32, i32]),
            "oracle_attention": (None, [f32p, f32p, f32p, i32, i32, i32, i32, i32, i32, sz, f32,
                                        f32p, i32, i32, f32p]),
            "oracle_kv_capacity": (sz, [sz, sz]),
            "oracle_top_k": (i32, [f32p, sz, i32, u32p, f32p]),
            "oracle_sample": (u32, [f32p, sz, i32, f32, f32, i32, i32, f32, f32, f32, f32, f32p, u32p, i32, u64, u64,
                                    u32, f32p]),
            "oracle_quantize": (i32, [f32p, sz, u32, u8p]),
            "oracle_normal": (None, [u64, f32, sz, f32p]),
            "oracle_random_qweights": (i32, [u64, f32, sz, u32, u8p]),
            "oracle_llama_create": (vp, [i32] * 8 + [f32, f32, i32, i32]),
            "oracle_llama_free": (None, [vp]),
            "oracle_llama_set_rope": (None, [vp, f32, f32, f32, i32, f32p]),
            "oracle_rope_tables_w": (None, [i32, i32, f32, f32, f32, f32, i32, f32p, f32p, f32p]),
            "oracle_llama_set_qmatrix": (i32, [vp, i32, i32, u32, sz, sz, u8p, sz]),
            "oracle_llama_set_norm": (i32, [vp, i32, i32, f32p, sz]),
            "oracle_llama_reset": (None, [vp]),
            "oracle_llama_pos": (i32, [vp]),
            "oracle_llama_truncate": (i32, [vp, i32]),
            "oracle_llama_forward": (i32, [vp, u32p, i32, f32p]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def num_threads() -> int:
    return lib().oracle_num_threads()


def nbytes_for(ty: int, n_elems: int) -> int:
    bs, bb = BLOCK[ty]
    assert n_elems % bs == 0
    return n_elems // bs * bb


def dequantize(raw: np.ndarray, ty: int, n_elems: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    assert raw.size == nbytes_for(ty, n_elems)
    out = np.empty(n_elems, dtype=np.float32)
    rc = lib().oracle_dequantize(_p(raw), ty, n_elems, _p(out))
    if rc:
        raise ValueError(f"oracle_dequantize rc={rc}")
    return out


def q_mat_mul(x: np.ndarray, raw: np.ndarray, ty: int, n: int, k: int) -> np.ndarray:
    x = _f32(x)
    x2 = x.reshape(-1, k)
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    assert raw.size == nbytes_for(ty, n * k)
    y = np.empty((x2.shape[0], n), dtype=np.float32)
    rc = lib().oracle_q_mat_mul(_p(x2), x2.shape[0], k, _p(raw), ty, n, _p(y))
    if rc:
        raise ValueError(f"oracle_q_mat_mul rc={rc}")
    return y.reshape(x.shape[:-1] + (n,))


def rms_norm(x, w, eps, residual=None, bias=None):
    x = _f32(x)
    n = x.shape[-1]
    rows = x.size // n
    res = None if residual is None else _f32(residual)
    b = None if bias is None else _f32(bias)
    w = _f32(w)
    y = np.empty_like(x)
    lib().oracle_rms_norm(_p(x), _p(res), _p(w), _p(b), eps, rows, n, _p(y))
    return y


def silu_mul(gate, up):
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().oracle_silu_mul(_p(gate), _p(up), gate.size, _p(out))
    return out


def rope_tables(head_dim, ctx, theta, scaling=None):
    cos = np.empty((ctx, head_dim // 2), dtype=np.float32)
    sin = np.empty_like(cos)
    factor, low, high, orig = (0.0, 1.0, 4.0, ctx) if scaling is None else scaling
    lib().oracle_rope_tables(head_dim, ctx, theta, factor, low, high, orig, _p(cos), _p(sin))
    return cos, sin


def rope(x, cos, sin, start_pos=0, interleaved=True):
    x = _f32(x).copy()
    b, h, s, d = x.shape
    cos, sin = _f32(cos), _f32(sin)
    lib().oracle_rope(_p(x), b, h, s, d, _p(cos), _p(sin), start_pos, 1 if interleaved else 0)
    return x


def attention(q, k, v, scale, mask=None, mask_kind=0, causal=False):
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, h, sq, d = q.shape
    _, hkv, skv, _ = k.shape
    m = None if mask is None else _f32(mask)
    out = np.empty_like(q)
    lib().oracle_attention(_p(q), _p(k), _p(v), b, h, hkv, sq, skv, d, skv * d, scale, _p(m),
                           mask_kind, 1 if causal else 0, _p(out))
    return out


def kv_capacity(required, max_len):
    return lib().oracle_kv_capacity(required, max_len)


def top_k(logits, k):
    logits = _f32(logits)
    ids = np.empty(max(k, 1), dtype=np.uint32)
    vals = np.empty(max(k, 1), dtype=np.float32)
    n = lib().oracle_top_k(_p(logits), logits.size, k, _p(ids), _p(vals))
    return ids[:n], vals[:n]


def sample(logits, *, strategy=0, temperature=1.0, repetition_penalty=1.0, repetition_penalty_range=64, top_k=64,
           top_p=float("nan"), min_p=float("nan"), tau=5.0, eta=0.1, mu=None, previous=None, seed=0, counter=0, row=0):
    """One draw of the reference's CPU sampler (models/kalosm-llama/src/sampler.rs) on one row of logits.
    Returns (token id, margin, new mu): margin = relative distance of the draw from the nearest
    cumulative boundary; mu only for Mirostat 2 (strategy 1)."""
    logits = _f32(logits).reshape(-1)
    prev = None if previous is None else np.ascontiguousarray(previous, dtype=np.uint32).reshape(-1)
    mu_arr = np.array([10.0 if mu is None else mu], dtype=np.float32)
    margin = np.ones(1, dtype=np.float32)
    tok = lib().oracle_sample(_p(logits), logits.size, strategy, temperature, repetition_penalty,
                              repetition_penalty_range, top_k, top_p, min_p, tau, eta, _p(mu_arr), _p(prev),
                              0 if prev is None else prev.size, seed, counter, row, _p(margin))
    return int(tok), float(margin[0]), float(mu_arr[0])


def quantize(x, ty):
    x = _f32(x).reshape(-1)
    out = np.empty(nbytes_for(ty, x.size), dtype=np.uint8)
    rc = lib().oracle_quantize(_p(x), x.size, ty, _p(out))
    if rc:
        raise ValueError(f"oracle_quantize rc={rc}")
    return out


def normal(seed, sigma, n):
    out = np.empty(n, dtype=np.float32)
    lib().oracle_normal(seed, sigma, n, _p(out))
    return out


def random_qweights(seed, sigma, n_elems, ty):
    out = np.empty(nbytes_for(ty, n_elems), dtype=np.uint8)
    rc = lib().oracle_random_qweights(seed, sigma, n_elems, ty, _p(out))
    if rc:
        raise ValueError(f"oracle_random_qweights rc={rc}")
    return out


class Llama:
    """Llama decoder oracle (order of operations of kalosm-llama's CPU forward)."""

    WHICH = {"token_embd": 0, "output": 1, "wq": 2, "wk": 3, "wv": 4, "wo": 5, "gate": 6, "up": 7,
             "down": 8}
    NORMS = {"attn_norm": 0, "ffn_norm": 1, "output_norm": 2}

    def __init__(self, n_layer, hidden, ffn, n_head, n_kv_head, head_dim, vocab, ctx, eps=1e-5,
                 theta=500000.0, batch=1, kv_f16=True):
        self.cfg = dict(n_layer=n_layer, hidden=hidden, ffn=ffn, n_head=n_head,
                        n_kv_head=n_kv_head, head_dim=head_dim, vocab=vocab, ctx=ctx, eps=eps,
                        theta=theta, batch=batch)
        self.h = lib().oracle_llama_create(n_layer, hidden, ffn, n_head, n_kv_head, head_dim,
                                           vocab, ctx, eps, theta, batch, 1 if kv_f16 else 0)
        self.vocab, self.batch = vocab, batch

    def set_qmatrix(self, name, layer, ty, n, k, raw):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        rc = lib().oracle_llama_set_qmatrix(self.h, layer, self.WHICH[name], ty, n, k, _p(raw),
                                            raw.size)
        if rc:
            raise ValueError(f"set_qmatrix {name} rc={rc}")

    def set_norm(self, name, layer, w):
        w = _f32(w)
        rc = lib().oracle_llama_set_norm(self.h, layer, self.NORMS[name], _p(w), w.size)
        if rc:
            raise ValueError(f"set_norm {name} rc={rc}")

    def set_rope(self, scaling=None, freq_weight=None):
        """RoPE scaling (factor, low_freq_factor, high_freq_factor, original_ctx) and/or rope_freqs.weight."""
        factor, low, high, orig = (0.0, 1.0, 4.0, self.cfg["ctx"]) if scaling is None else scaling
        fw = None if freq_weight is None else _f32(freq_weight)
        lib().oracle_llama_set_rope(self.h, factor, low, high, orig, _p(fw))

    def reset(self):
        lib().oracle_llama_reset(self.h)

    def truncate(self, length):
        if lib().oracle_llama_truncate(self.h, length):
            raise ValueError(f"cannot truncate {self.pos} positions to {length}")

    @property
    def pos(self):
        return lib().oracle_llama_pos(self.h)

    def forward(self, tokens):
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(self.batch, -1)
        logits = np.empty((self.batch, self.vocab), dtype=np.float32)
        rc = lib().oracle_llama_forward(self.h, _p(tokens), tokens.shape[1], _p(logits))
        if rc:
            raise ValueError(f"oracle_llama_forward rc={rc}")
        return logits

    def __del__(self):
        try:
            lib().oracle_llama_free(self.h)
        except Exception:
            pass
