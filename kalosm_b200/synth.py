"""Synthetic GGUF-block weights: seeded N(0, sigma) values encoded as Q4_0 / Q8_0 / Q4_K / Q6_K.

The reference only ever loads pre-quantised GGUF files and ships no f32 -> Q4_K / Q6_K encoder,
so random-weight models need one. These encoders are simple (min/max per sub-block, absmax per
group) and vectorised with torch so that an 8B-parameter model is generated in seconds on the
device that will run it; their only duty is to emit structurally valid blocks (layouts of
fusor-ml/gguf/src/lib.rs:764-769, 1124-1127, 1427-1432, 1935-1944) with finite scales.
Returns raw block bytes as a uint8 tensor, ready for ``QMatrix.from_raw_bytes``.
"""
from __future__ import annotations

import torch

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _f16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).to(torch.float32)


def _safe_inv(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 0, 1.0 / x, torch.zeros_like(x))


def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    b = x.reshape(-1, 32).float()
    d = _f16_round(b.abs().amax(dim=1) / 7.0)
    q = (torch.round(b * _safe_inv(d)[:, None]) + 8).clamp_(0, 15).to(torch.uint8)
    qs = q[:, :16] | (q[:, 16:] << 4)
    return torch.cat([_f16_bytes(d), qs], dim=1).reshape(-1)


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    b = x.reshape(-1, 32).float()
    d = _f16_round(b.abs().amax(dim=1) / 127.0)
    q = torch.round(b * _safe_inv(d)[:, None]).clamp_(-127, 127).to(torch.int8).view(torch.uint8)
    return torch.cat([_f16_bytes(d), q], dim=1).reshape(-1)


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    b = x.reshape(-1, 8, 32).float()  # [super-block, sub-block, element]
    lo, hi = b.amin(dim=2), b.amax(dim=2)
    off = (-lo).clamp_(min=0)
    scale = (hi + off) / 15.0
    d = _f16_round(scale.amax(dim=1) / 63.0)
    dmin = _f16_round(off.amax(dim=1) / 63.0)
    sc = torch.round(scale * _safe_inv(d)[:, None]).clamp_(0, 63).to(torch.uint8)
    mn = torch.round(off * _safe_inv(dmin)[:, None]).clamp_(0, 63).to(torch.uint8)
    s_eff = d[:, None] * sc.float()
    o_eff = dmin[:, None] * mn.float()
    q = torch.round((b + o_eff[:, :, None]) * _safe_inv(s_eff)[:, :, None]).clamp_(0, 15).to(torch.uint8)
    # 6-bit packing (inverse of unpack_k4_scales_offsets, fusor-ml/gguf/src/lib.rs:2138-2208)
    p = torch.empty(b.shape[0], 12, dtype=torch.uint8, device=x.device)
    p[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    p[:, 4:8] = mn[:, 0:4] | ((mn[:, 4:8] >> 4) << 6)
    p[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mn[:, 4:8] & 0xF) << 4)
    qs = (q[:, 0::2, :] | (q[:, 1::2, :] << 4)).reshape(-1, 128)
    return torch.cat([_f16_bytes(d), _f16_bytes(dmin), p, qs], dim=1).reshape(-1)


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    b = x.reshape(-1, 16, 16).float()  # [super-block, group, element]
    gs = b.abs().amax(dim=2) / 31.0
    d = _f16_round(gs.amax(dim=1) / 127.0)
    sc = torch.round(gs * _safe_inv(d)[:, None]).clamp_(0, 127).to(torch.int8)
    s_eff = d[:, None] * sc.float()
    q = (torch.round(b * _safe_inv(s_eff)[:, :, None]) + 32).clamp_(0, 63).to(torch.uint8).reshape(-1, 2, 4, 32)
    q1, q2, q3, q4 = q[:, :, 0], q[:, :, 1], q[:, :, 2], q[:, :, 3]  # [sb, half, 32]
    ql = torch.stack([(q1 & 0xF) | ((q3 & 0xF) << 4), (q2 & 0xF) | ((q4 & 0xF) << 4)], dim=2).reshape(-1, 128)
    qh = ((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)).reshape(-1, 64)
    return torch.cat([ql, qh, sc.view(torch.uint8), _f16_bytes(d)], dim=1).reshape(-1)


_ENCODERS = {Q4_0: quantize_q4_0, Q8_0: quantize_q8_0, Q4_K: quantize_q4_k, Q6_K: quantize_q6_k}
_BLOCK = {Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256}


def quantize(x: torch.Tensor, ggml_type: int) -> torch.Tensor:
    if x.numel() % _BLOCK[ggml_type]:
        raise ValueError("element count is not a multiple of the block size")
    return _ENCODERS[ggml_type](x)


def random_qweights(seed: int, sigma: float, n: int, k: int, ggml_type: int, device="cpu",
                    chunk_rows: int = 8192) -> torch.Tensor:
    """Raw block bytes of a seeded N(0, sigma) [n, k] matrix, generated in row chunks."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    parts = []
    for r0 in range(0, n, chunk_rows):
        rows = min(chunk_rows, n - r0)
        w = torch.randn(rows, k, generator=gen, device=device, dtype=torch.float32) * sigma
        parts.append(quantize(w, ggml_type))
    return torch.cat(parts) if len(parts) > 1 else parts[0]
