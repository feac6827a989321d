#!/usr/bin/env python
"""Benchmark: Llama-3-8B-shaped Q4_K_M-style greedy decode on B200 through libfusor_b200.so.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

A step is one decode step (one new token per sequence) after a 512-token prompt. Prints ONE JSON
line. `value` = tokens/s of the device-resident greedy loop (CUDA-graph replays, only token ids
leave the GPU at the end); `e2e` = the same metric with the token id uploaded from pinned host
memory and the next id read back every step through fb200_llama_forward. With --gpus N > 1
(under torchrun) every rank runs an independent replica of the model on its own GPU (the model
fits one GPU, so the path does not shard: replicas only, no collective on the data path).

--impl reference times the reference's CPU algorithm (the C++ restatement under oracle/, the
reference itself is Rust and cannot be built here) on the host cores: each step is 1/32 of a
decode step's work (one transformer layer + 1/32 of the output head rows).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(n_layer=32, hidden=4096, ffn=14336, n_head=32, n_kv_head=8, head_dim=128, vocab=128256)
PROMPT = 512
# DRAM traffic of the dominant kernel (the fused decode-step kernel) per ALGORITHMIC byte, from the
# profiler capture summarised under profiles/ (a 4-layer model of the same shapes, one step:
# dram__bytes_read.sum + dram__bytes_write.sum = 1 002 517 760 B for 995 057 664 algorithmic bytes);
# traffic grows in proportion to the layers, so a full launch is scaled by its algorithmic bytes.
FUSED_TRAFFIC_PER_BYTE = 1002517760 / 995057664
Q4_0, Q8_0, Q4_K, Q6_K, F32 = 2, 8, 12, 14, 0
BLOCK_BYTES = {Q4_0: 18 * 8, Q8_0: 34 * 8, Q4_K: 144, Q6_K: 210}  # bytes per 256 elements
METRIC = "Llama-3-8B Q4_K decode tok/s @1 GPU; quant GEMV HBM GB/s vs ~8 TB/s peak"


def tensor_plan(cfg):
    """Q4_K_M-style: Q4_K body, Q6_K for attn_v, ffn_down and the output head."""
    e, f = cfg["hidden"], cfg["ffn"]
    qd, kvd = cfg["n_head"] * cfg["head_dim"], cfg["n_kv_head"] * cfg["head_dim"]
    plan = [("token_embd", -1, Q4_K, (cfg["vocab"], e)), ("output", -1, Q6_K, (cfg["vocab"], e))]
    for i in range(cfg["n_layer"]):
        plan += [("attn_q", i, Q4_K, (qd, e)), ("attn_k", i, Q4_K, (kvd, e)),
                 ("attn_v", i, Q6_K, (kvd, e)), ("attn_output", i, Q4_K, (e, qd)),
                 ("ffn_gate", i, Q4_K, (f, e)), ("ffn_up", i, Q4_K, (f, e)),
                 ("ffn_down", i, Q6_K, (e, f))]
    return plan


def qbytes(ty, n, k):
    return n * k // 256 * BLOCK_BYTES[ty]


def weight_bytes_per_step(cfg):
    """Algorithmic bytes one decode step streams: every matrix but the embedding table."""
    return sum(qbytes(ty, *shape) for name, _l, ty, shape in tensor_plan(cfg) if name != "token_embd")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    """Dense bf16 tensor-core peak in TFLOP/s (burst figure: the product kernels are timed alone)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l.split(", ") for ts, l in self.lines if t0 - 0.05 <= ts <= t1 + 0.15] or \
               [l.split(", ") for _ts, l in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for nm, v in zip(names, r[5:9]):
                    if v.strip().lower().startswith("active"):
                        reasons.add(nm)
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_gpu_model(dev, torch, cfg, batch, ctx, seed, keep=None):
    """Random Q4_K_M-style weights generated and encoded on the GPU (kalosm_b200.synth)."""
    import kalosm_b200 as kb
    from kalosm_b200 import synth
    m = kb.Llama(dev, n_layer=cfg["n_layer"], hidden=cfg["hidden"], ffn=cfg["ffn"], n_head=cfg["n_head"],
                 n_kv_head=cfg["n_kv_head"], head_dim=cfg["head_dim"], vocab=cfg["vocab"], max_seq_len=ctx,
                 max_batch=batch)
    for j, (name, layer, ty, (n, k)) in enumerate(tensor_plan(cfg)):
        raw = synth.random_qweights(seed * 100003 + j, 0.02, n, k, ty, device="cuda").cpu().numpy()
        m.set_tensor(name, layer, ty, (n, k), raw)
        if keep is not None and (layer <= 0):
            keep[(name, layer)] = raw
    g = torch.Generator().manual_seed(seed + 77)
    for i in range(cfg["n_layer"] + 1):
        for nm in (("attn_norm", "ffn_norm") if i < cfg["n_layer"] else ("output_norm",)):
            w = (1.0 + 0.02 * torch.randn(cfg["hidden"], generator=g)).numpy().astype(np.float32)
            m.set_tensor(nm, i if i < cfg["n_layer"] else -1, F32, (cfg["hidden"],), w)
            if keep is not None and i in (0, cfg["n_layer"]):
                keep[(nm, i if i < cfg["n_layer"] else -1)] = w
    return m


def cpu_layer_sample(cfg, keep, threads=None, min_seconds=0.0, steps=None, warmup=0):
    """Times the oracle's decode step on a 1-layer slice: one transformer layer plus 1/32 of the
    output head rows = 1/32 of a full decode step's weight bytes. Returns seconds per slice."""
    from oracle import oracle as O
    if threads:
        O.set_threads(threads)
    vocab_slice = cfg["vocab"] // cfg["n_layer"] // 256 * 256
    m = O.Llama(1, cfg["hidden"], cfg["ffn"], cfg["n_head"], cfg["n_kv_head"], cfg["head_dim"], vocab_slice,
                64, batch=1, kv_f16=True)
    names = {"attn_q": "wq", "attn_k": "wk", "attn_v": "wv", "attn_output": "wo", "ffn_gate": "gate",
             "ffn_up": "up", "ffn_down": "down"}
    for name, layer, ty, (n, k) in tensor_plan(cfg):
        if layer == 0:
            m.set_qmatrix(names[name], 0, ty, n, k, keep[(name, 0)])
    row_bytes = cfg["hidden"] // 256
    m.set_qmatrix("token_embd", 0, Q4_K, vocab_slice, cfg["hidden"],
                  keep[("token_embd", -1)][: vocab_slice * row_bytes * 144])
    m.set_qmatrix("output", 0, Q6_K, vocab_slice, cfg["hidden"],
                  keep[("output", -1)][: vocab_slice * row_bytes * 210])
    m.set_norm("attn_norm", 0, keep[("attn_norm", 0)])
    m.set_norm("ffn_norm", 0, keep[("ffn_norm", 0)])
    m.set_norm("output_norm", -1, keep[("output_norm", -1)])
    tok = np.array([[1]], dtype=np.uint32)
    for _ in range(max(warmup, 1)):
        m.forward(tok)
    times = []
    t_start = time.perf_counter()
    while True:
        if m.pos >= 60:
            m.reset()
        t0 = time.perf_counter()
        m.forward(tok)
        times.append(time.perf_counter() - t0)
        if steps is not None and len(times) >= steps:
            break
        if steps is None and time.perf_counter() - t_start >= min_seconds and len(times) >= 3:
            break
    return times, O.num_threads()


def host_weights(cfg, seed):
    """Layer-0 and model-level tensors on the host for the CPU arm (torch CPU generator)."""
    from kalosm_b200 import synth
    import torch
    keep = {}
    for j, (name, layer, ty, (n, k)) in enumerate(tensor_plan(cfg)):
        if layer == 0:
            keep[(name, 0)] = synth.random_qweights(seed * 100003 + j, 0.02, n, k, ty).numpy()
        elif layer < 0:
            n_s = cfg["vocab"] // cfg["n_layer"] // 256 * 256
            keep[(name, -1)] = synth.random_qweights(seed * 100003 + j, 0.02, n_s, k, ty).numpy()
    g = torch.Generator().manual_seed(seed + 77)
    for key in (("attn_norm", 0), ("ffn_norm", 0), ("output_norm", -1)):
        keep[key] = (1.0 + 0.02 * torch.randn(cfg["hidden"], generator=g)).numpy().astype(np.float32)
    return keep


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    keep = host_weights(CFG, 1)
    times, threads = cpu_layer_sample(CFG, keep, steps=args.steps, warmup=args.warmup)
    total = float(np.sum(times))
    step_ms = total / len(times) * 1e3
    tok_s = 1.0 / (CFG["n_layer"] * total / len(times))
    sample = ("each step = 1 transformer layer + 1/32 of the output-head rows of the 8B-shaped model "
              "(1/32 of a decode step's weight bytes), batch 1, short context; tok/s = 1 / (32 x step time)")
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"llama3-8b-shaped Q4_K_M-style greedy decode, batch 1, prompt {PROMPT}, "
                                   f"{args.steps} decode steps per replica", "batch": 1, "prompt": PROMPT,
                       "note": "CPU arm: C++ restatement of Fusor's f32-dequantize q_mat_mul path, bounded sample"},
            "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def max_over_ranks(values, world, device):
    """Element-wise maximum of a list of floats over all ranks of the default process group
    (replicas are independent: the only exchange of a multi-GPU run is this timing reduction)."""
    if world <= 1:
        return list(values)
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def whole_job_rate(world, batch, steps, ms):
    """tok/s of the whole job: every replica decodes batch * steps tokens in the slowest rank's time."""
    return world * batch * steps / (ms / 1e3)


def gemv_roofline(kb, dev, torch, stream, reps, rows=1):
    """The dominant kernel timed alone: product of `rows` activation rows with SwiGLU epilogue over 16
    distinct gate+up matrices (16 x 66 MB, larger than L2, so every launch streams from HBM)."""
    from kalosm_b200 import synth
    f, e = CFG["ffn"], CFG["hidden"]
    mats = []
    for i in range(16):
        raw = synth.random_qweights(900 + i, 0.02, 2 * f, e, Q4_K, device="cuda").cpu().numpy()
        mats.append(kb.QMatrix.from_raw_bytes(dev, (2 * f, e), raw, Q4_K))
    x = dev.tensor(np.random.default_rng(5).standard_normal((rows, e)).astype(np.float32))
    y = dev.empty((rows, f))
    for w in mats:
        x.q_mat_mul(w, epilogue=kb.EPI_SWIGLU, out=y)
    torch.cuda.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    for _ in range(reps):
        for w in mats:
            x.q_mat_mul(w, epilogue=kb.EPI_SWIGLU, out=y)
    g1.record(stream)
    torch.cuda.synchronize()
    us = g0.elapsed_time(g1) * 1e3 / (reps * len(mats))
    kbytes = qbytes(Q4_K, 2 * f, e) + (0 if rows == 1 else 4 * rows * (e + f))
    peak, which = peaks()
    achieved = kbytes / us / 1e3
    for w in mats:
        w.free()
    name = ("qgemv1_kernel<Q4_K, SwiGLU>" if rows == 1 else
            f"pack_x16v_kernel + qgemm16s_kernel<Q4_K, SwiGLU> ({rows} rows)" if rows <= 16 else
            f"pack_x16v_kernel + qgemm16_kernel<Q4_K, SwiGLU> ({rows} rows)")
    return {"bound": "hbm", "kernel": name + " on ffn gate+up [28672 x 4096]",
            "achieved": achieved, "peak": peak, "peak_source": which, "unit": "GB/s",
            "frac": achieved / peak, "us_per_launch": us, "bytes_per_launch": kbytes, "traffic": None}


def run_gemv_only(args):
    """Only the dominant-kernel leg (1 GB on the device): the small case profiler captures use."""
    import torch
    import kalosm_b200 as kb
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = kb.Device(0, stream.cuda_stream)
    print(json.dumps({"roofline": gemv_roofline(kb, dev, torch, stream, max(1, args.gemv_reps), rows=max(1, min(32, args.batch)))}),
          flush=True)


def run_q5_only(args):
    """Products with Q5_K (the kernel that reads GGUF byte order) and Q5_0 weights (widened to Q8_0 tiles) on the FFN up shape
    [14336 x 4096] at 1, 8 and 32 activation rows: 8 distinct matrices per type (8 x 40 MB, larger than L2).
    Quant bytes are random, block scales in a realistic range; bytes per launch = the matrix + f32 rows in and out."""
    import torch
    import kalosm_b200 as kb
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = kb.Device(0, stream.cuda_stream)
    n, k = CFG["ffn"], CFG["hidden"]
    peak, which = peaks()
    out = []
    for ty, name, be, bb in ((13, "Q5_K", 256, 176), (6, "Q5_0", 32, 22)):
        mats = []
        for i in range(8):
            rng = np.random.default_rng(40 + i)
            raw = rng.integers(0, 256, size=(n * k // be, bb), dtype=np.uint8)
            d = rng.uniform(1e-4 if be == 256 else 1e-3, 2e-4 if be == 256 else 2e-3, size=(raw.shape[0], 1)).astype(np.float16)
            raw[:, 0:2] = d.view(np.uint8)
            if be == 256:
                raw[:, 2:4] = d.view(np.uint8)
            mats.append(kb.QMatrix.from_raw_bytes(dev, (n, k), raw.reshape(-1), ty))
        for rows in (1, 8, 32):
            x = dev.tensor(np.random.default_rng(5).standard_normal((rows, k)).astype(np.float32))
            y = dev.empty((rows, n))
            for w in mats:
                x.q_mat_mul(w, out=y)
            torch.cuda.synchronize()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(1, args.gemv_reps)
            g0.record(stream)
            for _ in range(reps):
                for w in mats:
                    x.q_mat_mul(w, out=y)
            g1.record(stream)
            torch.cuda.synchronize()
            us = g0.elapsed_time(g1) * 1e3 / (reps * len(mats))
            kbytes = n * k // be * bb + 4 * rows * (n + k)
            # device time of each kernel of the product (CUPTI, one extra pass over the matrices, not timed above)
            kern = {}
            prof = None
            if args.kernel_table:
                from torch.profiler import ProfilerActivity, profile
                with profile(activities=[ProfilerActivity.CUDA]) as prof:
                    for w in mats:
                        x.q_mat_mul(w, out=y)
                    torch.cuda.synchronize()
            for ev in (prof.key_averages() if prof is not None else []):
                t = getattr(ev, "device_time_total", None)
                t = ev.cuda_time_total if t is None else t
                if t > 0:
                    kern[ev.key.replace("void ", "").replace("(anonymous namespace)::", "").split("(")[0][:40]] = round(t / len(mats), 2)
            out.append({"kernel": f"product with {name} weights ({rows} rows) on [{n} x {k}]", "bound": "hbm",
                        "us_per_launch": us, "bytes_per_launch": kbytes, "achieved": kbytes / us / 1e3, "peak": peak,
                        "peak_source": which, "unit": "GB/s", "frac": kbytes / us / 1e3 / peak, "device_us_per_kernel": kern})
        for w in mats:
            w.free()
    print(json.dumps({"q5_products": out}), flush=True)


def run_attn_decode_only(args):
    """One decode-attention case (batch 32, 4096 cached keys, Llama-3-8B heads: 0.54 GB of fp16 K and V per
    launch, two distinct caches): the small case profiler captures use."""
    import torch
    import kalosm_b200 as kb
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = kb.Device(0, stream.cuda_stream)
    b, h, hkv, d, L = 32, 32, 8, 128, 4096
    ks = [dev.tensor((np.random.default_rng(3 * i).standard_normal((b, hkv, L, d)) * 0.5).astype(np.float16)) for i in range(2)]
    vs = [dev.tensor((np.random.default_rng(3 * i + 1).standard_normal((b, hkv, L, d)) * 0.5).astype(np.float16)) for i in range(2)]
    q = dev.tensor(np.random.default_rng(9).standard_normal((b, h, 1, d)).astype(np.float32))
    o = dev.empty((b, h, 1, d))
    for i in range(4):
        dev.flash_attention(q, ks[i % 2], vs[i % 2], 1.0 / np.sqrt(d), out=o)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(16):
        dev.flash_attention(q, ks[i % 2], vs[i % 2], 1.0 / np.sqrt(d), out=o)
    e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 16
    nbytes = b * L * hkv * d * 2 * 2 + 2 * b * h * d * 4
    peak, which = peaks()
    print(json.dumps({"case": "decode_attention", "batch": b, "context": L, "us": us, "algorithmic_bytes": nbytes,
                      "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak, "peak": peak, "peak_source": which}), flush=True)


def run_prefill_only(args):
    """One prefill-sized case of each tensor-core kernel (a few hundred MB on the device): the small
    case profiler captures use. Q4_K 14336 x 4096 product at M = 2048, causal attention at S = 2048."""
    import torch
    import kalosm_b200 as kb
    from kalosm_b200 import synth
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = kb.Device(0, stream.cuda_stream)
    tf_peak = tensor_peak()

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    n, k, m = 14336, 4096, 2048
    raw = synth.random_qweights(700, 0.02, n, k, Q4_K, device="cuda").cpu().numpy()
    w = kb.QMatrix.from_raw_bytes(dev, (n, k), raw, Q4_K)
    x = dev.tensor(np.random.default_rng(m).standard_normal((m, k)).astype(np.float32))
    y = dev.empty((m, n))
    us = timed(lambda: x.q_mat_mul(w, out=y), max(1, args.gemv_reps))
    tf = 2.0 * m * n * k / us / 1e6
    print(json.dumps({"case": "q_mat_mul_prefill", "type": "Q4_K", "n": n, "k": k, "m": m, "us": us, "tflops": tf,
                      "frac": tf / tf_peak[0], "peak": tf_peak[0], "peak_source": tf_peak[1], "bound": "tensor"}), flush=True)
    h, hkv, d, S = 32, 8, 128, 2048
    rng = np.random.default_rng(S)
    kt = dev.tensor((rng.standard_normal((1, hkv, S, d)) * 0.5).astype(np.float16))
    vt = dev.tensor((rng.standard_normal((1, hkv, S, d)) * 0.5).astype(np.float16))
    q = dev.tensor(rng.standard_normal((1, h, S, d)).astype(np.float32))
    o = dev.empty((1, h, S, d))
    us = timed(lambda: dev.flash_attention(q, kt, vt, 1.0 / np.sqrt(d), mask_kind=kb.MASK_CAUSAL, out=o), max(1, args.gemv_reps))
    tf = 2.0 * S * (S + 1) * d * h / us / 1e6
    print(json.dumps({"case": "prefill_attention", "seq": S, "us": us, "tflops": tf, "frac": tf / tf_peak[0],
                      "peak": tf_peak[0], "peak_source": tf_peak[1], "bound": "tensor"}), flush=True)


CFG70 = dict(n_layer=80, hidden=8192, ffn=28672, n_head=64, n_kv_head=8, head_dim=128, vocab=128256)


def _tp_measure(torch, dist, kb, dev, stream, m, comm, cfg, rank, world, local, batch, steps, warmup, prompt_len,
                local_bytes, use_nccl, barrier):
    """One batch size of the tensor-parallel leg on an already loaded model."""
    e = cfg["hidden"]
    m.reset()
    prompt = np.random.default_rng(0).integers(0, cfg["vocab"], size=(batch, prompt_len), dtype=np.uint32)
    m.forward(prompt, want_logits=False)
    m.reset()
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(stream)
    _, nxt = m.forward(prompt, want_logits=False)
    p1.record(stream)
    barrier()
    ms_prefill = p0.elapsed_time(p1)
    m.generate_greedy(nxt, warmup)
    last = m.generate_greedy(nxt, 1)[:, -1]
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = dev.launch_count
    t0 = time.time()
    e0.record(stream)
    toks = m.generate_greedy(last, steps)
    e1.record(stream)
    barrier()
    t1 = time.time()
    launches = dev.launch_count - launches0
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t0, t1)
    # the all-reduce alone: the payload of one decode step's sums, back to back
    ar_us = None
    if comm is not None:
        buf = dev.tensor(np.zeros((batch, e), np.float32))
        for _ in range(20):
            comm.all_reduce_sum(buf)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for _ in range(2 * cfg["n_layer"]):
            comm.all_reduce_sum(buf)
        a1.record(stream)
        barrier()
        ar_us = a0.elapsed_time(a1) * 1e3 / (2 * cfg["n_layer"])
    same = True
    if world > 1:
        parts = [None] * world
        dist.all_gather_object(parts, toks.tolist())
        same = all(p == parts[0] for p in parts)
    ms, ms_prefill = max_over_ranks([ms, ms_prefill], world, "cuda")
    status = dev.status()
    out = None
    if rank == 0:
        peak, which = peaks()
        kv = 2 * cfg["n_layer"] * (cfg["n_kv_head"] // world) * cfg["head_dim"] * 2 * (prompt_len + warmup + steps // 2) * batch
        gbs = (local_bytes + kv) / (ms / steps / 1e3) / 1e9
        out = {
            "metric": "Llama-3-70B-shaped Q4_K greedy decode tok/s, tensor parallel", "value": batch * steps / ms * 1e3,
            "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
            "higher_is_better": True, "scaling": "strong", "data": "synthetic (seeded N(0, 0.02) weights as Q4_K blocks)",
            "config": {"workload": f"llama3-70b-shaped all-Q4_K greedy decode, TP={world}, batch {batch}, prompt "
                                   f"{prompt_len}, {steps} steps" + ("" if cfg["n_layer"] == 80 else
                                                                     f" (REDUCED: {cfg['n_layer']} layers)"),
                       "parallelism": f"tp{world}",
                       "step": ("kernel per operation, NCCL all-reduce" if use_nccl or world == 1 or batch > 1 else
                                "one persistent kernel per rank, sums over NVLink peer memory inside it")},
            "gpu_launches": int(launches),
            "per_gpu": {"weight_bytes_per_step": local_bytes, "kv_bytes_per_step": kv, "achieved_gbs": gbs,
                        "peak": peak, "peak_source": which, "frac": gbs / peak},
            "all_reduce": None if ar_us is None else {"per_step": 2 * cfg["n_layer"], "payload_bytes": batch * e * 4,
                                                      "us_each_back_to_back": ar_us,
                                                      "ms_per_step_alone": ar_us * 2 * cfg["n_layer"] / 1e3},
            "prefill": {"tokens": batch * prompt_len, "ms": ms_prefill, "tok_s": batch * prompt_len / ms_prefill * 1e3},
            "ranks_agree_on_tokens": same, "device_status": status, "clocks": clocks}
    return out


def tensor_parallel_leg(args, torch, dist, kb, dev, stream, rank, world, local, batches, steps, warmup, prompt_len,
                        n_layer=80, use_nccl=False):
    """Llama-3-70B-shaped, all Q4_K, greedy decode with the model split over the ranks (tensor
    parallel: every rank streams 1 / N of the weights per step; two sums over the ranks per layer).
    One model, measured once per entry of `batches`. Every rank calls this; rank 0 gets the list of
    result dictionaries (one per batch), the others None."""
    from kalosm_b200 import synth, tp
    comm = None
    if world > 1:
        uid = [kb.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, 0)
        comm = kb.Comm(dev, world, rank, uid[0])
        if not use_nccl:
            # the decode step sums its partial rows over NVLink peer memory inside the persistent kernel
            def gather(obj):
                parts = [None] * world
                dist.all_gather_object(parts, obj)
                return parts
            comm.enable_peer_exchange(CFG70["hidden"], gather)
    cfg = dict(CFG70, n_layer=n_layer)
    ctx = prompt_len + 2 * (steps + warmup) + 64
    m = kb.Llama(dev, n_layer=cfg["n_layer"], hidden=cfg["hidden"], ffn=cfg["ffn"], n_head=cfg["n_head"],
                 n_kv_head=cfg["n_kv_head"], head_dim=cfg["head_dim"], vocab=cfg["vocab"], max_seq_len=ctx,
                 max_batch=max(batches), comm=comm)
    e, f = cfg["hidden"], cfg["ffn"]
    qd, kvd = cfg["n_head"] * cfg["head_dim"], cfg["n_kv_head"] * cfg["head_dim"]
    plan = [("token_embd", -1, (cfg["vocab"], e)), ("output", -1, (cfg["vocab"], e))]
    for i in range(cfg["n_layer"]):
        plan += [("attn_q", i, (qd, e)), ("attn_k", i, (kvd, e)), ("attn_v", i, (kvd, e)), ("attn_output", i, (e, qd)),
                 ("ffn_gate", i, (f, e)), ("ffn_up", i, (f, e)), ("ffn_down", i, (e, f))]
    local_bytes = 0
    for j, (name, layer, (n, k)) in enumerate(plan):
        # this rank's shard is generated directly (random weights: no whole matrix to cut)
        if name in tp.ROW_SPLIT:
            n //= world
        elif name in tp.COL_SPLIT:
            k //= world
        seed = 1000003 * (rank if name != "token_embd" else 0) + j
        raw = synth.random_qweights(seed, 0.02, n, k, Q4_K, device="cuda").cpu().numpy()
        m.set_tensor(name, layer, Q4_K, (n, k), raw)
        if name != "token_embd":
            local_bytes += raw.size
    g = torch.Generator().manual_seed(77)
    for i in range(cfg["n_layer"] + 1):
        for nm in (("attn_norm", "ffn_norm") if i < cfg["n_layer"] else ("output_norm",)):
            w = (1.0 + 0.02 * torch.randn(e, generator=g)).numpy().astype(np.float32)
            m.set_tensor(nm, i if i < cfg["n_layer"] else -1, F32, (e,), w)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    results = []
    for batch in batches:
        results.append(_tp_measure(torch, dist, kb, dev, stream, m, comm, cfg, rank, world, local, batch, steps,
                                   warmup, prompt_len, local_bytes, use_nccl, barrier))
    out = results if rank == 0 else None
    m.free()
    if comm is not None:
        comm.destroy()
    return out


def run_tensor_parallel(args):
    """`--tp`: only the tensor-parallel leg, one JSON line from rank 0 (not the bench line: that is the
    8B replica metric). Exits non-zero when a kernel recorded a time-out or the ranks disagree."""
    import torch
    import torch.distributed as dist
    import kalosm_b200 as kb
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = kb.Device(local, stream.cuda_stream)
    outs = tensor_parallel_leg(args, torch, dist, kb, dev, stream, rank, world, local, [args.batch], args.steps,
                               max(args.warmup, 3), args.tp_prompt, n_layer=args.layers if args.layers != 32 else 80,
                               use_nccl=args.tp_nccl)
    bad = 0
    if rank == 0:
        out = outs[0]
        print(json.dumps(out), flush=True)
        bad = int(out["device_status"] != 0 or not out["ranks_agree_on_tokens"])
    if world > 1:
        dist.destroy_process_group()
    if bad:
        sys.exit(3)


def run_sweep(args):
    """Per-kernel table of the other configurations of the path, one JSON line each (not the bench
    line): single-row and small-batch quantised products over the Llama-3-8B matrix shapes, and
    decode attention over an fp16 cache. Every case rotates over enough distinct buffers to exceed
    the L2 (126 MB) several times."""
    import torch
    import kalosm_b200 as kb
    from kalosm_b200 import synth
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = kb.Device(0, stream.cuda_stream)
    peak, which = peaks()

    def timed(fn, n):
        for i in range(n):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        reps = 4
        for _ in range(reps):
            for i in range(n):
                fn(i)
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * n)

    types = {"Q4_0": Q4_0, "Q8_0": Q8_0, "Q4_K": Q4_K, "Q6_K": Q6_K}
    cases = [("Q4_0", 4096, 4096)] + [(t, n, k) for t in ("Q4_K", "Q8_0")
                                       for (n, k) in ((4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336))] + \
            [("Q6_K", 128256, 4096)]
    for tname, n, k in cases:
        ty = types[tname]
        wbytes = qbytes(ty, n, k)
        copies = max(2, min(24, int(600e6 // wbytes) + 1))
        mats = []
        for i in range(copies):
            raw = synth.random_qweights(700 + i, 0.02, n, k, ty, device="cuda").cpu().numpy()
            mats.append(kb.QMatrix.from_raw_bytes(dev, (n, k), raw, ty))
        for m in (1, 8, 32):
            x = dev.tensor(np.random.default_rng(m).standard_normal((m, k)).astype(np.float32))
            y = dev.empty((m, n))
            us = timed(lambda i: x.q_mat_mul(mats[i % copies], out=y), copies)
            nbytes = wbytes + 4 * m * (k + n)
            print(json.dumps({"case": "q_mat_mul", "type": tname, "n": n, "k": k, "m": m, "us": us,
                              "algorithmic_bytes": nbytes, "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak,
                              "peak": peak, "peak_source": which, "distinct_weight_buffers": copies}), flush=True)
        if tname != "Q4_0" and n <= 14336:
            # prefill product (tcgen05): bound by the tensor cores, not HBM
            tf_peak = tensor_peak()
            for m in (512, 2048):
                x = dev.tensor(np.random.default_rng(m).standard_normal((m, k)).astype(np.float32))
                y = dev.empty((m, n))
                us = timed(lambda i: x.q_mat_mul(mats[i % copies], out=y), copies)
                tf = 2.0 * m * n * k / us / 1e6
                print(json.dumps({"case": "q_mat_mul_prefill", "type": tname, "n": n, "k": k, "m": m, "us": us,
                                  "tflops": tf, "frac": tf / tf_peak[0], "peak": tf_peak[0], "peak_source": tf_peak[1],
                                  "bound": "tensor"}), flush=True)
        for w in mats:
            w.free()
    # decode attention: one query position per sequence against L cached keys (fp16), Llama-3-8B heads
    h, hkv, d = 32, 8, 128
    for L in (1024, 4096, 16384):
        for b in (1, 8, 32):
            kv_bytes = b * L * hkv * d * 2 * 2
            copies = max(2, min(16, int(400e6 // kv_bytes) + 1))
            if copies * kv_bytes > 40e9:
                continue
            ks = [dev.tensor((np.random.default_rng(3 * i).standard_normal((b, hkv, L, d)) * 0.5).astype(np.float16))
                  for i in range(copies)]
            vs = [dev.tensor((np.random.default_rng(3 * i + 1).standard_normal((b, hkv, L, d)) * 0.5).astype(np.float16))
                  for i in range(copies)]
            q = dev.tensor(np.random.default_rng(9).standard_normal((b, h, 1, d)).astype(np.float32))
            o = dev.empty((b, h, 1, d))
            us = timed(lambda i: dev.flash_attention(q, ks[i % copies], vs[i % copies], 1.0 / np.sqrt(d), out=o), copies)
            nbytes = kv_bytes + 2 * b * h * d * 4
            print(json.dumps({"case": "decode_attention", "batch": b, "context": L, "us": us, "algorithmic_bytes": nbytes,
                              "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak, "peak": peak,
                              "peak_source": which, "distinct_kv_buffers": copies}), flush=True)
            del ks, vs
    # prefill attention: causal, Llama-3-8B heads, fp16 cache; causal-effective flops 2 S (S + 1) D Hq
    tf_peak = tensor_peak()
    for S in (512, 2048, 8192):
        rng = np.random.default_rng(S)
        kt = dev.tensor((rng.standard_normal((1, hkv, S, d)) * 0.5).astype(np.float16))
        vt = dev.tensor((rng.standard_normal((1, hkv, S, d)) * 0.5).astype(np.float16))
        q = dev.tensor(rng.standard_normal((1, h, S, d)).astype(np.float32))
        o = dev.empty((1, h, S, d))
        us = timed(lambda i: dev.flash_attention(q, kt, vt, 1.0 / np.sqrt(d), mask_kind=kb.MASK_CAUSAL, out=o), 4)
        tf = 2.0 * S * (S + 1) * d * h / us / 1e6
        print(json.dumps({"case": "prefill_attention", "seq": S, "us": us, "tflops": tf, "frac": tf / tf_peak[0],
                          "peak": tf_peak[0], "peak_source": tf_peak[1], "bound": "tensor"}), flush=True)
        del kt, vt, q


def run_ours(args):
    # stdout carries exactly one line, the JSON record: whatever libraries print while they start
    # (NCCL announces its version on stdout) goes to stderr instead
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    import torch
    import torch.distributed as dist
    import kalosm_b200 as kb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = kb.Device(local, stream.cuda_stream)
    batch, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
    ctx = PROMPT + 2 * (steps + warmup) + 64
    keep = {} if rank == 0 else None
    model = build_gpu_model(dev, torch, CFG, batch, ctx, seed=1 + rank, keep=keep)
    rng = np.random.default_rng(rank)
    prompt = rng.integers(0, CFG["vocab"], size=(batch, PROMPT), dtype=np.uint32)
    model.forward(prompt, want_logits=False)
    # prefill of the prompt (host ids in, next token out), timed once warm; reported beside the
    # decode metric, not part of it
    model.reset()
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(stream)
    _, nxt = model.forward(prompt, want_logits=False)
    p1.record(stream)
    torch.cuda.synchronize()
    ms_prefill = p0.elapsed_time(p1)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident loop (value) ----------------------------------------------------
    # The timed region is EXACTLY `steps` decode steps, bracketed by barrier + synchronize. It is
    # repeated (the KV caches rewound to the same position each time, so every repetition covers
    # the same contexts) until about a second of GPU time has been measured; the reported time is
    # the median repetition of the per-repetition maximum over ranks.
    model.generate_greedy(nxt, warmup)
    last = model.generate_greedy(nxt, 1)[:, -1]
    start_pos = model.position
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)

    def bail_if_any(reason):
        """Ends the job on every rank (non-zero exit) when any rank has a reason to; a rank that
        left alone would strand the others in the next barrier."""
        flag = max_over_ranks([1.0 if reason else 0.0], world, "cuda")[0]
        if reason:
            sys.stderr.write(f"bench (rank {rank}): {reason}\n")
        if flag:
            if world > 1:
                dist.destroy_process_group()
            sys.exit(3)

    def timed_generate():
        model.truncate(start_pos)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = dev.launch_count
        e0.record(stream)
        out = model.generate_greedy(last, steps)
        e1.record(stream)
        barrier()
        return max_over_ranks([e0.elapsed_time(e1)], world, "cuda")[0], dev.launch_count - n0, out

    t0 = time.time()
    first_ms, launches, toks = timed_generate()
    repeats = int(min(32, max(3, np.ceil(1000.0 / max(first_ms, 1e-3)))))
    rep_ms = [first_ms]
    differ = False
    for _ in range(repeats - 1):
        ms_i, launches, toks_i = timed_generate()
        rep_ms.append(ms_i)
        differ = differ or not np.array_equal(toks_i, toks)
    t1 = time.time()
    ms = float(np.median(rep_ms))
    clocks = sampler.stop(t0, t1)
    status = dev.status()
    bail_if_any(f"device status {status} after the timed region (a wait inside a kernel gave up)" if status else
                "two repetitions of the same greedy decode gave different tokens" if differ else None)

    # ---- end to end: one fb200_llama_forward per step, ids through pinned host memory -------
    pinned = torch.empty(batch, dtype=torch.int32).pin_memory()
    tok = pinned.numpy().view(np.uint32)

    def timed_forward_steps():
        model.truncate(start_pos)
        tok[:] = last
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(steps):
            _, n2 = model.forward(tok.reshape(batch, 1), want_logits=False)
            tok[:] = n2
        f1.record(stream)
        barrier()
        return max_over_ranks([f0.elapsed_time(f1)], world, "cuda")[0]

    model.truncate(start_pos)
    tok[:] = last
    for _ in range(3):
        _, n2 = model.forward(tok.reshape(batch, 1), want_logits=False)
        tok[:] = n2
    e2e_ms = [timed_forward_steps() for _ in range(repeats)]
    ms_e2e = float(np.median(e2e_ms))
    bail_if_any(None if np.array_equal(tok, toks[:, -1]) else
                "stepping through forward() and the device-resident loop gave different tokens")

    # ---- optional: device time per kernel of the decode step (CUPTI through torch.profiler; the
    # profiled steps are extra steps after the timed regions, never part of a reported number)
    kernel_table = None
    if args.kernel_table and rank == 0:
        from torch.profiler import ProfilerActivity, profile
        model.truncate(start_pos)
        n_prof = 8
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            model.generate_greedy(last, n_prof)
            torch.cuda.synchronize()
        rows = []
        for ev in prof.key_averages():
            t = getattr(ev, "device_time_total", None)
            t = ev.cuda_time_total if t is None else t
            if t > 0:
                rows.append({"kernel": ev.key[:120], "us_per_step": t / n_prof, "launches_per_step": ev.count / n_prof})
        rows.sort(key=lambda r: -r["us_per_step"])
        kernel_table = {"steps": n_prof, "device_us_per_step": sum(r["us_per_step"] for r in rows), "kernels": rows[:24]}

    # ---- the stand-alone single-row product (the kernel behind fb200_q_mat_mul at M = 1) ----
    roof_gemv = gemv_roofline(kb, dev, torch, stream, 8) if rank == 0 else None

    # ---- tensor parallel (only when the job has more than one GPU): the 70B-shaped model split over
    # the same ranks, reported under its own key; `value` stays the replica metric
    tp_leg = None
    if world > 1 and not args.no_tp:
        model.free()
        model = None
        try:
            tp_leg = tensor_parallel_leg(args, torch, dist, kb, dev, stream, rank, world, local, [1, 8], 128, 3,
                                         args.tp_prompt)
        except kb.FusorError as exc:  # every rank runs the same calls, so a refusal is raised on all of them
            tp_leg = [{"error": str(exc)}]
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    tok_s = whole_job_rate(world, batch, steps, ms)
    tok_s_e2e = whole_job_rate(world, batch, steps, ms_e2e)
    wb = weight_bytes_per_step(CFG)
    kv = 2 * CFG["n_layer"] * CFG["n_kv_head"] * CFG["head_dim"] * 2 * (PROMPT + warmup + 1 + steps // 2) * batch
    peak, which = peaks()
    step_gbs = (wb + kv) / (ms / steps / 1e3) / 1e9
    # dominant kernel: the fused decode-step kernel; the timed region above is `launches` launches
    # of it (one per 256 steps) and nothing else, timed with CUDA events on its stream
    per_launch = (wb + kv) * steps / max(1, launches)
    roof = {"bound": "hbm",
            "kernel": "fused_step_kernel: whole decode steps (embedding, 32 x [q/k/v, attention, o, gate/up + SwiGLU, "
                      "down + residuals], output head + argmax) in one persistent cooperative launch",
            "achieved": step_gbs, "peak": peak, "peak_source": which, "unit": "GB/s", "frac": step_gbs / peak,
            "us_per_launch": ms * 1e3 / max(1, launches), "bytes_per_launch": per_launch,
            "traffic": per_launch * FUSED_TRAFFIC_PER_BYTE if CFG["n_layer"] == 32 else None}
    # CPU baseline beside it (rank 0, N = 1 only): bounded sample of the oracle's decode step
    cpu = None
    if world == 1 and not args.no_cpu:
        times, threads = cpu_layer_sample(CFG, keep, min_seconds=10.0)
        per_tok = CFG["n_layer"] * float(np.median(times))
        cpu = {"value": 1.0 / per_tok, "unit": "tok/s", "cores": threads, "kind": "port",
               "sample": f"{len(times)} timed decode steps of a 1-layer slice (1 transformer layer + 1/32 of the "
                         "output-head rows = 1/32 of a step's weight bytes), scaled x32; C++ restatement of "
                         "Fusor's CPU q_mat_mul path"}
    line = {"metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 x int8 -> s32 tensor-core dot products of GGUF quants and 4 x 7-bit activation limbs, "
                     "f32 scales and accumulation",
            "data": "synthetic (seeded N(0, 0.02) weights encoded as Q4_K / Q6_K blocks on the GPU, uniform-random "
                    "token ids)",
            "config": {"workload": f"llama3-8b-shaped Q4_K_M-style greedy decode, batch {batch}, prompt {PROMPT}, "
                                   f"{steps} decode steps per replica" +
                                   ("" if CFG["n_layer"] == 32 else f" (PROFILING CASE: {CFG['n_layer']} layers)"),
                       "batch": batch, "prompt": PROMPT,
                       "l2": "4.9 GB of weights per step, far larger than L2",
                       "parallelism": "replicas only" if world > 1 else "single GPU"},
            "e2e": {"value": tok_s_e2e, "unit": "tok/s", "h2d_bytes_per_step": 4 * batch,
                    "d2h_bytes_per_step": 4 * batch, "ms_per_step": ms_e2e / steps},
            "gpu_launches": int(launches), "device_status": status, "clocks": clocks,
            "timing": {"repeats": repeats, "ms_per_repeat": rep_ms, "reported": "median repetition, each the maximum over ranks",
                       "e2e_ms_per_repeat": e2e_ms},
            "roofline": roof, "roofline_gemv_alone": roof_gemv,
            "prefill": {"tokens": batch * PROMPT, "ms": ms_prefill, "tok_s": batch * PROMPT / ms_prefill * 1e3,
                        "kernel": "quantised products on tcgen05 tensor cores (fp16 operands, fp32 TMEM accumulator)"},
            "step_hbm": {"bytes_per_step": wb + kv, "achieved_gbs": step_gbs, "frac_of_peak": step_gbs / peak,
                         "peak_source": which},
            "cpu_baseline": cpu}
    if kernel_table is not None:
        line["kernel_table"] = kernel_table
    if tp_leg is not None:
        line["tensor_parallel"] = {"tp": world, "model": "llama3-70b-shaped, all Q4_K, prompt %d, 128 greedy steps" % args.tp_prompt,
                                   "by_batch": tp_leg}
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--layers", type=int, default=CFG["n_layer"],
                    help="decoder layers of the model (fewer than 32 only for profiler captures; not a bench value)")
    ap.add_argument("--gemv-only", action="store_true", help="run only the dominant-kernel leg")
    ap.add_argument("--q5-only", action="store_true", help="time the Q5_K / Q5_0 products at 1, 8 and 32 rows")
    ap.add_argument("--attn-decode-only", action="store_true",
                    help="run only one decode-attention case (batch 32, 4096 keys): the small case of profiler captures")
    ap.add_argument("--prefill-only", action="store_true",
                    help="run one prefill product and one prefill attention (profiling case)")
    ap.add_argument("--tp", action="store_true",
                    help="70B-shaped model split over the ranks (tensor parallel) instead of 8B replicas")
    ap.add_argument("--tp-prompt", type=int, default=2048)
    ap.add_argument("--tp-nccl", action="store_true", help="with --tp: keep the decode step on NCCL all-reduces")
    ap.add_argument("--no-tp", action="store_true", help="with --gpus N > 1: skip the tensor-parallel leg after the replicas")
    ap.add_argument("--gemv-reps", type=int, default=8)
    ap.add_argument("--kernel-table", action="store_true",
                    help="add the device time per kernel of 8 extra decode steps (torch.profiler) as `kernel_table`")
    ap.add_argument("--sweep", action="store_true",
                    help="per-kernel table over the other product shapes and decode attention (several JSON lines)")
    args = ap.parse_args()
    CFG["n_layer"] = args.layers
    if args.impl == "reference":
        run_reference(args)
    elif args.sweep:
        run_sweep(args)
    elif args.gemv_only:
        run_gemv_only(args)
    elif args.q5_only:
        run_q5_only(args)
    elif args.attn_decode_only:
        run_attn_decode_only(args)
    elif args.prefill_only:
        run_prefill_only(args)
    elif args.tp:
        run_tensor_parallel(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
