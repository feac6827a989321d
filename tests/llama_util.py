"""Builds the same random-weight Llama model on the GPU (kalosm_b200) and in the oracle."""
import numpy as np

import kalosm_b200 as kb
from kalosm_b200 import tp
from oracle import oracle as O


def tiny_cfg():
    return dict(n_layer=2, hidden=256, ffn=512, n_head=4, n_kv_head=2, head_dim=64, vocab=1024, ctx=64)


def tp_cfg(world=2):
    """Smallest shapes that still cut on 256-element blocks over `world` ranks: every rank gets four
    query heads, one KV head and 512 FFN columns (attn_output K = 256 per rank, ffn_down K = 512)."""
    return dict(n_layer=2, hidden=512, ffn=512 * world, n_head=4 * world, n_kv_head=world, head_dim=64,
                vocab=1024, ctx=96)


def llama3_8b_cfg(ctx=1024):
    return dict(n_layer=32, hidden=4096, ffn=14336, n_head=32, n_kv_head=8, head_dim=128,
                vocab=128256, ctx=ctx)


def tensor_plan(cfg):
    """(name, which_layer, ggml type, [N, K]) in Q4_K_M style: Q4_K body, Q6_K for attn_v,
    ffn_down and the output head."""
    e, f = cfg["hidden"], cfg["ffn"]
    qd, kvd = cfg["n_head"] * cfg["head_dim"], cfg["n_kv_head"] * cfg["head_dim"]
    plan = [("token_embd", -1, O.Q4K, (cfg["vocab"], e)), ("output", -1, O.Q6K, (cfg["vocab"], e))]
    for i in range(cfg["n_layer"]):
        plan += [("attn_q", i, O.Q4K, (qd, e)), ("attn_k", i, O.Q4K, (kvd, e)),
                 ("attn_v", i, O.Q6K, (kvd, e)), ("attn_output", i, O.Q4K, (e, qd)),
                 ("ffn_gate", i, O.Q4K, (f, e)), ("ffn_up", i, O.Q4K, (f, e)),
                 ("ffn_down", i, O.Q6K, (e, f))]
    return plan


ORACLE_NAMES = {"token_embd": "token_embd", "output": "output", "attn_q": "wq", "attn_k": "wk",
                "attn_v": "wv", "attn_output": "wo", "ffn_gate": "gate", "ffn_up": "up",
                "ffn_down": "down"}


def build_models(dev, cfg, batch=1, seed=0, want_cpu=True, sigma=0.02, comm=None, tied=False, types=None):
    """With `comm` the GPU model is this rank's shard of the same (whole) seeded weights. With
    `tied` the GPU model gets no output head and must fall back to the embedding matrix
    (models/kalosm-llama/src/raw/mod.rs:480-486), as the oracle does when it has no head.
    `types` overrides the block type per tensor name (Q5_0 / Q5_K come from the tests' own encoders)."""
    gpu = kb.Llama(dev, n_layer=cfg["n_layer"], hidden=cfg["hidden"], ffn=cfg["ffn"],
                   n_head=cfg["n_head"], n_kv_head=cfg["n_kv_head"], head_dim=cfg["head_dim"],
                   vocab=cfg["vocab"], max_seq_len=cfg["ctx"], max_batch=batch, comm=comm)
    rank, size = (comm.rank, comm.size) if comm is not None else (0, 1)
    cpu = None
    if want_cpu:
        cpu = O.Llama(cfg["n_layer"], cfg["hidden"], cfg["ffn"], cfg["n_head"], cfg["n_kv_head"],
                      cfg["head_dim"], cfg["vocab"], cfg["ctx"], batch=batch, kv_f16=True)
    for j, (name, layer, ty, (n, k)) in enumerate(tensor_plan(cfg)):
        ty = (types or {}).get(name, ty)
        if ty in (O.Q5_0, O.Q5K):
            import fixtures
            raw = fixtures.random_q5_weights(seed * 100003 + j, sigma, n, k, ty)
        else:
            raw = O.random_qweights(seed * 100003 + j, sigma, n * k, ty)
        if tied and name == "output":
            continue
        part, part_shape = tp.shard(name, raw, ty, (n, k), rank, size)
        gpu.set_tensor(name, layer, ty, part_shape, part)
        if cpu:
            cpu.set_qmatrix(ORACLE_NAMES[name], layer, ty, n, k, raw)
    rng = np.random.default_rng(seed + 77)
    for i in range(cfg["n_layer"] + 1):
        for nm in (("attn_norm", "ffn_norm") if i < cfg["n_layer"] else ("output_norm",)):
            w = (1.0 + 0.02 * rng.standard_normal(cfg["hidden"])).astype(np.float32)
            gpu.set_tensor(nm, i if i < cfg["n_layer"] else -1, kb.F32, (cfg["hidden"],), w)
            if cpu:
                cpu.set_norm(nm, i if i < cfg["n_layer"] else -1, w)
    return gpu, cpu


def write_checkpoint(path, cfg, seed=0, sigma=0.02):
    """The same seeded model as build_models, as a GGUF file (kalosm_b200.gguf.write_gguf)."""
    from kalosm_b200 import gguf
    md = {"general.architecture": (gguf.STRING, "llama"), "llama.block_count": (gguf.U32, cfg["n_layer"]),
          "llama.embedding_length": (gguf.U32, cfg["hidden"]), "llama.feed_forward_length": (gguf.U32, cfg["ffn"]),
          "llama.attention.head_count": (gguf.U32, cfg["n_head"]),
          "llama.attention.head_count_kv": (gguf.U32, cfg["n_kv_head"]),
          "llama.attention.key_length": (gguf.U32, cfg["head_dim"]),
          "llama.context_length": (gguf.U32, cfg["ctx"]),
          "llama.attention.layer_norm_rms_epsilon": (gguf.F32, 1e-5), "llama.rope.freq_base": (gguf.F32, 500000.0)}
    tensors = []
    for j, (name, layer, ty, (n, k)) in enumerate(tensor_plan(cfg)):
        full = f"{name}.weight" if layer < 0 else f"blk.{layer}.{name}.weight"
        tensors.append((full, (n, k), ty, O.random_qweights(seed * 100003 + j, sigma, n * k, ty)))
    rng = np.random.default_rng(seed + 77)
    for i in range(cfg["n_layer"] + 1):
        for nm in (("attn_norm", "ffn_norm") if i < cfg["n_layer"] else ("output_norm",)):
            w = (1.0 + 0.02 * rng.standard_normal(cfg["hidden"])).astype(np.float32)
            full = f"blk.{i}.{nm}.weight" if i < cfg["n_layer"] else "output_norm.weight"
            tensors.append((full, (cfg["hidden"],), kb.F32, w))
    gguf.write_gguf(path, md, tensors)
