"""Shards of GGUF-quantised weight matrices for tensor parallelism.

A weight is raw GGUF blocks of a row-major [N, K] matrix, blocks contiguous along K. Splitting N
is a byte sub-range; splitting K gathers whole block columns (K / size must be a multiple of the
block size). Which tensor splits which way (one all-reduce per pair):
  attn_q / attn_k / attn_v, ffn_gate / ffn_up, output : rows
  attn_output, ffn_down                               : K columns
  token_embd, norms                                   : replicated
"""
import numpy as np

# (elements, bytes) per block, fusor-ml/gguf/src/lib.rs:99-121
BLOCK = {0: (1, 4), 1: (1, 2), 2: (32, 18), 6: (32, 22), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}

ROW_SPLIT = ("attn_q", "attn_k", "attn_v", "ffn_gate", "ffn_up", "output")
COL_SPLIT = ("attn_output", "ffn_down")


def shard_rows(raw, ggml_type, n, k, rank, size):
    """Rows [rank * n / size, (rank + 1) * n / size) of an [n, k] matrix -> (bytes, (n / size, k))."""
    bs, bb = BLOCK[ggml_type]
    if n % size or k % bs:
        raise ValueError(f"{n} rows are not divisible by {size} ranks")
    raw8 = np.ascontiguousarray(raw).view(np.uint8).reshape(n, k // bs * bb)
    rows = n // size
    return np.ascontiguousarray(raw8[rank * rows:(rank + 1) * rows]).reshape(-1), (rows, k)


def shard_cols(raw, ggml_type, n, k, rank, size):
    """Columns [rank * k / size, (rank + 1) * k / size) of an [n, k] matrix -> (bytes, (n, k / size))."""
    bs, bb = BLOCK[ggml_type]
    if k % (size * bs):
        raise ValueError(f"K = {k} over {size} ranks does not cut on blocks of {bs}")
    raw8 = np.ascontiguousarray(raw).view(np.uint8).reshape(n, k // bs, bb)
    cols = k // bs // size
    return np.ascontiguousarray(raw8[:, rank * cols:(rank + 1) * cols]).reshape(-1), (n, k // size)


def shard(name, raw, ggml_type, shape, rank, size):
    """This rank's part of tensor `name` (blk.{i}.<name>.weight) -> (bytes, shape)."""
    if size == 1 or name not in ROW_SPLIT + COL_SPLIT:
        return np.ascontiguousarray(raw).view(np.uint8).reshape(-1), tuple(shape)
    n, k = int(shape[0]), int(shape[1])
    return (shard_rows if name in ROW_SPLIT else shard_cols)(raw, ggml_type, n, k, rank, size)
