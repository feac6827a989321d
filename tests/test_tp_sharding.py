"""Host logic of tensor parallelism: shards of quantised matrices and the sum over ranks, checked
with the oracle on the CPU; the exchange itself by two gloo ranks."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import fixtures as F
from kalosm_b200 import tp
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("ty", [O.Q4_0, O.Q8_0, O.Q4K, O.Q6K])
@pytest.mark.parametrize("size", [2, 4])
def test_row_and_column_shards_reassemble_the_product(ty, size):
    n, k, m = 64, 2048, 3
    raw = O.random_qweights(11, 0.02, n * k, ty)
    x = O.normal(12, 1.0, m * k).reshape(m, k)
    full = O.q_mat_mul(x, raw, ty, n, k)
    rows, cols = [], np.zeros_like(full)
    for r in range(size):
        part, (pn, pk) = tp.shard_rows(raw, ty, n, k, r, size)
        assert (pn, pk) == (n // size, k) and part.size == raw.size // size
        rows.append(O.q_mat_mul(x, part, ty, pn, pk))
        part, (pn, pk) = tp.shard_cols(raw, ty, n, k, r, size)
        assert (pn, pk) == (n, k // size) and part.size == raw.size // size
        cols += O.q_mat_mul(np.ascontiguousarray(x[:, r * pk:(r + 1) * pk]), part, ty, pn, pk)
    assert np.array_equal(np.concatenate(rows, axis=1), full)  # rows are independent: bit-exact
    assert F.rel_l2(cols, full) < 1e-5                          # another summation order


def test_shard_rules():
    raw = O.random_qweights(1, 0.02, 8 * 512, O.Q4K)
    with pytest.raises(ValueError):
        tp.shard_cols(raw, O.Q4K, 8, 512, 0, 4)  # 128 columns per rank < one 256-element block
    with pytest.raises(ValueError):
        tp.shard_rows(raw, O.Q4K, 8, 512, 0, 3)
    part, shape = tp.shard("token_embd", raw, O.Q4K, (8, 512), 1, 2)  # replicated
    assert shape == (8, 512) and np.array_equal(part, raw)
    assert tp.shard("attn_q", raw, O.Q4K, (8, 512), 1, 2)[1] == (4, 512)
    assert tp.shard("ffn_down", raw, O.Q4K, (8, 512), 1, 2)[1] == (8, 256)


RANK_SCRIPT = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
    import numpy as np, torch, torch.distributed as dist
    from kalosm_b200 import tp
    from oracle import oracle as O
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    # one FFN of a layer, split the tensor-parallel way: gate/up by rows, down by columns, one sum
    e, f, m, ty = 256, 1024, 2, O.Q4K
    g, u, d = (O.random_qweights(s, 0.02, f * e, ty) for s in (1, 2, 3))
    x = O.normal(4, 1.0, m * e).reshape(m, e)
    want = O.q_mat_mul(O.silu_mul(O.q_mat_mul(x, g, ty, f, e), O.q_mat_mul(x, u, ty, f, e)), d, ty, e, f)
    gp, gs = tp.shard("ffn_gate", g, ty, (f, e), rank, world)
    up, us = tp.shard("ffn_up", u, ty, (f, e), rank, world)
    dp, ds = tp.shard("ffn_down", d, ty, (e, f), rank, world)
    h = O.silu_mul(O.q_mat_mul(x, gp, ty, *gs), O.q_mat_mul(x, up, ty, *us))
    part = torch.from_numpy(O.q_mat_mul(h, dp, ty, *ds))
    dist.all_reduce(part)
    err = np.linalg.norm(part.numpy() - want) / np.linalg.norm(want)
    assert err < 1e-5, err
    # every rank holds the same bits after the sum
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    assert all(torch.equal(parts[0], p) for p in parts)
    dist.barrier(); dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_ranks_sum_partial_products_over_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29735", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out
        assert f"rank {r} ok" in out
