"""One rank of the tensor-parallel parity run (started by test_gpu_tp.py under torch.distributed.run).

Every rank builds its shard of the same seeded model; rank 0 also builds the oracle. Checks: the
gathered logits of a 40-token prefill and of single-token steps against the oracle (2e-3 relative
L2), identical greedy ids on all ranks, greedy ids equal to the oracle's where its top-1 / top-2
margin exceeds the measured error."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import fixtures as F  # noqa: E402
import kalosm_b200 as kb  # noqa: E402
from llama_util import build_models, tp_cfg  # noqa: E402
from oracle import oracle as O  # noqa: E402


def gather(x):
    parts = [None] * dist.get_world_size()
    dist.all_gather_object(parts, x)
    return parts


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = kb.Device(local)
    uid = [kb.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, 0)
    comm = kb.Comm(dev, world, rank, uid[0])
    # the collective itself
    t = dev.tensor(np.full((3, 5), float(rank + 1), np.float32))
    assert np.all(comm.all_reduce_sum(t).as_slice() == world * (world + 1) / 2)

    cfg, batch = tp_cfg(world), 2
    gpu, cpu = build_models(dev, cfg, batch=batch, seed=5, want_cpu=(rank == 0), comm=comm)
    prompt = np.random.default_rng(6).integers(0, cfg["vocab"], size=(batch, 40), dtype=np.uint32)
    lg, nxt = gpu.forward(prompt)
    assert lg.shape == (batch, cfg["vocab"] // world)
    full = np.concatenate(gather(lg), axis=1)
    ids = gather(nxt)
    assert all(np.array_equal(ids[0], i) for i in ids), ids
    if rank == 0:
        lo = cpu.forward(prompt)
        assert F.rel_l2(full, lo) < 2e-3, F.rel_l2(full, lo)
        # the pick over the shards follows the tie rule of the whole row
        assert np.array_equal(nxt, [O.top_k(full[b], 1)[0][0] for b in range(batch)])
    tok = nxt.copy()
    for step in range(4):
        lg, nxt = gpu.forward(tok[:, None])
        full = np.concatenate(gather(lg), axis=1)
        ids = gather(nxt)
        assert all(np.array_equal(ids[0], i) for i in ids), ids
        assert np.array_equal(nxt, [O.top_k(full[b], 1)[0][0] for b in range(batch)])
        want = [None]
        if rank == 0:
            lo = cpu.forward(tok[:, None])
            assert F.rel_l2(full, lo) < 2e-3, (step, F.rel_l2(full, lo))
            want = [np.array([O.top_k(lo[b], 1)[0][0] for b in range(batch)], dtype=np.uint32)]
        dist.broadcast_object_list(want, 0)
        tok = want[0]
    # device-side greedy loop (captured graph with the collectives inside): same ids everywhere
    out = gpu.generate_greedy(tok, 6)
    outs = gather(out)
    assert all(np.array_equal(outs[0], o) for o in outs), outs
    assert gpu.position == 40 + 4 + 6
    assert dev.status() == 0
    gpu.free()

    # one sequence: the whole step is one persistent kernel per rank; the partial rows of the o and
    # down projections and the greedy key cross NVLink inside it (peer exchange), no NCCL call
    comm.enable_peer_exchange(cfg["hidden"], gather)
    one, cpu1 = build_models(dev, cfg, batch=1, seed=7, want_cpu=(rank == 0), comm=comm)
    prompt = np.random.default_rng(8).integers(0, cfg["vocab"], size=(1, 11), dtype=np.uint32)
    lg, nxt = one.forward(prompt)
    launches = dev.launch_count
    lg, nxt2 = one.forward(nxt[:, None])
    assert dev.launch_count - launches == 1, "a single-sequence step must be one launch"
    full = np.concatenate(gather(lg), axis=1)
    ids = gather(nxt2)
    assert all(np.array_equal(ids[0], i) for i in ids), ids
    assert np.array_equal(nxt2, [O.top_k(full[0], 1)[0][0]])
    if rank == 0:
        cpu1.forward(prompt)
        lo = cpu1.forward(nxt[:, None])
        assert F.rel_l2(full, lo) < 2e-3, F.rel_l2(full, lo)
    out = one.generate_greedy(nxt2, 12)
    outs = gather(out)
    assert all(np.array_equal(outs[0], o) for o in outs), outs
    if rank == 0:
        tok1 = nxt2.copy()
        for step in range(12):
            lo = cpu1.forward(tok1[:, None])
            want = O.top_k(lo[0], 1)[0][0]
            srt = np.sort(lo[0])
            if out[0, step] != want:
                assert srt[-1] - srt[-2] < 1e-3, (step, srt[-1] - srt[-2])
                break
            tok1 = np.array([want], dtype=np.uint32)
    assert dev.status() == 0
    one.free()
    comm.destroy()
    dist.barrier()
    dist.destroy_process_group()
    print(f"TP_OK rank {rank}", flush=True)


if __name__ == "__main__":
    main()
