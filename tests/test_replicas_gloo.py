"""Multi-GPU runs are independent replicas: the only exchange is the max-over-ranks of the timings.
Two gloo ranks on the CPU exercise that reduction and the whole-job rate."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_SCRIPT = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r})
    import torch.distributed as dist
    import bench
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    ms, ms_e2e = bench.max_over_ranks([10.0 + rank, 30.0 - rank], world, "cpu")
    assert (ms, ms_e2e) == (11.0, 30.0), (ms, ms_e2e)
    # 2 replicas x batch 1 x 64 steps in the slowest rank's 11 ms
    assert abs(bench.whole_job_rate(world, 1, 64, ms) - 2 * 64 / 0.011) < 1e-6
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_replicas_reduce_timings_over_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29731", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out
        assert f"rank {r} ok" in out


def test_single_process_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.max_over_ranks([1.5, 2.5], 1, "cpu") == [1.5, 2.5]
