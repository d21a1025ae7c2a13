"""Host-side logic that needs no GPU: workload generators, point sharding, and the multi-rank
bookkeeping of the benchmark (two gloo ranks on CPU)."""

import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_generators_are_deterministic_and_shaped():
    from sphericart_b200 import workloads

    for name, (wl, _) in workloads.CONFIGS.items():
        a = workloads.make_points(name, n_points=1000)
        b = workloads.make_points(name, n_points=1000)
        assert a.shape == (1000, 3) and a.dtype == wl.np_dtype and np.array_equal(a, b)
        assert not np.array_equal(a, workloads.make_points(name, n_points=1000, seed_offset=1))
    r = np.linalg.norm(workloads.make_points("cfg2", 20000).astype(np.float64), axis=1)
    assert r.max() <= 5.0 + 1e-5 and 3.5 < np.median(r) < 4.3            # uniform in a ball of radius 5
    r = np.linalg.norm(workloads.make_points("cfg3", 20000).astype(np.float64), axis=1)
    assert 0.5 - 1e-5 <= r.min() and r.max() <= 6.0 + 1e-5
    s = workloads.make_points("cfg5", 100000)
    r = np.linalg.norm(s, axis=1)
    assert (r == 0).sum() == 100 and ((r > 0) & (r < 1e-5)).sum() == 1000
    assert abs(workloads.make_points("cfg4", 200000).astype(np.float64).var() - 2.0) < 0.05


def test_bytes_per_point_match_the_scope_table():
    from sphericart_b200 import workloads

    want = {"metric": 1308, "cfg1": 2616, "cfg2": 796, "cfg3": 15040, "cfg4": 124, "cfg5": 34872}
    for name, b in want.items():
        assert workloads.CONFIGS[name][0].bytes_per_point() == b


def test_shards_partition_the_points():
    from sphericart_b200 import workloads

    for n in (0, 1, 31, 32, 33, 1000, 2_000_000, 50_000_000, 4_194_304 * 8 + 5):
        for world in (1, 2, 4, 8):
            covered = 0
            for rank in range(world):
                lo, hi = workloads.shard_bounds(n, world, rank)
                assert lo == covered or lo == n
                assert lo % 32 == 0 or lo == n
                covered = max(covered, hi)
            assert covered == n


RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
import bench
from sphericart_b200 import workloads
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
n = 100_000
lo, hi = workloads.shard_bounds(n, world, rank)
total = bench.reduce_sum(float(hi - lo), world)
slowest = bench.reduce_max(10.0 + rank, world)     # pretend rank r took 10 + r ms
a = workloads.make_points("metric", n_points=64, seed_offset=rank)
gathered = [None] * world
dist.all_gather_object(gathered, a.tobytes())
if rank == 0:
    assert total == n, total
    assert slowest == 10.0 + world - 1, slowest
    assert len(set(gathered)) == world, "every rank draws its own shard"
    print("RANKS_OK", world)
dist.destroy_process_group()
"""


def test_two_rank_bookkeeping_over_gloo(tmp_path):
    script = tmp_path / "ranks.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", "29617", str(script), ROOT],
        capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "RANKS_OK 2" in out.stdout


def test_reference_arm_prints_one_json_line():
    import json

    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "points/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["e2e"]["h2d_bytes_per_step"] == 0
