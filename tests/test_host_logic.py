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


LAUNCH_RULES_PROGRAM = r"""
#include "sph_launch.hpp"
#include <cstdio>
using namespace sph_b200;
int main() {
    // work_grid(ctas wanted at one item per warp, resident CTAs, items per warp)
    std::printf("grid %d %d %d %d %d %d %d\n", work_grid(100, 444, 0), work_grid(100000, 444, 0), work_grid(131072, 740, 1),
                work_grid(16384, 444, 32, true), work_grid(500000, 444, 32, true), work_grid(1LL << 40, 444, 1),
                work_grid(40000, 1184, 4));
    // tile_serves(kind, l_max, element bytes): kind 0..2 forward level, 3 VJP, 4 second-order VJP
    for (int kind = 0; kind < 5; ++kind) {
        for (int elem = 4; elem <= 8; elem += 4) {
            int last = -1;
            for (int l = 0; l <= 40; ++l) if (tile_serves(kind, l, elem)) last = l;
            std::printf("serves %d %d %d\n", kind, elem, last);
        }
    }
    return 0;
}
"""


def test_launch_rules(tmp_path):
    """The host-side rules that size grids and pick the kernel family, compiled from the library's
    own header: persistent launches take min(wanted, resident) CTAs; short-lived launches divide the
    work by the items per warp, unless that leaves fewer than sixteen waves of CTAs (then fewer items
    per warp, or - for the band kernel - a persistent launch); grids never exceed the hardware limit;
    the tile kernels end where the measured crossovers put them."""
    src = tmp_path / "rules.cpp"
    src.write_text(LAUNCH_RULES_PROGRAM)
    exe = tmp_path / "rules"
    csrc = os.path.join(ROOT, "sphericart_b200", "csrc")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    subprocess.run(["g++", "-std=c++17", "-I", csrc, "-I", cuda_inc, str(src), "-o", str(exe)], check=True)
    lines = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n")
    grid = [int(v) for v in lines[0].split()[1:]]
    assert grid[0] == 100 and grid[1] == 444          # persistent
    assert grid[2] == 131072                          # one item per warp: one CTA per item
    assert grid[3] == 444                             # 512 CTAs would be 1.2 waves: persistent instead
    assert grid[4] == (500000 + 31) // 32             # large call: the full 32 items per warp
    assert grid[5] == 2 ** 31 - 1                     # clamped; the kernels' loops cover the rest
    assert grid[6] == 20000                           # 4 items asked, 2 kept: 40000 / (16 * 1184) = 2
    serves = {(int(a), int(b)): int(c) for a, b, c in (ln.split()[1:] for ln in lines[1:] if ln.startswith("serves"))}
    assert serves[(0, 4)] == 20 and serves[(0, 8)] == 20          # values
    assert serves[(1, 4)] == 9 and serves[(1, 8)] == 8            # gradients: the panel kernels take over earlier in float64
    assert serves[(2, 4)] == 4 and serves[(2, 8)] == 4            # Hessians
    assert serves[(3, 4)] == 20 and serves[(3, 8)] == 20          # VJP: two tiles of upstream rows per SM
    assert serves[(4, 4)] == 10 and serves[(4, 8)] == 8           # second-order VJP


def test_out_buffers_are_validated_before_they_reach_a_kernel():
    """The ``out=`` buffers of the Python front end go to the kernels as bare pointers; a wrong
    count, device, dtype, shape or a non-contiguous tensor must be refused on the host."""
    import pytest
    import torch

    from sphericart_b200.spherical_harmonics import _BaseHarmonics

    check = _BaseHarmonics._validate_out
    xyz = torch.zeros((5, 3), dtype=torch.float64)
    shapes = [(5, 9), (5, 3, 9)]
    good = (torch.empty((5, 9), dtype=torch.float64), torch.empty((5, 3, 9), dtype=torch.float64))
    assert check(good, xyz, shapes, require_cuda=False) == (good[0], good[1], None)
    assert check(good + (None,), xyz, shapes, require_cuda=False)[2] is None
    with pytest.raises(ValueError, match="CUDA tensor"):
        check(good, xyz, shapes)                                          # CPU tensors never reach a kernel
    with pytest.raises(ValueError, match="exactly 2"):
        check(good[:1], xyz, shapes, require_cuda=False)                  # gradients asked for, one buffer given
    with pytest.raises(ValueError, match="exactly 2"):
        check(good + (torch.empty(1),), xyz, shapes, require_cuda=False)  # one buffer too many
    with pytest.raises(ValueError, match="shape"):
        check((good[0], torch.empty((5, 3, 8), dtype=torch.float64)), xyz, shapes, require_cuda=False)
    with pytest.raises(ValueError, match="dtype"):
        check((good[0].float(), good[1]), xyz, shapes, require_cuda=False)
    with pytest.raises(ValueError, match="contiguous"):
        check((torch.empty((9, 5), dtype=torch.float64).t(), good[1]), xyz, shapes, require_cuda=False)
    with pytest.raises(ValueError, match="CUDA tensor"):
        check(([1.0], good[1]), xyz, shapes, require_cuda=False)          # not a tensor at all
    with pytest.raises(ValueError, match="xyz_grad"):
        check(torch.empty((5, 4), dtype=torch.float64), xyz, [(5, 3)], names=("xyz_grad",), require_cuda=False)


def test_kernel_family_map():
    """Which kernel family serves which call, asked of the library itself (no launch, no GPU needed): the
    compile-time tile kernels up to their measured crossovers, the run-time-degree panel kernels above
    (forward levels and the first-order VJP), the band kernel for the second-order VJP above the tile
    range and for rows too long for a panel image."""
    from sphericart_b200 import _c_lib

    def switches(kind, elem, l_top):
        out, prev = [], None
        for l_max in range(0, l_top + 1):
            family = _c_lib.kernel_family(kind, l_max, elem)
            if family != prev:
                out.append((l_max, family))
                prev = family
        return out

    assert switches(0, 4, 28) == [(0, "sph_tile_kernel"), (21, "sph_panel_kernel")]
    assert switches(0, 8, 40) == [(0, "sph_tile_kernel"), (21, "sph_panel_kernel")]
    assert switches(1, 4, 28) == [(0, "sph_tile_kernel"), (10, "sph_panel_kernel")]
    assert switches(1, 8, 40) == [(0, "sph_tile_kernel"), (9, "sph_panel_kernel"), (37, "sph_band_kernel")]
    assert switches(2, 4, 28) == [(0, "sph_tile_kernel"), (5, "sph_panel_kernel")]
    assert switches(2, 8, 40) == [(0, "sph_tile_kernel"), (5, "sph_panel_kernel"), (31, "sph_band_kernel")]
    assert switches(3, 4, 28) == [(0, "sph_vjp_tile_kernel"), (21, "sph_panel_vjp_kernel")]
    assert switches(3, 8, 40) == [(0, "sph_vjp_tile_kernel"), (21, "sph_panel_vjp_kernel")]
    assert switches(4, 4, 28) == [(0, "sph_vjp2_tile_kernel"), (11, "sph_band_kernel")]
    assert switches(4, 8, 40) == [(0, "sph_vjp2_tile_kernel"), (9, "sph_band_kernel")]
    assert _c_lib.kernel_family(7, 4, 4) == "" and _c_lib.kernel_family(1, 4, 2) == ""
