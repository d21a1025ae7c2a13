"""Point sharding on more than one GPU (skipped on a single-GPU machine).

Points are independent, so a multi-GPU run is the same calculator applied to contiguous shards
(``workloads.shard_bounds``), each on its own device, with no exchange step. What must hold is that
the shards' outputs, laid end to end, are bit for bit the output of the one-GPU call: the same
kernels evaluate the same arithmetic per point wherever the point sits in the launch.
Shapes: configuration 3 (l_max = 16 float32 Hessians, the run-time-degree kernel) and configuration
4 (l_max = 4 float32 forward and fused VJP, the compile-time tile kernels; 2^24 of its points).
"""

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _shards(n, world):
    from sphericart_b200 import workloads

    return [workloads.shard_bounds(n, world, r) for r in range(world)]


def test_config3_shards_concatenate_bitwise():
    import sphericart_b200 as sb
    from sphericart_b200 import workloads

    wl, _ = workloads.CONFIGS["cfg3"]
    xyz_host = torch.from_numpy(workloads.make_points("cfg3"))
    n = xyz_host.shape[0]
    calc = sb.SphericalHarmonics(wl.l_max)
    whole = calc.compute_with_hessians(xyz_host.to("cuda:0"))
    world = torch.cuda.device_count()
    for rank, (lo, hi) in enumerate(_shards(n, world)):
        dev = f"cuda:{rank}"
        part = calc.compute_with_hessians(xyz_host[lo:hi].to(dev))
        torch.cuda.synchronize(dev)
        for a, b in zip(part, whole):
            assert torch.equal(a.to("cuda:0"), b[lo:hi]), (rank, lo, hi)
        del part
    assert torch.cuda.current_device() == 0


def test_config4_forward_and_vjp_shards_concatenate_bitwise():
    import sphericart_b200 as sb
    from sphericart_b200 import workloads

    wl, _ = workloads.CONFIGS["cfg4"]
    n = 1 << 24     # a third of the configuration's 5e7 points: the same kernels, less host time
    xyz_host = torch.from_numpy(workloads.make_points("cfg4", n_points=n))
    g_host = torch.from_numpy(workloads.make_upstream_grad("cfg4", n_points=n))
    calc = sb.SphericalHarmonics(wl.l_max)
    xyz0 = xyz_host.to("cuda:0")
    whole_sph = calc.compute(xyz0)
    whole_vjp = calc.compute_vjp(xyz0, g_host.to("cuda:0"))
    world = torch.cuda.device_count()
    for rank, (lo, hi) in enumerate(_shards(n, world)):
        dev = f"cuda:{rank}"
        xyz = xyz_host[lo:hi].to(dev)
        sph = calc.compute(xyz)
        vjp = calc.compute_vjp(xyz, g_host[lo:hi].to(dev))
        torch.cuda.synchronize(dev)
        assert torch.equal(sph.to("cuda:0"), whole_sph[lo:hi]), (rank, "values")
        assert torch.equal(vjp.to("cuda:0"), whole_vjp[lo:hi]), (rank, "vjp")
