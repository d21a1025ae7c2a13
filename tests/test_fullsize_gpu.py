"""The benchmark configurations at their full sizes, checked through properties that need no
CPU run: the addition theorem, Euler's homogeneity relation, the Laplacian, Hessian symmetry,
the NaN mask of the origin points, and agreement of the fused VJP with the explicit contraction.
All calls go through the C ABI."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _points(config, n=None):
    from sphericart_b200 import workloads

    wl, _ = workloads.CONFIGS[config]
    return wl, torch.from_numpy(workloads.make_points(config, n_points=n)).to(DEV)


def _addition_theorem_error(sph, l_max, rows=slice(None)):
    """max over points and l of |sum_m Y_lm^2 - (2l+1)/(4 pi)| / ((2l+1)/(4 pi)), ignoring NaN rows."""
    worst = 0.0
    for l in range(l_max + 1):
        want = (2 * l + 1) / (4 * math.pi)
        s = (sph[rows, l * l:(l + 1) ** 2].double() ** 2).sum(dim=1)
        s = s[~torch.isnan(s)]
        worst = max(worst, float(((s - want).abs() / want).max()))
    return worst


def _radial_error(xyz, dsph, l_max):
    """max |r . grad Y_lm| / (|r| max_block |grad Y|): zero for a function of the direction only. The
    scale is the largest gradient entry of the same degree block of the same point."""
    radial = torch.einsum("na,nak->nk", xyz, dsph).abs()
    rnorm = xyz.norm(dim=1)
    worst = 0.0
    for l in range(1, l_max + 1):
        sl = slice(l * l, (l + 1) ** 2)
        scale = (rnorm * dsph[:, :, sl].abs().amax(dim=(1, 2))).clamp_min(1e-300)
        worst = max(worst, float((radial[:, sl].amax(dim=1) / scale).max()))
    return worst


def test_metric_workload_full_size():
    import sphericart_b200 as sb

    wl, xyz = _points("metric")
    sph, dsph = sb.SphericalHarmonics(wl.l_max).compute_with_gradients(xyz)
    assert _addition_theorem_error(sph, wl.l_max) < 2e-5
    # Y depends on direction only: r . grad Y = 0 (relative to |r| |grad Y|)
    worst = 0.0
    for lo in range(0, xyz.shape[0], 1 << 20):
        sl = slice(lo, lo + (1 << 20))
        worst = max(worst, _radial_error(xyz[sl], dsph[sl], wl.l_max))
    assert worst < 5e-5


def test_config2_solid_full_size():
    import sphericart_b200 as sb

    wl, xyz = _points("cfg2")
    sph, dsph = sb.SolidHarmonics(wl.l_max).compute_with_gradients(xyz)
    for l in range(wl.l_max + 1):
        sl = slice(l * l, (l + 1) ** 2)
        euler = torch.einsum("na,nak->nk", xyz, dsph[:, :, sl])  # r . grad = l * value
        scale = (xyz.norm(dim=1) * dsph[:, :, sl].abs().amax(dim=(1, 2))).clamp_min(1e-30)
        assert float(((euler - l * sph[:, sl]).abs().amax(dim=1) / scale).max()) < 2e-5
    r = xyz.norm(dim=1, keepdim=True)
    unit = sb.SphericalHarmonics(wl.l_max).compute(xyz)
    for l in range(wl.l_max + 1):
        sl = slice(l * l, (l + 1) ** 2)
        ok = (r[:, 0] > 1e-3)
        diff = (sph[ok][:, sl] - unit[ok][:, sl] * r[ok] ** l).abs().amax(dim=1) / (r[ok][:, 0] ** l)
        assert float(diff.max()) < 2e-5   # |Y_lm| <= sqrt((2l+1)/(4 pi)) ~ 1, so this is relative to the block


def test_config3_hessians_full_size():
    import sphericart_b200 as sb

    wl, xyz = _points("cfg3")
    n = xyz.shape[0]
    sph, dsph, ddsph = sb.SphericalHarmonics(wl.l_max).compute_with_hessians(xyz)
    assert _addition_theorem_error(sph, wl.l_max) < 4e-5
    r2 = (xyz.double() ** 2).sum(dim=1, keepdim=True)
    lfac = torch.cat([torch.full((2 * l + 1,), float(l * (l + 1)), device=DEV, dtype=torch.float64)
                      for l in range(wl.l_max + 1)])
    worst_lap, sym_ok = 0.0, True
    for lo in range(0, n, 1 << 17):
        sl = slice(lo, lo + (1 << 17))
        h = ddsph[sl]
        sym_ok &= bool(torch.equal(h[:, 0, 1], h[:, 1, 0]) and torch.equal(h[:, 0, 2], h[:, 2, 0])
                       and torch.equal(h[:, 1, 2], h[:, 2, 1]))
        lap = (h[:, 0, 0].double() + h[:, 1, 1].double() + h[:, 2, 2].double())
        want = -lfac * sph[sl].double() / r2[sl]           # Laplacian of Y_lm(r/|r|)
        err = (lap - want).abs()
        for l in range(wl.l_max + 1):
            cs = slice(l * l, (l + 1) ** 2)
            scale = h[:, :, :, cs].abs().amax(dim=(1, 2, 3)).double().clamp_min(1e-30)
            worst_lap = max(worst_lap, float((err[:, cs].amax(dim=1) / scale).max()))
    assert sym_ok, "Hessian halves must be bitwise equal"
    assert worst_lap < 1e-4


def test_config4_forward_and_vjp_full_size():
    import sphericart_b200 as sb
    from sphericart_b200 import workloads

    wl, xyz = _points("cfg4")
    n = xyz.shape[0]
    calc = sb.SphericalHarmonics(wl.l_max)
    sph = calc.compute(xyz)
    assert _addition_theorem_error(sph, wl.l_max) < 1e-5
    del sph
    g = torch.from_numpy(workloads.make_upstream_grad("cfg4", n_points=1 << 22)).to(DEV)
    head = xyz[: 1 << 22]
    fused = calc.compute_vjp(head, g)
    _, dsph = calc.compute_with_gradients(head)
    explicit = torch.einsum("nak,nk->na", dsph.double(), g.double())
    scale = torch.einsum("nak,nk->na", dsph.abs().double(), g.abs().double()).amax(dim=1, keepdim=True)
    assert float(((fused.double() - explicit).abs() / scale).max()) < 1e-5
    # the whole 50M-point shard in one launch: finite everywhere (no point is at the origin)
    g_all = torch.randn(n, wl.ny, device=DEV)
    out = calc.compute_vjp(xyz, g_all)
    assert bool(torch.isfinite(out).all())


def test_config5_stress_full_size():
    import sphericart_b200 as sb

    wl, xyz = _points("cfg5")
    sph, dsph = sb.SphericalHarmonics(wl.l_max).compute_with_gradients(xyz)
    at_origin = (xyz == 0).all(dim=1)
    assert int(at_origin.sum()) == 1000
    nan_rows = torch.isnan(sph[:, 1:]).any(dim=1)
    assert torch.equal(nan_rows, at_origin), "NaN exactly at the origin points"
    assert bool(torch.isfinite(sph[:, 0]).all())
    assert bool(torch.isnan(dsph[at_origin]).all()) and bool(torch.isfinite(dsph[~at_origin]).all())
    assert _addition_theorem_error(sph, wl.l_max) < 1e-12
    tiny = (xyz.norm(dim=1) < 1e-5) & ~at_origin
    assert int(tiny.sum()) == 10000
    assert _radial_error(xyz[tiny], dsph[tiny], wl.l_max) < 1e-12
