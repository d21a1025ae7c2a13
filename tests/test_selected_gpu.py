"""Selected degree blocks, packed, scaled and axis-permuted by one kernel, against the CPU checker.

The reference composes this from a full evaluation, a slice, an axis permutation and a
multiplication (sphericart-torch/python/sphericart/torch/e3nn.py:47-80); the expected values here
are built the same way on the host from the reference CPU library's output (the CPU restatement
where that library was not built). Values and the fused backward go through the C ABI; the torch
operator is checked with gradcheck.
"""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {np.dtype(np.float64): 1e-12, np.dtype(np.float32): 1e-5}
AXIS = (2, 0, 1)   # e3nn's (y, z, x) columns hold this library's x at 2, y at 0, z at 1
L_LISTS = ([2], [0, 2, 4], [1, 3], list(range(9)), [5, 0], [12, 3])


def _scales(l_list, normalization):
    out = []
    for l in l_list:
        s = 1.0 if normalization == "integral" else math.sqrt(4 * math.pi)
        if normalization == "norm":
            s /= math.sqrt(2 * l + 1)
        out.append(s)
    return out


def _reference_full(oracle_mod, xyz, l_max, normalized, level):
    if oracle_mod.have_ref():
        return oracle_mod.ref_compute(xyz, l_max, normalized, level)
    return oracle_mod.port_compute(xyz, l_max, normalized, level)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("normalization", ["integral", "norm", "component"])
def test_selected_values_and_vjp_match_the_composed_reference(oracle_mod, dtype, normalization):
    import sphericart_b200 as sb

    rng = np.random.default_rng(17)
    for cls, normalized in ((sb.SphericalHarmonics, True), (sb.SolidHarmonics, False)):
        for l_list in L_LISTS:
            l_max = max(l_list)
            scales = _scales(l_list, normalization)
            for n in (1, 33, 1000):
                pts = (rng.standard_normal((n, 3)) * 1.4).astype(dtype)        # columns in the caller's order
                own = np.ascontiguousarray(pts[:, list(AXIS)])                 # columns (x, y, z)
                sph, dsph, _ = _reference_full(oracle_mod, own, l_max, normalized, 1)
                calc = cls(l_max)
                got = calc.compute_selected(torch.from_numpy(pts).cuda(), l_list, AXIS, scales).cpu().numpy()
                assert got.shape == (n, sum(2 * l + 1 for l in l_list))
                g = rng.standard_normal(got.shape).astype(dtype)
                got_vjp = calc.compute_selected_vjp(torch.from_numpy(pts).cuda(), torch.from_numpy(g).cuda(), l_list,
                                                    AXIS, scales).cpu().numpy()
                want_vjp = np.zeros((n, 3))
                scale_vjp = np.zeros((n, 1))
                col = 0
                for l, s in zip(l_list, scales):
                    block = slice(l * l, (l + 1) ** 2)
                    want = sph[:, block].astype(np.float64) * s
                    have = got[:, col:col + 2 * l + 1].astype(np.float64)
                    ref_scale = np.maximum(np.abs(want).max(axis=1, keepdims=True), np.finfo(dtype).tiny)
                    err = (np.abs(have - want) / ref_scale).max()
                    assert err <= TOL[np.dtype(dtype)], (cls.__name__, l_list, normalization, n, l, err)
                    gb = g[:, col:col + 2 * l + 1].astype(np.float64) * s
                    d = dsph[:, :, block].astype(np.float64)
                    contrib = np.einsum("nak,nk->na", d, gb)                    # d / d(x, y, z)
                    for a in range(3):
                        want_vjp[:, AXIS[a]] += contrib[:, a]                   # back to the caller's columns
                    scale_vjp += np.einsum("nak,nk->na", np.abs(d), np.abs(gb)).max(axis=1, keepdims=True)
                    col += 2 * l + 1
                err = (np.abs(got_vjp - want_vjp) / np.maximum(scale_vjp, 1e-300)).max()
                assert err <= TOL[np.dtype(dtype)], (cls.__name__, l_list, normalization, n, "vjp", err)


def test_selected_rejects_what_it_cannot_serve():
    import sphericart_b200 as sb

    xyz = torch.randn(10, 3, device="cuda")
    with pytest.raises(ValueError):
        sb.SphericalHarmonics(4).compute_selected(xyz, [1, 1])
    with pytest.raises(ValueError):
        sb.SphericalHarmonics(4).compute_selected(xyz, [5])
    with pytest.raises(ValueError):
        sb.SphericalHarmonics(4).compute_selected(xyz, [2], axis_order=(0, 0, 1))
    with pytest.raises(RuntimeError, match="l_max <= 20"):
        sb.SphericalHarmonics(21).compute_selected(xyz, [2])


def test_selected_operator_autograd_and_e3nn_entry_point():
    import sphericart_b200.torch_ops as sbt

    torch.manual_seed(4)
    x = torch.randn(40, 3, dtype=torch.float64, device="cuda", requires_grad=True)
    scales = _scales([1, 3], "norm")
    for op in (sbt.ops.spherical_harmonics_selected, sbt.ops.solid_harmonics_selected):
        assert torch.autograd.gradcheck(lambda t: op(t, [1, 3], [2, 0, 1], scales), (x,), eps=1e-6, atol=1e-7)
    # the e3nn-style function is one call of the operator: same numbers as the composition it replaces
    full = sbt.ops.spherical_harmonics(x[:, [2, 0, 1]], 3)
    got = sbt.e3nn_spherical_harmonics([1, 3], x, normalize=True, normalization="norm")
    want = torch.cat([full[:, 1:4] * scales[0], full[:, 9:16] * scales[1]], dim=1)
    assert torch.allclose(got, want, rtol=1e-13, atol=1e-14)
    (gx,) = torch.autograd.grad(got.square().sum(), x)
    (wx,) = torch.autograd.grad(want.square().sum(), x)
    assert torch.allclose(gx, wx, rtol=1e-10, atol=1e-12)
    # degrees beyond the compile-time kernels take the composed route
    high = sbt.e3nn_spherical_harmonics([22], x, normalize=True)
    assert tuple(high.shape) == (40, 45)
    # tracing sees the packed shape
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        fake = torch.empty((7, 3), device="cuda")
        assert tuple(sbt.ops.solid_harmonics_selected(fake, [0, 2], [0, 1, 2], []).shape) == (7, 6)
