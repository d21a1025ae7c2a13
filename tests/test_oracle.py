"""Pins the CPU restatement in oracle/ to the reference: committed outputs of the reference's
CPU library, the live reference library when it has been built, scipy's known answers (the
reference's python/tests/test_vs_scipy.py), and finite differences (the reference's
sphericart/tests/test_derivatives.cpp). CPU only."""

import numpy as np
import pytest
import scipy.special

TOL = {np.dtype(np.float64): 1e-12, np.dtype(np.float32): 1e-5}


def _golden_cases(golden):
    for key in golden.files:
        if key.endswith("_sph_A") or key.endswith("_sph_B"):
            cls, dt, l, lv, _, tag = key.split("_")
            yield cls, dt, int(l[1:]), int(lv[2:]), tag


def test_port_matches_golden_vectors(oracle_mod, golden):
    n_cases = 0
    for cls, dt, L, level, tag in _golden_cases(golden):
        dtype = np.float64 if dt == "f64" else np.float32
        xyz = golden[f"xyz_{tag}"].astype(dtype)
        got = oracle_mod.port_compute(xyz, L, cls == "spherical", level)
        base = f"{cls}_{dt}_l{L}_lv{level}"
        for name, arr in zip(("sph", "dsph", "ddsph")[: level + 1], got):
            want = golden[f"{base}_{name}_{tag}"]
            err, bad = oracle_mod.scaled_error(arr, want, L)
            assert bad == 0, (base, name, "NaN/inf pattern differs")
            assert err <= TOL[np.dtype(dtype)], (base, name, err)
        n_cases += 1
    assert n_cases >= 60


def test_golden_corner_cases_follow_the_origin_convention(golden):
    """Origin: Y_00 finite and everything else NaN for the normalised harmonics; finite for solid."""
    sph = golden["spherical_f64_l8_lv1_sph_A"]
    dsph = golden["spherical_f64_l8_lv1_dsph_A"]
    assert np.isfinite(sph[0, 0]) and np.isnan(sph[0, 1:]).all() and np.isnan(dsph[0]).all()
    assert np.isfinite(sph[1]).all() and np.isfinite(dsph[1]).all()  # r = 1e-9
    assert np.abs(dsph[1]).max() > 1e8
    assert np.isfinite(golden["solid_f64_l8_lv1_sph_A"]).all()
    assert np.isfinite(golden["solid_f64_l8_lv1_dsph_A"]).all()


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("normalized", [True, False])
def test_port_matches_live_reference(oracle_mod, dtype, normalized):
    if not oracle_mod.have_ref():
        pytest.skip("reference CPU library not built on this machine")
    rng = np.random.default_rng(7)
    for L in (0, 1, 2, 5, 6, 7, 8, 11, 16, 20):
        xyz = (rng.standard_normal((200, 3)) * 2.0).astype(dtype)
        for level in (0, 1, 2):
            got = oracle_mod.port_compute(xyz, L, normalized, level)
            want = oracle_mod.ref_compute(xyz, L, normalized, level)
            for a, b in zip(got[: level + 1], want[: level + 1]):
                err, bad = oracle_mod.scaled_error(a, b, L)
                assert bad == 0 and err <= TOL[np.dtype(dtype)], (L, level, err, bad)


def test_port_prefactors_match_reference_recipe(oracle_mod):
    """F[l][m]^2 = (2l+1)/(2 pi) (l-m)!/(l+m)! (halved for m = 0); K[l][l] = (-1)^l (2l-1)!!."""
    from math import factorial, pi

    L = 12
    f = oracle_mod.port_prefactors(L, np.float64)
    nq = (L + 1) * (L + 2) // 2
    for l in range(L + 1):
        for m in range(l + 1):
            want = (2 * l + 1) / (2 * pi) * factorial(l - m) / factorial(l + m)
            if m == 0:
                want /= 2
            got = f[l * (l + 1) // 2 + m]
            assert abs(got * got / want - 1) < 1e-13
            assert (got < 0) == (m % 2 == 1)
        dfact = 1.0
        for j in range(1, 2 * l, 2):
            dfact *= j
        assert f[nq + l * (l + 1) // 2 + l] == pytest.approx((-1) ** l * dfact, rel=1e-14)


def _scipy_real_sph(xyz, l, m):
    x, y, z = xyz[:, 0], xyz[:, 1], xyz[:, 2]
    r = np.sqrt(x**2 + y**2 + z**2)
    theta = np.arccos(z / r)
    phi = np.arctan2(y, x)
    pos = scipy.special.sph_harm_y(l, abs(m), theta, phi)
    neg = scipy.special.sph_harm_y(l, -abs(m), theta, phi)
    if m > 0:
        return ((neg + (-1) ** m * pos) / np.sqrt(2.0)).real
    if m < 0:
        mm = -m
        return ((-neg + (-1) ** mm * pos) / np.sqrt(2.0)).imag * (-1) ** mm * (-1) ** mm * -1 * -1
    return pos.real


def test_port_against_scipy(oracle_mod):
    """Known answers, as in the reference's python/tests/test_vs_scipy.py:12-61 (l <= 15)."""
    rng = np.random.default_rng(0)
    xyz = rng.random((100, 3))
    L = 15
    r = np.linalg.norm(xyz, axis=1)
    sph = oracle_mod.port_compute(xyz, L, True, 0)[0]
    solid = oracle_mod.port_compute(xyz, L, False, 0)[0]
    theta = np.arccos(xyz[:, 2] / r)
    phi = np.arctan2(xyz[:, 1], xyz[:, 0])
    for l in range(L + 1):
        for m in range(-l, l + 1):
            if m == 0:
                want = scipy.special.sph_harm_y(l, 0, theta, phi).real
            else:
                ylm = scipy.special.sph_harm_y(l, abs(m), theta, phi)
                # real harmonics: sqrt(2) (-1)^m Re / Im of the complex Y_l^|m|
                want = np.sqrt(2.0) * (-1) ** abs(m) * (ylm.real if m > 0 else ylm.imag)
            k = l * l + l + m
            assert np.allclose(sph[:, k], want, rtol=1e-9, atol=1e-11), (l, m)
            assert np.allclose(solid[:, k] / r**l, want, rtol=1e-9, atol=1e-11), (l, m)


@pytest.mark.parametrize("normalized", [True, False])
def test_port_derivatives_by_finite_differences(oracle_mod, normalized):
    """Central differences, as in sphericart/tests/test_derivatives.cpp:168-205 (l_max up to 14)."""
    L = 14
    rng = np.random.default_rng(3)
    xyz = rng.standard_normal((6, 3))
    _, dsph, ddsph = oracle_mod.port_compute(xyz, L, normalized, 2)
    h = 1e-5
    for a in range(3):
        step = np.zeros(3)
        step[a] = h
        yp, dp, _ = oracle_mod.port_compute(xyz + step, L, normalized, 1)
        ym, dm, _ = oracle_mod.port_compute(xyz - step, L, normalized, 1)
        fd1 = (yp - ym) / (2 * h)
        scale = np.abs(dsph[:, a]).max() + 1e-30
        assert np.abs(fd1 - dsph[:, a]).max() / scale < 1e-6
        fd2 = (dp - dm) / (2 * h)  # d/dx_a of the gradient = row a of the Hessian
        scale2 = np.abs(ddsph[:, a]).max() + 1e-30
        assert np.abs(fd2 - ddsph[:, a]).max() / scale2 < 1e-6


def test_port_invariants(oracle_mod):
    rng = np.random.default_rng(11)
    xyz = rng.standard_normal((50, 3)) * 3.0
    L = 10
    sph, dsph, ddsph = oracle_mod.port_compute(xyz, L, True, 2)
    solid, dsolid, ddsolid = oracle_mod.port_compute(xyz, L, False, 2)
    for l in range(L + 1):
        sl = slice(l * l, (l + 1) ** 2)
        # addition theorem on the unit sphere
        assert np.allclose((sph[:, sl] ** 2).sum(axis=1), (2 * l + 1) / (4 * np.pi), rtol=1e-12)
        # Euler: r . grad(solid) = l solid ; r . grad(spherical) = 0
        assert np.allclose(np.einsum("na,nak->nk", xyz, dsolid[:, :, sl]), l * solid[:, sl], rtol=1e-9, atol=1e-9 * np.abs(solid[:, sl]).max())
        assert np.abs(np.einsum("na,nak->nk", xyz, dsph[:, :, sl])).max() < 1e-11
    # solid harmonics are harmonic; Hessians are symmetric bit for bit
    lap = ddsolid[:, 0, 0] + ddsolid[:, 1, 1] + ddsolid[:, 2, 2]
    assert np.abs(lap).max() <= 1e-9 * np.abs(ddsolid).max()
    assert np.array_equal(ddsph, ddsph.transpose(0, 2, 1, 3))
    assert np.array_equal(ddsolid, ddsolid.transpose(0, 2, 1, 3))


def test_port_vjp_is_gradient_contraction(oracle_mod):
    rng = np.random.default_rng(5)
    for dtype in (np.float64, np.float32):
        xyz = rng.standard_normal((300, 3)).astype(dtype)
        for L in (0, 3, 4, 9):
            g = rng.standard_normal((300, (L + 1) ** 2)).astype(dtype)
            for normalized in (True, False):
                got = oracle_mod.port_vjp(xyz, g, L, normalized)
                _, dsph, _ = oracle_mod.port_compute(xyz, L, normalized, 1)
                want = np.einsum("nak,nk->na", dsph.astype(np.float64), g.astype(np.float64))
                tol = 1e-12 if dtype == np.float64 else 2e-5
                scale = np.einsum("nak,nk->na", np.abs(dsph).astype(np.float64), np.abs(g).astype(np.float64)).max() + 1e-30
                assert np.abs(got - want).max() / scale < tol
