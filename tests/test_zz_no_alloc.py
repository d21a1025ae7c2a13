"""The allocation-free entry point against the regular one, through the C ABI.

Some hosts give a plugin its input and output buffers and nothing else: the device arena was
reserved when the process started, or a cudaMalloc (which synchronises the whole device) is not
allowed inside the service loop. For them the library has one entry point that keeps its tables
in a fixed device array instead of allocating them. This file checks that it returns what the
regular entry point returns, twice in a row (the second call reuses what the first left in the
array) and again after the array's content has to change, and that it refuses degrees beyond its
fixed capacity. It is named to be collected last, so a run that stops at the first failure has
already run everything else; it passes alone in a fresh process as well.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-12  # float64 bar used throughout the GPU tests, relative to the degree block's maximum


def _both(lib, calc, normalized, l_max, xyz):
    dev = xyz.device
    n, ny = xyz.shape[0], (l_max + 1) ** 2
    stream = torch.cuda.current_stream(dev).cuda_stream
    sph_a = torch.empty((n, ny), dtype=torch.float64, device=dev)
    dsph_a = torch.empty((n, 3, ny), dtype=torch.float64, device=dev)
    sph_b = torch.full((n, ny), 7.0, dtype=torch.float64, device=dev)
    dsph_b = torch.full((n, 3, ny), 7.0, dtype=torch.float64, device=dev)
    calc.compute_raw(torch.float64, 1, xyz.data_ptr(), n, sph_a.data_ptr(), dsph_a.data_ptr(), None, stream)
    status = lib.sphericart_cuda_harmonics_with_gradients_no_alloc(
        int(normalized), l_max, xyz.data_ptr(), n, sph_b.data_ptr(), dsph_b.data_ptr(), stream)
    assert status == 0, lib.sphericart_cuda_last_error()
    torch.cuda.synchronize(dev)
    return (sph_a.cpu().numpy(), dsph_a.cpu().numpy()), (sph_b.cpu().numpy(), dsph_b.cpu().numpy())


def test_no_alloc_entry_point_matches_regular_entry_point(oracle_mod):
    import sphericart_b200 as sb
    from sphericart_b200 import _c_lib

    lib = _c_lib.get_library()
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(2024)
    # two calls in a row with the same degree, then the array's content changes twice
    plan = [(sb.SphericalHarmonics, True, 12, 1000), (sb.SphericalHarmonics, True, 12, 777),
            (sb.SolidHarmonics, False, 20, 300), (sb.SphericalHarmonics, True, 5, 64),
            (sb.SphericalHarmonics, True, 32, 150)]
    for cls, normalized, l_max, n in plan:
        xyz = torch.from_numpy(rng.standard_normal((n, 3)) * 1.3).to(dev)
        regular, no_alloc = _both(lib, cls(l_max), normalized, l_max, xyz)
        for a, b in zip(no_alloc, regular):
            err, bad = oracle_mod.scaled_error(a, b, l_max)
            assert bad == 0 and err <= TOL, (cls.__name__, l_max, n, err, bad)
        # and directly against the CPU checker (the reference's own library where it was built)
        xyz_np = xyz.cpu().numpy()
        want = (oracle_mod.ref_compute(xyz_np, l_max, normalized, 1) if oracle_mod.have_ref()
                else oracle_mod.port_compute(xyz_np, l_max, normalized, 1))
        for a, b in zip(no_alloc, want[:2]):
            err, bad = oracle_mod.scaled_error(a, b, l_max)
            assert bad == 0 and err <= TOL, (cls.__name__, l_max, n, "against the CPU checker", err, bad)


def test_no_alloc_entry_point_rejects_what_it_cannot_hold():
    from sphericart_b200 import _c_lib

    lib = _c_lib.get_library()
    dev = torch.device("cuda", 0)
    xyz = torch.randn(8, 3, dtype=torch.float64, device=dev)
    sph = torch.empty((8, 34 * 34), dtype=torch.float64, device=dev)
    dsph = torch.empty((8, 3, 34 * 34), dtype=torch.float64, device=dev)
    status = lib.sphericart_cuda_harmonics_with_gradients_no_alloc(1, 33, xyz.data_ptr(), 8, sph.data_ptr(),
                                                                   dsph.data_ptr(), None)
    assert status != 0 and "l_max <= 32" in _c_lib.last_error()
    status = lib.sphericart_cuda_harmonics_with_gradients_no_alloc(1, 4, xyz.data_ptr(), 8, None, dsph.data_ptr(), None)
    assert status != 0
    # zero points: nothing to do, nothing touched
    assert lib.sphericart_cuda_harmonics_with_gradients_no_alloc(1, 4, None, 0, None, None, None) == 0
