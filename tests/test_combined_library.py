"""One shared library with both halves of the reference's C API.

The reference's ctypes front end loads a single ``libsphericart`` and binds, at load time, the 36
CPU functions and the 20 CUDA functions of ``sphericart/include/sphericart.h``
(``python/src/sphericart/_c_lib.py:41-400``). ``oracle/Makefile`` (target ``combined``) links the
reference's own CPU translation units into ``oracle/_ref/libsphericart_combined.so`` with this
repository's CUDA library as its dependency, so that one load handle answers for all 56 functions
(a maintainer's build links the CUDA objects in directly); these tests check that the result is what that front
end needs: every symbol binds (through the reference's own ``setup_functions`` where the
reference checkout is present), the CPU half computes what the reference CPU library computes, and
the CUDA half - this repository's kernels - answers through the very same library handle.
The combined library is test infrastructure; the package never loads it.
"""

import ctypes
import importlib.util
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMBINED = os.path.join(ROOT, "oracle", "_ref", "libsphericart_combined.so")

needs_library = pytest.mark.skipif(not os.path.exists(COMBINED), reason="combined library not built (needs the "
                                   "reference checkout: make -C oracle REF=<checkout> combined)")


def _c_api_names():
    """The 56 functions of the reference's C header, CPU half then CUDA half."""
    cpu, cuda = [], []
    for kind in ("spherical", "solid"):
        for sfx in ("", "_f"):
            base = f"sphericart_{kind}_harmonics"
            cpu += [f"{base}_new{sfx}", f"{base}_delete{sfx}", f"{base}_omp_num_threads{sfx}"]
            for shape in ("array", "sample"):
                for level in ("", "_with_gradients", "_with_hessians"):
                    cpu.append(f"{base}_compute_{shape}{level}{sfx}")
            cbase = f"sphericart_cuda_{kind}_harmonics"
            cuda += [f"{cbase}_new{sfx}", f"{cbase}_delete{sfx}"]
            for level in ("", "_with_gradients", "_with_hessians"):
                cuda.append(f"{cbase}_compute_array{level}{sfx}")
    return cpu, cuda


@needs_library
def test_combined_library_exports_both_halves():
    lib = ctypes.CDLL(COMBINED)
    cpu, cuda = _c_api_names()
    assert len(cpu) == 36 and len(cuda) == 20
    for name in cpu + cuda:
        assert getattr(lib, name) is not None, name
    # the additions of this repository come along with its objects
    assert lib.sphericart_cuda_last_error is not None and lib.sphericart_cuda_spherical_harmonics_compute_vjp is not None


@needs_library
def test_reference_front_end_binds_every_symbol():
    """The reference's own binding code, run against the combined library."""
    from oracle import oracle

    root = oracle.reference_root()
    if root is None:
        pytest.skip("reference checkout not available on this machine (set SPHERICART_REF)")
    spec = importlib.util.spec_from_file_location(
        "reference_c_lib", os.path.join(root, "python", "src", "sphericart", "_c_lib.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    lib = ctypes.cdll.LoadLibrary(COMBINED)
    module.setup_functions(lib)     # raises AttributeError on the first missing symbol
    # a CPU call with the argument types the reference's binding has just declared
    xyz = np.random.default_rng(5).standard_normal((7, 3))
    sph = np.empty((7, 25))
    calc = lib.sphericart_spherical_harmonics_new(4)
    dptr = ctypes.POINTER(ctypes.c_double)
    lib.sphericart_spherical_harmonics_compute_array(calc, xyz.ctypes.data_as(dptr), xyz.size,
                                                     sph.ctypes.data_as(dptr), sph.size)
    lib.sphericart_spherical_harmonics_delete(calc)
    assert abs(sph[0, 0] - 0.282094791773878) < 1e-15 and np.isfinite(sph).all()


@needs_library
def test_cpu_half_is_the_reference_cpu_code(oracle_mod):
    if not oracle_mod.have_ref():
        pytest.skip("reference CPU library not built")
    lib = ctypes.CDLL(COMBINED)
    lib.sphericart_solid_harmonics_new_f.restype = ctypes.c_void_p
    lib.sphericart_solid_harmonics_new_f.argtypes = [ctypes.c_size_t]
    lib.sphericart_solid_harmonics_delete_f.argtypes = [ctypes.c_void_p]
    fn = lib.sphericart_solid_harmonics_compute_array_with_gradients_f
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t,
                   ctypes.c_void_p, ctypes.c_size_t]
    xyz = np.random.default_rng(6).standard_normal((300, 3)).astype(np.float32)
    sph = np.empty((300, 81), dtype=np.float32)
    dsph = np.empty((300, 3, 81), dtype=np.float32)
    calc = lib.sphericart_solid_harmonics_new_f(8)
    fn(calc, xyz.ctypes.data, xyz.size, sph.ctypes.data, sph.size, dsph.ctypes.data, dsph.size)
    lib.sphericart_solid_harmonics_delete_f(calc)
    want = oracle_mod.ref_compute(xyz, 8, False, 1)
    assert np.array_equal(sph, want[0]) and np.array_equal(dsph, want[1])   # same sources, same flags


@needs_library
@pytest.mark.gpu
def test_cuda_half_answers_through_the_same_handle(oracle_mod):
    """CPU and CUDA calculators created from ONE library handle; the CUDA results (this repository's
    kernels behind the reference's symbol names) agree with the CPU results of the same library."""
    import torch

    lib = ctypes.CDLL(COMBINED)
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    lib.sphericart_spherical_harmonics_new.restype = vp
    lib.sphericart_spherical_harmonics_new.argtypes = [sz]
    lib.sphericart_spherical_harmonics_delete.argtypes = [vp]
    cpu = lib.sphericart_spherical_harmonics_compute_array_with_gradients
    cpu.restype = None
    cpu.argtypes = [vp, vp, sz, vp, sz, vp, sz]
    lib.sphericart_cuda_spherical_harmonics_new.restype = vp
    lib.sphericart_cuda_spherical_harmonics_new.argtypes = [sz]
    lib.sphericart_cuda_spherical_harmonics_delete.argtypes = [vp]
    gpu = lib.sphericart_cuda_spherical_harmonics_compute_array_with_gradients
    gpu.restype = None
    gpu.argtypes = [vp, vp, sz, vp, vp, vp]

    for l_max in (6, 12):
        ny = (l_max + 1) ** 2
        xyz = np.random.default_rng(7 + l_max).standard_normal((1000, 3))
        sph = np.empty((1000, ny))
        dsph = np.empty((1000, 3, ny))
        c = lib.sphericart_spherical_harmonics_new(l_max)
        cpu(c, xyz.ctypes.data, xyz.size, sph.ctypes.data, sph.size, dsph.ctypes.data, dsph.size)
        lib.sphericart_spherical_harmonics_delete(c)
        d_xyz = torch.from_numpy(xyz).cuda()
        d_sph = torch.empty((1000, ny), dtype=torch.float64, device="cuda")
        d_dsph = torch.empty((1000, 3, ny), dtype=torch.float64, device="cuda")
        g = lib.sphericart_cuda_spherical_harmonics_new(l_max)
        assert g, "CUDA calculator construction failed"
        gpu(g, d_xyz.data_ptr(), 1000, d_sph.data_ptr(), d_dsph.data_ptr(), None)
        torch.cuda.synchronize()
        lib.sphericart_cuda_spherical_harmonics_delete(g)
        for got, want in ((d_sph, sph), (d_dsph, dsph)):
            err, bad = oracle_mod.scaled_error(got.cpu().numpy(), want, l_max)
            assert bad == 0 and err <= 1e-12, (l_max, err, bad)
