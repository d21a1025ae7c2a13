"""Behaviour at the drop-in boundary that the reference documents or relies on: the abort
convention of the reference-named C entry points, calls from several threads and streams on
one calculator, and the "device follows the pointer" rule on a multi-GPU machine."""

import os
import subprocess
import sys
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

ABORT_CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1])
import torch
from sphericart_b200 import _c_lib
lib = _c_lib.get_library()
calc = lib.sphericart_cuda_spherical_harmonics_new_f(3)
assert calc
xyz = torch.randn(4, 3, device="cuda")
print("BEFORE", flush=True)
# null sph with a non-zero point count: the reference-named entry point reports and aborts
lib.sphericart_cuda_spherical_harmonics_compute_array_f(calc, xyz.data_ptr(), 4, None, None)
print("AFTER", flush=True)
"""


def test_reference_named_entry_points_abort_on_error(tmp_path):
    """sphericart/src/sphericart-capi.cpp:653-696: print "fatal error: ..." and abort()."""
    script = tmp_path / "abort_child.py"
    script.write_text(ABORT_CHILD)
    out = subprocess.run([sys.executable, str(script), ROOT], capture_output=True, text=True, timeout=300)
    assert out.returncode < 0 or out.returncode == 134, out.returncode   # killed by SIGABRT
    assert "BEFORE" in out.stdout and "AFTER" not in out.stdout
    assert "fatal error:" in out.stdout and "sph" in out.stdout


def test_reference_named_entry_points_compute(oracle_mod):
    """The 20 reference-named symbols themselves (not the status-returning twins)."""
    from sphericart_b200 import _c_lib

    lib = _c_lib.get_library()
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(8)
    for kind, normalized in (("spherical", True), ("solid", False)):
        for sfx, dtype, tdtype in (("", np.float64, torch.float64), ("_f", np.float32, torch.float32)):
            l_max, n = 5, 300
            ny = (l_max + 1) ** 2
            base = f"sphericart_cuda_{kind}_harmonics"
            calc = getattr(lib, f"{base}_new{sfx}")(l_max)
            assert calc
            xyz_np = rng.standard_normal((n, 3)).astype(dtype)
            xyz = torch.from_numpy(xyz_np).to(dev)
            sph = torch.empty((n, ny), dtype=tdtype, device=dev)
            dsph = torch.empty((n, 3, ny), dtype=tdtype, device=dev)
            ddsph = torch.empty((n, 3, 3, ny), dtype=tdtype, device=dev)
            getattr(lib, f"{base}_compute_array{sfx}")(calc, xyz.data_ptr(), n, sph.data_ptr(), None)
            first = sph.clone()
            getattr(lib, f"{base}_compute_array_with_gradients{sfx}")(calc, xyz.data_ptr(), n, sph.data_ptr(),
                                                                      dsph.data_ptr(), None)
            getattr(lib, f"{base}_compute_array_with_hessians{sfx}")(calc, xyz.data_ptr(), n, sph.data_ptr(),
                                                                     dsph.data_ptr(), ddsph.data_ptr(), None)
            torch.cuda.synchronize(dev)
            want = oracle_mod.port_compute(xyz_np, l_max, normalized, 2)
            tol = 1e-12 if dtype == np.float64 else 1e-5
            for got, ref in zip((first, dsph, ddsph), want):
                err, bad = oracle_mod.scaled_error(got.cpu().numpy(), ref, l_max)
                assert bad == 0 and err <= tol
            getattr(lib, f"{base}_delete{sfx}")(calc)
            getattr(lib, f"{base}_delete{sfx}")(None)  # deleting nothing is harmless


def test_one_calculator_many_threads_and_streams():
    """Bindings share a calculator between threads and streams (sphericart-jax keeps a static map,
    sphericart-jax/src/sphericart_jax_cuda.cpp:29-40); calls must be re-entrant, including the
    first call that uploads the tables of a run-time-degree calculator."""
    import sphericart_b200 as sb

    dev = torch.device("cuda", 0)
    calc = sb.SphericalHarmonics(11)          # band kernel: lazy per-device table upload
    xyz = torch.randn(20000, 3, dtype=torch.float64, device=dev)
    results, errors = [None] * 8, []

    def work(i):
        try:
            stream = torch.cuda.Stream(device=dev)
            stream.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(stream):
                out = calc.compute_with_gradients(xyz)
            stream.synchronize()
            results[i] = out
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for out in results[1:]:
        assert torch.equal(out[0], results[0][0]) and torch.equal(out[1], results[0][1])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_device_follows_the_pointer(oracle_mod):
    """sphericart/src/sphericart_cuda.cpp:115-125,157-159: run on the device that owns xyz and
    restore the caller's current device; each device gets its own tables."""
    import sphericart_b200 as sb

    rng = np.random.default_rng(1)
    xyz_np = rng.standard_normal((500, 3))
    for l_max in (6, 12):
        calc = sb.SphericalHarmonics(l_max)
        want = oracle_mod.port_compute(xyz_np, l_max, True, 1)
        torch.cuda.set_device(0)
        for d in (1, 0, 1):
            xyz = torch.from_numpy(xyz_np).to(f"cuda:{d}")
            sph = torch.empty((500, (l_max + 1) ** 2), dtype=torch.float64, device=f"cuda:{d}")
            dsph = torch.empty((500, 3, (l_max + 1) ** 2), dtype=torch.float64, device=f"cuda:{d}")
            # launch on the stream of the OWNING device while another device is current
            calc.compute_raw(torch.float64, 1, xyz.data_ptr(), 500, sph.data_ptr(), dsph.data_ptr(), None,
                             torch.cuda.current_stream(d).cuda_stream)
            torch.cuda.synchronize(d)
            assert torch.cuda.current_device() == 0
            for got, ref in zip((sph, dsph), want):
                err, bad = oracle_mod.scaled_error(got.cpu().numpy(), ref, l_max)
                assert bad == 0 and err <= 1e-12


def test_threads_alternating_degrees_on_one_kernel(oracle_mod):
    """Two calculators whose calls run the same kernel instantiation with different shared-memory
    sizes (l_max = 12 and 14, float64 gradients), driven from several host threads at once: raising the
    kernel's shared-memory limit for one must never break a launch of the other."""
    import threading

    import sphericart_b200 as sb

    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(3)
    xyz_np = rng.standard_normal((257, 3))
    degrees = (12, 14)
    calcs = {l: sb.SphericalHarmonics(l) for l in degrees}
    want = {l: oracle_mod.port_compute(xyz_np, l, True, 1) for l in degrees}
    errors, results = [], {}

    def work(tid):
        try:
            torch.cuda.set_device(dev)
            stream = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(stream):
                xyz = torch.from_numpy(xyz_np).to(dev)
                for it in range(20):
                    l = degrees[(tid + it) % 2]
                    out = calcs[l].compute_with_gradients(xyz)
            stream.synchronize()
            results[tid] = (l, out)
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for l, out in results.values():
        for got, ref in zip(out, want[l]):
            err, bad = oracle_mod.scaled_error(got.cpu().numpy(), ref, l)
            assert bad == 0 and err <= 1e-12
