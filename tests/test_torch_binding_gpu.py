"""The reference's own, unmodified torch binding (sphericart-torch/src/torch.cpp) compiled against
the reference's headers and linked against this library: its CUDA ops must give what its CPU ops
give. These are the reference's GPU tests (sphericart-torch/python/tests/test_cuda.py,
test_cuda_stream.py, test_no_points.py; python/tests/test_cupy.py for the float32 tolerances) run
through ``torch.ops.sphericart_torch``. The binding is built by ``oracle/Makefile`` where the
reference checkout is available; elsewhere its absence skips this file."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINDING = os.path.join(ROOT, "oracle", "_ref", "libsphericart_torch_binding.so")


@pytest.fixture(scope="module")
def ops():
    if not os.path.exists(BINDING):
        pytest.skip("the reference torch binding has not been built on this machine")
    torch.ops.load_library(BINDING)
    return torch.ops.sphericart_torch


def _ops_for(ops, kind):
    return (getattr(ops, f"{kind}_harmonics"), getattr(ops, f"{kind}_harmonics_with_gradients"),
            getattr(ops, f"{kind}_harmonics_with_hessians"))


@pytest.mark.parametrize("kind", ["spherical", "solid"])
def test_cpu_vs_cuda_lmax20_float64(ops, kind):
    """sphericart-torch/python/tests/test_cuda.py:15-31."""
    torch.manual_seed(0)
    xyz = 6 * torch.randn(100, 3, dtype=torch.float64)
    values, gradients, _ = _ops_for(ops, kind)
    sph_cpu, dsph_cpu = gradients(xyz, 20)
    sph_gpu, dsph_gpu = gradients(xyz.cuda(), 20)
    assert sph_gpu.is_cuda and dsph_gpu.shape == (100, 3, 441)
    assert torch.allclose(sph_cpu, sph_gpu.cpu())
    assert torch.allclose(dsph_cpu, dsph_gpu.cpu())
    assert torch.allclose(values(xyz, 20), values(xyz.cuda(), 20).cpu())


@pytest.mark.parametrize("kind", ["spherical", "solid"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_cpu_vs_cuda_hessians_lmax4(ops, kind, dtype):
    """python/tests/test_cupy.py:26-49: rtol = atol = 1e-5 (float32), 1e-12 (float64)."""
    torch.manual_seed(0)
    xyz = torch.randn(8, 3, dtype=dtype)
    _, _, hessians = _ops_for(ops, kind)
    tol = 1e-5 if dtype == torch.float32 else 1e-12
    for a, b in zip(hessians(xyz, 4), hessians(xyz.cuda(), 4)):
        assert torch.allclose(a, b.cpu(), rtol=tol, atol=tol)


def test_streams(ops):
    """sphericart-torch/python/tests/test_cuda_stream.py:15-29."""
    xyz = 6 * torch.randn(100, 3, dtype=torch.float64, device="cuda")
    values, _, _ = _ops_for(ops, "spherical")
    base = values(xyz, 20)
    for _ in range(2):
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            other = values(xyz, 20)
        stream.synchronize()
        assert torch.allclose(base, other)


def test_no_points(ops):
    """sphericart-torch/python/tests/test_no_points.py:10-45."""
    for l_max in (0, 3, 7, 10, 20, 50):
        xyz = torch.empty((0, 3), dtype=torch.float64, device="cuda")
        ny = (l_max + 1) ** 2
        for kind in ("spherical", "solid"):
            values, gradients, hessians = _ops_for(ops, kind)
            assert values(xyz, l_max).shape == (0, ny)
            sph, dsph = gradients(xyz, l_max)
            assert sph.shape == (0, ny) and dsph.shape == (0, 3, ny)
            sph, dsph, ddsph = hessians(xyz, l_max)
            assert ddsph.shape == (0, 3, 3, ny)


def test_non_contiguous_input_and_large_batch(ops):
    values, gradients, _ = _ops_for(ops, "spherical")
    big = torch.randn(3, 200_000, dtype=torch.float32, device="cuda")
    xyz = big.t()  # (200000, 3), not contiguous
    sph, dsph = gradients(xyz, 8)
    ref_sph, ref_dsph = gradients(xyz.cpu(), 8)
    assert torch.allclose(sph.cpu(), ref_sph, rtol=1e-5, atol=1e-5)
    assert torch.allclose(dsph.cpu(), ref_dsph, rtol=2e-5, atol=2e-5 * float(ref_dsph.abs().max()))
