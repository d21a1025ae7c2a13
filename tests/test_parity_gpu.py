"""Parity of the CUDA library with the reference CPU implementation. Every call goes through
the C ABI (``libsphericart_b200.so`` via ctypes). The checker is the reference's own CPU library
when its build travelled with the tree (``oracle/_ref``), the CPU restatement otherwise; the
committed golden vectors are checked in either case.

Tolerances (the stated bar): 1e-12 for float64 and 1e-5 for float32, relative to the largest
|reference| in the same degree block of the same point; NaN positions must coincide.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {np.dtype(np.float64): 1e-12, np.dtype(np.float32): 1e-5}
SENTINEL = 1234567.0


@pytest.fixture(scope="module")
def sb():
    import sphericart_b200

    return sphericart_b200


def _reference(oracle_mod, xyz, l_max, normalized, level):
    if oracle_mod.have_ref():
        return oracle_mod.ref_compute(xyz, l_max, normalized, level)
    return oracle_mod.port_compute(xyz, l_max, normalized, level)


def _classes(sb):
    return ((sb.SphericalHarmonics, True), (sb.SolidHarmonics, False))


def _run_guarded(calc, xyz_np, level, misalign=0):
    """Runs the calculator into buffers surrounded by guard bands; returns outputs as numpy.
    ``misalign`` shifts every output by that many elements to force the unaligned copy-out path."""
    dev = torch.device("cuda", 0)
    n = xyz_np.shape[0]
    ny = (calc.l_max + 1) ** 2
    tdtype = torch.float64 if xyz_np.dtype == np.float64 else torch.float32
    xyz = torch.from_numpy(xyz_np).to(dev)
    pad = 4096 + misalign
    outs, raws = [], []
    for comps in (1, 3, 9)[: level + 1]:
        raw = torch.full((n * comps * ny + 2 * pad,), SENTINEL, dtype=tdtype, device=dev)
        raws.append(raw)
        outs.append(raw[pad: pad + n * comps * ny])
    ptrs = [o.data_ptr() for o in outs] + [None, None]
    calc.compute_raw(tdtype, level, xyz.data_ptr(), n, ptrs[0], ptrs[1], ptrs[2],
                     torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize(dev)
    for raw in raws:
        assert bool((raw[:pad] == SENTINEL).all()) and bool((raw[-pad:] == SENTINEL).all()), "guard band overwritten"
    shapes = [(n, ny), (n, 3, ny), (n, 3, 3, ny)]
    return [o.cpu().numpy().reshape(shapes[i]) for i, o in enumerate(outs)]


def _assert_close(oracle_mod, got, want, l_max, dtype, what):
    for name, a, b in zip(("sph", "dsph", "ddsph"), got, want):
        if b is None:
            continue
        err, bad = oracle_mod.scaled_error(a, b, l_max)
        assert bad == 0, (what, name, "NaN/inf pattern differs", bad)
        assert err <= TOL[np.dtype(dtype)], (what, name, err)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("level", [0, 1, 2])
def test_all_degrees_small(sb, oracle_mod, dtype, level):
    """l_max 0..21, 24 for both classes (the tile kernels end at 20; every degree with its own measured panel
    shape is in the list); sizes around the 32-point tile; guard bands intact."""
    rng = np.random.default_rng(42 + level)
    for cls, normalized in _classes(sb):
        for l_max in list(range(0, 22)) + [24]:
            calc = cls(l_max)
            for n in (1, 2, 31, 32, 33, 95, 257):
                xyz = (rng.standard_normal((n, 3)) * 1.7).astype(dtype)
                got = _run_guarded(calc, xyz, level)
                want = _reference(oracle_mod, xyz, l_max, normalized, level)
                _assert_close(oracle_mod, got, want, l_max, dtype, (cls.__name__, l_max, level, n))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_unaligned_outputs_take_the_plain_store_path(sb, oracle_mod, dtype):
    rng = np.random.default_rng(9)
    for cls, normalized in _classes(sb):
        for l_max in (3, 6, 7, 8):  # 3 and 7: padded rows in the tile images
            calc = cls(l_max)
            xyz = rng.standard_normal((1000, 3)).astype(dtype)
            for level in (0, 1, 2):
                got = _run_guarded(calc, xyz, level, misalign=1)
                want = _reference(oracle_mod, xyz, l_max, normalized, level)
                _assert_close(oracle_mod, got, want, l_max, dtype, (cls.__name__, l_max, level, "misaligned"))


def test_high_degree_float64(sb, oracle_mod):
    rng = np.random.default_rng(77)
    for cls, normalized in _classes(sb):
        for l_max, level, n in ((32, 1, 300), (32, 2, 70), (50, 2, 9), (50, 0, 40)):
            xyz = rng.standard_normal((n, 3))
            got = _run_guarded(cls(l_max), xyz, level)
            want = _reference(oracle_mod, xyz, l_max, normalized, level)
            _assert_close(oracle_mod, got, want, l_max, np.float64, (cls.__name__, l_max, level))


def test_golden_vectors(sb, oracle_mod, golden):
    """The committed outputs of the reference CPU library, corner cases included (origin, r = 1e-9,
    points on the axes)."""
    n_cases = 0
    for key in golden.files:
        if not (key.endswith("_sph_A") or key.endswith("_sph_B")):
            continue
        cls_name, dt, l, lv, _, tag = key.split("_")
        l_max, level = int(l[1:]), int(lv[2:])
        dtype = np.float64 if dt == "f64" else np.float32
        cls = sb.SphericalHarmonics if cls_name == "spherical" else sb.SolidHarmonics
        xyz = golden[f"xyz_{tag}"].astype(dtype)
        got = _run_guarded(cls(l_max), xyz, level)
        base = f"{cls_name}_{dt}_l{l_max}_lv{level}"
        want = [golden[f"{base}_sph_{tag}"], golden[f"{base}_dsph_{tag}"],
                golden[f"{base}_ddsph_{tag}"] if level == 2 else None]
        _assert_close(oracle_mod, got, want, l_max, dtype, base)
        n_cases += 1
    assert n_cases >= 60


def test_origin_and_tiny_radius_convention(sb):
    """Normalised harmonics: at the origin Y_00 is finite and everything else is NaN; any
    representable radius gives finite values with |dY| ~ l/r. Solid harmonics stay finite."""
    dev = torch.device("cuda", 0)
    for dtype in (torch.float32, torch.float64):
        xyz = torch.tensor([[0.0, 0.0, 0.0], [3e-9, -4e-9, 0.0], [0.0, 0.0, 2.0]], dtype=dtype, device=dev)
        for l_max in (4, 8, 12):
            sph, dsph, ddsph = sb.SphericalHarmonics(l_max).compute_with_hessians(xyz)
            assert torch.isfinite(sph[0, 0]) and abs(float(sph[0, 0]) - 0.282094791773878) < 1e-6
            assert torch.isnan(sph[0, 1:]).all() and torch.isnan(dsph[0]).all() and torch.isnan(ddsph[0]).all()
            assert torch.isfinite(sph[1:]).all() and torch.isfinite(dsph[1:]).all() and torch.isfinite(ddsph[1:]).all()
            assert float(dsph[1].abs().max()) > 1e7
            s, d, h = sb.SolidHarmonics(l_max).compute_with_hessians(xyz)
            assert torch.isfinite(s).all() and torch.isfinite(d).all() and torch.isfinite(h).all()


CONFIG_SAMPLES = [("cfg1", 10_000), ("cfg2", 100_000), ("cfg3", 20_000), ("cfg5", 20_000), ("metric", 100_000)]


@pytest.mark.parametrize("config,n", CONFIG_SAMPLES)
def test_benchmark_configurations_sampled(sb, oracle_mod, config, n):
    """Each benchmark configuration's distribution, at a size the CPU checker finishes in seconds."""
    from sphericart_b200 import workloads

    wl, _ = workloads.CONFIGS[config]
    xyz = workloads.make_points(config, n_points=n)
    cls = sb.SphericalHarmonics if wl.normalized else sb.SolidHarmonics
    got = _run_guarded(cls(wl.l_max), xyz, wl.level)
    want = _reference(oracle_mod, xyz, wl.l_max, wl.normalized, wl.level)
    _assert_close(oracle_mod, got, want, wl.l_max, wl.np_dtype, config)
    if config == "cfg5":
        assert np.isnan(want[0]).any(), "the stress sample must contain origin points"


def _vjp_reference(oracle_mod, xyz, g, l_max, normalized):
    """What the reference's backward computes (gradients, then product and sum:
    sphericart-torch/python/sphericart/torch/register.py:90-108), with the sum taken in float64:
    the checker's gradients in the precision of the input - beyond l_max = 18 the float32 prefactors
    of the reference's own recipe lose bits (1 / (2 l)! leaves the normal range), and parity is with
    the reference in the same precision - contracted in float64."""
    _, dsph, _ = _reference(oracle_mod, xyz, l_max, normalized, 1)
    dsph = dsph.astype(np.float64)
    want = np.einsum("nak,nk->na", dsph, g.astype(np.float64))
    scale = np.einsum("nak,nk->na", np.abs(dsph), np.abs(g.astype(np.float64))).max(axis=1, keepdims=True)
    return want, np.maximum(scale, 1e-300)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_fused_vjp(sb, oracle_mod, dtype):
    """The fused backward against gradient-then-contract, scaled by sum_k |g_k dY_k| per point."""
    rng = np.random.default_rng(4)
    dev = torch.device("cuda", 0)
    tol = 1e-12 if dtype == np.float64 else 1e-5
    for cls, normalized in _classes(sb):
        for l_max in list(range(0, 15)) + [16, 19, 20, 21, 24]:  # tile kernels up to 13 / 19 / 20, band kernel beyond
            for n in (1, 33, 1000):
                xyz = (rng.standard_normal((n, 3)) * 1.4).astype(dtype)
                g = rng.standard_normal((n, (l_max + 1) ** 2)).astype(dtype)
                got = cls(l_max).compute_vjp(torch.from_numpy(xyz).to(dev), torch.from_numpy(g).to(dev)).cpu().numpy()
                want, scale = _vjp_reference(oracle_mod, xyz, g, l_max, normalized)
                assert (np.abs(got - want) / scale).max() <= tol, (cls.__name__, l_max, n)


def test_config4_forward_and_vjp_sampled(sb, oracle_mod):
    from sphericart_b200 import workloads

    n = 200_000
    xyz = workloads.make_points("cfg4", n_points=n)
    g = workloads.make_upstream_grad("cfg4", n_points=n)
    dev = torch.device("cuda", 0)
    calc = sb.SphericalHarmonics(4)
    t_xyz = torch.from_numpy(xyz).to(dev).requires_grad_(True)
    sph = calc(t_xyz)
    sph.backward(torch.from_numpy(g).to(dev))
    want_sph = _reference(oracle_mod, xyz, 4, True, 0)[0]
    err, bad = oracle_mod.scaled_error(sph.detach().cpu().numpy(), want_sph, 4)
    assert bad == 0 and err <= 1e-5
    want, scale = _vjp_reference(oracle_mod, xyz, g, 4, True)
    assert (np.abs(t_xyz.grad.cpu().numpy() - want) / scale).max() <= 1e-5


def test_autograd_gradcheck(sb):
    """As the reference's sphericart-torch/python/tests/test_autograd.py:10-47 (first order)."""
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    xyz = (6 * torch.randn(20, 3, dtype=torch.float64, device=dev)).requires_grad_(True)
    for cls in (sb.SphericalHarmonics, sb.SolidHarmonics):
        calc = cls(4)
        assert torch.autograd.gradcheck(lambda t: calc(t), (xyz,), fast_mode=True)


def test_streams_and_empty_inputs(sb, oracle_mod):
    """Non-default streams give the same numbers (sphericart-torch/python/tests/test_cuda_stream.py);
    zero points return empty outputs for any l_max (python/tests/test_corner_cases.py:7-17)."""
    dev = torch.device("cuda", 0)
    xyz = torch.randn(5000, 3, dtype=torch.float64, device=dev)
    calc = sb.SphericalHarmonics(6)
    base = calc.compute_with_gradients(xyz)
    for _ in range(2):
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            other = calc.compute_with_gradients(xyz)
        s.synchronize()
        assert torch.equal(base[0], other[0]) and torch.equal(base[1], other[1])
    for l_max in (0, 3, 7, 10, 20, 50):
        empty = torch.empty((0, 3), dtype=torch.float32, device=dev)
        sph, dsph, ddsph = sb.SolidHarmonics(l_max).compute_with_hessians(empty)
        ny = (l_max + 1) ** 2
        assert sph.shape == (0, ny) and dsph.shape == (0, 3, ny) and ddsph.shape == (0, 3, 3, ny)


def test_errors_are_reported_not_fatal(sb):
    """Null outputs and host pointers fail with a message through the status-returning entry points."""
    dev = torch.device("cuda", 0)
    calc = sb.SphericalHarmonics(3)
    xyz = torch.randn(10, 3, device=dev)
    sph = torch.empty(10, 16, device=dev)
    with pytest.raises(RuntimeError, match="sph"):
        calc.compute_raw(torch.float32, 0, xyz.data_ptr(), 10, None)
    with pytest.raises(RuntimeError, match="dsph"):
        calc.compute_raw(torch.float32, 1, xyz.data_ptr(), 10, sph.data_ptr(), None)
    with pytest.raises(RuntimeError, match="ddsph"):
        calc.compute_raw(torch.float32, 2, xyz.data_ptr(), 10, sph.data_ptr(), sph.data_ptr(), None)
    host = torch.randn(10, 3)
    with pytest.raises(RuntimeError):
        calc.compute_raw(torch.float32, 0, host.data_ptr(), 10, sph.data_ptr())
    # n == 0 returns at once even with null outputs (sphericart/src/sphericart_cuda.cpp:85-89)
    calc.compute_raw(torch.float32, 2, None, 0, None, None, None)
    with pytest.raises(TypeError):
        calc.compute(host)
    # the context is still usable
    assert torch.isfinite(calc.compute(xyz)).all()


def test_host_pipeline_round_trip(sb, oracle_mod):
    """Host buffers in, host buffers out (the end-to-end path the benchmark times)."""
    from sphericart_b200.host_pipeline import HostPipeline

    dev = torch.device("cuda", 0)
    n, l_max = 70_001, 8
    xyz = np.random.default_rng(3).standard_normal((n, 3)).astype(np.float32)
    calc = sb.SphericalHarmonics(l_max)
    pipe = HostPipeline(calc, 1, torch.float32, dev, chunk_points=16384)
    sph = torch.empty((n, 81), dtype=torch.float32, pin_memory=True)
    dsph = torch.empty((n, 3, 81), dtype=torch.float32, pin_memory=True)
    pipe.run(torch.from_numpy(xyz).pin_memory(), [sph, dsph])
    want = _reference(oracle_mod, xyz, l_max, True, 1)
    _assert_close(oracle_mod, [sph.numpy(), dsph.numpy()], want, l_max, np.float32, "host pipeline")


def _vjp2_reference(oracle_mod, xyz, g_sph, g_dsph, l_max, normalized):
    """float64 contraction of the checker's float64 gradients and Hessians."""
    x64 = xyz.astype(np.float64)
    _, dsph, ddsph = _reference(oracle_mod, x64, l_max, normalized, 2)
    want = np.einsum("nak,nabk->nb", g_dsph.astype(np.float64), ddsph)
    scale = np.einsum("nak,nabk->nb", np.abs(g_dsph.astype(np.float64)), np.abs(ddsph))
    if g_sph is not None:
        want = want + np.einsum("nbk,nk->nb", dsph, g_sph.astype(np.float64))
        scale = scale + np.einsum("nbk,nk->nb", np.abs(dsph), np.abs(g_sph.astype(np.float64)))
    return want, np.maximum(scale.max(axis=1, keepdims=True), 1e-300)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_fused_second_order_backward(sb, oracle_mod, dtype):
    """VJP of (values, gradients) in one kernel against Hessian-then-contract
    (sphericart-torch/python/sphericart/torch/register.py:117-145), scaled by sum |g| |ddY| per point."""
    rng = np.random.default_rng(14)
    dev = torch.device("cuda", 0)
    tol = 1e-12 if dtype == np.float64 else 1e-5
    for cls, normalized in _classes(sb):
        for l_max in list(range(0, 12)) + [12, 16]:  # tile kernels up to 10 (float32) / 8 (float64), band kernel beyond
            for n in (1, 33, 500):
                ny = (l_max + 1) ** 2
                xyz = (rng.standard_normal((n, 3)) * 1.4).astype(dtype)
                g_sph = rng.standard_normal((n, ny)).astype(dtype)
                g_dsph = rng.standard_normal((n, 3, ny)).astype(dtype)
                calc = cls(l_max)
                t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
                for with_values in (True, False):
                    got = calc.compute_vjp_with_gradients(t(xyz), t(g_sph) if with_values else None, t(g_dsph))
                    want, scale = _vjp2_reference(oracle_mod, xyz, g_sph if with_values else None, g_dsph, l_max,
                                                  normalized)
                    assert (np.abs(got.cpu().numpy() - want) / scale).max() <= tol, (cls.__name__, l_max, n, with_values)


def test_autograd_of_values_and_gradients(sb):
    """gradcheck of the (values, gradients) map, as the reference checks its with_gradients op
    (sphericart-torch/python/tests/test_autograd.py:126-146)."""
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    xyz = (2 * torch.randn(12, 3, dtype=torch.float64, device=dev)).requires_grad_(True)
    for cls in (sb.SphericalHarmonics, sb.SolidHarmonics):
        for l_max in (3, 10):
            calc = cls(l_max)
            assert torch.autograd.gradcheck(lambda t: calc.forward_with_gradients(t), (xyz,), fast_mode=True)


def test_calls_can_be_recorded_in_a_cuda_graph(sb):
    """After one ordinary call per calculator, kind of output and device (which builds the per-device
    tables and kernel attributes), compute calls only enqueue kernels: recorded into a CUDA graph
    and replayed on new input data they give the results of ordinary calls."""
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(5)
    n = 5000
    cases = [(sb.SphericalHarmonics(8), torch.float32, 1), (sb.SolidHarmonics(12), torch.float64, 1),
             (sb.SphericalHarmonics(4), torch.float32, 0)]
    for calc, tdtype, level in cases:
        ny = (calc.l_max + 1) ** 2
        xyz = torch.from_numpy(rng.standard_normal((n, 3))).to(dev, tdtype)
        grad = torch.from_numpy(rng.standard_normal((n, ny))).to(dev, tdtype)
        outs = [torch.zeros(s, dtype=tdtype, device=dev) for s in [(n, ny), (n, 3, ny)][: level + 1]]
        xyz_grad = torch.zeros((n, 3), dtype=tdtype, device=dev)
        ptrs = [o.data_ptr() for o in outs] + [None, None]

        def enqueue(stream):
            calc.compute_raw(tdtype, level, xyz.data_ptr(), n, ptrs[0], ptrs[1], None, stream.cuda_stream)
            calc.compute_vjp_raw(tdtype, xyz.data_ptr(), n, grad.data_ptr(), xyz_grad.data_ptr(), stream.cuda_stream)

        enqueue(torch.cuda.current_stream(dev))  # ordinary first call
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            enqueue(torch.cuda.current_stream(dev))
        for _ in range(2):
            xyz.copy_(torch.from_numpy(rng.standard_normal((n, 3))).to(dev, tdtype))
            for o in outs:
                o.zero_()
            xyz_grad.zero_()
            graph.replay()
            torch.cuda.synchronize(dev)
            replayed = [o.clone() for o in outs] + [xyz_grad.clone()]
            enqueue(torch.cuda.current_stream(dev))
            torch.cuda.synchronize(dev)
            for a, b in zip(replayed, outs + [xyz_grad]):
                assert torch.equal(a, b)


def test_cuda_array_interface_inputs(sb):
    """Any array that exposes ``__cuda_array_interface__`` (CuPy, Numba) is accepted in place, as the
    reference's front end accepts CuPy arrays (python/src/sphericart/spherical_harmonics.py:140-178).
    CuPy is not installed here, so a minimal stand-in carries the interface of a torch tensor."""

    class DeviceArray:
        def __init__(self, tensor):
            self._keep = tensor
            self.__cuda_array_interface__ = tensor.__cuda_array_interface__

    torch.manual_seed(2)
    xyz = torch.randn(77, 3, dtype=torch.float64, device="cuda")
    calc = sb.SolidHarmonics(5)
    want = calc.compute_with_gradients(xyz)
    got = calc.compute_with_gradients(DeviceArray(xyz))
    for a, b in zip(got, want):
        assert torch.equal(torch.as_tensor(a, device="cuda"), b)
    with pytest.raises(TypeError):
        calc.compute(xyz.cpu().numpy())


def test_out_buffers_of_the_python_front_end(sb, oracle_mod):
    """Caller-provided output tensors (``out=``): filled in place with the same results, and refused
    when they do not match the call."""
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(31)
    xyz_np = rng.standard_normal((100, 3))
    xyz = torch.from_numpy(xyz_np).to(dev)
    for cls, normalized in _classes(sb):
        calc = cls(5)
        out = (torch.empty((100, 36), dtype=torch.float64, device=dev),
               torch.empty((100, 3, 36), dtype=torch.float64, device=dev))
        sph, dsph = calc.compute_with_gradients(xyz, out=out)
        assert sph.data_ptr() == out[0].data_ptr() and dsph.data_ptr() == out[1].data_ptr()
        want = _reference(oracle_mod, xyz_np, 5, normalized, 1)
        _assert_close(oracle_mod, [sph.cpu().numpy(), dsph.cpu().numpy()], want[:2], 5, np.float64, "out=")
        g = torch.from_numpy(rng.standard_normal((100, 36))).to(dev)
        buf = torch.empty((100, 3), dtype=torch.float64, device=dev)
        assert calc.compute_vjp(xyz, g, out=buf).data_ptr() == buf.data_ptr()
        assert torch.allclose(buf, torch.einsum("nak,nk->na", dsph, g), rtol=1e-11, atol=1e-12)
        with pytest.raises(ValueError):
            calc.compute_with_gradients(xyz, out=out[:1])
        with pytest.raises(ValueError):
            calc.compute(xyz, out=torch.empty((100, 35), dtype=torch.float64, device=dev))
        with pytest.raises(ValueError):
            calc.compute(xyz, out=torch.empty((100, 36), dtype=torch.float32, device=dev))
        with pytest.raises(ValueError):
            calc.compute(xyz, out=torch.empty((100, 36), dtype=torch.float64))
        with pytest.raises(ValueError):
            calc.compute_vjp(xyz, g, out=torch.empty((3, 100), dtype=torch.float64, device=dev).t())
