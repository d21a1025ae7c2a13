"""CPU-side checks of the drop-in boundary: the shared library loads, exports every function
the C header declares and the C++ calculator symbols, keeps the reference's object layout, and
fails loudly (no fallback) when there is no GPU."""

import os
import re
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sphericart_b200.h")


def _reference_header_dir():
    from oracle import oracle

    root = oracle.reference_root()
    return None if root is None else os.path.join(root, "sphericart", "include")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"SPHERICART_EXPORT\s+[\w\s\*]+?\b(sphericart_cuda_\w+)\s*\(", text)


def test_library_exports_every_declared_function():
    from sphericart_b200 import _c_lib

    lib = _c_lib.get_library()
    declared = _declared_functions()
    assert len(declared) == 52, declared
    for name in declared:
        assert getattr(lib, name) is not None
    assert sorted(declared) == sorted(_c_lib.exported_names())


def test_header_cites_the_reference_for_every_reference_entry_point():
    text = open(HEADER).read()
    for kind in ("spherical", "solid"):
        for sfx in ("", "_f"):
            for fn in ("new", "delete", "compute_array", "compute_array_with_gradients", "compute_array_with_hessians"):
                name = f"sphericart_cuda_{kind}_harmonics_{fn}{sfx}("
                idx = text.index(name)
                preceding = text[max(0, idx - 200):idx]
                assert "replaces sphericart/include/sphericart.h:" in preceding, name


def test_cxx_calculator_symbols_are_exported():
    from sphericart_b200 import _c_lib

    out = subprocess.run(["nm", "-DC", "--defined-only", _c_lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    for cls in ("SphericalHarmonics", "SolidHarmonics"):
        for t in ("float", "double"):
            assert f"sphericart::cuda::{cls}<{t}>::{cls}(unsigned long)" in out
    for t in ("float", "double"):
        for method in ("compute(", "compute_with_gradients(", "compute_with_hessians(", "compute_vjp("):
            assert f"sphericart::cuda::SphericalHarmonics<{t}>::{method}" in out


def test_object_layout_matches_the_reference_header(tmp_path):
    """Bindings built against the reference header allocate the calculators themselves, so size and
    alignment must agree. Needs the reference checkout; skipped where it is absent."""
    reference_header_dir = _reference_header_dir()
    if reference_header_dir is None:
        pytest.skip("reference headers not available on this machine (set SPHERICART_REF)")
    prog = r"""
#include <cstdio>
#include "sphericart_cuda.hpp"
int main() {
    std::printf("%zu %zu %zu %zu\n", sizeof(sphericart::cuda::SphericalHarmonics<float>),
                alignof(sphericart::cuda::SphericalHarmonics<float>),
                sizeof(sphericart::cuda::SolidHarmonics<double>), alignof(sphericart::cuda::SolidHarmonics<double>));
}
"""
    src = tmp_path / "layout.cpp"
    src.write_text(prog)
    results = []
    for inc in (os.path.join(ROOT, "include"), reference_header_dir):
        exe = tmp_path / ("layout_" + str(len(results)))
        subprocess.run(["g++", "-std=c++17", "-I", inc, str(src), "-o", str(exe)], check=True)
        results.append(subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout)
    assert results[0] == results[1], results


def test_front_end_validates_before_touching_the_device():
    import sphericart_b200 as sb

    calc = sb.SphericalHarmonics(3)
    with pytest.raises(TypeError, match="CUDA"):
        calc.compute(torch.zeros(4, 3))
    with pytest.raises(TypeError):
        calc.compute([[0.0, 0.0, 1.0]])
    with pytest.raises(ValueError):
        sb.SolidHarmonics(-1)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_deleted_calculators_refuse_work():
    """python/tests/test_corner_cases.py:20-32: deleting twice is harmless, use after deletion raises."""
    import sphericart_b200

    for cls in (sphericart_b200.SphericalHarmonics, sphericart_b200.SolidHarmonics):
        calc = cls(4)
        calc.__del__()
        calc.__del__()
        with pytest.raises(ValueError, match="can not use a deleted calculator"):
            calc._calculator(torch.float64)


def test_no_gpu_means_failure_not_fallback():
    from sphericart_b200 import _c_lib

    lib = _c_lib.get_library()
    handle = lib.sphericart_cuda_spherical_harmonics_new_f(4)
    assert not handle, "calculator creation must fail without a CUDA device"
    assert "no CPU code path" in _c_lib.last_error()


def test_product_code_never_touches_the_oracle():
    """The checker is test infrastructure: nothing under the package may import or load it."""
    pkg = os.path.join(ROOT, "sphericart_b200")
    for dirpath, _, files in os.walk(pkg):
        if "_build" in dirpath:
            continue
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".hpp", ".h", ".cpp")):
                text = open(os.path.join(dirpath, name)).read()
                assert "oracle" not in text.lower(), (dirpath, name)


def test_torch_operator_library_loads_and_serves_cuda_tensors_only():
    """The operator library registers the reference's six operator schemas (under its own
    namespace) plus the fused backward operators; without a GPU nothing can be computed, and a CPU
    tensor is refused by the dispatcher rather than served by some other path."""
    import torch

    import sphericart_b200.torch_ops as t

    for prefix in ("spherical_harmonics", "solid_harmonics"):
        assert str(getattr(t.ops, prefix).default._schema) == f"sphericart_b200::{prefix}(Tensor xyz, int l_max) -> Tensor"
        assert str(getattr(t.ops, prefix + "_with_gradients").default._schema).endswith("-> (Tensor, Tensor)")
        assert str(getattr(t.ops, prefix + "_with_hessians").default._schema).endswith("-> (Tensor, Tensor, Tensor)")
        assert "Tensor? sph_grad" in str(getattr(t.ops, prefix + "_vjp_with_gradients").default._schema)
    with pytest.raises(NotImplementedError):
        t.ops.spherical_harmonics(torch.zeros(4, 3), 3)
    # shape inference needs no device
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(10, 3, device="cuda")
        shapes = [tuple(o.shape) for o in t.ops.solid_harmonics_with_hessians(x, 4)]
        assert shapes == [(10, 25), (10, 3, 25), (10, 3, 3, 25)]
        assert tuple(t.ops.spherical_harmonics_vjp(x, torch.empty(10, 25, device="cuda"), 4).shape) == (10, 3)


def test_gpulite_stand_in_compiles_and_checks(tmp_path):
    """``include/gpulite/gpulite.hpp`` is what lets the reference's JAX binding
    (sphericart-jax/src/sphericart_jax_cuda.cpp:15,83,127,177) compile against this library without
    the run-time loader it normally uses: the macro passes a successful call through and turns a
    failing one into an exception that names the error. Needs no GPU: the macro is given status
    values directly."""
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    if not os.path.exists(os.path.join(cuda_home, "include", "cuda_runtime_api.h")):
        pytest.skip("CUDA toolkit headers not found")
    prog = r"""
#include <gpulite/gpulite.hpp>
#include <cstdio>
#include <cstring>
int main() {
    cudaStream_t stream = nullptr;             // the types the binding uses come with the header
    cudaPointerAttributes attributes;
    (void)stream; (void)attributes;
    int thrown = 0;
    try {
        GPULITE_CUDART_CALL(cudaErrorInvalidValue);   // any expression of type cudaError_t
    } catch (const std::runtime_error& e) {
        thrown = std::strstr(e.what(), "cudaErrorInvalidValue") != nullptr;
    }
    GPULITE_CUDART_CALL(cudaSuccess);
    std::printf("%d\n", thrown);
    return thrown ? 0 : 1;
}
"""
    src = tmp_path / "shim.cpp"
    src.write_text(prog)
    exe = tmp_path / "shim"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda_home, "include"),
                    str(src), "-L", os.path.join(cuda_home, "lib64"), "-lcudart", "-o", str(exe)], check=True)
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.join(cuda_home, "lib64") + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    out = subprocess.run([str(exe)], capture_output=True, text=True, env=env)
    assert out.returncode == 0 and out.stdout.strip() == "1", out.stdout + out.stderr
