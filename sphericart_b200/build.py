"""Builds ``libsphericart_b200.so`` in-tree with nvcc for sm_100a.

The kernels are instantiated per (type, l_max) and per (type, lanes-per-point) in separate
objects so the compile parallelises; objects are rebuilt only when a source is newer.

    python -m sphericart_b200.build            # build if out of date (CUDA library, then the torch operator library)
    python -m sphericart_b200.build --force
"""

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libsphericart_b200.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I", CSRC, "-I", INCLUDE,
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _units():
    """(object name, source, extra defines)"""
    units = [("sphericart_cuda.o", "sphericart_cuda.cu", [])]
    for tname, t in (("f32", "float"), ("f64", "double")):
        for l in range(0, 21):
            units.append((f"tile_{tname}_l{l}.o", "tile_inst.cu", [f"-DSPH_T={t}", f"-DSPH_LMAX={l}"]))
        for g in (1, 2, 4, 8, 16, 32):
            units.append((f"band_{tname}_g{g}.o", "band_inst.cu", [f"-DSPH_T={t}", f"-DSPH_G={g}"]))
            units.append((f"panel_{tname}_p{g}.o", "panel_inst.cu", [f"-DSPH_T={t}", f"-DSPH_TP={g}"]))
    return units


def _newest_source():
    newest = os.path.getmtime(os.path.abspath(__file__))
    for root in (CSRC, INCLUDE):
        for name in os.listdir(root):
            newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def _compile(unit, force, newest, verbose):
    obj_name, src, defines = unit
    obj = os.path.join(OBJ, obj_name)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj, False
    cmd = [_nvcc()] + NVCC_FLAGS + defines + ["-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    out = subprocess.run(cmd, capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError(f"nvcc failed for {obj_name}:\n{out.stdout}\n{out.stderr}")
    if verbose:
        sys.stderr.write(out.stderr)
    return obj, True


def build(force=False, verbose=False, jobs=None):
    """Compile (if needed) and return the path of the shared library."""
    os.makedirs(OBJ, exist_ok=True)
    newest = _newest_source()
    units = _units()
    jobs = jobs or max(1, (os.cpu_count() or 2))
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        results = list(pool.map(lambda u: _compile(u, force, newest, verbose), units))
    objs = [r[0] for r in results]
    rebuilt = any(r[1] for r in results)
    if rebuilt or force or not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
        out = subprocess.run(cmd, capture_output=True, text=True)
        if out.returncode != 0:
            raise RuntimeError(f"link failed:\n{out.stdout}\n{out.stderr}")
    return LIB


TORCH_OPS_SRC = os.path.join(HERE, "torch_csrc", "torch_ops.cpp")
TORCH_OPS_LIB = os.path.join(HERE, "libsphericart_b200_torch.so")


def build_torch_ops(force=False):
    """Compile (if needed) the PyTorch operator library over ``libsphericart_b200.so`` with the host
    compiler against the installed torch's headers; returns its path."""
    import torch

    build(force=False)
    newest = max(os.path.getmtime(TORCH_OPS_SRC), os.path.getmtime(os.path.join(INCLUDE, "sphericart_cuda.hpp")))
    if not force and os.path.exists(TORCH_OPS_LIB) and os.path.getmtime(TORCH_OPS_LIB) >= newest:
        return TORCH_OPS_LIB
    tdir = os.path.dirname(torch.__file__)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [
        "g++", "-std=c++17", "-O2", "-fPIC", "-shared",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        f"-I{tdir}/include", f"-I{tdir}/include/torch/csrc/api/include", f"-I{cuda_home}/include", f"-I{INCLUDE}",
        TORCH_OPS_SRC, f"-L{HERE}", "-lsphericart_b200", f"-L{tdir}/lib", "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
        "-lc10", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tdir}/lib", "-o", TORCH_OPS_LIB,
    ]
    out = subprocess.run(cmd, capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError(f"building the torch operator library failed:\n{out.stdout}\n{out.stderr}")
    return TORCH_OPS_LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    if "--no-torch-ops" not in sys.argv:
        print(build_torch_ops(force="--force" in sys.argv))
