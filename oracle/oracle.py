"""ctypes access to the two CPU checkers. TEST INFRASTRUCTURE ONLY.

``port``  : the C restatement in ``sph_oracle.c`` (``libsph_oracle.so``), always buildable.
``ref``   : the reference's own CPU library compiled from its sources by ``oracle/Makefile``
            into ``oracle/_ref/libsphericart_ref.so``; present only where it was built (the
            built file travels with the working tree, the reference sources do not).

Only the tests, the smoke check and the benchmark's CPU-baseline legs import this module.
The CUDA library and its Python front end never do.
"""

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_PATH = os.path.join(_HERE, "libsph_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libsphericart_ref.so")

_port = None
_ref = None


def reference_root():
    """Where the reference's source tree is: ``$SPHERICART_REF``, else a checkout named
    ``reference`` beside this repository; ``None`` when neither has the reference's headers (the
    prebuilt files under ``oracle/_ref`` are then used as they are)."""
    candidates = [os.environ.get("SPHERICART_REF"),
                  os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for root in candidates:
        if root and os.path.exists(os.path.join(root, "sphericart", "include", "templates.hpp")):
            return os.path.abspath(root)
    return None


def build(quiet=True):
    """Compile the restatement (and the reference library when its sources are reachable)."""
    ref = reference_root()
    out = subprocess.run(["make", "-C", _HERE] + ([f"REF={ref}"] if ref else []), capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def use_all_host_threads():
    """Make OpenMP use every core this process may run on, whatever OMP_NUM_THREADS says (launchers
    such as torchrun export OMP_NUM_THREADS=1 to their workers). Call before creating a
    calculator: the reference sizes its per-thread buffers from omp_get_max_threads() at
    construction (sphericart/src/sphericart.cpp:36). Returns the thread count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    load_port()  # pulls in libgomp
    gomp = ctypes.CDLL("libgomp.so.1")
    gomp.omp_set_num_threads(ctypes.c_int(n))
    return n


def _ctype(dtype):
    return ctypes.c_double if np.dtype(dtype) == np.float64 else ctypes.c_float


def _ptr(arr):
    if arr is None:
        return None
    return arr.ctypes.data_as(ctypes.c_void_p)


def load_port():
    global _port
    if _port is None:
        if not os.path.exists(_PORT_PATH):
            build()
        lib = ctypes.CDLL(_PORT_PATH)
        for sfx in ("f64", "f32"):
            f = getattr(lib, f"sph_oracle_compute_{sfx}")
            f.restype = ctypes.c_int
            f.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
            f = getattr(lib, f"sph_oracle_vjp_{sfx}")
            f.restype = ctypes.c_int
            f.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                          ctypes.c_void_p, ctypes.c_int]
            f = getattr(lib, f"sph_oracle_prefactors_{sfx}")
            f.restype = None
            f.argtypes = [ctypes.c_int, ctypes.c_void_p]
        _port = lib
    return _port


def have_ref():
    return os.path.exists(_REF_PATH)


def load_ref():
    """The reference's CPU C API (sphericart/include/sphericart.h:118-639)."""
    global _ref
    if _ref is None:
        if not have_ref():
            return None
        lib = ctypes.CDLL(_REF_PATH)
        for kind in ("spherical", "solid"):
            for sfx in ("", "_f"):
                base = f"sphericart_{kind}_harmonics"
                getattr(lib, f"{base}_new{sfx}").restype = ctypes.c_void_p
                getattr(lib, f"{base}_new{sfx}").argtypes = [ctypes.c_size_t]
                getattr(lib, f"{base}_delete{sfx}").restype = None
                getattr(lib, f"{base}_delete{sfx}").argtypes = [ctypes.c_void_p]
                getattr(lib, f"{base}_omp_num_threads{sfx}").restype = ctypes.c_int
                getattr(lib, f"{base}_omp_num_threads{sfx}").argtypes = [ctypes.c_void_p]
                for nout, name in ((1, "compute_array"), (2, "compute_array_with_gradients"),
                                   (3, "compute_array_with_hessians")):
                    f = getattr(lib, f"{base}_{name}{sfx}")
                    f.restype = None
                    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t] + \
                        [ctypes.c_void_p, ctypes.c_size_t] * nout
        _ref = lib
    return _ref


def _alloc(n, ny, level, dtype):
    sph = np.empty((n, ny), dtype=dtype)
    dsph = np.empty((n, 3, ny), dtype=dtype) if level >= 1 else None
    ddsph = np.empty((n, 3, 3, ny), dtype=dtype) if level >= 2 else None
    return sph, dsph, ddsph


def port_compute(xyz, l_max, normalized, level, nthreads=0, out=None):
    """Run the restatement. Returns (sph, dsph|None, ddsph|None)."""
    xyz = np.ascontiguousarray(xyz)
    assert xyz.dtype in (np.float32, np.float64) and xyz.ndim == 2 and xyz.shape[1] == 3
    lib = load_port()
    n = xyz.shape[0]
    ny = (l_max + 1) ** 2
    sph, dsph, ddsph = out if out is not None else _alloc(n, ny, level, xyz.dtype)
    sfx = "f64" if xyz.dtype == np.float64 else "f32"
    getattr(lib, f"sph_oracle_compute_{sfx}")(l_max, int(bool(normalized)), level, _ptr(xyz), n,
                                             _ptr(sph), _ptr(dsph), _ptr(ddsph), nthreads)
    return sph, dsph, ddsph


def port_vjp(xyz, sph_grad, l_max, normalized, nthreads=0):
    xyz = np.ascontiguousarray(xyz)
    sph_grad = np.ascontiguousarray(sph_grad)
    lib = load_port()
    n = xyz.shape[0]
    out = np.empty((n, 3), dtype=xyz.dtype)
    sfx = "f64" if xyz.dtype == np.float64 else "f32"
    getattr(lib, f"sph_oracle_vjp_{sfx}")(l_max, int(bool(normalized)), _ptr(xyz), _ptr(sph_grad), n,
                                         _ptr(out), nthreads)
    return out


def port_prefactors(l_max, dtype):
    nq = (l_max + 1) * (l_max + 2) // 2
    out = np.empty(2 * nq, dtype=dtype)
    sfx = "f64" if np.dtype(dtype) == np.float64 else "f32"
    getattr(load_port(), f"sph_oracle_prefactors_{sfx}")(l_max, _ptr(out))
    return out


class RefCalculator:
    """One reference CPU calculator (``sphericart::SphericalHarmonics<T>`` or
    ``SolidHarmonics<T>`` behind the reference C API)."""

    def __init__(self, l_max, normalized, dtype):
        self.lib = load_ref()
        if self.lib is None:
            raise RuntimeError("reference CPU library has not been built (oracle/_ref)")
        self.l_max = l_max
        self.dtype = np.dtype(dtype)
        self.sfx = "" if self.dtype == np.float64 else "_f"
        self.base = f"sphericart_{'spherical' if normalized else 'solid'}_harmonics"
        self.handle = getattr(self.lib, f"{self.base}_new{self.sfx}")(l_max)
        if not self.handle:
            raise RuntimeError("reference calculator construction failed")

    def omp_num_threads(self):
        return getattr(self.lib, f"{self.base}_omp_num_threads{self.sfx}")(self.handle)

    def compute(self, xyz, level, out=None):
        xyz = np.ascontiguousarray(xyz, dtype=self.dtype)
        n = xyz.shape[0]
        ny = (self.l_max + 1) ** 2
        sph, dsph, ddsph = out if out is not None else _alloc(n, ny, level, self.dtype)
        name = ("compute_array", "compute_array_with_gradients", "compute_array_with_hessians")[level]
        args = [self.handle, _ptr(xyz), xyz.size, _ptr(sph), sph.size]
        if level >= 1:
            args += [_ptr(dsph), dsph.size]
        if level >= 2:
            args += [_ptr(ddsph), ddsph.size]
        getattr(self.lib, f"{self.base}_{name}{self.sfx}")(*args)
        return sph, dsph, ddsph

    def close(self):
        if self.handle:
            getattr(self.lib, f"{self.base}_delete{self.sfx}")(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ref_compute(xyz, l_max, normalized, level):
    calc = RefCalculator(l_max, normalized, xyz.dtype)
    try:
        return calc.compute(xyz, level)
    finally:
        calc.close()


def ref_vjp(xyz, sph_grad, l_max, normalized, chunk=1 << 20):
    """What the reference's autograd backward does on CPU: gradients, then a product and a
    sum over the (l,m) axis (sphericart-torch/python/sphericart/torch/register.py:98-99)."""
    calc = RefCalculator(l_max, normalized, xyz.dtype)
    out = np.empty((xyz.shape[0], 3), dtype=xyz.dtype)
    try:
        for lo in range(0, xyz.shape[0], chunk):
            hi = min(xyz.shape[0], lo + chunk)
            _, dsph, _ = calc.compute(xyz[lo:hi], 1)
            out[lo:hi] = np.einsum("naj,nj->na", dsph, sph_grad[lo:hi])
    finally:
        calc.close()
    return out


def scaled_error(got, want, l_max):
    """Largest |got - want| divided by the per-point, per-l block maximum of |want|.

    ``got`` and ``want`` have the (l,m) axis last. For every point and every degree l the
    scale is the largest |want| over that l block and over all derivative components, which is
    the "relative tolerance scaled by max|Y_l|" the parity bar is stated in. Positions where
    ``want`` is NaN must be NaN in ``got`` and vice versa; infinities must agree in sign.
    The scale is floored at the smallest normal number of ``want``'s dtype: below it results
    are denormal and only absolutely, not relatively, accurate.
    Returns (max_scaled_error, nan_mismatches).
    """
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, (got.shape, want.shape)
    n = want.shape[0]
    ny = want.shape[-1]
    g = got.reshape(n, -1, ny).astype(np.float64)
    w = want.reshape(n, -1, ny).astype(np.float64)
    nan_mismatch = int(np.count_nonzero(np.isnan(g) != np.isnan(w)))
    inf_w = np.isinf(w)
    inf_mismatch = int(np.count_nonzero(inf_w & (g != w))) + int(np.count_nonzero(np.isinf(g) & ~inf_w))
    finite = np.isfinite(w) & np.isfinite(g)
    worst = 0.0
    tiny = float(np.finfo(want.dtype if want.dtype.kind == "f" else np.float64).tiny)
    for l in range(l_max + 1):
        sl = slice(l * l, (l + 1) * (l + 1))
        wb = w[:, :, sl]
        gb = g[:, :, sl]
        fb = finite[:, :, sl]
        scale = np.where(fb, np.abs(wb), 0.0).max(axis=(1, 2), keepdims=True)
        scale = np.maximum(scale, tiny)
        err = np.where(fb, np.abs(gb - wb), 0.0) / scale
        if err.size:
            worst = max(worst, float(err.max()))
    return worst, nan_mismatch + inf_mismatch
