"""ctypes binding of ``libsphericart_b200.so`` (the C ABI declared in ``include/sphericart_b200.h``).

Plays the role of the reference's ``python/src/sphericart/_c_lib.py:240-400`` for the CUDA half
of the API. There is no fallback: if the library has not been built this raises.
"""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsphericart_b200.so")

_lib = None

_KINDS = ("spherical", "solid")
_SUFFIXES = ("", "_f")


def exported_names():
    """Every function the C header declares, in declaration-family order."""
    names = ["sphericart_cuda_last_error", "sphericart_cuda_kernel_family", "sphericart_cuda_device_wait_errors",
             "sphericart_cuda_harmonics_with_gradients_no_alloc"]
    for kind in _KINDS:
        for sfx in _SUFFIXES:
            base = f"sphericart_cuda_{kind}_harmonics"
            for fn in ("new", "delete", "compute_array", "compute_array_with_gradients",
                       "compute_array_with_hessians", "compute_vjp", "try_compute", "try_compute_vjp",
                       "compute_vjp_with_gradients", "try_compute_vjp_with_gradients",
                       "compute_selected", "compute_selected_vjp"):
                names.append(f"{base}_{fn}{sfx}")
    return names


def get_library():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m sphericart_b200.build` "
            "(there is no CPU or PyTorch fallback)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.sphericart_cuda_last_error.restype = ctypes.c_char_p
    lib.sphericart_cuda_last_error.argtypes = []
    lib.sphericart_cuda_kernel_family.restype = ctypes.c_char_p
    lib.sphericart_cuda_kernel_family.argtypes = [ci, sz, ci]
    lib.sphericart_cuda_device_wait_errors.restype = ci
    lib.sphericart_cuda_device_wait_errors.argtypes = []
    lib.sphericart_cuda_harmonics_with_gradients_no_alloc.restype = ci
    lib.sphericart_cuda_harmonics_with_gradients_no_alloc.argtypes = [ci, sz, vp, sz, vp, vp, vp]
    for kind in _KINDS:
        for sfx in _SUFFIXES:
            base = f"sphericart_cuda_{kind}_harmonics"

            def bind(fn, restype, argtypes):
                f = getattr(lib, f"{base}_{fn}{sfx}")
                f.restype = restype
                f.argtypes = argtypes

            bind("new", vp, [sz])
            bind("delete", None, [vp])
            bind("compute_array", None, [vp, vp, sz, vp, vp])
            bind("compute_array_with_gradients", None, [vp, vp, sz, vp, vp, vp])
            bind("compute_array_with_hessians", None, [vp, vp, sz, vp, vp, vp, vp])
            bind("compute_vjp", None, [vp, vp, sz, vp, vp, vp])
            bind("try_compute", ci, [vp, ci, vp, sz, vp, vp, vp, vp])
            bind("try_compute_vjp", ci, [vp, vp, sz, vp, vp, vp])
            bind("compute_vjp_with_gradients", None, [vp, vp, sz, vp, vp, vp, vp])
            bind("try_compute_vjp_with_gradients", ci, [vp, vp, sz, vp, vp, vp, vp])
            bind("compute_selected", ci, [vp, vp, sz, vp, sz, vp, vp, vp, vp])
            bind("compute_selected_vjp", ci, [vp, vp, sz, vp, sz, vp, vp, vp, vp, vp])
    _lib = lib
    return lib


def last_error():
    msg = get_library().sphericart_cuda_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def kernel_family(kind, l_max, elem_bytes):
    """Name of the kernel family that serves a call (kind 0..2 forward level, 3 VJP, 4 second-order VJP)."""
    return get_library().sphericart_cuda_kernel_family(int(kind), int(l_max), int(elem_bytes)).decode()
