"""Calculators for torch CUDA tensors on top of the C ABI.

Same shape as the reference's array front end (``python/src/sphericart/spherical_harmonics.py:9-245``:
``SphericalHarmonics(l_max).compute / compute_with_gradients / compute_with_hessians``), with
torch CUDA tensors where the reference takes CuPy arrays, plus the fused ``compute_vjp`` and an
autograd-aware ``forward`` that uses it (the reference's backward re-runs the gradients kernel
and reduces with two more kernels: ``sphericart-torch/python/sphericart/torch/register.py:90-108``).

Everything here launches CUDA kernels through ``libsphericart_b200.so``; CPU tensors are
rejected, there is no other code path.
"""

from typing import Optional, Tuple

import torch

from . import _c_lib


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class _BaseHarmonics:
    _prefix = ""
    normalized = True

    def __init__(self, l_max: int):
        if l_max < 0:
            raise ValueError("l_max must be non-negative")
        self._l_max = int(l_max)
        self._lib = _c_lib.get_library()
        self._calculators = {}
        self._deleted = False

    @property
    def l_max(self) -> int:
        return self._l_max

    def __del__(self):
        lib = getattr(self, "_lib", None)
        for dtype, handle in getattr(self, "_calculators", {}).items():
            if handle:
                sfx = "" if dtype == torch.float64 else "_f"
                getattr(lib, f"{self._prefix}_delete{sfx}")(handle)
        self._calculators = {}
        self._deleted = True  # as in the reference front end: deleting twice is fine, using it afterwards is not

    # -- plumbing ---------------------------------------------------------------------------
    def _calculator(self, dtype):
        if self._deleted:
            raise ValueError("can not use a deleted calculator")
        handle = self._calculators.get(dtype)
        if handle is None:
            sfx = "" if dtype == torch.float64 else "_f"
            handle = getattr(self._lib, f"{self._prefix}_new{sfx}")(self._l_max)
            if not handle:
                raise RuntimeError("failed to create the CUDA calculator: " + _c_lib.last_error())
            self._calculators[dtype] = handle
        return handle

    def _validate_xyz(self, xyz):
        if not isinstance(xyz, torch.Tensor):
            if not hasattr(xyz, "__cuda_array_interface__"):
                raise TypeError("xyz must be a torch.Tensor or a CUDA array (CuPy, Numba) on a CUDA device")
            xyz = torch.as_tensor(xyz, device="cuda")  # no copy: the same device memory
        if not xyz.is_cuda:
            raise TypeError("xyz must live on a CUDA device: this library has no CPU code path")
        if xyz.dtype not in (torch.float32, torch.float64):
            raise TypeError("xyz must be a tensor of 32 or 64-bit floats")
        if xyz.dim() != 2 or xyz.shape[1] != 3:
            raise ValueError("xyz tensor must be a `N x 3` array")
        return xyz.detach().contiguous()

    @staticmethod
    def _validate_out(out, xyz, shapes, names=("sph", "dsph", "ddsph"), require_cuda=True):
        """Caller-provided output buffers are handed to the kernels as bare pointers, so everything
        the kernels assume is checked here: one CUDA tensor per requested output, on the device of
        ``xyz``, of its dtype, contiguous and of exactly the output's shape. Returns the buffers padded
        with ``None`` to three entries. (``require_cuda=False`` lets the CPU-only tests reach the other checks.)"""
        if isinstance(out, torch.Tensor):
            out = (out,)
        out = tuple(out)
        if len(out) < len(shapes) or any(t is not None for t in out[len(shapes):]):
            raise ValueError(f"out must hold exactly {len(shapes)} tensor(s) for this call, got {len(out)}")
        for name, t, shape in zip(names, out, shapes):
            if not isinstance(t, torch.Tensor) or (require_cuda and not t.is_cuda):
                raise ValueError(f"out: {name} must be a CUDA tensor")
            if t.device != xyz.device or t.dtype != xyz.dtype:
                raise ValueError(f"out: {name} must be on {xyz.device} with dtype {xyz.dtype}, "
                                 f"got {t.device} / {t.dtype}")
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"out: {name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
            if not t.is_contiguous():
                raise ValueError(f"out: {name} must be contiguous")
        return (out[: len(shapes)] + (None, None))[:3]

    def compute_raw(self, dtype, level, xyz_ptr, n_samples, sph_ptr, dsph_ptr=None, ddsph_ptr=None, stream=None):
        """Thin wrapper of ``*_try_compute``: device pointers in, work enqueued on ``stream``."""
        sfx = "" if dtype == torch.float64 else "_f"
        status = getattr(self._lib, f"{self._prefix}_try_compute{sfx}")(
            self._calculator(dtype), level, xyz_ptr, n_samples, sph_ptr, dsph_ptr, ddsph_ptr, stream)
        if status != 0:
            raise RuntimeError(_c_lib.last_error())

    def compute_vjp_raw(self, dtype, xyz_ptr, n_samples, sph_grad_ptr, xyz_grad_ptr, stream=None):
        sfx = "" if dtype == torch.float64 else "_f"
        status = getattr(self._lib, f"{self._prefix}_try_compute_vjp{sfx}")(
            self._calculator(dtype), xyz_ptr, n_samples, sph_grad_ptr, xyz_grad_ptr, stream)
        if status != 0:
            raise RuntimeError(_c_lib.last_error())

    def _compute_impl(self, xyz, level, out=None):
        xyz = self._validate_xyz(xyz)
        n = xyz.shape[0]
        ny = (self._l_max + 1) ** 2
        if out is None:
            sph = torch.empty((n, ny), dtype=xyz.dtype, device=xyz.device)
            dsph = torch.empty((n, 3, ny), dtype=xyz.dtype, device=xyz.device) if level >= 1 else None
            ddsph = torch.empty((n, 3, 3, ny), dtype=xyz.dtype, device=xyz.device) if level >= 2 else None
        else:
            sph, dsph, ddsph = self._validate_out(out, xyz, [(n, ny), (n, 3, ny), (n, 3, 3, ny)][: level + 1])
        stream = torch.cuda.current_stream(xyz.device).cuda_stream
        self.compute_raw(xyz.dtype, level, _ptr(xyz), n, _ptr(sph), _ptr(dsph), _ptr(ddsph), stream)
        return sph, dsph, ddsph

    @staticmethod
    def _like_input(xyz, tensors):
        """Outputs in the array type of the input: torch tensors for torch tensors; for another
        CUDA array type (the reference's front end serves CuPy arrays:
        python/src/sphericart/spherical_harmonics.py:140-178) CuPy arrays over the same memory when
        CuPy is installed, torch tensors otherwise."""
        if isinstance(xyz, torch.Tensor):
            return tensors
        try:
            import cupy
        except ImportError:
            return tensors
        return tuple(None if t is None else cupy.asarray(t) for t in tensors)

    # -- public API -------------------------------------------------------------------------
    def compute(self, xyz, out=None) -> torch.Tensor:
        """Harmonics for an ``(n_samples, 3)`` CUDA tensor (or CuPy / Numba array) -> ``(n_samples, (l_max+1)^2)``."""
        return self._like_input(xyz, self._compute_impl(xyz, 0, out))[0]

    def compute_with_gradients(self, xyz, out=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Values and Cartesian gradients ``(n_samples, 3, (l_max+1)^2)``."""
        return self._like_input(xyz, self._compute_impl(xyz, 1, out))[:2]

    def compute_with_hessians(self, xyz, out=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Values, gradients and Hessians ``(n_samples, 3, 3, (l_max+1)^2)``."""
        return self._like_input(xyz, self._compute_impl(xyz, 2, out))

    def compute_vjp(self, xyz, sph_grad, out=None) -> torch.Tensor:
        """``xyz_grad[i, a] = sum_k sph_grad[i, k] * dsph[i, a, k]`` in one kernel, no dsph in memory."""
        xyz = self._validate_xyz(xyz)
        n = xyz.shape[0]
        ny = (self._l_max + 1) ** 2
        if sph_grad.shape != (n, ny) or sph_grad.dtype != xyz.dtype or sph_grad.device != xyz.device:
            raise ValueError("sph_grad must match xyz in dtype and device and have shape (n_samples, (l_max+1)^2)")
        sph_grad = sph_grad.detach().contiguous()
        xyz_grad = (torch.empty((n, 3), dtype=xyz.dtype, device=xyz.device) if out is None
                    else self._validate_out(out, xyz, [(n, 3)], names=("xyz_grad",))[0])
        stream = torch.cuda.current_stream(xyz.device).cuda_stream
        self.compute_vjp_raw(xyz.dtype, _ptr(xyz), n, _ptr(sph_grad), _ptr(xyz_grad), stream)
        return xyz_grad

    def compute_vjp_with_gradients(self, xyz, sph_grad, dsph_grad, out=None) -> torch.Tensor:
        """Second-order backward in one kernel: ``xyz_grad[i, b] = sum_k sph_grad[i, k] dsph[i, b, k] +
        sum_{a,k} dsph_grad[i, a, k] ddsph[i, a, b, k]`` with neither dsph nor ddsph in memory.
        ``sph_grad`` may be ``None``."""
        xyz = self._validate_xyz(xyz)
        n = xyz.shape[0]
        ny = (self._l_max + 1) ** 2
        if dsph_grad.shape != (n, 3, ny) or dsph_grad.dtype != xyz.dtype or dsph_grad.device != xyz.device:
            raise ValueError("dsph_grad must match xyz in dtype and device and have shape (n_samples, 3, (l_max+1)^2)")
        if sph_grad is not None:
            if sph_grad.shape != (n, ny) or sph_grad.dtype != xyz.dtype or sph_grad.device != xyz.device:
                raise ValueError("sph_grad must match xyz in dtype and device and have shape (n_samples, (l_max+1)^2)")
            sph_grad = sph_grad.detach().contiguous()
        dsph_grad = dsph_grad.detach().contiguous()
        xyz_grad = (torch.empty((n, 3), dtype=xyz.dtype, device=xyz.device) if out is None
                    else self._validate_out(out, xyz, [(n, 3)], names=("xyz_grad",))[0])
        stream = torch.cuda.current_stream(xyz.device).cuda_stream
        sfx = "" if xyz.dtype == torch.float64 else "_f"
        status = getattr(self._lib, f"{self._prefix}_try_compute_vjp_with_gradients{sfx}")(
            self._calculator(xyz.dtype), _ptr(xyz), n, _ptr(sph_grad), _ptr(dsph_grad), _ptr(xyz_grad), stream)
        if status != 0:
            raise RuntimeError(_c_lib.last_error())
        return xyz_grad

    def _selection_args(self, l_list, axis_order, scales, dtype):
        import ctypes

        degrees = [int(l) for l in l_list]
        if not degrees:
            raise ValueError("l_list must name at least one degree")
        if len(set(degrees)) != len(degrees) or min(degrees) < 0 or max(degrees) > self._l_max:
            raise ValueError(f"l_list must hold distinct degrees between 0 and l_max = {self._l_max}, got {degrees}")
        axis = [0, 1, 2] if axis_order is None else [int(a) for a in axis_order]
        if sorted(axis) != [0, 1, 2]:
            raise ValueError("axis_order must be a permutation of (0, 1, 2)")
        ctype = ctypes.c_double if dtype == torch.float64 else ctypes.c_float
        c_scales = None
        if scales is not None:
            if len(scales) != len(degrees):
                raise ValueError("scales must hold one factor per listed degree")
            c_scales = (ctype * len(degrees))(*[float(v) for v in scales])
        c_l = (ctypes.c_int * len(degrees))(*degrees)
        c_axis = (ctypes.c_int * 3)(*axis)
        return degrees, c_l, c_axis, c_scales, sum(2 * l + 1 for l in degrees)

    def compute_selected(self, xyz, l_list, axis_order=None, scales=None, out=None) -> torch.Tensor:
        """Values of the listed degree blocks only, ``(n_samples, sum(2l+1))``, in one kernel: block ``l`` of
        the output is ``scales[j] * Y_l`` for ``l = l_list[j]``, evaluated at points whose columns
        ``axis_order`` hold (x, y, z). What the reference's e3nn adaptor composes from a full evaluation, a
        slice, a permutation and a multiplication (``sphericart-torch/python/sphericart/torch/e3nn.py:47-80``).
        Needs ``l_max <= 20``."""
        xyz = self._validate_xyz(xyz)
        n = xyz.shape[0]
        _, c_l, c_axis, c_scales, ny_out = self._selection_args(l_list, axis_order, scales, xyz.dtype)
        res = (torch.empty((n, ny_out), dtype=xyz.dtype, device=xyz.device) if out is None
               else self._validate_out(out, xyz, [(n, ny_out)], names=("out",))[0])
        stream = torch.cuda.current_stream(xyz.device).cuda_stream
        sfx = "" if xyz.dtype == torch.float64 else "_f"
        status = getattr(self._lib, f"{self._prefix}_compute_selected{sfx}")(
            self._calculator(xyz.dtype), _ptr(xyz), n, c_l, len(c_l), c_axis, c_scales, _ptr(res), stream)
        if status != 0:
            raise RuntimeError(_c_lib.last_error())
        return res

    def compute_selected_vjp(self, xyz, out_grad, l_list, axis_order=None, scales=None, out=None) -> torch.Tensor:
        """Fused backward of :meth:`compute_selected`: ``out_grad`` is ``(n_samples, sum(2l+1))`` in the packed
        layout; returns ``(n_samples, 3)`` in the caller's axis order."""
        xyz = self._validate_xyz(xyz)
        n = xyz.shape[0]
        _, c_l, c_axis, c_scales, ny_out = self._selection_args(l_list, axis_order, scales, xyz.dtype)
        if out_grad.shape != (n, ny_out) or out_grad.dtype != xyz.dtype or out_grad.device != xyz.device:
            raise ValueError("out_grad must match xyz in dtype and device and have shape (n_samples, sum(2l+1))")
        out_grad = out_grad.detach().contiguous()
        res = (torch.empty((n, 3), dtype=xyz.dtype, device=xyz.device) if out is None
               else self._validate_out(out, xyz, [(n, 3)], names=("xyz_grad",))[0])
        stream = torch.cuda.current_stream(xyz.device).cuda_stream
        sfx = "" if xyz.dtype == torch.float64 else "_f"
        status = getattr(self._lib, f"{self._prefix}_compute_selected_vjp{sfx}")(
            self._calculator(xyz.dtype), _ptr(xyz), n, c_l, len(c_l), c_axis, c_scales, _ptr(out_grad), _ptr(res), stream)
        if status != 0:
            raise RuntimeError(_c_lib.last_error())
        return res

    def forward(self, xyz) -> torch.Tensor:
        """Values with autograd support: the backward pass is the fused VJP kernel."""
        return _HarmonicsFunction.apply(xyz, self)

    def forward_with_gradients(self, xyz) -> Tuple[torch.Tensor, torch.Tensor]:
        """Values and gradients with autograd support (as the reference's ``*_with_gradients`` op):
        the backward pass is the fused second-order kernel, no Hessian tensor is materialised."""
        return _HarmonicsWithGradientsFunction.apply(xyz, self)

    __call__ = forward


class _HarmonicsFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xyz, calculator):
        ctx.calculator = calculator
        ctx.save_for_backward(xyz)
        return calculator.compute(xyz)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_sph):
        (xyz,) = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return None, None
        return ctx.calculator.compute_vjp(xyz, grad_sph), None


class _HarmonicsWithGradientsFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xyz, calculator):
        ctx.calculator = calculator
        ctx.save_for_backward(xyz)
        return calculator.compute_with_gradients(xyz)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_sph, grad_dsph):
        (xyz,) = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return None, None
        if grad_dsph is None:
            return ctx.calculator.compute_vjp(xyz, grad_sph), None
        return ctx.calculator.compute_vjp_with_gradients(xyz, grad_sph, grad_dsph), None


class SphericalHarmonics(_BaseHarmonics):
    """Real spherical harmonics Y_l^m of the direction of each point, up to degree ``l_max``."""

    _prefix = "sphericart_cuda_spherical_harmonics"
    normalized = True


class SolidHarmonics(_BaseHarmonics):
    """Solid harmonics r^l Y_l^m (homogeneous polynomials of x, y, z), up to degree ``l_max``."""

    _prefix = "sphericart_cuda_solid_harmonics"
    normalized = False
