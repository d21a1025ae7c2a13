"""PyTorch operators over the CUDA library: ``torch.ops.sphericart_b200.*``.

The operators and their autograd are implemented in C++ (``torch_csrc/torch_ops.cpp``: output
allocation, current stream, kernel launch and backward with no Python in between); this module
loads that library and registers shape inference for tracing and the vmap rules, as the reference
does from Python for its own operators
(``sphericart-torch/python/sphericart/torch/register.py:60-80``). Unlike the reference, whose
backward passes materialise ``dsph`` / ``ddsph`` and reduce them with tensor expressions
(``register.py:90-108, 117-145``), the backward passes call the fused kernels:

* values                 -> ``*_vjp`` (gradients never written to memory); that operator is itself
                            differentiable, which gives the second-order path of the values;
* values and gradients   -> ``*_vjp_with_gradients`` (neither gradients nor Hessians written);
* values, gradients and Hessians -> contraction of the saved outputs, as in the reference
                            (third derivatives are not supported).

    import sphericart_b200.torch_ops as sbt     # registers the operators
    sph = torch.ops.sphericart_b200.spherical_harmonics(xyz_cuda, 8)
    sph = sbt.SphericalHarmonics(8)(xyz_cuda)    # the same through a (scriptable) torch.nn.Module

Only CUDA tensors are served; a CPU tensor raises ``NotImplementedError`` from the dispatcher.
"""

import os
from typing import Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(_HERE, "libsphericart_b200_torch.so")

if not os.path.exists(LIBRARY):
    raise ImportError(
        f"{LIBRARY} is missing: build it with `python -m sphericart_b200.build` (needs nvcc, g++ and torch's headers)"
    )
torch.ops.load_library(LIBRARY)

_NS = "sphericart_b200"
ops = torch.ops.sphericart_b200


def _ny(l_max):
    return (l_max + 1) ** 2


def _register_fakes(prefix):
    @torch.library.register_fake(f"{_NS}::{prefix}")
    def _(xyz, l_max):
        return xyz.new_empty((xyz.shape[0], _ny(l_max)))

    @torch.library.register_fake(f"{_NS}::{prefix}_with_gradients")
    def _(xyz, l_max):
        n, ny = xyz.shape[0], _ny(l_max)
        return xyz.new_empty((n, ny)), xyz.new_empty((n, 3, ny))

    @torch.library.register_fake(f"{_NS}::{prefix}_with_hessians")
    def _(xyz, l_max):
        n, ny = xyz.shape[0], _ny(l_max)
        return xyz.new_empty((n, ny)), xyz.new_empty((n, 3, ny)), xyz.new_empty((n, 3, 3, ny))

    @torch.library.register_fake(f"{_NS}::{prefix}_vjp")
    def _(xyz, sph_grad, l_max):
        return xyz.new_empty((xyz.shape[0], 3))

    @torch.library.register_fake(f"{_NS}::{prefix}_vjp_with_gradients")
    def _(xyz, sph_grad, dsph_grad, l_max):
        return xyz.new_empty((xyz.shape[0], 3))

    @torch.library.register_fake(f"{_NS}::{prefix}_selected")
    def _(xyz, l_list, axis_order, scales):
        return xyz.new_empty((xyz.shape[0], sum(2 * l + 1 for l in l_list)))

    @torch.library.register_fake(f"{_NS}::{prefix}_selected_vjp")
    def _(xyz, out_grad, l_list, axis_order, scales):
        return xyz.new_empty((xyz.shape[0], 3))


def _register_vmap(prefix):
    # a function of one point, vmapped over the points: the batch is the operator's own first axis
    for suffix, n_out in (("", 1), ("_with_gradients", 2), ("_with_hessians", 3)):
        op = getattr(ops, prefix + suffix).default

        def rule(info, in_dims, xyz, l_max, _op=op, _n_out=n_out):
            if in_dims[0] not in (None, 0):
                xyz = xyz.movedim(in_dims[0], 0)
            return _op(xyz, l_max), (0 if _n_out == 1 else (0,) * _n_out)

        torch.library.register_vmap(op, rule)


for _prefix in ("spherical_harmonics", "solid_harmonics"):
    _register_fakes(_prefix)
    _register_vmap(_prefix)


class SphericalHarmonics(torch.nn.Module):
    """Real spherical harmonics of CUDA points as a ``torch.nn.Module`` over the operators above:
    the interface of the reference's ``sphericart.torch.SphericalHarmonics``
    (``sphericart-torch/python/sphericart/torch/spherical_hamonics.py:7-161``) - ``forward`` and
    ``compute`` return ``(n_samples, (l_max+1)^2)`` values and are differentiable (twice) through
    the fused backward kernels; ``compute_with_gradients`` / ``compute_with_hessians`` also return
    ``(n_samples, 3, ny)`` gradients and ``(n_samples, 3, 3, ny)`` Hessians. Works under
    ``torch.jit.script``. There is no CPU code path: CPU tensors are refused."""

    def __init__(self, l_max: int):
        super().__init__()
        self._l_max = l_max

    def forward(self, xyz: torch.Tensor) -> torch.Tensor:
        return torch.ops.sphericart_b200.spherical_harmonics(xyz, self._l_max)

    @torch.jit.export
    def compute(self, xyz: torch.Tensor) -> torch.Tensor:
        return self.forward(xyz)

    @torch.jit.export
    def compute_with_gradients(self, xyz: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return torch.ops.sphericart_b200.spherical_harmonics_with_gradients(xyz, self._l_max)

    @torch.jit.export
    def compute_with_hessians(self, xyz: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return torch.ops.sphericart_b200.spherical_harmonics_with_hessians(xyz, self._l_max)

    @torch.jit.export
    def l_max(self) -> int:
        return self._l_max


class SolidHarmonics(torch.nn.Module):
    """Solid harmonics ``r^l Y_l^m``: same interface as :class:`SphericalHarmonics`
    (reference: ``spherical_hamonics.py:164-209``)."""

    def __init__(self, l_max: int):
        super().__init__()
        self._l_max = l_max

    def forward(self, xyz: torch.Tensor) -> torch.Tensor:
        return torch.ops.sphericart_b200.solid_harmonics(xyz, self._l_max)

    @torch.jit.export
    def compute(self, xyz: torch.Tensor) -> torch.Tensor:
        return self.forward(xyz)

    @torch.jit.export
    def compute_with_gradients(self, xyz: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return torch.ops.sphericart_b200.solid_harmonics_with_gradients(xyz, self._l_max)

    @torch.jit.export
    def compute_with_hessians(self, xyz: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return torch.ops.sphericart_b200.solid_harmonics_with_hessians(xyz, self._l_max)

    @torch.jit.export
    def l_max(self) -> int:
        return self._l_max


# largest degree the compile-time kernels behind the `*_selected` operators cover
_SELECTED_LMAX = 20


def e3nn_spherical_harmonics(l_list, x: torch.Tensor, normalize: bool = False, normalization: str = "integral"):
    """Harmonics in the conventions of ``e3nn.o3.spherical_harmonics``: the function the reference
    offers in ``sphericart-torch/python/sphericart/torch/e3nn.py:10-80``, for CUDA tensors.

    ``l_list``: one degree or a list of degrees, returned in the listed order; ``x``: ``(n, 3)`` points
    with e3nn's axis order (y, z, x in this library's terms); ``normalize``: spherical (True) or solid
    (False) harmonics; ``normalization``: "integral" (this library's), "component" (times sqrt(4 pi)) or
    "norm" (times sqrt(4 pi / (2 l + 1))).

    One kernel writes the listed blocks, scaled, from the points as they are (the axis permutation is
    part of the kernel's load); its backward pass is one fused kernel as well. The reference evaluates
    every degree and then slices, permutes and rescales. Lists the kernel does not serve (a degree
    above 20, a repeated degree) take that composed route here too, as does second-order autograd."""
    import math

    degrees = [int(v) for v in l_list] if hasattr(l_list, "__len__") else [int(l_list)]
    if normalization not in ("integral", "norm", "component"):
        raise ValueError('normalization must be "integral", "norm" or "component"')
    scales = []
    for l in degrees:
        scale = 1.0 if normalization == "integral" else math.sqrt(4 * math.pi)
        if normalization == "norm":
            scale /= math.sqrt(2 * l + 1)
        scales.append(scale)
    if max(degrees) <= _SELECTED_LMAX and len(set(degrees)) == len(degrees):
        op = ops.spherical_harmonics_selected if normalize else ops.solid_harmonics_selected
        return op(x, degrees, [2, 0, 1], scales)
    l_max = max(degrees)
    op = ops.spherical_harmonics if normalize else ops.solid_harmonics
    sh = op(x[:, [2, 0, 1]], l_max)
    columns, factors = [], []
    for l, scale in zip(degrees, scales):
        columns.extend(range(l * l, (l + 1) * (l + 1)))
        factors.extend([scale] * (2 * l + 1))
    sh = sh[:, torch.tensor(columns, dtype=torch.long, device=sh.device)]
    return sh * torch.tensor(factors, dtype=sh.dtype, device=sh.device)
