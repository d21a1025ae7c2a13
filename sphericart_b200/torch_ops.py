"""PyTorch operators over the CUDA library: ``torch.ops.sphericart_b200.*``.

The operators are implemented in C++ (``torch_csrc/torch_ops.cpp``: output allocation, current
stream and kernel launch with no Python in between); this module loads that library and registers
what the reference registers from Python for its own operators
(``sphericart-torch/python/sphericart/torch/register.py:60-196``): shape inference for tracing,
vmap rules and autograd. Unlike the reference, whose backward passes materialise ``dsph`` /
``ddsph`` and reduce them with tensor expressions (``register.py:90-108, 117-145``), the backward
passes here call the fused kernels:

* values                 -> ``*_vjp`` (gradients never written to memory); that operator is itself
                            differentiable, which gives the second-order path of the values;
* values and gradients   -> ``*_vjp_with_gradients`` (neither gradients nor Hessians written);
* values, gradients and Hessians -> contraction of the saved outputs, as in the reference
                            (third derivatives are not supported).

    import sphericart_b200.torch_ops            # registers the operators
    sph = torch.ops.sphericart_b200.spherical_harmonics(xyz_cuda, 8)

Only CUDA tensors are served; a CPU tensor raises ``NotImplementedError`` from the dispatcher.
"""

import os

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


def _register_vmap(prefix):
    # a function of one point, vmapped over the points: the batch is the operator's own first axis
    for suffix, n_out in (("", 1), ("_with_gradients", 2), ("_with_hessians", 3)):
        op = getattr(ops, prefix + suffix).default

        def rule(info, in_dims, xyz, l_max, _op=op, _n_out=n_out):
            if in_dims[0] not in (None, 0):
                xyz = xyz.movedim(in_dims[0], 0)
            return _op(xyz, l_max), (0 if _n_out == 1 else (0,) * _n_out)

        torch.library.register_vmap(op, rule)


def _register_autograd(prefix):
    with_gradients = getattr(ops, f"{prefix}_with_gradients").default
    vjp = getattr(ops, f"{prefix}_vjp").default
    vjp_with_gradients = getattr(ops, f"{prefix}_vjp_with_gradients").default

    # ---- values: backward is the fused VJP
    def values_setup(ctx, inputs, output):
        xyz, ctx.l_max = inputs
        ctx.save_for_backward(xyz)
        ctx.set_materialize_grads(False)

    def values_backward(ctx, grad_sph):
        if not ctx.needs_input_grad[0] or grad_sph is None:
            return None, None
        (xyz,) = ctx.saved_tensors
        return vjp(xyz, grad_sph.contiguous(), ctx.l_max), None

    torch.library.register_autograd(f"{_NS}::{prefix}", values_backward, setup_context=values_setup)

    # ---- the VJP itself: out[i][a] = sum_k g[i][k] dY[i][a][k]
    def vjp_setup(ctx, inputs, output):
        xyz, sph_grad, ctx.l_max = inputs
        ctx.save_for_backward(xyz, sph_grad)
        ctx.set_materialize_grads(False)

    def vjp_backward(ctx, v):
        xyz, sph_grad = ctx.saved_tensors
        xyz_grad = g_grad = None
        if v is None:
            return None, None, None
        v = v.contiguous()
        if ctx.needs_input_grad[0]:
            # d/dxyz[b] = sum_{a,k} v[a] g[k] ddY[a][b][k]: the second-order kernel with dsph_grad = v (x) g
            xyz_grad = vjp_with_gradients(xyz, None, (v.unsqueeze(2) * sph_grad.unsqueeze(1)).contiguous(), ctx.l_max)
        if ctx.needs_input_grad[1]:
            dsph = with_gradients(xyz, ctx.l_max)[1]
            g_grad = torch.einsum("na,nak->nk", v, dsph)
        return xyz_grad, g_grad, None

    torch.library.register_autograd(f"{_NS}::{prefix}_vjp", vjp_backward, setup_context=vjp_setup)

    # ---- values and gradients: backward is the fused second-order kernel
    def gradients_setup(ctx, inputs, output):
        xyz, ctx.l_max = inputs
        ctx.save_for_backward(xyz)
        ctx.set_materialize_grads(False)  # an unused output arrives as None, not as a tensor of zeros

    def gradients_backward(ctx, grad_sph, grad_dsph):
        if not ctx.needs_input_grad[0]:
            return None, None
        (xyz,) = ctx.saved_tensors
        if grad_dsph is None:
            if grad_sph is None:
                return None, None
            return vjp(xyz, grad_sph.contiguous(), ctx.l_max), None
        grad_sph = None if grad_sph is None else grad_sph.contiguous()
        return vjp_with_gradients(xyz, grad_sph, grad_dsph.contiguous(), ctx.l_max), None

    torch.library.register_autograd(f"{_NS}::{prefix}_with_gradients", gradients_backward, setup_context=gradients_setup)

    # ---- values, gradients and Hessians: everything needed was an output
    def hessians_setup(ctx, inputs, output):
        ctx.save_for_backward(output[1], output[2])
        ctx.set_materialize_grads(False)

    def hessians_backward(ctx, grad_sph, grad_dsph, grad_ddsph):
        if grad_ddsph is not None:
            raise RuntimeError(
                "Third derivatives of the spherical harmonics with respect to the Cartesian coordinates are not supported."
            )
        dsph, ddsph = ctx.saved_tensors
        xyz_grad = None
        if grad_sph is not None:
            xyz_grad = torch.einsum("nk,nak->na", grad_sph, dsph)
        if grad_dsph is not None:
            extra = torch.einsum("nak,nabk->nb", grad_dsph, ddsph)
            xyz_grad = extra if xyz_grad is None else xyz_grad + extra
        return xyz_grad, None

    torch.library.register_autograd(f"{_NS}::{prefix}_with_hessians", hessians_backward, setup_context=hessians_setup)


for _prefix in ("spherical_harmonics", "solid_harmonics"):
    _register_fakes(_prefix)
    _register_vmap(_prefix)
    _register_autograd(_prefix)
