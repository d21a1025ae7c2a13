// PyTorch operator library over the B200 calculators: CUDA tensors in, CUDA tensors out, no Python
// between the dispatcher and the kernel launch.
//
// Operators (namespace sphericart_b200). The first six have the schemas of the reference's
// operators (sphericart-torch/src/torch.cpp:367-376); the vjp operators have no counterpart there.
//   {spherical,solid}_harmonics(Tensor xyz, int l_max) -> Tensor
//   {spherical,solid}_harmonics_with_gradients(Tensor xyz, int l_max) -> (Tensor, Tensor)
//   {spherical,solid}_harmonics_with_hessians(Tensor xyz, int l_max) -> (Tensor, Tensor, Tensor)
//   {spherical,solid}_harmonics_vjp(Tensor xyz, Tensor sph_grad, int l_max) -> Tensor
//   {spherical,solid}_harmonics_vjp_with_gradients(Tensor xyz, Tensor? sph_grad, Tensor dsph_grad, int l_max) -> Tensor
//   {spherical,solid}_harmonics_selected(Tensor xyz, int[] l_list, int[] axis_order, float[] scales) -> Tensor
//   {spherical,solid}_harmonics_selected_vjp(Tensor xyz, Tensor out_grad, int[] l_list, int[] axis_order, float[] scales) -> Tensor
//     (chosen degree blocks only, packed, scaled, input axes permuted: what the reference's e3nn adaptor,
//      sphericart-torch/python/sphericart/torch/e3nn.py:47-80, composes from four tensor expressions)
//
// Differences from the reference's operator layer (sphericart-torch/src/torch.cpp:117-143,340-349):
//  * only the CUDA dispatch key is implemented; a CPU tensor finds no kernel and the dispatcher
//    raises (this library has no CPU code path);
//  * one calculator per (kind, element type, l_max) for the whole process - the calculators keep
//    their per-device state themselves and may be called from several threads - instead of one
//    set of four calculators (two of them CPU ones) per thread, l_max and device;
//  * the current stream comes from c10 directly rather than from a helper library loaded at run
//    time.
//  * autograd is registered here, in C++, on the fused backward kernels (the reference registers
//    Python backward functions that materialise dsph / ddsph and reduce them with tensor
//    expressions: sphericart-torch/python/sphericart/torch/register.py:82-175):
//      values                  -> *_vjp (gradients never written to memory); that operator is
//                                 differentiable again, which gives the values' second-order path;
//      values and gradients    -> *_vjp_with_gradients (neither gradients nor Hessians written);
//      values, gradients and Hessians -> contraction of the saved outputs, third derivatives refused.
// Shape inference for tracing and the vmap rules are registered from Python
// (sphericart_b200/torch_ops.py), as the reference does for its own operators.
#include <ATen/ATen.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/autograd/autograd_not_implemented_fallback.h>
#include <torch/csrc/autograd/custom_function.h>
#include <torch/library.h>

#include <map>
#include <memory>
#include <mutex>
#include <tuple>
#include <vector>

#include "sphericart_cuda.hpp"

namespace {

template <typename Calc> Calc& calculator(int64_t l_max) {
    // the calculators live for the whole process, so each thread may remember the one it used last
    // and skip the lock and the map on a steady stream of calls with one l_max
    thread_local int64_t last_l_max = -1;
    thread_local Calc* last = nullptr;
    if (last != nullptr && last_l_max == l_max) return *last;
    static std::mutex mutex;
    static std::map<int64_t, std::unique_ptr<Calc>> cache;
    std::lock_guard<std::mutex> lock(mutex);
    auto& slot = cache[l_max];
    if (!slot) slot = std::make_unique<Calc>(static_cast<size_t>(l_max));
    last = slot.get();
    last_l_max = l_max;
    return *slot;
}

template <bool NORMALIZED, typename T>
using Calculator = std::conditional_t<NORMALIZED, sphericart::cuda::SphericalHarmonics<T>, sphericart::cuda::SolidHarmonics<T>>;

at::Tensor checked_points(const at::Tensor& xyz, int64_t l_max) {
    TORCH_CHECK(l_max >= 0, "l_max must not be negative, got ", l_max);
    TORCH_CHECK(xyz.is_cuda(), "xyz must be a CUDA tensor");
    TORCH_CHECK(xyz.dim() == 2 && xyz.size(1) == 3, "xyz must have shape (n_samples, 3), got ", xyz.sizes());
    TORCH_CHECK(xyz.scalar_type() == at::kFloat || xyz.scalar_type() == at::kDouble,
                "this code only runs on float64 and float32 arrays");
    return xyz.contiguous();
}

at::Tensor checked_like(const at::Tensor& t, const at::Tensor& xyz, at::IntArrayRef shape, const char* name) {
    TORCH_CHECK(t.device() == xyz.device() && t.scalar_type() == xyz.scalar_type(), name,
                " must have the device and dtype of xyz");
    TORCH_CHECK(t.sizes() == shape, name, " must have shape ", shape, ", got ", t.sizes());
    return t.contiguous();
}

// level 0: values; 1: + gradients; 2: + Hessians
template <bool NORMALIZED> std::tuple<at::Tensor, at::Tensor, at::Tensor> forward(const at::Tensor& xyz_in, int64_t l_max, int level) {
    const at::Tensor xyz = checked_points(xyz_in, l_max);
    const int64_t n = xyz.size(0), ny = (l_max + 1) * (l_max + 1);
    const c10::cuda::CUDAGuard guard(xyz.device());
    void* stream = c10::cuda::getCurrentCUDAStream(xyz.device().index()).stream();
    at::Tensor sph = at::empty({n, ny}, xyz.options());
    at::Tensor dsph = level >= 1 ? at::empty({n, 3, ny}, xyz.options()) : at::Tensor();
    at::Tensor ddsph = level >= 2 ? at::empty({n, 3, 3, ny}, xyz.options()) : at::Tensor();
    AT_DISPATCH_FLOATING_TYPES(xyz.scalar_type(), "sphericart_b200_forward", [&] {
        auto& calc = calculator<Calculator<NORMALIZED, scalar_t>>(l_max);
        const scalar_t* p = xyz.data_ptr<scalar_t>();
        if (level == 0) {
            calc.compute(p, size_t(n), sph.data_ptr<scalar_t>(), stream);
        } else if (level == 1) {
            calc.compute_with_gradients(p, size_t(n), sph.data_ptr<scalar_t>(), dsph.data_ptr<scalar_t>(), stream);
        } else {
            calc.compute_with_hessians(p, size_t(n), sph.data_ptr<scalar_t>(), dsph.data_ptr<scalar_t>(),
                                       ddsph.data_ptr<scalar_t>(), stream);
        }
    });
    return {sph, dsph, ddsph};
}

template <bool NORMALIZED> at::Tensor values(const at::Tensor& xyz, int64_t l_max) {
    return std::get<0>(forward<NORMALIZED>(xyz, l_max, 0));
}

template <bool NORMALIZED> std::tuple<at::Tensor, at::Tensor> with_gradients(const at::Tensor& xyz, int64_t l_max) {
    auto r = forward<NORMALIZED>(xyz, l_max, 1);
    return {std::get<0>(r), std::get<1>(r)};
}

template <bool NORMALIZED>
std::tuple<at::Tensor, at::Tensor, at::Tensor> with_hessians(const at::Tensor& xyz, int64_t l_max) {
    return forward<NORMALIZED>(xyz, l_max, 2);
}

// xyz_grad[i][a] = sum_k sph_grad[i][k] dY[i][a][k]
template <bool NORMALIZED> at::Tensor vjp(const at::Tensor& xyz_in, const at::Tensor& sph_grad_in, int64_t l_max) {
    const at::Tensor xyz = checked_points(xyz_in, l_max);
    const int64_t n = xyz.size(0), ny = (l_max + 1) * (l_max + 1);
    const at::Tensor sph_grad = checked_like(sph_grad_in, xyz, {n, ny}, "sph_grad");
    const c10::cuda::CUDAGuard guard(xyz.device());
    void* stream = c10::cuda::getCurrentCUDAStream(xyz.device().index()).stream();
    at::Tensor out = at::empty({n, 3}, xyz.options());
    AT_DISPATCH_FLOATING_TYPES(xyz.scalar_type(), "sphericart_b200_vjp", [&] {
        calculator<Calculator<NORMALIZED, scalar_t>>(l_max).compute_vjp(
            xyz.data_ptr<scalar_t>(), size_t(n), sph_grad.data_ptr<scalar_t>(), out.data_ptr<scalar_t>(), stream);
    });
    return out;
}

// xyz_grad[i][b] = sum_k sph_grad[i][k] dY[i][b][k] + sum_{a,k} dsph_grad[i][a][k] ddY[i][a][b][k]
template <bool NORMALIZED>
at::Tensor vjp_with_gradients(const at::Tensor& xyz_in, const c10::optional<at::Tensor>& sph_grad_in,
                              const at::Tensor& dsph_grad_in, int64_t l_max) {
    const at::Tensor xyz = checked_points(xyz_in, l_max);
    const int64_t n = xyz.size(0), ny = (l_max + 1) * (l_max + 1);
    const at::Tensor dsph_grad = checked_like(dsph_grad_in, xyz, {n, 3, ny}, "dsph_grad");
    at::Tensor sph_grad;
    if (sph_grad_in.has_value() && sph_grad_in->defined()) sph_grad = checked_like(*sph_grad_in, xyz, {n, ny}, "sph_grad");
    const c10::cuda::CUDAGuard guard(xyz.device());
    void* stream = c10::cuda::getCurrentCUDAStream(xyz.device().index()).stream();
    at::Tensor out = at::empty({n, 3}, xyz.options());
    AT_DISPATCH_FLOATING_TYPES(xyz.scalar_type(), "sphericart_b200_vjp_with_gradients", [&] {
        calculator<Calculator<NORMALIZED, scalar_t>>(l_max).compute_vjp_with_gradients(
            xyz.data_ptr<scalar_t>(), size_t(n), sph_grad.defined() ? sph_grad.data_ptr<scalar_t>() : nullptr,
            dsph_grad.data_ptr<scalar_t>(), out.data_ptr<scalar_t>(), stream);
    });
    return out;
}

// Selected degree blocks: l_max of the calculator = the largest listed degree.
struct SelectionArgs {
    std::vector<int> degrees;
    int axis[3];
    int64_t l_max = 0, ny_out = 0;
};

SelectionArgs checked_selection(at::IntArrayRef l_list, at::IntArrayRef axis_order, at::ArrayRef<double> scales) {
    SelectionArgs sel;
    TORCH_CHECK(!l_list.empty(), "l_list must name at least one degree");
    TORCH_CHECK(scales.empty() || scales.size() == l_list.size(), "scales must hold one factor per listed degree");
    TORCH_CHECK(axis_order.size() == 3, "axis_order must hold three entries");
    for (int64_t l : l_list) {
        TORCH_CHECK(l >= 0, "degrees must not be negative, got ", l);
        sel.degrees.push_back(int(l));
        sel.l_max = std::max<int64_t>(sel.l_max, l);
        sel.ny_out += 2 * l + 1;
    }
    for (int a = 0; a < 3; ++a) sel.axis[a] = int(axis_order[a]);
    return sel;
}

template <bool NORMALIZED>
at::Tensor selected(const at::Tensor& xyz_in, at::IntArrayRef l_list, at::IntArrayRef axis_order, at::ArrayRef<double> scales) {
    const SelectionArgs sel = checked_selection(l_list, axis_order, scales);
    const at::Tensor xyz = checked_points(xyz_in, sel.l_max);
    const int64_t n = xyz.size(0);
    const c10::cuda::CUDAGuard guard(xyz.device());
    void* stream = c10::cuda::getCurrentCUDAStream(xyz.device().index()).stream();
    at::Tensor out = at::empty({n, sel.ny_out}, xyz.options());
    AT_DISPATCH_FLOATING_TYPES(xyz.scalar_type(), "sphericart_b200_selected", [&] {
        std::vector<scalar_t> factors(scales.begin(), scales.end());
        calculator<Calculator<NORMALIZED, scalar_t>>(sel.l_max).compute_selected(
            xyz.data_ptr<scalar_t>(), size_t(n), sel.degrees.data(), sel.degrees.size(), sel.axis,
            factors.empty() ? nullptr : factors.data(), out.data_ptr<scalar_t>(), stream);
    });
    return out;
}

template <bool NORMALIZED>
at::Tensor selected_vjp(const at::Tensor& xyz_in, const at::Tensor& out_grad_in, at::IntArrayRef l_list,
                        at::IntArrayRef axis_order, at::ArrayRef<double> scales) {
    const SelectionArgs sel = checked_selection(l_list, axis_order, scales);
    const at::Tensor xyz = checked_points(xyz_in, sel.l_max);
    const int64_t n = xyz.size(0);
    const at::Tensor out_grad = checked_like(out_grad_in, xyz, {n, sel.ny_out}, "out_grad");
    const c10::cuda::CUDAGuard guard(xyz.device());
    void* stream = c10::cuda::getCurrentCUDAStream(xyz.device().index()).stream();
    at::Tensor xyz_grad = at::empty({n, 3}, xyz.options());
    AT_DISPATCH_FLOATING_TYPES(xyz.scalar_type(), "sphericart_b200_selected_vjp", [&] {
        std::vector<scalar_t> factors(scales.begin(), scales.end());
        calculator<Calculator<NORMALIZED, scalar_t>>(sel.l_max).compute_selected_vjp(
            xyz.data_ptr<scalar_t>(), size_t(n), sel.degrees.data(), sel.degrees.size(), sel.axis,
            factors.empty() ? nullptr : factors.data(), out_grad.data_ptr<scalar_t>(), xyz_grad.data_ptr<scalar_t>(), stream);
    });
    return xyz_grad;
}

// ---------------------------------------------------------------------------------------------
// Autograd. Every operator called below goes back through the dispatcher, so what a backward
// pass computes is recorded when a graph of it is asked for (create_graph).
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

// No graph is recorded when nothing asks for one: the operator then goes straight to the kernel.
inline bool wants_graph(const at::Tensor& t) { return at::GradMode::is_enabled() && t.defined() && t.requires_grad(); }

template <bool NORMALIZED> std::string op_name(const char* suffix) {
    return std::string("sphericart_b200::") + (NORMALIZED ? "spherical" : "solid") + "_harmonics" + suffix;
}

template <bool NORMALIZED> at::Tensor call_values(const at::Tensor& xyz, int64_t l_max) {
    static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(op_name<NORMALIZED>("").c_str(), "")
                         .template typed<at::Tensor(const at::Tensor&, int64_t)>();
    return op.call(xyz, l_max);
}
template <bool NORMALIZED> std::tuple<at::Tensor, at::Tensor> call_with_gradients(const at::Tensor& xyz, int64_t l_max) {
    static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(op_name<NORMALIZED>("_with_gradients").c_str(), "")
                         .template typed<std::tuple<at::Tensor, at::Tensor>(const at::Tensor&, int64_t)>();
    return op.call(xyz, l_max);
}
template <bool NORMALIZED>
std::tuple<at::Tensor, at::Tensor, at::Tensor> call_with_hessians(const at::Tensor& xyz, int64_t l_max) {
    static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(op_name<NORMALIZED>("_with_hessians").c_str(), "")
                         .template typed<std::tuple<at::Tensor, at::Tensor, at::Tensor>(const at::Tensor&, int64_t)>();
    return op.call(xyz, l_max);
}
template <bool NORMALIZED> at::Tensor call_vjp(const at::Tensor& xyz, const at::Tensor& sph_grad, int64_t l_max) {
    static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(op_name<NORMALIZED>("_vjp").c_str(), "")
                         .template typed<at::Tensor(const at::Tensor&, const at::Tensor&, int64_t)>();
    return op.call(xyz, sph_grad, l_max);
}
template <bool NORMALIZED>
at::Tensor call_vjp_with_gradients(const at::Tensor& xyz, const c10::optional<at::Tensor>& sph_grad,
                                   const at::Tensor& dsph_grad, int64_t l_max) {
    static auto op =
        c10::Dispatcher::singleton().findSchemaOrThrow(op_name<NORMALIZED>("_vjp_with_gradients").c_str(), "")
            .template typed<at::Tensor(const at::Tensor&, const c10::optional<at::Tensor>&, const at::Tensor&, int64_t)>();
    return op.call(xyz, sph_grad, dsph_grad, l_max);
}

template <bool NORMALIZED> struct ValuesFunction : torch::autograd::Function<ValuesFunction<NORMALIZED>> {
    static at::Tensor forward(AutogradContext* ctx, const at::Tensor& xyz, int64_t l_max) {
        at::AutoDispatchBelowADInplaceOrView below;
        ctx->save_for_backward({xyz});
        ctx->saved_data["l_max"] = l_max;
        ctx->set_materialize_grads(false);
        return call_values<NORMALIZED>(xyz, l_max);
    }
    static variable_list backward(AutogradContext* ctx, variable_list grads) {
        if (!grads[0].defined()) return {at::Tensor(), at::Tensor()};
        const auto saved = ctx->get_saved_variables();
        return {call_vjp<NORMALIZED>(saved[0], grads[0].contiguous(), ctx->saved_data["l_max"].toInt()), at::Tensor()};
    }
};

// out[i][a] = sum_k g[i][k] dY[i][a][k]
template <bool NORMALIZED> struct VjpFunction : torch::autograd::Function<VjpFunction<NORMALIZED>> {
    static at::Tensor forward(AutogradContext* ctx, const at::Tensor& xyz, const at::Tensor& sph_grad, int64_t l_max) {
        at::AutoDispatchBelowADInplaceOrView below;
        ctx->save_for_backward({xyz, sph_grad});
        ctx->saved_data["l_max"] = l_max;
        ctx->set_materialize_grads(false);
        return call_vjp<NORMALIZED>(xyz, sph_grad, l_max);
    }
    static variable_list backward(AutogradContext* ctx, variable_list grads) {
        if (!grads[0].defined()) return {at::Tensor(), at::Tensor(), at::Tensor()};
        const auto saved = ctx->get_saved_variables();
        const at::Tensor& xyz = saved[0];
        const at::Tensor& g = saved[1];
        const int64_t l_max = ctx->saved_data["l_max"].toInt();
        const at::Tensor v = grads[0].contiguous();
        at::Tensor xyz_grad, g_grad;
        if (ctx->needs_input_grad(0)) {
            // d/dxyz[b] = sum_{a,k} v[a] g[k] ddY[a][b][k]: the second-order kernel with dsph_grad = v (x) g
            xyz_grad = call_vjp_with_gradients<NORMALIZED>(xyz, c10::nullopt, (v.unsqueeze(2) * g.unsqueeze(1)).contiguous(),
                                                           l_max);
        }
        if (ctx->needs_input_grad(1)) {
            const at::Tensor dsph = std::get<1>(call_with_gradients<NORMALIZED>(xyz, l_max));
            g_grad = at::einsum("na,nak->nk", {v, dsph});
        }
        return {xyz_grad, g_grad, at::Tensor()};
    }
};

template <bool NORMALIZED> struct GradientsFunction : torch::autograd::Function<GradientsFunction<NORMALIZED>> {
    static variable_list forward(AutogradContext* ctx, const at::Tensor& xyz, int64_t l_max) {
        at::AutoDispatchBelowADInplaceOrView below;
        ctx->save_for_backward({xyz});
        ctx->saved_data["l_max"] = l_max;
        ctx->set_materialize_grads(false);  // an unused output arrives undefined, not as zeros
        auto r = call_with_gradients<NORMALIZED>(xyz, l_max);
        return {std::get<0>(r), std::get<1>(r)};
    }
    static variable_list backward(AutogradContext* ctx, variable_list grads) {
        const auto saved = ctx->get_saved_variables();
        const int64_t l_max = ctx->saved_data["l_max"].toInt();
        if (!grads[1].defined()) {
            if (!grads[0].defined()) return {at::Tensor(), at::Tensor()};
            return {call_vjp<NORMALIZED>(saved[0], grads[0].contiguous(), l_max), at::Tensor()};
        }
        c10::optional<at::Tensor> g0;
        if (grads[0].defined()) g0 = grads[0].contiguous();
        return {call_vjp_with_gradients<NORMALIZED>(saved[0], g0, grads[1].contiguous(), l_max), at::Tensor()};
    }
};

template <bool NORMALIZED> struct HessiansFunction : torch::autograd::Function<HessiansFunction<NORMALIZED>> {
    static variable_list forward(AutogradContext* ctx, const at::Tensor& xyz, int64_t l_max) {
        at::AutoDispatchBelowADInplaceOrView below;
        auto r = call_with_hessians<NORMALIZED>(xyz, l_max);
        ctx->save_for_backward({std::get<1>(r), std::get<2>(r)});
        ctx->set_materialize_grads(false);
        return {std::get<0>(r), std::get<1>(r), std::get<2>(r)};
    }
    static variable_list backward(AutogradContext* ctx, variable_list grads) {
        TORCH_CHECK(!grads[2].defined(),
                    "Third derivatives of the spherical harmonics with respect to the Cartesian coordinates are not "
                    "supported.");
        const auto saved = ctx->get_saved_variables();
        at::Tensor xyz_grad;
        if (grads[0].defined()) xyz_grad = at::einsum("nk,nak->na", {grads[0], saved[0]});
        if (grads[1].defined()) {
            const at::Tensor extra = at::einsum("nak,nabk->nb", {grads[1], saved[1]});
            xyz_grad = xyz_grad.defined() ? xyz_grad + extra : extra;
        }
        return {xyz_grad, at::Tensor()};
    }
};

template <bool NORMALIZED>
at::Tensor call_selected(const at::Tensor& xyz, at::IntArrayRef l_list, at::IntArrayRef axis_order, at::ArrayRef<double> scales) {
    static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(op_name<NORMALIZED>("_selected").c_str(), "")
                         .template typed<at::Tensor(const at::Tensor&, at::IntArrayRef, at::IntArrayRef, at::ArrayRef<double>)>();
    return op.call(xyz, l_list, axis_order, scales);
}
template <bool NORMALIZED>
at::Tensor call_selected_vjp(const at::Tensor& xyz, const at::Tensor& out_grad, at::IntArrayRef l_list,
                             at::IntArrayRef axis_order, at::ArrayRef<double> scales) {
    static auto op =
        c10::Dispatcher::singleton().findSchemaOrThrow(op_name<NORMALIZED>("_selected_vjp").c_str(), "")
            .template typed<at::Tensor(const at::Tensor&, const at::Tensor&, at::IntArrayRef, at::IntArrayRef, at::ArrayRef<double>)>();
    return op.call(xyz, out_grad, l_list, axis_order, scales);
}

// selected values -> the fused selected VJP (first order only: the VJP operator itself is not differentiable)
template <bool NORMALIZED> struct SelectedFunction : torch::autograd::Function<SelectedFunction<NORMALIZED>> {
    static at::Tensor forward(AutogradContext* ctx, const at::Tensor& xyz, at::IntArrayRef l_list,
                              at::IntArrayRef axis_order, at::ArrayRef<double> scales) {
        at::AutoDispatchBelowADInplaceOrView below;
        ctx->save_for_backward({xyz});
        ctx->saved_data["l_list"] = l_list.vec();
        ctx->saved_data["axis_order"] = axis_order.vec();
        ctx->saved_data["scales"] = scales.vec();
        ctx->set_materialize_grads(false);
        return call_selected<NORMALIZED>(xyz, l_list, axis_order, scales);
    }
    static variable_list backward(AutogradContext* ctx, variable_list grads) {
        if (!grads[0].defined()) return {at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
        const auto saved = ctx->get_saved_variables();
        const std::vector<int64_t> l_list = ctx->saved_data["l_list"].toIntVector();
        const std::vector<int64_t> axis_order = ctx->saved_data["axis_order"].toIntVector();
        const std::vector<double> scales = ctx->saved_data["scales"].toDoubleVector();
        return {call_selected_vjp<NORMALIZED>(saved[0], grads[0].contiguous(), l_list, axis_order, scales), at::Tensor(),
                at::Tensor(), at::Tensor()};
    }
};

template <bool NORMALIZED>
at::Tensor selected_autograd(const at::Tensor& xyz, at::IntArrayRef l_list, at::IntArrayRef axis_order, at::ArrayRef<double> scales) {
    if (!wants_graph(xyz)) {
        at::AutoDispatchBelowADInplaceOrView below;
        return call_selected<NORMALIZED>(xyz, l_list, axis_order, scales);
    }
    return SelectedFunction<NORMALIZED>::apply(xyz, l_list, axis_order, scales);
}

template <bool NORMALIZED> at::Tensor values_autograd(const at::Tensor& xyz, int64_t l_max) {
    if (!wants_graph(xyz)) {
        at::AutoDispatchBelowADInplaceOrView below;
        return call_values<NORMALIZED>(xyz, l_max);
    }
    return ValuesFunction<NORMALIZED>::apply(xyz, l_max);
}
template <bool NORMALIZED> at::Tensor vjp_autograd(const at::Tensor& xyz, const at::Tensor& sph_grad, int64_t l_max) {
    if (!wants_graph(xyz) && !wants_graph(sph_grad)) {
        at::AutoDispatchBelowADInplaceOrView below;
        return call_vjp<NORMALIZED>(xyz, sph_grad, l_max);
    }
    return VjpFunction<NORMALIZED>::apply(xyz, sph_grad, l_max);
}
template <bool NORMALIZED> std::tuple<at::Tensor, at::Tensor> with_gradients_autograd(const at::Tensor& xyz, int64_t l_max) {
    if (!wants_graph(xyz)) {
        at::AutoDispatchBelowADInplaceOrView below;
        return call_with_gradients<NORMALIZED>(xyz, l_max);
    }
    auto r = GradientsFunction<NORMALIZED>::apply(xyz, l_max);
    return {r[0], r[1]};
}
template <bool NORMALIZED>
std::tuple<at::Tensor, at::Tensor, at::Tensor> with_hessians_autograd(const at::Tensor& xyz, int64_t l_max) {
    if (!wants_graph(xyz)) {
        at::AutoDispatchBelowADInplaceOrView below;
        return call_with_hessians<NORMALIZED>(xyz, l_max);
    }
    auto r = HessiansFunction<NORMALIZED>::apply(xyz, l_max);
    return {r[0], r[1], r[2]};
}

}  // namespace

TORCH_LIBRARY(sphericart_b200, m) {
    for (const char* kind : {"spherical", "solid"}) {
        const std::string p = std::string(kind) + "_harmonics";
        m.def((p + "(Tensor xyz, int l_max) -> Tensor").c_str());
        m.def((p + "_with_gradients(Tensor xyz, int l_max) -> (Tensor, Tensor)").c_str());
        m.def((p + "_with_hessians(Tensor xyz, int l_max) -> (Tensor, Tensor, Tensor)").c_str());
        m.def((p + "_vjp(Tensor xyz, Tensor sph_grad, int l_max) -> Tensor").c_str());
        m.def((p + "_vjp_with_gradients(Tensor xyz, Tensor? sph_grad, Tensor dsph_grad, int l_max) -> Tensor").c_str());
        m.def((p + "_selected(Tensor xyz, int[] l_list, int[] axis_order, float[] scales) -> Tensor").c_str());
        m.def((p + "_selected_vjp(Tensor xyz, Tensor out_grad, int[] l_list, int[] axis_order, float[] scales) -> Tensor").c_str());
    }
}

TORCH_LIBRARY_IMPL(sphericart_b200, CUDA, m) {
    m.impl("spherical_harmonics", &values<true>);
    m.impl("spherical_harmonics_with_gradients", &with_gradients<true>);
    m.impl("spherical_harmonics_with_hessians", &with_hessians<true>);
    m.impl("spherical_harmonics_vjp", &vjp<true>);
    m.impl("spherical_harmonics_vjp_with_gradients", &vjp_with_gradients<true>);
    m.impl("spherical_harmonics_selected", &selected<true>);
    m.impl("spherical_harmonics_selected_vjp", &selected_vjp<true>);
    m.impl("solid_harmonics_selected", &selected<false>);
    m.impl("solid_harmonics_selected_vjp", &selected_vjp<false>);
    m.impl("solid_harmonics", &values<false>);
    m.impl("solid_harmonics_with_gradients", &with_gradients<false>);
    m.impl("solid_harmonics_with_hessians", &with_hessians<false>);
    m.impl("solid_harmonics_vjp", &vjp<false>);
    m.impl("solid_harmonics_vjp_with_gradients", &vjp_with_gradients<false>);
}

TORCH_LIBRARY_IMPL(sphericart_b200, Autograd, m) {
    m.impl("spherical_harmonics", &values_autograd<true>);
    m.impl("spherical_harmonics_with_gradients", &with_gradients_autograd<true>);
    m.impl("spherical_harmonics_with_hessians", &with_hessians_autograd<true>);
    m.impl("spherical_harmonics_vjp", &vjp_autograd<true>);
    m.impl("spherical_harmonics_vjp_with_gradients", torch::autograd::autogradNotImplementedFallback());
    m.impl("spherical_harmonics_selected", &selected_autograd<true>);
    m.impl("spherical_harmonics_selected_vjp", torch::autograd::autogradNotImplementedFallback());
    m.impl("solid_harmonics_selected", &selected_autograd<false>);
    m.impl("solid_harmonics_selected_vjp", torch::autograd::autogradNotImplementedFallback());
    m.impl("solid_harmonics", &values_autograd<false>);
    m.impl("solid_harmonics_with_gradients", &with_gradients_autograd<false>);
    m.impl("solid_harmonics_with_hessians", &with_hessians_autograd<false>);
    m.impl("solid_harmonics_vjp", &vjp_autograd<false>);
    m.impl("solid_harmonics_vjp_with_gradients", torch::autograd::autogradNotImplementedFallback());
}
