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
//
// Differences from the reference's operator layer (sphericart-torch/src/torch.cpp:117-143,340-349):
//  * only the CUDA dispatch key is implemented; a CPU tensor finds no kernel and the dispatcher
//    raises (this library has no CPU code path);
//  * one calculator per (kind, element type, l_max) for the whole process - the calculators keep
//    their per-device state themselves and may be called from several threads - instead of one
//    set of four calculators (two of them CPU ones) per thread, l_max and device;
//  * the current stream comes from c10 directly rather than from a helper library loaded at run
//    time.
// Autograd, shape inference for tracing and vmap rules are registered from Python
// (sphericart_b200/torch_ops.py), as the reference does for its own operators.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <map>
#include <memory>
#include <mutex>
#include <tuple>

#include "sphericart_cuda.hpp"

namespace {

template <typename Calc> Calc& calculator(int64_t l_max) {
    static std::mutex mutex;
    static std::map<int64_t, std::unique_ptr<Calc>> cache;
    std::lock_guard<std::mutex> lock(mutex);
    auto& slot = cache[l_max];
    if (!slot) slot = std::make_unique<Calc>(static_cast<size_t>(l_max));
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

}  // namespace

TORCH_LIBRARY(sphericart_b200, m) {
    for (const char* kind : {"spherical", "solid"}) {
        const std::string p = std::string(kind) + "_harmonics";
        m.def((p + "(Tensor xyz, int l_max) -> Tensor").c_str());
        m.def((p + "_with_gradients(Tensor xyz, int l_max) -> (Tensor, Tensor)").c_str());
        m.def((p + "_with_hessians(Tensor xyz, int l_max) -> (Tensor, Tensor, Tensor)").c_str());
        m.def((p + "_vjp(Tensor xyz, Tensor sph_grad, int l_max) -> Tensor").c_str());
        m.def((p + "_vjp_with_gradients(Tensor xyz, Tensor? sph_grad, Tensor dsph_grad, int l_max) -> Tensor").c_str());
    }
}

TORCH_LIBRARY_IMPL(sphericart_b200, CUDA, m) {
    m.impl("spherical_harmonics", &values<true>);
    m.impl("spherical_harmonics_with_gradients", &with_gradients<true>);
    m.impl("spherical_harmonics_with_hessians", &with_hessians<true>);
    m.impl("spherical_harmonics_vjp", &vjp<true>);
    m.impl("spherical_harmonics_vjp_with_gradients", &vjp_with_gradients<true>);
    m.impl("solid_harmonics", &values<false>);
    m.impl("solid_harmonics_with_gradients", &with_gradients<false>);
    m.impl("solid_harmonics_with_hessians", &with_hessians<false>);
    m.impl("solid_harmonics_vjp", &vjp<false>);
    m.impl("solid_harmonics_vjp_with_gradients", &vjp_with_gradients<false>);
}
