// C++ interface of the B200 (sm_100a) implementation of sphericart's CUDA calculators.
//
// Drop-in for the reference header sphericart/include/sphericart_cuda.hpp:33-187: the same
// namespace, class names, constructor and compute / compute_with_gradients /
// compute_with_hessians signatures, and the same object size and member offsets (the
// reference's bindings allocate these objects themselves: sphericart-torch/src/torch.cpp:340-349,
// sphericart-jax/src/sphericart_jax_cuda.cpp:25-40), so code compiled against either header links
// against this library. Two methods are added, compute_vjp and compute_vjp_with_gradients, which
// nothing in the reference calls.
//
// Contract of every compute call (reference: sphericart/src/sphericart_cuda.cpp:74-160):
//  * xyz, sph, dsph, ddsph are DEVICE pointers to caller-owned contiguous buffers of
//    n_samples x 3, n_samples x (l_max+1)^2, n_samples x 3 x (l_max+1)^2 and
//    n_samples x 3 x 3 x (l_max+1)^2 elements; column (l, m) sits at l*l + l + m.
//  * cuda_stream is a cudaStream_t cast to void* (nullptr = default stream). The call only
//    enqueues work; it never allocates or frees the caller's buffers and, with one exception,
//    never synchronises: the first call per calculator and device that is served by the
//    run-time-degree kernel (values: l_max > 20, gradients: l_max > 10, Hessians: l_max > 5)
//    allocates a few KB on that device for the calculator's tables and fills them with a blocking
//    copy. Make that call once before recording a CUDA graph or entering a latency-critical loop.
//  * The work runs on the device that owns xyz; the caller's current device is restored.
//  * n_samples == 0 returns at once, even with null outputs. A null sph (or a null dsph / ddsph
//    when that output was asked for) and every CUDA failure throw std::runtime_error.
//  * Calls on one calculator may come from several threads and streams at once.
#ifndef SPHERICART_CUDA_HPP
#define SPHERICART_CUDA_HPP

#include <cstddef>
#include <cstdint>
#include <mutex>

namespace sphericart {
namespace cuda {

/// Real spherical harmonics Y_l^m(r/|r|) for l <= l_max, T = float or double.
template <typename T> class SphericalHarmonics {
  public:
    SphericalHarmonics(size_t l_max);
    ~SphericalHarmonics();

    /// Values only.
    void compute(const T* xyz, const size_t n_samples, T* sph, void* cuda_stream = nullptr);

    /// Values and gradients d/dx, d/dy, d/dz.
    void compute_with_gradients(const T* xyz, const size_t n_samples, T* sph, T* dsph, void* cuda_stream = nullptr);

    /// Values, gradients and Hessians (all nine second derivatives, both symmetric halves).
    void compute_with_hessians(
        const T* xyz, const size_t n_samples, T* sph, T* dsph, T* ddsph, void* cuda_stream = nullptr
    );

    /// Fused vector-Jacobian product (no counterpart in the reference's C++ classes):
    /// xyz_grad[i][a] = sum_k sph_grad[i][k] * dsph[i][a][k], with dsph never written to memory.
    /// sph_grad is n_samples x (l_max+1)^2, xyz_grad is n_samples x 3, both device pointers.
    void compute_vjp(const T* xyz, const size_t n_samples, const T* sph_grad, T* xyz_grad, void* cuda_stream = nullptr);

    /// Fused second-order backward (no counterpart in the reference's C++ classes): the
    /// vector-Jacobian product of the values-and-gradients map,
    /// xyz_grad[i][b] = sum_k sph_grad[i][k] dsph[i][b][k] + sum_{a,k} dsph_grad[i][a][k] ddsph[i][a][b][k],
    /// with neither dsph nor ddsph written to memory. sph_grad (n_samples x (l_max+1)^2) may be null,
    /// dsph_grad is n_samples x 3 x (l_max+1)^2, xyz_grad is n_samples x 3; device pointers.
    void compute_vjp_with_gradients(
        const T* xyz, const size_t n_samples, const T* sph_grad, const T* dsph_grad, T* xyz_grad,
        void* cuda_stream = nullptr
    );

    /// Values of selected degree blocks only, packed, scaled and with the input axes permuted, in one
    /// pass (no counterpart in the reference's C++ classes; it serves callers such as the reference's
    /// e3nn adaptor, sphericart-torch/python/sphericart/torch/e3nn.py:47-80, which evaluates every degree
    /// and then slices, permutes and rescales). l_list: n_l distinct degrees <= l_max (HOST pointer), in
    /// the order their blocks appear in the output; out is n_samples x sum(2l+1) (device pointer);
    /// axis_order: three HOST ints, a permutation of 0, 1, 2 giving the input columns that hold x, y, z
    /// (null: 0, 1, 2); scales: n_l HOST factors, one per listed degree (null: all 1). Needs
    /// l_max <= 20 (the compile-time kernels); throws std::runtime_error otherwise.
    void compute_selected(
        const T* xyz, const size_t n_samples, const int* l_list, const size_t n_l, const int* axis_order,
        const T* scales, T* out, void* cuda_stream = nullptr
    );

    /// Fused vector-Jacobian product of compute_selected: out_grad is n_samples x sum(2l+1) in the
    /// packed layout, xyz_grad is n_samples x 3 in the caller's axis order; the gradients of the
    /// harmonics are never written to memory.
    void compute_selected_vjp(
        const T* xyz, const size_t n_samples, const int* l_list, const size_t n_l, const int* axis_order,
        const T* scales, const T* out_grad, T* xyz_grad, void* cuda_stream = nullptr
    );

    template <typename U> friend class SolidHarmonics;

  private:
    // The member list mirrors the reference class so that sizeof and offsets agree. Members this
    // implementation has no use for are kept as placeholders.
    size_t l_max;
    size_t nprefactors;            // 2 * (l_max+1)(l_max+2)/2 table entries
    bool normalized;               // true: spherical harmonics, false: solid harmonics
    T* prefactors_cpu = nullptr;   // host copy of the F and K tables
    T* prefactors_cuda = nullptr;  // opaque handle to library-owned state (per-device tables, plans)
    int device_count = 0;
    int64_t CUDA_GRID_DIM_X_ = 8;  // placeholder
    int64_t CUDA_GRID_DIM_Y_ = 8;  // placeholder
    bool cached_compute_with_gradients = false;  // placeholder
    bool cached_compute_with_hessian = false;    // placeholder
    int64_t _current_shared_mem_allocation = 0;  // placeholder

    void compute_internal(
        const T* xyz,
        const size_t n_samples,
        bool compute_with_gradients,
        bool compute_with_hessian,
        T* sph,
        T* dsph,
        T* ddsph,
        void* cuda_stream
    );
};

/// Solid harmonics r^l Y_l^m (homogeneous polynomials of x, y, z): same interface.
template <typename T> class SolidHarmonics : public SphericalHarmonics<T> {
  public:
    SolidHarmonics(size_t l_max);
};

}  // namespace cuda
}  // namespace sphericart

#endif
