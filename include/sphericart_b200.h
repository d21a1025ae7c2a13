/*
 * C ABI of the B200 (sm_100a) implementation of sphericart's CUDA calculators.
 *
 * The first 20 functions are, name for name and argument for argument, the CUDA half of the
 * reference's C API (sphericart/include/sphericart.h:641-779, implemented in
 * sphericart/src/sphericart-capi.cpp:637-876); each declaration cites the line it replaces.
 * They keep the reference's conventions: *_new returns NULL on any failure, *_delete swallows
 * errors, *_compute_* prints "fatal error: <what>" to stdout and aborts the process on failure.
 *
 * The remaining functions are additions that the reference does not have: the fused
 * vector-Jacobian product, and status-returning twins of the compute calls for hosts that must
 * not be aborted (an interpreter, a server). The twins return 0 on success and non-zero on
 * failure, with the message available from sphericart_cuda_last_error().
 *
 * Common contract: xyz, sph, dsph, ddsph, sph_grad, xyz_grad are DEVICE pointers to caller-owned
 * contiguous arrays; n_samples counts points; cuda_stream is a cudaStream_t cast to void*
 * (NULL = default stream); calls enqueue work on that stream and return without synchronising;
 * the work runs on the device that owns xyz. Array shapes: xyz [n][3], sph [n][(l_max+1)^2],
 * dsph [n][3][(l_max+1)^2], ddsph [n][3][3][(l_max+1)^2], sph_grad like sph, xyz_grad like xyz.
 */
#ifndef SPHERICART_B200_H
#define SPHERICART_B200_H

#include <stddef.h>

#if defined(_WIN32)
#define SPHERICART_EXPORT __declspec(dllexport)
#else
#define SPHERICART_EXPORT __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
namespace sphericart {
namespace cuda {
template <typename T> class SphericalHarmonics;
template <typename T> class SolidHarmonics;
}  // namespace cuda
}  // namespace sphericart
/* opaque handles are the C++ calculators themselves (sphericart/include/sphericart.h:32-37) */
using sphericart_cuda_spherical_harmonics_calculator_t = sphericart::cuda::SphericalHarmonics<double>;
using sphericart_cuda_spherical_harmonics_calculator_f_t = sphericart::cuda::SphericalHarmonics<float>;
using sphericart_cuda_solid_harmonics_calculator_t = sphericart::cuda::SolidHarmonics<double>;
using sphericart_cuda_solid_harmonics_calculator_f_t = sphericart::cuda::SolidHarmonics<float>;
extern "C" {
#else
/* sphericart/include/sphericart.h:91-104 */
struct sphericart_cuda_spherical_harmonics_calculator_t;
typedef struct sphericart_cuda_spherical_harmonics_calculator_t sphericart_cuda_spherical_harmonics_calculator_t;
struct sphericart_cuda_spherical_harmonics_calculator_f_t;
typedef struct sphericart_cuda_spherical_harmonics_calculator_f_t sphericart_cuda_spherical_harmonics_calculator_f_t;
struct sphericart_cuda_solid_harmonics_calculator_t;
typedef struct sphericart_cuda_solid_harmonics_calculator_t sphericart_cuda_solid_harmonics_calculator_t;
struct sphericart_cuda_solid_harmonics_calculator_f_t;
typedef struct sphericart_cuda_solid_harmonics_calculator_f_t sphericart_cuda_solid_harmonics_calculator_f_t;
#endif

/* ---- spherical harmonics: the reference's entry points ---- */

/* replaces sphericart/include/sphericart.h:641 */
SPHERICART_EXPORT sphericart_cuda_spherical_harmonics_calculator_t* sphericart_cuda_spherical_harmonics_new(size_t l_max);

/* replaces sphericart/include/sphericart.h:649 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_delete(sphericart_cuda_spherical_harmonics_calculator_t* calculator);

/* replaces sphericart/include/sphericart.h:657 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_array(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, double* sph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:673 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_array_with_gradients(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, double* sph, double* dsph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:691 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_array_with_hessians(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, double* sph, double* dsph, double* ddsph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:645 */
SPHERICART_EXPORT sphericart_cuda_spherical_harmonics_calculator_f_t* sphericart_cuda_spherical_harmonics_new_f(size_t l_max);

/* replaces sphericart/include/sphericart.h:653 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_delete_f(sphericart_cuda_spherical_harmonics_calculator_f_t* calculator);

/* replaces sphericart/include/sphericart.h:665 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_array_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, float* sph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:682 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_array_with_gradients_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, float* sph, float* dsph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:701 */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_array_with_hessians_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, float* sph, float* dsph, float* ddsph, void* cuda_stream);

/* ---- solid harmonics: the reference's entry points ---- */

/* replaces sphericart/include/sphericart.h:711 */
SPHERICART_EXPORT sphericart_cuda_solid_harmonics_calculator_t* sphericart_cuda_solid_harmonics_new(size_t l_max);

/* replaces sphericart/include/sphericart.h:719 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_delete(sphericart_cuda_solid_harmonics_calculator_t* calculator);

/* replaces sphericart/include/sphericart.h:727 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_array(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, double* sph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:743 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_array_with_gradients(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, double* sph, double* dsph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:761 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_array_with_hessians(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, double* sph, double* dsph, double* ddsph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:715 */
SPHERICART_EXPORT sphericart_cuda_solid_harmonics_calculator_f_t* sphericart_cuda_solid_harmonics_new_f(size_t l_max);

/* replaces sphericart/include/sphericart.h:723 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_delete_f(sphericart_cuda_solid_harmonics_calculator_f_t* calculator);

/* replaces sphericart/include/sphericart.h:735 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_array_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, float* sph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:752 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_array_with_gradients_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, float* sph, float* dsph, void* cuda_stream);

/* replaces sphericart/include/sphericart.h:771 */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_array_with_hessians_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, float* sph, float* dsph, float* ddsph, void* cuda_stream);

/* ---- additions (no counterpart in the reference's C API) ---- */

/* Message of the last failure reported on the calling thread by a *_try_* function or by
 * *_new (empty string if none). The pointer stays valid until the thread's next failing call. */
SPHERICART_EXPORT const char* sphericart_cuda_last_error(void);

/* No counterpart in the reference. Name of the kernel family that serves a call on a B200:
 * kind 0, 1, 2 = values, + gradients, + Hessians; 3 = fused VJP; 4 = fused second-order VJP;
 * elem_bytes 4 (float) or 8 (double). Returns "sph_tile_kernel", "sph_vjp_tile_kernel",
 * "sph_vjp2_tile_kernel", "sph_panel_kernel", "sph_panel_vjp_kernel" or "sph_band_kernel" (a static string; "" for arguments
 * out of range). Launches nothing; benchmarks and profiles use it to label what they time. */
SPHERICART_EXPORT const char* sphericart_cuda_kernel_family(int kind, size_t l_max, int elem_bytes);

/* The kernels' only waits are on their own asynchronous copies and are bounded; a wait that ever
 * gave up records it on the device. Returns 1 if that happened on the current device since the
 * library was loaded, 0 if not, -1 if the flags could not be read. Synchronises the device. */
SPHERICART_EXPORT int sphericart_cuda_device_wait_errors(void);

/* Fused backward of the values: xyz_grad[i][a] = sum_k sph_grad[i][k] * dsph[i][a][k], dsph never
 * materialised. Fuses what sphericart-torch/python/sphericart/torch/register.py:90-108 does with a
 * gradients launch plus a product and a reduction. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_vjp(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, double* xyz_grad, void* cuda_stream);

/* Status-returning form of the three compute calls: level 0 = values (dsph, ddsph ignored),
 * 1 = + gradients, 2 = + Hessians. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_try_compute(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, int level, const double* xyz, size_t n_samples, double* sph, double* dsph, double* ddsph,
    void* cuda_stream);

/* Status-returning form of compute_vjp. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_try_compute_vjp(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, double* xyz_grad, void* cuda_stream);

/* Fused backward of the values: xyz_grad[i][a] = sum_k sph_grad[i][k] * dsph[i][a][k], dsph never
 * materialised. Fuses what sphericart-torch/python/sphericart/torch/register.py:90-108 does with a
 * gradients launch plus a product and a reduction. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_vjp_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, float* xyz_grad, void* cuda_stream);

/* Status-returning form of the three compute calls: level 0 = values (dsph, ddsph ignored),
 * 1 = + gradients, 2 = + Hessians. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_try_compute_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, int level, const float* xyz, size_t n_samples, float* sph, float* dsph, float* ddsph,
    void* cuda_stream);

/* Status-returning form of compute_vjp. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_try_compute_vjp_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, float* xyz_grad, void* cuda_stream);

/* Fused backward of the values: xyz_grad[i][a] = sum_k sph_grad[i][k] * dsph[i][a][k], dsph never
 * materialised. Fuses what sphericart-torch/python/sphericart/torch/register.py:90-108 does with a
 * gradients launch plus a product and a reduction. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_vjp(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, double* xyz_grad, void* cuda_stream);

/* Status-returning form of the three compute calls: level 0 = values (dsph, ddsph ignored),
 * 1 = + gradients, 2 = + Hessians. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_try_compute(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, int level, const double* xyz, size_t n_samples, double* sph, double* dsph, double* ddsph,
    void* cuda_stream);

/* Status-returning form of compute_vjp. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_try_compute_vjp(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, double* xyz_grad, void* cuda_stream);

/* Fused backward of the values: xyz_grad[i][a] = sum_k sph_grad[i][k] * dsph[i][a][k], dsph never
 * materialised. Fuses what sphericart-torch/python/sphericart/torch/register.py:90-108 does with a
 * gradients launch plus a product and a reduction. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_vjp_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, float* xyz_grad, void* cuda_stream);

/* Status-returning form of the three compute calls: level 0 = values (dsph, ddsph ignored),
 * 1 = + gradients, 2 = + Hessians. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_try_compute_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, int level, const float* xyz, size_t n_samples, float* sph, float* dsph, float* ddsph,
    void* cuda_stream);

/* Status-returning form of compute_vjp. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_try_compute_vjp_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, float* xyz_grad, void* cuda_stream);

/* Fused second-order backward (no counterpart in the reference's C API): the VJP of the
 * values-and-gradients map, xyz_grad[i][b] = sum_k sph_grad[i][k] dsph[i][b][k]
 * + sum_(a,k) dsph_grad[i][a][k] ddsph[i][a][b][k], without materialising dsph or ddsph. Fuses what
 * sphericart-torch/python/sphericart/torch/register.py:117-145 does with a Hessians launch plus products and
 * reductions. sph_grad may be NULL. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_vjp_with_gradients(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, const double* dsph_grad, double* xyz_grad,
    void* cuda_stream);

/* Status-returning form of compute_vjp_with_gradients. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_try_compute_vjp_with_gradients(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, const double* dsph_grad, double* xyz_grad,
    void* cuda_stream);

/* Fused second-order backward (no counterpart in the reference's C API): the VJP of the
 * values-and-gradients map, xyz_grad[i][b] = sum_k sph_grad[i][k] dsph[i][b][k]
 * + sum_(a,k) dsph_grad[i][a][k] ddsph[i][a][b][k], without materialising dsph or ddsph. Fuses what
 * sphericart-torch/python/sphericart/torch/register.py:117-145 does with a Hessians launch plus products and
 * reductions. sph_grad may be NULL. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_spherical_harmonics_compute_vjp_with_gradients_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, const float* dsph_grad, float* xyz_grad,
    void* cuda_stream);

/* Status-returning form of compute_vjp_with_gradients. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_try_compute_vjp_with_gradients_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, const float* dsph_grad, float* xyz_grad,
    void* cuda_stream);

/* Fused second-order backward (no counterpart in the reference's C API): the VJP of the
 * values-and-gradients map, xyz_grad[i][b] = sum_k sph_grad[i][k] dsph[i][b][k]
 * + sum_(a,k) dsph_grad[i][a][k] ddsph[i][a][b][k], without materialising dsph or ddsph. Fuses what
 * sphericart-torch/python/sphericart/torch/register.py:117-145 does with a Hessians launch plus products and
 * reductions. sph_grad may be NULL. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_vjp_with_gradients(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, const double* dsph_grad, double* xyz_grad,
    void* cuda_stream);

/* Status-returning form of compute_vjp_with_gradients. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_try_compute_vjp_with_gradients(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const double* sph_grad, const double* dsph_grad, double* xyz_grad,
    void* cuda_stream);

/* Fused second-order backward (no counterpart in the reference's C API): the VJP of the
 * values-and-gradients map, xyz_grad[i][b] = sum_k sph_grad[i][k] dsph[i][b][k]
 * + sum_(a,k) dsph_grad[i][a][k] ddsph[i][a][b][k], without materialising dsph or ddsph. Fuses what
 * sphericart-torch/python/sphericart/torch/register.py:117-145 does with a Hessians launch plus products and
 * reductions. sph_grad may be NULL. Aborts on failure like the reference's compute calls. */
SPHERICART_EXPORT void sphericart_cuda_solid_harmonics_compute_vjp_with_gradients_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, const float* dsph_grad, float* xyz_grad,
    void* cuda_stream);

/* Status-returning form of compute_vjp_with_gradients. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_try_compute_vjp_with_gradients_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const float* sph_grad, const float* dsph_grad, float* xyz_grad,
    void* cuda_stream);

/* No counterpart in the reference's C API. Values of selected degree blocks of the spherical (normalised) harmonics
 * only, packed, scaled and with the input axes permuted, in one pass (what the reference's e3nn adaptor,
 * sphericart-torch/python/sphericart/torch/e3nn.py:47-80, composes from a full evaluation, a slice, a
 * permutation and a multiplication). l_list: n_l distinct degrees <= l_max, HOST pointer, in output order;
 * out: n_samples x sum(2l+1), device pointer; axis_order: 3 HOST ints, the input columns holding x, y, z
 * (NULL: 0, 1, 2); scales: n_l HOST factors (NULL: 1). Needs l_max <= 20. Returns 0 on success, otherwise
 * non-zero with the message in sphericart_cuda_last_error(). */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_compute_selected(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const double* scales, double* out, void* cuda_stream);

/* No counterpart in the reference's C API. Fused vector-Jacobian product of compute_selected:
 * out_grad is n_samples x sum(2l+1) in the packed layout, xyz_grad n_samples x 3 in the caller's axis
 * order (device pointers); gradients of the harmonics are never written to memory. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_compute_selected_vjp(
    sphericart_cuda_spherical_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const double* scales, const double* out_grad, double* xyz_grad, void* cuda_stream);

/* No counterpart in the reference's C API. Values of selected degree blocks of the spherical (normalised) harmonics
 * only, packed, scaled and with the input axes permuted, in one pass (what the reference's e3nn adaptor,
 * sphericart-torch/python/sphericart/torch/e3nn.py:47-80, composes from a full evaluation, a slice, a
 * permutation and a multiplication). l_list: n_l distinct degrees <= l_max, HOST pointer, in output order;
 * out: n_samples x sum(2l+1), device pointer; axis_order: 3 HOST ints, the input columns holding x, y, z
 * (NULL: 0, 1, 2); scales: n_l HOST factors (NULL: 1). Needs l_max <= 20. Returns 0 on success, otherwise
 * non-zero with the message in sphericart_cuda_last_error(). */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_compute_selected_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const float* scales, float* out, void* cuda_stream);

/* No counterpart in the reference's C API. Fused vector-Jacobian product of compute_selected_f:
 * out_grad is n_samples x sum(2l+1) in the packed layout, xyz_grad n_samples x 3 in the caller's axis
 * order (device pointers); gradients of the harmonics are never written to memory. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_spherical_harmonics_compute_selected_vjp_f(
    sphericart_cuda_spherical_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const float* scales, const float* out_grad, float* xyz_grad, void* cuda_stream);

/* No counterpart in the reference's C API. Values of selected degree blocks of the solid harmonics
 * only, packed, scaled and with the input axes permuted, in one pass (what the reference's e3nn adaptor,
 * sphericart-torch/python/sphericart/torch/e3nn.py:47-80, composes from a full evaluation, a slice, a
 * permutation and a multiplication). l_list: n_l distinct degrees <= l_max, HOST pointer, in output order;
 * out: n_samples x sum(2l+1), device pointer; axis_order: 3 HOST ints, the input columns holding x, y, z
 * (NULL: 0, 1, 2); scales: n_l HOST factors (NULL: 1). Needs l_max <= 20. Returns 0 on success, otherwise
 * non-zero with the message in sphericart_cuda_last_error(). */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_compute_selected(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const double* scales, double* out, void* cuda_stream);

/* No counterpart in the reference's C API. Fused vector-Jacobian product of compute_selected:
 * out_grad is n_samples x sum(2l+1) in the packed layout, xyz_grad n_samples x 3 in the caller's axis
 * order (device pointers); gradients of the harmonics are never written to memory. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_compute_selected_vjp(
    sphericart_cuda_solid_harmonics_calculator_t* calculator, const double* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const double* scales, const double* out_grad, double* xyz_grad, void* cuda_stream);

/* No counterpart in the reference's C API. Values of selected degree blocks of the solid harmonics
 * only, packed, scaled and with the input axes permuted, in one pass (what the reference's e3nn adaptor,
 * sphericart-torch/python/sphericart/torch/e3nn.py:47-80, composes from a full evaluation, a slice, a
 * permutation and a multiplication). l_list: n_l distinct degrees <= l_max, HOST pointer, in output order;
 * out: n_samples x sum(2l+1), device pointer; axis_order: 3 HOST ints, the input columns holding x, y, z
 * (NULL: 0, 1, 2); scales: n_l HOST factors (NULL: 1). Needs l_max <= 20. Returns 0 on success, otherwise
 * non-zero with the message in sphericart_cuda_last_error(). */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_compute_selected_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const float* scales, float* out, void* cuda_stream);

/* No counterpart in the reference's C API. Fused vector-Jacobian product of compute_selected_f:
 * out_grad is n_samples x sum(2l+1) in the packed layout, xyz_grad n_samples x 3 in the caller's axis
 * order (device pointers); gradients of the harmonics are never written to memory. Returns 0 on success. */
SPHERICART_EXPORT int sphericart_cuda_solid_harmonics_compute_selected_vjp_f(
    sphericart_cuda_solid_harmonics_calculator_f_t* calculator, const float* xyz, size_t n_samples, const int* l_list, size_t n_l, const int* axis_order,
    const float* scales, const float* out_grad, float* xyz_grad, void* cuda_stream);

/* No counterpart in the reference. Values and gradients (float64, level 1) for hosts that do not
 * let a plugin allocate device memory of its own - a runtime that reserved the whole device arena
 * at start-up, or a latency-bound service loop where cudaMalloc's device-wide synchronisation is
 * not acceptable. The calculators above cudaMalloc their tables on first use of their run-time-
 * degree kernel (values and gradients: l_max > 10); this
 * entry point instead keeps them in a fixed 16 KiB array that is part of the library image (every
 * GPU that loads the library holds it until the process exits) and calls no allocating routine.
 * Limit: l_max <= 32; larger values are rejected with an error. normalized != 0 selects spherical
 * harmonics, 0 solid harmonics. The first call on each device looks up the array's device address
 * and opts the kernel into its shared memory, so make that call before any stream capture. The
 * first call on a device and any call whose l_max differs from the previous call's also enqueue a
 * small host-to-device copy of the tables (from a host table the library keeps for the life of the
 * process) in front of the kernel; a call made during stream capture always records that copy. All
 * calls on a device share the array: calls that can overlap on the GPU race on it, so order them.
 * Returns 0 on success; otherwise non-zero, message in sphericart_cuda_last_error(). */
SPHERICART_EXPORT int sphericart_cuda_harmonics_with_gradients_no_alloc(
    int normalized, size_t l_max, const double* xyz, size_t n_samples, double* sph, double* dsph, void* cuda_stream);

#ifdef __cplusplus
}
#endif

#endif
