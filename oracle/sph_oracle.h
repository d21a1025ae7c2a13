/*
 * CPU restatement of sphericart's harmonics evaluation. TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA library and the "port" CPU baseline of the benchmark.
 * The shipped library never links, loads or calls it.
 *
 * Parity status: pinned. tests/test_oracle.py checks this restatement against outputs of
 * the reference's own CPU library (committed fixtures under tests/golden/, and the live
 * library under oracle/_ref/ when it has been built) and against scipy's known answers.
 *
 * Conventions (sphericart/include/templates.hpp:54-97,333-615 and
 * sphericart/include/templates_core.hpp:29-427 in the reference):
 *   ny = (l_max+1)^2, column of (l,m) is l*l + l + m
 *   sph   [n][ny]
 *   dsph  [n][3][ny]       order x, y, z
 *   ddsph [n][3][3][ny]    order xx, xy, xz, yx, yy, yz, zx, zy, zz
 *   level: 0 = values, 1 = + gradients, 2 = + Hessians
 *   normalized != 0 evaluates Y(r/|r|) ("SphericalHarmonics"), 0 evaluates the
 *   homogeneous polynomials r^l Y ("SolidHarmonics").
 */
#ifndef SPH_ORACLE_H
#define SPH_ORACLE_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* factors has 2*nq entries, nq = (l_max+1)(l_max+2)/2: F table then K table. */
void sph_oracle_prefactors_f64(int l_max, double* factors);
void sph_oracle_prefactors_f32(int l_max, float* factors);

/* nthreads <= 0 means "all OpenMP threads". Returns the thread count used. */
int sph_oracle_compute_f64(int l_max, int normalized, int level, const double* xyz, size_t n,
                           double* sph, double* dsph, double* ddsph, int nthreads);
int sph_oracle_compute_f32(int l_max, int normalized, int level, const float* xyz, size_t n,
                           float* sph, float* dsph, float* ddsph, int nthreads);

/* xyz_grad[i][a] = sum_k sph_grad[i][k] * dsph[i][a][k]  (what the reference's autograd
 * backward computes, sphericart-torch/python/sphericart/torch/register.py:90-108) */
int sph_oracle_vjp_f64(int l_max, int normalized, const double* xyz, const double* sph_grad,
                       size_t n, double* xyz_grad, int nthreads);
int sph_oracle_vjp_f32(int l_max, int normalized, const float* xyz, const float* sph_grad,
                       size_t n, float* xyz_grad, int nthreads);

#ifdef __cplusplus
}
#endif
#endif
