// "Band" kernels: any maximum degree (run-time l_max), any derivative level, and the fused
// vector-Jacobian product. Used wherever the compile-time tile kernels do not apply: l_max > 8,
// and the cases whose 32-point tile image would not fit shared memory.
//
// Work split. A group of G lanes (G = 1, 2, 4, ... 32) shares one point, so a warp holds
// P = 32 / G consecutive points. The degrees l >= 2 are independent channels (each runs its own
// downward-in-m recurrence), and a channel costs l + 1 steps; the host deals the channels to the
// G lanes with a longest-first greedy schedule so every lane gets nearly the same number of
// steps, and each lane walks its list in ONE flat loop (channel changes happen inside the loop),
// so lanes that own several short channels finish together with the lane that owns the longest.
//
// Data movement. The P points' complete output rows are built in shared memory exactly as they
// lie in global memory ([P][ny], [P][3][ny], [P][9][ny] are contiguous spans of the outputs) and
// copied out by the whole warp with fully coalesced stores. When even a single point's rows do
// not fit, the degrees are cut into bands of consecutive l and the image holds one band of
// columns at a time. c_m, s_m and 2(m+1)z of each point are computed once and kept in shared
// memory; the prefactor tables are staged into shared memory once per CTA.
//
// No inter-warp, inter-CTA or inter-GPU communication; the only barrier is the one after the
// table load. Replaces spherical_harmonics_kernel (sphericart/src/sphericart_impl.cu:207-615)
// and, for the VJP, the reference's materialise-then-reduce backward
// (sphericart-torch/python/sphericart/torch/register.py:90-108).
#pragma once

#include "sph_core.cuh"

namespace sph_b200 {

// Layout of the host-built plan (ints, in global memory, staged to shared memory):
//   [0] number of bands   [1] slots per lane (channel list length, -1 terminated)
//   then per band: l_lo, l_hi, steps (largest per-lane step count), G * slots channel ids
constexpr int PLAN_HEADER = 2;
constexpr int PLAN_BAND_HEADER = 3;

template <typename T> struct BandArgs {
    const T* xyz;
    long long n;
    T* sph;
    T* dsph;
    T* ddsph;
    const T* sph_grad;   // VJP only
    T* xyz_grad;         // VJP only
    const T* tables;     // F then K, n_table(l_max) entries each
    const int* plan;
    int l_max;
    int plan_ints;
    int image_elems;     // per-warp image size in elements of T
};

template <typename T, int LEVEL, bool NORM, int G, bool VJP>
__global__ void __launch_bounds__(128) sph_band_kernel(const BandArgs<T> a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int P = 32 / G;
    constexpr int NCOMP = level_components(LEVEL);
    const int L = a.l_max;
    const int ny = (L + 1) * (L + 1);
    const int nq = (L + 1) * (L + 2) / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int g = lane % G;    // lane within the point's group
    const int pt = lane / G;   // point slot within the warp

    // shared memory carve-up: tables | per-warp (c, s, 2mz) | per-warp image | plan
    T* sF = reinterpret_cast<T*>(smem_raw);
    T* sK = sF + nq;
    const int csz_elems = P * 3 * (L + 1);
    T* warp_base = sK + nq + size_t(warp) * (csz_elems + a.image_elems);
    T* sc = warp_base + pt * 3 * (L + 1);
    T* ss = sc + (L + 1);
    T* stz = ss + (L + 1);
    T* image = warp_base + csz_elems;
    int* splan = reinterpret_cast<int*>(sK + nq + size_t(nwarps) * (csz_elems + a.image_elems));

    for (int e = threadIdx.x; e < 2 * nq; e += blockDim.x) sF[e] = a.tables[e];
    for (int e = threadIdx.x; e < a.plan_ints; e += blockDim.x) splan[e] = a.plan[e];
    __syncthreads();
    const int nbands = splan[0];
    const int slots = splan[1];

    const long long ngroups = (a.n + P - 1) / P;
    const long long stride = (long long)gridDim.x * nwarps;
    for (long long grp = (long long)blockIdx.x * nwarps + warp; grp < ngroups; grp += stride) {
        const long long first = grp * P;
        const long long i = first + pt;
        const bool valid = i < a.n;
        const int nvalid = (a.n - first) < P ? int(a.n - first) : P;

        T x = T(1), y = T(0), z = T(0);
        if (valid) {
            x = a.xyz[3 * i + 0];
            y = a.xyz[3 * i + 1];
            z = a.xyz[3 * i + 2];
        }
        UnitSphere<T> us{x, y, z, T(0), T(0)};
        if constexpr (NORM) {
            const T ir = T(1) / sqrt(x * x + y * y + z * z);
            x *= ir;
            y *= ir;
            z *= ir;
            us = UnitSphere<T>{x, y, z, ir, ir * ir};
        }
        const T x2 = x * x, y2 = y * y, xy = x * y;
        const T rho = x2 + y2;

        __syncwarp();  // the previous group's readers of c/s/tz and of the image are done

        // c_m, s_m, 2(m+1)z: every lane of the group runs the recurrence, lane g keeps m = g mod G
        {
            T cc = T(1), cs = T(0);
            const T twoz = z + z;
            T ctz = twoz;
            if (g == 0) {
                sc[0] = cc;
                ss[0] = cs;
                stz[0] = ctz;
            }
            for (int m = 1; m <= L; ++m) {
                const T nc = cc * x - cs * y;
                const T ns = cc * y + cs * x;
                cc = nc;
                cs = ns;
                ctz += twoz;
                if (m % G == g) {
                    sc[m] = cc;
                    ss[m] = cs;
                    stz[m] = ctz;
                }
            }
        }

        [[maybe_unused]] T ax = T(0), ay = T(0), az = T(0);  // VJP accumulators
        if constexpr (VJP) {
            // stage the P rows of the upstream gradient (one contiguous span) into the image
            const T* gsrc = a.sph_grad + first * ny;
            for (int e = lane; e < nvalid * ny; e += 32) image[e] = gsrc[e];
        }
        __syncwarp();

        for (int b = 0; b < nbands; ++b) {
            const int* band = splan + PLAN_HEADER + b * (PLAN_BAND_HEADER + G * slots);
            const int l_lo = band[0], l_hi = band[1], nsteps = band[2];
            const int kb = l_lo * l_lo;                       // first column of the band
            const int cols = (l_hi + 1) * (l_hi + 1) - kb;    // columns in the band
            T* img_sph = image + pt * cols;
            T* img_d = image + P * cols + pt * 3 * cols;
            T* img_dd = image + 4 * P * cols + pt * 9 * cols;
            const T* grow = image + pt * ny;  // VJP: this point's upstream-gradient row

            auto put = [&](int k, Column<T> v) {
                if constexpr (NORM && LEVEL >= 1) to_cartesian<T, LEVEL>(v, us);
                if constexpr (VJP) {
                    const T gk = grow[k];
                    ax += gk * v.gx;
                    ay += gk * v.gy;
                    az += gk * v.gz;
                } else {
                    const int kc = k - kb;
                    img_sph[kc] = v.y;
                    if constexpr (LEVEL >= 1) {
                        img_d[kc] = v.gx;
                        img_d[cols + kc] = v.gy;
                        img_d[2 * cols + kc] = v.gz;
                    }
                    if constexpr (LEVEL >= 2) {
                        img_dd[0 * cols + kc] = v.hxx;
                        img_dd[1 * cols + kc] = v.hxy;
                        img_dd[2 * cols + kc] = v.hxz;
                        img_dd[3 * cols + kc] = v.hxy;
                        img_dd[4 * cols + kc] = v.hyy;
                        img_dd[5 * cols + kc] = v.hyz;
                        img_dd[6 * cols + kc] = v.hxz;
                        img_dd[7 * cols + kc] = v.hyz;
                        img_dd[8 * cols + kc] = v.hzz;
                    }
                }
            };

            // l = 0 and l = 1: closed forms, done by the group's first lane
            if (g == 0 && valid && l_lo == 0) {
                Column<T> v{};
                v.y = T(0.282094791773878);
                put(0, v);
                if (L >= 1) {
                    const T a1 = T(0.48860251190292);
                    Column<T> vy{}, vz{}, vx{};
                    vy.y = a1 * y;
                    vy.gy = a1;
                    vz.y = a1 * z;
                    vz.gz = a1;
                    vx.y = a1 * x;
                    vx.gx = a1;
                    put(1, vy);
                    put(2, vz);
                    put(3, vx);
                }
            }

            // flat loop over this lane's channels
            const int* mine = band + PLAN_BAND_HEADER + g * slots;
            int ci = 0;
            int l = valid ? mine[0] : -1;
            int m = l;
            T q1 = T(0), q2 = T(0);                     // Q_l^{m+1},     Q_l^{m+2}
            [[maybe_unused]] T p1 = T(0), p2 = T(0);    // Q_{l-1}^{m+1}, Q_{l-1}^{m+2}
            [[maybe_unused]] T r1 = T(0), r2 = T(0);    // Q_{l-2}^{m+1}, Q_{l-2}^{m+2}
            for (int step = 0; step < nsteps; ++step) {
                if (l < 0) continue;
                const int rl = tri(l, 0);
                const T tzm = stz[m];
                const T cm = sc[m], sm = ss[m];
                // Q_l^m: Q_l^l is tabulated, Q_l^{l-1} = -z Q_l^l, then the recurrence
                const T q0 = (m == l) ? sK[rl + l] : ((m == l - 1) ? -z * q1 : sK[rl + m] * (tzm * q1 + rho * q2));
                const T f = sF[rl + m];
                const T pq = q0 * f;
                Column<T> vp{}, vm{};
                vp.y = pq * cm;
                vm.y = pq * sm;
                if constexpr (LEVEL >= 1) {
                    // Q_{l-1}^m by the same recurrence with row l-1 of K, started from Q_{l-1}^{l-1}
                    const int rl1 = rl - l;  // tri(l-1, 0)
                    const T p0 = (m >= l) ? T(0) : ((m == l - 1) ? sK[rl1 + m] : sK[rl1 + m] * (tzm * p1 + rho * p2));
                    const int m1 = m >= 1 ? m - 1 : 0;
                    const T cm1 = sc[m1], sm1 = ss[m1];
                    const T fm = T(m);
                    const T pqm = pq * fm;
                    const T pqs = pqm * sm1, pqc = pqm * cm1;
                    const T pdq = f * p1;
                    const T pdqx = pdq * x, pdqy = pdq * y;
                    vm.gx = pdqx * sm + pqs;
                    vp.gx = pdqx * cm + pqc;
                    vm.gy = pdqy * sm + pqc;
                    vp.gy = pdqy * cm - pqs;
                    const T flm = T(l + m);
                    const T pdz = f * flm * p0;
                    vm.gz = pdz * sm;
                    vp.gz = pdz * cm;
                    if constexpr (LEVEL >= 2) {
                        const int rl2 = rl1 - (l - 1);  // tri(l-2, 0)
                        const T r0 = (m >= l - 1) ? T(0)
                                                  : ((m == l - 2) ? sK[rl2 + m] : sK[rl2 + m] * (tzm * r1 + rho * r2));
                        const int m2 = m >= 2 ? m - 2 : 0;
                        const T cm2 = sc[m2], sm2 = ss[m2];
                        const T A = f * p1, D = f * p0, B = f * r2, E = f * r1, C = f * r0;
                        const T fmm = T(m * (m - 1));
                        const T Pc = fmm * pq * cm2, Ps = fmm * pq * sm2;
                        const T f2m = T(2 * m);
                        vp.hxx = A * cm + x2 * B * cm + f2m * x * A * cm1 + Pc;
                        vm.hxx = A * sm + x2 * B * sm + f2m * x * A * sm1 + Ps;
                        vp.hyy = A * cm + y2 * B * cm - f2m * y * A * sm1 - Pc;
                        vm.hyy = A * sm + y2 * B * sm + f2m * y * A * cm1 - Ps;
                        const T fz = T((l + m) * (l + m - 1));
                        vp.hzz = fz * C * cm;
                        vm.hzz = fz * C * sm;
                        vp.hxy = xy * B * cm + y * A * fm * cm1 - x * A * fm * sm1 - Ps;
                        vm.hxy = xy * B * sm + y * A * fm * sm1 + x * A * fm * cm1 + Pc;
                        vp.hxz = x * flm * E * cm + flm * D * fm * cm1;
                        vm.hxz = x * flm * E * sm + flm * D * fm * sm1;
                        vp.hyz = y * flm * E * cm - flm * D * fm * sm1;
                        vm.hyz = y * flm * E * sm + flm * D * fm * cm1;
                        r2 = r1;
                        r1 = r0;
                    }
                    p2 = p1;
                    p1 = p0;
                }
                q2 = q1;
                q1 = q0;
                const int mid = l * l + l;
                put(mid + m, vp);
                if (m > 0) {
                    put(mid - m, vm);
                    --m;
                } else {
                    // next channel: rows l-1 and l-2 start from "nothing above the diagonal"
                    ++ci;
                    l = mine[ci];
                    m = l;
                    if constexpr (LEVEL >= 1) p1 = p2 = T(0);
                    if constexpr (LEVEL >= 2) r1 = r2 = T(0);
                }
            }

            if constexpr (!VJP) {
                __syncwarp();  // image complete
                const long long row0 = first;
                if (cols == ny) {
                    // the image IS the global layout of these points: three linear copies
                    T* dst = a.sph + row0 * ny;
                    for (int e = lane; e < nvalid * ny; e += 32) dst[e] = image[e];
                    if constexpr (LEVEL >= 1) {
                        T* dst1 = a.dsph + row0 * 3 * ny;
                        const T* src1 = image + P * cols;
                        for (int e = lane; e < nvalid * 3 * ny; e += 32) dst1[e] = src1[e];
                    }
                    if constexpr (LEVEL >= 2) {
                        T* dst2 = a.ddsph + row0 * 9 * ny;
                        const T* src2 = image + 4 * P * cols;
                        for (int e = lane; e < nvalid * 9 * ny; e += 32) dst2[e] = src2[e];
                    }
                } else {
                    // one band of columns: a fragment of `cols` elements per (point, component)
                    for (int r = 0; r < nvalid; ++r)
                        for (int e = lane; e < cols; e += 32) a.sph[(row0 + r) * ny + kb + e] = image[r * cols + e];
                    if constexpr (LEVEL >= 1) {
                        const T* src1 = image + P * cols;
                        for (int r = 0; r < nvalid * 3; ++r)
                            for (int e = lane; e < cols; e += 32)
                                a.dsph[(row0 * 3 + r) * ny + kb + e] = src1[r * cols + e];
                    }
                    if constexpr (LEVEL >= 2) {
                        const T* src2 = image + 4 * P * cols;
                        for (int r = 0; r < nvalid * 9; ++r)
                            for (int e = lane; e < cols; e += 32)
                                a.ddsph[(row0 * 9 + r) * ny + kb + e] = src2[r * cols + e];
                    }
                }
                __syncwarp();  // image free for the next band
            }
        }

        if constexpr (VJP) {
            // sum the G partial results of each point (G is a power of two: butterfly within the group)
#pragma unroll
            for (int off = G / 2; off >= 1; off >>= 1) {
                ax += __shfl_xor_sync(0xffffffffu, ax, off);
                ay += __shfl_xor_sync(0xffffffffu, ay, off);
                az += __shfl_xor_sync(0xffffffffu, az, off);
            }
            if (g == 0 && valid) {
                a.xyz_grad[3 * i + 0] = ax;
                a.xyz_grad[3 * i + 1] = ay;
                a.xyz_grad[3 * i + 2] = az;
            }
        }
    }
}

}  // namespace sph_b200
