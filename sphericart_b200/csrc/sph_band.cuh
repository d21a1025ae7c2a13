// "Band" kernels: any maximum degree (run-time l_max), any derivative level, and the fused
// vector-Jacobian product. Used wherever the compile-time tile kernels do not apply (see
// tile_serves() in sph_launch.hpp: high degrees, and the cases with rows so long that too few tile
// images fit an SM).
//
// Two phases per point, G lanes (1, 2, 4, ... 32) sharing a point, P = 32 / G points per warp:
//
//  A. The point's whole table Q_l^m (0 <= m <= l <= l_max) is built in shared memory with the
//     reference's downward-in-m recurrence, one row (one degree) per lane, together with
//     c_m, s_m and 2(m+1)z. Rows carry four zeros after the diagonal, two all-zero rows precede
//     row 0, and c, s carry two zeros before m = 0, so that every "term absent" case of the
//     derivative formulas (and the degrees 0 and 1) reads a zero instead of branching.
//  B. The (l, m) pairs are independent once the table exists. They are dealt round-robin to the
//     G lanes (pair t goes to lane t mod G), so the load is balanced to within one pair for any
//     l_max, consecutive lanes work on consecutive m of the same degree (their table reads and
//     their output writes are consecutive words), and there is no per-lane recurrence state,
//     hence no serial dependence between a lane's steps; two pairs are in flight per lane.
//
// Data movement, two modes chosen on the host:
//  * IMAGE: the P points' complete output rows are built in shared memory exactly as they lie in
//    global memory ([P][ny], [P][3][ny], [P][9][ny] are contiguous spans of the outputs) and each
//    span is handed to the TMA engine as a 1-D bulk store (cp.async.bulk.global.shared::cta).
//    A span may start at any 4- or 8-byte boundary, so its image is placed in shared memory at the
//    same offset modulo 16 bytes; the few elements before the first and after the last 16-byte
//    boundary are written with plain stores and the aligned body goes through the engine.
//  * DIRECT: for rows so long that an image would leave room for only a few warps per SM, phase B
//    stores straight to global memory. Consecutive lanes hold consecutive m, so every store
//    instruction writes one contiguous run of a row; neighbouring runs are written by the same
//    warp moments later and merge in L2. No image, so many more warps fit and hide latency.
//
// No inter-warp, inter-CTA or inter-GPU communication; the only block-wide barrier is the one
// after the prefactor tables are staged. Replaces spherical_harmonics_kernel
// (sphericart/src/sphericart_impl.cu:207-615) and, for the VJP, the reference's
// materialise-then-reduce backward (sphericart-torch/python/sphericart/torch/register.py:90-108).
#pragma once

#include <cstdint>

#include "sph_core.cuh"
#include "sph_packed.cuh"  // float32: both columns of a pair with packed two-wide instructions
#include "sph_tile.cuh"    // bulk-store helpers

namespace sph_b200 {

constexpr int BAND_ROW_PAD = 4;    // zeros after the diagonal of every Q row
constexpr int BAND_ZERO_ROWS = 2;  // all-zero rows standing in for degrees -1 and -2

// Row stride of the per-point Q table: room for the padding, and even so that lanes working on
// different rows at the same distance from the diagonal hit different banks.
__host__ __device__ constexpr int band_row_stride(int l_max) {
    return (l_max + 1 + BAND_ROW_PAD) + ((l_max + 1 + BAND_ROW_PAD) & 1);
}

// Elements of per-point state: 2 + (l_max+1) for c, the same for s, then the Q table.
__host__ __device__ constexpr int band_point_state(int l_max) {
    return 2 * (l_max + 3) + (l_max + 1 + BAND_ZERO_ROWS) * band_row_stride(l_max);
}

// Round an element count up so that the next region starts 16-byte aligned.
template <typename T> __host__ __device__ constexpr int align16_elems(int n) {
    constexpr int q = 16 / int(sizeof(T));
    return (n + q - 1) / q * q;
}

// Image regions of one warp (elements): each has one 16-byte slot of slack for the alignment shift.
template <typename T> __host__ __device__ constexpr int band_region(int points, int comps, int cols) {
    return align16_elems<T>(points * comps * cols) + 16 / int(sizeof(T));
}

enum BandMode : int { BAND_IMAGE_BULK = 0, BAND_IMAGE_PLAIN = 1, BAND_DIRECT = 2 };

template <typename T> struct BandArgs {
    const T* xyz;
    long long n;
    T* sph;
    T* dsph;
    T* ddsph;
    const T* sph_grad;   // VJP only (may be null in the second-order VJP)
    const T* dsph_grad;  // second-order VJP only
    T* xyz_grad;         // VJP only
    const T* tables;    // F then K, n_table(l_max) entries each
    int l_max;
    int mode;           // BAND_IMAGE_BULK or BAND_IMAGE_PLAIN (ignored by the VJP and by DIRECT kernels)
};

// ---- explicit shared-memory access with 32-bit addresses and constant offsets -----------------
template <typename T, int OFF_ELEMS> __device__ __forceinline__ T lds_at(unsigned addr) {
    T v;
    if constexpr (sizeof(T) == 4) {
        asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(OFF_ELEMS * 4));
    } else {
        asm volatile("ld.shared.f64 %0, [%1+%2];" : "=d"(v) : "r"(addr), "n"(OFF_ELEMS * 8));
    }
    return v;
}

template <typename T> __device__ __forceinline__ void sts_to(unsigned addr, T v) {
    if constexpr (sizeof(T) == 4) {
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
    } else {
        asm volatile("st.shared.f64 [%0], %1;" ::"r"(addr), "d"(v) : "memory");
    }
}

// Per-pair constants, the same for every point, built once per CTA: where the pair's inputs sit
// in the per-point state and in F, which column it produces, and the integer factors of the
// derivative formulas as floating-point numbers.
struct PairDesc {
    int q_off;  // byte offset of Q_{l-2}^{m} in the point's Q table (rows l-1, l at +row stride)
    int f_off;  // byte offset of F[l][m]
    int kp;     // column l*l + l + m  (the -m column is kp - 2m)
    int m;
};
__host__ __device__ constexpr int band_pair_factors(int level) { return level == 0 ? 0 : (level == 1 ? 2 : 4); }

// Everything phase B reads for one (l, m) pair.
template <typename T, int LEVEL> struct PairInputs {
    int kp, m;
    T f, q, cm, sm;
    T q1a, q1b, cm1, sm1;       // Q_{l-1}^{m+1}, Q_{l-1}^{m}, c_{m-1}, s_{m-1}
    T q2a, q2b, q2c, cm2, sm2;  // Q_{l-2}^{m+2}, Q_{l-2}^{m+1}, Q_{l-2}^{m}, c_{m-2}, s_{m-2}
    T fm, flm, fmm, fz;         // m, l+m, m(m-1), (l+m)(l+m-1)
};

// sQ_addr: shared address of the point's row -2; sc_addr, ss_addr: of c_{-2}, s_{-2};
// row_b: Q row stride in bytes.
template <typename T, int LEVEL>
__device__ __forceinline__ PairInputs<T, LEVEL> band_load_pair(const PairDesc d, unsigned sF_addr, unsigned sQ_addr,
                                                               unsigned sc_addr, unsigned ss_addr, unsigned row_b,
                                                               unsigned fac_addr) {
    PairInputs<T, LEVEL> in;
    in.kp = d.kp;
    in.m = d.m;
    const unsigned m_b = unsigned(d.m) * unsigned(sizeof(T));
    const unsigned a2 = sQ_addr + unsigned(d.q_off);  // row l-2, column m
    const unsigned a1 = a2 + row_b;                   // row l-1
    const unsigned a0 = a1 + row_b;                   // row l
    const unsigned ac = sc_addr + m_b;                // c_{m-2}
    const unsigned as = ss_addr + m_b;                // s_{m-2}
    in.f = lds_at<T, 0>(sF_addr + unsigned(d.f_off));
    in.q = lds_at<T, 0>(a0);
    in.cm = lds_at<T, 2>(ac);
    in.sm = lds_at<T, 2>(as);
    if constexpr (LEVEL >= 1) {
        in.q1a = lds_at<T, 1>(a1);
        in.q1b = lds_at<T, 0>(a1);
        in.cm1 = lds_at<T, 1>(ac);
        in.sm1 = lds_at<T, 1>(as);
        in.fm = lds_at<T, 0>(fac_addr);
        in.flm = lds_at<T, 1>(fac_addr);
    }
    if constexpr (LEVEL >= 2) {
        in.q2a = lds_at<T, 2>(a2);
        in.q2b = lds_at<T, 1>(a2);
        in.q2c = lds_at<T, 0>(a2);
        in.cm2 = lds_at<T, 0>(ac);
        in.sm2 = lds_at<T, 0>(as);
        in.fmm = lds_at<T, 2>(fac_addr);
        in.fz = lds_at<T, 3>(fac_addr);
    }
    return in;
}

// Raw columns +m (cosine-like) and -m (sine-like) of one pair; same expressions as the
// reference's channel code (sphericart/include/templates_core.hpp:201-292, 392-426) with the
// out-of-range Q entries reading as zero.
template <typename T, int LEVEL>
__device__ __forceinline__ void band_eval_pair(const PairInputs<T, LEVEL>& in, T x, T y, T x2, T y2, T xy,
                                               Column<T>& vp, Column<T>& vm) {
    const T f = in.f, cm = in.cm, sm = in.sm;
    const T pq = in.q * f;
    vp.y = pq * cm;
    vm.y = pq * sm;
    if constexpr (LEVEL >= 1) {
        const T cm1 = in.cm1, sm1 = in.sm1;
        const T fm = in.fm;
        const T pqm = pq * fm;
        const T pqs = pqm * sm1, pqc = pqm * cm1;
        const T pdq = f * in.q1a;
        const T pdqx = pdq * x, pdqy = pdq * y;
        vm.gx = pdqx * sm + pqs;
        vp.gx = pdqx * cm + pqc;
        vm.gy = pdqy * sm + pqc;
        vp.gy = pdqy * cm - pqs;
        const T flm = in.flm;
        const T pdz = f * flm * in.q1b;
        vm.gz = pdz * sm;
        vp.gz = pdz * cm;
        if constexpr (LEVEL >= 2) {
            const T A = f * in.q1a, D = f * in.q1b;
            const T B = f * in.q2a, E = f * in.q2b, C = f * in.q2c;
            const T fmm = in.fmm;
            const T Pc = fmm * pq * in.cm2, Ps = fmm * pq * in.sm2;
            const T f2m = fm + fm;
            vp.hxx = A * cm + x2 * B * cm + f2m * x * A * cm1 + Pc;
            vm.hxx = A * sm + x2 * B * sm + f2m * x * A * sm1 + Ps;
            vp.hyy = A * cm + y2 * B * cm - f2m * y * A * sm1 - Pc;
            vm.hyy = A * sm + y2 * B * sm + f2m * y * A * cm1 - Ps;
            const T fz = in.fz;
            vp.hzz = fz * C * cm;
            vm.hzz = fz * C * sm;
            vp.hxy = xy * B * cm + y * A * fm * cm1 - x * A * fm * sm1 - Ps;
            vm.hxy = xy * B * sm + y * A * fm * sm1 + x * A * fm * cm1 + Pc;
            vp.hxz = x * flm * E * cm + flm * D * fm * cm1;
            vm.hxz = x * flm * E * sm + flm * D * fm * sm1;
            vp.hyz = y * flm * E * cm - flm * D * fm * sm1;
            vm.hyz = y * flm * E * sm + flm * D * fm * cm1;
        }
    }
}

template <typename T, int LEVEL, bool NORM, int G, bool VJP, bool DIRECT>
__global__ void __launch_bounds__(128) sph_band_kernel(const __grid_constant__ BandArgs<T> a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int P = 32 / G;
    const int L = a.l_max;
    const int ny = (L + 1) * (L + 1);
    const int nq = (L + 1) * (L + 2) / 2;
    const int RS = band_row_stride(L);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int g = lane % G;   // lane within the point's group
    const int pt = lane / G;  // point slot within the warp
    constexpr bool direct = DIRECT;  // store straight to global memory, no image
    static_assert(!(VJP && DIRECT), "the VJP has no output image");
    const bool bulk = !VJP && !DIRECT && a.mode == BAND_IMAGE_BULK;

    // shared memory carve-up: F | K | pair factors | pair descriptors | per warp: P point states,
    // then the image regions
    constexpr int NF = band_pair_factors(LEVEL);
    T* sF = reinterpret_cast<T*>(smem_raw);
    T* sK = sF + nq;
    T* sFac = sF + align16_elems<T>(2 * nq);
    PairDesc* sDesc = reinterpret_cast<PairDesc*>(sFac + align16_elems<T>(nq * NF));
    T* warps_base = reinterpret_cast<T*>(sDesc + nq);
    const int state_elems = align16_elems<T>(P * band_point_state(L));
    // VJP: the staged upstream gradients, [P][ny] of sph_grad (+ [P][3][ny] of dsph_grad at LEVEL 2)
    constexpr int VJP_ROWS = LEVEL >= 2 ? 4 : 1;
    const int reg0 = VJP ? align16_elems<T>(P * VJP_ROWS * ny) : (direct ? 0 : band_region<T>(P, 1, ny));
    const int reg1 = (!VJP && !direct && LEVEL >= 1) ? band_region<T>(P, 3, ny) : 0;
    const int reg2 = (!VJP && !direct && LEVEL >= 2) ? band_region<T>(P, 9, ny) : 0;
    T* warp_base = warps_base + size_t(warp) * (state_elems + reg0 + reg1 + reg2);
    T* state = warp_base + pt * band_point_state(L);
    T* sc = state + 2;             // sc[-2], sc[-1] are zeros
    T* ss = sc + (L + 1) + 2;      // ss[-2], ss[-1] are zeros
    T* sQ = ss + (L + 1) + BAND_ZERO_ROWS * RS;  // sQ[l * RS + m], rows -2 and -1 are zeros
    T* region0 = warp_base + state_elems;
    T* region1 = region0 + reg0;
    T* region2 = region1 + reg1;

    for (int e = threadIdx.x; e < 2 * nq; e += blockDim.x) sF[e] = a.tables[e];
    // pair t of the flattened (l, m) list: l = largest integer with l(l+1)/2 <= t
    for (int t = threadIdx.x; t < nq; t += blockDim.x) {
        int l = int((sqrtf(8.0f * float(t) + 1.0f) - 1.0f) * 0.5f);
        while (tri(l + 1, 0) <= t) ++l;
        while (tri(l, 0) > t) --l;
        const int m = t - tri(l, 0);
        PairDesc d;
        d.q_off = (l * RS + m) * int(sizeof(T));  // relative to row -2, i.e. row l-2 of the table
        d.f_off = t * int(sizeof(T));
        d.kp = l * l + l + m;
        d.m = m;
        sDesc[t] = d;
        if constexpr (NF >= 2) {
            sFac[t * NF + 0] = T(m);
            sFac[t * NF + 1] = T(l + m);
        }
        if constexpr (NF >= 4) {
            sFac[t * NF + 2] = T(m * (m - 1));
            sFac[t * NF + 3] = T((l + m) * (l + m - 1));
        }
    }
    // the zero rows and the zeros before c_0, s_0 never change
    for (int e = g; e < BAND_ZERO_ROWS * RS; e += G) sQ[e - BAND_ZERO_ROWS * RS] = T(0);
    if (g == 0) sc[-2] = sc[-1] = ss[-2] = ss[-1] = T(0);
    __syncthreads();

    const long long ngroups = (a.n + P - 1) / P;
    const long long stride = (long long)gridDim.x * nwarps;
    // A group's point is fetched while the previous group is evaluated: under a saturated write
    // stream a DRAM read takes microseconds, and a warp has nothing else to do until it has its point.
    auto fetch_point = [&](long long group, T& px, T& py, T& pz) {
        px = T(1);
        py = T(0);
        pz = T(0);
        const long long ip = group * P + pt;
        if (group < ngroups && ip < a.n) {
            px = a.xyz[3 * ip + 0];
            py = a.xyz[3 * ip + 1];
            pz = a.xyz[3 * ip + 2];
        }
    };
    T next_x, next_y, next_z;
    fetch_point((long long)blockIdx.x * nwarps + warp, next_x, next_y, next_z);
    for (long long grp = (long long)blockIdx.x * nwarps + warp; grp < ngroups; grp += stride) {
        const long long first = grp * P;
        const long long i = first + pt;
        const bool valid = i < a.n;
        const int nvalid = (a.n - first) < P ? int(a.n - first) : P;

        T x = next_x, y = next_y, z = next_z;
        fetch_point(grp + stride, next_x, next_y, next_z);
        UnitSphere<T> us{x, y, z, T(0), T(0)};
        if constexpr (NORM) {
            const T ir = T(1) / sqrt(x * x + y * y + z * z);
            x *= ir;
            y *= ir;
            z *= ir;
            us = UnitSphere<T>{x, y, z, ir, ir * ir};
        }
        const T x2 = x * x, y2 = y * y, xy = x * y;

        __syncwarp();  // the previous group's phase B has finished reading the state

        // ---- phase A, in float64 for both element types. The recurrences below are where rounding
        // accumulates (an error growing with l_max in the element type); carried in float64 and rounded
        // once on storing, they make the float32 results essentially exact up to this point, so that
        // what separates them from the reference's float32 output is the reference's own rounding
        // only. The float64 pipe is otherwise idle in the float32 kernels. The inputs are the
        // element-type coordinates (normalised in the element type, as the reference does).
        const double xd = double(x), yd = double(y), zd = double(z);
        const double rhod = xd * xd + yd * yd;

        // A1: c_m + i s_m = (x + i y)^m. Lane g builds the powers m = g, g + G, ... from the repeated
        // squares of x + i y: a dozen dependent operations instead of a serial chain of 2 l_max.
        for (int m = g; m <= L; m += G) {
            double pr = 1.0, pi = 0.0;  // running product
            double wr = xd, wi = yd;    // (x + i y)^(2^b)
            for (int bits = m; bits != 0; bits >>= 1) {
                if (bits & 1) {
                    const double nr = pr * wr - pi * wi;
                    pi = pr * wi + pi * wr;
                    pr = nr;
                }
                const double sr = wr * wr - wi * wi;
                wi = (wr + wr) * wi;
                wr = sr;
            }
            sc[m] = T(pr);
            ss[m] = T(pi);
        }

        // A2: the Q table, one degree per lane, downward in m (the reference's recurrence,
        // sphericart/include/templates_core.hpp:123,155,202, with 2(m+1)z formed directly)
        for (int l = g; l <= L; l += G) {
            T* row = sQ + l * RS;
            const T* Kl = sK + tri(l, 0);
            double q2 = double(Kl[l]);  // Q_l^l is tabulated
            row[l] = T(q2);
#pragma unroll
            for (int j = 1; j <= BAND_ROW_PAD; ++j) row[l + j] = T(0);
            if (l >= 1) {
                double q1 = -zd * q2;  // Q_l^{l-1}
                row[l - 1] = T(q1);
                for (int m = l - 2; m >= 0; --m) {
                    const double q0 = double(Kl[m]) * (double(2 * (m + 1)) * zd * q1 + rhod * q2);
                    row[m] = T(q0);
                    q2 = q1;
                    q1 = q0;
                }
            }
        }

        // where this point's rows go
        T* gsph = VJP ? nullptr : a.sph + first * ny;
        T* gd = (VJP || LEVEL < 1) ? nullptr : a.dsph + first * 3 * ny;
        T* gdd = (VJP || LEVEL < 2) ? nullptr : a.ddsph + first * 9 * ny;
        // image mode: images placed so that shared and global addresses agree modulo 16 bytes
        int shift0 = 0, shift1 = 0, shift2 = 0;
        if (bulk) {
            shift0 = int((reinterpret_cast<uintptr_t>(gsph) & 15u) / sizeof(T));
            if constexpr (LEVEL >= 1) shift1 = int((reinterpret_cast<uintptr_t>(gd) & 15u) / sizeof(T));
            if constexpr (LEVEL >= 2) shift2 = int((reinterpret_cast<uintptr_t>(gdd) & 15u) / sizeof(T));
        }
        T* image0 = region0 + shift0;
        T* image1 = region1 + shift1;
        T* image2 = region2 + shift2;
        // destination of this lane's point, indexed by the column k: the image or global memory
        T* out_sph = direct ? gsph + size_t(pt) * ny : image0 + pt * ny;
        T* out_d = direct ? gd + size_t(pt) * 3 * ny : image1 + pt * 3 * ny;
        T* out_dd = direct ? gdd + size_t(pt) * 9 * ny : image2 + pt * 9 * ny;
        const T* grow = region0 + pt * ny;  // VJP: this point's upstream-gradient row

        [[maybe_unused]] T ax = T(0), ay = T(0), az = T(0);  // VJP accumulators
        // second-order VJP of the normalised harmonics: sums of raw derivatives, projected once per
        // point (see Vjp2RawSink in sph_tile.cuh for the algebra): B and C next to A = (ax, ay, az)
        constexpr bool RAW2 = VJP && LEVEL >= 2 && NORM;
        [[maybe_unused]] T rb[3] = {T(0), T(0), T(0)};
        [[maybe_unused]] T rc[9] = {T(0), T(0), T(0), T(0), T(0), T(0), T(0), T(0), T(0)};
        if constexpr (VJP) {
            // the P rows of each upstream gradient are one contiguous span: coalesced loads
            if (a.sph_grad != nullptr) {
                const T* gsrc = a.sph_grad + first * ny;
                for (int e = lane; e < nvalid * ny; e += 32) region0[e] = gsrc[e];
            } else {
                for (int e = lane; e < nvalid * ny; e += 32) region0[e] = T(0);
            }
            if constexpr (LEVEL >= 2) {
                const T* dsrc = a.dsph_grad + first * 3 * ny;
                T* ddst = region0 + P * ny;
                for (int e = lane; e < nvalid * 3 * ny; e += 32) ddst[e] = dsrc[e];
            }
        } else {
            // the engine must be done reading the images of the previous group
            if (bulk && lane == 0) bulk_wait_read_all();
        }
        __syncwarp();  // table, c/s and (VJP) gradient rows visible; images free

        // shared-memory addresses of this lane's image rows (image modes) or gradient row (VJP)
        const unsigned ny_b = unsigned(ny) * unsigned(sizeof(T));
        [[maybe_unused]] const unsigned img0_addr = static_cast<unsigned>(__cvta_generic_to_shared(VJP ? grow : out_sph));
        [[maybe_unused]] const unsigned vjp_d_addr =
            static_cast<unsigned>(__cvta_generic_to_shared(region0 + P * ny + pt * 3 * ny));
        [[maybe_unused]] const unsigned img1_addr = direct ? 0u : static_cast<unsigned>(__cvta_generic_to_shared(out_d));
        [[maybe_unused]] const unsigned img2_addr = direct ? 0u : static_cast<unsigned>(__cvta_generic_to_shared(out_dd));

        auto store_column = [&](int k, const Column<T>& v) {
            if constexpr (VJP) {
                const unsigned k_b = unsigned(k) * unsigned(sizeof(T));
                const T gk = lds_at<T, 0>(img0_addr + k_b);
                ax += gk * v.gx;
                ay += gk * v.gy;
                az += gk * v.gz;
                if constexpr (LEVEL >= 2) {
                    // second-order backward: contract the Hessian column with the dsph_grad column
                    unsigned ad = vjp_d_addr + k_b;
                    const T wx = lds_at<T, 0>(ad);
                    ad += ny_b;
                    const T wy = lds_at<T, 0>(ad);
                    ad += ny_b;
                    const T wz = lds_at<T, 0>(ad);
                    if constexpr (RAW2) {
                        const T t = T(us.x) * wx + T(us.y) * wy + T(us.z) * wz;
                        const T px = wx - T(us.x) * t, py = wy - T(us.y) * t, pz = wz - T(us.z) * t;
                        rb[0] += v.hxx * px + v.hxy * py + v.hxz * pz;
                        rb[1] += v.hxy * px + v.hyy * py + v.hyz * pz;
                        rb[2] += v.hxz * px + v.hyz * py + v.hzz * pz;
                        rc[0] += wx * v.gx;  rc[1] += wx * v.gy;  rc[2] += wx * v.gz;
                        rc[3] += wy * v.gx;  rc[4] += wy * v.gy;  rc[5] += wy * v.gz;
                        rc[6] += wz * v.gx;  rc[7] += wz * v.gy;  rc[8] += wz * v.gz;
                    } else {
                        ax += wx * v.hxx + wy * v.hxy + wz * v.hxz;
                        ay += wx * v.hxy + wy * v.hyy + wz * v.hyz;
                        az += wx * v.hxz + wy * v.hyz + wz * v.hzz;
                    }
                }
            } else if constexpr (DIRECT) {
                // streaming stores: the data is written once and never read back by this kernel
                __stcs(out_sph + k, v.y);
                if constexpr (LEVEL >= 1) {
                    T* d = out_d + k;
                    __stcs(d, v.gx);
                    __stcs(d + ny, v.gy);
                    __stcs(d + 2 * ny, v.gz);
                }
                if constexpr (LEVEL >= 2) {
                    T* h = out_dd + k;
                    __stcs(h, v.hxx);
                    __stcs(h + ny, v.hxy);
                    __stcs(h + 2 * ny, v.hxz);
                    __stcs(h + 3 * ny, v.hxy);
                    __stcs(h + 4 * ny, v.hyy);
                    __stcs(h + 5 * ny, v.hyz);
                    __stcs(h + 6 * ny, v.hxz);
                    __stcs(h + 7 * ny, v.hyz);
                    __stcs(h + 8 * ny, v.hzz);
                }
            } else {
                const unsigned k_b = unsigned(k) * unsigned(sizeof(T));
                sts_to<T>(img0_addr + k_b, v.y);
                if constexpr (LEVEL >= 1) {
                    unsigned ad = img1_addr + k_b;
                    sts_to<T>(ad, v.gx);
                    ad += ny_b;
                    sts_to<T>(ad, v.gy);
                    ad += ny_b;
                    sts_to<T>(ad, v.gz);
                }
                if constexpr (LEVEL >= 2) {
                    unsigned ah = img2_addr + k_b;
                    sts_to<T>(ah, v.hxx);
                    ah += ny_b;
                    sts_to<T>(ah, v.hxy);
                    ah += ny_b;
                    sts_to<T>(ah, v.hxz);
                    ah += ny_b;
                    sts_to<T>(ah, v.hxy);
                    ah += ny_b;
                    sts_to<T>(ah, v.hyy);
                    ah += ny_b;
                    sts_to<T>(ah, v.hyz);
                    ah += ny_b;
                    sts_to<T>(ah, v.hxz);
                    ah += ny_b;
                    sts_to<T>(ah, v.hyz);
                    ah += ny_b;
                    sts_to<T>(ah, v.hzz);
                }
            }
        };
        // float32 with derivatives: the pair's two columns go through the packed two-wide path
        constexpr bool PACKED = sizeof(T) == 4 && LEVEL >= 1;
        [[maybe_unused]] UnitSphere2 us2{};
        // (the first-order VJP applies the linear chain rule once to its sum; everything else per column)
        constexpr bool CHAIN_PER_COLUMN = NORM && LEVEL >= 1 && !VJP;
        if constexpr (PACKED && CHAIN_PER_COLUMN) {
            UnitSphere<float> usf{float(us.x), float(us.y), float(us.z), float(us.ir), float(us.irsq)};
            us2 = make_unit_sphere2<LEVEL>(usf);
        }
        auto finish_pair = [&](const PairInputs<T, LEVEL>& in) {
            if constexpr (PACKED) {
                PairScalars ps{};
                ps.f = float(in.f);
                ps.q = float(in.q);
                ps.q1a = float(in.q1a);
                ps.q1b = float(in.q1b);
                ps.fm = float(in.fm);
                ps.flm = float(in.flm);
                F2 cs2 = bc(0.0f);
                if constexpr (LEVEL >= 2) {
                    ps.q2a = float(in.q2a);
                    ps.q2b = float(in.q2b);
                    ps.q2c = float(in.q2c);
                    ps.fmm = float(in.fmm);
                    ps.fz = float(in.fz);
                    cs2 = f2(float(in.cm2), float(in.sm2));
                }
                Column2 v{};
                eval_pair2<LEVEL>(ps, f2(float(in.cm), float(in.sm)), f2(float(in.cm1), float(in.sm1)), cs2, float(x),
                                  float(y), float(x2), float(y2), float(xy), v);
                if constexpr (CHAIN_PER_COLUMN) to_cartesian2<LEVEL>(v, us2);
                Column<T> vp{}, vm{};
                vp.y = T(v.y.v.x);    vm.y = T(v.y.v.y);
                vp.gx = T(v.gx.v.x);  vm.gx = T(v.gx.v.y);
                vp.gy = T(v.gy.v.x);  vm.gy = T(v.gy.v.y);
                vp.gz = T(v.gz.v.x);  vm.gz = T(v.gz.v.y);
                if constexpr (LEVEL >= 2) {
                    vp.hxx = T(v.hxx.v.x);  vm.hxx = T(v.hxx.v.y);
                    vp.hxy = T(v.hxy.v.x);  vm.hxy = T(v.hxy.v.y);
                    vp.hxz = T(v.hxz.v.x);  vm.hxz = T(v.hxz.v.y);
                    vp.hyy = T(v.hyy.v.x);  vm.hyy = T(v.hyy.v.y);
                    vp.hyz = T(v.hyz.v.x);  vm.hyz = T(v.hyz.v.y);
                    vp.hzz = T(v.hzz.v.x);  vm.hzz = T(v.hzz.v.y);
                }
                store_column(in.kp, vp);
                if (in.m > 0) store_column(in.kp - 2 * in.m, vm);
            } else {
                Column<T> vp{}, vm{};
                band_eval_pair<T, LEVEL>(in, x, y, x2, y2, xy, vp, vm);
                if constexpr (CHAIN_PER_COLUMN) {
                    to_cartesian<T, LEVEL>(vp, us);
                    to_cartesian<T, LEVEL>(vm, us);
                }
                store_column(in.kp, vp);
                if (in.m > 0) store_column(in.kp - 2 * in.m, vm);
            }
        };

        // ---- phase B: pairs t = g, g + G, ... of the flattened (l, m) list, two in flight per lane
        const unsigned sF_addr = static_cast<unsigned>(__cvta_generic_to_shared(sF));
        const unsigned sQ_addr = static_cast<unsigned>(__cvta_generic_to_shared(sQ - BAND_ZERO_ROWS * RS));
        const unsigned sc_addr = static_cast<unsigned>(__cvta_generic_to_shared(sc - 2));
        const unsigned ss_addr = static_cast<unsigned>(__cvta_generic_to_shared(ss - 2));
        const unsigned fac_addr = static_cast<unsigned>(__cvta_generic_to_shared(sFac));
        const unsigned row_b = unsigned(RS) * unsigned(sizeof(T));
        constexpr unsigned FAC_B = unsigned(NF) * unsigned(sizeof(T));
        const unsigned desc_addr = static_cast<unsigned>(__cvta_generic_to_shared(sDesc));
        auto load = [&](int t) {
            PairDesc d;
            asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(d.q_off), "=r"(d.f_off), "=r"(d.kp), "=r"(d.m)
                         : "r"(desc_addr + unsigned(t) * 16u));
            return band_load_pair<T, LEVEL>(d, sF_addr, sQ_addr, sc_addr, ss_addr, row_b, fac_addr + unsigned(t) * FAC_B);
        };
        int t = valid ? g : nq;
        if constexpr (sizeof(T) == 8) {
            // float64 arithmetic has long dependent chains: four independent pairs per lane in flight
            for (; t + 3 * G < nq; t += 4 * G) {
                const PairInputs<T, LEVEL> in0 = load(t);
                const PairInputs<T, LEVEL> in1 = load(t + G);
                const PairInputs<T, LEVEL> in2 = load(t + 2 * G);
                const PairInputs<T, LEVEL> in3 = load(t + 3 * G);
                finish_pair(in0);
                finish_pair(in1);
                finish_pair(in2);
                finish_pair(in3);
            }
        }
        for (; t + G < nq; t += 2 * G) {
            const PairInputs<T, LEVEL> in0 = load(t);
            const PairInputs<T, LEVEL> in1 = load(t + G);
            finish_pair(in0);
            finish_pair(in1);
        }
        if (t < nq) finish_pair(load(t));

        if constexpr (!VJP) {
            if (bulk) {
                // each image is one span of the output. Elements before the first and after the last
                // 16-byte boundary go out with plain stores, the body through TMA.
                fence_proxy_async_smem();
                __syncwarp();
                constexpr int Q16 = 16 / int(sizeof(T));
                auto copy_out = [&](T* gdst, const T* img, int shift, int count) {
                    const int head = shift == 0 ? 0 : (Q16 - shift < count ? Q16 - shift : count);
                    const int body = (count - head) / Q16 * Q16;
                    const int tail = count - head - body;
                    if (lane < head) gdst[lane] = img[lane];
                    if (lane >= 8 && lane - 8 < tail) gdst[head + body + lane - 8] = img[head + body + lane - 8];
                    if (lane == 0 && body > 0)
                        bulk_store_smem_to_global(gdst + head, img + head, unsigned(body) * unsigned(sizeof(T)));
                };
                copy_out(gsph, image0, shift0, nvalid * ny);
                if constexpr (LEVEL >= 1) copy_out(gd, image1, shift1, nvalid * 3 * ny);
                if constexpr (LEVEL >= 2) copy_out(gdd, image2, shift2, nvalid * 9 * ny);
                if (lane == 0) bulk_commit();
            } else if (!direct) {
                __syncwarp();  // image complete
                for (int e = lane; e < nvalid * ny; e += 32) gsph[e] = image0[e];
                if constexpr (LEVEL >= 1)
                    for (int e = lane; e < nvalid * 3 * ny; e += 32) gd[e] = image1[e];
                if constexpr (LEVEL >= 2)
                    for (int e = lane; e < nvalid * 9 * ny; e += 32) gdd[e] = image2[e];
            }
        }

        if constexpr (VJP) {
            // sum the G partial results of each point (G is a power of two: butterfly within the group)
#pragma unroll
            for (int off = G / 2; off >= 1; off >>= 1) {
                ax += __shfl_xor_sync(0xffffffffu, ax, off);
                ay += __shfl_xor_sync(0xffffffffu, ay, off);
                az += __shfl_xor_sync(0xffffffffu, az, off);
                if constexpr (RAW2) {
#pragma unroll
                    for (int q = 0; q < 3; ++q) rb[q] += __shfl_xor_sync(0xffffffffu, rb[q], off);
#pragma unroll
                    for (int q = 0; q < 9; ++q) rc[q] += __shfl_xor_sync(0xffffffffu, rc[q], off);
                }
            }
            if constexpr (NORM && LEVEL == 1) {
                // linear chain rule, applied once to the sum of raw gradients
                const T t = ax * us.x + ay * us.y + az * us.z;
                ax = (ax - us.x * t) * us.ir;
                ay = (ay - us.y * t) * us.ir;
                az = (az - us.z * t) * us.ir;
            }
            if constexpr (RAW2) {
                const T ux = T(us.x), uy = T(us.y), uz = T(us.z), ir = T(us.ir);
                const T sx = ax + rb[0] * ir, sy = ay + rb[1] * ir, sz = az + rb[2] * ir;
                const T d = ux * sx + uy * sy + uz * sz;
                const T tr = rc[0] + rc[4] + rc[8];
                const T ucx = ux * rc[0] + uy * rc[3] + uz * rc[6];
                const T ucy = ux * rc[1] + uy * rc[4] + uz * rc[7];
                const T ucz = ux * rc[2] + uy * rc[5] + uz * rc[8];
                const T cux = rc[0] * ux + rc[1] * uy + rc[2] * uz;
                const T cuy = rc[3] * ux + rc[4] * uy + rc[5] * uz;
                const T cuz = rc[6] * ux + rc[7] * uy + rc[8] * uz;
                const T k = T(3) * (ucx * ux + ucy * uy + ucz * uz) - tr;
                const T irsq = ir * ir;
                ax = (sx - ux * d) * ir + (ux * k - ucx - cux) * irsq;
                ay = (sy - uy * d) * ir + (uy * k - ucy - cuy) * irsq;
                az = (sz - uz * d) * ir + (uz * k - ucz - cuz) * irsq;
            }
            if (g == 0 && valid) {
                a.xyz_grad[3 * i + 0] = ax;
                a.xyz_grad[3 * i + 1] = ay;
                a.xyz_grad[3 * i + 2] = az;
            }
        }
    }
    // shared memory must outlive the engine's reads
    if (bulk && lane == 0) bulk_wait_read_all();
}

}  // namespace sph_b200
