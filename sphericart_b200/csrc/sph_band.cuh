// "Band" kernels: any maximum degree (run-time l_max), any derivative level, and the fused
// vector-Jacobian product. Used wherever the compile-time tile kernels do not apply: l_max > 8,
// and the cases whose 32-point tile image would not fit shared memory.
//
// Two phases per point, G lanes (1, 2, 4, ... 32) sharing a point, P = 32 / G points per warp:
//
//  A. The point's whole table Q_l^m (0 <= m <= l <= l_max) is built in shared memory with the
//     reference's downward-in-m recurrence, one row (one degree) per lane, together with
//     c_m, s_m and 2(m+1)z. Rows carry four zeros after the diagonal and c, s carry two zeros
//     before m = 0, so that "term absent" cases of the derivative formulas read a zero instead of
//     branching.
//  B. The (l, m) pairs are independent once the table exists. They are dealt round-robin to the
//     G lanes (pair t goes to lane t mod G), so the load is balanced to within one pair for any
//     l_max, consecutive lanes work on consecutive m of the same degree (their table reads and
//     their writes into the output image are consecutive words: no bank conflicts), and there is
//     no per-lane recurrence state, hence no serial dependence between a lane's steps.
//
// Data movement. The P points' complete output rows are built in shared memory exactly as they
// lie in global memory ([P][ny], [P][3][ny], [P][9][ny] are contiguous spans of the outputs).
// Each span is handed to the TMA engine as a 1-D bulk store (cp.async.bulk.global.shared::cta);
// because a span may start at any 4- or 8-byte boundary, its image is placed in shared memory at
// the same offset modulo 16 bytes, the few elements before the first and after the last 16-byte
// boundary are written with plain stores, and the aligned body goes through the engine. When even
// one point's rows do not fit shared memory the degrees are cut into bands of consecutive l; the
// image then holds one band of columns at a time and is copied out with coalesced plain stores.
//
// No inter-warp, inter-CTA or inter-GPU communication; the only block-wide barrier is the one
// after the prefactor tables are staged. Replaces spherical_harmonics_kernel
// (sphericart/src/sphericart_impl.cu:207-615) and, for the VJP, the reference's
// materialise-then-reduce backward (sphericart-torch/python/sphericart/torch/register.py:90-108).
#pragma once

#include <cstdint>

#include "sph_core.cuh"
#include "sph_tile.cuh"  // bulk-store helpers

namespace sph_b200 {

constexpr int MAX_BANDS = 32;
constexpr int BAND_ROW_PAD = 4;  // zeros after the diagonal of every Q row

// Row stride of the per-point Q table: room for the padding, and even so that lanes working on
// different rows at the same distance from the diagonal hit different banks.
__host__ __device__ constexpr int band_row_stride(int l_max) { return (l_max + 1 + BAND_ROW_PAD) + ((l_max + 1 + BAND_ROW_PAD) & 1); }

// Elements of per-point state: 2 + (l_max+1) for c, the same for s, l_max+1 for 2(m+1)z, the Q table.
__host__ __device__ constexpr int band_point_state(int l_max) {
    return 2 * (l_max + 3) + (l_max + 1) + (l_max + 1) * band_row_stride(l_max);
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

template <typename T> struct BandArgs {
    const T* xyz;
    long long n;
    T* sph;
    T* dsph;
    T* ddsph;
    const T* sph_grad;  // VJP only
    T* xyz_grad;        // VJP only
    const T* tables;    // F then K, n_table(l_max) entries each
    int l_max;
    int nbands;
    int max_cols;       // widest band, columns
    int use_bulk;       // single band and TMA copy-out allowed
    short band_lo[MAX_BANDS + 1];  // band b covers degrees band_lo[b] .. band_lo[b+1] - 1
};

template <typename T, int LEVEL, bool NORM, int G, bool VJP>
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

    // shared memory carve-up: F | K | per warp: P point states, then the image regions
    T* sF = reinterpret_cast<T*>(smem_raw);
    T* sK = sF + nq;
    const int state_elems = align16_elems<T>(P * band_point_state(L));
    const int reg0 = VJP ? align16_elems<T>(P * ny) : band_region<T>(P, 1, a.max_cols);
    const int reg1 = (!VJP && LEVEL >= 1) ? band_region<T>(P, 3, a.max_cols) : 0;
    const int reg2 = (!VJP && LEVEL >= 2) ? band_region<T>(P, 9, a.max_cols) : 0;
    T* warp_base = sF + align16_elems<T>(2 * nq) + size_t(warp) * (state_elems + reg0 + reg1 + reg2);
    T* state = warp_base + pt * band_point_state(L);
    T* sc = state + 2;             // sc[-2], sc[-1] are zeros
    T* ss = sc + (L + 1) + 2;      // ss[-2], ss[-1] are zeros
    T* stz = ss + (L + 1);
    T* sQ = stz + (L + 1);         // sQ[l * RS + m]
    T* region0 = warp_base + state_elems;
    T* region1 = region0 + reg0;
    T* region2 = region1 + reg1;

    for (int e = threadIdx.x; e < 2 * nq; e += blockDim.x) sF[e] = a.tables[e];
    __syncthreads();

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

        __syncwarp();  // the previous group's phase B has finished reading the state

        // ---- phase A1: c_m, s_m, 2(m+1)z. Every lane of the group runs the (serial) recurrence,
        // lane g keeps the entries m = g mod G.
        {
            T cc = T(1), cs = T(0);
            const T twoz = z + z;
            T ctz = twoz;
            if (g == 0) {
                sc[-2] = sc[-1] = ss[-2] = ss[-1] = T(0);
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
        __syncwarp();

        // ---- phase A2: the Q table, one degree per lane, downward in m
        for (int l = g; l <= L; l += G) {
            T* row = sQ + l * RS;
            const T* Kl = sK + tri(l, 0);
            T q2 = Kl[l];  // Q_l^l is tabulated
            row[l] = q2;
#pragma unroll
            for (int j = 1; j <= BAND_ROW_PAD; ++j) row[l + j] = T(0);
            if (l >= 1) {
                T q1 = -z * q2;  // Q_l^{l-1}
                row[l - 1] = q1;
                for (int m = l - 2; m >= 0; --m) {
                    const T q0 = Kl[m] * (stz[m] * q1 + rho * q2);
                    row[m] = q0;
                    q2 = q1;
                    q1 = q0;
                }
            }
        }

        // output images: placed so that shared and global addresses agree modulo 16 bytes
        T* gsph = VJP ? nullptr : a.sph + first * ny;
        T* gd = (VJP || LEVEL < 1) ? nullptr : a.dsph + first * 3 * ny;
        T* gdd = (VJP || LEVEL < 2) ? nullptr : a.ddsph + first * 9 * ny;
        int shift0 = 0, shift1 = 0, shift2 = 0;
        if (a.use_bulk) {
            shift0 = int((reinterpret_cast<uintptr_t>(gsph) & 15u) / sizeof(T));
            if constexpr (LEVEL >= 1) shift1 = int((reinterpret_cast<uintptr_t>(gd) & 15u) / sizeof(T));
            if constexpr (LEVEL >= 2) shift2 = int((reinterpret_cast<uintptr_t>(gdd) & 15u) / sizeof(T));
        }
        T* image0 = region0 + shift0;
        T* image1 = region1 + shift1;
        T* image2 = region2 + shift2;

        [[maybe_unused]] T ax = T(0), ay = T(0), az = T(0);  // VJP accumulators
        if constexpr (VJP) {
            // the P rows of the upstream gradient are one contiguous span: coalesced load
            const T* gsrc = a.sph_grad + first * ny;
            for (int e = lane; e < nvalid * ny; e += 32) region0[e] = gsrc[e];
        } else {
            // the engine must be done reading the images of the previous group
            if (a.use_bulk && lane == 0) bulk_wait_read_all();
        }
        __syncwarp();  // table, c/s and (VJP) gradient rows visible; images free

        for (int b = 0; b < a.nbands; ++b) {
            const int l_lo = a.band_lo[b], l_hi = a.band_lo[b + 1] - 1;
            const int kb = l_lo * l_lo;                     // first column of the band
            const int cols = (l_hi + 1) * (l_hi + 1) - kb;  // columns in the band
            T* img_sph = image0 + pt * cols - kb;           // indexed by the global column k
            T* img_d = image1 + pt * 3 * cols - kb;
            T* img_dd = image2 + pt * 9 * cols - kb;
            const T* grow = region0 + pt * ny;              // VJP: this point's upstream-gradient row

            auto put = [&](int k, Column<T> v) {
                if constexpr (NORM && LEVEL >= 1) to_cartesian<T, LEVEL>(v, us);
                if constexpr (VJP) {
                    const T gk = grow[k];
                    ax += gk * v.gx;
                    ay += gk * v.gy;
                    az += gk * v.gz;
                } else {
                    img_sph[k] = v.y;
                    if constexpr (LEVEL >= 1) {
                        img_d[k] = v.gx;
                        img_d[cols + k] = v.gy;
                        img_d[2 * cols + k] = v.gz;
                    }
                    if constexpr (LEVEL >= 2) {
                        img_dd[0 * cols + k] = v.hxx;
                        img_dd[1 * cols + k] = v.hxy;
                        img_dd[2 * cols + k] = v.hxz;
                        img_dd[3 * cols + k] = v.hxy;
                        img_dd[4 * cols + k] = v.hyy;
                        img_dd[5 * cols + k] = v.hyz;
                        img_dd[6 * cols + k] = v.hxz;
                        img_dd[7 * cols + k] = v.hyz;
                        img_dd[8 * cols + k] = v.hzz;
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

            // ---- phase B: pairs (l, m), l >= 2, dealt round-robin to the group's lanes
            int l = l_lo < 2 ? 2 : l_lo;
            int m = g;
            while (l <= l_hi && m > l) {
                m -= l + 1;
                ++l;
            }
            if (!valid) l = l_hi + 1;
            while (l <= l_hi) {
                const T* Ql = sQ + l * RS;
                const T f = sF[tri(l, m)];
                const T cm = sc[m], sm = ss[m];
                const T pq = Ql[m] * f;
                Column<T> vp{}, vm{};  // +m (cosine-like) and -m (sine-like) columns
                vp.y = pq * cm;
                vm.y = pq * sm;
                if constexpr (LEVEL >= 1) {
                    const T* Ql1 = Ql - RS;
                    const T q1a = Ql1[m + 1];  // Q_{l-1}^{m+1}, zero past the diagonal
                    const T q1b = Ql1[m];      // Q_{l-1}^{m}
                    const T cm1 = sc[m - 1], sm1 = ss[m - 1];
                    const T fm = T(m);
                    const T pqm = pq * fm;
                    const T pqs = pqm * sm1, pqc = pqm * cm1;
                    const T pdq = f * q1a;
                    const T pdqx = pdq * x, pdqy = pdq * y;
                    vm.gx = pdqx * sm + pqs;
                    vp.gx = pdqx * cm + pqc;
                    vm.gy = pdqy * sm + pqc;
                    vp.gy = pdqy * cm - pqs;
                    const T flm = T(l + m);
                    const T pdz = f * flm * q1b;
                    vm.gz = pdz * sm;
                    vp.gz = pdz * cm;
                    if constexpr (LEVEL >= 2) {
                        const T* Ql2 = Ql1 - RS;
                        const T cm2 = sc[m - 2], sm2 = ss[m - 2];
                        const T A = f * q1a, D = f * q1b;
                        const T B = f * Ql2[m + 2], E = f * Ql2[m + 1], C = f * Ql2[m];
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
                    }
                }
                const int mid = l * l + l;
                put(mid + m, vp);
                if (m > 0) put(mid - m, vm);
                m += G;
                while (l <= l_hi && m > l) {
                    m -= l + 1;
                    ++l;
                }
            }

            if constexpr (!VJP) {
                if (a.use_bulk) {
                    // single band: each image is one span of the output. Elements before the first and
                    // after the last 16-byte boundary go out with plain stores, the body through TMA.
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
                } else {
                    __syncwarp();  // image complete
                    if (cols == ny) {
                        for (int e = lane; e < nvalid * ny; e += 32) gsph[e] = image0[e];
                        if constexpr (LEVEL >= 1)
                            for (int e = lane; e < nvalid * 3 * ny; e += 32) gd[e] = image1[e];
                        if constexpr (LEVEL >= 2)
                            for (int e = lane; e < nvalid * 9 * ny; e += 32) gdd[e] = image2[e];
                    } else {
                        // one band of columns: a fragment of `cols` elements per (point, component)
                        for (int r = 0; r < nvalid; ++r)
                            for (int e = lane; e < cols; e += 32) gsph[size_t(r) * ny + kb + e] = image0[r * cols + e];
                        if constexpr (LEVEL >= 1)
                            for (int r = 0; r < nvalid * 3; ++r)
                                for (int e = lane; e < cols; e += 32) gd[size_t(r) * ny + kb + e] = image1[r * cols + e];
                        if constexpr (LEVEL >= 2)
                            for (int r = 0; r < nvalid * 9; ++r)
                                for (int e = lane; e < cols; e += 32) gdd[size_t(r) * ny + kb + e] = image2[r * cols + e];
                    }
                    __syncwarp();  // image free for the next band
                }
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
    // shared memory must outlive the engine's reads
    if (!VJP && a.use_bulk && lane == 0) bulk_wait_read_all();
}

}  // namespace sph_b200
