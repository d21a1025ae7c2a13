// "Panel" kernels: forward evaluation (values, gradients, Hessians) for any maximum degree
// (run-time l_max) with a whole CTA working on a panel of tp consecutive points at a time
// (tp = 1 ... 32). They serve the cases with rows too long for the compile-time tile kernels (see
// the dispatch in sphericart_cuda.cu). The fused first-order backward of those cases is the second
// kernel of this file (sph_panel_vjp_kernel); the second-order backward stays with the band kernel.
//
// Work split. For a panel, thread t of a CTA is (point p = t mod tp, slice s = t / tp);
// S = blockDim.x / tp slices share each point. Neighbouring lanes therefore hold DIFFERENT POINTS and
// the SAME (l, m) pair, which makes the shared-memory accesses of the hot loop conflict-free by
// construction: the per-point tables are stored point-minor (element e of point q at e * TPT + q),
// the per-pair constants are read at one address by all lanes of a slice, and the image rows of
// neighbouring points are an odd number of 4-word groups apart. (The band kernel deals pairs to
// lanes instead; half of its image stores conflict where a warp straddles two degrees.)
//
//  A. Tables, for a batch of TPT points (TPT / tp panels) at once, all threads: c_m + i s_m =
//     (x + i y)^m (a slice builds a block of consecutive m from one power) and the triangular table
//     Q_l^m with the reference's downward-in-m recurrence
//     (sphericart/include/templates_core.hpp:123,155,202), rows dealt to the slices in pairs
//     (l, l_max - l) of constant total length. The recurrence is a serial chain, so batching several
//     panels' points gives this phase its parallelism. Carried in the element type (in float64 on
//     request); four steps per turn with the constants loaded ahead of the chain. Values-only calls
//     build no Q table at all: their slices carry whole rows in registers (see phase B of LEVEL 0).
//     Four zeros follow every diagonal, a block of
//     zeros stands for the rows -1 and -2, and c, s carry two zeros before m = 0, so that every "term
//     absent" case of the derivative formulas reads a zero.
//  B. Pairs, panel by panel. Slice s evaluates the pairs t = s, s + S, ... of the flattened
//     (l, m >= 0) list with the same per-pair code as the band kernel (band_eval_pair / eval_pair2 and
//     the unit-sphere chain rule) and writes both columns of each pair into the panel's image.
//  C. Copy-out. The image leaves through the TMA engine (cp.async.bulk.global.shared::cta).
//     Odd row lengths (even l_max): the panel's rows are one contiguous span of each output array;
//     its image is built at the span's own offset modulo 16 bytes and leaves as one bulk store per
//     array, the few elements before the first and after the last 16-byte boundary as plain stores.
//     Even row lengths (odd l_max: (l_max+1)^2 is a multiple of 4): every point's row is 16-byte
//     aligned by itself; rows get 16 bytes of padding where needed to keep neighbouring points an odd
//     number of 16-byte groups apart, and leave as one bulk store per point and array.
//     A CTA owns a ring of `slots` images: a panel's image is only waited for when its slot comes
//     round again, so the engine drains one image while the CTA fills the next (the launch plan has
//     never found more than one slot to pay: see make_panel_plan in sphericart_cuda.cu). What bounds
//     these kernels is the number of image bytes an SM keeps in flight towards HBM and the time its
//     CTAs spend at their barriers.
//
// No communication between CTAs or GPUs; the only waits are on this CTA's own TMA copies (bounded
// polls in the VJP kernel). Replaces spherical_harmonics_kernel
// (sphericart/src/sphericart_impl.cu:207-615).
#pragma once

#include <cstdint>

#include "sph_launch.hpp"  // layout constants shared with the host-side plan
#include "sph_band.cuh"  // per-pair evaluation, shared-memory access helpers, bulk-store helpers

namespace sph_b200 {

constexpr int PANEL_MAX_SLOTS = 4;  // images per CTA

// Elements between the image rows of neighbouring points for an array with `comps` rows of ny
// columns per point. Odd ny: the rows are packed (the image is the exact picture of global memory).
// Even ny: 16 bytes of padding where the packed distance would be an even number of 16-byte groups.
__host__ __device__ constexpr int panel_point_stride(int comps, int ny, int elem_bytes) {
    const int packed = comps * ny;
    if (ny % 2 != 0) return packed;
    const int q = 16 / elem_bytes;
    return (packed / q) % 2 == 0 ? packed + q : packed;
}

// One entry per (l, m >= 0) pair, built on the host (see make_panel_desc in sphericart_cuda.cu):
// element offsets of Q_l^m, Q_{l-1}^m and Q_{l-2}^m in the per-point table, and
// column (l*l + l + m) | m << 16 | l << 24.
struct PanelDesc {
    int off0, off1, off2, klm;
};

template <typename T> struct PanelArgs {
    const T* xyz;
    long long n;
    T* sph;
    T* dsph;
    T* ddsph;
    const T* tables;        // F then K, n_table(l_max) entries each
    const PanelDesc* desc;  // n_table(l_max) entries
    int l_max;
    int bulk;               // 1: TMA bulk copy-out, 0: plain stores
    int tp;                 // points per panel: a power of two that divides TPT
    int slots;              // images per CTA, 1 ... PANEL_MAX_SLOTS
    int tables_f64;         // 1: the table recurrences are carried in float64 whatever the element type
};

template <typename T, int TPT, int LEVEL>
__device__ __forceinline__ PairInputs<T, LEVEL> panel_load_pair(const PanelDesc d, T f, unsigned q_addr, unsigned c_addr,
                                                                unsigned s_addr) {
    constexpr unsigned E = unsigned(TPT) * unsigned(sizeof(T));  // bytes between consecutive table elements of one point
    PairInputs<T, LEVEL> in;
    const int m = (d.klm >> 16) & 0xff;
    const int l = (d.klm >> 24) & 0xff;
    in.kp = d.klm & 0xffff;
    in.m = m;
    in.f = f;
    const unsigned ac = c_addr + unsigned(m) * E;  // c_{m-2}
    const unsigned as = s_addr + unsigned(m) * E;  // s_{m-2}
    in.q = lds_at<T, 0>(q_addr + unsigned(d.off0));
    in.cm = lds_at<T, 2 * TPT>(ac);
    in.sm = lds_at<T, 2 * TPT>(as);
    if constexpr (LEVEL >= 1) {
        const unsigned a1 = q_addr + unsigned(d.off1);
        in.q1a = lds_at<T, TPT>(a1);
        in.q1b = lds_at<T, 0>(a1);
        in.cm1 = lds_at<T, TPT>(ac);
        in.sm1 = lds_at<T, TPT>(as);
        in.fm = T(m);
        in.flm = T(l + m);
    }
    if constexpr (LEVEL >= 2) {
        const unsigned a2 = q_addr + unsigned(d.off2);
        in.q2a = lds_at<T, 2 * TPT>(a2);
        in.q2b = lds_at<T, TPT>(a2);
        in.q2c = lds_at<T, 0>(a2);
        in.cm2 = lds_at<T, 0>(ac);
        in.sm2 = lds_at<T, 0>(as);
        in.fmm = T(m * (m - 1));
        in.fz = T((l + m) * (l + m - 1));
    }
    return in;
}

// Elements of one image region (one output array of one panel), with the slack the alignment shift needs.
template <typename T> __host__ __device__ constexpr int panel_region(int tp, int comps, int ny) {
    return align16_elems<T>(tp * panel_point_stride(comps, ny, int(sizeof(T)))) + 16 / int(sizeof(T));
}

// Waits until at most `pending` of this thread's committed bulk stores are still reading shared memory.
__device__ __forceinline__ void bulk_wait_read_pending(int pending) {
    switch (pending) {
        case 0: asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); break;
        default: asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory"); break;
    }
}

// Phase A for one (point, slice): the slice's block of c_m + i s_m = (x + i y)^m (one power by repeated
// squaring, then one complex product per m) and its rows of the Q table (pairs (j, L - j) of constant
// total length), with the reference's downward-in-m recurrence
// (sphericart/include/templates_core.hpp:123,155,202). A is the type the recurrences are carried in:
// double (rounded once on storing) or the element type itself.
template <typename T, typename A, int TPT, bool WITH_Q = true>
__device__ __forceinline__ void panel_build_tables(T x, T y, T z, int L, int sa, int SA, int qa, T* sc, T* ss, T* sQ,
                                                   const T* sK) {
    const A xd = A(x), yd = A(y), zd = A(z);
    const A rhod = xd * xd + yd * yd;
    const int block = (L + SA) / SA;  // ceil((L + 1) / SA)
    const int m0 = sa * block;
    if (m0 <= L) {
        A pr = A(1), pi = A(0);
        A wr = xd, wi = yd;
        for (int bits = m0; bits != 0; bits >>= 1) {
            if (bits & 1) {
                const A nr = pr * wr - pi * wi;
                pi = pr * wi + pi * wr;
                pr = nr;
            }
            const A sr = wr * wr - wi * wi;
            wi = (wr + wr) * wi;
            wr = sr;
        }
        const int m1 = (m0 + block - 1) < L ? (m0 + block - 1) : L;
        for (int m = m0; m <= m1; ++m) {
            sc[(m + 2) * TPT + qa] = T(pr);
            ss[(m + 2) * TPT + qa] = T(pi);
            const A nr = pr * xd - pi * yd;
            pi = pr * yd + pi * xd;
            pr = nr;
        }
    }
    if constexpr (!WITH_Q) return;  // values only: the rows are evaluated in registers as they are emitted
    auto build_row = [&](int l) {
        T* row = sQ + panel_row_start(l) * TPT + qa;
        const T* Kl = sK + tri(l, 0);
        A q2 = A(Kl[l]);  // Q_l^l is tabulated
        row[l * TPT] = T(q2);
        if (l >= 1) {
            A q1 = -zd * q2;  // Q_l^{l-1}
            row[(l - 1) * TPT] = T(q1);
            if constexpr (sizeof(A) == 8) {
                // float64: the coefficients K 2(m+1) z and K rho are formed off the dependent chain, which
                // is then one fused multiply-add per step instead of three operations; unrolled so that the
                // loads of K and the coefficient products of several steps are issued ahead of the chain
                // (the rounding differs from the reference's expression order by a few units of 1e-16 per step;
                // measured on l_max = 32 gradients, 1e6 points: 7.50 ms against 7.78 ms for the rolled loop)
                const A twoz = zd + zd;
                int m = l - 2;
                for (; m >= 3; m -= 4) {
                    const A k0 = A(Kl[m]), k1 = A(Kl[m - 1]), k2 = A(Kl[m - 2]), k3 = A(Kl[m - 3]);
                    const A a0 = k0 * (A(m + 1) * twoz), a1 = k1 * (A(m) * twoz), a2 = k2 * (A(m - 1) * twoz),
                            a3 = k3 * (A(m - 2) * twoz);
                    const A b0 = k0 * rhod, b1 = k1 * rhod, b2 = k2 * rhod, b3 = k3 * rhod;
                    const A r0 = a0 * q1 + b0 * q2;
                    const A r1 = a1 * r0 + b1 * q1;
                    const A r2 = a2 * r1 + b2 * r0;
                    const A r3 = a3 * r2 + b3 * r1;
                    row[m * TPT] = T(r0);
                    row[(m - 1) * TPT] = T(r1);
                    row[(m - 2) * TPT] = T(r2);
                    row[(m - 3) * TPT] = T(r3);
                    q2 = r2;
                    q1 = r3;
                }
                for (; m >= 0; --m) {
                    const A k = A(Kl[m]);
                    const A q0 = (k * (A(m + 1) * twoz)) * q1 + (k * rhod) * q2;
                    row[m * TPT] = T(q0);
                    q2 = q1;
                    q1 = q0;
                }
            } else {
                // the reference's expression order; four steps per turn so that the loads of K are issued
                // ahead of the dependent chain instead of inside it
                int m = l - 2;
                for (; m >= 3; m -= 4) {
                    const A k0 = A(Kl[m]), k1 = A(Kl[m - 1]), k2 = A(Kl[m - 2]), k3 = A(Kl[m - 3]);
                    const A r0 = k0 * (A(2 * (m + 1)) * zd * q1 + rhod * q2);
                    const A r1 = k1 * (A(2 * m) * zd * r0 + rhod * q1);
                    const A r2 = k2 * (A(2 * (m - 1)) * zd * r1 + rhod * r0);
                    const A r3 = k3 * (A(2 * (m - 2)) * zd * r2 + rhod * r1);
                    row[m * TPT] = T(r0);
                    row[(m - 1) * TPT] = T(r1);
                    row[(m - 2) * TPT] = T(r2);
                    row[(m - 3) * TPT] = T(r3);
                    q2 = r2;
                    q1 = r3;
                }
                for (; m >= 0; --m) {
                    const A q0 = A(Kl[m]) * (A(2 * (m + 1)) * zd * q1 + rhod * q2);
                    row[m * TPT] = T(q0);
                    q2 = q1;
                    q1 = q0;
                }
            }
        }
    };
    for (int j = sa; 2 * j <= L; j += SA) {
        build_row(L - j);
        if (L - j != j) build_row(j);
    }
}

// Points that share an arithmetic instruction: two in float32 (packed fma.rn.f32x2), one in float64.
template <typename T> struct PointPack;
template <> struct PointPack<float> {
    using type = F2;
    static constexpr int N = 2;
    static __device__ __forceinline__ type make(const float* v) { return f2(v[0], v[1]); }
    static __device__ __forceinline__ type all(float s) { return bc(s); }
    static __device__ __forceinline__ float get(type v, int j) { return j == 0 ? v.v.x : v.v.y; }
    static __device__ __forceinline__ type fma(type a, type b, type c) { return fma2(a, b, c); }
    static __device__ __forceinline__ type minus(type a) { return neg(a); }
};
template <> struct PointPack<double> {
    using type = double;
    static constexpr int N = 1;
    static __device__ __forceinline__ type make(const double* v) { return v[0]; }
    static __device__ __forceinline__ type all(double s) { return s; }
    static __device__ __forceinline__ double get(type v, int) { return v; }
    static __device__ __forceinline__ type fma(type a, type b, type c) { return a * b + c; }
    static __device__ __forceinline__ type minus(type a) { return -a; }
};

// 16 bytes of a point-minor table row (four float32 / two float64 neighbouring slots) as packs.
template <typename T, int NPK>
__device__ __forceinline__ void load_packs16(const T* ptr, typename PointPack<T>::type (&v)[NPK]) {
    if constexpr (sizeof(T) == 4) {
        const float4 t = *reinterpret_cast<const float4*>(ptr);
        v[0] = f2(t.x, t.y);
        v[1] = f2(t.z, t.w);
    } else {
        const double2 t = *reinterpret_cast<const double2*>(ptr);
        v[0] = t.x;
        v[1] = t.y;
    }
}

// Bytes of `count` table entries stored one pack each (the value broadcast to the pack's points), rounded
// up to 16: the kernels that carry rows in registers read their constants in this form.
__host__ __device__ constexpr size_t pack_table_bytes(int count) { return (size_t(count) * 8 + 15) / 16 * 16; }

template <typename T, int LEVEL, bool NORM, int TPT>
__global__ void __launch_bounds__(256) sph_panel_kernel(const __grid_constant__ PanelArgs<T> a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int L = a.l_max;
    const int ny = (L + 1) * (L + 1);
    const int nq = (L + 1) * (L + 2) / 2;
    const int tid = threadIdx.x;
    const int tp = a.tp;
    const int slots = a.slots;
    const bool bulk = a.bulk != 0;
    const bool packed_rows = (ny & 1) != 0;  // odd row length: the image is the exact picture of global memory
    constexpr unsigned E = unsigned(TPT) * unsigned(sizeof(T));
    constexpr int Q16 = 16 / int(sizeof(T));

    // phase A: thread = (point of the batch, table slice)
    const int qa = tid % TPT;
    const int sa = tid / TPT;
    const int SA = blockDim.x / TPT;
    // phase B: thread = (point of the panel, pair slice); values only: PPT points of the panel, lanes apart
    constexpr int PPT = LEVEL == 0 ? panel_values_ppt(int(sizeof(T))) : 1;
    const int lanes = tp / PPT;
    const int p = tid & (lanes - 1);
    const int s = tid / lanes;
    const int S = blockDim.x / lanes;
    // Table slot of phase A's point. Values only: the PPT points of a phase B thread (r = p + i lanes within
    // their panel) take the neighbouring slots PPT p + i, so that one vector load fetches them all.
    int qs = qa;
    if constexpr (LEVEL == 0) {
        const int r = qa & (tp - 1);
        qs = (qa - r) + PPT * (r & (lanes - 1)) + r / lanes;
    }

    // carve-up: F | K | descriptors | per-point state of a batch (point-minor) | slots x images
    // (values only: F then K with every entry broadcast to a pack of points, nothing else)
    using PP = PointPack<T>;
    using Pk = typename PP::type;
    T* sF = reinterpret_cast<T*>(smem_raw);
    T* sK = sF + nq;
    [[maybe_unused]] Pk* sF2 = reinterpret_cast<Pk*>(smem_raw);
    [[maybe_unused]] Pk* sK2 = sF2 + nq;
    PanelDesc* sDesc = reinterpret_cast<PanelDesc*>(sF + align16_elems<T>(2 * nq));
    T* state = LEVEL >= 1 ? reinterpret_cast<T*>(sDesc + nq) : reinterpret_cast<T*>(smem_raw + pack_table_bytes(2 * nq));
    T* sP = state;              // x, y, z, 1/r of point q at sP[c * TPT + q]
    T* sc = sP + 4 * TPT;       // c_m of point q at sc[(m + 2) * TPT + q]
    T* ss = sc + (L + 3) * TPT;  // s_m likewise
    T* sQ = ss + (L + 3) * TPT;  // element e of point q at sQ[e * TPT + q]
    T* images = state + align16_elems<T>(TPT * panel_point_state(L, LEVEL));
    const int st0 = panel_point_stride(1, ny, int(sizeof(T)));
    const int st1 = panel_point_stride(3, ny, int(sizeof(T)));
    const int st2 = panel_point_stride(9, ny, int(sizeof(T)));
    const int reg0 = panel_region<T>(tp, 1, ny);
    const int reg1 = LEVEL >= 1 ? panel_region<T>(tp, 3, ny) : 0;
    const int reg2 = LEVEL >= 2 ? panel_region<T>(tp, 9, ny) : 0;
    const int slot_elems = reg0 + reg1 + reg2;

    // ---- once per CTA: constants, and the zeros that never change
    if constexpr (LEVEL >= 1) {
        for (int e = tid; e < 2 * nq; e += blockDim.x) sF[e] = a.tables[e];
    } else {
        for (int e = tid; e < 2 * nq; e += blockDim.x) sF2[e] = PP::all(a.tables[e]);
    }
    for (int e = tid; e < 2 * TPT; e += blockDim.x) {
        sc[e] = T(0);
        ss[e] = T(0);
    }
    if constexpr (LEVEL >= 1) {
        for (int t = tid; t < nq; t += blockDim.x) {
            PanelDesc d = a.desc[t];
            d.off0 *= int(E);
            d.off1 *= int(E);
            d.off2 *= int(E);
            sDesc[t] = d;
        }
        for (int e = tid; e < PANEL_ROW_PAD * TPT; e += blockDim.x) sQ[e] = T(0);
        for (int e = tid; e < (L + 1) * PANEL_ROW_PAD * TPT; e += blockDim.x) {
            const int l = e / (PANEL_ROW_PAD * TPT);
            const int r = e % (PANEL_ROW_PAD * TPT);
            sQ[(panel_row_start(l) + l + 1) * TPT + r] = T(0);
        }
    }
    __syncthreads();

    const unsigned f_addr = static_cast<unsigned>(__cvta_generic_to_shared(sF));
    const unsigned desc_addr = static_cast<unsigned>(__cvta_generic_to_shared(sDesc));
    const unsigned ny_b = unsigned(ny) * unsigned(sizeof(T));

    const long long nbatches = (a.n + TPT - 1) / TPT;
    // rows past the end evaluate a harmless point; they are never copied out
    auto fetch_point = [&](long long batch, T& px, T& py, T& pz) {
        px = T(1);
        py = T(0);
        pz = T(0);
        const long long ip = batch * TPT + qa;
        if (batch < nbatches && ip < a.n) {
            px = a.xyz[3 * ip + 0];
            py = a.xyz[3 * ip + 1];
            pz = a.xyz[3 * ip + 2];
        }
    };
    T next_x = T(1), next_y = T(0), next_z = T(0);
    if (sa < SA) fetch_point(blockIdx.x, next_x, next_y, next_z);
    int slot = 0;
    int committed = 0;  // thread 0 only: bulk-store groups committed so far
    for (long long batch = blockIdx.x; batch < nbatches; batch += gridDim.x) {
        const long long batch_first = batch * TPT;

        // ---- phase A
        if (sa < SA) {
            T x = next_x, y = next_y, z = next_z, ir = T(1);
            // the next batch's point is fetched now and used an entire batch later: under a saturated
            // write stream a read from global memory takes microseconds
            fetch_point(batch + gridDim.x, next_x, next_y, next_z);
            if constexpr (NORM) {
                // IEEE square root and division, as on the CPU (sphericart/include/templates.hpp:392-400)
                ir = T(1) / sqrt(x * x + y * y + z * z);
                x *= ir;
                y *= ir;
                z *= ir;
            }
            if (sa == 0) {
                // phase B reads the point from here
                sP[0 * TPT + qs] = x;
                sP[1 * TPT + qs] = y;
                sP[2 * TPT + qs] = z;
                sP[3 * TPT + qs] = ir;
            }
            if (a.tables_f64 != 0) {
                panel_build_tables<T, double, TPT, LEVEL >= 1>(x, y, z, L, sa, SA, qs, sc, ss, sQ, sK);
            } else {
                panel_build_tables<T, T, TPT, LEVEL >= 1>(x, y, z, L, sa, SA, qs, sc, ss, sQ, sK);
            }
        }

        // ---- the batch's panels, one image each
        for (int sub = 0; sub < TPT; sub += tp) {
            const long long first = batch_first + sub;
            if (first >= a.n) break;  // the same for every thread
            const int nvalid = (a.n - first) < tp ? int(a.n - first) : tp;

            // where this panel's rows go; with packed rows the images are placed so that shared and
            // global addresses agree modulo 16 bytes
            T* gsph = a.sph + first * ny;
            T* gd = LEVEL >= 1 ? a.dsph + first * 3 * ny : nullptr;
            T* gdd = LEVEL >= 2 ? a.ddsph + first * 9 * ny : nullptr;
            int shift0 = 0, shift1 = 0, shift2 = 0;
            if (bulk && packed_rows) {
                shift0 = int((reinterpret_cast<uintptr_t>(gsph) & 15u) / sizeof(T));
                if constexpr (LEVEL >= 1) shift1 = int((reinterpret_cast<uintptr_t>(gd) & 15u) / sizeof(T));
                if constexpr (LEVEL >= 2) shift2 = int((reinterpret_cast<uintptr_t>(gdd) & 15u) / sizeof(T));
            }
            T* region0 = images + slot * slot_elems;
            T* image0 = region0 + shift0;
            T* image1 = region0 + reg0 + shift1;
            T* image2 = region0 + reg0 + reg1 + shift2;

            // the engine must be done reading this slot's previous image before phase B overwrites it:
            // of the groups committed so far all but the last slots - 1 must have been read
            if (tid == 0 && committed >= slots) bulk_wait_read_pending(slots - 1);
            __syncthreads();  // tables complete, slot free

            if (s < S) {
                const T x = sP[0 * TPT + sub + p], y = sP[1 * TPT + sub + p], z = sP[2 * TPT + sub + p];
                [[maybe_unused]] const T ir = sP[3 * TPT + sub + p];
                const UnitSphere<T> us{x, y, z, ir, ir * ir};
                const T x2 = x * x, y2 = y * y, xy = x * y;
                const unsigned q_addr = static_cast<unsigned>(__cvta_generic_to_shared(sQ + sub + p));
                const unsigned c_addr = static_cast<unsigned>(__cvta_generic_to_shared(sc + sub + p));
                const unsigned s_addr = static_cast<unsigned>(__cvta_generic_to_shared(ss + sub + p));
                const unsigned img0_addr = static_cast<unsigned>(__cvta_generic_to_shared(image0 + p * st0));
                [[maybe_unused]] const unsigned img1_addr = static_cast<unsigned>(__cvta_generic_to_shared(image1 + p * st1));
                [[maybe_unused]] const unsigned img2_addr = static_cast<unsigned>(__cvta_generic_to_shared(image2 + p * st2));

                auto store_column = [&](int k, const Column<T>& v) {
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
                };
                // float32 with derivatives: the pair's two columns go through the packed two-wide path
                constexpr bool PACKED = sizeof(T) == 4 && LEVEL >= 1;
                constexpr bool CHAIN = NORM && LEVEL >= 1;
                [[maybe_unused]] UnitSphere2 us2{};
                if constexpr (PACKED && CHAIN) {
                    UnitSphere<float> usf{float(us.x), float(us.y), float(us.z), float(us.ir), float(us.irsq)};
                    us2 = make_unit_sphere2<LEVEL>(usf);
                }
                auto finish_pair = [&](const PairInputs<T, LEVEL>& in) {
                    Column<T> vp{}, vm{};
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
                        eval_pair2<LEVEL>(ps, f2(float(in.cm), float(in.sm)), f2(float(in.cm1), float(in.sm1)), cs2,
                                          float(x), float(y), float(x2), float(y2), float(xy), v);
                        if constexpr (CHAIN) to_cartesian2<LEVEL>(v, us2);
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
                    } else {
                        band_eval_pair<T, LEVEL>(in, x, y, x2, y2, xy, vp, vm);
                        if constexpr (CHAIN) {
                            to_cartesian<T, LEVEL>(vp, us);
                            to_cartesian<T, LEVEL>(vm, us);
                        }
                    }
                    store_column(in.kp, vp);
                    if (in.m > 0) store_column(in.kp - 2 * in.m, vm);
                };

                // ---- phase B: pairs t = s, s + S, ...
                auto load = [&](int t) {
                    PanelDesc d;
                    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(d.off0), "=r"(d.off1), "=r"(d.off2), "=r"(d.klm)
                                 : "r"(desc_addr + unsigned(t) * 16u));
                    const T f = lds_at<T, 0>(f_addr + unsigned(t) * unsigned(sizeof(T)));
                    return panel_load_pair<T, TPT, LEVEL>(d, f, q_addr, c_addr, s_addr);
                };
                if constexpr (LEVEL >= 1) {
                    // two pairs in flight per thread (one for float64 Hessians: two pairs' inputs and thirteen outputs per
                    // column cost registers that are better spent on a second CTA per SM)
                    constexpr bool ONE_IN_FLIGHT = sizeof(T) == 8 && LEVEL == 2;
                    int t = s;
                    for (; !ONE_IN_FLIGHT && t + S < nq; t += 2 * S) {
                        const PairInputs<T, LEVEL> in0 = load(t);
                        const PairInputs<T, LEVEL> in1 = load(t + S);
                        finish_pair(in0);
                        finish_pair(in1);
                    }
                    for (; t < nq; t += S) finish_pair(load(t));
                } else {
                    // Values only: no Q table. A slice takes whole rows, in pairs (j, l_max - j) of constant
                    // total length, carries each row's recurrence in registers (the reference's own scheme,
                    // sphericart/include/templates_core.hpp:123,155,202, in the element type) and writes the
                    // two values of every m as it goes: Y_{l,+m} = F Q_l^m c_m, Y_{l,-m} = F Q_l^m s_m.
                    // A thread does this for PPT neighbouring points of the panel at once: their c_m (s_m) sit
                    // side by side in the point-minor tables and arrive as one 16-byte load, the row's
                    // constants are read once for all of them, and in float32 two points share each
                    // arithmetic instruction (packed fma.rn.f32x2).
                    // (thread p's points are p, p + lanes, ... of the panel: rows `lanes` apart in the image, which
                    // keeps a warp's image writes conflict-free; their table entries sit in neighbouring slots)
                    const int q0i = sub + PPT * p;     // first of this thread's table slots within the batch
                    const T* cp = sc + 2 * TPT + q0i;  // c_m of point i at cp[m * TPT + i]
                    const T* sp = ss + 2 * TPT + q0i;
                    T* out = image0 + p * st0;         // row of point i at out + i * pst
                    const int pst = lanes * st0;
                    constexpr int NPK = PPT / PP::N;
                    Pk nzz[NPK], rho[NPK], tzz[NPK];  // -z, x^2 + y^2, 2z
                    {
                        Pk px[NPK], py[NPK], pz[NPK];
                        load_packs16<T, NPK>(sP + 0 * TPT + q0i, px);
                        load_packs16<T, NPK>(sP + 1 * TPT + q0i, py);
                        load_packs16<T, NPK>(sP + 2 * TPT + q0i, pz);
#pragma unroll
                        for (int k = 0; k < NPK; ++k) {
                            rho[k] = PP::fma(px[k], px[k], py[k] * py[k]);
                            nzz[k] = PP::minus(pz[k]);
                            tzz[k] = pz[k] + pz[k];
                        }
                    }
                    // writes F Q (c_m, s_m) of every point for one m; q holds Q_l^m per point, cv / sv the points' c_m, s_m;
                    // pp / pm point at the columns +m / -m of each point's row
                    auto emit = [&](T* const (&pp)[PPT], T* const (&pm)[PPT], int off, const Pk (&cv)[NPK], const Pk (&sv)[NPK], Pk fm,
                                    const Pk (&q)[NPK], bool minus_too) {
#pragma unroll
                        for (int k = 0; k < NPK; ++k) {
                            const Pk pq = q[k] * fm;
                            const Pk yp = pq * cv[k];
                            const Pk ym = pq * sv[k];
#pragma unroll
                            for (int j = 0; j < PP::N; ++j) {
                                pp[k * PP::N + j][-off] = PP::get(yp, j);
                                if (minus_too) pm[k * PP::N + j][off] = PP::get(ym, j);
                            }
                        }
                    };
                    auto row_values = [&](int l) {
                        const Pk* Kl = sK2 + tri(l, 0);
                        const Pk* Fl = sF2 + tri(l, 0);
                        T* pp[PPT];  // column +m of each point's row
                        T* pm[PPT];  // column -m
#pragma unroll
                        for (int i = 0; i < PPT; ++i) {
                            pp[i] = out + i * pst + l * l + 2 * l;
                            pm[i] = out + i * pst + l * l;
                        }
                        const T* cpm = cp + l * TPT;
                        const T* spm = sp + l * TPT;
                        // the two newest values of the recurrence alternate between qa and qb
                        Pk qa[NPK], qb[NPK], c0[NPK], s0[NPK], c1[NPK], s1[NPK];
                        load_packs16<T, NPK>(cpm, c0);
                        load_packs16<T, NPK>(spm, s0);
                        load_packs16<T, NPK>(cpm - TPT, c1);  // (l = 0: the zero rows)
                        load_packs16<T, NPK>(spm - TPT, s1);
#pragma unroll
                        for (int k = 0; k < NPK; ++k) qa[k] = Kl[l];  // Q_l^l is tabulated
                        emit(pp, pm, 0, c0, s0, Fl[l], qa, l > 0);
                        if (l == 0) return;
#pragma unroll
                        for (int k = 0; k < NPK; ++k) qb[k] = nzz[k] * qa[k];  // Q_l^{l-1}
                        emit(pp, pm, 1, c1, s1, Fl[l - 1], qb, l > 1);
                        // 2 (m + 1) z as one product per step (a running difference would drift: float32 has no
                        // error budget to spare at these degrees)
                        T mp1 = T(l - 1);
                        int m = l - 2;
#pragma unroll
                        for (int i = 0; i < PPT; ++i) {
                            pp[i] -= 2;
                            pm[i] += 2;
                        }
                        cpm -= 2 * TPT;
                        spm -= 2 * TPT;
                        // Q_l^m = K (2 (m+1) z Q_l^{m+1} + rho Q_l^{m+2}), two steps per turn: the new value takes the
                        // place of the older of the two it was made from, so nothing is moved between registers, and
                        // both steps' table entries are requested before the first step's stores
                        for (; m >= 2; m -= 2) {
                            load_packs16<T, NPK>(cpm, c0);
                            load_packs16<T, NPK>(spm, s0);
                            load_packs16<T, NPK>(cpm - TPT, c1);
                            load_packs16<T, NPK>(spm - TPT, s1);
                            const Pk k0 = Kl[m], k1 = Kl[m - 1], f0 = Fl[m], f1 = Fl[m - 1];
                            const Pk t0 = PP::all(mp1), t1 = PP::all(mp1 - T(1));
                            mp1 -= T(2);
#pragma unroll
                            for (int k = 0; k < NPK; ++k) qa[k] = k0 * PP::fma(rho[k], qa[k], t0 * tzz[k] * qb[k]);
                            emit(pp, pm, 0, c0, s0, f0, qa, true);
#pragma unroll
                            for (int k = 0; k < NPK; ++k) qb[k] = k1 * PP::fma(rho[k], qb[k], t1 * tzz[k] * qa[k]);
                            emit(pp, pm, 1, c1, s1, f1, qb, true);
#pragma unroll
                            for (int i = 0; i < PPT; ++i) {
                                pp[i] -= 2;
                                pm[i] += 2;
                            }
                            cpm -= 2 * TPT;
                            spm -= 2 * TPT;
                        }
                        if (m >= 0) {
                            load_packs16<T, NPK>(cpm, c0);
                            load_packs16<T, NPK>(spm, s0);
                            load_packs16<T, NPK>(cpm - TPT, c1);  // (m = 0: the zero rows, not used)
                            load_packs16<T, NPK>(spm - TPT, s1);
                            const Pk t0 = PP::all(mp1), t1 = PP::all(mp1 - T(1));
#pragma unroll
                            for (int k = 0; k < NPK; ++k) qa[k] = Kl[m] * PP::fma(rho[k], qa[k], t0 * tzz[k] * qb[k]);
                            emit(pp, pm, 0, c0, s0, Fl[m], qa, m > 0);
                            if (m == 1) {
#pragma unroll
                                for (int k = 0; k < NPK; ++k) qb[k] = Kl[0] * PP::fma(rho[k], qb[k], t1 * tzz[k] * qa[k]);
                                emit(pp, pm, 1, c1, s1, Fl[0], qb, false);
                            }
                        }
                    };
                    for (int j = s; 2 * j <= L; j += S) {
                        row_values(L - j);
                        if (L - j != j) row_values(j);
                    }
                }
            }

            // ---- copy-out
            if (bulk) {
                fence_proxy_async_smem();  // this thread's image writes, visible to the TMA engine
                __syncthreads();           // image complete; phase B has finished reading the tables
                if (packed_rows) {
                    if (tid < 32) {
                        auto copy_out = [&](T* gdst, const T* img, int shift, int count) {
                            const int head = shift == 0 ? 0 : (Q16 - shift < count ? Q16 - shift : count);
                            const int body = (count - head) / Q16 * Q16;
                            const int tail = count - head - body;
                            if (tid < head) gdst[tid] = img[tid];
                            if (tid >= 8 && tid - 8 < tail) gdst[head + body + tid - 8] = img[head + body + tid - 8];
                            if (tid == 0 && body > 0)
                                bulk_store_smem_to_global(gdst + head, img + head, unsigned(body) * unsigned(sizeof(T)));
                        };
                        copy_out(gsph, image0, shift0, nvalid * ny);
                        if constexpr (LEVEL >= 1) copy_out(gd, image1, shift1, nvalid * 3 * ny);
                        if constexpr (LEVEL >= 2) copy_out(gdd, image2, shift2, nvalid * 9 * ny);
                    }
                } else if (tid == 0) {
                    // every point's row is 16-byte aligned on both sides: one store per point and array (issued by one
                    // thread: spreading the issue over a warp's lanes measured 1 - 3 % slower, 10 % for values only)
                    for (int r = 0; r < nvalid; ++r) {
                        bulk_store_smem_to_global(gsph + size_t(r) * ny, image0 + r * st0, ny_b);
                        if constexpr (LEVEL >= 1) bulk_store_smem_to_global(gd + size_t(r) * 3 * ny, image1 + r * st1, 3 * ny_b);
                        if constexpr (LEVEL >= 2) bulk_store_smem_to_global(gdd + size_t(r) * 9 * ny, image2 + r * st2, 9 * ny_b);
                    }
                }
                if (tid == 0) {
                    bulk_commit();
                    ++committed;
                }
            } else {
                __syncthreads();
                for (int r = 0; r < nvalid; ++r) {
                    for (int e = tid; e < ny; e += blockDim.x) gsph[size_t(r) * ny + e] = image0[r * st0 + e];
                    if constexpr (LEVEL >= 1)
                        for (int e = tid; e < 3 * ny; e += blockDim.x) gd[size_t(r) * 3 * ny + e] = image1[r * st1 + e];
                    if constexpr (LEVEL >= 2)
                        for (int e = tid; e < 9 * ny; e += blockDim.x) gdd[size_t(r) * 9 * ny + e] = image2[r * st2 + e];
                }
            }
            slot = slot + 1 == slots ? 0 : slot + 1;
        }
        // (the next batch's tables may be written at once: every thread has passed the barrier that
        // follows phase B of this batch's last panel)
    }
    // shared memory must outlive the engine's reads
    if (tid == 0 && committed > 0) bulk_wait_read_all();
}

// ---------------------------------------------------------------------------------------------
// Fused vector-Jacobian product with the maximum degree known only at run time:
//   xyz_grad[i][a] = sum_k sph_grad[i][k] dY[i][a][k],
// dY never in memory. A CTA takes batches of TPT points. Phase A builds the batch's c_m, s_m (all
// threads, point-minor) - no Q table: as in the values-only forward path a slice owns whole rows, in
// pairs (j, l_max - j) of constant total length, and carries the recurrences in registers - here two
// of them, row l and row l-1, because the derivatives of row l need Q_{l-1}^{m+1} and Q_{l-1}^m. The
// gradient columns are never formed (see eval_point_vjp in sph_core.cuh for the algebra): per (l, m)
// the thread reads the two upstream entries g+, g- and accumulates four sums. A thread does this for
// PPT points at once (their c_m, s_m arrive as one 16-byte load; float32: two points per packed
// instruction). The partial sums of a point's slices meet in shared memory; the linear unit-sphere
// chain rule is applied once to their total.
// The batch's TPT rows of sph_grad are one contiguous span of the input: the TMA engine fetches it
// (one bulk load when the rows are of odd length and packed, one per row into padded rows
// otherwise), completion on an mbarrier that every thread waits for with a bounded number of polls
// (on give-up the CTA records it in g_tile_wait_gave_up and returns: nothing else of it is in
// flight); the next batch's rows are requested as soon as phase B is over, so the load runs under the
// reduction and the next table phase. Replaces the reference's backward (a gradients launch that
// materialises dsph, a product and a reduction: sphericart-torch/python/sphericart/torch/register.py:90-108).
template <typename T> struct PanelVjpArgs {
    const T* xyz;
    const T* sph_grad;
    long long n;
    T* xyz_grad;
    const T* tables;  // F then K
    int l_max;
    int bulk;         // 1: sph_grad is 16-byte aligned, rows may come through the TMA engine
};

// Dynamic shared memory of sph_panel_vjp_kernel, in bytes: four tables of constants (F, K, F m, F (l + m), every
// entry broadcast to a pack of points), the batch's points and c/s, its upstream rows, the partial sums, the mbarrier.
template <typename T> __host__ __device__ constexpr size_t panel_vjp_smem_bytes(int l_max, int tpt, int threads) {
    const int nq = n_table(l_max);
    const int ny = n_columns(l_max);
    return pack_table_bytes(4 * nq) +
           size_t(align16_elems<T>(tpt * panel_point_state(l_max, 0)) + align16_elems<T>(tpt * panel_point_stride(1, ny, int(sizeof(T)))) +
                  align16_elems<T>(3 * threads * (16 / int(sizeof(T))))) * sizeof(T) + 16;
}

template <typename T, bool NORM, int TPT>
__global__ void __launch_bounds__(256) sph_panel_vjp_kernel(const __grid_constant__ PanelVjpArgs<T> a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using PP = PointPack<T>;
    using Pk = typename PP::type;
    constexpr int PPT = panel_values_ppt(int(sizeof(T)));  // points per thread in phase B
    constexpr int NPK = PPT / PP::N;                        // packs per thread
    constexpr int LANES = TPT / PPT;                        // threads side by side in a slice
    static_assert(TPT >= PPT, "a batch holds at least one thread's points");
    const int L = a.l_max;
    const int ny = (L + 1) * (L + 1);
    const int nq = (L + 1) * (L + 2) / 2;
    const int tid = threadIdx.x;
    // phase A: thread = (point of the batch, table slice)
    const int qa = tid % TPT;
    const int sa = tid / TPT;
    const int SA = blockDim.x / TPT;
    // phase B: thread = (PPT points of the batch, LANES apart; slice of rows)
    const int p = tid % LANES;
    const int s = tid / LANES;
    const int S = blockDim.x / LANES;
    // table slot of phase A's point: the PPT points of a phase B thread (r = p + i LANES) take the
    // neighbouring slots PPT p + i, so that one vector load fetches them all
    const int qs = PPT * (qa % LANES) + qa / LANES;

    // carve-up: F | K | F m | F (l + m) (packs) | per-point state of a batch (point-minor) | the batch's rows of sph_grad | partial sums | mbarrier
    Pk* sF2 = reinterpret_cast<Pk*>(smem_raw);
    Pk* sK2 = sF2 + nq;
    Pk* sFM2 = sK2 + nq;
    Pk* sFLM2 = sFM2 + nq;
    T* state = reinterpret_cast<T*>(smem_raw + pack_table_bytes(4 * nq));
    T* sP = state;               // x, y, z, 1/r of slot q at sP[c * TPT + q]
    T* sc = sP + 4 * TPT;        // c_m of slot q at sc[(m + 2) * TPT + q]
    T* ss = sc + (L + 3) * TPT;  // s_m likewise
    T* rows = state + align16_elems<T>(TPT * panel_point_state(L, 0));
    const int gst = panel_point_stride(1, ny, int(sizeof(T)));  // elements between neighbouring points' rows
    T* red = rows + align16_elems<T>(TPT * gst);                // partial sums [3][S][TPT]
    unsigned long long* bar =
        reinterpret_cast<unsigned long long*>(red + align16_elems<T>(3 * int(blockDim.x) * (16 / int(sizeof(T)))));

    for (int e = tid; e < nq; e += blockDim.x) {
        int l = int((sqrtf(8.0f * float(e) + 1.0f) - 1.0f) * 0.5f);
        while (tri(l + 1, 0) <= e) ++l;
        while (tri(l, 0) > e) --l;
        const int m = e - tri(l, 0);
        const T f = a.tables[e];
        sF2[e] = PP::all(f);
        sK2[e] = PP::all(a.tables[nq + e]);
        sFM2[e] = PP::all(f * T(m));
        sFLM2[e] = PP::all(f * T(l + m));
    }
    for (int e = tid; e < 2 * TPT; e += blockDim.x) {
        sc[e] = T(0);
        ss[e] = T(0);
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init_fence();
    }
    __syncthreads();

    const long long nbatches = (a.n + TPT - 1) / TPT;
    const bool packed_rows = (ny & 1) != 0;
    const unsigned row_bytes = unsigned(ny) * unsigned(sizeof(T));
    // a batch can come through the engine when it is full: its span (packed rows) or each of its rows
    // (rows of even length are multiples of 16 bytes) then starts and ends on 16-byte boundaries
    auto engine_batch = [&](long long batch) { return a.bulk != 0 && (batch + 1) * TPT <= a.n; };
    auto issue = [&](long long batch) {  // thread 0 only
        if (batch < nbatches && engine_batch(batch)) {
            const T* src = a.sph_grad + batch * TPT * ny;
            mbar_expect_tx(bar, unsigned(TPT) * row_bytes);
            if (packed_rows) {
                bulk_load_global_to_smem(rows, src, unsigned(TPT) * row_bytes, bar);
            } else {
                for (int r = 0; r < TPT; ++r) bulk_load_global_to_smem(rows + r * gst, src + size_t(r) * ny, row_bytes, bar);
            }
        }
    };
    auto fetch_point = [&](long long batch, T& px, T& py, T& pz) {
        px = T(1);
        py = T(0);
        pz = T(0);
        const long long ip = batch * TPT + qa;
        if (batch < nbatches && ip < a.n) {
            px = a.xyz[3 * ip + 0];
            py = a.xyz[3 * ip + 1];
            pz = a.xyz[3 * ip + 2];
        }
    };
    if (tid == 0) issue(blockIdx.x);
    T next_x = T(1), next_y = T(0), next_z = T(0);
    if (sa < SA) fetch_point(blockIdx.x, next_x, next_y, next_z);
    unsigned phase = 0u;
    for (long long batch = blockIdx.x; batch < nbatches; batch += gridDim.x) {
        // ---- phase A: the batch's points and their c_m, s_m
        if (sa < SA) {
            T x = next_x, y = next_y, z = next_z, ir = T(1);
            fetch_point(batch + gridDim.x, next_x, next_y, next_z);
            if constexpr (NORM) {
                // IEEE square root and division, as on the CPU (sphericart/include/templates.hpp:392-400)
                ir = T(1) / sqrt(x * x + y * y + z * z);
                x *= ir;
                y *= ir;
                z *= ir;
            }
            if (sa == 0) {
                sP[0 * TPT + qs] = x;
                sP[1 * TPT + qs] = y;
                sP[2 * TPT + qs] = z;
                sP[3 * TPT + qs] = ir;
            }
            panel_build_tables<T, T, TPT, false>(x, y, z, L, sa, SA, qs, sc, ss, nullptr, nullptr);
        }
        // ---- the batch's rows of sph_grad
        if (engine_batch(batch)) {
            if (!mbar_wait_bounded(bar, phase)) {
                g_tile_wait_gave_up = 1;
                return;  // nothing else of this CTA is in flight
            }
            phase ^= 1u;
        } else {
            // ragged last batch, or an input that is not 16-byte aligned: coalesced loads by all threads
            const long long first = batch * TPT;
            const int nvalid = (a.n - first) < TPT ? int(a.n - first) : TPT;
            const T* src = a.sph_grad + first * ny;
            for (int r = 0; r < TPT; ++r) {
                for (int e = tid; e < ny; e += blockDim.x) rows[r * gst + e] = r < nvalid ? src[size_t(r) * ny + e] : T(0);
            }
        }
        __syncthreads();  // c, s, the points and the rows are complete

        // ---- phase B
        Pk ax[NPK], ay[NPK], az[NPK], aw[NPK];  // aw: the sum that x and y multiply
#pragma unroll
        for (int k = 0; k < NPK; ++k) ax[k] = ay[k] = az[k] = aw[k] = PP::all(T(0));
        if (s < S) {
            const int q0i = PPT * p;             // first of this thread's table slots
            const T* cp = sc + 2 * TPT + q0i;    // c_m of the thread's points at cp[m * TPT ...]
            const T* sp = ss + 2 * TPT + q0i;
            const T* grow = rows + p * gst;      // row of point i at grow + i * LANES * gst
            Pk nzz[NPK], rho[NPK], tzz[NPK];  // -z, x^2 + y^2, 2z
            {
                Pk px[NPK], py[NPK], pz[NPK];
                load_packs16<T, NPK>(sP + 0 * TPT + q0i, px);
                load_packs16<T, NPK>(sP + 1 * TPT + q0i, py);
                load_packs16<T, NPK>(sP + 2 * TPT + q0i, pz);
#pragma unroll
                for (int k = 0; k < NPK; ++k) {
                    rho[k] = PP::fma(px[k], px[k], py[k] * py[k]);
                    nzz[k] = PP::minus(pz[k]);
                    tzz[k] = pz[k] + pz[k];
                }
            }
            // One (l, m). q = Q_l^m, bn = Q_{l-1}^{m+1}, bcur = Q_{l-1}^m (zeros where absent); cm, sm hold c_m, s_m;
            // c_{m-1}, s_{m-1} are loaded into cm1, sm1 (c_{-1} = s_{-1} = 0 from the tables' zero rows); gp / gm point
            // at the upstream entries of the columns +m / -m of each point, `off` columns further in.
            auto contract = [&](int idx, int off, const T* cpm1, const T* spm1, const T* const (&gp)[PPT],
                                const T* const (&gm)[PPT], const Pk (&q)[NPK], const Pk (&bn)[NPK], const Pk (&bcur)[NPK],
                                const Pk (&cm)[NPK], const Pk (&sm)[NPK], Pk (&cm1)[NPK], Pk (&sm1)[NPK]) {
                load_packs16<T, NPK>(cpm1, cm1);
                load_packs16<T, NPK>(spm1, sm1);
                const Pk f1 = sF2[idx], fm = sFM2[idx], flm = sFLM2[idx];
#pragma unroll
                for (int k = 0; k < NPK; ++k) {
                    T vp[PP::N], vm[PP::N];
#pragma unroll
                    for (int j = 0; j < PP::N; ++j) {
                        vp[j] = gp[k * PP::N + j][-off];
                        vm[j] = gm[k * PP::N + j][off];
                    }
                    const Pk g1 = PP::make(vp), g2 = PP::make(vm);
                    const Pk w = PP::fma(g1, cm[k], g2 * sm[k]);
                    const Pk u = PP::fma(g1, cm1[k], g2 * sm1[k]);
                    const Pk v = PP::fma(PP::minus(g1), sm1[k], g2 * cm1[k]);
                    const Pk pqm = q[k] * fm;
                    ax[k] = PP::fma(pqm, u, ax[k]);
                    ay[k] = PP::fma(pqm, v, ay[k]);
                    aw[k] = PP::fma(f1 * bn[k], w, aw[k]);
                    az[k] = PP::fma(flm * bcur[k], w, az[k]);
                }
            };
            auto row_vjp = [&](int l) {  // l >= 1 (the row l = 0 has no derivative)
                const int t0 = tri(l, 0);
                const Pk* Kl = sK2 + t0;
                const Pk* Kb = sK2 + tri(l - 1, 0);
                const T* gp[PPT];  // upstream entry of column +m of each point
                const T* gm[PPT];  // of column -m
#pragma unroll
                for (int i = 0; i < PPT; ++i) {
                    gp[i] = grow + (i * LANES) * gst + l * l + 2 * l;
                    gm[i] = grow + (i * LANES) * gst + l * l;
                }
                const T* cpm = cp + l * TPT;  // c_m of the current step
                const T* spm = sp + l * TPT;
                // the two newest values of each recurrence, and c/s of two neighbouring m, alternate between the
                // a and b registers, so nothing is moved between steps
                Pk qa[NPK], qb[NPK], ba[NPK], bb[NPK], ca[NPK], sa2[NPK], cb[NPK], sb[NPK], zero[NPK];
                load_packs16<T, NPK>(cpm, cb);
                load_packs16<T, NPK>(spm, sb);
#pragma unroll
                for (int k = 0; k < NPK; ++k) {
                    zero[k] = PP::all(T(0));
                    qa[k] = Kl[l];  // Q_l^l is tabulated
                }
                // m = l
                contract(t0 + l, 0, cpm - TPT, spm - TPT, gp, gm, qa, zero, zero, cb, sb, ca, sa2);
                // m = l - 1: Q_l^{l-1} = -z Q_l^l, Q_{l-1}^{l-1} tabulated
#pragma unroll
                for (int k = 0; k < NPK; ++k) {
                    qb[k] = nzz[k] * qa[k];
                    bb[k] = Kb[l - 1];
                }
                contract(t0 + l - 1, 1, cpm - 2 * TPT, spm - 2 * TPT, gp, gm, qb, zero, bb, ca, sa2, cb, sb);
                if (l < 2) return;
                // 2 (m + 1) z as one product per step (a running difference would drift)
                T mp1 = T(l - 1);
                Pk tz[NPK];
#pragma unroll
                for (int k = 0; k < NPK; ++k) {
                    tz[k] = PP::all(mp1) * tzz[k];
                    // m = l - 2: the general step for row l, Q_{l-1}^{l-2} = -z Q_{l-1}^{l-1}
                    qa[k] = Kl[l - 2] * PP::fma(rho[k], qa[k], tz[k] * qb[k]);
                    ba[k] = nzz[k] * bb[k];
                    tz[k] = PP::all(mp1 - T(1)) * tzz[k];
                }
                mp1 -= T(1);
                contract(t0 + l - 2, 2, cpm - 3 * TPT, spm - 3 * TPT, gp, gm, qa, bb, ba, cb, sb, ca, sa2);
                int m = l - 3;
#pragma unroll
                for (int i = 0; i < PPT; ++i) {
                    gp[i] -= 3;
                    gm[i] += 3;
                }
                cpm -= 3 * TPT;
                spm -= 3 * TPT;
                for (; m >= 1; m -= 2) {
#pragma unroll
                    for (int k = 0; k < NPK; ++k) {
                        qb[k] = Kl[m] * PP::fma(rho[k], qb[k], tz[k] * qa[k]);
                        bb[k] = Kb[m] * PP::fma(rho[k], bb[k], tz[k] * ba[k]);
                        tz[k] = PP::all(mp1 - T(1)) * tzz[k];
                    }
                    contract(t0 + m, 0, cpm - TPT, spm - TPT, gp, gm, qb, ba, bb, ca, sa2, cb, sb);
#pragma unroll
                    for (int k = 0; k < NPK; ++k) {
                        qa[k] = Kl[m - 1] * PP::fma(rho[k], qa[k], tz[k] * qb[k]);
                        ba[k] = Kb[m - 1] * PP::fma(rho[k], ba[k], tz[k] * bb[k]);
                        tz[k] = PP::all(mp1 - T(2)) * tzz[k];
                    }
                    mp1 -= T(2);
                    contract(t0 + m - 1, 1, cpm - 2 * TPT, spm - 2 * TPT, gp, gm, qa, bb, ba, cb, sb, ca, sa2);
#pragma unroll
                    for (int i = 0; i < PPT; ++i) {
                        gp[i] -= 2;
                        gm[i] += 2;
                    }
                    cpm -= 2 * TPT;
                    spm -= 2 * TPT;
                }
                if (m == 0) {
#pragma unroll
                    for (int k = 0; k < NPK; ++k) {
                        qb[k] = Kl[0] * PP::fma(rho[k], qb[k], tz[k] * qa[k]);
                        bb[k] = Kb[0] * PP::fma(rho[k], bb[k], tz[k] * ba[k]);
                    }
                    contract(t0, 0, cpm - TPT, spm - TPT, gp, gm, qb, ba, bb, ca, sa2, cb, sb);
                }
            };
            for (int j = s; 2 * j <= L; j += S) {
                if (L - j >= 1) row_vjp(L - j);
                if (L - j != j && j >= 1) row_vjp(j);
            }
            // x and y multiply the sums of their second terms once
            {
                Pk px[NPK], py[NPK];
                load_packs16<T, NPK>(sP + 0 * TPT + q0i, px);
                load_packs16<T, NPK>(sP + 1 * TPT + q0i, py);
#pragma unroll
                for (int k = 0; k < NPK; ++k) {
                    ax[k] = PP::fma(px[k], aw[k], ax[k]);
                    ay[k] = PP::fma(py[k], aw[k], ay[k]);
                }
            }
            // partial sums of point r = p + i LANES, slice s: red[(c * S + s) * TPT + r]
#pragma unroll
            for (int i = 0; i < PPT; ++i) {
                const int r = p + i * LANES;
                red[(0 * S + s) * TPT + r] = PP::get(ax[i / PP::N], i % PP::N);
                red[(1 * S + s) * TPT + r] = PP::get(ay[i / PP::N], i % PP::N);
                red[(2 * S + s) * TPT + r] = PP::get(az[i / PP::N], i % PP::N);
            }
        }
        // the threads that finish the reduction read their point before the next table phase overwrites it
        T ux = T(0), uy = T(0), uz = T(0), ir = T(1);
        if (tid < TPT) {
            const int slot = PPT * (tid % LANES) + tid / LANES;
            ux = sP[0 * TPT + slot];
            uy = sP[1 * TPT + slot];
            uz = sP[2 * TPT + slot];
            ir = sP[3 * TPT + slot];
        }
        fence_proxy_async_smem();  // the rows were read through ordinary loads and are written next by the engine
        __syncthreads();           // partial sums complete; rows, points and tables free
        if (tid == 0) issue(batch + gridDim.x);
        if (tid < TPT) {
            T gx = T(0), gy = T(0), gz = T(0);
            for (int j = 0; j < S; ++j) {
                gx += red[(0 * S + j) * TPT + tid];
                gy += red[(1 * S + j) * TPT + tid];
                gz += red[(2 * S + j) * TPT + tid];
            }
            if constexpr (NORM) {
                // the chain rule through r -> r/|r| is linear in the gradient: applied once to the sum
                const T t = gx * ux + gy * uy + gz * uz;
                gx = (gx - ux * t) * ir;
                gy = (gy - uy * t) * ir;
                gz = (gz - uz * t) * ir;
            }
            const long long ip = batch * TPT + tid;
            if (ip < a.n) {
                a.xyz_grad[3 * ip + 0] = gx;
                a.xyz_grad[3 * ip + 1] = gy;
                a.xyz_grad[3 * ip + 2] = gz;
            }
        }
        // (the partial sums are overwritten only after the next batch's first barrier, which the
        // reducing threads reach after they are done reading them)
    }
}

}  // namespace sph_b200
