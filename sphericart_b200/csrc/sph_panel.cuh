// "Panel" kernels: forward evaluation (values, gradients, Hessians) for any maximum degree
// (run-time l_max) with a whole CTA working on a panel of TP consecutive points (TP = 1 ... 32).
// They serve the cases with rows too long for the compile-time tile kernels (see panel_serves()
// in sph_launch.hpp); the fused backward passes of those cases stay with the band kernel.
//
// Work split. Thread t of a CTA is (point p = t mod TP, slice s = t / TP); S = blockDim.x / TP
// slices share each point. Neighbouring lanes therefore hold DIFFERENT POINTS and the SAME (l, m)
// pair, which makes every shared-memory access of the hot loop conflict-free by construction: the
// per-point tables are stored point-minor (element e of point p at e * TP + p), the per-pair
// constants are read at one address by all lanes of a slice, and the image rows of neighbouring
// points are an odd number of words apart. (The band kernel deals pairs to lanes instead; half of
// its image stores conflict where a warp straddles two degrees.)
//
//  A. Tables, once per panel, all threads: c_m + i s_m = (x + i y)^m (slice s builds a block of
//     consecutive m from one power) and the triangular table Q_l^m with the reference's
//     downward-in-m recurrence (sphericart/include/templates_core.hpp:123,155,202), rows dealt to
//     the slices in pairs (l, l_max - l) of constant total length. Carried in float64 for both
//     element types and rounded once on storing, as in the band kernel. Four zeros follow every
//     diagonal, a block of zeros stands for the rows -1 and -2, and c, s carry two zeros before
//     m = 0, so that every "term absent" case of the derivative formulas reads a zero.
//  B. Pairs. Slice s evaluates the pairs t = s, s + S, ... of the flattened (l, m >= 0) list with
//     the same per-pair code as the band kernel (band_eval_pair / eval_pair2 and the unit-sphere
//     chain rule), two pairs in flight, and writes both columns of each pair into the panel's image.
//  C. Copy-out. The panel's rows are one contiguous span of each output array; the image of each
//     span, built at the span's own offset modulo 16 bytes, leaves as a TMA 1-D bulk store
//     (cp.async.bulk.global.shared::cta), the few elements before the first and after the last
//     16-byte boundary as plain stores. The tables of the next panel are built while the engine
//     reads the image; only the first image store of the next panel waits for it.
//
// No communication between CTAs or GPUs, no spin-wait. Replaces spherical_harmonics_kernel
// (sphericart/src/sphericart_impl.cu:207-615).
#pragma once

#include <cstdint>

#include "sph_band.cuh"  // per-pair evaluation, shared-memory access helpers, bulk-store helpers

namespace sph_b200 {

constexpr int PANEL_ROW_PAD = 4;  // zeros after the diagonal of every Q row

// Element offset (for TP = 1) of row l of the triangular Q table: a block of PANEL_ROW_PAD zeros
// (standing for the rows -1 and -2), then row 0, row 1, ... each with its PANEL_ROW_PAD zeros.
__host__ __device__ constexpr int panel_row_start(int l) { return PANEL_ROW_PAD + l * (l - 1) / 2 + (PANEL_ROW_PAD + 1) * l; }
// Elements of per-point state: c and s with two leading zeros each, then the Q table.
__host__ __device__ constexpr int panel_point_state(int l_max) { return 2 * (l_max + 3) + panel_row_start(l_max + 1); }

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
};

template <typename T, int TP, int LEVEL>
__device__ __forceinline__ PairInputs<T, LEVEL> panel_load_pair(const PanelDesc d, T f, unsigned q_addr, unsigned c_addr,
                                                                unsigned s_addr) {
    constexpr unsigned E = unsigned(TP) * unsigned(sizeof(T));  // bytes between consecutive table elements of one point
    PairInputs<T, LEVEL> in;
    const int m = (d.klm >> 16) & 0xff;
    const int l = (d.klm >> 24) & 0xff;
    in.kp = d.klm & 0xffff;
    in.m = m;
    in.f = f;
    const unsigned ac = c_addr + unsigned(m) * E;  // c_{m-2}
    const unsigned as = s_addr + unsigned(m) * E;  // s_{m-2}
    in.q = lds_at<T, 0>(q_addr + unsigned(d.off0));
    in.cm = lds_at<T, 2 * TP>(ac);
    in.sm = lds_at<T, 2 * TP>(as);
    if constexpr (LEVEL >= 1) {
        const unsigned a1 = q_addr + unsigned(d.off1);
        in.q1a = lds_at<T, TP>(a1);
        in.q1b = lds_at<T, 0>(a1);
        in.cm1 = lds_at<T, TP>(ac);
        in.sm1 = lds_at<T, TP>(as);
        in.fm = T(m);
        in.flm = T(l + m);
    }
    if constexpr (LEVEL >= 2) {
        const unsigned a2 = q_addr + unsigned(d.off2);
        in.q2a = lds_at<T, 2 * TP>(a2);
        in.q2b = lds_at<T, TP>(a2);
        in.q2c = lds_at<T, 0>(a2);
        in.cm2 = lds_at<T, 0>(ac);
        in.sm2 = lds_at<T, 0>(as);
        in.fmm = T(m * (m - 1));
        in.fz = T((l + m) * (l + m - 1));
    }
    return in;
}

// Dynamic shared memory of one CTA, in bytes (also used by the host to plan the launch).
template <typename T> __host__ __device__ constexpr size_t panel_const_bytes(int l_max) {
    return size_t(align16_elems<T>(2 * n_table(l_max))) * sizeof(T) + size_t(n_table(l_max)) * sizeof(PanelDesc);
}
template <typename T> __host__ __device__ constexpr size_t panel_state_bytes(int l_max, int tp) {
    return size_t(align16_elems<T>(tp * panel_point_state(l_max))) * sizeof(T);
}
template <typename T> __host__ __device__ constexpr size_t panel_image_bytes(int l_max, int tp, int level) {
    const int ny = n_columns(l_max);
    size_t e = size_t(band_region<T>(tp, 1, ny));
    if (level >= 1) e += size_t(band_region<T>(tp, 3, ny));
    if (level >= 2) e += size_t(band_region<T>(tp, 9, ny));
    return e * sizeof(T);
}

template <typename T, int LEVEL, bool NORM, int TP>
__global__ void __launch_bounds__(256) sph_panel_kernel(const __grid_constant__ PanelArgs<T> a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int L = a.l_max;
    const int ny = (L + 1) * (L + 1);
    const int nq = (L + 1) * (L + 2) / 2;
    const int tid = threadIdx.x;
    const int p = tid % TP;  // point of the panel
    const int s = tid / TP;  // slice of the point's (l, m) pairs
    const int S = blockDim.x / TP;
    const bool bulk = a.bulk != 0;
    constexpr unsigned E = unsigned(TP) * unsigned(sizeof(T));

    // carve-up: F | K | descriptors | per-point state (point-minor) | images
    T* sF = reinterpret_cast<T*>(smem_raw);
    T* sK = sF + nq;
    PanelDesc* sDesc = reinterpret_cast<PanelDesc*>(sF + align16_elems<T>(2 * nq));
    T* state = reinterpret_cast<T*>(sDesc + nq);
    T* sc = state;                            // c_m of point p at sc[(m + 2) * TP + p]
    T* ss = sc + (L + 3) * TP;                // s_m likewise
    T* sQ = ss + (L + 3) * TP;                // element e of point p at sQ[e * TP + p]
    T* region0 = state + align16_elems<T>(TP * panel_point_state(L));
    T* region1 = region0 + band_region<T>(TP, 1, ny);
    T* region2 = region1 + (LEVEL >= 1 ? band_region<T>(TP, 3, ny) : 0);

    // ---- once per CTA: constants, and the zeros that never change
    for (int e = tid; e < 2 * nq; e += blockDim.x) sF[e] = a.tables[e];
    for (int t = tid; t < nq; t += blockDim.x) {
        PanelDesc d = a.desc[t];
        d.off0 *= int(E);
        d.off1 *= int(E);
        d.off2 *= int(E);
        sDesc[t] = d;
    }
    for (int e = tid; e < 2 * TP; e += blockDim.x) {
        sc[e] = T(0);
        ss[e] = T(0);
    }
    for (int e = tid; e < PANEL_ROW_PAD * TP; e += blockDim.x) sQ[e] = T(0);
    for (int e = tid; e < (L + 1) * PANEL_ROW_PAD * TP; e += blockDim.x) {
        const int l = e / (PANEL_ROW_PAD * TP);
        const int r = e % (PANEL_ROW_PAD * TP);
        sQ[(panel_row_start(l) + l + 1) * TP + r] = T(0);
    }
    __syncthreads();

    const unsigned q_addr = static_cast<unsigned>(__cvta_generic_to_shared(sQ + p));
    const unsigned c_addr = static_cast<unsigned>(__cvta_generic_to_shared(sc + p));
    const unsigned s_addr = static_cast<unsigned>(__cvta_generic_to_shared(ss + p));
    const unsigned f_addr = static_cast<unsigned>(__cvta_generic_to_shared(sF));
    const unsigned desc_addr = static_cast<unsigned>(__cvta_generic_to_shared(sDesc));
    const unsigned ny_b = unsigned(ny) * unsigned(sizeof(T));

    const long long npanels = (a.n + TP - 1) / TP;
    bool stores_in_flight = false;  // thread 0 only: committed bulk stores that may still read the images
    for (long long panel = blockIdx.x; panel < npanels; panel += gridDim.x) {
        const long long first = panel * TP;
        const long long i = first + p;
        const int nvalid = (a.n - first) < TP ? int(a.n - first) : TP;

        // rows past the end evaluate a harmless point; they are never copied out
        T x = T(1), y = T(0), z = T(0);
        if (i < a.n) {
            x = a.xyz[3 * i + 0];
            y = a.xyz[3 * i + 1];
            z = a.xyz[3 * i + 2];
        }
        UnitSphere<T> us{x, y, z, T(0), T(0)};
        if constexpr (NORM) {
            // IEEE square root and division, as on the CPU (sphericart/include/templates.hpp:392-400)
            const T ir = T(1) / sqrt(x * x + y * y + z * z);
            x *= ir;
            y *= ir;
            z *= ir;
            us = UnitSphere<T>{x, y, z, ir, ir * ir};
        }
        const T x2 = x * x, y2 = y * y, xy = x * y;

        // ---- phase A (float64 for both element types, rounded once on storing)
        {
            const double xd = double(x), yd = double(y), zd = double(z);
            const double rhod = xd * xd + yd * yd;
            // c_m + i s_m for a block of consecutive m: one power, then one complex product per m
            const int block = (L + S) / S;  // ceil((L + 1) / S)
            const int m0 = s * block;
            if (m0 <= L) {
                double pr = 1.0, pi = 0.0;
                double wr = xd, wi = yd;
                for (int bits = m0; bits != 0; bits >>= 1) {
                    if (bits & 1) {
                        const double nr = pr * wr - pi * wi;
                        pi = pr * wi + pi * wr;
                        pr = nr;
                    }
                    const double sr = wr * wr - wi * wi;
                    wi = (wr + wr) * wi;
                    wr = sr;
                }
                const int m1 = (m0 + block - 1) < L ? (m0 + block - 1) : L;
                for (int m = m0; m <= m1; ++m) {
                    sc[(m + 2) * TP + p] = T(pr);
                    ss[(m + 2) * TP + p] = T(pi);
                    const double nr = pr * xd - pi * yd;
                    pi = pr * yd + pi * xd;
                    pr = nr;
                }
            }
            // Q rows, dealt to the slices in pairs (j, L - j) of constant total length
            auto build_row = [&](int l) {
                T* row = sQ + panel_row_start(l) * TP + p;
                const T* Kl = sK + tri(l, 0);
                double q2 = double(Kl[l]);  // Q_l^l is tabulated
                row[l * TP] = T(q2);
                if (l >= 1) {
                    double q1 = -zd * q2;  // Q_l^{l-1}
                    row[(l - 1) * TP] = T(q1);
                    double tm = double(2 * (l - 1));  // 2 (m + 1)
                    for (int m = l - 2; m >= 0; --m) {
                        const double q0 = double(Kl[m]) * (tm * zd * q1 + rhod * q2);
                        row[m * TP] = T(q0);
                        q2 = q1;
                        q1 = q0;
                        tm -= 2.0;
                    }
                }
            };
            for (int j = s; 2 * j <= L; j += S) {
                build_row(L - j);
                if (L - j != j) build_row(j);
            }
        }

        // where this panel's rows go; images placed so that shared and global addresses agree modulo 16 bytes
        T* gsph = a.sph + first * ny;
        T* gd = LEVEL >= 1 ? a.dsph + first * 3 * ny : nullptr;
        T* gdd = LEVEL >= 2 ? a.ddsph + first * 9 * ny : nullptr;
        int shift0 = 0, shift1 = 0, shift2 = 0;
        if (bulk) {
            shift0 = int((reinterpret_cast<uintptr_t>(gsph) & 15u) / sizeof(T));
            if constexpr (LEVEL >= 1) shift1 = int((reinterpret_cast<uintptr_t>(gd) & 15u) / sizeof(T));
            if constexpr (LEVEL >= 2) shift2 = int((reinterpret_cast<uintptr_t>(gdd) & 15u) / sizeof(T));
        }
        T* image0 = region0 + shift0;
        T* image1 = region1 + shift1;
        T* image2 = region2 + shift2;

        // the engine must be done reading the previous panel's images before phase B overwrites them
        if (tid == 0 && stores_in_flight) {
            bulk_wait_read_all();
            stores_in_flight = false;
        }
        __syncthreads();  // tables complete, images free

        const unsigned img0_addr = static_cast<unsigned>(__cvta_generic_to_shared(image0 + p * ny));
        [[maybe_unused]] const unsigned img1_addr = static_cast<unsigned>(__cvta_generic_to_shared(image1 + p * 3 * ny));
        [[maybe_unused]] const unsigned img2_addr = static_cast<unsigned>(__cvta_generic_to_shared(image2 + p * 9 * ny));

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
                eval_pair2<LEVEL>(ps, f2(float(in.cm), float(in.sm)), f2(float(in.cm1), float(in.sm1)), cs2, float(x),
                                  float(y), float(x2), float(y2), float(xy), v);
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

        // ---- phase B: pairs t = s, s + S, ..., two in flight per thread
        auto load = [&](int t) {
            PanelDesc d;
            asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(d.off0), "=r"(d.off1), "=r"(d.off2), "=r"(d.klm)
                         : "r"(desc_addr + unsigned(t) * 16u));
            const T f = lds_at<T, 0>(f_addr + unsigned(t) * unsigned(sizeof(T)));
            return panel_load_pair<T, TP, LEVEL>(d, f, q_addr, c_addr, s_addr);
        };
        int t = s;
        for (; t + S < nq; t += 2 * S) {
            const PairInputs<T, LEVEL> in0 = load(t);
            const PairInputs<T, LEVEL> in1 = load(t + S);
            finish_pair(in0);
            finish_pair(in1);
        }
        if (t < nq) finish_pair(load(t));

        // ---- copy-out
        if (bulk) {
            fence_proxy_async_smem();  // this thread's image writes, visible to the TMA engine
            __syncthreads();           // images complete; phase B has finished reading the tables
            if (tid < 32) {
                constexpr int Q16 = 16 / int(sizeof(T));
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
                if (tid == 0) {
                    bulk_commit();
                    stores_in_flight = true;
                }
            }
        } else {
            __syncthreads();
            for (int e = tid; e < nvalid * ny; e += blockDim.x) gsph[e] = image0[e];
            if constexpr (LEVEL >= 1)
                for (int e = tid; e < nvalid * 3 * ny; e += blockDim.x) gd[e] = image1[e];
            if constexpr (LEVEL >= 2)
                for (int e = tid; e < nvalid * 9 * ny; e += blockDim.x) gdd[e] = image2[e];
            __syncthreads();  // images free for the next panel
        }
    }
    // shared memory must outlive the engine's reads
    if (tid == 0 && stores_in_flight) bulk_wait_read_all();
}

}  // namespace sph_b200
