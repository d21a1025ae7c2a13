// "Panel" kernels: forward evaluation (values, gradients, Hessians) for any maximum degree
// (run-time l_max). They serve the cases with rows too long for the compile-time tile kernels (see
// the dispatch in sphericart_cuda.cu); the fused backward passes of those cases stay with the band
// kernel.
//
// A CTA is a three-stage pipeline of specialised warps that never meet at a CTA-wide barrier; the
// stages hand buffers to one another through mbarriers in shared memory:
//
//  producer warps   build the per-point tables of a BATCH of TPT consecutive points into one of two
//                   table buffers: c_m + i s_m = (x + i y)^m (a lane builds a block of consecutive m
//                   from one power) and the triangular table Q_l^m with the reference's
//                   downward-in-m recurrence (sphericart/include/templates_core.hpp:123,155,202),
//                   rows dealt in pairs (l, l_max - l) of constant total length. The recurrence is
//                   a serial chain: off the critical path here, it costs the other warps nothing.
//                   Four zeros follow every diagonal, a block of zeros stands for the rows -1 and
//                   -2, and c, s carry two zeros before m = 0, so that every "term absent" case of
//                   the derivative formulas reads a zero.
//  consumer warps   evaluate the (l, m >= 0) pairs of the batch's PANELS (tp consecutive points
//                   each) with the same per-pair code as the band kernel (band_eval_pair /
//                   eval_pair2 and the unit-sphere chain rule) and write both columns of each pair
//                   into the panel's image, one of a ring of `slots` images. A lane is (point
//                   p = lane mod tp, pair slot = lane / tp): neighbouring lanes hold DIFFERENT
//                   POINTS and the SAME pair, so the tables (stored point-minor: element e of point
//                   q at e * TPT + q), the per-pair constants (one address per pair) and the image
//                   rows (neighbouring points an odd number of 4-word groups apart) are read and
//                   written without bank conflicts. A panel's pairs are cut into chunks of 32 / tp;
//                   chunk g of the CTA's running count goes to consumer warp g mod (number of
//                   consumers), so the load evens out across panels whatever the pair count.
//  the store warp   hands each finished image to the TMA engine
//                   (cp.async.bulk.global.shared::cta), waits until the engine has read it and
//                   returns the slot to the ring; the consumers meanwhile fill the other slots.
//                   Odd row lengths (even l_max): the panel's rows are one contiguous span of each
//                   output array; its image is built at the span's own offset modulo 16 bytes and
//                   leaves as one bulk store per array, the few elements before the first and after
//                   the last 16-byte boundary as plain stores. Even row lengths (odd l_max:
//                   (l_max+1)^2 is a multiple of 4): every point's row is 16-byte aligned by itself;
//                   rows get 16 bytes of padding where needed to keep neighbouring points an odd
//                   number of 16-byte groups apart, and leave as one bulk store per point and array.
//
// Every wait on an mbarrier is bounded: a wait that gives up sets a device flag (readable through
// sphericart_cuda_device_wait_errors()) and the warp leaves its loop; the other warps then run into
// their own bounds and leave as well, after the store warp has waited for its copies in flight.
// No communication between CTAs or GPUs. Replaces spherical_harmonics_kernel
// (sphericart/src/sphericart_impl.cu:207-615).
#pragma once

#include <cstdint>

#include "sph_band.cuh"  // per-pair evaluation, shared-memory access helpers, bulk-store helpers

namespace sph_b200 {

constexpr int PANEL_ROW_PAD = 4;    // zeros after the diagonal of every Q row
constexpr int PANEL_MAX_SLOTS = 4;  // images per CTA

// Element offset (for TPT = 1) of row l of the triangular Q table: a block of PANEL_ROW_PAD zeros
// (standing for the rows -1 and -2), then row 0, row 1, ... each with its PANEL_ROW_PAD zeros.
__host__ __device__ constexpr int panel_row_start(int l) { return PANEL_ROW_PAD + l * (l - 1) / 2 + (PANEL_ROW_PAD + 1) * l; }
// Elements of per-point state: the point itself (x, y, z - normalised where the harmonics are - and
// 1/r), c and s with two leading zeros each, then the Q table.
__host__ __device__ constexpr int panel_point_state(int l_max) { return 4 + 2 * (l_max + 3) + panel_row_start(l_max + 1); }

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
    int producers;          // warps that build tables (32 * producers >= TPT)
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

// Phase A for one (point, slice): the slice's block of c_m + i s_m = (x + i y)^m (one power by repeated
// squaring, then one complex product per m) and its rows of the Q table (pairs (j, L - j) of constant
// total length), with the reference's downward-in-m recurrence
// (sphericart/include/templates_core.hpp:123,155,202). A is the type the recurrences are carried in:
// double (rounded once on storing) or the element type itself.
template <typename T, typename A, int TPT>
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
    auto build_row = [&](int l) {
        T* row = sQ + panel_row_start(l) * TPT + qa;
        const T* Kl = sK + tri(l, 0);
        A q2 = A(Kl[l]);  // Q_l^l is tabulated
        row[l * TPT] = T(q2);
        if (l >= 1) {
            A q1 = -zd * q2;  // Q_l^{l-1}
            row[(l - 1) * TPT] = T(q1);
            A tm = A(2 * (l - 1));  // 2 (m + 1)
            for (int m = l - 2; m >= 0; --m) {
                const A q0 = A(Kl[m]) * (tm * zd * q1 + rhod * q2);
                row[m * TPT] = T(q0);
                q2 = q1;
                q1 = q0;
                tm -= A(2);
            }
        }
    };
    for (int j = sa; 2 * j <= L; j += SA) {
        build_row(L - j);
        if (L - j != j) build_row(j);
    }
}

// Set when a bounded wait gave up (it never does unless the device is misbehaving); one flag per
// translation unit, read by PanelLaunch::device_error_flag().
static __device__ int g_panel_wait_gave_up = 0;

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}

// Bytes of the mbarriers at the end of the dynamic shared memory: full / empty for the two table
// buffers and for up to PANEL_MAX_SLOTS images.
constexpr int PANEL_BARRIER_BYTES = 8 * (4 + 2 * PANEL_MAX_SLOTS);
// Polls before a wait between the stages gives up. A hand-over takes microseconds; each poll already
// blocks for a hardware-defined interval, so this bound is reached only if a stage has stopped.
constexpr int PANEL_WAIT_TRIES = 1 << 18;

// blockDim.x = 32 * (producers + 1 + consumers): warps 0 ... producers-1 build tables, warp
// `producers` is the store warp, the rest are consumers. 32 * producers >= TPT.
template <typename T, int LEVEL, bool NORM, int TPT>
__global__ void __launch_bounds__(384) sph_panel_kernel(const __grid_constant__ PanelArgs<T> a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int L = a.l_max;
    const int ny = (L + 1) * (L + 1);
    const int nq = (L + 1) * (L + 2) / 2;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int tp = a.tp;
    const int slots = a.slots;
    const int NP = a.producers;
    const int NB = int(blockDim.x >> 5) - NP - 1;
    const bool bulk = a.bulk != 0;
    const bool packed_rows = (ny & 1) != 0;  // odd row length: the image is the exact picture of global memory
    constexpr unsigned E = unsigned(TPT) * unsigned(sizeof(T));
    constexpr int Q16 = 16 / int(sizeof(T));

    // carve-up: F | K | descriptors | 2 x per-point state of a batch (point-minor) | slots x images | mbarriers
    T* sF = reinterpret_cast<T*>(smem_raw);
    T* sK = sF + nq;
    PanelDesc* sDesc = reinterpret_cast<PanelDesc*>(sF + align16_elems<T>(2 * nq));
    T* state0 = reinterpret_cast<T*>(sDesc + nq);
    const int state_elems = align16_elems<T>(TPT * panel_point_state(L));
    T* images = state0 + 2 * state_elems;
    const int st0 = panel_point_stride(1, ny, int(sizeof(T)));
    const int st1 = panel_point_stride(3, ny, int(sizeof(T)));
    const int st2 = panel_point_stride(9, ny, int(sizeof(T)));
    const int reg0 = panel_region<T>(tp, 1, ny);
    const int reg1 = LEVEL >= 1 ? panel_region<T>(tp, 3, ny) : 0;
    const int reg2 = LEVEL >= 2 ? panel_region<T>(tp, 9, ny) : 0;
    const int slot_elems = reg0 + reg1 + reg2;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(images + size_t(slots) * slot_elems);
    unsigned long long* tfull = bars;       // [2] tables of a batch complete (producers -> consumers)
    unsigned long long* tempty = bars + 2;  // [2] consumers done with a table buffer
    unsigned long long* ifull = bars + 4;   // [slots] image complete (consumers -> store warp)
    unsigned long long* iempty = bars + 4 + PANEL_MAX_SLOTS;  // [slots] image read by the engine, slot free
    // per-point state of table buffer b: x, y, z, 1/r, then c, s (two leading zeros each), then Q
    auto buf_P = [&](int b) { return state0 + b * state_elems; };
    auto buf_c = [&](int b) { return buf_P(b) + 4 * TPT; };
    auto buf_s = [&](int b) { return buf_c(b) + (L + 3) * TPT; };
    auto buf_Q = [&](int b) { return buf_s(b) + (L + 3) * TPT; };

    // ---- once per CTA, all warps: constants, the zeros that never change, the barriers
    for (int e = tid; e < 2 * nq; e += blockDim.x) sF[e] = a.tables[e];
    for (int t = tid; t < nq; t += blockDim.x) {
        PanelDesc d = a.desc[t];
        d.off0 *= int(E);
        d.off1 *= int(E);
        d.off2 *= int(E);
        sDesc[t] = d;
    }
    for (int b = 0; b < 2; ++b) {
        T* sc = buf_c(b);
        T* ss = buf_s(b);
        T* sQ = buf_Q(b);
        for (int e = tid; e < 2 * TPT; e += blockDim.x) {
            sc[e] = T(0);
            ss[e] = T(0);
        }
        for (int e = tid; e < PANEL_ROW_PAD * TPT; e += blockDim.x) sQ[e] = T(0);
        for (int e = tid; e < (L + 1) * PANEL_ROW_PAD * TPT; e += blockDim.x) {
            const int l = e / (PANEL_ROW_PAD * TPT);
            const int r = e % (PANEL_ROW_PAD * TPT);
            sQ[(panel_row_start(l) + l + 1) * TPT + r] = T(0);
        }
    }
    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], unsigned(NP));
            mbar_init(&tempty[b], unsigned(NB));
        }
        for (int sl = 0; sl < slots; ++sl) {
            mbar_init(&ifull[sl], unsigned(NB));
            mbar_init(&iempty[sl], 1u);
        }
        mbar_init_fence();
    }
    __syncthreads();  // the only CTA-wide barrier

    // The work of this CTA: batches blockIdx.x, blockIdx.x + gridDim.x, ...; every role walks the same
    // sequence of batches and panels, so the counts below agree between the roles.
    const long long nbatches = (a.n + TPT - 1) / TPT;
    auto panels_in = [&](long long batch) {
        const long long left = a.n - batch * TPT;
        const int pts = left < TPT ? int(left) : TPT;
        return (pts + tp - 1) / tp;
    };
    auto give_up = [&]() { g_panel_wait_gave_up = 1; };

    if (warp < NP) {
        // ================= producers: tables of batch `it` into buffer it & 1
        const int ptid = warp * 32 + lane;
        const int qa = ptid % TPT;
        const int sa = ptid / TPT;
        const int SA = (NP * 32) / TPT;
        int it = 0;
        for (long long batch = blockIdx.x; batch < nbatches; batch += gridDim.x, ++it) {
            const int b = it & 1;
            // the consumers must be done with this buffer's previous batch (its use (it >> 1) - 1)
            if (it >= 2 && !mbar_wait_bounded(&tempty[b], unsigned(((it >> 1) - 1) & 1), PANEL_WAIT_TRIES)) {
                give_up();
                break;
            }
            if (sa < SA) {
                // rows past the end evaluate a harmless point; they are never copied out
                T x = T(1), y = T(0), z = T(0), ir = T(1);
                const long long ip = batch * TPT + qa;
                if (ip < a.n) {
                    x = a.xyz[3 * ip + 0];
                    y = a.xyz[3 * ip + 1];
                    z = a.xyz[3 * ip + 2];
                }
                if constexpr (NORM) {
                    // IEEE square root and division, as on the CPU (sphericart/include/templates.hpp:392-400)
                    ir = T(1) / sqrt(x * x + y * y + z * z);
                    x *= ir;
                    y *= ir;
                    z *= ir;
                }
                T* sP = buf_P(b);
                if (sa == 0) {
                    sP[0 * TPT + qa] = x;
                    sP[1 * TPT + qa] = y;
                    sP[2 * TPT + qa] = z;
                    sP[3 * TPT + qa] = ir;
                }
                if (a.tables_f64 != 0) {
                    panel_build_tables<T, double, TPT>(x, y, z, L, sa, SA, qa, buf_c(b), buf_s(b), buf_Q(b), sK);
                } else {
                    panel_build_tables<T, T, TPT>(x, y, z, L, sa, SA, qa, buf_c(b), buf_s(b), buf_Q(b), sK);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&tfull[b]);  // release: the tables are visible to whoever sees the phase
        }
    } else if (warp == NP) {
        // ================= the store warp: image of panel `seq` (slot seq mod slots) to global memory
        int seq = 0;
        bool alive = true;
        for (long long batch = blockIdx.x; batch < nbatches && alive; batch += gridDim.x) {
            const int npanels = panels_in(batch);
            for (int j = 0; j < npanels; ++j, ++seq) {
                const int slot = seq % slots;
                if (!mbar_wait_bounded(&ifull[slot], unsigned((seq / slots) & 1), PANEL_WAIT_TRIES)) {
                    give_up();
                    alive = false;
                    break;
                }
                const long long first = batch * TPT + (long long)j * tp;
                const int nvalid = (a.n - first) < tp ? int(a.n - first) : tp;
                T* gsph = a.sph + first * ny;
                T* gd = LEVEL >= 1 ? a.dsph + first * 3 * ny : nullptr;
                T* gdd = LEVEL >= 2 ? a.ddsph + first * 9 * ny : nullptr;
                T* region0 = images + size_t(slot) * slot_elems;
                if (bulk && packed_rows) {
                    // one span per array; the image was built at the span's own offset modulo 16 bytes
                    const int shift0 = int((reinterpret_cast<uintptr_t>(gsph) & 15u) / sizeof(T));
                    const int shift1 = LEVEL >= 1 ? int((reinterpret_cast<uintptr_t>(gd) & 15u) / sizeof(T)) : 0;
                    const int shift2 = LEVEL >= 2 ? int((reinterpret_cast<uintptr_t>(gdd) & 15u) / sizeof(T)) : 0;
                    auto copy_out = [&](T* gdst, const T* img, int shift, int count) {
                        const int head = shift == 0 ? 0 : (Q16 - shift < count ? Q16 - shift : count);
                        const int body = (count - head) / Q16 * Q16;
                        const int tail = count - head - body;
                        if (lane < head) gdst[lane] = img[lane];
                        if (lane >= 8 && lane - 8 < tail) gdst[head + body + lane - 8] = img[head + body + lane - 8];
                        if (lane == 0 && body > 0)
                            bulk_store_smem_to_global(gdst + head, img + head, unsigned(body) * unsigned(sizeof(T)));
                    };
                    copy_out(gsph, region0 + shift0, shift0, nvalid * ny);
                    if constexpr (LEVEL >= 1) copy_out(gd, region0 + reg0 + shift1, shift1, nvalid * 3 * ny);
                    if constexpr (LEVEL >= 2) copy_out(gdd, region0 + reg0 + reg1 + shift2, shift2, nvalid * 9 * ny);
                    if (lane == 0) {
                        bulk_commit();
                        bulk_wait_read_all();
                    }
                } else if (bulk) {
                    // every point's row is 16-byte aligned on both sides: one store per point and array
                    const unsigned ny_b = unsigned(ny) * unsigned(sizeof(T));
                    if (lane == 0) {
                        for (int r = 0; r < nvalid; ++r) {
                            bulk_store_smem_to_global(gsph + size_t(r) * ny, region0 + r * st0, ny_b);
                            if constexpr (LEVEL >= 1)
                                bulk_store_smem_to_global(gd + size_t(r) * 3 * ny, region0 + reg0 + r * st1, 3 * ny_b);
                            if constexpr (LEVEL >= 2)
                                bulk_store_smem_to_global(gdd + size_t(r) * 9 * ny, region0 + reg0 + reg1 + r * st2, 9 * ny_b);
                        }
                        bulk_commit();
                        bulk_wait_read_all();
                    }
                } else {
                    for (int r = 0; r < nvalid; ++r) {
                        for (int e = lane; e < ny; e += 32) gsph[size_t(r) * ny + e] = region0[r * st0 + e];
                        if constexpr (LEVEL >= 1)
                            for (int e = lane; e < 3 * ny; e += 32) gd[size_t(r) * 3 * ny + e] = region0[reg0 + r * st1 + e];
                        if constexpr (LEVEL >= 2)
                            for (int e = lane; e < 9 * ny; e += 32)
                                gdd[size_t(r) * 9 * ny + e] = region0[reg0 + reg1 + r * st2 + e];
                    }
                }
                __syncwarp();  // every lane is done reading the image
                if (lane == 0) mbar_arrive(&iempty[slot]);
            }
        }
    } else {
        // ================= consumers
        const int cw = warp - NP - 1;
        const int p = lane & (tp - 1);  // point of the panel
        const int sl = lane / tp;       // pair slot of a chunk
        const int SPW = 32 / tp;        // pairs per chunk
        const int nchunks = (nq + SPW - 1) / SPW;
        const unsigned f_addr = static_cast<unsigned>(__cvta_generic_to_shared(sF));
        const unsigned desc_addr = static_cast<unsigned>(__cvta_generic_to_shared(sDesc));
        const unsigned ny_b = unsigned(ny) * unsigned(sizeof(T));
        int seq = 0;
        int owner = 0;  // consumer warp that owns the next chunk of the CTA's running count
        int it = 0;
        bool alive = true;
        for (long long batch = blockIdx.x; batch < nbatches && alive; batch += gridDim.x, ++it) {
            const int b = it & 1;
            if (!mbar_wait_bounded(&tfull[b], unsigned((it >> 1) & 1), PANEL_WAIT_TRIES)) {
                give_up();
                break;
            }
            const T* sP = buf_P(b);
            const int npanels = panels_in(batch);
            for (int j = 0; j < npanels; ++j, ++seq) {
                const int slot = seq % slots;
                // the slot's previous image (panel seq - slots) must have been read by the engine. Every
                // consumer waits, also one without a chunk in this panel: its arrival below must not be
                // counted towards the previous phase of the barrier.
                if (seq >= slots && !mbar_wait_bounded(&iempty[slot], unsigned(((seq / slots) - 1) & 1), PANEL_WAIT_TRIES)) {
                    give_up();
                    alive = false;
                    break;
                }
                // this warp's chunks of the panel: c = first_chunk, first_chunk + NB, ...
                int first_chunk = cw - owner;
                if (first_chunk < 0) first_chunk += NB;
                owner = (owner + nchunks) % NB;
                if (first_chunk < nchunks) {
                    const int sub = j * tp;
                    const long long first = batch * TPT + sub;
                    const T x = sP[0 * TPT + sub + p], y = sP[1 * TPT + sub + p], z = sP[2 * TPT + sub + p];
                    [[maybe_unused]] const T ir = sP[3 * TPT + sub + p];
                    const UnitSphere<T> us{x, y, z, ir, ir * ir};
                    const T x2 = x * x, y2 = y * y, xy = x * y;
                    // with packed rows the images are placed so that shared and global addresses agree modulo 16 bytes
                    int shift0 = 0, shift1 = 0, shift2 = 0;
                    if (bulk && packed_rows) {
                        shift0 = int((reinterpret_cast<uintptr_t>(a.sph + first * ny) & 15u) / sizeof(T));
                        if constexpr (LEVEL >= 1) shift1 = int((reinterpret_cast<uintptr_t>(a.dsph + first * 3 * ny) & 15u) / sizeof(T));
                        if constexpr (LEVEL >= 2) shift2 = int((reinterpret_cast<uintptr_t>(a.ddsph + first * 9 * ny) & 15u) / sizeof(T));
                    }
                    T* region0 = images + size_t(slot) * slot_elems;
                    const unsigned q_addr = static_cast<unsigned>(__cvta_generic_to_shared(buf_Q(b) + sub + p));
                    const unsigned c_addr = static_cast<unsigned>(__cvta_generic_to_shared(buf_c(b) + sub + p));
                    const unsigned s_addr = static_cast<unsigned>(__cvta_generic_to_shared(buf_s(b) + sub + p));
                    const unsigned img0_addr = static_cast<unsigned>(__cvta_generic_to_shared(region0 + shift0 + p * st0));
                    [[maybe_unused]] const unsigned img1_addr =
                        static_cast<unsigned>(__cvta_generic_to_shared(region0 + reg0 + shift1 + p * st1));
                    [[maybe_unused]] const unsigned img2_addr =
                        static_cast<unsigned>(__cvta_generic_to_shared(region0 + reg0 + reg1 + shift2 + p * st2));

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
                    auto load = [&](int t) {
                        PanelDesc d;
                        asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(d.off0), "=r"(d.off1), "=r"(d.off2), "=r"(d.klm)
                                     : "r"(desc_addr + unsigned(t) * 16u));
                        const T f = lds_at<T, 0>(f_addr + unsigned(t) * unsigned(sizeof(T)));
                        return panel_load_pair<T, TPT, LEVEL>(d, f, q_addr, c_addr, s_addr);
                    };
                    // pairs of this lane: chunk c holds the pairs c * SPW ... c * SPW + SPW - 1; two in flight
                    int c = first_chunk;
                    for (; c + NB < nchunks; c += 2 * NB) {
                        const int t0 = c * SPW + sl, t1 = (c + NB) * SPW + sl;
                        if (t1 < nq) {
                            const PairInputs<T, LEVEL> in0 = load(t0);
                            const PairInputs<T, LEVEL> in1 = load(t1);
                            finish_pair(in0);
                            finish_pair(in1);
                        } else if (t0 < nq) {
                            finish_pair(load(t0));
                        }
                    }
                    if (c < nchunks) {
                        const int t0 = c * SPW + sl;
                        if (t0 < nq) finish_pair(load(t0));
                    }
                }
                // this warp's share of the image is written: visible to the TMA engine, then to the store warp
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ifull[slot]);
            }
            if (!alive) break;
            // done with this table buffer
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[b]);
        }
    }
}

}  // namespace sph_b200
