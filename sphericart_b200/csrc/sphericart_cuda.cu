// Host side of the library: the sphericart::cuda calculator classes and the C ABI.
//
// Mirrors the behaviour of sphericart/src/sphericart_cuda.cpp:40-196 (argument checks, device
// follows the xyz pointer, lazy per-device state) and sphericart/src/sphericart-capi.cpp:637-876
// (C wrappers), with statically compiled sm_100a kernels instead of run-time compilation.
// There is deliberately no CPU code path: without a usable CUDA device every call fails.
#include "sphericart_b200.h"
#include "sphericart_cuda.hpp"

#include "sph_core.cuh"
#include "sph_launch.hpp"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace sph_b200 {

namespace {

void check(cudaError_t status, const char* what) {
    if (status != cudaSuccess) {
        throw std::runtime_error(std::string("sphericart::cuda: ") + what + " failed: " + cudaGetErrorString(status));
    }
}

// Switches for the kernel-variant tests, read from the environment once per process (0 = use the
// built-in choice). They select code paths the default dispatch reaches only for some inputs, so that
// every path can be checked against the CPU reference on the same inputs; none is a tuning knob.
struct Knobs {
    int band_lanes;     // force lanes per point (1..32, power of two)
    int band_warps;     // force warps per CTA of the band kernel (1..4)
    int tile_warps;     // force warps per CTA of the tile kernels (1..8)
    int force_band;     // route every call through the band kernel
    int no_bulk;        // copy tiles out with plain stores instead of TMA bulk stores
    int band_direct;    // 1: force direct global stores in the band kernel, -1: forbid them
    int tile_iters;     // work items per warp of the forward tile kernels (k > 0), -1: persistent launch
    int vjp_iters;      // the same for the backward tile kernels
    int band_iters;     // the same for the band kernels
    int tile_points;    // force the points per tile of the forward tile kernels (8, 16 or 32)
    int tile_lmax;      // largest l_max served by the tile kernels (default: all they are compiled for)
    int no_panel;       // route what the panel kernels would serve to the band kernel
    int panel_batch;    // force the points per table batch of the panel kernels (1, 2, 4, 8, 16 or 32)
    int panel_points;   // force the points per panel image (a power of two dividing the batch)
    int panel_slots;    // force the images per CTA (1..4)
    int panel_threads;  // force the threads per CTA of the panel kernels (<= 256)
    int panel_iters;    // table batches per CTA of the panel kernels (k > 0), -1: persistent launch
    int panel_tables_f64;  // 1: table recurrences of the panel kernels in float64 for float32 outputs too
};

int env_int(const char* name, int fallback) {
    const char* v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    return std::atoi(v);
}

const Knobs& knobs() {
    static const Knobs k = {env_int("SPH_B200_BAND_LANES", 0),  env_int("SPH_B200_BAND_WARPS", 0),
                            env_int("SPH_B200_TILE_WARPS", 0),  env_int("SPH_B200_FORCE_BAND", 0),
                            env_int("SPH_B200_NO_BULK", 0),     env_int("SPH_B200_BAND_DIRECT", 0),
                            env_int("SPH_B200_TILE_ITERS", 0),  env_int("SPH_B200_VJP_ITERS", 0),
                            env_int("SPH_B200_BAND_ITERS", 0),  env_int("SPH_B200_TILE_POINTS", 0),
                            env_int("SPH_B200_TILE_LMAX", TILE_LMAX), env_int("SPH_B200_NO_PANEL", 0),
                            env_int("SPH_B200_PANEL_BATCH", 0), env_int("SPH_B200_PANEL_POINTS", 0),
                            env_int("SPH_B200_PANEL_SLOTS", 0), env_int("SPH_B200_PANEL_THREADS", 0),
                            env_int("SPH_B200_PANEL_ITERS", 0), env_int("SPH_B200_PANEL_TABLES_F64", 0)};
    return k;
}

// A knob of the *_iters family against the built-in choice: the value handed to work_grid().
int resolve_iters(int knob, int builtin) { return knob < 0 ? 0 : (knob > 0 ? knob : builtin); }

struct DeviceProps {
    std::atomic<bool> known{false};
    int sm_count = 0;
    size_t smem_optin = 0;
};
std::mutex g_props_mutex;
DeviceProps g_props[MAX_DEVICES];

// Filled once per device; afterwards read without taking the lock.
const DeviceProps& device_props(int device) {
    DeviceProps& p = g_props[device];
    if (p.known.load(std::memory_order_acquire)) return p;
    std::lock_guard<std::mutex> lock(g_props_mutex);
    if (!p.known.load(std::memory_order_relaxed)) {
        int v = 0;
        check(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute");
        p.sm_count = v;
        check(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, device), "cudaDeviceGetAttribute");
        p.smem_optin = size_t(v);
        p.known.store(true, std::memory_order_release);
    }
    return p;
}

}  // namespace

int device_sm_count(int device) { return device_props(device).sm_count; }

int persistent_grid(const void* kernel, int block, size_t smem, int device) {
    const DeviceProps& props = device_props(device);
    if (smem > props.smem_optin) return 0;
    {
        // The dynamic shared-memory limit of a kernel is per-process state and one kernel may be
        // launched with several sizes (calculators of different l_max, different tile widths) from
        // several threads: the read-compare-raise sequence is serialised and the limit is only ever
        // raised, so a concurrent launch that needs more never finds it lowered.
        static std::mutex attribute_mutex;
        std::lock_guard<std::mutex> lock(attribute_mutex);
        cudaFuncAttributes attr;
        if (cudaFuncGetAttributes(&attr, kernel) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        if (size_t(attr.maxDynamicSharedSizeBytes) < smem &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return per_sm * props.sm_count;
}

// Prefactor tables in the working precision, built with the recipe of the reference
// (sphericart/include/templates.hpp:54-97) so that both sides start from the same constants:
// F[l][m] = (-1)^m sqrt((2l+1)/(2 pi) (l-m)!/(l+m)!) by iterated products, with 1/sqrt(2) folded
// into m = 0; K[l][l] = Q_l^l = -(2l-1) K[l-1][l-1], K[l][m<l] = -1/((l+m+1)(l-m)).
template <typename T> void build_tables(int l_max, T* out) {
    const int nq = n_table(l_max);
    T* F = out;
    T* K = out + nq;
    const T pi = static_cast<T>(3.141592653589793238462643383279502884L);
    const T inv_sqrt_two = static_cast<T>(0.707106781186547524400844362104849039L);
    for (int l = 0; l <= l_max; ++l) {
        T acc = (2 * l + 1) / (2 * pi);
        F[tri(l, 0)] = std::sqrt(acc) * inv_sqrt_two;
        for (int m = 1; m <= l; ++m) {
            acc *= static_cast<T>(1.0) / (l * (l + 1) + m * (1 - m));
            F[tri(l, m)] = (m % 2 == 0) ? std::sqrt(acc) : -std::sqrt(acc);
        }
    }
    K[0] = 1;
    for (int l = 1; l <= l_max; ++l) {
        K[tri(l, l)] = -(2 * l - 1) * K[tri(l - 1, l - 1)];
        for (int m = l - 1; m >= 0; --m) K[tri(l, m)] = static_cast<T>(-1.0) / ((l + m + 1) * (l - m));
    }
}

// ---------------------------------------------------------------------------------------------
// Band-kernel plan: lanes per point, warps per CTA, copy-out mode, shared-memory size.
struct BandPlan {
    int lanes = 1;    // G
    int warps = 1;    // warps per CTA
    int mode = 0;     // 0 image + TMA bulk stores, 1 image + plain stores, 2 direct global stores
    size_t smem = 0;  // dynamic shared memory per CTA
    int grid_cap = 0; // upper bound on CTAs of a persistent launch (0 = none)
    int iters = 0;    // groups of points per warp (see work_grid() in sph_launch.hpp)
    bool feasible = true;
};

// Sizes shared with the kernel (sph_band.cuh), restated for a run-time element size.
size_t band_align16(size_t elems, size_t elem) {
    const size_t q = 16 / elem;
    return (elems + q - 1) / q * q;
}
int band_row_stride_host(int l_max) { return (l_max + 5) + ((l_max + 5) & 1); }
size_t band_point_state_host(int l_max) {
    return 2 * size_t(l_max + 3) + size_t(l_max + 3) * band_row_stride_host(l_max);
}

// kind: 0..2 = forward level, 3 = VJP of the values, 4 = VJP of (values, gradients).
BandPlan make_band_plan(int l_max, int kind, size_t elem, size_t smem_limit, int sm_count) {
    const int L = l_max;
    const size_t ny = size_t(n_columns(L));
    const size_t nq = size_t(n_table(L));
    const bool vjp = kind >= 3;
    const size_t vjp_rows = kind == 4 ? 4 : 1;  // staged upstream-gradient rows per point, in units of ny
    // per CTA: F and K, the per-pair factors (2 per pair with gradients, 4 with Hessians) and the
    // 16-byte pair descriptors
    const size_t pair_factors = (kind == 1 || kind == 3) ? 2 : ((kind == 2 || kind == 4) ? 4 : 0);
    const size_t table_bytes =
        (band_align16(2 * nq, elem) + band_align16(nq * pair_factors, elem)) * elem + nq * 16;
    const size_t slack = 16 / elem;

    auto per_warp_bytes = [&](int P, bool with_image) {
        size_t e = band_align16(size_t(P) * band_point_state_host(L), elem);
        if (vjp) return (e + band_align16(size_t(P) * vjp_rows * ny, elem)) * elem;
        if (with_image) {
            e += band_align16(size_t(P) * ny, elem) + slack;
            if (kind >= 1) e += band_align16(size_t(P) * 3 * ny, elem) + slack;
            if (kind >= 2) e += band_align16(size_t(P) * 9 * ny, elem) + slack;
        }
        return e * elem;
    };
    // warps per SM that fit when CTAs of w warps share the tables
    auto warps_per_sm = [&](size_t per_warp, int w) {
        const size_t cta = table_bytes + w * per_warp;
        if (cta > smem_limit) return size_t(0);
        const size_t n_cta = std::min<size_t>(32, (smem_limit + 1024) / (cta + 1024));
        return std::min<size_t>(64, n_cta * w);
    };

    BandPlan plan;
    // Lanes per point. The pair loop is balanced for any G, so G is chosen for occupancy and for
    // amortising the per-group prologue: about four pairs per lane at least, and a warp's images
    // within the budget.
    const size_t budget = 64 * 1024;
    const int pairs = n_table(L);
    int G = 32;
    while (G > 1 && pairs / G < 4) G /= 2;
    while (G < 32 && per_warp_bytes(32 / G, true) > budget) G *= 2;
    const int forced = knobs().band_lanes;
    if (forced == 1 || forced == 2 || forced == 4 || forced == 8 || forced == 16 || forced == 32) G = forced;
    // whatever was asked for, one warp's state and images must fit next to the tables
    while (G < 32 && table_bytes + per_warp_bytes(32 / G, !vjp) > smem_limit) G *= 2;

    // Copy-out mode. With a whole warp per point, rows so long that their image leaves room for
    // fewer than eight warps per SM are stored straight to global memory instead, provided a
    // degree's run of columns is long enough to fill store sectors (>= 128 bytes at l_max).
    plan.mode = knobs().no_bulk != 0 ? 1 : 0;
    if (!vjp && G == 32) {
        const bool long_runs = size_t(L + 1) * elem >= 128;
        const bool image_fits = warps_per_sm(per_warp_bytes(1, true), 1) >= 1;
        const bool crowded = warps_per_sm(per_warp_bytes(1, true), 4) < 8 && warps_per_sm(per_warp_bytes(1, true), 1) < 8;
        if (!image_fits || (crowded && long_runs)) plan.mode = 2;
        if (knobs().band_direct == 1) plan.mode = 2;
        if (knobs().band_direct == -1 && image_fits) plan.mode = knobs().no_bulk != 0 ? 1 : 0;
    }
    plan.lanes = G;
    const int P = 32 / G;
    const size_t per_warp = per_warp_bytes(P, plan.mode != 2);

    // warps per CTA: up to 4; pick the count that packs the most warps into an SM
    int warps = 1;
    const int forced_warps = knobs().band_warps;
    if (forced_warps >= 1 && forced_warps <= 4) {
        warps = forced_warps;
    } else {
        size_t best = 0;
        for (int w = 4; w >= 1; --w) {
            const size_t per_sm = warps_per_sm(per_warp, w);
            if (per_sm > best) {
                best = per_sm;
                warps = w;
            }
        }
    }
    plan.warps = warps;
    plan.grid_cap = 0;
    if (plan.mode == 2 && forced_warps == 0) {
        // Direct stores: every warp keeps several write streams open in L2 / DRAM. In a persistent
        // launch (smaller calls, see work_grid()) measured throughput peaks at eight warps per SM
        // (12 warps: 12 % slower, 4 warps: 28 % slower on a B200 at l_max = 32, float64), hence the
        // cap of two CTAs of four warps per SM; a launch of short-lived CTAs is not capped.
        plan.warps = warps = 4;
        if (table_bytes + 4 * per_warp > smem_limit) plan.warps = warps = 1;
        plan.grid_cap = (warps == 4 ? 2 : 8) * sm_count;
    }
    while (warps > 1 && table_bytes + warps * per_warp > smem_limit) --warps;  // a forced count may not fit
    plan.warps = warps;
    plan.smem = table_bytes + warps * per_warp;
    if (plan.smem > smem_limit) plan.feasible = false;
    // Short-lived CTAs (see work_grid()); each one rebuilds the tables in shared memory, which a few
    // dozen groups per warp amortise. Measured on a B200: l_max = 16 float32 Hessians 0.78 -> 0.81 of
    // the copy peak at 32 groups per warp; l_max = 32 float64 gradients (direct stores) 0.73 -> 0.76
    // at 4.
    plan.iters = resolve_iters(knobs().band_iters, plan.mode == 2 ? 4 : 32);
    return plan;
}

// ---------------------------------------------------------------------------------------------
// Panel-kernel plan: points per panel (TP), threads per CTA, shared-memory size. The sizes restate
// panel_const_bytes / panel_state_bytes / panel_image_bytes of sph_panel.cuh for a run-time element size.
struct PanelPlan {
    int batch = 0;     // TPT: points whose tables are built at once
    int tp = 0;        // points per panel (image); a power of two dividing batch
    int slots = 0;     // images per CTA
    int threads = 0;   // threads per CTA; threads / tp slices share each point
    size_t smem = 0;   // dynamic shared memory per CTA
    int iters = 0;     // table batches per CTA (see work_grid() in sph_launch.hpp)
    bool feasible = false;
};

constexpr int PANEL_LMAX = 200;  // the descriptors hold l and m in 8 bits and the column in 16

// Bytes of one panel image: the regions of sph_panel.cuh (panel_region) for a run-time element size.
size_t panel_image_bytes(int l_max, int level, int tp, size_t elem) {
    const size_t ny = size_t(n_columns(l_max));
    const size_t q = 16 / elem;
    auto stride = [&](size_t comps) {
        const size_t packed = comps * ny;
        if (ny % 2 != 0) return packed;
        return (packed / q) % 2 == 0 ? packed + q : packed;
    };
    size_t image = band_align16(size_t(tp) * stride(1), elem) + q;
    if (level >= 1) image += band_align16(size_t(tp) * stride(3), elem) + q;
    if (level >= 2) image += band_align16(size_t(tp) * stride(9), elem) + q;
    return image * elem;
}

size_t panel_fixed_bytes(int l_max, int level, int batch, size_t elem) {
    const size_t nq = size_t(n_table(l_max));
    // (values only: F and K with every entry broadcast to a pack of points, 8 bytes each; no descriptors)
    const size_t consts = level >= 1 ? band_align16(2 * nq, elem) * elem + nq * 16 : (2 * nq * 8 + 15) / 16 * 16;
    const size_t per_point = size_t(panel_point_state(l_max, level));
    return consts + band_align16(size_t(batch) * per_point, elem) * elem;
}

// Chooses the panel shape. Measured on a B200 over a few hundred forced shapes, what counts is: enough
// image bytes per SM on their way to HBM (CTAs per SM x image size, up to about 160 KB - an image
// drains for microseconds once the memory system is saturated), warps per SM (beyond about twelve
// more did not help), how evenly the pairs divide among the slices of a point and into whole warps,
// MANY pairs per thread and panel (each panel costs two barriers, a copy-out and the wait for the
// previous image: l_max = 16 float32 Hessians, 2e6 points, four points per panel: 3 / 4 / 5 pairs per
// thread -> 0.87 / 0.86 / 0.93 of the copy peak with 21 / 15 / 12 warps per SM),
// and a table batch large enough to keep the threads busy during the table phase. A whole warp of
// points per panel (tp = 32: all lanes of a warp read the same per-pair constants) measured better
// than its score otherwise says, hence the bonus. One image per CTA: a ring of two halves the
// panel that fits and was slower in every case measured. `regs` = registers per thread (occupancy).
PanelPlan make_panel_plan(int l_max, int level, size_t elem, size_t smem_limit, int regs) {
    PanelPlan best;
    if (l_max > PANEL_LMAX) return best;
    // Rows so long that even one point's image leaves room for a single small CTA per SM stay with the
    // band kernel and its direct stores (measured, panel / band: float64 gradients l_max = 40, 54 KB per
    // point: 0.65 / 0.78; float64 Hessians l_max = 32, 113 KB per point: 0.37 / 0.49; below these sizes the
    // panel kernels win, e.g. float64 Hessians l_max = 24, 65 KB per point: 0.66 / 0.47).
    const size_t one_point = panel_image_bytes(l_max, level, 1, elem);
    if (knobs().panel_points <= 0 && ((level == 1 && one_point > 44 * 1024) || (level == 2 && one_point > 100 * 1024))) return best;
    const int nq = n_table(l_max);
    const bool even_rows = n_columns(l_max) % 2 == 0;
    if (regs <= 0) regs = level == 2 ? 176 : 64;
    const int regs_alloc = (regs + 7) / 8 * 8;
    const Knobs& k = knobs();
    double best_score = -1.0;
    for (int batch = 32; batch >= 1; batch /= 2) {
        if (k.panel_batch > 0 && batch != k.panel_batch) continue;
        const size_t fixed = panel_fixed_bytes(l_max, level, batch, elem);
        for (int tp = batch; tp >= 1; tp /= 2) {
            if (k.panel_points > 0 && tp != k.panel_points) continue;
            // table batches of 32 points only for whole-warp panels (measured, l_max = 16 float32 gradients,
            // 16 points per panel: batches of 16 / 32 points -> 0.86 / 0.79)
            if (batch == 32 && tp < 32 && k.panel_batch <= 0) continue;
            // rows of even length: neighbouring points sit a multiple of 16 bytes apart, which is
            // conflict-free for up to eight points side by side
            // (values only: the threads of a slice hold every fourth / second point)
            const int side_by_side = level == 0 ? tp / panel_values_ppt(int(elem)) : tp;
            if (even_rows && side_by_side > 8 && k.panel_points <= 0) continue;
            const size_t image = panel_image_bytes(l_max, level, tp, elem);
            for (int slots = 1; slots <= 4; ++slots) {
                if (k.panel_slots > 0 ? slots != k.panel_slots : slots != 1) continue;
                const size_t smem = fixed + slots * image;
                if (smem > smem_limit) break;
                // the work a slice divides: (l, m) pairs, or - values only - pairs of rows (j, l_max - j)
                const int items = level == 0 ? l_max / 2 + 1 : nq;
                // threads side by side in a slice: one per point, or - values only - one per 16 bytes' worth of points
                const int lanes = level == 0 ? tp / panel_values_ppt(int(elem)) : tp;
                if (lanes < 1) continue;
                for (int per_slice = 1; per_slice <= items; ++per_slice) {
                    const int slices = (items + per_slice - 1) / per_slice;
                    int threads = slices * lanes;
                    if (k.panel_threads > 0) threads = k.panel_threads;
                    if (threads > 256) continue;
                    if (threads < (level == 0 ? 32 : 64) && k.panel_threads <= 0) break;
                    if (threads < batch) continue;
                    const int warp_threads = (threads + 31) / 32 * 32;
                    long long ctas = std::min<long long>(32, (long long)(233472 / (smem + 1024)));
                    ctas = std::min<long long>(ctas, 2048 / warp_threads);
                    ctas = std::min<long long>(ctas, 65536 / (regs_alloc * warp_threads));
                    if (ctas < 1) continue;
                    const int real_slices = threads / lanes;
                    const int real_per_slice = (items + real_slices - 1) / real_slices;
                    const double in_flight = std::min<double>(double(ctas * slots) * double(image), 160.0 * 1024) / (160.0 * 1024);
                    const double warps = std::min<double>(double(ctas * warp_threads / 32), 12.0) / 12.0;
                    const double balance = double(items) / (double(real_slices) * real_per_slice) * threads / warp_threads;
                    // (a pair of rows is l_max + 2 steps of the recurrence, each writing a pair)
                    const double pairs_each = level == 0 ? double(real_per_slice) * (l_max + 2) : double(real_per_slice);
                    const double panel_cost = pairs_each / (pairs_each + 2.0);
                    const double table_busy = std::min(1.0, double(batch) * ((l_max + 2) / 2) / threads);
                    double score = in_flight * warps * balance * panel_cost * (0.7 + 0.3 * table_busy) *
                                   (ctas >= 2 ? 1.0 : 0.8) * (tp == 32 ? 1.15 : 1.0);
                    if (level == 0) {
                        // Values only: a thread carries 16 bytes' worth of points through whole rows, which gives
                        // it the independent work that the other levels get from many warps; the kernel is bound
                        // by shared-memory traffic (image writes, the engine's reads, the c/s loads), and four
                        // slices share a warp, so bank conflicts between slices vary with l_max. Measured: one
                        // pair of rows per thread is best (two: 0.49 against 0.79, float32 l_max = 24). Float32:
                        // eight threads side by side (32 points per panel) where two CTAs fit an SM (l_max = 24:
                        // 32 / 16 / 8 points -> 0.72 / 0.54 / 0.54 of the copy peak), half as many where only one
                        // would (l_max = 28: 0.55 against 0.61). Float64: four threads side by side (8 points per
                        // panel) at every degree measured (l_max = 22 / 26 / 32: 0.80 / 0.81 / 0.69 against
                        // 0.63 / 0.65 / 0.60 with 16 points).
                        // (rows of even length were only measured with eight threads side by side: float64 l_max = 21: 0.92)
                        const bool narrow = elem == 8 && !even_rows;
                        const int target = narrow ? 4 : 8;
                        const double side = lanes == target ? 1.0 : (lanes > target ? 0.8 : std::sqrt(double(lanes) / target));
                        // (a table batch larger than the panel measured lower: float64 l_max = 26, batches of 16 / 8
                        // points for panels of 8: 0.59 / 0.81; partly filled warps do not count against a shape here)
                        const double dealt = double(items) / (double(real_slices) * real_per_slice);
                        score = side * dealt / real_per_slice * (ctas >= 2 ? 1.0 : 0.7) * (0.85 + 0.05 * std::min<long long>(ctas, 3)) *
                                (tp >= (narrow ? 8 : 16) ? 1.0 : 0.85) * (batch == tp ? 1.0 : 0.9);
                    }
                    if (score > best_score + 1e-9) {
                        best_score = score;
                        best.batch = batch;
                        best.tp = tp;
                        best.slots = slots;
                        best.threads = threads;
                        best.smem = smem;
                        best.feasible = true;
                    }
                    if (k.panel_threads > 0) break;
                }
            }
        }
    }
    // Float32 gradients with rows of even length at moderate degrees: the score above settles on CTAs of two warps
    // (eight points, eight slices); table batches of sixteen points with sixteen slices measured better
    // (l_max = 11 / 13 / 15: 0.79 / 0.79 / 0.78 -> 0.83 / 0.82 / 0.87 of the copy peak; from l_max = 17 on and
    // in float64 the score's own choice is the best measured).
    if (level == 1 && elem == 4 && even_rows && best.feasible && best.tp == 8 && best.batch == 8 && best.threads < 128 &&
        k.panel_batch <= 0 && k.panel_points <= 0 && k.panel_threads <= 0) {
        const size_t smem = panel_fixed_bytes(l_max, level, 16, elem) + panel_image_bytes(l_max, level, 8, elem);
        if (smem <= smem_limit && 233472 / (smem + 1024) >= 4) {
            best.batch = 16;
            best.threads = 128;
            best.smem = smem;
        }
    }
    // Shapes measured on a B200 over twelve to twenty-five candidates per case (1.5 GB launches, fraction of the copy
    // peak, the score's choice -> the shape taken here). Hessians:
    //   float32 l_max 11: 0.85 -> 0.90   12: 0.74 -> 0.88   13: 0.78 -> 0.82   14: 0.84 -> 0.91   15: 0.75 -> 0.83
    //                 17: 0.81 -> 0.86   18: 0.75 -> 0.85   19: 0.71 -> 0.86
    //   float64 l_max  7: 0.76 -> 0.83   13: 0.74 -> 0.85   15: 0.75 -> 0.77   16: 0.77 -> 0.82   20: 0.72 -> 0.76
    //                 24: 0.59 -> 0.66
    // gradients: float32 l_max 16: 0.86 -> 0.90   21: 0.78 -> 0.82   26: 0.71 -> 0.75; float64 l_max 28: 0.59 -> 0.62.
    // Where a swept case is not listed (Hessians: float32 l_max = 16, 20, 24, float64 l_max = 5, 10; gradients: float32
    // l_max = 18, 20, 22, float64 l_max = 16 ... 24) the score's choice was the best measured or within 2 % of it; the
    // other degrees were not swept. For Hessians small panels of four, two or one point with about four warps per CTA
    // win: several CTAs per SM hide each other's barriers.
    // Values only, float32 l_max = 22: 16 points per panel 0.70 against 0.59 with 32.
    if (best.feasible && k.panel_batch <= 0 && k.panel_points <= 0 && k.panel_threads <= 0 && k.panel_slots <= 0) {
        struct Shape { int level, elem, l_max, batch, tp, threads; };
        static const Shape measured[] = {
            {2, 4, 11, 8, 4, 64},  {2, 4, 12, 8, 4, 128}, {2, 4, 13, 8, 4, 96},  {2, 4, 14, 8, 4, 96},  {2, 4, 15, 8, 4, 128},
            {2, 4, 17, 4, 2, 128}, {2, 4, 18, 4, 2, 128}, {2, 4, 19, 4, 2, 96},  {2, 8, 7, 16, 8, 128}, {2, 8, 13, 8, 2, 128},
            {2, 8, 15, 4, 2, 128}, {2, 8, 16, 4, 2, 128}, {2, 8, 20, 4, 1, 128}, {2, 8, 24, 2, 1, 96},
            {1, 4, 16, 16, 16, 192}, {1, 4, 21, 8, 4, 96}, {1, 4, 26, 8, 4, 192}, {1, 8, 28, 4, 2, 128},
            {0, 4, 22, 16, 16, 48}};
        for (const Shape& m : measured) {
            if (m.level != level || m.l_max != l_max || size_t(m.elem) != elem) continue;
            const size_t smem = panel_fixed_bytes(l_max, level, m.batch, elem) + panel_image_bytes(l_max, level, m.tp, elem);
            if (smem <= smem_limit) {
                best.batch = m.batch;
                best.tp = m.tp;
                best.slots = 1;
                best.threads = m.threads;
                best.smem = smem;
            }
        }
    }
    // Each CTA stages the constants once; enough table batches per CTA amortise that: at least eight,
    // and at least 256 points (measured: 8 batches per CTA 3 - 10 % faster than 4 and 15 - 25 % faster
    // than 1; l_max = 32 float64 gradients with batches of four points: 32 / 64 batches -> 0.73 / 0.80).
    best.iters = resolve_iters(k.panel_iters, std::max(8, best.batch > 0 ? (256 + best.batch - 1) / best.batch : 8));
    return best;
}

// Shape of the run-time-degree VJP kernel: points per table batch, threads per CTA (batch x slices), dynamic
// shared memory (panel_vjp_smem_bytes of sph_panel.cuh for a run-time element size), batches per CTA.
struct PanelVjpPlan {
    int batch = 0;
    int threads = 0;
    size_t smem = 0;
    int iters = 8;
    bool feasible = false;
};

size_t panel_vjp_bytes(int l_max, int batch, int threads, size_t elem) {
    const size_t nq = size_t(n_table(l_max));
    const size_t ny = size_t(n_columns(l_max));
    const size_t q = 16 / elem;
    const size_t stride = ny % 2 != 0 ? ny : ((ny / q) % 2 == 0 ? ny + q : ny);
    return (4 * nq * 8 + 15) / 16 * 16 +
           (band_align16(size_t(batch) * size_t(panel_point_state(l_max, 0)), elem) + band_align16(size_t(batch) * stride, elem) +
            band_align16(3 * size_t(threads) * q, elem)) * elem + 16;
}

// Same shape rules as the values-only forward path, whose structure the kernel shares (a thread carries
// 16 bytes' worth of points through one pair of rows): eight threads side by side where two CTAs fit an
// SM, half as many otherwise; one slice per pair of rows (j, l_max - j).
PanelVjpPlan make_panel_vjp_plan(int l_max, size_t elem, size_t smem_limit) {
    PanelVjpPlan best;
    if (l_max > PANEL_LMAX || knobs().no_panel != 0) return best;
    const int ppt = panel_values_ppt(int(elem));
    const int slices = l_max / 2 + 1;
    const bool even_rows = n_columns(l_max) % 2 == 0;
    double best_score = -1.0;
    for (int batch = 32; batch >= ppt; batch /= 2) {
        if (knobs().panel_batch > 0 && batch != knobs().panel_batch) continue;
        const int lanes = batch / ppt;
        if (even_rows && lanes > 8) continue;  // padded rows are conflict-free for eight threads side by side
        const int threads = lanes * slices;
        if (threads > 256 || threads < batch) continue;
        const size_t smem = panel_vjp_bytes(l_max, batch, threads, elem);
        if (smem > smem_limit) continue;
        const long long ctas = std::min<long long>(32, (long long)(233472 / (smem + 1024)));
        // (measured, fraction of the copy peak: float32 l_max = 24, 32 / 16 / 8 points per batch: 0.54 / 0.50 / 0.44;
        // float64 l_max = 32, 16 / 8 points: 0.50 / 0.44; float64 l_max = 24, 32 / 16 / 8 points: 0.58 / 0.62 / 0.58)
        const double score = std::sqrt(std::min(lanes, 8) / 8.0) * (ctas >= 2 ? 1.0 : 0.7) *
                             (0.85 + 0.05 * std::min<long long>(ctas, 3)) * (batch >= 16 ? 1.0 : 0.85);
        if (score > best_score + 1e-9) {
            best_score = score;
            best.batch = batch;
            best.threads = threads;
            best.smem = smem;
            best.feasible = true;
        }
    }
    best.iters = resolve_iters(knobs().panel_iters, std::max(8, best.batch > 0 ? 256 / best.batch : 8));
    return best;
}

// Descriptors of the (l, m >= 0) pairs for the panel kernels (PanelDesc in sph_panel.cuh): element
// offsets of Q_l^m, Q_{l-1}^m, Q_{l-2}^m in the triangular per-point table (rows -1 and -2 are the
// block of zeros at offset 0), and column | m << 16 | l << 24.
void make_panel_desc(int l_max, int* out) {
    auto row_start = [](int l) { return 4 + l * (l - 1) / 2 + 5 * l; };
    for (int l = 0; l <= l_max; ++l) {
        for (int m = 0; m <= l; ++m) {
            int* d = out + 4 * tri(l, m);
            d[0] = row_start(l) + m;
            d[1] = (l >= 1 ? row_start(l - 1) : 0) + m;
            d[2] = (l >= 2 ? row_start(l - 2) : 0) + m;
            d[3] = (l * l + l + m) | (m << 16) | (l << 24);
        }
    }
}

// Library-owned state of one calculator, reached through the class's prefactors_cuda slot.
template <typename T> struct CalculatorState {
    std::mutex mutex;
    BandPlan plans[5];
    bool plan_ready[5] = {false, false, false, false, false};
    PanelPlan panel_plans[3];
    bool panel_plan_ready[3] = {false, false, false};
    PanelVjpPlan panel_vjp_plan;
    bool panel_vjp_plan_ready = false;
    // device copies of the F and K tables followed (from the next 16-byte boundary) by the panel
    // kernels' pair descriptors, made on first use per device
    T* tables[MAX_DEVICES] = {};
};

template <typename T> size_t desc_offset_bytes(int l_max) { return band_align16(2 * size_t(n_table(l_max)), sizeof(T)) * sizeof(T); }

// Uploads the calculator's tables to `device` on first use (under the calculator's mutex).
template <typename T> const T* device_tables(CalculatorState<T>& st, const T* host_tables, int l_max, int device) {
    if (st.tables[device] == nullptr) {
        const size_t nq = size_t(n_table(l_max));
        const size_t desc_at = desc_offset_bytes<T>(l_max);
        const bool with_desc = l_max <= PANEL_LMAX;
        std::vector<unsigned char> staging(desc_at + (with_desc ? nq * 16 : 0), 0);
        std::memcpy(staging.data(), host_tables, 2 * nq * sizeof(T));
        if (with_desc) make_panel_desc(l_max, reinterpret_cast<int*>(staging.data() + desc_at));
        check(cudaMalloc(reinterpret_cast<void**>(&st.tables[device]), staging.size()), "cudaMalloc(prefactors)");
        check(cudaMemcpy(st.tables[device], staging.data(), staging.size(), cudaMemcpyHostToDevice), "cudaMemcpy(prefactors)");
    }
    return st.tables[device];
}

template <typename T>
void band_resources(CalculatorState<T>& st, const T* host_tables, int l_max, int kind, int device, size_t smem_limit,
                    int sm_count, const BandPlan*& plan, const T*& d_tables) {
    std::lock_guard<std::mutex> lock(st.mutex);
    if (!st.plan_ready[kind]) {
        st.plans[kind] = make_band_plan(l_max, kind, sizeof(T), smem_limit, sm_count);
        st.plan_ready[kind] = true;
    }
    plan = &st.plans[kind];
    d_tables = device_tables(st, host_tables, l_max, device);
}

template <typename T> int panel_registers(int level, bool normalized);

template <typename T>
void panel_resources(CalculatorState<T>& st, const T* host_tables, int l_max, int level, bool normalized, int device,
                     size_t smem_limit, const PanelPlan*& plan, const T*& d_tables) {
    std::lock_guard<std::mutex> lock(st.mutex);
    if (!st.panel_plan_ready[level]) {
        st.panel_plans[level] = make_panel_plan(l_max, level, sizeof(T), smem_limit, panel_registers<T>(level, normalized));
        st.panel_plan_ready[level] = true;
    }
    plan = &st.panel_plans[level];
    d_tables = plan->feasible ? device_tables(st, host_tables, l_max, device) : nullptr;
}

template <typename T>
BandLaunchArgs<T> band_launch_args(const BandPlan& plan, int l_max, const T* d_tables, const T* xyz, long long n,
                                   T* sph, T* dsph, T* ddsph, const T* sph_grad, const T* dsph_grad, T* xyz_grad) {
    BandLaunchArgs<T> a{};
    a.xyz = xyz;
    a.n = n;
    a.sph = sph;
    a.dsph = dsph;
    a.ddsph = ddsph;
    a.sph_grad = sph_grad;
    a.dsph_grad = dsph_grad;
    a.xyz_grad = xyz_grad;
    a.d_tables = d_tables;
    a.l_max = l_max;
    a.mode = plan.mode;
    a.warps = plan.warps;
    a.smem = plan.smem;
    a.grid_cap = plan.grid_cap;
    a.iters = plan.iters;
    return a;
}

// RAII: run on the device that owns `ptr`, restore the caller's device afterwards.
struct DeviceScope {
    int previous = -1;
    int device = -1;
    explicit DeviceScope(const void* ptr) {
        cudaPointerAttributes attr;
        check(cudaPointerGetAttributes(&attr, ptr), "cudaPointerGetAttributes");
        if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged) {
            throw std::runtime_error("sphericart::cuda: xyz is not a device pointer");
        }
        device = attr.device;
        check(cudaGetDevice(&previous), "cudaGetDevice");
        if (device < 0 || device >= MAX_DEVICES) throw std::runtime_error("sphericart::cuda: unsupported device index");
        if (previous != device) check(cudaSetDevice(device), "cudaSetDevice");
    }
    ~DeviceScope() {
        if (previous != device && previous >= 0) cudaSetDevice(previous);
    }
};

template <typename T> bool aligned16(const T* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, int LMAX = TILE_LMAX> struct TileDispatch {
    static size_t smem_per_warp(int l_max, int level) {
        if (l_max == LMAX) return TileLaunch<T, LMAX>::smem_per_warp(level);
        if constexpr (LMAX > 0) return TileDispatch<T, LMAX - 1>::smem_per_warp(l_max, level);
        return 0;
    }
    static cudaError_t forward(int l_max, int level, bool normalized, const T* xyz, long long n, T* sph, T* dsph,
                               T* ddsph, const T* tables, int warps, int span_tiles, bool use_bulk, int iters,
                               int tile_points, int device, cudaStream_t stream) {
        if (l_max == LMAX)
            return TileLaunch<T, LMAX>::forward(level, normalized, xyz, n, sph, dsph, ddsph, tables, warps, span_tiles,
                                                use_bulk, iters, tile_points, device, stream);
        if constexpr (LMAX > 0)
            return TileDispatch<T, LMAX - 1>::forward(l_max, level, normalized, xyz, n, sph, dsph, ddsph, tables, warps,
                                                      span_tiles, use_bulk, iters, tile_points, device, stream);
        return cudaErrorInvalidValue;
    }
    static cudaError_t vjp(int l_max, bool normalized, const T* xyz, const T* sph_grad, long long n, T* xyz_grad,
                           const T* tables, int warps, bool use_bulk, int iters, int device,
                           cudaStream_t stream) {
        if (l_max == LMAX)
            return TileLaunch<T, LMAX>::vjp(normalized, xyz, sph_grad, n, xyz_grad, tables, warps, use_bulk, iters,
                                            device, stream);
        if constexpr (LMAX > 0)
            return TileDispatch<T, LMAX - 1>::vjp(l_max, normalized, xyz, sph_grad, n, xyz_grad, tables, warps, use_bulk,
                                                  iters, device, stream);
        return cudaErrorInvalidValue;
    }
    static cudaError_t vjp2(int l_max, bool normalized, const T* xyz, const T* sph_grad, const T* dsph_grad, long long n,
                            T* xyz_grad, const T* tables, int warps, int iters, bool use_bulk, int device,
                            cudaStream_t stream) {
        if (l_max == LMAX)
            return TileLaunch<T, LMAX>::vjp2(normalized, xyz, sph_grad, dsph_grad, n, xyz_grad, tables, warps, iters,
                                             use_bulk, device, stream);
        if constexpr (LMAX > 0)
            return TileDispatch<T, LMAX - 1>::vjp2(l_max, normalized, xyz, sph_grad, dsph_grad, n, xyz_grad, tables, warps,
                                                   iters, use_bulk, device, stream);
        return cudaErrorInvalidValue;
    }
    static cudaError_t selected(int l_max, bool normalized, const T* xyz, long long n, T* out, const T* tables,
                                const Selection& selection, bool use_bulk, int device, cudaStream_t stream) {
        if (l_max == LMAX)
            return TileLaunch<T, LMAX>::selected(normalized, xyz, n, out, tables, selection, use_bulk, device, stream);
        if constexpr (LMAX > 0)
            return TileDispatch<T, LMAX - 1>::selected(l_max, normalized, xyz, n, out, tables, selection, use_bulk, device,
                                                       stream);
        return cudaErrorInvalidValue;
    }
    static cudaError_t selected_vjp(int l_max, bool normalized, const T* xyz, const T* out_grad, long long n,
                                    T* xyz_grad, const T* tables, const Selection& selection, int device,
                                    cudaStream_t stream) {
        if (l_max == LMAX)
            return TileLaunch<T, LMAX>::selected_vjp(normalized, xyz, out_grad, n, xyz_grad, tables, selection, device,
                                                     stream);
        if constexpr (LMAX > 0)
            return TileDispatch<T, LMAX - 1>::selected_vjp(l_max, normalized, xyz, out_grad, n, xyz_grad, tables,
                                                           selection, device, stream);
        return cudaErrorInvalidValue;
    }
    static int error_flags() {
        int flag = TileLaunch<T, LMAX>::device_error_flag();
        if constexpr (LMAX > 0) {
            const int rest = TileDispatch<T, LMAX - 1>::error_flags();
            flag = (flag < 0 || rest < 0) ? -1 : (flag | rest);
        }
        return flag;
    }
};

// Registers per thread of the panel kernels (they barely depend on the batch size; 8 is queried).
template <typename T> int panel_registers(int level, bool normalized) { return PanelLaunch<T, 8>::registers(level, normalized); }

template <typename T>
cudaError_t panel_dispatch(int tp, int level, bool normalized, const PanelLaunchArgs<T>& a, int device, cudaStream_t stream) {
    switch (tp) {
        case 1: return PanelLaunch<T, 1>::run(level, normalized, a, device, stream);
        case 2: return PanelLaunch<T, 2>::run(level, normalized, a, device, stream);
        case 4: return PanelLaunch<T, 4>::run(level, normalized, a, device, stream);
        case 8: return PanelLaunch<T, 8>::run(level, normalized, a, device, stream);
        case 16: return PanelLaunch<T, 16>::run(level, normalized, a, device, stream);
        case 32: return PanelLaunch<T, 32>::run(level, normalized, a, device, stream);
        default: return cudaErrorInvalidValue;
    }
}

template <typename T>
cudaError_t panel_vjp_dispatch(int batch, bool normalized, const PanelVjpLaunchArgs<T>& a, int device, cudaStream_t stream) {
    switch (batch) {
        case 2: return PanelLaunch<T, 2>::run_vjp(normalized, a, device, stream);
        case 4: return PanelLaunch<T, 4>::run_vjp(normalized, a, device, stream);
        case 8: return PanelLaunch<T, 8>::run_vjp(normalized, a, device, stream);
        case 16: return PanelLaunch<T, 16>::run_vjp(normalized, a, device, stream);
        case 32: return PanelLaunch<T, 32>::run_vjp(normalized, a, device, stream);
        default: return cudaErrorInvalidValue;
    }
}

template <typename T> int panel_error_flags() {
    const int flags[6] = {PanelLaunch<T, 1>::device_error_flag(), PanelLaunch<T, 2>::device_error_flag(),
                          PanelLaunch<T, 4>::device_error_flag(), PanelLaunch<T, 8>::device_error_flag(),
                          PanelLaunch<T, 16>::device_error_flag(), PanelLaunch<T, 32>::device_error_flag()};
    int all = 0;
    for (int f : flags) {
        if (f < 0) return -1;
        all |= f;
    }
    return all;
}

template <typename T>
cudaError_t band_dispatch(int lanes, int level, bool vjp, bool normalized, const BandLaunchArgs<T>& a, int device,
                          cudaStream_t stream) {
    switch (lanes) {
        case 1: return BandLaunch<T, 1>::run(level, vjp, normalized, a, device, stream);
        case 2: return BandLaunch<T, 2>::run(level, vjp, normalized, a, device, stream);
        case 4: return BandLaunch<T, 4>::run(level, vjp, normalized, a, device, stream);
        case 8: return BandLaunch<T, 8>::run(level, vjp, normalized, a, device, stream);
        case 16: return BandLaunch<T, 16>::run(level, vjp, normalized, a, device, stream);
        case 32: return BandLaunch<T, 32>::run(level, vjp, normalized, a, device, stream);
        default: return cudaErrorInvalidValue;
    }
}

// Tile images in flight per CTA of a persistent launch. What matters most is the number of images
// an SM can hold (each one is a tile being drained while others are computed); among the choices
// that reach the maximum, the largest CTA of at most five warps spreads the warps over the SM's
// schedulers.
int tile_warps(size_t smem_per_warp, size_t smem_limit) {
    if (smem_per_warp == 0) return 4;
    const int forced = knobs().tile_warps;
    int best = 1;
    size_t best_slots = 0;
    for (int w = 1; w <= 8; ++w) {
        const size_t cta = w * smem_per_warp;
        if (cta > smem_limit) break;
        size_t n_cta = (smem_limit + 1024) / (cta + 1024);
        n_cta = std::min<size_t>(n_cta, 32);
        const size_t slots = std::min<size_t>(64, n_cta * w);
        if (forced == w) return w;
        if (slots > best_slots || (slots == best_slots && w <= 5)) {
            best_slots = slots;
            best = w;
        }
    }
    return best;
}

// kind 0..2: forward level; 3: VJP of the values; 4: VJP of (values, gradients).
template <typename T>
void run(size_t l_max_, bool normalized, const T* host_tables, CalculatorState<T>& st, int kind, const T* xyz,
         size_t n_samples, T* sph, T* dsph, T* ddsph, const T* sph_grad, const T* dsph_grad, T* xyz_grad,
         void* cuda_stream) {
    const int l_max = int(l_max_);
    const long long n = (long long)n_samples;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    DeviceScope scope(xyz);
    const DeviceProps& props = device_props(scope.device);
    const bool vjp = kind >= 3;
    const bool force_band = knobs().force_band != 0;

    if (tile_serves(kind, l_max, int(sizeof(T))) && l_max <= knobs().tile_lmax && !force_band) {
        if (kind == 4) {
            const size_t vjp2_per_warp =
                size_t(32) * (4 * n_columns(l_max) + 2 * tile_row_pad(n_columns(l_max), int(sizeof(T)))) * sizeof(T) + 16;
            const bool use_bulk = knobs().no_bulk == 0 && aligned16(dsph_grad) && (sph_grad == nullptr || aligned16(sph_grad));
            check(TileDispatch<T>::vjp2(l_max, normalized, xyz, sph_grad, dsph_grad, n, xyz_grad, host_tables,
                                        tile_warps(vjp2_per_warp, props.smem_optin), resolve_iters(knobs().vjp_iters, 4),
                                        use_bulk, scope.device, stream),
                  "tile second-order VJP kernel launch");
            return;
        }
        // VJP: one image of upstream rows per warp (plus its mbarrier)
        const size_t vjp_image = size_t(32) * (n_columns(l_max) + tile_row_pad(n_columns(l_max), int(sizeof(T)))) * sizeof(T);
        const size_t per_warp = kind == 3 ? vjp_image + 16 : TileDispatch<T>::smem_per_warp(l_max, kind < 3 ? kind : 2);
        if (kind == 3) {
            const bool use_bulk = aligned16(sph_grad) && knobs().no_bulk == 0;
            // short-lived CTAs of four warps, one tile per warp
            const int iters = resolve_iters(knobs().vjp_iters, 1);
            int warps = tile_warps(per_warp, props.smem_optin);
            if (iters > 0 && knobs().tile_warps == 0) {
                // short-lived CTAs of up to four warps: the count that lets an SM hold the most warps (an
                // SM has 228 KB of shared memory, 1 KB reserved per CTA), the larger CTA on a tie. With long
                // rows this matters: at l_max = 16 float32 (37 KB per warp) CTAs of four warps fit once per
                // SM, CTAs of three or two warps give six warps per SM.
                size_t best = 0;
                for (int w = 1; w <= 4; ++w) {
                    if (w * per_warp > props.smem_optin) break;
                    const size_t resident = std::min<size_t>(32, size_t(233472) / (w * per_warp + 1024)) * w;
                    if (resident >= best) {
                        best = resident;
                        warps = w;
                    }
                }
            }
            check(TileDispatch<T>::vjp(l_max, normalized, xyz, sph_grad, n, xyz_grad, host_tables, warps, use_bulk,
                                       iters, scope.device, stream),
                  "tile VJP kernel launch");
            return;
        }
        if (kind < 3) {
            bool use_bulk = aligned16(sph) && (kind < 1 || aligned16(dsph)) && (kind < 2 || aligned16(ddsph));
            if (knobs().no_bulk != 0) use_bulk = false;
            // One warp and one image per short-lived CTA: a CTA's shared memory is released as soon
            // as its own image has been read by the TMA engine, and the block scheduler keeps every
            // SM as full as its shared memory allows (l_max = 8 float32 gradients: five images).
            const int iters = resolve_iters(knobs().tile_iters, 1);
            // tiles per image: small tiles are grouped so that each bulk store moves about 8 KB or more
            // (12 KB for a persistent launch)
            const size_t store_bytes = iters > 0 ? 8 * 1024 : 12 * 1024;
            int span_tiles = int(std::min<size_t>(8, std::max<size_t>(1, (store_bytes + per_warp - 1) / per_warp)));
            while (span_tiles > 1 && span_tiles * per_warp > props.smem_optin) --span_tiles;
            int warps = tile_warps(span_tiles * per_warp, props.smem_optin);
            if (iters > 0 && knobs().tile_warps == 0) warps = 1;
            int tile_points = knobs().tile_points;
            if (tile_points != 8 && tile_points != 16 && tile_points != 32) tile_points = 0;
            check(TileDispatch<T>::forward(l_max, kind, normalized, xyz, n, sph, dsph, ddsph, host_tables, warps,
                                           span_tiles, use_bulk, iters, tile_points, scope.device, stream),
                  "tile kernel launch");
            return;
        }
    }

    if (kind <= 2 && knobs().no_panel == 0 && !force_band) {
        const PanelPlan* pplan = nullptr;
        const T* d_tables = nullptr;
        panel_resources(st, host_tables, l_max, kind, normalized, scope.device, props.smem_optin, pplan, d_tables);
        if (pplan->feasible) {
            PanelLaunchArgs<T> a{};
            a.xyz = xyz;
            a.n = n;
            a.sph = sph;
            a.dsph = dsph;
            a.ddsph = ddsph;
            a.d_tables = d_tables;
            a.d_desc = reinterpret_cast<const unsigned char*>(d_tables) + desc_offset_bytes<T>(l_max);
            a.l_max = l_max;
            // bulk copy-out: rows of odd length go out as one span per array from an image placed at the
            // span's own alignment; rows of even length go out point by point and need 16-byte aligned arrays
            const bool aligned_out = aligned16(sph) && (kind < 1 || aligned16(dsph)) && (kind < 2 || aligned16(ddsph));
            a.bulk = (knobs().no_bulk != 0 || (n_columns(l_max) % 2 == 0 && !aligned_out)) ? 0 : 1;
            a.tp = pplan->tp;
            a.slots = pplan->slots;
            a.tables_f64 = knobs().panel_tables_f64;
            a.threads = pplan->threads;
            a.smem = pplan->smem;
            a.iters = pplan->iters;
            check(panel_dispatch<T>(pplan->batch, kind, normalized, a, scope.device, stream), "panel kernel launch");
            return;
        }
    }

    if (kind == 3 && knobs().no_panel == 0 && !force_band) {
        const PanelVjpPlan* vplan = nullptr;
        const T* d_tables = nullptr;
        {
            std::lock_guard<std::mutex> lock(st.mutex);
            if (!st.panel_vjp_plan_ready) {
                st.panel_vjp_plan = make_panel_vjp_plan(l_max, sizeof(T), props.smem_optin);
                st.panel_vjp_plan_ready = true;
            }
            vplan = &st.panel_vjp_plan;
            if (vplan->feasible) d_tables = device_tables(st, host_tables, l_max, scope.device);
        }
        if (vplan->feasible) {
            PanelVjpLaunchArgs<T> a{};
            a.xyz = xyz;
            a.sph_grad = sph_grad;
            a.n = n;
            a.xyz_grad = xyz_grad;
            a.d_tables = d_tables;
            a.l_max = l_max;
            a.bulk = (aligned16(sph_grad) && knobs().no_bulk == 0) ? 1 : 0;
            a.threads = vplan->threads;
            a.smem = vplan->smem;
            a.iters = vplan->iters;
            check(panel_vjp_dispatch<T>(vplan->batch, normalized, a, scope.device, stream), "panel VJP kernel launch");
            return;
        }
    }

    const BandPlan* plan = nullptr;
    const T* d_tables = nullptr;
    band_resources(st, host_tables, l_max, kind, scope.device, props.smem_optin, props.sm_count, plan, d_tables);
    if (!plan->feasible) {
        throw std::runtime_error("sphericart::cuda: l_max is too large for this device's shared memory");
    }
    const BandLaunchArgs<T> a =
        band_launch_args<T>(*plan, l_max, d_tables, xyz, n, sph, dsph, ddsph, sph_grad, dsph_grad, xyz_grad);
    check(band_dispatch<T>(plan->lanes, kind == 3 ? 1 : (kind == 4 ? 2 : kind), vjp, normalized, a, scope.device, stream),
          "band kernel launch");
}

// Selected degree blocks (values when out_grad is null, the fused VJP otherwise).
template <typename T>
void run_selected(size_t l_max_, bool normalized, const T* host_tables, const T* xyz, size_t n_samples,
                  const int* l_list, size_t n_l, const int* axis_order, const T* scales, T* out, const T* out_grad,
                  T* xyz_grad, void* cuda_stream) {
    const int l_max = int(l_max_);
    if (l_max > TILE_LMAX) {
        throw std::runtime_error("sphericart::cuda: selected outputs are served for l_max <= " + std::to_string(TILE_LMAX) +
                                 "; got l_max = " + std::to_string(l_max));
    }
    if (l_list == nullptr || n_l == 0) throw std::runtime_error("sphericart::cuda: l_list is empty");
    Selection sel{};
    for (int l = 0; l <= TILE_LMAX; ++l) {
        sel.dest[l] = -1;
        sel.scale[l] = 1.0;
    }
    int column = 0;
    for (size_t j = 0; j < n_l; ++j) {
        const int l = l_list[j];
        if (l < 0 || l > l_max) {
            throw std::runtime_error("sphericart::cuda: l_list holds " + std::to_string(l) +
                                     ", outside 0 ... l_max = " + std::to_string(l_max));
        }
        if (sel.dest[l] >= 0) throw std::runtime_error("sphericart::cuda: l_list holds " + std::to_string(l) + " twice");
        sel.dest[l] = column;
        sel.scale[l] = scales != nullptr ? double(scales[j]) : 1.0;
        column += 2 * l + 1;
    }
    sel.ny_out = column;
    for (int a = 0; a < 3; ++a) sel.axis[a] = axis_order != nullptr ? axis_order[a] : a;
    const bool permutation = ((1 << sel.axis[0]) | (1 << sel.axis[1]) | (1 << sel.axis[2])) == 7 && sel.axis[0] >= 0 &&
                             sel.axis[1] >= 0 && sel.axis[2] >= 0 && sel.axis[0] <= 2 && sel.axis[1] <= 2 && sel.axis[2] <= 2;
    if (!permutation) throw std::runtime_error("sphericart::cuda: axis_order must be a permutation of 0, 1, 2");
    if (n_samples == 0) return;
    if (xyz == nullptr) throw std::runtime_error("sphericart::cuda: xyz is a null pointer");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    DeviceScope scope(xyz);
    if (out_grad == nullptr) {
        if (out == nullptr) throw std::runtime_error("sphericart::cuda: out is a null pointer");
        check(TileDispatch<T>::selected(l_max, normalized, xyz, (long long)n_samples, out, host_tables, sel,
                                        aligned16(out) && knobs().no_bulk == 0, scope.device, stream),
              "selected kernel launch");
    } else {
        if (xyz_grad == nullptr) throw std::runtime_error("sphericart::cuda: xyz_grad is a null pointer");
        check(TileDispatch<T>::selected_vjp(l_max, normalized, xyz, out_grad, (long long)n_samples, xyz_grad, host_tables,
                                            sel, scope.device, stream),
              "selected VJP kernel launch");
    }
}

// The kernel family run() picks for a call of this kind; mirrors the order of the tests in run().
const char* kernel_family(int kind, int l_max, int elem_bytes, size_t smem_limit) {
    const bool force_band = knobs().force_band != 0;
    if (tile_serves(kind, l_max, elem_bytes) && l_max <= knobs().tile_lmax && !force_band) {
        return kind == 3 ? "sph_vjp_tile_kernel" : (kind == 4 ? "sph_vjp2_tile_kernel" : "sph_tile_kernel");
    }
    if (kind <= 2 && knobs().no_panel == 0 && !force_band &&
        make_panel_plan(l_max, kind, size_t(elem_bytes), smem_limit, 0).feasible) {
        return "sph_panel_kernel";
    }
    if (kind == 3 && !force_band && make_panel_vjp_plan(l_max, size_t(elem_bytes), smem_limit).feasible) {
        return "sph_panel_vjp_kernel";
    }
    return "sph_band_kernel";
}

}  // namespace sph_b200

// ---------------------------------------------------------------------------------------------
namespace sphericart {
namespace cuda {

using sph_b200::CalculatorState;

template <typename T> static CalculatorState<T>* state_of(T* slot) { return reinterpret_cast<CalculatorState<T>*>(slot); }

template <typename T> SphericalHarmonics<T>::SphericalHarmonics(size_t l_max) {
    this->l_max = l_max;
    this->nprefactors = (l_max + 1) * (l_max + 2);
    this->normalized = true;
    int count = 0;
    cudaError_t status = cudaGetDeviceCount(&count);
    if (status != cudaSuccess || count <= 0) {
        cudaGetLastError();
        throw std::runtime_error(
            std::string("sphericart::cuda: no usable CUDA device (") + cudaGetErrorString(status) +
            "); this library has no CPU code path"
        );
    }
    this->device_count = count;
    this->prefactors_cpu = new T[this->nprefactors];
    sph_b200::build_tables<T>(int(l_max), this->prefactors_cpu);
    this->prefactors_cuda = reinterpret_cast<T*>(new CalculatorState<T>());
}

template <typename T> SphericalHarmonics<T>::~SphericalHarmonics() {
    delete[] this->prefactors_cpu;
    this->prefactors_cpu = nullptr;
    // Device tables are left to the driver at process exit, as the reference does
    // (sphericart/src/sphericart_cuda.cpp:60-72): calculators often die during static
    // destruction, after the CUDA runtime has shut down.
    delete state_of<T>(this->prefactors_cuda);
    this->prefactors_cuda = nullptr;
}

template <typename T>
void SphericalHarmonics<T>::compute_internal(
    const T* xyz,
    const size_t n_samples,
    bool compute_with_gradients,
    bool compute_with_hessian,
    T* sph,
    T* dsph,
    T* ddsph,
    void* cuda_stream
) {
    if (n_samples == 0) return;  // callers may hold null pointers for empty arrays
    if (xyz == nullptr) throw std::runtime_error("sphericart::cuda: xyz is a null pointer");
    if (sph == nullptr) throw std::runtime_error("sphericart::cuda: sph is a null pointer; allocate it on the device");
    if (compute_with_gradients && dsph == nullptr)
        throw std::runtime_error("sphericart::cuda: gradients were requested but dsph is a null pointer");
    if (compute_with_hessian && ddsph == nullptr)
        throw std::runtime_error("sphericart::cuda: Hessians were requested but ddsph is a null pointer");
    const int level = compute_with_hessian ? 2 : (compute_with_gradients ? 1 : 0);
    sph_b200::run<T>(this->l_max, this->normalized, this->prefactors_cpu, *state_of<T>(this->prefactors_cuda), level, xyz,
                     n_samples, sph, dsph, ddsph, nullptr, nullptr, nullptr, cuda_stream);
}

template <typename T>
void SphericalHarmonics<T>::compute(const T* xyz, const size_t n_samples, T* sph, void* cuda_stream) {
    compute_internal(xyz, n_samples, false, false, sph, nullptr, nullptr, cuda_stream);
}

template <typename T>
void SphericalHarmonics<T>::compute_with_gradients(const T* xyz, const size_t n_samples, T* sph, T* dsph, void* cuda_stream) {
    compute_internal(xyz, n_samples, true, false, sph, dsph, nullptr, cuda_stream);
}

template <typename T>
void SphericalHarmonics<T>::compute_with_hessians(
    const T* xyz, const size_t n_samples, T* sph, T* dsph, T* ddsph, void* cuda_stream
) {
    compute_internal(xyz, n_samples, true, true, sph, dsph, ddsph, cuda_stream);
}

template <typename T>
void SphericalHarmonics<T>::compute_vjp(
    const T* xyz, const size_t n_samples, const T* sph_grad, T* xyz_grad, void* cuda_stream
) {
    if (n_samples == 0) return;
    if (xyz == nullptr) throw std::runtime_error("sphericart::cuda: xyz is a null pointer");
    if (sph_grad == nullptr) throw std::runtime_error("sphericart::cuda: sph_grad is a null pointer");
    if (xyz_grad == nullptr) throw std::runtime_error("sphericart::cuda: xyz_grad is a null pointer");
    sph_b200::run<T>(this->l_max, this->normalized, this->prefactors_cpu, *state_of<T>(this->prefactors_cuda), 3, xyz,
                     n_samples, nullptr, nullptr, nullptr, sph_grad, nullptr, xyz_grad, cuda_stream);
}

template <typename T>
void SphericalHarmonics<T>::compute_vjp_with_gradients(
    const T* xyz, const size_t n_samples, const T* sph_grad, const T* dsph_grad, T* xyz_grad, void* cuda_stream
) {
    if (n_samples == 0) return;
    if (xyz == nullptr) throw std::runtime_error("sphericart::cuda: xyz is a null pointer");
    if (dsph_grad == nullptr) throw std::runtime_error("sphericart::cuda: dsph_grad is a null pointer");
    if (xyz_grad == nullptr) throw std::runtime_error("sphericart::cuda: xyz_grad is a null pointer");
    sph_b200::run<T>(this->l_max, this->normalized, this->prefactors_cpu, *state_of<T>(this->prefactors_cuda), 4, xyz,
                     n_samples, nullptr, nullptr, nullptr, sph_grad, dsph_grad, xyz_grad, cuda_stream);
}

template <typename T>
void SphericalHarmonics<T>::compute_selected(
    const T* xyz, const size_t n_samples, const int* l_list, const size_t n_l, const int* axis_order, const T* scales,
    T* out, void* cuda_stream
) {
    sph_b200::run_selected<T>(this->l_max, this->normalized, this->prefactors_cpu, xyz, n_samples, l_list, n_l, axis_order,
                              scales, out, nullptr, nullptr, cuda_stream);
}

template <typename T>
void SphericalHarmonics<T>::compute_selected_vjp(
    const T* xyz, const size_t n_samples, const int* l_list, const size_t n_l, const int* axis_order, const T* scales,
    const T* out_grad, T* xyz_grad, void* cuda_stream
) {
    if (n_samples != 0 && out_grad == nullptr) throw std::runtime_error("sphericart::cuda: out_grad is a null pointer");
    sph_b200::run_selected<T>(this->l_max, this->normalized, this->prefactors_cpu, xyz, n_samples, l_list, n_l, axis_order,
                              scales, nullptr, out_grad, xyz_grad, cuda_stream);
}

template <typename T> SolidHarmonics<T>::SolidHarmonics(size_t l_max) : SphericalHarmonics<T>(l_max) {
    this->normalized = false;
}

// exported: the reference's torch and JAX bindings link against these C++ symbols directly
template class __attribute__((visibility("default"))) SphericalHarmonics<float>;
template class __attribute__((visibility("default"))) SphericalHarmonics<double>;
template class __attribute__((visibility("default"))) SolidHarmonics<float>;
template class __attribute__((visibility("default"))) SolidHarmonics<double>;

}  // namespace cuda
}  // namespace sphericart

// ---------------------------------------------------------------------------------------------
// C ABI
namespace {

thread_local std::string g_last_error;

template <typename Calculator> Calculator* capi_new(size_t l_max) {
    try {
        return new Calculator(l_max);
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return nullptr;
    } catch (...) {
        g_last_error = "unknown exception";
        return nullptr;
    }
}

template <typename Calculator> void capi_delete(Calculator* calculator) {
    try {
        delete calculator;
    } catch (...) {
    }
}

// Reference convention for compute calls: report and abort (sphericart/src/sphericart-capi.cpp:653-696).
template <typename Fn> void capi_or_abort(Fn&& fn) {
    try {
        fn();
    } catch (const std::exception& e) {
        std::printf("fatal error: %s\n", e.what());
        std::fflush(stdout);
        std::abort();
    } catch (...) {
        std::printf("fatal error: unknown exception type\n");
        std::fflush(stdout);
        std::abort();
    }
}

template <typename Fn> int capi_try(Fn&& fn) {
    try {
        fn();
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return 1;
    } catch (...) {
        g_last_error = "unknown exception";
        return 1;
    }
}

template <typename Calculator, typename T>
void level_call(Calculator* c, int level, const T* xyz, size_t n, T* sph, T* dsph, T* ddsph, void* stream) {
    if (c == nullptr) throw std::runtime_error("sphericart::cuda: calculator is a null pointer");
    switch (level) {
        case 0: c->compute(xyz, n, sph, stream); break;
        case 1: c->compute_with_gradients(xyz, n, sph, dsph, stream); break;
        case 2: c->compute_with_hessians(xyz, n, sph, dsph, ddsph, stream); break;
        default: throw std::runtime_error("sphericart::cuda: level must be 0, 1 or 2");
    }
}

template <typename Calculator, typename T>
void vjp2_call(Calculator* c, const T* xyz, size_t n, const T* sph_grad, const T* dsph_grad, T* xyz_grad, void* stream) {
    if (c == nullptr) throw std::runtime_error("sphericart::cuda: calculator is a null pointer");
    c->compute_vjp_with_gradients(xyz, n, sph_grad, dsph_grad, xyz_grad, stream);
}

template <typename Calculator, typename T>
void vjp_call(Calculator* c, const T* xyz, size_t n, const T* sph_grad, T* xyz_grad, void* stream) {
    if (c == nullptr) throw std::runtime_error("sphericart::cuda: calculator is a null pointer");
    c->compute_vjp(xyz, n, sph_grad, xyz_grad, stream);
}

}  // namespace

extern "C" const char* sphericart_cuda_last_error(void) { return g_last_error.c_str(); }

extern "C" const char* sphericart_cuda_kernel_family(int kind, size_t l_max, int elem_bytes) {
    if (kind < 0 || kind > 4 || (elem_bytes != 4 && elem_bytes != 8)) return "";
    // the largest dynamic shared memory a CTA may ask for on sm_100 (227 KB); the planning rule needs it
    return sph_b200::kernel_family(kind, int(l_max), elem_bytes, size_t(232448));
}

extern "C" int sphericart_cuda_device_wait_errors(void) {
    const int f = sph_b200::TileDispatch<float>::error_flags();
    const int d = sph_b200::TileDispatch<double>::error_flags();
    const int pf = sph_b200::panel_error_flags<float>();
    const int pd = sph_b200::panel_error_flags<double>();
    return (f < 0 || d < 0 || pf < 0 || pd < 0) ? -1 : (f | d | pf | pd);
}

#define SPH_CAPI_FAMILY(KIND, SFX, T)                                                                               \
    extern "C" sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* sphericart_cuda_##KIND##_harmonics_new##SFX( \
        size_t l_max) {                                                                                             \
        return capi_new<sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t>(l_max);                             \
    }                                                                                                               \
    extern "C" void sphericart_cuda_##KIND##_harmonics_delete##SFX(                                                 \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator) {                                       \
        capi_delete(calculator);                                                                                    \
    }                                                                                                               \
    extern "C" void sphericart_cuda_##KIND##_harmonics_compute_array##SFX(                                          \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples, T* sph, \
        void* cuda_stream) {                                                                                        \
        capi_or_abort([&] { level_call(calculator, 0, xyz, n_samples, sph, (T*)nullptr, (T*)nullptr, cuda_stream); }); \
    }                                                                                                               \
    extern "C" void sphericart_cuda_##KIND##_harmonics_compute_array_with_gradients##SFX(                           \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples, T* sph, \
        T* dsph, void* cuda_stream) {                                                                               \
        capi_or_abort([&] { level_call(calculator, 1, xyz, n_samples, sph, dsph, (T*)nullptr, cuda_stream); });     \
    }                                                                                                               \
    extern "C" void sphericart_cuda_##KIND##_harmonics_compute_array_with_hessians##SFX(                            \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples, T* sph, \
        T* dsph, T* ddsph, void* cuda_stream) {                                                                     \
        capi_or_abort([&] { level_call(calculator, 2, xyz, n_samples, sph, dsph, ddsph, cuda_stream); });           \
    }                                                                                                               \
    extern "C" void sphericart_cuda_##KIND##_harmonics_compute_vjp##SFX(                                            \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples,         \
        const T* sph_grad, T* xyz_grad, void* cuda_stream) {                                                        \
        capi_or_abort([&] { vjp_call(calculator, xyz, n_samples, sph_grad, xyz_grad, cuda_stream); });              \
    }                                                                                                               \
    extern "C" int sphericart_cuda_##KIND##_harmonics_try_compute##SFX(                                             \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, int level, const T* xyz,                \
        size_t n_samples, T* sph, T* dsph, T* ddsph, void* cuda_stream) {                                           \
        return capi_try([&] { level_call(calculator, level, xyz, n_samples, sph, dsph, ddsph, cuda_stream); });     \
    }                                                                                                               \
    extern "C" int sphericart_cuda_##KIND##_harmonics_try_compute_vjp##SFX(                                         \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples,         \
        const T* sph_grad, T* xyz_grad, void* cuda_stream) {                                                        \
        return capi_try([&] { vjp_call(calculator, xyz, n_samples, sph_grad, xyz_grad, cuda_stream); });            \
    }

#define SPH_CAPI_VJP2(KIND, SFX, T)                                                                                  \
    extern "C" void sphericart_cuda_##KIND##_harmonics_compute_vjp_with_gradients##SFX(                             \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples,         \
        const T* sph_grad, const T* dsph_grad, T* xyz_grad, void* cuda_stream) {                                    \
        capi_or_abort([&] { vjp2_call(calculator, xyz, n_samples, sph_grad, dsph_grad, xyz_grad, cuda_stream); });   \
    }                                                                                                               \
    extern "C" int sphericart_cuda_##KIND##_harmonics_try_compute_vjp_with_gradients##SFX(                          \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples,         \
        const T* sph_grad, const T* dsph_grad, T* xyz_grad, void* cuda_stream) {                                    \
        return capi_try([&] { vjp2_call(calculator, xyz, n_samples, sph_grad, dsph_grad, xyz_grad, cuda_stream); }); \
    }

#define SPH_CAPI_SELECTED(KIND, SFX, T)                                                                              \
    extern "C" int sphericart_cuda_##KIND##_harmonics_compute_selected##SFX(                                        \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples,         \
        const int* l_list, size_t n_l, const int* axis_order, const T* scales, T* out, void* cuda_stream) {         \
        return capi_try([&] {                                                                                       \
            if (calculator == nullptr) throw std::runtime_error("sphericart::cuda: calculator is a null pointer");  \
            calculator->compute_selected(xyz, n_samples, l_list, n_l, axis_order, scales, out, cuda_stream);        \
        });                                                                                                         \
    }                                                                                                               \
    extern "C" int sphericart_cuda_##KIND##_harmonics_compute_selected_vjp##SFX(                                    \
        sphericart_cuda_##KIND##_harmonics_calculator##SFX##_t* calculator, const T* xyz, size_t n_samples,         \
        const int* l_list, size_t n_l, const int* axis_order, const T* scales, const T* out_grad, T* xyz_grad,      \
        void* cuda_stream) {                                                                                        \
        return capi_try([&] {                                                                                       \
            if (calculator == nullptr) throw std::runtime_error("sphericart::cuda: calculator is a null pointer");  \
            calculator->compute_selected_vjp(xyz, n_samples, l_list, n_l, axis_order, scales, out_grad, xyz_grad,   \
                                             cuda_stream);                                                          \
        });                                                                                                         \
    }

SPH_CAPI_SELECTED(spherical, , double)
SPH_CAPI_SELECTED(spherical, _f, float)
SPH_CAPI_SELECTED(solid, , double)
SPH_CAPI_SELECTED(solid, _f, float)
#undef SPH_CAPI_SELECTED

SPH_CAPI_FAMILY(spherical, , double)
SPH_CAPI_FAMILY(spherical, _f, float)
SPH_CAPI_FAMILY(solid, , double)
SPH_CAPI_FAMILY(solid, _f, float)

SPH_CAPI_VJP2(spherical, , double)
SPH_CAPI_VJP2(spherical, _f, float)
SPH_CAPI_VJP2(solid, , double)
SPH_CAPI_VJP2(solid, _f, float)

#undef SPH_CAPI_FAMILY
#undef SPH_CAPI_VJP2

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point (an addition; the reference has nothing like it).
//
// Who needs it: hosts that hand a plugin its input and output buffers but do not let it take
// device memory of its own. Examples are runtimes that reserve the whole device arena when the
// process starts, so a later cudaMalloc from a plugin simply fails, and latency-bound service
// loops in which cudaMalloc is off limits because it synchronises the device and may block. The
// calculators above cannot serve such hosts whenever a call goes to their run-time-degree kernel
// (values and gradients: l_max > 10), which reads the prefactor tables from a device buffer that
// they cudaMalloc on first use.
//
// This variant runs the same kernel (float64, values + gradients, run-time l_max) with those
// tables placed in a fixed array that is part of the library image, so every GPU
// that loads the library carries NO_ALLOC_SCRATCH_BYTES (16 KiB) of it until the process ends. The
// function calls no cudaMalloc, cudaFree or any other allocating routine; the caller passes inputs
// and outputs as usual. The fixed size bounds the degree: l_max <= NO_ALLOC_MAX_L (32).
//
// In host code the array's name below is only a host-side stand-in for the device object: it is
// not an address a kernel may be given. The real device address is looked up once per device, with
// that device current, by cudaGetSymbolAddress, and that address is what the kernel receives.
// That look-up (plus the kernel's shared-memory opt-in) happens in the first call made on each
// device, so make that first call before any stream capture begins.
//
// All calls on one device share the one array, and it keeps what the last call left in it. A call
// overwrites, on the caller's stream, every byte the kernel will read unless the array already holds
// the data for the same l_max (nothing in it has to start at zero, nothing is read before it is
// written); so besides the first call on a device, every call whose l_max differs from the previous
// call's enqueues a small host-to-device copy in front of the kernel. The host side of that copy is
// a table the library keeps for the life of the process. A call made while its stream is being
// captured always records the copy with the kernel (the recorded work is then complete whatever the
// array holds when it is replayed), and from then on calls on that device no longer skip the copy.
// Calls that may overlap on the GPU - different streams with no ordering between them - race on the
// array; order such calls.
namespace {

constexpr int NO_ALLOC_MAX_L = 32;
constexpr size_t NO_ALLOC_SCRATCH_BYTES = 16384;  // holds 2 * n_table(32) doubles = 8976 bytes

static __device__ __align__(256) unsigned char g_no_alloc_scratch[NO_ALLOC_SCRATCH_BYTES];

struct NoAllocDevice {
    unsigned char* scratch = nullptr;  // device address of g_no_alloc_scratch on this device
    int resident_l_max = -1;           // whose tables the array holds now
    bool always_upload = false;        // a recorded (captured) call may rewrite the array at any time
};
std::mutex g_no_alloc_mutex;
NoAllocDevice g_no_alloc_devices[sph_b200::MAX_DEVICES];
// host tables per degree, built on first use and kept until the process ends: an asynchronous or
// recorded copy may read them long after the call that enqueued it has returned
std::vector<double> g_no_alloc_host_tables[NO_ALLOC_MAX_L + 1];

void no_alloc_run(bool normalized, size_t l_max_, const double* xyz, size_t n_samples, double* sph, double* dsph,
                  void* cuda_stream) {
    using namespace sph_b200;
    if (n_samples == 0) return;
    if (l_max_ > size_t(NO_ALLOC_MAX_L)) {
        throw std::runtime_error("sphericart::cuda: the allocation-free entry point supports l_max <= 32 (its fixed "
                                 "16 KiB device array cannot hold larger tables); got l_max = " + std::to_string(l_max_));
    }
    if (xyz == nullptr || sph == nullptr || dsph == nullptr) {
        throw std::runtime_error("sphericart::cuda: xyz, sph and dsph must be device pointers, got a null pointer");
    }
    const int l_max = int(l_max_);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    DeviceScope scope(xyz);
    const DeviceProps& props = device_props(scope.device);

    const BandPlan plan = make_band_plan(l_max, /*kind=*/1, sizeof(double), props.smem_optin, props.sm_count);
    const size_t table_bytes = 2 * size_t(n_table(l_max)) * sizeof(double);
    if (table_bytes > NO_ALLOC_SCRATCH_BYTES || !plan.feasible) {
        throw std::runtime_error("sphericart::cuda: internal tables do not fit the allocation-free array");
    }

    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    std::vector<double>& tables = g_no_alloc_host_tables[l_max];  // host heap only
    if (tables.empty()) {
        tables.resize(2 * size_t(n_table(l_max)));
        build_tables<double>(l_max, tables.data());
    }
    NoAllocDevice& dev = g_no_alloc_devices[scope.device];
    if (dev.scratch == nullptr) {
        // once per device, with that device current (DeviceScope made it so)
        void* address = nullptr;
        check(cudaGetSymbolAddress(&address, g_no_alloc_scratch), "cudaGetSymbolAddress(no-alloc array)");
        dev.scratch = static_cast<unsigned char*>(address);
    }
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    check(cudaStreamIsCapturing(stream, &capture), "cudaStreamIsCapturing");
    const bool capturing = capture != cudaStreamCaptureStatusNone;
    if (capturing) dev.always_upload = true;
    if (capturing || dev.always_upload || dev.resident_l_max != l_max) {
        check(cudaMemcpyAsync(dev.scratch, tables.data(), table_bytes, cudaMemcpyHostToDevice, stream),
              "cudaMemcpyAsync(tables)");
        dev.resident_l_max = l_max;
    }
    const BandLaunchArgs<double> a =
        band_launch_args<double>(plan, l_max, reinterpret_cast<const double*>(dev.scratch), xyz,
                                 (long long)n_samples, sph, dsph, nullptr, nullptr, nullptr, nullptr);
    check(band_dispatch<double>(plan.lanes, 1, false, normalized, a, scope.device, stream),
          "band kernel launch (allocation-free)");
}

}  // namespace

// Values and gradients in float64 for n_samples points, l_max <= 32, without any device
// allocation. normalized != 0: spherical harmonics, 0: solid harmonics. Returns 0 on success, else
// non-zero with the message in sphericart_cuda_last_error().
extern "C" int sphericart_cuda_harmonics_with_gradients_no_alloc(int normalized, size_t l_max, const double* xyz,
                                                                 size_t n_samples, double* sph, double* dsph,
                                                                 void* cuda_stream) {
    return capi_try([&] { no_alloc_run(normalized != 0, l_max, xyz, n_samples, sph, dsph, cuda_stream); });
}
