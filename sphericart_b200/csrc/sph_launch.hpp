// Host-side launch interface between the calculator classes (sphericart_cuda.cu) and the
// translation units that instantiate the kernels (tile_inst.cu, band_inst.cu, each compiled
// several times with different -D settings so the build parallelises).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

namespace sph_b200 {

constexpr int TILE_LMAX = 20;       // compile-time tile kernels cover l_max 0..20
constexpr int MAX_DEVICES = 64;

// Which cases the tile kernels (compile-time l_max, one lane per point) serve; the other forward
// calls go to the panel kernels (run-time l_max, a CTA per panel of points), the other backward
// calls to the band kernel (run-time l_max, lanes share a point). kind 0..2: forward level, 3: VJP
// of the values, 4: VJP of (values, gradients). The crossovers were measured on a B200 for both
// element types (fraction of the copy peak, tile / panel or band):
//   values        l = 9..20: 1.00-1.04 / 0.29-0.57              -> tile wherever compiled
//   gradients     float32 l = 9: 0.90 / 0.70, l = 10: 0.77 / 0.90, l = 11: 0.60 / 0.82;
//                 float64 l = 8: 1.03 / 0.87, l = 9: 0.68 / 0.87, l = 10: 0.70 / 0.89
//                                                               -> tile up to 9 (float32), 8 (float64)
//   Hessians      float32 l = 4: 0.88 / 0.86, l = 5: 0.57 / 0.67; float64 l = 4: 0.84 / 0.53, l = 5: 0.57 / 0.57
//                                                               -> tile up to 4
//   VJP           l = 9..20: 0.57-1.03 / 0.15-0.25 (band)       -> tile wherever compiled
//   2nd-order VJP float32 l = 5: 1.02, l = 8: 0.59, l = 10: 0.39 / 0.25 (band), float64 l = 8: 0.50 / 0.19 (band at l = 9)
//                                                               -> tile up to 10 (float32), 8 (float64)
constexpr bool tile_serves(int kind, int l_max, int elem_bytes) {
    if (l_max > TILE_LMAX) return false;
    if (kind == 1) return l_max <= (elem_bytes == 4 ? 9 : 8);
    if (kind == 2) return l_max <= 4;
    if (kind == 4) return l_max <= (elem_bytes == 4 ? 10 : 8);
    // the VJP kernel keeps a tile's upstream rows in shared memory: at least two tiles per SM
    if (kind == 3) return size_t(32) * (l_max + 1) * (l_max + 1) * elem_bytes <= 113 * 1024;
    return true;
}

// Number of CTAs that keep every SM of `device` full for a persistent launch of `kernel` with
// the given block size and dynamic shared memory (also raises the kernel's dynamic shared
// memory limit). Results are cached by the callers.
int persistent_grid(const void* kernel, int block, size_t smem, int device);
int device_sm_count(int device);

// persistent_grid() for one kernel (a function pointer known at compile time), remembered per host
// thread for the last few (device, threads, shared memory) combinations, so that a steady stream of
// calls pays for the occupancy query (and the raise of the shared-memory limit) once.
template <auto Kernel> int memo_grid(int threads, size_t smem, int device) {
    struct Slot {
        int device, threads, blocks;
        size_t smem;
    };
    thread_local Slot slots[4] = {{-1, 0, 0, 0}, {-1, 0, 0, 0}, {-1, 0, 0, 0}, {-1, 0, 0, 0}};
    thread_local int next_slot = 0;
    for (const Slot& s : slots)
        if (s.device == device && s.threads == threads && s.smem == smem) return s.blocks;
    const int blocks = persistent_grid(reinterpret_cast<const void*>(Kernel), threads, smem, device);
    slots[next_slot] = Slot{device, threads, blocks, smem};
    next_slot = (next_slot + 1) % 4;
    return blocks;
}

// Every kernel walks its work items (spans of tiles, groups of points) with a grid-stride loop, so
// the grid size alone decides how the work is divided:
//   iters = 0: persistent launch, `resident` CTAs (one per slot the SMs offer), items dealt
//              round-robin until none are left;
//   iters = k > 0: a grid of short-lived CTAs sized so that every warp handles about k items, handed
//              out by the hardware's block scheduler as CTAs retire.
// On a B200 the second form is markedly faster for the store-bound kernels (l_max = 8 float32
// values+gradients: 7.0 against 5.8 TB/s of output): work follows the SMs that drain their stores
// fastest instead of being split evenly in advance, and the CTAs' store bursts end up staggered.
// `ctas_wanted` is the number of CTAs at one item per warp.
inline int work_grid(long long ctas_wanted, int resident, int iters, bool all_or_nothing = false) {
    long long grid = ctas_wanted < resident ? ctas_wanted : resident;
    // Several items per warp only pay on large calls: below about sixteen waves of CTAs the partly
    // filled last wave costs more than the staggering gains. A smaller call gets fewer items per
    // warp; a kernel whose CTAs have a set-up to amortise (all_or_nothing: the band kernel and its
    // tables) is launched persistently instead (l_max = 16 Hessians, 262,144 points: 0.76 ms against
    // 0.80 ms).
    if (iters > 1 && resident > 0) {
        const long long fit = ctas_wanted / (16LL * resident);
        if (fit < iters) iters = all_or_nothing ? 0 : (fit < 1 ? 1 : int(fit));
    }
    if (iters > 0) grid = (ctas_wanted + iters - 1) / iters;
    if (grid > 0x7fffffffLL) grid = 0x7fffffffLL;  // the grid-stride loops cover the remainder
    return int(grid < 1 ? 1 : grid);
}

// Which degree blocks a "selected" call emits and where (see sph_select.cuh): block l goes to the
// packed columns dest[l] ... dest[l] + 2l (dest[l] < 0: not emitted) times scale[l]; axis[a] is the
// input column that holds coordinate a.
struct Selection {
    int dest[TILE_LMAX + 1];
    double scale[TILE_LMAX + 1];
    int ny_out;
    int axis[3];
};

// Tile kernels, l_max = LMAX known at compile time. host_tables = F then K (n_table each).
template <typename T, int LMAX> struct TileLaunch {
    static size_t smem_per_warp(int level);
    // warps: images in flight per CTA; span_tiles (1..8): consecutive 32-point tiles per image;
    // iters: see work_grid(); tile_points: 32, 16 or 8 points per tile, 0 = the widest tile with which
    // the call fits in one wave of resident CTAs (32 when none does)
    static cudaError_t forward(int level, bool normalized, const T* xyz, long long n, T* sph, T* dsph, T* ddsph,
                               const T* host_tables, int warps, int span_tiles, bool use_bulk, int iters,
                               int tile_points, int device, cudaStream_t stream);
    static cudaError_t vjp(bool normalized, const T* xyz, const T* sph_grad, long long n, T* xyz_grad,
                           const T* host_tables, int warps, bool use_bulk, int iters, int device,
                           cudaStream_t stream);
    // second-order backward: VJP of (values, gradients); sph_grad may be null; use_bulk: the upstream
    // gradients are 16-byte aligned and may be fetched by the TMA engine
    static cudaError_t vjp2(bool normalized, const T* xyz, const T* sph_grad, const T* dsph_grad, long long n,
                            T* xyz_grad, const T* host_tables, int warps, int iters, bool use_bulk, int device,
                            cudaStream_t stream);
    // values of selected degree blocks, packed / scaled / axis-permuted, and the matching fused VJP
    static cudaError_t selected(bool normalized, const T* xyz, long long n, T* out, const T* host_tables,
                                const Selection& selection, bool use_bulk, int device, cudaStream_t stream);
    static cudaError_t selected_vjp(bool normalized, const T* xyz, const T* out_grad, long long n, T* xyz_grad,
                                    const T* host_tables, const Selection& selection, int device, cudaStream_t stream);
    // 1 if a bounded wait inside one of this instantiation's kernels ever gave up on the current
    // device, 0 if not, -1 if the flag could not be read. Synchronises the device.
    static int device_error_flag();
};

// Band kernels, run-time l_max. G lanes per point. mode: 0 = image in shared memory copied out by
// TMA bulk stores, 1 = image copied out by plain stores, 2 = direct global stores (G = 32 only).
template <typename T> struct BandLaunchArgs {
    const T* xyz;
    long long n;
    T* sph;
    T* dsph;
    T* ddsph;
    const T* sph_grad;
    const T* dsph_grad;
    T* xyz_grad;
    const T* d_tables;
    int l_max;
    int mode;
    int warps;
    size_t smem;
    int grid_cap;  // upper bound on the number of CTAs of a persistent launch (0 = none)
    int iters;     // see work_grid()
};

// Layout of the panel kernels' per-point state in shared memory (used by the kernels and by the plan).
constexpr int PANEL_ROW_PAD = 4;    // zeros after the diagonal of every Q row

// Element offset (for TPT = 1) of row l of the triangular Q table: a block of PANEL_ROW_PAD zeros
// (standing for the rows -1 and -2), then row 0, row 1, ... each with its PANEL_ROW_PAD zeros.
__host__ __device__ constexpr int panel_row_start(int l) { return PANEL_ROW_PAD + l * (l - 1) / 2 + (PANEL_ROW_PAD + 1) * l; }
// Elements of per-point state: the point itself (x, y, z - normalised where the harmonics are - and
// 1/r), c and s with two leading zeros each, then the Q table.
// The values-only kernels keep no Q table (and stage no pair descriptors): they carry the rows in registers.
__host__ __device__ constexpr int panel_point_state(int l_max, int level) {
    return 4 + 2 * (l_max + 3) + (level >= 1 ? panel_row_start(l_max + 1) : 0);
}
// Values only: points per thread. A thread runs the same row for this many neighbouring points of the panel
// at once (16 bytes' worth: their table entries arrive as one vector load): independent recurrence chains,
// and the row's constants are read once for all of them.
__host__ __device__ constexpr int panel_values_ppt(int elem_bytes) { return 16 / elem_bytes; }

// Panel kernels, run-time l_max, forward levels only. Tables for TPT points at a time, tp points per
// image (a power of two dividing TPT), threads / tp slices per point, `slots` images per CTA.
template <typename T> struct PanelLaunchArgs {
    const T* xyz;
    long long n;
    T* sph;
    T* dsph;
    T* ddsph;
    const T* d_tables;   // F then K
    const void* d_desc;  // the per-pair descriptors (PanelDesc in sph_panel.cuh)
    int l_max;
    int bulk;            // 1: TMA bulk copy-out, 0: plain stores
    int tp;
    int slots;
    int tables_f64;      // 1: table recurrences in float64 for float32 outputs too
    int threads;         // threads per CTA
    size_t smem;
    int iters;           // table batches per CTA, see work_grid()
};

// Fused VJP with run-time l_max (sph_panel_vjp_kernel): tables and upstream rows for TPT points at a time.
template <typename T> struct PanelVjpLaunchArgs {
    const T* xyz;
    const T* sph_grad;
    long long n;
    T* xyz_grad;
    const T* d_tables;
    int l_max;
    int bulk;        // 1: the upstream rows may come through the TMA engine (sph_grad is 16-byte aligned)
    int threads;     // slices x (TPT / points per thread), at least TPT
    size_t smem;
    int iters;       // table batches per CTA, see work_grid()
};

template <typename T, int TPT> struct PanelLaunch {
    static cudaError_t run(int level, bool normalized, const PanelLaunchArgs<T>& a, int device, cudaStream_t stream);
    static cudaError_t run_vjp(bool normalized, const PanelVjpLaunchArgs<T>& a, int device, cudaStream_t stream);
    // registers per thread of the kernel that run() would launch (0 if it cannot be queried)
    static int registers(int level, bool normalized);
    // 1 if a kernel of this translation unit gave up waiting for a TMA load, 0 if not, -1 if unknown
    static int device_error_flag();
};

template <typename T, int G> struct BandLaunch {
    // level 0..2 forward; vjp with level 1: first-order VJP, with level 2: VJP of (values, gradients)
    static cudaError_t run(int level, bool vjp, bool normalized, const BandLaunchArgs<T>& a, int device,
                           cudaStream_t stream);
};

}  // namespace sph_b200
