// Instantiates the tile kernels for one (type, l_max) pair: compile with
//   -DSPH_T=float|double -DSPH_LMAX=0..20
#include "sph_launch.hpp"
#include "sph_select.cuh"
#include "sph_tile.cuh"

#include <atomic>

#ifndef SPH_T
#error "compile with -DSPH_T=float or -DSPH_T=double"
#endif
#ifndef SPH_LMAX
#error "compile with -DSPH_LMAX=<0..20>"
#endif

namespace sph_b200 {

namespace {

// Grid size per (kernel, device, warps per CTA), filled on first use. Races are benign: every
// writer stores the same value.
struct GridCache {
    std::atomic<int> blocks[MAX_DEVICES][9];
};

template <typename Kernel> int cached_grid(GridCache& cache, Kernel kernel, int warps, size_t smem, int device) {
    int v = cache.blocks[device][warps].load(std::memory_order_relaxed);
    if (v == 0) {
        v = persistent_grid(reinterpret_cast<const void*>(kernel), warps * 32, smem, device);
        cache.blocks[device][warps].store(v, std::memory_order_relaxed);
    }
    return v;
}

template <typename T, int LMAX> Tables<T, LMAX> make_tables(const T* host_tables) {
    Tables<T, LMAX> t;
    for (int i = 0; i < n_table(LMAX); ++i) {
        t.F[i] = host_tables[i];
        t.K[i] = host_tables[n_table(LMAX) + i];
    }
    return t;
}

template <typename T, int LMAX, int LEVEL, bool NORM>
cudaError_t launch_forward(const T* xyz, long long n, T* sph, T* dsph, T* ddsph, const T* host_tables, int warps,
                           int span_tiles, bool use_bulk, int iters, int tile_points, int device, cudaStream_t stream) {
    static GridCache cache[3][9] = {};
    if (span_tiles < 1 || span_tiles > 8) return cudaErrorInvalidValue;
    auto kernel = sph_tile_kernel<T, LMAX, LEVEL, NORM>;
    // Points per tile. For throughput: the widest tile of which an SM holds at least five images
    // (measured on a B200, l_max = 8 gradients, 10^6 points: float64 32 / 16 / 8 points -> 0.70 / 0.96 /
    // 0.84 of the copy peak with 2 / 5 / 10 images per SM; float32 32 / 16 -> 1.03 / 0.98 with 5 / 10;
    // l_max = 9 float32 32 / 16 -> 0.87 / 0.90 with 4 / 8), at least eight where padded rows leave
    // one by one (l_max = 7 float32 gradients 32 / 16 -> 0.76 / 0.91 with 6 / 12).
    // For calls that fit in one wave of resident CTAs a tile's latency is what counts: narrower
    // tiles still, as long as the call keeps fitting in one wave.
    const int candidates[3] = {32, 16, 8};
    constexpr int NY_ = n_columns(LMAX);
    constexpr bool ROW_WISE = tile_row_pad(NY_, int(sizeof(T))) != 0 && NY_ * sizeof(T) >= 256;
    constexpr int MIN_IMAGES = ROW_WISE ? 8 : 5;
    const int sms = device_sm_count(device);
    int chosen = -1, max_blocks = 0;
    size_t smem = 0;
    auto query = [&](int c) {
        smem = size_t(warps) * span_tiles * tile_smem_bytes<T, LMAX, LEVEL>() * candidates[c] / TILE_POINTS;
        max_blocks = cached_grid(cache[c][span_tiles], kernel, warps, smem, device);
    };
    auto ctas_needed = [&](int c) {
        const long long span_points = (long long)span_tiles * candidates[c];
        return ((n + span_points - 1) / span_points + warps - 1) / warps;
    };
    for (int c = 0; c < 3 && chosen < 0; ++c) {
        if (tile_points != 0 && tile_points != candidates[c]) continue;
        query(c);
        if (max_blocks <= 0) {
            if (tile_points != 0) return cudaErrorLaunchOutOfResources;
            continue;
        }
        if (tile_points != 0 || c == 2 || max_blocks * warps >= MIN_IMAGES * sms) chosen = c;
    }
    if (chosen < 0) return tile_points != 0 ? cudaErrorInvalidValue : cudaErrorLaunchOutOfResources;
    if (tile_points == 0 && ctas_needed(chosen) <= max_blocks) {
        // one wave: narrow the tile while the call still fits in one wave
        while (chosen < 2) {
            query(chosen + 1);
            if (max_blocks <= 0 || ctas_needed(chosen + 1) > max_blocks) break;
            ++chosen;
        }
    }
    query(chosen);
    const int tp = candidates[chosen];
    const long long span_points = (long long)span_tiles * tp;
    const long long nspans = (n + span_points - 1) / span_points;
    const long long want = (nspans + warps - 1) / warps;
    const int grid = work_grid(want, max_blocks, iters);
    kernel<<<grid, warps * 32, smem, stream>>>(xyz, n, sph, dsph, ddsph, make_tables<T, LMAX>(host_tables),
                                               use_bulk ? 1 : 0, span_tiles, tp);
    return cudaGetLastError();
}

template <typename T, int LMAX, bool NORM>
cudaError_t launch_vjp(const T* xyz, const T* sph_grad, long long n, T* xyz_grad, const T* host_tables, int warps,
                       bool use_bulk, int iters, int device, cudaStream_t stream) {
    static GridCache cache{};
    auto kernel = sph_vjp_tile_kernel<T, LMAX, NORM>;
    const size_t smem = size_t(warps) * vjp_tile_smem_bytes<T, LMAX>();
    const int max_blocks = cached_grid(cache, kernel, warps, smem, device);
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long want = (ntiles + warps - 1) / warps;
    const int grid = work_grid(want, max_blocks, iters);
    kernel<<<grid, warps * 32, smem, stream>>>(xyz, sph_grad, n, xyz_grad, make_tables<T, LMAX>(host_tables),
                                               use_bulk ? 1 : 0);
    return cudaGetLastError();
}

template <typename T, int LMAX, bool NORM>
cudaError_t launch_vjp2(const T* xyz, const T* sph_grad, const T* dsph_grad, long long n, T* xyz_grad,
                        const T* host_tables, int warps, int iters, bool use_bulk, int device, cudaStream_t stream) {
    static GridCache cache{};
    auto kernel = sph_vjp2_tile_kernel<T, LMAX, NORM>;
    // the warps' images, then one mbarrier slot (16 bytes) per warp
    const size_t smem = size_t(warps) * (vjp2_tile_smem_bytes<T, LMAX>() + 16);
    const int max_blocks = cached_grid(cache, kernel, warps, smem, device);
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long want = (ntiles + warps - 1) / warps;
    const int grid = work_grid(want, max_blocks, iters);
    kernel<<<grid, warps * 32, smem, stream>>>(xyz, sph_grad, dsph_grad, n, xyz_grad, make_tables<T, LMAX>(host_tables),
                                               use_bulk ? 1 : 0);
    return cudaGetLastError();
}

template <typename T, int LMAX> SelectMap<T, LMAX> make_select_map(const Selection& selection) {
    SelectMap<T, LMAX> map;
    for (int l = 0; l <= LMAX; ++l) {
        map.dest[l] = selection.dest[l];
        map.scale[l] = T(selection.scale[l]);
    }
    map.ny_out = selection.ny_out;
    for (int a = 0; a < 3; ++a) map.axis[a] = selection.axis[a];
    return map;
}

// Warps per CTA of the selected kernels: up to four, fewer when the packed images are large.
template <typename T> int select_warps(int ny_out, int device, size_t& smem_per_warp) {
    smem_per_warp = size_t(TILE_POINTS) * select_row_stride(ny_out) * sizeof(T);
    int warps = 4;
    while (warps > 1 && warps * smem_per_warp > size_t(100) * 1024) --warps;
    (void)device;
    return warps;
}

template <typename T, int LMAX, bool NORM>
cudaError_t launch_selected(const T* xyz, long long n, T* out, const T* host_tables, const Selection& selection,
                            bool use_bulk, int device, cudaStream_t stream) {
    auto kernel = sph_select_kernel<T, LMAX, NORM>;
    size_t per_warp = 0;
    const int warps = select_warps<T>(selection.ny_out, device, per_warp);
    const size_t smem = warps * per_warp;
    const int max_blocks = memo_grid<sph_select_kernel<T, LMAX, NORM>>(warps * 32, smem, device);
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const int grid = work_grid((ntiles + warps - 1) / warps, max_blocks, /*iters=*/2);
    kernel<<<grid, warps * 32, smem, stream>>>(xyz, n, out, make_tables<T, LMAX>(host_tables),
                                               make_select_map<T, LMAX>(selection), use_bulk ? 1 : 0);
    return cudaGetLastError();
}

template <typename T, int LMAX, bool NORM>
cudaError_t launch_selected_vjp(const T* xyz, const T* out_grad, long long n, T* xyz_grad, const T* host_tables,
                                const Selection& selection, int device, cudaStream_t stream) {
    auto kernel = sph_select_vjp_kernel<T, LMAX, NORM>;
    size_t per_warp = 0;
    const int warps = select_warps<T>(selection.ny_out, device, per_warp);
    const size_t smem = warps * per_warp;
    const int max_blocks = memo_grid<sph_select_vjp_kernel<T, LMAX, NORM>>(warps * 32, smem, device);
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const int grid = work_grid((ntiles + warps - 1) / warps, max_blocks, /*iters=*/1);
    kernel<<<grid, warps * 32, smem, stream>>>(xyz, out_grad, n, xyz_grad, make_tables<T, LMAX>(host_tables),
                                               make_select_map<T, LMAX>(selection));
    return cudaGetLastError();
}

template <typename T, int LMAX, int LEVEL> constexpr bool tile_fits() { return tile_serves(LEVEL, LMAX, int(sizeof(T))); }

}  // namespace

template <typename T, int LMAX> size_t TileLaunch<T, LMAX>::smem_per_warp(int level) {
    return size_t(TILE_POINTS) * tile_point_elems(n_columns(LMAX), level, int(sizeof(T))) * sizeof(T);
}

template <typename T, int LMAX>
cudaError_t TileLaunch<T, LMAX>::forward(int level, bool normalized, const T* xyz, long long n, T* sph, T* dsph,
                                         T* ddsph, const T* host_tables, int warps, int span_tiles, bool use_bulk,
                                         int iters, int tile_points, int device, cudaStream_t stream) {
#define SPH_CASE(LEVEL)                                                                                            \
    if constexpr (tile_fits<T, LMAX, LEVEL>()) {                                                                   \
        return normalized ? launch_forward<T, LMAX, LEVEL, true>(xyz, n, sph, dsph, ddsph, host_tables, warps,     \
                                                                 span_tiles, use_bulk, iters, tile_points, device,\
                                                                 stream)                                           \
                          : launch_forward<T, LMAX, LEVEL, false>(xyz, n, sph, dsph, ddsph, host_tables, warps,    \
                                                                  span_tiles, use_bulk, iters, tile_points,       \
                                                                  device, stream);                                 \
    } else {                                                                                                       \
        return cudaErrorInvalidConfiguration;                                                                      \
    }
    switch (level) {
        case 0: SPH_CASE(0)
        case 1: SPH_CASE(1)
        case 2: SPH_CASE(2)
        default: return cudaErrorInvalidValue;
    }
#undef SPH_CASE
}

template <typename T, int LMAX>
cudaError_t TileLaunch<T, LMAX>::vjp(bool normalized, const T* xyz, const T* sph_grad, long long n, T* xyz_grad,
                                     const T* host_tables, int warps, bool use_bulk, int iters, int device,
                                     cudaStream_t stream) {
    if constexpr (tile_serves(3, LMAX, int(sizeof(T)))) {
        return normalized ? launch_vjp<T, LMAX, true>(xyz, sph_grad, n, xyz_grad, host_tables, warps, use_bulk,
                                                      iters, device, stream)
                          : launch_vjp<T, LMAX, false>(xyz, sph_grad, n, xyz_grad, host_tables, warps, use_bulk,
                                                       iters, device, stream);
    } else {
        return cudaErrorInvalidConfiguration;
    }
}

template <typename T, int LMAX>
cudaError_t TileLaunch<T, LMAX>::vjp2(bool normalized, const T* xyz, const T* sph_grad, const T* dsph_grad, long long n,
                                      T* xyz_grad, const T* host_tables, int warps, int iters, bool use_bulk, int device,
                                      cudaStream_t stream) {
    if constexpr (tile_serves(4, LMAX, int(sizeof(T)))) {
        return normalized ? launch_vjp2<T, LMAX, true>(xyz, sph_grad, dsph_grad, n, xyz_grad, host_tables, warps, iters,
                                                       use_bulk, device, stream)
                          : launch_vjp2<T, LMAX, false>(xyz, sph_grad, dsph_grad, n, xyz_grad, host_tables, warps, iters,
                                                        use_bulk, device, stream);
    } else {
        return cudaErrorInvalidConfiguration;
    }
}

template <typename T, int LMAX>
cudaError_t TileLaunch<T, LMAX>::selected(bool normalized, const T* xyz, long long n, T* out, const T* host_tables,
                                          const Selection& selection, bool use_bulk, int device, cudaStream_t stream) {
    return normalized ? launch_selected<T, LMAX, true>(xyz, n, out, host_tables, selection, use_bulk, device, stream)
                      : launch_selected<T, LMAX, false>(xyz, n, out, host_tables, selection, use_bulk, device, stream);
}

template <typename T, int LMAX>
cudaError_t TileLaunch<T, LMAX>::selected_vjp(bool normalized, const T* xyz, const T* out_grad, long long n, T* xyz_grad,
                                              const T* host_tables, const Selection& selection, int device,
                                              cudaStream_t stream) {
    return normalized
               ? launch_selected_vjp<T, LMAX, true>(xyz, out_grad, n, xyz_grad, host_tables, selection, device, stream)
               : launch_selected_vjp<T, LMAX, false>(xyz, out_grad, n, xyz_grad, host_tables, selection, device, stream);
}

template <typename T, int LMAX> int TileLaunch<T, LMAX>::device_error_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, g_tile_wait_gave_up, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return flag;
}

template struct TileLaunch<SPH_T, SPH_LMAX>;

}  // namespace sph_b200
