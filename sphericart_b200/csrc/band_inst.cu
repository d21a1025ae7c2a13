// Instantiates the band kernels for one (type, lanes-per-point) pair: compile with
//   -DSPH_T=float|double -DSPH_G=1|2|4|8|16|32
#include "sph_band.cuh"
#include "sph_launch.hpp"


#ifndef SPH_T
#error "compile with -DSPH_T=float or -DSPH_T=double"
#endif
#ifndef SPH_G
#error "compile with -DSPH_G=<1,2,4,8,16,32>"
#endif

namespace sph_b200 {

namespace {

template <typename T, int LEVEL, bool NORM, int G, bool VJP, bool DIRECT>
cudaError_t launch_band(const BandLaunchArgs<T>& a, int device, cudaStream_t stream) {
    auto kernel = sph_band_kernel<T, LEVEL, NORM, G, VJP, DIRECT>;
    const int max_blocks = memo_grid<sph_band_kernel<T, LEVEL, NORM, G, VJP, DIRECT>>(a.warps * 32, a.smem, device);
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    constexpr int P = 32 / G;
    const long long ngroups = (a.n + P - 1) / P;
    const long long want = (ngroups + a.warps - 1) / a.warps;
    int grid = work_grid(want, max_blocks, a.iters, /*all_or_nothing=*/true);
    if (a.iters <= 0 && a.grid_cap > 0 && grid > a.grid_cap) grid = a.grid_cap;
    BandArgs<T> k{};
    k.xyz = a.xyz;
    k.n = a.n;
    k.sph = a.sph;
    k.dsph = a.dsph;
    k.ddsph = a.ddsph;
    k.sph_grad = a.sph_grad;
    k.dsph_grad = a.dsph_grad;
    k.xyz_grad = a.xyz_grad;
    k.tables = a.d_tables;
    k.l_max = a.l_max;
    k.mode = a.mode;
    kernel<<<grid, a.warps * 32, a.smem, stream>>>(k);
    return cudaGetLastError();
}

template <typename T, int LEVEL, int G>
cudaError_t launch_forward(bool normalized, const BandLaunchArgs<T>& a, int device, cudaStream_t stream) {
    if (a.mode == BAND_DIRECT) {
        // the direct-store variant exists for whole-warp-per-point launches only
        if constexpr (G == 32) {
            return normalized ? launch_band<T, LEVEL, true, G, false, true>(a, device, stream)
                              : launch_band<T, LEVEL, false, G, false, true>(a, device, stream);
        } else {
            return cudaErrorInvalidValue;
        }
    }
    return normalized ? launch_band<T, LEVEL, true, G, false, false>(a, device, stream)
                      : launch_band<T, LEVEL, false, G, false, false>(a, device, stream);
}

}  // namespace

template <typename T, int G>
cudaError_t BandLaunch<T, G>::run(int level, bool vjp, bool normalized, const BandLaunchArgs<T>& a, int device,
                                  cudaStream_t stream) {
    if (vjp) {
        if (level >= 2) {
            return normalized ? launch_band<T, 2, true, G, true, false>(a, device, stream)
                              : launch_band<T, 2, false, G, true, false>(a, device, stream);
        }
        return normalized ? launch_band<T, 1, true, G, true, false>(a, device, stream)
                          : launch_band<T, 1, false, G, true, false>(a, device, stream);
    }
    switch (level) {
        case 0: return launch_forward<T, 0, G>(normalized, a, device, stream);
        case 1: return launch_forward<T, 1, G>(normalized, a, device, stream);
        case 2: return launch_forward<T, 2, G>(normalized, a, device, stream);
        default: return cudaErrorInvalidValue;
    }
}

template struct BandLaunch<SPH_T, SPH_G>;

}  // namespace sph_b200
