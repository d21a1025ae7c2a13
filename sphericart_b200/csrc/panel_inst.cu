// Instantiates the panel kernels for one (type, points-per-panel) pair: compile with
//   -DSPH_T=float|double -DSPH_TP=1|2|4|8|16|32   (points per table batch)
#include "sph_launch.hpp"
#include "sph_panel.cuh"

#ifndef SPH_T
#error "compile with -DSPH_T=float or -DSPH_T=double"
#endif
#ifndef SPH_TP
#error "compile with -DSPH_TP=<1,2,4,8,16,32>"
#endif

namespace sph_b200 {

namespace {

template <typename T, int LEVEL, bool NORM, int TP>
cudaError_t launch_panel(const PanelLaunchArgs<T>& a, int device, cudaStream_t stream) {
    auto kernel = sph_panel_kernel<T, LEVEL, NORM, TP>;
    const int max_blocks = memo_grid<sph_panel_kernel<T, LEVEL, NORM, TP>>(a.threads, a.smem, device);
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    if (a.threads < TP || a.threads > 256 || a.tp < 1 || a.tp > TP || (a.tp & (a.tp - 1)) != 0 || a.slots < 1 ||
        a.slots > PANEL_MAX_SLOTS) {
        return cudaErrorInvalidValue;
    }
    const long long nbatches = (a.n + TP - 1) / TP;
    const int grid = work_grid(nbatches, max_blocks, a.iters, /*all_or_nothing=*/true);
    PanelArgs<T> k{};
    k.xyz = a.xyz;
    k.n = a.n;
    k.sph = a.sph;
    k.dsph = a.dsph;
    k.ddsph = a.ddsph;
    k.tables = a.d_tables;
    k.desc = static_cast<const PanelDesc*>(a.d_desc);
    k.l_max = a.l_max;
    k.bulk = a.bulk;
    k.tp = a.tp;
    k.slots = a.slots;
    k.tables_f64 = a.tables_f64;
    kernel<<<grid, a.threads, a.smem, stream>>>(k);
    return cudaGetLastError();
}

template <typename T, bool NORM, int TP>
cudaError_t launch_panel_vjp(const PanelVjpLaunchArgs<T>& a, int device, cudaStream_t stream) {
    if constexpr (TP < panel_values_ppt(int(sizeof(T)))) {
        return cudaErrorInvalidValue;  // a batch holds at least one thread's points
    } else {
    auto kernel = sph_panel_vjp_kernel<T, NORM, TP>;
    constexpr int LANES = TP / panel_values_ppt(int(sizeof(T)));
    if (a.threads < TP || a.threads > 256 || a.threads % LANES != 0 ||
        a.smem < panel_vjp_smem_bytes<T>(a.l_max, TP, a.threads)) {
        return cudaErrorInvalidValue;
    }
    const int max_blocks = memo_grid<sph_panel_vjp_kernel<T, NORM, TP>>(a.threads, a.smem, device);
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    const long long nbatches = (a.n + TP - 1) / TP;
    const int grid = work_grid(nbatches, max_blocks, a.iters, /*all_or_nothing=*/true);
    PanelVjpArgs<T> k{};
    k.xyz = a.xyz;
    k.sph_grad = a.sph_grad;
    k.n = a.n;
    k.xyz_grad = a.xyz_grad;
    k.tables = a.d_tables;
    k.l_max = a.l_max;
    k.bulk = a.bulk;
    kernel<<<grid, a.threads, a.smem, stream>>>(k);
    return cudaGetLastError();
    }
}

}  // namespace

template <typename T, int TP>
cudaError_t PanelLaunch<T, TP>::run_vjp(bool normalized, const PanelVjpLaunchArgs<T>& a, int device, cudaStream_t stream) {
    return normalized ? launch_panel_vjp<T, true, TP>(a, device, stream) : launch_panel_vjp<T, false, TP>(a, device, stream);
}

template <typename T, int TP> int PanelLaunch<T, TP>::device_error_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, g_tile_wait_gave_up, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return flag;
}

template <typename T, int TP>
cudaError_t PanelLaunch<T, TP>::run(int level, bool normalized, const PanelLaunchArgs<T>& a, int device,
                                    cudaStream_t stream) {
    switch (level) {
        case 0:
            return normalized ? launch_panel<T, 0, true, TP>(a, device, stream)
                              : launch_panel<T, 0, false, TP>(a, device, stream);
        case 1:
            return normalized ? launch_panel<T, 1, true, TP>(a, device, stream)
                              : launch_panel<T, 1, false, TP>(a, device, stream);
        case 2:
            return normalized ? launch_panel<T, 2, true, TP>(a, device, stream)
                              : launch_panel<T, 2, false, TP>(a, device, stream);
        default: return cudaErrorInvalidValue;
    }
}

template <typename T, int TP> int PanelLaunch<T, TP>::registers(int level, bool normalized) {
    const void* kernel = nullptr;
    switch (level) {
        case 0: kernel = normalized ? (const void*)sph_panel_kernel<T, 0, true, TP> : (const void*)sph_panel_kernel<T, 0, false, TP>; break;
        case 1: kernel = normalized ? (const void*)sph_panel_kernel<T, 1, true, TP> : (const void*)sph_panel_kernel<T, 1, false, TP>; break;
        case 2: kernel = normalized ? (const void*)sph_panel_kernel<T, 2, true, TP> : (const void*)sph_panel_kernel<T, 2, false, TP>; break;
        default: return 0;
    }
    cudaFuncAttributes attr;
    if (cudaFuncGetAttributes(&attr, kernel) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return attr.numRegs;
}

template struct PanelLaunch<SPH_T, SPH_TP>;

}  // namespace sph_b200
