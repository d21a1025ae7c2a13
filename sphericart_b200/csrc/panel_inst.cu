// Instantiates the panel kernels for one (type, points-per-panel) pair: compile with
//   -DSPH_T=float|double -DSPH_TP=1|2|4|8|16|32
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
    // the occupancy query (which also raises the kernel's shared-memory limit) is remembered per
    // thread for the last few (device, threads, shared memory) combinations of this instantiation
    struct Slot {
        int device, threads, blocks;
        size_t smem;
    };
    thread_local Slot slots[4] = {{-1, 0, 0, 0}, {-1, 0, 0, 0}, {-1, 0, 0, 0}, {-1, 0, 0, 0}};
    thread_local int next_slot = 0;
    int max_blocks = -1;
    for (const Slot& s : slots)
        if (s.device == device && s.threads == a.threads && s.smem == a.smem) max_blocks = s.blocks;
    if (max_blocks < 0) {
        max_blocks = persistent_grid(reinterpret_cast<const void*>(kernel), a.threads, a.smem, device);
        slots[next_slot] = Slot{device, a.threads, max_blocks, a.smem};
        next_slot = (next_slot + 1) % 4;
    }
    if (max_blocks <= 0) return cudaErrorLaunchOutOfResources;
    if (a.threads % TP != 0 || a.threads > 256) return cudaErrorInvalidValue;
    const long long npanels = (a.n + TP - 1) / TP;
    const int grid = work_grid(npanels, max_blocks, a.iters, /*all_or_nothing=*/true);
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
    kernel<<<grid, a.threads, a.smem, stream>>>(k);
    return cudaGetLastError();
}

}  // namespace

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

template struct PanelLaunch<SPH_T, SPH_TP>;

}  // namespace sph_b200
