// "Tile" kernels: one thread per point, one warp per tile of 32 consecutive points, maximum
// degree known at compile time (l_max <= 8).
//
// Data movement. The outputs are row-major [N][ny], [N][3][ny], [N][3][3][ny], so the rows of
// 32 consecutive points form ONE contiguous span in each output array. A warp builds the exact
// image of those spans in its own slice of shared memory (thread t writes row t; with ny odd the
// row stride is odd, so the 32 lanes hit 32 different banks) and then a single lane hands each
// span to the TMA engine as a 1-D bulk store (cp.async.bulk.global.shared::cta). The copy-out
// therefore costs no issue slots and is always made of full 128-byte lines, and the warp goes
// straight on to its next tile; it only waits, before overwriting the slice, for the engine to
// have finished READING shared memory. Spans start at multiples of 32*ny*sizeof(T) bytes from
// the array base, i.e. 16-byte aligned whenever the base is; a base that is not 16-byte aligned
// and the ragged last tile fall back to coalesced plain stores from the same image.
//
// There is no communication between warps, CTAs or GPUs and no spin-wait anywhere.
//
// Replaces spherical_harmonics_kernel (sphericart/src/sphericart_impl.cu:207-615) for l_max <= 8.
#pragma once

#include "sph_core.cuh"

namespace sph_b200 {

constexpr int TILE_POINTS = 32;

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void bulk_store_smem_to_global(void* gdst, const void* ssrc, unsigned bytes) {
    const unsigned saddr = static_cast<unsigned>(__cvta_generic_to_shared(ssrc));
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(saddr), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until every committed bulk store of this thread has finished reading shared memory.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// Writes one point's columns into the tile image held in shared memory.
template <typename T, int NY, int LEVEL> struct TileSink {
    T* sph;    // this point's row of the [32][NY] image
    T* dsph;   // this point's row of the [32][3][NY] image
    T* ddsph;  // this point's row of the [32][9][NY] image
    template <int K> __device__ __forceinline__ void put(const Column<T>& v) {
        sph[K] = v.y;
        if constexpr (LEVEL >= 1) {
            dsph[K] = v.gx;
            dsph[NY + K] = v.gy;
            dsph[2 * NY + K] = v.gz;
        }
        if constexpr (LEVEL >= 2) {
            ddsph[0 * NY + K] = v.hxx;
            ddsph[1 * NY + K] = v.hxy;
            ddsph[2 * NY + K] = v.hxz;
            ddsph[3 * NY + K] = v.hxy;
            ddsph[4 * NY + K] = v.hyy;
            ddsph[5 * NY + K] = v.hyz;
            ddsph[6 * NY + K] = v.hxz;
            ddsph[7 * NY + K] = v.hyz;
            ddsph[8 * NY + K] = v.hzz;
        }
    }
};

template <typename T, int LMAX, int LEVEL> constexpr size_t tile_smem_bytes() {
    return size_t(TILE_POINTS) * n_columns(LMAX) * level_components(LEVEL) * sizeof(T);
}

// blockDim.x = 32 * warps; dynamic shared memory = warps * tile_smem_bytes. Tiles are dealt
// round-robin over all warps of the (persistent) grid.
template <typename T, int LMAX, int LEVEL, bool NORM>
__global__ void __launch_bounds__(256)
sph_tile_kernel(const T* __restrict__ xyz, long long n, T* __restrict__ sph, T* __restrict__ dsph,
                T* __restrict__ ddsph, const __grid_constant__ Tables<T, LMAX> tab, int use_bulk) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NY = n_columns(LMAX);
    constexpr int ROW = NY * level_components(LEVEL);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;

    T* img_sph = reinterpret_cast<T*>(smem_raw) + size_t(warp) * TILE_POINTS * ROW;
    T* img_d = img_sph + TILE_POINTS * NY;
    T* img_dd = img_sph + TILE_POINTS * NY * 4;

    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long stride = (long long)gridDim.x * nwarps;
    for (long long tile = (long long)blockIdx.x * nwarps + warp; tile < ntiles; tile += stride) {
        const long long first = tile * TILE_POINTS;
        const long long i = first + lane;
        // lanes past the end evaluate a harmless point; their rows are never copied out
        T x = T(1), y = T(0), z = T(0);
        if (i < n) {
            x = xyz[3 * i + 0];
            y = xyz[3 * i + 1];
            z = xyz[3 * i + 2];
        }

        // the previous tile's bulk stores must be done reading this slice
        if (use_bulk && lane == 0) bulk_wait_read_all();
        __syncwarp();

        TileSink<T, NY, LEVEL> sink{img_sph + lane * NY, img_d + lane * 3 * NY, img_dd + lane * 9 * NY};
        eval_point<T, LMAX, LEVEL, NORM>(x, y, z, tab, sink);

        const int npts = (n - first) < TILE_POINTS ? int(n - first) : TILE_POINTS;
        if (use_bulk && npts == TILE_POINTS) {
            fence_proxy_async_smem();  // make this lane's image writes visible to the TMA engine
            __syncwarp();
            if (lane == 0) {
                bulk_store_smem_to_global(sph + first * NY, img_sph, unsigned(TILE_POINTS * NY * sizeof(T)));
                if constexpr (LEVEL >= 1)
                    bulk_store_smem_to_global(dsph + first * 3 * NY, img_d, unsigned(TILE_POINTS * 3 * NY * sizeof(T)));
                if constexpr (LEVEL >= 2)
                    bulk_store_smem_to_global(ddsph + first * 9 * NY, img_dd, unsigned(TILE_POINTS * 9 * NY * sizeof(T)));
                bulk_commit();
            }
        } else {
            __syncwarp();
            for (int e = lane; e < npts * NY; e += 32) sph[first * NY + e] = img_sph[e];
            if constexpr (LEVEL >= 1)
                for (int e = lane; e < npts * 3 * NY; e += 32) dsph[first * 3 * NY + e] = img_d[e];
            if constexpr (LEVEL >= 2)
                for (int e = lane; e < npts * 9 * NY; e += 32) ddsph[first * 9 * NY + e] = img_dd[e];
            __syncwarp();
        }
    }
    // shared memory must outlive the engine's reads
    if (use_bulk && lane == 0) bulk_wait_read_all();
}

// ---------------------------------------------------------------------------------------------
// Fused vector-Jacobian product: xyz_grad[i][a] = sum_k sph_grad[i][k] * dY[i][a][k], without
// ever writing dY to memory. The tile's 32 rows of sph_grad are one contiguous span of the
// input; the warp loads it with coalesced reads into shared memory, then thread t walks row t
// (odd stride: conflict-free) while it evaluates the gradient columns in registers.
//
// Replaces the reference's backward (a gradients launch that materialises dsph, then an
// element-wise product and a reduction: sphericart-torch/python/sphericart/torch/register.py:90-108)
// and its unused backward_kernel (sphericart/src/sphericart_impl.cu:650-684).
template <typename T, int NY> struct VjpSink {
    const T* g;  // this point's row of the upstream gradient, in shared memory
    T ax, ay, az;
    template <int K> __device__ __forceinline__ void put(const Column<T>& v) {
        const T gk = g[K];
        ax += gk * v.gx;
        ay += gk * v.gy;
        az += gk * v.gz;
    }
};

template <typename T, int LMAX> constexpr size_t vjp_tile_smem_bytes() {
    return size_t(TILE_POINTS) * n_columns(LMAX) * sizeof(T);
}

template <typename T, int LMAX, bool NORM>
__global__ void __launch_bounds__(256)
sph_vjp_tile_kernel(const T* __restrict__ xyz, const T* __restrict__ sph_grad, long long n,
                    T* __restrict__ xyz_grad, const __grid_constant__ Tables<T, LMAX> tab) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NY = n_columns(LMAX);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    T* img_g = reinterpret_cast<T*>(smem_raw) + size_t(warp) * TILE_POINTS * NY;

    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long stride = (long long)gridDim.x * nwarps;
    for (long long tile = (long long)blockIdx.x * nwarps + warp; tile < ntiles; tile += stride) {
        const long long first = tile * TILE_POINTS;
        const long long i = first + lane;
        const int npts = (n - first) < TILE_POINTS ? int(n - first) : TILE_POINTS;
        T x = T(1), y = T(0), z = T(0);
        if (i < n) {
            x = xyz[3 * i + 0];
            y = xyz[3 * i + 1];
            z = xyz[3 * i + 2];
        }
        __syncwarp();  // previous tile's reads of the image are complete
        const T* gsrc = sph_grad + first * NY;
        for (int e = lane; e < TILE_POINTS * NY; e += 32) img_g[e] = (e < npts * NY) ? gsrc[e] : T(0);
        __syncwarp();

        VjpSink<T, NY> sink{img_g + lane * NY, T(0), T(0), T(0)};
        eval_point<T, LMAX, 1, NORM>(x, y, z, tab, sink);
        if (i < n) {
            xyz_grad[3 * i + 0] = sink.ax;
            xyz_grad[3 * i + 1] = sink.ay;
            xyz_grad[3 * i + 2] = sink.az;
        }
    }
}

}  // namespace sph_b200
