// "Selected" kernels: values of chosen degree blocks only, written packed, scaled and with the
// input axes permuted - in one pass. Callers that follow other conventions (the e3nn adaptor of the
// reference, sphericart-torch/python/sphericart/torch/e3nn.py:47-80) want a few degrees l, each
// multiplied by a normalisation factor, from points whose axes are ordered (y, z, x); the reference
// evaluates every degree up to the largest, then slices, permutes and rescales with tensor
// expressions, so the output crosses memory three times. Here block l of a point's row goes
// straight to columns dest[l] ... dest[l] + 2l of a packed row of ny_out columns, times scale[l];
// blocks with dest[l] < 0 are evaluated (the recurrence needs them) but never stored. The fused
// vector-Jacobian product reads the upstream gradient in the same packed layout and returns the
// gradient in the caller's axis order.
//
// Same structure as the tile kernels (sph_tile.cuh): one thread per point, one warp per tile of 32
// points, maximum degree known at compile time, the tile's packed rows built in shared memory
// (row stride forced odd: conflict-free) and copied out as one contiguous span - by the TMA engine
// when the packed rows are themselves of odd length (the image is then the exact picture of the
// span), by coalesced warp stores otherwise.
#pragma once

#include "sph_tile.cuh"

namespace sph_b200 {

template <typename T, int LMAX> struct SelectMap {
    int dest[LMAX + 1];   // first packed column of block l, or -1
    T scale[LMAX + 1];    // factor applied to block l
    int ny_out;           // packed row length
    int axis[3];          // which input column holds x, y, z
};

__host__ __device__ constexpr int degree_of_column(int k) {
    int l = 0;
    while ((l + 1) * (l + 1) <= k) ++l;
    return l;
}

// Row stride of the packed image: the row length made odd.
__host__ __device__ constexpr int select_row_stride(int ny_out) { return ny_out | 1; }

template <typename T, int LMAX> struct SelectSink {
    T* row;  // this point's packed row in the image
    const SelectMap<T, LMAX>& map;
    template <int K> __device__ __forceinline__ void put(const Column<T>& v) {
        constexpr int l = degree_of_column(K);
        const int d = map.dest[l];
        if (d >= 0) row[d + (K - l * l)] = v.y * map.scale[l];
    }
};

template <typename T, int LMAX> struct SelectVjpSink {
    const T* g;  // this point's packed row of the upstream gradient, in shared memory
    const SelectMap<T, LMAX>& map;
    T ax, ay, az;
    template <int K> __device__ __forceinline__ void put(const Column<T>& v) {
        constexpr int l = degree_of_column(K);
        const int d = map.dest[l];
        if (d >= 0) {
            const T gk = g[d + (K - l * l)] * map.scale[l];
            ax += gk * v.gx;
            ay += gk * v.gy;
            az += gk * v.gz;
        }
    }
};

// blockDim.x = 32 * warps; dynamic shared memory = warps * 32 * select_row_stride(ny_out) * sizeof(T).
template <typename T, int LMAX, bool NORM>
__global__ void __launch_bounds__(128)
sph_select_kernel(const T* __restrict__ xyz, long long n, T* __restrict__ out, const __grid_constant__ Tables<T, LMAX> tab,
                  const __grid_constant__ SelectMap<T, LMAX> map, int use_bulk) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int len = map.ny_out;
    const int S = select_row_stride(len);
    const bool exact_image = S == len;
    T* img = reinterpret_cast<T*>(smem_raw) + size_t(warp) * TILE_POINTS * S;

    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long stride = (long long)gridDim.x * nwarps;
    bool store_in_flight = false;  // lane 0 only
    for (long long tile = (long long)blockIdx.x * nwarps + warp; tile < ntiles; tile += stride) {
        const long long first = tile * TILE_POINTS;
        const long long i = first + lane;
        const int npts = (n - first) < TILE_POINTS ? int(n - first) : TILE_POINTS;
        // lanes past the end evaluate a harmless point; their rows are never copied out
        T x = T(1), y = T(0), z = T(0);
        if (i < n) {
            x = xyz[3 * i + map.axis[0]];
            y = xyz[3 * i + map.axis[1]];
            z = xyz[3 * i + map.axis[2]];
        }
        if (lane == 0 && store_in_flight) {
            bulk_wait_read_all();  // the previous tile's bulk store must be done reading the image
            store_in_flight = false;
        }
        __syncwarp();
        SelectSink<T, LMAX> sink{img + lane * S, map};
        eval_point<T, LMAX, 0, NORM>(x, y, z, tab, sink);

        T* gdst = out + first * len;
        if (use_bulk && exact_image && npts == TILE_POINTS) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                bulk_store_smem_to_global(gdst, img, unsigned(TILE_POINTS * len * sizeof(T)));
                bulk_commit();
                store_in_flight = true;
            }
        } else {
            __syncwarp();
            // element e of the span lies in row e / len of the image; rows and columns are stepped, not divided
            int col = lane, row = 0;
            while (col >= len) {
                col -= len;
                ++row;
            }
            for (int e = lane; e < npts * len; e += 32) {
                gdst[e] = img[row * S + col];
                col += 32;
                while (col >= len) {
                    col -= len;
                    ++row;
                }
            }
            __syncwarp();
        }
    }
    if (lane == 0 && store_in_flight) bulk_wait_read_all();  // shared memory must outlive the engine's reads
}

// xyz_grad[i][axis[a]] = sum over the selected columns of out_grad[i][column] * scale * dY[i][a][k].
template <typename T, int LMAX, bool NORM>
__global__ void __launch_bounds__(128)
sph_select_vjp_kernel(const T* __restrict__ xyz, const T* __restrict__ out_grad, long long n, T* __restrict__ xyz_grad,
                      const __grid_constant__ Tables<T, LMAX> tab, const __grid_constant__ SelectMap<T, LMAX> map) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int len = map.ny_out;
    const int S = select_row_stride(len);
    T* img = reinterpret_cast<T*>(smem_raw) + size_t(warp) * TILE_POINTS * S;

    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long stride = (long long)gridDim.x * nwarps;
    for (long long tile = (long long)blockIdx.x * nwarps + warp; tile < ntiles; tile += stride) {
        const long long first = tile * TILE_POINTS;
        const long long i = first + lane;
        const int npts = (n - first) < TILE_POINTS ? int(n - first) : TILE_POINTS;
        T x = T(1), y = T(0), z = T(0);
        if (i < n) {
            x = xyz[3 * i + map.axis[0]];
            y = xyz[3 * i + map.axis[1]];
            z = xyz[3 * i + map.axis[2]];
        }
        __syncwarp();  // the previous tile's reads of the image are complete
        {
            // the tile's rows of the upstream gradient are one contiguous span: coalesced loads
            const T* gsrc = out_grad + first * len;
            int col = lane, row = 0;
            while (col >= len) {
                col -= len;
                ++row;
            }
            for (int e = lane; e < TILE_POINTS * len; e += 32) {
                img[row * S + col] = e < npts * len ? gsrc[e] : T(0);
                col += 32;
                while (col >= len) {
                    col -= len;
                    ++row;
                }
            }
        }
        __syncwarp();
        // the chain rule through r -> r/|r| is linear in the gradient: applied once to the sum
        SelectVjpSink<T, LMAX> sink{img + lane * S, map, T(0), T(0), T(0)};
        eval_point<T, LMAX, 1, NORM, SelectVjpSink<T, LMAX>, true>(x, y, z, tab, sink);
        if constexpr (NORM) {
            const T ir = T(1) / sqrt(x * x + y * y + z * z);
            const T ux = x * ir, uy = y * ir, uz = z * ir;
            const T t = sink.ax * ux + sink.ay * uy + sink.az * uz;
            sink.ax = (sink.ax - ux * t) * ir;
            sink.ay = (sink.ay - uy * t) * ir;
            sink.az = (sink.az - uz * t) * ir;
        }
        if (i < n) {
            xyz_grad[3 * i + map.axis[0]] = sink.ax;
            xyz_grad[3 * i + map.axis[1]] = sink.ay;
            xyz_grad[3 * i + map.axis[2]] = sink.az;
        }
    }
}

}  // namespace sph_b200
