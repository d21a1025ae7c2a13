// "Tile" kernels: one thread per point, one warp per tile of 32 (or 16, or 8) consecutive points,
// maximum degree known at compile time (l_max <= 20; which cases they serve: tile_serves() in
// sph_launch.hpp).
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
// and the ragged last tile fall back to coalesced plain stores from the same image. Row lengths
// that are multiples of 16 elements get padded rows (tile_row_pad() in sph_core.cuh) and leave row
// by row.
//
// There is no communication between warps, CTAs or GPUs and no spin-wait anywhere.
//
// Replaces spherical_harmonics_kernel (sphericart/src/sphericart_impl.cu:207-615) for the cases
// tile_serves() lists.
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

__device__ __forceinline__ int lane_of_warp() { return int(threadIdx.x & 31); }

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until every committed bulk store of this thread has finished reading shared memory.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// Writes one point's columns into the tile image held in shared memory.
template <typename T, int NY, int LEVEL> struct TileSink {
    T* sph;    // this point's row of the [points][NY] image
    T* dsph;   // this point's row of the [points][3][NY] image
    T* ddsph;  // this point's row of the [points][9][NY] image
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

// Copies `rows` rows of LEN elements, kept in shared memory with row stride STRIDE, to a contiguous
// 16-byte aligned span of global memory in 16-byte pieces (LEN is a multiple of 16 elements, so a
// piece never straddles two rows; the shared-memory side is read element by element because
// padded rows are not 16-byte aligned).
template <typename T, int LEN, int STRIDE>
__device__ __forceinline__ void copy_rows_out_16(T* __restrict__ gdst, const T* img, int rows, int lane) {
    constexpr int Q = 16 / int(sizeof(T));
    const int pieces = rows * (LEN / Q);
    for (int v = lane; v < pieces; v += 32) {
        const int e = v * Q;
        const T* src = img + (e / LEN) * STRIDE + (e % LEN);
        if constexpr (sizeof(T) == 4) {
            const float4 piece = make_float4(src[0], src[1], src[2], src[3]);
            reinterpret_cast<float4*>(gdst)[v] = piece;
        } else {
            const double2 piece = make_double2(src[0], src[1]);
            reinterpret_cast<double2*>(gdst)[v] = piece;
        }
    }
}

// The reverse: a contiguous 16-byte aligned span of global memory into padded rows, at most
// MAXROWS of them (a compile-time trip count, so that the loop unrolls and its loads overlap).
template <typename T, int LEN, int STRIDE, int MAXROWS>
__device__ __forceinline__ void copy_rows_in_16(T* img, const T* __restrict__ gsrc, int rows, int lane) {
    constexpr int Q = 16 / int(sizeof(T));
    const int pieces = rows * (LEN / Q);
#pragma unroll
    for (int v0 = 0; v0 < MAXROWS * (LEN / Q); v0 += 32) {
        const int v = v0 + lane;
        if (v >= pieces) continue;
        const int e = v * Q;
        T* dst = img + (e / LEN) * STRIDE + (e % LEN);
        if constexpr (sizeof(T) == 4) {
            const float4 piece = reinterpret_cast<const float4*>(gsrc)[v];
            dst[0] = piece.x;
            dst[1] = piece.y;
            dst[2] = piece.z;
            dst[3] = piece.w;
        } else {
            const double2 piece = reinterpret_cast<const double2*>(gsrc)[v];
            dst[0] = piece.x;
            dst[1] = piece.y;
        }
    }
}

template <typename T, int LMAX, int LEVEL> constexpr size_t tile_smem_bytes() {
    return size_t(TILE_POINTS) * tile_point_elems(n_columns(LMAX), LEVEL, int(sizeof(T))) * sizeof(T);
}

// blockDim.x = 32 * warps; dynamic shared memory = warps * span_tiles * tile_smem_bytes * tile_points / 32.
// A warp's unit of work is a span of `span_tiles` consecutive tiles (span_tiles * tile_points
// points): it evaluates them one after the other into one image and hands the whole span to the
// TMA engine at once, so that small tiles (low l_max, values only) still leave as stores of several
// KB. Spans are dealt round-robin over all warps of the grid.
// tile_points is 32, or 16 or 8 where whole-warp tiles would leave SMs without work (small calls)
// or with too few images in flight (large rows). The lanes beyond tile_points repeat the work of
// lane (lane mod tile_points) and store the same values to the same places, so the evaluation
// code carries no predicate.
template <typename T, int LMAX, int LEVEL, bool NORM>
__global__ void __launch_bounds__(256)
sph_tile_kernel(const T* __restrict__ xyz, long long n, T* __restrict__ sph, T* __restrict__ dsph,
                T* __restrict__ ddsph, const __grid_constant__ Tables<T, LMAX> tab, int use_bulk, int span_tiles,
                int tile_points) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NY = n_columns(LMAX);
    // padded rows (see tile_row_pad) are not an image of global memory: they leave row by row
    constexpr int PAD = tile_row_pad(NY, int(sizeof(T)));
    constexpr int S0 = NY + PAD, S1 = 3 * NY + PAD, S2 = 9 * NY + PAD;
    constexpr int ROW = tile_point_elems(NY, LEVEL, int(sizeof(T)));
    // (measured: worthwhile from 256-byte rows on; shorter padded rows are copied out by the warp,
    // in 16-byte pieces when the outputs are 16-byte aligned - which is what use_bulk says)
    const bool aligned16_out = use_bulk != 0;
    if constexpr (PAD != 0 && NY * sizeof(T) < 256) use_bulk = 0;
    // bulk-store groups are per thread: with padded rows every lane issues and waits for its own
    const bool bulk_lane = use_bulk && (PAD != 0 || lane_of_warp() == 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int span_points = span_tiles * tile_points;
    const int pt = lane & (tile_points - 1);  // this lane's point within a tile

    // image of one span: [span_points][NY], then [span_points][3][NY], then [span_points][9][NY]
    T* img_sph = reinterpret_cast<T*>(smem_raw) + size_t(warp) * span_points * ROW;
    T* img_d = img_sph + span_points * S0;
    T* img_dd = img_d + span_points * S1;

    const long long nspans = (n + span_points - 1) / span_points;
    const long long stride = (long long)gridDim.x * nwarps;
    for (long long span = (long long)blockIdx.x * nwarps + warp; span < nspans; span += stride) {
        const long long first = span * span_points;
        // lanes past the end evaluate a harmless point; their rows are never copied out
        T x = T(1), y = T(0), z = T(0);
        if (first + pt < n) {
            x = xyz[3 * (first + pt) + 0];
            y = xyz[3 * (first + pt) + 1];
            z = xyz[3 * (first + pt) + 2];
        }

        // the previous span's bulk stores must be done reading this slice
        if (bulk_lane) bulk_wait_read_all();
        __syncwarp();

        for (int t = 0; t < span_tiles; ++t) {
            // fetch the next tile's point while this one is evaluated
            T nx = T(1), ny_ = T(0), nz = T(0);
            const long long inext = first + (t + 1) * tile_points + pt;
            if (t + 1 < span_tiles && inext < n) {
                nx = xyz[3 * inext + 0];
                ny_ = xyz[3 * inext + 1];
                nz = xyz[3 * inext + 2];
            }
            const int row = t * tile_points + pt;
            TileSink<T, NY, LEVEL> sink{img_sph + row * S0, img_d + row * S1, img_dd + row * S2};
            eval_point<T, LMAX, LEVEL, NORM>(x, y, z, tab, sink);
            x = nx;
            y = ny_;
            z = nz;
        }

        const int npts = (n - first) < span_points ? int(n - first) : span_points;
        if (use_bulk && npts == span_points) {
            fence_proxy_async_smem();  // make this lane's image writes visible to the TMA engine
            __syncwarp();
            if constexpr (PAD == 0) {
                if (lane == 0) {
                    bulk_store_smem_to_global(sph + first * NY, img_sph, unsigned(span_points * NY * sizeof(T)));
                    if constexpr (LEVEL >= 1)
                        bulk_store_smem_to_global(dsph + first * 3 * NY, img_d, unsigned(span_points * 3 * NY * sizeof(T)));
                    if constexpr (LEVEL >= 2)
                        bulk_store_smem_to_global(ddsph + first * 9 * NY, img_dd,
                                                  unsigned(span_points * 9 * NY * sizeof(T)));
                    bulk_commit();
                }
            } else {
                // one store per point and array, issued by the lanes side by side
                for (int r = lane; r < span_points; r += 32) {
                    bulk_store_smem_to_global(sph + (first + r) * NY, img_sph + r * S0, unsigned(NY * sizeof(T)));
                    if constexpr (LEVEL >= 1)
                        bulk_store_smem_to_global(dsph + (first + r) * 3 * NY, img_d + r * S1, unsigned(3 * NY * sizeof(T)));
                    if constexpr (LEVEL >= 2)
                        bulk_store_smem_to_global(ddsph + (first + r) * 9 * NY, img_dd + r * S2,
                                                  unsigned(9 * NY * sizeof(T)));
                }
                bulk_commit();
            }
        } else if (PAD != 0 && aligned16_out) {
            __syncwarp();
            copy_rows_out_16<T, NY, S0>(sph + first * NY, img_sph, npts, lane);
            if constexpr (LEVEL >= 1) copy_rows_out_16<T, 3 * NY, S1>(dsph + first * 3 * NY, img_d, npts, lane);
            if constexpr (LEVEL >= 2) copy_rows_out_16<T, 9 * NY, S2>(ddsph + first * 9 * NY, img_dd, npts, lane);
            __syncwarp();
        } else {
            __syncwarp();
            // element e of a span's output lies in row e / row_length of the image
            for (int e = lane; e < npts * NY; e += 32) sph[first * NY + e] = img_sph[e + PAD * (e / NY)];
            if constexpr (LEVEL >= 1)
                for (int e = lane; e < npts * 3 * NY; e += 32) dsph[first * 3 * NY + e] = img_d[e + PAD * (e / (3 * NY))];
            if constexpr (LEVEL >= 2)
                for (int e = lane; e < npts * 9 * NY; e += 32)
                    ddsph[first * 9 * NY + e] = img_dd[e + PAD * (e / (9 * NY))];
            __syncwarp();
        }
    }
    // shared memory must outlive the engine's reads
    if (bulk_lane) bulk_wait_read_all();
}

// ---------------------------------------------------------------------------------------------
// Fused vector-Jacobian product: xyz_grad[i][a] = sum_k sph_grad[i][k] * dY[i][a][k], without
// ever writing dY to memory. The tile's 32 rows of sph_grad are one contiguous span of the
// input; the warp loads it with coalesced reads into shared memory, then thread t walks row t
// (odd stride: conflict-free) while it accumulates the contraction in registers
// (eval_point_vjp in sph_core.cuh: the gradient columns themselves are never formed).
//
// Replaces the reference's backward (a gradients launch that materialises dsph, then an
// element-wise product and a reduction: sphericart-torch/python/sphericart/torch/register.py:90-108)
// and its unused backward_kernel (sphericart/src/sphericart_impl.cu:650-684).

// ---- mbarrier + TMA 1-D bulk load (global -> the issuing CTA's own shared memory) ----------
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_load_global_to_smem(void* sdst, const void* gsrc, unsigned bytes,
                                                         unsigned long long* bar) {
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(sdst));
    const unsigned b = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(d),
                 "l"(gsrc), "r"(bytes), "r"(b)
                 : "memory");
}

// Waits for the phase with the given parity, giving up after a bounded number of polls (each
// poll already blocks for a hardware-defined interval). Returns false on give-up.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity, int max_tries = 1 << 22) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(bar));
    for (int tries = 0; tries < max_tries; ++tries) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Set when a bounded wait gave up (it never does unless the device is misbehaving); one flag per
// translation unit, read by TileLaunch::device_error_flag().
static __device__ int g_tile_wait_gave_up = 0;

// Per warp: one image of the tile's sph_grad rows followed by its mbarrier (16 bytes reserved). One
// image, not two: a double buffer that fetched one tile ahead halves the warps an SM holds and
// measured slower at every degree (l_max = 10 float32: 0.61 against 1.03 of the copy peak).
template <typename T, int LMAX> __host__ __device__ constexpr size_t vjp_tile_smem_bytes() {
    return size_t(TILE_POINTS) * (n_columns(LMAX) + tile_row_pad(n_columns(LMAX), int(sizeof(T)))) * sizeof(T) + 16;
}

// use_bulk != 0: the rows of sph_grad are fetched by the TMA engine (1-D bulk load, completion on
// an mbarrier), so the warp spends no issue slots on the staging copy; the next tile is requested
// as soon as the current one has been consumed and the other resident warps cover the wait.
// Requires a 16-byte aligned sph_grad; otherwise, and for the ragged last tile, the warp stages
// the rows itself with coalesced loads.
template <typename T, int LMAX, bool NORM>
__global__ void __launch_bounds__(256)
sph_vjp_tile_kernel(const T* __restrict__ xyz, const T* __restrict__ sph_grad, long long n,
                    T* __restrict__ xyz_grad, const __grid_constant__ Tables<T, LMAX> tab, int use_bulk) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NY = n_columns(LMAX);
    constexpr unsigned TILE_BYTES = unsigned(TILE_POINTS * NY * sizeof(T));
    // padded rows (see tile_row_pad) arrive as one bulk load per row, issued by the row's lane
    // (measured: worthwhile from 256-byte rows on; shorter padded rows are staged by the warp)
    constexpr int PAD = tile_row_pad(NY, int(sizeof(T)));
    constexpr int S = NY + PAD;
    const bool aligned16_in = use_bulk != 0;
    if constexpr (PAD != 0 && NY * sizeof(T) < 256) use_bulk = 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    unsigned char* mine = smem_raw + size_t(warp) * vjp_tile_smem_bytes<T, LMAX>();
    T* img = reinterpret_cast<T*>(mine);
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(mine + size_t(TILE_POINTS) * S * sizeof(T));

    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long stride = (long long)gridDim.x * nwarps;
    const long long tile0 = (long long)blockIdx.x * nwarps + warp;

    // a tile can come through the engine when it is full (its byte count is then a multiple of 16)
    auto engine_tile = [&](long long tile) { return use_bulk && (tile + 1) * TILE_POINTS <= n; };
    auto issue = [&](long long tile) {
        if (tile < ntiles && engine_tile(tile)) {  // the same for every lane
            if constexpr (PAD == 0) {
                if (lane == 0) {
                    mbar_expect_tx(bar, TILE_BYTES);
                    bulk_load_global_to_smem(img, sph_grad + tile * TILE_POINTS * NY, TILE_BYTES, bar);
                }
            } else {
                if (lane == 0) mbar_expect_tx(bar, TILE_BYTES);
                __syncwarp();
                bulk_load_global_to_smem(img + lane * S, sph_grad + (tile * TILE_POINTS + lane) * NY, unsigned(NY * sizeof(T)),
                                         bar);
            }
        }
    };

    if (use_bulk) {
        if (lane == 0) {
            mbar_init(bar, 1);
            mbar_init_fence();
        }
        __syncwarp();
        issue(tile0);
    }

    unsigned phase = 0u;
    for (long long tile = tile0; tile < ntiles; tile += stride) {
        const long long first = tile * TILE_POINTS;
        const long long i = first + lane;
        const int npts = (n - first) < TILE_POINTS ? int(n - first) : TILE_POINTS;
        T x = T(1), y = T(0), z = T(0);
        if (i < n) {
            x = xyz[3 * i + 0];
            y = xyz[3 * i + 1];
            z = xyz[3 * i + 2];
        }

        if (engine_tile(tile)) {
            if (!mbar_wait_bounded(bar, phase)) {
                g_tile_wait_gave_up = 1;
                return;  // nothing else of this warp is in flight: the next tile is only requested below
            }
            phase ^= 1u;
        } else {
            const T* gsrc = sph_grad + first * NY;
            if (PAD != 0 && aligned16_in) {
                // rows past the end of the input keep whatever they hold: their lanes write no result
                copy_rows_in_16<T, NY, S, TILE_POINTS>(img, gsrc, npts, lane);
            } else {
                for (int e = lane; e < TILE_POINTS * NY; e += 32) img[e + PAD * (e / NY)] = (e < npts * NY) ? gsrc[e] : T(0);
            }
            __syncwarp();
        }

        // The chain rule through r -> r/|r| is linear in the gradient, so it is applied once to the
        // accumulated sum of raw gradients instead of to each of the (l_max+1)^2 columns.
        T ax, ay, az;
        if constexpr (NORM) {
            // IEEE square root and division, as on the CPU (sphericart/include/templates.hpp:392-400)
            const T ir = T(1) / sqrt(x * x + y * y + z * z);
            const T ux = x * ir, uy = y * ir, uz = z * ir;
            eval_point_vjp<T, LMAX>(ux, uy, uz, tab, img + lane * S, ax, ay, az);
            const T t = ax * ux + ay * uy + az * uz;
            ax = (ax - ux * t) * ir;
            ay = (ay - uy * t) * ir;
            az = (az - uz * t) * ir;
        } else {
            eval_point_vjp<T, LMAX>(x, y, z, tab, img + lane * S, ax, ay, az);
        }
        if (i < n) {
            xyz_grad[3 * i + 0] = ax;
            xyz_grad[3 * i + 1] = ay;
            xyz_grad[3 * i + 2] = az;
        }
        // the image is written next by the TMA engine (async proxy) after having been read through
        // ordinary loads: order the two, then ask for the next tile
        fence_proxy_async_smem();
        __syncwarp();  // all lanes are done with the image
        issue(tile + stride);
    }
}

}  // namespace sph_b200

namespace sph_b200 {

// ---------------------------------------------------------------------------------------------
// Fused second-order backward: the vector-Jacobian product of the values-and-gradients map,
//   xyz_grad[i][b] = sum_k sph_grad[i][k] dY[i][b][k] + sum_{a,k} dsph_grad[i][a][k] ddY[i][a][b][k],
// with neither dY nor ddY written to memory. sph_grad may be null (second term only).
// Replaces the reference's backward of its with_gradients op, which materialises the whole
// Hessian tensor and then multiplies and reduces it
// (sphericart-torch/python/sphericart/torch/register.py:117-145, and :101-106, :165-167).
template <typename T, int NY, bool HAS_VALUE_GRAD> struct Vjp2Sink {
    const T* gs;  // this point's row of sph_grad (shared memory), unused without HAS_VALUE_GRAD
    const T* gd;  // this point's [3][NY] rows of dsph_grad (shared memory)
    T ax, ay, az;
    template <int K> __device__ __forceinline__ void put(const Column<T>& v) {
        const T wx = gd[K], wy = gd[NY + K], wz = gd[2 * NY + K];
        ax += wx * v.hxx + wy * v.hxy + wz * v.hxz;
        ay += wx * v.hxy + wy * v.hyy + wz * v.hyz;
        az += wx * v.hxz + wy * v.hyz + wz * v.hzz;
        if constexpr (HAS_VALUE_GRAD) {
            const T gk = gs[K];
            ax += gk * v.gx;
            ay += gk * v.gy;
            az += gk * v.gz;
        }
    }
};

// The same contraction for the normalised harmonics Y(x) = S(u), u = x / r, without the chain rule
// per column. With G_c = dS/du_c, H_cd = d2S/du_c du_d (what eval_point hands over in RAW mode),
// J = du/dx = (1 - u u^T) / r and K^c_ab = d2u_c/dx_a dx_b, the result is
//   out_b = sum_c J_cb (A_c + B_c) + sum_{a,c} K^c_ab C_ac,
//   A_c = sum_k g_k G_k,c,   B = (1/r) sum_k H_k (w_k - u (u . w_k)),   C_ac = sum_k w_a,k G_k,c,
// (w_k = the three dsph_grad entries of column k), so each column costs 27 multiply-adds on raw
// derivatives and the projection is applied once per point (finish()). The reference applies it to
// every Hessian column (sphericart/include/templates.hpp:214-254) before contracting.
template <typename T, int NY, bool HAS_VALUE_GRAD> struct Vjp2RawSink {
    const T* gs;
    const T* gd;
    T ux, uy, uz;
    T a[3], b[3], c[9];
    template <int K> __device__ __forceinline__ void put(const Column<T>& v) {
        const T wx = gd[K], wy = gd[NY + K], wz = gd[2 * NY + K];
        const T t = ux * wx + uy * wy + uz * wz;
        const T px = wx - ux * t, py = wy - uy * t, pz = wz - uz * t;
        b[0] += v.hxx * px + v.hxy * py + v.hxz * pz;
        b[1] += v.hxy * px + v.hyy * py + v.hyz * pz;
        b[2] += v.hxz * px + v.hyz * py + v.hzz * pz;
        c[0] += wx * v.gx;  c[1] += wx * v.gy;  c[2] += wx * v.gz;
        c[3] += wy * v.gx;  c[4] += wy * v.gy;  c[5] += wy * v.gz;
        c[6] += wz * v.gx;  c[7] += wz * v.gy;  c[8] += wz * v.gz;
        if constexpr (HAS_VALUE_GRAD) {
            const T gk = gs[K];
            a[0] += gk * v.gx;
            a[1] += gk * v.gy;
            a[2] += gk * v.gz;
        }
    }
    __device__ __forceinline__ void finish(T ir, T& ox, T& oy, T& oz) const {
        const T sx = a[0] + b[0] * ir, sy = a[1] + b[1] * ir, sz = a[2] + b[2] * ir;
        const T d = ux * sx + uy * sy + uz * sz;
        const T tr = c[0] + c[4] + c[8];
        const T ucx = ux * c[0] + uy * c[3] + uz * c[6];  // (u^T C)_b
        const T ucy = ux * c[1] + uy * c[4] + uz * c[7];
        const T ucz = ux * c[2] + uy * c[5] + uz * c[8];
        const T cux = c[0] * ux + c[1] * uy + c[2] * uz;  // (C u)_b
        const T cuy = c[3] * ux + c[4] * uy + c[5] * uz;
        const T cuz = c[6] * ux + c[7] * uy + c[8] * uz;
        const T ucu = ucx * ux + ucy * uy + ucz * uz;
        const T k = T(3) * ucu - tr;
        const T irsq = ir * ir;
        ox = (sx - ux * d) * ir + (ux * k - ucx - cux) * irsq;
        oy = (sy - uy * d) * ir + (uy * k - ucy - cuy) * irsq;
        oz = (sz - uz * d) * ir + (uz * k - ucz - cuz) * irsq;
    }
};

// Per warp: the tile's 32 rows of sph_grad ([32][NY]) followed by its rows of dsph_grad ([32][3][NY]);
// after all warps' images, one mbarrier per warp (16 bytes reserved each).
template <typename T, int LMAX> __host__ __device__ constexpr size_t vjp2_tile_smem_bytes() {
    return size_t(TILE_POINTS) * (4 * n_columns(LMAX) + 2 * tile_row_pad(n_columns(LMAX), int(sizeof(T)))) * sizeof(T);
}

// The upstream gradients of a tile are contiguous spans of their arrays. use_bulk != 0 (both arrays
// 16-byte aligned, rows without padding): full tiles are fetched by the TMA engine - one 1-D bulk
// load per array into the warp's image, completion on the warp's mbarrier, the next tile requested
// as soon as the current one has been consumed - so that the warp neither spends issue slots on the
// staging copy nor sits on a chain of dependent global loads (with warp-staged loads this kernel
// measured 11.7 stall cycles per issue on global loads, at 27 % of the DRAM bandwidth, for
// l_max = 4). Otherwise, and for the ragged last tile, the warp stages the rows itself.
template <typename T, int LMAX, bool NORM>
__global__ void __launch_bounds__(256)
sph_vjp2_tile_kernel(const T* __restrict__ xyz, const T* __restrict__ sph_grad, const T* __restrict__ dsph_grad,
                     long long n, T* __restrict__ xyz_grad, const __grid_constant__ Tables<T, LMAX> tab, int use_bulk) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NY = n_columns(LMAX);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    constexpr int PAD = tile_row_pad(NY, int(sizeof(T)));
    constexpr int S0 = NY + PAD, S1 = 3 * NY + PAD;
    // padded rows (see tile_row_pad) arrive as one bulk load per row and array, issued by the row's
    // lane; worthwhile from 256-byte rows on, shorter padded rows are staged by the warp
    const bool aligned16_in = use_bulk != 0;
    if constexpr (PAD != 0 && NY * sizeof(T) < 256) use_bulk = 0;
    T* img_s = reinterpret_cast<T*>(smem_raw) + size_t(warp) * TILE_POINTS * (S0 + S1);
    T* img_d = img_s + TILE_POINTS * S0;
    unsigned long long* bar =
        reinterpret_cast<unsigned long long*>(smem_raw + size_t(nwarps) * vjp2_tile_smem_bytes<T, LMAX>()) + 2 * warp;
    const bool has_value_grad = sph_grad != nullptr;
    constexpr unsigned BYTES_S = unsigned(TILE_POINTS * NY * sizeof(T));
    constexpr unsigned BYTES_D = unsigned(TILE_POINTS * 3 * NY * sizeof(T));

    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    const long long stride = (long long)gridDim.x * nwarps;
    const long long tile0 = (long long)blockIdx.x * nwarps + warp;
    // a tile can come through the engine when it is full (the same answer for every lane)
    auto engine_tile = [&](long long tile) { return use_bulk && tile < ntiles && (tile + 1) * TILE_POINTS <= n; };
    auto issue = [&](long long tile) {
        if (!engine_tile(tile)) return;
        if (lane == 0) mbar_expect_tx(bar, (has_value_grad ? BYTES_S : 0u) + BYTES_D);
        if constexpr (PAD == 0) {
            if (lane == 0) {
                if (has_value_grad) bulk_load_global_to_smem(img_s, sph_grad + tile * TILE_POINTS * NY, BYTES_S, bar);
                bulk_load_global_to_smem(img_d, dsph_grad + tile * TILE_POINTS * 3 * NY, BYTES_D, bar);
            }
        } else {
            __syncwarp();  // the expected byte count is set before any lane's copy can complete
            const long long row = tile * TILE_POINTS + lane;
            if (has_value_grad) bulk_load_global_to_smem(img_s + lane * S0, sph_grad + row * NY, unsigned(NY * sizeof(T)), bar);
            bulk_load_global_to_smem(img_d + lane * S1, dsph_grad + row * 3 * NY, unsigned(3 * NY * sizeof(T)), bar);
        }
    };
    if (use_bulk) {
        if (lane == 0) {
            mbar_init(bar, 1);
            mbar_init_fence();
        }
        __syncwarp();
        issue(tile0);
    }
    unsigned phase = 0u;
    for (long long tile = tile0; tile < ntiles; tile += stride) {
        const long long first = tile * TILE_POINTS;
        const long long i = first + lane;
        const int npts = (n - first) < TILE_POINTS ? int(n - first) : TILE_POINTS;
        T x = T(1), y = T(0), z = T(0);
        if (i < n) {
            x = xyz[3 * i + 0];
            y = xyz[3 * i + 1];
            z = xyz[3 * i + 2];
        }
        if (engine_tile(tile)) {
            if (!mbar_wait_bounded(bar, phase)) {
                g_tile_wait_gave_up = 1;
                return;  // nothing else of this warp is in flight: the next tile is only requested below
            }
            phase ^= 1u;
        } else {
            __syncwarp();  // previous tile's reads of the images are complete
            if (PAD != 0 && aligned16_in) {
                // short padded rows: 16-byte pieces, unrolled so that the loads overlap (rows past the end of
                // the input keep whatever they hold: their lanes write no result)
                if (has_value_grad) copy_rows_in_16<T, NY, S0, TILE_POINTS>(img_s, sph_grad + first * NY, npts, lane);
                copy_rows_in_16<T, 3 * NY, S1, TILE_POINTS>(img_d, dsph_grad + first * 3 * NY, npts, lane);
            } else {
                if (has_value_grad) {
                    const T* src = sph_grad + first * NY;
                    for (int e = lane; e < TILE_POINTS * NY; e += 32) img_s[e + PAD * (e / NY)] = (e < npts * NY) ? src[e] : T(0);
                }
                const T* src = dsph_grad + first * 3 * NY;
                for (int e = lane; e < TILE_POINTS * 3 * NY; e += 32)
                    img_d[e + PAD * (e / (3 * NY))] = (e < npts * 3 * NY) ? src[e] : T(0);
            }
            __syncwarp();
        }

        T ax, ay, az;
        if constexpr (NORM) {
            // same normalisation as eval_point (and the reference: sphericart/include/templates.hpp:392-396)
            const T ir = T(1) / sqrt(x * x + y * y + z * z);
            const T ux = x * ir, uy = y * ir, uz = z * ir;
            if (has_value_grad) {
                Vjp2RawSink<T, NY, true> sink{img_s + lane * S0, img_d + lane * S1, ux, uy, uz, {}, {}, {}};
                eval_point<T, LMAX, 2, NORM, Vjp2RawSink<T, NY, true>, true>(x, y, z, tab, sink);
                sink.finish(ir, ax, ay, az);
            } else {
                Vjp2RawSink<T, NY, false> sink{img_s, img_d + lane * S1, ux, uy, uz, {}, {}, {}};
                eval_point<T, LMAX, 2, NORM, Vjp2RawSink<T, NY, false>, true>(x, y, z, tab, sink);
                sink.finish(ir, ax, ay, az);
            }
        } else if (has_value_grad) {
            Vjp2Sink<T, NY, true> sink{img_s + lane * S0, img_d + lane * S1, T(0), T(0), T(0)};
            eval_point<T, LMAX, 2, NORM>(x, y, z, tab, sink);
            ax = sink.ax;
            ay = sink.ay;
            az = sink.az;
        } else {
            Vjp2Sink<T, NY, false> sink{img_s, img_d + lane * S1, T(0), T(0), T(0)};
            eval_point<T, LMAX, 2, NORM>(x, y, z, tab, sink);
            ax = sink.ax;
            ay = sink.ay;
            az = sink.az;
        }
        if (i < n) {
            xyz_grad[3 * i + 0] = ax;
            xyz_grad[3 * i + 1] = ay;
            xyz_grad[3 * i + 2] = az;
        }
        if (use_bulk) {
            // the images are written next by the TMA engine (async proxy) after having been read through
            // ordinary loads: order the two, then ask for the next tile
            fence_proxy_async_smem();
            __syncwarp();
            issue(tile + stride);
        }
    }
}

}  // namespace sph_b200
