// Fused vector-Jacobian product for the higher compile-time degrees: the warps of a CTA SHARE one
// tile of 32 points and split its degrees among themselves.
//
// Why. The one-warp-per-tile VJP kernel (sph_tile.cuh) keeps the tile's 32 upstream-gradient rows
// in shared memory, one image per warp. From l_max = 11 or so that image (32 (l_max+1)^2 elements:
// 37 KB at l_max = 16 in float32) leaves room for a handful of warps per SM - four at l_max = 16,
// 6 % of the warp slots - with nothing to hide the latency of the bulk load, of instruction fetch
// (the fully unrolled body does not fit the instruction cache) or of the arithmetic chains:
// 0.56 of the copy peak at l_max = 16. Here W warps work on the same image, so an SM holds W times
// as many warps for the same shared memory.
//
// How. Thread t of every warp is point t of the tile. Degree l belongs to warp owner(l) (degrees
// dealt from the top in snake order, which balances the (l+1) pairs per degree to a few percent);
// a warp evaluates only its own degrees, each with its own two rows of the Q table (Q_l and
// Q_{l-1}, both by the reference's downward-in-m recurrence,
// sphericart/include/templates_core.hpp:123,155,202 - rows are independent of one another, so
// nothing is shared between degrees) and accumulates sum_k g_k dY_k / d(unit vector) for its columns.
// The W partial sums meet in shared memory; warp 0 adds them, applies the chain rule through
// r -> r/|r| once (it is linear in the gradient) and writes the three results of each point.
// The branch on the owner is uniform within a warp: no divergence, each warp simply runs its own
// part of the unrolled body.
//
// The tile's upstream rows are one contiguous span of the input and arrive by a TMA 1-D bulk load
// (completion on an mbarrier, bounded wait) when sph_grad is 16-byte aligned, the tile is full and
// the rows carry no padding; otherwise the CTA stages them with coalesced loads.
//
// Replaces, for these degrees, the reference's backward (a gradients launch that materialises dsph,
// then an element-wise product and a reduction:
// sphericart-torch/python/sphericart/torch/register.py:90-108).
#pragma once

#include "sph_tile.cuh"

namespace sph_b200 {

// Which of W warps evaluates degree l: degrees LMAX, LMAX-1, ... dealt 0, 1, ..., W-1, W-1, ..., 1, 0, 0, 1, ...
__host__ __device__ constexpr int split_owner(int l, int lmax, int w) {
    const int rank = lmax - l;  // 0 for the highest degree
    const int round = rank / w, pos = rank % w;
    return (round % 2 == 0) ? pos : (w - 1 - pos);
}

// Accumulates, for the degrees this warp owns, the raw gradient (with respect to the evaluation
// point, i.e. the unit vector for the normalised harmonics) contracted with the row g.
template <typename T, int LMAX, int W>
__device__ __forceinline__ void eval_owned_degrees_vjp(T x, T y, T z, const Tables<T, LMAX>& tab, const T* g, int w,
                                                       T& ax, T& ay, T& az) {
    const T rho = x * x + y * y;
    // c[m] = r_xy^m cos(m phi), s[m] = r_xy^m sin(m phi), tz[m] = 2(m+1)z (sphericart/include/templates.hpp:451-466)
    T c[LMAX + 1], s[LMAX + 1], tz[LMAX + 1];
    c[0] = T(1);
    s[0] = T(0);
    const T twoz = z + z;
    tz[0] = twoz;
    static_for<1, LMAX + 1>([&](auto mc) {
        constexpr int m = decltype(mc)::value;
        c[m] = c[m - 1] * x - s[m - 1] * y;
        s[m] = c[m - 1] * y + s[m - 1] * x;
        tz[m] = tz[m - 1] + twoz;
    });
    // degree 1 in closed form, as in eval_point (degree 0 has no gradient)
    if constexpr (LMAX >= 1) {
        if (split_owner(1, LMAX, W) == w) {
            const T a1 = T(0.48860251190292);
            ay += g[1] * a1;
            az += g[2] * a1;
            ax += g[3] * a1;
        }
    }
    static_for<2, LMAX + 1>([&](auto lc) {
        constexpr int l = decltype(lc)::value;
        if (split_owner(l, LMAX, W) != w) return;  // uniform within the warp
        constexpr int mid = l * l + l;
        // rows l and l-1 of the Q table, downward in m
        T Ql[l + 1], Qp[l];
        Ql[l] = tab.K[tri(l, l)];
        Ql[l - 1] = -z * Ql[l];
        static_for_down<l - 2, 0>([&](auto mc) {
            constexpr int m = decltype(mc)::value;
            Ql[m] = tab.K[tri(l, m)] * (tz[m] * Ql[m + 1] + rho * Ql[m + 2]);
        });
        Qp[l - 1] = tab.K[tri(l - 1, l - 1)];
        if constexpr (l >= 2) Qp[l - 2] = -z * Qp[l - 1];
        static_for_down<l - 3, 0>([&](auto mc) {
            constexpr int m = decltype(mc)::value;
            Qp[m] = tab.K[tri(l - 1, m)] * (tz[m] * Qp[m + 1] + rho * Qp[m + 2]);
        });
        // the same expressions as eval_point (sph_core.cuh), gradients only
        static_for_down<l, 1>([&](auto mc) {
            constexpr int m = decltype(mc)::value;
            const T f = tab.F[tri(l, m)];
            const T pq = Ql[m] * f;
            const T pqm = pq * T(m);
            const T pqs = pqm * s[m - 1], pqc = pqm * c[m - 1];
            T mgx, pgx, mgy, pgy, mgz = T(0), pgz = T(0);
            if constexpr (m + 1 <= l - 1) {
                const T pdq = f * Qp[m + 1];
                const T pdqx = pdq * x, pdqy = pdq * y;
                mgx = pdqx * s[m] + pqs;
                pgx = pdqx * c[m] + pqc;
                mgy = pdqy * s[m] + pqc;
                pgy = pdqy * c[m] - pqs;
            } else {
                mgx = pqs;
                pgx = pqc;
                mgy = pqc;
                pgy = -pqs;
            }
            if constexpr (m <= l - 1) {
                const T pdz = f * T(l + m) * Qp[m];
                mgz = pdz * s[m];
                pgz = pdz * c[m];
            }
            const T gm = g[mid - m], gp = g[mid + m];
            ax += gm * mgx;
            ay += gm * mgy;
            az += gm * mgz;
            ax += gp * pgx;
            ay += gp * pgy;
            az += gp * pgz;
        });
        {
            const T f = tab.F[tri(l, 0)];
            const T g0 = g[mid];
            ax += g0 * (f * x * Qp[1]);
            ay += g0 * (f * y * Qp[1]);
            az += g0 * (f * T(l) * Qp[0]);
        }
    });
}

// Dynamic shared memory: the tile's image of sph_grad rows, W x 32 x 3 partial sums, one mbarrier.
template <typename T, int LMAX, int W> __host__ __device__ constexpr size_t vjp_split_smem_bytes() {
    return size_t(TILE_POINTS) * (n_columns(LMAX) + tile_row_pad(n_columns(LMAX), int(sizeof(T)))) * sizeof(T) +
           size_t(W) * TILE_POINTS * 3 * sizeof(T) + 16;
}

// blockDim.x = 32 * W. One tile per CTA at a time, tiles dealt round-robin over the grid.
template <typename T, int LMAX, bool NORM, int W>
__global__ void __launch_bounds__(32 * W)
sph_vjp_split_kernel(const T* __restrict__ xyz, const T* __restrict__ sph_grad, long long n, T* __restrict__ xyz_grad,
                     const __grid_constant__ Tables<T, LMAX> tab, int use_bulk) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int NY = n_columns(LMAX);
    constexpr int PAD = tile_row_pad(NY, int(sizeof(T)));
    constexpr int S = NY + PAD;
    constexpr unsigned TILE_BYTES = unsigned(TILE_POINTS * NY * sizeof(T));
    if constexpr (PAD != 0) use_bulk = 0;  // padded rows are not an image of global memory
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* img = reinterpret_cast<T*>(smem_raw);
    T* part = img + TILE_POINTS * S;  // [W][32][3]
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(part + W * TILE_POINTS * 3);

    const long long ntiles = (n + TILE_POINTS - 1) / TILE_POINTS;
    // a tile can come through the engine when it is full (the same answer for every thread)
    auto engine_tile = [&](long long tile) { return use_bulk && tile < ntiles && (tile + 1) * TILE_POINTS <= n; };
    auto issue = [&](long long tile) {
        if (engine_tile(tile) && threadIdx.x == 0) {
            mbar_expect_tx(bar, TILE_BYTES);
            bulk_load_global_to_smem(img, sph_grad + tile * TILE_POINTS * NY, TILE_BYTES, bar);
        }
    };
    if (use_bulk) {
        if (threadIdx.x == 0) {
            mbar_init(bar, 1);
            mbar_init_fence();
        }
        __syncthreads();
        issue(blockIdx.x);
    }
    unsigned phase = 0u;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long first = tile * TILE_POINTS;
        const long long i = first + lane;
        const int npts = (n - first) < TILE_POINTS ? int(n - first) : TILE_POINTS;
        T x = T(1), y = T(0), z = T(0);
        if (i < n) {
            x = xyz[3 * i + 0];
            y = xyz[3 * i + 1];
            z = xyz[3 * i + 2];
        }
        T ir = T(1);
        if constexpr (NORM) {
            // IEEE square root and division, as on the CPU (sphericart/include/templates.hpp:392-400)
            ir = T(1) / sqrt(x * x + y * y + z * z);
            x *= ir;
            y *= ir;
            z *= ir;
        }
        if (engine_tile(tile)) {
            if (!mbar_wait_bounded(bar, phase)) {
                g_tile_wait_gave_up = 1;
                return;  // nothing else of this CTA is in flight: the next tile is only requested below
            }
            phase ^= 1u;
        } else {
            // rows past the end of the input are zero: their lanes write no result
            const T* gsrc = sph_grad + first * NY;
            for (int e = threadIdx.x; e < TILE_POINTS * NY; e += 32 * W) img[e + PAD * (e / NY)] = (e < npts * NY) ? gsrc[e] : T(0);
            __syncthreads();
        }

        T ax = T(0), ay = T(0), az = T(0);
        eval_owned_degrees_vjp<T, LMAX, W>(x, y, z, tab, img + lane * S, warp, ax, ay, az);
        part[(warp * TILE_POINTS + lane) * 3 + 0] = ax;
        part[(warp * TILE_POINTS + lane) * 3 + 1] = ay;
        part[(warp * TILE_POINTS + lane) * 3 + 2] = az;
        // the image is written next by the TMA engine (async proxy) after having been read through
        // ordinary loads: order the two; the barrier also publishes the partial sums
        fence_proxy_async_smem();
        __syncthreads();
        issue(tile + gridDim.x);  // the image is free: the next tile streams in during the reduction
        if (warp == 0) {
            T sx = T(0), sy = T(0), sz = T(0);
#pragma unroll
            for (int w = 0; w < W; ++w) {
                sx += part[(w * TILE_POINTS + lane) * 3 + 0];
                sy += part[(w * TILE_POINTS + lane) * 3 + 1];
                sz += part[(w * TILE_POINTS + lane) * 3 + 2];
            }
            if constexpr (NORM) {
                // x, y, z hold the unit vector here
                const T t = sx * x + sy * y + sz * z;
                sx = (sx - x * t) * ir;
                sy = (sy - y * t) * ir;
                sz = (sz - z * t) * ir;
            }
            if (i < n) {
                xyz_grad[3 * i + 0] = sx;
                xyz_grad[3 * i + 1] = sy;
                xyz_grad[3 * i + 2] = sz;
            }
        }
        __syncthreads();  // the partial sums are free again
    }
}

}  // namespace sph_b200
