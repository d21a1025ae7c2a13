// Per-point evaluation of real spherical / solid harmonics with the maximum degree known at
// compile time. Every loop over (l, m) is unrolled by template recursion, so the prefactor
// tables are read with constant indices (they sit in the kernel's parameter bank) and the
// Q_l^m rows live in registers; row l-1 and row l-2, which the derivatives need, are the rows
// the two previous degrees already produced, so nothing is recomputed.
//
// The arithmetic follows the reference CPU implementation (the parity target):
//   prefactors      sphericart/include/templates.hpp:54-97   (built on the host, same recipe)
//   normalisation   sphericart/include/templates.hpp:392-400
//   c_m, s_m, 2mz   sphericart/include/templates.hpp:451-466
//   Q recurrence    sphericart/include/templates_core.hpp:123,155,202
//   Y, dY, ddY      sphericart/include/templates_core.hpp:122-426
//   unit-sphere chain rule  sphericart/include/templates.hpp:553-614
#pragma once

#include <cuda_runtime.h>

#include <type_traits>

namespace sph_b200 {

__host__ __device__ constexpr int tri(int l, int m) { return l * (l + 1) / 2 + m; }
__host__ __device__ constexpr int n_columns(int l_max) { return (l_max + 1) * (l_max + 1); }
__host__ __device__ constexpr int n_table(int l_max) { return (l_max + 1) * (l_max + 2) / 2; }
// number of output scalars per column for a derivative level (values, +gradient, +Hessian)
__host__ __device__ constexpr int level_components(int level) { return level == 0 ? 1 : (level == 1 ? 4 : 13); }

// Tile kernels keep one row per lane in shared memory. When the row length is a multiple of 16
// elements (l_max = 3, 7: 16 and 64 columns) all lanes of a warp would hit the same few banks, so
// such rows are padded. Rows of 256 bytes or more get 16 bytes: at most four lanes then share a
// bank and every row still starts on a 16-byte boundary, so the rows can travel through the TMA
// engine one by one. Shorter rows are copied by the warp itself, in 16-byte pieces on the global
// side, and get one element (odd stride, no conflicts). Measured on a B200, float32 gradients:
// l_max = 7: 0.18 of the copy peak unpadded, 0.64 with one element and warp copies, 0.75 with
// row-wise engine copies; l_max = 3: 0.36 unpadded, 0.79 with element-wise warp copies, 1.00 with
// 16-byte pieces.
__host__ __device__ constexpr int tile_row_pad(int ny, int elem_bytes) {
    return ny % 16 != 0 ? 0 : (ny * elem_bytes >= 256 ? 16 / elem_bytes : 1);
}
// elements one point occupies in the forward tile image: rows of ny, 3 ny and 9 ny elements
__host__ __device__ constexpr int tile_point_elems(int ny, int level, int elem_bytes) {
    return (ny + tile_row_pad(ny, elem_bytes)) + (level >= 1 ? 3 * ny + tile_row_pad(ny, elem_bytes) : 0) +
           (level >= 2 ? 9 * ny + tile_row_pad(ny, elem_bytes) : 0);
}

// F: normalisation factors of Y_l^m, K: constants of the Q_l^m recurrence, both indexed tri(l,m).
template <typename T, int LMAX> struct Tables {
    T F[n_table(LMAX)];
    T K[n_table(LMAX)];
};

template <int I> using Int = std::integral_constant<int, I>;

// f(Int<B>), f(Int<B+1>), ..., f(Int<E-1>)
template <int B, int E, typename Fn> __device__ __forceinline__ void static_for(Fn&& f) {
    if constexpr (B < E) {
        f(Int<B>{});
        static_for<B + 1, E>(f);
    }
}

// f(Int<HI>), f(Int<HI-1>), ..., f(Int<LO>)
template <int HI, int LO, typename Fn> __device__ __forceinline__ void static_for_down(Fn&& f) {
    if constexpr (HI >= LO) {
        f(Int<HI>{});
        static_for_down<HI - 1, LO>(f);
    }
}

// One column's raw outputs (derivatives taken with respect to the possibly normalised point).
template <typename T> struct Column {
    T y;
    T gx, gy, gz;
    T hxx, hxy, hxz, hyy, hyz, hzz;
};

// Per-point constants of the chain rule through r -> r/|r|.
template <typename T> struct UnitSphere {
    T x, y, z, ir, irsq;
};

// Turns derivatives with respect to the unit vector into derivatives with respect to the
// original point. With u the unit vector, g the raw gradient, H the raw Hessian, t = u.g:
//   grad    = (g - u t) / r
//   hess_ab = [H_ab - u_a (Hu)_b - u_b (Hu)_a + u_a u_b (u.Hu) + (3 u_a u_b - d_ab) t
//              - u_a g_b - u_b g_a] / r^2
// The expression order is the reference's so that float32 results round alike.
template <typename T, int LEVEL>
__device__ __forceinline__ void to_cartesian(Column<T>& v, const UnitSphere<T>& u) {
    const T x = u.x, y = u.y, z = u.z;
    const T t = v.gx * x + v.gy * y + v.gz * z;
    if constexpr (LEVEL >= 2) {
        const T hux = x * v.hxx + y * v.hxy + z * v.hxz;
        const T huy = x * v.hxy + y * v.hyy + z * v.hyz;
        const T huz = x * v.hxz + y * v.hyz + z * v.hzz;
        const T uhu = x * x * v.hxx + y * y * v.hyy + z * z * v.hzz + 2 * x * y * v.hxy +
                      2 * x * z * v.hxz + 2 * y * z * v.hyz;
        const T nxx = (-2 * x * hux + v.hxx + 3 * x * x * t - t - 2 * x * v.gx + x * x * uhu) * u.irsq;
        const T nyy = (-2 * y * huy + v.hyy + 3 * y * y * t - t - 2 * y * v.gy + y * y * uhu) * u.irsq;
        const T nzz = (-2 * z * huz + v.hzz + 3 * z * z * t - t - 2 * z * v.gz + z * z * uhu) * u.irsq;
        const T nxy = (-x * huy - y * hux + v.hxy + 3 * x * y * t - x * v.gy - y * v.gx + x * y * uhu) * u.irsq;
        const T nxz = (-x * huz - z * hux + v.hxz + 3 * x * z * t - x * v.gz - z * v.gx + x * z * uhu) * u.irsq;
        const T nyz = (-z * huy - y * huz + v.hyz + 3 * y * z * t - z * v.gy - y * v.gz + y * z * uhu) * u.irsq;
        v.hxx = nxx;
        v.hyy = nyy;
        v.hzz = nzz;
        v.hxy = nxy;
        v.hxz = nxz;
        v.hyz = nyz;
    }
    v.gx = (v.gx - x * t) * u.ir;
    v.gy = (v.gy - y * t) * u.ir;
    v.gz = (v.gz - z * t) * u.ir;
}

// Evaluates all (l_max+1)^2 columns for one point and hands each to sink.put<column>(Column).
// LEVEL 0: values; 1: + gradient; 2: + Hessian. NORM: evaluate at r/|r| and chain-rule back.
// RAW: hand over the derivatives with respect to the unit vector instead (a caller that only
// needs a linear combination of the columns applies the linear chain rule once, to the sum).
template <typename T, int LMAX, int LEVEL, bool NORM, typename Sink, bool RAW = false>
__device__ __forceinline__ void eval_point(T x, T y, T z, const Tables<T, LMAX>& tab, Sink& sink) {
    UnitSphere<T> us{x, y, z, T(0), T(0)};
    if constexpr (NORM) {
        // IEEE square root and division, as on the CPU: the r -> 0 behaviour (NaN at the
        // origin, finite for any representable r) depends on it.
        const T ir = T(1) / sqrt(x * x + y * y + z * z);
        x *= ir;
        y *= ir;
        z *= ir;
        us = UnitSphere<T>{x, y, z, ir, ir * ir};
    }
    const T x2 = x * x, y2 = y * y, xy = x * y;
    const T rho = x2 + y2;

    auto emit = [&](auto kc, Column<T> v) {
        constexpr int k = decltype(kc)::value;
        if constexpr (NORM && LEVEL >= 1 && !RAW) to_cartesian<T, LEVEL>(v, us);
        sink.template put<k>(v);
    };

    // c[m] = r_xy^m cos(m phi), s[m] = r_xy^m sin(m phi), tz[m] = 2(m+1)z
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

    // l = 0, 1: closed forms with literal constants
    {
        Column<T> v{};
        v.y = T(0.282094791773878);
        emit(Int<0>{}, v);
    }
    if constexpr (LMAX >= 1) {
        const T a1 = T(0.48860251190292);
        Column<T> vy{}, vz{}, vx{};
        vy.y = a1 * y;
        vy.gy = a1;
        vz.y = a1 * z;
        vz.gz = a1;
        vx.y = a1 * x;
        vx.gx = a1;
        emit(Int<1>{}, vy);
        emit(Int<2>{}, vz);
        emit(Int<3>{}, vx);
    }

    if constexpr (LMAX >= 2) {
        // Q[tri(l,m)]; only the rows still needed stay live in registers.
        T Q[n_table(LMAX)];
        Q[tri(0, 0)] = tab.K[tri(0, 0)];
        Q[tri(1, 1)] = tab.K[tri(1, 1)];
        Q[tri(1, 0)] = -z * Q[tri(1, 1)];

        static_for<2, LMAX + 1>([&](auto lc) {
            constexpr int l = decltype(lc)::value;
            constexpr int mid = l * l + l;
            // row l of the Q table, downward in m
            Q[tri(l, l)] = tab.K[tri(l, l)];
            Q[tri(l, l - 1)] = -z * Q[tri(l, l)];
            static_for_down<l - 2, 0>([&](auto mc) {
                constexpr int m = decltype(mc)::value;
                Q[tri(l, m)] = tab.K[tri(l, m)] * (tz[m] * Q[tri(l, m + 1)] + rho * Q[tri(l, m + 2)]);
            });

            static_for_down<l, 1>([&](auto mc) {
                constexpr int m = decltype(mc)::value;
                const T f = tab.F[tri(l, m)];
                const T pq = Q[tri(l, m)] * f;
                Column<T> vp{}, vm{};  // +m (cosine-like) and -m (sine-like) columns
                vm.y = pq * s[m];
                vp.y = pq * c[m];
                if constexpr (LEVEL >= 1) {
                    const T pqm = pq * T(m);
                    const T pqs = pqm * s[m - 1], pqc = pqm * c[m - 1];
                    if constexpr (m + 1 <= l - 1) {
                        const T pdq = f * Q[tri(l - 1, m + 1)];
                        const T pdqx = pdq * x, pdqy = pdq * y;
                        vm.gx = pdqx * s[m] + pqs;
                        vp.gx = pdqx * c[m] + pqc;
                        vm.gy = pdqy * s[m] + pqc;
                        vp.gy = pdqy * c[m] - pqs;
                    } else {
                        vm.gx = pqs;
                        vp.gx = pqc;
                        vm.gy = pqc;
                        vp.gy = -pqs;
                    }
                    if constexpr (m <= l - 1) {
                        const T pdz = f * T(l + m) * Q[tri(l - 1, m)];
                        vm.gz = pdz * s[m];
                        vp.gz = pdz * c[m];
                    }
                }
                if constexpr (LEVEL >= 2) {
                    // A = F Q_{l-1}^{m+1}, D = F Q_{l-1}^{m}, B = F Q_{l-2}^{m+2},
                    // E = F Q_{l-2}^{m+1}, C = F Q_{l-2}^{m}; absent entries are zero
                    T Pc = T(0), Ps = T(0);
                    if constexpr (m >= 2) {
                        Pc = T(m * (m - 1)) * pq * c[m - 2];
                        Ps = T(m * (m - 1)) * pq * s[m - 2];
                    }
                    T xxp = Pc, xxm = Ps, yyp = -Pc, yym = -Ps, xyp = -Ps, xym = Pc;
                    T xzp = T(0), xzm = T(0), yzp = T(0), yzm = T(0), zzp = T(0), zzm = T(0);
                    if constexpr (m + 1 <= l - 1) {
                        const T A = f * Q[tri(l - 1, m + 1)];
                        T B = T(0);
                        if constexpr (m + 2 <= l - 2) B = f * Q[tri(l - 2, m + 2)];
                        xxp = A * c[m] + x2 * B * c[m] + T(2 * m) * x * A * c[m - 1] + Pc;
                        xxm = A * s[m] + x2 * B * s[m] + T(2 * m) * x * A * s[m - 1] + Ps;
                        yyp = A * c[m] + y2 * B * c[m] - T(2 * m) * y * A * s[m - 1] - Pc;
                        yym = A * s[m] + y2 * B * s[m] + T(2 * m) * y * A * c[m - 1] - Ps;
                        xyp = xy * B * c[m] + y * A * T(m) * c[m - 1] - x * A * T(m) * s[m - 1] - Ps;
                        xym = xy * B * s[m] + y * A * T(m) * s[m - 1] + x * A * T(m) * c[m - 1] + Pc;
                    }
                    if constexpr (m <= l - 1) {
                        const T D = f * Q[tri(l - 1, m)];
                        T E = T(0);
                        if constexpr (m + 1 <= l - 2) E = f * Q[tri(l - 2, m + 1)];
                        xzp = x * T(l + m) * E * c[m] + T(l + m) * D * T(m) * c[m - 1];
                        xzm = x * T(l + m) * E * s[m] + T(l + m) * D * T(m) * s[m - 1];
                        yzp = y * T(l + m) * E * c[m] - T(l + m) * D * T(m) * s[m - 1];
                        yzm = y * T(l + m) * E * s[m] + T(l + m) * D * T(m) * c[m - 1];
                    }
                    if constexpr (m <= l - 2) {
                        const T C = f * Q[tri(l - 2, m)];
                        zzp = T((l + m) * (l + m - 1)) * C * c[m];
                        zzm = T((l + m) * (l + m - 1)) * C * s[m];
                    }
                    vp.hxx = xxp; vm.hxx = xxm;
                    vp.hyy = yyp; vm.hyy = yym;
                    vp.hzz = zzp; vm.hzz = zzm;
                    vp.hxy = xyp; vm.hxy = xym;
                    vp.hxz = xzp; vm.hxz = xzm;
                    vp.hyz = yzp; vm.hyz = yzm;
                }
                emit(Int<mid - m>{}, vm);
                emit(Int<mid + m>{}, vp);
            });

            // m = 0
            {
                const T f = tab.F[tri(l, 0)];
                Column<T> v{};
                v.y = Q[tri(l, 0)] * f;
                if constexpr (LEVEL >= 1) {
                    v.gx = f * x * Q[tri(l - 1, 1)];
                    v.gy = f * y * Q[tri(l - 1, 1)];
                    v.gz = f * T(l) * Q[tri(l - 1, 0)];
                }
                if constexpr (LEVEL >= 2) {
                    const T A = f * Q[tri(l - 1, 1)];
                    T B = T(0), E = T(0);
                    if constexpr (l - 2 >= 2) B = f * Q[tri(l - 2, 2)];
                    if constexpr (l - 2 >= 1) E = f * Q[tri(l - 2, 1)];
                    const T C = f * Q[tri(l - 2, 0)];
                    v.hxx = A + x2 * B;
                    v.hyy = A + y2 * B;
                    v.hzz = T(l * (l - 1)) * C;
                    v.hxy = xy * B;
                    v.hxz = x * T(l) * E;
                    v.hyz = y * T(l) * E;
                }
                emit(Int<mid>{}, v);
            }
        });
    }
}

// Vector-Jacobian product of one point with the maximum degree known at compile time:
//   (ax, ay, az) = sum_k g[k] dY_k/d(x, y, z)
// at the point (x, y, z) as given (for the normalised harmonics the caller passes the unit vector and
// applies the linear chain rule to the result). Same Q recurrence and prefactors as eval_point, but the
// gradient columns are never formed: with W = g+ c_m + g- s_m, U = g+ c_{m-1} + g- s_{m-1},
// V = g- c_{m-1} - g+ s_{m-1} (g+, g- the upstream entries of the columns +m and -m) the reference's
// expressions for the pair's six derivatives (sphericart/include/templates_core.hpp:201-292) contract to
//   ax += m F Q_l^m U + x F Q_{l-1}^{m+1} W,   ay += m F Q_l^m V + y F Q_{l-1}^{m+1} W,
//   az += (l+m) F Q_{l-1}^m W,
// and the common factors x, y of the second terms are applied once to their sum: 15 operations per pair
// instead of 21, and a third less code to fetch (the fully unrolled body is bound by instruction issue
// and fetch from l_max = 14 on).
template <typename T, int LMAX>
__device__ __forceinline__ void eval_point_vjp(T x, T y, T z, const Tables<T, LMAX>& tab, const T* g, T& ax, T& ay, T& az) {
    const T rho = x * x + y * y;
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
    T sx = T(0), sy = T(0), sz = T(0), sw = T(0);  // sw: the sum that x and y multiply
    if constexpr (LMAX >= 1) {
        const T a1 = T(0.48860251190292);
        sy = a1 * g[1];
        sz = a1 * g[2];
        sx = a1 * g[3];
    }
    if constexpr (LMAX >= 2) {
        T Q[n_table(LMAX)];
        Q[tri(0, 0)] = tab.K[tri(0, 0)];
        Q[tri(1, 1)] = tab.K[tri(1, 1)];
        Q[tri(1, 0)] = -z * Q[tri(1, 1)];
        static_for<2, LMAX + 1>([&](auto lc) {
            constexpr int l = decltype(lc)::value;
            constexpr int mid = l * l + l;
            Q[tri(l, l)] = tab.K[tri(l, l)];
            Q[tri(l, l - 1)] = -z * Q[tri(l, l)];
            static_for_down<l - 2, 0>([&](auto mc) {
                constexpr int m = decltype(mc)::value;
                Q[tri(l, m)] = tab.K[tri(l, m)] * (tz[m] * Q[tri(l, m + 1)] + rho * Q[tri(l, m + 2)]);
            });
            static_for_down<l, 1>([&](auto mc) {
                constexpr int m = decltype(mc)::value;
                const T f = tab.F[tri(l, m)];
                const T gp = g[mid + m], gm = g[mid - m];
                const T u = gp * c[m - 1] + gm * s[m - 1];
                const T v = gm * c[m - 1] - gp * s[m - 1];
                const T pqm = Q[tri(l, m)] * f * T(m);
                sx += pqm * u;
                sy += pqm * v;
                if constexpr (m <= l - 1) {
                    const T w = gp * c[m] + gm * s[m];
                    if constexpr (m + 1 <= l - 1) sw += f * Q[tri(l - 1, m + 1)] * w;
                    sz += f * T(l + m) * Q[tri(l - 1, m)] * w;
                }
            });
            {
                const T fg = tab.F[tri(l, 0)] * g[mid];
                sw += fg * Q[tri(l - 1, 1)];
                sz += fg * T(l) * Q[tri(l - 1, 0)];
            }
        });
    }
    ax = sx + x * sw;
    ay = sy + y * sw;
    az = sz;
}

}  // namespace sph_b200
