// float32 only: the +m (cosine-like) and -m (sine-like) columns of one (l, m) pair evaluated
// together with Blackwell's packed two-wide FP32 instructions (fma.rn.f32x2 and friends, exposed
// as __ffma2_rn / __fmul2_rn / __fadd2_rn on sm_100). The two columns run exactly the same
// formulas with (c_m, s_m) exchanged, so one packed instruction does the work of two scalar ones;
// each half is rounded exactly like the scalar operation, and the multiply-adds are fused in the
// same places as in the scalar code path, so the results agree with it to the last bits.
//
// Layout of a packed value: .x = the +m column, .y = the -m column.
#pragma once

#include "sph_core.cuh"

namespace sph_b200 {

struct F2 {
    float2 v;
};

__device__ __forceinline__ F2 f2(float lo, float hi) { return F2{make_float2(lo, hi)}; }
__device__ __forceinline__ F2 bc(float s) { return F2{make_float2(s, s)}; }
__device__ __forceinline__ F2 operator*(F2 a, F2 b) { return F2{__fmul2_rn(a.v, b.v)}; }
__device__ __forceinline__ F2 operator+(F2 a, F2 b) { return F2{__fadd2_rn(a.v, b.v)}; }
__device__ __forceinline__ F2 fma2(F2 a, F2 b, F2 c) { return F2{__ffma2_rn(a.v, b.v, c.v)}; }
__device__ __forceinline__ F2 neg(F2 a) { return f2(-a.v.x, -a.v.y); }
__device__ __forceinline__ F2 operator-(F2 a, F2 b) { return a + neg(b); }
// (c, s) -> (-s, c): the combination the y-derivatives need
__device__ __forceinline__ F2 rot(F2 a) { return f2(-a.v.y, a.v.x); }

// The two columns of a pair, packed.
struct Column2 {
    F2 y;
    F2 gx, gy, gz;
    F2 hxx, hxy, hxz, hyy, hyz, hzz;
};

// Per-point constants of the unit-sphere chain rule, broadcast to both halves.
struct UnitSphere2 {
    F2 x, y, z, mx, my, mz;           // u and -u
    F2 m2x, m2y, m2z;                 // -2u
    F2 xx, yy, zz, xy, xz, yz;        // u_a u_b
    F2 xx3, yy3, zz3, xy3, xz3, yz3;  // 3 u_a u_b
    F2 xy2, xz2, yz2;                 // 2 u_a u_b
    F2 ir, irsq;
};

template <int LEVEL> __device__ __forceinline__ UnitSphere2 make_unit_sphere2(const UnitSphere<float>& u) {
    UnitSphere2 p{};
    const float x = u.x, y = u.y, z = u.z;
    p.x = bc(x);
    p.y = bc(y);
    p.z = bc(z);
    p.mx = bc(-x);
    p.my = bc(-y);
    p.mz = bc(-z);
    p.ir = bc(u.ir);
    if constexpr (LEVEL >= 2) {
        p.m2x = bc(-2 * x);
        p.m2y = bc(-2 * y);
        p.m2z = bc(-2 * z);
        p.xx = bc(x * x);
        p.yy = bc(y * y);
        p.zz = bc(z * z);
        p.xy = bc(x * y);
        p.xz = bc(x * z);
        p.yz = bc(y * z);
        p.xx3 = bc(3 * x * x);
        p.yy3 = bc(3 * y * y);
        p.zz3 = bc(3 * z * z);
        p.xy3 = bc(3 * x * y);
        p.xz3 = bc(3 * x * z);
        p.yz3 = bc(3 * y * z);
        p.xy2 = bc(2 * x * y);
        p.xz2 = bc(2 * x * z);
        p.yz2 = bc(2 * y * z);
        p.irsq = bc(u.irsq);
    }
    return p;
}

// Same expressions, in the same order, as to_cartesian() in sph_core.cuh.
template <int LEVEL> __device__ __forceinline__ void to_cartesian2(Column2& v, const UnitSphere2& u) {
    const F2 t = fma2(v.gz, u.z, fma2(v.gy, u.y, v.gx * u.x));
    if constexpr (LEVEL >= 2) {
        const F2 hux = fma2(u.z, v.hxz, fma2(u.y, v.hxy, u.x * v.hxx));
        const F2 huy = fma2(u.z, v.hyz, fma2(u.y, v.hyy, u.x * v.hxy));
        const F2 huz = fma2(u.z, v.hzz, fma2(u.y, v.hyz, u.x * v.hxz));
        F2 uhu = u.xx * v.hxx;
        uhu = fma2(u.yy, v.hyy, uhu);
        uhu = fma2(u.zz, v.hzz, uhu);
        uhu = fma2(u.xy2, v.hxy, uhu);
        uhu = fma2(u.xz2, v.hxz, uhu);
        uhu = fma2(u.yz2, v.hyz, uhu);
        const F2 mt = neg(t);
        // diagonal: (-2 a (Hu)_a + H_aa + 3 a a t - t - 2 a g_a + a a uHu) / r^2
        F2 nxx = fma2(u.m2x, hux, v.hxx);
        nxx = fma2(u.xx3, t, nxx) + mt;
        nxx = fma2(u.xx, uhu, fma2(u.m2x, v.gx, nxx)) * u.irsq;
        F2 nyy = fma2(u.m2y, huy, v.hyy);
        nyy = fma2(u.yy3, t, nyy) + mt;
        nyy = fma2(u.yy, uhu, fma2(u.m2y, v.gy, nyy)) * u.irsq;
        F2 nzz = fma2(u.m2z, huz, v.hzz);
        nzz = fma2(u.zz3, t, nzz) + mt;
        nzz = fma2(u.zz, uhu, fma2(u.m2z, v.gz, nzz)) * u.irsq;
        // off-diagonal: (-a (Hu)_b - b (Hu)_a + H_ab + 3 a b t - a g_b - b g_a + a b uHu) / r^2
        F2 nxy = fma2(u.my, hux, u.mx * huy) + v.hxy;
        nxy = fma2(u.my, v.gx, fma2(u.mx, v.gy, fma2(u.xy3, t, nxy)));
        nxy = fma2(u.xy, uhu, nxy) * u.irsq;
        F2 nxz = fma2(u.mz, hux, u.mx * huz) + v.hxz;
        nxz = fma2(u.mz, v.gx, fma2(u.mx, v.gz, fma2(u.xz3, t, nxz)));
        nxz = fma2(u.xz, uhu, nxz) * u.irsq;
        F2 nyz = fma2(u.my, huz, u.mz * huy) + v.hyz;
        nyz = fma2(u.my, v.gz, fma2(u.mz, v.gy, fma2(u.yz3, t, nyz)));
        nyz = fma2(u.yz, uhu, nyz) * u.irsq;
        v.hxx = nxx;
        v.hyy = nyy;
        v.hzz = nzz;
        v.hxy = nxy;
        v.hxz = nxz;
        v.hyz = nyz;
    }
    v.gx = fma2(u.mx, t, v.gx) * u.ir;
    v.gy = fma2(u.my, t, v.gy) * u.ir;
    v.gz = fma2(u.mz, t, v.gz) * u.ir;
}

// Inputs of one pair as the scalar path loads them (see PairInputs in sph_band.cuh); passed field by
// field to keep this header independent of it.
struct PairScalars {
    float f, q, q1a, q1b, q2a, q2b, q2c;
    float fm, flm, fmm, fz;
};

// Raw packed columns of one pair; the formulas of band_eval_pair() with (c, s) packed.
template <int LEVEL>
__device__ __forceinline__ void eval_pair2(const PairScalars& in, F2 cs, F2 cs1, F2 cs2, float x, float y, float x2,
                                           float y2, float xy, Column2& v) {
    const float f = in.f;
    const float pq = in.q * f;
    v.y = bc(pq) * cs;
    if constexpr (LEVEL >= 1) {
        const float pqm = pq * in.fm;
        const F2 pqcs1 = bc(pqm) * cs1;  // (m F Q c_{m-1}, m F Q s_{m-1})
        const float pdq = f * in.q1a;
        v.gx = fma2(bc(pdq * x), cs, pqcs1);
        v.gy = fma2(bc(pdq * y), cs, rot(pqcs1));
        v.gz = bc(f * in.flm * in.q1b) * cs;
        if constexpr (LEVEL >= 2) {
            const float A = f * in.q1a, D = f * in.q1b;
            const float B = f * in.q2a, E = f * in.q2b, C = f * in.q2c;
            const float fm = in.fm, flm = in.flm;
            const F2 P = bc(in.fmm * pq) * cs2;  // (Pc, Ps)
            const float f2m = fm + fm;
            const F2 acs = bc(A) * cs;
            v.hxx = fma2(bc(f2m * x * A), cs1, fma2(bc(x2 * B), cs, acs)) + P;
            v.hyy = fma2(bc(f2m * y * A), rot(cs1), fma2(bc(y2 * B), cs, acs)) - P;
            v.hzz = bc(in.fz * C) * cs;
            v.hxy = fma2(bc(x * A * fm), rot(cs1), fma2(bc(y * A * fm), cs1, bc(xy * B) * cs)) + rot(P);
            const float dfm = flm * D * fm;
            v.hxz = fma2(bc(dfm), cs1, bc(x * flm * E) * cs);
            v.hyz = fma2(bc(dfm), rot(cs1), bc(y * flm * E) * cs);
        }
    }
}

}  // namespace sph_b200
