"""Seeded synthetic point clouds for the benchmark configurations.

The reference's own benchmarks draw random points (benchmarks/cpp/benchmark.cpp:78-81,
benchmarks/pytorch/benchmark.py:47); no dataset is involved, so these generators ARE the
workloads. Everything is drawn in float64 from numpy's PCG64 and cast afterwards, so the CPU
checker and the GPU see identical bits.
"""

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Workload:
    name: str
    normalized: bool       # True: SphericalHarmonics, False: SolidHarmonics
    l_max: int
    level: int             # 0 values, 1 + gradients, 2 + Hessians
    dtype: str             # "f32" / "f64"
    n_points: int
    seed: int
    vjp: bool = False      # the step also runs the fused VJP of the values
    vjp2: bool = False     # the step also runs the fused second-order VJP (of values and gradients)

    @property
    def np_dtype(self):
        return np.float64 if self.dtype == "f64" else np.float32

    @property
    def ny(self):
        return (self.l_max + 1) ** 2

    def bytes_per_point(self):
        """Algorithmic HBM bytes per point: the xyz read plus every output written once."""
        size = 8 if self.dtype == "f64" else 4
        if self.vjp:
            return size * (3 + self.ny + 3)
        if self.vjp2:
            return size * (3 + 4 * self.ny + 3)
        return size * (3 + self.ny * (1, 4, 13)[self.level])


def _directions(rng, n):
    d = rng.standard_normal((n, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    return d


def _gen_normal(rng, n):
    return rng.standard_normal((n, 3))


def _gen_ball(rng, n):
    d = _directions(rng, n)
    r = 5.0 * rng.random(n) ** (1.0 / 3.0)
    return d * r[:, None]


def _gen_shell(rng, n):
    d = _directions(rng, n)
    r = rng.uniform(0.5, 6.0, n)
    return d * r[:, None]


def _gen_var2(rng, n):
    return np.sqrt(2.0) * rng.standard_normal((n, 3))


def _gen_stress(rng, n):
    """98.9 % on the unit sphere, 1 % with r log-uniform in [1e-8, 1e-6], 0.1 % at the origin."""
    d = _directions(rng, n)
    n_tiny = int(round(0.01 * n))
    n_zero = int(round(0.001 * n))
    perm = rng.permutation(n)
    r = np.ones(n)
    r[perm[:n_tiny]] = 10.0 ** rng.uniform(-8.0, -6.0, n_tiny)
    r[perm[n_tiny:n_tiny + n_zero]] = 0.0
    return d * r[:, None]


_GENERATORS = {
    "normal": _gen_normal,
    "ball5": _gen_ball,
    "shell": _gen_shell,
    "var2": _gen_var2,
    "stress": _gen_stress,
}

# name -> (workload, generator key). "metric" is the case the headline number is quoted on.
CONFIGS = {
    "metric": (Workload("spherical_l8_f32_grad", True, 8, 1, "f32", 4_194_304, 1000), "normal"),
    "cfg1": (Workload("spherical_l8_f64_grad_n1e4", True, 8, 1, "f64", 10_000, 1001), "normal"),
    "cfg2": (Workload("solid_l6_f32_grad_n1e6", False, 6, 1, "f32", 1_000_000, 1002), "ball5"),
    "cfg3": (Workload("spherical_l16_f32_hess_n2e6", True, 16, 2, "f32", 2_000_000, 1003), "shell"),
    "cfg4": (Workload("spherical_l4_f32_fwd_vjp_n5e7", True, 4, 0, "f32", 50_000_000, 1004, vjp=True), "var2"),
    "cfg5": (Workload("spherical_l32_f64_grad_n1e6", True, 32, 1, "f64", 1_000_000, 1005), "stress"),
    # Not benchmark configurations: cases of the backward kernels that the profiles under profiles/
    # capture (forward values, then the fused first- or second-order VJP).
    "aux_vjp_l16": (Workload("spherical_l16_f32_fwd_vjp", True, 16, 0, "f32", 1_048_576, 1016, vjp=True), "var2"),
    "aux_vjp2_l4": (Workload("spherical_l4_f32_fwd_vjp2", True, 4, 0, "f32", 4_194_304, 1024, vjp2=True), "var2"),
    "aux_vjp2_l16": (Workload("spherical_l16_f32_fwd_vjp2", True, 16, 0, "f32", 262_144, 1026, vjp2=True), "var2"),
    "aux_vjp_l24": (Workload("spherical_l24_f32_fwd_vjp", True, 24, 0, "f32", 524_288, 1027, vjp=True), "var2"),
    "aux_values_l24": (Workload("spherical_l24_f32_values", True, 24, 0, "f32", 524_288, 1028), "var2"),
}


def make_points(config, n_points=None, seed_offset=0):
    """Points of one configuration as an (n, 3) array of the configuration's dtype.

    ``n_points`` overrides the configured size (parity tests use a prefix-sized sample of the
    same distribution); ``seed_offset`` gives each rank of a multi-GPU run its own shard.
    """
    wl, gen = CONFIGS[config]
    n = wl.n_points if n_points is None else int(n_points)
    rng = np.random.default_rng(wl.seed + seed_offset)
    return np.ascontiguousarray(_GENERATORS[gen](rng, n).astype(wl.np_dtype))


def make_upstream_grad(config, n_points=None, seed_offset=0):
    """Upstream gradient dL/dY for the VJP configuration: iid N(0,1), shape (n, ny)."""
    wl, _ = CONFIGS[config]
    n = wl.n_points if n_points is None else int(n_points)
    rng = np.random.default_rng(wl.seed + 100 + seed_offset)
    return rng.standard_normal((n, wl.ny), dtype=np.float32).astype(wl.np_dtype)


def make_upstream_gradient_of_gradients(config, n_points=None, seed_offset=0):
    """Upstream gradient dL/d(dY) for the second-order VJP cases: iid N(0,1), shape (n, 3, ny)."""
    wl, _ = CONFIGS[config]
    n = wl.n_points if n_points is None else int(n_points)
    rng = np.random.default_rng(wl.seed + 200 + seed_offset)
    return rng.standard_normal((n, 3, wl.ny), dtype=np.float32).astype(wl.np_dtype)


def shard_bounds(n_points, world_size, rank, multiple=32):
    """Contiguous range [lo, hi) of points owned by ``rank``.

    Boundaries are rounded to a multiple of the kernels' tile (32 points) so that every
    shard's output rows start 16-byte aligned. Points are independent, so no exchange step
    follows: each rank's outputs stay in its own GPU's memory.
    """
    per = -(-n_points // world_size)
    per = -(-per // multiple) * multiple
    lo = min(n_points, rank * per)
    hi = min(n_points, lo + per)
    return lo, hi
