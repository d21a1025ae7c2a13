"""Regenerate ``ref_cpu_vectors.npz``: outputs of the reference's own CPU library.

Run where the reference checkout is available (``make -C oracle`` builds
``oracle/_ref/libsphericart_ref.so`` from the reference sources first)::

    python tests/golden/make_golden.py

The fixture pins the CPU restatement in ``oracle/`` and, on a GPU box, the CUDA library, to
the reference's CPU implementation on fixed inputs that include the corner cases the
reference's tests do not cover (origin, tiny radius, points on the axes).

Keys: ``xyz_A`` / ``xyz_B`` (float64 inputs; float32 cases use ``.astype(float32)`` of them) and
``{spherical|solid}_{f64|f32}_l{L}_lv{level}_{sph|dsph|ddsph}_{A|B}``. Values-only outputs of
the reference equal the ``sph`` of the gradients call, so level 0 is not stored.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle  # noqa: E402

# (point set, l_max list for gradients, l_max list for Hessians, dtypes)
PLAN = {
    "A": dict(grad=(0, 1, 2, 3, 4, 5, 6, 7, 8), hess=(0, 1, 2, 4, 7), dtypes=("f64", "f32")),
    "B": dict(grad=(12, 16, 32), hess=(16,), dtypes=("f64", "f32")),
}


def point_sets():
    rng = np.random.default_rng(20240607)
    a = rng.standard_normal((12, 3))
    a[0] = (0.0, 0.0, 0.0)                       # origin
    a[1] = 1e-9 * a[1] / np.linalg.norm(a[1])    # tiny radius
    a[2] = (0.0, 0.0, 1.3)                       # on +z: x^2 + y^2 == 0
    a[3] = (0.0, 0.0, -0.7)                      # on -z
    a[4] = (2.5, 0.0, 0.0)                       # on x
    a[5] = (0.0, -0.4, 0.0)                      # on y
    a[6] = (0.3, -1.1, 0.0)                      # in the xy plane
    a[7] *= 40.0                                 # far away
    # the reference test's points: xyz = 0.01*i - 0.3*alpha^2 pattern is covered by randoms;
    # test_cupy's are 8 N(0,1) points with seed 0, reproduced here as the tail of the set
    a[8:12] = np.random.default_rng(0).normal(size=(8, 3))[:4]
    b = rng.standard_normal((3, 3)) * 1.5
    return {"A": a, "B": b}


def main():
    if not oracle.have_ref():
        oracle.build()
    if not oracle.have_ref():
        raise SystemExit("reference library unavailable: cannot regenerate the fixture")
    sets = point_sets()
    out = {f"xyz_{k}": v for k, v in sets.items()}
    for tag, plan in PLAN.items():
        for dt in plan["dtypes"]:
            dtype = np.float64 if dt == "f64" else np.float32
            xyz = sets[tag].astype(dtype)
            for normalized, cls in ((True, "spherical"), (False, "solid")):
                for level, key in ((1, "grad"), (2, "hess")):
                    for L in plan[key]:
                        if dt == "f32" and L > 20:
                            continue  # (2l-1)!! overflows float32 above l = 28; keep clear of it
                        sph, dsph, ddsph = oracle.ref_compute(xyz, L, normalized, level)
                        base = f"{cls}_{dt}_l{L}_lv{level}"
                        out[f"{base}_sph_{tag}"] = sph
                        out[f"{base}_dsph_{tag}"] = dsph
                        if level == 2:
                            out[f"{base}_ddsph_{tag}"] = ddsph
    path = os.path.join(HERE, "ref_cpu_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
