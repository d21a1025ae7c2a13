"""Parity of the kernel variants that the default dispatch does not reach on every input: the
run-time-degree kernels (panel and band) for low degrees, their plain-store and direct-store copy-out
modes, forced lane counts and panel shapes, the tile kernels without TMA, and persistent launches
against grids of short-lived CTAs. The variants are selected by the library's
development environment variables, which are read once per process, so each runs in a child
process that prints its worst scaled error against the CPU checker."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch
import sphericart_b200 as sb
from oracle import oracle
cases = eval(sys.argv[2])
import os
if os.environ.get("EXPECT_PANEL"):
    # the forced shape must be one the library accepts: otherwise the calls would quietly go elsewhere
    from sphericart_b200 import _c_lib
    assert _c_lib.kernel_family(1, 12, 4) == "sph_panel_kernel"
rng = np.random.default_rng(11)
worst = {"f32": 0.0, "f64": 0.0}
for normalized, dt, l_max, level, n in cases:
    dtype = np.float64 if dt == "f64" else np.float32
    xyz = (rng.standard_normal((n, 3)) * 1.6).astype(dtype)
    xyz[0] = 0.0                      # the origin: NaN pattern must match too
    cls = sb.SphericalHarmonics if normalized else sb.SolidHarmonics
    calc = cls(l_max)
    t = torch.from_numpy(xyz).cuda()
    got = calc._compute_impl(t, level)
    want = oracle.ref_compute(xyz, l_max, normalized, level) if oracle.have_ref() else \
        oracle.port_compute(xyz, l_max, normalized, level)
    for a, b in zip(got[: level + 1], want[: level + 1]):
        err, bad = oracle.scaled_error(a.cpu().numpy(), b, l_max)
        assert bad == 0, (normalized, dt, l_max, level, n, "NaN pattern")
        worst[dt] = max(worst[dt], err)
    g = rng.standard_normal((n, (l_max + 1) ** 2)).astype(dtype)
    vj = calc.compute_vjp(t[1:], torch.from_numpy(g[1:]).cuda()).cpu().numpy()
    x64 = xyz[1:].astype(np.float64)
    _, dref, _ = oracle.ref_compute(x64, l_max, normalized, 1) if oracle.have_ref() else \
        oracle.port_compute(x64, l_max, normalized, 1)
    ref = np.einsum("nak,nk->na", dref, g[1:].astype(np.float64))
    scale = np.einsum("nak,nk->na", np.abs(dref), np.abs(g[1:].astype(np.float64))).max(axis=1, keepdims=True)
    worst[dt] = max(worst[dt], float((np.abs(vj - ref) / scale).max()))
print("WORST", worst["f32"], worst["f64"])
"""

CASES = [(True, "f32", 3, 2, 70), (False, "f32", 8, 1, 333), (True, "f64", 6, 2, 65), (True, "f32", 12, 1, 257),
         (True, "f64", 20, 1, 100), (False, "f64", 33, 2, 33), (True, "f32", 16, 2, 129), (True, "f64", 32, 1, 64),
         # values only (the panel kernels carry the rows in registers there): even and odd row lengths; float32 stays
         # below l_max = 19, where its gradients - the VJP half of the check is against float64 - lose their accuracy
         (True, "f32", 18, 0, 100), (False, "f64", 9, 0, 77), (True, "f64", 31, 0, 45)]

VARIANTS = [
    {},
    {"SPH_B200_FORCE_BAND": "1"},
    {"SPH_B200_NO_BULK": "1"},
    {"SPH_B200_FORCE_BAND": "1", "SPH_B200_NO_BULK": "1"},
    {"SPH_B200_FORCE_BAND": "1", "SPH_B200_BAND_LANES": "32", "SPH_B200_BAND_DIRECT": "1"},
    {"SPH_B200_FORCE_BAND": "1", "SPH_B200_BAND_LANES": "1"},
    {"SPH_B200_FORCE_BAND": "1", "SPH_B200_BAND_LANES": "4", "SPH_B200_BAND_WARPS": "3"},
    {"SPH_B200_BAND_DIRECT": "-1"},
    {"SPH_B200_TILE_WARPS": "3"},
    # persistent launches instead of grids of short-lived CTAs, and a different split of the work
    {"SPH_B200_TILE_ITERS": "-1", "SPH_B200_VJP_ITERS": "-1", "SPH_B200_BAND_ITERS": "-1"},
    {"SPH_B200_TILE_ITERS": "3", "SPH_B200_VJP_ITERS": "1", "SPH_B200_BAND_ITERS": "2", "SPH_B200_TILE_WARPS": "2"},
    # tiles narrower than a warp (chosen by the library for small calls and large rows)
    {"SPH_B200_TILE_POINTS": "8"},
    {"SPH_B200_TILE_POINTS": "16", "SPH_B200_TILE_ITERS": "-1"},
    {"SPH_B200_TILE_POINTS": "32"},
    # every degree above l_max = 2 through the run-time-degree kernels: the panel kernels (forward) ...
    {"SPH_B200_TILE_LMAX": "2"},
    # ... and the band kernel alone
    {"SPH_B200_TILE_LMAX": "2", "SPH_B200_NO_PANEL": "1"},
    {"SPH_B200_NO_PANEL": "1"},
    # panel shapes that the plan picks only for some degrees: one point per image (spans at any
    # alignment), whole-warp panels with a persistent launch, plain-store copy-out, several panels per
    # table batch with a ring of three images, table recurrences in float64
    {"SPH_B200_TILE_LMAX": "2", "SPH_B200_PANEL_POINTS": "1", "SPH_B200_PANEL_THREADS": "96", "EXPECT_PANEL": "1"},
    {"SPH_B200_TILE_LMAX": "2", "SPH_B200_PANEL_POINTS": "32", "SPH_B200_PANEL_THREADS": "64",
     "SPH_B200_PANEL_ITERS": "-1", "EXPECT_PANEL": "1"},
    {"SPH_B200_TILE_LMAX": "2", "SPH_B200_PANEL_POINTS": "4", "SPH_B200_NO_BULK": "1", "EXPECT_PANEL": "1"},
    {"SPH_B200_TILE_LMAX": "2", "SPH_B200_PANEL_BATCH": "8", "SPH_B200_PANEL_POINTS": "2", "SPH_B200_PANEL_SLOTS": "3",
     "EXPECT_PANEL": "1"},
    {"SPH_B200_TILE_LMAX": "2", "SPH_B200_PANEL_BATCH": "16", "SPH_B200_PANEL_TABLES_F64": "1", "EXPECT_PANEL": "1"},
]


@pytest.mark.parametrize("variant", VARIANTS, ids=lambda v: ",".join(f"{k[9:]}={x}" for k, x in v.items() if k.startswith("SPH_B200_")) or "default")
def test_variant_parity(variant, tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ)
    env.update(variant)
    out = subprocess.run([sys.executable, str(script), ROOT, repr(CASES)], capture_output=True, text=True, env=env,
                         timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("WORST")][-1].split()
    assert float(line[1]) <= 1e-5, line      # float32 bar
    assert float(line[2]) <= 1e-12, line     # float64 bar
