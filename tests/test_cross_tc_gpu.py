"""GPU parity of the tcgen05 cross-term kernel at every tree level.

By default only the widest level of a 64-site tree takes `cross_tc_kernel`; the switch
`HZ_CROSS_MP=15` sends every level through it (all four template instances: 12, 24, 48 and 96
Jacobian rows per child) and `HZ_CROSS=legacy` none. The switches are read once per process, so
each setting runs in a child process; the local energies of the same seeded walkers are compared
with the fp64 oracle and with each other (tolerances of test_walker_gpu.py: 1e-5 of the term
scale, 1e-4 relative)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from hamiltonzero_b200 import systems as S
from oracle import walker as W

pytestmark = pytest.mark.gpu

DIMS = dict(d_o=16, d_m=256, d_r=32, r_leaf=32, r_merge=64, r_ro=16)
N, WALKERS = 64, 5          # five walkers: the second group of four is ragged

CHILD = r"""
import json, sys
import numpy as np
import hamiltonzero_b200 as hz
from hamiltonzero_b200 import systems as S
dims = json.loads(sys.argv[1]); n = int(sys.argv[2]); walkers = int(sys.argv[3])
frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(n, 0.5, seed=7), n)
wf = S.synthetic_wavefunction(0, n, n_real=n, **dims)
q = S.random_unit_quaternions(np.random.default_rng(11), (walkers, n))
cw = hz.CompiledWaveFunction(wf)
got = hz.vmc_energy_custom_lap_compiled(cw, frame, q)
out = [[np.asarray(g, dtype=np.complex128).real.tolist(), np.asarray(g, dtype=np.complex128).imag.tolist()]
       for g in got]
print("RESULT" + json.dumps(out))
"""


def _run(env_extra):
    env = dict(os.environ)
    env.pop("HZ_CROSS", None)
    env.pop("HZ_CROSS_MP", None)
    env.update(env_extra)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    res = subprocess.run([sys.executable, "-c", CHILD, json.dumps(DIMS), str(N), str(WALKERS)],
                         capture_output=True, text=True, env=env, cwd=root, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT")][-1]
    return [np.asarray(re) + 1j * np.asarray(im) for re, im in json.loads(line[len("RESULT"):])]


def test_cross_term_on_tcgen05_at_every_level_matches_oracle_and_mma_sync_kernel(hz_lib):
    frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(N, 0.5, seed=7), N)
    wf = S.synthetic_wavefunction(0, N, n_real=N, **DIMS)
    q = S.random_unit_quaternions(np.random.default_rng(11), (WALKERS, N))
    ref = W.local_energy(wf, frame, q)
    _, _, lap = W.forward_laplacian(wf, frame, q.reshape(-1, N, 4))
    scale = np.abs(lap[:, 0] + 1j * lap[:, 1]) + abs(float(frame.radial_const)) + 1.0

    tc = _run({"HZ_CROSS_MP": "15"})
    legacy = _run({"HZ_CROSS": "legacy"})
    for name, got in (("tcgen05 at every level", tc), ("mma.sync at every level", legacy)):
        total = got[0].reshape(-1)
        assert np.isfinite(total.view(np.float64)).all(), name
        err = np.abs(total - np.asarray(ref[0]).reshape(-1))
        assert (err / scale).max() <= 1e-5, f"{name}: {(err / scale).max():.2e} of the term scale"
        rel = err / np.maximum(np.abs(np.asarray(ref[0]).reshape(-1)), 1e-2 * scale)
        assert rel.max() <= 1e-4, f"{name}: relative error {rel.max():.2e}"
    diff = np.abs(tc[0].reshape(-1) - legacy[0].reshape(-1))
    assert (diff / scale).max() <= 1e-5, f"kernels differ by {(diff / scale).max():.2e} of the term scale"
