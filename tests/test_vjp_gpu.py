"""GPU parity of the reverse pass (hz_logpsi_vjp, through the C ABI) against the fp64 oracle
(torch autograd over the restated executor).

Tolerance: the north star asks gradient samples within 1e-4 relative; every gradient array is
held to 1e-4 of its own largest magnitude (floor 1e-6 of the cotangent scale for arrays that
are identically zero, such as the factors of a tree without a merged node)."""
import numpy as np
import pytest

from hamiltonzero_b200 import systems as S
from oracle import walker as W

pytestmark = pytest.mark.gpu

SMALL = dict(d_o=8, d_m=64, d_r=32, r_leaf=16, r_merge=16, r_ro=8)
MID = dict(d_o=16, d_m=256, d_r=32, r_leaf=32, r_merge=64, r_ro=32)

CASES = [
    # n, dims, n_real, walkers
    (1, SMALL, None, 5),
    (2, SMALL, None, 7),
    (8, SMALL, None, 9),
    (8, SMALL, 5, 6),
    (4, MID, None, 5),
    (16, MID, None, 6),
    (16, MID, 11, 19),
    (32, MID, 19, 4),
    (64, MID, 45, 3),
    (128, MID, 100, 2),
    (128, None, None, 1),            # default model sizes
    (256, SMALL, None, 2),
    (256, MID, 200, 1),
]


def _close(got, want, what, tol=1e-4):
    got = np.asarray(got, dtype=np.float64)
    scale = max(np.abs(want).max(), 1e-6)
    err = np.abs(got - want).max() / scale
    assert np.isfinite(got).all(), f"{what}: non-finite"
    assert err <= tol, f"{what}: {err:.2e} of scale {scale:.2e}"


@pytest.mark.parametrize("n,dims,n_real,walkers", CASES)
def test_vjp_matches_oracle(hz_lib, n, dims, n_real, walkers):
    import hamiltonzero_b200 as hz
    wf = S.synthetic_wavefunction(3, n, n_real=n if n_real is None else n_real, **(dims or {}))
    rng = np.random.default_rng(100 + n + walkers)
    q = S.random_unit_quaternions(rng, (walkers, n))
    ca = rng.standard_normal(walkers).astype(np.float32)
    cp = rng.standard_normal(walkers).astype(np.float32)
    cw = hz.CompiledWaveFunction(wf)
    g, dq, la, ph = cw.vjp(q, ca, cp, chunk_size=4)
    g0, dq0, la0, ph0 = W.logpsi_vjp(wf, q, ca, cp)
    assert np.abs(la - la0).max() <= 1e-5 * np.abs(la0).max() + 1e-5
    assert np.abs(np.angle(np.exp(1j * (ph - ph0)))).max() <= (2e-5 if n <= 32 else 5e-5)
    _close(dq, dq0, "dq")
    for k, want in g0.items():
        if k == "merge_h":
            for lvl, (a, b) in enumerate(zip(g.get(k, []), want)):
                _close(a, b, f"merge_h[{lvl}]")
        elif k in g:
            _close(g[k], want, k)


def test_vjp_is_independent_of_chunking_and_linear_in_cotangents(hz_lib):
    import hamiltonzero_b200 as hz
    n, walkers = 16, 24
    wf = S.synthetic_wavefunction(5, n, **MID)
    rng = np.random.default_rng(9)
    q = S.random_unit_quaternions(rng, (walkers, n))
    ca = rng.standard_normal(walkers).astype(np.float32)
    cp = rng.standard_normal(walkers).astype(np.float32)
    cw = hz.CompiledWaveFunction(wf)
    g1, dq1, _, _ = cw.vjp(q, ca, cp, chunk_size=walkers)
    g2, dq2, _, _ = cw.vjp(q, ca, cp, chunk_size=5)
    g3, _, _, _ = cw.vjp(q, 2 * ca, 2 * cp, chunk_size=walkers)
    np.testing.assert_allclose(dq1, dq2, rtol=0, atol=1e-5 * np.abs(dq1).max())
    for k in ("merge_T", "merge_V", "merge_U", "leaf_U", "readout_V", "q_weight"):
        s = np.abs(g1[k]).max()
        np.testing.assert_allclose(g1[k], g2[k], rtol=0, atol=2e-5 * s)
        np.testing.assert_allclose(2 * g1[k], g3[k], rtol=0, atol=4e-5 * s)


@pytest.mark.parametrize("n,dims,n_real,walkers", [(8, SMALL, 5, 7), (16, MID, 11, 9), (2, MID, None, 5)])
def test_kfac_factor_sums_match_oracle(hz_lib, n, dims, n_real, walkers):
    import hamiltonzero_b200 as hz
    n_real = n if n_real is None else n_real
    wf = S.synthetic_wavefunction(4, n, n_real=n_real, **dims)
    rng = np.random.default_rng(7 + n)
    q = S.random_unit_quaternions(rng, (walkers, n))
    ca = rng.choice([-1.0, 1.0], walkers).astype(np.float32)      # the reference's Fisher signs
    cp = rng.choice([-1.0, 1.0], walkers).astype(np.float32)
    mask = (np.arange(n) < n_real).astype(np.uint8)
    cw = hz.CompiledWaveFunction(wf)
    g, dq, la, ph, f = cw.vjp(q, ca, cp, chunk_size=4, factors=True, leaf_mask=mask)
    g0, dq0, la0, ph0, f0 = W.logpsi_vjp(wf, q, ca, cp, with_factors=True, leaf_mask=mask)
    _close(dq, dq0, "dq")
    _close(g["merge_T"], g0["merge_T"], "merge_T")
    for k, want in f0.items():
        if k == "merge_h_diag":
            for lvl, (a, b) in enumerate(zip(f.get(k, []), want)):
                _close(a, b, f"merge_h_diag[{lvl}]")
        else:
            _close(f[k], want, k)
            if np.ndim(want) == 2 and want.shape[0] == want.shape[1]:
                assert np.array_equal(f[k], f[k].T), f"{k} is not exactly symmetric"


@pytest.mark.parametrize("n,dims,n_real,walkers", [(8, SMALL, 5, 7), (16, MID, 11, 5), (4, MID, None, 9)])
def test_quadrilinear_tag_marginals(hz_lib, n, dims, n_real, walkers):
    """The sums behind the two-Kronecker marginals of the merge tensor's curvature block
    (optim/spin_blocks.py:140-171,505-556) against the oracle's einsum restatement, their
    symmetry, and the host-side normalisation."""
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200.walker import two_kron_marginals
    wf = S.synthetic_wavefunction(4, n, n_real=n if n_real is None else n_real, **dims)
    rng = np.random.default_rng(31 + n)
    q = S.random_unit_quaternions(rng, (walkers, n))
    ca = rng.standard_normal(walkers).astype(np.float32)
    cp = rng.standard_normal(walkers).astype(np.float32)
    cw = hz.CompiledWaveFunction(wf)
    g, dq, la, ph, f = cw.vjp(q, ca, cp, chunk_size=4, factors="marginals")
    _, _, _, _, f0 = W.logpsi_vjp(wf, q, ca, cp, with_factors="marginals")
    for k in ("merge_T_left", "merge_T_right", "merge_T_stats", "merge_V_in", "merge_U_out"):
        _close(f[k], f0[k], k)
    assert np.array_equal(f["merge_T_right"], f["merge_T_right"].T)
    merged = sum(int((np.asarray(o) == 0).sum()) for o in wf.opcodes) * walkers
    assert abs(float(f["merge_T_stats"][1]) - merged) < 0.5
    left, right, repeats = two_kron_marginals(f, walkers, walkers)
    l0, r0, rep0 = two_kron_marginals(f0, walkers, walkers)
    assert abs(repeats - rep0) < 1e-6
    _close(left, l0, "sigma_left"); _close(right, r0, "sigma_right")
    # the trace normalisation makes tr(sigma_left) tr(sigma_right) = repeats^2 tr_L tr_R / trace
    assert np.isfinite(left).all() and np.isfinite(right).all()
    # the plain factor request is unchanged by the new fields
    _, _, _, _, f1 = cw.vjp(q, ca, cp, chunk_size=4, factors=True)
    assert "merge_T_left" not in f1 and np.allclose(f1["merge_V_in"], f["merge_V_in"], rtol=1e-5, atol=1e-6)


def test_vjp_default_model_sizes_at_64_sites(hz_lib):
    """The headline benchmark's wavefunction (64 sites, d_m 1536, ranks 256/256/128): two walkers
    against the oracle, with the factor sums."""
    import hamiltonzero_b200 as hz
    n = 64
    wf = S.synthetic_wavefunction(0, n)
    q = S.corner_quaternions(np.random.default_rng(4).integers(0, 2, (2, n)))
    ca = np.array([1.0, -1.0], np.float32)
    cp = np.array([-1.0, 1.0], np.float32)
    cw = hz.CompiledWaveFunction(wf)
    g, dq, la, ph, f = cw.vjp(q, ca, cp, factors=True)
    g0, dq0, la0, ph0, f0 = W.logpsi_vjp(wf, q, ca, cp, with_factors=True)
    assert np.abs(la - la0).max() <= 1e-5 * np.abs(la0).max()
    _close(dq, dq0, "dq")
    for k in ("q_weight", "leaf_V", "leaf_U", "leaf_h", "merge_T", "merge_V", "merge_U", "readout_V",
              "readout_U", "readout_h"):
        _close(g[k], g0[k], k)
    for a, b in zip(g["merge_h"], g0["merge_h"]):
        _close(a, b, "merge_h")
    for k in ("merge_V_in", "merge_V_out", "merge_U_in", "merge_U_out", "leaf_U_out", "leaf_V_out",
              "readout_V_in", "q_out"):
        _close(f[k], f0[k], k)


def test_vjp_is_bitwise_reproducible(hz_lib):
    """Gradients and factor sums of two identical calls are equal bit for bit: the split
    A^T B products add their partial tiles in a fixed order (no atomic accumulation), at a size
    where every product is split over many CTAs (64 sites, default widths, 96 walkers)."""
    import hamiltonzero_b200 as hz
    n = 64
    wf = S.synthetic_wavefunction(0, n)
    rng = np.random.default_rng(11)
    q = S.random_unit_quaternions(rng, (96, n))
    ca = rng.choice([-1.0, 1.0], 96).astype(np.float32)
    cp = rng.standard_normal(96).astype(np.float32)
    cw = hz.CompiledWaveFunction(wf)
    runs = [cw.vjp(q, ca, cp, chunk_size=32, factors="marginals") for _ in range(2)]
    (g1, dq1, la1, ph1, f1), (g2, dq2, la2, ph2, f2) = runs
    assert np.array_equal(dq1, dq2) and np.array_equal(la1, la2) and np.array_equal(ph1, ph2)
    for k in g1:
        a, b = g1[k], g2[k]
        if isinstance(a, (list, tuple)):
            assert all(np.array_equal(x, y) for x, y in zip(a, b)), k
        else:
            assert np.array_equal(a, b), k
    for k in f1:
        a, b = f1[k], f2[k]
        if isinstance(a, (list, tuple)):
            assert all(np.array_equal(x, y) for x, y in zip(a, b)), k
        else:
            assert np.array_equal(a, b), k


def test_vjp_argument_checks(hz_lib):
    """Status codes of the C entry point: missing arrays, a workspace that is too small or
    misaligned, and shapes the host mirror refuses."""
    import ctypes
    import torch
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200 import _lib
    lib = _lib.load()
    wf = S.synthetic_wavefunction(1, 4, **SMALL)
    cw = hz.CompiledWaveFunction(wf)
    q = torch.from_numpy(S.random_unit_quaternions(np.random.default_rng(0), (3, 4))).cuda()
    c = torch.ones(3, device="cuda")
    need = lib.hz_vjp_workspace_bytes(ctypes.byref(cw.c), 3, 0)
    assert need > 0 and lib.hz_vjp_workspace_bytes(ctypes.byref(cw.c), 0, 0) == -1
    assert lib.hz_vjp_workspace_bytes(ctypes.byref(cw.c), 3, 1) > need
    ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    g = {k: torch.empty_like(cw.t[k]) for k in cw.GRAD_NAMES}
    full = _lib.WavefunctionGrads(**{k: g[k].data_ptr() for k in cw.GRAD_NAMES})
    call = lambda grads, wptr, nbytes: lib.hz_logpsi_vjp(
        ctypes.byref(cw.c), q.data_ptr(), 3, c.data_ptr(), c.data_ptr(), grads, None, 0, 0, 0, wptr,
        nbytes, None)
    assert call(ctypes.byref(full), ws.data_ptr(), need) == 0
    assert call(None, ws.data_ptr(), need) == 1                         # HZ_ERR_NULL_POINTER
    holes = _lib.WavefunctionGrads(**{k: (0 if k == "merge_T" else g[k].data_ptr()) for k in cw.GRAD_NAMES})
    assert call(ctypes.byref(holes), ws.data_ptr(), need) == 1
    assert call(ctypes.byref(full), ws.data_ptr(), 1024) == 7           # HZ_ERR_WORKSPACE
    assert call(ctypes.byref(full), ws.data_ptr() + 4, need) == 4       # HZ_ERR_MISALIGNED
    torch.cuda.synchronize()
    with pytest.raises(ValueError):
        cw.vjp(np.zeros((3, 8, 4), np.float32), np.ones(3), np.ones(3))
    with pytest.raises(ValueError):
        cw.vjp(q, np.ones(2, np.float32), np.ones(3, np.float32))
