"""GPU tests of the replica-exchange MALA sweep (through the C ABI).

Single moves are compared with the host restatement on identical random numbers (the draws
are injected); the sampler with its own Philox stream is checked through invariants: unit
quaternions, a cache that matches a recomputation, reproducibility, bounded counters."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import systems as S
from oracle import mcmc as M

pytestmark = pytest.mark.gpu
DIMS = dict(d_o=8, d_m=64, d_r=32, r_leaf=16, r_merge=16, r_ro=8)


MID = dict(d_o=16, d_m=256, d_r=32, r_leaf=32, r_merge=64, r_ro=16)


def _setup(n, n_real, B, R, seed=0, dims=DIMS):
    import hamiltonzero_b200 as hz
    wf = S.synthetic_wavefunction(seed, n, n_real=n_real, **(dims or {}))
    cw = hz.CompiledWaveFunction(wf)
    mask = (np.arange(n) < n_real).astype(np.int32)
    st = hz.mcmc.init_batched_state(seed + 1, mask, B, R, initial_m=2)
    return hz, wf, cw, mask, st


@pytest.mark.parametrize("n,n_real,B,R,steps,dims,chunk", [
    (4, 4, 16, 4, 2, DIMS, None),
    (8, 6, 16, 4, 2, DIMS, None),
    (64, 64, 2, 2, 1, None, None),        # default model sizes (d_m = 1536, rank 256)
    (64, 50, 6, 3, 2, MID, 4),            # ragged 64-site tree, chunked value-and-gradient passes
    (256, 256, 5, 2, 1, MID, 2),          # the largest tree, chunked
])
def test_one_sweep_matches_the_oracle_on_injected_draws(hz_lib, n, n_real, B, R, steps, dims, chunk):
    hz, wf, cw, mask, st = _setup(n, n_real, B, R, dims=dims)
    rng = np.random.default_rng(7)
    noise = dict(haar_scores=rng.random((B, R, n)), haar_raw=rng.standard_normal((B, R, n, 4)),
                 haar_logu=np.log(rng.random((B, R))),
                 local_noise=rng.standard_normal((steps, B, R, n, 3)),
                 local_logu=np.log(rng.random((steps, B, R))),
                 swap_logu=np.log(rng.random((steps, B, R - 1))))
    noise = {k: v.astype(np.float32) for k, v in noise.items()}
    new, la = hz.mcmc.run_batched(cw, st, steps, walker_chunk_size=chunk, noise=noise,
                                  return_log_alpha=True)
    torch.cuda.synchronize()
    # host restatement with the same numbers
    q = st.q.cpu().numpy().astype(np.float64)
    beta = st.beta.cpu().numpy().astype(np.float64); sigma = st.sigma.cpu().numpy().astype(np.float64)
    m = st.m.cpu().numpy()
    lp, dr = M.value_and_drift(wf, q)
    margin = np.full((B, R), np.inf)
    q, lp, dr, acc_h, la_h = M.haar_move(wf, q, lp, dr, beta, mask, m,
                                         noise["haar_scores"].astype(np.float64),
                                         noise["haar_raw"].astype(np.float64),
                                         noise["haar_logu"].astype(np.float64))
    margin = np.minimum(margin, np.abs(noise["haar_logu"] - la_h))
    log_alpha_ref = []
    for i in range(steps):
        q, lp, dr, acc, la_ref = M.mala_step(wf, q, lp, dr, beta, sigma, mask,
                                             noise["local_noise"][i].astype(np.float64),
                                             noise["local_logu"][i].astype(np.float64))
        log_alpha_ref.append(la_ref)
        margin = np.minimum(margin, np.abs(noise["local_logu"][i] - la_ref))
        q, lp, dr, eacc, elig, la_s = M.swap_move(q, lp, dr, beta, st.step + i,
                                                  noise["swap_logu"][i].astype(np.float64))
        sm = np.where(elig, np.abs(noise["swap_logu"][i] - la_s), np.inf).min(axis=1)
        margin = np.minimum(margin, sm[:, None])
    # the first MALA move starts from identical states: its log acceptance ratio must agree
    np.testing.assert_allclose(la[0].cpu().numpy(), log_alpha_ref[0], rtol=1e-4, atol=2e-3)
    # whole-sweep comparison for the walkers whose accept decisions were not marginal
    good = margin.min(axis=1) > 1e-2
    assert good.sum() >= min(3, B - 1)
    got_q = new.q.cpu().numpy()
    got_lp = new.log_p.cpu().numpy()
    np.testing.assert_allclose(got_q[good], q[good], rtol=0, atol=2e-5)
    np.testing.assert_allclose(got_lp[good], lp[good], rtol=0, atol=5e-4)
    # gradient samples: 1e-4 relative, with a floor of 1e-4 of the largest component
    np.testing.assert_allclose(new.drift.cpu().numpy()[good], dr[good], rtol=1e-4,
                               atol=1e-4 * max(np.abs(dr).max(), 1.0))


def test_sweep_invariants_with_internal_random_numbers(hz_lib):
    B, R, n, steps = 64, 4, 8, 6
    hz, wf, cw, mask, st = _setup(n, n, B, R, seed=3)
    a = hz.mcmc.run_batched(cw, st, steps)
    b = hz.mcmc.run_batched(cw, st, steps)                 # same seed and sweep counter
    c = hz.mcmc.run_batched(cw, a, steps)                  # next sweep: new draws
    torch.cuda.synchronize()
    assert torch.equal(a.q, b.q) and torch.equal(a.log_p, b.log_p)
    assert not torch.equal(a.q, c.q)
    for s in (a, c):
        assert torch.isfinite(s.q).all() and torch.isfinite(s.log_p).all()
        assert ((s.q * s.q).sum(-1) - 1).abs().max().item() < 1e-5
        la, _ = cw(s.q)                                    # cache equals a recomputation
        assert (2 * la - s.log_p).abs().max().item() < 2e-4 * max(1.0, s.log_p.abs().max().item())
        assert s.n_local_accept.min().item() >= 0 and s.n_local_accept.max().item() <= s.n_local
        assert s.n_swap.max().item() <= s.step
    assert a.step == steps and a.n_local == steps and a.n_haar == 1 and c.sweeps == 2
    # some moves are accepted and some rejected at sigma = 0.3
    rate = a.n_local_accept.sum().item() / (B * R * steps)
    assert 0.02 < rate < 0.999
    # chunked value-and-gradient passes give the same chain
    d = hz.mcmc.run_batched(cw, st, steps, walker_chunk_size=7)
    assert torch.equal(a.q, d.q)
    # adaptation keeps shapes and resets the counters
    e = hz.mcmc.adapt_beta_equi_rej(hz.mcmc.adapt_m(hz.mcmc.adapt_sigma(a)))
    assert e.n_local == 0 and e.n_haar == 0 and float(e.n_local_accept.sum()) == 0.0
    assert hz.mcmc.cold_samples(a).shape == (B, n, 4)


def test_large_tree_sweep_is_independent_of_the_walker_chunk(hz_lib):
    """The largest configuration's shape of call: a 256-site tree swept with
    ``walker_chunk_size = 64`` gives the chain of the unchunked call bit for bit, its cache
    equals a recomputation and the walkers stay unit quaternions."""
    B, R, n, steps = 130, 2, 256, 2
    hz, wf, cw, mask, st = _setup(n, n, B, R, seed=5, dims=MID)
    a = hz.mcmc.run_batched(cw, st, steps, walker_chunk_size=64)
    b = hz.mcmc.run_batched(cw, st, steps)
    torch.cuda.synchronize()
    assert torch.equal(a.q, b.q) and torch.equal(a.log_p, b.log_p) and torch.equal(a.drift, b.drift)
    assert torch.isfinite(a.q).all() and torch.isfinite(a.log_p).all()
    assert ((a.q * a.q).sum(-1) - 1).abs().max().item() < 1e-5
    la, _ = cw(a.q)
    assert (2 * la - a.log_p).abs().max().item() < 2e-4 * max(1.0, a.log_p.abs().max().item())


def test_sampler_targets_psi_squared_on_one_site(hz_lib):
    """Distributional check on a 1-site wavefunction: the cold chain's samples of
    log p must have the mean that direct Haar sampling reweighted by p gives."""
    import hamiltonzero_b200 as hz
    n = 1
    wf = S.synthetic_wavefunction(5, n, **DIMS)
    cw = hz.CompiledWaveFunction(wf)
    st = hz.mcmc.init_batched_state(11, np.ones(1, np.int32), 2048, 3, initial_m=1)
    for _ in range(6):
        st = hz.mcmc.run_batched(cw, st, 8)
    lp_cold = st.log_p[:, -1].double().cpu().numpy()
    rng = np.random.default_rng(0)
    qh = S.random_unit_quaternions(rng, (200000, 1))
    la, _ = cw(qh)
    w = np.exp(2 * la.astype(np.float64) - 2 * la.max())
    ref = (w * 2 * la).sum() / w.sum()
    spread = np.sqrt(((w * (2 * la - ref) ** 2).sum() / w.sum()))
    assert abs(lp_cold.mean() - ref) < 6 * spread / np.sqrt(len(lp_cold)) + 0.02 * spread
