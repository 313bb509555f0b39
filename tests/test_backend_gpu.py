"""The reference-shaped entry points of the walker path: the (kernel, tree) argument lists of
energy/compiled.py:17-31, observables.py:31-59 and mcmc/runtime.py:88-129, and the
EvalBackend-shaped class, against the oracle and against the package's short forms."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import systems as S
from oracle import walker as W

pytestmark = pytest.mark.gpu
MID = dict(d_o=16, d_m=256, d_r=32, r_leaf=32, r_merge=64, r_ro=16)


def test_reference_argument_lists(hz_lib):
    import hamiltonzero_b200 as hz
    n = 16
    frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(13, 0.4, seed=7), n)
    arrays = S.synthetic_wavefunction(1, n, n_real=13, **MID)
    kernel, tree = hz.types.from_arrays(arrays)
    assert kernel.merge_factors[0].V is arrays.merge_V and tree.merge_h[1] is arrays.merge_h[1]
    q = S.random_unit_quaternions(np.random.default_rng(3), (3, 2, n))
    # energy: (kernel, tree, energy_frame, q_routed, *, chunk_size)
    got = hz.vmc_energy_custom_lap_compiled(kernel, tree, frame, q, chunk_size=4)
    ref = W.local_energy(arrays, frame, q)
    assert got[0].shape == (3, 2)
    _, _, lap = W.forward_laplacian(arrays, frame, q.reshape(-1, n, 4))
    scale = (np.abs(lap[:, 0] + 1j * lap[:, 1]) + abs(float(frame.radial_const)) + 1.0).reshape(3, 2)
    assert (np.abs(got[0] - ref[0]) / scale).max() <= 1e-5
    wf = hz.CompiledWaveFunction(kernel, tree)
    same = hz.vmc_energy_custom_lap_compiled(wf, frame, q, chunk_size=None)
    assert np.array_equal(same[0], got[0])
    # spin: (wavefunction, context, q_routed, *, chunk_size) with context.mask
    spin = hz.local_spin(wf, frame, q, chunk_size=2)
    spin0 = W.local_spin(arrays, frame.mask, q)
    assert spin.shape == (3, 2, n, 3)
    assert np.abs(spin - spin0).max() <= 1e-4 * np.abs(spin0).max()
    assert np.all(spin[..., 13:, :] == 0)
    # the value-and-Jacobian pass agrees with the Jacobian of the energy pass
    la, ph, grad = hz.logpsi_and_chart_gradient(wf, q)
    la0, ph0 = W.execute_wavefunction(arrays, q)
    assert np.abs(la.cpu().numpy() - la0).max() <= 1e-5 * np.abs(la0).max() + 1e-5
    with pytest.raises(ValueError):
        hz.local_spin(wf, frame, q[..., :8, :])
    with pytest.raises(ValueError):
        hz.vmc_energy_custom_lap_compiled(kernel, tree, frame, q, chunk_size=0)
    bad = hz.types.CompiledTree(**{**tree.__dict__, "leaf_combiner_h": (arrays.leaf_h,)})
    with pytest.raises(ValueError, match="combiners"):
        hz.CompiledWaveFunction(kernel, bad)


def test_eval_backend_cycle(hz_lib):
    """initialize -> prepare -> burn-in steps with adaptation -> cold walkers -> energy, through
    the EvalBackend-shaped class, with the reference's configuration objects."""
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200.backend import EnergyConfig, EvalMCMCConfig
    n = 8
    frame = S.frame_from_graph(S.chain_graph(n), n)
    arrays = S.synthetic_wavefunction(2, n, **MID)
    backend = hz.build_eval_backend()
    model = hz.CompiledWaveFunction(*hz.types.from_arrays(arrays))
    cfg = EvalMCMCConfig(batch_size=32, replicas=4, steps=3, walker_chunk_size=8)
    state = backend.initialize_mcmc(5, model, frame, cfg)
    model, context, state = backend.prepare_singular(model, frame, state)
    assert state.q.shape == (32, 4, n, 4)
    sigma0 = state.sigma.clone()
    for _ in range(2):
        state = backend.step_mcmc(state, model, context, replica_steps=cfg.steps,
                                  walker_chunk_size=cfg.walker_chunk_size)
        state = backend.adapt_mcmc(state, cfg)
    backend.block_until_ready(state.q)
    assert state.n_local == 0 and float(state.n_local_accept.sum()) == 0.0
    assert not torch.equal(state.sigma, sigma0)
    pop = backend.mcmc_population(state)
    state = backend.replace_mcmc_population(state, pop)
    q = backend.cold_walkers(state)
    assert q.shape == (32, n, 4)
    total, exchange, casimir, field = backend.custom_lap_energy(model, context, q, EnergyConfig(chunk_size=16))
    assert total.shape == (1, 32) and torch.isfinite(torch.view_as_real(total)).all()
    ref = W.local_energy(arrays, frame, q.cpu().numpy())
    assert np.abs(total[0].cpu().numpy() - ref[0]).max() <= 1e-3 * max(np.abs(ref[0]).max(), 1.0)
    # adapt_batched = the three adaptations in the reference's order with its defaults
    st = backend.step_mcmc(state, model, context, replica_steps=2, walker_chunk_size=8)
    a = hz.mcmc.adapt_batched(st)
    b = hz.mcmc.adapt_beta_equi_rej(hz.mcmc.adapt_m(hz.mcmc.adapt_sigma(st)), ema=0.9)
    assert torch.equal(a.sigma, b.sigma) and torch.equal(a.beta, b.beta) and torch.equal(a.m, b.m)
