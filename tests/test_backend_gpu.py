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


def test_finetune_cycle_sweep_energy_gradient_factors(hz_lib):
    """One cycle of the fine-tune configuration on a small lattice: sampler sweep with
    walker_chunk_size 64 -> local energy of the cold chain -> gradient of the centred-energy loss
    -> Fisher pass with the factor sums and the quadrilinear tag's marginals -> moving averages,
    damped inverses and a preconditioned gradient of every block kind. Energies and the gradient
    are checked against the oracle on the sampled walkers; the preconditioned directions against
    a direct solve with the damped factors."""
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200 import finetune, kfac
    n, B, R = 16, 96, 4
    frame = S.frame_from_graph(S.j1j2_square_graph(4), n)
    arrays = S.synthetic_wavefunction(3, n, **MID)
    model = hz.CompiledWaveFunction(arrays)
    state = hz.mcmc.init_batched_state(9, frame.mask, B, R)
    state = hz.mcmc.run_batched(model, frame, state, 6, 64)
    state = hz.mcmc.adapt_batched(state)
    q = hz.mcmc.cold_samples(state)                                     # [B, n, 4]
    total = hz.vmc_energy_custom_lap_compiled(model, hz.DeviceEnergyFrame(frame), q)[0]
    ref = W.local_energy(arrays, frame, q.cpu().numpy())
    scale = np.maximum(np.abs(ref[0]), 1.0)
    assert (np.abs(total.cpu().numpy() - ref[0]) / scale).max() <= 1e-3
    energy = total.reshape(1, B)
    loss, grads = finetune.finetune_loss_and_gradient(model, q[None], energy, chunk_size=40)
    assert abs(float(loss) - float(total.real.mean())) <= 1e-5 * max(abs(float(loss)), 1.0)
    e = total.cpu().numpy().astype(np.complex128)
    delta = e - e.mean()
    n_eff = max(int((np.abs(delta) > 0).sum()), 1)
    g0, _, _, _ = W.logpsi_vjp(arrays, q.cpu().numpy(), 2 * delta.real / n_eff, 2 * delta.imag / n_eff)
    for k in ("merge_V", "merge_U", "merge_T", "leaf_U", "readout_V"):
        want = np.asarray(g0[k], np.float64)
        got = grads[k].double().cpu().numpy()
        assert np.abs(got - want).max() <= 2e-4 * max(np.abs(want).max(), 1e-8), k
    signs = finetune.make_fisher_signs(1, q[None])
    factors, walkers = finetune.fisher_factor_sums(model, q[None], signs,
                                                   leaf_mask=np.asarray(frame.mask, np.uint8))
    assert walkers == B
    nodes = n - 1
    dense = kfac.DenseBlock(arrays.merge_V.shape[0], arrays.merge_V.shape[1], device="cuda")
    dense.update(factors["merge_V_in"], factors["merge_V_out"], float(B * nodes), logical_batch=B,
                 batch_size=B, ema_old=0.95, ema_new=1.0).update_inverse(1e-3)
    pre = dense.precondition(grads["merge_V"])
    a_d, g_d = kfac.pi_adjusted_kronecker_factors(dense.a.value, dense.g.value, damping=1e-3 / dense.scale())
    back = (a_d @ pre @ g_d) * dense.scale()
    assert (back - grads["merge_V"].double()).abs().max() <= 1e-6 * grads["merge_V"].abs().max()
    left, right, repeats = hz.walker.two_kron_marginals(factors, batch_size=B, logical_batch=B)
    G = arrays.merge_T.shape[0]
    tk = kfac.TwoKroneckerBlock(G * 32, 1024, device="cuda")
    tk.update(left, right, repeats, ema_old=0.95, ema_new=1.0).update_inverse(1e-3)
    pt = tk.precondition(grads["merge_T"])
    assert pt.shape == grads["merge_T"].shape and torch.isfinite(pt).all()
    assert float((pt.double() * grads["merge_T"].double()).sum()) > 0        # a descent direction
    diag = kfac.DiagonalBlock(tuple(factors["merge_h_diag"][0].shape), device="cuda")
    diag.update(factors["merge_h_diag"][0], batch_size=B, ema_old=0.95, ema_new=1.0)
    ph = diag.precondition(grads["merge_h"][0], 1e-3)
    assert torch.isfinite(ph).all() and ph.shape == grads["merge_h"][0].shape
