"""Basis-state sampler and SWAP estimator: host rules on CPU, and on the GPU a 4-spin system whose
16 amplitudes are enumerated, so that the sampled distribution and the purity of a subsystem have
exact answers."""
import itertools
import math

import numpy as np
import pytest
import torch

from hamiltonzero_b200 import systems as S


def test_acceptance_rules_and_log_polar_mean():
    from hamiltonzero_b200 import renyi2 as R
    inf = math.inf
    cur = torch.tensor([0.0, 0.0, -inf, -inf, float("nan"), 0.0, 1.0])
    prop = torch.tensor([1.0, -1.0, -inf, 0.5, 0.0, float("nan"), -inf])
    got = R.metropolis_log_acceptance(cur, prop)
    want = [0.0, -2.0, 0.0, 0.0, 0.0, -inf, -inf]
    assert all((g == w) or (math.isinf(w) and math.isinf(g)) for g, w in zip(got.tolist(), want))
    # mean of e^{i pi/3} * {1, e^2}: pivoted, no overflow at large logs
    la, ph = R.complex_mean_log_polar(torch.tensor([1000.0, 1002.0]), torch.tensor([math.pi / 3] * 2))
    assert abs(la - (1000.0 + math.log((1 + math.e ** 2) / 2))) < 1e-9 and abs(ph - math.pi / 3) < 1e-6
    assert R.complex_mean_log_polar(torch.tensor([-inf]), torch.tensor([0.0])) == (-inf, 0.0)
    with pytest.raises(ValueError):
        R.complex_mean_log_polar(torch.tensor([inf]), torch.tensor([0.0]))
    m = R.subsystem_mask([0, 2], n_spins=4)
    assert m.tolist() == [True, False, True, False]
    with pytest.raises(ValueError):
        R.subsystem_mask([0, 0], n_spins=4)
    q = R.routed_corners(torch.tensor([[True, False, True]]), torch.tensor([1, 0, 3, 2]), n_spins=3)
    # routed bits (padded with up): [bits[1], bits[0], pad, bits[2]] = [up, down, up, down]
    assert q[0].tolist() == [[1, 0, 0, 0], [0, 0, 1, 0], [1, 0, 0, 0], [0, 0, 1, 0]]


@pytest.mark.gpu
def test_basis_chain_and_swap_estimator_against_enumeration(hz_lib):
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200 import renyi2 as R
    n = 4
    dims = dict(d_o=8, d_m=64, d_r=32, r_leaf=16, r_merge=16, r_ro=8)
    wf = hz.CompiledWaveFunction(S.synthetic_wavefunction(7, n, **dims))
    route = np.arange(n)
    states = np.array(list(itertools.product([0, 1], repeat=n)), dtype=bool)           # [16, 4]
    la, ph = R.basis_log_wavefunction(wf, torch.tensor(states), route, n_spins=n)
    amp = np.exp(la.double().cpu().numpy() + 1j * ph.double().cpu().numpy())
    prob = np.abs(amp) ** 2
    prob /= prob.sum()
    psi = amp / np.sqrt((np.abs(amp) ** 2).sum())
    # exact purity of sites {0, 1}: tr rho_A^2 with rho_A = M M^dagger, M[a, b] = psi[a b]
    M = psi.reshape(4, 4)
    rho = M @ M.conj().T
    purity = float(np.real(np.trace(rho @ rho)))
    sx, bits_x = R.burn_in_basis(wf, route, n, seed=1, batch_size=4096, burn_in=64)
    sy, bits_y = R.burn_in_basis(wf, route, n, seed=2, batch_size=4096, burn_in=64)
    assert 0 < sx.accepted <= sx.proposed == 4096 * 64
    code = (bits_x.long().cpu().numpy() * (2 ** np.arange(n - 1, -1, -1))).sum(1)
    hist = np.bincount(code, minlength=16) / len(code)
    assert np.abs(hist - prob).max() < 5.0 * np.sqrt(prob.max() / len(code)) + 0.01
    sx, bits_x = R.step_basis(wf, route, n, sx, steps=4)
    out = R.renyi2(wf, route, n, [0, 1], bits_x, bits_y)
    ratios = np.exp(out["swap_log_abs"].double().cpu().numpy()) * np.cos(out["swap_phase"].double().cpu().numpy())
    err = ratios.std() / math.sqrt(len(ratios))
    assert abs(out["purity"] - purity) < 5 * err + 1e-3
    assert abs(out["renyi2_nats"] + math.log(purity)) < 0.1
    # the whole system and the empty set are exact identities
    assert R.renyi2(wf, route, n, [], bits_x, bits_y)["purity"] == pytest.approx(1.0, abs=1e-12)
    assert R.renyi2(wf, route, n, [0, 1, 2, 3], bits_x, bits_y)["purity"] == pytest.approx(1.0, abs=1e-12)
