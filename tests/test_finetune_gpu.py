"""The fine-tune loss around the reverse pass on the GPU: the gradient that
``finetune_loss_and_gradient`` returns is the transpose of the reference's loss tangent
(src/hamiltonzero/optim/production.py:194-226), checked against a central difference of the
float64 oracle along random parameter directions, and the Fisher pass against the oracle's
factor sums."""
from dataclasses import replace

import numpy as np
import pytest
import torch

from hamiltonzero_b200 import finetune, systems as S
from oracle import walker as W

pytestmark = pytest.mark.gpu

MID = dict(d_o=16, d_m=256, d_r=32, r_leaf=32, r_merge=64, r_ro=32)


def _loss_tangent(wf, q, energy, name, direction, eps=1e-6):
    """2 (sum tan_re Re dE + sum tan_im Im dE) / n_eff with the tangents of (log|psi|, phase)
    along ``direction`` of parameter ``name`` from a central difference of the oracle."""
    def at(sign):
        moved = replace(wf, **{name: (getattr(wf, name).astype(np.float64)
                                       + sign * eps * direction)})
        return W.execute_wavefunction(moved, q)
    (la_p, ph_p), (la_m, ph_m) = at(+1), at(-1)
    tan_re = (la_p - la_m) / (2 * eps)
    tan_im = np.angle(np.exp(1j * (ph_p - ph_m))) / (2 * eps)
    e = energy.astype(np.complex128)[0]
    delta = e - e.mean()
    n_eff = max((np.abs(delta) > 0).sum(), 1)
    return 2.0 * ((tan_re * delta.real).sum() + (tan_im * delta.imag).sum()) / n_eff


def test_gradient_is_the_transpose_of_the_loss_tangent(hz_lib):
    import hamiltonzero_b200 as hz
    n, walkers = 16, 24
    wf = S.synthetic_wavefunction(5, n, n_real=13, **MID)
    rng = np.random.default_rng(0)
    q = S.random_unit_quaternions(rng, (1, walkers, n))
    energy = (rng.standard_normal((1, walkers)) + 1j * rng.standard_normal((1, walkers))).astype(np.complex64)
    cw = hz.CompiledWaveFunction(wf)
    loss, g = finetune.finetune_loss_and_gradient(cw, torch.from_numpy(q), torch.from_numpy(energy),
                                                  chunk_size=7)
    assert abs(float(loss) - energy.real.mean()) < 1e-6
    for name in ("merge_V", "merge_U", "leaf_U", "readout_V", "merge_T"):
        direction = rng.standard_normal(getattr(wf, name).shape)
        want = _loss_tangent(wf, q[0], energy, name, direction)
        grad = g[name].double().cpu().numpy()
        got = float((grad * direction).sum())
        # gradient samples are held to 1e-4 relative: the contraction with a direction is then
        # good to 1e-4 of |grad| |direction| (Cauchy-Schwarz), which is what is asserted
        assert abs(got - want) <= 1e-4 * np.linalg.norm(grad) * np.linalg.norm(direction), (name, got, want)
        assert abs(got - want) <= 2e-3 * abs(want), (name, got, want)


def test_fisher_pass_uses_the_signs_as_cotangents(hz_lib):
    import hamiltonzero_b200 as hz
    n, walkers = 8, 11
    wf = S.synthetic_wavefunction(6, n, n_real=6, **MID)
    q = S.random_unit_quaternions(np.random.default_rng(1), (1, walkers, n))
    cw = hz.CompiledWaveFunction(wf)
    signs = finetune.make_fisher_signs(7, torch.from_numpy(q))
    assert signs.shape == (1, walkers, 3) and set(np.unique(signs.numpy())) <= {-1.0, 1.0}
    mask = (np.arange(n) < 6).astype(np.uint8)
    f, count = finetune.fisher_factor_sums(cw, torch.from_numpy(q), signs, leaf_mask=mask)
    assert count == walkers
    s = signs.numpy()[0]
    _, _, _, _, f0 = W.logpsi_vjp(wf, q[0], s[:, 0], s[:, 1], with_factors="marginals", leaf_mask=mask)
    for k in ("merge_V_in", "merge_V_out", "merge_U_out", "readout_V_in", "merge_T_left", "merge_T_right"):
        want = np.asarray(f0[k], np.float64)
        got = f[k].double().cpu().numpy()
        assert np.abs(got - want).max() <= 1e-4 * max(np.abs(want).max(), 1e-6), k
