"""CPU tests of the system featuriser: hand-worked polar split, presence rule and strength
features (which pin the oracle), and the vectorised torch code in float64 against the oracle's
per-bond and per-site loops, with absent bonds, absent fields and padded sites."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import context as C
from hamiltonzero_b200 import featurizer as F
from oracle import featurizer as O


def _dbl(t):
    if isinstance(t, dict):
        return {k: _dbl(v) for k, v in t.items()}
    return t.double() if isinstance(t, torch.Tensor) else t


def _params(seed=0):
    return F.init_system_featurizer(seed, d_bond=12, n_heads=2, head_dim=4, n_global_q=3, d_edge=10,
                                    d_hidden_edge=16, polar_group_norm_bond_hidden=24,
                                    polar_group_norm_n_bond_groups=4, polar_group_norm_d_bond_group=6,
                                    polar_group_norm_n_zeeman_groups=3, polar_group_norm_d_zeeman_group=4,
                                    zeeman_hidden_dim=12, global_hidden_dim=20, combine_hidden_dim=18,
                                    token_initial_scale=0.02, device="cpu")


def _system(seed, n, n_real, with_field=True, density=0.5):
    rng = np.random.default_rng(seed)
    J = np.zeros((n, n, 10))
    for i in range(n_real):
        for j in range(i + 1, n_real):
            if rng.random() < density:
                blk = rng.standard_normal((3, 3))
                J[i, j, :9] = blk.reshape(-1); J[j, i, :9] = blk.T.reshape(-1)
        J[i, i, 9] = 1.0
    h = np.zeros((n, 3))
    if with_field:
        h[:n_real:2] = rng.standard_normal((len(range(0, n_real, 2)), 3))      # every other site has a field
    mask = (np.arange(n) < n_real).astype(np.float64)
    return J, mask, h


def test_polar_split_presence_and_strengths_by_hand():
    r, u = O.polar_split(np.array([3.0, 4.0, 0.0]), 1e-3)
    assert abs(r[0] - 5.0) < 1e-12 and np.allclose(u, [0.6, 0.8, 0.0], atol=1e-7)
    r0, u0 = O.polar_split(np.zeros(3), 1e-3)
    assert r0[0] == 0.0 and np.all(u0 == 0.0)                      # no division by zero
    rt, ut = F.polar_split(torch.tensor([[3.0, 4.0, 0.0]], dtype=torch.float64), 1e-3)
    assert abs(float(rt) - 5.0) < 1e-12 and np.allclose(ut.numpy()[0], u, atol=1e-12)
    j = np.zeros(10)
    assert not O.bond_present(j)
    j[9] = 1.0
    assert O.bond_present(j)                                       # the diagonal flag alone
    j[9] = 0.0; j[4] = -0.2
    assert O.bond_present(j)
    # two sites, one bond of squared magnitude 9 in each direction, fields of squared length 16 and 0
    J = np.zeros((2, 2, 10)); J[0, 1, 0] = 3.0; J[1, 0, 0] = 3.0
    h = np.array([[4.0, 0.0, 0.0], [0.0, 0.0, 0.0]])
    f = O.strength_features(J, np.ones(2), h)
    rj, rh = 3.0, np.sqrt(8.0)
    th = np.arctan2(rh, rj)
    np.testing.assert_allclose(f, [np.log1p(rj), np.log1p(rh), np.sin(2 * th), np.cos(2 * th), np.sin(4 * th),
                                   np.cos(4 * th), np.sin(8 * th), np.cos(8 * th)], atol=1e-12)
    np.testing.assert_allclose(O.strength_features(np.zeros((2, 2, 10)), np.ones(2), np.zeros((2, 3))),
                               [0, 0, 0, 1, 0, 1, 0, 1], atol=1e-12)


@pytest.mark.parametrize("n,n_real,with_field", [(6, 6, True), (8, 5, True), (6, 4, False)])
def test_featurizer_matches_the_oracle_loops(n, n_real, with_field):
    p = _params(n)
    pd, pn = _dbl(p), C.to_numpy(p)
    J, mask, h = _system(n + n_real, n, n_real, with_field)
    tt = torch.from_numpy
    edge, local, glob = F.system_featurizer(pd, tt(J), tt(mask), tt(h))
    edge0, local0, glob0 = O.system_featurizer(pn, J, mask, h)
    np.testing.assert_allclose(glob.numpy(), glob0, rtol=2e-6, atol=2e-7)
    np.testing.assert_allclose(local.numpy(), local0, rtol=2e-6, atol=2e-7)
    np.testing.assert_allclose(edge.numpy(), edge0, rtol=2e-6, atol=2e-7)
    assert np.all(edge.numpy()[n_real:] == 0) and np.all(edge.numpy()[:, n_real:] == 0)
    assert np.all(local.numpy()[n_real:] == 0)
    assert edge.shape == (n, n, 10) and local.shape == (n, 8) and glob.shape == (24,)
    # padded sites carry no weight: changing their inputs changes nothing (their fields only where
    # some real site has one: "any field present" is taken over all slots, as in the reference)
    if n_real < n:
        J2, h2 = J.copy(), h.copy()
        J2[n_real:] += 1.0; J2[:, n_real:] -= 1.0
        if with_field:
            h2[n_real:] += 2.0
        e2, l2, g2 = F.system_featurizer(pd, tt(J2), tt(mask), tt(h2))
        np.testing.assert_allclose(g2.numpy(), glob.numpy(), rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(l2.numpy(), local.numpy(), rtol=1e-6, atol=1e-7)
