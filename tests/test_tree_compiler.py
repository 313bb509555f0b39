"""CPU tests of the context-only tree reduction: hand-worked clocks, count features and opcodes
(which pin the oracle), and the vectorised pieces in float64 against the oracle's per-pair and
per-cell loops. The whole reduction needs the attention kernel: tests/test_tree_compiler_gpu.py."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import context as C
from hamiltonzero_b200 import tree_compiler as T
from oracle import tree_compiler as O

MERGE, CARRY_LEFT, CARRY_RIGHT, EMPTY = 0, 1, 2, 3


def _dbl(t):
    if isinstance(t, dict):
        return {k: _dbl(v) for k, v in t.items()}
    if isinstance(t, list):
        return [_dbl(v) for v in t]
    return t.double() if isinstance(t, torch.Tensor) else t


def _params(edge_node_ctx_dim=None):
    return T.init_physical_compiler(5, d_e=20, d_edge=12, d_c=16, d_feat=24, d_g=10, tap_dim=8, r_leaf=6,
                                    r_merge=7, r_ro=5, alpha_init=0.3, n_heads=2, attn_dim=16, attn_impl="einsum",
                                    edge_node_ctx_dim=edge_node_ctx_dim, fwl_channels=8, pool_heads=2, pool_d_k=8,
                                    pool_d_v=8, device="cpu")


def test_clocks_by_hand():
    np.testing.assert_allclose(O.coord_clock(0.0, 4), [0, 0, 1, 1])
    # width 3: half = 2, frequencies 1 and 10000^-1/2 = 0.01; the second cosine is cut off
    np.testing.assert_allclose(O.coord_clock(100.0, 3), [np.sin(100.0), np.sin(1.0), np.cos(100.0)], atol=1e-12)
    # first pair of a two-leaf tree: its segment is the whole tree, centred on the root
    np.testing.assert_allclose(O.merge_clock(0, 0, 6, 1), [0, 0, 1, 1, np.sin(2.0), np.cos(2.0)], atol=1e-12)
    # third pair of the leaf level of a 16-leaf tree: leaves 4 and 5, centre 4.5 - 7.5
    np.testing.assert_allclose(O.merge_clock(0, 2, 4, 4)[:2], [np.sin(-3.0), np.cos(-3.0)], atol=1e-12)
    got = T.tree_merge_clock(1, torch.arange(4), 16, 3).numpy()
    want = np.stack([O.merge_clock(1, p, 16, 3) for p in range(4)])
    np.testing.assert_allclose(got, want, atol=2e-6)
    assert T.tree_coord_clock(torch.zeros(3), 0).shape == (3, 0)


def test_count_features_and_depth_by_hand():
    f = O.depth_count_features(1.0, 1.0, 2.0, 0, 1)
    s = np.sin(np.pi / np.array([1, 2, 4, 8])); c = np.cos(np.pi / np.array([1, 2, 4, 8]))
    want = np.concatenate([s, c, s, c, np.zeros(4), np.ones(4), [0, 0, 1, 1], [0, 0, 1, 1]])
    np.testing.assert_allclose(f, want, atol=1e-12)
    got = T.tree_depth_count_features(torch.tensor([1.0, 3.0]), torch.tensor([1.0, 2.0]), 11.0, 2, 4).numpy()
    np.testing.assert_allclose(got[0], O.depth_count_features(1.0, 1.0, 11.0, 2, 4), atol=2e-6)
    np.testing.assert_allclose(got[1], O.depth_count_features(3.0, 2.0, 11.0, 2, 4), atol=2e-6)
    for n, d in ((0, 1), (1, 1), (2, 1), (3, 2), (5, 3), (64, 6)):
        mask = np.arange(64) < n
        assert O.active_clock_depth(mask) == d and T.tree_active_clock_depth(torch.from_numpy(mask)) == d


def test_opcodes_by_hand():
    ops = T.classify_merge_opcodes(torch.tensor([1, 1, 1, 0, 0, 0, 0, 0]))
    assert [o.tolist() for o in ops] == [[MERGE, CARRY_LEFT, EMPTY, EMPTY], [MERGE, EMPTY], [CARRY_LEFT]]
    ops = T.classify_merge_opcodes(torch.tensor([0, 1, 1, 1]))
    assert [o.tolist() for o in ops] == [[CARRY_RIGHT, MERGE], [MERGE]]
    with pytest.raises(ValueError):
        T.classify_merge_opcodes(torch.ones(6))


@pytest.mark.parametrize("ctx_dim", [None, 5])
def test_level_pieces_match_the_oracle_loops(ctx_dim):
    """Candidate contexts, the edge merge over all cells, the 2-FWL edge update and the global
    update of one level (8 nodes, the last pair without structural children) in float64."""
    p = _params(ctx_dim)
    pd, pn = _dbl(p), C.to_numpy(p)
    rng = np.random.default_rng(2)
    n = 8
    c = rng.standard_normal((n, 16)); e = rng.standard_normal((n, n, 12)); g = rng.standard_normal(24)
    k = np.array([1, 1, 1, 1, 1, 0, 0, 0], dtype=np.float64)
    tt = torch.from_numpy
    g_level = g @ pn["gladder"]["tree_proj_w"] + pn["gladder"]["tree_proj_b"]
    depth = np.stack([O.depth_count_features(k[2 * i], k[2 * i + 1], 5.0, 1, 3) for i in range(4)])
    idx = np.arange(4)
    got = T.context_candidate(pd["merge"], tt(c[0::2]), tt(c[1::2]), tt(g_level), tt(e[2 * idx, 2 * idx + 1]),
                              tt(e[2 * idx + 1, 2 * idx]), 1, 3, tt(depth)).numpy()
    want = np.stack([O.context_candidate(pn["merge"], c[2 * i], c[2 * i + 1], g_level, e[2 * i, 2 * i + 1],
                                         e[2 * i + 1, 2 * i], 1, i, 3, depth[i]) for i in range(4)])
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)        # the clock is evaluated in fp32
    got = T.edge_merge_level(pd["merge"]["edge_merge"], tt(e), tt(c), tt(k)).numpy()
    want = np.stack([np.stack([O.edge_merge_cell(
        pn["merge"]["edge_merge"], (e[2 * i, 2 * j], e[2 * i, 2 * j + 1], e[2 * i + 1, 2 * j], e[2 * i + 1, 2 * j + 1]),
        (c[2 * i], c[2 * i + 1], c[2 * j], c[2 * j + 1]), (k[2 * i], k[2 * i + 1], k[2 * j], k[2 * j + 1]))
        for j in range(4)]) for i in range(4)])
    np.testing.assert_allclose(got, want, rtol=1e-11, atol=1e-12)
    assert np.all(got[2:] == 0) and np.all(got[:, 2:] == 0) and np.abs(got[:2, :2]).min() > 0
    both = k[0::2] * k[1::2]
    e4, c4 = rng.standard_normal((4, 4, 12)), rng.standard_normal((4, 16))
    got = T.edge_fwl_residual(pd["merge"]["tree_edge_fwl"], tt(e4), tt(c4), tt(both)).numpy()
    np.testing.assert_allclose(got, O.edge_fwl_residual(pn["merge"]["tree_edge_fwl"], e4, c4, both),
                               rtol=1e-11, atol=1e-12)
    np.testing.assert_array_equal(got[2:], e4[2:])                     # inactive cells keep their value
    pool = rng.standard_normal(16)
    got = T.tree_global_update(pd["gladder"]["tree_update"], tt(g), tt(pool), True).numpy()
    np.testing.assert_allclose(got, O.tree_global_update(pn["gladder"]["tree_update"], g, pool, True), rtol=1e-12)
    assert T.tree_global_update(pd["gladder"]["tree_update"], tt(g), tt(pool), False) is not None
    np.testing.assert_array_equal(T.tree_global_update(pd["gladder"]["tree_update"], tt(g), tt(pool), False).numpy(), g)


def test_conditioner_projections_and_assembly():
    p = _params()
    pd, pn = _dbl(p), C.to_numpy(p)
    rng = np.random.default_rng(3)
    tt = torch.from_numpy
    e_leaf, g10 = rng.standard_normal((4, 20)), rng.standard_normal(10)
    np.testing.assert_allclose(T.compile_target_leaf_h(pd["leaf"], tt(e_leaf), tt(g10))[0].numpy(),
                               O.leaf_h(pn["leaf"], e_leaf, g10), rtol=1e-12)
    e_root, c_root = rng.standard_normal(12), rng.standard_normal(16)
    np.testing.assert_allclose(T.compile_target_readout_h(pd["readout"], tt(e_root), tt(c_root), tt(g10))[0].numpy(),
                               O.readout_h(pn["readout"], e_root, c_root, g10), rtol=1e-12)
    g24 = rng.standard_normal(24)
    np.testing.assert_allclose(T.project_global(pd["root_projection"], tt(g24)).numpy(),
                               O.project_global(pn["root_projection"], g24), rtol=1e-12)
    tree = T.assemble_compiled_tree(perm=torch.tensor([2, 0, 3, 1]), leaf_real=torch.tensor([1, 1, 1, 0]),
                                    boundaries={"leaf_h": (torch.zeros(4, 6),), "leaf_combiner_h": (),
                                                "merge_h": (torch.zeros(2, 7), torch.zeros(1, 7)),
                                                "opcodes": T.classify_merge_opcodes(torch.tensor([1, 1, 1, 0])),
                                                "readout_h": (torch.zeros(5),), "readout_combiner_h": ()})
    assert tree.inv_perm.tolist() == [1, 3, 0, 2] and tree.leaf_real.tolist() == [True, True, True, False]
    assert [o.tolist() for o in tree.opcodes] == [[MERGE, CARRY_LEFT], [MERGE]]
    with pytest.raises(ValueError):
        T.assemble_compiled_tree(perm=torch.zeros(2, 2), leaf_real=torch.ones(2), boundaries={})
    with pytest.raises(ValueError):
        T.compile_context_only_reduction(pd["merge"], pd["gladder"], torch.zeros(6, 16), torch.ones(6),
                                         torch.zeros(24), torch.zeros(6, 6, 12), torch.ones(6))
    with pytest.raises(ValueError):
        T.init_physical_compiler(0, d_e=4, d_edge=4, d_c=4, d_feat=8, d_g=4, tap_dim=8, r_leaf=2, r_merge=2,
                                 r_ro=2, device="cpu")


def test_contextualiser_clock_and_argument_checks():
    from oracle import context as OC
    # five active slots: the subtree spans 8 leaves, positions are taken from its centre 3.5
    bmask = (np.arange(8) < 5).astype(np.float64)
    clock = OC._slot_clock(8, 4, bmask, 10000.0, 1.0)
    np.testing.assert_allclose(clock[0], [np.sin(-3.5), np.sin(-3.5 * 0.01), np.cos(-3.5), np.cos(-3.5 * 0.01)],
                               atol=1e-12)
    np.testing.assert_allclose(C._slot_clock(8, 4, torch.from_numpy(bmask), 10000.0, 1.0).numpy(), clock, atol=2e-6)
    assert OC._direction(3)[:, :, 0].tolist() == [[0, 1, 1], [-1, 0, 1], [-1, -1, 0]]
    good = dict(d_e=8, d_edge=4, n_layers=1, n_heads=2, summary_hidden=8, mlp_hidden=8, bias_hidden=8,
                edge_ffn_hidden=8, attn_dim=8, edge_node_ctx_dim=2, gladder_d_g=8, global_tap_dim=4, pool_heads=1,
                pool_d_k=4, pool_d_v=4, device="cpu")
    p = C.init_physical_readout_context(0, **good)
    assert p["layers"][0]["W_QKV"].shape == (8, 3 * 4 * 4) and p["layers"][0]["edge_ffn"]["in_proj"]["weight"].shape[0] == 4 + 4 + 64
    for bad in (dict(n_layers=0), dict(n_heads=0), dict(attn_dim=6), dict(d_e=7), dict(attn_dim=4, n_heads=4),
                dict(attn_impl="flash"), dict(rope_base=0.0), dict(global_tap_dim=8)):
        with pytest.raises(ValueError):
            C.init_physical_readout_context(0, **{**good, **bad})
    from hamiltonzero_b200 import types as Ty
    shared = Ty.SharedTrunk(torch.zeros(4, 8), torch.zeros(4, 4, 4), None, torch.zeros(8), torch.ones(4), torch.ones(4))
    with pytest.raises(ValueError):
        T.compile_physical_tree_from_shared_trunk({}, shared, torch.arange(3))
