"""GPU parity of the context-only tree reduction (level attention on hz_mhsea_fwd, 2-FWL
contraction on hz_fwl2_panel) against the float64 oracle, and the compiled tree it emits fed
to the walker path."""
import dataclasses

import numpy as np
import pytest
import torch

from hamiltonzero_b200 import context as C
from hamiltonzero_b200 import systems as S
from hamiltonzero_b200 import tree_compiler as T
from hamiltonzero_b200 import types as Ty
from oracle import tree_compiler as O
from oracle import walker as W

pytestmark = pytest.mark.gpu

DIMS = dict(d_e=40, d_edge=12, d_c=32, d_feat=24, d_g=16, tap_dim=8, r_leaf=16, r_merge=16, r_ro=8)


def _inputs(seed, n, n_real, n_struct, dev):
    rng = np.random.default_rng(seed)
    e_leaf = rng.standard_normal((n, DIMS["d_e"])).astype(np.float32)
    edge = rng.standard_normal((n, n, DIMS["d_edge"])).astype(np.float32)
    g = rng.standard_normal(DIMS["d_feat"]).astype(np.float32)
    real = (np.arange(n) < n_real).astype(np.float32)
    struct = (np.arange(n) < n_struct).astype(np.float32)
    t = lambda x: torch.from_numpy(x).to(dev)
    return (e_leaf, edge, g, real, struct), tuple(t(x) for x in (e_leaf, edge, g, real, struct))


def _close(a, b, tol, what):
    a = np.asarray(a, dtype=np.float64)
    assert np.isfinite(a).all(), what
    assert np.abs(a - b).max() <= tol * np.abs(b).max(), f"{what}: {np.abs(a - b).max() / np.abs(b).max():.2e}"


# n_struct: the balanced subtree that holds the real leaves (next power of two)
@pytest.mark.parametrize("n,n_real,n_struct,impl,ctx_dim", [
    (2, 2, 2, "mhsea_tuned", None),
    (16, 16, 16, "einsum", None),
    (16, 11, 16, "mhsea_tuned", 6),
    (16, 5, 8, "mhsea_tuned", None),        # the upper half of the tree is carried, not merged
    (64, 64, 64, "mhsea_tuned", 6),
    (64, 40, 64, "mhsea_tuned", None),
])
def test_compiled_tree_matches_oracle(hz_lib, n, n_real, n_struct, impl, ctx_dim):
    params = T.init_physical_compiler(n + n_real, alpha_init=0.3, n_heads=2, attn_dim=32, attn_impl=impl,
                                      edge_node_ctx_dim=ctx_dim, fwl_channels=8, pool_heads=2, pool_d_k=8,
                                      pool_d_v=8, **DIMS)
    dev = params["leaf"]["P_c"]["weight"].device
    host, devs = _inputs(n, n, n_real, n_struct, dev)
    tree = T.compile_physical_tree(params, *devs)
    leaf_h, merge_h, opcodes, readout_h = O.compile_tree(C.to_numpy(params), *[x.astype(np.float64) for x in host])
    tol = 2e-4 if n == 64 else 5e-5
    _close(tree.leaf_h[0], leaf_h, 1e-5, "leaf_h")
    assert len(tree.merge_h) == len(merge_h) == n.bit_length() - 1
    struct = host[4] > 0
    for lvl, (a, b, op, op0) in enumerate(zip(tree.merge_h, merge_h, tree.opcodes, opcodes)):
        np.testing.assert_array_equal(op, op0)
        assert a.shape == (n >> (lvl + 1), DIMS["r_merge"])
        # pairs outside the structural subtree carry padding that no opcode consumes
        struct = struct[0::2] | struct[1::2]
        _close(a[struct], b[struct], tol, f"merge_h[{lvl}]")
    _close(tree.readout_h[0], readout_h, tol, "readout_h")
    assert tree.leaf_real.tolist() == (host[3] > 0).tolist()
    assert [o.tolist() for o in T.classify_merge_opcodes(devs[3])] == [o.tolist() for o in opcodes]


def test_reduction_restarts_from_a_reduced_state(hz_lib):
    """The reduction started above the first level (the arguments that
    compile_physical_tree_from_reduced_state passes: counts, total, depths and level offset of
    the full tree) repeats what the full run's upper levels derive from masks and counts:
    opcodes, count features and the number of levels."""
    n = 16
    params = T.init_physical_compiler(9, alpha_init=0.3, n_heads=2, attn_dim=32, fwl_channels=8, pool_heads=2,
                                      pool_d_k=8, pool_d_v=8, **DIMS)
    dev = params["leaf"]["P_c"]["weight"].device
    _, (e_leaf, edge, g, real, struct) = _inputs(4, n, 13, 16, dev)
    c_leaf = C.tree_sphere(C._linear(params["leaf"]["P_c"], e_leaf))
    full = T.compile_context_only_reduction(params["merge"], params["gladder"], c_leaf, real, g, edge, struct)
    m1 = real[0::2] + real[1::2] - real[0::2] * real[1::2]
    k1 = struct[0::2] + struct[1::2] - struct[0::2] * struct[1::2]
    rest = T.compile_context_only_reduction(
        params["merge"], params["gladder"], full["c_carried"][0], m1, g, edge[0::2, 0::2].contiguous(), k1,
        n_total=real.sum(), clock_depth=T.tree_active_clock_depth(struct), initial_counts=real[0::2] + real[1::2],
        level_offset=1, feature_n_levels=T.tree_active_clock_depth(real))
    assert len(rest["merge_h"]) == 3 and rest["merge_h"][0].shape == (4, DIMS["r_merge"])
    for a, b in zip(rest["opcodes"], full["opcodes"][1:]):
        assert a.tolist() == b.tolist()
    for a, b in zip(rest["depth_features"], full["depth_features"][1:]):
        np.testing.assert_array_equal(a.cpu().numpy(), b.cpu().numpy())
    with pytest.raises(ValueError):
        T.compile_context_only_reduction(params["merge"], params["gladder"], c_leaf, real, g, edge, struct,
                                         initial_counts=real[:8])


@pytest.mark.parametrize("n,n_real", [(8, 8), (16, 11)])
def test_compiled_tree_drives_the_walker_path(hz_lib, n, n_real):
    """Conditioners from the compiler in place of the N(0,1) stand-ins: log-amplitude and phase
    of the walker path against the oracle run with the oracle's conditioners."""
    import hamiltonzero_b200 as hz
    params = T.init_physical_compiler(3 * n, alpha_init=0.3, n_heads=2, attn_dim=32, fwl_channels=8, pool_heads=2,
                                      pool_d_k=8, pool_d_v=8, **DIMS)
    dev = params["leaf"]["P_c"]["weight"].device
    host, devs = _inputs(n + 1, n, n_real, n, dev)
    tree = T.compile_physical_tree(params, *devs)
    wf = S.synthetic_wavefunction(1, n, n_real=n_real, d_o=8, d_m=64, d_r=32, r_leaf=16, r_merge=16, r_ro=8)
    kernel, _ = Ty.from_arrays(wf)
    arrays = Ty.to_arrays(kernel, tree)
    for a, b in zip(arrays.opcodes, wf.opcodes):
        np.testing.assert_array_equal(a, b)
    leaf_h, merge_h, _, readout_h = O.compile_tree(C.to_numpy(params), *[x.astype(np.float64) for x in host])
    wf0 = dataclasses.replace(wf, leaf_h=leaf_h, merge_h=list(merge_h), readout_h=readout_h)
    q = S.random_unit_quaternions(np.random.default_rng(n), (6, n))
    la, ph = hz.CompiledWaveFunction(arrays)(q)
    la0, ph0 = W.execute_wavefunction(wf0, q)
    assert np.abs(la - la0).max() <= 1e-4 * np.abs(la0).max() + 1e-4
    assert np.abs(np.angle(np.exp(1j * (ph - ph0)))).max() <= 2e-4


@pytest.mark.parametrize("n,n_real,n_struct", [(16, 11, 16), (16, 5, 8), (64, 64, 64)])
def test_features_to_compiled_tree_matches_oracle(hz_lib, n, n_real, n_struct):
    """The whole context path after the featuriser: trunk layers, global stream, routing by a
    permutation that puts the real sites first, leaf contextualiser (virtual slots, edge summary,
    edge update, gated attention with the LCA-ALiBi bias), global fork, tree reduction and
    conditioners, against the float64 oracle chained the same way."""
    d_e, d_edge, d_feat = DIMS["d_e"], DIMS["d_edge"], DIMS["d_feat"]
    blocks = [C.init_transformer_block(5 * n + i, d_e, 2, d_edge, d_feat, global_tap_dim=8, n_layers=2,
                                       attn_impl="mhsea_tuned", attn_dim=32, attn_bias_hidden_dim=16,
                                       ffn_hidden_dim=64, edge_hidden_dim=24, edge_node_ctx_dim=6,
                                       two_hop_channels=8, two_hop_hidden_dim=16, pool_heads=2, pool_d_k=8,
                                       pool_d_v=8) for i in range(2)]
    post = C.init_edge_rowcol_global_update(n + 3, d_feat, d_edge, tap_dim=8, n_heads=2, d_k=8, d_v=8)
    params = T.init_physical_compiler(n + 4, alpha_init=0.3, n_heads=2, attn_dim=32, fwl_channels=8, pool_heads=2,
                                      pool_d_k=8, pool_d_v=8, **DIMS)
    params["contextualizer"] = C.init_physical_readout_context(
        n + 5, d_e=d_e, d_edge=d_edge, n_layers=2, n_heads=2, summary_hidden=24, mlp_hidden=32, bias_hidden=16,
        edge_ffn_hidden=24, attn_dim=32, edge_node_ctx_dim=6, gladder_d_g=d_feat, global_tap_dim=8, pool_heads=2,
        pool_d_k=8, pool_d_v=8)
    params["global_fork"] = C.init_edge_rowcol_global_update(n + 6, d_feat, d_edge, tap_dim=8, n_heads=2, d_k=8,
                                                             d_v=8)
    dev = post["update"]["w1"].device
    rng = np.random.default_rng(n + n_real)
    local = rng.standard_normal((n, d_e)).astype(np.float32)
    edge = rng.standard_normal((n, n, d_edge)).astype(np.float32)
    gfeat = rng.standard_normal(d_feat).astype(np.float32)
    real = (rng.permutation(n) < n_real).astype(np.float32)
    struct = (np.arange(n) < n_struct).astype(np.float32)
    perm = np.argsort(-real, kind="stable")
    t = lambda x: torch.from_numpy(x).to(dev)
    shared = T.compile_shared_trunk_from_features(blocks, post, t(edge), t(local), t(gfeat), t(real), t(struct))
    tree = T.compile_physical_tree_from_shared_trunk(params, shared, perm)

    from oracle import context as OC
    f8 = lambda x: x.astype(np.float64)
    g_seed = OC.tree_sphere(f8(gfeat))
    node0, edge0, g0 = OC.trunk([C.to_numpy(b) for b in blocks], f8(local), f8(edge), real, g_seed)
    g_stream = OC.edge_rowcol_global_update(C.to_numpy(post), g0, edge0, real)
    _close(shared.global_stream.cpu().numpy(), g_stream, 1e-4, "global stream")
    leaf_h, merge_h, opcodes, readout_h = O.compile_tree_from_shared_trunk(C.to_numpy(params), node0, edge0, g_stream,
                                                                           real, struct, perm)
    tol = 3e-4 if n == 64 else 1e-4
    st = struct > 0
    _close(tree.leaf_h[0][st], leaf_h[st], tol, "leaf_h")
    for lvl, (a, b, op, op0) in enumerate(zip(tree.merge_h, merge_h, tree.opcodes, opcodes)):
        np.testing.assert_array_equal(op, op0)
        st = st[0::2] | st[1::2]
        _close(a[st], b[st], tol, f"merge_h[{lvl}]")
    _close(tree.readout_h[0], readout_h, tol, "readout_h")
    assert tree.perm.tolist() == perm.tolist() and tree.inv_perm[perm].tolist() == list(range(n))
    assert tree.leaf_real.tolist() == (real[perm] > 0).tolist()


def test_graph_inputs_to_compiled_tree_matches_oracle(hz_lib):
    """From the graph inputs (couplings with absent bonds, fields on some sites, padded sites) to
    the conditioners: featuriser, trunk, global stream, routing, contextualiser, fork, tree."""
    from hamiltonzero_b200 import featurizer as F
    from oracle import context as OC
    from oracle import featurizer as OF
    n, n_real = 16, 11
    d_e, d_edge, d_feat = DIMS["d_e"], DIMS["d_edge"], DIMS["d_feat"]
    # d_local = n_heads * head_dim = d_e, d_global = n_global_q * d_local / ... = d_feat
    feat = F.init_system_featurizer(21, d_bond=14, n_heads=5, head_dim=8, n_global_q=3, d_edge=d_edge,
                                    d_hidden_edge=16, polar_group_norm_bond_hidden=24,
                                    polar_group_norm_n_bond_groups=4, polar_group_norm_d_bond_group=6,
                                    polar_group_norm_n_zeeman_groups=3, polar_group_norm_d_zeeman_group=4,
                                    zeeman_hidden_dim=12, global_hidden_dim=20, combine_hidden_dim=18,
                                    token_initial_scale=0.02)
    d_glob = 3 * 5 * 8
    blocks = [C.init_transformer_block(31 + i, d_e, 2, d_edge, d_glob, global_tap_dim=8, n_layers=1,
                                       attn_impl="mhsea_tuned", attn_dim=32, attn_bias_hidden_dim=16,
                                       ffn_hidden_dim=64, edge_hidden_dim=24, edge_node_ctx_dim=6,
                                       two_hop_channels=8, two_hop_hidden_dim=16, pool_heads=2, pool_d_k=8,
                                       pool_d_v=8) for i in range(1)]
    post = C.init_edge_rowcol_global_update(41, d_glob, d_edge, tap_dim=8, n_heads=2, d_k=8, d_v=8)
    dims = dict(DIMS, d_feat=d_glob)
    params = T.init_physical_compiler(42, alpha_init=0.3, n_heads=2, attn_dim=32, fwl_channels=8, pool_heads=2,
                                      pool_d_k=8, pool_d_v=8, **dims)
    params["contextualizer"] = C.init_physical_readout_context(
        43, d_e=d_e, d_edge=d_edge, n_layers=1, n_heads=2, summary_hidden=24, mlp_hidden=32, bias_hidden=16,
        edge_ffn_hidden=24, attn_dim=32, edge_node_ctx_dim=6, gladder_d_g=d_glob, global_tap_dim=8, pool_heads=2,
        pool_d_k=8, pool_d_v=8)
    params["global_fork"] = C.init_edge_rowcol_global_update(44, d_glob, d_edge, tap_dim=8, n_heads=2, d_k=8, d_v=8)
    rng = np.random.default_rng(5)
    J = np.zeros((n, n, 10), np.float32)
    for i in range(n_real):
        for j in range(i + 1, n_real):
            if rng.random() < 0.4:
                blk = rng.standard_normal((3, 3)).astype(np.float32)
                J[i, j, :9] = blk.reshape(-1); J[j, i, :9] = blk.T.reshape(-1)
        J[i, i, 9] = 1.0
    h = np.zeros((n, 3), np.float32)
    h[:n_real:3] = rng.standard_normal((len(range(0, n_real, 3)), 3)).astype(np.float32)
    real = (np.arange(n) < n_real).astype(np.float32)
    struct = np.ones(n, np.float32)
    perm = rng.permutation(n_real).tolist() + list(range(n_real, n))
    dev = post["update"]["w1"].device
    t = lambda x: torch.from_numpy(x).to(dev)
    shared = T.compile_shared_trunk(feat, blocks, post, t(J), t(real), t(h), t(struct))
    tree = T.compile_physical_tree_from_shared_trunk(params, shared, perm)

    f8 = lambda x: x.astype(np.float64)
    edge0, local0, glob0 = OF.system_featurizer(C.to_numpy(feat), f8(J), real, f8(h))
    node0, edge1, g0 = OC.trunk([C.to_numpy(b) for b in blocks], local0, edge0, real, OC.tree_sphere(glob0))
    g_stream = OC.edge_rowcol_global_update(C.to_numpy(post), g0, edge1, real)
    leaf_h, merge_h, opcodes, readout_h = O.compile_tree_from_shared_trunk(C.to_numpy(params), node0, edge1, g_stream,
                                                                           real, struct, np.asarray(perm))
    _close(shared.global_raw.cpu().numpy(), glob0, 2e-5, "global features")
    _close(tree.leaf_h[0], leaf_h, 1e-4, "leaf_h")
    for lvl, (a, b, op, op0) in enumerate(zip(tree.merge_h, merge_h, tree.opcodes, opcodes)):
        np.testing.assert_array_equal(op, op0)
        _close(a, b, 1e-4, f"merge_h[{lvl}]")
    _close(tree.readout_h[0], readout_h, 1e-4, "readout_h")
