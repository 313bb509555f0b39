"""CPU checks of the context blocks' host pieces: the LCA-ALiBi bias against hand-worked levels,
the torch restatement of norms / MLPs / nGPT residual against the numpy oracle, and the
argument checks of the initialisers (the attention op itself needs a GPU)."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import context as C
from oracle import context as O


def test_lca_levels_by_hand():
    # leaves 0..7 of a depth-3 tree: siblings meet at level 1, cousins at 2, halves at 3
    want = {(0, 0): 0, (0, 1): 1, (2, 3): 1, (0, 2): 2, (1, 3): 2, (0, 4): 3, (3, 4): 3, (5, 7): 2, (6, 7): 1}
    idx = torch.arange(8)
    lvl = C.lca_level(idx, idx).numpy()
    for (a, b), l in want.items():
        assert lvl[a, b] == l and lvl[b, a] == l
    big = torch.arange(300)
    np.testing.assert_array_equal(C.lca_level(big, big).numpy(), O.lca_level(range(300), range(300)))
    assert int(C.lca_level(torch.tensor([0]), torch.tensor([2 ** 14]))[0, 0]) == 13      # capped


def test_lca_slopes_and_bias():
    s = C.lca_fixed_slopes(8).numpy()
    assert abs(s[0] - 1.5) < 1e-7 and abs(s[-1] - 1.5 / 16) < 1e-7
    np.testing.assert_allclose(s, O.lca_fixed_slopes(8), rtol=1e-6)
    assert float(C.lca_fixed_slopes(1)[0]) == 1.5
    idx = torch.arange(16)
    b = C.lca_alibi_bias(idx, idx, C.lca_fixed_slopes(4, torch.float64)).numpy()
    np.testing.assert_allclose(b, O.lca_alibi_bias(range(16), range(16), O.lca_fixed_slopes(4)), rtol=1e-6)  # slopes are formed in fp32
    assert b.shape == (4, 16, 16) and np.all(np.diagonal(b, axis1=1, axis2=2) == 0) and np.all(b <= 0)


def test_norms_mlps_and_residual_match_the_oracle():
    p = C.init_level_edge_attn(3, 24, 10, alpha_init=0.1, alpha_max=0.5, n_heads=2, attn_dim=16,
                               bias_mlp_n_blocks=2, device="cpu")
    q = C.init_even_edge_attention(4, 24, 2, 10, attn_impl="einsum", n_layers=4, attn_dim=16,
                                   bias_hidden_dim=12, device="cpu")
    assert p["w_qkv"].shape == (24, 3 * 4 * 8) and p["w_o"].shape == (16, 24) and p["ffn_w1"].shape == (24, 96)
    assert q["bias_mlp"]["inner_gain"] == 0.5 and "out_norm" not in q["bias_mlp"]
    g = torch.Generator().manual_seed(0)
    edge = torch.randn(6, 6, 10, generator=g, dtype=torch.float64)
    pn, qn = C.to_numpy(p), C.to_numpy(q)
    dbl = lambda t: {k: dbl(v) for k, v in t.items()} if isinstance(t, dict) else \
        [dbl(v) for v in t] if isinstance(t, list) else t.double() if isinstance(t, torch.Tensor) else t
    np.testing.assert_allclose(C.mlp(dbl(p["bias_mlp"]), edge).numpy(), O.mlp(pn["bias_mlp"], edge.numpy()),
                               rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(C.unnormalized_mlp(dbl(q["bias_mlp"]), edge).numpy(),
                               O.unnormalized_mlp(qn["bias_mlp"], edge.numpy()), rtol=1e-11, atol=1e-12)
    x = torch.randn(6, 24, generator=g, dtype=torch.float64)
    y = torch.randn(6, 24, generator=g, dtype=torch.float64)
    alpha = torch.randn(24, generator=g, dtype=torch.float64)
    mask = torch.tensor([1, 1, 0, 1, 0, 1.0], dtype=torch.float64)
    got = C.ngpt_residual(x, y, alpha, max_gain=0.5, update_mask=mask).numpy()
    np.testing.assert_allclose(got, O.ngpt_residual(x.numpy(), y.numpy(), alpha.numpy(), 0.5, mask.numpy()),
                               rtol=1e-12)
    np.testing.assert_array_equal(got[2], x.numpy()[2])                 # padded rows keep the skip
    np.testing.assert_allclose((got[[0, 1, 3, 5]] ** 2).mean(-1), 1.0, rtol=1e-12)   # on the sphere
    np.testing.assert_allclose(C.rms_norm(x, alpha, 1e-5).numpy(), O.rms_norm(x.numpy(), alpha.numpy(), 1e-5),
                               rtol=1e-12)


def test_initialiser_argument_checks():
    with pytest.raises(ValueError):
        C.init_level_edge_attn(0, 24, 8, alpha_init=0.1, alpha_max=0.5, n_heads=5, device="cpu")
    with pytest.raises(ValueError):
        C.init_level_edge_attn(0, 12, 8, alpha_init=0.1, alpha_max=0.5, n_heads=4, device="cpu")   # odd d_head
    with pytest.raises(ValueError):
        C.init_level_edge_attn(0, 16, 8, alpha_init=0.1, alpha_max=0.5, attn_impl="flash", device="cpu")
    with pytest.raises(ValueError):
        C.init_even_edge_attention(0, 16, 3, 8, attn_impl="einsum", n_layers=2, attn_dim=16,
                                   bias_hidden_dim=8, device="cpu")


def test_trunk_layer_pieces_match_the_oracle_on_cpu():
    """Edge update (2-FWL contraction through torch's einsum on CPU), global-stream pooling and
    update of one trunk layer in float64 against the numpy oracle; the attention inside the full
    layer needs the GPU and is covered by tests/test_context_gpu.py."""
    p = C.init_transformer_block(1, 48, 2, 12, 24, global_tap_dim=8, n_layers=2, attn_impl="einsum",
                                 attn_dim=32, attn_bias_hidden_dim=16, ffn_hidden_dim=64, edge_hidden_dim=24,
                                 edge_node_ctx_dim=6, two_hop_channels=8, two_hop_hidden_dim=16,
                                 pool_heads=2, pool_d_k=8, pool_d_v=8, device="cpu")
    assert p["residual_gain"] == 2 ** -0.5 and p["edge_update_ctx"]["ffn"]["in_proj"]["weight"].shape == (32, 24)
    rng = np.random.default_rng(0)
    e, edge = rng.standard_normal((10, 48)), rng.standard_normal((10, 10, 12))
    mask, g = (np.arange(10) < 8).astype(np.float64), rng.standard_normal(24)
    dbl = lambda t: {k: dbl(v) for k, v in t.items()} if isinstance(t, dict) else \
        [dbl(v) for v in t] if isinstance(t, list) else t.double() if isinstance(t, torch.Tensor) else t
    pd, pn = dbl(p), C.to_numpy(p)
    tt = torch.from_numpy
    got = C.edge_update_context_aware(pd["edge_update_ctx"], tt(edge), tt(e), tt(mask)).numpy()
    np.testing.assert_allclose(got, O.edge_update_context_aware(pn["edge_update_ctx"], edge, e, mask),
                               rtol=1e-11, atol=1e-12)
    pool = C.g_descriptor_pool(pd["g_pool"], tt(g), tt(e), tt(mask)).numpy()
    np.testing.assert_allclose(pool, O.g_descriptor_pool(pn["g_pool"], g, e, mask), rtol=1e-12, atol=1e-13)
    # masked nodes carry no weight in the pooling: changing them changes nothing
    e2 = e.copy(); e2[8:] += 5.0
    np.testing.assert_allclose(C.g_descriptor_pool(pd["g_pool"], tt(g), tt(e2), tt(mask)).numpy(), pool, rtol=1e-12)
    gu = C.residual_global_update(pd["g_update"], tt(g), tt(pool)).numpy()
    np.testing.assert_allclose(gu, O.residual_global_update(pn["g_update"], g, pool), rtol=1e-12, atol=1e-13)
    with pytest.raises(ValueError):
        C.init_transformer_block(1, 48, 2, 12, 24, global_tap_dim=24, n_layers=2, attn_impl="einsum",
                                 attn_dim=32, attn_bias_hidden_dim=16, ffn_hidden_dim=64, edge_hidden_dim=24,
                                 edge_node_ctx_dim=6, two_hop_channels=8, two_hop_hidden_dim=16, device="cpu")


def test_global_stream_after_the_trunk_matches_the_oracle_on_cpu():
    """Row, column and set pooling with the boundary update (model/global_ladder.py:420-503) in
    float64 against the numpy oracle, which loops over rows and columns one at a time; masked
    rows and columns carry no weight; the result sits on the unit-mean-square sphere."""
    p = C.init_edge_rowcol_global_update(3, 24, 12, tap_dim=8, n_heads=2, d_k=8, d_v=8, device="cpu")
    rng = np.random.default_rng(1)
    edge, g = rng.standard_normal((10, 10, 12)), rng.standard_normal(24)
    mask = (np.arange(10) < 7).astype(np.float64)
    dbl = lambda t: {k: dbl(v) for k, v in t.items()} if isinstance(t, dict) else \
        t.double() if isinstance(t, torch.Tensor) else t
    pd, pn = dbl(p), C.to_numpy(p)
    tt = torch.from_numpy
    got = C.edge_rowcol_global_update(pd, tt(g), tt(edge), tt(mask)).numpy()
    np.testing.assert_allclose(got, O.edge_rowcol_global_update(pn, g, edge, mask), rtol=1e-11, atol=1e-12)
    assert abs((got * got).mean() - 1.0) < 1e-12
    edge2 = edge.copy(); edge2[7:] += 3.0; edge2[:, 7:] -= 2.0
    np.testing.assert_allclose(C.edge_rowcol_global_update(pd, tt(g), tt(edge2), tt(mask)).numpy(), got, rtol=1e-11)
    with pytest.raises(ValueError):
        C.init_edge_rowcol_global_update(3, 24, 12, tap_dim=24, device="cpu")
