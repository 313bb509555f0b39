"""GPU parity of the context compiler's two attention call sites (trunk block, level-edge block
with the LCA-ALiBi bias) on the CUDA attention op against the float64 oracle.
Tolerance: 1e-5 relative to the output scale where the op contracts with the three-term TF32
split (every shape but n = 64), and the op's own 1e-4 at n = 64, where it runs the whole-sequence
kernels on their default two-term BF16 split (measured about 1e-5; the reference's Triton kernels
contract with one TF32 product there, about 1e-3)."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import context as C
from oracle import context as O

pytestmark = pytest.mark.gpu


def _inputs(seed, n, d_c, d_edge, n_real):
    rng = np.random.default_rng(seed)
    c = rng.standard_normal((n, d_c)).astype(np.float32)
    edge = rng.standard_normal((n, n, d_edge)).astype(np.float32)
    mask = (np.arange(n) < n_real).astype(np.float32)
    return c, edge, mask


# n = 16/32: the small-N full-AD kernels; 64/128: the tuned shapes; 24: outside both, keys-only twin
@pytest.mark.parametrize("n,n_real,n_heads,attn_dim,level_idx,impl", [
    (16, 16, 2, 16, None, "mhsea_tuned"),       # d_head 8 -> padded to 16
    (16, 11, 2, 32, 0, "mhsea_tuned"),
    (32, 20, 4, 64, 1, "mhsea_tuned"),
    (64, 64, 4, 64, 2, "mhsea_tuned"),
    (64, 45, 2, 64, 0, "mhsea_tuned"),          # d_head 32
    (128, 100, 4, 32, 3, "mhsea_tuned"),        # d_head 8 at a tuned shape
    (24, 17, 2, 16, 0, "mhsea_tuned"),
    (16, 11, 2, 16, 0, "einsum"),
])
def test_level_edge_attn_matches_oracle(hz_lib, n, n_real, n_heads, attn_dim, level_idx, impl):
    d_c, d_edge = 48, 12
    p = C.init_level_edge_attn(n + n_heads, d_c, d_edge, alpha_init=0.3, alpha_max=0.5, n_heads=n_heads,
                               attn_dim=attn_dim, attn_impl=impl, bias_mlp_n_blocks=2)
    c, edge, mask = _inputs(n, n, d_c, d_edge, n_real)
    dev = p["w_qkv"].device
    got = C.level_edge_attn(p, torch.from_numpy(c).to(dev), torch.from_numpy(edge).to(dev),
                            torch.from_numpy(mask).to(dev), level_idx).cpu().numpy()
    want = O.level_edge_attn(C.to_numpy(p), c.astype(np.float64), edge.astype(np.float64), mask, level_idx)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= (1e-4 if n == 64 else 1e-5) * np.abs(want).max()
    np.testing.assert_array_equal(got[n_real:], c[n_real:])            # padded nodes untouched


@pytest.mark.parametrize("n,n_real,n_heads,attn_dim,impl", [
    (16, 13, 2, 16, "mhsea_tuned"), (64, 64, 4, 64, "mhsea_tuned"), (64, 50, 4, 32, "mhsea_tuned"),
    (40, 33, 2, 32, "mhsea_tuned"), (32, 32, 2, 32, "einsum")])
def test_even_edge_attention_matches_oracle(hz_lib, n, n_real, n_heads, attn_dim, impl):
    d_e, n_edge = 40, 10
    p = C.init_even_edge_attention(n, d_e, n_heads, n_edge, attn_impl=impl, n_layers=4, attn_dim=attn_dim,
                                   bias_hidden_dim=24)
    e, edge, mask = _inputs(n + 1, n, d_e, n_edge, n_real)
    dev = p["W_QKV"].device
    got = C.even_edge_attention(p, torch.from_numpy(e).to(dev), torch.from_numpy(edge).to(dev),
                                torch.from_numpy(mask).to(dev)).cpu().numpy()
    want = O.even_edge_attention(C.to_numpy(p), e.astype(np.float64), edge.astype(np.float64), mask)
    real = slice(0, n_real)      # padded query rows are not consumed by the caller (masked residual)
    assert np.abs(got[real] - want[real]).max() <= (1e-4 if n == 64 else 1e-5) * np.abs(want[real]).max()


def test_level_block_is_differentiable_through_the_op(hz_lib):
    """d(sum w * out)/d(w_qkv) from torch.autograd (the op's backward kernel) against a central
    difference of the oracle along one direction."""
    n, d_c, d_edge = 16, 32, 8
    p = C.init_level_edge_attn(9, d_c, d_edge, alpha_init=0.3, alpha_max=0.5, n_heads=2, attn_dim=32)
    c, edge, mask = _inputs(5, n, d_c, d_edge, 13)
    dev = p["w_qkv"].device
    rng = np.random.default_rng(1)
    weight = rng.standard_normal((n, d_c))
    direction = rng.standard_normal(tuple(p["w_qkv"].shape))
    p["w_qkv"].requires_grad_(True)
    out = C.level_edge_attn(p, torch.from_numpy(c).to(dev), torch.from_numpy(edge).to(dev),
                            torch.from_numpy(mask).to(dev), 0)
    (out * torch.from_numpy(weight).to(dev, torch.float32)).sum().backward()
    got = float((p["w_qkv"].grad.double().cpu().numpy() * direction).sum())
    pn = C.to_numpy(p)
    def f(sign, eps=1e-6):
        moved = dict(pn, w_qkv=pn["w_qkv"] + sign * eps * direction)
        return (O.level_edge_attn(moved, c.astype(np.float64), edge.astype(np.float64), mask, 0) * weight).sum()
    want = (f(+1) - f(-1)) / 2e-6
    assert abs(got - want) <= 1e-4 * np.linalg.norm(p["w_qkv"].grad.cpu().numpy()) * np.linalg.norm(direction)


@pytest.mark.parametrize("n,n_real,layers,impl", [(16, 13, 2, "mhsea_tuned"), (64, 50, 2, "mhsea_tuned"),
                                                  (24, 24, 1, "mhsea_tuned"), (32, 20, 1, "einsum")])
def test_trunk_layers_match_oracle(hz_lib, n, n_real, layers, impl):
    """The stack of trunk layers (edge update with the 2-FWL contraction on hz_fwl2_panel,
    attention on hz_mhsea_fwd, feed-forward, global-stream pooling and update) against the
    float64 oracle: node stream, edge stream and global stream after the last layer."""
    d_e, n_edge, d_g = 48, 12, 24
    blocks = [C.init_transformer_block(100 * n + i, d_e, 2, n_edge, d_g, global_tap_dim=8, n_layers=layers,
                                       attn_impl=impl, attn_dim=32, attn_bias_hidden_dim=16,
                                       ffn_hidden_dim=64, edge_hidden_dim=24, edge_node_ctx_dim=6,
                                       two_hop_channels=8, two_hop_hidden_dim=16, pool_heads=2, pool_d_k=8,
                                       pool_d_v=8) for i in range(layers)]
    e, edge, mask = _inputs(n + 7, n, d_e, n_edge, n_real)
    g = np.random.default_rng(n).standard_normal(d_g).astype(np.float32)
    dev = blocks[0]["g_ffn_proj_w"].device
    t = lambda x: torch.from_numpy(x).to(dev)
    got = C.trunk(blocks, t(e), t(edge), t(mask), t(g))
    want = O.trunk([C.to_numpy(b) for b in blocks], e.astype(np.float64), edge.astype(np.float64), mask,
                   g.astype(np.float64))
    real = mask.astype(bool)
    tol = 1e-4 if n == 64 else 2e-5
    for name, a, b in zip(("nodes", "edges", "global"), got, want):
        a = a.cpu().numpy().astype(np.float64)
        if name == "nodes":
            a, b = a[real], b[real]           # padded nodes are not consumed (masked downstream)
        elif name == "edges":
            a, b = a[np.ix_(real, real)], b[np.ix_(real, real)]
        assert np.isfinite(a).all(), name
        assert np.abs(a - b).max() <= tol * np.abs(b).max(), f"{name}: {np.abs(a - b).max() / np.abs(b).max():.2e}"


def test_fwl2_product_is_differentiable(hz_lib):
    """Cotangents of the 2-FWL contraction from the panel kernel on transposed operands against
    torch's einsum autograd."""
    rng = np.random.default_rng(3)
    a = torch.from_numpy(rng.standard_normal((20, 20, 6)).astype(np.float32)).cuda().requires_grad_(True)
    b = torch.from_numpy(rng.standard_normal((20, 20, 6)).astype(np.float32)).cuda().requires_grad_(True)
    w = torch.from_numpy(rng.standard_normal((20, 20, 6)).astype(np.float32)).cuda()
    (C.fwl2_product(a, b) * w).sum().backward()
    a2, b2 = a.detach().double().requires_grad_(True), b.detach().double().requires_grad_(True)
    (torch.einsum("ikc,kjc->ijc", a2, b2) * w.double()).sum().backward()
    assert (a.grad.double() - a2.grad).abs().max() <= 1e-5 * a2.grad.abs().max()
    assert (b.grad.double() - b2.grad).abs().max() <= 1e-5 * b2.grad.abs().max()


@pytest.mark.parametrize("n,n_real", [(16, 11), (64, 64)])
def test_shared_trunk_global_stream_matches_oracle(hz_lib, n, n_real):
    """Trunk layers followed by the row/column/set pooling of the edge stream and the boundary
    update: the global stream handed to the tree compiler, against the float64 oracle."""
    d_e, n_edge, d_g = 48, 12, 24
    blocks = [C.init_transformer_block(7 * n + i, d_e, 2, n_edge, d_g, global_tap_dim=8, n_layers=2,
                                       attn_impl="mhsea_tuned", attn_dim=32, attn_bias_hidden_dim=16,
                                       ffn_hidden_dim=64, edge_hidden_dim=24, edge_node_ctx_dim=6,
                                       two_hop_channels=8, two_hop_hidden_dim=16, pool_heads=2, pool_d_k=8,
                                       pool_d_v=8) for i in range(2)]
    post = C.init_edge_rowcol_global_update(n, d_g, n_edge, tap_dim=8, n_heads=2, d_k=8, d_v=8)
    e, edge, mask = _inputs(n + 3, n, d_e, n_edge, n_real)
    g = np.random.default_rng(n + 1).standard_normal(d_g).astype(np.float32)
    dev = post["update"]["w1"].device
    t = lambda x: torch.from_numpy(x).to(dev)
    _, _, got = C.shared_trunk(blocks, post, t(e), t(edge), t(mask), t(g))
    _, edge_w, g_w = O.trunk([C.to_numpy(b) for b in blocks], e.astype(np.float64), edge.astype(np.float64),
                             mask, g.astype(np.float64))
    want = O.edge_rowcol_global_update(C.to_numpy(post), g_w, edge_w, mask)
    got = got.cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
