"""The attention blocks of the context compiler on the CUDA attention op.

The reference compiles a system once per lane by running its eager context path
(src/hamiltonzero/compiled/trunk.py:108-157, compiled/tree.py:96-303) whose attention call sites
are the trunk's ``EvenEdgeAttention`` (src/hamiltonzero/model/trunk.py:70-144) and the tree's
``LevelEdgeAttn`` (src/hamiltonzero/model/tree.py:1356-1544, with the LCA-ALiBi bias of
src/hamiltonzero/model/readout_leaf_context.py:150-170). Both are restated here over
``gated_edge_attention`` (zero-padded heads, Q rescaling, sigmoid gate) so that the op's
in-product consumers run on it, and the whole trunk layer around the first one
(``TransformerBlock``, model/trunk.py:298-434: context-aware edge update with its learned 2-FWL
contraction on ``hz_fwl2_panel``, attention, feed-forward, global-stream pooling and update of
src/hamiltonzero/model/global_ladder.py:28-287) with the stack of layers ``trunk``: projections, RMS norms, the bias MLPs and the nGPT residuals
are plain torch on the device (a few small matmuls per block, once per system), the attention
itself is ``hz_mhsea_fwd``. Parameters are dicts of fp32 tensors with the reference's field
names; ``init_*`` draw them with the reference's initialisers (normal * fan_in^-1/2, unit norm
scales, zero biases) from a seeded torch generator (not jax.random's bits).
Everything is differentiable under ``torch.autograd`` (the op's backward is ``hz_mhsea_bwd``)."""
from __future__ import annotations

import numpy as np
import torch

from .attention import gated_edge_attention

_LCA_MAX_LEVELS = 13                      # readout_leaf_context.py:131


# ------------------------------------------------------------------ small pieces
def rms_norm(x, scale, eps: float = 1e-5):
    """``x * scale * rsqrt(mean(x^2) + eps)`` over the last axis (model/tree.py:339-376)."""
    return x * (scale * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps))


def tree_sphere(x):
    """Unit mean square over the last axis, floor 1e-4 (model/tree.py:104-106)."""
    return x * torch.rsqrt(torch.clamp((x * x).mean(dim=-1, keepdim=True), min=1e-4))


def silu(x):
    return x * torch.sigmoid(x)


def ngpt_residual(skip, proposal, alpha, *, max_gain: float, update_mask=None):
    """Normalised residual (model/tree.py:431-495): both arguments are put on the sphere, the
    step towards the proposal is scaled by ``max_gain * sigmoid(alpha)`` per feature and the
    result is normalised again; rows outside ``update_mask`` keep ``skip``."""
    skip_n, prop_n = tree_sphere(skip), tree_sphere(proposal)
    direction = prop_n - skip_n
    updated = tree_sphere(skip_n + (max_gain * torch.sigmoid(alpha)) * direction)
    if update_mask is None:
        return updated
    active = update_mask.to(torch.bool)
    while active.ndim < updated.ndim:
        active = active[..., None]
    return torch.where(active, updated, skip)


def lca_level(pos_q, pos_k):
    """Level of the lowest common ancestor of two leaf positions of a perfect binary tree:
    the number of thresholds ``2^l`` (``l < 13``) that ``pos_q xor pos_k`` reaches
    (readout_leaf_context.py:150-158)."""
    xor = torch.bitwise_xor(pos_q.to(torch.int32)[..., :, None], pos_k.to(torch.int32)[..., None, :])
    thresholds = (2 ** torch.arange(_LCA_MAX_LEVELS, device=xor.device)).to(torch.int32)
    return (xor[..., None] >= thresholds).sum(dim=-1).to(torch.int32)


def lca_fixed_slopes(n_heads: int, dtype=torch.float32, device=None):
    """``1.5 * 2^(-4 h / max(H - 1, 1))`` (readout_leaf_context.py:166-169)."""
    head = torch.arange(n_heads, dtype=torch.float32, device=device)
    return (1.5 * torch.exp2(-(head * 4.0 / max(float(n_heads - 1), 1.0)))).to(dtype)


def lca_alibi_bias(pos_q, pos_k, slopes):
    """``-slope_h * level(q, k)``, ``[H, n_q, n_k]`` (readout_leaf_context.py:161-163)."""
    return -(slopes[:, None, None] * lca_level(pos_q, pos_k).to(slopes.dtype)[None])


def _linear(p, x):
    return x @ p["weight"] + p["bias"]


def mlp(p, x):
    """Normalised residual MLP (model/odd_ops.py:218-276)."""
    x = _linear(p["in_proj"], x)
    for nrm, l1, l2 in zip(p["block_norms"], p["block_l1s"], p["block_l2s"]):
        x = x + p["inner_gain"] * _linear(l2, silu(_linear(l1, rms_norm(x, nrm["weight"], nrm["eps"]))))
    return _linear(p["out_proj"], rms_norm(x, p["out_norm"]["weight"], p["out_norm"]["eps"]))


def unnormalized_mlp(p, x):
    """Residual MLP without norms (model/odd_ops.py:279-328)."""
    x = _linear(p["in_proj"], x)
    for l1, l2 in zip(p["block_l1s"], p["block_l2s"]):
        x = x + p["inner_gain"] * _linear(l2, silu(_linear(l1, x)))
    return _linear(p["out_proj"], x)


# ------------------------------------------------------------------ initialisers
def _gen(seed, device):
    return torch.Generator(device=device).manual_seed(int(seed))


def _normal(gen, shape, std, device):
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std


def _init_linear(gen, d_in, d_out, device):
    return {"weight": _normal(gen, (d_in, d_out), d_in ** -0.5, device),
            "bias": torch.zeros(d_out, device=device)}


def _init_rms(d, device):
    return {"weight": torch.ones(d, device=device), "eps": 1e-5}


def _init_mlp(gen, d_in, d_hidden, d_out, n_blocks, inner_gain, device, normalized):
    p = {"in_proj": _init_linear(gen, d_in, d_hidden, device),
         "block_l1s": [_init_linear(gen, d_hidden, d_hidden, device) for _ in range(n_blocks)],
         "block_l2s": [_init_linear(gen, d_hidden, d_hidden, device) for _ in range(n_blocks)],
         "out_proj": _init_linear(gen, d_hidden, d_out, device), "inner_gain": float(inner_gain)}
    if normalized:
        p["block_norms"] = [_init_rms(d_hidden, device) for _ in range(n_blocks)]
        p["out_norm"] = _init_rms(d_hidden, device)
    return p


def init_level_edge_attn(seed: int, d_c: int, d_edge: int, *, alpha_init: float, alpha_max: float,
                         n_heads: int = 4, attn_dim: int | None = None, attn_impl: str = "mhsea_tuned",
                         bias_mlp_hidden: int | None = None, bias_mlp_n_blocks: int = 1,
                         ffn_d_hidden: int | None = None, ln_eps: float = 1e-5, device="cuda"):
    """Parameters of ``LevelEdgeAttn`` (model/tree.py:1284-1354)."""
    d_attn = int(d_c) if attn_dim is None else int(attn_dim)
    if d_attn < 1 or d_attn % n_heads:
        raise ValueError("attn_dim must be positive and divisible by n_heads")
    if attn_impl not in ("einsum", "mhsea_tuned"):
        raise ValueError("attn_impl must be 'einsum' or 'mhsea_tuned'")
    d_head = d_attn // n_heads
    if d_head % 2:
        raise ValueError("LevelEdgeAttn requires an even d_head")
    hk = 2 * n_heads
    gen = _gen(seed, device)
    hidden = max(32, hk * 2) if bias_mlp_hidden is None else bias_mlp_hidden
    d_ffn = 4 * d_c if ffn_d_hidden is None else ffn_d_hidden
    return {
        "w_qkv": _normal(gen, (d_c, 3 * hk * d_head), d_c ** -0.5, device),
        "w_o": _normal(gen, (n_heads * d_head, d_c), (n_heads * d_head) ** -0.5, device),
        "bias_mlp": _init_mlp(gen, d_edge, hidden, hk, bias_mlp_n_blocks, 1.0, device, True),
        "ln_scale": torch.ones(d_c, device=device), "ffn_ln_scale": torch.ones(d_c, device=device),
        "ffn_w1": _normal(gen, (d_c, d_ffn), d_c ** -0.5, device), "ffn_b1": torch.zeros(d_ffn, device=device),
        "ffn_w2": _normal(gen, (d_ffn, d_c), d_ffn ** -0.5, device), "ffn_b2": torch.zeros(d_c, device=device),
        "alpha_attn": torch.full((d_c,), float(alpha_init), device=device),
        "alpha_ffn": torch.full((d_c,), float(alpha_init), device=device),
        "n_heads": n_heads, "d_head": d_head, "attn_impl": attn_impl, "ln_eps": float(ln_eps),
        "ngpt_alpha_max": float(alpha_max),
    }


def init_even_edge_attention(seed: int, d_e: int, n_heads: int, n_edge: int, *, attn_impl: str,
                             n_layers: int, attn_dim: int, bias_hidden_dim: int, device="cuda"):
    """Parameters of the trunk's ``EvenEdgeAttention`` (model/trunk.py:25-68)."""
    if n_heads < 1 or attn_dim < 1 or attn_dim % n_heads:
        raise ValueError("attn_dim must be positive and divisible by n_heads >= 1")
    if attn_impl not in ("einsum", "mhsea_tuned"):
        raise ValueError("attn_impl must be 'einsum' or 'mhsea_tuned'")
    d_head, hk = attn_dim // n_heads, 2 * n_heads
    gen = _gen(seed, device)
    return {
        "W_QKV": _normal(gen, (d_e, 3 * hk * d_head), d_e ** -0.5, device),
        "W_O": _normal(gen, (attn_dim, d_e), attn_dim ** -0.5, device),
        "bias_mlp": _init_mlp(gen, n_edge, bias_hidden_dim, hk, 1, float(n_layers) ** -0.5, device, False),
        "ln_edge": _init_rms(n_edge, device),
        "n_heads": n_heads, "d_head": d_head, "attn_impl": attn_impl,
    }


# ------------------------------------------------------------------ the two call sites
def even_edge_attention(p, e, edge, mask):
    """Trunk attention block (model/trunk.py:70-144): ``e [n, d_e]``, ``edge [n, n, n_edge]``,
    ``mask [n]`` -> ``[n, d_e]``."""
    n, hk, d = e.shape[0], 2 * p["n_heads"], p["d_head"]
    qkv = (e @ p["W_QKV"]).reshape(n, 3, hk, d)
    edge_pre = rms_norm(edge, p["ln_edge"]["weight"], p["ln_edge"]["eps"])
    coup_bias = unnormalized_mlp(p["bias_mlp"], edge_pre) / float(d) ** 0.5
    out = gated_edge_attention(qkv[:, 0].contiguous(), qkv[:, 1].contiguous(), qkv[:, 2].contiguous(),
                               coup_bias.contiguous(), mask, p["n_heads"], p["attn_impl"])
    return out @ p["W_O"]


def level_edge_attn(p, c_level, edge, mask, level_idx=None):
    """One tree level's attention + FFN block (model/tree.py:1356-1544): ``c_level [n, d_c]``,
    ``edge [n, n, d_edge]``, ``mask [n]`` (float or bool) -> ``[n, d_c]``. With ``level_idx`` the
    LCA-ALiBi bias of the node positions is added to the coupling bias."""
    n, hk, d = c_level.shape[0], 2 * p["n_heads"], p["d_head"]
    maskf = mask.to(c_level.dtype)
    x = rms_norm(c_level, p["ln_scale"], p["ln_eps"])
    qkv = (x @ p["w_qkv"]).reshape(n, 3, hk, d)
    coup_bias = mlp(p["bias_mlp"], edge) / float(d) ** 0.5
    if level_idx is not None:
        idx = torch.arange(n, dtype=torch.int32, device=c_level.device)
        lca = lca_alibi_bias(idx, idx, lca_fixed_slopes(hk, x.dtype, x.device))
        coup_bias = coup_bias + lca.permute(1, 2, 0)
    out_flat = gated_edge_attention(qkv[:, 0].contiguous(), qkv[:, 1].contiguous(), qkv[:, 2].contiguous(),
                                    coup_bias.contiguous(), maskf, p["n_heads"], p["attn_impl"])
    mask_q = maskf.reshape(-1, 1)
    c_attn = ngpt_residual(c_level, mask_q * (out_flat @ p["w_o"]), p["alpha_attn"],
                           max_gain=p["ngpt_alpha_max"], update_mask=maskf)
    x_ffn = rms_norm(c_attn, p["ffn_ln_scale"], p["ln_eps"])
    delta_ffn = silu(x_ffn @ p["ffn_w1"] + p["ffn_b1"]) @ p["ffn_w2"] + p["ffn_b2"]
    return ngpt_residual(c_attn, mask_q * delta_ffn, p["alpha_ffn"], max_gain=p["ngpt_alpha_max"],
                         update_mask=maskf)


# ------------------------------------------------------------------ the trunk layer
class _Fwl2Product(torch.autograd.Function):
    """``P[i, j, c] = sum_k A[i, k, c] B[k, j, c]`` (the learned 2-FWL contraction of the edge
    update, model/trunk.py:275) on ``hz_fwl2_panel``; the two cotangents are the same product on
    transposed operands."""

    @staticmethod
    def forward(ctx, a, b):
        from .sequence_parallel import fwl2_panel
        a, b = a.contiguous(), b.contiguous()
        ctx.save_for_backward(a, b)
        out = torch.empty(a.shape[0], b.shape[1], a.shape[2], dtype=a.dtype, device=a.device)
        return fwl2_panel(a, b, out, 0, False)

    @staticmethod
    def backward(ctx, dp):
        from .sequence_parallel import fwl2_panel
        a, b = ctx.saved_tensors
        dp = dp.contiguous()
        # dA[i, k, c] = sum_j dP[i, j, c] B[k, j, c];  dB[k, j, c] = sum_i A[i, k, c] dP[i, j, c]
        da = fwl2_panel(dp, b.transpose(0, 1).contiguous(), torch.empty_like(a), 0, False)
        db = fwl2_panel(a.transpose(0, 1).contiguous(), dp, torch.empty_like(b), 0, False)
        return da, db


def fwl2_product(a, b):
    """``einsum("ikc,kjc->ijc", a, b)``: the CUDA panel kernel for device tensors (differentiable),
    torch's einsum for host tensors (tests of the surrounding arithmetic on CPU)."""
    if a.is_cuda:
        return _Fwl2Product.apply(a, b)
    return torch.einsum("ikc,kjc->ijc", a, b)


def edge_update_context_aware(p, edge, even, mask):
    """The trunk's edge update (model/trunk.py:232-296): pair features ``[edge | ctx_i | ctx_j]``,
    two learned pair maps ``A, B`` contracted over the middle node (2-FWL), the path feature
    normalised and concatenated, a residual MLP back to the edge width."""
    n = even.shape[0]
    edge_ln = rms_norm(edge, p["ln_edge"]["weight"], p["ln_edge"]["eps"])
    even_ctx = rms_norm(even, p["ln_even"]["weight"], p["ln_even"]["eps"]) @ p["node_ctx_proj"]
    d_ctx = even_ctx.shape[-1]
    pair_ij = torch.cat([edge_ln, even_ctx[:, None, :].expand(n, n, d_ctx),
                         even_ctx[None, :, :].expand(n, n, d_ctx)], dim=-1)
    psi = lambda l_in, l_out: _linear(l_out, silu(_linear(l_in, pair_ij)))
    m = mask.to(edge.dtype)
    a = psi(p["psi_L_in"], p["psi_L_out"]) * (m[:, None, None] * m[None, :, None])
    b = psi(p["psi_R_in"], p["psi_R_out"]) * m[None, :, None]
    n_eff = torch.clamp(m.sum(), min=1.0)
    path = fwl2_product(a, b) / torch.sqrt(n_eff)
    p_ij = rms_norm(path, p["ln_path"]["weight"], p["ln_path"]["eps"])
    return mlp(p["ffn"], torch.cat([pair_ij, p_ij], dim=-1))


def g_descriptor_pool(p, g, xs, mask):
    """Attention pooling of the node stream by the global stream (model/global_ladder.py:63-136):
    one query per head from ``g``, keys and values from the normalised nodes, masked softmax."""
    n, h, dk, dv = xs.shape[0], p["n_heads"], p["d_k"], p["d_v"]
    xn = rms_norm(xs, p["ln_in"]["weight"], p["ln_in"]["eps"])
    q = (g @ p["W_q"]).reshape(h, dk)
    k = _linear(p["K"], xn).reshape(n, h, dk)
    v = _linear(p["V"], xn).reshape(n, h, dv)
    scores = torch.einsum("hd,nhd->hn", q, k) / float(dk) ** 0.5
    scores = torch.where(mask[None, :] > 0, scores, torch.full_like(scores, -1.0e30))
    return torch.einsum("hn,nhv->hv", torch.softmax(scores, dim=-1), v).reshape(-1)


def residual_global_update(p, g, pool):
    """``g + gain * MLP(rms([g W_tap | pool]))`` (model/global_ladder.py:156-287)."""
    x = torch.cat([g @ p["g_tap_w"], pool.to(g.dtype)])
    x = rms_norm(x, p["ln_s"], 1e-5)
    return g + p["residual_gain"] * (silu(x @ p["w1"] + p["b1"]) @ p["w2"] + p["b2"])


def transformer_block(p, e, edge, mask, g):
    """One trunk layer (``TransformerBlock._even_edge_step``, model/trunk.py:372-424): edge
    update, attention, feed-forward with the projected global stream added to its input, then
    the global stream pooled from the nodes and updated. Returns ``(e, edge, g)``."""
    gain = p["residual_gain"]
    edge = edge + gain * edge_update_context_aware(p["edge_update_ctx"], edge, e, mask)
    e = e + gain * even_edge_attention(p["attn"], rms_norm(e, p["ln_attn"]["weight"], p["ln_attn"]["eps"]),
                                       edge, mask)
    e_pre = rms_norm(e, p["ln_ffn"]["weight"], p["ln_ffn"]["eps"]) + (g @ p["g_ffn_proj_w"])[None, :]
    e = e + gain * _linear(p["ffn"]["l2"], silu(_linear(p["ffn"]["l1"], e_pre)))
    pooled = g_descriptor_pool(p["g_pool"], g, e, mask)
    g = residual_global_update(p["g_update"], g, pooled)
    return e, edge, g


def trunk(blocks, local_feat, edge_feat, mask, g):
    """The stack of trunk layers (``Trunk.__call__``, model/trunk.py:498-529): ``(e, edge, g)``
    after every block in turn (the reference scans over stacked block parameters)."""
    e, edge = local_feat.to(torch.float32), edge_feat.to(torch.float32)
    for p in blocks:
        e, edge, g = transformer_block(p, e, edge, mask, g)
    return e, edge, g


def init_transformer_block(seed: int, d_e: int, n_heads: int, n_edge: int, gladder_d_g: int, *,
                           global_tap_dim: int, n_layers: int, attn_impl: str, attn_dim: int,
                           attn_bias_hidden_dim: int, ffn_hidden_dim: int, edge_hidden_dim: int,
                           edge_node_ctx_dim: int, two_hop_channels: int, two_hop_hidden_dim: int,
                           pool_heads: int = 4, pool_d_k: int = 64, pool_d_v: int = 64, device="cuda"):
    """Parameters of one ``TransformerBlock`` (model/trunk.py:309-370 with
    ``EdgeUpdateContextAware`` :182-230, ``GDescriptorPool`` and ``ResidualGlobalUpdate`` of
    model/global_ladder.py:38-57,139-153) with the reference's initialiser scales."""
    if edge_node_ctx_dim < 1:
        raise ValueError("edge_node_ctx_dim must be positive")
    if not (0 < global_tap_dim < gladder_d_g):
        raise ValueError("global tap dimension must be positive and smaller than d_g")
    gen = _gen(seed, device)
    d_pair = n_edge + 2 * edge_node_ctx_dim
    inner = float(n_layers) ** -0.5
    d_pool = pool_heads * pool_d_v
    d_in = global_tap_dim + d_pool
    edge_update = {
        "ln_edge": _init_rms(n_edge, device), "ln_even": _init_rms(d_e, device),
        "node_ctx_proj": _normal(gen, (d_e, edge_node_ctx_dim), d_e ** -0.5, device),
        "ffn": _init_mlp(gen, d_pair + two_hop_channels, edge_hidden_dim, n_edge, 1, inner, device, True),
        "psi_L_in": _init_linear(gen, d_pair, two_hop_hidden_dim, device),
        "psi_L_out": _init_linear(gen, two_hop_hidden_dim, two_hop_channels, device),
        "psi_R_in": _init_linear(gen, d_pair, two_hop_hidden_dim, device),
        "psi_R_out": _init_linear(gen, two_hop_hidden_dim, two_hop_channels, device),
        "ln_path": _init_rms(two_hop_channels, device),
    }
    return {
        "edge_update_ctx": edge_update,
        "ln_attn": _init_rms(d_e, device),
        "attn": init_even_edge_attention(seed + 1, d_e, n_heads, n_edge, attn_impl=attn_impl, n_layers=n_layers,
                                         attn_dim=attn_dim, bias_hidden_dim=attn_bias_hidden_dim, device=device),
        "ln_ffn": _init_rms(d_e, device),
        "ffn": {"l1": _init_linear(gen, d_e, ffn_hidden_dim, device),
                "l2": _init_linear(gen, ffn_hidden_dim, d_e, device)},
        "g_pool": {"W_q": _normal(gen, (gladder_d_g, pool_heads * pool_d_k), gladder_d_g ** -0.5, device),
                   "K": _init_linear(gen, d_e, pool_heads * pool_d_k, device),
                   "V": _init_linear(gen, d_e, pool_heads * pool_d_v, device),
                   "ln_in": _init_rms(d_e, device), "n_heads": pool_heads, "d_k": pool_d_k, "d_v": pool_d_v},
        "g_update": {"w1": _normal(gen, (d_in, 2 * gladder_d_g), d_in ** -0.5, device),
                     "b1": torch.zeros(2 * gladder_d_g, device=device),
                     "w2": _normal(gen, (2 * gladder_d_g, gladder_d_g), (2 * gladder_d_g) ** -0.5, device),
                     "b2": torch.zeros(gladder_d_g, device=device), "ln_s": torch.ones(d_in, device=device),
                     "g_tap_w": _normal(gen, (gladder_d_g, global_tap_dim), gladder_d_g ** -0.5, device),
                     "residual_gain": inner},
        "g_ffn_proj_w": _normal(gen, (gladder_d_g, d_e), gladder_d_g ** -0.5, device),
        "residual_gain": inner,
    }


def boundary_global_update(p, g, pool):
    """The update of :func:`residual_global_update` without the gain, put back on the sphere
    (``BoundaryGlobalUpdate``, model/global_ladder.py:289-334)."""
    x = torch.cat([g @ p["g_tap_w"], pool.to(g.dtype)])
    x = rms_norm(x, p["ln_s"], 1e-5)
    return tree_sphere(g + silu(x @ p["w1"] + p["b1"]) @ p["w2"] + p["b2"])


def _descriptor_pool_rows(p, g, xs, mask):
    """:func:`g_descriptor_pool` of every ``xs[b]`` with the same query and mask: ``[b, h*dv]``."""
    b, n, h, dk, dv = xs.shape[0], xs.shape[1], p["n_heads"], p["d_k"], p["d_v"]
    xn = rms_norm(xs, p["ln_in"]["weight"], p["ln_in"]["eps"])
    q = (g @ p["W_q"]).reshape(h, dk)
    k = _linear(p["K"], xn).reshape(b, n, h, dk)
    v = _linear(p["V"], xn).reshape(b, n, h, dv)
    scores = torch.einsum("hd,bnhd->bhn", q, k) / float(dk) ** 0.5
    scores = torch.where(mask[None, None, :] > 0, scores, torch.full_like(scores, -1.0e30))
    return torch.einsum("bhn,bnhv->bhv", torch.softmax(scores, dim=-1), v).reshape(b, -1)


def edge_rowcol_global_update(p, g, edge, mask):
    """The global stream after the trunk (``EdgeRowColGlobalUpdate.__call__``,
    model/global_ladder.py:461-503): one descriptor per edge row and one per edge column, each
    pooled by the global stream; the 2n descriptors pooled again; the boundary update."""
    rows = _descriptor_pool_rows(p["row_pool"], g, edge, mask)
    cols = _descriptor_pool_rows(p["col_pool"], g, edge.transpose(0, 1), mask)
    descs = torch.cat([rows, cols], dim=0)
    dmask = torch.cat([mask, mask], dim=0)
    return boundary_global_update(p["update"], g, g_descriptor_pool(p["set_pool"], g, descs, dmask))


def _init_pool(gen, d_g, d_x, heads, d_k, d_v, device):
    return {"W_q": _normal(gen, (d_g, heads * d_k), d_g ** -0.5, device),
            "K": _init_linear(gen, d_x, heads * d_k, device), "V": _init_linear(gen, d_x, heads * d_v, device),
            "ln_in": _init_rms(d_x, device), "n_heads": heads, "d_k": d_k, "d_v": d_v}


def init_edge_rowcol_global_update(seed: int, d_g: int, d_edge: int, *, tap_dim: int, n_heads: int = 4,
                                   d_k: int = 64, d_v: int = 64, device="cuda"):
    """Parameters of ``EdgeRowColGlobalUpdate`` (model/global_ladder.py:427-459) with the
    reference's initialiser scales (``_global_update_parameters``, :139-153)."""
    if not (0 < tap_dim < d_g):
        raise ValueError("global tap dimension must be positive and smaller than d_g")
    gen = _gen(seed, device)
    d_pool = n_heads * d_v
    d_in = tap_dim + d_pool
    return {
        "row_pool": _init_pool(gen, d_g, d_edge, n_heads, d_k, d_v, device),
        "col_pool": _init_pool(gen, d_g, d_edge, n_heads, d_k, d_v, device),
        "set_pool": _init_pool(gen, d_g, d_pool, n_heads, d_k, d_v, device),
        "update": {"w1": _normal(gen, (d_in, 2 * d_g), d_in ** -0.5, device),
                   "b1": torch.zeros(2 * d_g, device=device),
                   "w2": _normal(gen, (2 * d_g, d_g), (2 * d_g) ** -0.5, device),
                   "b2": torch.zeros(d_g, device=device), "ln_s": torch.ones(d_in, device=device),
                   "g_tap_w": _normal(gen, (d_g, tap_dim), d_g ** -0.5, device)},
    }


def shared_trunk(blocks, post, local_feat, edge_feat, mask, g):
    """Trunk and global stream of one system from its featurised inputs (the part of
    ``compile_shared_trunk`` after the featuriser, compiled/trunk.py:22-48 with
    ``HamiltonZero.trunk_outputs``, model/model.py:515-533): ``(e, edge, g_stream)``."""
    e, edge, g_trunk = trunk(blocks, local_feat, edge_feat, mask, g)
    return e, edge, edge_rowcol_global_update(post, g_trunk, edge, mask)


# ------------------------------------------------------------------ the leaf contextualiser
def _slot_clock(n: int, d_e: int, bmask, rope_base: float, rope_scaling: float):
    """Sin/cos clock of the slot position relative to the centre of the active balanced subtree
    (model/readout_leaf_context.py:543-562)."""
    n_active = max(int(bmask.to(torch.int64).sum()), 1)
    span = 2.0 ** float(np.ceil(np.log2(float(n_active))))
    pos = (torch.arange(n, dtype=torch.float32, device=bmask.device) - (span - 1.0) * 0.5) / float(rope_scaling)
    half = (d_e + 1) // 2
    band = torch.arange(half, dtype=torch.float32, device=bmask.device)
    inv = torch.exp(-float(np.log(rope_base)) * band / float(max(half, 1)))
    ang = pos[:, None] * inv[None, :]
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=-1)[:, :d_e]


def physical_readout_context_layer(p, c, edge, bmask, g):
    """One layer of the leaf contextualiser (``PhysicalReadoutContextLayer.__call__``,
    model/readout_leaf_context.py:732-836): node update from an LCA-weighted summary of the
    node's edges, global-stream pooling and update, edge update from the node contexts and the
    global stream, gated edge attention with the LCA-ALiBi bias. Returns ``(c, edge, g)``."""
    n, dtype = c.shape[0], c.dtype
    bm = bmask.to(dtype)
    st = bm > 0
    idx = torch.arange(n, dtype=torch.int32, device=c.device)
    rel = idx[:, None] - idx[None, :]
    direction = torch.where(rel < 0, 1.0, torch.where(rel > 0, -1.0, 0.0)).to(dtype)[..., None]
    edge_n = rms_norm(edge, p["ln_edge"]["weight"], p["ln_edge"]["eps"])
    clock = _slot_clock(n, c.shape[1], bm, p["rope_base"], p["rope_scaling"]).to(dtype)
    message = mlp(p["summary_mlp"], torch.cat([edge_n, edge_n.transpose(0, 1), direction], dim=-1))
    weight = bm[:, None] * bm[None, :] * (1.0 - torch.eye(n, dtype=dtype, device=c.device)) \
        * torch.exp(-0.5 * lca_level(idx, idx).to(dtype))
    summary = (message * weight[..., None]).sum(dim=1) / torch.clamp(weight.sum(dim=1, keepdim=True), min=1.0)
    ctx_in = torch.cat([rms_norm(c + clock, p["ln_c"]["weight"], p["ln_c"]["eps"]),
                        rms_norm(summary, p["ln_summary"]["weight"], p["ln_summary"]["eps"])], dim=-1)
    c1 = torch.where(st[:, None], c + p["residual_scale"] * mlp(p["ctx_mlp"], ctx_in), torch.zeros_like(c))
    g = residual_global_update(p["g_update"], g, g_descriptor_pool(p["g_pool"], g, c1, bm))
    edge_ctx = rms_norm(c1, p["ln_edge_ctx"]["weight"], p["ln_edge_ctx"]["eps"]) @ p["edge_node_ctx_proj"]
    pair = (bm[:, None] * bm[None, :])[..., None]
    g_edge = (g @ p["g_edge_proj_w"]).to(dtype)
    edge_in = torch.cat([pair * edge_n, edge_ctx[:, None, :].expand(n, n, -1), edge_ctx[None, :, :].expand(n, n, -1),
                         g_edge[None, None, :].expand(n, n, -1)], dim=-1)
    edge1 = torch.where(pair > 0, edge + p["residual_scale"] * mlp(p["edge_ffn"], edge_in), torch.zeros_like(edge))
    hk, d = 2 * p["n_heads"], p["d_head"]
    x = rms_norm(c1 + clock, p["ln_attn"]["weight"], p["ln_attn"]["eps"])
    e_att = rms_norm(edge1, p["ln_edge_attn"]["weight"], p["ln_edge_attn"]["eps"])
    qkv = (x @ p["W_QKV"]).reshape(n, 3, hk, d)
    bias = mlp(p["bias_mlp"], torch.cat([e_att, direction], dim=-1)) / float(d) ** 0.5
    bias = bias + lca_alibi_bias(idx, idx, lca_fixed_slopes(hk, dtype, c.device)).permute(1, 2, 0)
    out = gated_edge_attention(qkv[:, 0].contiguous(), qkv[:, 1].contiguous(), qkv[:, 2].contiguous(),
                               bias.contiguous(), bm, p["n_heads"], p["attn_impl"])
    out = torch.where(st[:, None], c1 + p["residual_scale"] * (out @ p["W_O"]), torch.zeros_like(c1))
    return out, edge1, g


def physical_readout_context(p, c, edge, mask, bmask, g):
    """``PhysicalReadoutContext.with_edge`` (model/readout_leaf_context.py:1078-1215): the virtual
    slots of the balanced subtree (structural but not real) get the learned node vector, edges
    between a real and a virtual slot or between two virtual slots the learned edge vectors,
    everything outside is zero; then the layers in turn."""
    c, edge = c.to(torch.float32), edge.to(torch.float32)
    real = mask > 0
    virtual = (bmask > 0) & ~real
    c = torch.where(real[:, None], c, torch.where(virtual[:, None], p["virtual_node"][None, :], torch.zeros_like(c)))
    real_pair = real[:, None] & real[None, :]
    mixed = (real[:, None] & virtual[None, :]) | (virtual[:, None] & real[None, :])
    both_virtual = virtual[:, None] & virtual[None, :]
    zero = torch.zeros_like(edge)
    edge = torch.where(real_pair[..., None], edge,
                       torch.where(mixed[..., None], p["edge_empty_nonempty"][None, None, :],
                                   torch.where(both_virtual[..., None], p["edge_empty_empty"][None, None, :], zero)))
    for layer in p["layers"]:
        c, edge, g = physical_readout_context_layer(layer, c, edge, bmask, g)
    return c, edge, g


def init_physical_readout_context(seed: int, *, d_e: int, d_edge: int, n_layers: int, n_heads: int,
                                  summary_hidden: int, mlp_hidden: int, bias_hidden: int, edge_ffn_hidden: int,
                                  attn_dim: int, edge_node_ctx_dim: int, attn_impl: str = "mhsea_tuned",
                                  rope_base: float = 10000.0, rope_scaling: float = 1.0, gladder_d_g: int,
                                  global_tap_dim: int, pool_heads: int = 4, pool_d_k: int = 64, pool_d_v: int = 64,
                                  device="cuda"):
    """Parameters of ``PhysicalReadoutContext`` (model/readout_leaf_context.py:453-541,1150-1208)
    with the reference's shapes and initialiser scales."""
    if n_layers < 1:
        raise ValueError("physical contextualizer layers must be positive")
    if n_heads < 1:
        raise ValueError("contextualizer n_heads must be positive")
    if attn_dim < 1 or attn_dim % n_heads:
        raise ValueError("contextualizer attention width must divide by n_heads")
    if d_e % 2:
        raise ValueError("physical contextualizer width must be even")
    d_head = attn_dim // n_heads
    if d_head % 2:
        raise ValueError("contextualizer attention head width must be even")
    if attn_impl not in ("einsum", "mhsea_tuned"):
        raise ValueError("attention must be 'einsum' or 'mhsea_tuned'")
    if rope_base <= 0.0 or rope_scaling <= 0.0:
        raise ValueError("physical contextualizer rope values must be positive")
    if not (0 < global_tap_dim < gladder_d_g):
        raise ValueError("global tap dimension must be positive and smaller than d_g")
    gen = _gen(seed, device)
    hk, scale = 2 * n_heads, float(n_layers) ** -0.5
    d_pool, d_g = pool_heads * pool_d_v, gladder_d_g
    d_in = global_tap_dim + d_pool

    def layer():
        return {
            "ln_edge": _init_rms(d_edge, device), "ln_edge_attn": _init_rms(d_edge, device),
            "ln_c": _init_rms(d_e, device), "ln_summary": _init_rms(d_e, device),
            "ln_attn": _init_rms(d_e, device), "ln_edge_ctx": _init_rms(d_e, device),
            "summary_mlp": _init_mlp(gen, 2 * d_edge + 1, summary_hidden, d_e, 1, 1.0, device, True),
            "ctx_mlp": _init_mlp(gen, 2 * d_e, mlp_hidden, d_e, 2, 1.0, device, True),
            "edge_node_ctx_proj": _normal(gen, (d_e, edge_node_ctx_dim), d_e ** -0.5, device),
            "edge_ffn": _init_mlp(gen, d_edge + 2 * edge_node_ctx_dim + 64, edge_ffn_hidden, d_edge, 1, 1.0, device,
                                  True),
            "g_pool": _init_pool(gen, d_g, d_e, pool_heads, pool_d_k, pool_d_v, device),
            "g_update": {"w1": _normal(gen, (d_in, 2 * d_g), d_in ** -0.5, device),
                         "b1": torch.zeros(2 * d_g, device=device),
                         "w2": _normal(gen, (2 * d_g, d_g), (2 * d_g) ** -0.5, device),
                         "b2": torch.zeros(d_g, device=device), "ln_s": torch.ones(d_in, device=device),
                         "g_tap_w": _normal(gen, (d_g, global_tap_dim), d_g ** -0.5, device),
                         "residual_gain": scale},
            "g_edge_proj_w": _normal(gen, (d_g, 64), d_g ** -0.5, device),
            "W_QKV": _normal(gen, (d_e, 3 * hk * d_head), d_e ** -0.5, device),
            "W_O": _normal(gen, (attn_dim, d_e), attn_dim ** -0.5, device),
            "bias_mlp": _init_mlp(gen, d_edge + 1, bias_hidden, hk, 1, 1.0, device, True),
            "n_heads": n_heads, "d_head": d_head, "attn_impl": attn_impl, "rope_base": float(rope_base),
            "rope_scaling": float(rope_scaling), "residual_scale": scale,
        }
    return {"layers": [layer() for _ in range(n_layers)],
            "virtual_node": _normal(gen, (d_e,), d_e ** -0.5, device),
            "edge_empty_nonempty": _normal(gen, (d_edge,), d_edge ** -0.5, device),
            "edge_empty_empty": _normal(gen, (d_edge,), d_edge ** -0.5, device)}


def to_numpy(p):
    """Parameter dict with every tensor as a float64 numpy array (for the oracle)."""
    if isinstance(p, dict):
        return {k: to_numpy(v) for k, v in p.items()}
    if isinstance(p, (list, tuple)):
        return [to_numpy(v) for v in p]
    if isinstance(p, torch.Tensor):
        return p.detach().cpu().numpy().astype(np.float64)
    return p


__all__ = ["boundary_global_update", "edge_rowcol_global_update", "edge_update_context_aware", "even_edge_attention", "fwl2_product", "g_descriptor_pool",
           "init_edge_rowcol_global_update", "init_even_edge_attention", "init_physical_readout_context", "init_level_edge_attn", "init_transformer_block", "lca_alibi_bias",
           "lca_fixed_slopes", "lca_level", "level_edge_attn", "mlp", "ngpt_residual", "physical_readout_context", "physical_readout_context_layer",
           "residual_global_update", "rms_norm", "shared_trunk", "to_numpy", "transformer_block", "tree_sphere", "trunk",
           "unnormalized_mlp"]
