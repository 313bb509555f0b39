"""Test infrastructure, not product code: float64 numpy restatement of the two attention blocks
of the reference's context path - the trunk's EvenEdgeAttention
(src/hamiltonzero/model/trunk.py:70-144) and the tree's LevelEdgeAttn
(src/hamiltonzero/model/tree.py:1356-1544) with the LCA-ALiBi bias
(src/hamiltonzero/model/readout_leaf_context.py:150-170), the leaf contextualiser
(model/readout_leaf_context.py:426-836,1078-1215), the global-stream updates
(src/hamiltonzero/model/global_ladder.py:63-503), the residual MLPs
(src/hamiltonzero/model/odd_ops.py:218-328), the RMS norm (model/tree.py:339-376) and the nGPT
residual (model/tree.py:104-106,431-495) - over the attention oracle. Parameters are the dicts
of hamiltonzero_b200.context converted with ``to_numpy``.
Parity unpinned for these blocks: the reference holds no golden vectors for them and JAX is
not installed where this was written; the LCA levels are pinned by hand-worked values in
tests/test_context_oracle.py."""
import numpy as np

from . import attention as A

LCA_MAX_LEVELS = 13


def rms_norm(x, scale, eps=1e-5):
    return x * (scale / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps))


def tree_sphere(x):
    return x / np.sqrt(np.maximum((x * x).mean(axis=-1, keepdims=True), 1e-4))


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def ngpt_residual(skip, proposal, alpha, max_gain, update_mask=None):
    skip_n, prop_n = tree_sphere(skip), tree_sphere(proposal)
    updated = tree_sphere(skip_n + max_gain * sigmoid(alpha) * (prop_n - skip_n))
    if update_mask is None:
        return updated
    return np.where(np.asarray(update_mask).astype(bool)[:, None], updated, skip)


def lca_level(pos_q, pos_k):
    """Bit length of ``q xor k`` (capped at 13): the loop form of the threshold count."""
    out = np.zeros((len(pos_q), len(pos_k)), dtype=np.int64)
    for i, a in enumerate(pos_q):
        for j, b in enumerate(pos_k):
            out[i, j] = min(int(a ^ b).bit_length(), LCA_MAX_LEVELS)
    return out


def lca_fixed_slopes(n_heads):
    head = np.arange(n_heads, dtype=np.float64)
    return 1.5 * np.exp2(-(head * 4.0 / max(n_heads - 1, 1)))


def lca_alibi_bias(pos_q, pos_k, slopes):
    return -(slopes[:, None, None] * lca_level(pos_q, pos_k)[None].astype(np.float64))


def _linear(p, x):
    return x @ p["weight"] + p["bias"]


def mlp(p, x):
    x = _linear(p["in_proj"], x)
    for nrm, l1, l2 in zip(p["block_norms"], p["block_l1s"], p["block_l2s"]):
        x = x + p["inner_gain"] * _linear(l2, silu(_linear(l1, rms_norm(x, nrm["weight"], nrm["eps"]))))
    return _linear(p["out_proj"], rms_norm(x, p["out_norm"]["weight"], p["out_norm"]["eps"]))


def unnormalized_mlp(p, x):
    x = _linear(p["in_proj"], x)
    for l1, l2 in zip(p["block_l1s"], p["block_l2s"]):
        x = x + p["inner_gain"] * _linear(l2, silu(_linear(l1, x)))
    return _linear(p["out_proj"], x)


def even_edge_attention(p, e, edge, mask):
    n, hk, d = e.shape[0], 2 * p["n_heads"], p["d_head"]
    qkv = (e @ p["W_QKV"]).reshape(n, 3, hk, d)
    coup = unnormalized_mlp(p["bias_mlp"], rms_norm(edge, p["ln_edge"]["weight"], p["ln_edge"]["eps"]))
    coup = coup / np.sqrt(float(d))
    out = A.gated_edge_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], coup, mask, p["n_heads"], p["attn_impl"])
    return out @ p["W_O"]


def level_edge_attn(p, c_level, edge, mask, level_idx=None):
    n, hk, d = c_level.shape[0], 2 * p["n_heads"], p["d_head"]
    maskf = np.asarray(mask, dtype=np.float64)
    x = rms_norm(c_level, p["ln_scale"], p["ln_eps"])
    qkv = (x @ p["w_qkv"]).reshape(n, 3, hk, d)
    coup = mlp(p["bias_mlp"], edge) / np.sqrt(float(d))
    if level_idx is not None:
        idx = np.arange(n)
        coup = coup + np.transpose(lca_alibi_bias(idx, idx, lca_fixed_slopes(hk)), (1, 2, 0))
    out = A.gated_edge_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], coup, maskf, p["n_heads"], p["attn_impl"])
    mask_q = maskf[:, None]
    c_attn = ngpt_residual(c_level, mask_q * (out @ p["w_o"]), p["alpha_attn"], p["ngpt_alpha_max"], maskf)
    x_ffn = rms_norm(c_attn, p["ffn_ln_scale"], p["ln_eps"])
    delta = silu(x_ffn @ p["ffn_w1"] + p["ffn_b1"]) @ p["ffn_w2"] + p["ffn_b2"]
    return ngpt_residual(c_attn, mask_q * delta, p["alpha_ffn"], p["ngpt_alpha_max"], maskf)


def edge_update_context_aware(p, edge, even, mask):
    """model/trunk.py:232-296."""
    n = even.shape[0]
    edge_ln = rms_norm(edge, p["ln_edge"]["weight"], p["ln_edge"]["eps"])
    even_ctx = rms_norm(even, p["ln_even"]["weight"], p["ln_even"]["eps"]) @ p["node_ctx_proj"]
    d_ctx = even_ctx.shape[-1]
    pair_ij = np.concatenate([edge_ln, np.broadcast_to(even_ctx[:, None, :], (n, n, d_ctx)),
                              np.broadcast_to(even_ctx[None, :, :], (n, n, d_ctx))], axis=-1)
    psi = lambda l_in, l_out: _linear(l_out, silu(_linear(l_in, pair_ij)))
    m = np.asarray(mask, dtype=np.float64)
    a = psi(p["psi_L_in"], p["psi_L_out"]) * (m[:, None, None] * m[None, :, None])
    b = psi(p["psi_R_in"], p["psi_R_out"]) * m[None, :, None]
    path = np.einsum("ikc,kjc->ijc", a, b) / np.sqrt(max(m.sum(), 1.0))
    p_ij = rms_norm(path, p["ln_path"]["weight"], p["ln_path"]["eps"])
    return mlp(p["ffn"], np.concatenate([pair_ij, p_ij], axis=-1))


def g_descriptor_pool(p, g, xs, mask):
    """model/global_ladder.py:63-136."""
    n, h, dk, dv = xs.shape[0], p["n_heads"], p["d_k"], p["d_v"]
    xn = rms_norm(xs, p["ln_in"]["weight"], p["ln_in"]["eps"])
    q = (g @ p["W_q"]).reshape(h, dk)
    k = _linear(p["K"], xn).reshape(n, h, dk)
    v = _linear(p["V"], xn).reshape(n, h, dv)
    scores = np.einsum("hd,nhd->hn", q, k) / np.sqrt(float(dk))
    scores = np.where(np.asarray(mask)[None, :] > 0, scores, -1.0e30)
    scores = scores - scores.max(axis=-1, keepdims=True)
    attn = np.exp(scores)
    attn = attn / attn.sum(axis=-1, keepdims=True)
    return np.einsum("hn,nhv->hv", attn, v).reshape(-1)


def residual_global_update(p, g, pool):
    """model/global_ladder.py:156-287."""
    x = rms_norm(np.concatenate([g @ p["g_tap_w"], pool]), p["ln_s"], 1e-5)
    return g + p["residual_gain"] * (silu(x @ p["w1"] + p["b1"]) @ p["w2"] + p["b2"])


def boundary_global_update(p, g, pool):
    """model/global_ladder.py:289-334: the update of :func:`residual_global_update` without the
    gain, put back on the sphere."""
    x = rms_norm(np.concatenate([g @ p["g_tap_w"], pool]), p["ln_s"], 1e-5)
    return tree_sphere(g + silu(x @ p["w1"] + p["b1"]) @ p["w2"] + p["b2"])


def edge_rowcol_global_update(p, g, edge, mask):
    """model/global_ladder.py:420-503: one descriptor per edge row and per edge column, pooled
    by the global stream, then the 2n descriptors pooled again and fed to the boundary update."""
    n = edge.shape[0]
    rows = np.stack([g_descriptor_pool(p["row_pool"], g, edge[i], mask) for i in range(n)])
    cols = np.stack([g_descriptor_pool(p["col_pool"], g, edge[:, j], mask) for j in range(n)])
    descs = np.concatenate([rows, cols], axis=0)
    dmask = np.concatenate([np.asarray(mask), np.asarray(mask)])
    return boundary_global_update(p["update"], g, g_descriptor_pool(p["set_pool"], g, descs, dmask))


def _slot_clock(n, d_e, bmask, rope_base, rope_scaling):
    """model/readout_leaf_context.py:543-562: sin/cos of the slot position relative to the centre
    of the active subtree."""
    n_active = max(int(np.asarray(bmask).astype(np.int64).sum()), 1)
    span = 2.0 ** np.ceil(np.log2(float(n_active)))
    pos = (np.arange(n, dtype=np.float64) - (span - 1.0) * 0.5) / rope_scaling
    half = (d_e + 1) // 2
    inv = np.exp(-np.log(rope_base) * np.arange(half) / max(half, 1))
    ang = pos[:, None] * inv[None, :]
    return np.concatenate([np.sin(ang), np.cos(ang)], axis=-1)[:, :d_e]


def _direction(n):
    """model/readout_leaf_context.py:139-147: +1 where the key sits right of the query."""
    idx = np.arange(n)
    rel = idx[:, None] - idx[None, :]
    return np.where(rel < 0, 1.0, np.where(rel > 0, -1.0, 0.0))[..., None]


def physical_readout_context_layer(p, c, edge, bmask, g):
    """model/readout_leaf_context.py:732-836 (with :564-588, :276-324, :680-730)."""
    n = c.shape[0]
    bm = np.asarray(bmask, dtype=np.float64)
    st = bm > 0
    edge_n = rms_norm(edge, p["ln_edge"]["weight"], p["ln_edge"]["eps"])
    direction = _direction(n)
    clock = _slot_clock(n, c.shape[1], bm, p["rope_base"], p["rope_scaling"])
    # edge summary: messages from every other active slot, weighted by exp(-level / 2)
    message = mlp(p["summary_mlp"], np.concatenate([edge_n, edge_n.transpose(1, 0, 2), direction], axis=-1))
    idx = np.arange(n)
    weight = bm[:, None] * bm[None, :] * (1.0 - np.eye(n)) * np.exp(-0.5 * lca_level(idx, idx))
    summary = (message * weight[..., None]).sum(axis=1) / np.maximum(weight.sum(axis=1, keepdims=True), 1.0)
    ctx_in = np.concatenate([rms_norm(c + clock, p["ln_c"]["weight"], p["ln_c"]["eps"]),
                             rms_norm(summary, p["ln_summary"]["weight"], p["ln_summary"]["eps"])], axis=-1)
    c1 = np.where(st[:, None], c + p["residual_scale"] * mlp(p["ctx_mlp"], ctx_in), 0.0)
    g = residual_global_update(p["g_update"], g, g_descriptor_pool(p["g_pool"], g, c1, bm))
    edge_ctx = rms_norm(c1, p["ln_edge_ctx"]["weight"], p["ln_edge_ctx"]["eps"]) @ p["edge_node_ctx_proj"]
    pair = (bm[:, None] * bm[None, :])[..., None]
    g_edge = g @ p["g_edge_proj_w"]
    edge_in = np.concatenate([pair * edge_n, np.broadcast_to(edge_ctx[:, None, :], (n, n, edge_ctx.shape[1])),
                              np.broadcast_to(edge_ctx[None, :, :], (n, n, edge_ctx.shape[1])),
                              np.broadcast_to(g_edge, (n, n, g_edge.shape[0]))], axis=-1)
    edge1 = np.where(pair > 0, edge + p["residual_scale"] * mlp(p["edge_ffn"], edge_in), 0.0)
    # attention
    hk, d = 2 * p["n_heads"], p["d_head"]
    x = rms_norm(c1 + clock, p["ln_attn"]["weight"], p["ln_attn"]["eps"])
    e_att = rms_norm(edge1, p["ln_edge_attn"]["weight"], p["ln_edge_attn"]["eps"])
    qkv = (x @ p["W_QKV"]).reshape(n, 3, hk, d)
    bias = mlp(p["bias_mlp"], np.concatenate([e_att, direction], axis=-1)) / np.sqrt(float(d))
    bias = bias + lca_alibi_bias(idx, idx, lca_fixed_slopes(hk)).transpose(1, 2, 0)
    out = A.gated_edge_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], bias, bm, p["n_heads"], p["attn_impl"])
    out = np.where(st[:, None], c1 + p["residual_scale"] * (out @ p["W_O"]), 0.0)
    return out, edge1, g


def physical_readout_context(p, c, edge, mask, bmask, g):
    """model/readout_leaf_context.py:1078-1215: learned fill-ins for the virtual slots of the
    balanced subtree, then the layers in turn."""
    real = np.asarray(mask) > 0
    virtual = (np.asarray(bmask) > 0) & ~real
    c = np.where(real[:, None], c, np.where(virtual[:, None], p["virtual_node"][None, :], 0.0))
    real_pair = real[:, None] & real[None, :]
    mixed = (real[:, None] & virtual[None, :]) | (virtual[:, None] & real[None, :])
    both_virtual = virtual[:, None] & virtual[None, :]
    edge = np.where(real_pair[..., None], edge,
                    np.where(mixed[..., None], p["edge_empty_nonempty"][None, None, :],
                             np.where(both_virtual[..., None], p["edge_empty_empty"][None, None, :], 0.0)))
    for layer in p["layers"]:
        c, edge, g = physical_readout_context_layer(layer, c, edge, bmask, g)
    return c, edge, g


def transformer_block(p, e, edge, mask, g):
    """model/trunk.py:372-424."""
    gain = p["residual_gain"]
    edge = edge + gain * edge_update_context_aware(p["edge_update_ctx"], edge, e, mask)
    e = e + gain * even_edge_attention(p["attn"], rms_norm(e, p["ln_attn"]["weight"], p["ln_attn"]["eps"]),
                                       edge, mask)
    e_pre = rms_norm(e, p["ln_ffn"]["weight"], p["ln_ffn"]["eps"]) + (g @ p["g_ffn_proj_w"])[None, :]
    e = e + gain * _linear(p["ffn"]["l2"], silu(_linear(p["ffn"]["l1"], e_pre)))
    g = residual_global_update(p["g_update"], g, g_descriptor_pool(p["g_pool"], g, e, mask))
    return e, edge, g


def trunk(blocks, local_feat, edge_feat, mask, g):
    """model/trunk.py:498-529."""
    e, edge = local_feat, edge_feat
    for p in blocks:
        e, edge, g = transformer_block(p, e, edge, mask, g)
    return e, edge, g
