"""Test infrastructure, not product code: float64 numpy restatement, one pair and one edge cell
at a time, of the reference's context-only tree reduction
(src/hamiltonzero/compiled/tree.py:96-303) that emits the merge conditioners, the opcodes and
the root context of a compiled tree, with the pieces it calls: the dyadic clocks and count
features (src/hamiltonzero/model/tree.py:20-130), the candidate context of a merge
(model/tree.py:1653-1807), the edge merge of four child cells (model/tree.py:636-729,1996-2052),
the 2-FWL edge update (model/tree.py:828-952), the tree-level global update
(src/hamiltonzero/model/global_ladder.py:337-417) and the conditioner projections
(compiled/tree.py:305-340). Parameters are the dicts of hamiltonzero_b200.tree_compiler
converted with ``to_numpy``.
Parity unpinned for these blocks: the reference holds no golden vectors for them and JAX is
not installed where this was written; clocks, count features and opcodes are pinned by
hand-worked values in tests/test_tree_compiler.py."""
import numpy as np

from . import context as C

MERGE, CARRY_LEFT, CARRY_RIGHT, EMPTY = 0, 1, 2, 3       # compiled/types.py:15-19
CLOCK_BASE = 10000.0
DEPTH_FEAT_DIM = 32


def coord_clock(pos, width, base=CLOCK_BASE):
    """model/tree.py:20-43: ``[sin(pos f_k) | cos(pos f_k)]`` cut to ``width`` entries."""
    if width <= 0:
        return np.zeros(0)
    half = (width + 1) // 2
    out = []
    for fn in (np.sin, np.cos):
        for k in range(half):
            out.append(fn(pos * np.exp(-np.log(max(base, 2.0)) * k / max(half, 1))))
    return np.array(out[:width])


def merge_clock(level, pair, width, max_depth):
    """model/tree.py:51-101: centre of the pair's leaf segment (relative to the centre of the
    tree of depth ``max_depth``) and the segment length, each as a clock."""
    if width <= 0:
        return np.zeros(0)
    center_width = max(1, width - 2)
    span = 2.0 ** (level + 1)
    root_center = (2.0 ** max(float(max_depth), 0.0) - 1.0) * 0.5
    center = pair * span + 0.5 * (span - 1.0) - root_center
    return np.concatenate([coord_clock(center, center_width), coord_clock(span, width - center_width)])


def depth_count_features(cnt_a, cnt_b, n_total, level, n_levels):
    """model/tree.py:109-130 for one pair: 24 count features and 8 level features."""
    feats = []
    for v in (np.log2(1.0 + cnt_a), np.log2(1.0 + cnt_b), np.log2(1.0 + max(n_total - cnt_a - cnt_b, 0.0))):
        ang = [v * np.pi / 2.0 ** k for k in range(4)]
        feats += [np.sin(a) for a in ang] + [np.cos(a) for a in ang]
    for v in (float(level), float(n_levels) - 1.0 - float(level)):
        ang = [v * np.pi / 2.0 ** k for k in range(2)]
        feats += [np.sin(a) for a in ang] + [np.cos(a) for a in ang]
    return np.array(feats)


def active_clock_depth(mask):
    """model/tree.py:2067-2070."""
    n_active = max(int(np.asarray(mask).astype(np.int64).sum()), 1)
    return max(int(np.ceil(np.log2(float(n_active)))), 1)


def rownorm_cols(w):
    """model/tree.py:208-210."""
    return w / np.sqrt(np.maximum((w * w).sum(axis=0, keepdims=True), 1e-4))


def _ngpt(skip, proposal, alpha, max_gain):
    skip_n, prop_n = C.tree_sphere(skip), C.tree_sphere(proposal)
    return C.tree_sphere(skip_n + max_gain * C.sigmoid(alpha) * (prop_n - skip_n))


def _mlp(p, x, weight_map=lambda w: w):
    lin = lambda l, v: v @ weight_map(l["weight"]) + l["bias"]
    x = lin(p["in_proj"], x)
    for nrm, l1, l2 in zip(p["block_norms"], p["block_l1s"], p["block_l2s"]):
        x = x + p["inner_gain"] * lin(l2, C.silu(lin(l1, C.rms_norm(x, nrm["weight"], nrm["eps"]))))
    return lin(p["out_proj"], C.rms_norm(x, p["out_norm"]["weight"], p["out_norm"]["eps"]))


def context_candidate(merge, c_a, c_b, g_level, e_lr, e_rl, level, pair, clock_depth, depth):
    """model/tree.py:1701-1807: MLP with column-normalised weights of ``[c_a | c_b | g | sibling
    edges | clock | count features]``, then the nGPT step from the children's mean."""
    x = np.concatenate([c_a, c_b, g_level, e_lr, e_rl, merge_clock(level, pair, c_a.shape[-1], clock_depth), depth])
    delta = _mlp(merge["mlp_c"], x, rownorm_cols)
    return _ngpt(0.5 * (c_a + c_b), delta, merge["alpha_c"], merge["ngpt_alpha_max"])


def edge_merge_cell(em, e4, c4, k4):
    """model/tree.py:1996-2052 for one parent cell: ``e4`` the child cells (2i,2j), (2i,2j+1),
    (2i+1,2j), (2i+1,2j+1); ``c4`` the contexts of 2i, 2i+1, 2j, 2j+1; ``k4`` their structural
    masks. Zero unless both parents have two structural children."""
    out_mask = k4[0] * k4[1] * k4[2] * k4[3]
    ctx = [c if em["node_ctx_proj"] is None else c @ em["node_ctx_proj"] for c in c4]
    proposal = _mlp(em["mlp"], np.concatenate(list(e4) + ctx))
    w = np.array([k4[0] * k4[2], k4[0] * k4[3], k4[1] * k4[2], k4[1] * k4[3]])
    mean = sum(wi * ei for wi, ei in zip(w, e4)) / max(w.sum(), 1.0)
    merged = _ngpt(mean, proposal, em["alpha"], em["ngpt_alpha_max"])
    return merged if out_mask > 0 else np.zeros_like(merged)


def edge_fwl_residual(p, edge, c_level, mask):
    """model/tree.py:828-952: pair features ``[rms(edge) | ctx_i | ctx_j]``, two pair maps
    contracted over the middle node, normalised path feature, one hidden layer, nGPT step on
    the cells whose two nodes are active."""
    n = c_level.shape[0]
    m = np.asarray(mask, dtype=np.float64)
    lin = lambda l, v: v @ l["weight"] + l["bias"]
    c_ln = C.rms_norm(c_level, p["ln_c"]["weight"], p["ln_c"]["eps"])
    c_ctx = c_ln if p["node_ctx_proj"] is None else c_ln @ p["node_ctx_proj"]
    pair = np.empty((n, n, edge.shape[-1] + 2 * c_ctx.shape[-1]))
    for i in range(n):
        for j in range(n):
            pair[i, j] = np.concatenate([C.rms_norm(edge[i, j], p["ln_edge"]["weight"], p["ln_edge"]["eps"]),
                                         c_ctx[i], c_ctx[j]])
    a = lin(p["psi_L_out"], C.silu(lin(p["psi_L_in"], pair))) * (m[:, None, None] * m[None, :, None])
    b = lin(p["psi_R_out"], C.silu(lin(p["psi_R_in"], pair))) * m[None, :, None]
    path = np.zeros((n, n, a.shape[-1]))
    for k in range(n):
        path += a[:, k, None, :] * b[None, k, :, :]
    path = path / np.sqrt(max(m.sum(), 1.0))
    p_ij = C.rms_norm(path, p["ln_path"]["weight"], p["ln_path"]["eps"])
    delta = lin(p["ffn_out"], C.silu(lin(p["ffn_in"], np.concatenate([pair, p_ij], axis=-1))))
    updated = _ngpt(edge, delta, p["alpha"], p["ngpt_alpha_max"])
    keep = (m[:, None] * m[None, :]) > 0
    return np.where(keep[..., None], updated, edge)


def tree_global_update(p, g, pool, update_mask):
    """global_ladder.py:337-417: nGPT step of the global stream towards its MLP proposal."""
    x = C.rms_norm(np.concatenate([g @ p["g_tap_w"], pool]), p["ln_s"], 1e-5)
    delta = C.silu(x @ p["w1"] + p["b1"]) @ p["w2"] + p["b2"]
    return _ngpt(g, delta, p["alpha"], p["alpha_max"]) if update_mask else g


def project_global(p, g):
    """compiled/tree.py:66-93."""
    return C.rms_norm(g @ p["weight"] + p["bias"], p["norm_scale"], 1e-5)


def context_only_reduction(merge, gladder, c_leaf, leaf_real, g_emb, edges, structural_mask):
    """compiled/tree.py:96-303 with the defaults of ``compile_physical_tree_from_shared_trunk``
    (counts start from the real leaves, level offset 0)."""
    c = np.asarray(c_leaf, dtype=np.float64)
    m = np.asarray(leaf_real, dtype=np.float64)
    k = np.asarray(structural_mask, dtype=np.float64)
    n = c.shape[0]
    if n == 0 or n & (n - 1):
        raise ValueError(f"context-only width must be a power of two, got {n}")
    n_total, n_levels, clock_depth = m.sum(), active_clock_depth(m), active_clock_depth(k)
    counts = m.copy()
    e_curr = C.tree_sphere(np.asarray(edges, dtype=np.float64))
    g_curr = np.asarray(g_emb, dtype=np.float64)
    candidates, carried, depth_levels, opcodes = [], [], [], []
    level = 0
    while c.shape[0] > 1:
        pairs = c.shape[0] // 2
        both = k[0::2] * k[1::2]
        depth = np.stack([depth_count_features(counts[2 * p], counts[2 * p + 1], n_total, level, n_levels)
                          for p in range(pairs)])
        counts = counts[0::2] + counts[1::2]
        depth_levels.append(depth)
        g_level = g_curr @ gladder["tree_proj_w"] + gladder["tree_proj_b"]
        cand = np.stack([context_candidate(merge, c[2 * p], c[2 * p + 1], g_level, e_curr[2 * p, 2 * p + 1],
                                           e_curr[2 * p + 1, 2 * p], level, p, clock_depth, depth[p])
                         for p in range(pairs)])
        candidates.append(cand)
        c_new = np.empty((pairs, c.shape[1]))
        op = np.empty(pairs, dtype=np.uint8)
        for p in range(pairs):
            ka, kb = k[2 * p], k[2 * p + 1]
            c_new[p] = ka * kb * cand[p] + ka * (1 - kb) * c[2 * p] + (1 - ka) * kb * c[2 * p + 1]
            ma, mb = m[2 * p] > 0, m[2 * p + 1] > 0
            op[p] = MERGE if ma and mb else CARRY_LEFT if ma else CARRY_RIGHT if mb else EMPTY
        opcodes.append(op)
        e_new = np.empty((pairs, pairs, e_curr.shape[-1]))
        for p in range(pairs):
            for q in range(pairs):
                e_new[p, q] = edge_merge_cell(
                    merge["edge_merge"],
                    (e_curr[2 * p, 2 * q], e_curr[2 * p, 2 * q + 1], e_curr[2 * p + 1, 2 * q],
                     e_curr[2 * p + 1, 2 * q + 1]),
                    (c[2 * p], c[2 * p + 1], c[2 * q], c[2 * q + 1]),
                    (k[2 * p], k[2 * p + 1], k[2 * q], k[2 * q + 1]))
        e00 = e_curr[0::2, 0::2]
        e_new = edge_fwl_residual(merge["tree_edge_fwl"], e_new, c_new, both)
        keep = ((both[:, None] * both[None, :]) > 0)[..., None]
        e_curr = np.where(keep, C.tree_sphere(np.where(keep, e_new, e00)), e00)
        c_att = C.level_edge_attn(merge["level_edge_attn"], c_new, e_curr, both, level_idx=level)
        c = np.where((both > 0)[:, None], C.tree_sphere(c_att), c_new)
        carried.append(c)
        m = m[0::2] + m[1::2] - m[0::2] * m[1::2]
        k = k[0::2] + k[1::2] - k[0::2] * k[1::2]
        active = bool((both > 0).any())
        pooled = C.g_descriptor_pool(gladder["tree_pool"], g_curr, c, k)
        g_curr = tree_global_update(gladder["tree_update"], g_curr, pooled, active)
        level += 1
    w_h = merge["output_hypernet"]["W_h"]
    return {"c_candidate": candidates, "c_carried": carried, "depth_features": depth_levels,
            "merge_h": [np.concatenate([cd, dp], axis=-1) @ w_h for cd, dp in zip(candidates, depth_levels)],
            "opcodes": opcodes, "c_root": c[0], "e_root": e_curr[0, 0], "g_final": g_curr}


def leaf_h(leaf, e_leaf, g_emb):
    """compiled/tree.py:309-317."""
    ctx = np.concatenate([e_leaf, np.broadcast_to(g_emb, (e_leaf.shape[0], g_emb.shape[0]))], axis=-1)
    return ctx @ leaf["P_u"]["W_h"]


def readout_h(readout, e_root, c_root, g_emb):
    """compiled/tree.py:332-340."""
    e_norm = C.rms_norm(e_root, readout["ln_e"]["weight"], readout["ln_e"]["eps"])
    return np.concatenate([e_norm, c_root, g_emb]) @ readout["output_hypernet"]["W_h"]


def compile_tree(params, e_leaf, edge_leaf, g_stream, leaf_real, structural_mask):
    """compiled/tree.py:470-530 after the contextualiser and the global fork: returns
    ``(leaf_h, merge_h per level, opcodes per level, readout_h)``."""
    leaf_g = project_global(params["leaf_projection"], g_stream)
    c_leaf = C.tree_sphere(e_leaf @ params["leaf"]["P_c"]["weight"] + params["leaf"]["P_c"]["bias"])
    red = context_only_reduction(params["merge"], params["gladder"], c_leaf, leaf_real, g_stream, edge_leaf,
                                 structural_mask)
    root_g = project_global(params["root_projection"], red["g_final"])
    return (leaf_h(params["leaf"], e_leaf, leaf_g), red["merge_h"], red["opcodes"],
            readout_h(params["readout"], red["e_root"], red["c_root"], root_g))


def compile_tree_from_shared_trunk(params, node_raw, edge_raw, global_stream, real_mask, balanced_mask, perm):
    """compiled/tree.py:470-494 in front of :func:`compile_tree`: route by ``perm``, leaf
    contextualiser, global fork."""
    perm = np.asarray(perm)
    node, edge, leaf_real = node_raw[perm], edge_raw[perm][:, perm], np.asarray(real_mask)[perm]
    e_leaf, edge_leaf, g = C.physical_readout_context(params["contextualizer"], node, edge, leaf_real, balanced_mask,
                                                      global_stream)
    g = C.edge_rowcol_global_update(params["global_fork"], g, edge_leaf, balanced_mask)
    return compile_tree(params, e_leaf, edge_leaf, g, leaf_real, balanced_mask)
