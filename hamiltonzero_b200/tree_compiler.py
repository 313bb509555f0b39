"""The context-only tree reduction of the context compiler: from the contextualised leaves of
one system to the conditioners the walker path consumes.

The reference compiles a lane by reducing the leaf contexts up the balanced tree without any
walker (src/hamiltonzero/compiled/tree.py:96-303): per level a candidate parent context from
the two children, the global stream, the sibling edges, a dyadic clock and count features
(``MergeOp.context_candidate``, src/hamiltonzero/model/tree.py:1701-1807); the edge stream merged
four cells at a time (``edge_merge_masked``, model/tree.py:1996-2052) and refined by a learned
2-FWL contraction (``EdgeFWLUpdate``, model/tree.py:828-952); the level's attention block
(``LevelEdgeAttn``, model/tree.py:1356-1544); the global stream pooled from the level and updated
(src/hamiltonzero/model/global_ladder.py:63-136,337-417). The conditioners are projections of
those contexts (compiled/tree.py:305-340) and come back as a ``CompiledTree``.

Here every level is vectorised over its pairs and cells; the attention runs on ``hz_mhsea_fwd``
through ``context.level_edge_attn`` and the 2-FWL contraction on ``hz_fwl2_panel`` through
``context.fwl2_product``; the small matmuls around them are plain torch on the device, once per
system. Inputs are the outputs of the reference's leaf contextualiser and global fork
(compiled/tree.py:479-494), which are not restated here. Parameters are dicts of fp32 tensors
with the reference's field names."""
from __future__ import annotations

import math

import numpy as np
import torch

from . import context as C
from .systems import CARRY_LEFT, CARRY_RIGHT, EMPTY, MERGE
from .types import CompiledTree, SharedTrunk

_CLOCK_BASE = 10000.0                     # model/tree.py:17
_DEPTH_FEAT_DIM = 32                      # model/tree.py:101


# ------------------------------------------------------------------ clocks and count features
def tree_coord_clock(pos, width: int, base: float = _CLOCK_BASE):
    """``[sin(pos f_k) | cos(pos f_k)]`` cut to ``width`` entries, ``f_k = base^(-k / half)``
    (model/tree.py:20-43)."""
    pos = torch.as_tensor(pos, dtype=torch.float32)
    if width <= 0:
        return pos.new_zeros(pos.shape + (0,))
    half = (width + 1) // 2
    band = torch.arange(half, dtype=torch.float32, device=pos.device)
    inv_freq = torch.exp(-math.log(max(base, 2.0)) * band / float(max(half, 1)))
    phase = pos[..., None] * inv_freq
    return torch.cat([torch.sin(phase), torch.cos(phase)], dim=-1)[..., :width]


def tree_merge_clock(level: int, pair_idx, width: int, max_depth):
    """Clock of the leaf segment a pair covers (model/tree.py:51-101): the segment's centre
    relative to the centre of a tree of depth ``max_depth`` in ``width - 2`` entries, its length
    ``2^(level + 1)`` in the last two."""
    pair = torch.as_tensor(pair_idx, dtype=torch.float32)
    if width <= 0:
        return pair.new_zeros(pair.shape + (0,))
    center_width = max(1, width - 2)
    span = 2.0 ** (level + 1)
    root_center = (2.0 ** max(float(max_depth), 0.0) - 1.0) * 0.5
    center = pair * span + 0.5 * (span - 1.0) - root_center
    return torch.cat([tree_coord_clock(center, center_width),
                      tree_coord_clock(torch.full_like(center, span), width - center_width)], dim=-1)


def tree_depth_count_features(cnt_a, cnt_b, n_total, level, n_levels):
    """24 features of the children's leaf counts and the leaves outside the pair (log2(1 + n) at
    four frequencies) and 8 of the level and the levels above it (model/tree.py:109-130)."""
    a, b = cnt_a.to(torch.float32), cnt_b.to(torch.float32)
    nt = torch.as_tensor(n_total, dtype=torch.float32, device=a.device)
    counts = torch.stack([torch.log2(1.0 + a), torch.log2(1.0 + b),
                          torch.log2(1.0 + torch.clamp(nt - a - b, min=0.0))], dim=-1)
    ang_c = counts[..., None] * (math.pi / 2.0 ** torch.arange(4, dtype=torch.float32, device=a.device))
    f_c = torch.cat([torch.sin(ang_c), torch.cos(ang_c)], dim=-1).reshape(a.shape + (24,))
    lv = torch.full_like(a, float(level))
    levels = torch.stack([lv, float(n_levels) - 1.0 - lv], dim=-1)
    ang_l = levels[..., None] * (math.pi / 2.0 ** torch.arange(2, dtype=torch.float32, device=a.device))
    f_l = torch.cat([torch.sin(ang_l), torch.cos(ang_l)], dim=-1).reshape(a.shape + (8,))
    return torch.cat([f_c, f_l], dim=-1)


def tree_active_clock_depth(mask) -> int:
    """``max(ceil(log2(active leaves)), 1)`` (model/tree.py:2067-2070)."""
    n_active = max(int(torch.as_tensor(mask).to(torch.int64).sum()), 1)
    return max(int(math.ceil(math.log2(float(n_active)))), 1)


def classify_merge_opcodes(leaf_real):
    """Per level the opcode of every pair from which of its children hold real leaves
    (compiled/tree.py:343-361)."""
    active = torch.as_tensor(leaf_real).to(torch.bool)
    n = active.shape[0]
    if n == 0 or n & (n - 1):
        raise ValueError(f"leaf_real width must be a nonzero power of two, got {n}")
    levels = []
    while active.shape[0] > 1:
        left, right = active[0::2], active[1::2]
        levels.append(_opcodes(left, right))
        active = left | right
    return tuple(levels)


def _opcodes(left, right):
    op = torch.full(left.shape, EMPTY, dtype=torch.uint8, device=left.device)
    op[left & right] = MERGE
    op[left & ~right] = CARRY_LEFT
    op[~left & right] = CARRY_RIGHT
    return op


# ------------------------------------------------------------------ the pieces of one level
def rownorm_cols(w):
    """Columns of a weight matrix at unit norm, floor 1e-4 (model/tree.py:208-210)."""
    return w * torch.rsqrt(torch.clamp((w * w).sum(dim=0, keepdim=True), min=1e-4))


def _mlp_rownorm(p, x):
    lin = lambda l, v: v @ rownorm_cols(l["weight"]) + l["bias"]
    x = lin(p["in_proj"], x)
    for nrm, l1, l2 in zip(p["block_norms"], p["block_l1s"], p["block_l2s"]):
        x = x + p["inner_gain"] * lin(l2, C.silu(lin(l1, C.rms_norm(x, nrm["weight"], nrm["eps"]))))
    return lin(p["out_proj"], C.rms_norm(x, p["out_norm"]["weight"], p["out_norm"]["eps"]))


def context_candidate(merge, c_a, c_b, g_level, e_lr, e_rl, level: int, clock_depth, depth):
    """Candidate parent contexts of all pairs of a level (model/tree.py:1701-1807)."""
    pairs = c_a.shape[0]
    clock = tree_merge_clock(level, torch.arange(pairs, device=c_a.device), c_a.shape[-1], clock_depth)
    x = torch.cat([c_a, c_b, g_level[None, :].expand(pairs, -1), e_lr, e_rl, clock.to(c_a.dtype),
                   depth.to(c_a.dtype)], dim=-1)
    return C.ngpt_residual(0.5 * (c_a + c_b), _mlp_rownorm(merge["mlp_c"], x), merge["alpha_c"],
                           max_gain=merge["ngpt_alpha_max"])


def edge_merge_level(em, e_curr, c, k):
    """The parent edge stream ``[P, P, d_edge]`` from the children's ``[2P, 2P, d_edge]``
    (``edge_merge_masked`` over all cells, model/tree.py:636-729,1996-2052): MLP proposal from
    the four child cells and the four child contexts, nGPT step from the structural mean of the
    child cells, zero where a parent lacks a structural child."""
    pairs, d_edge = c.shape[0] // 2, e_curr.shape[-1]
    blocks = e_curr.reshape(pairs, 2, pairs, 2, d_edge)
    e4 = [blocks[:, 0, :, 0], blocks[:, 0, :, 1], blocks[:, 1, :, 0], blocks[:, 1, :, 1]]
    ctx = c if em["node_ctx_proj"] is None else c @ em["node_ctx_proj"]
    ctx_a, ctx_b = ctx[0::2], ctx[1::2]
    rows = lambda v: v[:, None, :].expand(pairs, pairs, -1)
    cols = lambda v: v[None, :, :].expand(pairs, pairs, -1)
    proposal = C.mlp(em["mlp"], torch.cat(e4 + [rows(ctx_a), rows(ctx_b), cols(ctx_a), cols(ctx_b)], dim=-1))
    k_a, k_b = k[0::2], k[1::2]
    w = [k_a[:, None] * k_a[None, :], k_a[:, None] * k_b[None, :], k_b[:, None] * k_a[None, :],
         k_b[:, None] * k_b[None, :]]
    denom = torch.clamp(w[0] + w[1] + w[2] + w[3], min=1.0)
    mean = sum(wi[..., None] * ei for wi, ei in zip(w, e4)) / denom[..., None]
    merged = C.ngpt_residual(mean, proposal, em["alpha"], max_gain=em["ngpt_alpha_max"])
    both = k_a * k_b
    return merged * ((both[:, None] * both[None, :]) > 0)[..., None].to(merged.dtype)


def edge_fwl_residual(p, edge, c_level, mask):
    """The tree's 2-FWL edge update with its nGPT residual (model/tree.py:828-952)."""
    n = c_level.shape[0]
    m = mask.to(edge.dtype)
    c_ln = C.rms_norm(c_level, p["ln_c"]["weight"], p["ln_c"]["eps"])
    c_ctx = c_ln if p["node_ctx_proj"] is None else c_ln @ p["node_ctx_proj"]
    pair = torch.cat([C.rms_norm(edge, p["ln_edge"]["weight"], p["ln_edge"]["eps"]),
                      c_ctx[:, None, :].expand(n, n, -1), c_ctx[None, :, :].expand(n, n, -1)], dim=-1)
    psi = lambda l_in, l_out: C._linear(l_out, C.silu(C._linear(l_in, pair)))
    a = psi(p["psi_L_in"], p["psi_L_out"]) * (m[:, None, None] * m[None, :, None])
    b = psi(p["psi_R_in"], p["psi_R_out"]) * m[None, :, None]
    path = C.fwl2_product(a, b) / torch.sqrt(torch.clamp(m.sum(), min=1.0))
    p_ij = C.rms_norm(path, p["ln_path"]["weight"], p["ln_path"]["eps"])
    delta = C._linear(p["ffn_out"], C.silu(C._linear(p["ffn_in"], torch.cat([pair, p_ij], dim=-1))))
    return C.ngpt_residual(edge, delta, p["alpha"], max_gain=p["ngpt_alpha_max"],
                           update_mask=(m[:, None] * m[None, :]) > 0)


def tree_global_update(p, g, pool, update_active: bool):
    """nGPT step of the global stream towards its MLP proposal (``TreeGlobalUpdate``,
    global_ladder.py:337-417); a level without a structural merge leaves it unchanged."""
    if not update_active:
        return g
    x = C.rms_norm(torch.cat([g @ p["g_tap_w"], pool.to(g.dtype)]), p["ln_s"], 1e-5)
    delta = C.silu(x @ p["w1"] + p["b1"]) @ p["w2"] + p["b2"]
    return C.ngpt_residual(g, delta, p["alpha"], max_gain=p["alpha_max"])


def project_global(p, g):
    """Dense + RMS norm of a global stream (compiled/tree.py:66-93)."""
    return C.rms_norm(g @ p["weight"] + p["bias"], p["norm_scale"], 1e-5)


# ------------------------------------------------------------------ the reduction
def compile_context_only_reduction(merge, gladder, c_leaf, leaf_real, g_emb, edges, structural_mask, *,
                                   n_total=None, clock_depth=None, initial_counts=None, level_offset: int = 0,
                                   feature_n_levels=None):
    """The reduction of compiled/tree.py:96-303: per-level candidates, carried contexts, count
    features, merge conditioners and opcodes, and the root's context, edge and global stream.
    The optional arguments restart it from a partly reduced state
    (``compile_physical_tree_from_reduced_state``, compiled/tree.py:383-467)."""
    c = torch.as_tensor(c_leaf, dtype=torch.float32)
    m = torch.as_tensor(leaf_real).to(c)
    if c.shape[0] != m.shape[0]:
        raise ValueError("c_leaf and leaf_real widths differ")
    n = c.shape[0]
    if n == 0 or n & (n - 1):
        raise ValueError(f"context-only width must be a power of two, got {n}")
    k = torch.as_tensor(structural_mask).to(c)
    if k.shape != m.shape:
        raise ValueError("structural_mask and leaf_real widths differ")
    n_total = m.sum() if n_total is None else n_total
    feature_n_levels = tree_active_clock_depth(m) if feature_n_levels is None else feature_n_levels
    clock_depth = tree_active_clock_depth(k) if clock_depth is None else clock_depth
    counts = m if initial_counts is None else torch.as_tensor(initial_counts).to(m)
    if counts.shape != m.shape:
        raise ValueError("initial_counts and leaf_real widths differ")
    candidates, carried, depth_levels, opcode_levels = [], [], [], []
    g_curr = g_emb
    e_curr = C.tree_sphere(torch.as_tensor(edges, dtype=torch.float32))
    level = int(level_offset)
    while c.shape[0] > 1:
        pairs = c.shape[0] // 2
        idx = torch.arange(pairs, device=c.device)
        c_a, c_b, m_a, m_b, k_a, k_b = c[0::2], c[1::2], m[0::2], m[1::2], k[0::2], k[1::2]
        both = k_a * k_b
        depth = tree_depth_count_features(counts[0::2], counts[1::2], n_total, level, feature_n_levels)
        counts = counts[0::2] + counts[1::2]
        depth_levels.append(depth)
        g_level = g_curr @ gladder["tree_proj_w"] + gladder["tree_proj_b"]
        candidate = context_candidate(merge, c_a, c_b, g_level, e_curr[2 * idx, 2 * idx + 1],
                                      e_curr[2 * idx + 1, 2 * idx], level, clock_depth, depth)
        candidates.append(candidate)
        c_new = (both[:, None] * candidate + (k_a * (1.0 - k_b))[:, None] * c_a
                 + ((1.0 - k_a) * k_b)[:, None] * c_b)
        opcode_levels.append(_opcodes(m_a > 0, m_b > 0))
        e00 = e_curr[0::2, 0::2]
        e_new = edge_merge_level(merge["edge_merge"], e_curr, c, k)
        e_new = edge_fwl_residual(merge["tree_edge_fwl"], e_new, c_new, both)
        keep = ((both[:, None] * both[None, :]) > 0)[..., None]
        e_curr = torch.where(keep, C.tree_sphere(torch.where(keep, e_new, e00)), e00).contiguous()
        c_att = C.level_edge_attn(merge["level_edge_attn"], c_new, e_curr, both, level_idx=level)
        c = torch.where((both > 0)[:, None], C.tree_sphere(c_att), c_new)
        carried.append(c)
        m = m_a + m_b - m_a * m_b
        k = k_a + k_b - k_a * k_b
        pooled = C.g_descriptor_pool(gladder["tree_pool"], g_curr, c, k)
        g_curr = tree_global_update(gladder["tree_update"], g_curr, pooled, bool((both > 0).any()))
        level += 1
    merge_h = tuple(compile_merge_h(merge, cd, dp) for cd, dp in zip(candidates, depth_levels))
    return {"c_candidate": tuple(candidates), "c_carried": tuple(carried), "depth_features": tuple(depth_levels),
            "merge_h": merge_h, "opcodes": tuple(opcode_levels), "c_root": c[0], "e_root": e_curr[0, 0],
            "g_final": g_curr}


def compile_merge_h(merge, c_candidate, depth_features):
    """``[candidate | count features] W_h`` (compiled/tree.py:320-329)."""
    return torch.cat([c_candidate, depth_features.to(c_candidate.dtype)], dim=-1) @ merge["output_hypernet"]["W_h"]


def compile_target_leaf_h(leaf, e_leaf, g_emb):
    """``[e_leaf | g] W_h`` of the leaf hypernetwork (compiled/tree.py:309-317)."""
    ctx = torch.cat([e_leaf, g_emb[None, :].expand(e_leaf.shape[0], -1)], dim=-1)
    return (ctx @ leaf["P_u"]["W_h"],)


def compile_target_readout_h(readout, e_root, c_root, g_emb):
    """``[rms(e_root) | c_root | g] W_h`` of the readout hypernetwork (compiled/tree.py:332-340)."""
    e_norm = C.rms_norm(e_root, readout["ln_e"]["weight"], readout["ln_e"]["eps"])
    return (torch.cat([e_norm, c_root.to(e_norm.dtype), g_emb.to(e_norm.dtype)]) @ readout["output_hypernet"]["W_h"],)


def assemble_compiled_tree(*, perm, leaf_real, boundaries) -> CompiledTree:
    """compiled/tree.py:364-386, as host arrays ready for ``types.to_arrays``."""
    perm = np.asarray(torch.as_tensor(perm).cpu(), dtype=np.int32)
    if perm.ndim != 1:
        raise ValueError(f"perm must be rank one, got shape {perm.shape}")
    leaf_real = np.asarray(torch.as_tensor(leaf_real).cpu()).astype(bool)
    if leaf_real.shape != perm.shape:
        raise ValueError(f"leaf_real shape {leaf_real.shape} must match perm {perm.shape}")
    host = lambda seq: tuple(t.detach().cpu().numpy() for t in seq)
    return CompiledTree(
        perm=perm, inv_perm=np.argsort(perm).astype(np.int32), leaf_real=leaf_real,
        leaf_h=host(boundaries["leaf_h"]), leaf_combiner_h=host(boundaries["leaf_combiner_h"]),
        merge_h=host(boundaries["merge_h"]), opcodes=host(boundaries["opcodes"]),
        readout_h=host(boundaries["readout_h"]), readout_combiner_h=host(boundaries["readout_combiner_h"]))


def compile_physical_tree(params, e_leaf, edge_leaf, g_stream, leaf_real, structural_mask, perm=None) -> CompiledTree:
    """The part of ``compile_physical_tree_from_shared_trunk`` after the leaf contextualiser and
    the global fork (compiled/tree.py:495-530): leaf projection of the global stream, leaf
    contexts, the reduction, root projection, the three conditioner families."""
    n = e_leaf.shape[0]
    perm = torch.arange(n, dtype=torch.int32) if perm is None else perm
    leaf_g = project_global(params["leaf_projection"], g_stream)
    c_leaf = C.tree_sphere(C._linear(params["leaf"]["P_c"], e_leaf))
    reduced = compile_context_only_reduction(params["merge"], params["gladder"], c_leaf, leaf_real, g_stream,
                                             edge_leaf, structural_mask)
    root_g = project_global(params["root_projection"], reduced["g_final"])
    boundaries = {
        "leaf_h": compile_target_leaf_h(params["leaf"], e_leaf, leaf_g), "leaf_combiner_h": (),
        "merge_h": reduced["merge_h"], "opcodes": reduced["opcodes"],
        "readout_h": compile_target_readout_h(params["readout"], reduced["e_root"], reduced["c_root"], root_g),
        "readout_combiner_h": (),
    }
    return assemble_compiled_tree(perm=perm, leaf_real=leaf_real, boundaries=boundaries)


def compile_shared_trunk_from_features(blocks, post, edge_feat, local_feat, global_feat, real_mask,
                                       balanced_mask) -> SharedTrunk:
    """``compile_shared_trunk`` after the featuriser (compiled/trunk.py:108-131): the global seed
    on the sphere, the trunk layers, the global stream pooled from the trunk's edges."""
    g_seed = C.tree_sphere(global_feat.to(local_feat.dtype))
    node_raw, edge_raw, g_seed = C.trunk(blocks, local_feat, edge_feat, real_mask, g_seed)
    return SharedTrunk(node_raw=node_raw, edge_raw=edge_raw, global_raw=global_feat,
                       global_stream=C.edge_rowcol_global_update(post, g_seed.to(edge_raw.dtype), edge_raw, real_mask),
                       real_mask=real_mask, balanced_mask=balanced_mask)


def compile_shared_trunk(featurizer_params, blocks, post, J_double_prime, mask, h_prime, balanced_mask) -> SharedTrunk:
    """``compile_shared_trunk`` (compiled/trunk.py:108-131): the system featuriser on the graph
    inputs (couplings ``[n, n, 10]``, real-site mask, fields ``[n, 3]``), then the trunk and the
    global stream."""
    from .featurizer import system_featurizer
    edge_feat, local_feat, global_feat = system_featurizer(featurizer_params, J_double_prime, mask, h_prime)
    return compile_shared_trunk_from_features(blocks, post, edge_feat, local_feat, global_feat, mask, balanced_mask)


def compile_physical_tree_from_shared_trunk(params, shared: SharedTrunk, perm) -> CompiledTree:
    """compiled/tree.py:470-530: route the trunk state by ``perm``, contextualise the leaves
    (``params["contextualizer"]``), fork the global stream on the leaf edges
    (``params["global_fork"]``), then the reduction and the conditioners."""
    perm = torch.as_tensor(perm, dtype=torch.int64, device=shared.node_raw.device)
    if perm.ndim != 1 or perm.shape != shared.real_mask.shape:
        raise ValueError("perm must be rank one and match the shared trunk site width")
    node = shared.node_raw[perm]
    edge = shared.edge_raw[perm][:, perm]
    leaf_real = shared.real_mask[perm]
    structural = shared.balanced_mask
    e_leaf, edge_leaf, g_stream = C.physical_readout_context(params["contextualizer"], node, edge, leaf_real,
                                                             structural, shared.global_stream)
    g_stream = C.edge_rowcol_global_update(params["global_fork"], g_stream, edge_leaf, structural)
    return compile_physical_tree(params, e_leaf, edge_leaf.contiguous(), g_stream, leaf_real, structural, perm=perm)


# ------------------------------------------------------------------ initialiser
def init_physical_compiler(seed: int, *, d_e: int, d_edge: int, d_c: int, d_feat: int, d_g: int, tap_dim: int,
                           r_leaf: int, r_merge: int, r_ro: int, alpha_init: float = 0.0, alpha_max: float = 0.5,
                           n_heads: int = 4, attn_dim: int | None = None, attn_impl: str = "mhsea_tuned",
                           edge_node_ctx_dim: int | None = None, fwl_channels: int = 64,
                           edge_mlp_hidden: int | None = None, edge_mlp_n_blocks: int = 2,
                           merge_c_mlp_hidden: int | None = None, pool_heads: int = 4, pool_d_k: int = 64,
                           pool_d_v: int = 64, device="cuda"):
    """Parameters of the physical compiler's context side with the reference's shapes and
    initialiser scales: ``MergeOp`` without the carrier (model/tree.py:1560-1651), the tree
    ladder and the two projections (src/hamiltonzero/model/model.py:305-332), ``LeafBuilder.P_c``
    and the three ``W_h`` (model/tree.py:527-549, src/hamiltonzero/model/odd_ops.py:123-129,
    model/tree.py:2342-2363). ``d_feat`` is the width of the global stream, ``d_g`` of its
    projections."""
    node_ctx = d_c if edge_node_ctx_dim is None else int(edge_node_ctx_dim)
    if node_ctx < 1:
        raise ValueError(f"tree edge_node_ctx_dim must be positive or None, got {edge_node_ctx_dim}")
    if not (0 < tap_dim < d_feat):
        raise ValueError("global tap dimension must be positive and smaller than d_g")
    gen = C._gen(seed, device)
    nrm, lin, rms = C._normal, C._init_linear, C._init_rms
    ctx_proj = lambda: None if node_ctx == d_c else nrm(gen, (d_c, node_ctx), d_c ** -0.5, device)
    extra = d_g + 2 * d_edge + d_c + _DEPTH_FEAT_DIM
    c_hidden = max(d_c, 16) if merge_c_mlp_hidden is None else int(merge_c_mlp_hidden)
    e_hidden = max(2 * d_edge, 64) if edge_mlp_hidden is None else int(edge_mlp_hidden)
    d_pair = d_edge + 2 * node_ctx
    alpha = lambda d: torch.full((d,), float(alpha_init), device=device)
    d_pool = pool_heads * pool_d_v
    d_in = tap_dim + d_pool
    merge = {
        "mlp_c": C._init_mlp(gen, 2 * d_c + extra, c_hidden, d_c, 2, 1.0, device, True),
        "alpha_c": alpha(d_c), "ngpt_alpha_max": float(alpha_max),
        "output_hypernet": {"W_h": nrm(gen, (d_c + _DEPTH_FEAT_DIM, r_merge), (d_c + _DEPTH_FEAT_DIM) ** -0.5, device)},
        "edge_merge": {"mlp": C._init_mlp(gen, 4 * d_edge + 4 * node_ctx, e_hidden, d_edge, edge_mlp_n_blocks, 1.0,
                                          device, True),
                       "node_ctx_proj": ctx_proj(), "alpha": alpha(d_edge), "ngpt_alpha_max": float(alpha_max)},
        "level_edge_attn": C.init_level_edge_attn(seed + 1, d_c, d_edge, alpha_init=alpha_init, alpha_max=alpha_max,
                                                  n_heads=n_heads, attn_dim=attn_dim, attn_impl=attn_impl,
                                                  device=device),
        "tree_edge_fwl": {
            "ln_edge": rms(d_edge, device), "ln_c": rms(d_c, device), "node_ctx_proj": ctx_proj(),
            "psi_L_in": lin(gen, d_pair, 2 * fwl_channels, device),
            "psi_L_out": lin(gen, 2 * fwl_channels, fwl_channels, device),
            "psi_R_in": lin(gen, d_pair, 2 * fwl_channels, device),
            "psi_R_out": lin(gen, 2 * fwl_channels, fwl_channels, device),
            "ln_path": rms(fwl_channels, device),
            "ffn_in": lin(gen, d_pair + fwl_channels, max(d_edge, 2 * fwl_channels), device),
            "ffn_out": lin(gen, max(d_edge, 2 * fwl_channels), d_edge, device),
            "alpha": alpha(d_edge), "ngpt_alpha_max": float(alpha_max)},
    }
    gladder = {
        "tree_pool": C._init_pool(gen, d_feat, d_c, pool_heads, pool_d_k, pool_d_v, device),
        "tree_update": {"w1": nrm(gen, (d_in, 2 * d_feat), d_in ** -0.5, device),
                        "b1": torch.zeros(2 * d_feat, device=device),
                        "w2": nrm(gen, (2 * d_feat, d_feat), (2 * d_feat) ** -0.5, device),
                        "b2": torch.zeros(d_feat, device=device), "ln_s": torch.ones(d_in, device=device),
                        "g_tap_w": nrm(gen, (d_feat, tap_dim), d_feat ** -0.5, device),
                        "alpha": alpha(d_feat), "alpha_max": float(alpha_max)},
        "tree_proj_w": nrm(gen, (d_feat, d_g), d_feat ** -0.5, device), "tree_proj_b": torch.zeros(d_g, device=device),
    }
    projection = lambda: {"weight": nrm(gen, (d_feat, d_g), d_feat ** -0.5, device),
                          "bias": torch.zeros(d_g, device=device), "norm_scale": torch.ones(d_g, device=device)}
    return {
        "merge": merge, "gladder": gladder, "leaf_projection": projection(), "root_projection": projection(),
        "leaf": {"P_c": lin(gen, d_e, d_c, device),
                 "P_u": {"W_h": nrm(gen, (d_e + d_g, r_leaf), (d_e + d_g) ** -0.5, device)}},
        "readout": {"ln_e": rms(d_edge, device),
                    "output_hypernet": {"W_h": nrm(gen, (d_edge + d_c + d_g, r_ro), (d_edge + d_c + d_g) ** -0.5,
                                                   device)}},
    }


__all__ = ["assemble_compiled_tree", "classify_merge_opcodes", "compile_context_only_reduction",
           "compile_merge_h", "compile_physical_tree", "compile_physical_tree_from_shared_trunk",
           "compile_shared_trunk", "compile_shared_trunk_from_features", "compile_target_leaf_h", "compile_target_readout_h",
           "context_candidate", "edge_fwl_residual", "edge_merge_level", "init_physical_compiler",
           "project_global", "rownorm_cols", "tree_active_clock_depth", "tree_coord_clock",
           "tree_depth_count_features", "tree_global_update", "tree_merge_clock"]
