"""The system featuriser in front of the trunk: graph inputs to edge, node and global features.

``SystemFeaturizer.__call__`` (src/hamiltonzero/model/featurizer.py:886-1119) restated in torch:
bond embedding with a polar split and grouped RMS norm (:274-349), column attention of every
site over its bonds with learned queries (:916-935), Zeeman embedding of the field (:351-404),
two row descriptors pooled by learned global queries (:937-960), eight features of the mean
coupling and field strengths (:981-1012), the global MLP, the node update, and the edge features
conditioned on both end nodes with a FiLM modulation by the global vector (:1038-1119). Learned
tokens stand in for absent bonds and absent fields. Everything is plain torch on the device,
once per system (its attentions have learned queries and no edge bias: they are not the MHSEA
op); the outputs feed ``tree_compiler.compile_shared_trunk_from_features``. Parameters are a
dict of fp32 tensors with the reference's field names."""
from __future__ import annotations

import math

import torch

from . import context as C


def _lin(p, x):
    return x @ p["weight"] + p["bias"]


def _rms(p, x):
    return C.rms_norm(x, p["weight"], p["eps"])


def polar_split(x, tau: float):
    """Length and regularised direction of the last axis (featurizer.py:274-282)."""
    sq = (x * x).sum(dim=-1, keepdim=True)
    return torch.sqrt(sq), x * torch.rsqrt(sq + tau * tau)


def group_rms(x, weight, eps: float):
    """RMS norm inside each group of the trailing ``[groups, d_group]`` axes (featurizer.py:13-75)."""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def bond_present(J):
    """A bond slot counts as present when any coupling entry is non-zero or its diagonal flag is
    set (featurizer.py:331-333)."""
    return (J[..., :9] != 0).any(dim=-1) | (J[..., 9] > 0.5)


def embed_bonds(p, J):
    """``[n, n, 10]`` couplings (nine entries and a diagonal flag) -> ``[n, n, d_bond]``
    (featurizer.py:296-349)."""
    J9 = J[..., :9]
    r, u = polar_split(J9, p["tau"])
    z = C.silu(_lin(p["bond_group_w1"], torch.cat([J9, r, u, J[..., 9:]], dim=-1)))
    z = _lin(p["bond_group_w2"], z)
    g, dg = p["bond_group_ln"]["weight"].shape
    z = group_rms(z.reshape(*J.shape[:-1], g, dg), p["bond_group_ln"]["weight"], p["bond_group_ln"]["eps"])
    z = torch.where(bond_present(J)[..., None, None], z, p["tok_bond_gln"].to(z.dtype))
    z = C.silu(_lin(p["bond_group_post"], z.reshape(*J.shape[:-1], g * dg)))
    return C.silu(_lin(p["bond_group_out"], z))


def embed_zeeman(p, h):
    """``[n, 3]`` fields -> ``[n, d_local]`` (featurizer.py:351-404)."""
    r, u = polar_split(h, p["tau"])
    z = C.silu(_lin(p["zeeman_w1"], torch.cat([h, r, u], dim=-1)))
    z = _lin(p["zeeman_group_proj"], z)
    g, dg = p["zeeman_group_ln"]["weight"].shape
    z = group_rms(z.reshape(h.shape[0], g, dg), p["zeeman_group_ln"]["weight"], p["zeeman_group_ln"]["eps"])
    z = torch.where((h != 0).any(dim=-1)[:, None, None], z, p["tok_zeeman_gln"].to(z.dtype))
    z = C.silu(_lin(p["zeeman_group_post"], z.reshape(h.shape[0], g * dg)))
    return _lin(p["zeeman_w2"], z)


def _row_descriptor(p, x, ln, Q, K, V, m, present=None):
    """Learned global queries pooling the nodes (featurizer.py:937-960): ``[d_global]``."""
    n, heads, hd = x.shape[0], p["n_heads"], p["head_dim"]
    xn = _rms(ln, x)
    if present is not None:
        xn = torch.where(present[:, None], xn, p["tok_field_row"].to(xn.dtype))
    kr = (xn @ K).reshape(n, 2 * heads, hd)
    vr = (xn @ V).reshape(n, 2 * heads, hd)
    sc = torch.einsum("qhd,ihd->qhi", Q, kr) * hd ** -0.5
    sc = torch.where(m[None, None, :] > 0, sc, torch.full_like(sc, -1.0e9))
    ro = torch.einsum("qhi,ihd->qhd", torch.softmax(sc, dim=-1), vr)
    return (torch.sigmoid(ro[:, :heads]) * ro[:, heads:]).reshape(-1)


def system_featurizer(p, J_double_prime, mask, h_prime):
    """``(edge [n, n, d_edge], local [n, d_local], global [d_global])`` of one system
    (featurizer.py:886-1119)."""
    dtype = p["Q_col"].dtype             # fp32 in the product; the CPU tests run it in fp64
    J = J_double_prime.to(dtype)
    h = h_prime.to(dtype)
    n, heads, hd = J.shape[0], p["n_heads"], p["head_dim"]
    m = mask.to(dtype)
    pair = m[:, None] * m[None, :]
    bond_emb = embed_bonds(p, J) * pair[..., None]
    bond_norm = torch.where(bond_present(J)[..., None], _rms(p["ln_bond"], bond_emb), p["tok_bond_key"])
    # column attention: every site over its bonds, one learned query per kernel head
    K = (bond_norm @ p["K_col"]).reshape(n, n, 2 * heads, hd)
    V = (bond_norm @ p["V_col"]).reshape(n, n, 2 * heads, hd)
    scores = torch.einsum("hd,ijhd->ijh", p["Q_col"], K) * hd ** -0.5
    scores = torch.where(pair[..., None] > 0, scores, torch.full_like(scores, -1.0e9))
    col = torch.einsum("ijh,ijhd->ihd", torch.softmax(scores, dim=1), V)
    local_raw = (torch.sigmoid(col[:, :heads]) * col[:, heads:]).reshape(n, -1) * m[:, None]
    local_prime = embed_zeeman(p, h) * m[:, None]
    h_present = (h != 0).any(dim=-1)
    g_edge = _row_descriptor(p, local_raw, p["ln_local_pre_row"], p["Q_row"], p["K_row"], p["V_row"], m)
    g_zee = _row_descriptor(p, local_prime, p["ln_local_pre_row2"], p["Q_row2"], p["K_row2"], p["V_row2"], m,
                            present=h_present)
    # mean coupling and field strengths, their ratio as an angle
    off = pair * (1.0 - torch.eye(n, dtype=pair.dtype, device=pair.device))
    mean_j2 = ((J[..., :9] ** 2).sum(dim=-1) * off).sum() / torch.clamp(off.sum(), min=1.0)
    mean_h2 = ((h ** 2).sum(dim=-1) * m).sum() / torch.clamp(m.sum(), min=1.0)
    rj, rh = torch.sqrt(torch.clamp(mean_j2, min=0.0)), torch.sqrt(torch.clamp(mean_h2, min=0.0))
    nonzero = (rj + rh) > 0
    theta = torch.atan2(torch.where(nonzero, rh, torch.zeros_like(rh)), torch.where(nonzero, rj, torch.ones_like(rj)))
    jh = torch.stack([torch.log1p(rj), torch.log1p(rh), torch.sin(2 * theta), torch.cos(2 * theta),
                      torch.sin(4 * theta), torch.cos(4 * theta), torch.sin(8 * theta), torch.cos(8 * theta)])
    zee_part = _rms(p["ln_g_zee"], g_zee) if bool(h_present.any()) else p["tok_field_global"]
    global_cat = torch.cat([_rms(p["ln_g_edge"], g_edge), zee_part, jh])
    global_feat = _rms(p["ln_global_out"], _lin(p["global_w2"], C.silu(_lin(p["global_w1"], global_cat))))
    combine_in = torch.cat([torch.where(h_present[:, None], _rms(p["ln_c1"], local_prime), p["tok_field_combine"]),
                            _rms(p["ln_c2"], local_raw),
                            _rms(p["ln_c3"], global_feat)[None, :].expand(n, -1)], dim=-1)
    local = _rms(p["ln_local_out"], local_prime + _lin(p["combine_w2"], C.silu(_lin(p["combine_w1"], combine_in))))
    local = local * m[:, None]
    cond = torch.cat([bond_emb, local[:, None, :].expand(n, n, -1), local[None, :, :].expand(n, n, -1)], dim=-1)
    core = _lin(p["edge_cond_w2"], C.silu(_lin(p["edge_cond_w1"], _rms(p["ln_edge_cond"], cond))))
    film = _lin(p["edge_global_film"], _rms(p["ln_edge_global"], global_feat))
    gamma, beta = 0.1 * torch.tanh(film[: film.shape[0] // 2]), 0.1 * film[film.shape[0] // 2:]
    edge = _rms(p["ln_edge_out"], bond_emb @ p["edge_residual_proj"] + core * (1.0 + gamma) + beta)
    return edge * pair[..., None], local, global_feat


def init_system_featurizer(seed: int, *, d_bond: int, n_heads: int, head_dim: int, n_global_q: int, d_edge: int,
                           d_hidden_edge: int, polar_group_norm_tau: float = 1e-3,
                           polar_group_norm_bond_hidden: int = 128, polar_group_norm_n_bond_groups: int = 16,
                           polar_group_norm_d_bond_group: int = 16, polar_group_norm_n_zeeman_groups: int = 16,
                           polar_group_norm_d_zeeman_group: int = 16, zeeman_hidden_dim: int,
                           global_hidden_dim: int, combine_hidden_dim: int, token_initial_scale: float,
                           device="cuda"):
    """Parameters of ``SystemFeaturizer`` (featurizer.py:149-272) with the reference's shapes and
    initialiser scales (weights normal * fan_in^-1/2, learned queries normal * head_dim^-1/2,
    tokens normal * ``token_initial_scale``, unit norm scales, zero biases)."""
    gen = C._gen(seed, device)
    lin, rms, nrm = C._init_linear, C._init_rms, C._normal
    d_local, d_global = n_heads * head_dim, n_global_q * n_heads * head_dim
    hk, dk = 2 * n_heads, 2 * n_heads * head_dim
    bh = polar_group_norm_bond_hidden
    gb, db = polar_group_norm_n_bond_groups, polar_group_norm_d_bond_group
    gz, dz = polar_group_norm_n_zeeman_groups, polar_group_norm_d_zeeman_group
    cond_in = d_bond + 2 * d_local
    free = lambda d_in, d_out: nrm(gen, (d_in, d_out), d_in ** -0.5, device)
    tok = lambda *shape: nrm(gen, shape, float(token_initial_scale), device)
    return {
        "tau": float(polar_group_norm_tau), "n_heads": n_heads, "head_dim": head_dim,
        "bond_group_w1": lin(gen, 20, bh, device), "bond_group_w2": lin(gen, bh, gb * db, device),
        "bond_group_post": lin(gen, gb * db, bh, device), "bond_group_out": lin(gen, bh, d_bond, device),
        "bond_group_ln": {"weight": torch.ones(gb, db, device=device), "eps": 1e-5},
        "Q_col": nrm(gen, (hk, head_dim), head_dim ** -0.5, device),
        "K_col": free(d_bond, dk), "V_col": free(d_bond, dk), "ln_bond": rms(d_bond, device),
        "Q_row": nrm(gen, (n_global_q, hk, head_dim), head_dim ** -0.5, device),
        "K_row": free(d_local, dk), "V_row": free(d_local, dk), "ln_local_pre_row": rms(d_local, device),
        "ln_edge_cond": rms(cond_in, device), "edge_cond_w1": lin(gen, cond_in, d_hidden_edge, device),
        "edge_cond_w2": lin(gen, d_hidden_edge, d_edge, device), "ln_edge_global": rms(d_global, device),
        "edge_global_film": lin(gen, d_global, 2 * d_edge, device), "edge_residual_proj": free(d_bond, d_edge),
        "zeeman_w1": lin(gen, 7, zeeman_hidden_dim, device),
        "zeeman_group_proj": lin(gen, zeeman_hidden_dim, gz * dz, device),
        "zeeman_group_ln": {"weight": torch.ones(gz, dz, device=device), "eps": 1e-5},
        "zeeman_group_post": lin(gen, gz * dz, zeeman_hidden_dim, device),
        "zeeman_w2": lin(gen, zeeman_hidden_dim, d_local, device),
        "Q_row2": nrm(gen, (n_global_q, hk, head_dim), head_dim ** -0.5, device),
        "K_row2": free(d_local, dk), "V_row2": free(d_local, dk), "ln_local_pre_row2": rms(d_local, device),
        "ln_g_edge": rms(d_global, device), "ln_g_zee": rms(d_global, device),
        "global_w1": lin(gen, 2 * d_global + 8, global_hidden_dim, device),
        "global_w2": lin(gen, global_hidden_dim, d_global, device),
        "ln_c1": rms(d_local, device), "ln_c2": rms(d_local, device), "ln_c3": rms(d_global, device),
        "combine_w1": lin(gen, 2 * d_local + d_global, combine_hidden_dim, device),
        "combine_w2": lin(gen, combine_hidden_dim, d_local, device),
        "ln_edge_out": rms(d_edge, device), "ln_local_out": rms(d_local, device),
        "ln_global_out": rms(d_global, device),
        "tok_bond_gln": tok(gb, db), "tok_zeeman_gln": tok(gz, dz), "tok_bond_key": tok(d_bond),
        "tok_field_row": tok(d_local), "tok_field_global": tok(d_global), "tok_field_combine": tok(d_local),
    }


__all__ = ["bond_present", "embed_bonds", "embed_zeeman", "group_rms", "init_system_featurizer", "polar_split",
           "system_featurizer"]
