"""Test infrastructure, not product code: float64 numpy restatement, one bond and one site at a
time, of the reference's system featuriser (src/hamiltonzero/model/featurizer.py:13-75,274-404,
886-1119). Parameters are the dict of hamiltonzero_b200.featurizer converted with
``context.to_numpy``.
Parity unpinned: the reference holds no golden vectors for the featuriser and JAX is not
installed where this was written; the polar split, the presence rule and the eight strength
features are pinned by hand-worked values in tests/test_featurizer.py."""
import numpy as np

from . import context as C


def lin(p, x):
    return x @ p["weight"] + p["bias"]


def rms(p, x):
    return C.rms_norm(x, p["weight"], p["eps"])


def polar_split(x, tau):
    sq = float((x * x).sum())
    return np.array([np.sqrt(sq)]), x / np.sqrt(sq + tau * tau)


def group_rms(z, w, eps):
    return np.stack([z[g] / np.sqrt((z[g] ** 2).mean() + eps) * w[g] for g in range(z.shape[0])])


def bond_present(j10):
    return bool((j10[:9] != 0).any() or j10[9] > 0.5)


def embed_bond(p, j10):
    """featurizer.py:296-349 for one bond slot."""
    r, u = polar_split(j10[:9], p["tau"])
    z = lin(p["bond_group_w2"], C.silu(lin(p["bond_group_w1"], np.concatenate([j10[:9], r, u, j10[9:]]))))
    g, dg = p["bond_group_ln"]["weight"].shape
    z = group_rms(z.reshape(g, dg), p["bond_group_ln"]["weight"], p["bond_group_ln"]["eps"])
    if not bond_present(j10):
        z = p["tok_bond_gln"]
    return C.silu(lin(p["bond_group_out"], C.silu(lin(p["bond_group_post"], z.reshape(-1)))))


def embed_field(p, h3):
    """featurizer.py:351-404 for one site."""
    r, u = polar_split(h3, p["tau"])
    z = lin(p["zeeman_group_proj"], C.silu(lin(p["zeeman_w1"], np.concatenate([h3, r, u]))))
    g, dg = p["zeeman_group_ln"]["weight"].shape
    z = group_rms(z.reshape(g, dg), p["zeeman_group_ln"]["weight"], p["zeeman_group_ln"]["eps"])
    if not (h3 != 0).any():
        z = p["tok_zeeman_gln"]
    return lin(p["zeeman_w2"], C.silu(lin(p["zeeman_group_post"], z.reshape(-1))))


def _softmax(x):
    e = np.exp(x - x.max())
    return e / e.sum()


def _gate(out, heads):
    return (C.sigmoid(out[:heads]) * out[heads:]).reshape(-1)


def strength_features(J, mask, h):
    """featurizer.py:981-1012."""
    n = J.shape[0]
    num = den = 0.0
    for i in range(n):
        for j in range(n):
            if i != j and mask[i] > 0 and mask[j] > 0:
                num += float((J[i, j, :9] ** 2).sum()); den += 1.0
    rj = np.sqrt(num / max(den, 1.0))
    rh = np.sqrt(sum(float((h[i] ** 2).sum()) for i in range(n) if mask[i] > 0) / max(float(np.sum(mask > 0)), 1.0))
    theta = np.arctan2(rh, rj) if rj + rh > 0 else 0.0
    return np.array([np.log1p(rj), np.log1p(rh), np.sin(2 * theta), np.cos(2 * theta), np.sin(4 * theta),
                     np.cos(4 * theta), np.sin(8 * theta), np.cos(8 * theta)])


def system_featurizer(p, J, mask, h):
    """featurizer.py:886-1119."""
    n, heads, hd = J.shape[0], p["n_heads"], p["head_dim"]
    m = np.asarray(mask, dtype=np.float64)
    real = m > 0
    bond = np.zeros((n, n, p["bond_group_out"]["weight"].shape[1]))
    for i in range(n):
        for j in range(n):
            if real[i] and real[j]:
                bond[i, j] = embed_bond(p, J[i, j])
    # column attention of site i over its bonds j
    local_raw = np.zeros((n, heads * hd))
    for i in range(n):
        if not real[i]:
            continue
        keys = np.stack([rms(p["ln_bond"], bond[i, j]) if bond_present(J[i, j]) else p["tok_bond_key"]
                         for j in range(n)])
        K = (keys @ p["K_col"]).reshape(n, 2 * heads, hd)
        V = (keys @ p["V_col"]).reshape(n, 2 * heads, hd)
        out = np.zeros((2 * heads, hd))
        for hh in range(2 * heads):
            sc = np.array([K[j, hh] @ p["Q_col"][hh] * hd ** -0.5 if real[j] else -1.0e9 for j in range(n)])
            out[hh] = _softmax(sc) @ V[:, hh]
        local_raw[i] = _gate(out, heads)
    local_prime = np.stack([embed_field(p, h[i]) if real[i] else np.zeros(heads * hd) for i in range(n)])
    h_present = np.array([(h[i] != 0).any() for i in range(n)])

    def row_descriptor(x, ln, Q, K, V, present=None):
        xn = np.stack([rms(ln, x[i]) if (present is None or present[i]) else p["tok_field_row"] for i in range(n)])
        kr, vr = (xn @ K).reshape(n, 2 * heads, hd), (xn @ V).reshape(n, 2 * heads, hd)
        out = []
        for q in range(Q.shape[0]):
            ro = np.zeros((2 * heads, hd))
            for hh in range(2 * heads):
                sc = np.array([kr[i, hh] @ Q[q, hh] * hd ** -0.5 if real[i] else -1.0e9 for i in range(n)])
                ro[hh] = _softmax(sc) @ vr[:, hh]
            out.append(_gate(ro, heads))
        return np.concatenate(out)

    g_edge = row_descriptor(local_raw, p["ln_local_pre_row"], p["Q_row"], p["K_row"], p["V_row"])
    g_zee = row_descriptor(local_prime, p["ln_local_pre_row2"], p["Q_row2"], p["K_row2"], p["V_row2"], h_present)
    zee = rms(p["ln_g_zee"], g_zee) if h_present.any() else p["tok_field_global"]
    global_cat = np.concatenate([rms(p["ln_g_edge"], g_edge), zee, strength_features(J, m, h)])
    global_feat = rms(p["ln_global_out"], lin(p["global_w2"], C.silu(lin(p["global_w1"], global_cat))))
    g3 = rms(p["ln_c3"], global_feat)
    local = np.zeros_like(local_prime)
    for i in range(n):
        if not real[i]:
            continue
        first = rms(p["ln_c1"], local_prime[i]) if h_present[i] else p["tok_field_combine"]
        cin = np.concatenate([first, rms(p["ln_c2"], local_raw[i]), g3])
        local[i] = rms(p["ln_local_out"], local_prime[i] + lin(p["combine_w2"], C.silu(lin(p["combine_w1"], cin))))
    film = lin(p["edge_global_film"], rms(p["ln_edge_global"], global_feat))
    half = film.shape[0] // 2
    gamma, beta = 0.1 * np.tanh(film[:half]), 0.1 * film[half:]
    edge = np.zeros((n, n, half))
    for i in range(n):
        for j in range(n):
            if real[i] and real[j]:
                cond = rms(p["ln_edge_cond"], np.concatenate([bond[i, j], local[i], local[j]]))
                core = lin(p["edge_cond_w2"], C.silu(lin(p["edge_cond_w1"], cond)))
                edge[i, j] = rms(p["ln_edge_out"], bond[i, j] @ p["edge_residual_proj"] + core * (1.0 + gamma) + beta)
    return edge, local, global_feat
