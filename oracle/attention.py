"""NumPy restatement of the reference's masked multi-head softmax attention with
additive edge bias ("MHSEA"): forward, forward-mode tangent and backward.

TEST INFRASTRUCTURE: checker for the CUDA kernels; never imported by the package.
Parity unpinned: the reference holds no golden vectors for this op.

Follows, line by line:
  * forward      src/hamiltonzero/model/_pallas_attn/mhsea.py:13-31 and the
                 wrapper's zeroing of masked query rows
                 src/hamiltonzero/model/_pallas_attn/mhsea_tuned.py:76-92
  * masked score src/hamiltonzero/model/_pallas_attn/utils.py:52-53 (-10000.0)
  * tangent      src/hamiltonzero/model/_pallas_attn/mhsea_tuned_jvp.py:20-91
                 (small-N twin: mhsea_full_ad_jvp.py:19-69 — same mathematics)
  * backward     src/hamiltonzero/model/_pallas_attn/custom_gradients.py:231-347
  * dispatcher   src/hamiltonzero/model/pallas_attention.py:22-67

Layouts: q,k,v,out,tangents,grads [B,N,H,D]; e,de [B,N,H,N]; mask [B,N]; lse [B,N,H].
``q`` at primitive level is already multiplied by D**-0.5.  All functions take a
``dtype`` so the same code gives the fp64 truth and an fp32 yardstick.
"""
from __future__ import annotations

import numpy as np

BIG_NEGATIVE = -10000.0          # utils.py:52-53
EINSUM_KEY_MASK = -1e9           # pallas_attention.py:33


def _prep(q, k, e, v, mask, dtype):
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    B, N, H, D = q.shape
    if e is None:
        e = np.zeros((B, N, H, N), dtype=dtype)
    e = np.asarray(e, dtype=dtype)
    if mask is None:
        mask = np.ones((B, N), dtype=bool)
    mask = np.asarray(mask).astype(bool)
    m4 = mask[:, :, None, None]
    qz = np.where(m4, q, 0)                    # mhsea.py:20
    kz = np.where(m4, k, 0)                    # mhsea.py:21
    vz = np.where(m4, v, 0)                    # mhsea.py:23
    square = mask[:, :, None, None] & mask[:, None, None, :]   # [B,Nq,1,Nk]  mhsea.py:19
    return qz, kz, e, vz, mask, square


def _scores(qz, kz, e, square):
    # s[b,i,h,j] = q[b,i,h,:]·k[b,j,h,:] + e[b,i,h,j]  (mhsea.py:24-26)
    s = np.einsum("bihd,bjhd->bihj", qz, kz) + e
    return np.where(square, s, np.asarray(BIG_NEGATIVE, dtype=s.dtype))


def mhsea_fwd(q, k, e, v, mask, dtype=np.float64):
    """Primal primitive ``mhsea_tuned_ad`` / ``mhsea_full_ad``: returns (out, lse)."""
    qz, kz, e, vz, mask, square = _prep(q, k, e, v, mask, dtype)
    s = _scores(qz, kz, e, square)
    mx = s.max(axis=-1)                                        # mhsea.py:27
    lse = mx + np.log(np.exp(s - mx[..., None]).sum(axis=-1))  # mhsea.py:28
    p = np.exp(s - lse[..., None])                             # mhsea.py:29
    out = np.einsum("bihj,bjhd->bihd", p, vz)                  # mhsea.py:31
    out = np.where(mask[:, :, None, None], out, 0)             # mhsea_tuned.py:91
    return out, lse


def mhsea_jvp(q, k, e, v, mask, out, lse, qt, kt, et, vt, dtype=np.float64):
    """Linear tangent primitive ``mhsea_tuned_ad_lin`` (mhsea_tuned_jvp.py:20-91)."""
    qz, kz, e, vz, mask, square = _prep(q, k, e, v, mask, dtype)
    qtz, ktz, et, vtz, _, _ = _prep(qt, kt, et, vt, mask, dtype)
    out = np.asarray(out, dtype=dtype)
    lse = np.asarray(lse, dtype=dtype)
    s = _scores(qz, kz, e, square)
    p = np.exp(s - lse[..., None])                             # :67
    sd = (np.einsum("bihd,bjhd->bihj", qtz, kz)
          + np.einsum("bihd,bjhd->bihj", qz, ktz) + et)        # :68-72
    sd = np.where(square, sd, 0)                               # :73
    psd = p * sd                                               # :74
    mean = psd.sum(axis=-1)                                    # :75
    tangent = (np.einsum("bihj,bjhd->bihd", psd, vz)           # :76-78
               + np.einsum("bihj,bjhd->bihd", p, vtz)          # :79-81
               - mean[..., None] * out)                        # :88
    return np.where(mask[:, :, None, None], tangent, 0)        # :89


def mhsea_bwd(q, k, e, v, mask, lse, out, dout, dtype=np.float64):
    """Transpose of the tangent primitive (custom_gradients.py:231-347):
    returns (dq, dk, de, dv); ``dq`` is the gradient w.r.t. the pre-scaled q."""
    qz, kz, e, vz, mask, square = _prep(q, k, e, v, mask, dtype)
    out = np.asarray(out, dtype=dtype)
    lse = np.asarray(lse, dtype=dtype)
    do = np.where(mask[:, :, None, None], np.asarray(dout, dtype=dtype), 0)  # :263-265
    s = _scores(qz, kz, e, square)
    p = np.exp(s - lse[..., None])                             # :262
    delta = (out * do).sum(axis=-1)                            # sum_columns(o*o_vjp) :267-268
    ds = (np.einsum("bihd,bjhd->bihj", do, vz) - delta[..., None]) * p
    ds = ds * square                                           # :270
    dq = np.einsum("bihj,bjhd->bihd", ds, kz)                  # :271
    dk = np.einsum("bihj,bihd->bjhd", ds, qz)                  # :336
    dv = np.einsum("bihj,bihd->bjhd", p, do)                   # :337
    return dq, dk, ds, dv                                      # de = dS :273


# ---------------------------------------------------------------- dispatcher level
def reference_edge_attention(Q, K, V, edge_bias, mask, dtype=np.float64):
    """Einsum twin (pallas_attention.py:22-37): keys-only additive -1e9 mask."""
    Q = np.asarray(Q, dtype=dtype); K = np.asarray(K, dtype=dtype); V = np.asarray(V, dtype=dtype)
    n, h, d = Q.shape
    logits = np.einsum("ihd,jhd->hij", Q, K) * (float(d) ** -0.5)
    logits = logits + np.transpose(np.asarray(edge_bias, dtype=dtype), (2, 0, 1))
    logits = logits + (1.0 - np.asarray(mask).astype(dtype))[None, None, :] * EINSUM_KEY_MASK
    logits = logits - logits.max(axis=-1, keepdims=True)
    alpha = np.exp(logits)
    alpha = alpha / alpha.sum(axis=-1, keepdims=True)
    return np.einsum("hij,jhd->ihd", alpha, V)


def supports_tuned(n, d):       # mhsea_tuned.py:53-60
    return n >= 64 and n % 32 == 0 and d in (8, 16, 32, 64)


def supports_full_ad(n, d):     # mhsea_tuned.py:63-69
    return 0 < n < 64 and not (n & (n - 1)) and d in (8, 16, 32, 64)


def mhsea_tuned_edge_attention(Q, K, V, edge_bias, mask, dtype=np.float64):
    """Dispatcher (pallas_attention.py:40-67): Q,K,V [N,H,D], edge_bias [N,N,H], mask [N]."""
    n, h, d = np.shape(Q)
    if not (supports_tuned(n, d) or supports_full_ad(n, d)):
        return reference_edge_attention(Q, K, V, edge_bias, mask, dtype)
    q4 = (np.asarray(Q, dtype=dtype) * (float(d) ** -0.5))[None]
    e4 = np.transpose(np.asarray(edge_bias, dtype=dtype), (0, 2, 1))[None]
    out, _ = mhsea_fwd(q4, np.asarray(K)[None], e4, np.asarray(V)[None],
                       np.asarray(mask).astype(bool)[None], dtype)
    return out[0]


def gated_edge_attention(Q, K, V, coup_bias, mask, n_heads, attn_impl="mhsea_tuned",
                         dtype=np.float64):
    """What the attention blocks do around the op (model/trunk.py:108-137, model/tree.py:
    1457-1479): the einsum twin, or the tuned op on heads zero-padded to max(16, d_head)
    with Q scaled by sqrt(d_pad / d_head) so that the op's own d_pad^-1/2 leaves the scores
    unchanged; then the first n_heads kernel heads gate the other n_heads through a sigmoid.
    Q,K,V [n, 2 n_heads, d_head], coup_bias [n, n, 2 n_heads], mask [n] -> [n, n_heads d_head]."""
    Q, K, V = (np.asarray(x, dtype=dtype) for x in (Q, K, V))
    n, hk, d = Q.shape
    if hk != 2 * n_heads:
        raise ValueError("the op runs on 2 * n_heads kernel heads")
    if attn_impl == "einsum":
        out = reference_edge_attention(Q, K, V, coup_bias, mask, dtype)
    elif attn_impl == "mhsea_tuned":
        d_pad = max(16, d)
        z = np.zeros((n, hk, d_pad - d), dtype=dtype)
        scale = np.sqrt(dtype(d_pad / d))
        out = mhsea_tuned_edge_attention(np.concatenate([Q * scale, z], -1), np.concatenate([K, z], -1),
                                         np.concatenate([V, z], -1), coup_bias, mask, dtype)[..., :d]
    else:
        raise ValueError("attn_impl must be 'einsum' or 'mhsea_tuned'")
    gate, value = out[:, :n_heads, :], out[:, n_heads:, :]
    return (value / (1.0 + np.exp(-gate))).reshape(n, n_heads * d)


def rectangular_edge_attention(q_local, k_global, v_global, edge_bias_local, key_mask, dtype=np.float64):
    """pallas_rectangular_edge_attention (src/hamiltonzero/evaluation/sequence_parallel.py:59-95
    over src/hamiltonzero/evaluation/pallas_mha.py:43-161) without the blocking: masked keys
    get a bias of -1e30, scores q k^T D^-1/2 + bias, softmax over all keys, times v.
    q [Lq,H,D], k, v [Lk,H,D], bias [Lq,Lk,H], key_mask [Lk] -> [Lq,H,D]."""
    q = np.asarray(q_local, dtype=dtype); k = np.asarray(k_global, dtype=dtype)
    v = np.asarray(v_global, dtype=dtype)
    bias = np.where(np.asarray(key_mask).astype(bool)[None, :, None],
                    np.asarray(edge_bias_local, dtype=dtype), -1.0e30)
    s = np.einsum("ihd,jhd->ijh", q, k) * (float(q.shape[-1]) ** -0.5) + bias
    s = s - s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=1, keepdims=True)
    return np.einsum("ijh,jhd->ihd", p, v)
