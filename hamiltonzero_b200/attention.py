"""Host-side mirror of the reference's attention interface, backed by libhz_b200.so.

Mirrors ``src/hamiltonzero/model/pallas_attention.py`` (``reference_edge_attention``
:22-37, ``mhsea_tuned_edge_attention`` :40-67) and the batched entry
``mhsea_with_tuned_ad`` (``src/hamiltonzero/model/_pallas_attn/mhsea_tuned.py:243-255``)
together with the three primitive-level operators the reference lowers to Pallas
kernels: the primal (``mhsea_tuned_ad``), the linear tangent (``mhsea_tuned_ad_lin``)
and its transpose. Names, argument order, layouts and error behaviour follow the
reference; tensors are ``torch`` CUDA tensors (or NumPy arrays, which are copied
to the current device and back). Every operator runs in CUDA through the C ABI;
there is no eager or CPU fallback.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from ._lib import AttnShape

HZ_MASK_SQUARE = 0
HZ_MASK_KEYS = 1
HZ_ATTN_TF32 = 0x100     # flag OR-ed into mask_mode: single-pass TF32 contractions allowed
HZ_ATTN_TCGEN05 = 0x200  # flag OR-ed into mask_mode (forward): use the tcgen05 kernel where it applies
HZ_ATTN_TF32X3 = 0x1000  # flag OR-ed into mask_mode: three-term TF32 split (fp32-faithful) instead of the default BF16 split
HZ_ATTN_BF16X3 = 0x400   # flag OR-ed into mask_mode: two-term BF16 split (three products) allowed
HZ_ATTN_FP16X3 = 0x800   # flag OR-ed into mask_mode: two-term FP16 split allowed (operands inside the FP16 range)

_SUPPORTED_MHSEA_HEAD_DIMS = frozenset((8, 16, 32, 64))   # pallas_attention.py:13
MAX_TOKENS = 256


def _require_fp32(*values) -> None:
    # pallas_attention.py:16-19
    for value in values:
        if value is None:
            continue
        dt = value.dtype
        if dt not in (torch.float32, np.dtype(np.float32)):
            raise TypeError(f"attention tensors must be float32, got {dt}")


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("hamiltonzero_b200 needs a CUDA device; there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def _dev(x, dtype=torch.float32):
    """Contiguous tensor on the current CUDA device (NumPy / CPU inputs are copied)."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(np.ascontiguousarray(x))
    if not x.is_cuda:
        x = x.to(_device(), non_blocking=True)
    if x.dtype != dtype:
        x = x.to(dtype)
    return x.contiguous()


def _ptr(x):
    return ctypes.c_void_p(0 if x is None else x.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _shape(q, mask_mode) -> AttnShape:
    if q.ndim != 4:
        raise ValueError(f"q must have rank 4 [B, N, H, D], got shape {tuple(q.shape)}")
    B, N, H, D = q.shape
    return AttnShape(B, N, H, D, mask_mode)


def _check_primals(q, k, e, v, mask):
    # _validate_primals, mhsea_tuned.py:29-50
    B, N, H, D = q.shape
    if tuple(k.shape) != (B, N, H, D):
        raise ValueError(f"k shape {tuple(k.shape)} != q shape {tuple(q.shape)}")
    if tuple(v.shape) != (B, N, H, D):
        raise ValueError(f"v shape {tuple(v.shape)} != q shape {tuple(q.shape)}")
    if e is not None and tuple(e.shape) != (B, N, H, N):
        raise ValueError(f"e shape {tuple(e.shape)} != ({B}, {N}, {H}, {N})")
    if mask is not None and tuple(mask.shape) != (B, N):
        raise ValueError(f"mask shape {tuple(mask.shape)} != ({B}, {N})")


# --------------------------------------------------------------- primitive level
def mhsea_fwd(q, k, e, v, mask, mask_mode: int = HZ_MASK_SQUARE):
    """Primal primitive: ``(out [B,N,H,D], lse [B,N,H])``; ``q`` pre-scaled by D**-0.5.
    ``e`` and ``mask`` may be None (no bias / every token real)."""
    _require_fp32(q, k, e, v)
    q, k, e, v = _dev(q), _dev(k), _dev(e), _dev(v)
    mask = _dev(mask, torch.uint8) if mask is not None else None
    _check_primals(q, k, e, v, mask)
    shape = _shape(q, mask_mode)
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    st = _lib.load().hz_mhsea_fwd(ctypes.byref(shape), _ptr(q), _ptr(k), _ptr(e), _ptr(v),
                                  _ptr(mask), _ptr(out), _ptr(lse), _stream())
    _lib.check(st, "hz_mhsea_fwd")
    return out, lse


def mhsea_jvp(q, k, e, v, mask, out, lse, qt, kt, et, vt, mask_mode: int = HZ_MASK_SQUARE):
    """Linear tangent primitive given the saved ``out, lse``."""
    _require_fp32(q, k, e, v, out, lse, qt, kt, et, vt)
    q, k, e, v = _dev(q), _dev(k), _dev(e), _dev(v)
    out, lse = _dev(out), _dev(lse)
    qt, kt, et, vt = _dev(qt), _dev(kt), _dev(et), _dev(vt)
    mask = _dev(mask, torch.uint8) if mask is not None else None
    _check_primals(q, k, e, v, mask)
    _check_primals(qt, kt, et, vt, mask)
    shape = _shape(q, mask_mode)
    tangent = torch.empty_like(q)
    st = _lib.load().hz_mhsea_jvp(ctypes.byref(shape), _ptr(q), _ptr(k), _ptr(e), _ptr(v),
                                  _ptr(mask), _ptr(out), _ptr(lse), _ptr(qt), _ptr(kt),
                                  _ptr(et), _ptr(vt), _ptr(tangent), _stream())
    _lib.check(st, "hz_mhsea_jvp")
    return tangent


def mhsea_bwd(q, k, e, v, mask, lse, out, dout, need_de: bool = True,
              mask_mode: int = HZ_MASK_SQUARE):
    """Transpose of the tangent primitive: ``(dq, dk, de, dv)``; ``de`` is None when
    ``need_de`` is false."""
    _require_fp32(q, k, e, v, out, lse, dout)
    q, k, e, v = _dev(q), _dev(k), _dev(e), _dev(v)
    out, lse, dout = _dev(out), _dev(lse), _dev(dout)
    mask = _dev(mask, torch.uint8) if mask is not None else None
    _check_primals(q, k, e, v, mask)
    shape = _shape(q, mask_mode)
    B, N, H, D = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    de = torch.empty((B, N, H, N), dtype=torch.float32, device=q.device) if need_de else None
    st = _lib.load().hz_mhsea_bwd(ctypes.byref(shape), _ptr(q), _ptr(k), _ptr(e), _ptr(v),
                                  _ptr(mask), _ptr(lse), _ptr(out), _ptr(dout), _ptr(dq),
                                  _ptr(dk), _ptr(de), _ptr(dv), _stream())
    _lib.check(st, "hz_mhsea_bwd")
    return dq, dk, de, dv


# --------------------------------------------------------------- differentiable op
def _zeros_like_opt(t, ref):
    return torch.zeros_like(ref) if t is None else t.contiguous()


class _MhseaLinFunction(torch.autograd.Function):
    """The linear tangent primitive (``mhsea_tuned_ad_lin_p``, mhsea_tuned.py:175-198) as a
    differentiable op of its four tangent arguments: forward = tangent kernel, backward = the
    transpose rule (``_inner_transpose``, mhsea_tuned.py:206-221 = the backward kernel). The
    primals and the saved ``out, lse`` are constants of the linear map."""

    @staticmethod
    def forward(ctx, q, k, e, v, mask, out, lse, qt, kt, et, vt, mask_mode):
        ctx.save_for_backward(q, k, e, v, mask, out, lse)
        ctx.mask_mode = mask_mode
        ctx.has_et = et is not None
        return mhsea_jvp(q, k, e, v, mask, out, lse, qt, kt, et, vt, mask_mode)

    @staticmethod
    def backward(ctx, dtan):
        q, k, e, v, mask, out, lse = ctx.saved_tensors
        need_de = ctx.has_et and ctx.needs_input_grad[9]
        dq, dk, de, dv = mhsea_bwd(q, k, e, v, mask, lse, out, dtan.contiguous(), need_de=need_de,
                                   mask_mode=ctx.mask_mode)
        return (None,) * 7 + (dq, dk, de if need_de else None, dv, None)


def mhsea_linear_tangent(q, k, e, v, mask, out, lse, qt, kt, et, vt,
                         mask_mode: int = HZ_MASK_SQUARE):
    """``tangent = d out[q,k,e,v] . (qt, kt, et, vt)``, differentiable (linear) in the tangents:
    reverse mode through it is the JVP-then-transpose route by which the reference's KFAC loss
    reaches the backward kernel (src/hamiltonzero/optim/production.py:181-228)."""
    return _MhseaLinFunction.apply(q, k, e, v, mask, out, lse, qt, kt, et, vt, mask_mode)


class _MhseaFunction(torch.autograd.Function):
    """The primal primitive with both differentiation rules of the reference
    (mhsea_tuned.py:104-118,206-221): forward mode (``jvp``) binds the primal kernel and the
    linear tangent kernel, with a symbolically zero tangent for ``lse``; reverse mode
    (``backward``) is the transpose of that tangent, i.e. the backward kernel."""

    @staticmethod
    def forward(ctx, q, k, e, v, mask, mask_mode):
        out, lse = mhsea_fwd(q, k, e, v, mask, mask_mode)
        ctx.save_for_backward(q, k, e, v, mask, out, lse)
        ctx.save_for_forward(q, k, e, v, mask, out, lse)
        ctx.mask_mode = mask_mode
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def jvp(ctx, qt, kt, et, vt, _mask_t, _mode_t):
        q, k, e, v, mask, out, lse = ctx.saved_tensors
        if e is None:
            et = None
        elif et is None:
            et = torch.zeros_like(e)
        tan = mhsea_jvp(q, k, e, v, mask, out, lse, _zeros_like_opt(qt, q), _zeros_like_opt(kt, k),
                        et.contiguous() if et is not None else None, _zeros_like_opt(vt, v),
                        ctx.mask_mode)
        return tan, None

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, e, v, mask, out, lse = ctx.saved_tensors
        need_de = e is not None and ctx.needs_input_grad[2]
        dq, dk, de, dv = mhsea_bwd(q, k, e, v, mask, lse, out, dout.contiguous(),
                                   need_de=need_de, mask_mode=ctx.mask_mode)
        return dq, dk, de, dv, None, None


def _supports_tuned_shape(n: int, d: int) -> bool:        # mhsea_tuned.py:53-60
    return n >= 64 and n % 32 == 0 and d in _SUPPORTED_MHSEA_HEAD_DIMS


def _supports_full_ad_shape(n: int, d: int) -> bool:      # mhsea_tuned.py:63-69
    return 0 < n < 64 and not (n & (n - 1)) and d in _SUPPORTED_MHSEA_HEAD_DIMS


def mhsea_with_tuned_ad(q, k, e, v, mask):
    """Batched entry (mhsea_tuned.py:243-255): ``out [B,N,H,D]`` with masked query rows
    zero; differentiable w.r.t. q, k, e, v under ``torch.autograd``."""
    host = isinstance(q, np.ndarray)
    _require_fp32(q, k, e, v)
    q, k, e, v = _dev(q), _dev(k), _dev(e), _dev(v)
    mask = _dev(mask, torch.uint8) if mask is not None else None
    n, d = q.shape[1], q.shape[-1]
    if not (_supports_tuned_shape(n, d) or _supports_full_ad_shape(n, d)):
        raise ValueError(
            "mhsea requires a power-of-two N and head dimension in "
            f"{sorted(_SUPPORTED_MHSEA_HEAD_DIMS)}")
    out, _lse = _MhseaFunction.apply(q, k, e, v, mask, HZ_MASK_SQUARE)
    return out.cpu().numpy() if host else out


def _pad_head_dim(x, d_pad):
    d = x.shape[-1]
    if d == d_pad:
        return x
    return torch.nn.functional.pad(x, (0, d_pad - d))


def _kernel_head_dim(d: int) -> int:
    for cand in (8, 16, 32, 64):
        if d <= cand:
            return cand
    raise _lib.HzError(3, "attention", f"head dimension {d} > 64 is not implemented")


def reference_edge_attention(Q, K, V, edge_bias, mask):
    """Einsum twin (pallas_attention.py:22-37): ``softmax_j(QK^T D^-1/2 + bias^T +
    (1-mask_j)(-1e9)) V`` with a keys-only mask, evaluated by the CUDA kernels in
    HZ_MASK_KEYS mode. Q,K,V ``[n,h,d]``, edge_bias ``[n,n,h]``, mask ``[n]``."""
    host = isinstance(Q, np.ndarray)
    _require_fp32(Q, K, V, edge_bias)
    Q, K, V, edge_bias = _dev(Q), _dev(K), _dev(V), _dev(edge_bias)
    n, _h, d = Q.shape
    if n > MAX_TOKENS:
        raise _lib.HzError(3, "attention", f"N={n} > {MAX_TOKENS} is not implemented")
    dk = _kernel_head_dim(d)
    q4 = _pad_head_dim(Q * (float(d) ** -0.5), dk)[None]
    k4 = _pad_head_dim(K, dk)[None]
    v4 = _pad_head_dim(V, dk)[None]
    e4 = edge_bias.permute(0, 2, 1)[None].contiguous()
    m4 = _dev(mask, torch.uint8).ne(0).to(torch.uint8)[None]
    out, _ = _MhseaFunction.apply(q4.contiguous(), k4.contiguous(), e4, v4.contiguous(), m4,
                                  HZ_MASK_KEYS)
    out = out[0, :, :, :d]
    return out.cpu().numpy() if host else out


def mhsea_tuned_edge_attention(Q, K, V, edge_bias, mask):
    """Dispatcher (pallas_attention.py:40-67). Shapes the reference sends to its tuned
    or small-N Pallas kernels take the square-mask kernels; every other shape takes
    the keys-only convention of ``reference_edge_attention``, as in the reference."""
    host = isinstance(Q, np.ndarray)
    _require_fp32(Q, K, V, edge_bias)
    Qd, Kd, Vd, Ed = _dev(Q), _dev(K), _dev(V), _dev(edge_bias)
    n, n_heads, d_head = Qd.shape
    sm_scale = float(d_head) ** -0.5
    square = (tuple(Kd.shape) == tuple(Qd.shape) and tuple(Vd.shape) == tuple(Qd.shape)
              and tuple(Ed.shape) == (n, n, n_heads) and tuple(np.shape(mask)) == (n,))
    supports_tuned = square and n >= 64 and n % 32 == 0
    supports_full_ad = square and 0 < n < 64 and not (n & (n - 1))
    if d_head not in _SUPPORTED_MHSEA_HEAD_DIMS or not (supports_tuned or supports_full_ad):
        out = reference_edge_attention(Qd, Kd, Vd, Ed, mask)
        return out.cpu().numpy() if host else out
    if n > MAX_TOKENS:
        raise _lib.HzError(3, "attention", f"N={n} > {MAX_TOKENS} is not implemented")
    q4 = (Qd * sm_scale)[None]
    e4 = Ed.permute(0, 2, 1)[None].contiguous()
    m4 = _dev(mask, torch.uint8).ne(0).to(torch.uint8)[None]
    out, _ = _MhseaFunction.apply(q4, Kd[None], e4, Vd[None], m4, HZ_MASK_SQUARE)
    out = out[0]
    return out.cpu().numpy() if host else out


def gated_edge_attention(Q, K, V, coup_bias, mask, n_heads, attn_impl="mhsea_tuned"):
    """The callers' shell around the op (model/trunk.py:108-137, model/tree.py:1457-1479):
    ``attn_impl`` "einsum" takes the einsum twin, "mhsea_tuned" zero-pads the heads to
    max(16, d_head), scales Q by sqrt(d_pad / d_head) (so the op's d_pad^-1/2 leaves the
    scores as they were), runs the dispatcher and drops the padding; then the first
    ``n_heads`` kernel heads gate the remaining ``n_heads`` through a sigmoid and the heads
    are flattened. Q,K,V ``[n, 2 n_heads, d_head]``, coup_bias ``[n, n, 2 n_heads]``, mask
    ``[n]`` -> ``[n, n_heads * d_head]``; differentiable under ``torch.autograd``."""
    host = isinstance(Q, np.ndarray)
    _require_fp32(Q, K, V, coup_bias)
    Qd, Kd, Vd, Ed = _dev(Q), _dev(K), _dev(V), _dev(coup_bias)
    n, hk, d = Qd.shape
    if hk != 2 * n_heads:
        raise ValueError("the op runs on 2 * n_heads kernel heads")
    if attn_impl == "einsum":
        out = reference_edge_attention(Qd, Kd, Vd, Ed, mask)
    elif attn_impl == "mhsea_tuned":
        d_pad = max(16, d)
        scale = float(d_pad / d) ** 0.5
        out = mhsea_tuned_edge_attention(_pad_head_dim(Qd * scale, d_pad).contiguous(),
                                         _pad_head_dim(Kd, d_pad).contiguous(),
                                         _pad_head_dim(Vd, d_pad).contiguous(), Ed, mask)[..., :d]
    else:
        raise ValueError("attn_impl must be 'einsum' or 'mhsea_tuned'")
    out = torch.sigmoid(out[:, :n_heads, :]) * out[:, n_heads:, :]
    out = out.reshape(n, n_heads * d)
    return out.cpu().numpy() if host else out


__all__ = [
    "gated_edge_attention",
    "HZ_ATTN_BF16X3", "HZ_ATTN_FP16X3", "HZ_ATTN_TCGEN05", "HZ_ATTN_TF32", "HZ_ATTN_TF32X3", "HZ_MASK_KEYS", "HZ_MASK_SQUARE", "mhsea_bwd", "mhsea_fwd", "mhsea_jvp",
    "mhsea_linear_tangent", "mhsea_tuned_edge_attention", "mhsea_with_tuned_ad",
    "reference_edge_attention",
]
