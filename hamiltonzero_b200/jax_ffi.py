"""JAX binding of libhz_b200: XLA FFI targets and the differentiation rules around them.

Importing this module needs JAX (the reference pins jax 0.11); nothing else in the package
imports it, and it cannot be exercised where JAX is absent. ``register()`` loads
``libhz_ffi.so`` (built from csrc/hz_ffi.cc by ``build.build_ffi`` when jaxlib's headers are
present) and registers one FFI target per handler for platform "CUDA".

The attention op keeps the contract of the reference's primitives
(src/hamiltonzero/model/_pallas_attn/mhsea_tuned.py:72-240, mhsea_full_ad.py:32-185):

* a primal call returning ``out, lse`` (``mhsea_tuned_ad_p``);
* a tangent call that is linear in ``(qt, kt, et, vt)`` given the saved ``out, lse``
  (``mhsea_tuned_ad_lin_p``), expressed with ``jax.custom_derivatives.linear_call`` so that JAX
  can transpose it: the transpose is the backward kernel (``_inner_transpose``);
* the JVP rule binds both (``_outer_jvp``), with a symbolically zero tangent for ``lse``;
* ``vmap`` adds leading axes (``vmap_method="broadcast_all"``), which the handlers fold into
  the batch, as the reference's batching rules do.

``mhsea_with_tuned_ad`` and ``mhsea_tuned_edge_attention`` have the reference's signatures, so
that ``ModelConfig.attention = "tuned"`` can route here by replacing the two imports of
src/hamiltonzero/model/pallas_attention.py. The walker operators are exposed as plain functions
of the reference's ``kernel`` / ``tree`` / ``energy_frame`` pytrees.
"""
from __future__ import annotations

import ctypes
from functools import partial
from pathlib import Path

import jax
import jax.numpy as jnp
import numpy as np

HZ_MASK_SQUARE, HZ_MASK_KEYS = 0, 1
_FFI_LIB = Path(__file__).resolve().parent / "libhz_ffi.so"
_TARGETS = ("hz_ffi_mhsea_fwd", "hz_ffi_mhsea_jvp", "hz_ffi_mhsea_bwd", "hz_ffi_logpsi",
            "hz_ffi_local_energy", "hz_ffi_logpsi_grad", "hz_ffi_logpsi_vjp")
_registered = False


def register() -> None:
    """Register the FFI targets (idempotent). Raises if libhz_ffi.so has not been built."""
    global _registered
    if _registered:
        return
    if not _FFI_LIB.exists():
        raise ImportError(f"{_FFI_LIB} is missing: build it with hamiltonzero_b200.build.build_ffi() "
                          "on a machine that has jaxlib's headers")
    ctypes.CDLL(str(_FFI_LIB.parent / "libhz_b200.so"), mode=ctypes.RTLD_GLOBAL)
    lib = ctypes.CDLL(str(_FFI_LIB))
    for name in _TARGETS:
        jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(lib, name)), platform="CUDA")
    _registered = True


def _f32(x):
    x = jnp.asarray(x)
    if x.dtype != jnp.float32:
        raise TypeError("the CUDA operators take float32 operands")     # pallas_attention.py:16-19
    return x


def _absent(shape_tail):
    return jnp.zeros((0,) + tuple(shape_tail), jnp.float32)


# ----------------------------------------------------------------------------- attention
def _fwd_call(q, k, e, v, mask, mask_mode):
    out_t = jax.ShapeDtypeStruct(q.shape, jnp.float32)
    lse_t = jax.ShapeDtypeStruct(q.shape[:-1], jnp.float32)
    return jax.ffi.ffi_call("hz_ffi_mhsea_fwd", (out_t, lse_t), vmap_method="broadcast_all")(
        q, k, e, v, mask, mask_mode=np.int32(mask_mode))


def _jvp_call(q, k, e, v, mask, out, lse, qt, kt, et, vt, mask_mode):
    return jax.ffi.ffi_call("hz_ffi_mhsea_jvp", jax.ShapeDtypeStruct(q.shape, jnp.float32),
                            vmap_method="broadcast_all")(
        q, k, e, v, mask, out, lse, qt, kt, et, vt, mask_mode=np.int32(mask_mode))


def _bwd_call(q, k, e, v, mask, lse, out, dout, mask_mode):
    t = jax.ShapeDtypeStruct(q.shape, jnp.float32)
    de_t = jax.ShapeDtypeStruct(e.shape, jnp.float32)
    return jax.ffi.ffi_call("hz_ffi_mhsea_bwd", (t, t, de_t, t), vmap_method="broadcast_all")(
        q, k, e, v, mask, lse, out, dout, mask_mode=np.int32(mask_mode))


def _linear_tangent(residuals, tangents, *, mask_mode):
    q, k, e, v, mask, out, lse = residuals
    qt, kt, et, vt = tangents
    return _jvp_call(q, k, e, v, mask, out, lse, qt, kt, et, vt, mask_mode)


def _linear_tangent_transpose(residuals, dtangent, *, mask_mode):
    q, k, e, v, mask, out, lse = residuals
    dq, dk, de, dv = _bwd_call(q, k, e, v, mask, lse, out, dtangent, mask_mode)
    return dq, dk, de, dv


@partial(jax.custom_jvp, nondiff_argnums=(5,))
def _mhsea(q, k, e, v, mask, mask_mode):
    return _fwd_call(q, k, e, v, mask, mask_mode)


@_mhsea.defjvp
def _mhsea_jvp(mask_mode, primals, tangents):
    q, k, e, v, mask = primals
    qt, kt, et, vt, _ = tangents
    out, lse = _fwd_call(q, k, e, v, mask, mask_mode)
    tangent = jax.custom_derivatives.linear_call(
        partial(_linear_tangent, mask_mode=mask_mode),
        partial(_linear_tangent_transpose, mask_mode=mask_mode),
        (q, k, e, v, mask, out, lse), (qt, kt, et, vt))
    return (out, lse), (tangent, jnp.zeros_like(lse))


def mhsea_with_tuned_ad(q, k, e, v, mask):
    """``[B,N,H,D]`` batched entry (mhsea_tuned.py:243-255); masked query rows of the result
    are zero; differentiable in forward and reverse mode."""
    register()
    q, k, e, v = _f32(q), _f32(k), _f32(e), _f32(v)
    out, _lse = _mhsea(q, k, e, v, jnp.asarray(mask).astype(jnp.uint8), HZ_MASK_SQUARE)
    return out


def mhsea_tuned_edge_attention(Q, K, V, edge_bias, mask):
    """Dispatcher with the reference's signature and gating (pallas_attention.py:40-67): shapes
    outside the kernels' reach take the einsum twin's keys-only convention."""
    register()
    Q, K, V, edge_bias = _f32(Q), _f32(K), _f32(V), _f32(edge_bias)
    n, n_heads, d_head = Q.shape
    square = K.shape == Q.shape and V.shape == Q.shape and edge_bias.shape == (n, n, n_heads) \
        and jnp.shape(mask) == (n,)
    tuned = square and n >= 64 and n % 32 == 0
    full_ad = square and 0 < n < 64 and not (n & (n - 1))
    mode = HZ_MASK_SQUARE if (d_head in (8, 16, 32, 64) and (tuned or full_ad)) else HZ_MASK_KEYS
    if d_head not in (8, 16, 32, 64):
        pad = next(c for c in (8, 16, 32, 64) if d_head <= c) - d_head
        widen = lambda x: jnp.pad(x, ((0, 0), (0, 0), (0, pad)))
        Qp, Kp, Vp = widen(Q), widen(K), widen(V)
    else:
        Qp, Kp, Vp = Q, K, V
    q4 = (Qp * (float(d_head) ** -0.5))[None]
    e4 = jnp.transpose(edge_bias, (0, 2, 1))[None]
    m4 = (jnp.asarray(mask) != 0).astype(jnp.uint8)[None]
    out, _ = _mhsea(q4, Kp[None], e4, Vp[None], m4, mode)
    return out[0, :, :, :d_head]


# ----------------------------------------------------------------------------- walker operators
def _wavefunction_operands(kernel, tree):
    """Twelve operands in the order of hz_wavefunction, from the reference's pytrees
    (compiled/types.py:38-45,131-140; one factor per stage, no combiners: execute.py:79-92)."""
    if len(tree.leaf_combiner_h) != 0 or len(tree.readout_combiner_h) != 0:
        raise ValueError("single-head compiled HT executor does not accept combiners")
    leaf, merge, readout = kernel.leaf_factors[0], kernel.merge_factors[0], kernel.readout_factors[0]
    merge_h = jnp.concatenate([h.reshape(-1) for h in tree.merge_h]) if tree.merge_h else _absent(())
    opcodes = jnp.concatenate([jnp.asarray(o, jnp.uint8) for o in tree.opcodes]) if tree.opcodes \
        else jnp.zeros((0,), jnp.uint8)
    return (kernel.q_to_odd.weight, leaf.V, leaf.U, tree.leaf_h[0], kernel.merge_T, merge.V, merge.U,
            merge_h, opcodes, readout.V, readout.U, tree.readout_h[0])


def execute_wavefunction(kernel, tree, q_routed, *, chunk_size: int = 4096):
    """``(log_abs, phase)`` of routed walkers ``q_routed [..., N, 4]`` (compiled/execute.py:79-118)."""
    register()
    lead = q_routed.shape[:-2]
    t = jax.ShapeDtypeStruct(lead, jnp.float32)
    return jax.ffi.ffi_call("hz_ffi_logpsi", (t, t))(
        _f32(q_routed), *_wavefunction_operands(kernel, tree),
        merge_eps=np.float32(kernel.merge_eps), chunk_size=np.int64(chunk_size))


def vmc_energy_custom_lap_compiled(kernel, tree, energy_frame, q_routed, *, chunk_size: int | None = 512):
    """``(total, exchange, casimir, field)`` complex64 (energy/compiled.py:17-31)."""
    register()
    lead = q_routed.shape[:-2]
    n_items = int(np.prod(lead)) if lead else 1
    n = q_routed.shape[-2]
    outs = jax.ffi.ffi_call(
        "hz_ffi_local_energy",
        (jax.ShapeDtypeStruct((4, n_items, 2), jnp.float32), jax.ShapeDtypeStruct((n_items,), jnp.float32),
         jax.ShapeDtypeStruct((n_items,), jnp.float32), jax.ShapeDtypeStruct((0, 3 * n, 2), jnp.float32)))(
        _f32(q_routed), *_wavefunction_operands(kernel, tree),
        _f32(energy_frame.custom_lap_J_eff), _f32(energy_frame.one_body_fields[0]),
        merge_eps=np.float32(kernel.merge_eps),
        radial_const=np.float32(energy_frame.custom_lap_radial_const),
        chunk_size=np.int64(chunk_size or n_items))
    e = outs[0]
    return tuple((e[i, :, 0] + 1j * e[i, :, 1]).astype(jnp.complex64).reshape(lead) for i in range(4))


def local_spin(wavefunction, context, q_routed, *, chunk_size: int | None = 512):
    """``-i/2 d(log psi)/dz`` masked (observables.py:31-59), from one value-and-Jacobian pass."""
    register()
    lead = q_routed.shape[:-2]
    n_items = int(np.prod(lead)) if lead else 1
    n = q_routed.shape[-2]
    t = jax.ShapeDtypeStruct((n_items,), jnp.float32)
    _la, _ph, grad = jax.ffi.ffi_call(
        "hz_ffi_logpsi_grad", (t, t, jax.ShapeDtypeStruct((n_items, 3 * n, 2), jnp.float32)))(
        _f32(q_routed), *_wavefunction_operands(wavefunction.kernel, wavefunction.tree),
        merge_eps=np.float32(wavefunction.kernel.merge_eps), chunk_size=np.int64(chunk_size or n_items))
    g = (grad[..., 0] + 1j * grad[..., 1]).reshape(lead + (n, 3))
    return (-0.5j * g * jnp.asarray(context.mask, jnp.float32)[..., None]).astype(jnp.complex64)


def logpsi_vjp(kernel, tree, q_routed, cot_log_abs, cot_phase, *, chunk_size: int = 512):
    """Gradients of ``sum_w cot_log_abs[w] log|psi_w| + cot_phase[w] phase_w`` with respect to the
    twelve arrays of the compiled wavefunction (in hz_wavefunction order, opcodes excepted) and to
    ``q_routed``, plus the forward values: what ``jax.vjp`` of ``call_tagged``
    (compiled/model.py:179-310) delivers to the loss tangent of optim/production.py:168-228."""
    register()
    ops = _wavefunction_operands(kernel, tree)
    lead = q_routed.shape[:-2]
    n_items = int(np.prod(lead)) if lead else 1
    like = lambda a: jax.ShapeDtypeStruct(a.shape, jnp.float32)
    grads_t = tuple(like(a) for i, a in enumerate(ops) if i != 8)
    t = jax.ShapeDtypeStruct((n_items,), jnp.float32)
    outs = jax.ffi.ffi_call("hz_ffi_logpsi_vjp", grads_t + (like(q_routed), t, t))(
        _f32(q_routed), _f32(cot_log_abs).reshape(-1), _f32(cot_phase).reshape(-1), *ops,
        merge_eps=np.float32(kernel.merge_eps), chunk_size=np.int64(chunk_size))
    return outs[:11], outs[11], outs[12].reshape(lead), outs[13].reshape(lead)


__all__ = ["execute_wavefunction", "local_spin", "logpsi_vjp", "mhsea_tuned_edge_attention",
           "mhsea_with_tuned_ad", "register", "vmc_energy_custom_lap_compiled"]
