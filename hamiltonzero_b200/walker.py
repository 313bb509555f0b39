"""Host-side mirror of the reference's walker-batch interface, backed by libhz_b200.so.

Mirrors ``CompiledWaveFunction.__call__`` (src/hamiltonzero/compiled/types.py:146-153),
``vmc_energy_custom_lap_compiled`` (src/hamiltonzero/energy/compiled.py:17-31) and
``local_spin`` (src/hamiltonzero/observables.py:31-59): same names, argument meaning
and result layout, with ``torch`` CUDA tensors (NumPy inputs are copied to the current
device and results copied back). There is no eager or CPU fallback.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .attention import _dev, _device, _ptr, _stream
from .systems import EnergyFrame, WavefunctionArrays
from .types import CompiledTree, SharedKernel, to_arrays


class CompiledWaveFunction:
    """Device-resident ``SharedKernel`` + ``CompiledTree``; callable like the reference's
    ``CompiledWaveFunction``: ``wf(q_routed) -> (log_abs, phase)``. Built either like the
    reference's module, ``CompiledWaveFunction(kernel, tree)`` (compiled/types.py:146-153), or
    from the flat arrays, ``CompiledWaveFunction(arrays)``."""

    def __init__(self, kernel, tree=None, device=None):
        dev = _device() if device is None else torch.device(device)
        self.device = dev
        if isinstance(kernel, SharedKernel):
            if not isinstance(tree, CompiledTree):
                raise TypeError("CompiledWaveFunction(kernel, tree) needs a CompiledTree")
            self.kernel, self.tree = kernel, tree
            arrays = to_arrays(kernel, tree)
        else:
            arrays = kernel
            self.kernel = self.tree = None
        self.arrays = arrays
        f = lambda a: torch.as_tensor(np.ascontiguousarray(a, dtype=np.float32), device=dev)
        self.n_sites = arrays.n_sites
        self.t = dict(
            q_weight=f(arrays.q_weight), leaf_V=f(arrays.leaf_V), leaf_U=f(arrays.leaf_U),
            leaf_h=f(arrays.leaf_h), merge_T=f(arrays.merge_T), merge_V=f(arrays.merge_V),
            merge_U=f(arrays.merge_U), readout_V=f(arrays.readout_V),
            readout_U=f(arrays.readout_U), readout_h=f(arrays.readout_h))
        levels = len(arrays.merge_h)
        if len(arrays.opcodes) != levels:
            raise ValueError("merge_h and opcodes must have one entry per tree level")
        if (1 << levels) != self.n_sites:
            raise ValueError("compiled tree did not reduce to one root")
        if levels:
            self.t["merge_h"] = f(np.concatenate([np.asarray(h, np.float32).reshape(-1)
                                                  for h in arrays.merge_h]))
            self.t["opcodes"] = torch.as_tensor(
                np.concatenate([np.asarray(o, np.uint8) for o in arrays.opcodes]), device=dev)
        d_r = arrays.merge_T.shape[1]
        t = self.t
        self.c = _lib.Wavefunction(
            n_sites=self.n_sites, d_o=arrays.q_weight.shape[1], d_m=arrays.leaf_U.shape[1],
            d_r=d_r, r_leaf=arrays.leaf_V.shape[1], r_merge=arrays.merge_V.shape[1],
            r_ro=arrays.readout_V.shape[1], merge_eps=float(arrays.merge_eps),
            q_weight=t["q_weight"].data_ptr(), leaf_V=t["leaf_V"].data_ptr(),
            leaf_U=t["leaf_U"].data_ptr(), leaf_h=t["leaf_h"].data_ptr(),
            merge_T=t["merge_T"].data_ptr(), merge_V=t["merge_V"].data_ptr(),
            merge_U=t["merge_U"].data_ptr(),
            merge_h=t["merge_h"].data_ptr() if levels else 0,
            opcodes=t["opcodes"].data_ptr() if levels else 0,
            readout_V=t["readout_V"].data_ptr(), readout_U=t["readout_U"].data_ptr(),
            readout_h=t["readout_h"].data_ptr())
        self._workspace = None

    # scratch owned by this object and reused across calls on the same stream
    def workspace(self, with_jets: bool, n_items: int, chunk_size):
        lib = _lib.load()
        chunk = n_items if chunk_size is None else max(1, min(int(chunk_size), n_items))
        need = lib.hz_walker_workspace_bytes(ctypes.byref(self.c), 1 if with_jets else 0, chunk)
        if need < 0:
            raise _lib.HzError(3, "hz_walker_workspace_bytes",
                               "wavefunction extents outside what the kernels implement")
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = None
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._workspace, need

    def __call__(self, q_routed, _ctx=None, _t=0.0, *, chunk_size=4096):
        host = isinstance(q_routed, np.ndarray)
        q = _dev(q_routed)
        if q.ndim < 2 or q.shape[-1] != 4 or q.shape[-2] != self.n_sites:
            raise ValueError(f"q_routed must have shape [..., {self.n_sites}, 4]")
        lead = tuple(q.shape[:-2])
        n_items = int(np.prod(lead)) if lead else 1
        log_abs = torch.empty(n_items, dtype=torch.float32, device=q.device)
        phase = torch.empty_like(log_abs)
        ws, nbytes = self.workspace(False, n_items, chunk_size)
        st = _lib.load().hz_logpsi(ctypes.byref(self.c), _ptr(q), n_items, _ptr(log_abs),
                                   _ptr(phase), _ptr(ws), nbytes, _stream())
        _lib.check(st, "hz_logpsi")
        log_abs, phase = log_abs.reshape(lead), phase.reshape(lead)
        return (log_abs.cpu().numpy(), phase.cpu().numpy()) if host else (log_abs, phase)


    GRAD_NAMES = ("q_weight", "leaf_V", "leaf_U", "leaf_h", "merge_T", "merge_V", "merge_U",
                  "merge_h", "readout_V", "readout_U", "readout_h")

    def _factor_shapes(self, marginals=False):
        a = self.arrays
        d_o, rl = a.leaf_V.shape
        d, r = a.merge_V.shape
        rr = a.readout_V.shape[1]
        n = self.n_sites
        d_r = a.merge_T.shape[1]
        extra = dict(merge_T_left=(d, d), merge_T_right=(d_r * d_r, d_r * d_r), merge_T_stats=(2,)) \
            if (marginals and n > 1) else {}
        return dict(**extra, q_in=(4, 4), q_out=(d_o, d_o), leaf_V_in=(d_o, d_o), leaf_V_out=(rl, rl),
                    leaf_U_in=(rl, rl), leaf_U_out=(d, d), leaf_h_diag=(n, rl),
                    merge_V_in=(d, d), merge_V_out=(r, r), merge_U_in=(r, r), merge_U_out=(d, d),
                    merge_h_diag=(max(n - 1, 0) * r,), readout_V_in=(d, d), readout_V_out=(rr, rr),
                    readout_U_in=(rr, rr), readout_U_out=(2, 2), readout_h_diag=(rr,))

    def vjp(self, q_routed, cot_log_abs, cot_phase, *, want_dq=True, chunk_size=512,
            factors=False, leaf_mask=None):
        """Reverse pass: ``(grads, dq, log_abs, phase)`` with ``grads[name]`` the sum over
        walkers of ``cot_log_abs * d log|psi| + cot_phase * d phase`` with respect to the
        parameter array ``name`` (shapes of the arrays given at construction; ``merge_h`` as a
        list, one ``[nodes, r]`` array per level) and ``dq [..., N, 4]`` the same combination
        differentiated with respect to the walker's quaternions. With ``factors=True`` a fifth
        item holds the KFAC second-moment sums of every dense and scale tag (see
        ``hz_kfac_factors``; ``leaf_mask [N]`` marks the real leaves); ``factors="marginals"`` adds
        the sums behind the two-Kronecker marginals of the quadrilinear tag (``merge_T_left``,
        ``merge_T_right``, ``merge_T_stats``; see ``two_kron_marginals``). This is what JAX's transpose
        of ``CompiledFinetuneWaveFunction.call_tagged`` delivers to the loss tangent of
        src/hamiltonzero/optim/production.py:168-228 (cotangents ``2 Re/Im(delta E) / n``)."""
        host = isinstance(q_routed, np.ndarray)
        q = _dev(q_routed)
        if q.ndim < 2 or q.shape[-1] != 4 or q.shape[-2] != self.n_sites:
            raise ValueError(f"q_routed must have shape [..., {self.n_sites}, 4]")
        lead = tuple(q.shape[:-2])
        n_items = int(np.prod(lead)) if lead else 1
        ca = _dev(np.ascontiguousarray(cot_log_abs, np.float32) if isinstance(cot_log_abs, np.ndarray)
                  else cot_log_abs).reshape(-1)
        cp = _dev(np.ascontiguousarray(cot_phase, np.float32) if isinstance(cot_phase, np.ndarray)
                  else cot_phase).reshape(-1)
        if ca.numel() != n_items or cp.numel() != n_items:
            raise ValueError("one cotangent pair per walker is required")
        lib = _lib.load()
        g = {k: torch.empty_like(self.t[k]) for k in self.GRAD_NAMES if k in self.t}
        gp = lambda k: g[k].data_ptr() if k in g else 0
        cg = _lib.WavefunctionGrads(**{k: gp(k) for k in self.GRAD_NAMES})
        dq = torch.empty_like(q) if want_dq else None
        log_abs = torch.empty(n_items, dtype=torch.float32, device=q.device)
        phase = torch.empty_like(log_abs)
        chunk = max(1, min(int(chunk_size or n_items), n_items))
        fac, cf = None, None
        if factors:
            fac = {k: torch.empty(shape, dtype=torch.float32, device=q.device)
                   for k, shape in self._factor_shapes(factors == "marginals").items()
                   if int(np.prod(shape)) > 0}
            mask_t = None
            if leaf_mask is not None:
                mask_t = torch.as_tensor(np.ascontiguousarray(leaf_mask, dtype=np.uint8), device=q.device)
            cf = _lib.KfacFactors(leaf_mask=mask_t.data_ptr() if mask_t is not None else 0,
                                  **{k: (fac[k].data_ptr() if k in fac else 0)
                                     for k in _lib.KfacFactors.NAMES})
        need = lib.hz_vjp_workspace_bytes(ctypes.byref(self.c), chunk,
                                          (2 if factors == "marginals" else 1) if factors else 0)
        if need < 0:
            raise _lib.HzError(3, "hz_vjp_workspace_bytes",
                               "wavefunction extents outside what the kernels implement")
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = None
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        st = lib.hz_logpsi_vjp(ctypes.byref(self.c), _ptr(q), n_items, _ptr(ca), _ptr(cp),
                               ctypes.byref(cg), ctypes.byref(cf) if cf is not None else None,
                               _ptr(dq) if want_dq else 0, _ptr(log_abs),
                               _ptr(phase), _ptr(self._workspace), need, _stream())
        _lib.check(st, "hz_logpsi_vjp")
        if "merge_h" in g:
            r = self.arrays.merge_V.shape[1]
            flat, out, off = g["merge_h"], [], 0
            for h in self.arrays.merge_h:
                n = int(np.asarray(h).shape[0])
                out.append(flat[off:off + n * r].reshape(n, r))
                off += n * r
            g["merge_h"] = out
        if fac is not None and "merge_h_diag" in fac:
            r = self.arrays.merge_V.shape[1]
            flat, out, off = fac["merge_h_diag"], [], 0
            for h in self.arrays.merge_h:
                n = int(np.asarray(h).shape[0])
                out.append(flat[off:off + n * r].reshape(n, r))
                off += n * r
            fac["merge_h_diag"] = out
        log_abs, phase = log_abs.reshape(lead), phase.reshape(lead)
        conv = lambda v: [x.cpu().numpy() for x in v] if isinstance(v, list) else v.cpu().numpy()
        if host:
            res = ({k: conv(v) for k, v in g.items()}, dq.cpu().numpy() if want_dq else None,
                   log_abs.cpu().numpy(), phase.cpu().numpy())
            return res + ({k: conv(v) for k, v in fac.items()},) if factors else res
        return (g, dq, log_abs, phase, fac) if factors else (g, dq, log_abs, phase)


class DeviceEnergyFrame:
    """Device copy of the routed energy frame."""

    def __init__(self, frame: EnergyFrame, device=None):
        dev = _device() if device is None else torch.device(device)
        self.frame = frame
        self.J_eff = torch.as_tensor(np.ascontiguousarray(frame.J_eff, np.float32), device=dev)
        self.field = torch.as_tensor(np.ascontiguousarray(frame.one_body_field, np.float32),
                                     device=dev)
        self.mask = torch.as_tensor(np.ascontiguousarray(frame.mask, np.float32), device=dev)
        self.c = _lib.EnergyFrame(J_eff=self.J_eff.data_ptr(),
                                  one_body_field=self.field.data_ptr(),
                                  radial_const=float(frame.radial_const))


def _energy_call(wf: CompiledWaveFunction, frame: DeviceEnergyFrame, q_routed, chunk_size,
                 want_grad: bool):
    q = _dev(q_routed)
    n = wf.n_sites
    if q.ndim < 2 or q.shape[-1] != 4:
        raise ValueError("q_routed must have shape [..., N, 4]")
    if q.shape[-2] != n or frame.J_eff.shape[0] != 3 * n:
        raise ValueError("walkers, wavefunction and energy frame must have the same site width")
    lead = tuple(q.shape[:-2])
    n_items = int(np.prod(lead)) if lead else 1
    energies = torch.empty((4, n_items, 2), dtype=torch.float32, device=q.device)
    log_abs = torch.empty(n_items, dtype=torch.float32, device=q.device)
    phase = torch.empty_like(log_abs)
    grad = torch.empty((n_items, 3 * n, 2), dtype=torch.float32, device=q.device) \
        if want_grad else None
    ws, nbytes = wf.workspace(True, n_items, chunk_size)
    st = _lib.load().hz_local_energy(ctypes.byref(wf.c), ctypes.byref(frame.c), _ptr(q), n_items,
                                     _ptr(energies), _ptr(log_abs), _ptr(phase), _ptr(grad),
                                     _ptr(ws), nbytes, _stream())
    _lib.check(st, "hz_local_energy")
    return lead, energies, log_abs, phase, grad


def two_kron_marginals(factors: dict, batch_size: int, logical_batch: int):
    """``(sigma_left, sigma_right, repeats)`` of the quadrilinear tag's curvature block from the
    sums of ``vjp(..., factors="marginals")``, normalised as the reference's
    ``StructuralQuadrilinearMergeBlock.update_curvature_matrix_estimate`` does before its moving
    averages (src/hamiltonzero/optim/spin_blocks.py:505-556): division by the sample count, trace
    normalisation with the repeat mass (``_trace_normalize_two_kron_marginals``, :174-197),
    symmetrisation. ``batch_size`` is the number of walkers behind the sums, ``logical_batch`` the
    number of (walker) rows the structural grouping counts (walkers, for the scan-shared tag)."""
    left, right, stats = factors["merge_T_left"], factors["merge_T_right"], factors["merge_T_stats"]
    to_np = lambda x: x.detach().cpu().numpy().astype(np.float64) if isinstance(x, torch.Tensor) \
        else np.asarray(x, np.float64)
    left, right, stats = to_np(left), to_np(right), to_np(stats)
    divisor = max(float(batch_size), 1.0)
    left, right = left / divisor, right / divisor
    repeats = stats[1] / float(logical_batch)
    trace_mass = stats[0] / divisor
    if not (np.isfinite(trace_mass) and np.isfinite(repeats)):
        left, right = np.full_like(left, np.nan), np.full_like(right, np.nan)
    elif trace_mass <= 0 or repeats <= 0:
        left, right = np.zeros_like(left), np.zeros_like(right)
    else:
        scale = np.sqrt(repeats / trace_mass)
        left, right = scale * left, scale * right
    return 0.5 * (left + left.T), 0.5 * (right + right.T), repeats


# Device copies of what callers pass by value every time (the reference passes pytrees that XLA
# keeps on the device): keyed by object identity, a handful of entries.
_WF_CACHE: dict = {}
_FRAME_CACHE: dict = {}


def _cached(cache: dict, key, owners, build):
    hit = cache.get(key)
    if hit is not None and all(a is b for a, b in zip(hit[0], owners)):
        return hit[1]
    if len(cache) >= 8:
        cache.pop(next(iter(cache)))
    value = build()
    cache[key] = (tuple(owners), value)
    return value


def as_wavefunction(kernel, tree=None) -> CompiledWaveFunction:
    """``CompiledWaveFunction`` for a reference-style ``(kernel, tree)`` pair, cached."""
    if isinstance(kernel, CompiledWaveFunction):
        return kernel
    return _cached(_WF_CACHE, (id(kernel), id(tree)), (kernel, tree),
                   lambda: CompiledWaveFunction(kernel, tree))


def as_device_frame(energy_frame, device) -> DeviceEnergyFrame:
    if isinstance(energy_frame, DeviceEnergyFrame):
        return energy_frame
    return _cached(_FRAME_CACHE, id(energy_frame), (energy_frame,),
                   lambda: DeviceEnergyFrame(energy_frame, device))


def vmc_energy_custom_lap_compiled(kernel, tree, energy_frame, q_routed=None, *,
                                   chunk_size: int | None = 512):
    """``vmc_energy_custom_lap_compiled(kernel, tree, energy_frame, q_routed, *, chunk_size)``
    -> ``(total, exchange, casimir, field)``, complex64 of shape ``q_routed.shape[:-2]``, the
    reference's signature (src/hamiltonzero/energy/compiled.py:17-31). ``chunk_size`` caps the
    scratch memory only; results do not depend on it. The three-argument form
    ``(wavefunction, energy_frame, q_routed)`` with a ``CompiledWaveFunction`` is accepted too."""
    if isinstance(kernel, CompiledWaveFunction) and q_routed is None:
        wavefunction, energy_frame, q_routed = kernel, tree, energy_frame
    else:
        wavefunction = as_wavefunction(kernel, tree)
    if chunk_size is not None and chunk_size < 1:
        raise ValueError("chunk_size must be positive or None")
    host = isinstance(q_routed, np.ndarray)
    energy_frame = as_device_frame(energy_frame, wavefunction.device)
    lead, energies, *_ = _energy_call(wavefunction, energy_frame, q_routed, chunk_size, False)
    out = tuple(torch.view_as_complex(energies[i]).reshape(lead) for i in range(4))
    return tuple(o.cpu().numpy() for o in out) if host else out


def logpsi_and_chart_gradient(wavefunction: CompiledWaveFunction, q_routed, *,
                              chunk_size: int | None = 512):
    """``(log_abs, phase, grad)`` with ``grad [..., 3N, 2]`` the derivatives of (log|psi|, phase)
    along the right-SU(2) chart at z = 0 (hz_logpsi_grad: value and Jacobian rows only)."""
    q = _dev(q_routed)
    n = wavefunction.n_sites
    if q.ndim < 2 or q.shape[-1] != 4:
        raise ValueError("q_routed must have shape [..., N, 4]")
    if q.shape[-2] != n:
        raise ValueError("walkers and wavefunction must have the same site width")
    lead = tuple(q.shape[:-2])
    n_items = int(np.prod(lead)) if lead else 1
    log_abs = torch.empty(n_items, dtype=torch.float32, device=q.device)
    phase = torch.empty_like(log_abs)
    grad = torch.empty((n_items, 3 * n, 2), dtype=torch.float32, device=q.device)
    lib = _lib.load()
    chunk = n_items if chunk_size is None else max(1, min(int(chunk_size), n_items))
    need = lib.hz_walker_workspace_bytes(ctypes.byref(wavefunction.c), 2, chunk)
    if need < 0:
        raise _lib.HzError(3, "hz_walker_workspace_bytes",
                           "wavefunction extents outside what the kernels implement")
    if wavefunction._workspace is None or wavefunction._workspace.numel() < need:
        wavefunction._workspace = None
        wavefunction._workspace = torch.empty(need, dtype=torch.uint8, device=wavefunction.device)
    st = lib.hz_logpsi_grad(ctypes.byref(wavefunction.c), _ptr(q), n_items, _ptr(log_abs),
                            _ptr(phase), _ptr(grad), _ptr(wavefunction._workspace), need, _stream())
    _lib.check(st, "hz_logpsi_grad")
    return log_abs.reshape(lead), phase.reshape(lead), grad.reshape(*lead, 3 * n, 2)


def local_spin(wavefunction, context, q_routed, *, chunk_size: int | None = 512):
    """``local_spin(wavefunction, context, q_routed, *, chunk_size)``: ``-i/2 d(log psi)/dz`` per
    site, complex64 ``[..., N, 3]``, times ``context.mask`` (src/hamiltonzero/observables.py:15-59;
    ``context`` is anything with the routed real-site ``mask [N]``: the reference's context, an
    energy frame, or the mask itself). The derivative comes from one value-and-Jacobian forward
    pass (the reference takes the same Jacobian by ``jacrev``)."""
    host = isinstance(q_routed, np.ndarray)
    wavefunction = as_wavefunction(wavefunction)
    mask = getattr(context, "mask", context)
    if isinstance(context, DeviceEnergyFrame):
        mask = context.mask
    mask = torch.as_tensor(np.asarray(mask.cpu() if isinstance(mask, torch.Tensor) else mask,
                                      dtype=np.float32), device=wavefunction.device)
    if np.ndim(q_routed) < 2 or np.shape(q_routed)[-1] != 4:
        raise ValueError("q_routed must have shape [..., N, 4]")
    if mask.shape[-1] != np.shape(q_routed)[-2]:
        raise ValueError("context mask and q_routed must have the same site width")
    if chunk_size is not None and chunk_size < 1:
        raise ValueError("chunk_size must be positive or None")
    _la, _ph, grad = logpsi_and_chart_gradient(wavefunction, q_routed, chunk_size=chunk_size)
    lead = tuple(grad.shape[:-2])
    g = torch.view_as_complex(grad.contiguous()).reshape(*lead, wavefunction.n_sites, 3)
    out = (-0.5j) * g * mask[:, None]
    return out.cpu().numpy() if host else out


__all__ = ["CompiledWaveFunction", "DeviceEnergyFrame", "as_device_frame", "as_wavefunction",
           "local_spin", "logpsi_and_chart_gradient", "two_kron_marginals",
           "vmc_energy_custom_lap_compiled"]
