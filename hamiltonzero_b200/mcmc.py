"""Host-side mirror of the reference's sampler interface, backed by libhz_b200.so.

Mirrors ``REState`` (src/hamiltonzero/mcmc/replica_exchange.py:21-36), ``init_batched_state``,
``run_batched``, ``cold_samples`` (src/hamiltonzero/mcmc/runtime.py:43-64,88-129,198-199) and
the two counter-driven adaptations ``adapt_sigma`` / ``adapt_m``
(replica_exchange.py:316-376). The sweep itself (refresh, Haar move, MALA moves, swaps) runs in
CUDA through ``hz_mcmc_sweep``; there is no eager or CPU fallback.

Differences from the reference, by construction: ``drift`` [B,R,N,3] replaces the cached
``grad_log_p`` [B,R,N,4] (the reference only ever uses that gradient projected on the frame
e_1..e_3), and random numbers come from Philox(seed, sweep counter) instead of JAX's threefry,
so agreement with the reference's chains is distributional, not bitwise.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, replace

import numpy as np
import torch

from . import _lib
from .attention import _device, _ptr, _stream
from .walker import CompiledWaveFunction


@dataclass
class REState:
    q: torch.Tensor                # [B, R, N, 4]
    log_p: torch.Tensor            # [B, R]
    drift: torch.Tensor            # [B, R, N, 3]
    beta: torch.Tensor             # [R]
    sigma: torch.Tensor            # [R]
    step: int
    seed: int
    sweeps: int                    # Philox offset: number of sweeps run so far
    n_local_accept: torch.Tensor   # [B, R]
    n_local: int
    n_swap_accept: torch.Tensor    # [B, R-1]
    n_swap: torch.Tensor           # [B, R-1] int32
    mask: torch.Tensor             # [N] int32
    m: torch.Tensor                # [R] int32
    n_haar_accept: torch.Tensor    # [B, R]
    n_haar: int


def annealing_geometric(n_replicas: int, base: float = 2.0 ** 0.5) -> np.ndarray:
    """Inverse-temperature ladder, hot chain (beta 0) first, cold chain (beta 1) last
    (replica_exchange.py:39-49)."""
    if n_replicas < 2:
        raise ValueError("n_replicas must be at least two")
    if n_replicas == 2:
        return np.array([0.0, 1.0], dtype=np.float32)
    powers = np.power(base, -np.arange(n_replicas - 1, dtype=np.float64))
    return np.append(powers, 0.0)[::-1].astype(np.float32)


def init_batched_state(seed: int, mask, batch_size: int, n_replicas: int, initial_m: int = 1,
                       initial_sigma: float = 0.3, device=None) -> REState:
    """Normalised Gaussian walkers and zeroed counters (replica_exchange.py:52-93,
    runtime.py:43-64)."""
    dev = _device() if device is None else torch.device(device)
    mask_np = np.asarray(mask).astype(np.int32)
    n = mask_np.shape[-1]
    gen = torch.Generator(device=dev).manual_seed(int(seed))
    q = torch.randn(batch_size, n_replicas, n, 4, device=dev, generator=gen)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-12)
    beta = annealing_geometric(n_replicas)
    n_active = int(mask_np.sum())
    m = np.full(n_replicas, min(max(int(initial_m), 1), max(n_active, 1)), np.int32)
    m[beta == 0.0] = n_active
    f = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
    return REState(
        q=q.contiguous(), log_p=torch.full((batch_size, n_replicas), -1e30, device=dev),
        drift=f(batch_size, n_replicas, n, 3), beta=torch.as_tensor(beta, device=dev),
        sigma=torch.full((n_replicas,), float(initial_sigma), device=dev), step=0, seed=int(seed),
        sweeps=0, n_local_accept=f(batch_size, n_replicas), n_local=0,
        n_swap_accept=f(batch_size, n_replicas - 1),
        n_swap=torch.zeros(batch_size, n_replicas - 1, dtype=torch.int32, device=dev),
        mask=torch.as_tensor(mask_np, device=dev), m=torch.as_tensor(m, device=dev),
        n_haar_accept=f(batch_size, n_replicas), n_haar=0)


def run_batched(model: CompiledWaveFunction, context, state=None, n_steps=None,
                walker_chunk_size: int | None = None, *, noise: dict | None = None,
                return_log_alpha: bool = False):
    """``run_batched(model, context, state, n_steps, walker_chunk_size)``, the reference's
    signature (src/hamiltonzero/mcmc/runtime.py:88-129): one sampler call on every walker -
    refresh, global Haar move, then ``n_steps`` x (MALA move per replica + even-odd swaps).
    ``context`` is not read (log p = 2 log|psi| depends on the walkers only,
    runtime.py:66-72; the real-site mask travels in ``state.mask``); the shorter form
    ``run_batched(model, state, n_steps, walker_chunk_size)`` is accepted too.
    ``walker_chunk_size`` caps the scratch of the value-and-gradient passes only; results do not
    depend on it. ``noise`` (testing) replaces the internal draws: keys of ``hz_mcmc_noise``."""
    if isinstance(context, REState):                       # (model, state, n_steps[, chunk])
        if walker_chunk_size is None and n_steps is not None and state is not None:
            walker_chunk_size = n_steps
        state, n_steps = context, state
    if not isinstance(state, REState) or n_steps is None:
        raise TypeError("run_batched(model, context, state, n_steps, walker_chunk_size)")
    n_steps = int(n_steps)
    from .walker import as_wavefunction
    model = as_wavefunction(model)
    lib = _lib.load()
    B, R, N, _ = state.q.shape
    if N != model.n_sites:
        raise ValueError("state and wavefunction must have the same site width")
    chunk = B * R if walker_chunk_size is None else max(1, min(B, int(walker_chunk_size))) * R
    chunk = min(chunk, 2048)
    nbytes = lib.hz_mcmc_workspace_bytes(ctypes.byref(model.c), B, R, chunk)
    if nbytes < 0:
        raise _lib.HzError(3, "hz_mcmc_workspace_bytes", "extents outside what the kernels implement")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=state.q.device)
    new = replace(state, q=state.q.clone(), log_p=state.log_p.clone(), drift=state.drift.clone(),
                  n_local_accept=state.n_local_accept.clone(),
                  n_swap_accept=state.n_swap_accept.clone(), n_swap=state.n_swap.clone(),
                  n_haar_accept=state.n_haar_accept.clone())
    c = _lib.McmcState(
        n_walkers=B, n_replicas=R, n_sites=N, step=state.step, seed=state.seed, offset=state.sweeps,
        q=new.q.data_ptr(), log_p=new.log_p.data_ptr(), drift=new.drift.data_ptr(),
        beta=new.beta.data_ptr(), sigma=new.sigma.data_ptr(), mask=new.mask.data_ptr(),
        m=new.m.data_ptr(), n_local_accept=new.n_local_accept.data_ptr(),
        n_swap_accept=new.n_swap_accept.data_ptr(), n_swap=new.n_swap.data_ptr(),
        n_haar_accept=new.n_haar_accept.data_ptr())
    keep, cn = [], None
    if noise is not None:
        vals = {}
        for key in ("haar_scores", "haar_raw", "haar_logu", "local_noise", "local_logu", "swap_logu"):
            t = noise.get(key)
            if t is not None:
                t = torch.as_tensor(np.ascontiguousarray(t, dtype=np.float32), device=state.q.device)
                keep.append(t)
                vals[key] = t.data_ptr()
        cn = _lib.McmcNoise(**vals)
    la = torch.empty(max(n_steps, 1), B, R, device=state.q.device) if return_log_alpha else None
    st = lib.hz_mcmc_sweep(ctypes.byref(model.c), ctypes.byref(c), int(n_steps),
                           ctypes.byref(cn) if cn is not None else None, _ptr(la), _ptr(ws), nbytes,
                           _stream())
    _lib.check(st, "hz_mcmc_sweep")
    new = replace(new, step=state.step + n_steps, sweeps=state.sweeps + 1,
                  n_local=state.n_local + n_steps, n_haar=state.n_haar + 1)
    return (new, la) if return_log_alpha else new


def cold_samples(state: REState) -> torch.Tensor:
    """Walkers of the cold chain (beta = 1), ``q[:, -1]`` (runtime.py:198-199)."""
    return state.q[:, -1]


def adapt_sigma(state: REState, *, target: float = 0.574, factor: float = 1.1, lo: float = 1e-4,
                hi: float = 3.14, pooled=None) -> REState:
    """Widen or narrow each replica's proposal from its pooled acceptance rate and reset the
    local counters (replica_exchange.py:316-345, pooled over walkers as in
    ``adapt_batched``, runtime.py:132-156). ``pooled``: the result of ``all_reduce_counters``
    when the walkers are sharded over ranks."""
    pooled = pooled_counters(state) if pooled is None else pooled
    B = float(pooled[4, 0])
    rate = pooled[0].to(state.sigma.dtype) / max(B * state.n_local, 1)
    sigma = torch.where(rate > target, state.sigma * factor, state.sigma / factor).clamp(lo, hi)
    return replace(state, sigma=sigma, n_local_accept=torch.zeros_like(state.n_local_accept),
                   n_local=0)


def adapt_m(state: REState, *, target: float = 0.234, pooled=None) -> REState:
    """Adjust the number of Haar-refreshed sites from the pooled Haar acceptance rate
    (replica_exchange.py:357-386)."""
    pooled = pooled_counters(state) if pooled is None else pooled
    B = float(pooled[4, 0])
    rate = pooled[2].to(torch.float32) / max(B * state.n_haar, 1)
    n_active = int(state.mask.sum().item())
    delta = torch.where(rate > target, 1, -1).to(torch.int32)
    m = (state.m + delta).clamp(1, n_active)
    m = torch.where(state.beta == 0, torch.full_like(m, n_active), m)
    return replace(state, m=m, n_haar_accept=torch.zeros_like(state.n_haar_accept), n_haar=0)


def _monotone_slopes(t: np.ndarray, y: np.ndarray) -> np.ndarray:
    """Knot derivatives of a monotonicity-preserving cubic Hermite interpolant (Hyman's
    filter on the three-point estimate), as mcmc/_monotone_cubic.py:11-45 builds them."""
    h = np.diff(t)
    m = np.diff(y) / h

    def end(h0, h1, m0, m1):
        d = ((2.0 * h0 + h1) * m0 - h0 * m1) / (h0 + h1)
        if np.sign(d) != np.sign(m0):
            return 0.0
        if np.sign(m0) != np.sign(m1) and abs(d) > 3.0 * abs(m0):
            return 3.0 * m0
        return d

    inner = (h[1:] * m[:-1] + h[:-1] * m[1:]) / (h[:-1] + h[1:])
    cap = 3.0 * np.minimum(np.abs(m[:-1]), np.abs(m[1:]))
    inner = np.where(m[:-1] * m[1:] > 0, np.sign(m[1:]) * np.minimum(np.abs(inner), cap), 0.0)
    return np.concatenate([[end(h[0], h[1], m[0], m[1])], inner, [end(h[-1], h[-2], m[-1], m[-2])]])


def _hermite(t: np.ndarray, y: np.ndarray, d: np.ndarray, x: float) -> float:
    i = int(np.clip(np.searchsorted(t, x, side="right") - 1, 0, len(t) - 2))
    h = t[i + 1] - t[i]
    u = (x - t[i]) / h
    return (y[i] * (2 * u ** 3 - 3 * u ** 2 + 1) + h * d[i] * (u ** 3 - 2 * u ** 2 + u)
            + y[i + 1] * (-2 * u ** 3 + 3 * u ** 2) + h * d[i + 1] * (u ** 3 - u ** 2))


def equi_rejection_schedule(beta, rejection, *, offset: float = 1e-4, ema: float = 0.99) -> np.ndarray:
    """New inverse-temperature ladder that equalises the swap rejection between neighbours
    (replica_exchange.py:380-450): the cumulative rejection Lambda(beta) is interpolated by a
    monotone cubic, the interior temperatures are placed at equal steps of Lambda by bisection
    (50 iterations at most), and the result is mixed into the old ladder with weight 1 - ema."""
    beta = np.asarray(beta, dtype=np.float64)
    R = beta.shape[0]
    if R < 3:
        return beta.astype(np.float32)
    lam = np.concatenate([[0.0], np.cumsum(np.maximum(np.asarray(rejection, np.float64), offset))])
    slopes = _monotone_slopes(beta, lam)
    interior = []
    for i in range(1, R - 1):
        target = i * lam[-1] / (R - 1)
        lo, hi = offset, 1.0 - offset
        for _ in range(50):
            if hi - lo <= offset * 1e-3:
                break
            mid = 0.5 * (lo + hi)
            if _hermite(beta, lam, slopes, mid) - target < 0.0:
                lo = mid
            else:
                hi = mid
        interior.append(0.5 * (lo + hi))
    new = np.concatenate([[0.0], interior, [1.0]])
    return np.clip((1.0 - ema) * new + ema * beta, 0.0, 1.0).astype(np.float32)


def adapt_beta_equi_rej(state: REState, *, ema: float = 0.99, pooled=None) -> REState:
    """Refit the ladder from the pooled swap rejection rates and reset the swap counters
    (replica_exchange.py:453-477; pooled over walkers like the other adaptations)."""
    pooled = pooled_counters(state) if pooled is None else pooled
    R = state.q.shape[1]
    attempts = pooled[3, :R - 1].clamp(min=1.0)
    rejection = 1.0 - pooled[1, :R - 1] / attempts
    beta = equi_rejection_schedule(state.beta.cpu().numpy(), rejection.cpu().numpy(), ema=ema)
    return replace(state, beta=torch.as_tensor(beta, device=state.beta.device, dtype=state.beta.dtype),
                   n_swap_accept=torch.zeros_like(state.n_swap_accept),
                   n_swap=torch.zeros_like(state.n_swap))


def adapt_batched(state: REState, *, beta_history_weight: float = 0.9, sigma_target: float = 0.574,
                  sigma_scale: float = 1.1, haar_target: float = 0.234, group=None) -> REState:
    """The adaptation the reference applies between sampler calls, in its order and with its
    defaults (src/hamiltonzero/mcmc/runtime.py:132-195): counters pooled over the walkers, then
    the proposal widths, the Haar site counts and the ladder (history weight 0.9), then every
    counter reset. With the walkers sharded over the ranks of an initialised process group the
    counters are summed over the ranks first (one all-reduce of ``5 R`` numbers), so that every
    rank adapts to the same ladder."""
    pooled = all_reduce_counters(state, group)
    adapted = adapt_sigma(state, target=sigma_target, factor=sigma_scale, pooled=pooled)
    adapted = adapt_m(adapted, target=haar_target, pooled=pooled)
    adapted = adapt_beta_equi_rej(adapted, ema=beta_history_weight, pooled=pooled)
    return adapted


def pooled_counters(state: REState):
    """``[5, R]`` float64 summed over this rank's walkers: local accepts, swap accepts, Haar
    accepts, swap attempts (the swap rows padded to R) and, in every entry of the last row, the
    number of walkers - what ranks sum before a sharded ``adapt_batched``
    (runtime.py:148-156)."""
    B, R = state.q.shape[:2]
    out = torch.zeros(5, R, dtype=torch.float64, device=state.q.device)
    out[0] = state.n_local_accept.sum(0)
    out[1, :R - 1] = state.n_swap_accept.sum(0)
    out[2] = state.n_haar_accept.sum(0)
    out[3, :R - 1] = state.n_swap.sum(0)
    out[4] = float(B)
    return out


def all_reduce_counters(state: REState, group=None):
    """``pooled_counters`` summed over the ranks (NCCL for device tensors, gloo on CPU); the
    local counters when no process group is initialised."""
    import torch.distributed as dist
    pooled = pooled_counters(state)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(pooled, op=dist.ReduceOp.SUM, group=group)
    return pooled


__all__ = ["REState", "adapt_batched", "all_reduce_counters", "adapt_beta_equi_rej", "adapt_m", "adapt_sigma",
           "annealing_geometric", "cold_samples", "equi_rejection_schedule", "init_batched_state",
           "pooled_counters", "run_batched"]
