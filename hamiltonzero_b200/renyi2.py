"""Basis-state sampler and SWAP estimator of the second Renyi entropy on the CUDA log-psi op.

Host-side mirror of the reference's computational-basis chains
(src/hamiltonzero/renyi2.py:87-297): spin configurations enter the wavefunction as corner
quaternions (up -> (1,0,0,0), down -> (0,0,1,0), ``_routed_corners`` :87-97), a chain flips one
uniformly chosen site per step and accepts with min(1, |psi'|^2 / |psi|^2) with the reference's
rules for zero and non-finite amplitudes (``_metropolis_log_acceptance`` :113-124), and the
purity of a subsystem is the mean over pairs of independent samples of
psi(x_A' , x_B) psi(x_A, x_B') / (psi(x) psi(x')) (``_swap_log_ratios`` :258-297), averaged in
log-polar form (``_complex_mean_log_polar`` :300-321). Every wavefunction value comes from
``hz_logpsi``; the random numbers come from a seeded ``torch.Generator`` instead of JAX's
threefry, so agreement with the reference's chains is distributional.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .walker import as_wavefunction


@dataclass
class BasisSamplerState:
    bits: torch.Tensor            # [B, n_spins] bool, True = down
    log_abs: torch.Tensor         # [B]
    generator: torch.Generator
    accepted: int = 0
    proposed: int = 0


def routed_corners(bits, route, *, n_spins: int) -> torch.Tensor:
    """``[B, n_spins]`` bits -> routed corner quaternions ``[B, N, 4]`` (renyi2.py:87-97)."""
    bits = torch.as_tensor(bits)
    route = torch.as_tensor(route, device=bits.device, dtype=torch.long)
    width = int(route.shape[0])
    padding = width - int(n_spins)
    if padding < 0:
        raise ValueError("physical spin count exceeds compiled width")
    full = torch.nn.functional.pad(bits.to(torch.bool), (0, padding), value=False)
    routed = full.index_select(-1, route)
    down = routed.to(torch.float32)
    up = 1.0 - down
    zeros = torch.zeros_like(up)
    return torch.stack((up, zeros, down, zeros), dim=-1).contiguous()


def basis_log_wavefunction(wavefunction, bits, route, *, n_spins: int):
    wf = as_wavefunction(wavefunction)
    q = routed_corners(torch.as_tensor(bits, device=wf.device), route, n_spins=n_spins)
    return wf(q)


def metropolis_log_acceptance(current_log_abs, proposed_log_abs):
    """log min(1, |psi'|^2/|psi|^2) with the reference's edge rules (renyi2.py:113-124): a move
    between two exact zeros or out of a non-finite state is always accepted, a move into a
    non-finite state never."""
    cur, prop = torch.as_tensor(current_log_abs), torch.as_tensor(proposed_log_abs)
    cur_fin, prop_fin = torch.isfinite(cur), torch.isfinite(prop)
    log_ratio = 2.0 * (prop - cur)
    log_accept = torch.minimum(torch.zeros_like(log_ratio), log_ratio)
    both_zero = torch.isneginf(cur) & torch.isneginf(prop)
    recover = ~cur_fin & prop_fin
    invalid = ~prop_fin & ~both_zero
    log_accept = torch.where(both_zero | recover, torch.zeros_like(log_accept), log_accept)
    return torch.where(invalid, torch.full_like(log_accept, -math.inf), log_accept)


def _basis_step(state: BasisSamplerState, wavefunction, route, n_spins: int) -> BasisSamplerState:
    bits, gen = state.bits, state.generator
    B = bits.shape[0]
    sites = torch.randint(0, n_spins, (B,), device=bits.device, generator=gen)
    rows = torch.arange(B, device=bits.device)
    proposed = bits.clone()
    proposed[rows, sites] = ~bits[rows, sites]
    prop_log_abs, _ = basis_log_wavefunction(wavefunction, proposed, route, n_spins=n_spins)
    log_accept = metropolis_log_acceptance(state.log_abs, prop_log_abs)
    log_u = torch.log(torch.rand(B, device=bits.device, generator=gen))
    accept = log_u < log_accept
    return BasisSamplerState(bits=torch.where(accept[:, None], proposed, bits),
                             log_abs=torch.where(accept, prop_log_abs, state.log_abs),
                             generator=gen, accepted=state.accepted + int(accept.sum()),
                             proposed=state.proposed + B)


def _require_finite_state(state: BasisSamplerState) -> None:
    if not bool(torch.isfinite(state.log_abs).all()):
        raise RuntimeError("basis burn-in ended with a zero or non-finite wavefunction coefficient")


def burn_in_basis(wavefunction, route, n_spins: int, seed: int, *, batch_size: int = 256,
                  burn_in: int = 1024):
    """Random bit strings, then ``burn_in`` single-site-flip Metropolis steps
    (renyi2.py:176-207). Returns ``(state, bits)``."""
    if int(batch_size) < 1:
        raise ValueError("batch_size must be positive")
    if int(burn_in) < 0:
        raise ValueError("burn_in must be non-negative")
    wf = as_wavefunction(wavefunction)
    gen = torch.Generator(device=wf.device).manual_seed(int(seed))
    bits = torch.rand(int(batch_size), n_spins, device=wf.device, generator=gen) < 0.5
    log_abs, _ = basis_log_wavefunction(wf, bits, route, n_spins=n_spins)
    state = BasisSamplerState(bits=bits, log_abs=log_abs, generator=gen)
    for _ in range(int(burn_in)):
        state = _basis_step(state, wf, route, n_spins)
    _require_finite_state(state)
    return state, state.bits


def step_basis(wavefunction, route, n_spins: int, state: BasisSamplerState, *, steps: int = 24):
    """``steps`` more Metropolis steps (renyi2.py:210-233)."""
    if not isinstance(state, BasisSamplerState):
        raise TypeError("state must be a BasisSamplerState")
    if int(steps) < 1:
        raise ValueError("steps must be positive")
    if state.bits.shape[-1] != n_spins:
        raise ValueError("basis state width does not match the prepared system")
    for _ in range(int(steps)):
        state = _basis_step(state, wavefunction, route, n_spins)
    _require_finite_state(state)
    return state, state.bits


def subsystem_mask(subsystem, *, n_spins: int) -> np.ndarray:
    """Boolean region mask from site indices or a boolean mask (renyi2.py:236-262)."""
    value = np.asarray(subsystem)
    if value.ndim == 1 and value.size == 0:
        return np.zeros((n_spins,), dtype=bool)
    if value.dtype == np.bool_:
        if value.shape != (n_spins,):
            raise ValueError(f"boolean subsystem mask must have shape [{n_spins}]")
        return value
    if value.ndim != 1:
        raise ValueError("subsystem site indices must be one-dimensional")
    if not np.issubdtype(value.dtype, np.integer):
        raise TypeError("subsystem must contain integer sites or booleans")
    sites = value.astype(np.int64)
    if len(np.unique(sites)) != sites.size:
        raise ValueError("subsystem site indices must be unique")
    if np.any(sites < 0) or np.any(sites >= n_spins):
        raise ValueError("subsystem site index is out of range")
    mask = np.zeros((n_spins,), dtype=bool)
    mask[sites] = True
    return mask


def swap_log_ratios(wavefunction, replica_x, replica_y, route, region_mask, *, n_spins: int):
    """``(log_abs, phase, valid)`` of psi(swap_x) psi(swap_y) / (psi(x) psi(y)) per pair
    (renyi2.py:265-297)."""
    wf = as_wavefunction(wavefunction)
    x = torch.as_tensor(replica_x, device=wf.device).to(torch.bool)
    y = torch.as_tensor(replica_y, device=wf.device).to(torch.bool)
    region = torch.as_tensor(np.asarray(region_mask, dtype=bool), device=wf.device)
    sx = torch.where(region[None, :], y, x)
    sy = torch.where(region[None, :], x, y)
    # one batched evaluation of the four configurations of every pair
    la, ph = basis_log_wavefunction(wf, torch.cat([x, y, sx, sy]), route, n_spins=n_spins)
    n = x.shape[0]
    dx, dy, nx, ny = (la[i * n:(i + 1) * n] for i in range(4))
    px, py, pnx, pny = (ph[i * n:(i + 1) * n] for i in range(4))
    valid = torch.isfinite(dx) & torch.isfinite(dy)
    log_abs = nx + ny - dx - dy
    phase = pnx + pny - px - py
    phase = torch.atan2(torch.sin(phase), torch.cos(phase))
    log_abs = torch.where(valid, log_abs, torch.full_like(log_abs, -math.inf))
    phase = torch.where(valid, phase, torch.zeros_like(phase))
    if bool((~region).all()) or bool(region.all()):
        log_abs = torch.where(valid, torch.zeros_like(log_abs), log_abs)
        phase = torch.where(valid, torch.zeros_like(phase), phase)
    return log_abs, phase, valid


def complex_mean_log_polar(log_abs, phase):
    """Mean of exp(log_abs + i phase) returned as ``(log |mean|, arg mean)``, with a pivot so
    that nothing overflows (renyi2.py:300-321)."""
    logs = np.asarray(torch.as_tensor(log_abs).cpu(), dtype=np.float64).reshape(-1)
    phases = np.asarray(torch.as_tensor(phase).cpu(), dtype=np.float64).reshape(-1)
    if logs.shape != phases.shape or logs.size == 0:
        raise ValueError("log_abs and phase must have matching nonempty shapes")
    if np.any(np.isnan(logs)) or np.any(np.isposinf(logs)) or np.any(~np.isfinite(phases)):
        raise ValueError("non-finite SWAP log-polar sample")
    finite = np.isfinite(logs)
    if not np.any(finite):
        return -math.inf, 0.0
    pivot = float(np.max(logs[finite]))
    scaled = np.zeros(logs.shape, dtype=np.complex128)
    scaled[finite] = np.exp(logs[finite] - pivot + 1j * phases[finite])
    mean = np.mean(scaled)
    if abs(mean) == 0.0:
        return -math.inf, 0.0
    return pivot + math.log(abs(mean)), float(np.angle(mean))


def renyi2(wavefunction, route, n_spins: int, subsystem, bits_x, bits_y):
    """Second Renyi entropy (nats) of ``subsystem`` from two sets of independent samples of
    |psi|^2: ``-log Re mean(SWAP ratio)``, with the purity and the per-pair ratios."""
    mask = subsystem_mask(subsystem, n_spins=n_spins)
    log_abs, phase, valid = swap_log_ratios(wavefunction, bits_x, bits_y, route, mask, n_spins=n_spins)
    mean_log, mean_phase = complex_mean_log_polar(log_abs, phase)
    purity = 0.0 if mean_log == -math.inf else math.exp(mean_log) * math.cos(mean_phase)
    return {"purity": purity, "renyi2_nats": -math.log(purity) if purity > 0 else None,
            "mean_log_abs": mean_log, "mean_phase": mean_phase, "swap_log_abs": log_abs,
            "swap_phase": phase, "valid_denominator": valid}


__all__ = ["BasisSamplerState", "basis_log_wavefunction", "burn_in_basis", "complex_mean_log_polar",
           "metropolis_log_acceptance", "renyi2", "routed_corners", "step_basis", "subsystem_mask",
           "swap_log_ratios"]
