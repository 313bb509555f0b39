"""Walker-path evaluation backend with the reference's method names.

The reference's inference API (``burn_in``, ``step``, ``energy``: src/hamiltonzero/inference.py:
159-259) drives an object that satisfies the ``EvalBackend`` protocol
(src/hamiltonzero/evaluation/backend.py:39-148). ``WalkerEvalBackend`` implements the part of
that protocol that runs per walker - ``initialize_mcmc``, ``prepare_singular``, ``step_mcmc``,
``adapt_mcmc``, ``mcmc_population`` / ``replace_mcmc_population``, ``cold_walkers``,
``custom_lap_energy``, ``block_until_ready`` - on the CUDA operators of this package, with the
argument lists of ``DefaultEvalBackend`` (src/hamiltonzero/evaluation/runtime.py:997-1253).
The remaining protocol methods (system and checkpoint loading, routing, the context
compiler, beam search) belong to the reference's control plane and are not provided here:
calling one raises ``AttributeError`` like any missing method.

``context`` is whatever carries the routed system: an ``systems.EnergyFrame`` (it holds the
real-site ``mask`` and the energy frame), or an object with ``mask`` and ``energy_frame``
attributes. ``model`` is a ``walker.CompiledWaveFunction``. ``config`` objects are read by
attribute, with the reference's defaults (src/hamiltonzero/config.py:141-144,209-221).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any

import numpy as np
import torch

from . import mcmc
from .walker import CompiledWaveFunction, as_device_frame, as_wavefunction, \
    vmc_energy_custom_lap_compiled


@dataclass(frozen=True)
class EvalMCMCConfig:
    """Defaults of src/hamiltonzero/config.py:209-221."""
    batch_size: int = 256
    replicas: int = 8
    steps: int = 24
    burn_in: int = 1024
    burn_in_replica_steps: int = 2
    walker_chunk_size: int = 16
    initial_sigma: float = 0.3
    initial_haar_sites: int = 1
    sigma_scale: float = 1.1
    langevin_target_acceptance: float = 0.574
    haar_target_acceptance: float = 0.234
    beta_history_weight: float = 0.9


@dataclass(frozen=True)
class EnergyConfig:
    """Defaults of src/hamiltonzero/config.py:141-144."""
    mu: float | None = None
    eps: float = 0.1
    chunk_size: int = 512


@dataclass(frozen=True)
class MCMCPopulation:
    """src/hamiltonzero/evaluation/backend.py:30-36."""
    q: Any
    sigma: Any
    beta: Any


def _mask_of(context):
    mask = getattr(context, "mask", None)
    if mask is None:
        raise TypeError("context must carry the routed real-site mask")
    return mask.cpu().numpy() if isinstance(mask, torch.Tensor) else np.asarray(mask)


def _frame_of(context):
    return getattr(context, "energy_frame", context)


class WalkerEvalBackend:
    def __init__(self, device=None):
        self.device = device

    # ---- placement (runtime.py:997-1019): everything of one system lives on this rank's GPU
    def prepare_singular(self, model, context, state):
        if state.q.ndim != 4:
            raise ValueError("post-selection eval MCMC state must have shape [B, R, N, 4]")
        model = as_wavefunction(model)
        as_device_frame(_frame_of(context), model.device)          # device copy, cached
        return model, context, state

    # ---- sampler (runtime.py:1021-1140)
    def initialize_mcmc(self, key, model, context, config=EvalMCMCConfig()):
        del model
        seed = int(np.asarray(key).reshape(-1)[-1]) if not isinstance(key, int) else key
        return mcmc.init_batched_state(seed, _mask_of(context), int(config.batch_size),
                                       int(config.replicas),
                                       initial_m=int(config.initial_haar_sites),
                                       initial_sigma=float(config.initial_sigma),
                                       device=self.device)

    def step_mcmc(self, state, model, context, *, replica_steps: int, walker_chunk_size: int):
        return mcmc.run_batched(as_wavefunction(model), context, state, int(replica_steps),
                                int(walker_chunk_size))

    def adapt_mcmc(self, state, config=EvalMCMCConfig()):
        return mcmc.adapt_batched(state, beta_history_weight=float(config.beta_history_weight),
                                  sigma_target=float(config.langevin_target_acceptance),
                                  sigma_scale=float(config.sigma_scale),
                                  haar_target=float(config.haar_target_acceptance))

    def mcmc_population(self, state) -> MCMCPopulation:
        return MCMCPopulation(q=state.q, sigma=state.sigma, beta=state.beta)

    def replace_mcmc_population(self, state, population: MCMCPopulation):
        """New walkers, widths and ladder; the cached log p and drift are refreshed by the next
        sampler call, as in the reference (replica_exchange.py:96-109)."""
        return replace(state, q=population.q.contiguous(), sigma=population.sigma,
                       beta=population.beta)

    def cold_walkers(self, state):
        return mcmc.cold_samples(state)

    # ---- energy (runtime.py:1198-1253): outputs carry the leading system axis of size one
    def custom_lap_energy(self, model, context, q, config=EnergyConfig()):
        if not isinstance(model, CompiledWaveFunction):
            model = as_wavefunction(model)
        outputs = vmc_energy_custom_lap_compiled(model, _frame_of(context), q,
                                                 chunk_size=int(config.chunk_size))
        return tuple(o[None] for o in outputs)

    def block_until_ready(self, value) -> None:
        torch.cuda.synchronize()


def build_eval_backend(device=None) -> WalkerEvalBackend:
    """src/hamiltonzero/evaluation/runtime.py: ``build_eval_backend``."""
    return WalkerEvalBackend(device)


__all__ = ["EnergyConfig", "EvalMCMCConfig", "MCMCPopulation", "WalkerEvalBackend",
           "build_eval_backend"]
