"""The loss around the reverse pass: centring, loss tangent and Fisher registration of the
fine-tune step (src/hamiltonzero/optim/production.py:32-80,168-228).

The reference's ``total_energy`` is a ``custom_jvp`` whose primal is the mean energy and whose
tangent is ``2 (sum tan_re * Re dE + sum tan_im * Im dE) / n_eff`` with ``dE`` the centred,
gradient-stopped local energies and ``(tan_re, tan_im)`` the tangents of ``(log|psi|, phase)``.
Transposed, the parameter gradient is one reverse pass of ``hz_logpsi_vjp`` with the cotangents
``2 Re dE / n_eff`` and ``2 Im dE / n_eff``; the Fisher registration (``_register_fisher_output``
with the Rademacher ``_signed_identity``) is a second reverse pass whose cotangents are the
signs themselves, which is what the KFAC second-moment sums are taken from. Sums that the
reference takes with ``psum`` over the ``"batch"`` axis are all-reduces over the process group
here (NCCL on GPUs, gloo on CPU)."""
from __future__ import annotations

import torch

from . import sharding

_FISHER_SIGN_STREAM = 1262895427          # production.py:21
_FISHER_CHANNELS = 3                      # production.py:22


def _all_reduce(t: torch.Tensor, group=None) -> torch.Tensor:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def make_fisher_signs(seed: int, q_cold: torch.Tensor) -> torch.Tensor:
    """Rademacher signs ``[systems, walkers, 3]`` in the dtype of the walkers
    (production.py:32-49). The stream is this library's (a torch generator seeded with the key
    folded with the reference's stream constant), not jax.random's bits; each rank of a sharded
    batch folds its rank in as well so that shards draw independent signs."""
    import torch.distributed as dist
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    gen = torch.Generator(device="cpu").manual_seed((int(seed) * 1000003 + _FISHER_SIGN_STREAM + rank)
                                                    % (2 ** 63 - 1))
    bits = torch.randint(0, 2, tuple(q_cold.shape[:2]) + (_FISHER_CHANNELS,), generator=gen)
    return (2 * bits - 1).to(dtype=q_cold.dtype if q_cold.dtype.is_floating_point else torch.float32,
                             device=q_cold.device)


def center_preprocessed_energy(energy: torch.Tensor, group=None):
    """``(delta, mean)``: local energies ``[systems, walkers]`` minus the per-system mean over
    the walkers of ALL ranks (production.py:63-80). One all-reduce of ``2 systems + 1`` numbers."""
    e = energy.to(torch.complex128)
    packed = torch.cat([torch.view_as_real(e.sum(dim=1)).reshape(-1),
                        torch.tensor([float(e.shape[1])], dtype=torch.float64, device=e.device)])
    _all_reduce(packed, group)
    total = torch.view_as_complex(packed[:-1].reshape(-1, 2).contiguous())
    mean = total / torch.clamp(packed[-1], min=1.0)
    return (e - mean[:, None]).to(energy.dtype), mean.to(energy.dtype)


def loss_cotangents(energy: torch.Tensor, group=None):
    """``(cot_log_abs, cot_phase, loss)`` of the fine-tune loss for this rank's walkers:
    ``2 Re dE / n_eff`` and ``2 Im dE / n_eff`` with ``n_eff`` the number of walkers of all ranks
    whose centred energy is non-zero, and the loss value ``mean_systems Re <E>``
    (production.py:201-226)."""
    delta, mean = center_preprocessed_energy(energy, group)
    n_eff = _all_reduce((delta.abs() > 0).sum().to(torch.float64).reshape(1), group)
    scale = 2.0 / torch.clamp(n_eff, min=1.0)
    real_dtype = delta.real.dtype
    return ((delta.real.to(torch.float64) * scale).to(real_dtype),
            (delta.imag.to(torch.float64) * scale).to(real_dtype), mean.real.mean())


def finetune_loss_and_gradient(wavefunction, q_cold, energy, *, group=None, chunk_size=512):
    """``(loss, grads)``: the mean energy and its parameter gradient, summed over all ranks.
    ``q_cold [systems = 1, walkers, N, 4]`` and ``energy [1, walkers]`` are this rank's shard of
    the preprocessed batch (production.py:168-228); ``grads`` has the layout of
    ``CompiledWaveFunction.vjp``."""
    q = torch.as_tensor(q_cold)
    e = torch.as_tensor(energy).to(q.device if q.is_cuda else wavefunction.device)
    if q.ndim != 4 or q.shape[0] != 1 or tuple(e.shape) != tuple(q.shape[:2]):
        raise ValueError("q_cold must be [1, walkers, N, 4] and energy [1, walkers]")
    ca, cp, loss = loss_cotangents(e, group)
    grads, _, _, _ = wavefunction.vjp(q[0].to(wavefunction.device), ca[0].float().contiguous(),
                                      cp[0].float().contiguous(), want_dq=False, chunk_size=chunk_size)
    sharding.reduce_gradients(grads, group=group)
    return loss, grads


def fisher_factor_sums(wavefunction, q_cold, fisher_signs, *, leaf_mask=None, marginals=True,
                       group=None, chunk_size=512):
    """The reverse pass behind the Fisher registration: cotangents are the Rademacher signs of
    channels 0 (``log|psi|``) and 1 (phase); returns ``(factors, walkers)`` with the
    second-moment sums of every tag and the walker count, both summed over all ranks (one
    all-reduce of the packed sums)."""
    q = torch.as_tensor(q_cold)
    s = torch.as_tensor(fisher_signs)
    if q.ndim != 4 or q.shape[0] != 1 or tuple(s.shape[:2]) != tuple(q.shape[:2]):
        raise ValueError("q_cold must be [1, walkers, N, 4] and fisher_signs [1, walkers, 3]")
    out = wavefunction.vjp(q[0].to(wavefunction.device), s[0, :, 0].float().contiguous(),
                           s[0, :, 1].float().contiguous(), want_dq=False, chunk_size=chunk_size,
                           factors="marginals" if marginals else True, leaf_mask=leaf_mask)
    factors = out[4]
    count = {"walkers": torch.tensor([float(q.shape[1])], device=wavefunction.device)}
    sharding.reduce_gradients(factors, count, group=group)
    return factors, int(count["walkers"].item())


__all__ = ["center_preprocessed_energy", "finetune_loss_and_gradient", "fisher_factor_sums",
           "loss_cotangents", "make_fisher_signs"]
