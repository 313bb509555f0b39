"""Walker sharding across ranks and the one small reduction the energy path needs.

Walkers are independent, so the batch is cut contiguously on its leading axis, one shard
per rank, exactly like the reference's ``P("batch")`` partition
(src/hamiltonzero/evaluation/runtime.py:280-316,398-417); parameters and the energy frame
are replicated. The only data that crosses ranks is the energy moments used for centring
(src/hamiltonzero/optim/production.py:63-80: a psum of the summed local energy and the
count): one all-reduce of five numbers over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).
The fine-tune step adds the psum of the parameter gradients and KFAC factor statistics that
each rank accumulated over its own walkers (kfac_jax's ``pmean`` over the ``"batch"`` axis):
``reduce_gradients`` packs them into one flat buffer so that it is a single all-reduce.
"""
from __future__ import annotations

import torch


def shard_bounds(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """[start, stop) of this rank's contiguous shard; the first ``n_items % world`` ranks
    hold one extra item (ragged batches are allowed, empty shards too)."""
    if world <= 0 or not (0 <= rank < world) or n_items < 0:
        raise ValueError("need 0 <= rank < world and n_items >= 0")
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard(tensor, rank: int, world: int):
    a, b = shard_bounds(tensor.shape[0], rank, world)
    return tensor[a:b]


def local_moments(total: torch.Tensor) -> torch.Tensor:
    """``[sum Re E, sum Im E, sum |E|^2, count, 0]`` in float64 for this rank's samples
    (NaN samples are skipped and not counted)."""
    e = total.reshape(-1).to(torch.complex128)
    ok = torch.isfinite(e.real) & torch.isfinite(e.imag)
    e = torch.where(ok, e, torch.zeros_like(e))
    return torch.stack([e.real.sum(), e.imag.sum(), (e.real ** 2 + e.imag ** 2).sum(),
                        ok.sum().to(torch.float64), torch.zeros((), dtype=torch.float64,
                                                               device=e.device)])


def all_reduce_moments(moments: torch.Tensor, group=None, async_op: bool = False):
    """The exchange step alone: sum the five moments over the ranks, in place, on the device
    (one NCCL all-reduce of 40 bytes; no host synchronisation). With ``async_op`` the call
    returns ``(moments, work)`` and the launching stream does not wait for the reduction: the
    caller waits on ``work`` (``None`` without a process group) where it consumes the moments,
    so that ranks are not put in lockstep after every step."""
    import torch.distributed as dist
    work = None
    if dist.is_available() and dist.is_initialized():
        work = dist.all_reduce(moments, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
    return (moments, work) if async_op else moments


def reduce_moments(moments: torch.Tensor, group=None) -> dict:
    """All-reduce the moments and return the batch mean, variance and count."""
    all_reduce_moments(moments, group)
    m = moments.tolist()
    n = max(m[3], 1.0)
    mean = complex(m[0] / n, m[1] / n)
    var = max(m[2] / n - abs(mean) ** 2, 0.0)
    return {"mean": mean, "variance": var, "count": int(m[3])}


def centred(total: torch.Tensor, stats: dict) -> torch.Tensor:
    """``E - <E>`` with the global mean (the ``delta_E`` the fine-tune loss uses)."""
    return total - torch.as_tensor(stats["mean"], dtype=total.dtype, device=total.device)


def _flatten(tree):
    """Leaves of a dict of tensors / lists of tensors, in a deterministic order."""
    leaves = []
    for key in sorted(tree):
        v = tree[key]
        leaves.extend(v if isinstance(v, (list, tuple)) else [v])
    return leaves


def reduce_gradients(*trees, group=None):
    """Sum the per-rank results of ``CompiledWaveFunction.vjp`` (gradient dicts, factor
    dicts) over all ranks, in place: every leaf is copied into one flat fp32 buffer, the buffer
    is all-reduced once and copied back (bucketed for launch latency, not for link count).
    Returns the number of elements that crossed."""
    import torch.distributed as dist
    leaves = [t for tree in trees if tree is not None for t in _flatten(tree)]
    if not leaves:
        return 0
    flat = torch.cat([t.reshape(-1).to(torch.float32) for t in leaves])
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for t in leaves:
        n = t.numel()
        t.copy_(flat[off:off + n].reshape(t.shape))
        off += n
    return off
