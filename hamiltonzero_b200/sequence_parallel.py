"""The large-N context path's attention and 2-FWL ring on this library's kernels.

The reference shards a long node sequence over the devices of one axis: every device keeps its
rows of the queries and of the edge stream, all-gathers keys and values, and calls a
rectangular flash kernel (src/hamiltonzero/evaluation/pallas_mha.py:43-161, driven by
``pallas_rectangular_edge_attention``, src/hamiltonzero/evaluation/sequence_parallel.py:59-95);
the learned 2-FWL edge update passes column panels around a ring
(``ring_learned_fwl2_columns_local``, sequence_parallel.py:112-173). Here the kernel is
``hz_mha_rect_fwd`` (CUDA, forward only like the reference's), the gather and the ring are
``torch.distributed`` over the process group (NCCL between GPUs; the ring steps are paired
send/receive, the panel product of each step is ``hz_fwl2_panel``). One process per GPU; the
rank plays the role of ``jax.lax.axis_index``."""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from .attention import _dev, _ptr, _require_fp32, _stream


def noncausal_bias_mha(q, k, v, bias, key_mask=None):
    """``softmax_k(q k^T D^-1/2 + bias) v`` over all keys. q ``[B, Lq, H, D]`` (unscaled: note
    that the reference's kernel takes q already scaled by its caller, pallas_mha.py:70-72 and
    sequence_parallel.py:88-93; here the scale is applied inside), k, v ``[B, Lk, H, D]``, bias
    ``[B, Lq, Lk, H]``, key_mask ``[B, Lk]`` or None -> ``[B, Lq, H, D]``."""
    host = isinstance(q, np.ndarray)
    _require_fp32(q, k, v, bias)
    qd, kd, vd, bd = (_dev(x).contiguous() for x in (q, k, v, bias))
    if qd.ndim != 4 or kd.ndim != 4 or vd.shape != kd.shape:
        raise ValueError("q, k, v must be [batch, sequence, heads, head_dim] with k and v alike")
    B, Lq, H, D = qd.shape
    Lk = kd.shape[1]
    if tuple(kd.shape) != (B, Lk, H, D):
        raise ValueError("q, k, and v must have the same batch, head count and head dimension")
    if tuple(bd.shape) != (B, Lq, Lk, H):
        raise ValueError(f"bias must have shape [batch, query, key, heads]; got {tuple(bd.shape)}")
    md = None
    if key_mask is not None:
        md = _dev(key_mask, torch.uint8).ne(0).to(torch.uint8).contiguous()
        if tuple(md.shape) != (B, Lk):
            raise ValueError(f"key mask must have shape {(B, Lk)}, got {tuple(md.shape)}")
    out = torch.empty_like(qd)
    lib = _lib.load()
    need = lib.hz_mha_rect_workspace_bytes(B, Lq, Lk, H, D)
    ws = torch.empty(max(need, 0), dtype=torch.uint8, device=qd.device) if need > 0 else None
    st = lib.hz_mha_rect_fwd(B, Lq, Lk, H, D, _ptr(qd), _ptr(kd), _ptr(vd), _ptr(bd),
                             _ptr(md) if md is not None else 0, _ptr(out),
                             _ptr(ws) if ws is not None else 0, max(need, 0), _stream())
    _lib.check(st, "hz_mha_rect_fwd")
    return out.cpu().numpy() if host else out


def rectangular_edge_attention(q_local, k_global, v_global, edge_bias_local, key_mask, *, block_k=None):
    """``pallas_rectangular_edge_attention`` (sequence_parallel.py:59-95): q_local
    ``[Lq, H, D]``, k_global, v_global ``[Lk, H, D]``, edge_bias_local ``[Lq, Lk, H]``, key_mask
    ``[Lk]`` -> ``[Lq, H, D]``. ``block_k`` is accepted for signature parity (the kernel's key
    block is fixed; results do not depend on it beyond rounding)."""
    del block_k
    for x in (q_local, k_global, v_global):
        if np.ndim(x) != 3:
            raise ValueError("q, k, and v must have shapes [sequence, heads, head_dim]")
    if tuple(np.shape(edge_bias_local)) != (np.shape(q_local)[0], np.shape(k_global)[0], np.shape(q_local)[1]):
        raise ValueError("edge bias must have shape [local_queries, global_keys, heads]")
    if tuple(np.shape(key_mask)) != (np.shape(k_global)[0],):
        raise ValueError(f"key mask must have shape {(np.shape(k_global)[0],)}")
    out = noncausal_bias_mha(q_local[None], k_global[None], v_global[None], edge_bias_local[None],
                             key_mask[None])
    return out[0]


pallas_rectangular_edge_attention = rectangular_edge_attention      # the reference's name


def _group_info(group=None):
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def all_gather_sequence(x_local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenation of every rank's rows along axis 0 (equal shard sizes, as the reference's
    mesh sharding requires)."""
    import torch.distributed as dist
    rank, world = _group_info(group)
    if world == 1:
        return x_local
    parts = [torch.empty_like(x_local) for _ in range(world)]
    dist.all_gather(parts, x_local.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def sequence_parallel_edge_attention(q_local, k_local, v_local, edge_bias_local, key_mask_local, *,
                                     group=None, attention=None):
    """Attention of this rank's query rows over the keys of all ranks: keys, values and the key
    mask are all-gathered (the bias rows are local), then the rectangular kernel runs.
    ``attention`` replaces the kernel (host-side tests on CPU pass the einsum twin)."""
    k_global = all_gather_sequence(k_local, group)
    v_global = all_gather_sequence(v_local, group)
    mask_global = all_gather_sequence(key_mask_local, group)
    fn = rectangular_edge_attention if attention is None else attention
    return fn(q_local, k_global, v_global, edge_bias_local, mask_global)


def fwl2_panel(a_local, b_panel, out, origin: int, accumulate: bool):
    """``out[i, j, c] (+)= sum_k a_local[i, origin * rows + k, c] * b_panel[k, j, c]`` on the
    device (one ring step's contribution, sequence_parallel.py:148-153)."""
    rows, a_cols, C = a_local.shape
    panel, cols, _ = b_panel.shape
    st = _lib.load().hz_fwl2_panel(_ptr(a_local), _ptr(b_panel), _ptr(out), rows, a_cols, origin * panel,
                                   panel, cols, C, 1 if accumulate else 0, _stream())
    _lib.check(st, "hz_fwl2_panel")
    return out


def _fwl2_panel_torch(a_local, b_panel, out, origin, accumulate):
    rows = b_panel.shape[0]
    contrib = torch.einsum("ikc,kjc->ijc", a_local[:, origin * rows:(origin + 1) * rows], b_panel)
    return out.add_(contrib) if accumulate else out.copy_(contrib)


def ring_learned_fwl2_columns_local(a_local, b_local_columns, *, group=None, panel_product=None):
    """``out[i, j, c] = sum_k a[i, k, c] b[k, j, c]`` with ``a`` sharded by rows
    (``a_local [rows, rows * world, C]``) and ``b`` by rows too (``b_local_columns
    [rows, cols, C]``): every rank multiplies the panel it holds into the matching column block
    of its ``a`` rows, then passes the panel to the next rank, ``world - 1`` times
    (sequence_parallel.py:112-173). ``panel_product`` replaces the CUDA panel kernel (host-side
    tests on CPU)."""
    import torch.distributed as dist
    if a_local.ndim != 3 or b_local_columns.ndim != 3:
        raise ValueError("local 2-FWL operands must both be rank three")
    rows, global_columns, C = a_local.shape
    if b_local_columns.shape[0] != rows or b_local_columns.shape[2] != C:
        raise ValueError("local A/B row and channel counts must match")
    if a_local.dtype != b_local_columns.dtype:
        raise TypeError("local A/B dtypes must match")
    rank, world = _group_info(group)
    if global_columns != rows * world:
        raise ValueError("2-FWL row shards must evenly tile the contracted axis")
    product = panel_product or (fwl2_panel if a_local.is_cuda else _fwl2_panel_torch)
    a_local = a_local.contiguous()
    panel = b_local_columns.contiguous()
    out = torch.empty(rows, panel.shape[1], C, dtype=a_local.dtype, device=a_local.device)
    origin = rank
    product(a_local, panel, out, origin, False)
    for _ in range(world - 1):
        incoming = torch.empty_like(panel)
        ops = [dist.P2POp(dist.isend, panel, (rank + 1) % world, group),
               dist.P2POp(dist.irecv, incoming, (rank - 1) % world, group)]
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        panel = incoming
        origin = (origin - 1) % world
        product(a_local, panel, out, origin, True)
    return out


def ring_learned_fwl2_local(a_local, b_local, *, group=None, panel_product=None):
    """sequence_parallel.py:98-109: the square case (``b`` has the shape of ``a``)."""
    if tuple(b_local.shape) != tuple(a_local.shape):
        raise ValueError(f"local 2-FWL shapes must match; got {tuple(a_local.shape)}, {tuple(b_local.shape)}")
    return ring_learned_fwl2_columns_local(a_local, b_local, group=group, panel_product=panel_product)


__all__ = ["all_gather_sequence", "fwl2_panel", "noncausal_bias_mha", "pallas_rectangular_edge_attention",
           "rectangular_edge_attention", "ring_learned_fwl2_columns_local", "ring_learned_fwl2_local",
           "sequence_parallel_edge_attention"]
