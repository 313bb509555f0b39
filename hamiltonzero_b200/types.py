"""Plain-array mirrors of the reference's compiled-wavefunction types.

``SharedKernel`` and ``CompiledTree`` carry the same field names as the reference's
equinox modules (src/hamiltonzero/compiled/types.py:22-45,131-140), so that code written
against ``kernel.merge_T``, ``kernel.leaf_factors[0].V``, ``tree.merge_h[level]`` ... reads
the same here. The single-head executor takes exactly one factor per stage and no combiners
(src/hamiltonzero/compiled/execute.py:79-92); ``to_arrays`` enforces that with the reference's
messages.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import numpy as np

from .systems import WavefunctionArrays


@dataclass
class QSideLeafInput:
    weight: Any                     # [4, d_o]


@dataclass
class FactorizedQSide:
    V: Any                          # [d_in, r]
    U: Any                          # [r, d_out]


@dataclass
class SharedKernel:
    q_to_odd: QSideLeafInput
    leaf_factors: Sequence[FactorizedQSide]
    leaf_combiner_factors: Sequence[FactorizedQSide]
    merge_T: Any                    # [G, d_r, d_r, d_r]
    merge_factors: Sequence[FactorizedQSide]
    readout_factors: Sequence[FactorizedQSide]
    merge_eps: float = 1e-6


@dataclass
class CompiledTree:
    perm: Any
    inv_perm: Any
    leaf_real: Any
    leaf_h: Sequence[Any]           # ([N, r_leaf],)
    leaf_combiner_h: Sequence[Any]
    merge_h: Sequence[Any]          # level l: [N >> (l + 1), r_merge]
    opcodes: Sequence[Any]          # level l: [N >> (l + 1)] uint8
    readout_h: Sequence[Any]        # ([r_ro],)
    readout_combiner_h: Sequence[Any] = field(default_factory=tuple)


@dataclass
class SharedTrunk:
    """Route-independent trunk state of one system (compiled/types.py:122-128)."""
    node_raw: Any                   # [N, d_e]
    edge_raw: Any                   # [N, N, d_edge]
    global_raw: Any                 # [d_g] featurizer output
    global_stream: Any              # [d_g] after the trunk's global update
    real_mask: Any                  # [N]
    balanced_mask: Any              # [N] the balanced subtree that holds the real sites


def _single(values, name: str):
    if len(values) != 1:
        raise ValueError(f"compiled HT executor requires exactly one {name}; got {len(values)}")
    return values[0]


def to_arrays(kernel: SharedKernel, tree: CompiledTree) -> WavefunctionArrays:
    """The flat arrays the C ABI takes, with the executor's checks (execute.py:79-92)."""
    if len(tree.leaf_combiner_h) != 0 or len(tree.readout_combiner_h) != 0:
        raise ValueError("single-head compiled HT executor does not accept combiners")
    if len(tree.merge_h) != len(tree.opcodes):
        raise ValueError("merge_h and opcodes must have one entry per tree level")
    leaf = _single(kernel.leaf_factors, "leaf factor")
    merge = _single(kernel.merge_factors, "merge factor")
    readout = _single(kernel.readout_factors, "readout factor")
    f = lambda a: np.asarray(a, dtype=np.float32)
    return WavefunctionArrays(
        q_weight=f(kernel.q_to_odd.weight), leaf_V=f(leaf.V), leaf_U=f(leaf.U),
        leaf_h=f(_single(tree.leaf_h, "leaf conditioner")), merge_T=f(kernel.merge_T),
        merge_V=f(merge.V), merge_U=f(merge.U), merge_h=[f(h) for h in tree.merge_h],
        opcodes=[np.asarray(o, dtype=np.uint8) for o in tree.opcodes],
        readout_V=f(readout.V), readout_U=f(readout.U),
        readout_h=f(_single(tree.readout_h, "readout conditioner")),
        merge_eps=float(kernel.merge_eps))


def from_arrays(a: WavefunctionArrays, leaf_real=None) -> tuple[SharedKernel, CompiledTree]:
    """``(SharedKernel, CompiledTree)`` over the arrays of ``a`` with the identity route."""
    n = a.n_sites
    kernel = SharedKernel(
        q_to_odd=QSideLeafInput(a.q_weight), leaf_factors=(FactorizedQSide(a.leaf_V, a.leaf_U),),
        leaf_combiner_factors=(), merge_T=a.merge_T,
        merge_factors=(FactorizedQSide(a.merge_V, a.merge_U),),
        readout_factors=(FactorizedQSide(a.readout_V, a.readout_U),), merge_eps=a.merge_eps)
    tree = CompiledTree(
        perm=np.arange(n, dtype=np.int32), inv_perm=np.arange(n, dtype=np.int32),
        leaf_real=np.ones(n, dtype=bool) if leaf_real is None else np.asarray(leaf_real, bool),
        leaf_h=(a.leaf_h,), leaf_combiner_h=(), merge_h=tuple(a.merge_h),
        opcodes=tuple(a.opcodes), readout_h=(a.readout_h,), readout_combiner_h=())
    return kernel, tree


__all__ = ["CompiledTree", "FactorizedQSide", "QSideLeafInput", "SharedKernel", "SharedTrunk", "from_arrays",
           "to_arrays"]
