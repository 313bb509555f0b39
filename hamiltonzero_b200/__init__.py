"""hamiltonzero_b200: CUDA (sm_100a) operators for HamiltonZero's hot path behind
the reference's own Python interface. The arithmetic lives in libhz_b200.so
(C ABI: include/hz_b200.h); PyTorch is used for device memory and streams only."""
from . import _lib  # noqa: F401
from .attention import (  # noqa: F401
    HZ_ATTN_BF16X3,
    HZ_ATTN_FP16X3,
    HZ_ATTN_TCGEN05,
    HZ_ATTN_TF32,
    HZ_ATTN_TF32X3,
    HZ_MASK_KEYS,
    HZ_MASK_SQUARE,
    gated_edge_attention,
    mhsea_bwd,
    mhsea_fwd,
    mhsea_jvp,
    mhsea_linear_tangent,
    mhsea_tuned_edge_attention,
    mhsea_with_tuned_ad,
    reference_edge_attention,
)
from . import mcmc, sharding, systems, types  # noqa: F401
from .types import CompiledTree, FactorizedQSide, QSideLeafInput, SharedKernel  # noqa: F401
from .walker import (  # noqa: F401
    CompiledWaveFunction,
    DeviceEnergyFrame,
    local_spin,
    logpsi_and_chart_gradient,
    vmc_energy_custom_lap_compiled,
)
from . import backend, context, featurizer, finetune, kfac, renyi2, sequence_parallel, tree_compiler  # noqa: F401
from .backend import WalkerEvalBackend, build_eval_backend  # noqa: F401

__version__ = "0.1.0"
