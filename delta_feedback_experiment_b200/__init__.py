"""B200-native PKDA delta-rule attention kernels behind the reference's own
operator interface.  See ``fla_ops`` (custom ops) and ``pkda`` (stateful
operators and the recurrence dispatch)."""

from .fla_ops import (CHUNK_SIZE, PKDA_INTERMEDIATES, PKDA_RETAINED, fla_ops_available,
                      pkda_recurrence)
from .pkda import (chunk_precond_kda, fused_recurrent_precond_kda, pkda_cuda_available,
                   pkda_cuda_recurrence)
from .layer_ops import pkda_norm_gate, pkda_qkv_conv
from .host_pipeline import HostStep

__all__ = [
    "CHUNK_SIZE", "PKDA_INTERMEDIATES", "PKDA_RETAINED", "fla_ops_available", "pkda_recurrence",
    "chunk_precond_kda", "fused_recurrent_precond_kda", "pkda_cuda_available",
    "pkda_cuda_recurrence", "pkda_qkv_conv", "pkda_norm_gate", "HostStep",
]
