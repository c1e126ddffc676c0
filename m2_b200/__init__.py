"""m2_b200: the M2-BERT sequence-mixer / BlockdiagLinear GLU MLP forward path on B200.

Drop-in modules with the reference's constructor signatures and state_dict layout:

    from m2_b200 import MonarchMixerSequenceMixing, BlockdiagLinear, HyenaFilter

The kernels live in libm2b200.so (C ABI in include/m2_b200.h) and are reached through
ctypes; there is no CPU or eager fallback.
"""
from .blockdiag_linear import (BlockdiagLinear, StructuredLinear, blockdiag_multiply,  # noqa: F401
                               blockdiag_weight_to_dense_weight)
from .hyena_filter import (ExponentialModulation, HyenaFilter, OptimModule,  # noqa: F401
                           PositionalEmbedding, Sin)
from .sequence_mixer import MonarchMixerSequenceMixing  # noqa: F401
from .glu_mlp import BertGatedLinearUnitMLP  # noqa: F401
from .graph import GraphedForward  # noqa: F401

__all__ = [
    "MonarchMixerSequenceMixing", "HyenaFilter", "BlockdiagLinear", "StructuredLinear",
    "BertGatedLinearUnitMLP", "blockdiag_multiply", "Sin", "PositionalEmbedding",
    "ExponentialModulation", "OptimModule", "GraphedForward",
]
