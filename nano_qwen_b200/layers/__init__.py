from .activation import SiluAndMul
from .layernorm import GemmaRMSNorm, RMSNorm
from .quantized import QuantizedActivation
from .linear import (
    ColumnParallelLinear,
    LinearBase,
    MergedColumnParallelLinear,
    QKVParallelLinear,
    ReplicatedLinear,
    RowParallelLinear,
    divide,
)

__all__ = [
    "LinearBase",
    "ReplicatedLinear",
    "ColumnParallelLinear",
    "MergedColumnParallelLinear",
    "QKVParallelLinear",
    "RowParallelLinear",
    "divide",
    "SiluAndMul",
    "RMSNorm",
    "GemmaRMSNorm",
    "QuantizedActivation",
]
