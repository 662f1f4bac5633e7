"""``SiluAndMul`` that hands the next linear layer FP8 directly (reference ``nano_qwen/layers/activation.py:6-11``)."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from .quantized import QuantizedActivation


class SiluAndMul(nn.Module):
    """``silu(x[..., :I]) * x[..., I:]``.

    With ``emit_fp8=True`` (default) a CUDA bf16 input yields a :class:`QuantizedActivation` — the bf16 result of the
    reference, quantised per token and 128-wide group by the same kernel pass — which ``RowParallelLinear`` (down_proj)
    consumes without a quantiser launch; any other input raises (the FP8 path has no CPU or other-dtype fallback).
    ``emit_fp8=False`` is not part of the FP8 path: it is the reference's eager arithmetic in torch.
    """

    def __init__(self, emit_fp8: bool = True):
        super().__init__()
        self.emit_fp8 = emit_fp8

    def forward(self, x: torch.Tensor):
        if not self.emit_fp8:
            gate, up = x.chunk(2, -1)
            return F.silu(gate) * up
        if not x.is_cuda or x.dtype != torch.bfloat16:
            raise RuntimeError(f"SiluAndMul(emit_fp8=True) needs a CUDA bfloat16 tensor, got {x.device.type} {x.dtype}: "
                               "there is no CPU fallback (construct it with emit_fp8=False for the eager op)")
        inter = x.shape[-1] // 2
        xq, sx = ops.silu_mul_quant(x.reshape(-1, x.shape[-1]))
        return QuantizedActivation(xq, sx, (*x.shape[:-1], inter))
