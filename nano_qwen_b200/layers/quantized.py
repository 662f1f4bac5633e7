"""An activation that already is what an FP8 linear layer consumes: e4m3 values plus 1x128 group scales.

Produced by the fused producers (``SiluAndMul``, ``RMSNorm`` / ``GemmaRMSNorm`` with ``emit_fp8=True``) and accepted
by every linear layer of ``nano_qwen_b200.layers.linear`` in place of a bf16 tensor, so the model code
``down_proj(act_fn(gate_up))`` (reference ``models/qwen3_5.py:164-165``) runs unchanged and one quantiser launch
disappears.
"""
from __future__ import annotations

import torch


class QuantizedActivation:
    """``xq`` ``[M, K]`` float8_e4m3fn, ``sx`` ``[M, ceil(K/128)]`` fp32 (K-group major storage), ``shape`` of the bf16
    tensor it stands for (leading dimensions kept for the layer's output)."""

    __slots__ = ("xq", "sx", "shape")

    def __init__(self, xq: torch.Tensor, sx: torch.Tensor, shape: torch.Size | tuple):
        self.xq, self.sx, self.shape = xq, sx, tuple(shape)

    @property
    def device(self):
        return self.xq.device

    @property
    def is_cuda(self) -> bool:
        return self.xq.is_cuda

    def dequantize(self) -> torch.Tensor:
        """The bf16 tensor this stands for, up to the quantisation error (for consumers that are not FP8 linears)."""
        M, K = self.xq.shape
        scales = self.sx.repeat_interleave(128, dim=1)[:, :K]
        return (self.xq.to(torch.float32) * scales).to(torch.bfloat16).view(*self.shape)
