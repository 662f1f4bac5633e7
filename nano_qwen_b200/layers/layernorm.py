"""RMS norms that hand the next linear layer FP8 directly (reference ``nano_qwen/layers/layernorm.py``).

``RMSNorm`` (``:5-56``) scales by ``weight``; ``GemmaRMSNorm`` (``:59-120``) by ``1 + weight``.  Same constructor,
parameter name and call convention as the reference: ``forward(x)`` or ``forward(x, residual) -> (out, residual)``.
With ``emit_fp8=True`` the first result is a :class:`QuantizedActivation` for the FP8 linear layers (qkv_proj,
gate_up_proj) and the input must be a CUDA bf16 tensor: anything else raises (the FP8 path has no CPU or other-dtype
fallback).  ``emit_fp8=False`` (default) is not part of the FP8 path: it is the reference's own eager arithmetic in
torch, for norms whose consumer is not an FP8 linear (q_norm / k_norm, the final norm).
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from .quantized import QuantizedActivation


class _NormBase(nn.Module):
    gemma = False

    def __init__(self, hidden_size: int, eps: float = 1e-6, emit_fp8: bool = False):
        super().__init__()
        self.eps = eps
        self.emit_fp8 = emit_fp8
        init = torch.zeros if self.gemma else torch.ones
        self.weight = nn.Parameter(init(hidden_size))

    def _eager(self, x: torch.Tensor, residual: torch.Tensor | None):
        """The reference's eager arithmetic (``layernorm.py:16-40`` / ``:79-105``), out of place."""
        orig = x.dtype
        v = x.float()
        if residual is not None:
            v = v + residual.float()
            residual = v.to(orig)
        var = v.pow(2).mean(dim=-1, keepdim=True)
        n = (v * torch.rsqrt(var + self.eps)).to(orig)
        out = n * (1.0 + self.weight) if self.gemma else n * self.weight
        return out if residual is None else (out, residual)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if not self.emit_fp8:
            return self._eager(x, residual)
        if not x.is_cuda or x.dtype != torch.bfloat16:
            raise RuntimeError(f"{type(self).__name__}(emit_fp8=True) needs a CUDA bfloat16 tensor, got {x.device.type} "
                               f"{x.dtype}: there is no CPU fallback (construct it with emit_fp8=False for the eager op)")
        H = x.shape[-1]
        res2 = residual.reshape(-1, H) if residual is not None else None
        xq, sx, new_res, _ = ops.rmsnorm_quant(x.reshape(-1, H), self.weight, self.eps, res2, gemma=self.gemma)
        out = QuantizedActivation(xq, sx, x.shape)
        return out if residual is None else (out, new_res.view(x.shape))


class RMSNorm(_NormBase):
    gemma = False


class GemmaRMSNorm(_NormBase):
    gemma = True
