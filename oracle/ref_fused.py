"""CPU restatement of the two producers of linear-layer inputs (TEST INFRASTRUCTURE: only tests, the smoke check
and the bench's CPU arm may import this).

Follows the reference's *eager* arithmetic, i.e. every intermediate that the Python code materialises as a bf16 tensor
is rounded to bf16 here too:

* ``silu_and_mul``  — ``nano_qwen/layers/activation.py:8-11``: ``F.silu(gate) * up`` on bf16 tensors.
* ``rms_norm``      — ``nano_qwen/layers/layernorm.py:16-40`` (RMSNorm) and ``:79-105`` (GemmaRMSNorm, ``1 + weight``):
  fp32 add of the residual, new residual = bf16 of the sum, fp32 mean of squares, ``rsqrt``, result cast to bf16 and
  multiplied by the bf16 weight.

The reference decorates these functions with ``torch.compile``; a fused evaluation may skip an intermediate rounding,
which moves a result by at most one bf16 unit in the last place.  The fixtures in ``tests/golden/fused_ops.npz`` were
produced by the reference's own modules with the compiler switched off.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    gate, up = x.chunk(2, -1)
    return F.silu(gate) * up


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
             gemma: bool = False):
    orig = x.dtype
    v = x.float()
    if residual is not None:
        v = v + residual.float()
        residual = v.to(orig)
    var = v.pow(2).mean(dim=-1, keepdim=True)
    n = (v * torch.rsqrt(var + eps)).to(orig)
    out = n * (1.0 + weight) if gemma else n * weight
    return out if residual is None else (out, residual)
