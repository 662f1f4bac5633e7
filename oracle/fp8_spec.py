"""Arithmetic specification of the FP8 (e4m3) W8A8 block-scaled linear path.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Parity unpinned by the
reference: nano_qwen has no quantisation code, so this module restates the
recipe that the benchmark contract gives in words:

* weights ``W[N, K]`` (bf16): one fp32 scale per 128x128 block,
  ``scale = max(amax, 1e-10) / 448``, ``Wq = RNE_e4m3(float(W) / scale)``;
* activations ``x[M, K]`` (bf16): one fp32 scale per token and per 128-wide
  K-group, same formula, computed at run time;
* linear: dequantise both operands to fp32 and apply the reference's matmul,
  ``F.linear`` (nano_qwen ``src/nano_qwen/layers/linear.py:51,73,153``),
  accumulate in fp32, round the result to bf16.

Everything here is plain torch on CPU plus an independent numpy e4m3 encoder
that pins what "RNE_e4m3" means without relying on torch's cast.
Ragged edges: a last K-group / last block that is not full takes its amax over
the elements that exist.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

E4M3_MAX = 448.0
GROUP = 128          # activation group width along K, weight block edge
AMAX_FLOOR = 1e-10   # keeps an all-zero group/block from dividing by zero


# --------------------------------------------------------------------------- #
# e4m3 ("fn": no infinities, 0x7f/0xff are NaN) in numpy, independent of torch #
# --------------------------------------------------------------------------- #
def e4m3_decode_table() -> np.ndarray:
    """All 256 e4m3fn code points as float32 (NaN for 0x7f and 0xff)."""
    out = np.empty(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exp = (code >> 3) & 0xF
        man = code & 0x7
        if exp == 0xF and man == 0x7:
            val = float("nan")
        elif exp == 0:
            val = sign * man * 2.0 ** -9          # subnormals: man/8 * 2^-6
        else:
            val = sign * (1.0 + man / 8.0) * 2.0 ** (exp - 7)
        out[code] = val
    return out


def e4m3_encode_rne(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> e4m3fn code points, saturating at +-448.

    Pure integer/float numpy arithmetic: scales each value to the spacing of
    its binade, rounds with ``np.rint`` (ties to even) and rebuilds the code.
    """
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    a = np.minimum(a, E4M3_MAX)                    # satfinite
    # exponent of the binade, clamped to the subnormal binade (2^-6)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)                          # 3 mantissa bits
    q = np.rint(a / step)                          # ties-to-even, in units of step
    # a mantissa that rounded up to 16 steps moves to the next binade
    bump = q >= 16
    e = np.where(bump, e + 1, e)
    q = np.where(bump, 8, q)
    val = q * 2.0 ** (e - 3)
    val = np.minimum(val, E4M3_MAX)
    # rebuild the code from the rounded value
    is_sub = val < 2.0 ** -6
    man_sub = np.rint(val / 2.0 ** -9).astype(np.int64)
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(val > 0, val, 1.0))).astype(np.int64)
    man_norm = np.rint((val / 2.0 ** e2 - 1.0) * 8).astype(np.int64)
    code = np.where(is_sub, man_sub, ((e2 + 7) << 3) | man_norm).astype(np.uint8)
    return (code | sign).astype(np.uint8)


# --------------------------------------------------------------------------- #
# quantisers                                                                   #
# --------------------------------------------------------------------------- #
def _pad_to(x: torch.Tensor, dim: int, multiple: int) -> torch.Tensor:
    size = x.shape[dim]
    pad = (-size) % multiple
    if pad == 0:
        return x
    shape = list(x.shape)
    shape[dim] = pad
    return torch.cat([x, x.new_zeros(shape)], dim=dim)


def quantize_act_group128(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token 1x128 dynamic activation quantiser.

    ``x``: ``[M, K]`` bf16 (or fp32 holding bf16-representable values).
    Returns ``xq`` ``[M, K]`` float8_e4m3fn and ``sx`` ``[M, ceil(K/128)]`` fp32
    (the dequantisation multiplier).
    """
    assert x.dim() == 2
    M, K = x.shape
    xf = _pad_to(x.float(), 1, GROUP)
    G = xf.shape[1] // GROUP
    g = xf.view(M, G, GROUP)
    amax = g.abs().amax(dim=2)                                   # fp32
    sx = amax.clamp(min=AMAX_FLOOR) / E4M3_MAX                   # IEEE fp32 divide
    q = (g / sx.unsqueeze(2)).to(torch.float8_e4m3fn)            # RNE
    return q.view(M, G * GROUP)[:, :K].contiguous(), sx.contiguous()


def quantize_weight_block128(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Offline 128x128 block weight quantiser.

    ``w``: ``[N, K]`` bf16.  Returns ``wq`` ``[N, K]`` float8_e4m3fn and
    ``sw`` ``[ceil(N/128), ceil(K/128)]`` fp32 (what FP8 checkpoints store as
    ``weight_scale_inv``).
    """
    assert w.dim() == 2
    N, K = w.shape
    wf = _pad_to(_pad_to(w.float(), 0, GROUP), 1, GROUP)
    NB, KB = wf.shape[0] // GROUP, wf.shape[1] // GROUP
    b = wf.view(NB, GROUP, KB, GROUP)
    amax = b.abs().amax(dim=(1, 3))
    sw = amax.clamp(min=AMAX_FLOOR) / E4M3_MAX
    q = (b / sw.view(NB, 1, KB, 1)).to(torch.float8_e4m3fn)
    return q.view(NB * GROUP, KB * GROUP)[:N, :K].contiguous(), sw.contiguous()


def dequantize_act(xq: torch.Tensor, sx: torch.Tensor) -> torch.Tensor:
    M, K = xq.shape
    s = sx.repeat_interleave(GROUP, dim=1)[:, :K]
    return xq.float() * s


def dequantize_weight(wq: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
    N, K = wq.shape
    s = sw.repeat_interleave(GROUP, dim=0)[:N].repeat_interleave(GROUP, dim=1)[:, :K]
    return wq.float() * s


# --------------------------------------------------------------------------- #
# the linear itself                                                            #
# --------------------------------------------------------------------------- #
def linear_dequant_matmul(xq, sx, wq, sw, bias=None) -> torch.Tensor:
    """Dequantise-then-matmul: the parity target (fp32 accumulate, bf16 out).

    The matmul is the reference's, ``F.linear(x, W, b)``
    (nano_qwen ``src/nano_qwen/layers/linear.py:73``), fed fp32 operands.
    """
    y = F.linear(dequantize_act(xq, sx), dequantize_weight(wq, sw),
                 None if bias is None else bias.float())
    return y.to(torch.bfloat16)


def linear_tile_promotion(xq, sx, wq, sw, bias=None) -> torch.Tensor:
    """Same linear evaluated in the order the device kernels use.

    ``y[m,n] = bf16( sum_t sx[m,t]*sw[n//128,t] * (xq[m,tile t] . wq[n,tile t]) + b[n] )``
    with the inner dot product exact in fp32 and the outer sum in fp32.  Used
    for tight (few-ulp) checks; it differs from ``linear_dequant_matmul`` only
    by fp32 summation order.
    """
    M, K = xq.shape
    N = wq.shape[0]
    G = sx.shape[1]
    xf, wf = xq.float(), wq.float()
    acc = torch.zeros(M, N, dtype=torch.float32)
    swn = sw.repeat_interleave(GROUP, dim=0)[:N]                 # [N, G]
    for t in range(G):
        k0, k1 = t * GROUP, min((t + 1) * GROUP, K)
        p = xf[:, k0:k1].double() @ wf[:, k0:k1].double().t()    # exact: |p| < 2^24 * tiny
        acc += (sx[:, t:t + 1] * swn[:, t].unsqueeze(0)) * p.float()
    if bias is not None:
        acc += bias.float()
    return acc.to(torch.bfloat16)


def max_rel_err(y: torch.Tensor, y_ref: torch.Tensor) -> float:
    """The parity metric: ``max|y - y_ref| / max|y_ref|`` over the whole output."""
    yr = y_ref.float()
    denom = yr.abs().max().item()
    if denom == 0.0:
        return (y.float() - yr).abs().max().item()
    return ((y.float() - yr).abs().max() / denom).item()
