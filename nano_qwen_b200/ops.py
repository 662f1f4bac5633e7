"""Functional host API over the C ABI (``include/nq_fp8.h``).

Tensors must live on the current CUDA device; all work is enqueued on
``torch.cuda.current_stream()`` without host synchronisation, so these calls
can be captured in a CUDA graph (call :func:`init` once before capturing).
There is no CPU path: a CPU tensor raises.
"""
from __future__ import annotations

import torch

from . import _cabi
from ._cabi import (ALGO_AUTO, ALGO_TOKEN_LANE, ALGO_TOKEN_LANE_128, ALGO_TOKEN_LANE_192,  # noqa: F401  (re-exported)
                    ALGO_TOKEN_LANE_256, ALGO_TOKEN_PAIR, ALGO_TOKEN_PAIR_128, ALGO_WEIGHT_LANE,
                    ALGO_WEIGHT_LANE_FUSED)

GROUP = 128
FP8 = torch.float8_e4m3fn


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("nano_qwen_b200 runs on CUDA (sm_100a) tensors only; got a "
                               f"{t.device.type} tensor and there is no CPU fallback")


def init() -> None:
    """Per-device set-up of the native library for the current device."""
    _cabi.check(_cabi.lib().nq_init(), "nq_init")


def set_sm_reserve(n: int) -> int:
    """SMs the persistent GEMM leaves free for a kernel running beside it (a collective); returns the old value."""
    old = _cabi.lib().nq_set_sm_reserve(int(n))
    if old < 0:
        _cabi.check(old, "nq_set_sm_reserve")
    return old


def launch_count() -> int:
    return int(_cabi.lib().nq_launch_count())


def act_quant(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Dynamic per-token 1x128 quantiser.

    ``x``: ``[M, K]`` bf16, unit stride along K.  Returns ``xq`` ``[M, K]``
    (float8_e4m3fn, row stride = K rounded up to 16 bytes) and ``sx``
    ``[M, ceil(K/128)]`` fp32 stored K-group major (``sx.stride() == (1, ld)``).
    """
    _require_cuda(x)
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise TypeError("act_quant expects a 2-D bfloat16 tensor")
    if x.stride(1) != 1 and x.shape[1] > 1:
        x = x.contiguous()
    M, K = x.shape
    G = (K + GROUP - 1) // GROUP
    ld_xq = _round_up(max(K, 1), 16)
    ld_sx = _round_up(max(M, 1), 4)
    xq_buf = torch.empty((M, ld_xq), dtype=FP8, device=x.device)
    sx_buf = torch.empty((G, ld_sx), dtype=torch.float32, device=x.device)
    if M > 0 and K > 0:
        st = _cabi.lib().nq_act_quant_e4m3_g128(x.data_ptr(), M, K, x.stride(0) if M > 1 else max(K, x.stride(0)),
                                                xq_buf.data_ptr(), ld_xq, sx_buf.data_ptr(), ld_sx, _stream())
        _cabi.check(st, "nq_act_quant_e4m3_g128")
    return xq_buf[:, :K], sx_buf[:, :M].t()


def weight_quant(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Offline 128x128 block quantiser: bf16 ``[N, K]`` -> (e4m3 ``[N, K]``, fp32 ``[ceil(N/128), ceil(K/128)]``)."""
    _require_cuda(w)
    if w.dtype != torch.bfloat16 or w.dim() != 2:
        raise TypeError("weight_quant expects a 2-D bfloat16 tensor")
    w = w.contiguous()
    N, K = w.shape
    ld_wq = _round_up(max(K, 1), 16)
    wq_buf = torch.empty((N, ld_wq), dtype=FP8, device=w.device)
    sw = torch.empty(((N + GROUP - 1) // GROUP, (K + GROUP - 1) // GROUP), dtype=torch.float32, device=w.device)
    if N > 0 and K > 0:
        st = _cabi.lib().nq_weight_quant_e4m3_b128(w.data_ptr(), N, K, K, wq_buf.data_ptr(), ld_wq,
                                                   sw.data_ptr(), sw.stride(0), _stream())
        _cabi.check(st, "nq_weight_quant_e4m3_b128")
    return wq_buf[:, :K], sw


def fp8_gemm(xq: torch.Tensor, sx: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor,
             bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
             algo: int = ALGO_AUTO, split_k: int = 0) -> torch.Tensor:
    """Block-scaled FP8 GEMM ``y = (xq*sx) @ (wq*sw)^T + bias`` -> bf16 ``[M, N]``.

    ``xq`` ``[M,K]`` / ``wq`` ``[N,K]`` e4m3 with unit stride along K and row
    strides that are multiples of 16; ``sx`` ``[M, G]`` K-group major as
    returned by :func:`act_quant`; ``sw`` ``[ceil(N/128), G]`` row-major.
    """
    _require_cuda(xq, sx, wq, sw, bias, out)
    M, K = xq.shape
    N = wq.shape[0]
    if wq.shape[1] != K:
        raise ValueError(f"K mismatch: xq {tuple(xq.shape)} vs wq {tuple(wq.shape)}")
    if K > 1 and (xq.stride(1) != 1 or wq.stride(1) != 1):
        raise ValueError("xq and wq need unit stride along K")
    if M > 1 and sx.stride(0) != 1:
        sx = sx.t().contiguous().t()     # make it K-group major
    if sw.dim() != 2 or (sw.shape[1] > 1 and sw.stride(1) != 1):
        sw = sw.contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    if M == 0 or N == 0:
        return out
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_contiguous()):
        bias = bias.to(torch.bfloat16).contiguous()
    G = (K + GROUP - 1) // GROUP
    ld_xq = xq.stride(0) if M > 1 else _round_up(K, 16)
    ld_sx = sx.stride(1) if G > 1 else _round_up(M, 4)
    st = _cabi.lib().nq_fp8_gemm_bs128(
        xq.data_ptr(), ld_xq, sx.data_ptr(), ld_sx,
        wq.data_ptr(), wq.stride(0) if N > 1 else _round_up(K, 16), sw.data_ptr(), sw.stride(0) if sw.shape[0] > 1 else G,
        bias.data_ptr() if bias is not None else None, out.data_ptr(), out.stride(0) if M > 1 else N,
        M, N, K, None, 0, algo, split_k, _stream())
    _cabi.check(st, "nq_fp8_gemm_bs128")
    return out


def fp8_linear(x: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, bias: torch.Tensor | None = None,
               algo: int = ALGO_AUTO, split_k: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear`` with FP8 weights: quantise ``x`` on the fly, then the FP8 GEMM.

    Accepts any leading dimensions, like ``F.linear``; returns bf16.  ``out``, if given, is a
    row-contiguous bf16 ``[tokens, N]`` tensor (rows may be a slice of a larger buffer).
    """
    _require_cuda(x, wq, sw, bias)
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    lead = x.shape[:-1]
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if K > 1 and x2.stride(1) != 1:
        x2 = x2.contiguous()
    M, N = x2.shape[0], wq.shape[0]
    if wq.shape[1] != K:
        raise ValueError(f"K mismatch: x {tuple(x.shape)} vs wq {tuple(wq.shape)}")
    if K > 1 and wq.stride(1) != 1:
        raise ValueError("wq needs unit stride along K")
    if sw.dim() != 2 or (sw.shape[1] > 1 and sw.stride(1) != 1):
        sw = sw.contiguous()
    if out is None:
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    else:
        if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N) or (N > 1 and out.stride(1) != 1):
            raise ValueError("out must be a bf16 [tokens, N] tensor with unit stride along N")
        y = out
    if M == 0 or N == 0:
        return y if out is not None else y.view(*lead, N)
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_contiguous()):
        bias = bias.to(torch.bfloat16).contiguous()
    G = (K + GROUP - 1) // GROUP
    ldx = x2.stride(0) if M > 1 else max(K, x2.stride(0))
    # Decode batches that the library quantises inside the GEMM kernel need no scratch (same rule as the library's;
    # if the two ever disagreed the call would be rejected for its null scratch, not miscomputed).
    limit = {ALGO_AUTO: _cabi.FUSED_AUTO_TOKENS, ALGO_WEIGHT_LANE_FUSED: _cabi.FUSED_MAX_TOKENS}.get(algo, 0)
    fused = M <= limit and K % 8 == 0 and ldx % 8 == 0 and x2.data_ptr() % 16 == 0
    xq = None if fused else torch.empty((M, _round_up(K, 16)), dtype=FP8, device=x.device)
    sx = None if fused else torch.empty((G, _round_up(M, 4)), dtype=torch.float32, device=x.device)
    st = _cabi.lib().nq_fp8_linear(
        x2.data_ptr(), ldx,
        wq.data_ptr(), wq.stride(0) if N > 1 else _round_up(K, 16), sw.data_ptr(), sw.stride(0) if sw.shape[0] > 1 else G,
        bias.data_ptr() if bias is not None else None, y.data_ptr(), y.stride(0) if M > 1 else N, M, N, K,
        None if fused else xq.data_ptr(), None if fused else sx.data_ptr(), None, 0, algo, split_k, _stream())
    _cabi.check(st, "nq_fp8_linear")
    return y if out is not None else y.view(*lead, N)
