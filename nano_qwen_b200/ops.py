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
                    ALGO_TOKEN_LANE_256, ALGO_TOKEN_PAIR, ALGO_WEIGHT_LANE,
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


def check_device_status(reset: bool = True) -> None:
    """Raises :class:`_cabi.NqError` if a bounded device-side wait ran out since the last check.

    The kernels never trap: a wait that expires (a peer of the row-parallel sum that never arrived, a pipeline
    barrier that was never signalled) lets its kernel finish with an incomplete result and records the fact in a
    status block.  Call this where the host synchronises anyway (after a step's outputs were read); it does not
    synchronise itself.  ``reset`` clears the block so that the next check reports only new events.
    """
    st = _cabi.device_status()
    if st["code"] != 0:
        if reset:
            _cabi.device_status(reset=True)
        raise _cabi.NqError(st["code"], "device status",
                            f"{_cabi.lib().nq_status_string(st['code']).decode()}: wait site {st['where']}, "
                            f"block {st['block']}, aux {st['aux']}")


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


def _quant_buffers(M: int, K: int, device) -> tuple[torch.Tensor, torch.Tensor, int, int]:
    G = (K + GROUP - 1) // GROUP
    ld_xq = _round_up(max(K, 1), 16)
    ld_sx = _round_up(max(M, 1), 4)
    return (torch.empty((M, ld_xq), dtype=FP8, device=device), torch.empty((G, ld_sx), dtype=torch.float32, device=device),
            ld_xq, ld_sx)


def silu_mul_quant(gate_up: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``silu(gate) * up`` of a ``[M, 2*I]`` bf16 tensor (gate first), emitted as FP8 + 1x128 group scales.

    Stands in for the reference's ``SiluAndMul.forward`` (``layers/activation.py:8-11``) followed by the activation
    quantiser of the next linear layer.  Returns ``(xq, sx)`` laid out like :func:`act_quant`'s.
    """
    _require_cuda(gate_up)
    if gate_up.dtype != torch.bfloat16 or gate_up.dim() != 2 or gate_up.shape[1] % 2:
        raise TypeError("silu_mul_quant expects a 2-D bfloat16 tensor with an even number of columns")
    if gate_up.stride(1) != 1:
        gate_up = gate_up.contiguous()
    M, I = gate_up.shape[0], gate_up.shape[1] // 2
    xq_buf, sx_buf, ld_xq, ld_sx = _quant_buffers(M, I, gate_up.device)
    if M > 0 and I > 0:
        st = _cabi.lib().nq_silu_mul_quant_e4m3_g128(gate_up.data_ptr(), M, I, gate_up.stride(0) if M > 1 else 2 * I,
                                                     xq_buf.data_ptr(), ld_xq, sx_buf.data_ptr(), ld_sx, _stream())
        _cabi.check(st, "nq_silu_mul_quant_e4m3_g128")
    return xq_buf[:, :I], sx_buf[:, :M].t()


def rmsnorm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                  gemma: bool = False, want_bf16: bool = False):
    """RMS norm of ``[M, H]`` bf16 rows (optionally after adding ``residual``), emitted as FP8 + group scales.

    Stands in for ``RMSNorm.forward`` / ``GemmaRMSNorm.forward`` (``layers/layernorm.py:16-56``, ``:79-120``) followed
    by the activation quantiser.  Returns ``(xq, sx, new_residual_or_None, bf16_result_or_None)``.
    """
    _require_cuda(x, weight, residual)
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise TypeError("rmsnorm_quant expects a 2-D bfloat16 tensor")
    if x.stride(1) != 1:
        x = x.contiguous()
    M, H = x.shape
    if weight.dtype != torch.bfloat16 or weight.numel() != H:
        weight = weight.to(torch.bfloat16)
    weight = weight.contiguous()
    res_out = None
    if residual is not None:
        if residual.dtype != torch.bfloat16 or residual.shape != x.shape:
            raise TypeError("residual must be bfloat16 with the shape of x")
        if residual.stride(1) != 1:
            residual = residual.contiguous()
        res_out = torch.empty((M, H), dtype=torch.bfloat16, device=x.device)
    y = torch.empty((M, H), dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    xq_buf, sx_buf, ld_xq, ld_sx = _quant_buffers(M, H, x.device)
    if M > 0 and H > 0:
        st = _cabi.lib().nq_rmsnorm_quant_e4m3_g128(
            x.data_ptr(), residual.data_ptr() if residual is not None else None, weight.data_ptr(), float(eps),
            int(bool(gemma)), M, H, x.stride(0) if M > 1 else H,
            (residual.stride(0) if M > 1 else H) if residual is not None else 0,
            res_out.data_ptr() if res_out is not None else None, y.data_ptr() if y is not None else None, H,
            xq_buf.data_ptr(), ld_xq, sx_buf.data_ptr(), ld_sx, _stream())
        _cabi.check(st, "nq_rmsnorm_quant_e4m3_g128")
    return xq_buf[:, :H], sx_buf[:, :M].t(), res_out, y


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
