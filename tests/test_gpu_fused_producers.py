"""SiluAndMul + quantiser and RMSNorm + quantiser kernels against the oracle and the reference modules' outputs.

Tolerances.  The value that is quantised is a bf16 tensor computed from fp32 intermediates (exp, reciprocal square
root, a sum of squares) whose last bit may differ between the GPU and the CPU evaluation; a different last bit can
move a bf16 result by one unit in the last place, and a group's amax with it.  So:
  * the new residual (one fp32 add, one rounding) must be bit-exact;
  * the bf16 result may differ by one bf16 ulp (2^-8 relative) on at most 0.5 % of the elements;
  * scales within 2^-7 relative; at least 99 % of the e4m3 bytes identical to "oracle op, then oracle quantiser";
  * every dequantised element within the e4m3 rounding bound of the oracle's bf16 value:
    |xq*sx - h| <= max(|h| * 2^-4, sx * 2^-10) * 1.02 + |h| * 2^-7;
  * end to end (producer -> FP8 linear) max|y - y_ref| / max|y_ref| <= 2e-2 against dequantise-then-matmul.
"""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import fp8_spec as S
from oracle import ref_fused as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_library):
    from nano_qwen_b200 import ops
    ops.init()
    return ops


def golden():
    with np.load(os.path.join(GOLDEN, "fused_ops.npz")) as z:
        return {k: torch.from_numpy(z[k].copy()).view(torch.bfloat16) for k in z.files}


def check_quantised(xq, sx, h_ref):
    """xq/sx from the kernel (device tensors) against the oracle's bf16 result h_ref (CPU)."""
    xq, sx = xq.cpu(), sx.cpu().contiguous()
    q_ref, s_ref = S.quantize_act_group128(h_ref)
    assert xq.shape == q_ref.shape and sx.shape == s_ref.shape
    rel = ((sx - s_ref).abs() / s_ref).max().item()
    assert rel <= 2 ** -7, f"scales differ by {rel}"
    same = (xq.view(torch.uint8) == q_ref.view(torch.uint8)).float().mean().item()
    assert same >= 0.99, f"only {same:.4f} of the bytes equal the oracle's"
    K = xq.shape[1]
    scales = sx.repeat_interleave(128, dim=1)[:, :K]
    deq = xq.to(torch.float32) * scales
    h = h_ref.float()
    bound = torch.maximum(h.abs() * 2 ** -4, scales * 2 ** -10) * 1.02 + h.abs() * 2 ** -7
    worst = ((deq - h).abs() - bound).max().item()
    assert worst <= 0, f"dequantised value off by {worst} beyond the rounding bound"
    return same


def check_bf16(y, ref):
    y, ref = y.cpu().float(), ref.float()
    diff = (y - ref).abs()
    assert (diff <= ref.abs() * 2 ** -7 + 1e-30).all(), "more than one bf16 ulp away"
    assert (diff > 0).float().mean().item() <= 5e-3


def test_silu_mul_quant_golden_case(ops):
    g = golden()
    xq, sx = ops.silu_mul_quant(g["silu_in"].cuda())
    torch.cuda.synchronize()
    check_quantised(xq, sx, g["silu_out"])


@pytest.mark.parametrize("m,inter", [(1, 12288), (7, 3072), (64, 12288), (300, 1024), (5, 208), (2048, 3072)])
def test_silu_mul_quant_matches_oracle(ops, m, inter):
    gen = torch.Generator().manual_seed(m + inter)
    x = (torch.randn(m, 2 * inter, generator=gen) * 2.0).to(torch.bfloat16)
    if m > 4:
        x[3] = 0                                             # an all-zero token
        x[4, :inter] = -30.0                                 # silu underflows to -0
    xq, sx = ops.silu_mul_quant(x.cuda())
    torch.cuda.synchronize()
    check_quantised(xq, sx, R.silu_and_mul(x))


@pytest.mark.parametrize("gemma", [False, True])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_quant_golden_cases(ops, gemma, with_res):
    g = golden()
    name = "gemma" if gemma else "rms"
    res = g["norm_res"].cuda() if with_res else None
    xq, sx, new_res, y = ops.rmsnorm_quant(g["norm_x"].cuda(), g[name + "_w"].cuda(), 1e-6, res, gemma=gemma, want_bf16=True)
    torch.cuda.synchronize()
    ref = g[name + ("_add_out" if with_res else "_out")]
    check_quantised(xq, sx, ref)
    check_bf16(y, ref)
    if with_res:
        assert torch.equal(new_res.cpu().view(torch.int16), g[name + "_add_res"].view(torch.int16))
    else:
        assert new_res is None


@pytest.mark.parametrize("m,h", [(1, 4096), (3, 5120), (64, 4096), (257, 1024), (9, 8192), (4, 208), (2, 16384)])
@pytest.mark.parametrize("gemma", [False, True])
def test_rmsnorm_quant_matches_oracle(ops, m, h, gemma):
    gen = torch.Generator().manual_seed(m * 3 + h)
    x = (torch.randn(m, h, generator=gen) * 3.0).to(torch.bfloat16)
    res = torch.randn(m, h, generator=gen).to(torch.bfloat16)
    w = (torch.randn(h, generator=gen) * 0.2 + (0.0 if gemma else 1.0)).to(torch.bfloat16)
    ref, ref_res = R.rms_norm(x, w, 1e-6, res, gemma)
    xq, sx, new_res, y = ops.rmsnorm_quant(x.cuda(), w.cuda(), 1e-6, res.cuda(), gemma=gemma, want_bf16=True)
    torch.cuda.synchronize()
    assert torch.equal(new_res.cpu().view(torch.int16), ref_res.view(torch.int16))
    check_bf16(y, ref)
    check_quantised(xq, sx, ref)


def test_full_size_producers_sampled_rows(ops):
    """Prefill-sized inputs (larger than L2): 48 sampled token rows against the oracle."""
    gen = torch.Generator(device="cuda").manual_seed(31)
    rows = torch.linspace(0, 8191, 48).long()
    gu = (torch.randn(8192, 2 * 12288, generator=gen, device="cuda") * 2.0).to(torch.bfloat16)
    xq, sx = ops.silu_mul_quant(gu)
    torch.cuda.synchronize()
    check_quantised(xq[rows.cuda()], sx[rows.cuda()], R.silu_and_mul(gu[rows.cuda()].cpu()))
    del gu, xq, sx
    x = (torch.randn(8192, 4096, generator=gen, device="cuda") * 3.0).to(torch.bfloat16)
    res = torch.randn(8192, 4096, generator=gen, device="cuda").to(torch.bfloat16)
    w = (torch.randn(4096, generator=gen, device="cuda") * 0.2).to(torch.bfloat16)
    xq, sx, new_res, _ = ops.rmsnorm_quant(x, w, 1e-6, res, gemma=True)
    torch.cuda.synchronize()
    ref, ref_res = R.rms_norm(x[rows.cuda()].cpu(), w.cpu(), 1e-6, res[rows.cuda()].cpu(), gemma=True)
    assert torch.equal(new_res[rows.cuda()].cpu().view(torch.int16), ref_res.view(torch.int16))
    check_quantised(xq[rows.cuda()], sx[rows.cuda()], ref)


def test_rmsnorm_residual_in_place_through_the_c_abi(ops):
    """residual_out may be the residual_in buffer (what the reference's in-place variant does)."""
    from nano_qwen_b200 import _cabi
    m, h = 33, 4096
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(m, h, generator=gen).to(torch.bfloat16)
    res = torch.randn(m, h, generator=gen).to(torch.bfloat16)
    w = torch.ones(h, dtype=torch.bfloat16)
    ref, ref_res = R.rms_norm(x, w, 1e-6, res)
    xd, rd, wd = x.cuda(), res.cuda(), w.cuda()
    xq = torch.empty(m, h, dtype=torch.uint8, device="cuda")
    sx = torch.empty(h // 128, 36, dtype=torch.float32, device="cuda")
    st = _cabi.lib().nq_rmsnorm_quant_e4m3_g128(xd.data_ptr(), rd.data_ptr(), wd.data_ptr(), 1e-6, 0, m, h, h, h,
                                                rd.data_ptr(), None, 0, xq.data_ptr(), h, sx.data_ptr(), 36,
                                                torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert torch.equal(rd.cpu().view(torch.int16), ref_res.view(torch.int16))
    check_quantised(xq.view(torch.float8_e4m3fn), sx[:, :m].t(), ref)


def test_unsupported_layouts_are_refused(ops):
    from nano_qwen_b200._cabi import NqError
    with pytest.raises(NqError):
        ops.silu_mul_quant(torch.zeros(4, 2 * 24, dtype=torch.bfloat16, device="cuda"))      # I not a multiple of 16
    with pytest.raises(NqError):
        ops.rmsnorm_quant(torch.zeros(4, 40, dtype=torch.bfloat16, device="cuda"),
                          torch.ones(40, dtype=torch.bfloat16, device="cuda"), 1e-6)


def test_mlp_block_with_fused_producers_matches_the_oracle_chain(built_library, single_rank_group):
    """post-norm -> gate_up -> SiluAndMul -> down, the reference's MLP (models/qwen3_5.py:152-165), with the fused
    producers in front of both linears, against the same chain evaluated by the oracle."""
    from nano_qwen_b200 import layers as L
    hid, inter, m = 1024, 3072, 48
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(m, hid, generator=gen).to(torch.bfloat16)
    res = torch.randn(m, hid, generator=gen).to(torch.bfloat16)
    wn = (torch.randn(hid, generator=gen) * 0.1).to(torch.bfloat16)
    w1 = (torch.randn(2 * inter, hid, generator=gen) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(hid, inter, generator=gen) * 0.02).to(torch.bfloat16)
    torch.set_default_device("cuda")
    torch.set_default_dtype(torch.bfloat16)
    try:
        norm = L.GemmaRMSNorm(hid, eps=1e-6, emit_fp8=True)
        gate_up = L.MergedColumnParallelLinear(hid, [inter, inter])
        act = L.SiluAndMul()
        down = L.RowParallelLinear(inter, hid)
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)
    norm.weight.data.copy_(wn)
    gate_up.weight.weight_loader(gate_up.weight, w1[:inter], 0)
    gate_up.weight.weight_loader(gate_up.weight, w1[inter:], 1)
    down.weight.weight_loader(down.weight, w2)
    h, new_res = norm(x.cuda(), res.cuda())
    assert isinstance(h, L.QuantizedActivation)
    y = down(act(gate_up(h)))
    torch.cuda.synchronize()
    # oracle chain: every linear = quantise input, dequantise both operands, fp32 matmul, bf16 out
    def lin(a, w):
        aq, sa = S.quantize_act_group128(a)
        wq, sw = S.quantize_weight_block128(w)
        return S.linear_dequant_matmul(aq, sa, wq, sw, None)
    h_ref, res_ref = R.rms_norm(x, wn, 1e-6, res, gemma=True)
    y_ref = lin(R.silu_and_mul(lin(h_ref, w1)), w2)
    assert torch.equal(new_res.cpu().view(torch.int16), res_ref.view(torch.int16))
    assert S.max_rel_err(y.cpu(), y_ref) <= 2e-2
