"""Decode path with the activation quantiser inside the GEMM kernel (NQ_ALGO_WEIGHT_LANE_FUSED), through the C ABI.

The fused kernel must reproduce the two-launch path (quantiser kernel, then weight-lane GEMM) bit for bit: the
quantiser arithmetic is the same, the K-tiles are accumulated in the same order with the same split.  It is also
held to the oracle directly, with the tolerances of the GEMM tests.
"""
import pytest
import torch

from oracle import fp8_spec as S

pytestmark = pytest.mark.gpu

TIGHT = 8e-3
PARITY = 2e-2


@pytest.fixture(scope="module")
def ops(built_library):
    from nano_qwen_b200 import ops
    ops.init()
    return ops


def make(m, n, k, seed, bias, outliers=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    if outliers:                       # heavy-tailed rows, a zero row and a tiny row: exercises scale clamping
        x = x * torch.exp(2.0 * torch.randn(m, 1, generator=g))
        x[0] = 0.0
        if m > 1:
            x[m - 1] *= 1e-30
    x = x.to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    b = torch.randn(n, generator=g).to(torch.bfloat16) if bias else None
    wq, sw = S.quantize_weight_block128(w)
    return x, wq, sw, b


def both(ops, x, wq, sw, b, split_k=0):
    xd, wd, sd = x.cuda(), wq.cuda(), sw.cuda()
    bd = None if b is None else b.cuda()
    two = ops.fp8_linear(xd, wd, sd, bd, algo=ops.ALGO_WEIGHT_LANE, split_k=split_k)
    one = ops.fp8_linear(xd, wd, sd, bd, algo=ops.ALGO_WEIGHT_LANE_FUSED, split_k=split_k)
    torch.cuda.synchronize()
    return one.cpu(), two.cpu()


def check_oracle(y, x, wq, sw, b):
    xq, sx = S.quantize_act_group128(x)
    case = (xq, sx, wq, sw, b)
    e1 = S.max_rel_err(y, S.linear_tile_promotion(*case))
    e2 = S.max_rel_err(y, S.linear_dequant_matmul(*case))
    assert e1 <= TIGHT, f"vs tile-promotion oracle: {e1}"
    assert e2 <= PARITY, f"vs dequantise-then-matmul: {e2}"


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 24, 31, 32])
@pytest.mark.parametrize("n,k", [(1024, 1024), (200, 320), (4096, 512), (384, 2048 + 64), (128, 144)])
def test_fused_equals_two_launch_path_and_oracle(ops, m, n, k):
    x, wq, sw, b = make(m, n, k, seed=m * 7 + n, bias=(m % 2 == 1))
    one, two = both(ops, x, wq, sw, b)
    assert torch.equal(one, two)
    check_oracle(one, x, wq, sw, b)


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("m", [1, 5, 32])
def test_fused_split_k(ops, split, m):
    x, wq, sw, b = make(m, 512, 4096, seed=split + m, bias=True)
    one, two = both(ops, x, wq, sw, b, split_k=split)
    assert torch.equal(one, two)
    check_oracle(one, x, wq, sw, b)


@pytest.mark.parametrize("m", [1, 2, 9, 32])
def test_fused_outlier_rows_and_zero_rows(ops, m):
    x, wq, sw, b = make(m, 768, 1536, seed=m, bias=False, outliers=True)
    one, two = both(ops, x, wq, sw, b)
    assert torch.equal(one, two)
    assert torch.all(one[0] == 0)
    check_oracle(one, x, wq, sw, b)


def test_fused_on_request_is_one_launch_and_auto_is_two_with_the_same_bits(ops):
    """NQ_ALGO_AUTO keeps quantiser and GEMM as two launches at every batch size (the GEMM's set-up overlaps the
    quantiser through programmatic dependent launch, which measured faster); the one-launch kernel stays selectable."""
    T = 8
    x, wq, sw, b = make(T, 1024, 1024, seed=1, bias=False)
    xd, wd, sd = x.cuda(), wq.cuda(), sw.cuda()
    n0 = ops.launch_count()
    y_fused = ops.fp8_linear(xd, wd, sd, algo=ops.ALGO_WEIGHT_LANE_FUSED)
    n1 = ops.launch_count()
    assert n1 - n0 == 1
    y_auto = ops.fp8_linear(xd, wd, sd)
    assert ops.launch_count() - n1 == 2
    torch.cuda.synchronize()
    assert torch.equal(y_auto.cpu(), y_fused.cpu())


def test_strided_rows_and_guarded_output(ops):
    m, n, k = 27, 640, 1024
    x, wq, sw, b = make(m, n, k, seed=3, bias=True)
    wide = torch.full((m, k + 64), 9.0, dtype=torch.bfloat16, device="cuda")
    wide[:, 8:8 + k] = x.cuda()
    xv = wide[:, 8:8 + k]                                     # row stride k+64, 16-byte aligned start
    buf = torch.full((m + 4, n + 8), -777.0, dtype=torch.bfloat16, device="cuda")
    out = buf[2:2 + m, :n]
    ops.fp8_linear(xv, wq.cuda(), sw.cuda(), b.cuda(), algo=ops.ALGO_WEIGHT_LANE_FUSED, out=out)
    ref = ops.fp8_linear(x.cuda(), wq.cuda(), sw.cuda(), b.cuda(), algo=ops.ALGO_WEIGHT_LANE)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    assert torch.all(buf[:2] == -777.0) and torch.all(buf[2 + m:] == -777.0) and torch.all(buf[:, n:] == -777.0)


def test_ineligible_inputs_fall_back_or_are_rejected(ops):
    from nano_qwen_b200._cabi import NqError
    # K not a multiple of 8: AUTO uses the two-launch path, the explicit request is refused
    x, wq, sw, b = make(8, 256, 324, seed=5, bias=False)
    pad = torch.zeros(256, 336, dtype=torch.uint8, device="cuda")     # weight rows need a 16-byte stride
    pad[:, :324] = wq.view(torch.uint8).cuda()
    xd, wd, sd = x.cuda(), pad.view(torch.float8_e4m3fn)[:, :324], sw.cuda()
    n0 = ops.launch_count()
    y = ops.fp8_linear(xd, wd, sd)
    assert ops.launch_count() - n0 == 2
    torch.cuda.synchronize()
    check_oracle(y.cpu(), x, wq, sw, b)
    with pytest.raises(NqError):
        ops.fp8_linear(xd, wd, sd, algo=ops.ALGO_WEIGHT_LANE_FUSED)
    # more tokens than the fused kernel takes
    x, wq, sw, b = make(33, 256, 512, seed=6, bias=False)
    with pytest.raises(NqError):
        ops.fp8_linear(x.cuda(), wq.cuda(), sw.cuda(), algo=ops.ALGO_WEIGHT_LANE_FUSED)
    # rows that start 2 bytes off a 16-byte boundary
    x, wq, sw, b = make(4, 256, 512, seed=7, bias=False)
    wide = torch.zeros(4, 520, dtype=torch.bfloat16, device="cuda")           # M = 4: AUTO would fuse if it could
    wide[:, 1:513] = x.cuda()
    n0 = ops.launch_count()
    y = ops.fp8_linear(wide[:, 1:513], wq.cuda(), sw.cuda())
    assert ops.launch_count() - n0 == 2
    torch.cuda.synchronize()
    check_oracle(y.cpu(), x, wq, sw, b)


def test_status_block_clean_after_fused_runs(ops):
    from nano_qwen_b200 import _cabi
    torch.cuda.synchronize()
    assert _cabi.device_status()["code"] == 0
