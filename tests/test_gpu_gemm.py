"""Block-scaled FP8 GEMM kernels vs the oracle (through the C ABI).

Tolerances: against the oracle evaluated in the kernels' own order
(``linear_tile_promotion``) the result may differ by fp32 summation order
inside a K-tile and one bf16 rounding flip (one bf16 ulp of the largest
element is 2^-7 of it): max|d|/max|ref| <= 8e-3.  Against the
parity target proper, dequantise-then-matmul: <= 2e-2 (the contract's bound).
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


def make_case(m, n, k, seed=0, bias=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    b = torch.randn(n, generator=g).to(torch.bfloat16) if bias else None
    xq, sx = S.quantize_act_group128(x)
    wq, sw = S.quantize_weight_block128(w)
    return xq, sx, wq, sw, b


def run_gemm(ops, case, algo, split_k=0, guard=2):
    """Runs the kernel into a buffer with sentinel guard rows/columns and checks they stay untouched."""
    xq, sx, wq, sw, b = case
    m, n = xq.shape[0], wq.shape[0]
    ldy = (n + 8 + 7) // 8 * 8
    buf = torch.full((m + 2 * guard, ldy), -777.0, dtype=torch.bfloat16, device="cuda")
    out = buf[guard:guard + m, :n]
    k = xq.shape[1]
    kp = (k + 15) // 16 * 16
    xq_d = torch.zeros(m, kp, dtype=torch.uint8, device="cuda")
    xq_d[:, :k] = xq.view(torch.uint8).cuda()
    wq_d = torch.zeros(n, kp, dtype=torch.uint8, device="cuda")
    wq_d[:, :k] = wq.view(torch.uint8).cuda()
    y = ops.fp8_gemm(xq_d.view(torch.float8_e4m3fn)[:, :k], sx.cuda(), wq_d.view(torch.float8_e4m3fn)[:, :k], sw.cuda(),
                     None if b is None else b.cuda(), out=out, algo=algo, split_k=split_k)
    torch.cuda.synchronize()
    assert y.data_ptr() == out.data_ptr()
    assert torch.all(buf[:guard] == -777.0) and torch.all(buf[guard + m:] == -777.0), "wrote outside the rows of y"
    assert torch.all(buf[:, n:] == -777.0), "wrote outside the columns of y"
    return out.cpu().clone()


def check(y, case):
    ref_tight = S.linear_tile_promotion(*case)
    ref = S.linear_dequant_matmul(*case)
    e1, e2 = S.max_rel_err(y, ref_tight), S.max_rel_err(y, ref)
    assert e1 <= TIGHT, f"vs tile-promotion oracle: {e1}"
    assert e2 <= PARITY, f"vs dequantise-then-matmul: {e2}"


SHAPES_SMALL = [(128, 128), (256, 512), (1024, 1024), (4096, 1024), (384, 2048), (200, 320), (136, 144), (128, 4096 + 128)]


@pytest.mark.parametrize("m", [1, 7, 8, 16, 17, 63, 64, 65, 128, 200, 256, 300])
@pytest.mark.parametrize("n,k", [(1024, 1024), (200, 320), (4096, 512)])
def test_weight_lane_matches_oracle(ops, m, n, k):
    case = make_case(m, n, k, seed=m + n, bias=(m % 2 == 0))
    check(run_gemm(ops, case, ops.ALGO_WEIGHT_LANE), case)


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("m", [3, 16, 24, 64, 130])
def test_weight_lane_split_k(ops, split, m):
    case = make_case(m, 512, 2048, seed=split, bias=True)
    check(run_gemm(ops, case, ops.ALGO_WEIGHT_LANE, split_k=split), case)


@pytest.mark.parametrize("m", [1, 16, 100, 128, 129, 256, 640, 1000])
@pytest.mark.parametrize("n,k", SHAPES_SMALL)
def test_token_lane_matches_oracle(ops, m, n, k):
    if m > 300 and n * k > 2 ** 21:
        pytest.skip("oracle time")
    case = make_case(m, n, k, seed=m * 3 + n, bias=(m % 2 == 1))
    check(run_gemm(ops, case, ops.ALGO_TOKEN_LANE), case)


@pytest.mark.parametrize("width", ["128", "192", "256"])
@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (130, 200, 320), (256, 1024, 1024), (300, 576, 2048), (129, 4096 + 128, 128)])
def test_token_lane_every_tile_width(ops, width, m, n, k):
    algo = getattr(ops, "ALGO_TOKEN_LANE_" + width)
    case = make_case(m, n, k, seed=m + n + int(width), bias=True)
    check(run_gemm(ops, case, algo), case)


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (1, 128, 256), (130, 200, 320), (256, 512, 512), (300, 520, 1024),
                                   (1000, 1024, 1024), (2304, 4352, 384), (640, 4096 + 128, 256)])
@pytest.mark.parametrize("algo", ["ALGO_TOKEN_PAIR"])
def test_token_pair_matches_oracle(ops, m, n, k, algo):
    """256x256 tiles computed by CTA pairs (UMMAs spanning two SMs, half a K-tile per accumulator slot)."""
    case = make_case(m, n, k, seed=m + n + k, bias=(m % 2 == 0))
    check(run_gemm(ops, case, getattr(ops, algo)), case)


@pytest.mark.parametrize("width", ["128", "192", "256"])
@pytest.mark.parametrize("split", [2, 3, 5, 8])
def test_token_lane_split_k_over_a_cluster(ops, width, split):
    """Few tiles: K is split over a cluster of CTAs and the partial tiles are summed through distributed shared memory."""
    case = make_case(200, 520, 2048 + 128, seed=split, bias=True)      # 17 K-tiles: uneven split
    check(run_gemm(ops, case, getattr(ops, "ALGO_TOKEN_LANE_" + width), split_k=split), case)


def test_token_lane_auto_split_for_mid_sized_batches(ops):
    case = make_case(256, 1024, 4096, seed=21, bias=True)
    a = run_gemm(ops, case, ops.ALGO_TOKEN_LANE)
    check(a, case)
    assert torch.equal(a.view(torch.int16), run_gemm(ops, case, ops.ALGO_TOKEN_LANE).view(torch.int16))


@pytest.mark.parametrize("width", ["128", "192", "256"])
def test_token_lane_many_tiles_persistent_loop(ops, width):
    """More output tiles than SMs: every CTA walks several tiles and ring phases wrap many times."""
    case = make_case(2304, 4352, 384, seed=11, bias=True)       # 18 x 17 tiles of 128x256 = 306 > 148
    check(run_gemm(ops, case, getattr(ops, "ALGO_TOKEN_LANE_" + width)), case)


def test_known_answers_exact(ops):
    """All-ones operands with unit scales: every output is exactly K (and K + bias)."""
    for algo, m in ((ops.ALGO_TOKEN_LANE, 130), (ops.ALGO_WEIGHT_LANE, 20), (ops.ALGO_TOKEN_PAIR, 300)):
        n, k = 384, 1024
        one = torch.full((1,), 1.0).to(torch.float8_e4m3fn)
        xq = one.expand(m, k).contiguous()
        wq = one.expand(n, k).contiguous()
        sx = torch.ones(m, k // 128)
        sw = torch.ones(n // 128, k // 128)
        y = run_gemm(ops, (xq, sx, wq, sw, None), algo)
        assert torch.all(y.float() == float(k))
        # per-tile scales: tile t weighted by 2^-t on the token side, block (bn, t) by (bn+1) on the weight side
        sx2 = (2.0 ** -torch.arange(k // 128, dtype=torch.float32)).expand(m, -1).contiguous()
        sw2 = torch.arange(1, n // 128 + 1, dtype=torch.float32).unsqueeze(1).expand(-1, k // 128).contiguous()
        y = run_gemm(ops, (xq, sx2, wq, sw2, None), algo)
        expect = (128.0 * sx2[0].sum()) * sw2[:, 0].repeat_interleave(128)
        assert torch.equal(y.float(), expect.to(torch.bfloat16).float().expand(m, -1))
        # a single non-zero element per operand row picks out one product
        xq3 = torch.zeros(m, k).to(torch.float8_e4m3fn)
        wq3 = torch.zeros(n, k).to(torch.float8_e4m3fn)
        xq3.view(torch.uint8)[:, 257] = torch.tensor(2.0).to(torch.float8_e4m3fn).view(torch.uint8)
        wq3.view(torch.uint8)[:, 257] = torch.tensor(-3.0).to(torch.float8_e4m3fn).view(torch.uint8)
        y = run_gemm(ops, (xq3, sx, wq3, sw, None), algo)
        assert torch.all(y.float() == -6.0)



def test_auto_dispatch_on_seeded_random_shapes(ops):
    """NQ_ALGO_AUTO picks kernel, tile width and K split from the shape: 40 seeded shapes across those boundaries."""
    import random
    rng = random.Random(20240607)
    for i in range(40):
        m = rng.choice([1, 5, 33, 64, 65, 100, 128, 129, 200, 256, 257, 384, 500, 600])
        n = rng.choice([8, 72, 128, 136, 256, 520, 1024, 1536, 2048])
        k = rng.choice([16, 128, 144, 512, 1024, 2048])
        case = make_case(m, n, k, seed=1000 + i, bias=bool(i & 1))
        check(run_gemm(ops, case, ops.ALGO_AUTO), case)


def test_auto_takes_cta_pairs_for_prefill_sizes_with_ragged_edges(ops):
    """Prefill-sized launches (>= 2048 tokens and at least one 256 x 256 tile per SM) run on CTA pairs under
    NQ_ALGO_AUTO: ragged M and N, a K that is not a multiple of 128, bias; also with SMs held back for a neighbour."""
    case = make_case(2048 + 75, 4096 + 136, 640 + 16, seed=77, bias=True)       # 9 x 17 tiles of 256 x 256 = 153 >= 148
    a = run_gemm(ops, case, ops.ALGO_AUTO)
    check(a, case)
    assert torch.equal(a.view(torch.int16), run_gemm(ops, case, ops.ALGO_TOKEN_PAIR).view(torch.int16))
    old = ops.set_sm_reserve(20)
    try:
        b = run_gemm(ops, case, ops.ALGO_AUTO)
    finally:
        ops.set_sm_reserve(old)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))              # the grid size does not change the sums


def test_results_are_deterministic(ops):
    case = make_case(48, 1024, 4096, seed=5)
    a = run_gemm(ops, case, ops.ALGO_WEIGHT_LANE, split_k=4)
    b = run_gemm(ops, case, ops.ALGO_WEIGHT_LANE, split_k=4)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    case = make_case(512, 1024, 1024, seed=6)
    a = run_gemm(ops, case, ops.ALGO_TOKEN_LANE)
    b = run_gemm(ops, case, ops.ALGO_TOKEN_LANE)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_bad_arguments_are_rejected_not_computed(ops):
    from nano_qwen_b200 import _cabi
    lib = _cabi.lib()
    x = torch.zeros(16, 128, dtype=torch.uint8, device="cuda")
    s = torch.ones(4, 16, device="cuda")
    y = torch.zeros(16, 128, dtype=torch.bfloat16, device="cuda")
    st = lib.nq_fp8_gemm_bs128(x.data_ptr() + 1, 128, s.data_ptr(), 16, x.data_ptr(), 128, s.data_ptr(), 1,
                               None, y.data_ptr(), 128, 16, 16, 128, None, 0, 0, 0, None)
    assert st == -1
    st = lib.nq_fp8_gemm_bs128(x.data_ptr(), 100, s.data_ptr(), 16, x.data_ptr(), 128, s.data_ptr(), 1,
                               None, y.data_ptr(), 128, 16, 16, 128, None, 0, 0, 0, None)
    assert st == -1
    st = lib.nq_fp8_gemm_bs128(None, 128, s.data_ptr(), 16, x.data_ptr(), 128, s.data_ptr(), 1,
                               None, y.data_ptr(), 128, 16, 16, 128, None, 0, 0, 0, None)
    assert st == -1
    assert lib.nq_fp8_gemm_bs128(x.data_ptr(), 128, s.data_ptr(), 16, x.data_ptr(), 128, s.data_ptr(), 1,
                                 None, y.data_ptr(), 128, 0, 16, 128, None, 0, 0, 0, None) == 0   # M = 0: nothing to do


def test_status_block_clean_after_all_gemms(ops):
    from nano_qwen_b200 import _cabi
    torch.cuda.synchronize()
    assert _cabi.device_status()["code"] == 0
