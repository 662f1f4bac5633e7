"""Every shape of the benchmark contract against the oracle, on one GPU.

Covers what the small-shape GEMM tests do not reach: the Qwen3-32B-shaped layers, the per-rank shard shapes of
the 8B- and 32B-shaped stacks at tensor-parallel degrees 2, 4 and 8 (each shard is a plain one-GPU GEMM: the
oracle's operands are sliced with ``oracle/ref_linear.py``'s ``column_shard`` / ``row_shard``, which restate
nano_qwen ``layers/linear.py:65-70,142-150``), a 16 384-token prefill, and the module API paths the stack tests
leave out (``ReplicatedLinear``, a biased ``RowParallelLinear``).

The oracle dequantises to fp32 on the CPU, so it is evaluated on sampled token rows and sampled 128-row
weight blocks (first, last and some in between); the kernel always computes the full product.
Tolerance: max|y - ref| / max|ref| <= 2e-2 against dequantise-then-matmul (the contract's bound).
"""
import pytest
import torch

from oracle import fp8_spec as S, ref_linear as R, synth

pytestmark = pytest.mark.gpu

PARITY = 2e-2


@pytest.fixture(scope="module")
def ops(built_library):
    from nano_qwen_b200 import ops
    ops.init()
    return ops


_weights = {}


def quantised_weight(ops, stack: str, name: str):
    """Full (unsharded) FP8 weight + block scales of one layer, generated and quantised on the device once."""
    key = (stack, name)
    if key not in _weights:
        _weights.clear()                                   # keep one layer resident at a time
        K, N = synth.STACKS[stack][name]
        g = torch.Generator(device="cuda").manual_seed(sum(map(ord, stack + name)))
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        _weights[key] = ops.weight_quant(w)
    return _weights[key]


def sample_blocks(n_rows: int, count: int = 6) -> torch.Tensor:
    nb = (n_rows + 127) // 128
    return torch.linspace(0, nb - 1, min(count, nb)).long().unique()


def check_sampled(y: torch.Tensor, x: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, bias=None, rows=24):
    """Compares sampled rows x sampled 128-row weight blocks of ``y = linear(x, wq, sw)`` with the oracle."""
    m, n = y.shape
    ridx = torch.linspace(0, m - 1, min(rows, m)).long().unique()
    xq_ref, sx_ref = S.quantize_act_group128(x[ridx.cuda()].cpu())
    worst = 0.0
    for b in sample_blocks(n).tolist():
        lo, hi = b * 128, min(b * 128 + 128, n)
        ref = S.linear_dequant_matmul(xq_ref, sx_ref, wq[lo:hi].cpu(), sw[b:b + 1].cpu(),
                                      None if bias is None else bias[lo:hi].cpu())
        got = y[ridx.cuda()][:, lo:hi].cpu()
        err = S.max_rel_err(got, ref)                      # relative to the largest reference value of the block
        assert err <= PARITY, (b, err)
        worst = max(worst, err)
    return worst


# ---------------------------------------------------------------------------------------------------------------
# Qwen3-32B-shaped layers, unsharded
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m", [1, 64, 8192])
@pytest.mark.parametrize("name", synth.LAYER_ORDER)
def test_qwen3_32b_layers_against_the_oracle(ops, name, m):
    K, N = synth.STACKS["qwen3-32b"][name]
    wq, sw = quantised_weight(ops, "qwen3-32b", name)
    g = torch.Generator(device="cuda").manual_seed(m + 5)
    x = torch.randn(m, K, generator=g, device="cuda").to(torch.bfloat16)
    y = ops.fp8_linear(x, wq, sw)
    torch.cuda.synchronize()
    assert y.shape == (m, N) and y.dtype == torch.bfloat16
    check_sampled(y, x, wq, sw)


# ---------------------------------------------------------------------------------------------------------------
# Per-rank shards at tp = 2, 4, 8 (what each rank of a tensor-parallel run executes)
# ---------------------------------------------------------------------------------------------------------------
def column_rank_param(stack, name, wq, sw, rank, tp):
    """This rank's rows of a column-parallel layer: [q_r; k_r; v_r] for qkv, [gate_r; up_r] for gate_up."""
    K, N = synth.STACKS[stack][name]
    if name == "qkv":
        nq = N - 2 * 8 * 128                               # 8 kv heads of 128
        parts = [(0, nq), (nq, nq + 1024), (nq + 1024, N)]
    else:
        parts = [(0, N // 2), (N // 2, N)]
    w_r = torch.cat([wq[lo:hi].view(torch.uint8).chunk(tp, 0)[rank] for lo, hi in parts]).view(torch.float8_e4m3fn)
    s_r = torch.cat([sw[lo // 128:hi // 128].chunk(tp, 0)[rank] for lo, hi in parts])
    return w_r, s_r


@pytest.mark.parametrize("tp", [2, 4, 8])
@pytest.mark.parametrize("stack", ["qwen3-8b", "qwen3-32b"])
@pytest.mark.parametrize("name", ["qkv", "gate_up"])
def test_column_parallel_shards_against_the_oracle(ops, stack, name, tp):
    """Rank 0 and the last rank of a column-parallel layer (N / tp rows: 8B at tp 8 is 768 and 3072, 32B 1280 and 6400)."""
    K, N = synth.STACKS[stack][name]
    wq, sw = quantised_weight(ops, stack, name)
    for rank in (0, tp - 1):
        w_r, s_r = column_rank_param(stack, name, wq, sw, rank, tp)
        assert w_r.shape == (N // tp, K)
        for m in (64, 8192):
            g = torch.Generator(device="cuda").manual_seed(tp * 100 + rank + m)
            x = torch.randn(m, K, generator=g, device="cuda").to(torch.bfloat16)
            y = ops.fp8_linear(x, w_r.contiguous(), s_r.contiguous())
            torch.cuda.synchronize()
            check_sampled(y, x, w_r, s_r)


@pytest.mark.parametrize("tp", [2, 4, 8])
@pytest.mark.parametrize("stack", ["qwen3-8b", "qwen3-32b"])
@pytest.mark.parametrize("name", ["o_proj", "down"])
def test_row_parallel_shards_sum_to_the_unsharded_oracle(ops, stack, name, tp):
    """Every rank's K-slice (8B at tp 8: 512 and 1536 columns; 32B: 1024 and 3200 = 25 K-tiles) through the kernel;
    each partial against the oracle of the slice, and their sum (what the all-reduce leaves) against the oracle
    of the whole layer."""
    K, N = synth.STACKS[stack][name]
    wq, sw = quantised_weight(ops, stack, name)
    for m in (64, 8192):
        g = torch.Generator(device="cuda").manual_seed(tp * 10 + m)
        x = torch.randn(m, K, generator=g, device="cuda").to(torch.bfloat16)
        total = torch.zeros(m, N, dtype=torch.float32, device="cuda")
        for rank in range(tp):
            if m == 8192 and rank not in (0, tp - 1):
                continue                                   # prefill size: first and last rank only
            w_r = R.row_shard(wq.view(torch.uint8), rank, tp).contiguous().view(torch.float8_e4m3fn)
            s_r = R.row_shard(sw, rank, tp).contiguous()
            x_r = R.row_shard(x, rank, tp).contiguous()    # the rank's slice of the activations (dim 1, like the weight)
            y = ops.fp8_linear(x_r, w_r, s_r)
            torch.cuda.synchronize()
            check_sampled(y, x_r, w_r, s_r, rows=12)
            total += y.float()                             # bf16 partials summed, as the all-reduce does
        if m == 64:
            # group scales are per 128 columns and shards are 128-aligned, so quantising slices == slicing the quantised
            ridx = torch.linspace(0, m - 1, 12).long().unique()
            xq_ref, sx_ref = S.quantize_act_group128(x[ridx.cuda()].cpu())
            for b in sample_blocks(N, 4).tolist():
                ref = S.linear_dequant_matmul(xq_ref, sx_ref, wq[b * 128:b * 128 + 128].cpu(), sw[b:b + 1].cpu())
                got = total[ridx.cuda()][:, b * 128:b * 128 + 128].cpu()
                assert S.max_rel_err(got.to(torch.bfloat16), ref) <= PARITY


# ---------------------------------------------------------------------------------------------------------------
# The runner's warm-up size: 16 384 tokens
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["gate_up", "down"])
def test_prefill_of_16384_tokens_against_the_oracle(ops, name):
    K, N = synth.STACKS["qwen3-8b"][name]
    wq, sw = quantised_weight(ops, "qwen3-8b", name)
    g = torch.Generator(device="cuda").manual_seed(16384)
    x = torch.randn(16384, K, generator=g, device="cuda").to(torch.bfloat16)
    y = ops.fp8_linear(x, wq, sw)
    torch.cuda.synchronize()
    check_sampled(y, x, wq, sw, rows=32)
    # the second half of the batch alone gives the same rows (tiles do not leak between tokens)
    tail = ops.fp8_linear(x[8192:], wq, sw)
    assert S.max_rel_err(tail.cpu(), y[8192:].cpu()) <= 8e-3


# ---------------------------------------------------------------------------------------------------------------
# Module API: ReplicatedLinear, and a biased row-parallel layer
# ---------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def L(ops, single_rank_group):
    from nano_qwen_b200.layers import linear
    return linear


def _on_cuda(make):
    torch.set_default_device("cuda")
    torch.set_default_dtype(torch.bfloat16)
    try:
        return make()
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)


@pytest.mark.parametrize("kind", ["ReplicatedLinear", "RowParallelLinear", "ColumnParallelLinear"])
@pytest.mark.parametrize("m", [1, 48, 300])
def test_biased_layers_through_the_module_api(L, kind, m):
    """``F.linear(x, W, b)`` of nano_qwen ``layers/linear.py:51`` (Replicated), ``:73`` (Column) and ``:153`` (Row:
    the bias is added on rank 0, which a one-rank group is)."""
    K, N = 1536, 640
    g = torch.Generator().manual_seed(m)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    b = torch.randn(N, generator=g).to(torch.bfloat16)
    x = torch.randn(m, K, generator=g).to(torch.bfloat16)
    wq, sw = S.quantize_weight_block128(w)
    layer = _on_cuda(lambda: getattr(L, kind)(K, N, bias=True))
    assert layer.bias is not None and layer.bias.dtype == torch.bfloat16 and layer.bias.is_cuda
    layer.weight.weight_loader(layer.weight, wq)
    layer.weight_scale_inv.weight_loader(layer.weight_scale_inv, sw)
    layer.bias.weight_loader(layer.bias, b)
    y = layer(x.cuda())
    torch.cuda.synchronize()
    xq, sx = S.quantize_act_group128(x)
    ref = S.linear_dequant_matmul(xq, sx, wq, sw, b)
    assert S.max_rel_err(y.cpu(), ref) <= PARITY
    # and without the bias the difference is exactly the bias up to one bf16 rounding of the sum
    plain = _on_cuda(lambda: getattr(L, kind)(K, N))
    assert plain.bias is None
    plain.weight.weight_loader(plain.weight, wq)
    plain.weight_scale_inv.weight_loader(plain.weight_scale_inv, sw)
    y0 = plain(x.cuda())
    ref0 = S.linear_dequant_matmul(xq, sx, wq, sw, None)
    assert S.max_rel_err(y0.cpu(), ref0) <= PARITY
