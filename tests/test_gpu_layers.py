"""The drop-in layers on the GPU: reference-derived goldens, graph capture, shapes, full-size properties."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import fp8_spec as S, synth

pytestmark = pytest.mark.gpu

PARITY = 2e-2


@pytest.fixture(scope="module")
def L(built_library, single_rank_group):
    from nano_qwen_b200 import ops
    from nano_qwen_b200.layers import linear
    ops.init()
    return linear


@pytest.fixture(scope="module")
def stack06():
    return synth.make_stack("qwen3-0.6b", 16, seed=0)


def build_layers(L, weights, quantised_checkpoint):
    """The four layers of the 0.6B-shaped stack on cuda, loaded through weight_loader."""
    shapes = synth.STACKS["qwen3-0.6b"]
    torch.set_default_device("cuda")
    torch.set_default_dtype(torch.bfloat16)
    try:
        K, N = shapes["qkv"]
        qkv = L.QKVParallelLinear(K, 128, N // 128 - 16, 8)
        K, N = shapes["gate_up"]
        gu = L.MergedColumnParallelLinear(K, [N // 2, N // 2])
        o = L.RowParallelLinear(*shapes["o_proj"])
        down = L.RowParallelLinear(*shapes["down"])
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)

    def pieces(name):
        w = weights[name]
        if quantised_checkpoint:                        # an FP8 checkpoint: weight + weight_scale_inv tensors
            wq, sw = S.quantize_weight_block128(w)
            return [(wq, sw)]
        return [(w, None)]                              # a bf16 checkpoint: quantised on load, on the device

    def load(mod, name, splits):
        (w, s), = pieces(name)
        for sid, lo, hi in splits:
            args = () if sid is None else (sid,)
            mod.weight.weight_loader(mod.weight, w[lo:hi] if sid is not None else w, *args)
            if s is not None:
                mod.weight_scale_inv.weight_loader(mod.weight_scale_inv, s[lo // 128:hi // 128] if sid is not None else s, *args)

    N = shapes["qkv"][1]
    nq = N - 2048
    load(qkv, "qkv", [("q", 0, nq), ("k", nq, nq + 1024), ("v", nq + 1024, N)])
    N = shapes["gate_up"][1]
    load(gu, "gate_up", [(0, 0, N // 2), (1, N // 2, N)])
    load(o, "o_proj", [(None, 0, 0)])
    load(down, "down", [(None, 0, 0)])
    return {"qkv": qkv, "gate_up": gu, "o_proj": o, "down": down}


@pytest.mark.parametrize("quantised_checkpoint", [True, False])
def test_stack_matches_reference_modules_golden(L, stack06, quantised_checkpoint):
    """Outputs equal what nano_qwen's own modules returned for the dequantised operands (<= 2e-2)."""
    weights, acts = stack06
    layers = build_layers(L, weights, quantised_checkpoint)
    with np.load(os.path.join(GOLDEN, "linear_tp1.npz")) as z:
        for name in synth.LAYER_ORDER:
            assert synth.digest(acts[name].view(torch.int16)) == str(z[f"sha_x_{name}"])
            y = layers[name](acts[name].cuda())
            torch.cuda.synchronize()
            gold = torch.from_numpy(z[f"y_{name}_r0"]).view(torch.bfloat16)
            assert y.dtype == torch.bfloat16 and tuple(y.shape) == tuple(gold.shape)
            assert S.max_rel_err(y.cpu(), gold) <= PARITY, name
            if not quantised_checkpoint:                 # quantise-on-load produced the oracle's bytes
                wq, sw = S.quantize_weight_block128(weights[name])
                assert torch.equal(layers[name].weight.data.cpu().view(torch.uint8) & 0x7F, wq.view(torch.uint8) & 0x7F)
                assert torch.equal(layers[name].weight_scale_inv.data.cpu(), sw)


def test_forward_shapes_like_f_linear(L, stack06):
    weights, acts = stack06
    layers = build_layers(L, weights, True)
    qkv = layers["qkv"]
    x = acts["qkv"].cuda()
    y2 = qkv(x)
    y3 = qkv(x.view(2, 8, -1))                           # leading dims are flattened and restored
    assert y3.shape == (2, 8, y2.shape[1]) and torch.equal(y3.view(16, -1), y2)
    y0 = qkv(x[:0])                                      # no tokens
    assert y0.shape == (0, y2.shape[1])
    wide = torch.zeros(16, 2048, dtype=torch.bfloat16, device="cuda")
    wide[:, ::2] = x
    assert torch.equal(qkv(wide[:, ::2]), y2)            # odd strides are made contiguous, not rejected
    assert torch.equal(qkv(x), y2)                       # input not modified, result reproducible


def test_cuda_graph_replay_equals_eager(L, stack06):
    """The runner captures decode steps in CUDA graphs; the layers must be capturable and replay bit-identically."""
    weights, acts = stack06
    layers = build_layers(L, weights, True)
    xs = {n: acts[n].cuda() for n in synth.LAYER_ORDER}
    eager = {n: layers[n](xs[n]).clone() for n in synth.LAYER_ORDER}
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for n in synth.LAYER_ORDER:                      # warm-up on the capture stream
            layers[n](xs[n])
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        outs = {n: layers[n](xs[n]) for n in synth.LAYER_ORDER}
    for _ in range(3):
        for n in synth.LAYER_ORDER:
            outs[n].fill_(0)
        graph.replay()
        torch.cuda.synchronize()
        for n in synth.LAYER_ORDER:
            assert torch.equal(outs[n].view(torch.int16), eager[n].view(torch.int16)), n


@pytest.mark.parametrize("name,m", [("qkv", 8192), ("down", 4096), ("gate_up", 2048), ("o_proj", 256), ("gate_up", 256), ("gate_up", 64),
                                    ("gate_up", 4), ("down", 1)])
def test_full_size_8b_layers_sampled_rows_and_linearity(L, name, m):
    """Qwen3-8B-sized layers: sampled rows against the oracle, plus size-independent properties."""
    from nano_qwen_b200 import ops
    K, N = synth.STACKS["qwen3-8b"][name]
    g = torch.Generator(device="cuda").manual_seed(7)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    x = torch.randn(m, K, generator=g, device="cuda").to(torch.bfloat16)
    wq, sw = ops.weight_quant(w)
    y = ops.fp8_linear(x, wq, sw)
    torch.cuda.synchronize()
    rows = torch.linspace(0, m - 1, 24).long().unique()
    xq_ref, sx_ref = S.quantize_act_group128(x[rows].cpu())
    ref = S.linear_dequant_matmul(xq_ref, sx_ref, wq.cpu(), sw.cpu())
    assert S.max_rel_err(y[rows.cuda()].cpu(), ref) <= PARITY
    # tokens are independent: a permuted batch gives the permuted result, bit for bit
    perm = torch.randperm(m, generator=torch.Generator().manual_seed(1)).cuda()
    assert torch.equal(ops.fp8_linear(x[perm], wq, sw), y[perm])
    # scaling the input by a power of two scales the group scales, not the codes: y doubles exactly
    assert torch.equal(ops.fp8_linear(x * 2, wq, sw).float(), y.float() * 2)
    # a batch is the concatenation of its halves (tile boundaries do not leak between tokens); a different batch size
    # may run on a different kernel or K split, i.e. another fp32 summation order: equal up to one bf16 rounding
    h = m // 2 + 3
    halves = torch.cat([ops.fp8_linear(x[:h], wq, sw), ops.fp8_linear(x[h:], wq, sw)])
    assert S.max_rel_err(halves.cpu(), y.cpu()) <= 8e-3
