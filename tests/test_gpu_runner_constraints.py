"""The drop-in layers under the model runner's real constraints (nano_qwen ``engine/model_runner.py``).

* ``capture_cudagraph`` (``model_runner.py:421-456``) captures the decode forward once per batch size of
  ``[1, 2, 4, 8] + range(16, 513, 16)`` (36 graphs), largest first, all sharing one memory pool, on slices of static
  input/output buffers; ``run_model`` (``:323-336``) copies fresh inputs into the static buffers and replays.
  Here the same is done to one Qwen3-8B-sized decoder layer's linear path — add + RMSNorm -> qkv_proj -> o_proj ->
  add + RMSNorm -> gate_up_proj -> SiluAndMul -> down_proj, in the data flow of ``models/qwen3_5.py:248-277`` with
  attention (outside this path) replaced by "take the query columns" — and every replay must equal the eager
  forward of the same inputs bit for bit.
* ``warmup_model`` (``model_runner.py:171-184``) runs one eager prefill of ``max_num_batched_tokens`` = 16 384 tokens;
  the same pass is checked stage by stage against the oracle on sampled token rows.
"""
import pytest
import torch

from oracle import fp8_spec as S, ref_fused as F, synth

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER = 4096, 32, 8, 128, 12288
GRAPH_BS = [1, 2, 4, 8] + list(range(16, 513, 16))
PARITY = 2e-2


class LinearPath(torch.nn.Module):
    def __init__(self, L):
        super().__init__()
        self.input_layernorm = L.RMSNorm(HIDDEN, eps=1e-6, emit_fp8=True)
        self.qkv_proj = L.QKVParallelLinear(HIDDEN, HEAD_DIM, HEADS, KV_HEADS)
        self.o_proj = L.RowParallelLinear(HEADS * HEAD_DIM, HIDDEN)
        self.post_attention_layernorm = L.RMSNorm(HIDDEN, eps=1e-6, emit_fp8=True)
        self.gate_up_proj = L.MergedColumnParallelLinear(HIDDEN, [INTER, INTER])
        self.down_proj = L.RowParallelLinear(INTER, HIDDEN)
        self.act_fn = L.SiluAndMul()

    def forward(self, hidden, residual, keep=None):
        h, residual = self.input_layernorm(hidden, residual)
        qkv = self.qkv_proj(h)
        attn = qkv[:, :HEADS * HEAD_DIM]                      # stand-in for attention: a strided view of the queries
        o = self.o_proj(attn)
        h2, residual = self.post_attention_layernorm(o, residual)
        gate_up = self.gate_up_proj(h2)
        act = self.act_fn(gate_up)
        out = self.down_proj(act)
        if keep is not None:
            keep.update(h=h, qkv=qkv, attn=attn, o=o, h2=h2, gate_up=gate_up, act=act, out=out, residual=residual)
        return out, residual


@pytest.fixture(scope="module")
def layer(built_library, single_rank_group):
    from nano_qwen_b200 import layers as L, ops
    ops.init()
    torch.set_default_device("cuda")
    torch.set_default_dtype(torch.bfloat16)
    try:
        mod = LinearPath(L)
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)
    g = torch.Generator(device="cuda").manual_seed(2025)
    for name in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj"):
        lin = getattr(mod, name)
        n, k = lin.weight.shape
        wq, sw = ops.weight_quant((torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
        lin.weight.data.copy_(wq)
        lin.weight_scale_inv.data.copy_(sw)
    for name in ("input_layernorm", "post_attention_layernorm"):
        w = getattr(mod, name).weight
        w.data.copy_(1.0 + 0.1 * torch.randn(w.shape, generator=g, device="cuda"))
    return mod


@torch.inference_mode()
def test_thirty_six_decode_graphs_share_one_pool_and_replay_bit_exactly(layer):
    max_bs = GRAPH_BS[-1]
    hidden = torch.zeros(max_bs, HIDDEN, dtype=torch.bfloat16, device="cuda")
    residual = torch.zeros(max_bs, HIDDEN, dtype=torch.bfloat16, device="cuda")
    outputs = torch.zeros(max_bs, HIDDEN, dtype=torch.bfloat16, device="cuda")
    res_out = torch.zeros(max_bs, HIDDEN, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    graphs, pool = {}, None
    for bs in reversed(GRAPH_BS):                                       # largest first, as the runner does
        graph = torch.cuda.CUDAGraph()
        y, r = layer(hidden[:bs], residual[:bs])                        # warm-up
        outputs[:bs], res_out[:bs] = y, r
        with torch.cuda.graph(graph, pool):
            y, r = layer(hidden[:bs], residual[:bs])
            outputs[:bs], res_out[:bs] = y, r
        if pool is None:
            pool = graph.pool()
        graphs[bs] = graph
        torch.cuda.synchronize()
    captured_bytes = torch.cuda.max_memory_allocated() - base
    # one shared pool: the 36 graphs together may not need more than a few times the largest one's intermediates
    # (largest: 512 tokens x (qkv 6144 + gate_up 24576 + ...) bf16, about 50 MB)
    assert captured_bytes < 512 << 20, f"graph pool grew to {captured_bytes >> 20} MiB"
    print(f"\n36 decode graphs captured; allocator peak above the weights: {captured_bytes / 2**20:.1f} MiB")

    g = torch.Generator(device="cuda").manual_seed(77)
    for rnd in range(2):
        for bs in GRAPH_BS:
            x = torch.randn(bs, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)
            res = torch.randn(bs, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)
            hidden[:bs], residual[:bs] = x, res                          # run_model: fresh inputs into the static buffers
            outputs.fill_(float("nan"))
            graphs[bs].replay()
            want_y, want_r = layer(x, res)                               # eager forward of the same inputs
            torch.cuda.synchronize()
            assert torch.equal(outputs[:bs].view(torch.int16), want_y.view(torch.int16)), bs
            assert torch.equal(res_out[:bs].view(torch.int16), want_r.view(torch.int16)), bs
    from nano_qwen_b200 import _cabi
    assert _cabi.device_status()["code"] == 0


@torch.inference_mode()
def test_warmup_pass_of_16384_tokens_against_the_oracle(layer):
    m = 16384
    g = torch.Generator(device="cuda").manual_seed(16384)
    x = torch.randn(m, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)
    res = torch.randn(m, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    keep = {}
    out, new_res = layer(x, res, keep)
    torch.cuda.synchronize()
    print(f"\neager pass of {m} tokens: allocator peak above the resident tensors {((torch.cuda.max_memory_allocated() - base) >> 20)} MiB")
    assert out.shape == (m, HIDDEN) and out.dtype == torch.bfloat16
    rows = torch.linspace(0, m - 1, 16).long().unique()
    rc = rows.cuda()

    def deq(qa):                                                         # sampled rows of a QuantizedActivation, fp32
        return S.dequantize_act(qa.xq[rc].cpu(), qa.sx[rc].cpu())

    def linear_rows(x_rows_fp32, lin, blocks):
        outs = []
        for b in blocks:
            w = S.dequantize_weight(lin.weight.data[b * 128:(b + 1) * 128].cpu(), lin.weight_scale_inv.data[b:b + 1].cpu())
            outs.append(torch.nn.functional.linear(x_rows_fp32, w).to(torch.bfloat16))
        return outs

    def check_linear(x_rows_fp32, lin, y, name):
        blocks = torch.linspace(0, lin.weight.shape[0] // 128 - 1, 5).long().unique().tolist()
        for b, ref in zip(blocks, linear_rows(x_rows_fp32, lin, blocks)):
            assert S.max_rel_err(y[rc][:, b * 128:(b + 1) * 128].cpu(), ref) <= PARITY, (name, b)

    # add + RMSNorm + quantiser: the new residual is bit-exact, the emitted FP8 is the quantised bf16 norm output
    ref_h, ref_res = F.rms_norm(x[rc].cpu(), layer.input_layernorm.weight.data.cpu(), 1e-6, res[rc].cpu(), False)
    xq_ref, sx_ref = S.quantize_act_group128(ref_h)
    assert torch.equal(keep["residual"][rc].cpu().view(torch.int16), F.rms_norm(
        keep["o"][rc].cpu(), layer.post_attention_layernorm.weight.data.cpu(), 1e-6, ref_res, False)[1].view(torch.int16))
    err = (deq(keep["h"]) - S.dequantize_act(xq_ref, sx_ref)).abs().max() / ref_h.float().abs().max()
    assert err <= 2 ** -3                                               # at most one e4m3 rounding step (32/448 of a group maximum)
    # each linear against the oracle, fed what the device actually fed it (errors do not chain)
    check_linear(deq(keep["h"]), layer.qkv_proj, keep["qkv"], "qkv")
    xq, sx = S.quantize_act_group128(keep["attn"][rc].cpu())
    check_linear(S.dequantize_act(xq, sx), layer.o_proj, keep["o"], "o_proj")
    check_linear(deq(keep["h2"]), layer.gate_up_proj, keep["gate_up"], "gate_up")
    check_linear(deq(keep["act"]), layer.down_proj, keep["out"], "down")
    # SiluAndMul + quantiser on the device's own gate_up rows
    ref_act = F.silu_and_mul(keep["gate_up"][rc].cpu())
    xq_ref, sx_ref = S.quantize_act_group128(ref_act)
    err = (deq(keep["act"]) - S.dequantize_act(xq_ref, sx_ref)).abs().max() / ref_act.float().abs().max()
    assert err <= 2 ** -3                                               # at most one e4m3 rounding step (32/448 of a group maximum)
