"""Regenerates the fixtures in this directory from the reference's own modules.

Run once, in a container that has the reference checked out (it is not needed,
and not read, when the tests run):

    python tests/golden/make_golden.py /path/to/nano_qwen

What it records
---------------
``sharding.json``
    For every layer class of ``nano_qwen/layers/linear.py`` and every
    ``tp in {1,2,4,8}`` and rank: which checkpoint rows / columns end up in the
    rank's parameter.  Obtained by pushing an index-coded tensor
    (``value = row * K + col``) through the reference ``weight_loader`` inside
    real gloo ranks (the modules read ``dist.get_rank()/get_world_size()``).
``linear_tp{1,2}.npz``
    The Qwen3-0.6B-shaped stack at M=16, seed 0: FP8-quantised (oracle recipe),
    dequantised to fp32, loaded into the reference's QKV / Merged / Row modules
    through their loaders and run through their ``forward`` on CPU in fp32
    (row-parallel layers all-reduced over gloo).  Outputs are stored as bf16
    bit patterns, inputs as sha256 digests.
``checkpoint_digests.json``, ``checkpoint_probe_tp{1,2}.npz``
    The synthetic tiny Qwen3-dense-shaped checkpoint of ``oracle/synth_checkpoint.py`` (dequantised variant) loaded
    by the reference's own ``load_model`` (``nano_qwen/utils/loader.py:12-28``) into a tree of the reference's
    ``QKVParallelLinear`` / ``MergedColumnParallelLinear`` / ``RowParallelLinear`` / ``VocabParallelEmbedding`` /
    ``RMSNorm`` under real gloo ranks, tp in {1,2,4,8}: sha256 of every rank's parameters (as fp32), and for tp in
    {1,2} the outputs of every packed linear on seeded probe activations (quantised and dequantised by the oracle
    recipe first).  The script also checks that ``oracle/ref_loader.py`` places exactly what ``load_model`` places.
``fused_ops.npz``
    The reference's ``SiluAndMul``, ``RMSNorm`` and ``GemmaRMSNorm`` (``layers/activation.py``, ``layers/layernorm.py``)
    run on CPU in bf16 with ``torch.compile`` switched off (``TORCHDYNAMO_DISABLE=1``), on seeded inputs of the
    Qwen3-0.6B shapes at M=16: inputs and outputs as bf16 bit patterns.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import fp8_spec, ref_loader, synth, synth_checkpoint  # noqa: E402

SHARD_CASES = {
    # kind: constructor args for the small index-coded case
    "replicated": dict(K=256, N=512),
    "column": dict(K=256, N=1024),
    "merged": dict(K=256, sizes=[1024, 2048]),
    "qkv": dict(K=256, head=128, heads=16, kv=8),
    "row": dict(K=2048, N=256),
}


def index_coded(n: int, k: int) -> torch.Tensor:
    return (torch.arange(n, dtype=torch.float32).unsqueeze(1) * k + torch.arange(k, dtype=torch.float32))


def segments(vals: list[int]) -> list[list[int]]:
    """Run-length encode consecutive integers as [dst_start, src_start, length]."""
    out, i = [], 0
    while i < len(vals):
        j = i
        while j + 1 < len(vals) and vals[j + 1] == vals[j] + 1:
            j += 1
        out.append([i, vals[i], j - i + 1])
        i = j + 1
    return out


def describe(param: torch.Tensor, k_full: int) -> dict:
    if param.dim() == 1:
        return {"shape": list(param.shape), "rows": segments([int(v) for v in param.tolist()])}
    rows = (param[:, 0] // k_full).long().tolist()
    cols = (param[0, :] % k_full).long().tolist()
    assert torch.equal(param, index_coded(max(rows) + 1, k_full)[rows][:, cols])
    return {"shape": list(param.shape), "rows": segments(rows), "cols": segments(cols)}


def worker(rank: int, tp: int, port: int, ref_src: str, outdir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=tp)
    sys.path.insert(0, ref_src)
    torch.set_default_dtype(torch.float32)
    from nano_qwen.layers import linear as ref

    out: dict = {}
    # ---- sharding ----
    c = SHARD_CASES["replicated"]
    m = ref.ReplicatedLinear(c["K"], c["N"], bias=True)
    m.weight.weight_loader(m.weight, index_coded(c["N"], c["K"]))
    m.bias.weight_loader(m.bias, torch.arange(c["N"], dtype=torch.float32))
    out["replicated"] = {"weight": describe(m.weight.data, c["K"]), "bias": describe(m.bias.data, 1)}

    c = SHARD_CASES["column"]
    m = ref.ColumnParallelLinear(c["K"], c["N"], bias=True)
    m.weight.weight_loader(m.weight, index_coded(c["N"], c["K"]))
    m.bias.weight_loader(m.bias, torch.arange(c["N"], dtype=torch.float32))
    out["column"] = {"weight": describe(m.weight.data, c["K"]), "bias": describe(m.bias.data, 1)}

    c = SHARD_CASES["merged"]
    m = ref.MergedColumnParallelLinear(c["K"], c["sizes"])
    full = index_coded(sum(c["sizes"]), c["K"])
    off = 0
    for i, sz in enumerate(c["sizes"]):
        m.weight.weight_loader(m.weight, full[off:off + sz], i)
        off += sz
    out["merged"] = {"weight": describe(m.weight.data, c["K"])}

    c = SHARD_CASES["qkv"]
    m = ref.QKVParallelLinear(c["K"], c["head"], c["heads"], c["kv"])
    nq, nk = c["heads"] * c["head"], c["kv"] * c["head"]
    full = index_coded(nq + 2 * nk, c["K"])
    m.weight.weight_loader(m.weight, full[:nq], "q")
    m.weight.weight_loader(m.weight, full[nq:nq + nk], "k")
    m.weight.weight_loader(m.weight, full[nq + nk:], "v")
    out["qkv"] = {"weight": describe(m.weight.data, c["K"]),
                  "num_heads": m.num_heads, "num_kv_heads": m.num_kv_heads}

    c = SHARD_CASES["row"]
    m = ref.RowParallelLinear(c["K"], c["N"], bias=True)
    m.weight.weight_loader(m.weight, index_coded(c["N"], c["K"]))
    m.bias.weight_loader(m.bias, torch.arange(c["N"], dtype=torch.float32))
    out["row"] = {"weight": describe(m.weight.data, c["K"]), "bias": describe(m.bias.data, 1)}

    with open(os.path.join(outdir, f"shard_tp{tp}_r{rank}.json"), "w") as f:
        json.dump(out, f)

    # ---- the 0.6B-shaped stack through the reference's forward ----
    if tp in (1, 2):
        weights, acts = synth.make_stack("qwen3-0.6b", 16, seed=0)
        shapes = synth.STACKS["qwen3-0.6b"]
        res = {}
        dq_w, dq_x = {}, {}
        for name in synth.LAYER_ORDER:
            wq, sw = fp8_spec.quantize_weight_block128(weights[name])
            xq, sx = fp8_spec.quantize_act_group128(acts[name])
            dq_w[name] = fp8_spec.dequantize_weight(wq, sw)
            dq_x[name] = fp8_spec.dequantize_act(xq, sx)
            if rank == 0:
                res[f"sha_w_{name}"] = synth.digest(weights[name].view(torch.int16))
                res[f"sha_x_{name}"] = synth.digest(acts[name].view(torch.int16))
                res[f"sha_wq_{name}"] = synth.digest(wq.view(torch.uint8))
                res[f"sha_xq_{name}"] = synth.digest(xq.view(torch.uint8))
        K, N = shapes["qkv"]
        qkv = ref.QKVParallelLinear(K, 128, (N // 128) - 16, 8)
        nq = N - 2 * 8 * 128
        qkv.weight.weight_loader(qkv.weight, dq_w["qkv"][:nq], "q")
        qkv.weight.weight_loader(qkv.weight, dq_w["qkv"][nq:nq + 1024], "k")
        qkv.weight.weight_loader(qkv.weight, dq_w["qkv"][nq + 1024:], "v")
        y_qkv = qkv(dq_x["qkv"])

        K, N = shapes["gate_up"]
        gu = ref.MergedColumnParallelLinear(K, [N // 2, N // 2])
        gu.weight.weight_loader(gu.weight, dq_w["gate_up"][:N // 2], 0)
        gu.weight.weight_loader(gu.weight, dq_w["gate_up"][N // 2:], 1)
        y_gu = gu(dq_x["gate_up"])

        ys = {"qkv": y_qkv, "gate_up": y_gu}
        for name in ("o_proj", "down"):
            K, N = shapes[name]
            row = ref.RowParallelLinear(K, N)
            row.weight.weight_loader(row.weight, dq_w[name])
            ks = K // tp
            ys[name] = row(dq_x[name][:, rank * ks:(rank + 1) * ks].contiguous())
        for name, y in ys.items():
            res[f"y_{name}_r{rank}"] = y.detach().to(torch.bfloat16).view(torch.int16).numpy()
        np.savez(os.path.join(outdir, f"linear_tp{tp}_r{rank}.npz"), **res)
    dist.barrier()
    dist.destroy_process_group()


def param_digests(model) -> dict:
    return {name: synth.digest(p.data.float().contiguous().view(torch.uint8)) for name, p in model.named_parameters()}


def checkpoint_worker(rank: int, tp: int, port: int, ref_src: str, ckpt: str, outdir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=tp)
    sys.path.insert(0, ref_src)
    torch.set_default_dtype(torch.float32)
    from nano_qwen.layers import linear as ref
    from nano_qwen.layers.embed_head import VocabParallelEmbedding
    from nano_qwen.layers.layernorm import RMSNorm
    from nano_qwen.utils.loader import load_model

    def tree():
        return synth_checkpoint.build_tree(ref, rank, tp, embed_cls=VocabParallelEmbedding,
                                           norm_cls=lambda n: RMSNorm(n, eps=1e-6))
    model = tree()
    load_model(model, ckpt)                                   # the reference's own loop
    digests = param_digests(model)
    again = tree()
    ref_loader.load_model(again, ckpt)                        # the restatement must place the same bytes
    assert param_digests(again) == digests, "oracle/ref_loader.py disagrees with nano_qwen.utils.loader.load_model"
    with open(os.path.join(outdir, f"ckpt_tp{tp}_r{rank}.json"), "w") as f:
        json.dump(digests, f)
    if tp in (1, 2):
        res = {}
        for name, x in synth_checkpoint.probe_inputs().items():
            mod = model.model.get_submodule(name)
            xq, sx = fp8_spec.quantize_act_group128(x)
            xd = fp8_spec.dequantize_act(xq, sx)
            if isinstance(mod, ref.RowParallelLinear):
                ks = xd.shape[1] // tp
                xd = xd[:, rank * ks:(rank + 1) * ks].contiguous()
            res[f"{name}_r{rank}"] = mod(xd).detach().to(torch.bfloat16).view(torch.int16).numpy()
        np.savez(os.path.join(outdir, f"ckpt_probe_tp{tp}_r{rank}.npz"), **res)
    dist.barrier()
    dist.destroy_process_group()


def checkpoint_case(ref_src: str, port: int) -> None:
    tmp = tempfile.mkdtemp()
    ckpt = synth_checkpoint.write(os.path.join(tmp, "dequantised"), seed=0, quantised=False)
    digests = {}
    for i, tp in enumerate((1, 2, 4, 8)):
        mp.spawn(checkpoint_worker, args=(tp, port + i, ref_src, ckpt, tmp), nprocs=tp, join=True)
        digests[f"tp{tp}"] = [json.load(open(os.path.join(tmp, f"ckpt_tp{tp}_r{r}.json"))) for r in range(tp)]
        if tp in (1, 2):
            merged = {}
            for r in range(tp):
                with np.load(os.path.join(tmp, f"ckpt_probe_tp{tp}_r{r}.npz")) as z:
                    merged.update({k: z[k] for k in z.files})
            np.savez_compressed(os.path.join(HERE, f"checkpoint_probe_tp{tp}.npz"), **merged)
    with open(os.path.join(HERE, "checkpoint_digests.json"), "w") as f:
        json.dump(digests, f, separators=(",", ":"))


def fused_ops(ref_src: str) -> None:
    """Runs in a child interpreter: the compiler switch has to be set before torch is imported."""
    import subprocess
    code = r'''
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from nano_qwen.layers.activation import SiluAndMul
from nano_qwen.layers.layernorm import RMSNorm, GemmaRMSNorm
g = torch.Generator().manual_seed(2024)
bits = lambda t: t.contiguous().view(torch.int16).numpy()
M, H, I = 16, 1024, 3072
out = {}
gate_up = (torch.randn(M, 2 * I, generator=g) * 1.5).to(torch.bfloat16)
out["silu_in"] = bits(gate_up)
out["silu_out"] = bits(SiluAndMul()(gate_up))
x = torch.randn(M, H, generator=g).to(torch.bfloat16)
res = torch.randn(M, H, generator=g).to(torch.bfloat16)
out["norm_x"], out["norm_res"] = bits(x), bits(res)
for name, cls in (("rms", RMSNorm), ("gemma", GemmaRMSNorm)):
    mod = cls(H, eps=1e-6).to(torch.bfloat16)
    w = (torch.randn(H, generator=g) * 0.3 + (0.0 if name == "gemma" else 1.0)).to(torch.bfloat16)
    mod.weight.data.copy_(w)
    out[name + "_w"] = bits(w)
    out[name + "_out"] = bits(mod(x.clone()).detach())
    y, r = mod(x.clone(), res.clone())
    out[name + "_add_out"], out[name + "_add_res"] = bits(y.detach()), bits(r.detach())
np.savez_compressed(sys.argv[2], **out)
'''
    env = dict(os.environ, TORCHDYNAMO_DISABLE="1")
    subprocess.run([sys.executable, "-c", code, ref_src, os.path.join(HERE, "fused_ops.npz")], check=True, env=env)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/nano_qwen [--only-checkpoint]")
    ref_src = os.path.join(sys.argv[1], "src")
    assert os.path.isdir(ref_src), ref_src
    checkpoint_case(ref_src, 29631)
    if "--only-checkpoint" in sys.argv:
        return
    fused_ops(ref_src)
    tmp = tempfile.mkdtemp()
    sharding = {"cases": SHARD_CASES}
    for i, tp in enumerate((1, 2, 4, 8)):
        mp.spawn(worker, args=(tp, 29611 + i, ref_src, tmp), nprocs=tp, join=True)
        sharding[f"tp{tp}"] = [json.load(open(os.path.join(tmp, f"shard_tp{tp}_r{r}.json"))) for r in range(tp)]
        if tp in (1, 2):
            merged = {}
            for r in range(tp):
                with np.load(os.path.join(tmp, f"linear_tp{tp}_r{r}.npz")) as z:
                    merged.update({k: z[k] for k in z.files})
            np.savez_compressed(os.path.join(HERE, f"linear_tp{tp}.npz"), **merged)
    with open(os.path.join(HERE, "sharding.json"), "w") as f:
        json.dump(sharding, f, separators=(",", ":"))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
