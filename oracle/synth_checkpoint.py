"""A synthetic FP8 block-quantised checkpoint of a tiny Qwen3-dense-shaped model, and the module tree that loads it.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  No real checkpoint is available offline; this one has the
tensor names, dtypes and layouts public block-FP8 checkpoints use: every linear projection as ``<module>.weight``
(float8_e4m3fn ``[N, K]``) plus ``<module>.weight_scale_inv`` (fp32 ``[N/128, K/128]``), everything else (embeddings,
norms, ``lm_head``) unquantised bf16.  q/k/v and gate/up are stored as separate projections, so loading them into
``QKVParallelLinear`` / ``MergedColumnParallelLinear`` exercises ``packed_modules_mapping`` the way
``nano_qwen/models/qwen3_5.py:330-333`` uses it for gate/up.

Sizes are the smallest that keep every shard of every tensor on 128-row / 128-column block boundaries up to 8 ranks.
All values come from one seeded CPU generator, so the script that records the reference's behaviour and the tests
regenerate the same bytes instead of committing megabytes.
"""
from __future__ import annotations

import os

import torch
from torch import nn

from . import fp8_spec

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, VOCAB, LAYERS = 256, 16, 8, 128, 1024, 512, 2
PROBE_TOKENS = 4

PACKED = {
    "q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
    "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1),
}

# projection name -> (N, K)
PROJECTIONS = {
    "self_attn.q_proj": (HEADS * HEAD_DIM, HIDDEN), "self_attn.k_proj": (KV_HEADS * HEAD_DIM, HIDDEN),
    "self_attn.v_proj": (KV_HEADS * HEAD_DIM, HIDDEN), "self_attn.o_proj": (HIDDEN, HEADS * HEAD_DIM),
    "mlp.gate_proj": (INTER, HIDDEN), "mlp.up_proj": (INTER, HIDDEN), "mlp.down_proj": (HIDDEN, INTER),
}


def tensors(seed: int = 0, quantised: bool = True) -> dict[str, torch.Tensor]:
    """Name -> CPU tensor.  ``quantised=False`` gives the same model with every projection dequantised to fp32 and
    no scale tensors: what a model without FP8 support (the reference) can load."""
    g = torch.Generator().manual_seed(seed)
    out: dict[str, torch.Tensor] = {}

    def bf16(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    out["model.embed_tokens.weight"] = bf16(VOCAB, HIDDEN, std=0.05)
    for i in range(LAYERS):
        pre = f"model.layers.{i}."
        out[pre + "input_layernorm.weight"] = bf16(HIDDEN, std=0.1, mean=1.0)
        out[pre + "post_attention_layernorm.weight"] = bf16(HIDDEN, std=0.1, mean=1.0)
        out[pre + "self_attn.q_norm.weight"] = bf16(HEAD_DIM, std=0.1, mean=1.0)
        out[pre + "self_attn.k_norm.weight"] = bf16(HEAD_DIM, std=0.1, mean=1.0)
        for proj, (n, k) in PROJECTIONS.items():
            wq, sw = fp8_spec.quantize_weight_block128(bf16(n, k, std=0.02))
            if quantised:
                out[pre + proj + ".weight"] = wq
                out[pre + proj + ".weight_scale_inv"] = sw
            else:
                out[pre + proj + ".weight"] = fp8_spec.dequantize_weight(wq, sw)
    out["model.norm.weight"] = bf16(HIDDEN, std=0.1, mean=1.0)
    out["lm_head.weight"] = bf16(VOCAB, HIDDEN, std=0.05)
    return out


def write(path: str, seed: int = 0, quantised: bool = True) -> str:
    """Writes the checkpoint as two ``*.safetensors`` files under ``path`` (a loader must walk several files)."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    all_t = tensors(seed, quantised)
    names = list(all_t)
    half = len(names) // 2
    for idx, part in enumerate((names[:half], names[half:])):
        save_file({n: all_t[n].contiguous() for n in part}, os.path.join(path, f"model-{idx + 1:05d}-of-00002.safetensors"))
    return path


def probe_inputs(seed: int = 1) -> dict[str, torch.Tensor]:
    """One seeded bf16 activation matrix per packed linear of every layer: ``layers.<i>.<module>`` -> ``[4, K]``."""
    g = torch.Generator().manual_seed(seed)
    k_of = {"self_attn.qkv_proj": HIDDEN, "self_attn.o_proj": HEADS * HEAD_DIM, "mlp.gate_up_proj": HIDDEN,
            "mlp.down_proj": INTER}
    return {f"layers.{i}.{name}": torch.randn(PROBE_TOKENS, k, generator=g).to(torch.bfloat16)
            for i in range(LAYERS) for name, k in k_of.items()}


class VocabShard(nn.Module):
    """Stand-in for the unquantised vocabulary-parallel tables (``nano_qwen/layers/embed_head.py:9-33``): each rank
    keeps rows ``[rank * V / tp, (rank + 1) * V / tp)``."""

    def __init__(self, vocab: int, hidden: int, rank: int, tp: int):
        super().__init__()
        self.rank = rank
        self.weight = nn.Parameter(torch.empty(vocab // tp, hidden), requires_grad=False)
        self.weight.weight_loader = self.weight_loader

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor) -> None:
        rows = param.data.size(0)
        param.data.copy_(loaded.narrow(0, self.rank * rows, rows))


class NormWeight(nn.Module):
    """A norm's parameter holder without a ``weight_loader`` (takes the loader's plain-copy branch)."""

    def __init__(self, size: int):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size), requires_grad=False)


def build_tree(linear_classes, rank: int, tp: int, embed_cls=None, norm_cls=None) -> nn.Module:
    """The module tree of the tiny model from a namespace that provides ``QKVParallelLinear``,
    ``MergedColumnParallelLinear`` and ``RowParallelLinear`` (the reference's module or the drop-in one).
    Parameter names equal the checkpoint's after ``PACKED`` is applied."""
    L = linear_classes
    embed = embed_cls or (lambda v, h: VocabShard(v, h, rank, tp))
    norm = norm_cls or NormWeight

    def layer():
        attn = nn.Module()
        attn.qkv_proj = L.QKVParallelLinear(HIDDEN, HEAD_DIM, HEADS, KV_HEADS)
        attn.o_proj = L.RowParallelLinear(HEADS * HEAD_DIM, HIDDEN)
        attn.q_norm, attn.k_norm = norm(HEAD_DIM), norm(HEAD_DIM)
        mlp = nn.Module()
        mlp.gate_up_proj = L.MergedColumnParallelLinear(HIDDEN, [INTER, INTER])
        mlp.down_proj = L.RowParallelLinear(INTER, HIDDEN)
        blk = nn.Module()
        blk.self_attn, blk.mlp = attn, mlp
        blk.input_layernorm, blk.post_attention_layernorm = norm(HIDDEN), norm(HIDDEN)
        return blk

    root = nn.Module()
    root.packed_modules_mapping = dict(PACKED)
    root.model = nn.Module()
    root.model.embed_tokens = embed(VOCAB, HIDDEN)
    root.model.layers = nn.ModuleList([layer() for _ in range(LAYERS)])
    root.model.norm = norm(HIDDEN)
    root.lm_head = embed(VOCAB, HIDDEN)
    return root
