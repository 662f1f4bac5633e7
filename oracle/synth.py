"""Seeded synthetic inputs for the FP8 linear stacks (CPU generator).

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Real checkpoints and
prompts are not available offline; these tensors have the shapes and value
distributions the benchmark contract names: weights bf16 N(0, 0.02),
activations bf16 N(0, 1), one independent activation matrix per layer input.

Generation order for one stack (fixed so a seed reproduces): for the layers
in the order qkv, o_proj, gate_up, down: all four weights first, then the four
activation matrices, all drawn from one ``torch.Generator`` seeded once.
"""
from __future__ import annotations

import hashlib

import torch

# (K, N) per layer kind; qkv N = (heads + 2*kv_heads) * 128 with 8 kv heads
STACKS = {
    "qwen3-0.6b": {"qkv": (1024, 4096), "o_proj": (2048, 1024), "gate_up": (1024, 6144), "down": (3072, 1024)},
    "qwen3-8b": {"qkv": (4096, 6144), "o_proj": (4096, 4096), "gate_up": (4096, 24576), "down": (12288, 4096)},
    "qwen3-32b": {"qkv": (5120, 10240), "o_proj": (8192, 5120), "gate_up": (5120, 51200), "down": (25600, 5120)},
}
LAYER_ORDER = ("qkv", "o_proj", "gate_up", "down")


def make_weight(gen: torch.Generator, n: int, k: int) -> torch.Tensor:
    return (torch.randn(n, k, generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)


def make_act(gen: torch.Generator, m: int, k: int) -> torch.Tensor:
    return torch.randn(m, k, generator=gen, dtype=torch.float32).to(torch.bfloat16)


def make_stack(stack: str, m: int, seed: int = 0):
    """Returns ``(weights, acts)``: dicts keyed by layer kind, bf16 CPU tensors."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    shapes = STACKS[stack]
    weights = {name: make_weight(gen, shapes[name][1], shapes[name][0]) for name in LAYER_ORDER}
    acts = {name: make_act(gen, m, shapes[name][0]) for name in LAYER_ORDER}
    return weights, acts


def digest(t: torch.Tensor) -> str:
    """sha256 of the raw bytes, to detect a drifting RNG before blaming a kernel."""
    raw = t.contiguous().view(torch.uint8) if t.dtype != torch.uint8 else t.contiguous()
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()
