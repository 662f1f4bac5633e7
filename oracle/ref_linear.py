"""CPU restatement of nano_qwen's tensor-parallel linear layers.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Functional (not
``nn.Module``) restatement of ``src/nano_qwen/layers/linear.py`` of the
reference: where each rank's parameter rows/columns come from in the
checkpoint tensor, and what the forward pass of each layer kind computes.
It is validated against the reference's own modules through the fixtures in
``tests/golden`` (made by ``tests/golden/make_golden.py``).

All tensors are CPU tensors; matmuls are fp32 ``F.linear``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def divide(numerator: int, denominator: int) -> int:
    """Exact division; raises ``AssertionError`` otherwise (linear.py:7-9)."""
    assert numerator % denominator == 0
    return numerator // denominator


# ----------------------------- sharding ----------------------------------- #
def column_shard(full: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """Rows ``[rank*N/tp, (rank+1)*N/tp)`` of a ``[N, ...]`` tensor.

    ``ColumnParallelLinear.weight_loader`` (linear.py:65-70); also used for a
    1-D bias (dim 0).
    """
    shard = divide(full.shape[0], tp)
    return full.narrow(0, rank * shard, shard)


def row_shard(full: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """Columns ``[rank*K/tp, (rank+1)*K/tp)`` of ``[N, K]``; a 1-D bias whole.

    ``RowParallelLinear.weight_loader`` (linear.py:142-150).
    """
    if full.dim() == 1:
        return full
    shard = divide(full.shape[1], tp)
    return full.narrow(1, rank * shard, shard)


def merged_column_param(parts: list[torch.Tensor], rank: int, tp: int) -> torch.Tensor:
    """Per-rank parameter of ``MergedColumnParallelLinear`` (linear.py:87-93).

    Part *i* (``[output_sizes[i], K]``) contributes its ``rank``-th of ``tp``
    row chunks, placed at row offset ``sum(output_sizes[:i]) / tp``.
    """
    return torch.cat([p.chunk(tp, 0)[rank] for p in parts], dim=0)


def qkv_param(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """Per-rank parameter of ``QKVParallelLinear``: ``[q_r; k_r; v_r]`` (linear.py:114-128)."""
    return torch.cat([q.chunk(tp, 0)[rank], k.chunk(tp, 0)[rank], v.chunk(tp, 0)[rank]], dim=0)


def qkv_output_size(head_size: int, total_num_heads: int, total_num_kv_heads: int | None) -> int:
    """``(heads + 2*kv_heads) * head_size`` (linear.py:107-111)."""
    total_num_kv_heads = total_num_kv_heads or total_num_heads
    return (total_num_heads + 2 * total_num_kv_heads) * head_size


def block_rows(t: torch.Tensor, block: int = 128) -> int:
    return (t.shape[0] + block - 1) // block


# ----------------------------- forward ------------------------------------ #
def column_forward(x: torch.Tensor, w_rank: torch.Tensor, b_rank: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear(x, W_r, b_r)``, no collective (linear.py:72-73)."""
    return F.linear(x, w_rank, b_rank)


def row_forward_partial(x_rank: torch.Tensor, w_rank: torch.Tensor, bias: torch.Tensor | None, rank: int) -> torch.Tensor:
    """One rank's partial sum; the bias is added on rank 0 only (linear.py:153)."""
    return F.linear(x_rank, w_rank, bias if rank == 0 else None)


def row_forward(x_full: torch.Tensor, w_full: torch.Tensor, bias: torch.Tensor | None, tp: int) -> torch.Tensor:
    """All ranks' partials summed, i.e. the value after ``dist.all_reduce`` (linear.py:154-155)."""
    y = None
    for r in range(tp):
        part = row_forward_partial(row_shard(x_full, r, tp), row_shard(w_full, r, tp), bias, r)
        y = part if y is None else y + part
    return y
