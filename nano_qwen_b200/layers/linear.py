"""FP8 drop-in replacements for ``nano_qwen.layers.linear``.

Same class names, constructor signatures, public attributes and
``param.weight_loader(param, tensor[, shard_id])`` protocol as the reference
(nano_qwen ``src/nano_qwen/layers/linear.py:12-156``), so the model code and
``nano_qwen.utils.loader.load_model`` (``utils/loader.py:12-28``) work
unchanged.  What differs is the storage and the arithmetic:

* ``weight``            float8_e4m3fn ``[N_shard, K_shard]``
* ``weight_scale_inv``  float32 ``[ceil(N_shard/128), ceil(K_shard/128)]`` —
  one dequantisation multiplier per 128x128 block (the name FP8 block
  checkpoints use)
* ``bias``              optional, default dtype, as in the reference
* ``forward``           dynamic 1x128 activation quantisation + block-scaled
  FP8 GEMM on the tensor cores (``nano_qwen_b200.ops.fp8_linear``), bf16 out;
  ``RowParallelLinear`` then all-reduces exactly like the reference
  (``linear.py:152-156``).

Loading: an fp8 checkpoint tensor is sharded like the reference shards bf16
(element units); its ``weight_scale_inv`` is sharded with the same rule in
units of 128-blocks.  A bf16/fp16/fp32 checkpoint tensor given to ``weight``'s
loader is sharded first and quantised on the device, which also fills the
matching rows of ``weight_scale_inv``.  Shard boundaries must fall on
128-multiples whenever tp_size > 1 (true for every Qwen3 shape at tp <= 8).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from . import p2p_reduce, sym_reduce
from .quantized import QuantizedActivation

BLOCK = 128
FP8 = torch.float8_e4m3fn


def divide(numerator: int, denominator: int) -> int:
    """Exact integer division; ``AssertionError`` if not divisible (reference ``linear.py:7-9``)."""
    assert numerator % denominator == 0, f"{numerator} is not divisible by {denominator}"
    return numerator // denominator


def _blocks(n: int) -> int:
    return (n + BLOCK - 1) // BLOCK


def _is_quantised(t: torch.Tensor) -> bool:
    return t.dtype == FP8


class LinearBase(nn.Module):
    """Owns the FP8 parameters and the loader plumbing (reference ``linear.py:12-34``).

    ``input_size`` / ``output_size`` are the PER-RANK sizes, as in the
    reference; ``tp_dim`` is the sharded dimension of ``weight`` (0 = N,
    1 = K, None = replicated).
    """

    def __init__(self, input_size: int, output_size: int, bias: bool = False, tp_dim: int | None = None):
        super().__init__()
        self.tp_dim = tp_dim
        self.tp_rank = dist.get_rank()
        self.tp_size = dist.get_world_size()
        self.input_size = input_size
        self.output_size = output_size
        k_storage = (input_size + 15) // 16 * 16          # TMA needs 16-byte row strides
        storage = torch.empty(output_size, k_storage, dtype=FP8)
        self.weight = nn.Parameter(storage[:, :input_size], requires_grad=False)
        self.weight.weight_loader = self.weight_loader
        self.weight.block = (1, 1)
        self.weight_scale_inv = nn.Parameter(
            torch.ones(_blocks(output_size), _blocks(input_size), dtype=torch.float32), requires_grad=False)
        self.weight_scale_inv.weight_loader = self.weight_loader
        self.weight_scale_inv.block = (BLOCK, BLOCK)
        if bias:
            self.bias = nn.Parameter(torch.empty(output_size), requires_grad=False)
            self.bias.weight_loader = self.weight_loader
            self.bias.block = (1,)
        else:
            self.register_parameter("bias", None)

    # ---- helpers shared by the loaders -------------------------------------
    def _unit(self, param: nn.Parameter, dim: int) -> int:
        """Rows (dim 0) or columns (dim 1) of the logical weight that one index of ``param`` covers."""
        return param.block[dim] if dim < len(param.block) else 1

    def _to_units(self, param: nn.Parameter, dim: int, offset: int, size: int) -> tuple[int, int]:
        unit = self._unit(param, dim)
        if unit == 1:
            return offset, size
        if self.tp_size > 1 or offset != 0:
            assert offset % unit == 0 and size % unit == 0, (
                f"shard [{offset}, {offset + size}) along dim {dim} is not aligned to {unit}-blocks; "
                "block scales cannot be split across ranks")
        return offset // unit, _blocks(size)

    def _store(self, param: nn.Parameter, dst_offset: int, dst_size: int, dim: int, piece: torch.Tensor):
        """Writes ``piece`` into ``param[dst_offset : dst_offset+dst_size]`` along ``dim`` (element units of the logical weight)."""
        if param is self.weight and not _is_quantised(piece):
            self._quantise_into(piece, dst_offset, dst_size, dim)
            return
        off, size = self._to_units(param, dim, dst_offset, dst_size)
        param.data.narrow(dim, off, size).copy_(piece)

    def _quantise_into(self, piece: torch.Tensor, dst_offset: int, dst_size: int, dim: int):
        """bf16/fp16/fp32 checkpoint shard -> FP8 rows + their block scales, on the device."""
        if not self.weight.is_cuda:
            raise RuntimeError("quantising an unquantised checkpoint tensor needs the module on a CUDA device "
                               "(no CPU fallback); load pre-quantised float8 tensors instead")
        wq, sw = ops.weight_quant(piece.to(device=self.weight.device, dtype=torch.bfloat16))
        self.weight.data.narrow(dim, dst_offset, dst_size).copy_(wq)
        off, size = self._to_units(self.weight_scale_inv, dim, dst_offset, dst_size)
        self.weight_scale_inv.data.narrow(dim, off, size).copy_(sw)

    def _linear(self, x, bias: torch.Tensor | None) -> torch.Tensor:
        if isinstance(x, QuantizedActivation):       # a fused producer already quantised it: GEMM only
            y = ops.fp8_gemm(x.xq, x.sx, self.weight, self.weight_scale_inv, bias)
            return y.view(*x.shape[:-1], y.shape[-1])
        return ops.fp8_linear(x, self.weight, self.weight_scale_inv, bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class ReplicatedLinear(LinearBase):
    """Unsharded layer (reference ``linear.py:37-51``)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        super().__init__(input_size, output_size, bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        self._store(param, 0, self.output_size, 0, loaded_weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._linear(x, self.bias)


class ColumnParallelLinear(LinearBase):
    """Output features split across ranks; no collective (reference ``linear.py:54-73``)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        tp_size = dist.get_world_size()
        super().__init__(input_size, divide(output_size, tp_size), bias, 0)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        # rank r takes rows [r*N/tp, (r+1)*N/tp) of the checkpoint tensor (weight, scale rows or bias)
        shard = self.output_size
        src_off, src_size = (self.tp_rank * shard, shard)
        if not (param is self.weight and not _is_quantised(loaded_weight)):
            src_off, src_size = self._to_units(param, 0, src_off, src_size)
        self._store(param, 0, shard, 0, loaded_weight.narrow(0, src_off, src_size))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._linear(x, self.bias)


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel matrices sharing one input, e.g. gate and up (reference ``linear.py:76-93``).

    The per-rank parameter is ``[part0_r; part1_r; ...]``.
    """

    def __init__(self, input_size: int, output_sizes: list[int], bias: bool = False):
        self.output_sizes = output_sizes
        super().__init__(input_size, sum(output_sizes), bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: int):
        shard_offset = sum(self.output_sizes[:loaded_shard_id]) // self.tp_size
        shard_size = self.output_sizes[loaded_shard_id] // self.tp_size
        piece = loaded_weight.chunk(self.tp_size, 0)[self.tp_rank]
        self._store(param, shard_offset, shard_size, 0, piece)


class QKVParallelLinear(ColumnParallelLinear):
    """Fused q/k/v projection, heads split across ranks (reference ``linear.py:96-128``).

    The per-rank parameter is ``[q_r; k_r; v_r]``.
    """

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: int | None = None, bias: bool = False):
        tp_size = dist.get_world_size()
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        self.head_size = head_size
        self.num_heads = divide(total_num_heads, tp_size)
        self.num_kv_heads = divide(total_num_kv_heads, tp_size)
        super().__init__(hidden_size, (total_num_heads + 2 * total_num_kv_heads) * head_size, bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: str):
        assert loaded_shard_id in ["q", "k", "v"]
        q_rows = self.num_heads * self.head_size
        kv_rows = self.num_kv_heads * self.head_size
        shard_offset, shard_size = {"q": (0, q_rows), "k": (q_rows, kv_rows), "v": (q_rows + kv_rows, kv_rows)}[loaded_shard_id]
        piece = loaded_weight.chunk(self.tp_size, 0)[self.tp_rank]
        self._store(param, shard_offset, shard_size, 0, piece)


class RowParallelLinear(LinearBase):
    """Input features split across ranks; partial outputs summed (reference ``linear.py:131-156``).

    How the sum is formed depends on the size of the output (always the same bits on every rank):

    * decode-sized outputs on an NCCL group of 2..8 ranks: one kernel per rank pushes the partial into every peer's
      inbox and adds what arrived, fp32 accumulation in rank order (``p2p_reduce``; ``p2p_reduce = False`` or
      ``NQ_P2P_REDUCE=0`` keeps NCCL);
    * prefill-sized outputs (at least ``overlap_min_rows`` token rows, eager mode) on 2 or 8 ranks, or on 4 ranks on
      request (``sym_reduce = True``): the GEMM writes its partial output into a peer-mapped buffer and one kernel
      per rank sums it over the group (``sym_reduce.py``: a two-shot exchange done with bulk copies over NVLink, 32
      thread blocks).  Measured on B200s for 64 MiB: 219 us against NCCL's 274 us on 8 ranks, 140 us against 152 us
      on 2; the 36-layer prefill + decode step 31.4 ms against 35.3 ms on 8 ranks, 1-3 % faster on 2 (46.9 ms against
      48.5 ms on one box, 48.9-49.0 ms against 49.4-49.8 ms on another), and 35.6 ms against 35.4 ms on 4, which
      therefore keep NCCL.  ``sym_reduce = False`` or ``NQ_SYM_REDUCE=0`` keeps
      NCCL everywhere;
    * anything else: NCCL's all-reduce, as in the reference.

    With ``overlap_chunks`` > 1 the GEMM runs in chunks of token rows and the exchange of chunk *i* runs on a second
    stream beside the GEMM of chunk *i + 1*, which leaves it its SMs.  Measured slower than one GEMM followed by one
    exchange (2 ranks: 49.2 ms against 44.7 ms with NCCL; 8 ranks: 33.2 ms against 32.1 ms), so the default is one chunk.
    """

    p2p_reduce = True            # small outputs are summed over peer memory instead of NCCL (see p2p_reduce.py)
    sym_reduce = None            # large outputs over a peer-mapped buffer (see sym_reduce.py): None = on 2 and 8 ranks
    sym_auto_ranks = (2, 8)      # group sizes where that measured faster than NCCL on B200s
    overlap_chunks = 1
    overlap_min_rows = 2048      # smaller batches take one GEMM and one reduction
    overlap_chunk_rows = 1024    # a chunk is never smaller than this (and always a multiple of 128 rows)

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        tp_size = dist.get_world_size()
        super().__init__(divide(input_size, tp_size), output_size, bias, 1)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        if param.data.ndim == 1:            # the bias is replicated; only rank 0 adds it
            param.data.copy_(loaded_weight)
            return
        shard = self.input_size
        src_off, src_size = (self.tp_rank * shard, shard)
        if not (param is self.weight and not _is_quantised(loaded_weight)):
            src_off, src_size = self._to_units(param, 1, src_off, src_size)
        self._store(param, 0, shard, 1, loaded_weight.narrow(1, src_off, src_size))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bias = self.bias if self.tp_rank == 0 else None          # added once, before the sum
        if self.tp_size == 1:
            return self._linear(x, bias)
        rows = math.prod(x.shape[:-1])
        use_sym = self.sym_reduce if self.sym_reduce is not None else self.tp_size in self.sym_auto_ranks
        if (use_sym and x.is_cuda and rows >= self.overlap_min_rows
                and not torch.cuda.is_current_stream_capturing()):
            sym = sym_reduce.get_reducer()
            if sym is not None and sym.fits(rows, self.output_size):
                return self._forward_overlapped(x, bias, rows, sym)
        y = self._linear(x, bias)
        reducer = p2p_reduce.get_reducer() if (self.p2p_reduce and x.is_cuda) else None
        if reducer is not None and reducer.fits(y):
            reducer.reduce_(y)               # decode-sized: one kernel over peer memory
        else:
            dist.all_reduce(y)
        return y

    def _forward_overlapped(self, x, bias, rows: int, sym) -> torch.Tensor:
        """The partial output goes to the peer-mapped buffer and is summed from there; with several chunks of token
        rows, the GEMM of chunk i + 1 runs on the current stream beside the exchange of chunk i."""
        if isinstance(x, QuantizedActivation):
            xq, sx, lead = x.xq, x.sx, x.shape[:-1]
        else:
            x2 = x.reshape(rows, x.shape[-1])
            if x2.dtype != torch.bfloat16:
                x2 = x2.to(torch.bfloat16)
            xq, sx = ops.act_quant(x2)                   # one quantiser launch for all chunks
            lead = x.shape[:-1]
        n = self.output_size
        part = sym.partial(rows, n)
        y = torch.empty((rows, n), dtype=torch.bfloat16, device=xq.device)
        chunks = max(1, min(self.overlap_chunks, rows // self.overlap_chunk_rows))
        if chunks == 1:                                  # one GEMM on every SM, then one exchange, on this stream
            ops.fp8_gemm(xq, sx, self.weight, self.weight_scale_inv, bias, out=part)
            sym.reduce_pull(part, y)
            return y.view(*lead, n)
        step = ((rows + chunks - 1) // chunks + 127) // 128 * 128
        main = torch.cuda.current_stream()
        old = ops.set_sm_reserve(sym.blocks)             # the GEMMs leave the exchange kernel its SMs
        try:
            for lo in range(0, rows, step):
                hi = min(lo + step, rows)
                ops.fp8_gemm(xq[lo:hi], sx[lo:hi], self.weight, self.weight_scale_inv, bias, out=part[lo:hi])
                done = torch.cuda.Event()
                done.record(main)
                sym.stream.wait_event(done)
                with torch.cuda.stream(sym.stream):
                    sym.reduce_pull(part[lo:hi], y[lo:hi])
        finally:
            ops.set_sm_reserve(old)
        main.wait_stream(sym.stream)
        return y.view(*lead, n)
