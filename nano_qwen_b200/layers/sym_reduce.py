"""Row-parallel SUM over peer-mapped buffers for prefill-sized outputs (``nq_row_reduce_pull``).

Stands in for the ``dist.all_reduce(y)`` that ends the reference's ``RowParallelLinear.forward``
(``nano_qwen/layers/linear.py:154-155``) when ``y`` is large.  The row-parallel GEMM writes its partial output
straight into a buffer that every GPU of the group has mapped; one kernel per rank then sums its slice of the
message from all peers and collects the other slices' sums (a two-shot exchange done with loads over NVLink).
Measured on B200s for 64 MiB: 219 us on 8 GPUs with 32 thread blocks (more do not help) against NCCL's 274 us;
140 us on 2 GPUs against 152 us.  The kernel needs only a few dozen thread blocks, so it can also run on a second
stream beside the GEMM of the next chunk of token rows; that overlap measured slower than one GEMM followed by one
exchange and is off by default.

``torch.distributed`` is the plumbing: its symmetric-memory allocator provides the peer-mapped buffer and the
rendezvous between the ranks; the kernels only see raw pointers.  All ranks must be processes on one node, one
GPU each, with peer access between the GPUs.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _cabi

PAD_BYTES = 3 * 160 * 8 * 4         # NQ_SYM_PAD_BYTES
DEFAULT_CAPACITY = 192 << 20        # bytes of partial output the buffer can hold (16384 tokens x 6144 bf16)


class SymRowReducer:
    """One per process: the symmetric partial-output buffer, signal pads, call counter and the side stream."""

    def __init__(self, capacity_bytes: int = DEFAULT_CAPACITY, group=None, blocks: int = 32):
        import torch.distributed._symmetric_memory as symm_mem
        pg = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(pg)
        self.tp = dist.get_world_size(pg)
        if self.tp not in (2, 4, 8):
            raise ValueError("the peer-memory exchange is built for 2, 4 or 8 ranks")
        self.blocks = blocks
        dev = torch.device("cuda", torch.cuda.current_device())
        self.capacity = (int(capacity_bytes) + 4095) // 4096 * 4096
        self.buf = symm_mem.empty(self.capacity, dtype=torch.uint8, device=dev)
        handle = symm_mem.rendezvous(self.buf, pg.group_name)
        self._peer_bufs = [int(q) for q in handle.buffer_ptrs]
        self._pad = symm_mem.empty(PAD_BYTES, dtype=torch.uint8, device=dev)
        self._pad.zero_()
        pad_handle = symm_mem.rendezvous(self._pad, pg.group_name)
        self._pads = (ctypes.c_void_p * self.tp)(*[int(p) for p in pad_handle.buffer_ptrs])
        self._state = torch.zeros(16, dtype=torch.uint8, device=dev)
        self._handles = (handle, pad_handle)            # keep the mappings alive
        self.stream = torch.cuda.Stream(device=dev)     # the exchange runs here, beside the GEMM of the next chunk
        torch.cuda.synchronize()
        dist.barrier(group=pg)                          # every pad is zero before anyone signals

    def fits(self, rows: int, cols: int) -> bool:
        return rows * cols * 2 <= self.capacity and cols % 8 == 0

    def partial(self, rows: int, cols: int, offset_bytes: int = 0) -> torch.Tensor:
        """A bf16 ``[rows, cols]`` view of the symmetric buffer for the GEMM to write its partial output into."""
        n = rows * cols * 2
        assert offset_bytes % 16 == 0 and offset_bytes + n <= self.capacity
        return self.buf[offset_bytes:offset_bytes + n].view(torch.bfloat16).view(rows, cols)

    def reduce_pull(self, part: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """SUM over the ranks of a tensor returned by :meth:`partial` (or a row slice of one); the result goes to
        ``out`` (a private contiguous bf16 tensor of the same shape, allocated if not given).  Enqueued on the
        current stream; capturable."""
        off = part.data_ptr() - self.buf.data_ptr()
        assert 0 <= off and off + part.numel() * 2 <= self.capacity and part.is_contiguous()
        if out is None:
            out = torch.empty(part.shape, dtype=torch.bfloat16, device=part.device)
        assert out.is_contiguous() and out.numel() == part.numel()
        bufs = (ctypes.c_void_p * self.tp)(*[b + off for b in self._peer_bufs])
        st = _cabi.lib().nq_row_reduce_pull(bufs, out.data_ptr(), part.numel(), self._pads, self.rank, self.tp,
                                            self._state.data_ptr(), self.blocks, torch.cuda.current_stream().cuda_stream)
        _cabi.check(st, "nq_row_reduce_pull")
        return out


_reducer: SymRowReducer | None = None
_failed = False


def get_reducer() -> SymRowReducer | None:
    """The process-wide reducer of the default group, created on first use (a collective call).  ``NQ_SYM_REDUCE=0``
    switches it off; if symmetric memory is unavailable the row layers keep NCCL."""
    global _reducer, _failed
    if _reducer is not None or _failed:
        return _reducer
    if os.environ.get("NQ_SYM_REDUCE", "") == "0" or not dist.is_initialized() or dist.get_backend() != "nccl":
        _failed = True
        return None
    if dist.get_world_size() not in (2, 4, 8):
        _failed = True
        return None
    if torch.cuda.is_current_stream_capturing():
        return None                                     # set-up allocates and talks to the peers: not during a capture
    try:
        _reducer = SymRowReducer(int(os.environ.get("NQ_SYM_REDUCE_BYTES", DEFAULT_CAPACITY)),
                                 blocks=int(os.environ.get("NQ_SYM_REDUCE_BLOCKS", 32)))
    except Exception as exc:                            # no symmetric memory on this system: the reference's collective stays
        import warnings
        warnings.warn(f"peer-memory row reduction unavailable, keeping NCCL: {exc}")
        _failed = True
    return _reducer


def init() -> bool:
    """Creates the reducer now (collective; call before CUDA-graph capture).  Returns whether it is in use."""
    return get_reducer() is not None
