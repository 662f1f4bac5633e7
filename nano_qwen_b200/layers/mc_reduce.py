"""Row-parallel SUM inside the NVLink switch for prefill-sized outputs (``nq_row_reduce_mc``).

Stands in for the ``dist.all_reduce(y)`` that ends the reference's ``RowParallelLinear.forward``
(``nano_qwen/layers/linear.py:154-155``) when ``y`` is large.  The row-parallel GEMM writes its partial output
straight into a buffer that is mapped on every GPU of the group and bound to an NVLink multicast address; one
kernel per rank then lets the switch add the copies (``multimem.ld_reduce``) and write the sum back into all of
them (``multimem.st``).  Per GPU one message leaves and one arrives, whatever the group size.

``torch.distributed`` is the plumbing: its symmetric-memory allocator provides the peer-mapped buffer, the
multicast address and the rendezvous between the ranks; the kernels only see raw pointers.  All ranks must be
processes on one node with NVLS-capable GPUs, one GPU each.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _cabi

PAD_BYTES = 3 * 160 * 8 * 4         # NQ_MC_PAD_BYTES
DEFAULT_CAPACITY = 192 << 20        # bytes of partial output the buffer can hold (16384 tokens x 6144 bf16)


class McRowReducer:
    """One per process: the symmetric partial-output buffer, its multicast address, signal pads and call counter."""

    def __init__(self, capacity_bytes: int = DEFAULT_CAPACITY, group=None, blocks: int = 48):
        import torch.distributed._symmetric_memory as symm_mem
        pg = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(pg)
        self.tp = dist.get_world_size(pg)
        if not 2 <= self.tp <= 8:
            raise ValueError("in-switch reduction needs 2..8 ranks")
        self.blocks = blocks
        dev = torch.device("cuda", torch.cuda.current_device())
        self.capacity = (int(capacity_bytes) + 4095) // 4096 * 4096
        self.buf = symm_mem.empty(self.capacity, dtype=torch.uint8, device=dev)
        handle = symm_mem.rendezvous(self.buf, pg.group_name)
        self.mc_base = int(handle.multicast_ptr or 0)
        if self.mc_base == 0:
            raise RuntimeError("the symmetric-memory allocator returned no multicast address (NVLS unavailable)")
        self._peer_bufs = [int(q) for q in handle.buffer_ptrs]
        self._pad = symm_mem.empty(PAD_BYTES, dtype=torch.uint8, device=dev)
        self._pad.zero_()
        pad_handle = symm_mem.rendezvous(self._pad, pg.group_name)
        self._pads = (ctypes.c_void_p * self.tp)(*[int(p) for p in pad_handle.buffer_ptrs])
        self._state = torch.zeros(16, dtype=torch.uint8, device=dev)
        self._handles = (handle, pad_handle)            # keep the mappings alive
        torch.cuda.synchronize()
        dist.barrier(group=pg)                          # every pad is zero before anyone signals

    def fits(self, rows: int, cols: int) -> bool:
        return rows * cols * 2 <= self.capacity and (rows * cols) % 8 == 0

    def partial(self, rows: int, cols: int, offset_bytes: int = 0) -> torch.Tensor:
        """A bf16 ``[rows, cols]`` view of the symmetric buffer for the GEMM to write its partial output into."""
        n = rows * cols * 2
        assert offset_bytes % 16 == 0 and offset_bytes + n <= self.capacity
        return self.buf[offset_bytes:offset_bytes + n].view(torch.bfloat16).view(rows, cols)

    def reduce_(self, part: torch.Tensor) -> torch.Tensor:
        """In-place SUM over the ranks of a tensor returned by :meth:`partial`; enqueued on the current stream
        (capturable).  Afterwards ``part`` holds the sum on every rank."""
        off = part.data_ptr() - self.buf.data_ptr()
        assert 0 <= off and off + part.numel() * 2 <= self.capacity and part.is_contiguous()
        st = _cabi.lib().nq_row_reduce_mc(self.mc_base + off, part.numel(), self._pads, self.rank, self.tp,
                                          self._state.data_ptr(), self.blocks, torch.cuda.current_stream().cuda_stream)
        _cabi.check(st, "nq_row_reduce_mc")
        return part


    def reduce_pull(self, part: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """SUM over the ranks of a tensor returned by :meth:`partial`, by loads from the peers' buffers (no multicast);
        the result goes to ``out`` (a private bf16 tensor of the same shape, allocated if not given)."""
        off = part.data_ptr() - self.buf.data_ptr()
        assert 0 <= off and off + part.numel() * 2 <= self.capacity and part.is_contiguous()
        if out is None:
            out = torch.empty(part.shape, dtype=torch.bfloat16, device=part.device)
        bufs = (ctypes.c_void_p * self.tp)(*[b + off for b in self._peer_bufs])
        st = _cabi.lib().nq_row_reduce_pull(bufs, out.data_ptr(), part.numel(), self._pads, self.rank, self.tp,
                                            self._state.data_ptr(), self.blocks, torch.cuda.current_stream().cuda_stream)
        _cabi.check(st, "nq_row_reduce_pull")
        return out


_reducer: McRowReducer | None = None
_failed = False


def get_reducer() -> McRowReducer | None:
    """The process-wide reducer of the default group, created on first use (a collective call).  ``NQ_MC_REDUCE=0``
    switches it off; if symmetric memory or the multicast address is unavailable the row layers keep NCCL."""
    global _reducer, _failed
    if _reducer is not None or _failed:
        return _reducer
    if os.environ.get("NQ_MC_REDUCE", "") == "0" or not dist.is_initialized() or dist.get_backend() != "nccl":
        _failed = True
        return None
    if not 2 <= dist.get_world_size() <= 8:
        _failed = True
        return None
    if torch.cuda.is_current_stream_capturing():
        return None                                     # set-up allocates and talks to the peers: not during a capture
    try:
        _reducer = McRowReducer(int(os.environ.get("NQ_MC_REDUCE_BYTES", DEFAULT_CAPACITY)),
                                blocks=int(os.environ.get("NQ_MC_REDUCE_BLOCKS", 48)))
    except Exception as exc:                            # no NVLS on this system: the reference's collective stays
        import warnings
        warnings.warn(f"in-switch row reduction unavailable, keeping NCCL: {exc}")
        _failed = True
    return _reducer


def init() -> bool:
    """Creates the reducer now (collective; call before CUDA-graph capture).  Returns whether it is in use."""
    return get_reducer() is not None
