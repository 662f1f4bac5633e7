"""Row-parallel SUM over peer memory for decode-sized outputs (``nq_row_reduce_p2p``).

Stands in for the ``dist.all_reduce(y)`` that ends the reference's ``RowParallelLinear.forward``
(``nano_qwen/layers/linear.py:154-155``) when ``y`` is small: NCCL's all-reduce costs a fixed latency per call that
dominates a 16-512 KiB message, one kernel that pushes the partial to every peer over NVLink (data and call number in the same 8-byte words) and
adds what the peers pushed does not.  Larger messages keep NCCL (a one-shot exchange moves ``tp - 1`` copies of the message per GPU).

``torch.distributed`` is only the plumbing: it carries the 64-byte IPC handles between the ranks at set-up.
All ranks must be processes on one node, one GPU each.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _cabi

_HANDLE_BYTES = 64             # NQ_P2P_HANDLE_BYTES


class P2PRowReducer:
    """One per process: inbox and call counter of this rank plus the mapped inboxes of the peers."""

    def __init__(self, slot_bytes: int, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.tp = dist.get_world_size(group)
        if not 2 <= self.tp <= 8:
            raise ValueError("peer-memory reduction needs 2..8 ranks")
        self.slot_bytes = (int(slot_bytes) + 255) // 256 * 256
        lib = _cabi.lib()

        def alloc(nbytes: int) -> int:
            ptr = ctypes.c_void_p()
            _cabi.check(lib.nq_p2p_alloc(nbytes, ctypes.byref(ptr)), "nq_p2p_alloc")
            return ptr.value

        # a slot holds the message twice over: every 8-byte word is 4 bytes of data + the call number
        inbox = alloc(2 * self.tp * 2 * self.slot_bytes)
        self._state = alloc(256)
        handle = (ctypes.c_ubyte * _HANDLE_BYTES)()
        _cabi.check(lib.nq_p2p_export(inbox, handle), "nq_p2p_export")
        gathered = [None] * self.tp
        dist.all_gather_object(gathered, bytes(handle), group=group)
        ptrs = []
        for r in range(self.tp):
            if r == self.rank:
                ptrs.append(inbox)
                continue
            raw = (ctypes.c_ubyte * _HANDLE_BYTES).from_buffer_copy(gathered[r])
            ptr = ctypes.c_void_p()
            _cabi.check(lib.nq_p2p_import(raw, ctypes.byref(ptr)), "nq_p2p_import")
            ptrs.append(ptr.value)
        self._inbox = (ctypes.c_void_p * self.tp)(*ptrs)   # kept for the life of the process (never unmapped)
        dist.barrier(group=group)          # every inbox exists and is zero before anyone pushes

    def fits(self, y: torch.Tensor) -> bool:
        n = y.numel()
        return (y.dtype == torch.bfloat16 and y.is_contiguous() and n % 8 == 0 and n * 2 <= self.slot_bytes
                and y.data_ptr() % 16 == 0)

    def reduce_(self, y: torch.Tensor) -> torch.Tensor:
        """In-place SUM of ``y`` over the ranks; enqueued on the current stream (capturable)."""
        st = _cabi.lib().nq_row_reduce_p2p(y.data_ptr(), y.data_ptr(), y.numel(), self._inbox, self.rank,
                                           self.tp, self.slot_bytes, self._state,
                                           torch.cuda.current_stream().cuda_stream)
        _cabi.check(st, "nq_row_reduce_p2p")
        return y


_reducer: P2PRowReducer | None = None
_reducer_failed = False


def max_message_bytes(tp: int) -> int:
    """Largest ``y`` the peer-memory path takes.  A one-shot exchange receives ``tp - 1`` messages per GPU, so the
    limit shrinks with the number of ranks: 2 MiB of inbound traffic per call, except where a larger message was
    measured to win on B200s (4 ranks: 1 MiB takes 19.5 us against 25.2 us for NCCL, 1.5 MiB loses 31 to 26).
    ``NQ_P2P_REDUCE_MAX_BYTES`` overrides."""
    env = os.environ.get("NQ_P2P_REDUCE_MAX_BYTES")
    if env is not None:
        return int(env)
    if tp == 4:
        return 1 << 20
    return (2 << 20) // max(tp - 1, 1)


# Group sizes on which the peer-memory path has been run and checked against NCCL on B200s; it is the default there.
MEASURED_GROUP_SIZES = (2, 4, 8)


def get_reducer() -> P2PRowReducer | None:
    """The process-wide reducer of the default group, created on first use (a collective call: every rank reaches
    it in its first row-parallel forward).  ``NQ_P2P_REDUCE=0`` keeps NCCL for every size; ``NQ_P2P_REDUCE=1`` turns
    the peer-memory path on for any group of 2..8 ranks; unset, it is on for the group sizes it has been measured on."""
    global _reducer, _reducer_failed
    if _reducer is not None or _reducer_failed:
        return _reducer
    mode = os.environ.get("NQ_P2P_REDUCE", "")
    if mode == "0" or not dist.is_initialized() or dist.get_backend() != "nccl":
        _reducer_failed = True
        return None
    tp = dist.get_world_size()
    if not 2 <= tp <= 8 or (mode != "1" and tp not in MEASURED_GROUP_SIZES):
        _reducer_failed = True
        return None
    if torch.cuda.is_current_stream_capturing():
        return None                        # set-up allocates and talks to the peers: not during a capture
    _reducer = P2PRowReducer(max_message_bytes(tp))
    return _reducer


def init() -> bool:
    """Creates the peer-memory reducer now instead of inside the first row-parallel ``forward``.

    A collective call (every rank of the default group must make it) that allocates and exchanges handles, so it
    must not happen during CUDA-graph capture: a model runner calls it once after ``init_process_group`` and before
    ``capture_cudagraph``; otherwise a first forward that happens under capture keeps NCCL for that graph.
    Returns whether the peer-memory path is in use.
    """
    return get_reducer() is not None
