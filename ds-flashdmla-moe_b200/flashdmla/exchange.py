"""Exchange and merge of the ranks' partial decode results in one kernel over NVLink peer memory.

`PeerExchange` is the host side of `fdmla_exchange_merge` (include/flashdmla.h): every rank of a node owns an
exchange buffer in device memory that its peers have mapped through CUDA IPC; one kernel launch per rank sends the
rows of the rank's message [O | m | l] to the ranks that own them, merges the rows it owns once its peers' have landed
and stores the merged rows into every peer's buffer - the fused form of `all_gather_into_tensor` + `merge_partials`,
with bit-identical results and a fraction of the NVLink traffic.  It stands where the reference's
MPI wrapper gathers on the host (csrc/attention/fa2_fwd_mpi.cu:65-74).  CUDA only; one process per GPU, all on one
node.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from ._lib import FlashDMLAError, check


class PeerExchange:
    """Exchange buffers of one process group for messages of `rows` rows of `d_v` columns.

    Collective: every rank of `group` must construct it at the same point (the IPC handles travel with
    `all_gather_object`, and a barrier follows).  `merge(msg, out)` is then one kernel launch per step on the current
    stream; every rank must issue the same sequence of steps.  After a time-out (device error flag 31) the object
    must be rebuilt on all ranks.
    """

    def __init__(self, rows: int, d_v: int, device, group: Optional[dist.ProcessGroup] = None, timeout_ms: int = 10000):
        device = torch.device(device)
        if device.type != "cuda":
            raise FlashDMLAError("PeerExchange needs CUDA devices (there is no CPU path)")
        self.rows, self.d_v, self.device, self.group, self.timeout_ms = int(rows), int(d_v), device, group, int(timeout_ms)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        L = _lib.lib()
        nbytes = L.fdmla_exchange_bytes(self.world, self.rows, self.d_v)
        if nbytes == 0:
            raise FlashDMLAError("unsupported exchange shape (world <= 16, d_v a multiple of 4)")
        self._own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        self._peers = {}
        self._bufs = (ctypes.c_void_p * self.world)()
        # Every rank goes through the same collectives whether its own set-up works or not; a failure anywhere is
        # agreed on with an all-reduce and raised on all ranks together, so that no rank is left in a barrier alone.
        failure = None
        with torch.cuda.device(device):
            rc = L.fdmla_exchange_alloc(nbytes, ctypes.byref(self._own), handle)
            if rc != 0:
                failure = f"fdmla_exchange_alloc failed with status {rc}"
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw) if failure is None else None, group=group)
            if failure is None and any(h is None for h in handles):
                failure = "a peer could not allocate its exchange buffer"
            if failure is None:
                for p in range(self.world):
                    if p == self.rank:
                        self._bufs[p] = self._own.value
                        continue
                    ptr = ctypes.c_void_p()
                    rc = L.fdmla_exchange_open(ctypes.create_string_buffer(handles[p], 64), ctypes.byref(ptr))
                    if rc != 0:
                        failure = f"fdmla_exchange_open of rank {p}'s buffer failed with status {rc} (CUDA IPC between the ranks' processes)"
                        break
                    self._peers[p] = ptr
                    self._bufs[p] = ptr.value
            ok = torch.tensor([0 if failure else 1], dtype=torch.int32, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                for ptr in self._peers.values():
                    L.fdmla_exchange_close(ptr)
                self._peers = {}
                dist.barrier(group=group)           # nobody frees a buffer that a peer may still be unmapping
                if self._own:
                    L.fdmla_exchange_free(self._own)
                    self._own = ctypes.c_void_p()
                raise FlashDMLAError("peer exchange not set up: " + (failure or "the set-up failed on another rank"))
        dist.barrier(group=group)       # every buffer is zeroed and mapped before anyone stores into it

    def merge(self, msg: torch.Tensor, out):
        """msg: this rank's fp32 message [rows * (d_v + 2)]; out = (O [..., d_v] fp32 or bf16, m, l fp32), contiguous."""
        O, m, l = out
        n = self.rows * (self.d_v + 2)
        if not (msg.is_cuda and msg.dtype == torch.float32 and msg.is_contiguous() and msg.numel() == n):
            raise FlashDMLAError("message must be a contiguous CUDA float32 tensor of rows * (d_v + 2) elements")
        if (O.numel() != self.rows * self.d_v or m.numel() != self.rows or l.numel() != self.rows
                or not (O.is_contiguous() and m.is_contiguous() and l.is_contiguous())
                or O.dtype not in (torch.float32, torch.bfloat16) or m.dtype != torch.float32 or l.dtype != torch.float32):
            raise FlashDMLAError("out tensors do not match the merged result")
        code = _lib.F32 if O.dtype == torch.float32 else _lib.BF16
        with torch.cuda.device(self.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            check(_lib.lib().fdmla_exchange_merge(msg.data_ptr(), self._bufs, self.world, self.rank, self.rows, self.d_v,
                                                  O.data_ptr(), m.data_ptr(), l.data_ptr(), code, self.timeout_ms, stream),
                  "fdmla_exchange_merge")
        return out

    def merge_parts(self, parts, msg: torch.Tensor, out):
        """The same step when the rank's own partial result is still in pieces: parts = (O_part [S, rows.., d_v], m_part,
        l_part [S, rows..]) fp32, dense (what `flash_dmla_paged_decode_partial(..., pieces_only=True)` leaves in its
        scratch).  The kernel first merges the pieces into `msg` (which it overwrites), then exchanges and merges as
        `merge` does: one launch for the local merge, the exchange and the final merge."""
        Op, mp, lp = parts
        S = Op.shape[0]
        n = self.rows * (self.d_v + 2)
        for t, k in ((Op, S * self.rows * self.d_v), (mp, S * self.rows), (lp, S * self.rows)):
            if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == k):
                raise FlashDMLAError("parts must be dense CUDA float32 tensors [S, rows, d_v], [S, rows], [S, rows]")
        if not (msg.is_cuda and msg.dtype == torch.float32 and msg.is_contiguous() and msg.numel() == n):
            raise FlashDMLAError("message must be a contiguous CUDA float32 tensor of rows * (d_v + 2) elements")
        O, m, l = out
        if (O.numel() != self.rows * self.d_v or m.numel() != self.rows or l.numel() != self.rows
                or not (O.is_contiguous() and m.is_contiguous() and l.is_contiguous())
                or O.dtype not in (torch.float32, torch.bfloat16) or m.dtype != torch.float32 or l.dtype != torch.float32):
            raise FlashDMLAError("out tensors do not match the merged result")
        code = _lib.F32 if O.dtype == torch.float32 else _lib.BF16
        with torch.cuda.device(self.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            check(_lib.lib().fdmla_exchange_merge_parts(Op.data_ptr(), mp.data_ptr(), lp.data_ptr(), int(S), msg.data_ptr(),
                                                        self._bufs, self.world, self.rank, self.rows, self.d_v,
                                                        O.data_ptr(), m.data_ptr(), l.data_ptr(), code, self.timeout_ms, stream),
                  "fdmla_exchange_merge_parts")
        return out

    def close(self):
        """Unmap the peers' buffers and free this rank's own (collective in effect: peers must have stopped using it)."""
        L = _lib.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for ptr in self._peers.values():
                L.fdmla_exchange_close(ptr)
            self._peers = {}
            if self._own:
                dist.barrier(group=self.group)      # nobody frees a buffer a peer still has mapped and in use
                L.fdmla_exchange_free(self._own)
                self._own = ctypes.c_void_p()
