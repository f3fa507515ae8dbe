"""Paged latent KV cache: the writer side of the format `flash_dmla_paged_decode` reads.

The reference only says that the decode path should "consume K_lat/V_lat from the
KV-cache" (README.md:15); it ships no cache.  This module defines one on the device
format the kernels use - a pool `[num_pages, page_size, d_qk]` of latent rows, a page
table `[max_seqs, max_pages]` int32 and sequence lengths `[max_seqs]` int32 - with a
host-side page allocator:

    cache = PagedLatentCache(num_pages, page_size=64, d_qk=576, max_seqs=128, max_pages_per_seq=64)
    slot = cache.new_sequence()
    cache.append([slot], rows)               # rows [1, n_tokens, d_qk]: prefill or one decode step
    O, m, l = cache.decode(Q, [slot], d_v=512, scale=...)
    cache.free_sequence(slot)

Page bookkeeping (free list, lengths, the host copy of the page table) is plain Python and
runs without a GPU (`device="cpu"`: the pool then only exists as metadata and `append`
needs `rows=None`); the row copies and the attention run through the CUDA library.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import ops
from ._lib import FlashDMLAError


class PagedLatentCache:
    def __init__(self, num_pages: int, page_size: int, d_qk: int, max_seqs: int, max_pages_per_seq: int,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if num_pages <= 0 or page_size <= 0 or d_qk <= 0 or max_seqs <= 0 or max_pages_per_seq <= 0:
            raise FlashDMLAError("cache dimensions must be positive")
        self.num_pages, self.page_size, self.d_qk = int(num_pages), int(page_size), int(d_qk)
        self.max_seqs, self.max_pages = int(max_seqs), int(max_pages_per_seq)
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        self.pool = (torch.zeros(num_pages, page_size, d_qk, dtype=dtype, device=self.device) if self.on_gpu else None)
        # host truth, device mirror (the kernels read the mirror)
        self.h_table = torch.zeros(max_seqs, max_pages_per_seq, dtype=torch.int32)
        self.h_len = torch.zeros(max_seqs, dtype=torch.int32)
        self.d_table = self.h_table.to(self.device) if self.on_gpu else None
        self.d_len = self.h_len.to(self.device) if self.on_gpu else None
        self._free_pages: List[int] = list(range(num_pages - 1, -1, -1))      # pop() hands out page 0 first
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self._live = [False] * max_seqs
        self._pages_of: List[List[int]] = [[] for _ in range(max_seqs)]

    # ------------------------------------------------------------------ allocator (host only)
    @property
    def free_pages(self) -> int:
        return len(self._free_pages)

    def length(self, slot: int) -> int:
        self._check_slot(slot)
        return int(self.h_len[slot])

    def pages_of(self, slot: int) -> List[int]:
        self._check_slot(slot)
        return list(self._pages_of[slot])

    def new_sequence(self) -> int:
        if not self._free_slots:
            raise FlashDMLAError("no free sequence slot")
        slot = self._free_slots.pop()
        self._live[slot] = True
        self.h_len[slot] = 0
        return slot

    def free_sequence(self, slot: int) -> None:
        self._check_slot(slot)
        self._free_pages.extend(reversed(self._pages_of[slot]))
        self._pages_of[slot] = []
        self.h_len[slot] = 0
        self.h_table[slot].zero_()
        self._live[slot] = False
        self._free_slots.append(slot)
        self._sync_rows([slot])

    def reserve(self, slots: Sequence[int], n_tokens: int) -> torch.Tensor:
        """Make room for n_tokens more rows in every listed sequence (allocating pages as needed),
        advance the lengths and return the positions the new rows start at, [len(slots)] int32.
        Nothing is changed if any sequence cannot be extended."""
        if n_tokens < 0:
            raise FlashDMLAError("n_tokens must be >= 0")
        if len(set(slots)) != len(slots):
            raise FlashDMLAError("a sequence may appear only once per append")
        need = []
        for s in slots:
            self._check_slot(s)
            have = len(self._pages_of[s])
            want = (int(self.h_len[s]) + n_tokens + self.page_size - 1) // self.page_size
            if want > self.max_pages:
                raise FlashDMLAError(f"sequence {s} would exceed max_pages_per_seq = {self.max_pages}")
            need.append(max(0, want - have))
        if sum(need) > len(self._free_pages):
            raise FlashDMLAError(f"out of cache pages: need {sum(need)}, {len(self._free_pages)} free")
        start = torch.empty(len(slots), dtype=torch.int32)
        for i, (s, k) in enumerate(zip(slots, need)):
            for _ in range(k):
                pg = self._free_pages.pop()
                self.h_table[s, len(self._pages_of[s])] = pg
                self._pages_of[s].append(pg)
            start[i] = self.h_len[s]
            self.h_len[s] += n_tokens
        self._sync_rows(slots)
        return start

    # ------------------------------------------------------------------ device side
    def append(self, slots: Sequence[int], rows: Optional[torch.Tensor]) -> torch.Tensor:
        """Append rows [len(slots), n_tokens, d_qk] (the RoPE'd 64 columns after the 512 latent ones, as the
        decode kernel expects) to the listed sequences; returns their start positions."""
        if rows is None:
            raise FlashDMLAError("append needs the rows; use reserve() for bookkeeping only")
        if rows.dim() != 3 or rows.shape[0] != len(slots) or rows.shape[2] != self.d_qk:
            raise FlashDMLAError("rows must be [len(slots), n_tokens, d_qk]")
        if not self.on_gpu:
            raise FlashDMLAError("append needs a CUDA cache (there is no CPU fallback)")
        start = self.reserve(slots, rows.shape[1])
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        ops.cache_append(rows, self.pool, self.d_table.index_select(0, idx), start.to(self.device))
        return start

    def tables(self, slots: Sequence[int]):
        """(page_table [n, max_pages], seqlens [n]) on the device for the listed sequences."""
        if not self.on_gpu:
            raise FlashDMLAError("device tables need a CUDA cache")
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        return self.d_table.index_select(0, idx), self.d_len.index_select(0, idx)

    def decode(self, Q: torch.Tensor, slots: Sequence[int], d_v: int, scale: Optional[float] = None, **kw):
        """One decode step of the listed sequences: Q [len(slots), H, d_qk] -> (O, m, l)."""
        table, lens = self.tables(slots)
        longest = max((int(self.h_len[s]) for s in slots), default=0)
        return ops.flash_dmla_paged_decode(Q, self.pool, table, lens, d_v, scale, max_seqlen=max(longest, 1), **kw)

    def gather(self, slots: Sequence[int], n_tokens: int) -> torch.Tensor:
        table, lens = self.tables(slots)
        return ops.cache_gather(self.pool, table, lens, n_tokens)

    # ------------------------------------------------------------------ helpers
    def _check_slot(self, slot: int) -> None:
        if not (0 <= slot < self.max_seqs) or not self._live[slot]:
            raise FlashDMLAError(f"sequence slot {slot} is not live")

    def _sync_rows(self, slots: Sequence[int]) -> None:
        if not self.on_gpu or not slots:
            return
        idx = torch.tensor(list(slots), dtype=torch.long)
        didx = idx.to(self.device)
        self.d_table.index_copy_(0, didx, self.h_table.index_select(0, idx).to(self.device))
        self.d_len.index_copy_(0, didx, self.h_len.index_select(0, idx).to(self.device))
