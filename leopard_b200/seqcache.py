"""Cache and state manager of the decoder-only language models (leopard_b200/seqlm.py).

Two kinds of per-request memory, both owned here and handed to the kernels as pools plus small index tables:

* a PAGED row cache for attention layers: pages of `page_size` token rows; every caching layer has its own pool
  [pages, page_size, row width] fp32 and all layers share one page numbering, so a request needs one page table.  Layers with a
  sliding window never look further back than their window, so pages that have fallen out of every layer's window are given back
  while the request is still running: a windowed model's cache per request is bounded by its largest window, not by its length.
  A layer may also keep its first `keep_first` tokens visible for ever: the pages that hold them are never given back.
* SUMMARY pools for layers that see far-away tokens only as one row per block of `every` tokens (pooled attention): the same paging,
  one row per block, a page table of its own per distinct block size, kept for the whole life of the request (a request of n tokens
  holds n / every rows there).  The token pages such a layer still needs are the window AND the block that is being filled, so the
  caller passes max(window, every) as that layer's look-back.
* a SLOT pool for recurrent layers: one fp32 state (any shape, [heads, dim, vdim] for retention, [width] for a gated recurrence) per
  (layer, slot).  A slot is not cleared when it is handed
  out again: the kernels start a request at position 0 from a zero state without reading the slot.

Pools grow (by reallocation) when a batch needs more than the configured size; `max_tokens` only sizes the first allocation.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence as Seq

import torch


@dataclass
class Sequence:
    key: Hashable
    slot: int
    length: int = 0                       # tokens already in the cache / state
    pages: List[int] = field(default_factory=list)   # page of logical block i, -1 once it has been given back
    summary_pages: List[List[int]] = field(default_factory=list)   # per summary stream: pages of block rows


class SequenceCache:
    def __init__(self, row_widths: Seq[int], state_shapes: Seq[Seq[int]], window: Optional[int], device, max_tokens: int = 4096,
                 page_size: int = 64, max_seqs: int = 8, keep_first: int = 0, summaries: Seq[Seq[int]] = ()):
        """row_widths[i]: floats per token of caching layer i; state_shapes[j]: state shape of recurrent layer j;
        window: the largest look-back (tokens, the current one included) of all caching layers, None if one of them sees everything;
        keep_first: the most first tokens any layer keeps visible; summaries[k] = (floats per row, tokens per row) of summary pool k."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.device = torch.device(device)
        self.page_size = int(page_size)
        self.window = window
        self.row_widths = [int(w) for w in row_widths]
        self.state_shapes = [tuple(int(x) for x in s) for s in state_shapes]
        self.n_pages = 0
        self.n_slots = 0
        self.pools: List[torch.Tensor] = [torch.empty((0, self.page_size, w), dtype=torch.float32, device=self.device) for w in self.row_widths]
        self.states: List[torch.Tensor] = [torch.empty((0, *s), dtype=torch.float32, device=self.device) for s in self.state_shapes]
        self.free_pages: List[int] = []
        self.free_slots: List[int] = []
        self.seqs: Dict[Hashable, Sequence] = {}
        self.generation = 0                # bumped whenever a pool is reallocated (captured pointers become stale)
        self.keep_first = int(keep_first)
        # summary streams: one per distinct block size; summary pool k is pool summary_index[k][1] of stream summary_index[k][0]
        self.summary_every: List[int] = sorted({int(e) for _, e in summaries})
        if any(e <= 0 for e in self.summary_every):
            raise ValueError("a summary pool needs a positive block size")
        self.summary_widths: List[List[int]] = [[] for _ in self.summary_every]
        self.summary_index: List[tuple] = []
        for w, e in summaries:
            k = self.summary_every.index(int(e))
            self.summary_index.append((k, len(self.summary_widths[k])))
            self.summary_widths[k].append(int(w))
        self.summary_pools: List[List[torch.Tensor]] = [[torch.empty((0, self.page_size, w), dtype=torch.float32, device=self.device)
                                                         for w in ws] for ws in self.summary_widths]
        self.summary_n_pages: List[int] = [0] * len(self.summary_every)
        self.summary_free: List[List[int]] = [[] for _ in self.summary_every]
        for k, e in enumerate(self.summary_every):
            self._grow_summary(k, -(-max(int(max_tokens) // e, 1) // self.page_size) + max_seqs)
        if self.row_widths:
            self._grow_pages(-(-max(int(max_tokens), 1) // self.page_size) + max_seqs)
        self._grow_slots(max_seqs)

    # ------------------------------------------------------------------ pools
    def _grow_pages(self, n_new: int):
        total = self.n_pages + n_new
        for i, w in enumerate(self.row_widths):
            pool = torch.empty((total, self.page_size, w), dtype=torch.float32, device=self.device)
            if self.n_pages:
                pool[: self.n_pages].copy_(self.pools[i])
            self.pools[i] = pool
        self.free_pages.extend(range(total - 1, self.n_pages - 1, -1))   # pop() hands out low numbers first
        self.n_pages = total
        self.generation += 1

    def _grow_summary(self, k: int, n_new: int):
        total = self.summary_n_pages[k] + n_new
        for i, w in enumerate(self.summary_widths[k]):
            pool = torch.empty((total, self.page_size, w), dtype=torch.float32, device=self.device)
            if self.summary_n_pages[k]:
                pool[: self.summary_n_pages[k]].copy_(self.summary_pools[k][i])
            self.summary_pools[k][i] = pool
        self.summary_free[k].extend(range(total - 1, self.summary_n_pages[k] - 1, -1))
        self.summary_n_pages[k] = total
        self.generation += 1

    def summary_pool(self, index: int) -> torch.Tensor:
        """The pool of summary layer `index` (the order of `summaries`)."""
        k, i = self.summary_index[index]
        return self.summary_pools[k][i]

    def _grow_slots(self, n_new: int):
        total = self.n_slots + n_new
        for j, s in enumerate(self.state_shapes):
            st = torch.zeros((total, *s), dtype=torch.float32, device=self.device)
            if self.n_slots:
                st[: self.n_slots].copy_(self.states[j])
            self.states[j] = st
        self.free_slots.extend(range(total - 1, self.n_slots - 1, -1))
        self.n_slots = total
        self.generation += 1

    # ------------------------------------------------------------------ requests
    def open(self, key: Hashable) -> Sequence:
        if key in self.seqs:
            raise KeyError(f"request {key!r} is already open")
        if not self.free_slots:
            self._grow_slots(max(4, self.n_slots))
        seq = Sequence(key=key, slot=self.free_slots.pop(), summary_pages=[[] for _ in self.summary_every])
        self.seqs[key] = seq
        return seq

    def get(self, key: Hashable) -> Optional[Sequence]:
        return self.seqs.get(key)

    def reserve(self, seq: Sequence, n_tokens: int) -> None:
        """Make sure pages exist for positions [seq.length, seq.length + n_tokens) and for the blocks they complete."""
        if not self.row_widths:
            return
        need = -(-(seq.length + n_tokens) // self.page_size)
        while len(seq.pages) < need:
            if not self.free_pages:
                self._grow_pages(max(8, self.n_pages // 2))
            seq.pages.append(self.free_pages.pop())
        for k, e in enumerate(self.summary_every):
            need = -(-((seq.length + n_tokens) // e) // self.page_size)
            while len(seq.summary_pages[k]) < need:
                if not self.summary_free[k]:
                    self._grow_summary(k, max(8, self.summary_n_pages[k] // 2))
                seq.summary_pages[k].append(self.summary_free[k].pop())

    def advance(self, seq: Sequence, n_tokens: int) -> None:
        """The step wrote n_tokens more; pages that no later query can see go back to the pool."""
        seq.length += n_tokens
        if self.window is None or not self.row_widths:
            return
        first_needed = seq.length - self.window + 1          # the oldest position the NEXT query (at seq.length) sees
        kept = -(-self.keep_first // self.page_size)           # pages that hold a token some layer keeps for ever
        for b in range(kept, min(len(seq.pages), max(first_needed, 0) // self.page_size)):
            if seq.pages[b] >= 0:
                self.free_pages.append(seq.pages[b])
                seq.pages[b] = -1

    def close(self, key: Hashable) -> None:
        seq = self.seqs.pop(key)
        self.free_pages.extend(p for p in seq.pages if p >= 0)
        for k, pages in enumerate(seq.summary_pages):
            self.summary_free[k].extend(pages)
        self.free_slots.append(seq.slot)

    def live_tokens(self) -> int:
        return sum(s.length for s in self.seqs.values())

    def pages_in_use(self) -> int:
        return self.n_pages - len(self.free_pages)
