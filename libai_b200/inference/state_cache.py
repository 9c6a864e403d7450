"""Per-sequence state of the stateful sequence mixers, kept in slots.

A model registers one entry per layer run (a layer that is run several times in a row keeps one state per pass):

* ``"latent"`` — a ring of the last ``ring_len`` low-rank key/value latents, ``[slots, ring_len, C]`` in the compute dtype
  (position ``p`` lives at ``p % ring_len``; a sliding window never needs more than its own length);
* ``"kv"`` — a ring of the last ``ring_len`` key/value rows of an attention layer whose mask reaches back a bounded number
  of positions, ``[slots, ring_len, C]`` (position ``p`` at ``p % ring_len``), and the rows of the first ``first_len``
  positions, ``[slots, first_len, C]``, which a mask that keeps the first tokens goes on reading after they left the ring;
* ``"recurrent"`` — the matrix state of a delta-rule or linear-attention layer, ``[slots, H, D, V]`` in fp32, and the last
  ``taps - 1`` inputs of its short convolutions, ``[slots, taps - 1, C]`` (empty for a layer without convolutions);
* ``"token"`` — the last token of the sequence, ``[slots]`` int32 (an embedding that looks at the previous token);
* ``"paged"`` — the key/value rows of an attention layer that sees the whole past: a pool ``[pages, page_size, C]`` in the compute
  dtype, shared by all sequences, and the last ``taps - 1`` inputs of the layer's short convolutions,
  ``[slots, taps - 1, conv_channels]``.  Position ``p`` of a sequence lives in row ``p % page_size`` of page
  ``page_table[slot, p // page_size]``; all paged entries share one page table (a page id names the same page of every pool).
  Pages are handed to a sequence as it grows (:meth:`SequenceStateCache.prepare`, before the step that needs them) and go
  back to the free list with its slot; a reused page is not cleared.  The pools grow (doubling) when the free list is empty.

A request holds one slot in every entry from its first token until it is finished.  Slots are handed out from a free list
and reused as they come back; a reused slot is not cleared — the kernels ignore a slot's contents for a sequence whose
``past`` is 0.  The cache grows (doubling) when more sequences are live than it has slots.
"""
from __future__ import annotations

from typing import Dict, List

import torch


class SequenceStateCache:
    def __init__(self, device, dtype, max_slots: int = 4, page_size: int = 64):
        self.device, self.dtype = torch.device(device), dtype
        self.page_size = max(1, int(page_size))
        self.num_pages = 0                                    # pages of every paged pool
        self.page_table = torch.zeros(max(1, int(max_slots)), 1, dtype=torch.int32, device=self.device)
        self._table_host = torch.zeros(max(1, int(max_slots)), 1, dtype=torch.int32)
        self._pages: Dict[int, List[int]] = {}                # live slot -> its pages, in order
        self._free_pages: List[int] = []
        self._paged = False
        self.capacity = max(1, int(max_slots))
        self._specs: List[dict] = []
        self._bufs: List[Dict[str, torch.Tensor]] = []
        self._free: List[int] = list(range(self.capacity - 1, -1, -1))
        self.length: Dict[int, int] = {}                      # live slot -> tokens folded into its state
        self.generation = 0                                   # bumped when the buffers move (captured graphs are stale then)

    # ------------------------------------------------------------------ layout
    def register(self, kind: str, **shape) -> int:
        """Add one entry; returns its handle.  ``latent``: ``ring_len, channels``; ``kv``: ``ring_len, first_len, channels``;
        ``recurrent``: ``heads, dim, vdim, taps, conv_channels``; ``token``: nothing; ``paged``: ``channels, taps,
        conv_channels``."""
        assert kind in ("latent", "kv", "recurrent", "token", "paged"), kind
        self._paged = self._paged or kind == "paged"
        self._specs.append(dict(kind=kind, **shape))
        self._bufs.append(self._make(self._specs[-1], self.capacity))
        return len(self._specs) - 1

    def _make(self, spec, n):
        if spec["kind"] == "latent":
            return {"ring": torch.zeros(n, spec["ring_len"], spec["channels"], dtype=self.dtype, device=self.device)}
        if spec["kind"] == "kv":
            return {"ring": torch.zeros(n, spec["ring_len"], spec["channels"], dtype=self.dtype, device=self.device),
                    "first": torch.zeros(n, spec["first_len"], spec["channels"], dtype=self.dtype, device=self.device)}
        if spec["kind"] == "token":
            return {"last": torch.zeros(n, dtype=torch.int32, device=self.device)}
        if spec["kind"] == "paged":
            return {"pool": torch.zeros(self.num_pages, self.page_size, spec["channels"], dtype=self.dtype, device=self.device),
                    "tail": torch.zeros(n, max(spec["taps"] - 1, 0), spec["conv_channels"], dtype=self.dtype, device=self.device)}
        return {
            "S": torch.zeros(n, spec["heads"], spec["dim"], spec["vdim"], dtype=torch.float32, device=self.device),
            "tail": torch.zeros(n, max(spec["taps"] - 1, 0), spec["conv_channels"], dtype=self.dtype, device=self.device),
        }

    def buffers(self, handle: int) -> Dict[str, torch.Tensor]:
        b = self._bufs[handle]
        if "pool" in b:
            return dict(b, table=self.page_table)             # with the table the pages of this entry are found by
        return b

    def bytes_per_slot(self) -> int:
        """Bytes of the per-slot state (the paged pools are counted by :meth:`bytes_per_token`)."""
        return sum(t[0].numel() * t.element_size() for b in self._bufs for name, t in b.items() if name != "pool")

    def bytes_per_token(self) -> int:
        return sum(b["pool"][0, 0].numel() * b["pool"].element_size() for b in self._bufs if "pool" in b and self.num_pages)

    # ------------------------------------------------------------------ slots
    def allocate(self, n: int = 1) -> List[int]:
        while len(self._free) < n:
            self._grow()
        slots = [self._free.pop() for _ in range(n)]
        for s in slots:
            self.length[s] = 0
            self._pages[s] = []
        return slots

    def free(self, slots) -> None:
        for s in slots:
            if s in self.length:
                del self.length[s]
                self._free.append(s)
                self._free_pages.extend(reversed(self._pages.pop(s, [])))

    def advance(self, slots, lens) -> None:
        for s, n in zip(slots, lens):
            self.length[s] += n

    def live(self) -> int:
        return len(self.length)

    # ------------------------------------------------------------------ pages
    def reserve(self, tokens: int) -> None:
        """Make room for ``tokens`` cached positions in all (a hint: the pools grow on demand anyway)."""
        if self._paged and tokens:
            want = -(-int(tokens) // self.page_size) + self.capacity
            if want > self.num_pages:
                self._grow_pages(want)

    def prepare(self, slots, lens) -> None:
        """Before a step that brings ``lens[i]`` tokens to ``slots[i]``: hand out the pages those positions fall into."""
        if not self._paged:
            return
        ps = self.page_size
        for s, n in zip(slots, lens):
            need = -(-(self.length[s] + n) // ps)
            mine = self._pages[s]
            if need <= len(mine):
                continue
            if need > self.page_table.shape[1]:
                self._widen_table(need)
            while len(mine) < need:
                if not self._free_pages:
                    self._grow_pages(max(2 * self.num_pages, need - len(mine), 4))
                page = self._free_pages.pop()
                self._table_host[s, len(mine)] = page
                mine.append(page)
            self.page_table[s].copy_(self._table_host[s])

    def _widen_table(self, width: int) -> None:
        width = max(width, 2 * self.page_table.shape[1])
        host = torch.zeros(self.capacity, width, dtype=torch.int32)
        host[:, : self._table_host.shape[1]] = self._table_host
        self._table_host = host
        self.page_table = host.to(self.device)
        self.generation += 1

    def _grow_pages(self, pages: int) -> None:
        old = self.num_pages
        self.num_pages = int(pages)
        for i, spec in enumerate(self._specs):
            if spec["kind"] == "paged":
                pool = torch.zeros(self.num_pages, self.page_size, spec["channels"], dtype=self.dtype, device=self.device)
                pool[:old].copy_(self._bufs[i]["pool"])
                self._bufs[i]["pool"] = pool
        self._free_pages = list(range(self.num_pages - 1, old - 1, -1)) + self._free_pages
        self.generation += 1

    def _grow(self):
        old, new = self.capacity, self.capacity * 2
        for i, spec in enumerate(self._specs):
            bigger = self._make(spec, new)
            for name, t in self._bufs[i].items():
                if name == "pool":                            # pages are not per slot
                    bigger[name] = t
                else:
                    bigger[name][:old].copy_(t)
            self._bufs[i] = bigger
        self._free = list(range(new - 1, old - 1, -1)) + self._free
        host = torch.zeros(new, self._table_host.shape[1], dtype=torch.int32)
        host[:old] = self._table_host
        self._table_host = host
        self.page_table = host.to(self.device)
        self.capacity = new
        self.generation += 1
