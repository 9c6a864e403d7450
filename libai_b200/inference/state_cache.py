"""Per-sequence state of the stateful sequence mixers, kept in slots.

A model registers one entry per layer run (a layer that is run several times in a row keeps one state per pass):

* ``"latent"`` — a ring of the last ``ring_len`` low-rank key/value latents, ``[slots, ring_len, C]`` in the compute dtype
  (position ``p`` lives at ``p % ring_len``; a sliding window never needs more than its own length);
* ``"kv"`` — a ring of the last ``ring_len`` key/value rows of an attention layer whose mask reaches back a bounded number
  of positions, ``[slots, ring_len, C]`` (position ``p`` at ``p % ring_len``), and the rows of the first ``first_len``
  positions, ``[slots, first_len, C]``, which a mask that keeps the first tokens goes on reading after they left the ring;
* ``"recurrent"`` — the matrix state of a delta-rule or linear-attention layer, ``[slots, H, D, V]`` in fp32, and the last
  ``taps - 1`` inputs of its short convolutions, ``[slots, taps - 1, C]`` (empty for a layer without convolutions);
* ``"token"`` — the last token of the sequence, ``[slots]`` int32 (an embedding that looks at the previous token).

A request holds one slot in every entry from its first token until it is finished.  Slots are handed out from a free list
and reused as they come back; a reused slot is not cleared — the kernels ignore a slot's contents for a sequence whose
``past`` is 0.  The cache grows (doubling) when more sequences are live than it has slots.
"""
from __future__ import annotations

from typing import Dict, List

import torch


class SequenceStateCache:
    def __init__(self, device, dtype, max_slots: int = 4):
        self.device, self.dtype = torch.device(device), dtype
        self.capacity = max(1, int(max_slots))
        self._specs: List[dict] = []
        self._bufs: List[Dict[str, torch.Tensor]] = []
        self._free: List[int] = list(range(self.capacity - 1, -1, -1))
        self.length: Dict[int, int] = {}                      # live slot -> tokens folded into its state
        self.generation = 0                                   # bumped when the buffers move (captured graphs are stale then)

    # ------------------------------------------------------------------ layout
    def register(self, kind: str, **shape) -> int:
        """Add one entry; returns its handle.  ``latent``: ``ring_len, channels``; ``kv``: ``ring_len, first_len, channels``;
        ``recurrent``: ``heads, dim, vdim, taps, conv_channels``; ``token``: nothing."""
        assert kind in ("latent", "kv", "recurrent", "token"), kind
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
        return {
            "S": torch.zeros(n, spec["heads"], spec["dim"], spec["vdim"], dtype=torch.float32, device=self.device),
            "tail": torch.zeros(n, max(spec["taps"] - 1, 0), spec["conv_channels"], dtype=self.dtype, device=self.device),
        }

    def buffers(self, handle: int) -> Dict[str, torch.Tensor]:
        return self._bufs[handle]

    def bytes_per_slot(self) -> int:
        return sum(t[0].numel() * t.element_size() for b in self._bufs for t in b.values())

    # ------------------------------------------------------------------ slots
    def allocate(self, n: int = 1) -> List[int]:
        while len(self._free) < n:
            self._grow()
        slots = [self._free.pop() for _ in range(n)]
        for s in slots:
            self.length[s] = 0
        return slots

    def free(self, slots) -> None:
        for s in slots:
            if s in self.length:
                del self.length[s]
                self._free.append(s)

    def advance(self, slots, lens) -> None:
        for s, n in zip(slots, lens):
            self.length[s] += n

    def live(self) -> int:
        return len(self.length)

    def _grow(self):
        old, new = self.capacity, self.capacity * 2
        for i, spec in enumerate(self._specs):
            bigger = self._make(spec, new)
            for name, t in self._bufs[i].items():
                bigger[name][:old].copy_(t)
            self._bufs[i] = bigger
        self._free = list(range(new - 1, old - 1, -1)) + self._free
        self.capacity = new
        self.generation += 1
