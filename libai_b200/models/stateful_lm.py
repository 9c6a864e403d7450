"""Causal language models that generate against a :class:`~libai_b200.inference.state_cache.SequenceStateCache`.

The shared part of such models: the state cache and its handles, the one step function on ragged batches —
:meth:`StatefulCausalLM.step`, which ``forward`` (and through it ``Generator.generate``), the request scheduler and the trace
runner all call — and the ``Generator`` protocol on left-padded batches.  A model supplies ``self.model.register_state(cache)``
(one cache entry per layer run) and ``step_device(tokens, rb, logits_rows, tap)`` (the kernel launches of one step).
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from libai_b200.inference.generator.generation_utils import Generator
from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.state_cache import SequenceStateCache


class StatefulCausalLM(nn.Module, Generator):
    def __init__(self):
        super().__init__()
        self.state: Optional[SequenceStateCache] = None
        self._handles: List[int] = []
        self._gen_slots: Optional[List[int]] = None

    # ------------------------------------------------------------------ state
    def state_cache(self) -> SequenceStateCache:
        p = self.head
        if self.state is None or self.state.device != p.device or self.state.dtype != p.dtype:
            self.state = SequenceStateCache(p.device, p.dtype, page_size=getattr(self, "kv_page_size", 64))
            self._handles = self.model.register_state(self.state)
            self._gen_slots = None
        return self.state

    # ------------------------------------------------------------------ the step function
    @torch.no_grad()
    def step(self, tokens, rb: RaggedBatch, logits_rows=None, tap=None):
        """One step of a ragged batch: ``tokens`` ``[rb.tokens]`` int64 on the model's device; advances the state of the
        step's slots.  Returns fp32 logits of the packed rows ``logits_rows`` (default: all), ``[rows, vocab]``."""
        cache = self.state_cache()
        tokens = tokens.to(self.head.device, torch.long).contiguous()
        cache.prepare(rb.slot_list, rb.lens)                   # pages of the positions this step writes (paged entries only)
        logits = self.step_device(tokens, rb, logits_rows, tap=tap)
        cache.advance(rb.slot_list, rb.lens)
        return logits

    # ------------------------------------------------------------------ Generator protocol
    def forward(self, input_ids, attention_mask=None, use_cache=False, last_only=False):
        """``input_ids`` ``[b, s]`` (left-padded when ``attention_mask`` says so; masked positions are not fed at all).
        With ``use_cache`` the sequences continue from the state the previous call left; otherwise they start at their
        first token and the state is dropped afterwards.  Returns ``{"logits": [b, s, vocab]}`` (masked positions zero),
        or ``[b, 1, vocab]`` = the last fed position of every sequence with ``last_only``."""
        cache = self.state_cache()
        b, s = input_ids.shape
        dev = self.head.device
        input_ids = input_ids.to(dev)
        mask = torch.ones(b, s, dtype=torch.bool) if attention_mask is None else attention_mask[:, -s:].bool().cpu()
        lens = mask.sum(1).tolist()
        if min(lens) == 0:
            raise ValueError("every sequence of a step needs at least one unmasked token")
        if use_cache:
            if self._gen_slots is None:
                self._gen_slots = cache.allocate(b)
            slots = self._gen_slots
        else:
            slots = cache.allocate(b)
        if len(slots) != b:
            raise ValueError(f"the cached batch has {len(slots)} sequences, the step has {b}")
        rb = RaggedBatch(lens, slots, [cache.length[q] for q in slots], dev)
        full = bool(mask.all())
        flat = None if full else mask.view(-1).nonzero().squeeze(1).to(dev)
        tokens = input_ids.reshape(-1) if full else input_ids.reshape(-1).index_select(0, flat)
        try:
            if last_only:
                rows = torch.tensor(rb.last_rows(), dtype=torch.long, device=dev)
                return {"logits": self.step(tokens, rb, rows)[:, None, :]}
            logits = self.step(tokens, rb)
        finally:
            if not use_cache:
                cache.free(slots)
        if full:
            return {"logits": logits.view(b, s, -1)}
        out = logits.new_zeros(b * s, logits.shape[-1])
        out.index_copy_(0, flat, logits)
        return {"logits": out.view(b, s, -1)}

    @property
    def past_key_values(self):
        return [self._gen_slots]

    def set_cache(self, past):
        """``None`` ends the running generation: its slots go back to the state cache."""
        if past is None and self._gen_slots is not None and self.state is not None:
            self.state.free(self._gen_slots)
            self._gen_slots = None

    def prepare_inputs_for_generation(self, input_ids, past=None, attention_mask=None, use_cache=None, **kwargs):
        if past is not None and use_cache:
            input_ids = input_ids[:, -1:]
        out = {"input_ids": input_ids, "use_cache": bool(use_cache), "last_only": True}
        if attention_mask is not None and not bool(attention_mask.all()):
            out["attention_mask"] = attention_mask
        return out

    def _reorder_cache(self, past, beam_idx):
        raise NotImplementedError("beam search needs per-beam copies of the recurrent state; use greedy search or sampling")


def _plain(node):
    """Config containers → plain dict / list (the mixer records are consumed as dictionaries)."""
    if node is None:
        return None
    if hasattr(node, "items"):
        return {k: _plain(v) for k, v in node.items()}
    if isinstance(node, (list, tuple)) or (hasattr(node, "__iter__") and not isinstance(node, (str, bytes))):
        return [_plain(v) for v in node]
    return node
