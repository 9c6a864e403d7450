"""Request scheduler of the stateful models: requests → slots of the state cache → ragged steps of the model's step function.

A request enters with its first tokens, goes on with whatever tokens later steps bring (one at a time while decoding, or a
further portion of its prompt) and gives its slot back when it is finished.  All entries of a step run as ONE ragged batch;
nothing is padded.  :meth:`RequestScheduler.generate` is batched generation on top of it: one step for all prompts, then one
token per live request per step, requests leaving the batch as they finish; the next token is chosen by the framework's
logits processors / warpers (greedy when none samples).
"""
from __future__ import annotations

import os
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from libai_b200.inference.generator.generation_logits_processor import (
    LogitsProcessorList,
    TemperatureLogitsWarper,
    TopKLogitsWarper,
    TopPLogitsWarper,
)
from libai_b200.inference.ragged import RaggedBatch


class _SingleTokenGraph:
    """A captured CUDA graph of one single-token step for a fixed set of slots: tokens and past lengths live in persistent
    device buffers that are refreshed before every replay; the logits come back in a persistent buffer."""

    def __init__(self, model, slots, generation):
        self.generation = generation
        dev = model.head.device
        self.n = len(slots)
        self.rb = RaggedBatch(self.n * [1], slots, self.n * [0], dev)
        self.io = torch.zeros(2 * self.n, dtype=torch.long, device=dev)       # [tokens | past lengths], refreshed per step
        self.graph = torch.cuda.CUDAGraph()
        self.logits = None
        self.model = model

    def capture(self):
        torch.cuda.synchronize()
        with torch.cuda.graph(self.graph):
            self.rb.past.copy_(self.io[self.n:])                              # int64 → the descriptor's int32, on the device
            self.logits = self.model.step_device(self.io[: self.n], self.rb)

    def run(self, tokens, past):
        # one copy from a fresh pageable tensor: the host may not touch a staging buffer that a queued copy still reads
        self.io.copy_(torch.tensor(list(tokens) + list(past), dtype=torch.long))
        self.graph.replay()
        return self.logits


class RequestScheduler:
    MAX_GRAPHS = 8

    def __init__(self, model, max_tokens: Optional[int] = None, cuda_graphs: Optional[bool] = None):
        self.model = model
        self.cache = model.state_cache()
        # single-token steps of a batch that stays together replay from a CUDA graph (captured at the batch's second such step)
        self.cuda_graphs = (os.environ.get("LIBAI_B200_DECODE_GRAPHS", "1") == "1") if cuda_graphs is None else cuda_graphs
        self._graphs: Dict[tuple, object] = {}
        self.max_tokens = max_tokens          # sizes the paged key/value pools; other state does not grow with the tokens held
        if max_tokens:
            self.cache.reserve(max_tokens)
        self.slot_of: Dict[Hashable, int] = {}
        self.device = model.head.device

    def live_tokens(self) -> int:
        return sum(self.cache.length[s] for s in self.slot_of.values())

    def step(self, entries: Sequence[Tuple[Hashable, Sequence[int], Sequence[int]]]):
        """``entries``: ``(request id, next tokens, positions among them whose logits are wanted)``.  Returns the wanted
        logits ``[Σ wanted, vocab]`` fp32 in the order of the entries (``None`` when nothing is wanted)."""
        if not entries:
            return None
        for rid, _, _ in entries:
            if rid not in self.slot_of:
                self.slot_of[rid] = self.cache.allocate(1)[0]
        slots = [self.slot_of[rid] for rid, _, _ in entries]
        lens = [len(toks) for _, toks, _ in entries]
        self.cache.prepare(slots, lens)                         # may move the buffers: before a captured graph is looked up
        if self.cuda_graphs and self.device.type == "cuda" and all(n == 1 for n in lens) and hasattr(self.model, "step_device"):
            logits = self._graphed_single_tokens(entries, slots)
            if logits is not None:
                return logits if any(want for _, _, want in entries) else None
        rb = RaggedBatch(lens, slots, [self.cache.length[s] for s in slots], self.device)
        flat = [t for _, toks, _ in entries for t in toks]
        rows = [rb.offsets[b] + w for b, (_, _, want) in enumerate(entries) for w in want]
        packed = torch.tensor(flat + rows, dtype=torch.long).to(self.device, non_blocking=True)
        tokens, row_idx = packed[: len(flat)], packed[len(flat):]
        logits = self.model.step(tokens, rb, row_idx)
        return logits if rows else None

    def _graphed_single_tokens(self, entries, slots):
        """Replay (or capture) the graph of this slot set; ``None`` = run this step eagerly (first time the set is seen, or
        capture is not possible).  Returns the wanted logits rows (a fresh tensor)."""
        key = tuple(slots)
        state = self._graphs.get(key)
        if state is not None and state != "seen" and state.generation != self.cache.generation:
            state = None                                        # the cache grew: its buffers moved
        if state is None:
            if len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = "seen"                          # the eager step warms everything a capture must not initialise
            return None
        past = [self.cache.length[s] for s in slots]
        if state == "seen":
            try:
                state = _SingleTokenGraph(self.model, slots, self.cache.generation)
                state.capture()
            except Exception:                                   # capture refused (an operation that cannot be captured): stay eager
                self.cuda_graphs = False
                self._graphs.clear()
                return None
            self._graphs[key] = state
        logits = state.run([toks[0] for _, toks, _ in entries], past)
        self.cache.advance(slots, [1] * len(slots))
        rows = [b for b, (_, _, want) in enumerate(entries) if want]
        if len(rows) == len(entries):
            return logits.clone()
        return logits[torch.tensor(rows, dtype=torch.long, device=logits.device)] if rows else logits[:0]

    def finish(self, request_ids) -> None:
        for rid in request_ids:
            slot = self.slot_of.pop(rid, None)
            if slot is not None:
                self.cache.free([slot])

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, eos_token_id: Optional[int] = None,
                 do_sample: bool = False, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                 logits_processor: Optional[LogitsProcessorList] = None) -> List[List[int]]:
        """Prompts of any lengths → the generated continuations (without the prompt, ending with ``eos_token_id`` when it
        was produced)."""
        processors = logits_processor if logits_processor is not None else LogitsProcessorList()
        warpers = LogitsProcessorList()
        if do_sample:
            if temperature != 1.0:
                warpers.append(TemperatureLogitsWarper(float(temperature)))
            if top_k:
                warpers.append(TopKLogitsWarper(top_k=int(top_k)))
            if top_p < 1.0:
                warpers.append(TopPLogitsWarper(top_p=float(top_p)))
        ids = [("gen", id(prompts), i) for i in range(len(prompts))]
        seqs = [list(p) for p in prompts]
        out: List[List[int]] = [[] for _ in prompts]
        live = list(range(len(prompts)))
        entries = [(ids[i], seqs[i], [len(seqs[i]) - 1]) for i in live]
        try:
            while live and max_new_tokens > 0:
                logits = self.step(entries)
                nxt = []
                for row, i in enumerate(live):
                    so_far = torch.tensor([seqs[i]], dtype=torch.long, device=logits.device)
                    scores = warpers(so_far, processors(so_far, logits[row:row + 1]))
                    tok = int(torch.multinomial(torch.softmax(scores, -1), 1)) if do_sample else int(scores.argmax(-1))
                    nxt.append(tok)
                still = []
                for i, tok in zip(live, nxt):
                    seqs[i].append(tok)
                    out[i].append(tok)
                    if (eos_token_id is not None and tok == eos_token_id) or len(out[i]) >= max_new_tokens:
                        self.finish([ids[i]])
                    else:
                        still.append(i)
                live = still
                entries = [(ids[i], [seqs[i][-1]], [0]) for i in live]
        finally:
            self.finish(ids)
        return out
