"""Grouped-query attention whose mask reaches back a bounded number of positions, on per-sequence key/value rings.

``q = W_q h`` (``H`` heads), ``k = W_k h``, ``v = W_v h`` (``G`` heads; query head h reads key/value head ``h // (H/G)``).
Options, all constructor arguments:

* ``qk_norm="full"`` — RMS norm over the whole query (key) projection with a weight of that size, before rotation;
  ``qk_norm="head_unit"`` — every head divided by its root mean square, without a weight, after rotation;
* rotary positions on the first ``rot_dims`` channels of every head in the rotate-half pairing, frequencies from
  :func:`libai_b200.ops.kv_functional.rotary_frequencies` (optionally blended per dimension towards ``f / factor``);
* the mask: ``chunk`` — position i sees j ≤ i of its own chunk of that many positions (chunks are counted from position 0
  of the sequence); or ``window`` with ``keep_first`` — j ≤ i with ``i − j < window`` or ``j < keep_first``;
* ``out_gate`` — head h of the result is multiplied by ``sigmoid(W_g h)_h`` (``True`` / ``"head"``: one gate logit per head),
  or every channel of the concatenated heads by its own ``sigmoid(W_g h)`` (``"channel"``: ``W_g`` is ``[H·V, width]``);
* ``kv_source`` — the layer has no key/value projections and reads the cache of another layer (keys as that layer stored them);
* ``value_from_key`` — there is no ``W_v``: the values are the keys as projected, before norm and rotation (``vdim = dim``);
* ``softcap`` — scaled scores pass through ``cap · tanh(score / cap)``; ``sink`` — the softmax has one more entry of score 0
  that carries no value: ``p_j = exp(s_j) / (1 + Σ exp(s))``.

State per sequence (:class:`libai_b200.inference.state_cache.SequenceStateCache`, kind ``kv``): a ring of the last
``ring_len`` rows ``[keys | values]`` and the rows of the first ``first_len`` positions.  Prompt steps read
``[kept-first rows | cached rows the step still sees | the step's rows]`` (gathered once per cache and step, shared with the
layers that read the same cache; a step whose sequences all start at position 0 reads the projection output in place) through
the masked attention kernel; single-token steps write their row first and read ring and kept-first rows directly.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from libai_b200.ops import kv_functional as KF

from ._param import create_parameter, ones_, xavier_normal_


class RingAttention(nn.Module):
    def __init__(self, width, heads, kv_heads, dim, vdim, *, window=0, chunk=0, keep_first=0, scale=None, rot_dims=0,
                 rot_base=10000.0, rot_scaling=None, qk_norm: Optional[str] = None, out_gate=False, kv_source: Optional[int] = None,
                 value_from_key=False, softcap=None, sink=False, eps=1e-6, init_method=xavier_normal_, layer_idx=0):
        super().__init__()
        assert heads % kv_heads == 0 and (chunk > 0) != (window > 0), "one of chunk / window bounds the mask"
        assert qk_norm in (None, "full", "head_unit") and rot_dims % 2 == 0 and rot_dims <= dim
        assert out_gate in (False, True, None, "head", "channel")
        assert not value_from_key or (vdim == dim and kv_source is None), "values that are the keys have the keys' size"
        self.value_from_key, self.softcap, self.sink = bool(value_from_key), float(softcap or 0.0), bool(sink)
        self.gate_wide = out_gate == "channel"
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.window, self.chunk, self.keep_first = int(window), int(chunk), int(keep_first) if window > 0 else 0
        self.scale, self.eps, self.qk_norm, self.kv_source = float(scale if scale is not None else dim ** -0.5), eps, qk_norm, kv_source
        self.rot_dims, self.layer_idx = int(rot_dims), layer_idx
        mk = lambda shape, init=init_method: create_parameter(shape, init, layer_idx=layer_idx)
        self.q = mk((heads * dim, width))
        self.q_norm = mk((heads * dim,), ones_) if qk_norm == "full" else None
        if kv_source is None:
            self.k = mk((kv_heads * dim, width))
            self.v = None if value_from_key else mk((kv_heads * vdim, width))
            self.k_norm = mk((kv_heads * dim,), ones_) if qk_norm == "full" else None
        else:
            self.k = self.v = self.k_norm = None
        self.g = mk((heads * vdim if self.gate_wide else heads, width)) if out_gate else None
        self.o = mk((width, heads * vdim))
        freq, self.rot_mscale = KF.rotary_frequencies(self.rot_dims, rot_base, rot_scaling) if rot_dims else (torch.zeros(0), 1.0)
        self.register_buffer("rot_freq", freq.float(), persistent=False)
        # set by the model: masks of every layer reading this layer's cache (this one included), and the cache's sizes
        self.cache_masks = [self.mask]
        self.ring_len, self.first_len = self.reach, self.keep_first

    @property
    def mask(self):
        return (self.window, self.chunk, self.keep_first)

    @property
    def reach(self) -> int:
        """Most positions behind (and including) a query's own that its contiguous range covers."""
        return self.chunk if self.chunk > 0 else self.window

    @property
    def mix_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self):
        return "kv", dict(ring_len=self.ring_len, first_len=self.first_len, channels=self.kv_heads * (self.dim + self.vdim))

    def input_weights(self):
        out = [("q", self.q)]
        if self.kv_source is None:                            # values that are the keys: W_k twice in the stacked product
            out += [("k", self.k), ("v", self.k if self.value_from_key else self.v)]
        if self.g is not None:
            out.append(("g", self.g))
        return out

    def output_weight(self):
        return self.o

    def mix(self, parts, rb, bufs, y, shared, out_scale: float = 1.0):
        """``parts``: the projections of the step's rows (column slices of one product); ``bufs``: the cache entry this layer
        reads; ``shared``: per-step dictionary through which a layer hands the key / value rows of a prompt step to the layers
        that read its cache; ``y`` ``[tokens, H·V]`` receives the heads' outputs (gated, times ``out_scale``)."""
        extra = dict(softcap=self.softcap, sink=self.sink, gate_wide=self.gate_wide, out_scale=out_scale)
        H, G, D, V = self.heads, self.kv_heads, self.dim, self.vdim
        q, k, v, gate = parts["q"], parts.get("k"), parts.get("v"), parts.get("g")
        if self.rot_freq.device != q.device:
            self.rot_freq = self.rot_freq.to(q.device)
        KF.qk_prepare(q, k, self.q_norm, self.k_norm, self.rot_freq, self.rot_mscale, rb, H, G, D, self.eps,
                      self.qk_norm == "full", self.qk_norm == "head_unit")
        ring, first = bufs["ring"], bufs["first"]
        own = self.kv_source is None
        if rb.single:
            if own:
                KF.kv_write(ring, first, k, v, rb)
            KF.ring_attention(q, ring, first, gate, rb, y, H, G, D, V, self.window, self.chunk, self.keep_first, self.scale, **extra)
            return y
        if own:
            ext = rb.kv_ext(self.cache_masks)
            if ext.cached:
                rows = KF.kv_gather(ring, first, k, v, rb, ext)
                kmat, vmat = rows[:, :G * D], rows[:, G * D:]
            else:
                kmat, vmat = k, v                              # every sequence starts at position 0: the projections are the rows
            shared[self.layer_idx] = (ext, kmat, vmat)
            KF.kv_write(ring, first, k, v, rb)
        else:
            ext, kmat, vmat = shared[self.kv_source]
        KF.masked_attention(q, kmat, vmat, ext, gate, rb, y, H, G, D, V, self.window, self.chunk, self.keep_first, self.scale, **extra)
        return y

    def forward(self, h, rb, bufs, shared=None):
        parts = {name: KF.linear(h, w) for name, w in self.input_weights()}
        y = torch.empty(h.shape[0], self.mix_features, dtype=h.dtype, device=h.device)
        return KF.linear(self.mix(parts, rb, bufs, y, {} if shared is None else shared), self.o)
