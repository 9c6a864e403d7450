"""Grouped-query softmax attention over the whole past of a sequence, on a paged key/value cache.

``q = W_q h`` (``H`` heads of ``dim``), ``k = W_k h``, ``v = W_v h`` (``G`` heads; query head h reads key/value head ``h // (H/G)``).
Options, all constructor arguments:

* ``conv`` — a causal convolution over time of that many taps on every channel of ``q``, ``k`` and ``v``, directly after the
  projections (weights ``[channels, taps]``, the last column multiplies the current token; no bias, no activation);
* ``qk_norm`` — RMS norm of every query and key head with one weight ``[dim]`` shared by the heads, before the rotation;
* ``v_norm`` — every value head is divided by its root mean square (no weight); it is cached so;
* rotary positions on the first ``rot_dims`` channels of every head in the rotate-half pairing, frequencies from
  :func:`libai_b200.ops.kv_functional.rotary_frequencies`;
* ``talk`` — the heads' scaled scores are mixed by a learned ``[H, H]`` matrix before the mask and the softmax
  (talking-heads attention: Shazeer et al., "Talking-Heads Attention", 2020; only the mix before the softmax);
* ``sink`` — a learned number per head whose exponential joins the softmax denominator without a key or a value.

State per sequence (:class:`libai_b200.inference.state_cache.SequenceStateCache`, kind ``paged``): the rows ``[keys | values]`` of
all its positions in pages, and the last ``conv − 1`` projections.  A step prepares its rows (one kernel: convolution, norms,
rotation, page write), then every query attends over the pages; prompt steps and single-token steps run the same kernel with
different tilings.
"""
from __future__ import annotations

import torch
from torch import nn

from libai_b200.ops import kv_functional as KF
from libai_b200.ops import paged_functional as PF

from ._param import create_parameter, ones_, xavier_normal_, zeros_


def _last_tap_(t, generator=None):
    """A convolution that passes its input through: one in the last column."""
    t.zero_()
    t[:, -1] = 1.0
    return t


def _identity_(t, generator=None):
    t.zero_()
    return t.fill_diagonal_(1.0)


class PagedAttention(nn.Module):
    def __init__(self, width, heads, kv_heads, dim, vdim, *, scale=None, conv=1, qk_norm=True, v_norm=False, rot_dims=0, rot_base=10000.0,
                 rot_scaling=None, talk=False, sink=False, eps=1e-6, init_method=xavier_normal_, layer_idx=0):
        super().__init__()
        assert heads % kv_heads == 0 and rot_dims % 2 == 0 and rot_dims <= dim and conv >= 1
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.eps, self.taps, self.layer_idx = float(scale if scale is not None else dim ** -0.5), eps, int(conv), layer_idx
        self.qk_norm, self.v_norm, self.rot_dims = bool(qk_norm), bool(v_norm), int(rot_dims)
        assert self.qk_norm and self.v_norm, "the preparation kernel is built with query/key norms and unit-RMS values"
        mk = lambda shape, init=init_method: create_parameter(shape, init, layer_idx=layer_idx)
        self.q, self.k, self.v = mk((heads * dim, width)), mk((kv_heads * dim, width)), mk((kv_heads * vdim, width))
        self.o = mk((width, heads * vdim))
        self.q_conv, self.k_conv, self.v_conv = (mk((n, self.taps), _last_tap_) for n in (heads * dim, kv_heads * dim, kv_heads * vdim))
        self.q_norm, self.k_norm = mk((dim,), ones_), mk((dim,), ones_)
        self.talk = mk((heads, heads), _identity_) if talk else None
        self.sink = mk((heads,), zeros_) if sink else None
        freq, mscale = KF.rotary_frequencies(self.rot_dims, rot_base, rot_scaling) if rot_dims else (torch.zeros(0), 1.0)
        assert mscale == 1.0, "frequency scalings that rescale cos / sin are not built into the preparation kernel"
        self.register_buffer("rot_freq", freq.float(), persistent=False)

    @property
    def mix_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self):
        H, G, D, V = self.heads, self.kv_heads, self.dim, self.vdim
        return "paged", dict(channels=G * (D + V), taps=self.taps, conv_channels=H * D + G * D + G * V)

    def input_weights(self):
        return [("q", self.q), ("k", self.k), ("v", self.v)]

    def output_weight(self):
        return self.o

    def _fp32(self, name):
        """fp32 copy of a small parameter that enters the scores (cached until the parameter changes)."""
        p = getattr(self, name)
        if p is None:
            return None
        key = (p.device, p._version)
        cache = self.__dict__.setdefault("_f32", {})
        if name not in cache or cache[name][0] != key:
            cache[name] = (key, p.detach().float().contiguous())
        return cache[name][1]

    def mix(self, parts, rb, bufs, y, shared=None, out_scale: float = 1.0, h=None):
        """``parts``: the projections of the step's rows (column slices of one product); ``bufs``: this layer's cache entry
        (``pool``, ``tail``, ``table``); ``y`` ``[tokens, H·V]`` receives the heads' outputs times ``out_scale``."""
        H, G, D, V = self.heads, self.kv_heads, self.dim, self.vdim
        if self.rot_freq.device != parts["q"].device:
            self.rot_freq = self.rot_freq.to(parts["q"].device)
        q = PF.conv_qkv_prepare(parts["q"], parts["k"], parts["v"], self.q_conv, self.k_conv, self.v_conv, bufs["tail"], self.q_norm,
                                self.k_norm, self.rot_freq, self.eps, rb, bufs["pool"], bufs["table"], H, G, D, V)
        return PF.talk_attention(q, bufs["pool"], bufs["table"], rb, y, H, G, D, V, self.scale, talk=self._fp32("talk"),
                                 sink=self._fp32("sink"), out_scale=out_scale)

    def forward(self, h, rb, bufs, shared=None):
        """Unfused form: ``h`` ``[tokens, width]`` packed rows → ``[tokens, width]``."""
        proj = KF.linear(h, torch.cat([self.q, self.k, self.v], 0))
        a, b = self.heads * self.dim, (self.heads + self.kv_heads) * self.dim
        parts = {"q": proj[:, :a], "k": proj[:, a:b], "v": proj[:, b:]}
        y = torch.empty(h.shape[0], self.mix_features, dtype=h.dtype, device=h.device)
        return KF.linear(self.mix(parts, rb, bufs, y), self.o)
