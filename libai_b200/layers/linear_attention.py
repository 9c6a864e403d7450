"""Linear attention with a decay: a sequence mixer whose state is one fp32 matrix per head.

Per head, with the state ``S`` ``[dim, vdim]`` (zero at the start of a sequence) and, for every token, ``q, k`` ``[dim]``,
``v`` ``[vdim]`` (projections of the layer input) and a decay ``a``::

    S ← diag(a) S + k vᵀ;   o = Sᵀ q

Options, all constructor arguments, cover the usual members of the family:

* ``decay`` — a list of fixed numbers, one per head (retention: Sun et al., "Retentive Network: A Successor to Transformer for
  Large Language Models", 2023), or ``"channel"``: one decay per key channel and token, ``a = sigmoid(W_a2 W_a1 h + b)^(1/tau)``
  through a low-rank pair (gated linear attention), or ``"tied"``: a forget gate per key channel and token that is bounded from
  below and also decides what is written, ``a = l + (1 − l) · sigmoid(W_f h + b)`` with a learned bound ``l`` per channel and
  the written key ``k = 1 − a`` — the layer has no key projection (HGRN2: Qin et al., "HGRN2: Gated Linear RNNs with State
  Expansion", 2024);
* ``qkv_act="silu"`` — ``q``, ``k`` and ``v`` pass through SiLU (``"silu_q"``: the queries only); ``q_scale`` / ``k_scale`` — constant
  factors (applied after the rotation);
* ``rot_dims`` / ``rot_base`` / ``rot_scaling`` — rotary positions on the first ``rot_dims`` channels of every query and key head;
* ``norm`` — the read-out is RMS-normalised per head (``"head"``) or over all heads together (``"all"``), with a weight
  (``[vdim]`` shared by the heads, or ``[heads·vdim]``) or without one (``norm_weight=False``);
* ``gate`` — the normalised read-out is multiplied by ``silu(W_g h)`` or ``sigmoid(W_g h)`` (``None``: no gate and no ``W_g``);
  ``W_o`` projects the result.

The decays, the recurrence, the norm and the gate's activation are fp32 in every compute dtype.  State per sequence: ``S``
(:class:`libai_b200.inference.state_cache.SequenceStateCache`, kind ``recurrent`` without convolution tails).
"""
from __future__ import annotations

import torch
from torch import nn

from libai_b200.ops import kv_functional as KF
from libai_b200.ops import lin_functional as LF

from ._param import create_parameter, ones_, xavier_normal_, zeros_


class DecayLinearAttention(nn.Module):
    def __init__(self, width, heads, dim, vdim, *, decay, tau=1.0, decay_rank=None, qkv_act=None, q_scale=1.0, k_scale=1.0,
                 rot_dims=0, rot_base=10000.0, rot_scaling=None, norm="head", norm_weight=True, gate="silu", eps=1e-6,
                 init_method=xavier_normal_, layer_idx=0):
        super().__init__()
        assert norm in ("head", "all") and gate in ("silu", "sigmoid", None) and qkv_act in (None, "silu", "silu_q")
        assert rot_dims % 2 == 0 and rot_dims <= dim
        self.width, self.heads, self.dim, self.vdim, self.eps, self.layer_idx = width, heads, dim, vdim, eps, layer_idx
        self.tied = isinstance(decay, str) and decay == "tied"
        self.channel_decay = isinstance(decay, str) and not self.tied
        self.tau, self.qkv_act, self.q_scale, self.k_scale = float(tau), qkv_act, float(q_scale), float(k_scale)
        self.norm_mode, self.gate = norm, gate
        self.rot_dims = int(rot_dims)
        mk = lambda shape, init=init_method: create_parameter(shape, init, layer_idx=layer_idx)
        self.q, self.v = mk((heads * dim, width)), mk((heads * vdim, width))
        self.k = None if self.tied else mk((heads * dim, width))
        self.g = mk((heads * vdim, width)) if gate is not None else None
        self.o = mk((width, heads * vdim))
        if self.tied:
            self.f, self.f_b, self.lower = mk((heads * dim, width)), mk((heads * dim,), zeros_), mk((heads * dim,), zeros_)
        elif self.channel_decay:
            assert decay == "channel" and decay_rank, "a data-dependent decay needs the inner size of its low-rank pair"
            self.a1, self.a2, self.a2_b = mk((decay_rank, width)), mk((heads * dim, decay_rank)), mk((heads * dim,), zeros_)
        else:
            assert len(decay) == heads, "one decay per head"
            self.register_buffer("decay", torch.tensor([float(d) for d in decay], dtype=torch.float32), persistent=False)
        self.norm = mk((vdim,) if norm == "head" else (heads * vdim,), ones_) if norm_weight else None
        freq, self.rot_mscale = KF.rotary_frequencies(self.rot_dims, rot_base, rot_scaling) if rot_dims else (torch.zeros(0), 1.0)
        self.register_buffer("rot_freq", freq.float(), persistent=False)
        self._bias32 = None

    # ------------------------------------------------------------------ protocol of the blocks
    @property
    def mix_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self):
        return "recurrent", dict(heads=self.heads, dim=self.dim, vdim=self.vdim, taps=1, conv_channels=0)

    def input_weights(self):
        out = [(n, w) for n, w in (("q", self.q), ("k", self.k), ("v", self.v), ("g", self.g)) if w is not None]
        if self.channel_decay:
            out.append(("a1", self.a1))
        return out

    def output_weight(self):
        return self.o

    def _fp32(self, name):
        """fp32 copy of a small parameter that enters the recurrence (cached until the parameter changes)."""
        p = getattr(self, name)
        key = (p.device, p._version)
        cache = self.__dict__.setdefault("_f32", {})
        if name not in cache or cache[name][0] != key:
            cache[name] = (key, p.detach().float().contiguous())
        return cache[name][1]

    def mix(self, parts, rb, bufs, y, shared=None, out_scale: float = 1.0, h=None):
        """From the projections of the layer input (``parts``: name → column view) to the gated, normalised read-out written
        into ``y`` ``[tokens, heads·vdim]`` (the input of ``W_o``), times ``out_scale``.  A tied decay takes the layer input ``h``
        as well: its gate logits are an fp32 product of their own."""
        q, k, v = parts["q"], parts.get("k"), parts["v"]
        dev = q.device
        if self.rot_dims:
            if self.rot_freq.device != dev:
                self.rot_freq = self.rot_freq.to(dev)
            KF.qk_prepare(q, k, None, None, self.rot_freq, self.rot_mscale, rb, self.heads, self.heads, self.dim, self.eps, False, False)
        kw = dict(q_scale=self.q_scale, k_scale=self.k_scale, act=LF.ACT_Q if self.qkv_act == "silu_q" else self.qkv_act == "silu")
        if self.tied:
            z = KF.linear_f32(h, self.f)                      # gate logits leave the product in fp32
            o = LF.decay_scan(q, None, v, bufs["S"], rb, z=z, zb=self._fp32("f_b"), lower=self._fp32("lower"), **kw)
        elif self.channel_decay:
            key = (self.a2_b.device, self.a2_b._version)
            if self._bias32 is None or self._bias32[0] != key:
                self._bias32 = (key, self.a2_b.detach().float().contiguous())
            z = KF.linear_f32(parts["a1"], self.a2)            # decay logits leave the product in fp32
            o = LF.decay_scan(q, k, v, bufs["S"], rb, z=z, zb=self._bias32[1], tau=self.tau, **kw)
        else:
            if self.decay.device != dev:
                self.decay = self.decay.to(dev)
            o = LF.decay_scan(q, k, v, bufs["S"], rb, decay=self.decay, **kw)
        act = LF.GATE_NONE if self.gate is None else (LF.GATE_SILU if self.gate == "silu" else LF.GATE_SIGMOID)
        LF.gated_norm(o, parts.get("g"), self.norm, self.eps, act, y, self.heads,
                      self.vdim, per_head=self.norm_mode == "head", out_scale=out_scale)
        return y

    def forward(self, h, rb, bufs):
        """Unfused form: ``h`` ``[tokens, width]`` packed rows → ``[tokens, width]``."""
        parts = {name: KF.linear(h, w) for name, w in self.input_weights()}
        y = torch.empty(h.shape[0], self.mix_features, dtype=h.dtype, device=h.device)
        return KF.linear(self.mix(parts, rb, bufs, y, h=h), self.o)
