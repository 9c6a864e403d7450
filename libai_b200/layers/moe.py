"""Mixture-of-experts feed-forward: a router chooses ``top`` of ``experts`` gated feed-forward layers per token.

Router (fp32 logits ``z = W_r h``, plus a bias with ``router_bias``): ``router="sigmoid"`` — ``s = sigmoid(z)``, the ``top``
largest scores, weights ``s_k / (Σ_chosen s + 1e-20) · scale``; ``router="sigmoid_raw"`` — the same choice, weights ``s_k · scale``
(not normalised); ``router="softmax"`` — the ``top`` largest logits, weights = the softmax over the chosen logits only, times
``scale``.  Expert: ``W_down (act(W_gate h) · W_up h)`` without biases (``act="swish_clamp"`` with ``limit``: ``g = min(W_gate h, limit)``,
``u = clamp(W_up h, ±limit)``, ``W_down (g · sigmoid(1.702 g) · (u + 1))``); the layer's output is the weighted sum over the chosen
experts, or — ``weight_input`` — the plain sum of the experts run on ``weight · h``.  The expert
matrices are stacked — ``gate_up`` ``[E, 2·ff, width]`` (gate rows, then up rows) and ``down`` ``[E, width, ff]`` — so that an
expert's two input matrices are one product.

Two execution forms (:mod:`libai_b200.ops.kv_functional`): prompt steps sort the (token, expert) pairs by expert and run every
expert as dense products on its rows; single-token steps (and anything as small) let every pair read its expert's matrices in
two kernels without any host-side decision, so that the step can be captured in a CUDA graph.
"""
from __future__ import annotations

import torch
from torch import nn

from libai_b200.ops import kv_functional as KF

from ._param import create_parameter, xavier_normal_, zeros_


class MoEFeedForward(nn.Module):
    PAIR_FORM_MAX_TOKENS = 16          # at most this many tokens run pair by pair even when the step is not single-token

    def __init__(self, width, ff, experts, top, *, router_scale=1.0, act="silu", router="sigmoid", router_bias=False, limit=0.0,
                 weight_input=False, init_method=xavier_normal_, layer_idx=0):
        super().__init__()
        assert 1 <= top <= experts and router in ("sigmoid", "softmax", "sigmoid_raw")
        self.width, self.ff, self.experts, self.top, self.router_scale, self.act = width, ff, experts, top, float(router_scale), act
        self.limit, self.weight_input = float(limit), bool(weight_input)
        self.route_mode = {"sigmoid": KF.ROUTE_SIGMOID, "softmax": KF.ROUTE_SOFTMAX, "sigmoid_raw": KF.ROUTE_SIGMOID_RAW}[router]
        mk = lambda shape: create_parameter(shape, init_method, layer_idx=layer_idx)
        self.router = mk((experts, width))
        self.router_b = create_parameter((experts,), zeros_, layer_idx=layer_idx) if router_bias else None
        self._bias32 = None
        self.gate_up = mk((experts, 2 * ff, width))
        self.down = mk((experts, width, ff))

    def forward(self, h, graph_safe: bool = False):
        """``h`` ``[tokens, width]`` → ``(y, pos, wts)``: either ``y`` fp32 ``[tokens, width]`` with ``pos = wts = None``, or the
        sorted expert outputs ``y`` ``[tokens·top, width]`` with the row ``pos[t, k]`` and weight ``wts[t, k]`` of every pair —
        the caller's residual operator gathers the weighted sum (``wts`` is ``None`` with ``weight_input``: a plain sum)."""
        act = KF.ACTS[self.act]
        bias = None
        if self.router_b is not None:                          # the router's arithmetic is fp32: a float copy of the bias
            key = (self.router_b.device, self.router_b._version)
            if self._bias32 is None or self._bias32[0] != key:
                self._bias32 = (key, self.router_b.detach().float().contiguous())
            bias = self._bias32[1]
        if graph_safe or h.shape[0] <= self.PAIR_FORM_MAX_TOKENS:
            idx, wts = KF.moe_route(h, self.router, self.top, self.router_scale, bias=bias, mode=self.route_mode)
            return KF.moe_pairs(h, self.gate_up, self.down, idx, wts, act, self.limit, self.weight_input), None, None
        counts = torch.zeros(self.experts, dtype=torch.int32, device=h.device)
        idx, wts = KF.moe_route(h, self.router, self.top, self.router_scale, counts, bias=bias, mode=self.route_mode)
        ys, pos = KF.moe_sorted(h, self.gate_up, self.down, idx, counts, act, self.limit, wts if self.weight_input else None)
        return ys, pos, (None if self.weight_input else wts)


class GatedFeedForward(nn.Module):
    """``W_down (act(W_gate h) · W_up h)`` without biases; ``gate_up`` stacks the two input matrices (gate rows, then up rows).
    ``act`` names an activation of :data:`libai_b200.ops.kv_functional.ACTS` (``"swish_clamp"`` takes ``limit``)."""

    def __init__(self, width, ff, act="gelu_tanh", *, limit=0.0, init_method=xavier_normal_, layer_idx=0):
        super().__init__()
        self.act, self.ff, self.limit = act, ff, float(limit)
        self.gate_up = create_parameter((2 * ff, width), init_method, layer_idx=layer_idx)
        self.down = create_parameter((width, ff), init_method, layer_idx=layer_idx)

    def forward(self, h):
        """``h`` ``[rows, width]`` → fp32 ``[rows, width]``."""
        gu = KF.linear(h, self.gate_up)
        a = torch.empty(h.shape[0], self.ff, dtype=h.dtype, device=h.device)
        KF.act_rows(gu, a, KF.ACTS[self.act], gated=True, limit=self.limit)
        return KF.linear_f32(a, self.down)
