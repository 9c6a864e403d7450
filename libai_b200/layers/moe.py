"""Mixture-of-experts feed-forward: a router chooses ``top`` of ``experts`` gated feed-forward layers per token.

Router (fp32 logits ``z = W_r h``, plus a bias with ``router_bias``): ``router="sigmoid"`` — ``s = sigmoid(z)``, the ``top``
largest scores, weights ``s_k / (Σ_chosen s + 1e-20) · scale``; ``router="softmax"`` — the ``top`` largest logits, weights = the
softmax over the chosen logits only, times ``scale``.  Expert:
``W_down (act(W_gate h) · W_up h)`` without biases; the layer's output is the weighted sum over the chosen experts.  The expert
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

    def __init__(self, width, ff, experts, top, *, router_scale=1.0, act="silu", router="sigmoid", router_bias=False,
                 init_method=xavier_normal_, layer_idx=0):
        super().__init__()
        assert 1 <= top <= experts and router in ("sigmoid", "softmax")
        self.width, self.ff, self.experts, self.top, self.router_scale, self.act = width, ff, experts, top, float(router_scale), act
        self.route_mode = KF.ROUTE_SOFTMAX if router == "softmax" else KF.ROUTE_SIGMOID
        mk = lambda shape: create_parameter(shape, init_method, layer_idx=layer_idx)
        self.router = mk((experts, width))
        self.router_b = create_parameter((experts,), zeros_, layer_idx=layer_idx) if router_bias else None
        self._bias32 = None
        self.gate_up = mk((experts, 2 * ff, width))
        self.down = mk((experts, width, ff))

    def forward(self, h, graph_safe: bool = False):
        """``h`` ``[tokens, width]`` → ``(y, pos, wts)``: either ``y`` fp32 ``[tokens, width]`` with ``pos = wts = None``, or the
        sorted expert outputs ``y`` ``[tokens·top, width]`` with the row ``pos[t, k]`` and weight ``wts[t, k]`` of every pair —
        the caller's residual operator gathers the weighted sum."""
        act = KF.ACTS[self.act]
        bias = None
        if self.router_b is not None:                          # the router's arithmetic is fp32: a float copy of the bias
            key = (self.router_b.device, self.router_b._version)
            if self._bias32 is None or self._bias32[0] != key:
                self._bias32 = (key, self.router_b.detach().float().contiguous())
            bias = self._bias32[1]
        if graph_safe or h.shape[0] <= self.PAIR_FORM_MAX_TOKENS:
            idx, wts = KF.moe_route(h, self.router, self.top, self.router_scale, bias=bias, mode=self.route_mode)
            return KF.moe_pairs(h, self.gate_up, self.down, idx, wts, act), None, None
        counts = torch.zeros(self.experts, dtype=torch.int32, device=h.device)
        idx, wts = KF.moe_route(h, self.router, self.top, self.router_scale, counts, bias=bias, mode=self.route_mode)
        ys, pos = KF.moe_sorted(h, self.gate_up, self.down, idx, counts, act)
        return ys, pos, wts
