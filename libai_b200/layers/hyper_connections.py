"""Hyper-connections: several residual streams instead of one (Zhu et al., "Hyper-Connections", 2024; the static form).

A sublayer reads ``u = Σ_s in[s] · x_s``, runs on ``norm(u)`` and its output ``y`` is written back to every stream while the
streams are mixed among themselves: ``x_t ← Σ_s mix[s, t] · x_s + out[t] · y`` (all ``t`` at once from the old streams; ``mix`` is
indexed ``[from, to]``).  With one stream, ``in = out = mix = 1`` this is the plain residual sum.  The module only holds the
coefficients; :func:`libai_b200.ops.lin_functional.hc_step` applies the closing of one sublayer and the opening (read + RMS norm)
of the next in one pass over the fp32 streams.
"""
from __future__ import annotations

import torch
from torch import nn

from ._param import create_parameter, ones_


def _eye(t, generator=None):
    with torch.no_grad():
        t.copy_(torch.eye(t.shape[0], dtype=t.dtype, device=t.device))
    return t


class HyperConnection(nn.Module):
    def __init__(self, streams: int, *, layer_idx=0):
        super().__init__()
        self.streams = int(streams)
        mk = lambda shape, init: create_parameter(shape, init, layer_idx=layer_idx)
        self.inw, self.outw, self.mix = mk((streams,), ones_), mk((streams,), ones_), mk((streams, streams), _eye)
        self._f32 = None

    def coefficients(self):
        """``(in [S], out [S], mix [S, S])`` as contiguous fp32 tensors (what the stream operator takes)."""
        key = (self.mix.device, self.inw._version, self.outw._version, self.mix._version)
        if self._f32 is None or self._f32[0] != key:
            self._f32 = (key, tuple(t.detach().float().contiguous() for t in (self.inw, self.outw, self.mix)))
        return self._f32[1]

    def extra_repr(self) -> str:
        return f"streams={self.streams}"
