"""Salizen: a decoder-only language model of pre-norm blocks on several residual streams (hyper-connections) whose sequence
mixers are linear-attention recurrences, alone or side by side with sink-softmax window attention.

Structure (every size and constant comes from the configuration):

* embedding: ``embed[token] · embedding.scale`` plus one row of a bigram table chosen by ``(previous token · mul_prev + token ·
  mul_cur) mod buckets`` (a sequence's first token takes the table's last row); the previous token is sequence state;
* ``streams`` copies of the embedding output are the residual streams.  A sublayer (mixer, then feed-forward) reads
  ``u = Σ_s in[s] x_s``, runs on ``rmsnorm(u)`` and is written back with ``x_t ← Σ_s mix[s, t] x_s + out[t] y``
  (:class:`libai_b200.layers.HyperConnection`); the model's output is the sum of the streams;
* mixers: ``parallel`` — grouped-query sliding-window attention (rotary positions with wavelength-blended frequencies, values =
  keys before rotation, tanh-capped scores, a softmax with a value-less entry of score 0, a channel-wise sigmoid output gate:
  :class:`libai_b200.layers.RingAttention`) beside gated linear attention with a data-dependent decay per key channel, their
  outputs weighted by two constants; ``retention`` — rotary positions, one fixed decay per head, unit-RMS heads, SiLU gate;
  ``lightning`` — SiLU on queries, keys and values, one fixed decay per head, one RMS norm over all heads, sigmoid gate (all three
  recurrences: :class:`libai_b200.layers.DecayLinearAttention`);
* feed-forwards: ``dense`` — ``W_down (gelu_tanh(W_gate h) · W_up h)``; ``moe`` — :class:`libai_b200.layers.MoEFeedForward` with a
  biased router whose weights are the softmax over the chosen logits; a block may have none;
* RMS norm of the summed streams and the output projection.

The streams, the norms, attention scores, the router, the decays and the recurrent state are fp32 whatever the compute dtype.
Execution is the framework's generation path for stateful models: packed rows (:class:`~libai_b200.inference.ragged.RaggedBatch`)
against a :class:`~libai_b200.inference.state_cache.SequenceStateCache`; a block is one stacked input product, its mixer kernels,
one output product and one stream kernel per sublayer (closing write-back + opening read and norm of the next sublayer).
"""
from __future__ import annotations

from typing import List

import torch
from torch import nn

from libai_b200.config import configurable
from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.state_cache import SequenceStateCache
from libai_b200.layers import DecayLinearAttention, GatedFeedForward, HyperConnection, MoEFeedForward, RingAttention, RMSLayerNorm
from libai_b200.layers._param import create_parameter, normal_init, xavier_normal_
from libai_b200.ops import kv_functional as KF
from libai_b200.ops import lin_functional as LF
from libai_b200.ops import seq_functional as SF

from .stateful_lm import StatefulCausalLM, _plain


def build_sequence_mixer(kind: str, width: int, m: dict, eps: float, layer_idx: int):
    """Mixer of one block from its ``type`` and ``mixer`` record."""
    if kind == "parallel":
        return ParallelMixer(width, m, eps, layer_idx)
    if kind in ("retention", "lightning"):
        rot = m.get("rot") or {}
        common = dict(decay=list(m["decay"]), eps=eps, layer_idx=layer_idx)
        if kind == "retention":
            return DecayLinearAttention(width, m["heads"], m["dim"], m["vdim"], k_scale=m["dim"] ** -0.5, rot_dims=rot.get("dims", 0),
                                        rot_base=rot.get("base", 10000.0), rot_scaling=rot.get("scaling"), norm="head",
                                        norm_weight=False, gate="silu", **common)
        return DecayLinearAttention(width, m["heads"], m["dim"], m["vdim"], qkv_act="silu", norm="all", norm_weight=True,
                                    gate="sigmoid", **common)
    raise ValueError(f"unknown mixer type {kind!r}")


class ParallelMixer(nn.Module):
    """Two mixers side by side on the same input: ``left_scale · left(h) + right_scale · right(h)``; the constants are applied
    to the mixers' gated outputs, so both output projections are one product on the concatenated heads."""

    def __init__(self, width, m, eps, layer_idx=0):
        super().__init__()
        a, b = m["left"], m["right"]
        rot = a.get("rot") or {}
        self.left = RingAttention(width, a["heads"], a["kv_heads"], a["dim"], a["vdim"], window=a["mask"]["size"], scale=a.get("scale"),
                                  rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 10000.0), rot_scaling=rot.get("scaling"),
                                  out_gate="channel", value_from_key=True, softcap=a.get("softcap"), sink=True, eps=eps,
                                  layer_idx=layer_idx)
        self.right = DecayLinearAttention(width, b["heads"], b["dim"], b["vdim"], decay="channel", tau=b["tau"],
                                          decay_rank=b.get("decay_rank") or max(1, b["dim"] // 4), q_scale=b["dim"] ** -0.5,
                                          norm="head", norm_weight=True, gate="silu", eps=eps, layer_idx=layer_idx)
        self.left_scale, self.right_scale = float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))

    def parts(self):
        return [("left", self.left, self.left_scale), ("right", self.right, self.right_scale)]


def mixer_parts(mix):
    """``[(prefix, module, output factor)]`` of a block's mixer: one entry, or the two sides of a parallel mixer."""
    return mix.parts() if isinstance(mix, ParallelMixer) else [("", mix, 1.0)]


GatedFF = GatedFeedForward          # the dense feed-forward of a block


class HyperBlock(nn.Module):
    """Mixer and feed-forward sublayers on the residual streams ``x`` ``[streams, rows, width]`` (fp32).  The read and norm that
    open a sublayer are done by the kernel that closes the sublayer before it, so a block receives ``h = norm1(Σ in·x)`` and
    returns the next block's."""

    def __init__(self, width, kind, mixer_cfg, mlp_cfg, streams, eps, *, layer_idx=0):
        super().__init__()
        self.kind, self.width, self.eps = kind, width, eps
        self.norm1 = RMSLayerNorm(width, eps=eps, layer_idx=layer_idx)
        self.hc1 = HyperConnection(streams, layer_idx=layer_idx)
        self.mix = build_sequence_mixer(kind, width, mixer_cfg, eps, layer_idx)
        self.mlp = None
        if mlp_cfg:
            self.norm2 = RMSLayerNorm(width, eps=eps, layer_idx=layer_idx)
            self.hc2 = HyperConnection(streams, layer_idx=layer_idx)
            kind_ff = mlp_cfg.get("kind", "dense")
            if kind_ff == "dense":
                self.mlp = GatedFF(width, mlp_cfg["ff"], layer_idx=layer_idx)
            elif kind_ff == "moe":
                r = mlp_cfg["router"]
                self.mlp = MoEFeedForward(width, mlp_cfg["expert"]["ff"], r["experts"], r["top"], router="softmax", router_bias=True,
                                          layer_idx=layer_idx)
            else:
                raise ValueError(f"unknown feed-forward kind {kind_ff!r}")
        self._fused = None

    def state_specs(self):
        return [m.state_spec() for _, m, _ in mixer_parts(self.mix)]

    def opening(self):
        """``(in, norm weight)`` of the block's first sublayer."""
        return self.hc1.coefficients()[0], self.norm1.weight

    def _fuse(self):
        w = self.norm1.weight
        if self._fused is None or self._fused[0].dtype != w.dtype or self._fused[0].device != w.device:
            parts = mixer_parts(self.mix)
            ins = [(p + n, t.detach()) for p, m, _ in parts for n, t in m.input_weights()]
            outs = [(p, m.output_weight().detach()) for p, m, _ in parts]
            self._fused = SF.fuse_rows(ins) + SF.fuse_cols(outs)
        return self._fused

    def forward(self, x, h, rb, bufs, nxt):
        """``bufs``: the state entries of the mixer's parts; ``nxt``: ``(in, norm weight)`` of the sublayer that follows the
        block (``None`` after the last one).  Returns that sublayer's normed input."""
        w_in, cols, w_out, kcols = self._fuse()
        dt, dev, T = w_in.dtype, h.device, h.shape[0]
        proj = KF.linear(h, w_in)
        full = w_out.shape[1] == sum(size for _, size in kcols.values())
        y = (torch.empty if full else torch.zeros)(T, w_out.shape[1], dtype=dt, device=dev)
        shared: dict = {}
        for (p, m, factor), buf in zip(mixer_parts(self.mix), bufs):
            parts = {n[len(p):]: proj[:, lo:lo + size] for n, (lo, size) in cols.items() if n.startswith(p)}
            lo, size = kcols[p]
            m.mix(parts, rb, buf, y[:, lo:lo + size], shared, out_scale=factor)
        o = KF.linear_f32(y, w_out)
        _, out1, mix1 = self.hc1.coefficients()
        after = (self.hc2.coefficients()[0], self.norm2.weight) if self.mlp is not None else nxt
        h = torch.empty(T, self.width, dtype=dt, device=dev) if after is not None else None
        LF.hc_step(x, o, post=(mix1, out1), nxt=after, h=h, eps=self.eps)
        if self.mlp is None:
            return h
        pos = cw = None
        if isinstance(self.mlp, MoEFeedForward):
            d, pos, cw = self.mlp(h, graph_safe=rb.single)
        else:
            d = self.mlp(h)
        _, out2, mix2 = self.hc2.coefficients()
        h = torch.empty(T, self.width, dtype=dt, device=dev) if nxt is not None else None
        LF.hc_step(x, d, post=(mix2, out2), nxt=nxt, h=h, pos=pos, cw=cw, eps=self.eps)
        return h


class SalizenModel(nn.Module):
    def __init__(self, vocab, width, layers, streams=1, embedding=None, eps=1e-6, initializer_range=0.02):
        super().__init__()
        emb = embedding or {}
        bg = emb.get("bigram") or {}
        self.vocab, self.width, self.eps, self.streams = vocab, width, eps, int(streams)
        self.embedding_scale = float(emb.get("scale", 1.0))
        self.buckets, self.mul_prev, self.mul_cur = int(bg.get("buckets", 1)), int(bg.get("mul_prev", 0)), int(bg.get("mul_cur", 0))
        self.embed = create_parameter((vocab, width), normal_init(initializer_range), layer_idx=0)
        self.bigram = create_parameter((self.buckets + 1, width), normal_init(initializer_range), layer_idx=0)
        self.layers = nn.ModuleList(
            [HyperBlock(width, lc["type"], lc["mixer"], lc.get("mlp"), self.streams, eps, layer_idx=i) for i, lc in enumerate(layers)])
        self.final_norm = RMSLayerNorm(width, eps=eps, layer_idx=-1)

    def register_state(self, cache: SequenceStateCache) -> List:
        """The previous token of every sequence, then per block the state entries of its mixer's parts."""
        handles: List = [cache.register("token")]
        for blk in self.layers:
            handles.append([cache.register(kind, **shape) for kind, shape in blk.state_specs()])
        return handles

    def forward(self, tokens, rb: RaggedBatch, cache: SequenceStateCache, handles, tap=None):
        """``tokens`` ``[rows]`` int64 packed → the fp32 streams after the last block ``[streams, rows, width]``.
        ``tap(run, x)`` is called with the sum of the streams after every block (diagnostics)."""
        dt, dev, T = self.embed.dtype, tokens.device, tokens.shape[0]
        x = torch.empty(self.streams, T, self.width, dtype=torch.float32, device=dev)
        LF.embed_bigram(self.embed, self.bigram, tokens, cache.buffers(handles[0])["last"], rb, self.embedding_scale, self.mul_prev,
                        self.mul_cur, self.buckets, x)
        h = None
        if len(self.layers):
            h = torch.empty(T, self.width, dtype=dt, device=dev)
            LF.hc_step(x, nxt=self.layers[0].opening(), h=h, eps=self.eps)
        for i, blk in enumerate(self.layers):
            nxt = self.layers[i + 1].opening() if i + 1 < len(self.layers) else None
            h = blk(x, h, rb, [cache.buffers(q) for q in handles[1 + i]], nxt)
            if tap is not None:
                tap(i, x.sum(0))
        return x


class SalizenForCausalLM(StatefulCausalLM):
    @configurable
    def __init__(self, vocab, width, layers, streams=1, embedding=None, norm_eps=1e-6, initializer_range=0.02, cfg=None):
        super().__init__()
        self.cfg = cfg
        self.model = SalizenModel(vocab, width, layers, streams=streams, embedding=embedding, eps=norm_eps,
                                  initializer_range=initializer_range)
        self.head = create_parameter((vocab, width), normal_init(initializer_range), layer_idx=-1)
        self._ones = None

    @classmethod
    def from_config(cls, cfg):
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        norm = get("norm") or {}
        return dict(vocab=get("vocab"), width=get("width"), layers=_plain(get("layers")), streams=get("streams") or 1,
                    embedding=_plain(get("embedding")), norm_eps=norm.get("eps", 1e-6) if hasattr(norm, "get") else 1e-6,
                    initializer_range=get("initializer_range") or 0.02, cfg=cfg)

    @torch.no_grad()
    def step_device(self, tokens, rb: RaggedBatch, logits_rows=None, tap=None):
        """The device work of :meth:`step` alone (kernel launches only, no host-side bookkeeping): this is what a CUDA graph of a
        single-token step captures."""
        cache = self.state_cache()
        x = self.model(tokens, rb, cache, self._handles, tap=tap)
        if logits_rows is not None:
            x = x.index_select(1, logits_rows)
        if self._ones is None or self._ones.device != x.device:
            self._ones = torch.ones(self.model.streams, dtype=torch.float32, device=x.device)
        h = torch.empty(x.shape[1], x.shape[2], dtype=self.head.dtype, device=x.device)
        LF.hc_step(x, nxt=(self._ones, self.model.final_norm.weight), h=h, eps=self.model.eps)    # norm of the summed streams
        return KF.linear_f32(h, self.head)
