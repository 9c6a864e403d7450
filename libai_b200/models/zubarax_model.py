"""Zubarax: a decoder-only language model of post-norm blocks whose sequence mixer runs full softmax attention and a gated
linear recurrence side by side, with mixture-of-experts feed-forwards and an output projection tied to the embedding.

Structure (every size and constant comes from the configuration):

* embedding: ``embed[token] · embedding.scale``; the same table, unscaled, projects the final norm's output to the logits;
* a block: ``x ← norm1(α x + mixer(x))``, then ``x ← norm2(α x + ff(x))`` with ``α = postln_alpha`` — the sublayers read the normed
  residual itself; the norms are RMS norms whose stored weight is the deviation from one
  (:func:`libai_b200.ops.paged_functional.postnorm_residual`); a block may have no feed-forward;
* mixer ``parallel``: ``left_scale · left(h) + right_scale · right(h)`` on the same input.  Left — grouped-query attention over the
  whole past: short causal convolutions on the projected queries, keys and values, per-head RMS norm of queries and keys, rotary
  positions on the leading channels, unit-RMS values, scores mixed across heads before the softmax, a learned sink per head in
  the denominator (:class:`libai_b200.layers.PagedAttention`).  Right — HGRN2: linear attention whose forget gate, bounded from
  below by a learned number per channel, also decides what is written; SiLU queries, per-head RMS norm of the read-out
  (:class:`libai_b200.layers.DecayLinearAttention` with a tied decay);
* feed-forward ``moe``: a sigmoid router picks ``top`` experts, their scores (not normalised) multiply the experts' *inputs*,
  the experts are clamped gated layers ``W_down (g σ(1.702 g) (u + 1))``, and a shared expert of the same form runs for every token
  (:class:`libai_b200.layers.MoEFeedForward`, :class:`libai_b200.layers.GatedFeedForward`);
* a block entry with ``weights_of: j`` runs block j's parameters with a cache and state of its own.

The residual, the norms, attention scores and softmax, the router, gates and the recurrent state are fp32 whatever the compute
dtype.  Execution is the framework's generation path for stateful models: packed rows
(:class:`~libai_b200.inference.ragged.RaggedBatch`) against a :class:`~libai_b200.inference.state_cache.SequenceStateCache`; a
block is one stacked input product, the mixers' kernels, one output product on the concatenated heads and one residual kernel
per sublayer.
"""
from __future__ import annotations

from typing import List

import torch
from torch import nn

from libai_b200.config import configurable
from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.state_cache import SequenceStateCache
from libai_b200.layers import DecayLinearAttention, GatedFeedForward, MoEFeedForward, PagedAttention, RMSLayerNorm
from libai_b200.layers._param import create_parameter, normal_init
from libai_b200.ops import kv_functional as KF
from libai_b200.ops import paged_functional as PF
from libai_b200.ops import seq_functional as SF

from .stateful_lm import StatefulCausalLM, _plain


class ParallelHeadsMixer(nn.Module):
    """Softmax attention over the pages beside a tied-gate linear recurrence, ``left_scale · left(h) + right_scale · right(h)``; the
    constants are applied to the mixers' head outputs, so both output projections are one product on the concatenated heads."""

    def __init__(self, width, m, eps, layer_idx=0):
        super().__init__()
        a, b = m["left"], m["right"]
        rot = a.get("rot") or {}
        self.left = PagedAttention(width, a["heads"], a["kv_heads"], a["dim"], a["vdim"], scale=a.get("scale"), conv=int(a.get("conv") or 1),
                                   qk_norm=True, v_norm=True, rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 10000.0),
                                   talk=True, sink=True, eps=eps, layer_idx=layer_idx)
        self.right = DecayLinearAttention(width, b["heads"], b["dim"], b["vdim"], decay="tied", qkv_act="silu_q", norm="head",
                                          norm_weight=True, gate=None, eps=eps, layer_idx=layer_idx)
        self.left_scale, self.right_scale = float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))

    def parts(self):
        return [("left.", self.left, self.left_scale), ("right.", self.right, self.right_scale)]


def build_mixer(kind: str, width: int, m: dict, eps: float, layer_idx: int):
    if kind == "parallel":
        return ParallelHeadsMixer(width, m, eps, layer_idx)
    raise ValueError(f"unknown mixer type {kind!r}")


class PostNormBlock(nn.Module):
    """``x ← norm1(α x + mixer(x))``, ``x ← norm2(α x + ff(x))`` on the fp32 residual ``x`` ``[rows, width]`` (updated in place); ``h`` is
    its copy in the compute dtype (``x`` itself in fp32), which the products read."""

    def __init__(self, width, kind, mixer_cfg, mlp_cfg, alpha, eps, *, bare_norm2=False, layer_idx=0):
        super().__init__()
        self.kind, self.width, self.alpha, self.eps = kind, width, float(alpha), eps
        self.norm1 = RMSLayerNorm(width, eps=eps, layer_idx=layer_idx, zero_centered=True)
        self.mix = build_mixer(kind, width, mixer_cfg, eps, layer_idx)
        self.mlp = self.shared = self.norm2 = None
        if mlp_cfg or bare_norm2:                              # a block without a feed-forward may still own a second norm
            self.norm2 = RMSLayerNorm(width, eps=eps, layer_idx=layer_idx, zero_centered=True)
        if mlp_cfg:
            if mlp_cfg.get("kind", "moe") != "moe":
                raise ValueError(f"unknown feed-forward kind {mlp_cfg.get('kind')!r}")
            r, e = mlp_cfg["router"], mlp_cfg["expert"]
            self.mlp = MoEFeedForward(width, e["ff"], r["experts"], r["top"], router="sigmoid_raw", act="swish_clamp", limit=e["limit"],
                                      weight_input=True, layer_idx=layer_idx)
            sh = mlp_cfg.get("shared")
            if sh:
                self.shared = GatedFeedForward(width, sh["ff"], "swish_clamp", limit=sh["limit"], layer_idx=layer_idx)
        self._fused = None

    def state_specs(self):
        return [m.state_spec() for _, m, _ in self.mix.parts()]

    def _fuse(self):
        w = self.norm1.weight
        if self._fused is None or self._fused[0].dtype != w.dtype or self._fused[0].device != w.device:
            parts = self.mix.parts()
            ins = [(p + n, t.detach()) for p, m, _ in parts for n, t in m.input_weights()]
            outs = [(p, m.output_weight().detach()) for p, m, _ in parts]
            self._fused = SF.fuse_rows(ins) + SF.fuse_cols(outs)
        return self._fused

    def _copy(self, x):
        """Where the next products read the residual from: a compute-dtype buffer, or ``None`` when that is ``x`` itself."""
        dt = self.norm1.weight.dtype
        return None if dt == torch.float32 else torch.empty(x.shape, dtype=dt, device=x.device)

    def forward(self, x, h, rb, bufs):
        """``bufs``: the state entries of the mixer's parts, in their order.  Returns the copy of the new ``x`` for the products."""
        w_in, cols, w_out, kcols = self._fuse()
        T = x.shape[0]
        proj = KF.linear(h, w_in)
        full = w_out.shape[1] == sum(size for _, size in kcols.values())
        y = (torch.empty if full else torch.zeros)(T, w_out.shape[1], dtype=w_in.dtype, device=x.device)
        for (p, m, factor), buf in zip(self.mix.parts(), bufs):
            parts = {n[len(p):]: proj[:, lo:lo + size] for n, (lo, size) in cols.items() if n.startswith(p)}
            lo, size = kcols[p]
            m.mix(parts, rb, buf, y[:, lo:lo + size], None, out_scale=factor, h=h)
        o = KF.linear_f32(y, w_out)
        hb = self._copy(x)
        PF.postnorm_residual(x, self.norm1.weight, self.eps, alpha=self.alpha, y=o, h=hb)
        h = x if hb is None else hb
        if self.mlp is None:
            if self.norm2 is None:
                return h
            hb = self._copy(x)                                 # x ← norm2(α x): the second step with an empty sublayer
            PF.postnorm_residual(x, self.norm2.weight, self.eps, alpha=self.alpha, h=hb)
            return x if hb is None else hb
        d, pos, cw = self.mlp(h, graph_safe=rb.single)
        shared = self.shared(h) if self.shared is not None else None
        hb = self._copy(x)
        if pos is None:                                        # the experts' sum came back per token
            PF.postnorm_residual(x, self.norm2.weight, self.eps, alpha=self.alpha, y=shared, y2=d, h=hb)
        else:
            PF.postnorm_residual(x, self.norm2.weight, self.eps, alpha=self.alpha, y=shared, y2=d, pos=pos, cw=cw, h=hb)
        return x if hb is None else hb


class ZubaraxModel(nn.Module):
    def __init__(self, vocab, width, layers, postln_alpha=1.0, embedding=None, eps=1e-6, initializer_range=0.02):
        super().__init__()
        self.vocab, self.width, self.eps = vocab, width, eps
        self.embedding_scale = float((embedding or {}).get("scale", 1.0))
        self.embed = create_parameter((vocab, width), normal_init(initializer_range), layer_idx=0)
        # a run of the stack names the block whose parameters it uses; blocks exist for the entries that own parameters
        owners = [i for i, lc in enumerate(layers) if lc.get("weights_of") is None]

        def owner(i):
            while layers[i].get("weights_of") is not None:
                i = int(layers[i]["weights_of"])
            return i

        self.runs = [owners.index(owner(i)) for i in range(len(layers))]
        self.owner_ids = owners                                # block k holds the tensors of entry owner_ids[k]
        self.layers = nn.ModuleList(
            [PostNormBlock(width, layers[i]["type"], layers[i]["mixer"], layers[i].get("mlp"), postln_alpha, eps,
                           bare_norm2=bool(layers[i].get("bare_norm2")), layer_idx=i) for i in owners])
        self.final_norm = RMSLayerNorm(width, eps=eps, layer_idx=-1, zero_centered=True)

    def register_state(self, cache: SequenceStateCache) -> List:
        """Per run of the stack the state entries of its mixer's parts (a block that runs twice keeps two states)."""
        return [[cache.register(kind, **shape) for kind, shape in self.layers[k].state_specs()] for k in self.runs]

    def forward(self, tokens, rb: RaggedBatch, cache: SequenceStateCache, handles, tap=None):
        """``tokens`` ``[rows]`` int64 packed → the fp32 residual after the last block ``[rows, width]``.  ``tap(run, x)`` is called
        with the residual after every run (diagnostics)."""
        dt, dev, T = self.embed.dtype, tokens.device, tokens.shape[0]
        x = torch.empty(T, self.width, dtype=torch.float32, device=dev)
        KF.embed_scale(self.embed, tokens, self.embedding_scale, x)
        h = x if dt == torch.float32 else x.to(dt)
        for run, k in enumerate(self.runs):
            h = self.layers[k](x, h, rb, [cache.buffers(q) for q in handles[run]])
            if tap is not None:
                tap(run, x)
        return x


class ZubaraxForCausalLM(StatefulCausalLM):
    @configurable
    def __init__(self, vocab, width, layers, postln_alpha=1.0, embedding=None, norm_eps=1e-6, initializer_range=0.02, kv_page_size=64,
                 cfg=None):
        super().__init__()
        self.cfg = cfg
        self.kv_page_size = int(kv_page_size)                 # positions per page of the attention layers' key/value pools
        self.model = ZubaraxModel(vocab, width, layers, postln_alpha=postln_alpha, embedding=embedding, eps=norm_eps,
                                  initializer_range=initializer_range)

    @property
    def head(self):
        """The output projection is the embedding table."""
        return self.model.embed

    @classmethod
    def from_config(cls, cfg):
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        norm = get("norm") or {}
        alpha = get("postln_alpha")
        return dict(vocab=get("vocab"), width=get("width"), layers=_plain(get("layers")), postln_alpha=1.0 if alpha is None else alpha,
                    embedding=_plain(get("embedding")), norm_eps=norm.get("eps", 1e-6) if hasattr(norm, "get") else 1e-6,
                    initializer_range=get("initializer_range") or 0.02, kv_page_size=get("kv_page_size") or 64, cfg=cfg)

    @torch.no_grad()
    def step_device(self, tokens, rb: RaggedBatch, logits_rows=None, tap=None):
        """The device work of :meth:`step` alone (kernel launches only, no host-side bookkeeping): this is what a CUDA graph of a
        single-token step captures."""
        cache = self.state_cache()
        x = self.model(tokens, rb, cache, self._handles, tap=tap)
        if logits_rows is not None:
            x = x.index_select(0, logits_rows)
        dt = self.head.dtype
        h = torch.empty(x.shape, dtype=dt, device=x.device)
        PF.postnorm_residual(x, self.model.final_norm.weight, self.model.eps, h=h, inplace=False)
        return KF.linear_f32(h, self.head)
