"""Operators of decoders built from linear-attention recurrences on several residual streams (``csrc/lin_mixers.cu``): token +
bigram embedding with the previous token carried as sequence state, hyper-connection streams fused with the RMS norm that
opens the next sublayer, the decayed outer-product recurrence with its fp32 state, and the gated RMS norm of its read-out.

Every operator takes the step's :class:`~libai_b200.inference.ragged.RaggedBatch`.  On a CUDA device the native kernels run
(a missing extension is an error, there is no fallback); on the CPU the same operators are plain PyTorch, sequence by
sequence, which is what the CPU tests use.  Streams, norms, decays and the recurrence are fp32 in both.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import count_launch, impl, load_lin_ext

GATE_SILU, GATE_SIGMOID, GATE_NONE = 0, 1, 2
ACT_Q, ACT_K, ACT_V = 1, 2, 4          # which of q, k, v pass through SiLU in decay_scan


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and impl() == "native"


# --------------------------------------------------------------------------------------------------------------- embedding
def embed_bigram(table, bigram, ids, last, rb, scale: float, mul_prev: int, mul_cur: int, buckets: int, x):
    """``x[s, r] = table[ids[r]] · scale + bigram[row(r)]`` into every stream ``s`` of ``x`` ``[streams, rows, width]`` (fp32).
    ``row(r) = (previous token · mul_prev + token · mul_cur) mod buckets``; the first token of a sequence takes row ``buckets``.
    ``last`` (int32 ``[slots]``) holds every sequence's previous token between steps: it is read for a step's first row when the
    sequence has a past, and left at the step's last token."""
    if _native(table):
        count_launch(2)
        load_lin_ext().embed_bigram(table, bigram, ids, last, rb.tok_seq, rb.seq_off, rb.slots, rb.past, float(scale), int(mul_prev),
                                    int(mul_cur), int(buckets), x)
        return x
    for b in range(rb.B):
        lo, n, slot = rb.offsets[b], rb.lens[b], rb.slot_list[b]
        toks = ids[lo:lo + n].long()
        prev = torch.cat([last[slot:slot + 1].long() if rb.past_list[b] > 0 else toks.new_full((1,), -1), toks[:-1]])
        rows = torch.where(prev < 0, torch.full_like(toks, buckets), (prev * mul_prev + toks * mul_cur) % buckets)
        x[:, lo:lo + n] = (table[toks].float() * scale + bigram[rows].float())[None]
        last[slot] = toks[-1].to(last.dtype)
    return x


# -------------------------------------------------------------------------------------------------------- hyper-connections
def hc_step(x, y=None, post=None, nxt=None, h=None, pos=None, cw=None, eps: float = 1e-6):
    """One sublayer boundary on the residual streams ``x`` ``[streams, rows, width]`` (fp32, updated in place).

    Closing (``y`` given, ``post = (mix [S, S], out [S])`` fp32): ``x_t ← Σ_s mix[s, t] x_s + out[t] · y`` for all ``t`` at once
    from the old streams; ``y`` are the rows of the sublayer's output or — ``pos`` / ``cw`` ``[rows, top]`` given — the weighted
    sums ``Σ_k cw[r, k] · y[pos[r, k]]`` over sorted expert rows.  Opening (``h`` given, ``nxt = (in [S] fp32, w [width])``):
    ``u = Σ_s in[s] x_s``, ``h = u / sqrt(mean(u²) + eps) · w``."""
    if _native(x):
        count_launch()
        mix, outw = post if y is not None else (None, None)
        inw, w = nxt if h is not None else (None, None)
        load_lin_ext().hc_step(x, y, pos, cw, mix, outw, inw, w, float(eps), h)
        return x
    if y is not None:
        mix, outw = post
        yv = y.float()
        if pos is not None:
            yv = (yv[pos.long()] * cw[:, :, None]).sum(1)
        x.copy_(torch.einsum("st,srn->trn", mix.float(), x) + outw.float()[:, None, None] * yv[None])
    if h is not None:
        inw, w = nxt
        u = torch.einsum("s,srn->rn", inw.float(), x)
        h.copy_(u * torch.rsqrt(u.pow(2).mean(-1, keepdim=True) + eps) * w.float())
    return x


# ------------------------------------------------------------------------------------------------------- decayed recurrence
def decay_scan(q, k, v, S, rb, *, decay=None, z=None, zb=None, tau: float = 1.0, q_scale: float = 1.0, k_scale: float = 1.0,
               act=False, lower=None):
    """Linear attention with a decay over the packed rows: per head ``S ← diag(a_t) S + k_t v_tᵀ``, ``o_t = Sᵀ q_t``.

    ``q``, ``k`` ``[tokens, H·D]`` and ``v`` ``[tokens, H·V]`` may be column slices of one projection output; ``act`` says which of
    them pass through SiLU (``True``: all three, or a sum of ``ACT_Q``, ``ACT_K``, ``ACT_V``); ``q`` is multiplied by ``q_scale`` and
    ``k`` by ``k_scale``.  The decay is either ``decay`` (fp32 ``[H]``, one fixed number per head) or, per token and key channel,
    ``sigmoid(z + zb)^(1/tau)`` from the fp32 logits ``z`` ``[tokens, H·D]`` and their bias ``zb`` ``[H·D]``.  With ``lower`` (fp32
    ``[H·D]``) the decay is ``a = lower + (1 − lower) · sigmoid(z + zb)`` and the written key is ``1 − a`` (``k`` is ignored and may
    be ``None``): a forget gate bounded from below that also decides what is written.  ``S`` ``[slots, H, D, V]`` fp32 is read (unless ``past == 0``) and left at
    the state after the last row.  Returns the read-outs ``[tokens, H·V]`` in fp32."""
    H, D, V = S.shape[1], S.shape[2], S.shape[3]
    out = torch.empty(q.shape[0], H * V, dtype=torch.float32, device=q.device)
    act = 7 if act is True else int(act)
    if _native(q):
        count_launch()
        load_lin_ext().decay_scan(q, q if k is None else k, v, decay, z, zb, 1.0 / float(tau), float(q_scale), float(k_scale), act, S,
                                  rb.seq_off, rb.slots, rb.past, out, lower)
        return out
    for b in range(rb.B):
        lo, n, slot = rb.offsets[b], rb.lens[b], rb.slot_list[b]
        st = S[slot].clone() if rb.past_list[b] > 0 else torch.zeros(H, D, V, device=q.device)
        qq, vv = q[lo:lo + n].float(), v[lo:lo + n].float()
        kk = k[lo:lo + n].float() if lower is None else None
        if act & ACT_Q:
            qq = F.silu(qq)
        if act & ACT_K and kk is not None:
            kk = F.silu(kk)
        if act & ACT_V:
            vv = F.silu(vv)
        if lower is not None:
            a = (lower.float() + (1.0 - lower.float()) * torch.sigmoid(z[lo:lo + n].float() + zb.float())).view(n, H, D)
            kk = (1.0 - a).reshape(n, H * D)
        qq, kk, vv = (qq * q_scale).view(n, H, D), (kk * k_scale).view(n, H, D), vv.view(n, H, V)
        if lower is not None:
            pass
        elif z is not None:
            a = torch.exp(F.logsigmoid(z[lo:lo + n].float() + zb.float()) / tau).view(n, H, D)
        else:
            a = decay.float()[None, :, None].expand(n, H, D)
        for t in range(n):
            st = st * a[t][:, :, None] + kk[t][:, :, None] * vv[t][:, None, :]
            out[lo + t] = torch.einsum("hdv,hd->hv", st, qq[t]).reshape(-1)
        S[slot] = st
    return out


def gated_norm(o, gate, w, eps: float, act: int, y, H: int, V: int, *, per_head: bool, out_scale: float = 1.0):
    """``y = o / sqrt(mean(o²) + eps) · w · act(gate) · out_scale`` for the fp32 read-outs ``o`` ``[rows, H·V]``; the mean runs
    over the ``V`` channels of every head (``per_head``; ``w`` ``[V]`` shared by the heads) or over the whole row (``w``
    ``[H·V]``); ``w = None`` leaves the weight out; ``act``: ``GATE_SILU``, ``GATE_SIGMOID`` or ``GATE_NONE`` (no gate: ``gate`` may be
    ``None``)."""
    if _native(o):
        count_launch()
        load_lin_ext().gated_norm(o, gate, w, float(eps), int(act), float(out_scale), y, H, V, bool(per_head))
        return y
    of = o.view(-1, H, V) if per_head else o.view(-1, 1, H * V)
    v = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps) * out_scale
    if act != GATE_NONE:
        g = gate.float().reshape(of.shape)
        v = v * (F.silu(g) if act == GATE_SILU else torch.sigmoid(g))
    if w is not None:
        v = v * w.float()
    y.copy_(v.reshape(-1, H * V))
    return y
