"""Operators of decoders that keep keys and values in per-sequence rings (``csrc/kv_mixers.cu``): Dynamic-Tanh norms fused
around the fp32 residual sum, query/key preparation (RMS norms, rotary positions with per-dimension frequencies), the ring /
kept-first-token cache, grouped-query attention under a position mask and a mixture-of-experts feed-forward.

Every operator takes the step's :class:`~libai_b200.inference.ragged.RaggedBatch`.  On a CUDA device the native kernels run
(a missing extension is an error, there is no fallback); on the CPU the same operators are plain PyTorch, sequence by
sequence, which is what the CPU tests use.  Norms, softmax, the router and the residual sum are fp32 in both.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import count_launch, impl, load_kv_ext
from .seq_functional import _tcgen05_gemm, linear, linear_accumulate  # noqa: F401  (projections are shared)

ACT_COPY, ACT_GELU, ACT_SILU, ACT_GELU_TANH, ACT_RELU2, ACT_SWISH_CLAMP = 0, 1, 2, 3, 4, 5
ACTS = {"copy": ACT_COPY, "gelu": ACT_GELU, "silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "relu2": ACT_RELU2,
        "swish_clamp": ACT_SWISH_CLAMP}


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and impl() == "native"


def _act(v, act: int):
    if act == ACT_GELU:
        return F.gelu(v)
    if act == ACT_SILU:
        return F.silu(v)
    if act == ACT_GELU_TANH:
        return F.gelu(v, approximate="tanh")
    if act == ACT_RELU2:
        return torch.relu(v) ** 2
    return v


def _gated_pair(g, u, act: int, limit: float = 0.0):
    """A gated pair: ``act(g) · u``, or — ``ACT_SWISH_CLAMP`` — ``g' · sigmoid(1.702 g') · (u' + 1)`` with ``g' = min(g, limit)`` and
    ``u' = clamp(u, −limit, limit)``."""
    if act == ACT_SWISH_CLAMP:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        return g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return _act(g, act) * u


# ------------------------------------------------------------------------------------------------------------ projections
def linear_into(a, w, out):
    """``out = a @ wᵀ`` into a given row-major matrix (bf16, or fp32 so that a sublayer's output reaches its norm unrounded):
    the tcgen05 GEMM writes it from its epilogue; shapes it does not take, fp32 operands and CPU tensors go to the vendor /
    PyTorch product."""
    from . import use_native

    a, w = a.detach(), w.detach()                               # an inference operator: nothing is recorded for autograd
    if (a.is_cuda and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and use_native(a) and a.dim() == 2
            and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and w.shape[0] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
            and out.stride(0) % 8 == 0 and a.shape[0] > 0):
        if _tcgen05_gemm(a, w, out, False, out.dtype) is not None:
            return out
    if out.dtype == a.dtype:
        return torch.mm(a, w.t(), out=out) if out.is_contiguous() else out.copy_(F.linear(a, w))
    if a.is_cuda and a.dtype == torch.bfloat16:
        try:                                                    # vendor product with an fp32 result: nothing is rounded to bf16
            return out.copy_(torch.mm(a, w.t(), out_dtype=torch.float32))
        except (TypeError, RuntimeError):
            pass
    return out.copy_(F.linear(a, w))


def linear_f32(a, w):
    """``a @ wᵀ`` as a fresh fp32 matrix."""
    return linear_into(a, w, torch.empty(a.shape[0], w.shape[0], dtype=torch.float32, device=a.device))


# ------------------------------------------------------------------------------------------------------- stream and norms
def embed_scale(table, ids, scale: float, x):
    """``x[r] = table[ids[r]] · scale`` into the fp32 stream ``x``."""
    if _native(table):
        count_launch()
        load_kv_ext().embed_scale(table, ids, float(scale), x)
        return x
    x.copy_(table[ids].float() * scale)
    return x


def dyt_residual(x, y=None, post=None, nxt=None, h=None, pos=None, cw=None):
    """The residual update around a sublayer with Dynamic-Tanh norms, ``dyt(v; w, b, α) = tanh(α v)·w + b``:
    ``x += dyt(y; post)`` when ``y`` is given, then ``h = dyt(x; nxt)`` when ``h`` is given.  ``x`` is the fp32 stream
    (updated in place); ``post`` / ``nxt`` are ``(w, b, alpha)``.  With ``pos`` / ``cw`` ``[rows, top]`` the sublayer output
    of row r is gathered, ``Σ_k cw[r, k] · y[pos[r, k]]`` (expert outputs sorted by expert)."""
    if _native(x):
        count_launch()
        pw, pb, pa = post if y is not None else (None, None, None)
        nw, nb, na = nxt if h is not None else (None, None, None)
        load_kv_ext().dyt_residual(x, y, pos, cw, pw, pb, pa, nw, nb, na, h)
        return x
    if y is not None:
        yv = y.float()
        if pos is not None:
            yv = (yv[pos.long()] * cw[:, :, None]).sum(1)
        w, b, a = post
        x.add_(torch.tanh(a.float() * yv) * w.float() + b.float())
    if h is not None:
        w, b, a = nxt
        h.copy_(torch.tanh(a.float() * x) * w.float() + b.float())
    return x


def act_rows(inp, out, act: int, gated: bool = False, limit: float = 0.0):
    """``out = act(inp)``, or — ``gated`` — ``out = act(inp[:, :n]) · inp[:, n:]`` (column slices of row-major matrices;
    ``ACT_SWISH_CLAMP`` is gated only and takes ``limit``, see :func:`_gated_pair`)."""
    if _native(inp):
        count_launch()
        load_kv_ext().act_rows(inp, out, act, gated, float(limit))
        return out
    n = out.shape[1]
    v = _gated_pair(inp[:, :n].float(), inp[:, n:].float(), act, limit) if gated else _act(inp[:, :n].float(), act)
    out.copy_(v)
    return out


def softcap(logits, cap: float):
    """``logits ← cap · tanh(logits / cap)`` in place (fp32)."""
    if _native(logits):
        count_launch()
        load_kv_ext().softcap(logits, float(cap))
        return logits
    return logits.copy_(cap * torch.tanh(logits / cap))


# ------------------------------------------------------------------------------------------------------- rotary positions
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """Per-pair angular frequencies ``[dims/2]`` (fp32) and the factor on cos / sin.  Plain: ``f_i = base^(-2i/dims)``, factor 1.
    With ``scaling`` = ``{factor, original, fast, slow}`` the frequencies are blended per dimension between ``f_i`` (dimensions
    that turn more than ``fast`` times within ``original`` positions) and ``f_i / factor`` (fewer than ``slow`` turns), linearly
    in the dimension index in between, and cos / sin are multiplied by ``0.1 ln(factor) + 1``.  With ``scaling`` =
    ``{factor, original, low, high}`` the blend is by wavelength ``λ = 2π / f``: ``f`` stays where ``λ < original / high``, becomes
    ``f / factor`` where ``λ > original / low`` and ``(1 − s) f / factor + s f`` with ``s = (original / λ − low) / (high − low)`` in
    between; cos / sin keep the factor 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    mscale = 1.0
    if scaling and "low" in scaling:
        factor, original, low, high = (float(scaling[k]) for k in ("factor", "original", "low", "high"))
        turns = original * f / (2.0 * math.pi)                                 # original / wavelength
        s = (turns - low) / (high - low) if high != low else torch.ones_like(turns)
        blended = (1.0 - s) * f / factor + s * f
        f = torch.where(turns > high, f, torch.where(turns < low, f / factor, blended))
    elif scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def turns_dim(t):
            return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turns_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turns_dim(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mscale = 0.1 * math.log(factor) + 1.0
    return f.float(), mscale


def qk_prepare(q, k, qw, kw, freq, mscale: float, rb, H: int, G: int, D: int, eps: float, full_norm: bool, unit_norm: bool):
    """Query / key preparation in place on the packed rows ``q`` ``[tokens, H·D]`` and ``k`` ``[tokens, G·D]`` (or ``None``):
    ``full_norm`` — RMS norm over the whole projection with weights ``qw`` / ``kw`` (before rotation); rotation of the first
    ``2·len(freq)`` channels of every head (channel i with i + len(freq)) by ``position · freq[i]``; ``unit_norm`` — every head
    divided by its root mean square (after rotation)."""
    if _native(q):
        count_launch()
        load_kv_ext().qk_prepare(q, k, qw if full_norm else None, kw if (full_norm and k is not None) else None, freq, float(mscale),
                                 H, G, D, float(eps), full_norm, unit_norm, rb.tok_seq, rb.seq_off, rb.past)
        return
    half = freq.numel()
    pos = torch.cat([torch.arange(p, p + n) for p, n in zip(rb.past_list, rb.lens)]).to(q.device).float()
    ang = pos[:, None] * freq.float()[None, :]
    cos, sin = (ang.cos() * mscale)[:, None, :], (ang.sin() * mscale)[:, None, :]
    for t, w, heads in ((q, qw, H), (k, kw, G)):
        if t is None:
            continue
        v = t.float()
        if full_norm:
            v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        v = v.view(-1, heads, D)
        a, b = v[..., :half], v[..., half:2 * half]
        v = torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., 2 * half:]], -1)
        if unit_norm:
            v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        t.copy_(v.reshape(-1, heads * D))


# ----------------------------------------------------------------------------------------------------------- cache rows
def kv_write(ring, first, knew, vnew, rb):
    """Store the step's key / value rows: position p of a sequence goes to ``ring[slot, p % L]`` and, for ``p < nfirst``, to
    ``first[slot, p]``."""
    if _native(knew):
        count_launch()
        load_kv_ext().kv_write(ring, first, knew, vnew, rb.tok_seq, rb.seq_off, rb.slots, rb.past)
        return
    L, nf = ring.shape[1], first.shape[1]
    for b in range(rb.B):
        lo, n, slot, past = rb.offsets[b], rb.lens[b], rb.slot_list[b], rb.past_list[b]
        for t in range(n):
            row = torch.cat([knew[lo + t], vnew[lo + t]])
            if n - t <= L:
                ring[slot, (past + t) % L] = row
            if past + t < nf:
                first[slot, past + t] = row
    return


def kv_gather(ring, first, knew, vnew, rb, ext):
    """The key / value rows a prompt step reads (``ext``: a :class:`~libai_b200.inference.ragged.KvExt`): per sequence the
    kept-first rows older than the contiguous part, the cached contiguous part, the step's own rows."""
    out = torch.empty(ext.rows, ring.shape[2], dtype=ring.dtype, device=ring.device)
    if _native(knew):
        count_launch()
        load_kv_ext().kv_gather(ring, first, knew, vnew, ext.ext_seq, ext.ext_off, ext.nsink, ext.cstart, rb.seq_off, rb.slots, rb.past, out)
        return out
    L = ring.shape[1]
    for b in range(rb.B):
        lo, n, slot, past = rb.offsets[b], rb.lens[b], rb.slot_list[b], rb.past_list[b]
        at = ext.offsets[b]
        for p in range(ext.nsink_list[b]):
            out[at] = first[slot, p]
            at += 1
        for p in range(ext.cstart_list[b], past):
            out[at] = ring[slot, p % L]
            at += 1
        out[at:at + n] = torch.cat([knew[lo:lo + n], vnew[lo:lo + n]], 1)
    return out


def _visible(pi: int, window: int, chunk: int, keep: int):
    """Positions the query at ``pi`` sees, in ascending order."""
    if chunk > 0:
        lo = (pi // chunk) * chunk
    elif window > 0:
        lo = max(0, pi - window + 1)
    else:
        lo = 0
    first = list(range(min(keep, lo))) if chunk <= 0 else []
    return first + list(range(lo, pi + 1))


def _attend_rows(qrow, keys, vals, H, G, D, V, scale, softcap=0.0, sink=False):
    """``qrow`` ``[H·D]``; ``keys`` ``[n, G·D]``, ``vals`` ``[n, G·V]`` → ``[H, V]`` fp32."""
    rep = H // G
    k = keys.float().view(-1, G, D).repeat_interleave(rep, 1)
    v = vals.float().view(-1, G, V).repeat_interleave(rep, 1)
    s = torch.einsum("hd,jhd->hj", qrow.float().view(H, D), k) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    if sink:                                                    # one more entry of score 0 that carries no value
        p = torch.softmax(torch.cat([s, s.new_zeros(H, 1)], -1), -1)[:, :-1]
    else:
        p = torch.softmax(s, -1)
    return torch.einsum("hj,jhv->hv", p, v)


def _gated(o, gate_row, wide: bool, out_scale: float):
    """``o`` ``[H, V]`` times ``sigmoid`` of the row's gate logits (one per head, or — ``wide`` — one per channel) and ``out_scale``."""
    if gate_row is not None:
        g = torch.sigmoid(gate_row.float())
        o = o * (g.view(o.shape) if wide else g[:, None])
    return o * out_scale if out_scale != 1.0 else o


def masked_attention(q, kmat, vmat, ext, gate, rb, y, H: int, G: int, D: int, V: int, window: int, chunk: int, keep: int,
                     scale: float, mma: bool = True, softcap: float = 0.0, sink: bool = False, gate_wide: bool = False,
                     out_scale: float = 1.0):
    """Grouped-query softmax attention of every packed query over the rows of the ext matrix (``kmat`` ``[rows, G·D]``,
    ``vmat`` ``[rows, G·V]``: column slices with one row stride) that its mask admits: position j ≤ i with
    ``j ≥ ⌊i/chunk⌋·chunk`` (``chunk > 0``) or ``j > i − window or j < keep`` (``window > 0``).  Head h of the result is
    multiplied by ``sigmoid(gate[t, h])`` when a gate is given (``gate_wide``: channel c of head h by
    ``sigmoid(gate[t, h·V + c])``) and by ``out_scale``.  ``softcap`` > 0: scaled scores pass through ``cap · tanh(s / cap)``;
    ``sink``: the softmax has one more entry of score 0 without a value.  bf16 inputs with head sizes the tensor-core kernel is
    built for take it; ``mma=False`` keeps them on the generic kernel (fp32 inputs always are)."""
    if _native(q):
        count_launch()
        tiles = (None, None)
        if mma and q.dtype == torch.bfloat16 and mma_eligible(q, kmat, vmat, y, D, V) and (
                gate is None or not gate_wide or (gate.data_ptr() % 4 == 0 and gate.stride(0) % 2 == 0 and V % 2 == 0)):
            tiles = rb.query_tiles(64)
        load_kv_ext().masked_attention(q, kmat, vmat, ext.ext_off, ext.nsink, ext.cstart, gate, rb.tok_seq, rb.seq_off, rb.past,
                                       tiles[0], tiles[1], y, H, G, D, V, window, chunk, keep, float(scale), float(softcap), bool(sink),
                                       bool(gate_wide), float(out_scale))
        return y
    for b in range(rb.B):
        lo, n, past, eo, ns, cs = rb.offsets[b], rb.lens[b], rb.past_list[b], ext.offsets[b], ext.nsink_list[b], ext.cstart_list[b]
        for t in range(n):
            rows = [eo + (p if p < cs else ns + p - cs) for p in _visible(past + t, window, chunk, keep)]
            o = _attend_rows(q[lo + t], kmat[rows], vmat[rows], H, G, D, V, scale, softcap, sink)
            o = _gated(o, None if gate is None else gate[lo + t], gate_wide, out_scale)
            y[lo + t] = o.reshape(-1).to(y.dtype)
    return y


MMA_HEAD_SIZES = (32, 48, 64, 96, 128)       # head sizes (keys = values) the tensor-core prompt kernel is built for
GROUPED_DECODE = True                      # single-token steps: the grouped split kernel where its sizes allow


def mma_eligible(q, kmat, vmat, y, D: int, V: int) -> bool:
    return (D == V and D in MMA_HEAD_SIZES and all(t.data_ptr() % 16 == 0 and t.stride(0) % 8 == 0 for t in (q, kmat, vmat, y)))


def ring_attention(q, ring, first, gate, rb, y, H: int, G: int, D: int, V: int, window: int, chunk: int, keep: int, scale: float,
                   splits: Optional[int] = None, softcap: float = 0.0, sink: bool = False, gate_wide: bool = False,
                   out_scale: float = 1.0):
    """Single-token steps: the same attention with keys and values read straight from ``ring`` / ``first`` (the step's own row
    has been written).  ``splits``: 0 = one warp per (token, head); n > 0 = the grouped kernel with the visible keys of a
    (sequence, key head) cut into n parts; ``None`` chooses by the mask's reach.  ``softcap``, ``sink``, ``gate_wide`` and
    ``out_scale`` as in :func:`masked_attention`."""
    if _native(q):
        if splits is None:
            reach = (chunk if chunk > 0 else window) + keep
            if not GROUPED_DECODE or H // G > 8 or V > 128 or (H // G * D + 4 * H // G * (V + 2)) * 4 > 48 * 1024:
                splits = 0
            else:                                               # enough blocks for the device, at least 64 positions each
                splits = max(1, min(32, (reach + 63) // 64, -(-296 // (q.shape[0] * G))))
        count_launch(1 if splits == 0 else 2)
        load_kv_ext().ring_attention(q, ring, first, gate, rb.tok_seq, rb.seq_off, rb.slots, rb.past, y, H, G, D, V, window, chunk, keep,
                                     float(scale), splits, float(softcap), bool(sink), bool(gate_wide), float(out_scale))
        return y
    L, nf, KC = ring.shape[1], first.shape[1], G * D
    for b in range(rb.B):
        slot, pi = rb.slot_list[b], rb.past_list[b]
        rows = torch.stack([first[slot, p] if p < nf else ring[slot, p % L] for p in _visible(pi, window, chunk, keep)])
        o = _attend_rows(q[b], rows[:, :KC], rows[:, KC:], H, G, D, V, scale, softcap, sink)
        o = _gated(o, None if gate is None else gate[b], gate_wide, out_scale)
        y[b] = o.reshape(-1).to(y.dtype)
    return y


# ------------------------------------------------------------------------------------------------------ mixture of experts
ROUTE_SIGMOID, ROUTE_SOFTMAX, ROUTE_SIGMOID_RAW = 0, 1, 2


def moe_route(h, wr, top: int, rscale: float, counts=None, bias=None, mode: int = ROUTE_SIGMOID):
    """Router on the fp32 logits ``z = W_r h`` (``+ bias``, fp32 ``[E]``).  ``ROUTE_SIGMOID``: the ``top`` largest
    ``s = sigmoid(z)``, weights ``s / (Σ s + 1e-20) · rscale``; ``ROUTE_SOFTMAX``: the ``top`` largest logits, weights = softmax
    over the chosen logits only, times ``rscale``; ``ROUTE_SIGMOID_RAW``: the ``top`` largest ``s = sigmoid(z)``, weights
    ``s · rscale`` (not normalised).  Ties go to the lower index.  Returns ``idx`` int32 and ``wts`` fp32, both
    ``[tokens, top]``; ``counts`` (int32 ``[E]``, zeroed by the caller) receives the number of tokens of every expert."""
    T = h.shape[0]
    idx = torch.empty(T, top, dtype=torch.int32, device=h.device)
    wts = torch.empty(T, top, dtype=torch.float32, device=h.device)
    if _native(h):
        z = router_logits(h, wr)
        count_launch()
        load_kv_ext().moe_topk(z, bias, mode, top, float(rscale), idx, wts, counts)
        return idx, wts
    z = F.linear(h.float(), wr.float())
    if bias is not None:
        z = z + bias.float()
    if mode == ROUTE_SOFTMAX:
        tv, ti = z.topk(top, -1)
        w = torch.softmax(tv, -1) * rscale
    else:
        tv, ti = torch.sigmoid(z).topk(top, -1)
        w = tv * rscale if mode == ROUTE_SIGMOID_RAW else tv / (tv.sum(-1, keepdim=True) + 1e-20) * rscale
    idx.copy_(ti)
    wts.copy_(w)
    if counts is not None:
        counts.add_(torch.bincount(ti.reshape(-1), minlength=counts.numel()).to(counts.dtype))
    return idx, wts


def router_logits(h, wr):
    """``h @ W_rᵀ`` in fp32: bf16 operands go through the tcgen05 GEMM with its fp32 epilogue (products of bf16 numbers are
    exact in fp32 and the accumulator is fp32, so nothing is rounded to 16 bits); anything else is an fp32 product."""
    from . import use_native

    h, wr = h.detach(), wr.detach()
    if (h.dtype == torch.bfloat16 and wr.dtype == torch.bfloat16 and use_native(h) and h.stride(1) == 1 and h.stride(0) % 8 == 0
            and h.shape[1] % 8 == 0 and wr.is_contiguous() and wr.shape[0] % 8 == 0 and h.data_ptr() % 16 == 0 and h.shape[0] > 0):
        z = torch.empty(h.shape[0], wr.shape[0], dtype=torch.float32, device=h.device)
        if _tcgen05_gemm(h, wr, z, False, torch.float32) is not None:
            return z
    return F.linear(h.float(), wr.float())


def moe_pairs(h, wgu, wd, idx, wts, act: int, limit: float = 0.0, weight_input: bool = False):
    """Experts for few tokens: every (token, chosen expert) pair reads its expert's matrices.  ``wgu`` ``[E, 2·ff, width]``
    (gate rows, then up rows), ``wd`` ``[E, width, ff]``.  Returns ``Σ_k wts[t,k] · W_down,k (act(W_gate,k h) · W_up,k h)`` as
    fp32 ``[tokens, width]``; with ``weight_input`` the weight multiplies the expert's input instead (``wts[t,k] · h`` rounded to
    the compute dtype) and the outputs are summed."""
    T, n = h.shape
    top, ff = idx.shape[1], wgu.shape[1] // 2
    out = torch.empty(T, n, dtype=torch.float32, device=h.device)
    if _native(h):
        count_launch(2)
        a = torch.empty(T * top, ff, dtype=h.dtype, device=h.device)
        load_kv_ext().moe_pairs(h, wgu, wd, idx, wts, a, out, act, float(limit), bool(weight_input))
        return out
    for t in range(T):
        acc = torch.zeros(n)
        for k in range(top):
            e = int(idx[t, k])
            hin = (wts[t, k] * h[t].float()).to(h.dtype).float() if weight_input else h[t].float()
            gu = wgu[e].float() @ hin
            a = _gated_pair(gu[:ff], gu[ff:], act, limit).to(h.dtype).float()
            acc += (1.0 if weight_input else wts[t, k]) * (wd[e].float() @ a)
        out[t] = acc
    return out


def moe_sorted(h, wgu, wd, idx, counts, act: int, limit: float = 0.0, in_wts=None):
    """Experts for many tokens: the rows are copied into a matrix sorted by expert, every expert runs as two dense products on
    its row range, and the caller gathers the weighted sum (:func:`dyt_residual` with ``pos``).  Returns
    ``(ys fp32 [rows, width], pos int32 [tokens, top])``: the output row of pair (t, k) is ``ys[pos[t, k]]``.  With ``in_wts``
    (fp32 ``[tokens, top]``) the copied row of pair (t, k) is ``in_wts[t, k] · h[t]``: routing weights on the experts' inputs.

    bf16 on the GPU: every expert's range starts on a multiple of 128 rows and each product is ONE launch of the tcgen05 GEMM
    in its grouped mode (the expert of every 128-row block is a device-side list), so nothing is read back by the host and the
    step can be captured.  Otherwise (fp32, CPU) the per-expert row counts are read back and the experts run one by one."""
    T, n = h.shape
    top, E, ff = idx.shape[1], wgu.shape[0], wgu.shape[1] // 2
    P = T * top
    dev = h.device
    pos = torch.empty(T, top, dtype=torch.int32, device=dev)
    if _native(h) and h.dtype == torch.bfloat16 and n % 8 == 0 and ff % 8 == 0 and E * max(2 * ff, n) < 2 ** 31:
        from . import load_ext

        rows = (P + E * 127 + 127) // 128 * 128
        xs = torch.empty(rows, n, dtype=h.dtype, device=dev)
        meta = torch.empty(2 * E + 1 + rows // 128, dtype=torch.int32, device=dev)
        groups = meta[2 * E + 1:]
        count_launch(5)
        load_kv_ext().moe_sort(h, idx, counts, meta[: E + 1], meta[E + 1: 2 * E + 1], pos, xs, 128, groups, in_wts)
        gu = torch.empty(rows, 2 * ff, dtype=h.dtype, device=dev)
        load_ext().gemm_grouped_blocks(xs, wgu.detach(), groups, gu)
        a = torch.empty(rows, ff, dtype=h.dtype, device=dev)
        act_rows(gu, a, act, gated=True, limit=limit)
        ys = torch.empty(rows, n, dtype=torch.float32, device=dev)
        load_ext().gemm_grouped_blocks(a, wd.detach(), groups, ys)
        return ys, pos
    xs = torch.empty(P, n, dtype=h.dtype, device=dev)
    if _native(h):
        count_launch(2)
        meta = torch.empty(2 * E + 1, dtype=torch.int32, device=dev)
        load_kv_ext().moe_sort(h, idx, counts, meta[: E + 1], meta[E + 1:], pos, xs, 1, None, in_wts)
        cnt = counts.tolist()
    else:
        order = torch.sort(idx.reshape(-1).long(), stable=True).indices
        pos.view(-1)[order] = torch.arange(P, dtype=torch.int32)
        xs.copy_(h[order // top] if in_wts is None else in_wts.reshape(-1)[order][:, None] * h[order // top].float())
        cnt = torch.bincount(idx.reshape(-1).long(), minlength=E).tolist()
    gu = torch.empty(P, 2 * ff, dtype=h.dtype, device=dev)
    a = torch.empty(P, ff, dtype=h.dtype, device=dev)
    ys = torch.empty(P, n, dtype=torch.float32, device=dev)
    _grouped_products(xs, wgu, cnt, gu, False)
    act_rows(gu, a, act, gated=True, limit=limit)
    _grouped_products(a, wd, cnt, ys, False)
    return ys, pos


def _grouped_products(a, w, counts, out, grouped: bool):
    """Rows ``[Σ counts[:e], +counts[e])`` of ``a`` times ``w[e]ᵀ`` into the same rows of ``out``: on the tcgen05 GEMM all
    groups are launched from one native call; otherwise group by group."""
    if grouped:
        from . import load_ext

        try:
            load_ext().gemm_grouped(a, w.detach(), counts, out)
            count_launch(sum(1 for c in counts if c))
            return
        except RuntimeError as e:
            if "failed with code -" not in str(e):      # a CUDA error, not a refusal by the launcher's shape checks
                raise
    at = 0
    for e, c in enumerate(counts):
        if c:
            linear_into(a[at:at + c], w[e], out[at:at + c])
            at += c
