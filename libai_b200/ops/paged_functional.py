"""Operators of decoders whose attention sees the whole past through a paged key/value cache (``csrc/paged_mixers.cu``): the
post-norm residual, the convolved and normalised query / key / value preparation that writes keys and values into their pages,
and softmax attention over the pages with mixed heads and a learned sink.

Every operator takes the step's :class:`~libai_b200.inference.ragged.RaggedBatch`.  On a CUDA device the native kernels run
(a missing extension is an error, there is no fallback); on the CPU the same operators are plain PyTorch, sequence by
sequence, which is what the CPU tests use.  Norms, angles, scores, the softmax and the residual are fp32 in both.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import count_launch, impl, load_kv_ext


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and impl() == "native"


# ------------------------------------------------------------------------------------------------------------ residual
def postnorm_residual(x, w, eps: float, *, alpha: float = 1.0, y=None, y2=None, pos=None, cw=None, h=None, inplace: bool = True):
    """``v = alpha · x + y + y2'``, ``out = v / sqrt(mean(v²) + eps) · (1 + w)`` on the fp32 residual ``x`` ``[rows, width]``.
    ``y`` ``[rows, width]`` (fp32 or the compute dtype) and ``y2`` (fp32) are optional sublayer outputs; with ``pos``
    ``[rows, top]`` the second one is gathered, ``y2' = Σ_k cw[r, k] · y2[pos[r, k]]`` (``cw`` absent: plain sum), which is how
    expert outputs sorted by expert come back to their tokens.  ``out`` replaces ``x`` (``inplace``) and is also written to
    ``h`` (compute dtype) when given — the copy the next sublayer's products read."""
    if _native(x):
        count_launch()
        load_kv_ext().postnorm_residual(x, x if inplace else None, y, y2, pos, cw, float(alpha), w, float(eps), h)
        return x
    v = alpha * x
    if y is not None:
        v = v + y.float()
    if y2 is not None:
        if pos is not None:
            g = y2[pos.long()]
            v = v + (g * cw[:, :, None] if cw is not None else g).sum(1)
        else:
            v = v + y2
    out = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())
    if inplace:
        x.copy_(out)
    if h is not None:
        h.copy_(out)
    return x


# ------------------------------------------------------------------------------------------------- query / key / value rows
def _page_rows(table, slot: int, lo: int, hi: int, page_size: int):
    """(page, row) of the positions ``lo … hi - 1`` of the sequence in ``slot``."""
    p = torch.arange(lo, hi, device=table.device)
    return table[slot, p // page_size].long(), p % page_size


def conv_qkv_prepare(q, k, v, wq, wk, wv, tail, qn, kn, freq, eps: float, rb, pool, table, H: int, G: int, D: int, V: int):
    """From the projections of a step's rows (``q`` ``[tokens, H·D]``, ``k`` ``[tokens, G·D]``, ``v`` ``[tokens, G·V]``: column
    slices of one matrix) to attention inputs:

    * per-channel causal convolution over time, ``y_t = Σ_j w[c, j] · u_(t − taps + 1 + j)`` (``w*`` ``[channels, taps]``, zeros
      before the sequence's start; ``tail`` ``[slots, taps − 1, H·D + G·D + G·V]`` carries the last projections of every
      sequence between steps and is updated);
    * queries and keys: RMS norm over every head with the weights ``qn`` / ``kn`` ``[D]`` shared by the heads, then rotation of
      the pairs ``(c, c + len(freq))`` by ``position · freq[c]``; values: every head divided by its root mean square;
    * keys and values go into the sequence's pages (``pool`` ``[pages, page_size, G·D + G·V]``, ``table`` ``[slots, max_pages]``).

    Returns the prepared queries ``[tokens, H·D]``."""
    qout = torch.empty(q.shape[0], H * D, dtype=q.dtype, device=q.device)
    if _native(q):
        count_launch(2 if wq.shape[1] > 1 else 1)
        load_kv_ext().conv_qkv_prepare(q, k, v, wq, wk, wv, tail, qn, kn, freq, float(eps), qout, pool, table, rb.tok_seq, rb.seq_off,
                                       rb.slots, rb.past, H, G, D, V)
        return qout
    taps, R, half, ps = wq.shape[1], wq.shape[1] - 1, freq.numel(), pool.shape[1]
    w = torch.cat([wq, wk, wv], 0).float()                                    # [C, taps]
    for b in range(rb.B):
        lo, n, slot, past = rb.offsets[b], rb.lens[b], rb.slot_list[b], rb.past_list[b]
        rows = torch.cat([q[lo:lo + n], k[lo:lo + n], v[lo:lo + n]], 1).float()
        prev = tail[slot].float().clone() if R else rows.new_zeros(0, rows.shape[1])
        for r in range(R):
            if past - R + r < 0:
                prev[r] = 0
        full = torch.cat([prev, rows], 0)
        y = sum(full[j:j + n] * w[:, j] for j in range(taps))
        if R:
            tail[slot] = full[full.shape[0] - R:].to(tail.dtype)
        yq, yk, yv = y[:, :H * D].view(n, H, D), y[:, H * D:H * D + G * D].view(n, G, D), y[:, H * D + G * D:].view(n, G, V)
        unit = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)
        yq, yk, yv = unit(yq) * qn.float(), unit(yk) * kn.float(), unit(yv)
        ang = torch.arange(past, past + n, device=q.device).float()[:, None] * freq.float()[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

        def turn(t):
            a, c = t[..., :half], t[..., half:2 * half]
            return torch.cat([a * cos - c * sin, c * cos + a * sin, t[..., 2 * half:]], -1)

        qout[lo:lo + n] = turn(yq).reshape(n, H * D).to(qout.dtype)
        page, row = _page_rows(table, slot, past, past + n, ps)
        pool[page, row] = torch.cat([turn(yk).reshape(n, G * D), yv.reshape(n, G * V)], 1).to(pool.dtype)
    return qout


# --------------------------------------------------------------------------------------------------------------- attention
PROMPT_QUERY_TILE = 8          # most queries of one sequence that a block of the generic prompt kernel takes
MMA_QUERY_TILE = 16            # queries per block of the tensor-core prompt kernel
MMA_HEAD_SIZES = (64, 128)     # head sizes (keys = values) the tensor-core prompt kernel is built for
MMA_MAX_HEADS = 16


def mma_eligible(q, pool, y, H: int, G: int, D: int, V: int) -> bool:
    """bf16 prompt steps whose sizes the tensor-core kernel is built for (its shared memory must hold a tile of all heads)."""
    smem = 2 * (2 * 32 * (G * D + 8) + 16 * (H * D + 8) + H * (16 * 40 + 8)) + 4 * (H * 16 * 33 + 2 * H * 16 + H * H)
    return (q.dtype == torch.bfloat16 and D == V and D in MMA_HEAD_SIZES and H <= MMA_MAX_HEADS and smem <= 220 * 1024
            and H % G == 0 and (H * 32) % (G * D // 8) == 0
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and y.stride(0) % 2 == 0 and y.data_ptr() % 4 == 0)


def talk_attention(q, pool, table, rb, y, H: int, G: int, D: int, V: int, scale: float, *, talk=None, sink=None,
                   out_scale: float = 1.0, parts: Optional[int] = None, mma: bool = True):
    """Causal softmax attention of every packed query over the positions ``0 … its own`` of its sequence, keys and values read
    from the pages (the step's own rows have been written).  ``talk`` (fp32 ``[H, H]``): the heads' scaled scores are mixed
    before the softmax, ``s'_h = Σ_g talk[h, g] · s_g``; ``sink`` (fp32 ``[H]``): the denominator also holds ``exp(sink_h)``, an
    entry without a key or a value.  Query head h reads key/value head ``h // (H/G)``.  The result, times ``out_scale``, goes to
    ``y`` ``[tokens, H·V]``.  ``parts``: into how many parts the keys of a query tile are cut (``None`` chooses: single-token
    steps spread every sequence over the device, prompt steps keep a tile's keys together).  bf16 prompt steps with head sizes
    the tensor-core kernel is built for take it; ``mma=False`` keeps them on the generic kernel (fp32 inputs always are)."""
    if _native(q):
        ext = load_kv_ext()
        if mma and not rb.single and parts in (None, 1) and mma_eligible(q, pool, y, H, G, D, V):
            seq, start = rb.query_tiles(MMA_QUERY_TILE)
            count_launch()
            ext.talk_attention(q, pool, table, talk, sink, seq, start, MMA_QUERY_TILE, 32, rb.seq_off, rb.slots, rb.past, y, None, 1, H, G,
                               D, V, float(scale), float(out_scale))
            return y
        qt, kt = ext.talk_attention_tiles(1 if rb.single else PROMPT_QUERY_TILE, H, G, D, V)
        if qt == 0:
            raise RuntimeError(f"talk_attention: heads of {H}x{D} / {G}x{V} do not fit a block's shared memory")
        # single-token steps: a tile per token, named by the step's own descriptor (nothing is built on the host, so the step
        # can be captured in a CUDA graph)
        seq, start = (rb.tok_seq, None) if rb.single else rb.query_tiles(qt)
        if parts is None:
            parts = max(1, min(16, -(-296 // max(1, seq.numel())))) if rb.single else 1
        part = torch.empty(q.shape[0] * parts * H * (V + 2), dtype=torch.float32, device=q.device) if parts > 1 else None
        count_launch(2 if parts > 1 else 1)
        ext.talk_attention(q, pool, table, talk, sink, seq, start, qt, kt, rb.seq_off, rb.slots, rb.past, y, part, parts, H, G, D, V,
                           float(scale), float(out_scale))
        return y
    rep, ps = H // G, pool.shape[1]
    for b in range(rb.B):
        lo, n, slot, past = rb.offsets[b], rb.lens[b], rb.slot_list[b], rb.past_list[b]
        page, row = _page_rows(table, slot, 0, past + n, ps)
        rows = pool[page, row].float()
        kk = rows[:, :G * D].view(-1, G, D).repeat_interleave(rep, 1)
        vv = rows[:, G * D:].view(-1, G, V).repeat_interleave(rep, 1)
        s = torch.einsum("ihd,jhd->hij", q[lo:lo + n].float().view(n, H, D), kk) * scale
        if talk is not None:
            s = torch.einsum("hg,gij->hij", talk.float(), s)
        i = torch.arange(past, past + n, device=q.device)[:, None]
        j = torch.arange(past + n, device=q.device)[None, :]
        s = s.masked_fill((j > i)[None], float("-inf"))
        if sink is not None:
            s = torch.cat([s, sink.float()[:, None, None].expand(H, n, 1)], -1)
        p = torch.softmax(s, -1)[..., :past + n]
        y[lo:lo + n] = (torch.einsum("hij,jhv->ihv", p, vv).reshape(n, H * V) * out_scale).to(y.dtype)
    return y
