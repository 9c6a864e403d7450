"""Prefill / decode throughput of the stateful models (Bumodra: delta-rule and latent-attention mixers; Nefelorn: ring-cached
attention with chunk / kept-first window masks and mixture-of-experts feed-forwards) beside Llama at equal width, depth and
(active) feed-forward size, and of Salizen (hyper-connection streams, linear-attention recurrences, sink-softmax window
attention) beside Nefelorn, and of Zubarax (post-norm blocks, paged attention with mixed heads beside an HGRN2 recurrence,
input-weighted experts) beside Salizen, random weights, one GPU.  ``bench.py --serving [--serving-model nefelorn|salizen|zubarax]`` prints the result
as one JSON line; ``--serving-kernels`` adds device times of the individual kernels of one block at the same sizes with their
roofline fractions.

Timing: CUDA events on the launching stream after warm-up steps, a synchronize on both sides, an L2 flush (a write larger
than L2) between timed iterations of the kernel table.
"""
from __future__ import annotations

import json
import os
import time

import torch

SIZES = {
    # name: width, ff, heads, head dim, latent ranks, window, blocks
    "w1024": dict(width=1024, ff=4096, heads=8, dim=128, q_rank=512, kv_rank=256, window=512, blocks=4, vocab=32000),
    "w2048": dict(width=2048, ff=8192, heads=16, dim=128, q_rank=768, kv_rank=512, window=1024, blocks=4, vocab=32000),
}


def bumodra_config(s):
    att = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": s["ff"]},
           "mixer": {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "q_rank": s["q_rank"], "kv_rank": s["kv_rank"],
                     "mask": {"size": s["window"]}, "scale": s["dim"] ** -0.5}}
    delta = {"type": "delta", "mlp": {"kind": "dense", "ff": s["ff"]},
             "mixer": {"heads": s["heads"], "kv_heads": s["heads"] // 2, "dim": s["dim"], "vdim": s["dim"], "conv": 4}}
    chan = {"type": "channel_delta", "mlp": {"kind": "dense", "ff": s["ff"]},
            "mixer": {"heads": s["heads"], "kv_heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "conv": 4,
                      "decay_rank": 64, "gate_rank": 64}}
    kinds = [att, delta, delta, chan]
    return dict(vocab=s["vocab"], width=s["width"], norm={"eps": 1e-6}, layers=[kinds[i % 4] for i in range(s["blocks"])])


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]) * 1e9, float(p["bf16_tflops"]) * 1e12, "measured"
    except Exception:
        return 6.65e12, 1.59e15, "fallback"


def _time(fn, warmup=3, iters=10, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def build_models(s, device="cuda"):
    from libai_b200.config import DictConfig
    from libai_b200.layers._param import param_defaults
    from libai_b200.models import BumodraForCausalLM, LlamaForCausalLM

    with param_defaults(dtype=torch.bfloat16, device=device, seed=1):
        bum = BumodraForCausalLM(DictConfig(bumodra_config(s))).eval()
        # SwiGLU has three matrices where the dense feed-forward has two: 2/3 of ff gives the same parameter count
        llama = LlamaForCausalLM(DictConfig(dict(
            hidden_layers=s["blocks"], vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=(2 * s["ff"] // 3 + 127) // 128 * 128,
            num_attention_heads=s["heads"] if s["width"] // s["heads"] in (64, 128) else s["width"] // 128,
            max_position_embeddings=8192, rms_norm_eps=1e-6, initializer_range=0.02, use_scaled_init_for_output_weights=True,
            scale_mask_softmax_fusion=False, amp_enabled=False))).eval()
    return bum.cuda(), llama.cuda()            # .cuda(): the rotary tables are buffers built on the host


@torch.no_grad()
def throughput(s, batch, prompt, new_tokens, steps, warmup):
    from libai_b200.inference.scheduler import RequestScheduler

    bum, llama = build_models(s)
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(1, s["vocab"], (batch, prompt), generator=gen)
    out = {}
    # ---- the stateful model through its scheduler: one ragged prefill step, then single-token steps
    sched = RequestScheduler(bum)
    prompts = [row.tolist() for row in ids]

    def prefill():
        sched.step([(("p", i), p, [len(p) - 1]) for i, p in enumerate(prompts)])
        sched.finish([("p", i) for i in range(batch)])

    out["bumodra_prefill_ms"] = _time(prefill, warmup, steps)
    sched.step([(("d", i), p, []) for i, p in enumerate(prompts)])
    entries = [(("d", i), [7], [0]) for i in range(batch)]
    out["bumodra_decode_ms"] = _time(lambda: sched.step(entries), warmup, new_tokens)
    sched.finish([("d", i) for i in range(batch)])
    # ---- Llama: the prompt through the packed flash-attention path (no cache), single tokens against a key/value cache of
    # `prompt` positions per layer (filled with random values: only the time matters) as Generator.generate drives them
    dev_ids = ids.cuda()
    out["llama_prefill_ms"] = _time(lambda: llama(dev_ids), warmup, steps)
    a, d = llama.model.layers[0].self_attn.local_heads, llama.model.layers[0].self_attn.head_size
    one = dev_ids[:, :1].contiguous()

    def llama_decode():
        llama(one, use_cache=True)

    def fill_cache():
        llama.set_cache([(torch.randn(batch, a, prompt, d, device="cuda").to(torch.bfloat16),
                          torch.randn(batch, a, prompt, d, device="cuda").to(torch.bfloat16)) for _ in range(s["blocks"])])

    fill_cache()
    out["llama_decode_ms"] = _time(llama_decode, warmup, new_tokens)
    llama.set_cache(None)
    for name in ("bumodra", "llama"):
        out[f"{name}_prefill_tokens_per_s"] = batch * prompt / out[f"{name}_prefill_ms"] * 1e3
        out[f"{name}_decode_tokens_per_s"] = batch / out[f"{name}_decode_ms"] * 1e3
    out["params_bumodra"] = sum(p.numel() for p in bum.parameters())
    out["params_llama"] = sum(p.numel() for p in llama.parameters())
    return out


@torch.no_grad()
def kernel_table(s, batch, prompt):
    """Device time of every kernel of the mixers at these sizes (prefill rows = batch·prompt; decode rows = batch), with the
    bytes / FLOPs the operation needs and the fraction of the measured roofline that this is."""
    from libai_b200.inference.ragged import RaggedBatch
    from libai_b200.ops import functional as OF
    from libai_b200.ops import seq_functional as SF

    hbm, flops, src = _peaks()
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, D, W, C = s["heads"], s["dim"], s["window"], s["kv_rank"]
    rows = []

    def add(name, ms, bytes_=0.0, fl=0.0):
        ideal = max(bytes_ / hbm, fl / flops) * 1e3
        rows.append(dict(kernel=name, ms=round(ms, 4), ideal_ms=round(ideal, 5), roofline_fraction=round(ideal / ms, 4),
                         bound="memory" if bytes_ / hbm >= fl / flops else "tensor"))

    for phase, lens, past in (("prefill", [prompt] * batch, [0] * batch), ("decode", [1] * batch, [prompt] * batch)):
        rb = RaggedBatch(lens, list(range(batch)), past, dev)
        T = rb.tokens
        x = torch.randn(T, s["width"], device=dev)
        w = torch.zeros(s["width"], dtype=bf, device=dev)
        h = torch.empty(T, s["width"], dtype=bf, device=dev)
        add(f"{phase}: rms norm fp32→bf16", _time(lambda: SF.rms_norm_rows(x, w, offset=1.0, eps=1e-6, out=h), flush=flush), T * s["width"] * 6)
        # delta rule: convolution, scan, gated norm
        KH = H // 2
        Cq = 2 * KH * D + H * D
        qkv = torch.randn(T, Cq, device=dev).to(bf)
        cw = torch.randn(Cq, 4, device=dev).to(bf)
        tail = torch.zeros(batch, 3, Cq, dtype=bf, device=dev)
        conv = torch.empty_like(qkv)
        add(f"{phase}: short conv + silu", _time(lambda: SF.short_conv(qkv, cw, tail, rb, conv), flush=flush), T * Cq * 4)
        a, b = torch.randn(T, H, device=dev).to(bf), torch.randn(T, H, device=dev).to(bf)
        A_log, dtb = torch.zeros(H, dtype=bf, device=dev), torch.zeros(H, dtype=bf, device=dev)
        S = torch.zeros(batch, H, D, D, device=dev)
        state_bytes = batch * H * D * D * 4 * (2 if phase == "decode" else 1)
        add(f"{phase}: delta scan (per-head decay)", _time(lambda: SF.delta_scan(conv, KH * D, 2 * KH * D, a, b, A_log, dtb, S, rb, KH, False), flush=flush),
            T * (Cq * 2 + H * D * 4) + state_bytes, 0.0)
        o = torch.randn(T, H * D, device=dev)
        g, nw, y = torch.randn(T, H * D, device=dev).to(bf), torch.ones(D, dtype=bf, device=dev), torch.empty(T, H * D, dtype=bf, device=dev)
        add(f"{phase}: gated rms norm", _time(lambda: SF.gated_rmsnorm(o, g, nw, 1e-6, 0, y, H, D), flush=flush), T * H * D * 8)
        # latent attention
        ring = torch.randn(batch, W, C, device=dev).to(bf)
        c = torch.randn(T, C, device=dev).to(bf)
        q = torch.randn(T, H * D, device=dev).to(bf)
        gate = torch.randn(T, H, device=dev).to(bf)
        if phase == "prefill":
            kv = torch.randn(rb.ext(W).rows, 2 * H * D, device=dev).to(bf)
            pairs = sum(min(t + 1, W) for t in range(prompt)) * batch
            add("prefill: window attention", _time(lambda: SF.window_attention(q, kv, gate, rb, y, H, D, D, W, D ** -0.5), flush=flush),
                T * H * D * 4 + kv.numel() * 2, pairs * H * D * 4.0)
            qkv4 = torch.randn(batch, prompt, H, 3 * D, device=dev).to(bf)
            add("prefill: Llama causal flash attention (same heads, full context)",
                _time(lambda: OF.attention_qkvpacked(qkv4, causal=True, scale=D ** -0.5), flush=flush),
                qkv4.numel() * 2 + T * H * D * 2, batch * prompt * (prompt + 1) / 2 * H * D * 4.0)
        else:
            qa = torch.randn(batch, H, C, device=dev)
            add("decode: absorbed latent attention", _time(lambda: SF.latent_decode(qa, ring, c, rb, W, D ** -0.5), flush=flush),
                batch * W * C * 2 + batch * H * C * 8)
            k = torch.randn(batch, H, prompt, D, device=dev).to(bf)
            v = torch.randn(batch, H, prompt, D, device=dev).to(bf)
            q1 = torch.randn(batch, H, 1, D, device=dev).to(bf)
            add("decode: Llama attention over its key/value cache",
                _time(lambda: OF.attention(q1, k, v, causal=False, scale=D ** -0.5), flush=flush), k.numel() * 4)
    return {"peaks": src, "hbm_bytes_per_s": hbm, "bf16_flops": flops, "rows": rows}


# ======================================================================================================================
# Nefelorn beside Llama
# ======================================================================================================================
NEFELORN_SIZES = {
    # heads × dim with grouped keys, mask reach, experts (top of them active; top · expert_ff = Llama's intermediate size)
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, reach=512, keep=8, ff=4096, experts=16, top=2, expert_ff=1408,
                  blocks=4, vocab=32000),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, reach=1024, keep=8, ff=8192, experts=32, top=2, expert_ff=2816,
                  blocks=4, vocab=32000),
}


def nefelorn_config(s):
    D = s["dim"]
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"], "scale": 1.0}}

    def chunked(mlp, kv_from=None):
        m = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": D, "vdim": D, "mask": {"size": s["reach"]}, "scale": D ** -0.5,
             "rot": {"dims": D, "base": 500000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 24.0, "slow": 2.0}}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "attention", "mixer": m, "mlp": mlp}

    def windowed(mlp):
        return {"type": "attention_2", "mlp": mlp,
                "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": D, "vdim": D, "scale": D ** -0.5,
                          "mask": {"size": s["reach"], "keep_first": s["keep"]}, "rot": {"dims": D // 2, "base": 10000.0}}}

    kinds = [chunked({"kind": "dense", "ff": s["ff"]}), windowed(moe), chunked(moe, kv_from=0), windowed(moe)]
    layers = []
    for i in range(s["blocks"]):
        lc = json.loads(json.dumps(kinds[i % 4]))
        if "kv_from" in lc["mixer"]:
            lc["mixer"]["kv_from"] = i - 2
        layers.append(lc)
    return dict(vocab=s["vocab"], width=s["width"], norm={"eps": 1e-6}, embedding={"scale": s["width"] ** 0.5}, logit_softcap=50.0,
                layers=layers)


def build_nefelorn_and_llama(s, device="cuda"):
    from libai_b200.config import DictConfig
    from libai_b200.layers._param import param_defaults
    from libai_b200.models import LlamaForCausalLM, NefelornForCausalLM

    with param_defaults(dtype=torch.bfloat16, device=device, seed=1):
        nef = NefelornForCausalLM(DictConfig(nefelorn_config(s))).eval()
        llama = LlamaForCausalLM(DictConfig(dict(
            hidden_layers=s["blocks"], vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["top"] * s["expert_ff"],
            num_attention_heads=s["heads"], max_position_embeddings=8192, rms_norm_eps=1e-6, initializer_range=0.02,
            use_scaled_init_for_output_weights=True, scale_mask_softmax_fusion=False, amp_enabled=False))).eval()
    return nef.cuda(), llama.cuda()


@torch.no_grad()
def throughput_nefelorn(s, batch, prompt, new_tokens, steps, warmup):
    from libai_b200.inference.scheduler import RequestScheduler

    nef, llama = build_nefelorn_and_llama(s)
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(1, s["vocab"], (batch, prompt), generator=gen)
    out = {}
    sched = RequestScheduler(nef)
    prompts = [row.tolist() for row in ids]

    def prefill():
        sched.step([(("p", i), p, [len(p) - 1]) for i, p in enumerate(prompts)])
        sched.finish([("p", i) for i in range(batch)])

    out["nefelorn_prefill_ms"] = _time(prefill, warmup, steps)
    sched.step([(("d", i), p, []) for i, p in enumerate(prompts)])
    entries = [(("d", i), [7], [0]) for i in range(batch)]
    out["nefelorn_decode_ms"] = _time(lambda: sched.step(entries), warmup, new_tokens)
    sched.cuda_graphs = False
    out["nefelorn_decode_eager_ms"] = _time(lambda: sched.step(entries), warmup, new_tokens)
    sched.finish([("d", i) for i in range(batch)])
    dev_ids = ids.cuda()
    out["llama_prefill_ms"] = _time(lambda: llama(dev_ids), warmup, steps)
    a, d = llama.model.layers[0].self_attn.local_heads, llama.model.layers[0].self_attn.head_size
    one = dev_ids[:, :1].contiguous()
    llama.set_cache([(torch.randn(batch, a, prompt, d, device="cuda").to(torch.bfloat16),
                      torch.randn(batch, a, prompt, d, device="cuda").to(torch.bfloat16)) for _ in range(s["blocks"])])
    out["llama_decode_ms"] = _time(lambda: llama(one, use_cache=True), warmup, new_tokens)
    llama.set_cache(None)
    for name in ("nefelorn", "llama"):
        out[f"{name}_prefill_tokens_per_s"] = batch * prompt / out[f"{name}_prefill_ms"] * 1e3
        out[f"{name}_decode_tokens_per_s"] = batch / out[f"{name}_decode_ms"] * 1e3
    out["params_nefelorn"] = sum(p.numel() for p in nef.parameters())
    out["params_llama"] = sum(p.numel() for p in llama.parameters())
    return out


@torch.no_grad()
def kernel_table_nefelorn(s, batch, prompt):
    """Device time of every kernel of a Nefelorn block at these sizes (prefill rows = batch·prompt; decode rows = batch) beside
    the like kernel of Llama, with the bytes / FLOPs the operation needs and the fraction of the measured roofline."""
    from libai_b200.config import DictConfig
    from libai_b200.inference.ragged import RaggedBatch
    from libai_b200.layers import DynamicTanh, MoEFeedForward
    from libai_b200.layers._param import param_defaults
    from libai_b200.models.llama_model import LlamaMLP
    from libai_b200.ops import functional as OF
    from libai_b200.ops import kv_functional as KF

    hbm, flops, src = _peaks()
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    n, H, G, D, R, keep = s["width"], s["heads"], s["kv_heads"], s["dim"], s["reach"], s["keep"]
    E, top, ff = s["experts"], s["top"], s["expert_ff"]
    C = G * 2 * D
    rows = []

    def add(name, ms, bytes_=0.0, fl=0.0):
        ideal = max(bytes_ / hbm, fl / flops) * 1e3
        rows.append(dict(kernel=name, ms=round(ms, 4), ideal_ms=round(ideal, 5), roofline_fraction=round(ideal / ms, 4),
                         bound="memory" if bytes_ / hbm >= fl / flops else "tensor"))

    with param_defaults(dtype=bf, device=dev, seed=2):
        na, nb = DynamicTanh(n), DynamicTanh(n)
        moe = MoEFeedForward(n, ff, E, top)
        lmlp = LlamaMLP(n, top * ff)
    freq, ms_ = KF.rotary_frequencies(D, 5e5, {"factor": 4.0, "original": 4096, "fast": 24.0, "slow": 2.0})
    freq = freq.to(dev)
    for phase, lens, past in (("prefill", [prompt] * batch, [0] * batch), ("decode", [1] * batch, [prompt] * batch)):
        rb = RaggedBatch(lens, list(range(batch)), past, dev)
        T = rb.tokens
        x, y32 = torch.randn(T, n, device=dev), torch.randn(T, n, device=dev)
        h = torch.empty(T, n, dtype=bf, device=dev)
        add(f"{phase}: closing norm + residual + opening norm (Dynamic Tanh)",
            _time(lambda: KF.dyt_residual(x, y32, post=na.triple(), nxt=nb.triple(), h=h), flush=flush), T * n * 14)
        xb = torch.randn(T, n, device=dev).to(bf)
        w = torch.ones(n, dtype=bf, device=dev)
        add(f"{phase}: Llama RMS norm", _time(lambda: OF.rms_norm(xb, w, 1e-6), flush=flush), T * n * 4)
        q = torch.randn(T, H * D, device=dev).to(bf)
        kv = torch.randn(T, C, device=dev).to(bf)
        qw, kw = torch.ones(H * D, dtype=bf, device=dev), torch.ones(G * D, dtype=bf, device=dev)
        add(f"{phase}: query/key norm + rotation (whole-projection norm)",
            _time(lambda: KF.qk_prepare(q, kv[:, :G * D], qw, kw, freq, ms_, rb, H, G, D, 1e-6, True, False), flush=flush), T * (H + G) * D * 4)
        ring = torch.randn(batch, R, C, device=dev).to(bf)
        first = torch.randn(batch, keep, C, device=dev).to(bf)
        add(f"{phase}: cache write", _time(lambda: KF.kv_write(ring, first, kv[:, :G * D], kv[:, G * D:], rb), flush=flush),
            min(T, batch * R) * C * 4)
        gate = torch.randn(T, H, device=dev).to(bf)
        yb = torch.empty(T, H * D, dtype=bf, device=dev)
        if phase == "prefill":
            ext = rb.kv_ext([(R, 0, keep)])
            pairs = sum(min(t + 1, R) + (min(keep, t + 1 - R) if t + 1 > R else 0) for t in range(prompt)) * batch
            add("prefill: sliding-window + kept-first attention (mma.sync)",
                _time(lambda: KF.masked_attention(q, kv[:, :G * D], kv[:, G * D:], ext, None, rb, yb, H, G, D, D, R, 0, keep, D ** -0.5), flush=flush),
                T * H * D * 4 + T * C * 2, pairs * H * D * 4.0)
            ext2 = rb.kv_ext([(0, R, 0)])
            pairs2 = sum(t % R + 1 for t in range(prompt)) * batch
            add("prefill: chunked attention with head gate (mma.sync)",
                _time(lambda: KF.masked_attention(q, kv[:, :G * D], kv[:, G * D:], ext2, gate, rb, yb, H, G, D, D, 0, R, 0, D ** -0.5), flush=flush),
                T * H * D * 4 + T * C * 2, pairs2 * H * D * 4.0)
            qkv4 = torch.randn(batch, prompt, H, 3 * D, device=dev).to(bf)
            add("prefill: Llama causal flash attention (tcgen05; same heads, full context)",
                _time(lambda: OF.attention_qkvpacked(qkv4, causal=True, scale=D ** -0.5), flush=flush),
                qkv4.numel() * 2 + T * H * D * 2, batch * prompt * (prompt + 1) / 2 * H * D * 4.0)
        else:
            add("decode: grouped ring attention (window + kept-first)",
                _time(lambda: KF.ring_attention(q, ring, first, None, rb, yb, H, G, D, D, R, 0, keep, D ** -0.5), flush=flush),
                batch * (min(prompt + 1, R) + keep) * C * 2)
            add("decode: one-warp-per-head ring attention (the generic kernel)",
                _time(lambda: KF.ring_attention(q, ring, first, None, rb, yb, H, G, D, D, R, 0, keep, D ** -0.5, splits=0), flush=flush),
                batch * (min(prompt + 1, R) + keep) * C * 2)
            k = torch.randn(batch, H, prompt, D, device=dev).to(bf)
            v = torch.randn(batch, H, prompt, D, device=dev).to(bf)
            q1 = torch.randn(batch, H, 1, D, device=dev).to(bf)
            add("decode: Llama attention over its key/value cache",
                _time(lambda: OF.attention(q1, k, v, causal=False, scale=D ** -0.5), flush=flush), k.numel() * 4)
        hb = torch.randn(T, n, device=dev).to(bf)
        add(f"{phase}: router (sigmoid, top-{top} of {E})", _time(lambda: KF.moe_route(hb, moe.router, top, 1.0), flush=flush),
            T * n * 2 + E * n * 2)
        if phase == "prefill":
            add("prefill: experts (sort by expert, two grouped tcgen05 GEMM launches, gated activation)",
                _time(lambda: moe(hb), flush=flush), 0.0, T * top * 3 * ff * n * 2.0)
            add("prefill: Llama gated feed-forward of the active size (tcgen05 GEMMs)", _time(lambda: lmlp(hb), flush=flush), 0.0,
                T * 3 * top * ff * n * 2.0)
        else:
            idx, wts = KF.moe_route(hb, moe.router, top, 1.0)
            used = int(torch.unique(idx).numel())
            add("decode: experts, pair by pair (two kernels)",
                _time(lambda: KF.moe_pairs(hb, moe.gate_up, moe.down, idx, wts, KF.ACT_SILU), flush=flush), used * 3 * ff * n * 2)
            add("decode: Llama gated feed-forward of the active size", _time(lambda: lmlp(hb), flush=flush), 3 * top * ff * n * 2)
    return {"peaks": src, "hbm_bytes_per_s": hbm, "bf16_flops": flops, "rows": rows}


# ======================================================================================================================
# Salizen beside Nefelorn (the framework's closest model: ring-cached window attention, experts, the same scheduler)
# ======================================================================================================================
def salizen_config(s):
    """The sizes of :data:`NEFELORN_SIZES`: the attention side of the parallel block has Nefelorn's heads and reach, the
    recurrences have as many heads of the same size, dense and expert feed-forwards have Nefelorn's sizes."""
    D, H = s["dim"], s["heads"]
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    left = {"heads": H, "kv_heads": s["kv_heads"], "dim": D, "vdim": D, "mask": {"size": s["reach"]}, "scale": D ** -0.5, "softcap": 30.0,
            "rot": {"dims": D // 2, "base": 1000000.0, "scaling": {"factor": 8.0, "original": 8192, "low": 1.0, "high": 4.0}}}
    right = {"heads": H, "dim": D // 2, "vdim": D, "tau": 8.0, "decay_rank": 64}
    decay = [1.0 - 2.0 ** (-3 - (i % 8)) for i in range(H)]
    kinds = [{"type": "parallel", "mlp": {"kind": "dense", "ff": s["ff"]},
              "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.7}},
             {"type": "retention", "mlp": moe, "mixer": {"heads": H, "dim": D, "vdim": D, "decay": decay, "rot": {"dims": D, "base": 10000.0}}},
             {"type": "lightning", "mlp": moe, "mixer": {"heads": H, "dim": D, "vdim": D, "decay": decay}},
             {"type": "lightning", "mlp": moe, "mixer": {"heads": H, "dim": D, "vdim": D, "decay": decay}}]
    return dict(vocab=s["vocab"], width=s["width"], streams=2, norm={"eps": 1e-6},
                embedding={"scale": s["width"] ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 13}},
                layers=[json.loads(json.dumps(kinds[i % 4])) for i in range(s["blocks"])])


def _stateful_throughput(model, name, ids, batch, new_tokens, steps, warmup, out):
    """Prefill (one ragged step for all prompts) and single-token steps (graph replay, and eager launches) through the scheduler."""
    from libai_b200.inference.scheduler import RequestScheduler

    sched = RequestScheduler(model)
    prompts = [row.tolist() for row in ids]

    def prefill():
        sched.step([(("p", i), p, [len(p) - 1]) for i, p in enumerate(prompts)])
        sched.finish([("p", i) for i in range(batch)])

    out[f"{name}_prefill_ms"] = _time(prefill, warmup, steps)
    sched.step([(("d", i), p, []) for i, p in enumerate(prompts)])
    entries = [(("d", i), [7], [0]) for i in range(batch)]
    out[f"{name}_decode_ms"] = _time(lambda: sched.step(entries), warmup, new_tokens)
    sched.cuda_graphs = False
    out[f"{name}_decode_eager_ms"] = _time(lambda: sched.step(entries), warmup, new_tokens)
    sched.finish([("d", i) for i in range(batch)])
    out[f"{name}_prefill_tokens_per_s"] = batch * ids.shape[1] / out[f"{name}_prefill_ms"] * 1e3
    out[f"{name}_decode_tokens_per_s"] = batch / out[f"{name}_decode_ms"] * 1e3
    out[f"params_{name}"] = sum(p.numel() for p in model.parameters())


@torch.no_grad()
def throughput_salizen(s, batch, prompt, new_tokens, steps, warmup):
    from libai_b200.config import DictConfig
    from libai_b200.layers._param import param_defaults
    from libai_b200.models import NefelornForCausalLM, SalizenForCausalLM

    ids = torch.randint(1, s["vocab"], (batch, prompt), generator=torch.Generator().manual_seed(0))
    out = {}
    for name, cls, cfg in (("salizen", SalizenForCausalLM, salizen_config(s)), ("nefelorn", NefelornForCausalLM, nefelorn_config(s))):
        with param_defaults(dtype=torch.bfloat16, device="cuda", seed=1):
            model = cls(DictConfig(cfg)).eval().cuda()
        _stateful_throughput(model, name, ids, batch, new_tokens, steps, warmup, out)
        del model
        torch.cuda.empty_cache()
    return out


@torch.no_grad()
def kernel_table_salizen(s, batch, prompt):
    """Device time of every kernel of a Salizen block at these sizes (prefill rows = batch·prompt; decode rows = batch) beside the
    like kernel of Nefelorn (or, for the recurrence, of Bumodra), with the bytes / FLOPs the operation needs and the fraction of
    the measured roofline."""
    from libai_b200.inference.ragged import RaggedBatch
    from libai_b200.layers import DynamicTanh
    from libai_b200.layers._param import param_defaults
    from libai_b200.ops import kv_functional as KF
    from libai_b200.ops import lin_functional as LF
    from libai_b200.ops import seq_functional as SF

    hbm, flops, src = _peaks()
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    n, H, G, D, R = s["width"], s["heads"], s["kv_heads"], s["dim"], s["reach"]
    E, top, S = s["experts"], s["top"], 2
    C = G * 2 * D
    rows = []

    def add(name, ms, bytes_=0.0, fl=0.0):
        ideal = max(bytes_ / hbm, fl / flops) * 1e3
        rows.append(dict(kernel=name, ms=round(ms, 4), ideal_ms=round(ideal, 5), roofline_fraction=round(ideal / ms, 4),
                         bound="memory" if bytes_ / hbm >= fl / flops else "tensor"))

    with param_defaults(dtype=bf, device=dev, seed=2):
        na, nb = DynamicTanh(n), DynamicTanh(n)
    mix, outw, inw = torch.eye(S, device=dev) * 0.9 + 0.05, torch.ones(S, device=dev), torch.ones(S, device=dev) * 0.5
    table = torch.randn(s["vocab"], n, device=dev).to(bf)
    bigram = torch.randn(65522, n, device=dev).to(bf)
    for phase, lens, past in (("prefill", [prompt] * batch, [0] * batch), ("decode", [1] * batch, [prompt] * batch)):
        rb = RaggedBatch(lens, list(range(batch)), past, dev)
        T = rb.tokens
        ids = torch.randint(0, s["vocab"], (T,), device=dev)
        last = torch.zeros(batch, dtype=torch.int32, device=dev)
        xs = torch.randn(S, T, n, device=dev)
        add(f"{phase}: token + bigram embedding into {S} streams", _time(lambda: LF.embed_bigram(table, bigram, ids, last, rb, 30.0, 31, 13, 65521, xs), flush=flush),
            T * n * (4 + 4 * S))
        x1 = torch.randn(T, n, device=dev)
        add(f"{phase}: Nefelorn embedding", _time(lambda: KF.embed_scale(table, ids, 30.0, x1), flush=flush), T * n * 6)
        y32 = torch.randn(T, n, device=dev)
        h = torch.empty(T, n, dtype=bf, device=dev)
        w = torch.ones(n, dtype=bf, device=dev)
        add(f"{phase}: stream write-back + read + RMS norm ({S} streams)",
            _time(lambda: LF.hc_step(xs, y32, post=(mix, outw), nxt=(inw, w), h=h, eps=1e-6), flush=flush), T * n * (8 * S + 6))
        add(f"{phase}: Nefelorn closing norm + residual + opening norm (one stream)",
            _time(lambda: KF.dyt_residual(x1, y32, post=na.triple(), nxt=nb.triple(), h=h), flush=flush), T * n * 14)
        # attention side: rotation, cache write, attention with cap + sink + channel gate beside the same kernel without them
        q = torch.randn(T, H * D, device=dev).to(bf)
        kv = torch.randn(T, C, device=dev).to(bf)
        freq, ms_ = KF.rotary_frequencies(D // 2, 1e6, {"factor": 8.0, "original": 8192, "low": 1.0, "high": 4.0})
        freq = freq.to(dev)
        add(f"{phase}: rotation of queries and keys", _time(lambda: KF.qk_prepare(q, kv[:, :G * D], None, None, freq, ms_, rb, H, G, D, 1e-6, False, False), flush=flush),
            T * (H + G) * D * 4)
        ring = torch.randn(batch, R, C, device=dev).to(bf)
        first = torch.zeros(batch, 0, C, dtype=bf, device=dev)
        wide, narrow = torch.randn(T, H * D, device=dev).to(bf), torch.randn(T, H, device=dev).to(bf)
        yb = torch.empty(T, H * D, dtype=bf, device=dev)
        extra = dict(softcap=30.0, sink=True, gate_wide=True, out_scale=0.7)
        if phase == "prefill":
            ext = rb.kv_ext([(R, 0, 0)])
            pairs = sum(min(t + 1, R) for t in range(prompt)) * batch
            add("prefill: window attention with score cap, sink and channel gate (mma.sync)",
                _time(lambda: KF.masked_attention(q, kv[:, :G * D], kv[:, G * D:], ext, wide, rb, yb, H, G, D, D, R, 0, 0, D ** -0.5, **extra), flush=flush),
                T * H * D * 6 + T * C * 2, pairs * H * D * 4.0)
            add("prefill: Nefelorn window attention with head gate (same kernel without them)",
                _time(lambda: KF.masked_attention(q, kv[:, :G * D], kv[:, G * D:], ext, narrow, rb, yb, H, G, D, D, R, 0, 0, D ** -0.5), flush=flush),
                T * H * D * 4 + T * C * 2, pairs * H * D * 4.0)
        else:
            add("decode: grouped ring attention with score cap, sink and channel gate",
                _time(lambda: KF.ring_attention(q, ring, first, wide, rb, yb, H, G, D, D, R, 0, 0, D ** -0.5, **extra), flush=flush),
                batch * min(prompt + 1, R) * C * 2)
            add("decode: Nefelorn grouped ring attention (same kernel without them)",
                _time(lambda: KF.ring_attention(q, ring, first, narrow, rb, yb, H, G, D, D, R, 0, 0, D ** -0.5), flush=flush),
                batch * min(prompt + 1, R) * C * 2)
        # recurrences: fixed decay per head (retention / lightning), decay logits per key channel (gated linear attention)
        k2, v2 = torch.randn(T, H * D, device=dev).to(bf), torch.randn(T, H * D, device=dev).to(bf)
        St = torch.zeros(batch, H, D, D, device=dev)
        decay = torch.full((H,), 0.97, device=dev)
        state_bytes = batch * H * D * D * 4 * (2 if phase == "decode" else 1)
        fma = T * H * D * D * 2.0                                    # state update + read-out, fused multiply-adds
        add(f"{phase}: decay scan, one decay per head (state {D} x {D})",
            _time(lambda: LF.decay_scan(q, k2, v2, St, rb, decay=decay, k_scale=D ** -0.5), flush=flush), T * H * D * (6 + 4) + state_bytes)
        rows[-1]["fp32_fma"] = fma
        add(f"{phase}: decay scan with SiLU on q, k, v", _time(lambda: LF.decay_scan(q, k2, v2, St, rb, decay=decay, act=True), flush=flush),
            T * H * D * (6 + 4) + state_bytes)
        Dg = D // 2
        qg, kg = torch.randn(T, H * Dg, device=dev).to(bf), torch.randn(T, H * Dg, device=dev).to(bf)
        z, zb = torch.randn(T, H * Dg, device=dev), torch.randn(H * Dg, device=dev) + 2.0
        Sg = torch.zeros(batch, H, Dg, D, device=dev)
        add(f"{phase}: decay scan, decay logits per key channel (state {Dg} x {D})",
            _time(lambda: LF.decay_scan(qg, kg, v2, Sg, rb, z=z, zb=zb, tau=8.0, q_scale=Dg ** -0.5), flush=flush),
            T * H * (Dg * 8 + D * 6) + state_bytes // 2)
        KH = H // 2
        Cq = 2 * KH * D + H * D
        conv = torch.randn(T, Cq, device=dev).to(bf)
        a, b = torch.randn(T, H, device=dev).to(bf), torch.randn(T, H, device=dev).to(bf)
        A_log, dtb = torch.zeros(H, dtype=bf, device=dev), torch.zeros(H, dtype=bf, device=dev)
        add(f"{phase}: Bumodra delta scan (per-head decay, state {D} x {D})",
            _time(lambda: SF.delta_scan(conv, KH * D, 2 * KH * D, a, b, A_log, dtb, St, rb, KH, False), flush=flush),
            T * (Cq * 2 + H * D * 4) + state_bytes)
        o = torch.randn(T, H * D, device=dev)
        nw, nall = torch.ones(D, dtype=bf, device=dev), torch.ones(H * D, dtype=bf, device=dev)
        add(f"{phase}: gated RMS norm per head", _time(lambda: LF.gated_norm(o, wide, nw, 1e-6, LF.GATE_SILU, yb, H, D, per_head=True), flush=flush), T * H * D * 8)
        add(f"{phase}: gated RMS norm over all heads", _time(lambda: LF.gated_norm(o, wide, nall, 1e-6, LF.GATE_SIGMOID, yb, H, D, per_head=False), flush=flush),
            T * H * D * 8)
        add(f"{phase}: Bumodra gated RMS norm per head", _time(lambda: SF.gated_rmsnorm(o, wide, nw, 1e-6, 0, yb, H, D), flush=flush), T * H * D * 8)
        hb = torch.randn(T, n, device=dev).to(bf)
        wr, rbias = torch.randn(E, n, device=dev).to(bf), torch.randn(E, device=dev)
        add(f"{phase}: router (bias, softmax over the top-{top} of {E})",
            _time(lambda: KF.moe_route(hb, wr, top, 1.0, bias=rbias, mode=KF.ROUTE_SOFTMAX), flush=flush), T * n * 2 + E * n * 2)
        add(f"{phase}: Nefelorn router (sigmoid)", _time(lambda: KF.moe_route(hb, wr, top, 1.0), flush=flush), T * n * 2 + E * n * 2)
    return {"peaks": src, "hbm_bytes_per_s": hbm, "bf16_flops": flops, "rows": rows}

# ======================================================================================================================
# Zubarax beside Salizen
# ======================================================================================================================
def zubarax_config(s):
    """The sizes of :data:`NEFELORN_SIZES`: the softmax side has Nefelorn's heads, the recurrence as many heads with half-size
    keys (Salizen's gated linear attention), the experts Nefelorn's sizes plus a shared expert of one expert's size; the last
    two entries run the first two blocks again."""
    D, H = s["dim"], s["heads"]
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"], "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"]},
           "shared": {"ff": s["expert_ff"], "limit": 7.0}}
    left = {"heads": H, "kv_heads": s["kv_heads"], "dim": D, "vdim": D, "conv": 4, "scale": D ** -0.5, "rot": {"dims": D // 2, "base": 1000000.0}}
    right = {"heads": H, "dim": D // 2, "vdim": D}
    entry = {"type": "parallel", "mlp": moe, "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.7}}
    layers = [json.loads(json.dumps(entry)) for _ in range(s["blocks"])]
    for i in range(s["blocks"] // 2, s["blocks"]):
        layers[i]["weights_of"] = i - s["blocks"] // 2
    return dict(vocab=s["vocab"], width=s["width"], norm={"eps": 1e-6}, postln_alpha=2.0, embedding={"scale": s["width"] ** 0.5}, layers=layers)


def salizen_full_window_config(s, prompt):
    """Salizen with every block a parallel one (window attention beside gated linear attention) with experts, its window as long
    as the prompt and the decoded tokens, one stream: the same work per block as Zubarax's."""
    cfg = salizen_config(dict(s, reach=prompt + 64))
    first = cfg["layers"][0]
    first["mlp"] = json.loads(json.dumps(cfg["layers"][1]["mlp"]))
    cfg["layers"] = [json.loads(json.dumps(first)) for _ in range(s["blocks"])]
    cfg["streams"] = 1
    return cfg


@torch.no_grad()
def throughput_zubarax(s, batch, prompt, new_tokens, steps, warmup):
    from libai_b200.config import DictConfig
    from libai_b200.layers._param import param_defaults
    from libai_b200.models import SalizenForCausalLM, ZubaraxForCausalLM

    ids = torch.randint(1, s["vocab"], (batch, prompt), generator=torch.Generator().manual_seed(0))
    out = {}
    for name, cls, cfg in (("zubarax", ZubaraxForCausalLM, zubarax_config(s)), ("salizen", SalizenForCausalLM, salizen_full_window_config(s, prompt))):
        with param_defaults(dtype=torch.bfloat16, device="cuda", seed=1):
            model = cls(DictConfig(cfg)).eval().cuda()
        _stateful_throughput(model, name, ids, batch, new_tokens, steps, warmup, out)
        del model
        torch.cuda.empty_cache()
    return out


@torch.no_grad()
def kernel_table_zubarax(s, batch, prompt):
    """Device time of every kernel of a Zubarax block at these sizes (prefill rows = batch·prompt; decode rows = batch) beside the
    like kernel of Salizen (or Nefelorn), with the bytes / FLOPs the operation needs and the fraction of the measured roofline."""
    from libai_b200.inference.ragged import RaggedBatch
    from libai_b200.inference.state_cache import SequenceStateCache
    from libai_b200.layers import DynamicTanh
    from libai_b200.layers._param import param_defaults
    from libai_b200.ops import kv_functional as KF
    from libai_b200.ops import lin_functional as LF
    from libai_b200.ops import paged_functional as PF

    hbm, flops, src = _peaks()
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    n, H, G, D = s["width"], s["heads"], s["kv_heads"], s["dim"]
    E, top = s["experts"], s["top"]
    C = G * 2 * D
    rows = []

    def add(name, ms, bytes_=0.0, fl=0.0):
        ideal = max(bytes_ / hbm, fl / flops) * 1e3
        rows.append(dict(kernel=name, ms=round(ms, 4), ideal_ms=round(ideal, 5), roofline_fraction=round(ideal / ms, 4),
                         bound="memory" if bytes_ / hbm >= fl / flops else "tensor"))

    with param_defaults(dtype=bf, device=dev, seed=2):
        na, nb = DynamicTanh(n), DynamicTanh(n)
    cache = SequenceStateCache(dev, bf, max_slots=batch, page_size=64)
    handle = cache.register("paged", channels=C, taps=4, conv_channels=H * D + C)
    slots = cache.allocate(batch)
    cache.prepare(slots, [prompt + 1] * batch)
    bufs = cache.buffers(handle)
    bufs["pool"].copy_(torch.randn(bufs["pool"].shape, device=dev).to(bf))
    talk = (torch.eye(H) + 0.1 * torch.randn(H, H)).to(dev)
    sink = torch.zeros(H, device=dev)
    for phase, lens, past in (("prefill", [prompt] * batch, [0] * batch), ("decode", [1] * batch, [prompt] * batch)):
        rb = RaggedBatch(lens, slots, past, dev)
        T = rb.tokens
        x1, y32 = torch.randn(T, n, device=dev), torch.randn(T, n, device=dev)
        h = torch.empty(T, n, dtype=bf, device=dev)
        w = torch.zeros(n, dtype=bf, device=dev)
        add(f"{phase}: post-norm residual (alpha x + y, RMS norm, fp32 residual + bf16 copy)",
            _time(lambda: PF.postnorm_residual(x1, w, 1e-6, alpha=2.0, y=y32, h=h), flush=flush), T * n * 14)
        add(f"{phase}: Nefelorn closing norm + residual + opening norm",
            _time(lambda: KF.dyt_residual(x1, y32, post=na.triple(), nxt=nb.triple(), h=h), flush=flush), T * n * 14)
        proj = torch.randn(T, H * D + C, device=dev).to(bf)
        pq, pk, pv = proj[:, :H * D], proj[:, H * D:H * D + G * D], proj[:, H * D + G * D:]
        cw = [torch.randn(c, 4, device=dev).to(bf) for c in (H * D, G * D, G * D)]
        nw = torch.ones(D, dtype=bf, device=dev)
        freq = KF.rotary_frequencies(D // 2, 1e6)[0].to(dev)
        add(f"{phase}: convolution + head norms + rotation + page write of q, k, v",
            _time(lambda: PF.conv_qkv_prepare(pq, pk, pv, cw[0], cw[1], cw[2], bufs["tail"], nw, nw, freq, 1e-6, rb, bufs["pool"], bufs["table"], H, G, D, D),
                  flush=flush), T * (H * D + C) * 4)
        q = torch.randn(T, H * D, device=dev).to(bf)
        kv = torch.randn(T, C, device=dev).to(bf)
        R = prompt + 64
        ring = torch.randn(batch, R, C, device=dev).to(bf)
        first = torch.zeros(batch, 0, C, dtype=bf, device=dev)

        def salizen_prepare():
            KF.qk_prepare(q, kv[:, :G * D], None, None, freq, 1.0, rb, H, G, D, 1e-6, False, False)
            KF.kv_write(ring, first, kv[:, :G * D], kv[:, G * D:], rb)

        add(f"{phase}: Salizen rotation of q, k + ring write (two kernels, no convolution, no norms)", _time(salizen_prepare, flush=flush), T * (H * D * 4 + C * 6))
        from libai_b200.ops import seq_functional as SF

        cw_all, tail3 = torch.cat(cw, 0), torch.zeros(batch, 3, H * D + C, dtype=bf, device=dev)
        conv_out = torch.empty_like(proj)
        add(f"{phase}: Bumodra short convolution of the same channels (two kernels; convolution + SiLU only)",
            _time(lambda: SF.short_conv(proj, cw_all, tail3, rb, conv_out), flush=flush), T * (H * D + C) * 4)
        yb = torch.empty(T, H * D, dtype=bf, device=dev)
        if phase == "prefill":
            pairs = prompt * (prompt + 1) // 2 * batch
            fl = pairs * H * D * 4.0
            add("prefill: attention over the pages with mixed heads and sink (mma.m16n8k16, mix on the fp32 pipe)",
                _time(lambda: PF.talk_attention(q, bufs["pool"], bufs["table"], rb, yb, H, G, D, D, D ** -0.5, talk=talk, sink=sink), flush=flush),
                T * H * D * 4 + T * C * 2, fl)
            rows[-1]["fp32_mix_fma"] = pairs * H * H * 1.0
            ext = rb.kv_ext([(R, 0, 0)])
            add("prefill: Salizen window attention with sink, window = prompt (mma.m16n8k16)",
                _time(lambda: KF.masked_attention(q, kv[:, :G * D], kv[:, G * D:], ext, None, rb, yb, H, G, D, D, R, 0, 0, D ** -0.5, sink=True), flush=flush),
                T * H * D * 4 + T * C * 2, fl)
        else:
            add("decode: attention over the pages with mixed heads and sink (keys in parts + merge)",
                _time(lambda: PF.talk_attention(q, bufs["pool"], bufs["table"], rb, yb, H, G, D, D, D ** -0.5, talk=talk, sink=sink), flush=flush),
                batch * (prompt + 1) * C * 2)
            add("decode: Salizen grouped ring attention with sink, window = prompt",
                _time(lambda: KF.ring_attention(q, ring, first, None, rb, yb, H, G, D, D, R, 0, 0, D ** -0.5, sink=True), flush=flush),
                batch * (prompt + 1) * C * 2)
        Dg = D // 2
        qg, kg, v2 = (torch.randn(T, H * c, device=dev).to(bf) for c in (Dg, Dg, D))
        z, zb, low = torch.randn(T, H * Dg, device=dev), torch.randn(H * Dg, device=dev) + 2.0, torch.rand(H * Dg, device=dev) * 0.9
        Sg = torch.zeros(batch, H, Dg, D, device=dev)
        state_bytes = batch * H * Dg * D * 4 * (2 if phase == "decode" else 1)
        add(f"{phase}: decay scan, bounded forget gate that also writes (state {Dg} x {D})",
            _time(lambda: LF.decay_scan(qg, None, v2, Sg, rb, z=z, zb=zb, lower=low, act=LF.ACT_Q), flush=flush), T * H * (Dg * 6 + D * 6) + state_bytes)
        add(f"{phase}: Salizen decay scan, decay logits per key channel (state {Dg} x {D})",
            _time(lambda: LF.decay_scan(qg, kg, v2, Sg, rb, z=z, zb=zb, tau=8.0, q_scale=Dg ** -0.5), flush=flush), T * H * (Dg * 8 + D * 6) + state_bytes)
        o = torch.randn(T, H * D, device=dev)
        gate = torch.randn(T, H * D, device=dev).to(bf)
        nw2 = torch.ones(D, dtype=bf, device=dev)
        add(f"{phase}: RMS norm per head of the read-out (no gate)", _time(lambda: LF.gated_norm(o, None, nw2, 1e-6, LF.GATE_NONE, yb, H, D, per_head=True), flush=flush), T * H * D * 6)
        add(f"{phase}: Salizen gated RMS norm per head", _time(lambda: LF.gated_norm(o, gate, nw2, 1e-6, LF.GATE_SILU, yb, H, D, per_head=True), flush=flush), T * H * D * 8)
        hb = torch.randn(T, n, device=dev).to(bf)
        wr = torch.randn(E, n, device=dev).to(bf)
        add(f"{phase}: router (sigmoid scores as they are, top-{top} of {E})", _time(lambda: KF.moe_route(hb, wr, top, 1.0, mode=KF.ROUTE_SIGMOID_RAW), flush=flush), T * n * 2 + E * n * 2)
        add(f"{phase}: Nefelorn router (sigmoid, normalised)", _time(lambda: KF.moe_route(hb, wr, top, 1.0), flush=flush), T * n * 2 + E * n * 2)
        if phase == "prefill":
            ff = s["expert_ff"]
            gu = torch.randn(T * top, 2 * ff, device=dev).to(bf)
            a = torch.empty(T * top, ff, dtype=bf, device=dev)
            add("prefill: clamped gated activation of the experts", _time(lambda: KF.act_rows(gu, a, KF.ACTS["swish_clamp"], gated=True, limit=7.0), flush=flush), T * top * ff * 6)
            add("prefill: Nefelorn gated SiLU activation", _time(lambda: KF.act_rows(gu, a, KF.ACTS["silu"], gated=True), flush=flush), T * top * ff * 6)
            idx, wts = KF.moe_route(hb, wr, top, 1.0, mode=KF.ROUTE_SIGMOID_RAW)
            P = T * top
            rows_p = (P + E * 127 + 127) // 128 * 128
            xs = torch.empty(rows_p, n, dtype=bf, device=dev)
            meta = torch.empty(2 * E + 1 + rows_p // 128, dtype=torch.int32, device=dev)
            pos = torch.empty(T, top, dtype=torch.int32, device=dev)
            counts = torch.bincount(idx.reshape(-1).long(), minlength=E).int()
            from libai_b200.ops import load_kv_ext

            def sort(wv):
                load_kv_ext().moe_sort(hb, idx, counts, meta[: E + 1], meta[E + 1: 2 * E + 1], pos, xs, 128, meta[2 * E + 1:], wv)

            add("prefill: rows sorted by expert, scaled by their routing weight", _time(lambda: sort(wts), flush=flush), P * n * 4)
            add("prefill: Nefelorn rows sorted by expert (copied)", _time(lambda: sort(None), flush=flush), P * n * 4)
    return {"peaks": src, "hbm_bytes_per_s": hbm, "bf16_flops": flops, "rows": rows}


def main(args):
    assert torch.cuda.is_available(), "the serving bench needs a GPU"
    from libai_b200 import ops

    ops.reset_launch_count()
    if getattr(args, "serving_model", "bumodra") == "zubarax":
        result = {"metric": "prefill / decode tokens per second, Zubarax beside Salizen (window = prompt, one stream) at equal width, depth, heads and expert sizes",
                  "dtype": "bf16", "data": "synthetic tokens, random-init weights", "n_gpus": 1, "sizes": {}}
        for name in (args.serving_sizes.split(",") if args.serving_sizes else list(NEFELORN_SIZES)):
            s = NEFELORN_SIZES[name]
            r = throughput_zubarax(s, args.serving_batch, args.serving_prompt, new_tokens=max(args.steps, 8),
                                   steps=max(args.steps // 2, 3), warmup=max(args.warmup, 3))
            if args.serving_kernels:
                r["kernels"] = kernel_table_zubarax(s, args.serving_batch, args.serving_prompt)
            result["sizes"][name] = {"config": dict(s), "batch": args.serving_batch, "prompt": args.serving_prompt, **r}
            torch.cuda.empty_cache()
        result["gpu_launches"] = ops.launch_count()
        print(json.dumps(result))
        return
    if getattr(args, "serving_model", "bumodra") == "salizen":
        result = {"metric": "prefill / decode tokens per second, Salizen beside Nefelorn at equal width, depth, heads and active feed-forward size",
                  "dtype": "bf16", "data": "synthetic tokens, random-init weights", "n_gpus": 1, "sizes": {}}
        for name in (args.serving_sizes.split(",") if args.serving_sizes else list(NEFELORN_SIZES)):
            s = NEFELORN_SIZES[name]
            r = throughput_salizen(s, args.serving_batch, args.serving_prompt, new_tokens=max(args.steps, 8),
                                   steps=max(args.steps // 2, 3), warmup=max(args.warmup, 3))
            if args.serving_kernels:
                r["kernels"] = kernel_table_salizen(s, args.serving_batch, args.serving_prompt)
            result["sizes"][name] = {"config": dict(s), "batch": args.serving_batch, "prompt": args.serving_prompt, **r}
            torch.cuda.empty_cache()
        result["gpu_launches"] = ops.launch_count()
        print(json.dumps(result))
        return
    if getattr(args, "serving_model", "bumodra") == "nefelorn":
        result = {"metric": "prefill / decode tokens per second, Nefelorn beside Llama at equal width, depth and active feed-forward size",
                  "dtype": "bf16", "data": "synthetic tokens, random-init weights", "n_gpus": 1, "sizes": {}}
        for name in (args.serving_sizes.split(",") if args.serving_sizes else list(NEFELORN_SIZES)):
            s = NEFELORN_SIZES[name]
            r = throughput_nefelorn(s, args.serving_batch, args.serving_prompt, new_tokens=max(args.steps, 8),
                                    steps=max(args.steps // 2, 3), warmup=max(args.warmup, 3))
            if args.serving_kernels:
                r["kernels"] = kernel_table_nefelorn(s, args.serving_batch, args.serving_prompt)
            result["sizes"][name] = {"config": dict(s), "batch": args.serving_batch, "prompt": args.serving_prompt, **r}
            torch.cuda.empty_cache()
        result["gpu_launches"] = ops.launch_count()
        print(json.dumps(result))
        return
    result = {"metric": "prefill / decode tokens per second, Bumodra beside Llama at equal width, depth and parameter count",
              "dtype": "bf16", "data": "synthetic tokens, random-init weights", "n_gpus": 1, "sizes": {}}
    for name in (args.serving_sizes.split(",") if args.serving_sizes else list(SIZES)):
        s = SIZES[name]
        r = throughput(s, args.serving_batch, args.serving_prompt, new_tokens=max(args.steps, 8), steps=max(args.steps // 2, 3),
                       warmup=max(args.warmup, 3))
        if args.serving_kernels:
            r["kernels"] = kernel_table(s, args.serving_batch, args.serving_prompt)
        result["sizes"][name] = {"config": {k: v for k, v in s.items()}, "batch": args.serving_batch, "prompt": args.serving_prompt, **r}
        torch.cuda.empty_cache()
    result["gpu_launches"] = ops.launch_count()
    print(json.dumps(result))
