"""Salizen against a plain float64 oracle (``salizen_oracle.py``): every mechanism alone, whole prompts, decoding through the
state cache, prompt portions, ragged batches, slot reuse, window edges and far keys made decisive, long decoding, odd sizes,
generation.

The CPU parametrisation exercises the framework's PyTorch operators; the ``cuda`` one (marked ``gpu``) the sm_100a kernels.
"""
import importlib.util
import json
import math
import os

import pytest
import torch

from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.scheduler import RequestScheduler
from libai_b200.inference.state_cache import SequenceStateCache
from libai_b200.layers import DecayLinearAttention, HyperConnection, MoEFeedForward, RingAttention
from libai_b200.layers._param import param_defaults
from libai_b200.models.utils.model_loader.auto import load_pretrained
from libai_b200.ops import kv_functional as KF
from libai_b200.ops import lin_functional as LF

from . import salizen_oracle as O

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda", id="cuda", marks=pytest.mark.gpu)]
REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
F64 = torch.float64


def rel_err(got, want):
    """Error of logits the way a user sees it: mean removed, RMS over the vocabulary, relative to the RMS of the target."""
    got, want = got.detach().cpu().double(), want.double()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    scale = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return float(d.pow(2).mean(-1).sqrt().max() / scale)


def save_model(tmp_path, cfg, weights, name="m"):
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


def make(tmp_path, cfg, device, dtype=torch.float32, seed=0, weights=None, rank=3):
    weights = weights if weights is not None else O.random_weights(cfg, seed, rank=rank)
    return load_pretrained(save_model(tmp_path, cfg, weights), dtype=dtype, device=device), weights


def run_schedule(model, prompts, cuts, **kw):
    """Feed ``prompts`` together: step s brings ``cuts[i][s]`` tokens of prompt i (requests that have nothing left drop out).
    Returns per prompt the logits of all its positions."""
    sched = RequestScheduler(model, **kw)
    at = [0] * len(prompts)
    got = [[] for _ in prompts]
    for s in range(max(len(c) for c in cuts)):
        entries, who = [], []
        for i, p in enumerate(prompts):
            if s < len(cuts[i]):
                n = cuts[i][s]
                entries.append((("r", i), p[at[i]:at[i] + n], list(range(n))))
                who.append((i, n))
                at[i] += n
        logits = sched.step(entries)
        o = 0
        for i, n in who:
            got[i].append(logits[o:o + n].clone())
            o += n
        sched.finish([("r", i) for i, p in enumerate(prompts) if at[i] == len(p)])
    assert sched.cache.live() == 0
    return [torch.cat(g) for g in got]


def tokens(n, vocab=50, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def mixed_cfg(**kw):
    """Every branch once: a parallel block with a dense feed-forward, a retention block with experts, a lightning block without
    a feed-forward, a lightning block with experts, a second parallel block of other sizes."""
    layers = [O.parallel_cfg(mlp=O.dense_cfg(20)),
              O.retention_cfg(mlp=O.moe_cfg()),
              O.lightning_cfg(mlp=None),
              O.lightning_cfg(heads=3, dim=4, vdim=6, mlp=O.moe_cfg(ff=4, experts=3, top=1)),
              O.parallel_cfg(left=O.left_cfg(heads=3, kv_heads=3, dim=4, window=3, rot=O.rot_cfg(4, 50.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 16}),
                                             scale=0.9, softcap=2.0),
                             right=O.right_cfg(heads=1, dim=10, vdim=6, tau=3.0), left_scale=1.2, right_scale=0.4, mlp=O.dense_cfg(12))]
    return O.model_cfg(layers, **kw)


def _f64(module_param):
    return module_param.detach().cpu().double()


# ------------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("device", DEVICES)
def test_bigram_embedding_carries_the_previous_token(device):
    g = torch.Generator().manual_seed(0)
    vocab, n, buckets, mp, mc, scale, S = 23, 12, 13, 7, 5, 2.5, 3
    W = {"embed": torch.randn(vocab, n, generator=g), "bigram": torch.randn(buckets + 1, n, generator=g)}
    emb = {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}
    seqs = [tokens(9, vocab, 1), tokens(5, vocab, 2), tokens(1, vocab, 3)]
    want = [O.embed_tokens(s, O.as_f64(W), emb) for s in seqs]
    last = torch.full((6,), 17, dtype=torch.int32, device=device)           # stale tokens of earlier owners of the slots
    slots = [4, 1, 3]
    table, bigram = W["embed"].to(device), W["bigram"].to(device)
    # step 1: the first 4 / 2 / 1 tokens (first rows take the table's last row whatever the slot holds); step 2: the rest
    for lens, past in (([4, 2, 1], [0, 0, 0]), ([5, 3], [4, 2])):
        rb = RaggedBatch(lens, slots[:len(lens)], past, device)
        ids = torch.tensor([t for s, n_, p in zip(seqs, lens, past) for t in s[p:p + n_]], device=device)
        x = torch.empty(S, sum(lens), n, device=device)
        LF.embed_bigram(table, bigram, ids, last, rb, scale, mp, mc, buckets, x)
        for b, (n_, p) in enumerate(zip(lens, past)):
            for s in range(S):
                assert torch.allclose(x[s, rb.offsets[b]:rb.offsets[b] + n_].cpu().double(), want[b][p:p + n_], atol=1e-5)
    assert last.tolist()[4] == seqs[0][-1] and last.tolist()[1] == seqs[1][-1] and last.tolist()[3] == seqs[2][-1]
    # the row really depends on the previous token and on both multipliers
    other = O.embed_tokens(seqs[0], O.as_f64(W), {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mc, "mul_cur": mp}})
    assert not torch.allclose(other[1:], want[0][1:], atol=1e-3)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("S,n", [(1, 8), (2, 20), (3, 7), (4, 64)])
def test_hyper_connection_step(device, S, n):
    g = torch.Generator().manual_seed(S)
    T, eps = 5, 1e-3
    streams = [torch.randn(T, n, generator=g, dtype=F64) for _ in range(S)]
    y = torch.randn(T, n, generator=g, dtype=F64)
    with param_defaults(dtype=torch.float32, device=device):
        hc, hc_next = HyperConnection(S), HyperConnection(S)
    with torch.no_grad():
        for mod in (hc, hc_next):
            for prm in (mod.inw, mod.outw, mod.mix):
                prm.copy_(torch.randn(prm.shape, generator=g))
    w_next = torch.randn(n, generator=g)
    W = {"l0.hc1.in": _f64(hc.inw), "l0.hc1.out": _f64(hc.outw), "l0.hc1.mix": _f64(hc.mix),
         "l0.hc2.in": _f64(hc_next.inw), "l0.hc2.out": _f64(hc_next.outw), "l0.hc2.mix": _f64(hc_next.mix)}
    seen = {}
    new = O.hyper_sublayer(streams, W, "l0.", 1, lambda hh: y, torch.ones(n, dtype=F64), eps)
    O.hyper_sublayer(new, W, "l0.", 2, lambda hh: seen.setdefault("h", hh) * 0, w_next.double(), eps)
    x = torch.stack(streams).float().to(device)
    h = torch.empty(T, n, device=device)
    _, outw, mix = hc.coefficients()
    LF.hc_step(x, y.float().to(device), post=(mix, outw), nxt=(hc_next.coefficients()[0], w_next.to(device)), h=h, eps=eps)
    assert torch.allclose(x.cpu().double(), torch.stack(new), atol=1e-5)
    assert torch.allclose(h.cpu().double(), seen["h"], atol=1e-4)
    if S > 1:                                                       # mix is indexed [from, to]: its transpose is another model
        assert not torch.allclose(torch.einsum("ts,srn->trn", _f64(hc.mix), torch.stack(streams)), torch.stack(new) - _f64(hc.outw)[:, None, None] * y, atol=1e-3)
    # the sublayer output gathered from sorted expert rows
    top = 2
    ys = torch.randn(3 * T, n, generator=g)
    pos = torch.randint(0, 3 * T, (T, top), generator=g).int()
    cw = torch.rand(T, top, generator=g)
    x2 = torch.stack(streams).float().to(device)
    LF.hc_step(x2, ys.to(device), post=(mix, outw), pos=pos.to(device), cw=cw.to(device), eps=eps)
    yg = (ys.double()[pos.long()] * cw.double()[:, :, None]).sum(1)
    want = O.hyper_sublayer(streams, W, "l0.", 1, lambda hh: yg, torch.ones(n, dtype=F64), eps)
    assert torch.allclose(x2.cpu().double(), torch.stack(want), atol=1e-5)


@pytest.mark.parametrize("rot", [O.rot_cfg(8, 100.0), O.rot_cfg(16, 250.0, {"factor": 4.0, "original": 64, "low": 1.0, "high": 4.0}),
                                 O.rot_cfg(32, 1e4, {"factor": 16.0, "original": 256, "low": 2.0, "high": 8.0}),
                                 O.rot_cfg(8, 10.0, {"factor": 2.0, "original": 1e6, "low": 1.0, "high": 2.0}),
                                 O.rot_cfg(8, 10.0, {"factor": 2.0, "original": 1, "low": 1.0, "high": 2.0})])
def test_rotary_frequencies_blended_by_wavelength(rot):
    freq, ms = KF.rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    want = torch.tensor(O.rotary_frequencies(rot), dtype=F64)
    assert torch.allclose(freq.double(), want, rtol=1e-6, atol=0) and ms == 1.0
    plain = torch.tensor(O.rotary_frequencies({"dims": rot["dims"], "base": rot["base"]}), dtype=F64)
    sc = rot.get("scaling")
    if sc and sc["original"] == 1:                                  # every wavelength is longer than original / low: all divided
        assert torch.allclose(want, plain / sc["factor"])
    elif sc and sc["original"] == 1e6:                              # every wavelength is shorter than original / high: unchanged
        assert torch.allclose(want, plain)
    elif sc:                                                        # all three branches occur
        ratio = plain / want
        assert float(ratio.min()) == 1.0 and abs(float(ratio.max()) - sc["factor"]) < 1e-9
        assert bool(((ratio > 1.0 + 1e-9) & (ratio < sc["factor"] - 1e-9)).any())


def _run_mixer(mod, h, device, lens, past_chunks=None):
    """A mixer module alone on one sequence ``h`` ``[n, width]`` fed in the portions ``lens``; returns ``[n, width]``."""
    cache = SequenceStateCache(device, torch.float32)
    kind, shape = mod.state_spec()
    handle = cache.register(kind, **shape)
    slot = cache.allocate(3)[1:2]                                   # not slot 0
    out, at = [], 0
    for n in lens:
        rb = RaggedBatch([n], slot, [at], device)
        out.append(mod(h[at:at + n].float().to(device), rb, cache.buffers(handle)).cpu().double())
        cache.advance(slot, [n])
        at += n
    return torch.cat(out)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("lens", [[17], [1] * 17, [5, 1, 9, 2]])
def test_sink_window_attention_alone(device, lens):
    width, m = 16, O.left_cfg(heads=4, kv_heads=2, dim=6, window=5, rot=O.rot_cfg(4, 30.0, {"factor": 3.0, "original": 20, "low": 1.0, "high": 3.0}),
                              scale=0.8, softcap=1.5)
    W = O.random_weights(O.model_cfg([O.parallel_cfg(left=m)], width=width), seed=3)
    with param_defaults(dtype=torch.float32, device=device):
        mod = RingAttention(width, 4, 2, 6, 6, window=5, scale=0.8, rot_dims=4, rot_base=30.0, rot_scaling=m["rot"]["scaling"],
                            out_gate="channel", value_from_key=True, softcap=1.5, sink=True)
    assert mod.v is None
    with torch.no_grad():
        for name in ("q", "k", "g", "o"):
            getattr(mod, name).copy_(W[f"l0.mix.left.{name}"])
    h = torch.randn(17, width, generator=torch.Generator().manual_seed(1), dtype=F64)
    want = O.sink_window_attention(h, O.as_f64(W), "l0.mix.left.", m)
    got = _run_mixer(mod, h, device, lens)
    assert torch.allclose(got, want, atol=2e-5)
    # each ingredient is visible: no sink, no cap, a window one longer
    assert not torch.allclose(O.sink_window_attention(h, O.as_f64(W), "l0.mix.left.", m, sink=0.0), want, atol=1e-2)
    assert not torch.allclose(O.sink_window_attention(h, O.as_f64(W), "l0.mix.left.", {**m, "softcap": 1e6}), want, atol=1e-2)
    assert not torch.allclose(O.sink_window_attention(h, O.as_f64(W), "l0.mix.left.", m, window_shift=1), want, atol=1e-3)


def _linear_attention(kind, device, width, m, W, rank=3):
    with param_defaults(dtype=torch.float32, device=device):
        if kind == "gla":
            mod = DecayLinearAttention(width, m["heads"], m["dim"], m["vdim"], decay="channel", tau=m["tau"], decay_rank=rank,
                                       q_scale=m["dim"] ** -0.5, norm="head", gate="silu", eps=1e-5)
        elif kind == "retention":
            mod = DecayLinearAttention(width, m["heads"], m["dim"], m["vdim"], decay=m["decay"], k_scale=m["dim"] ** -0.5,
                                       rot_dims=m["rot"]["dims"], rot_base=m["rot"]["base"], norm="head", norm_weight=False, gate="silu", eps=1e-5)
        else:
            mod = DecayLinearAttention(width, m["heads"], m["dim"], m["vdim"], decay=m["decay"], qkv_act="silu", norm="all",
                                       gate="sigmoid", eps=1e-5)
    p = "l0.mix.right." if kind == "gla" else "l0.mix."
    with torch.no_grad():
        for name, prm in mod.named_parameters():
            prm.copy_(W[p + name.replace("a2_b", "a2.b")])
    return mod


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("lens", [[19], [1] * 19, [2, 16, 1]])
@pytest.mark.parametrize("kind", ["gla", "retention", "lightning"])
def test_linear_attention_mixers_alone(device, kind, lens):
    width, eps = 16, 1e-5
    if kind == "gla":
        m = O.right_cfg(heads=3, dim=5, vdim=7, tau=4.0)
        cfg = O.model_cfg([O.parallel_cfg(right=m)], width=width)
        oracle = lambda h, W: O.gated_linear_attention(h, W, "l0.mix.right.", m, eps)
    elif kind == "retention":
        m = O.retention_cfg(heads=2, dim=6, vdim=9, rot=O.rot_cfg(4, 20.0))["mixer"]
        cfg = O.model_cfg([O.retention_cfg(heads=2, dim=6, vdim=9, rot=O.rot_cfg(4, 20.0))], width=width)
        oracle = lambda h, W: O.retention_mixer(h, W, "l0.mix.", m, eps)
    else:
        m = O.lightning_cfg(heads=3, dim=4, vdim=5)["mixer"]
        cfg = O.model_cfg([O.lightning_cfg(heads=3, dim=4, vdim=5)], width=width)
        oracle = lambda h, W: O.lightning_mixer(h, W, "l0.mix.", m, eps)
    W = O.random_weights(cfg, seed=5)
    mod = _linear_attention(kind, device, width, m, W)
    h = torch.randn(19, width, generator=torch.Generator().manual_seed(2), dtype=F64)
    want = oracle(h, O.as_f64(W))
    got = _run_mixer(mod, h, device, lens)
    assert torch.allclose(got, want, atol=5e-5), float((got - want).abs().max())


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("D,V,H", [(8, 8, 2), (24, 40, 1), (64, 32, 2), (100, 12, 1), (160, 72, 1)])
def test_decay_scan_sizes(device, D, V, H):
    """The recurrence alone for key sizes on both sides of every rows-per-lane choice of the kernel, with a fixed decay and with
    decay logits, in two portions, next to a direct evaluation of ``o_t = Σ_j (Π_{j<i≤t} a_i) (k_j·q_t) v_j``."""
    g = torch.Generator().manual_seed(D)
    n = 21
    q, k, v = (torch.randn(n, H * s, generator=g) for s in (D, D, V))
    z, zb = torch.randn(n, H * D, generator=g) * 2.0, torch.randn(H * D, generator=g) + 2.0
    decay = torch.linspace(0.8, 0.99, H)
    for mode in ("head", "channel"):
        if mode == "head":
            a = decay.double()[None, :, None].expand(n, H, D)
        else:
            a = torch.sigmoid(z.double() + zb.double()).pow(1.0 / 6.0).view(n, H, D)
        qd, kd, vd = q.double().view(n, H, D) * 0.5, k.double().view(n, H, D) * 2.0, v.double().view(n, H, V)
        want = torch.zeros(n, H, V, dtype=F64)
        for t in range(n):
            for j in range(t + 1):
                w = a[j + 1:t + 1].prod(0)                                         # [H, D]
                want[t] += ((qd[t] * kd[j] * w).sum(-1))[:, None] * vd[j]
        S = torch.full((3, H, D, V), 7.0, device=device)                          # a reused slot is not cleared
        outs = []
        for lo, hi in ((0, 13), (13, n)):
            rb = RaggedBatch([hi - lo], [2], [lo], device)
            kw = dict(decay=decay.to(device)) if mode == "head" else dict(z=z[lo:hi].to(device), zb=zb.to(device), tau=6.0)
            outs.append(LF.decay_scan(q[lo:hi].to(device), k[lo:hi].to(device), v[lo:hi].to(device), S, rb, q_scale=0.5, k_scale=2.0, **kw))
        got = torch.cat(outs).cpu().double().view(n, H, V)
        assert torch.allclose(got, want, atol=1e-3 * float(want.abs().max())), mode


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("experts,top", [(5, 2), (4, 1), (3, 3), (40, 6)])
def test_router_softmax_over_the_chosen_logits(device, experts, top):
    g = torch.Generator().manual_seed(experts)
    width, T = 12, 9
    W = {"l0.mlp.router": torch.randn(experts, width, generator=g), "l0.mlp.router.b": 4.0 * torch.randn(experts, generator=g)}
    h = torch.randn(T, width, generator=g)
    idx, wts = KF.moe_route(h.to(device), W["l0.mlp.router"].to(device), top, 1.0, bias=W["l0.mlp.router.b"].to(device), mode=KF.ROUTE_SOFTMAX)
    for t in range(T):
        order, w = O.router_choice(h[t].double(), O.as_f64(W), "l0.mlp.", {"experts": experts, "top": top})
        assert idx[t].tolist() == order
        assert torch.allclose(wts[t].cpu().double(), w, atol=1e-6)
        assert abs(float(wts[t].sum()) - 1.0) < 1e-5
    # the bias takes part in the choice, and the weights are no softmax over all experts
    push = torch.zeros(experts)
    push[experts - 1] = 100.0
    idx1, _ = KF.moe_route(h.to(device), W["l0.mlp.router"].to(device), top, 1.0, bias=push.to(device), mode=KF.ROUTE_SOFTMAX)
    assert all(row[0] == experts - 1 for row in idx1.tolist())


@pytest.mark.parametrize("device", DEVICES)
def test_feed_forwards(device):
    width, g = 16, torch.Generator().manual_seed(4)
    cfg = O.model_cfg([O.parallel_cfg(mlp=O.dense_cfg(24)), O.lightning_cfg(mlp=O.moe_cfg(ff=6, experts=5, top=2))], width=width)
    W = O.random_weights(cfg, seed=1)
    model_dir_weights = O.as_f64(W)
    h = torch.randn(7, width, generator=g)
    from libai_b200.models.salizen_model import GatedFF

    with param_defaults(dtype=torch.float32, device=device):
        ff = GatedFF(width, 24)
        moe = MoEFeedForward(width, 6, 5, 2, router="softmax", router_bias=True)
    with torch.no_grad():
        ff.gate_up.copy_(torch.cat([W["l0.mlp.gate"], W["l0.mlp.up"]]))
        ff.down.copy_(W["l0.mlp.down"])
        moe.router.copy_(W["l1.mlp.router"])
        moe.router_b.copy_(W["l1.mlp.router.b"])
        moe.gate_up.copy_(torch.stack([torch.cat([W[f"l1.mlp.e{e}.gate"], W[f"l1.mlp.e{e}.up"]]) for e in range(5)]))
        moe.down.copy_(torch.stack([W[f"l1.mlp.e{e}.down"] for e in range(5)]))
    want = O.feed_forward(h.double(), model_dir_weights, "l0.mlp.", cfg["layers"][0]["mlp"])
    assert torch.allclose(ff(h.to(device)).cpu().double(), want, atol=1e-5)
    erf_form = 0.5 * h * (1 + torch.erf(h / math.sqrt(2)))
    assert float((O.gelu_tanh(h.double()) - erf_form.double()).abs().max()) > 1e-4      # the tanh form, not erf
    want = O.feed_forward(h.double(), model_dir_weights, "l1.mlp.", cfg["layers"][1]["mlp"])
    pairs, _, _ = moe(h.to(device), graph_safe=True)
    assert torch.allclose(pairs.cpu().double(), want, atol=1e-5)
    many = torch.randn(40, width, generator=g)                      # enough rows for the sorted form
    ys, pos, cw = moe(many.to(device))
    assert pos is not None
    got = (ys.float()[pos.long()] * cw[:, :, None]).sum(1)
    assert torch.allclose(got.cpu().double(), O.feed_forward(many.double(), model_dir_weights, "l1.mlp.", cfg["layers"][1]["mlp"]), atol=1e-5)


# ------------------------------------------------------------------------------------------------- whole prompts, decoding
@pytest.mark.parametrize("device", DEVICES)
def test_whole_prompt_with_streams(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(19)
    streams = []
    want = O.forward(cfg, W, toks, streams)
    taps = []
    cache = model.state_cache()
    slots = cache.allocate(1)
    got = model.step(torch.tensor(toks, device=device), RaggedBatch([len(toks)], slots, [0], device),
                     tap=lambda i, x: taps.append(x.detach().cpu().double().clone()))
    cache.free(slots)
    assert len(taps) == len(streams) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(taps, streams)):
        assert torch.allclose(a, b, atol=2e-4), f"streams after block {i}"
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_prefill_against_token_by_token(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(26, seed=3)
    want = O.forward(cfg, W, toks)
    whole, = run_schedule(model, [toks], [[len(toks)]])
    single, = run_schedule(model, [toks], [[1] * len(toks)])
    mixed, = run_schedule(model, [toks], [[9] + [1] * 17])
    for got in (whole, single, mixed):
        assert rel_err(got, want) < 1e-4
    assert rel_err(single, whole.cpu()) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cuts", [[2] * 15, [3, 7, 2, 11, 7], [13, 2, 2, 13], [1, 29], [29, 1]])
def test_prompt_portions(device, tmp_path, cuts):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(30, seed=5)
    want = O.forward(cfg, W, toks)
    got, = run_schedule(model, [toks], [cuts])
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_ragged_batches_against_each_alone(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    prompts = [tokens(n, seed=n) for n in (1, 17, 4, 30, 9)]
    want = [O.forward(cfg, W, p) for p in prompts]
    cuts = [[1], [12] + [1] * 5, [2, 1, 1], [21] + [1] * 9, [9]]
    together = run_schedule(model, prompts, cuts)
    for i, p in enumerate(prompts):
        alone, = run_schedule(model, [p], [cuts[i]])
        assert rel_err(together[i], want[i]) < 1e-4
        assert rel_err(together[i], alone.cpu()) < 1e-5
    # unequal portions in one step: long and short prompt pieces beside single tokens
    cuts2 = [[1], [5, 12], [1, 3], [2, 20, 8], [4, 1, 4]]
    for got, w in zip(run_schedule(model, prompts, cuts2), want):
        assert rel_err(got, w) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_slots_are_reused_without_clearing(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    sched = RequestScheduler(model)
    a, b, c = tokens(23, seed=1), tokens(8, seed=2), tokens(15, seed=3)
    sched.step([("a", a, []), ("b", b, [])])
    slot_a = sched.slot_of["a"]
    sched.finish(["a"])
    got = sched.step([("c", c[:6], list(range(6)))])               # takes a's slot: its rings, states and last token are a's
    assert sched.slot_of["c"] == slot_a
    got = torch.cat([got] + [sched.step([("c", [t], [0]), ("b", [1], [])]) for t in c[6:]])
    assert rel_err(got, O.forward(cfg, W, c)) < 1e-4
    before = sched.cache.capacity
    many = [(("m", i), tokens(3 + i, seed=10 + i), [2 + i]) for i in range(before + 3)]      # more requests than slots: the cache grows
    logits = sched.step(many)
    assert sched.cache.capacity > before
    for row, (_, p, _) in enumerate(many):
        assert rel_err(logits[row:row + 1], O.forward(cfg, W, p)[-1:]) < 1e-4
    got = sched.step([("c", [7], [0])])                            # a request that lived through the growth goes on
    assert rel_err(got, O.forward(cfg, W, c + [7])[-1:]) < 1e-4


# --------------------------------------------------------------------------------------------------- window edges, far keys
def sharp_cfg():
    """A large score scale and a high cap make the softmax pick single keys, so a key that is wrongly seen or missed moves the
    logits; the linear-attention side is switched off by its factor."""
    left = O.left_cfg(heads=2, kv_heads=1, dim=8, window=7, rot=O.rot_cfg(4, 100.0), scale=3.0, softcap=30.0)
    return O.model_cfg([O.parallel_cfg(left=left, left_scale=1.0, right_scale=0.0, mlp=O.dense_cfg(16))])


@pytest.mark.parametrize("device", DEVICES)
def test_window_edge_shows_in_the_logits(device, tmp_path):
    cfg = sharp_cfg()
    model, W = make(tmp_path, cfg, device, seed=4)
    toks = tokens(40, seed=9)
    want = O.forward(cfg, W, toks)
    for cuts in ([40], [22] + [1] * 18, [1] * 40, [5, 2, 9, 24]):
        got, = run_schedule(model, [toks], [cuts])
        assert rel_err(got, want) < 2e-4, cuts
    for variant in (dict(window_shift=1), dict(window_shift=-1), dict(sink=0.0)):
        assert rel_err(O.forward(cfg, W, toks, **variant), want) > 20 * 2e-4, variant


@pytest.mark.parametrize("device", DEVICES)
def test_one_key_stands_out_at_the_window_edge(device, tmp_path):
    """One attention head without rotation whose keys equal its queries: a probe token equal to the last one gets the top score.
    It sits just inside or just outside the window — in a prompt, and with the query decoded alone."""
    left = O.left_cfg(heads=1, kv_heads=1, dim=4, window=9, rot=O.rot_cfg(0, 1.0), scale=0.6, softcap=40.0)
    cfg = O.model_cfg([O.parallel_cfg(left=left, left_scale=8.0, right_scale=0.0)], vocab=12, width=8, buckets=1, mul_prev=0, mul_cur=0)
    W = O.random_weights(cfg, seed=11)
    W["l0.mix.left.k"] = W["l0.mix.left.q"].clone()
    W["bigram"] = torch.zeros_like(W["bigram"])
    model, _ = make(tmp_path, cfg, device, weights=W)
    n = 37
    last = {}
    for probe_at in (n - 9, n - 10, 0, 3, n - 2):
        toks = [5] * n
        toks[probe_at] = 3
        toks[-1] = 3
        want = O.forward(cfg, W, toks)
        last[probe_at] = want[-1:]
        for cuts in ([n], [n - 1, 1], [n - 12] + [1] * 12):
            got, = run_schedule(model, [toks], [cuts])
            assert rel_err(got[-1:], want[-1:]) < 2e-4, (probe_at, cuts)
    assert rel_err(last[n - 9], last[n - 10]) > 100 * 2e-4          # seeing the probe or not moves the last logits
    assert rel_err(last[n - 10], last[0]) < 1e-6                    # outside the window it does not matter where


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("kind", ["retention", "lightning", "gla"])
def test_a_far_token_reaches_the_last_position(device, tmp_path, kind):
    """A recurrence with decays close to one keeps a token from hundreds of positions back: changing the token at position 2 moves
    the last logits, through prompts, portions and single-token steps alike."""
    if kind == "retention":
        layer = O.retention_cfg(heads=2, dim=4, vdim=4, decay=[1.0, 0.999], rot=O.rot_cfg(2, 10.0))
    elif kind == "lightning":
        layer = O.lightning_cfg(heads=1, dim=4, vdim=6, decay=[0.9995])
    else:
        layer = O.parallel_cfg(left=O.left_cfg(heads=1, kv_heads=1, dim=4, window=4), right=O.right_cfg(heads=1, dim=4, vdim=4, tau=5000.0),
                               left_scale=0.0, right_scale=6.0)
    cfg = O.model_cfg([layer], vocab=12, width=8, streams=1)
    W = O.random_weights(cfg, seed=6)
    model, _ = make(tmp_path, cfg, device, weights=W)
    n = 300
    toks = tokens(n, vocab=12, seed=1)
    other = list(toks)
    other[2] = (toks[2] + 5) % 12
    want, want_other = O.forward(cfg, W, toks)[-1:], O.forward(cfg, W, other)[-1:]
    effect = rel_err(want_other, want)                              # what losing (or misplacing) that one token would cost
    assert effect > 1e-3
    for cuts in ([n], [n - 20] + [1] * 20, [100, 2, 150, 48]):
        got, = run_schedule(model, [toks], [cuts])
        assert rel_err(got[-1:], want) < min(2e-4, effect / 20), cuts


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(75, seed=21)
    want = O.forward(cfg, W, toks)
    got, = run_schedule(model, [toks], [[4] + [1] * 71])
    assert rel_err(got, want) < 1e-4
    got2 = run_schedule(model, [toks, toks[:50]], [[4] + [1] * 71, [11] + [1] * 39])
    assert rel_err(got2[0], want) < 1e-4 and rel_err(got2[1], want[:50]) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("case", ["one_stream", "three_streams", "one_head_window_one", "all_experts", "wide_values", "no_rotation",
                                  "unit_constants"])
def test_other_sizes(device, tmp_path, case):
    kw = {}
    if case == "one_stream":
        layers, kw = [O.retention_cfg(mlp=O.dense_cfg(8)), O.parallel_cfg()], dict(streams=1)
    elif case == "three_streams":
        layers, kw = [O.lightning_cfg(mlp=O.moe_cfg(ff=3, experts=2, top=2)), O.parallel_cfg(mlp=O.dense_cfg(8))], dict(streams=3)
    elif case == "one_head_window_one":
        layers = [O.parallel_cfg(left=O.left_cfg(heads=1, kv_heads=1, dim=16, window=1, rot=O.rot_cfg(16, 7.0)),
                                 right=O.right_cfg(heads=1, dim=2, vdim=2, tau=1.0)), O.retention_cfg(heads=1, dim=2, vdim=2, decay=[0.5], rot=O.rot_cfg(2, 3.0))]
    elif case == "all_experts":
        layers = [O.lightning_cfg(heads=1, dim=3, vdim=3, mlp=O.moe_cfg(ff=5, experts=4, top=4)), O.lightning_cfg(mlp=O.moe_cfg(ff=2, experts=1, top=1))]
    elif case == "wide_values":
        layers = [O.lightning_cfg(heads=2, dim=3, vdim=40), O.retention_cfg(heads=1, dim=36, vdim=3, decay=[0.9], rot=O.rot_cfg(6, 20.0)),
                  O.parallel_cfg(left=O.left_cfg(heads=6, kv_heads=2, dim=4, window=11), right=O.right_cfg(heads=4, dim=3, vdim=5, tau=12.0))]
    elif case == "no_rotation":
        layers = [O.retention_cfg(heads=2, dim=6, vdim=4, decay=[0.9, 0.8], rot=O.rot_cfg(0, 1.0)),
                  O.parallel_cfg(left=O.left_cfg(heads=2, kv_heads=1, dim=6, window=5, rot=O.rot_cfg(0, 1.0)))]
    else:                                                           # constants that happen to be 1 or equal in some model
        layers = [O.parallel_cfg(left=O.left_cfg(heads=2, kv_heads=2, dim=4, window=6, scale=1.0, softcap=1.0), right=O.right_cfg(heads=2, dim=4, vdim=4, tau=1.0),
                                 left_scale=1.0, right_scale=1.0, mlp=O.dense_cfg(12)), O.retention_cfg(heads=2, dim=4, vdim=4, decay=[1.0, 1.0], rot=O.rot_cfg(4, 1.0))]
        kw = dict(scale=1.0, mul_prev=1, mul_cur=1, buckets=2)
    cfg = O.model_cfg(layers, vocab=31, width=12, **kw)
    model, W = make(tmp_path, cfg, device, seed=7, rank=2)
    toks = tokens(21, vocab=31, seed=2)
    want = O.forward(cfg, W, toks)
    for cuts in ([21], [6] + [1] * 15, [2, 8, 11]):
        got, = run_schedule(model, [toks], [cuts])
        assert rel_err(got, want) < 1e-4, cuts


# ------------------------------------------------------------------------------------------------------------- generation
@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_entry_points(device, tmp_path):
    cfg = mixed_cfg()
    W = O.random_weights(cfg, seed=2)
    path = save_model(tmp_path, cfg, W)
    model = load_pretrained(path, dtype=torch.float32, device=device)
    prompts = [tokens(7, seed=1), tokens(12, seed=2), tokens(3, seed=3)]
    want = [O.greedy(cfg, W, p, 9) for p in prompts]
    assert RequestScheduler(model).generate(prompts, max_new_tokens=9) == want
    assert model.state_cache().live() == 0
    # the Generator protocol of the other causal LMs: a left-padded batch
    width = max(len(p) for p in prompts)
    ids = torch.tensor([[0] * (width - len(p)) + p for p in prompts], device=device)
    mask = torch.tensor([[0] * (width - len(p)) + [1] * len(p) for p in prompts], device=device)
    out = model.generate(ids, attention_mask=mask, max_length=width + 9, do_sample=False, use_cache=True, eos_token_id=None,
                         pad_token_id=0)
    assert [row[width:].tolist() for row in out] == want
    spec = importlib.util.spec_from_file_location("generate_tool", os.path.join(REPO, "tools", "generate.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    out = tool.main(["--model", path, "--prompts", ";".join(" ".join(map(str, p)) for p in prompts), "--max-new-tokens", "9",
                     "--dtype", "float32", "--device", device])
    assert out == want


@pytest.mark.parametrize("device", DEVICES)
def test_random_init_from_the_config_record(device):
    from libai_b200.config import LazyConfig, instantiate

    node = LazyConfig.load(os.path.join(REPO, "configs", "common", "models", "salizen.py")).model
    node.cfg.width, node.cfg.vocab = 32, 90
    node.cfg.embedding["bigram"]["buckets"] = 11
    for lc in node.cfg.layers:
        m = lc["mixer"]
        if lc["type"] == "parallel":
            m["left"].update(heads=2, kv_heads=1, dim=8, vdim=8)
            m["left"]["rot"]["dims"] = 4
            m["right"].update(heads=2, dim=4, vdim=8)
        else:
            m.update(heads=2, dim=8, vdim=4, decay=[0.9, 0.99])
            if "rot" in m:
                m["rot"]["dims"] = 8
        if lc["mlp"] and lc["mlp"]["kind"] == "dense":
            lc["mlp"]["ff"] = 16
        elif lc["mlp"]:
            lc["mlp"]["expert"]["ff"] = 8
    with param_defaults(dtype=torch.float32, device=device, seed=3):
        model = instantiate(node).eval()
    out = RequestScheduler(model).generate([[1, 2, 3, 4, 5], [7]], max_new_tokens=5)
    assert [len(o) for o in out] == [5, 5] and all(0 <= t < 90 for o in out for t in o)


# ------------------------------------------------------------------------------------------------------ kernels (GPU only)
def _gpu_cfg(D, G, rep, window, width=64):
    left = O.left_cfg(heads=G * rep, kv_heads=G, dim=D, window=window, rot=O.rot_cfg(D // 2, 1e4), scale=D ** -0.5, softcap=20.0)
    layers = [O.parallel_cfg(left=left, right=O.right_cfg(heads=2, dim=16, vdim=32, tau=8.0), mlp=O.dense_cfg(32)),   # no experts here: in bf16 a
              O.retention_cfg(heads=2, dim=32, vdim=16, rot=O.rot_cfg(32, 1e4), mlp=O.dense_cfg(64)),               # close router call would flip a position
              O.lightning_cfg(heads=2, dim=16, vdim=32, decay=[0.7, 0.99])]
    return O.model_cfg(layers, vocab=64, width=width)


@pytest.mark.gpu
@pytest.mark.parametrize("D,G,rep", [(32, 2, 2), (48, 1, 3), (64, 2, 4), (96, 1, 1), (128, 1, 8)])
def test_tensor_core_prompts_and_grouped_decode_match_the_generic_kernels(tmp_path, monkeypatch, D, G, rep):
    """bf16: the tensor-core prompt kernel and the grouped split kernel of single-token steps (both with the score cap, the sink
    and the channel-wise gate) against the one-warp-per-head kernel, on prompts that cross many key tiles, continue from cached
    rows and decode past the window; and all of them against the oracle."""
    cfg = _gpu_cfg(D, G, rep, window=150)
    W = O.random_weights(cfg, seed=D, rank=8)
    model, _ = make(tmp_path, cfg, "cuda", dtype=torch.bfloat16, weights=W, rank=8)
    prompts = [tokens(n, vocab=64, seed=n) for n in (333, 64, 201)]
    cuts = [[200, 133], [64], [130, 71]]
    fast = run_schedule(model, prompts, cuts)
    dec_fast = run_schedule(model, prompts[:2], [[300] + [1] * 33, [30] + [1] * 34], cuda_graphs=False)
    monkeypatch.setattr(KF, "MMA_HEAD_SIZES", ())
    monkeypatch.setattr(KF, "GROUPED_DECODE", False)
    slow = run_schedule(model, prompts, cuts)
    dec_slow = run_schedule(model, prompts[:2], [[300] + [1] * 33, [30] + [1] * 34], cuda_graphs=False)
    want = [O.forward(cfg, W, p) for p in prompts]
    for a, b, w in zip(fast + dec_fast, slow + dec_slow, want + want[:2]):
        ea, eb = rel_err(a, w), rel_err(b, w)                      # both round to bf16, at different places: neither is the truth
        assert ea < 8e-2 and ea < 2.0 * eb + 1e-2, (ea, eb)
        assert rel_err(a, b.float().cpu()) < 8e-2
    # and the fp32 kernels, grouped and not, agree to rounding
    model32, _ = make(tmp_path, cfg, "cuda", dtype=torch.float32, weights=W, rank=8)
    one = run_schedule(model32, prompts[:1], [[300] + [1] * 33], cuda_graphs=False)
    monkeypatch.setattr(KF, "GROUPED_DECODE", True)
    two = run_schedule(model32, prompts[:1], [[300] + [1] * 33], cuda_graphs=False)
    assert rel_err(one[0], two[0].cpu()) < 1e-5
    assert rel_err(one[0][:64], O.forward(cfg, W, prompts[0][:64])) < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("width,vocab", [(20, 37), (36, 101)])
def test_sizes_the_fast_paths_refuse_in_bf16(tmp_path, width, vocab):
    """bf16 with a width, a vocabulary, head and expert sizes that are no multiples of 8 (or of 4): every product and kernel falls
    back to its general form and the result stays within bf16 rounding of the oracle."""
    layers = [O.parallel_cfg(left=O.left_cfg(heads=3, kv_heads=1, dim=6, window=9, rot=O.rot_cfg(4, 40.0)), right=O.right_cfg(heads=3, dim=5, vdim=7), mlp=O.dense_cfg(12)),
              O.retention_cfg(heads=2, dim=10, vdim=6, rot=O.rot_cfg(10, 40.0), mlp=O.dense_cfg(20)),
              O.lightning_cfg(heads=3, dim=5, vdim=3, mlp=O.dense_cfg(9))]
    cfg = O.model_cfg(layers, vocab=vocab, width=width, streams=3)
    W = O.random_weights(cfg, seed=width)
    model, _ = make(tmp_path, cfg, "cuda", dtype=torch.bfloat16, weights=W)
    prompts = [tokens(n, vocab=vocab, seed=n) for n in (33, 18)]
    want = [O.forward(cfg, W, p) for p in prompts]
    got = run_schedule(model, prompts, [[20] + [1] * 13, [18]])
    errs = [rel_err(g, w) for g, w in zip(got, want)]
    assert max(errs) < 8e-2, errs


@pytest.mark.gpu
def test_serving_precision_and_graphed_steps(tmp_path):
    cfg = mixed_cfg(width=32)
    for lc in cfg["layers"]:                                        # dense feed-forwards: a close router call would flip a position in bf16
        if lc["mlp"]:
            lc["mlp"] = O.dense_cfg(16)
    W = O.random_weights(cfg, seed=3)
    path = save_model(tmp_path, cfg, W)
    model = load_pretrained(path, dtype=torch.bfloat16, device="cuda")
    prompts = [tokens(n, seed=n) for n in (24, 9, 40)]
    want = [O.forward(cfg, W, p) for p in prompts]
    cuts = [[10] + [1] * 14, [5] + [1] * 4, [25] + [1] * 15]
    eager = run_schedule(model, prompts, cuts, cuda_graphs=False)
    graphed = run_schedule(model, prompts, cuts, cuda_graphs=True)
    for e, g_, w in zip(eager, graphed, want):
        assert rel_err(e, w) < 1e-1                             # five blocks of width 32 in bf16: the worst position
        assert float(torch.tensor([rel_err(e[i:i + 1], w[i:i + 1]) for i in range(len(w))]).median()) < 3e-2
        assert rel_err(g_, e.float().cpu()) < 1e-6              # a replayed step computes exactly what an eager one does


def test_trace_runner_replays_steps(tmp_path):
    """``bin/trace_run`` on a tiny checkpoint (CPU): a prompt step for two requests, single-token steps, one request ending early;
    the files it writes hold the wanted logits in the order of the entries."""
    import subprocess
    import sys

    import numpy as np

    cfg = mixed_cfg()
    W = O.random_weights(cfg, seed=8)
    path = save_model(tmp_path, cfg, W)
    a, b = tokens(9, seed=4), tokens(6, seed=5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:7], "want": [0, 6]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[7:8], "want": []}, {"id": "b", "tokens": b[5:6], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[8:9], "want": [0]}], "end": ["a"]}]
    out = os.path.join(str(tmp_path), "out")
    res = subprocess.run([sys.executable, os.path.join(REPO, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", out,
                          "--max-tokens", "64", "--device", "cpu"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.split("\n") if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = O.forward(cfg, W, a), O.forward(cfg, W, b)
    vocab = cfg["vocab"]
    got0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(-1, vocab).copy())
    assert rel_err(got0, torch.stack([wa[0], wa[6], wb[4]])) < 1e-4
    got1 = torch.from_numpy(np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").reshape(-1, vocab).copy())
    assert rel_err(got1, wb[5:6]) < 1e-4
    got2 = torch.from_numpy(np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(-1, vocab).copy())
    assert rel_err(got2, wa[8:9]) < 1e-4
