"""Zubarax against a plain float64 oracle (``zubarax_oracle.py``): every mechanism alone, whole prompts, decoding through the
paged cache and the recurrent state, prompt portions, ragged batches, pages and slots that are freed and used again, keys far
away and at page borders made decisive, the first tokens of a sequence, long decoding, other sizes, generation.

The CPU parametrisation exercises the framework's PyTorch operators; the ``cuda`` one (marked ``gpu``) the sm_100a kernels.
"""
import importlib.util
import json
import os

import pytest
import torch

from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.scheduler import RequestScheduler
from libai_b200.inference.state_cache import SequenceStateCache
from libai_b200.layers import DecayLinearAttention, GatedFeedForward, MoEFeedForward, PagedAttention
from libai_b200.layers._param import param_defaults
from libai_b200.models.utils.model_loader.auto import load_pretrained
from libai_b200.ops import kv_functional as KF
from libai_b200.ops import paged_functional as PF

from . import zubarax_oracle as O

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


def make(tmp_path, cfg, device, dtype=torch.float32, seed=0, weights=None, page_size=4):
    """The loaded model (pages of ``page_size`` positions: small, so that short prompts cross many page borders) and its weights."""
    weights = weights if weights is not None else O.random_weights(cfg, seed)
    model = load_pretrained(save_model(tmp_path, cfg, weights), dtype=dtype, device=device)
    model.kv_page_size = page_size
    return model, weights


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
    """Every branch once: experts with and without a shared one, a block without a feed-forward, grouped and ungrouped key
    heads, value heads wider and narrower than key heads, partial and full rotation, two to four taps, blocks that run again
    with a state of their own."""
    layers = [O.layer(O.side_cfgs(), mlp=O.moe_cfg()),
              O.layer(O.side_cfgs(heads=4, kv_heads=2, dim=6, vdim=10, conv=2, rot_dims=6, rot_base=30.0, rheads=1, rdim=10, rvdim=6,
                                  left_scale=1.1, right_scale=0.4), mlp=None),
              O.layer(O.side_cfgs(), mlp=O.moe_cfg(), weights_of=0),
              O.layer(O.side_cfgs(heads=3, kv_heads=3, dim=4, vdim=4, conv=4, rot_dims=2, rheads=3, rdim=4, rvdim=4),
                      mlp=O.moe_cfg(ff=4, experts=3, top=1, limit=0.7, shared_ff=0)),
              O.layer(O.side_cfgs(heads=4, kv_heads=2, dim=6, vdim=10, conv=2, rot_dims=6, rot_base=30.0, rheads=1, rdim=10, rvdim=6,
                                  left_scale=1.1, right_scale=0.4), mlp=None, weights_of=1)]
    return O.model_cfg(layers, **kw)


def _load_side(mod, W, prefix, names):
    with torch.no_grad():
        for attr, name in names.items():
            getattr(mod, attr).copy_(W[prefix + name])


def _run_mixer(mod, h, device, lens, page_size=4):
    """A mixer module alone on one sequence ``h`` ``[n, width]`` fed in the portions ``lens``; returns ``[n, width]``."""
    cache = SequenceStateCache(device, torch.float32, page_size=page_size)
    kind, shape = mod.state_spec()
    handle = cache.register(kind, **shape)
    slot = cache.allocate(3)[1:2]                                   # not slot 0
    out, at = [], 0
    for n in lens:
        cache.prepare(slot, [n])
        rb = RaggedBatch([n], slot, [at], device)
        with torch.no_grad():
            out.append(mod(h[at:at + n].float().to(device), rb, cache.buffers(handle)).cpu().double())
        cache.advance(slot, [n])
        at += n
    return torch.cat(out)


LEFT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "q_norm": "q.norm",
              "k_norm": "k.norm", "talk": "talk", "sink": "sink"}
RIGHT_NAMES = {"q": "q", "f": "f", "v": "v", "o": "o", "f_b": "f.b", "lower": "lower", "norm": "norm"}


# ------------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("lens", [[19], [1] * 19, [5, 1, 9, 2, 2]])
@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=6, vdim=10, conv=3, rot_dims=4), dict(heads=3, kv_heads=1, dim=8, vdim=4, conv=1, rot_dims=8),
                                   dict(heads=1, kv_heads=1, dim=4, vdim=6, conv=5, rot_dims=0)])
def test_softmax_side_alone(device, lens, sizes):
    width, eps = 16, 1e-5
    m = O.side_cfgs(**sizes)
    W = O.random_weights(O.model_cfg([O.layer(m)], width=width), seed=3)
    a = m["left"]
    with param_defaults(dtype=torch.float32, device=device):
        mod = PagedAttention(width, a["heads"], a["kv_heads"], a["dim"], a["vdim"], scale=a["scale"], conv=a["conv"], v_norm=True,
                             rot_dims=a["rot"]["dims"], rot_base=a["rot"]["base"], talk=True, sink=True, eps=eps)
    _load_side(mod, W, "l0.mix.left.", LEFT_NAMES)
    h = torch.randn(19, width, generator=torch.Generator().manual_seed(1), dtype=F64)
    want = O.softmax_side(h, W, "l0.mix.left.", a, eps)
    got = _run_mixer(mod, h, device, lens)
    assert torch.allclose(got, want, atol=3e-5)
    # each ingredient is visible in the result: the sink, the mix over heads, the convolution, the value norm
    p = "l0.mix.left."
    far = lambda Wx: not torch.allclose(O.softmax_side(h, Wx, p, a, eps), want, atol=1e-2)
    assert far({**W, p + "sink": W[p + "sink"] - 30.0})
    if a["heads"] > 1:
        assert far({**W, p + "talk": torch.eye(a["heads"], dtype=F64)})
    if a["conv"] > 1:
        assert far({**W, p + "k.conv": torch.roll(W[p + "k.conv"], 1, 1)})
    assert far({**W, p + "v": 3.0 * W[p + "v"]}) is False                     # unit-RMS values: a scaled projection changes nothing


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("lens", [[21], [1] * 21, [2, 16, 1, 2]])
@pytest.mark.parametrize("H,D,V", [(2, 4, 8), (1, 24, 40), (3, 16, 4)])
def test_recurrent_side_alone(device, lens, H, D, V):
    width, eps = 16, 1e-5
    m = O.side_cfgs(rheads=H, rdim=D, rvdim=V)
    W = O.random_weights(O.model_cfg([O.layer(m)], width=width), seed=4)
    with param_defaults(dtype=torch.float32, device=device):
        mod = DecayLinearAttention(width, H, D, V, decay="tied", qkv_act="silu_q", norm="head", norm_weight=True, gate=None, eps=eps)
    assert mod.k is None and mod.g is None
    _load_side(mod, W, "l0.mix.right.", RIGHT_NAMES)
    h = torch.randn(21, width, generator=torch.Generator().manual_seed(2), dtype=F64)
    want = O.recurrent_side(h, W, "l0.mix.right.", m["right"], eps)
    assert torch.allclose(_run_mixer(mod, h, device, lens), want, atol=3e-5)
    p = "l0.mix.right."
    assert not torch.allclose(O.recurrent_side(h, {**W, p + "lower": torch.zeros_like(W[p + "lower"])}, p, m["right"], eps), want, atol=1e-2)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("n", [24, 19, 1100])
def test_post_norm_residual(device, n):
    g = torch.Generator().manual_seed(5)
    rows, top = 9, 2
    x = torch.randn(rows, n, generator=g)
    y, ys = torch.randn(rows, n, generator=g), torch.randn(rows * top + 3, n, generator=g)
    w = (0.3 * torch.randn(n, generator=g)).to(torch.bfloat16).float()
    pos = torch.randperm(rows * top + 3, generator=g)[: rows * top].view(rows, top).int()
    want = O.centred_norm(1.75 * x.double() + y.double() + ys.double()[pos.long()].sum(1), w.double(), 1e-5)
    xd, h = x.clone().to(device), torch.empty(rows, n, device=device)
    PF.postnorm_residual(xd, w.to(device), 1e-5, alpha=1.75, y=y.to(device), y2=ys.to(device), pos=pos.to(device), h=h)
    assert torch.allclose(xd.cpu().double(), want, atol=1e-5) and torch.equal(xd, h)
    # the norm alone, the residual left as it is
    xd, h = x.clone().to(device), torch.empty(rows, n, device=device)
    PF.postnorm_residual(xd, w.to(device), 1e-5, h=h, inplace=False)
    assert torch.equal(xd.cpu(), x) and torch.allclose(h.cpu().double(), O.centred_norm(x.double(), w.double(), 1e-5), atol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("experts,top,rows", [(5, 2, 40), (4, 1, 7), (3, 3, 21), (40, 6, 3)])
def test_experts_weighted_on_their_inputs(device, experts, top, rows):
    width = 16
    mc = O.moe_cfg(ff=8, experts=experts, top=top, limit=0.8, shared_ff=12, shared_limit=0.5)
    W = O.random_weights(O.model_cfg([O.layer(mlp=mc)], width=width), seed=6)
    with param_defaults(dtype=torch.float32, device=device):
        mod = MoEFeedForward(width, 8, experts, top, router="sigmoid_raw", act="swish_clamp", limit=0.8, weight_input=True)
        shared = GatedFeedForward(width, 12, "swish_clamp", limit=0.5)
    p = "l0.mlp."
    with torch.no_grad():
        mod.router.copy_(W[p + "router"])
        mod.gate_up.copy_(torch.stack([torch.cat([W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"]]) for e in range(experts)]))
        mod.down.copy_(torch.stack([W[f"{p}e{e}.down"] for e in range(experts)]))
        shared.gate_up.copy_(torch.cat([W[p + "shared.gate"], W[p + "shared.up"]]))
        shared.down.copy_(W[p + "shared.down"])
    h = torch.randn(rows, width, generator=torch.Generator().manual_seed(7), dtype=F64)
    want = O.feed_forward(h, W, p, mc)
    scores, chosen = O.router(h, W, p, mc)
    hd = h.float().to(device)
    idx, wts = KF.moe_route(hd, mod.router, top, 1.0, mode=KF.ROUTE_SIGMOID_RAW)
    assert torch.equal(idx.cpu().long(), chosen) and torch.allclose(wts.cpu().double(), scores, atol=1e-6)
    with torch.no_grad():
        for graph_safe in (False, True):                           # sorted form (many rows) and pair form
            d, pos, cw = mod(hd, graph_safe=graph_safe)
            assert cw is None
            d = d if pos is None else d[pos.long()].sum(1)
            assert torch.allclose((d + shared(hd)).cpu().double(), want, atol=3e-5)
    # a weight on the output instead would be another function (the experts are not linear)
    wrong = sum(scores[:, k:k + 1] * torch.stack([O.clamped_expert(h[t], W, f"{p}e{int(chosen[t, k])}.", 0.8) for t in range(rows)]) for k in range(top))
    assert not torch.allclose(wrong + O.clamped_expert(h, W, p + "shared.", 0.5), want, atol=1e-3)


# ---------------------------------------------------------------------------------------------------------- whole model
@pytest.mark.parametrize("device", DEVICES)
def test_whole_prompt_with_residuals(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(19)
    residuals = []
    want = O.forward(cfg, W, toks, residuals)
    taps = []
    cache = model.state_cache()
    slots = cache.allocate(1)
    got = model.step(torch.tensor(toks, device=device), RaggedBatch([len(toks)], slots, [0], device),
                     tap=lambda i, x: taps.append(x.detach().cpu().double().clone()))
    cache.free(slots)
    assert len(taps) == len(residuals) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(taps, residuals)):
        assert torch.allclose(a, b, atol=2e-4), f"residual after entry {i}"
    assert rel_err(got, want) < 1e-4
    assert len(model.model.layers) == 3 and model.model.runs == [0, 1, 0, 2, 1]      # two entries run another entry's block


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
    cuts2 = [[1], [5, 12], [1, 3], [2, 20, 8], [4, 1, 4]]          # unequal portions in one step
    for got, w in zip(run_schedule(model, prompts, cuts2), want):
        assert rel_err(got, w) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_pages_and_slots_are_reused_without_clearing(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device, page_size=4)
    sched = RequestScheduler(model)
    cache = sched.cache
    a, b, c = tokens(23, seed=1), tokens(8, seed=2), tokens(15, seed=3)
    sched.step([("a", a, []), ("b", b, [])])
    slot_a, pages_a = sched.slot_of["a"], list(cache._pages[sched.slot_of["a"]])
    assert len(pages_a) == 6 and len(cache._pages[sched.slot_of["b"]]) == 2
    sched.finish(["a"])
    got = sched.step([("c", c[:6], list(range(6)))])               # takes a's slot and a's first pages: tails, states and rows are a's
    assert sched.slot_of["c"] == slot_a and cache._pages[slot_a] == pages_a[:2]
    got = torch.cat([got] + [sched.step([("c", [t], [0]), ("b", [1], [])]) for t in c[6:]])
    assert rel_err(got, O.forward(cfg, W, c)) < 1e-4
    before, pages_before = cache.capacity, cache.num_pages
    many = [(("m", i), tokens(3 + i, seed=10 + i), [2 + i]) for i in range(before + 3)]      # more requests than slots, more rows than pages
    logits = sched.step(many)
    assert cache.capacity > before and cache.num_pages > pages_before
    for row, (_, p, _) in enumerate(many):
        assert rel_err(logits[row:row + 1], O.forward(cfg, W, p)[-1:]) < 1e-4
    got = sched.step([("c", [7], [0])])                            # a request that lived through the growth goes on
    assert rel_err(got, O.forward(cfg, W, c + [7])[-1:]) < 1e-4
    sched.finish(["b", "c"] + [("m", i) for i in range(before + 3)])
    assert cache.live() == 0 and len(cache._free_pages) == cache.num_pages       # every page came back


# ------------------------------------------------------------------------------------------- far keys, page borders, starts
def sharp_model(tmp_path, device, n, key_at, page_size):
    """One block whose last query finds exactly one key: the inputs of the softmax side are built by hand (identity-like
    projections on one-hot embeddings), so that the score of position ``key_at`` stands far above all others, and that key's
    value is unlike every other value."""
    width = 16
    m = O.side_cfgs(heads=1, kv_heads=1, dim=8, vdim=8, conv=1, rot_dims=0, rheads=1, rdim=4, rvdim=4, left_scale=1.0, right_scale=0.0)
    m["left"]["scale"] = 1.0
    cfg = O.model_cfg([O.layer(m, mlp=None)], vocab=8, width=width, alpha=0.0, scale=1.0)
    W = O.random_weights(cfg, seed=9)
    p = "l0.mix.left."
    E = torch.zeros(8, width, dtype=F64)
    for t in range(8):
        E[t, t] = 1.0
    W["embed"] = E
    q, k, v = torch.zeros(8, width, dtype=F64), torch.zeros(8, width, dtype=F64), 0.1 * torch.ones(8, width, dtype=F64)
    q[0, 1] = q[0, 2] = 1.0           # token 1 (the probe) and token 2 (the needle) share a query/key direction; token 0 is filler
    k[0, 1] = k[0, 2] = 1.0
    k[1, 0] = q[1, 0] = 1.0           # the filler's direction
    v[3, 2] = 4.0                     # the needle's value is unlike the others
    v[4, 0] = 1.0
    v[5, 1] = 1.0
    W[p + "q"], W[p + "k"], W[p + "v"] = q, k, v
    W[p + "q.norm"], W[p + "k.norm"] = 6.0 * torch.ones(8, dtype=F64), 6.0 * torch.ones(8, dtype=F64)
    W[p + "q.conv"], W[p + "k.conv"], W[p + "v.conv"] = (torch.ones(8, 1, dtype=F64) for _ in range(3))
    W[p + "talk"], W[p + "sink"] = torch.ones(1, 1, dtype=F64), torch.tensor([-2.0], dtype=F64)
    toks = [0] * n
    toks[key_at] = 2
    toks[-1] = 1
    return cfg, W, toks


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("key_at,page_size", [(0, 8), (7, 8), (8, 8), (63, 8), (64, 8), (150, 64), (1, 3)])
def test_one_far_key_decides_the_last_position(device, tmp_path, key_at, page_size):
    n = 200
    cfg, W, toks = sharp_model(tmp_path, device, n, key_at, page_size)
    want = O.forward(cfg, W, toks)[-1:]
    moved = list(toks)
    moved[key_at] = 0
    assert rel_err(O.forward(cfg, W, moved)[-1:], want) > 0.3            # the key is decisive
    model, _ = make(tmp_path, cfg, device, weights=W, page_size=page_size)
    for cuts in ([n], [n - 1, 1], [key_at + 1] + [1] * (n - key_at - 1) if key_at > 100 else [n - 40] + [1] * 40):
        got, = run_schedule(model, [toks], [cuts])
        assert rel_err(got[-1:], want) < 1e-4, cuts


@pytest.mark.parametrize("device", DEVICES)
def test_the_first_tokens_of_a_sequence(device, tmp_path):
    """Convolution taps that reach before the start read zeros, whatever the slot held, also when the start is fed token by
    token; the state of the recurrence starts at zero."""
    cfg = O.model_cfg([O.layer(O.side_cfgs(conv=4), mlp=O.moe_cfg())])
    model, W = make(tmp_path, cfg, device)
    sched = RequestScheduler(model)
    sched.step([("old", tokens(11, seed=8), [])])                  # leaves tails, pages and a state behind in slot 0
    sched.finish(["old"])
    toks = tokens(6, seed=9)
    want = O.forward(cfg, W, toks)
    for cuts in ([6], [1] * 6, [2, 1, 3]):
        got, = run_schedule(model, [toks], [cuts])
        assert rel_err(got, want) < 1e-4, cuts


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding(device, tmp_path):
    cfg = O.model_cfg([O.layer(mlp=O.moe_cfg()), O.layer(weights_of=0, mlp=O.moe_cfg())])
    model, W = make(tmp_path, cfg, device, page_size=16)
    toks = tokens(150, seed=4)
    want = O.forward(cfg, W, toks)
    got, = run_schedule(model, [toks], [[10] + [1] * 140])
    assert rel_err(got, want) < 2e-4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("case", ["one_head", "one_tap", "all_experts", "wide_values", "no_rotation", "odd_sizes", "many_heads"])
def test_other_sizes(device, tmp_path, case):
    sides, mlp, kw = O.side_cfgs(), O.moe_cfg(), {}
    if case == "one_head":
        sides = O.side_cfgs(heads=1, kv_heads=1, dim=16, vdim=16, rot_dims=16, rheads=1, rdim=16, rvdim=16)
    elif case == "one_tap":
        sides = O.side_cfgs(conv=1)
    elif case == "all_experts":
        mlp = O.moe_cfg(experts=3, top=3, shared_ff=0)
    elif case == "wide_values":
        sides = O.side_cfgs(heads=2, kv_heads=2, dim=4, vdim=36, rvdim=40, rdim=12)
    elif case == "no_rotation":
        sides = O.side_cfgs(rot_dims=0)
    elif case == "odd_sizes":
        sides, kw = O.side_cfgs(heads=3, kv_heads=1, dim=10, vdim=7, rot_dims=6, rheads=3, rdim=5, rvdim=9), dict(width=20, vocab=37)
        mlp = O.moe_cfg(ff=5, experts=7, top=3, shared_ff=9)
    elif case == "many_heads":
        sides = O.side_cfgs(heads=12, kv_heads=4, dim=4, vdim=4, rot_dims=2)
    cfg = O.model_cfg([O.layer(sides, mlp=mlp), O.layer(sides, mlp=None)], **kw)
    model, W = make(tmp_path, cfg, device, seed=11)
    prompts = [tokens(n, vocab=cfg["vocab"], seed=n) for n in (13, 22)]
    want = [O.forward(cfg, W, p) for p in prompts]
    for got, w in zip(run_schedule(model, prompts, [[9] + [1] * 4, [22]]), want):
        assert rel_err(got, w) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_a_second_norm_without_a_feed_forward(device, tmp_path):
    """A checkpoint may carry the second norm of an entry that has no feed-forward: it then norms alpha · x alone, also in the
    entry that borrows the tensors."""
    sides = O.side_cfgs()
    cfg = O.model_cfg([O.layer(sides, mlp=None), O.layer(sides, mlp=O.moe_cfg()), O.layer(sides, mlp=None, weights_of=0)])
    W = O.random_weights(cfg, seed=6)
    plain = O.forward(cfg, W, tokens(11, vocab=cfg["vocab"], seed=3))
    W["l0.norm2"] = (0.3 * torch.randn(cfg["width"], dtype=torch.float64)).to(torch.bfloat16).double()
    model, _ = make(tmp_path, cfg, device, weights=W)
    p = tokens(11, vocab=cfg["vocab"], seed=3)
    want = O.forward(cfg, W, p)
    assert rel_err(want, plain) > 1e-2                        # the extra norm matters
    (got,) = run_schedule(model, [p], [[6, 2, 1, 1, 1]])
    assert rel_err(got, want) < 1e-4


# ------------------------------------------------------------------------------------------------------------- generation
@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_entry_points(device, tmp_path):
    cfg = mixed_cfg()
    W = O.random_weights(cfg, seed=2)
    path = save_model(tmp_path, cfg, W)
    model = load_pretrained(path, dtype=torch.float32, device=device)
    model.kv_page_size = 8
    prompts = [tokens(7, seed=1), tokens(12, seed=2), tokens(3, seed=3)]
    want = [O.greedy(cfg, W, p, 9) for p in prompts]
    assert RequestScheduler(model).generate(prompts, max_new_tokens=9) == want
    assert model.state_cache().live() == 0
    width = max(len(p) for p in prompts)                           # the Generator protocol of the other causal LMs: a left-padded batch
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

    node = LazyConfig.load(os.path.join(REPO, "configs", "common", "models", "zubarax.py")).model
    node.cfg.width, node.cfg.vocab = 32, 90
    for lc in node.cfg.layers:
        m = lc["mixer"]
        m["left"].update(heads=2, kv_heads=1, dim=8, vdim=8, scale=8 ** -0.5)
        m["left"]["rot"]["dims"] = 4
        m["right"].update(heads=2, dim=4, vdim=8)
        if lc["mlp"]:
            lc["mlp"]["expert"]["ff"] = 8
            lc["mlp"]["shared"]["ff"] = 8
    with param_defaults(dtype=torch.float32, device=device, seed=3):
        model = instantiate(node).eval()
    out = RequestScheduler(model).generate([[1, 2, 3, 4, 5], [7]], max_new_tokens=5)
    assert [len(o) for o in out] == [5, 5] and all(0 <= t < 90 for o in out for t in o)


def test_a_checkpoint_that_lacks_a_tensor_is_refused(tmp_path):
    cfg = O.model_cfg([O.layer(mlp=O.moe_cfg())])
    W = O.random_weights(cfg, seed=1)
    del W["l0.mix.left.sink"]
    with pytest.raises(RuntimeError, match="lacks tensors"):
        load_pretrained(save_model(tmp_path, cfg, W), dtype=torch.float32, device="cpu")


# ------------------------------------------------------------------------------------------------------ kernels (GPU only)
@pytest.mark.gpu
@pytest.mark.parametrize("H,G,D,V", [(8, 2, 64, 64), (16, 4, 128, 128), (4, 4, 32, 96)])
def test_attention_tilings_agree(H, G, D, V):
    """The prompt tiling, the single-token tiling with one part and with many parts compute the same attention (fp32 and bf16
    storage), at head sizes that make the kernel choose smaller tiles."""
    torch.manual_seed(0)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        n, ps = 150, 16
        cache = SequenceStateCache("cuda", dtype, page_size=ps)
        handle = cache.register("paged", channels=G * (D + V), taps=1, conv_channels=1)
        slots = cache.allocate(2)
        cache.prepare(slots, [n, n // 2])
        cache.advance(slots, [n, n // 2])
        bufs = cache.buffers(handle)
        bufs["pool"].copy_(torch.randn(bufs["pool"].shape, device="cuda").to(dtype))
        talk = (torch.eye(H) + 0.2 * torch.randn(H, H)).cuda()
        sink = torch.randn(H).cuda()
        q = torch.randn(n + n // 2, H * D, device="cuda").to(dtype)
        whole = RaggedBatch([n, n // 2], slots, [0, 0], "cuda")
        y = torch.empty(n + n // 2, H * V, device="cuda", dtype=dtype)
        PF.talk_attention(q, bufs["pool"], bufs["table"], whole, y, H, G, D, V, D ** -0.5, talk=talk, sink=sink, out_scale=0.7)
        last = RaggedBatch([1, 1], slots, [n - 1, n // 2 - 1], "cuda")
        ql = torch.stack([q[n - 1], q[-1]])
        for parts in (1, 5, None):
            yl = torch.empty(2, H * V, device="cuda", dtype=dtype)
            PF.talk_attention(ql, bufs["pool"], bufs["table"], last, yl, H, G, D, V, D ** -0.5, talk=talk, sink=sink, out_scale=0.7, parts=parts)
            assert torch.allclose(yl.float(), torch.stack([y[n - 1], y[-1]]).float(), atol=tol), (dtype, parts)


@pytest.mark.gpu
def test_serving_precision_and_graphed_steps(tmp_path):
    cfg = O.model_cfg([O.layer(O.side_cfgs(heads=4, kv_heads=2, dim=8, vdim=8, rot_dims=8, rheads=2, rdim=8, rvdim=8), mlp=None),
                       O.layer(O.side_cfgs(heads=4, kv_heads=2, dim=8, vdim=8, rot_dims=8, rheads=2, rdim=8, rvdim=8), mlp=None, weights_of=0)],
                      width=32)                                     # no experts: a close router call would flip a position in bf16
    W = O.random_weights(cfg, seed=3)
    model = load_pretrained(save_model(tmp_path, cfg, W), dtype=torch.bfloat16, device="cuda")
    model.kv_page_size = 8
    prompts = [tokens(n, seed=n) for n in (24, 9, 40)]
    want = [O.forward(cfg, W, p) for p in prompts]
    cuts = [[10] + [1] * 14, [5] + [1] * 4, [25] + [1] * 15]
    eager = run_schedule(model, prompts, cuts, cuda_graphs=False)
    graphed = run_schedule(model, prompts, cuts, cuda_graphs=True)
    for e, g_, w in zip(eager, graphed, want):
        assert rel_err(e, w) < 1e-1
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


@pytest.mark.gpu
@pytest.mark.parametrize("H,G,D", [(8, 2, 64), (8, 2, 128), (16, 4, 128), (6, 3, 64), (12, 12, 64), (5, 1, 128), (1, 1, 64)])
def test_tensor_core_prompts_match_the_generic_kernel(H, G, D):
    """bf16 prompt steps on the tensor-core kernel against the generic one: ragged lengths, a continued sequence (keys from
    earlier pages), tiles that end inside a page, heads that do and do not fill the padded register arrays."""
    torch.manual_seed(1)
    ps = 16
    cache = SequenceStateCache("cuda", torch.bfloat16, page_size=ps)
    handle = cache.register("paged", channels=2 * G * D, taps=1, conv_channels=1)
    slots = cache.allocate(3)
    lens, past = [70, 1, 37], [0, 45, 90]
    cache.prepare(slots, [a + b for a, b in zip(lens, past)])
    bufs = cache.buffers(handle)
    bufs["pool"].copy_(torch.randn(bufs["pool"].shape, device="cuda").to(torch.bfloat16))
    talk = (torch.eye(H) + 0.3 * torch.randn(H, H)).cuda()
    sink = torch.randn(H).cuda()
    rb = RaggedBatch(lens, slots, past, "cuda")
    q = (2.0 * torch.randn(sum(lens), H * D, device="cuda")).to(torch.bfloat16)
    assert PF.mma_eligible(q, bufs["pool"], q, H, G, D, D)
    got, want = torch.empty_like(q), torch.empty_like(q)
    PF.talk_attention(q, bufs["pool"], bufs["table"], rb, got, H, G, D, D, D ** -0.5, talk=talk, sink=sink, out_scale=0.8)
    PF.talk_attention(q, bufs["pool"], bufs["table"], rb, want, H, G, D, D, D ** -0.5, talk=talk, sink=sink, out_scale=0.8, mma=False)
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert float((got.float() - want.float()).abs().mean()) < 2e-3


@pytest.mark.gpu
def test_bf16_model_on_the_tensor_core_path(tmp_path, monkeypatch):
    """A whole bf16 model whose head size the tensor-core prompt kernel takes: against the oracle, and against the same model
    kept on the generic kernel."""
    sides = O.side_cfgs(heads=4, kv_heads=2, dim=64, vdim=64, conv=3, rot_dims=32, rheads=2, rdim=16, rvdim=32)
    cfg = O.model_cfg([O.layer(sides, mlp=None), O.layer(sides, mlp=None, weights_of=0)], width=64)
    W = O.random_weights(cfg, seed=5)
    model = load_pretrained(save_model(tmp_path, cfg, W), dtype=torch.bfloat16, device="cuda")
    model.kv_page_size = 16
    prompts = [tokens(70, seed=1), tokens(33, seed=2)]
    want = [O.forward(cfg, W, p) for p in prompts]
    cuts = [[60] + [1] * 10, [33]]
    fast = run_schedule(model, prompts, cuts)
    monkeypatch.setattr(PF, "mma_eligible", lambda *a: False)
    slow = run_schedule(model, prompts, cuts)
    for f, s_, w in zip(fast, slow, want):
        assert rel_err(f, w) < 1e-1 and rel_err(s_, w) < 1e-1
        assert rel_err(f, s_.float().cpu()) < 5e-2
        assert not torch.equal(f, s_)                              # the two paths did run different kernels
