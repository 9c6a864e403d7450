"""A plain, slow restatement of the Salizen design in float64, token by token, one function per mechanism.  It shares no code
with the package: the tests compare the framework's operators, layers, cache and scheduler against it.

Notation.  Positions count from 0.  Linear maps are stored ``[out, in]`` and applied as ``W @ v``.  ``W`` is the dictionary of
checkpoint tensors (float64), ``p`` the prefix of a block's tensors (``"l3."``).
"""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------------------ small pieces
def rms_divide(v, eps):
    return v / torch.sqrt((v * v).mean() + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def rotary_frequencies(rot):
    """Angular frequency of every rotated pair.  With ``scaling`` a frequency whose wavelength is longer than
    ``original / low`` is divided by ``factor``, one whose wavelength is shorter than ``original / high`` stays, and the ones
    between are blended linearly in ``original / wavelength``."""
    dims, base = rot["dims"], float(rot["base"])
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return freqs
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < sc["original"] / sc["high"]:
            out.append(f)
        elif wavelength > sc["original"] / sc["low"]:
            out.append(f / sc["factor"])
        else:
            s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * f / sc["factor"] + s * f)
    return out


def rotate_head(vec, position, rot):
    """One head ``[dim]``: channel i is paired with channel i + dims/2 for i < dims/2; the other channels pass."""
    dims = rot["dims"]
    freqs = rotary_frequencies(rot)
    out = vec.clone()
    for i in range(dims // 2):
        a = position * freqs[i]
        c, s = math.cos(a), math.sin(a)
        u, v = vec[i], vec[i + dims // 2]
        out[i] = u * c - v * s
        out[i + dims // 2] = v * c + u * s
    return out


# --------------------------------------------------------------------------------------------------------------- embedding
def embed_tokens(tokens, W, emb):
    """Scaled token rows plus a row of the bigram table chosen by (previous token, token); a sequence's first token takes the
    table's last row."""
    bg = emb["bigram"]
    rows = []
    for t, tok in enumerate(tokens):
        row = bg["buckets"] if t == 0 else (tokens[t - 1] * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"]
        rows.append(W["embed"][tok] * emb["scale"] + W["bigram"][row])
    return torch.stack(rows)


# ------------------------------------------------------------------------------------------------------------------ mixers
def sink_window_attention(h, W, p, m, window_shift=0, sink=1.0):
    """Grouped-query attention in a sliding window whose softmax has one more, value-less entry of score 0; values are the
    keys before rotation; scores pass through a tanh cap; the heads are gated channel by channel.  (``window_shift`` and ``sink``
    exist so that a test can show that a window that is one off, or a missing sink, would be noticed.)"""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    n = h.shape[0]
    keys, vals = [], []
    out = []
    for t in range(n):
        k = (W[p + "k"] @ h[t]).view(G, D)
        vals.append(k)
        keys.append(torch.stack([rotate_head(k[g], t, m["rot"]) for g in range(G)]))
        q = (W[p + "q"] @ h[t]).view(H, D)
        q = torch.stack([rotate_head(q[hh], t, m["rot"]) for hh in range(H)])
        seen = [j for j in range(t + 1) if t - j < m["mask"]["size"] + window_shift]
        heads = []
        for hh in range(H):
            g = hh // (H // G)
            s = torch.stack([(q[hh] * keys[j][g]).sum() * m["scale"] for j in seen])
            s = m["softcap"] * torch.tanh(s / m["softcap"])
            e = torch.exp(s)
            pr = e / (sink + e.sum())
            heads.append(sum(pj * vals[j][g] for pj, j in zip(pr, seen)))
        y = torch.cat(heads) * sigmoid(W[p + "g"] @ h[t])
        out.append(W[p + "o"] @ y)
    return torch.stack(out)


def decayed_outer_product_scan(qs, ks, vs, decays):
    """``S ← diag(decay_t) S + k_t v_tᵀ``, ``o_t = Sᵀ q_t`` for one head; ``decays[t]`` is a scalar or one number per key channel."""
    S = torch.zeros(ks[0].shape[0], vs[0].shape[0], dtype=F64)
    out = []
    for q, k, v, a in zip(qs, ks, vs, decays):
        a = a if torch.is_tensor(a) and a.dim() == 1 else torch.full((k.shape[0],), float(a), dtype=F64)
        S = a[:, None] * S + k[:, None] * v[None, :]
        out.append(S.t() @ q)
    return out


def gated_linear_attention(h, W, p, m, eps):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = [(W[p + "q"] @ h[t]).view(H, D) * D ** -0.5 for t in range(n)]
    k = [(W[p + "k"] @ h[t]).view(H, D) for t in range(n)]
    v = [(W[p + "v"] @ h[t]).view(H, V) for t in range(n)]
    alpha = [sigmoid(W[p + "a2"] @ (W[p + "a1"] @ h[t]) + W[p + "a2.b"]).pow(1.0 / m["tau"]).view(H, D) for t in range(n)]
    o = [decayed_outer_product_scan([x[hh] for x in q], [x[hh] for x in k], [x[hh] for x in v], [x[hh] for x in alpha])
         for hh in range(H)]
    out = []
    for t in range(n):
        y = torch.cat([rms_divide(o[hh][t], eps) * W[p + "norm"] for hh in range(H)]) * silu(W[p + "g"] @ h[t])
        out.append(W[p + "o"] @ y)
    return torch.stack(out)


def parallel_mixer(h, W, p, m, eps, **variant):
    left = sink_window_attention(h, W, p + "left.", m["left"], **variant)
    right = gated_linear_attention(h, W, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def retention_mixer(h, W, p, m, eps):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = [torch.stack([rotate_head(r, t, m["rot"]) for r in (W[p + "q"] @ h[t]).view(H, D)]) for t in range(n)]
    k = [torch.stack([rotate_head(r, t, m["rot"]) for r in (W[p + "k"] @ h[t]).view(H, D)]) * D ** -0.5 for t in range(n)]
    v = [(W[p + "v"] @ h[t]).view(H, V) for t in range(n)]
    o = [decayed_outer_product_scan([x[hh] for x in q], [x[hh] for x in k], [x[hh] for x in v], n * [m["decay"][hh]])
         for hh in range(H)]
    out = []
    for t in range(n):
        y = torch.cat([rms_divide(o[hh][t], eps) for hh in range(H)]) * silu(W[p + "g"] @ h[t])
        out.append(W[p + "o"] @ y)
    return torch.stack(out)


def lightning_mixer(h, W, p, m, eps):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = [silu(W[p + "q"] @ h[t]).view(H, D) for t in range(n)]
    k = [silu(W[p + "k"] @ h[t]).view(H, D) for t in range(n)]
    v = [silu(W[p + "v"] @ h[t]).view(H, V) for t in range(n)]
    o = [decayed_outer_product_scan([x[hh] for x in q], [x[hh] for x in k], [x[hh] for x in v], n * [m["decay"][hh]])
         for hh in range(H)]
    out = []
    for t in range(n):
        y = rms_divide(torch.cat([o[hh][t] for hh in range(H)]), eps) * W[p + "norm"] * sigmoid(W[p + "g"] @ h[t])
        out.append(W[p + "o"] @ y)
    return torch.stack(out)


def mixer(kind, h, W, p, m, eps, **variant):
    if kind == "parallel":
        return parallel_mixer(h, W, p, m, eps, **variant)
    if kind == "retention":
        return retention_mixer(h, W, p, m, eps)
    if kind == "lightning":
        return lightning_mixer(h, W, p, m, eps)
    raise ValueError(kind)


# ----------------------------------------------------------------------------------------------------------- feed-forwards
def gated_ff(v, gate, up, down, act):
    return down @ (act(gate @ v) * (up @ v))


def router_choice(v, W, p, r):
    """Chosen experts (largest logits first, ties to the lower index) and their weights: a softmax over the chosen logits."""
    z = W[p + "router"] @ v + W[p + "router.b"]
    order = sorted(range(r["experts"]), key=lambda e: (-float(z[e]), e))[: r["top"]]
    zs = torch.stack([z[e] for e in order])
    w = torch.exp(zs - zs.max())
    return order, w / w.sum()


def feed_forward(h, W, p, mlp):
    out = []
    for t in range(h.shape[0]):
        if mlp["kind"] == "dense":
            out.append(gated_ff(h[t], W[p + "gate"], W[p + "up"], W[p + "down"], gelu_tanh))
        else:
            order, w = router_choice(h[t], W, p, mlp["router"])
            out.append(sum(wk * gated_ff(h[t], W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"], W[f"{p}e{e}.down"], silu)
                           for wk, e in zip(w, order)))
    return torch.stack(out)


# ------------------------------------------------------------------------------------------------------------------- model
def norm_rows(x, w, eps):
    return torch.stack([rms_divide(r, eps) * w for r in x])


def hyper_sublayer(streams, W, p, q, fn, norm_w, eps):
    """One sublayer on several residual streams: read a weighted sum of them, then replace every stream by a mixture of the old
    streams plus its share of the sublayer's output."""
    n = len(streams)
    u = sum(W[f"{p}hc{q}.in"][s] * streams[s] for s in range(n))
    y = fn(norm_rows(u, norm_w, eps))
    return [sum(W[f"{p}hc{q}.mix"][s, t] * streams[s] for s in range(n)) + W[f"{p}hc{q}.out"][t] * y for t in range(n)]


def forward(cfg, W, tokens, taps=None, **variant):
    """Logits ``[n, vocab]`` of one sequence; ``taps`` (a list) receives the sum of the streams after every block."""
    W = as_f64(W)
    eps = cfg["norm"]["eps"]
    x = embed_tokens(tokens, W, cfg["embedding"])
    streams = [x.clone() for _ in range(cfg["streams"])]
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        streams = hyper_sublayer(streams, W, p, 1, lambda h: mixer(lc["type"], h, W, p + "mix.", lc["mixer"], eps, **variant),
                                 W[p + "norm1"], eps)
        if lc.get("mlp"):
            streams = hyper_sublayer(streams, W, p, 2, lambda h: feed_forward(h, W, p + "mlp.", lc["mlp"]), W[p + "norm2"], eps)
        if taps is not None:
            taps.append(sum(streams))
    return norm_rows(sum(streams), W["final.norm"], eps) @ W["head"].t()


def greedy(cfg, W, prompt, new_tokens):
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(cfg, W, seq)[-1].argmax()))
    return seq[len(prompt):]


# ---------------------------------------------------------------------------------------------------------- configurations
def rot_cfg(dims, base=10000.0, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling:
        out["scaling"] = scaling
    return out


def dense_cfg(ff=24):
    return {"kind": "dense", "ff": ff}


def moe_cfg(ff=8, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def left_cfg(heads=4, kv_heads=2, dim=8, window=5, rot=None, scale=0.4, softcap=6.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window},
            "rot": rot or rot_cfg(4, 100.0), "scale": scale, "softcap": softcap}


def right_cfg(heads=2, dim=6, vdim=4, tau=8.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def parallel_cfg(left=None, right=None, left_scale=0.7, right_scale=1.3, mlp=None):
    return {"type": "parallel", "mixer": {"left": left or left_cfg(), "right": right or right_cfg(), "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


def retention_cfg(heads=3, dim=8, vdim=4, decay=None, rot=None, mlp=None):
    decay = decay or [1.0 - 2.0 ** (-2 - i) for i in range(heads)]
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rot or rot_cfg(dim, 50.0)},
            "mlp": mlp}


def lightning_cfg(heads=2, dim=6, vdim=10, decay=None, mlp=None):
    decay = decay or [0.5 + 0.45 * i / max(heads - 1, 1) for i in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def model_cfg(layers, vocab=50, width=24, streams=2, eps=1e-5, scale=3.0, buckets=37, mul_prev=11, mul_cur=5):
    return {"architecture": "Salizen", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps},
            "embedding": {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
            "layers": layers}


def tensor_shapes(cfg, rank=3):
    """Name → shape of every checkpoint tensor of a configuration (``rank``: inner size of the decay logits' low-rank pair,
    which the configuration does not hold)."""
    n, s = cfg["width"], cfg["streams"]
    out = {"embed": (cfg["vocab"], n), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, n), "final.norm": (n,),
           "head": (cfg["vocab"], n)}
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        out[p + "norm1"] = (n,)
        for q in (1, 2) if lc.get("mlp") else (1,):
            out.update({f"{p}hc{q}.in": (s,), f"{p}hc{q}.out": (s,), f"{p}hc{q}.mix": (s, s)})
        if lc["type"] == "parallel":
            a, b = m["left"], m["right"]
            out.update({p + "mix.left.q": (a["heads"] * a["dim"], n), p + "mix.left.k": (a["kv_heads"] * a["dim"], n),
                        p + "mix.left.g": (a["heads"] * a["vdim"], n), p + "mix.left.o": (n, a["heads"] * a["vdim"])})
            out.update({p + "mix.right.q": (b["heads"] * b["dim"], n), p + "mix.right.k": (b["heads"] * b["dim"], n),
                        p + "mix.right.v": (b["heads"] * b["vdim"], n), p + "mix.right.g": (b["heads"] * b["vdim"], n),
                        p + "mix.right.o": (n, b["heads"] * b["vdim"]), p + "mix.right.norm": (b["vdim"],),
                        p + "mix.right.a1": (rank, n), p + "mix.right.a2": (b["heads"] * b["dim"], rank),
                        p + "mix.right.a2.b": (b["heads"] * b["dim"],)})
        else:
            out.update({p + "mix.q": (m["heads"] * m["dim"], n), p + "mix.k": (m["heads"] * m["dim"], n),
                        p + "mix.v": (m["heads"] * m["vdim"], n), p + "mix.g": (m["heads"] * m["vdim"], n),
                        p + "mix.o": (n, m["heads"] * m["vdim"])})
            if lc["type"] == "lightning":
                out[p + "mix.norm"] = (m["heads"] * m["vdim"],)
        mlp = lc.get("mlp")
        if mlp:
            out[p + "norm2"] = (n,)
            if mlp["kind"] == "dense":
                out.update({p + "mlp.gate": (mlp["ff"], n), p + "mlp.up": (mlp["ff"], n), p + "mlp.down": (n, mlp["ff"])})
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                out.update({p + "mlp.router": (E, n), p + "mlp.router.b": (E,)})
                for e in range(E):
                    out.update({f"{p}mlp.e{e}.gate": (ff, n), f"{p}mlp.e{e}.up": (ff, n), f"{p}mlp.e{e}.down": (n, ff)})
    return out


def random_weights(cfg, seed=0, rank=3):
    """Random tensors rounded to bfloat16 (what a checkpoint stores), as float32."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("a2.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif name.endswith("router.b"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif ".hc" in name:
            t = (torch.eye(shape[0]) if last == "mix" else torch.ones(shape) * (0.6 if last == "in" else 1.0)) \
                + 0.3 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = 0.3 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16).float()
    return out


def as_f64(weights):
    return {k: v.to(F64) for k, v in weights.items()}
