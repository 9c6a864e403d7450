"""A plain float64 implementation of Zubarax, one function per mechanism, written from the model's equations only: whole
sequences at once, no cache, no batching, no code shared with the framework.  The tests compare the framework with it.

Notation: ``x`` ``[n, width]`` is the residual of one sequence, ``W`` the dictionary of checkpoint tensors (float64), ``p`` a tensor
name prefix, ``m`` the part of the configuration that describes the mechanism."""
import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------------------------- helpers
def unit_rms(t, eps):
    return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)


def centred_norm(t, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return unit_rms(t, eps) * (1.0 + w)


def causal_conv(u, w):
    """``u`` ``[n, C]``, ``w`` ``[C, taps]``: out[t] = Σ_j w[:, j] u[t − (taps − 1) + j], zeros before the start."""
    n, taps = u.shape[0], w.shape[1]
    out = torch.zeros_like(u)
    for t in range(n):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def rotate(t, positions, dims, base):
    """``t`` ``[n, heads, D]``: channel i < dims/2 pairs with channel i + dims/2."""
    if not dims:
        return t
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = torch.tensor(positions, dtype=F64)[:, None] * f[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = t[..., :half], t[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, t[..., dims:]], -1)


# ----------------------------------------------------------------------------------------------------------------- mixers
def attention_inputs(x, W, p, m, eps):
    """Prepared queries ``[n, H, D]``, keys ``[n, G, D]`` and values ``[n, G, V]`` of the softmax side."""
    n = x.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(x @ W[p + "q"].T, W[p + "q.conv"]).view(n, H, D)
    k = causal_conv(x @ W[p + "k"].T, W[p + "k.conv"]).view(n, G, D)
    v = causal_conv(x @ W[p + "v"].T, W[p + "v.conv"]).view(n, G, V)
    rot = m.get("rot") or {}
    pos = list(range(n))
    q = rotate(unit_rms(q, eps) * W[p + "q.norm"], pos, rot.get("dims", 0), rot.get("base", 10000.0))
    k = rotate(unit_rms(k, eps) * W[p + "k.norm"], pos, rot.get("dims", 0), rot.get("base", 10000.0))
    return q, k, unit_rms(v, eps)


def softmax_side(x, W, p, m, eps):
    n = x.shape[0]
    H, G, V = m["heads"], m["kv_heads"], m["vdim"]
    q, k, v = attention_inputs(x, W, p, m, eps)
    out = torch.zeros(n, H, V, dtype=F64)
    for i in range(n):
        raw = torch.stack([(k[: i + 1, h // (H // G)] @ q[i, h]) * m["scale"] for h in range(H)])      # [H, i + 1]
        mixed = W[p + "talk"] @ raw
        for h in range(H):
            e = torch.exp(mixed[h] - mixed[h].max())
            denom = e.sum() + math.exp(float(W[p + "sink"][h]) - float(mixed[h].max()))
            out[i, h] = (e / denom) @ v[: i + 1, h // (H // G)]
    return out.reshape(n, H * V) @ W[p + "o"].T


def recurrent_side(x, W, p, m, eps):
    n = x.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(x @ W[p + "q"].T).view(n, H, D)
    v = (x @ W[p + "v"].T).view(n, H, V)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(x @ W[p + "f"].T + W[p + "f.b"])).view(n, H, D)
    S = torch.zeros(H, D, V, dtype=F64)
    out = torch.zeros(n, H, V, dtype=F64)
    for t in range(n):
        for h in range(H):
            S[h] = f[t, h][:, None] * S[h] + torch.outer(1.0 - f[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    out = unit_rms(out, eps) * W[p + "norm"]
    return out.reshape(n, H * V) @ W[p + "o"].T


def mixer(x, W, p, m, eps):
    return m["left_scale"] * softmax_side(x, W, p + "left.", m["left"], eps) + m["right_scale"] * recurrent_side(x, W, p + "right.", m["right"], eps)


# ----------------------------------------------------------------------------------------------------------- feed-forward
def clamped_expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def router(x, W, p, m):
    """Chosen experts and their scores, ``[n, top]`` each."""
    s = torch.sigmoid(x @ W[p + "router"].T)
    return s.topk(m["router"]["top"], -1)


def feed_forward(x, W, p, m):
    scores, chosen = router(x, W, p, m)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for s, e in zip(scores[t], chosen[t]):
            out[t] += clamped_expert(s * x[t], W, f"{p}e{int(e)}.", m["expert"]["limit"])
    if m.get("shared"):
        out = out + clamped_expert(x, W, p + "shared.", m["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------------------------------------------ model
def owner(cfg, i):
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def forward(cfg, W, tokens, residuals=None):
    """Logits ``[n, vocab]`` of one sequence; ``residuals`` collects the residual after every entry of ``layers``."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{owner(cfg, i)}."
        x = centred_norm(alpha * x + mixer(x, W, p + "mix.", lc["mixer"], eps), W[p + "norm1"], eps)
        if lc.get("mlp"):
            x = centred_norm(alpha * x + feed_forward(x, W, p + "mlp.", lc["mlp"]), W[p + "norm2"], eps)
        elif p + "norm2" in W:                                 # a second norm without a feed-forward norms alpha · x alone
            x = centred_norm(alpha * x, W[p + "norm2"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return centred_norm(x, W["final.norm"], eps) @ W["embed"].T


def greedy(cfg, W, prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(forward(cfg, W, seq)[-1].argmax())
        seq.append(tok)
        out.append(tok)
    return out


# ---------------------------------------------------------------------------------------------------------------- weights
def side_cfgs(heads=2, kv_heads=1, dim=8, vdim=8, conv=3, rot_dims=4, rot_base=100.0, rheads=2, rdim=4, rvdim=8, left_scale=0.7,
              right_scale=1.2):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, scale=dim ** -0.5, rot=dict(dims=rot_dims, base=rot_base))
    return dict(left=left, right=dict(heads=rheads, dim=rdim, vdim=rvdim), left_scale=left_scale, right_scale=right_scale)


def moe_cfg(ff=8, experts=4, top=2, limit=2.0, shared_ff=12, shared_limit=1.0):
    out = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))
    if shared_ff:
        out["shared"] = dict(ff=shared_ff, limit=shared_limit)
    return out


def layer(mixer_cfg=None, mlp=None, weights_of=None):
    out = dict(type="parallel", mixer=mixer_cfg or side_cfgs(), mlp=mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def model_cfg(layers, vocab=50, width=16, alpha=1.5, scale=3.0, eps=1e-5):
    return dict(architecture="Zubarax", vocab=vocab, width=width, postln_alpha=alpha, embedding=dict(scale=scale), norm=dict(eps=eps),
                layers=layers)


def random_weights(cfg, seed=0):
    """Checkpoint tensors with bf16-exact values (float64), so that saving them as bf16 loses nothing."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * std + mean).to(torch.bfloat16).to(F64)

    n = cfg["width"]
    W = {"embed": rnd(cfg["vocab"], n, std=0.5), "final.norm": rnd(n, std=0.2)}
    for i, lc in enumerate(cfg["layers"]):
        if lc.get("weights_of") is not None:
            continue
        p = f"l{i}."
        W[p + "norm1"] = rnd(n, std=0.2)
        a, b = lc["mixer"]["left"], lc["mixer"]["right"]
        H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        lp = p + "mix.left."
        for name, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
            W[lp + name] = rnd(rows, n, std=n ** -0.5)
            W[lp + name + ".conv"] = rnd(rows, a["conv"], std=0.6)
        W[lp + "q.norm"], W[lp + "k.norm"] = rnd(D, std=0.3, mean=1.0), rnd(D, std=0.3, mean=1.0)
        W[lp + "talk"] = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).to(torch.bfloat16).to(F64)
        W[lp + "sink"] = rnd(H, std=1.0)
        W[lp + "o"] = rnd(n, H * V, std=(H * V) ** -0.5)
        rp = p + "mix.right."
        Hr, Dr, Vr = b["heads"], b["dim"], b["vdim"]
        W[rp + "q"], W[rp + "f"], W[rp + "v"] = rnd(Hr * Dr, n, std=n ** -0.5), rnd(Hr * Dr, n, std=n ** -0.5), rnd(Hr * Vr, n, std=n ** -0.5)
        W[rp + "f.b"] = rnd(Hr * Dr, std=1.0, mean=1.0)
        W[rp + "lower"] = torch.rand(Hr * Dr, generator=g).mul(0.9).to(torch.bfloat16).to(F64)
        W[rp + "norm"] = rnd(Vr, std=0.3, mean=1.0)
        W[rp + "o"] = rnd(n, Hr * Vr, std=(Hr * Vr) ** -0.5)
        if lc.get("mlp"):
            mc = lc["mlp"]
            mp = p + "mlp."
            W[p + "norm2"] = rnd(n, std=0.2)
            W[mp + "router"] = rnd(mc["router"]["experts"], n, std=1.0)
            names = [f"e{e}." for e in range(mc["router"]["experts"])]
            sizes = [mc["expert"]["ff"]] * len(names)
            if mc.get("shared"):
                names.append("shared.")
                sizes.append(mc["shared"]["ff"])
            for name, ff in zip(names, sizes):
                W[mp + name + "gate"], W[mp + name + "up"] = rnd(ff, n, std=2.0 * n ** -0.5), rnd(ff, n, std=2.0 * n ** -0.5)
                W[mp + name + "down"] = rnd(n, ff, std=ff ** -0.5)
    return W
