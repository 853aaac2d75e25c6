"""Plain, slow float64 implementation of the Dibedra design (parallel blocks behind one Dynamic-Tanh norm, sliding-window
attention whose values are the un-normed keys, dense or routed feed-forward with identity experts), one function per
mechanism, written from the equations and sharing no code with the product path. It takes the config.json dictionary and a
{name: tensor} dict and processes a whole sequence at once: no cache, every row loops over the keys it sees.

Notation: h [T, width] is the block's normed input; rms(x) = x / sqrt(mean(x^2) + eps) over the last axis.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def dyt(x, w, b, alpha):
    """Dynamic Tanh: no statistics of the row enter."""
    return torch.tanh(alpha * x) * w + b


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def pair_frequencies(rot):
    """Frequency of every rotated pair and the factor on cos / sin (long-context interpolation when `scaling` is there)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor = float(sc["factor"])

    def where(turns):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, rot, start=0):
    """x [T, heads, D]: channels (2i, 2i+1), i < dims/2, turn by (start + t) * f_i; the other channels pass."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    f, mag = pair_frequencies(rot)
    p = torch.arange(start, start + x.shape[0], dtype=F64)
    ang = p[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def window_attention(q, k, v, scale, window):
    """q [T, H, D], k [T, G, D], v [T, G, DV]: row i sees rows j with 0 <= i - j < window; ordinary softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            w = torch.softmax(s, 0)
            out[i, h] = w @ v[lo:i + 1, g]
    return out


def attention_mixer(h, cfg, t, p, eps, start=0, window_off=False):
    """Gated sliding-window attention whose values are the keys as projected (before norm and rotation)."""
    H, G, D = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"])
    T = h.shape[0]
    q = (h @ t[p + "q"].T).view(T, H, D)
    k = (h @ t[p + "k"].T).view(T, G, D)
    v = k.clone()
    q = rms(q, eps) * t[p + "q.norm"]
    k = rms(k, eps) * t[p + "k.norm"]
    q, k = rotate_pairs(q, cfg["rot"], start), rotate_pairs(k, cfg["rot"], start)
    window = T + start + 1 if window_off else int(cfg["mask"]["size"])
    o = window_attention(q, k, v, float(cfg["scale"]), window).reshape(T, -1)
    o = o * torch.sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def dense_ff(h, t, p):
    return gelu_tanh(h @ t[p + "up"].T) @ t[p + "down"].T


def expert(h, t, p, limit):
    g = torch.clamp(h @ t[p + "gate"].T, max=limit)
    u = torch.clamp(h @ t[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[p + "down"].T


def route(h, mlp, t, p, use_correction=True, use_groups=True):
    """Chosen router outputs and their weights per row: ([T, top] indices, [T, top] weights)."""
    r = mlp["router"]
    n = int(r["experts"]) + int(r.get("identity", 0))
    top = int(r["top"])
    s = torch.softmax(h @ t[p + "router"].T, -1)
    choice = s + t[p + "correction"] if use_correction else s.clone()
    gr = r.get("groups")
    if gr and use_groups:
        count, keep = int(gr["count"]), int(gr["keep"])
        per = n // count
        best = choice.view(-1, count, per).max(-1).values
        kept = torch.topk(best, keep, -1).indices
        allow = torch.zeros(h.shape[0], count, dtype=torch.bool)
        allow.scatter_(1, kept, True)
        choice = torch.where(allow[:, :, None].expand(-1, -1, per).reshape(-1, n), choice, torch.full_like(choice, -math.inf))
    idx = torch.topk(choice, top, -1).indices
    return idx, torch.gather(s, 1, idx)


def routed_ff(h, mlp, t, p, **kw):
    """Weighted sum of the chosen experts; the last `identity` router outputs stand for experts that return h."""
    E = int(mlp["router"]["experts"])
    limit = float(mlp["expert"]["limit"])
    idx, w = route(h, mlp, t, p, **kw)
    out = torch.zeros_like(h)
    for r in range(h.shape[0]):
        for e, wt in zip(idx[r].tolist(), w[r]):
            out[r] += wt * (h[r] if e >= E else expert(h[r:r + 1], t, f"{p}e{e}.", limit)[0])
    return out


def forward(config, tensors, ids, layer_dump=False, **kw):
    """Logits [T, vocab] (and the residual stream after every layer [layers, T, width])."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = t["embed"][torch.tensor(ids, dtype=torch.long)]
    dump = []
    for i, L in enumerate(config["layers"]):
        p = f"l{L.get('weights_of', i)}."
        h = dyt(x, t[p + "norm1"], t[p + "norm1.b"], t[p + "norm1.alpha"])
        y = attention_mixer(h, L["mixer"], t, p + "mix.", eps, window_off=kw.get("window_off", False))
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "dense") == "dense":
                y = y + dense_ff(h, t, p + "mlp.")
            else:
                y = y + routed_ff(h, mlp, t, p + "mlp.", **{k: v for k, v in kw.items() if k in ("use_correction", "use_groups")})
        x = x + y
        dump.append(x.clone())
    h = dyt(x, t["final.norm"], t["final.norm.b"], t["final.norm.alpha"])
    logits = (h @ t["head"].T) * float(config.get("logit_scale", 1.0))
    return (logits, torch.stack(dump)) if layer_dump else logits


def greedy(config, tensors, prompt, n):
    """n greedy tokens after `prompt` (the whole sequence is recomputed for every token)."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(config, tensors, seq)[-1].argmax()))
    return seq[len(prompt):]
