"""Plain, slow float64 implementation of the Lugizen design, one function per mechanism, written from the equations and
sharing no code with the product path. It takes the config.json dictionary and a {name: tensor} dict and processes a whole
sequence at once: no cache, no carried state, every row loops over the keys it sees and every recurrence over its tokens.

The design: x <- x + n1(mixer(x + canon(x))), then x <- x + n2(ff(x)), where n(y) = y / sqrt(mean(y^2) + eps) * g with ONE
number g per norm, canon is a short causal convolution over time on every channel of the residual stream, and the mixer is
one of: a gated delta rule with a decay per key channel ("channel_delta"), causal softmax attention with rotary positions,
unit-rms q and k, a temperature per head and values mixed with the first such layer's ("attention"), or sliding-window
attention over a low-rank latent with one shared rotary key part ("latent_attention"). The feed-forward is two matrices
around a gelu, or a mixture of gated silu experts whose weights are the softmax over the chosen router logits.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def scalar_norm(y, g, eps):
    """y / sqrt(mean(y^2) + eps) * g over the last axis; g is a single number."""
    return y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps) * g


def rms(y, eps):
    return y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def time_conv(x, w):
    """x [T, C], w [C, taps]: out[t] = sum_j w[:, j] * x[t - taps + 1 + j], zeros before the first row."""
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * x[s]
    return out


def rotate_half(x, dims, base, start=0):
    """x [T, heads, D]: channel i < dims/2 turns with channel i + dims/2 by (start + t) * base^(-2i/dims); the rest pass."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = torch.arange(start, start + x.shape[0], dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, window=0):
    """q [T, H, D] (each head's scale factors already applied), k [T, G, D], v [T, G, DV]: row i sees j <= i, and with a
    window only those with i - j < window; ordinary softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1) if window > 0 else 0
        for h in range(H):
            g = h // (H // G)
            w = torch.softmax((k[lo:i + 1, g] @ q[i, h]) * scale, 0)
            out[i, h] = w @ v[lo:i + 1, g]
    return out


def delta_rule(q, k, v, beta, decay):
    """One head. q, k [T, N], v [T, P], beta [T], decay [T, N] in (0, 1]: S <- diag(decay_t) S; u = beta_t (v_t - S^T k_t);
    S <- S + k_t u^T; o_t = S^T q_t (the read-out sees the token's own write). S starts at zero."""
    T, N = k.shape
    S = torch.zeros(N, v.shape[1], dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta_mixer(h, cfg, t, p, eps):
    H, G, N, P = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"]), int(cfg["vdim"])
    T = h.shape[0]
    q = silu(time_conv(h @ t[p + "q"].T, t[p + "q.conv"])).view(T, G, N)
    k = silu(time_conv(h @ t[p + "k"].T, t[p + "k.conv"])).view(T, G, N)
    v = silu(time_conv(h @ t[p + "v"].T, t[p + "v.conv"])).view(T, H, P)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * N ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ t[p + "b"].T)                                   # [T, H]
    step = torch.nn.functional.softplus((h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "dt_bias"]).view(T, H, N)
    decay = torch.exp(-torch.exp(t[p + "A_log"])[None, :, None] * step)      # [T, H, N]
    o = torch.zeros(T, H, P, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        o[:, hd] = delta_rule(q[:, g], k[:, g], v[:, hd], beta[:, hd], decay[:, hd])
    o = rms(o, eps) * t[p + "norm"]
    o = o.reshape(T, H * P) * torch.sigmoid((h @ t[p + "g1"].T) @ t[p + "g2"].T)
    return o @ t[p + "o"].T


def attention_values(h, cfg, t, p):
    return (h @ t[p + "v"].T).view(h.shape[0], int(cfg["kv_heads"]), int(cfg["vdim"]))


def attention_mixer(h, cfg, t, p, eps, v_first=None, start=0, use_temp=True):
    """Returns (output, this layer's values as projected). v_first: the values of the first value-mixing layer (None in
    that layer itself and in layers that do not mix)."""
    H, G, D = int(cfg["heads"]), int(cfg["kv_heads"]), int(cfg["dim"])
    T = h.shape[0]
    q = (h @ t[p + "q"].T).view(T, H, D)
    k = (h @ t[p + "k"].T).view(T, G, D)
    v = attention_values(h, cfg, t, p)
    own = v
    rot = cfg.get("rot") or {"dims": 0, "base": 1.0}
    q = rms(rotate_half(q, int(rot["dims"]), float(rot["base"]), start), eps)
    k = rms(rotate_half(k, int(rot["dims"]), float(rot["base"]), start), eps)
    if use_temp:
        q = q * t[p + "temp"].view(1, H, 1)
    if v_first is not None:
        lam = t[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    o = softmax_attention(q, k, v, float(cfg["scale"])).reshape(T, -1)
    return o @ t[p + "o"].T, own


def latent_attention_mixer(h, cfg, t, p, eps, start=0, window_off=False):
    H, D, DR, DV, R = int(cfg["heads"]), int(cfg["dim"]), int(cfg["rot_dim"]), int(cfg["vdim"]), int(cfg["kv_rank"])
    T = h.shape[0]
    base = float(cfg["rot"]["base"])
    cq = rms(h @ t[p + "dq"].T, eps) * t[p + "dq.norm"]
    q = (cq @ t[p + "uq"].T).view(T, H, D + DR)
    q_rot = rotate_half(q[..., D:], DR, base, start)
    ckv = h @ t[p + "dkv"].T
    c = rms(ckv[:, :R], eps) * t[p + "dkv.norm"]
    k_rot = rotate_half(ckv[:, R:].view(T, 1, DR), DR, base, start)
    k = torch.cat([(c @ t[p + "uk"].T).view(T, H, D), k_rot.expand(T, H, DR)], -1)
    v = (c @ t[p + "uv"].T).view(T, H, DV)
    qq = torch.cat([q[..., :D], q_rot], -1)
    o = softmax_attention(qq, k, v, float(cfg["scale"]), 0 if window_off else int(cfg["mask"]["size"])).reshape(T, -1)
    return o @ t[p + "o"].T


def dense_ff(h, t, p):
    return gelu_tanh(h @ t[p + "up"].T) @ t[p + "down"].T


def expert(h, t, p):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def route(h, mlp, t, p, equal_weights=False):
    """([T, top] chosen experts, [T, top] weights = softmax over the chosen logits only; equal_weights: 1 / top each instead,
    which is what the design does not do. A softmax over every logit would differ from the design's by one factor per row,
    which the norm behind the feed-forward removes again)."""
    z = h @ t[p + "router"].T
    top = torch.topk(z, int(mlp["router"]["top"]), -1)
    if equal_weights:
        return top.indices, torch.full_like(top.values, 1.0 / top.values.shape[-1])
    return top.indices, torch.softmax(top.values, -1)


def routed_ff(h, mlp, t, p, equal_weights=False):
    idx, w = route(h, mlp, t, p, equal_weights)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=F64)
    for r in range(h.shape[0]):
        for j, e in enumerate(idx[r].tolist()):
            out[r] += w[r, j] * expert(h[r:r + 1], t, f"{p}e{e}.")[0]
    return out


def forward(cfg, tensors, ids, layer_outputs=False, leave_out=()):
    """Logits [T, vocab] of one sequence (and, with layer_outputs, the residual stream after every layer). leave_out names
    mechanisms to drop ("canon", "vmix", "temp", "window", "router_weights"): tests use it to show that their weights would
    expose a product that dropped one."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][torch.as_tensor(ids, dtype=torch.long)]
    v_first, outs = None, []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = x + time_conv(x, t[p + "canon1"]) if (p + "canon1" in t and "canon" not in leave_out) else x
        mx = L["mixer"]
        if L["type"] == "channel_delta":
            y = channel_delta_mixer(h, mx, t, p + "mix.", eps)
        elif L["type"] == "attention":
            mixes = bool(mx.get("v_mix")) and "vmix" not in leave_out
            y, own = attention_mixer(h, mx, t, p + "mix.", eps, v_first if mixes else None, use_temp="temp" not in leave_out)
            if mixes and v_first is None:
                v_first = own
        elif L["type"] == "latent_attention":
            y = latent_attention_mixer(h, mx, t, p + "mix.", eps, window_off="window" in leave_out)
        else:
            raise NotImplementedError(L["type"])
        x = x + scalar_norm(y, t[p + "norm1"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            y = dense_ff(x, t, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(x, mlp, t, p + "mlp.", "router_weights" in leave_out)
            x = x + scalar_norm(y, t[p + "norm2"], eps)
        outs.append(x)
    logits = scalar_norm(x, t["final.norm"], eps) @ t["head"].T
    return (logits, torch.stack(outs)) if layer_outputs else logits


def greedy(cfg, tensors, prompt, n_new):
    """The n_new tokens that greedy decoding appends to the prompt (the whole sequence is recomputed for every token)."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(forward(cfg, tensors, ids)[-1].argmax()))
    return ids[len(prompt):]
