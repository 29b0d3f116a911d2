"""Plain, slow implementation of the Kugirax decoder: whole sequences, no cache, no state carried between calls.

One function per mechanism, plain tensor arithmetic on the CPU (float64 unless told otherwise). It shares no code
with ``spissa_b200``: it reads config.json keys and a dict of tensors by their checkpoint names. Notation: x is the
residual stream [T, W], a = n(x) what both sublayers of a layer read.

    layer           a = n(x);  x ← x + mixer(a) + ff(a)                     (one norm, two readers)
    rms norm        n(x) = x / sqrt(mean(x²) + eps) ⊙ w
    attention       q, k through a short causal convolution; the values ARE the convolved keys (before rotation);
                    rotation of dim i with dim i + r/2; p_j = e^{s_j} / (1 + Σ e^{s_j}) over all earlier keys
    latent attn.    c_q = n(D_q a), q = U_q c_q;  c = n(D_kv a) (or another layer's c);  k = U_k c, v = U_v c;
                    window; p_j = e^{s_j} / (e^{sink_h} + Σ e^{s_j})
    feed-forward    dense SwiGLU, or routed SwiGLU experts (softmax router) plus a gated shared expert
    head            logits = cap · tanh(n_f(x) · Hᵀ / cap)
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: y_t = Σ_j w[:, j] ⊙ u_{t − taps + 1 + j}, zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * taps_w[:, j]
    return y


def rotate_half(v, dims: int, base: float):
    """v [T, heads, dim]: dim i pairs with dim i + dims/2 (i < dims/2), turned by t · base^(−2i/dims)."""
    if dims <= 0:
        return v
    T, half = v.shape[0], dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    ang = torch.arange(T, dtype=v.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = v.clone()
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def sink_softmax_mix(q, k, v, scale, window, sink):
    """q [T, H, d], k [T, H, d], v [T, H, vd] (kv heads already spread over the query heads); ``sink`` [H]: a score
    that joins every row's denominator once and carries no value. Query i sees j with 0 <= i − j < window (None:
    every j <= i). Returns [T, H, vd]."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    s = s.masked_fill(~seen, -math.inf)
    m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    p = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - m))
    return torch.einsum("hij,jhv->ihv", p, v)


def conv_attention(a, w, p, m):
    """Mixer 'attention'. ``p`` the tensors' prefix ('l3.mix.'), ``m`` the mixer's config dict."""
    T = a.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q, k = a @ w[p + "q"].T, a @ w[p + "k"].T
    if m.get("conv"):
        q, k = short_conv(q, w[p + "q.conv"]), short_conv(k, w[p + "k.conv"])
    q, k = q.reshape(T, H, d), k.reshape(T, G, d)
    v = k                                                    # the values: the keys as they leave the convolution
    rot = m.get("rot")
    if rot:
        q, k = rotate_half(q, rot["dims"], rot["base"]), rotate_half(k, rot["dims"], rot["base"])
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    mask = m.get("mask")
    o = sink_softmax_mix(q, k, v, m["scale"], mask["size"] if mask else None, torch.zeros(H, dtype=a.dtype))
    return o.reshape(T, -1) @ w[p + "o"].T


def latent(a, w, p, eps):
    """The normed low-rank row that a latent attention caches."""
    return rms_norm(a @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)


def latent_attention(a, w, p, m, eps, c):
    """Mixer 'latent_attention'; ``c`` [T, kv_rank] is the latent it reads (its own, or another layer's)."""
    T = a.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(a @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d)
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, vd)
    mask = m.get("mask")
    o = sink_softmax_mix(q, k, v, m["scale"], mask["size"] if mask else None, w[p + "sink"].to(a.dtype))
    return o.reshape(T, -1) @ w[p + "o"].T


def swiglu(a, w, p):
    return (silu(a @ w[p + "gate"].T) * (a @ w[p + "up"].T)) @ w[p + "down"].T


def route(a, w, p, router):
    """Chosen experts [T, top] and their weights [T, top]."""
    s = torch.softmax(a @ w[p + "router"].T, dim=-1)
    top = torch.topk(s, router["top"], dim=-1)
    wt = top.values / (top.values.sum(dim=-1, keepdim=True) + 1e-20) * router["scale"]
    return top.indices, wt


def moe_ff(a, w, p, mlp):
    ids, wt = route(a, w, p, mlp["router"])
    y = torch.zeros_like(a)
    for t in range(a.shape[0]):
        for e, g in zip(ids[t].tolist(), wt[t]):
            y[t] = y[t] + g * swiglu(a[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        y = y + torch.sigmoid(a @ w[p + "shared.sg"].T) * swiglu(a, w, p + "shared.")
    return y


def feed_forward(a, w, p, mlp):
    if mlp is None:
        return torch.zeros_like(a)
    return swiglu(a, w, p) if mlp["kind"] == "dense" else moe_ff(a, w, p, mlp)


def forward(cfg: dict, weights: dict, ids, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one sequence; ``layers_out`` collects the residual stream after every layer."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        a = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = conv_attention(a, w, p + "mix.", m)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent(a, w, p + "mix.", eps)
                src = i
            y = latent_attention(a, w, p + "mix.", m, eps, latents[src])
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + (y + feed_forward(a, w, p + "mlp.", layer.get("mlp")))
        if layers_out is not None:
            layers_out.append(x.clone())
    cap = cfg.get("logit_softcap")
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def generate_greedy(cfg, weights, prompt, n_new: int) -> list:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, weights, ids)[-1])))
    return ids[len(prompt):]
