"""Plain, slow implementation of the Fotulix decoder: whole sequences, no cache, no state carried between calls.

One function per mechanism, plain tensor arithmetic on the CPU (float64 unless told otherwise). It shares no code
with ``spissa_b200``: it reads config.json keys and a dict of tensors by their checkpoint names. Notation: x is the
residual stream [T, W], r the residual multiplier, n(·; w) an RMS norm whose weight is stored around zero.

    embedding       x_t = s · E[id_t] + B[(id_{t−1} · a + id_t · b) mod n]        (t = 0: the table's last row)
    norm            n(x; w) = x / sqrt(mean(x²) + eps) ⊙ (1 + w)
    layer           x ← x + r · n(mixer(n(x; w1)); w1b);   x ← x + r · n(ff(n(x; w2)); w2b);
                    y = P (gelu(G x) ⊙ S[id_t, layer's part]);   x ← x + r · y / rms(y) ⊙ w_s
    attention       biased q, k, v; q_t grows with ln of its position; a learned bias per (log-bucketed distance, head)
    attention_2     rotation of neighbouring pairs with the frequencies rescaled by bands of wavelength; a sink
    latent attn.    keys and values are images of a cached normed low-rank row, plus one rotated key part shared by
                    all heads; interpolated frequencies with a ramp; a sliding window; may read another layer's rows
    every mixer     head h's output times sigmoid of one number per head, a projection of the mixer's input
    feed-forward    SwiGLU
    head            logits = n(x; w_f) · Hᵀ
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(ids, w, emb: dict):
    """Token row times the scale, plus a row of the pair table chosen by the token and the one before it."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    x = w["embed"][ids] * emb["scale"]
    bg = emb.get("bigram")
    if bg:
        n = bg["buckets"]
        rows = torch.full_like(ids, n)
        rows[1:] = (ids[:-1] * bg["mul_prev"] + ids[1:] * bg["mul_cur"]) % n
        x = x + w["bigram"][rows]
    return x


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a distance-bias table with ``rows`` rows: distances below rows/2 have a row each, the others share
    rows on a logarithmic scale that reaches the last row at distance ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def rotate_pairs(v, freq, mult: float = 1.0):
    """v [T, heads, dims]: dim 2i pairs with 2i+1, turned by t · freq[i]; cos and sin times ``mult``."""
    T = v.shape[0]
    ang = torch.arange(T, dtype=v.dtype)[:, None] * freq.to(v.dtype)[None, :]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    a, b = v[..., 0::2], v[..., 1::2]
    out = torch.empty_like(v)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = b * c + a * s
    return out


def banded_frequencies(rot: dict):
    """base^(−2i/dims), rescaled by wavelength: short waves kept, long ones divided by the factor, a blend between."""
    dims = rot["dims"]
    f = [rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float64)


def ramped_frequencies(rot: dict):
    """(frequencies, multiplier of cos and sin): pairs below ``lo`` keep their frequency, pairs above ``hi`` have it
    divided by the factor, a linear ramp between; lo and hi are the pairs that turn ``fast`` and ``slow`` times over
    the original length."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=torch.float64), 1.0

    def pair_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(sc["factor"]) + 1.0


def softmax_mix(s, v, window=None, sink=None):
    """s [H, T, T] scores (scaled, biased), v [T, H, vd]. Query i sees j <= i, and with a window only i − j < window;
    ``sink`` [H] joins every row's denominator once with no value."""
    T = s.shape[-1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    s = s.masked_fill(~seen, -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return torch.einsum("hij,jhv->ihv", e / den, v)


def head_gate(o, a, w, p):
    """o [T, H, vd] times sigmoid(G a) [T, H]."""
    return o * torch.sigmoid(a @ w[p + "g"].T)[:, :, None]


def biased_attention(a, w, p, m):
    """Mixer 'attention'."""
    T = a.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (a @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (a @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, vd)
    qt = m.get("q_temp")
    if qt:
        pos = torch.arange(T)
        temp = 1.0 + qt["coef"] * torch.log(torch.floor((pos + 1) / qt["every"]).to(a.dtype) + 1.0)
        q = q * temp[:, None, None]
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    rel = w[p + "rel"]
    rows = torch.tensor([[distance_bucket(i - j, rel.shape[0], m["bias_max"]) if j <= i else 0 for j in range(T)]
                         for i in range(T)], dtype=torch.long)
    s = s + rel[rows].permute(2, 0, 1)
    o = head_gate(softmax_mix(s, v), a, w, p)
    return o.reshape(T, -1) @ w[p + "o"].T


def sink_attention(a, w, p, m):
    """Mixer 'attention_2'."""
    T = a.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T).reshape(T, H, d)
    k = (a @ w[p + "k"].T).reshape(T, G, d)
    v = (a @ w[p + "v"].T).reshape(T, G, vd)
    rot = m.get("rot")
    if rot:
        f, r = banded_frequencies(rot), rot["dims"]
        q = torch.cat([rotate_pairs(q[..., :r], f), q[..., r:]], dim=-1)
        k = torch.cat([rotate_pairs(k[..., :r], f), k[..., r:]], dim=-1)
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    o = head_gate(softmax_mix(s, v, sink=w[p + "sink"].to(a.dtype)), a, w, p)
    return o.reshape(T, -1) @ w[p + "o"].T


def latent_rows(a, w, p, m, eps):
    """What a latent attention caches per token: the normed low-rank row c [T, rank] and the rotated shared key part
    [T, rot_dim]."""
    T, r = a.shape[0], m["kv_rank"]
    d = a @ w[p + "dkv"].T
    c = rms_unit(d[:, :r], eps) * w[p + "dkv.norm"]
    f, mult = ramped_frequencies(m["rot"])
    kr = rotate_pairs(d[:, None, r:], f, mult)[:, 0]
    return c, kr


def latent_attention(a, w, p, m, rows):
    """Mixer 'latent_attention'; ``rows`` = (c, rotated key part) that it reads (its own, or another layer's)."""
    T = a.shape[0]
    H, d, rd, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = rows
    q = (a @ w[p + "q"].T).reshape(T, H, d + rd)
    f, mult = ramped_frequencies(m["rot"])
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], f, mult)
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, vd)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k) + torch.einsum("ihd,jd->hij", q_rot, kr)) * m["scale"]
    mask = m.get("mask")
    o = head_gate(softmax_mix(s, v, window=mask["size"] if mask else None), a, w, p)
    return o.reshape(T, -1) @ w[p + "o"].T


def swiglu(a, w, p):
    return (silu(a @ w[p + "gate"].T) * (a @ w[p + "up"].T)) @ w[p + "down"].T


def token_side(x, ids, w, p, layer: int, dim: int, eps):
    """The per-layer token input: a table row's part for this layer, gated by a projection of the stream, projected
    back and divided by its root mean square, with a plain weight."""
    e = w["side.embed"][torch.as_tensor(ids, dtype=torch.long)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms_unit(y, eps) * w[p + "norm"]


def forward(cfg: dict, weights: dict, ids, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one sequence; ``layers_out`` collects the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, r = cfg["norm"]["eps"], cfg["residual_mult"]
    side = cfg.get("token_side")
    x = embed(ids, w, cfg["embedding"])
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        a = norm_around_zero(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = biased_attention(a, w, p + "mix.", m)
        elif layer["type"] == "attention_2":
            y = sink_attention(a, w, p + "mix.", m)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                cached[i] = latent_rows(a, w, p + "mix.", m, eps)
                src = i
            y = latent_attention(a, w, p + "mix.", m, cached[src])
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + r * norm_around_zero(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = swiglu(norm_around_zero(x, w[p + "norm2"], eps), w, p + "mlp.")
            x = x + r * norm_around_zero(y, w[p + "norm2b"], eps)
        if side:
            x = x + r * token_side(x, ids, w, p + "side.", i, side["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T


def generate_greedy(cfg, weights, prompt, n_new: int) -> list:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, weights, ids)[-1])))
    return ids[len(prompt):]
