"""Small Fotulix configurations with random weights for tests, and models whose weights make one token stand out."""
import math
import os

import torch

from plain.llama_plain import read_model_folder


def biased(heads, kv, dim, vdim=None, scale=None, q_temp=None, far=None, rows=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim or dim, scale=scale or 1.0 / math.sqrt(dim))
    if q_temp:
        m["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    if far:
        m["bias_max"] = far
        m["bias_rows"] = rows
    return m


def turned(heads, kv, dim, vdim=None, rot=None, base=10000.0, scaling=None, scale=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim or dim, scale=scale or 1.0 / math.sqrt(dim))
    if rot:
        m["rot"] = dict(dims=rot, base=base)
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def through_rows(heads, dim, rot_dim, vdim, rank, window, base=10000.0, scaling=None, kv_from=None, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale or 1.0 / math.sqrt(dim + rot_dim),
             rot=dict(dims=rot_dim, base=base))
    if window:
        m["mask"] = dict(size=window)
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(kind, mixer, ff=None):
    return dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=ff) if ff else None)


def model(width, vocab, layers, mult=0.5, emb_scale=1.0, bigram=None, side=None, eps=1e-5):
    emb = dict(scale=emb_scale)
    if bigram:
        emb["bigram"] = dict(buckets=bigram[0], mul_prev=bigram[1], mul_cur=bigram[2])
    out = dict(architecture="Fotulix", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, embedding=emb,
               layers=layers)
    if side:
        out["token_side"] = dict(dim=side)
    return out


RAMP = (4.0, 16, 8.0, 1.0)         # factor, original length, turns of the fast and of the slow edge
BANDS = (4.0, 1.0, 4.0, 16)        # factor, low, high, original length

# sizes that differ from one another everywhere: grouped, multi-head and single-kv-head attention; key and value sizes
# equal or not; distance tables of 6 to 32 rows; query factors with a period of 1, 7, 16 or none; rotation over a part
# of a head, all of it or none, with and without rescaled frequencies; cached rows whose size the tensor-core kernels
# take (128, 256) and sizes they do not; windows of one token, below a page, above one and above two; readers of another
# layer's rows with a smaller and with a larger window than the writer's; layers without a feed-forward; with and without
# the pair table (also one of a single bucket) and the token side input; multipliers of 1, 0.5 and 0.25
CONFIGS = {
    "a": model(64, 200, [layer("latent_attention", through_rows(3, 8, 4, 12, 20, 9, base=100.0, scaling=RAMP), 56),
                         layer("attention", biased(4, 2, 16, q_temp=(0.35, 16), far=40, rows=12), 48),
                         layer("latent_attention", through_rows(2, 16, 4, 4, 20, 70, base=100.0, scaling=RAMP, kv_from=0)),
                         layer("attention_2", turned(3, 3, 8, rot=4, base=50.0, scaling=BANDS)),
                         layer("attention", biased(2, 1, 10, vdim=6, far=20, rows=8), 40)],
               mult=0.5, emb_scale=8.0, bigram=(37, 5, 3), side=6, eps=1e-4),
    "b": model(128, 333, [layer("attention_2", turned(4, 1, 32, rot=32), 96),
                          layer("latent_attention", through_rows(5, 16, 16, 32, 112, 100), 64),
                          layer("attention", biased(4, 2, 64, q_temp=(0.5, 1), far=300, rows=32)),
                          layer("latent_attention", through_rows(2, 32, 16, 16, 112, 33, kv_from=1), 32),
                          layer("attention_2", turned(2, 2, 64, rot=16, base=500.0, scaling=(8.0, 1.0, 2.0, 32)), 64)],
               mult=1.0, emb_scale=1.0, bigram=(1, 7, 11)),
    # nothing a multiple of four: the paths without wide accesses; a window of one token sees the token itself only
    "c": model(50, 97, [layer("attention", biased(3, 1, 10, vdim=7, q_temp=(0.2, 7), far=33, rows=6), 30),
                        layer("latent_attention", through_rows(2, 5, 6, 7, 11, 1, base=30.0), 22),
                        layer("attention_2", turned(1, 1, 6, rot=2, base=9.0)),
                        layer("latent_attention", through_rows(1, 6, 6, 3, 11, 130, base=30.0, kv_from=1), 14)],
               mult=0.25, emb_scale=3.0, side=5, eps=1e-3),
    "d": model(96, 150, [layer("latent_attention", through_rows(2, 24, 8, 24, 40, 65, scaling=(2.0, 64, 4.0, 2.0))),
                         layer("latent_attention", through_rows(3, 8, 8, 16, 248, 140), 64),
                         layer("attention", biased(6, 3, 16, q_temp=(1.0, 40), far=64.5, rows=16), 64),
                         layer("attention_2", turned(6, 2, 48, vdim=32, rot=32, base=1000.0), 40)],
               mult=0.5, emb_scale=2.0, bigram=(61, 1, 1), side=8),
}
INIT = {"a": dict(seed=5, std=0.1), "b": dict(seed=9, std=0.07), "c": dict(seed=13, std=0.12), "d": dict(seed=17, std=0.09)}


def make(cfg, folder, seed, std, patch=None):
    """A model folder from the library's random-weights mode, with the tensors that it draws too tamely spread out."""
    from spissa_b200.config import config_from_dict
    from spissa_b200.weights import write_random_model, write_safetensors
    write_random_model(config_from_dict(cfg), folder, seed=seed, std=std, norm_std=0.1)
    pcfg, w = read_model_folder(folder)
    g = torch.Generator().manual_seed(seed)
    for name in sorted(w):
        last = name.split(".")[-1]
        if last in ("sink", "rel"):                  # so that a sink left out or scaled, or a wrong row of the table, shows
            w[name] = (1.5 * torch.randn(w[name].shape, generator=g)).to(w[name].dtype)
        elif last == "g" or name.endswith("side.gate"):
            w[name] = (6.0 * w[name].float()).to(w[name].dtype)
        elif last == "b" or name.startswith("bigram") or name.startswith("side.embed"):
            w[name] = (0.5 * torch.randn(w[name].shape, generator=g)).to(w[name].dtype)
        elif "norm" in last:                         # stored around zero (or around one): visibly away from it
            w[name] = (w[name].float() + 0.3 * torch.randn(w[name].shape, generator=g)).to(w[name].dtype)
    if patch:
        patch(w)
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    return read_model_folder(folder)


# ---------------------------------------------------------------------------------------------- one token that stands out
NEEDLE, DIRECTION, CONST = 7, 3, 5


def _mark_embedding(w):
    """Token ``NEEDLE`` alone has a large entry along ``DIRECTION``; every token the same large one along ``CONST``."""
    for name in ("embed", "bigram"):
        if name in w:
            w[name][:, DIRECTION] = 0.0
            w[name][:, CONST] = 0.0
    w["embed"][NEEDLE, DIRECTION] = 6.0
    w["embed"][:, CONST] = 5.0


def _passes_marks(w, layer_no):
    """Layer ``layer_no`` leaves the two marks of the stream as they are."""
    w[f"l{layer_no}.mix.o"][DIRECTION] = 0.0
    w[f"l{layer_no}.mix.o"][CONST] = 0.0


def rows_needle_model(window, rank=20, rot_dim=4, reader_window=None):
    """An attention through cached rows that gives almost all its weight to the row of token ``NEEDLE`` wherever that
    row is visible, and whose values make the needle's presence large in the logits. With ``reader_window`` a second
    layer reads the first one's rows through a window of its own, and only that layer looks for the needle."""
    layers = [layer("latent_attention", through_rows(2, 8, rot_dim, 6, rank, window, base=100.0, scaling=RAMP, scale=1.0))]
    if reader_window:
        layers.append(layer("latent_attention", through_rows(3, 4, rot_dim, 8, rank, reader_window, base=100.0, scaling=RAMP,
                                                             scale=1.0, kv_from=0)))
    cfg = model(32, 64, layers, mult=1.0, emb_scale=1.0, bigram=(11, 3, 2))
    look = len(layers) - 1

    def patch(w):
        _mark_embedding(w)
        for i in range(len(layers)):
            w[f"l{i}.norm1"][DIRECTION] = w[f"l{i}.norm1"][CONST] = 0.0          # stored around zero: both pass as they are
        if look:
            _passes_marks(w, 0)
        p = f"l{look}.mix."
        H, d = (2, 8) if not look else (3, 4)
        qd = d + rot_dim
        w["l0.mix.dkv"][:, [DIRECTION, CONST]] = 0.0
        w[p + "q"][:, [DIRECTION, CONST]] = 0.0
        w["l0.mix.dkv"][0] = 0.0
        w["l0.mix.dkv"][0, DIRECTION] = 4.0                      # the needle's row points along entry 0, nobody else's does
        w["l0.mix.dkv.norm"][0] = 1.0
        for h in range(H):
            w[p + "uk"][h * d + d - 1] = 0.0
            w[p + "uk"][h * d + d - 1, 0] = 1.0                  # key dim d − 1 reads entry 0 of the row
            w[p + "q"][h * qd + d - 1] = 0.0
            w[p + "q"][h * qd + d - 1, CONST] = 1.0              # and every query looks along it
        w[p + "uv"][:, 0] = 3.0                                  # the needle's value stands out
        w[p + "g"][:] = 0.0                                      # every gate half open

    return cfg, patch


def keys_needle_model(kind, dim=16, rot=8, heads=2, kv=1, far=40, rows=12):
    """The same for the grouped-query attentions, which see every earlier key: ``kind`` 'attention' (biases, a query
    factor, a score by distance) or 'attention_2' (rotation over the first ``rot`` dims, a sink)."""
    if kind == "attention":
        mixer = biased(heads, kv, dim, q_temp=(0.25, 96), far=far, rows=rows, scale=1.0)
    else:
        mixer = turned(heads, kv, dim, rot=rot, base=100.0, scaling=BANDS, scale=1.0)
    cfg = model(32, 64, [layer(kind, mixer)], mult=1.0, emb_scale=1.0, bigram=(11, 3, 2))

    def patch(w):
        _mark_embedding(w)
        w["l0.norm1"][DIRECTION] = w["l0.norm1"][CONST] = 0.0
        for n in ("q", "k"):
            w[f"l0.mix.{n}"][:, [DIRECTION, CONST]] = 0.0
        j = dim - 1                                              # a dim that is not rotated
        for g in range(kv):
            w["l0.mix.k"][g * dim + j, :] = 0.0
            w["l0.mix.k"][g * dim + j, DIRECTION] = 1.0
        for h in range(heads):
            w["l0.mix.q"][h * dim + j, :] = 0.0
            w["l0.mix.q"][h * dim + j, CONST] = 1.0
        if kind == "attention":
            for n in ("q.b", "k.b"):
                w[f"l0.mix.{n}"].view(-1, dim)[:, j] = 0.0
            w["l0.mix.rel"] *= 0.3                               # the table shifts weights, the needle still leads
        else:
            w["l0.mix.sink"][:] = 0.5
        w["l0.mix.v"][:, DIRECTION] = 3.0
        w["l0.mix.g"][:] = 0.0

    return cfg, patch


def with_needle(base, place):
    toks = list(base)
    toks[place] = NEEDLE
    return toks
