"""Typed configuration of the Fotulix decoder, read from config.json keys.

A Fotulix model embeds a token as its table row times a scale plus a row of a pair table chosen by the token and the
one before it. Every sublayer of a layer stands between two RMS norms whose weights are stored around zero, and its
normed output enters the stream times ``residual_mult``: x ← x + r · n(mixer(n(x))), x ← x + r · n(ff(n(x))), then a
per-layer input chosen by the token, gated by a projection of the stream. Every layer names its mixer (``type``):

* ``attention``: grouped-query attention with biases on q, k, v, no rotation, a query factor that grows with the
  logarithm of the position (``q_temp.coef``, ``q_temp.every``) and a learned score per (log-bucketed distance, head)
  (``bias_max``: the distance that reaches the table's last row);
* ``attention_2``: grouped-query attention with neighbouring pairs rotated over the first ``rot.dims`` dims
  (``rot.base``; ``rot.scaling``: factor, low, high, original = rescaling by bands of wavelength) and a learned sink;
* ``latent_attention``: attention through a cached normed low-rank row (``kv_rank``) plus one rotated key part
  (``rot_dim``) shared by all heads (``rot.scaling``: factor, original, fast, slow = a ramp over the pairs), with a
  sliding window (``mask.size``); ``kv_from``: the layer whose cached rows it reads instead of making its own.

All mixers multiply every head's output by the sigmoid of one number per head. Feed-forwards (``mlp``) are dense
SwiGLUs (``{"kind": "dense", "ff": n}``) or absent (null).

config.json keys: ``architecture`` ("Fotulix"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult``,
``embedding.scale``, ``embedding.bigram.buckets|mul_prev|mul_cur``, ``token_side.dim``, ``layers[i].type|mixer|mlp``;
mixers: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale`` and the keys above. Absent keys mean "not there"
(``bigram``, ``token_side``, ``q_temp``, ``bias_max``, ``rot``, ``rot.scaling``, ``mask``, ``mlp``); ``kv_heads``
defaults to ``heads``, ``vdim`` to ``dim``, ``residual_mult`` and ``embedding.scale`` to 1. The rows of a distance
table are its tensor's first size (``bias_rows`` only says how many a random-weights model gets; default 32).
Tensor names: ``embed``, ``bigram``, ``side.embed``; ``l<i>.norm1|norm1b|norm2|norm2b``; ``l<i>.mix.q|k|v|g|o`` with
``q.b``, ``k.b``, ``v.b``, ``rel``, ``sink``; ``l<i>.mix.q|dkv|dkv.norm|uk|uv|g|o``; ``l<i>.mlp.gate|up|down``;
``l<i>.side.gate|proj|norm``; ``final.norm``; ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .duzinex import _NUM, _get
from .gozatar import _positive
from .llama import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXERS = ("attention", "attention_2", "latent_attention")


def _window(m: dict, where: str):
    mask = _get(m, "mask", where, (dict,), optional=True)
    return _positive(mask, "size", where + "mask.") if mask else None


def _rot(m: dict, where: str, dim: int, keys: tuple):
    """(dims, base, scaling dict or None) of a mixer's ``rot`` entry, or None; ``keys``: the scaling's numbers."""
    rot = _get(m, "rot", where, (dict,), optional=True)
    if not rot:
        return None
    rw = where + "rot."
    dims = _get(rot, "dims", rw)
    if dims <= 0 or dims % 2 or dims > dim:
        raise ConfigError(f"{rw}dims {dims} must be positive, even and at most {dim}")
    base = float(_get(rot, "base", rw, _NUM))
    if not base > 1.0:
        raise ConfigError(f"{rw}base must be larger than 1, got {base}")
    sc = _get(rot, "scaling", rw, (dict,), optional=True)
    scaling = None
    if sc:
        scaling = {k: float(_get(sc, k, rw + "scaling.", _NUM)) for k in keys}
        if any(not v > 0 for v in scaling.values()):
            raise ConfigError(f"{rw}scaling: every number must be positive")
    return dims, base, scaling


@dataclass(frozen=True)
class FotulixConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    bigram: Optional[tuple]          # (buckets, mul_prev, mul_cur) or None
    side_dim: Optional[int]
    layers: tuple                    # per layer the validated dict {type, mixer, mlp}
    raw: Optional[dict] = None       # config.json as it was read (written back by ``to_dict``)

    architecture = "Fotulix"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict) -> "FotulixConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json field 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(layer, "type", where, (str,))
            if kind not in MIXERS:
                raise ConfigError(f"config.json field {where}'type' is {kind!r}; known mixers: {MIXERS}")
            m = _get(layer, "mixer", where, (dict,))
            mw = where + "mixer."
            heads, dim = _positive(m, "heads", mw), _positive(m, "dim", mw)
            mixer = dict(heads=heads, dim=dim, vdim=_positive(m, "vdim", mw, optional=True) or dim,
                         scale=float(_get(m, "scale", mw, _NUM)), window=_window(m, mw))
            if kind in ("attention", "attention_2"):
                kvh = _positive(m, "kv_heads", mw, optional=True) or heads
                if heads % kvh:
                    raise ConfigError(f"{mw}heads {heads} must be a multiple of kv_heads {kvh}")
                mixer["kv_heads"] = kvh
            if kind == "attention":
                qt = _get(m, "q_temp", mw, (dict,), optional=True)
                mixer["q_temp"] = (float(_get(qt, "coef", mw + "q_temp.", _NUM)), _positive(qt, "every", mw + "q_temp.")) if qt else None
                far = _get(m, "bias_max", mw, _NUM, optional=True)
                mixer["bias_max"] = float(far) if far is not None else None
                # the table's rows are the tensor's to say; random weights take this many (``bias_rows``, else 32)
                mixer["bias_rows"] = _positive(m, "bias_rows", mw, optional=True)
            elif kind == "attention_2":
                mixer["rot"] = _rot(m, mw, dim, ("factor", "low", "high", "original"))
                sc = mixer["rot"][2] if mixer["rot"] else None
                if sc and not sc["high"] > sc["low"]:
                    raise ConfigError(f"{mw}rot.scaling.high must be larger than low")
            else:
                rd = _get(m, "rot_dim", mw, optional=True) or 0
                mixer.update(rot_dim=rd, kv_rank=_positive(m, "kv_rank", mw), kv_from=_get(m, "kv_from", mw, optional=True))
                mixer["rot"] = _rot(m, mw, rd, ("factor", "original", "fast", "slow")) if rd else None
                if rd and (mixer["rot"] is None or mixer["rot"][0] != rd):
                    raise ConfigError(f"{mw}rot.dims must equal rot_dim {rd}")
                src = mixer["kv_from"]
                if src is not None:
                    if not (0 <= src < i) or checked[src]["type"] != "latent_attention" or \
                            checked[src]["mixer"]["kv_from"] is not None:
                        raise ConfigError(f"{mw}kv_from {src} must name an earlier latent-attention layer with rows of its own")
                    theirs = checked[src]["mixer"]
                    if (theirs["kv_rank"], theirs["rot_dim"], theirs["rot"]) != (mixer["kv_rank"], rd, mixer["rot"]):
                        raise ConfigError(f"{mw}kv_rank, rot_dim and rot must equal layer {src}'s, whose rows it reads")
            mlp = layer.get("mlp")
            if mlp is not None:
                fw = where + "mlp."
                mk = _get(mlp, "kind", fw, (str,))
                if mk != "dense":
                    raise ConfigError(f"config.json field {fw}'kind' is {mk!r}; known: 'dense'")
                mlp = dict(kind=mk, ff=_positive(mlp, "ff", fw))
            checked.append(dict(type=kind, mixer=mixer, mlp=mlp))
        emb = _get(d, "embedding", "", (dict,), optional=True) or {}
        bg = _get(emb, "bigram", "embedding.", (dict,), optional=True)
        bigram = None
        if bg:
            bw = "embedding.bigram."
            bigram = (_positive(bg, "buckets", bw), _get(bg, "mul_prev", bw), _get(bg, "mul_cur", bw))
        side = _get(d, "token_side", "", (dict,), optional=True)
        mult = _get(d, "residual_mult", "", _NUM, optional=True)
        return cls(vocab=_positive(d, "vocab", ""), width=_positive(d, "width", ""),
                   norm_eps=float(_get(d.get("norm") or {}, "eps", "norm.", _NUM)),
                   residual_mult=float(mult) if mult is not None else 1.0,
                   embedding_scale=float(_get(emb, "scale", "embedding.", _NUM, optional=True) or 1.0),
                   bigram=bigram, side_dim=_positive(side, "dim", "token_side.") if side else None,
                   layers=tuple(checked), raw=dict(d))

    def to_dict(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        layers = []
        for l in self.layers:
            m = {k: v for k, v in l["mixer"].items() if v is not None}
            w = m.pop("window", None)
            if w:
                m["mask"] = dict(size=w)
            if "q_temp" in m:
                m["q_temp"] = dict(coef=m["q_temp"][0], every=m["q_temp"][1])
            if "rot" in m:
                dims, base, sc = m["rot"]
                m["rot"] = dict(dims=dims, base=base)
                if sc:
                    m["rot"]["scaling"] = dict(sc)
            if l["type"] == "latent_attention" and not m.get("rot_dim"):
                m.pop("rot_dim", None)
            layers.append(dict(type=l["type"], mixer=m, mlp=l["mlp"]))
        emb = dict(scale=self.embedding_scale)
        if self.bigram:
            emb["bigram"] = dict(buckets=self.bigram[0], mul_prev=self.bigram[1], mul_cur=self.bigram[2])
        out = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                   residual_mult=self.residual_mult, embedding=emb, layers=layers)
        if self.side_dim:
            out["token_side"] = dict(dim=self.side_dim)
        return out

    def stop_token_ids(self) -> list:
        return []

    # ------------------------------------------------------------------ model
    def cache_windows(self) -> dict:
        """Layer with cached rows of its own -> the window its cache keeps rows for: the widest among the layers that
        read it (None: one of them sees everything)."""
        out = {}
        for i, l in enumerate(self.layers):
            if l["type"] != "latent_attention":
                continue
            src = l["mixer"]["kv_from"] if l["mixer"]["kv_from"] is not None else i
            w = l["mixer"]["window"]
            if src not in out:
                out[src] = w
            elif out[src] is not None:
                out[src] = None if w is None else max(out[src], w)
        return out

    def to_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        windows = self.cache_windows()
        n_layers = len(self.layers)

        def norm(name, around_zero=True):
            return PartSpec("rmsnorm", dict(size=W, eps=eps, weight_name="", around_zero=around_zero), prefix=name)

        layers, schedule = [], []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            if l["type"] == "latent_attention":
                src = m["kv_from"]
                own = src is None
                rope = None
                if m["rot"]:
                    dims, base, sc = m["rot"]
                    rope = PartSpec("rotary", dict(theta=base, rotary_dim=dims, pairing="interleaved",
                                                   scaling=dict(sc, rope_type="ramp") if sc else None))
                mixer = PartSpec("rotary_latent_attention", dict(
                    hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
                    kv_rank=m["kv_rank"], scale=m["scale"], eps=eps, position=rope, window=m["window"],
                    cache_window=windows[i if own else src], shares_latent=not own), prefix=p + "mix.")
                schedule.append(ScheduleEntry(i, i if own else src, own))
            else:
                rope = None
                if l["type"] == "attention_2" and m["rot"]:
                    dims, base, sc = m["rot"]
                    scaling = None
                    if sc:
                        scaling = dict(rope_type="llama3", factor=sc["factor"], low_freq_factor=sc["low"],
                                       high_freq_factor=sc["high"], original_max_position_embeddings=sc["original"])
                    rope = PartSpec("rotary", dict(theta=base, rotary_dim=dims, pairing="interleaved", scaling=scaling))
                biased = l["type"] == "attention"
                params = dict(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                              v_head_dim=m["vdim"], scale=m["scale"], bias=biased, position=rope, sink=not biased,
                              window=m["window"])
                if biased:
                    params.update(q_temp=m["q_temp"], distance_rows=-(m["bias_rows"] or 32) if m["bias_max"] is not None else 0,
                                  distance_far=m["bias_max"] or 0.0)
                mixer = PartSpec("gated_attention", params, prefix=p + "mix.")
                schedule.append(ScheduleEntry(i, i, True))
            ffn, f = None, l["mlp"]
            if f is not None:
                ffn = PartSpec("swiglu", dict(hidden_size=W, intermediate_size=f["ff"],
                                              names=dict(gate="gate", up="up", down="down")), prefix=p + "mlp.")
            norms = {"mixer": norm(p + "norm1"), "mixer_out": norm(p + "norm1b")}
            if ffn is not None:
                norms.update({"ffn": norm(p + "norm2"), "ffn_out": norm(p + "norm2b")})
            side = None
            if self.side_dim:
                side = PartSpec("token_side", dict(hidden_size=W, dim=self.side_dim, vocab_size=self.vocab,
                                                   table_width=n_layers * self.side_dim, offset=i * self.side_dim,
                                                   table_name="side.embed"), prefix=p + "side.")
                norms["side_out"] = norm(p + "side.norm", around_zero=False)
            layers.append(LayerSpec(block="sandwich", mixer=mixer, ffn=ffn, norms=norms,
                                    params=dict(hidden_size=W, residual_mult=self.residual_mult, side=side)))
        if self.bigram:
            embedding = PartSpec("pair_embedding", dict(
                vocab_size=self.vocab, hidden_size=W, weight_name="embed", pair_name="bigram", scale=self.embedding_scale,
                buckets=self.bigram[0], mul_prev=self.bigram[1], mul_cur=self.bigram[2]))
        else:
            embedding = PartSpec("embedding", dict(vocab_size=self.vocab, hidden_size=W, weight_name="embed",
                                                   scale=self.embedding_scale))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, embedding=embedding,
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=W, weight_name="head")),
            max_position=0)
        spec.validate()
        return spec


register_architecture(FotulixConfig.architecture, FotulixConfig)
