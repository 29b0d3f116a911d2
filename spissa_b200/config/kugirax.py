"""Typed configuration of the Kugirax decoder, read from config.json keys.

A Kugirax model is a list of layers with ONE RMS norm each, whose output both sublayers read: with a = n(x),
x ← x + mixer(a) + ff(a). Every layer names its mixer (``type``: ``attention`` = grouped-query attention whose q and k
pass a short convolution, whose values are the convolved keys, with a rotation and one added to the softmax's
denominator; ``latent_attention`` = attention through a cached low-rank latent with a sliding window and a learned
sink per head, which may read the latent that another layer cached: ``kv_from``) with the mixer's sizes, and its
feed-forward (``mlp``: ``{"kind": "dense", "ff": n}`` = SwiGLU, ``{"kind": "moe", ...}`` = routed SwiGLU experts behind a
softmax router plus a shared expert with a gate per token, or null for none). The logits pass a tanh cap.

config.json keys: ``architecture`` ("Kugirax"), ``vocab``, ``width``, ``norm.eps``, ``logit_softcap``,
``layers[i].type | mixer | mlp``; attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``, ``rot.dims``,
``rot.base``, ``scale``; latent attention: ``heads``, ``dim``, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``,
``mask.size``, ``kv_from``; ``mlp.ff`` or ``mlp.expert.ff``, ``mlp.router.experts|top|scale``, ``mlp.shared.ff``.
Tensor names: ``embed``; ``l<i>.norm1``; ``l<i>.mix.q|k|o`` with ``q.conv``, ``k.conv``; ``l<i>.mix.dq|dq.norm|uq|dkv|
dkv.norm|uk|uv|sink|o``; ``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router|e<j>.gate|up|down|shared.gate|up|down|sg``;
``final.norm``; ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .duzinex import _NUM, _get
from .gozatar import _positive
from .llama import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXERS = ("attention", "latent_attention")
UNIT_SINK = 0.0                   # the design's attention adds one to the softmax's denominator: a sink whose score is 0


def _window(m: dict, where: str):
    mask = _get(m, "mask", where, (dict,), optional=True)
    return _positive(mask, "size", where + "mask.") if mask else None


@dataclass(frozen=True)
class KugiraxConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: Optional[float]
    layers: tuple                    # per layer the validated dict {type, mixer, mlp}
    raw: Optional[dict] = None       # config.json as it was read (written back by ``to_dict``)

    architecture = "Kugirax"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict) -> "KugiraxConfig":
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
            if kind == "attention":
                kvh = _positive(m, "kv_heads", mw, optional=True) or heads
                if heads % kvh:
                    raise ConfigError(f"{mw}heads {heads} must be a multiple of kv_heads {kvh}")
                if mixer["vdim"] != dim:
                    raise ConfigError(f"{mw}vdim {mixer['vdim']} differs from dim {dim}, but the values are the keys")
                mixer.update(kv_heads=kvh, conv=_positive(m, "conv", mw, optional=True), rot_dims=0, rot_base=10000.0)
                rot = _get(m, "rot", mw, (dict,), optional=True)
                if rot:
                    dims = _get(rot, "dims", mw + "rot.")
                    if dims < 0 or dims % 2 or dims > dim:
                        raise ConfigError(f"{mw}rot.dims {dims} must be even and at most dim {dim}")
                    mixer.update(rot_dims=dims, rot_base=float(_get(rot, "base", mw + "rot.", _NUM)))
            else:
                mixer.update(q_rank=_positive(m, "q_rank", mw), kv_rank=_positive(m, "kv_rank", mw),
                             kv_from=_get(m, "kv_from", mw, optional=True))
                src = mixer["kv_from"]
                if src is not None:
                    if not (0 <= src < i) or checked[src]["type"] != "latent_attention" or \
                            checked[src]["mixer"]["kv_from"] is not None:
                        raise ConfigError(f"{mw}kv_from {src} must name an earlier latent-attention layer with a latent of its own")
                    if checked[src]["mixer"]["kv_rank"] != mixer["kv_rank"]:
                        raise ConfigError(f"{mw}kv_rank {mixer['kv_rank']} differs from layer {src}'s, whose latent it reads")
            mlp = layer.get("mlp")
            if mlp is not None:
                fw = where + "mlp."
                mk = _get(mlp, "kind", fw, (str,))
                if mk == "dense":
                    mlp = dict(kind=mk, ff=_positive(mlp, "ff", fw))
                elif mk == "moe":
                    ro = _get(mlp, "router", fw, (dict,))
                    shared = _get(mlp, "shared", fw, (dict,), optional=True)
                    mlp = dict(kind=mk, ff=_positive(_get(mlp, "expert", fw, (dict,)), "ff", fw + "expert."),
                               experts=_positive(ro, "experts", fw + "router."), top=_positive(ro, "top", fw + "router."),
                               scale=float(_get(ro, "scale", fw + "router.", _NUM, optional=True) or 1.0),
                               shared_ff=_positive(shared, "ff", fw + "shared.") if shared else None)
                    if mlp["top"] > mlp["experts"]:
                        raise ConfigError(f"{fw}router.top {mlp['top']} is more than the {mlp['experts']} experts")
                else:
                    raise ConfigError(f"config.json field {fw}'kind' is {mk!r}; known: 'dense', 'moe'")
            checked.append(dict(type=kind, mixer=mixer, mlp=mlp))
        norm = d.get("norm") or {}
        cap = _get(d, "logit_softcap", "", _NUM, optional=True)
        if cap is not None and not cap > 0:
            raise ConfigError("config.json field 'logit_softcap' must be positive")
        return cls(vocab=_positive(d, "vocab", ""), width=_positive(d, "width", ""),
                   norm_eps=float(_get(norm, "eps", "norm.", _NUM)), logit_softcap=float(cap) if cap else None,
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
            if l["type"] == "attention":
                rd, rb = m.pop("rot_dims"), m.pop("rot_base")
                if rd:
                    m["rot"] = dict(dims=rd, base=rb)
            f = l["mlp"]
            if f is not None and f["kind"] == "moe":
                f = dict(kind="moe", expert=dict(ff=f["ff"]), router=dict(experts=f["experts"], top=f["top"], scale=f["scale"]),
                         shared=dict(ff=f["shared_ff"]) if f["shared_ff"] else None)
            layers.append(dict(type=l["type"], mixer=m, mlp=f))
        out = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                   layers=layers)
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out

    def stop_token_ids(self) -> list:
        return []

    # ------------------------------------------------------------------ model
    def cache_windows(self) -> dict:
        """Layer with a latent of its own -> the window its cache keeps rows for: the widest among the layers that
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
        swiglu_names = dict(gate="gate", up="up", down="down")

        def norm(name):
            return PartSpec("rmsnorm", dict(size=W, eps=eps, weight_name=""), prefix=name)

        layers, schedule = [], []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            if l["type"] == "attention":
                rope = None
                if m["rot_dims"] > 0:
                    rope = PartSpec("rotary", dict(theta=m["rot_base"], rotary_dim=m["rot_dims"]))
                mixer = PartSpec("conv_attention", dict(
                    hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], conv_taps=m["conv"],
                    scale=m["scale"], position=rope, window=m["window"], value_from_key=True, sink_logit=UNIT_SINK),
                    prefix=p + "mix.")
                schedule.append(ScheduleEntry(i, i, True))
            else:
                src = m["kv_from"]
                own = src is None
                mixer = PartSpec("latent_attention", dict(
                    hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"], q_rank=m["q_rank"],
                    kv_rank=m["kv_rank"], scale=m["scale"], eps=eps, window=m["window"],
                    cache_window=windows[i if own else src], shares_latent=not own), prefix=p + "mix.")
                schedule.append(ScheduleEntry(i, i if own else src, own))
            ffn, f = None, l["mlp"]
            if f is not None and f["kind"] == "dense":
                ffn = PartSpec("swiglu", dict(hidden_size=W, intermediate_size=f["ff"], names=swiglu_names), prefix=p + "mlp.")
            elif f is not None:
                shared = None
                if f["shared_ff"]:
                    shared = PartSpec("swiglu", dict(hidden_size=W, intermediate_size=f["shared_ff"], names=swiglu_names),
                                      prefix=p + "mlp.shared.")
                ffn = PartSpec("routed_experts", dict(
                    hidden_size=W, intermediate_size=f["ff"], experts=f["experts"], top=f["top"], activation="swiglu",
                    score="softmax", weight_scale=f["scale"], correction=False, shared=shared,
                    shared_gate="shared.sg" if shared else None), prefix=p + "mlp.")
            layers.append(LayerSpec(block="parallel_residual", mixer=mixer, ffn=ffn, norms={"input": norm(p + "norm1")}))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W,
            embedding=PartSpec("embedding", dict(vocab_size=self.vocab, hidden_size=W, weight_name="embed")),
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=W, weight_name="head",
                                          softcap=self.logit_softcap)),
            max_position=0)
        spec.validate()
        return spec


register_architecture(KugiraxConfig.architecture, KugiraxConfig)
