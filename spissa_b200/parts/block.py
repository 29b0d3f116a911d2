"""The pre-norm arrangement of a layer: h += mixer(norm(h)); h += ffn(norm(h)).

crates/spissa-runtime/src/models/llama/generate.rs:190-199 (norm before attention),
:459 (first residual sum), :465-471 (norm before the feed-forward), :773 (second sum).
The residual stream ``h`` is 32-bit in every mode; mixer and feed-forward add into it.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import Block, CacheBundle, StateRequest, WeightSpec
from .registry import build_part, register_part
from ..phases import phase


@register_part("block", "prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, mixer, ffn, norms: dict, prefix: str = ""):
        super().__init__(prefix)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None      # a layer may have no feed-forward
        self.mixer_norm = build_part("norm", norms["mixer"])
        self.ffn_norm = build_part("norm", norms["ffn"]) if ffn is not None else None

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def cache_request(self):
        return self.mixer.cache_request()

    def fused_fields(self):
        if self.ffn is None:
            return None
        f = dict(kind="prenorm", mixer_norm=self.mixer_norm.fused_fields(), mixer=self.mixer.fused_fields(),
                 ffn_norm=self.ffn_norm.fused_fields(), ffn=self.ffn.fused_fields())
        return None if any(v is None for v in f.values()) else f

    def forward(self, h, step, cache):
        with phase("attention_norm_ms"):
            x = self.mixer_norm.forward(h)
        self.mixer.forward(x, step, cache, h)
        if self.ffn is None:
            return
        with phase("mlp_norm_ms"):
            x = self.ffn_norm.forward(h)
        self.ffn.forward(x, step, h)


@register_part("block", "parallel_residual")
class ParallelResidualBlock(Block):
    """One norm, two readers: with a = norm(h), h += mixer(a) + ffn(a) (not in the reference). Both sublayers add into
    the 32-bit stream; the feed-forward may be absent. ``norms`` has the one place ``"input"``."""
    graph_safe = True

    def __init__(self, mixer, ffn, norms: dict, prefix: str = ""):
        super().__init__(prefix)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.input_norm = build_part("norm", norms["input"])

    def children(self):
        return [p for p in (self.input_norm, self.mixer, self.ffn) if p is not None]

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, h, step, cache):
        with phase("input_norm_ms"):
            x = self.input_norm.forward(h)
        self.mixer.forward(x, step, cache, h)
        if self.ffn is not None:
            self.ffn.forward(x, step, h)


@register_part("block", "prenorm_shift")
class ShiftedPreNormBlock(Block):
    """The pre-norm arrangement with a token shift in front of the mixer:

        a_t = norm(h_t);  x_t = a_t + (a_{t-1} − a_t) ⊙ mu;  h += mixer(x);  h += ffn(norm(h))

    with a_{-1} = 0 and ``mu`` a learned vector (``shift_name``). The last a of a sequence is state: the block asks
    the cache for one row of the stream's width per run beside whatever its mixer asks for, and hands the mixer the
    view named "mixer". The feed-forward sees no shift and may be absent (``ffn`` None). When the norm describes itself
    as dynamic tanh, norm and shift run as one kernel on the 32-bit stream."""
    graph_safe = True
    kernel_modules = ("seqmix",)

    def __init__(self, mixer, ffn, norms: dict, hidden_size: int, shift_name: str, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        self.shift_name = shift_name
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.mixer_norm = build_part("norm", norms["mixer"])
        self.ffn_norm = build_part("norm", norms["ffn"]) if ffn is not None else None
        self.mu = None

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def weight_specs(self):
        return [WeightSpec(self.shift_name, (self.hidden_size,))]

    def cache_request(self):
        return CacheBundle.of(mixer=self.mixer.cache_request(), shift=StateRequest((self.hidden_size,), torch.float32))

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.mu = tensors[self.shift_name].contiguous()

    def forward(self, h, step, cache):
        state = cache["shift"].state
        x = torch.empty(h.shape[0], self.hidden_size, dtype=self.rt.act_dtype, device=h.device)
        with phase("mixer_norm+shift_ms"):
            f = self.mixer_norm.fused_fields()
            if f is not None and f.get("kind") == "dyt":
                K.token_shift(h, self.mu, state, x, step, dyt=(f["weight"], f["bias"], f["alpha"]))
            else:
                K.token_shift(self.mixer_norm.forward(h), self.mu, state, x, step)
        self.mixer.forward(x, step, cache.get("mixer"), h)
        if self.ffn is not None:
            with phase("mlp_norm_ms"):
                x = self.ffn_norm.forward(h)
            self.ffn.forward(x, step, h)


@register_part("block", "hyper")
class HyperConnectionBlock(Block):
    """The pre-norm arrangement over several residual streams (hyper-connections). A token's row of ``h`` holds
    ``streams`` copies X_1 … X_S of the stream's width side by side. For each sublayer q (1 the mixer, 2 the
    feed-forward, which may be absent) with learned coefficients in_q [S], out_q [S] and mix_q [S, S] (from, to):

        a = norm_q(Σ_s in_q[s] X_s);   y = sublayer_q(a);   X_t ← Σ_s mix_q[s, t] X_s + out_q[t] · y   (all t at once)

    The sublayers keep their interface: they ADD into a 32-bit row buffer, which is zero when they get it. One kernel
    takes y into the streams, leaves the buffer zeroed and norms the next sublayer's input; the norms must describe
    themselves as layer norms (``fused_fields()`` kind ``layernorm``). ``names``: the tensors' names behind the prefix
    (``in1``, ``out1``, ``mix1``, ``in2``, ``out2``, ``mix2``)."""
    graph_safe = True
    kernel_modules = ("hybrid",)

    def __init__(self, mixer, ffn, norms: dict, hidden_size: int, streams: int, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.streams = int(hidden_size), int(streams)
        if self.streams < 1:
            raise ValueError(f"{prefix}: a layer needs at least one stream")
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.mixer_norm = build_part("norm", norms["mixer"])
        self.ffn_norm = build_part("norm", norms["ffn"]) if ffn is not None else None
        n = dict(in1="hc1.in", out1="hc1.out", mix1="hc1.mix", in2="hc2.in", out2="hc2.out", mix2="hc2.mix")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.coef = {}

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def weight_specs(self):
        S = self.streams
        specs = []
        for q in ("1", "2") if self.ffn is not None else ("1",):
            specs += [WeightSpec(self.names["in" + q], (S,), init=f"const:{1.0 / S}"),
                      WeightSpec(self.names["out" + q], (S,), init="const:1.0"),
                      WeightSpec(self.names["mix" + q], (S, S), init="eye")]
        return specs

    def cache_request(self):
        return self.mixer.cache_request()

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        # a handful of numbers per layer; the kernel reads them as 32-bit (exact for either storage type)
        self.coef = {k: tensors[name].float().contiguous() for k, name in self.names.items() if name in tensors}

    def _layer_norm(self, part) -> dict:
        f = part.fused_fields()
        if f is None or f.get("kind") != "layernorm":
            raise ValueError(f"{self.prefix}: the norms of this arrangement are layer norms")
        return f

    def forward(self, h, step, cache):
        S, W, c = self.streams, self.hidden_size, self.coef
        y = step.scratch.get("sublayer_sum")
        if y is None or y.shape[1] != W:
            y = step.scratch["sublayer_sum"] = torch.zeros(h.shape[0], W, dtype=torch.float32, device=h.device)
        x = torch.empty(h.shape[0], W, dtype=self.rt.act_dtype, device=h.device)
        n1 = self._layer_norm(self.mixer_norm)
        with phase("attention_norm_ms"):
            K.streams_norm(h, S, W, out=x, weight=n1["weight"], eps=n1["eps"], in_coef=c["in1"])
        self.mixer.forward(x, step, cache, y)
        if self.ffn is None:
            with phase("streams_update_ms"):
                K.streams_norm(h, S, W, y=y, mix=c["mix1"], out_coef=c["out1"])
            return
        n2 = self._layer_norm(self.ffn_norm)
        with phase("streams_update+mlp_norm_ms"):
            K.streams_norm(h, S, W, out=x, weight=n2["weight"], eps=n2["eps"], y=y, mix=c["mix1"], out_coef=c["out1"],
                           in_coef=c["in2"])
        self.ffn.forward(x, step, y)
        with phase("streams_update_ms"):
            K.streams_norm(h, S, W, y=y, mix=c["mix2"], out_coef=c["out2"])


NORMED_STREAM = "normed_stream"      # a step's scratch entry: the stream under the next block's first norm


@register_part("block", "sandwich")
class SandwichBlock(Block):
    """Every sublayer between two norms, its normed output scaled into the stream (not in the reference):

        h ← h + r · n_1b(mixer(n_1(h)));   h ← h + r · n_2b(ffn(n_2(h)));   h ← h + r · n_s(side(h))

    with r = ``residual_mult``. The feed-forward and the ``side`` sublayer (a feed-forward part that reads the stream
    itself, not a norm of it) may be absent. ``norms`` has the places ``mixer``, ``mixer_out``, ``ffn``, ``ffn_out``
    and ``side_out``; all are RMS norms (they hand their multiplying weight to the kernel that applies them). The
    sublayers keep their interface: they ADD into a 32-bit row buffer that is zero when they get it; one kernel takes
    the buffer's norm into the stream, leaves it zeroed and writes the next sublayer's input in the same pass."""
    graph_safe = True
    kernel_modules = ("sandwich",)

    def __init__(self, mixer, ffn, norms: dict, hidden_size: int, residual_mult: float = 1.0, side=None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.residual_mult = int(hidden_size), float(residual_mult)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.side = build_part("ffn", side) if side is not None else None
        self.mixer_norm, self.mixer_out = build_part("norm", norms["mixer"]), build_part("norm", norms["mixer_out"])
        self.ffn_norm = build_part("norm", norms["ffn"]) if ffn is not None else None
        self.ffn_out = build_part("norm", norms["ffn_out"]) if ffn is not None else None
        self.side_out = build_part("norm", norms["side_out"]) if side is not None else None
        for n in (self.mixer_norm, self.mixer_out, self.ffn_norm, self.ffn_out, self.side_out):
            if n is not None and not hasattr(n, "multiplier"):
                raise ValueError(f"{prefix}: the norms of this arrangement are RMS norms")
        self.next_norm, self.takes_normed = None, False      # see ``feeds``

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_out, self.ffn_norm, self.ffn, self.ffn_out, self.side,
                            self.side_out) if p is not None]

    def cache_request(self):
        return self.mixer.cache_request()

    def feeds(self, nxt) -> bool:
        """Told once, when the model is put together, that ``nxt`` always runs right behind this block on the same
        stream: this block's last pass over the stream then writes ``nxt``'s first norm as well. True if taken."""
        if (isinstance(nxt, SandwichBlock) and nxt.hidden_size == self.hidden_size
                and nxt.mixer_norm.eps == (self.side_out or self.ffn_out or self.mixer_out).eps):
            self.next_norm, nxt.takes_normed = nxt.mixer_norm, True
            return True
        return False

    def forward(self, h, step, cache):
        W, r = self.hidden_size, self.residual_mult
        y = step.scratch.get("sublayer_sum")
        if y is None or y.shape[1] != W:
            y = step.scratch["sublayer_sum"] = torch.zeros(h.shape[0], W, dtype=torch.float32, device=h.device)
        x = step.scratch.pop(NORMED_STREAM, None) if self.takes_normed else None    # the block before has normed the stream
        if x is None:
            with phase("attention_norm_ms"):
                x = self.mixer_norm.forward(h)
        nxt = self.next_norm
        ahead = nxt.multiplier() if nxt is not None else None
        self.mixer.forward(x, step, cache, y)
        last = self.mixer_out
        if self.ffn is not None:
            with phase("attention_out_norm+mlp_norm_ms"):
                x = torch.empty(h.shape[0], W, dtype=self.rt.act_dtype, device=h.device)
                K.stream_norm_add(h, y, last.multiplier(), r, last.eps, w_next=self.ffn_norm.multiplier(), out=x)
            self.ffn.forward(x, step, y)
            last = self.ffn_out
        with phase("out_norm_ms"):
            if self.side is None:
                xn = torch.empty(h.shape[0], W, dtype=self.rt.act_dtype, device=h.device) if nxt is not None else None
                K.stream_norm_add(h, y, last.multiplier(), r, last.eps, w_next=ahead, out=xn)
                if nxt is not None:
                    step.scratch[NORMED_STREAM] = xn
                return
            x = torch.empty(h.shape[0], W, dtype=self.rt.act_dtype, device=h.device)
            K.stream_norm_add(h, y, last.multiplier(), r, last.eps, out=x, raw=True)     # the side sublayer reads the stream itself
        self.side.forward(x, step, y)
        with phase("side_out_norm_ms"):
            xn = torch.empty(h.shape[0], W, dtype=self.rt.act_dtype, device=h.device) if nxt is not None else None
            K.stream_norm_add(h, y, self.side_out.multiplier(), r, self.side_out.eps, w_next=ahead, out=xn)
            if nxt is not None:
                step.scratch[NORMED_STREAM] = xn
