"""Grouped-query attention whose projections pass a short convolution over time, as a mixer (not in the reference).

    q = conv(x·Wqᵀ), k = conv(x·Wkᵀ), v = conv(x·Wvᵀ)          conv: y_t = Σ_j w[:, j] ⊙ u_{t−taps+1+j} per channel,
                                                                zeros before the sequence's start, no bias
    q, k: dim i turns with dim i + r/2 over the first r dims of each head (the position part's ``rotary_dim``)
    q, k ← q, k / sqrt(mean(·²) + eps) per head                 (``qk_norm_eps`` None: left as they are)
    score = (q · k) · scale over the visible keys (``window`` None: all earlier ones), softmax in 32-bit
    y += Wo · concat_h(softmax · v) · out_scale

``value_from_key``: there is no Wv; a token's values are its keys as they leave the convolution, before the rotation.
``sink_logit`` s: the softmax's denominator holds one more term e^{s} that has no key and no value (s = 0: one is
added to the sum of the exponentials).

Keys and values may have different sizes per head (``v_head_dim``). The last taps − 1 projected rows of a sequence are
its state beside the paged keys and values; the convolution, the rotation and the norm run in 32-bit on the unrounded
projections in one kernel that also writes the cache (the values already times ``out_scale``). The attention itself is
the grouped-query mixer's: its tensor-core kernels where key and value sizes agree, else the generic one.
"""
from __future__ import annotations

import math

import torch

from ..csrc import lib as K
from .attention import GQAAttention
from .base import CacheBundle, KVCacheRequest, Mixer, StateRequest, WeightSpec
from .linear import Linear
from .registry import register_part
from ..phases import phase


@register_part("mixer", "conv_attention")
class ConvAttention(GQAAttention):
    graph_safe = True
    kernel_modules = ("hybrid",)
    kernel_modules_bf16 = ("attention",)

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int | None = None,
                 conv_taps: int | None = None, scale: float | None = None, qk_norm_eps: float | None = None,
                 out_scale: float = 1.0, position=None, window=None, value_from_key: bool = False,
                 sink_logit: float | None = None, prefix: str = "", names: dict | None = None):
        n = dict(q="q", k="k", v="v", o="o", conv_suffix=".conv")
        n.update(names or {})
        self.conv_suffix = n.pop("conv_suffix")
        super().__init__(hidden_size, num_heads, num_kv_heads, head_dim, position=position, window=window,
                         prefix=prefix, names=n)
        self.v_head_dim = int(v_head_dim or head_dim)
        self.conv_taps = int(conv_taps or 0)       # 0: no convolution and no tensors for one; 1: a weight per channel
        if scale is not None:
            self.scale = float(scale)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.out_scale = float(out_scale)
        self.value_from_key = bool(value_from_key)
        if self.value_from_key and self.v_head_dim != self.head_dim:
            raise ValueError(f"{prefix}: values that are the keys have the keys' size")
        self.sink_logit = None if sink_logit is None else float(sink_logit)
        self.conv = None

    @property
    def channels(self) -> int:
        return (self.num_heads + self.num_kv_heads) * self.head_dim + (0 if self.value_from_key else self.num_kv_heads * self.v_head_dim)

    @property
    def _projected(self) -> tuple:
        return ("q", "k") if self.value_from_key else ("q", "k", "v")

    def weight_specs(self):
        H, nh, nkv, d, vd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        shapes = dict(q=(nh * d, H), k=(nkv * d, H), v=(nkv * vd, H))
        shapes = {k: shapes[k] for k in self._projected}
        specs = [WeightSpec(self.names[k], s) for k, s in shapes.items()] + [WeightSpec(self.names["o"], (H, nh * vd))]
        if self.conv_taps >= 1:
            specs += [WeightSpec(self.names[k] + self.conv_suffix, (s[0], self.conv_taps), init="const:0.5")
                      for k, s in shapes.items()]
        return specs

    def cache_request(self):
        vd = self.v_head_dim if self.v_head_dim != self.head_dim else None
        state = StateRequest((self.conv_taps - 1, self.channels), torch.float32) if self.conv_taps > 1 else None
        return CacheBundle.of(kv=KVCacheRequest(self.num_kv_heads, self.head_dim, self.window, v_head_dim=vd), conv=state)

    def fused_fields(self):
        return None

    def bind(self, tensors, rt):
        if self.value_from_key:
            Mixer.bind(self, tensors, rt)
            q, k = tensors[self.names["q"]], tensors[self.names["k"]]
            if q.dtype != k.dtype:
                raise ValueError(f"{self.prefix}: q and k projections must share a storage type")
            self.qkv = Linear(torch.cat([q, k], dim=0))
            self.o = Linear(tensors[self.names["o"]])
            self.counters = torch.zeros(4096, dtype=torch.int32, device=rt.device)
        else:
            super().bind(tensors, rt)
        if self.sink_logit is not None:
            self.sink = torch.full((self.num_heads,), self.sink_logit, dtype=torch.float32, device=rt.device)
        if self.conv_taps >= 1:
            self.conv = torch.cat([tensors[self.names[k] + self.conv_suffix] for k in self._projected], dim=0).contiguous()

    def forward(self, x, step, cache, residual):
        nh, nkv, d, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        kv = cache["kv"]
        if not kv.writes:
            raise ValueError(f"{self.prefix}: this mixer writes its own cache")
        state = cache["conv"].state if self.conv_taps > 1 else None
        inv_freq, rd = self.position.rotary() if self.position is not None else (None, 0)
        with phase("qkv_projection_ms"):
            qkv = self.qkv(x, out_dtype=torch.float32)             # convolution and rotation read unrounded products
        with phase("conv+rotary+kv_append_ms"):
            q = torch.empty(x.shape[0], nh * d, dtype=self.rt.act_dtype, device=x.device)
            K.conv_qk_store(qkv, self.conv, max(1, self.conv_taps), state, q, kv.k_pool, kv.v_pool, kv, step, inv_freq, nh, nkv,
                            d, vd, rd, self.qk_norm_eps or 0.0, v_scale=self.out_scale,
                            unit_rms=self.qk_norm_eps is not None, v_from_k=self.value_from_key)
        with phase("attention_ms"):
            if vd == d:
                ctx = self.attend(q, step, kv)
            else:
                ctx = torch.empty(x.shape[0], nh * vd, dtype=self.rt.act_dtype, device=x.device)
                K.attention_generic(q, kv.k_pool, kv.v_pool, ctx, kv, nh, nkv, d, self.window, self.scale, vd=vd,
                                    sink=self.sink)
        with phase("o_projection+attention_residual_ms"):
            self.o(ctx, out=residual, accumulate=True)
