"""Norms of the residual stream.

RMS norm: y = x / sqrt(mean(x²) + eps) · w, statistics in 32-bit
(crates/spissa-runtime/src/ops.rs:159-179: eps inside the root, the weight multiplies
directly, no ``1 + w``).

Dynamic tanh: y = tanh(alpha · x) ⊙ w + b with a learned scalar alpha: a norm that takes
no mean and no variance, so a token's row needs no reduction (not in the reference).

Layer norm: y = (x − mean) / sqrt(var + eps) ⊙ w with var the mean of the squared deviations, a weight and no bias
(not in the reference). Where a model keeps several copies of the residual stream side by side in a row
(``streams``), the norm reads their sum.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import Norm, WeightSpec
from .registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, prefix: str = "", weight_name: str = "weight", around_zero: bool = False):
        super().__init__(prefix)
        self.size = int(size)
        self.eps = float(eps)
        self.weight_name = prefix + weight_name
        self.around_zero = bool(around_zero)   # the stored weight w lies around zero and 1 + w multiplies (not in the reference)
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.size,), init="normal" if self.around_zero else "ones")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.weight_name].contiguous()
        if self.around_zero:
            self.weight = (1.0 + self.weight.float()).contiguous()     # 32-bit: 1 + w rounded to 16 bits would lose w

    def multiplier(self) -> torch.Tensor:
        """The weight as it multiplies, float32 [size] (for a kernel that applies this norm inside another pass)."""
        if self.weight.dtype != torch.float32:
            self.weight32 = getattr(self, "weight32", None)
            if self.weight32 is None:
                self.weight32 = self.weight.float().contiguous()
            return self.weight32
        return self.weight

    def fused_fields(self):
        if self.weight is None or self.weight.dtype != torch.bfloat16:
            return None
        return dict(kind="rmsnorm", weight=self.weight, eps=self.eps, size=self.size)

    def forward(self, h: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, self.size, dtype=self.rt.act_dtype, device=h.device)
        K.rmsnorm(h, self.weight, out, self.eps, rows)
        return out


@register_part("norm", "dyt")
class DynamicTanh(Norm):
    """``weight_name`` / ``bias_name`` / ``alpha_name`` are appended to the prefix (the weight's may be empty: some
    checkpoints store it under the norm's own name)."""
    graph_safe = True
    kernel_modules = ("seqmix",)

    def __init__(self, size: int, prefix: str = "", weight_name: str = "weight", bias_name: str = "bias",
                 alpha_name: str = "alpha"):
        super().__init__(prefix)
        self.size = int(size)
        self.names = dict(w=prefix + weight_name, b=prefix + bias_name, a=prefix + alpha_name)
        self.weight = self.bias = self.alpha = None

    def weight_specs(self):
        return [WeightSpec(self.names["w"], (self.size,), init="ones"), WeightSpec(self.names["b"], (self.size,)),
                WeightSpec(self.names["a"], (), init="const:0.5")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.names["w"]].contiguous()
        self.bias = tensors[self.names["b"]].contiguous()
        self.alpha = tensors[self.names["a"]].reshape(1).contiguous()
        if not (self.weight.dtype == self.bias.dtype == self.alpha.dtype):
            raise ValueError(f"{self.prefix}: weight, bias and alpha must share a storage type")

    def fused_fields(self):
        if self.weight is None:
            return None
        return dict(kind="dyt", weight=self.weight, bias=self.bias, alpha=self.alpha, size=self.size)

    def forward(self, h: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, self.size, dtype=self.rt.act_dtype, device=h.device)
        K.dyt_norm(h, self.weight, self.bias, self.alpha, out, rows)
        return out


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """``streams`` > 1: a row of ``h`` holds that many streams of ``size`` one after another and the norm reads their
    sum (how the final norm of a model with several residual streams takes them in)."""
    graph_safe = True
    kernel_modules = ("hybrid",)

    def __init__(self, size: int, eps: float, prefix: str = "", weight_name: str = "weight", streams: int = 1):
        super().__init__(prefix)
        self.size, self.eps, self.streams = int(size), float(eps), int(streams)
        self.weight_name = prefix + weight_name
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.size,), init="ones")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.weight_name].contiguous()

    def fused_fields(self):
        if self.weight is None:
            return None
        return dict(kind="layernorm", weight=self.weight, eps=self.eps, size=self.size)

    def forward(self, h: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, self.size, dtype=self.rt.act_dtype, device=h.device)
        K.streams_norm(h, self.streams, self.size, out=out, weight=self.weight, eps=self.eps, rows=rows)
        return out
