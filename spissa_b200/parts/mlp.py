"""Feed-forwards.

PolyNorm feed-forward: down( a·N(z) + b·N(z²) + c·N(z³) + e ) with z = x·Wupᵀ, powers element by element and
N(v) = v / sqrt(mean(v²) + eps) over a token's row; (a, b, c, e) is a learned tensor of four numbers (not in the
reference). The activation runs in 32-bit on the unrounded product.

SwiGLU feed-forward: down( silu(x·Wgᵀ) ⊙ (x·Wuᵀ) ), silu(z) = z / (1 + e^{-z}).

GELU feed-forward: down( gelu(x·Wupᵀ) ) with the tanh form gelu(z) = ½ z (1 + tanh(√(2/π) (z + 0.044715 z³))) (not in
the reference).

Clamped GLU feed-forward: g = min(x·Wgᵀ, limit), u = clamp(x·Wuᵀ, ±limit), down( g · sigmoid(slope · g) · (u + 1) ) (not
in the reference).

A SwiGLU may carry a gate of one number per token: the rows of silu(·) ⊙ (·) are multiplied by ``row_gate`` =
sigmoid(x · w_sgᵀ) before the down projection (which is linear, so its output is scaled by the same number).

Routed experts: ``experts`` gated feed-forwards (``activation``: ``clamped_glu`` or ``swiglu``) of which each token uses
``top``. The scores s are ``score`` of the router's 32-bit logits: ``sigmoid``, or ``softmax`` over all experts; the
weights are s_k / (Σ s_k + 1e-20) · ``weight_scale``. A shared expert may be gated per token by sigmoid(x · w_sgᵀ)
(``shared_gate`` names the row w_sg; it rides in the router's product). With the sigmoid score: s = sigmoid(x·Wrᵀ) in 32-bit;
the choice reads s + correction, the weights read s: the experts form ``groups`` equal groups of neighbours, a group's
score is the sum of its two largest choice scores, only experts of the ``keep_groups`` best groups can be chosen, the
``top`` largest choice scores among them are; weight_k = s_k / (Σ s_k + 1e-20); y += Σ_k weight_k · expert_k(x), plus a
shared expert that every token uses (not in the reference).

crates/spissa-runtime/src/models/llama/generate.rs:590-637 (gate, up), :642-763 (down);
crates/spissa-runtime/src/ops.rs:192-194 (silu). Gate and up run as one matrix product
over the stacked weight [Wg; Wu]; the down projection adds into the residual stream.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import FeedForward, WeightSpec
from .linear import GatedLinear, Linear
from .registry import build_part, register_part
from ..phases import phase


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        n = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.gate_up = self.down = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["gate"], (I, H)), WeightSpec(self.names["up"], (I, H)),
                WeightSpec(self.names["down"], (H, I))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        if g.dtype != u.dtype:
            raise ValueError(f"{self.prefix}: gate and up projections must share a storage type")
        self.gate_up = GatedLinear(g, u)
        self.down = Linear(tensors[self.names["down"]])

    def fused_fields(self):
        gu = self.gate_up
        if gu is None or not gu.block or gu.weight.dtype != torch.bfloat16 or self.down.weight.dtype != torch.bfloat16:
            return None
        return dict(kind="swiglu", gate_up=gu.weight, pair=gu.block, down=self.down.weight,
                    hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)

    takes_row_gate = True

    def forward(self, x, step, residual, row_gate=None):
        """``row_gate`` (float32 [T]): the token's output is multiplied by sigmoid(row_gate[t])."""
        with phase("gate_projection+up_projection+activation_multiply_ms"):
            act = self.gate_up(x, self.rt.act_dtype)
            if row_gate is not None:
                K.scale_rows_sigmoid(act, row_gate)
        with phase("down_projection+mlp_residual_ms"):
            self.down(act, out=residual, accumulate=True)


@register_part("ffn", "polynorm")
class PolyNormMLP(FeedForward):
    graph_safe = True
    kernel_modules = ("seqmix",)

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size, self.eps = int(hidden_size), int(intermediate_size), float(eps)
        n = dict(up="up", down="down", act="act")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.up = self.down = self.coef = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["up"], (I, H)), WeightSpec(self.names["down"], (H, I)),
                WeightSpec(self.names["act"], (4,), init="const:0.5")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.up = Linear(tensors[self.names["up"]])
        self.down = Linear(tensors[self.names["down"]])
        self.coef = tensors[self.names["act"]].contiguous()

    def forward(self, x, step, residual):
        with phase("up_projection_ms"):
            z = self.up(x, out_dtype=torch.float32)                # the activation's statistics read unrounded products
        with phase("activation_ms"):
            act = torch.empty(x.shape[0], self.intermediate_size, dtype=self.rt.act_dtype, device=x.device)
            K.polynorm(z, self.coef, act, self.eps)
        with phase("down_projection+mlp_residual_ms"):
            self.down(act, out=residual, accumulate=True)


@register_part("ffn", "gelu_mlp")
class GeluMLP(FeedForward):
    graph_safe = True
    kernel_modules = ("hybrid",)

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        n = dict(up="up", down="down")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.up = self.down = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["up"], (I, H)), WeightSpec(self.names["down"], (H, I))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.up = Linear(tensors[self.names["up"]])
        self.down = Linear(tensors[self.names["down"]])

    def forward(self, x, step, residual):
        with phase("up_projection_ms"):
            z = self.up(x, out_dtype=torch.float32)                # the activation reads unrounded products
        with phase("activation_ms"):
            act = torch.empty(x.shape[0], self.intermediate_size, dtype=self.rt.act_dtype, device=x.device)
            K.gelu_tanh(z, act)
        with phase("down_projection+mlp_residual_ms"):
            self.down(act, out=residual, accumulate=True)


@register_part("ffn", "clamped_glu")
class ClampedGLU(FeedForward):
    graph_safe = True
    kernel_modules = ("hybrid",)

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, slope: float = 1.702, prefix: str = "",
                 names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.slope = float(limit), float(slope)
        n = dict(gate="gate", up="up", down="down")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.gate_up = self.down = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["gate"], (I, H)), WeightSpec(self.names["up"], (I, H)),
                WeightSpec(self.names["down"], (H, I))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.gate_up = Linear(torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]], dim=0))
        self.down = Linear(tensors[self.names["down"]])

    def forward(self, x, step, residual):
        with phase("gate_projection+up_projection_ms"):
            gu = self.gate_up(x, out_dtype=torch.float32)
        with phase("activation_ms"):
            act = torch.empty(x.shape[0], self.intermediate_size, dtype=self.rt.act_dtype, device=x.device)
            K.clamped_glu(gu, act, self.limit, self.slope)
        with phase("down_projection+mlp_residual_ms"):
            self.down(act, out=residual, accumulate=True)


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    """``shared``: a feed-forward part (any kind) that every token uses besides its experts, or None. Tensor names:
    expert i's tensors stand under ``expert_prefix`` + i + "." (``e0.gate`` …)."""
    graph_safe = True
    kernel_modules = ("hybrid",)
    kernel_modules_bf16 = ("tc_gemm",)

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, limit: float = 0.0,
                 slope: float = 1.702, groups: int = 1, keep_groups: int = 1, shared=None, prefix: str = "",
                 names: dict | None = None, activation: str = "clamped_glu", score: str = "sigmoid",
                 weight_scale: float = 1.0, correction: bool = True, shared_gate: str | None = None):
        super().__init__(prefix)
        if activation not in ("clamped_glu", "swiglu") or score not in ("sigmoid", "softmax"):
            raise ValueError(f"{prefix}: unknown activation {activation!r} or score {score!r}")
        self.activation, self.score, self.weight_scale = activation, score, float(weight_scale)
        self.has_correction = bool(correction)
        self.shared_gate = shared_gate           # name (behind the prefix) of a row [1, hidden]: the shared expert's gate
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.experts, self.top = int(experts), int(top)
        self.groups, self.keep_groups = max(1, int(groups or 1)), int(keep_groups or 1)
        # the kernels read slope 0 as "the plain gated unit silu(g) · u"
        self.limit, self.slope = (float(limit), float(slope)) if activation == "clamped_glu" else (0.0, 0.0)
        if self.experts % self.groups:
            raise ValueError(f"{prefix}: {self.experts} experts do not form {self.groups} equal groups")
        allowed = self.experts if self.groups == 1 else self.keep_groups * (self.experts // self.groups)
        if not (1 <= self.top <= allowed):
            raise ValueError(f"{prefix}: {self.top} experts cannot be chosen among {allowed} allowed")
        n = dict(router="router", correction="correction", expert_prefix="e", gate="gate", up="up", down="down")
        n.update(names or {})
        self.names = n
        self.shared = build_part("ffn", shared) if shared is not None else None
        if shared_gate and (self.shared is None or not getattr(self.shared, "takes_row_gate", False)):
            raise ValueError(f"{prefix}: a gate per token needs a shared expert that takes one")
        self.router = self.correction = self.w_gate_up = self.w_down = None

    def _expert(self, i: int, which: str) -> str:
        return f"{self.prefix}{self.names['expert_prefix']}{i}.{self.names[which]}"

    def children(self):
        return [self.shared] if self.shared is not None else []

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        specs = [WeightSpec(self.prefix + self.names["router"], (self.experts, H))]
        if self.has_correction:
            specs.append(WeightSpec(self.prefix + self.names["correction"], (self.experts,)))
        if self.shared_gate:
            specs.append(WeightSpec(self.prefix + self.shared_gate, (1, H)))
        for i in range(self.experts):
            specs += [WeightSpec(self._expert(i, "gate"), (I, H)), WeightSpec(self._expert(i, "up"), (I, H)),
                      WeightSpec(self._expert(i, "down"), (H, I))]
        return specs

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        router = tensors[self.prefix + self.names["router"]]
        if self.shared_gate:
            router = torch.cat([router, tensors[self.prefix + self.shared_gate].reshape(1, -1)], dim=0)
        self.router = Linear(router)
        self.correction = tensors[self.prefix + self.names["correction"]].contiguous() if self.has_correction else None
        # [E, 2I, H] and [E, H, I]. An expert's gate rows, then its up rows; for bfloat16 sizes that the tensor-core
        # kernels take, in blocks (``glu_block`` gate rows, then the up rows of the same outputs), so that one tile of a
        # product holds both halves and applies the activation in its epilogue
        H, I = self.hidden_size, self.intermediate_size
        gate0 = tensors[self._expert(0, "gate")]
        self.glu_block = 0
        if gate0.dtype == torch.bfloat16 and H % 8 == 0 and I % 64 == 0:
            self.glu_block = 128 if I % 128 == 0 else 64
        b = self.glu_block

        def gate_up(i):
            g, u = tensors[self._expert(i, "gate")], tensors[self._expert(i, "up")]
            if not b:
                return torch.cat([g, u], dim=0)
            return torch.stack([g.reshape(I // b, b, H), u.reshape(I // b, b, H)], dim=1).reshape(2 * I, H)

        self.w_gate_up = torch.stack([gate_up(i) for i in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(i, "down")] for i in range(self.experts)]).contiguous()

    def forward(self, x, step, residual):
        T = x.shape[0]
        with phase("router_ms"):
            z = self.router(x, out_dtype=torch.float32)
            ids = torch.empty(T, self.top, dtype=torch.int32, device=x.device)
            wts = torch.empty(T, self.top, dtype=torch.float32, device=x.device)
            gate = torch.empty(T, dtype=torch.float32, device=x.device) if self.shared_gate else None
            K.moe_select(z, self.correction, ids, wts, self.top, self.groups, self.keep_groups,
                         softmax=self.score == "softmax", weight_scale=self.weight_scale, experts=self.experts, extra=gate)
        with phase("experts_ms"):
            K.moe_experts(x, ids, wts, self.w_gate_up, self.w_down, residual, self.top, self.limit, self.slope, self.glu_block)
        if self.shared is not None and self.shared_gate:
            self.shared.forward(x, step, residual, row_gate=gate)
        elif self.shared is not None:
            self.shared.forward(x, step, residual)


@register_part("ffn", "token_side")
class TokenSideInput(FeedForward):
    """A per-layer input chosen by the token (not in the reference): y += P · (gelu(G x) ⊙ S[id_t, offset : offset + dim])
    with S a table [vocab, table_width] that several layers share (each reads its own columns), G [dim, hidden],
    P [hidden, dim] and the tanh form of gelu. ``x`` is whatever the arrangement hands it (the stream itself)."""
    graph_safe = True
    kernel_modules = ("sandwich",)

    def __init__(self, hidden_size: int, dim: int, vocab_size: int, table_width: int, offset: int, table_name: str,
                 prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.dim, self.vocab_size = int(hidden_size), int(dim), int(vocab_size)
        self.table_width, self.offset = int(table_width), int(offset)
        if self.offset < 0 or self.offset + self.dim > self.table_width:
            raise ValueError(f"{prefix}: columns {self.offset}..{self.offset + self.dim} lie outside a table of width {self.table_width}")
        self.table_name = table_name                        # not under the prefix: the table belongs to all its readers
        n = dict(gate="gate", proj="proj")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.table = self.gate = self.proj = None

    def weight_specs(self):
        return [WeightSpec(self.table_name, (self.vocab_size, self.table_width)),
                WeightSpec(self.names["gate"], (self.dim, self.hidden_size)),
                WeightSpec(self.names["proj"], (self.hidden_size, self.dim))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.table = tensors[self.table_name].contiguous()
        self.gate, self.proj = Linear(tensors[self.names["gate"]]), Linear(tensors[self.names["proj"]])

    def forward(self, x, step, residual):
        with phase("side_gate_ms"):
            z = self.gate(x)
            g = torch.empty_like(z)
            K.gelu_gather_mul(z, self.table, step.tokens, g, self.offset)
        with phase("side_projection_ms"):
            self.proj(g, out=residual, accumulate=True)
