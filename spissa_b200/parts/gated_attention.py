"""Causal grouped-query attention with a gate per head on its output, as a mixer (not in the reference).

    q = Wq x (+ bq),  k = Wk x (+ bk),  v = Wv x (+ bv)          per head: q, k of size dim, v of size vdim
    q_t ← q_t · (1 + coef · ln(⌊(t + 1) / every⌋ + 1))            (``q_temp``: the query grows with its position t)
    rotation of neighbouring pairs over the first dims of q and k  (``position``: a rotary part with pairing "interleaved")
    s_h(i, j) = (q_i,h · k_j,g(h)) · scale + R[row(i − j), h]     (``distance_rows`` rows of a learned table R; the scale
                                                                    does not multiply it)
    p_h(i, j) = e^{s} / (Σ_j e^{s} (+ e^{sink_h}))                 over the visible j ≤ i (``window`` w: i − j < w);
                                                                    ``sink``: a learned score per head, no key, no value
    y += Wo · concat_h( sigmoid(w_g,h · x) · Σ_j p_h(i, j) v_j,g(h) )

Rows of the distance table, for B rows and the distance ``distance_far`` = D at which the last row is reached: distances
n < B/2 have a row each; n ≥ B/2 takes row min(B − 1, B/2 + ⌊ln(n / (B/2)) / ln(D / (B/2)) · (B − B/2)⌋). When the weights
are bound the table is spread out by distance once, [heads, distances up to the first that takes the last row], so
that the attention kernels look a score up by min(i − j, last).

Every option is a constructor parameter; a mixer without any of them is a grouped-query attention with a gate. The
projections of q, k, v and the gates run as ONE product over the stacked weight; one kernel then adds the biases,
applies the query factor and the rotation, writes q and the cache rows and hands the gates' arguments on. Scores,
softmax, gates, angles and the factor are 32-bit in every mode.
"""
from __future__ import annotations

import math

import torch

from ..csrc import lib as K
from .attention import attend_paged
from .base import KVCacheRequest, Mixer, WeightSpec
from .linear import Linear
from .registry import build_part, register_part
from ..phases import phase


def distance_row(n: int, rows: int, far: float) -> int:
    """The row of a table of ``rows`` rows that the distance ``n`` takes (see the module's text)."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_table(rel: torch.Tensor, far: float) -> torch.Tensor:
    """``rel`` [rows, heads] -> float32 [heads, distances]: entry n is the row that distance n takes; the last entry
    stands for every larger distance."""
    rows = rel.shape[0]
    picks, n = [], 0
    while True:
        r = distance_row(n, rows, far)
        picks.append(r)
        if r >= rows - 1 or n > (1 << 22):
            break
        n += 1
    idx = torch.tensor(picks, dtype=torch.long, device=rel.device)
    return rel.float().index_select(0, idx).t().contiguous()


@register_part("mixer", "gated_attention")
class GatedAttention(Mixer):
    graph_safe = True
    kernel_modules = ("sandwich",)
    kernel_modules_bf16 = ("attention",)

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float,
                 bias: bool = False, q_temp: tuple | None = None, distance_rows: int = 0, distance_far: float = 0.0,
                 position=None, sink: bool = False, window=None, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim, self.scale = int(head_dim), int(v_head_dim), float(scale)
        self.bias, self.has_sink = bool(bias), bool(sink)
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None          # (coef, every)
        # rows of the distance table; negative −n: the checkpoint's tensor decides (random weights take n)
        self.distance_rows, self.distance_far = int(distance_rows), float(distance_far)
        self.window = int(window) if window else None
        n = dict(q="q", k="k", v="v", g="g", o="o", rel="rel", sink="sink", bias_suffix=".b")
        n.update(names or {})
        self.bias_suffix = n.pop("bias_suffix")
        self.names = {k: prefix + v for k, v in n.items()}
        self.position = build_part("position", position) if position is not None else None
        if self.position is not None and getattr(self.position, "pairing", "half") != "interleaved":
            raise ValueError(f"{prefix}: this mixer's kernel rotates neighbouring pairs (pairing 'interleaved')")
        self.proj = self.o = self.qkv_bias = self.sink = self.dist = None

    def children(self):
        return [self.position] if self.position is not None else []

    def _shapes(self):
        W, nh, g, d, vd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        return dict(q=(nh * d, W), k=(g * d, W), v=(g * vd, W))

    def weight_specs(self):
        W, nh, vd = self.hidden_size, self.num_heads, self.v_head_dim
        specs = [WeightSpec(self.names[k], s) for k, s in self._shapes().items()]
        specs += [WeightSpec(self.names["g"], (nh, W)), WeightSpec(self.names["o"], (W, nh * vd))]
        if self.bias:
            specs += [WeightSpec(self.names[k] + self.bias_suffix, (s[0],)) for k, s in self._shapes().items()]
        if self.distance_rows:
            specs.append(WeightSpec(self.names["rel"], (self.distance_rows, nh)))
        if self.has_sink:
            specs.append(WeightSpec(self.names["sink"], (nh,)))
        return specs

    def cache_request(self):
        vd = self.v_head_dim if self.v_head_dim != self.head_dim else None
        return KVCacheRequest(self.num_kv_heads, self.head_dim, self.window, v_head_dim=vd)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        parts = [tensors[self.names[k]] for k in ("q", "k", "v", "g")]
        if len({p.dtype for p in parts}) != 1:
            raise ValueError(f"{self.prefix}: the projections of q, k, v and the gates must share a storage type")
        self.proj = Linear(torch.cat(parts, dim=0))
        self.o = Linear(tensors[self.names["o"]])
        if self.bias:
            self.qkv_bias = torch.cat([tensors[self.names[k] + self.bias_suffix] for k in ("q", "k", "v")]).contiguous()
        self.sink = tensors[self.names["sink"]].float().contiguous() if self.has_sink else None        # a score: 32-bit
        self.dist = None
        if self.distance_rows:
            rel = tensors[self.names["rel"]]
            if rel.shape[0] < 2 or not self.distance_far > rel.shape[0] // 2:
                raise ValueError(f"{self.prefix}: a distance table of {rel.shape[0]} rows and a last row reached at "
                                 f"{self.distance_far} do not fit together")
            self.dist = distance_table(rel, self.distance_far)
        # arrival counters of the split-key decode attention; the kernel returns them to zero
        self.counters = torch.zeros(4096, dtype=torch.int32, device=rt.device)

    def forward(self, x, step, cache, residual):
        nh, g, d, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        T, dev, act = x.shape[0], x.device, self.rt.act_dtype
        freq, rd, amp = None, 0, 1.0
        if self.position is not None:
            freq, rd = self.position.rotary()
            amp = getattr(self.position, "amplitude", 1.0)
        with phase("qkv_projection_ms"):
            proj = self.proj(x, out_dtype=torch.float32)            # biases, factor and rotation read unrounded products
        with phase("rotary+kv_append_ms"):
            q = torch.empty(T, nh * d, dtype=act, device=dev)
            gates = torch.empty(T, nh, dtype=torch.float32, device=dev)
            coef, every = self.q_temp or (0.0, 1)
            K.gated_qkv_store(proj, self.qkv_bias, q, cache.k_pool, cache.v_pool, cache, gates, freq, nh, g, d, vd, rd,
                              write_kv=cache.writes, rot_mult=amp, temp_coef=coef, temp_every=every)
        with phase("distance_attention_ms" if self.dist is not None else "attention_ms"):
            ctx = self.attend(q, step, cache)
        with phase("head_gate_ms"):
            K.scale_rows_sigmoid(ctx.view(T * nh, vd), gates.view(T * nh))
        with phase("o_projection+attention_residual_ms"):
            self.o(ctx, out=residual, accumulate=True)

    def attend(self, q, step, cache):
        """The heads' outputs [T, heads·vdim] over the cached keys and values, the step's own included."""
        nh, g, d, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        if d == vd:
            return attend_paged(q, step, cache, nh, g, d, self.window, self.scale, self.sink, self.counters, dist_bias=self.dist)
        T = q.shape[0]
        ctx = torch.empty(T, nh * vd, dtype=q.dtype, device=q.device)
        K.attention_generic(q, cache.k_pool, cache.v_pool, ctx, cache, nh, g, d, self.window, self.scale, vd=vd,
                            sink=self.sink, dist_bias=self.dist)
        return ctx
