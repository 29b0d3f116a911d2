"""Token embedding and output head.

Embedding: h[t,:] = E[id_t,:] (crates/spissa-runtime/src/ops.rs:6-30), times ``scale`` where a
model has one (1, the default, for the reference's models); the rows enter the 32-bit residual stream. Head: logits = x · Wᵀ with W either its own
tensor or the embedding table when the model ties them
(crates/spissa-runtime/src/models/llama/api.rs:176-181, :336-346); logits are 32-bit.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import Part, StateRequest, WeightSpec
from .linear import Linear
from .registry import register_part


@register_part("embedding", "embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, prefix: str = "", weight_name: str = "weight",
                 scale: float = 1.0):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight_name = prefix + weight_name
        self.scale = float(scale)                  # multiplies the rows on their way into the stream (not the table)
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.weight_name].contiguous()

    def fused_fields(self):
        """What a runner that gathers the rows itself needs: the table [vocab, hidden] (bfloat16)."""
        if self.weight is None or self.weight.dtype != torch.bfloat16 or type(self) is not TokenEmbedding \
                or self.scale != 1.0:
            return None
        return dict(kind="token_embedding", weight=self.weight, vocab_size=self.vocab_size, hidden_size=self.hidden_size)

    def forward(self, step) -> torch.Tensor:
        """The residual stream [T, H] (float32) of the step's tokens. An embedding that needs more than the token ids
        (positions, for a learned position table) finds it in ``step``. A token id outside the table gives a zero row
        and a fault code in the device's status word (ids that come from the host are checked there already)."""
        ids = step.tokens
        out = torch.empty(ids.shape[0], self.hidden_size, dtype=torch.float32, device=ids.device)
        K.embed_gather(self.weight, ids, out, K.status_word(ids.device), self.scale)
        return out


@register_part("embedding", "pair_embedding")
class PairEmbedding(TokenEmbedding):
    """The token's row times ``scale`` plus a row of a second table chosen by the token and the one before it (not in
    the reference): row (id_{t−1} · mul_prev + id_t · mul_cur) mod buckets of ``pair_name`` [buckets + 1, hidden]; a
    sequence's first token has no token before it and takes the last row. The token before a step's first one is a
    word of per-slot state (``cache_request``): the kernel reads it and leaves the step's last token there."""
    graph_safe = True
    kernel_modules = ("sandwich",)

    def __init__(self, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, prefix: str = "",
                 weight_name: str = "weight", pair_name: str = "pairs", scale: float = 1.0):
        super().__init__(vocab_size, hidden_size, prefix, weight_name, scale)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if self.buckets <= 0:
            raise ValueError(f"{prefix}: the pair table needs at least one bucket")
        self.pair_name = prefix + pair_name
        self.pairs = None

    def weight_specs(self):
        return super().weight_specs() + [WeightSpec(self.pair_name, (self.buckets + 1, self.hidden_size))]

    def cache_request(self):
        return StateRequest((1,), torch.int32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.pairs = tensors[self.pair_name].contiguous()
        if self.pairs.dtype != self.weight.dtype:
            raise ValueError(f"{self.prefix}: the token table and the pair table must share a storage type")

    def fused_fields(self):
        return None

    def forward(self, step, cache=None) -> torch.Tensor:
        if cache is None:
            raise ValueError(f"{self.prefix}: this embedding needs its per-slot state (the token before the step)")
        ids = step.tokens
        out = torch.empty(ids.shape[0], self.hidden_size, dtype=torch.float32, device=ids.device)
        K.pair_embed(self.weight, self.pairs, step, cache.state, out, self.buckets, self.mul_prev, self.mul_cur, self.scale,
                     K.status_word(ids.device))
        return out


@register_part("head", "lm_head")
class LMHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: str | None = None, prefix: str = "",
                 weight_name: str = "weight", softcap: float | None = None):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.softcap = float(softcap) if softcap else None       # logits ← cap · tanh(logits / cap)
        self.tied_to = tied_to
        self.weight_name = prefix + weight_name
        self.proj = None

    def weight_specs(self):
        return [] if self.tied_to else [WeightSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.proj = Linear(tensors[self.tied_to or self.weight_name])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.proj(x, out_dtype=torch.float32)
        if self.softcap:
            K.softcap(logits, self.softcap)
        return logits

    def fused_fields(self):
        """What a runner that computes the head itself needs: the weight [vocab, hidden] (bfloat16, contiguous)."""
        w = self.proj.weight if self.proj is not None else None
        if self.softcap:
            return None                     # the runners' heads write uncapped logits (a greedy choice needs no cap: ``greedy``)
        if w is None or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.data_ptr() % 16:
            return None
        return dict(kind="linear_head", weight=w, vocab_size=self.vocab_size, hidden_size=self.hidden_size)

    def greedy(self, x: torch.Tensor, note=None):
        """The index of the largest logit of every row (int32 [rows]) without the logits, as the reference's greedy
        head keeps only (best index, best value) while it streams the rows
        (crates/spissa-runtime/src/streaming/linear_argmax.rs:13, streaming/argmax.rs:30-51): the lowest index wins
        among equal logits (a cap of the logits is increasing, so it changes no choice and is left out). None when no kernel takes these operands (the caller then asks for the logits).
        ``note``: the tokens also go into the per-slot headers (an engine's ``step_note()``)."""
        w = self.proj.weight
        if not K.head_argmax_supported(x, w):
            return None
        rows = x.shape[0]
        n_cand = K.head_argmax_candidates(rows, w.shape[0])
        cand = torch.empty(rows, n_cand, 2, dtype=torch.float32, device=x.device)
        out = torch.empty(rows, dtype=torch.int32, device=x.device)
        K.head_argmax(x, w, cand, out, note)
        return out
