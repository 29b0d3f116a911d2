"""Attention through a cached low-rank latent, as a mixer (not in the reference).

    c_q = n(D_q x) ⊙ w_q                 a low-rank image of the token for the queries,  q_h = U_q,h c_q      [dim]
    c   = n(D_kv x) ⊙ w_c                the latent [rank]: the ONLY thing cached, one page row per token
    k_j,h = U_k,h c_j   v_j,h = U_v,h c_j                keys [dim] and values [vdim] of every head are images of c
    score_h(i, j) = (q_i,h · k_j,h) · scale              over the visible j (``window`` w: i − w < j <= i; None: all j <= i)
    p_h(i, j) = e^{score} / (e^{sink_h} + Σ_j e^{score})   a learned per-head sink joins the denominator (``sink`` False: none)
    y += W_o · concat_h(Σ_j p_h(i, j) v_j,h)

n is the RMS norm x / sqrt(mean(x²) + eps). No positions enter. Keys and values are never expanded: since
q · (U_k c) = (U_kᵀ q) · c and Σ p (U_v c) = U_v (Σ p c), the query is carried into the latent's space once per token,
the attention runs over the cached rows themselves (one row is key and value, for all heads), and the weighted sum of
latents is expanded once per token. A layer built with ``shares_latent`` has no D_kv and no norm weight of its own:
it reads the rows another layer cached (a run with ``cache.writes`` False), with its own U_k, U_v, queries, window
and sinks. ``cache_window``: the window the cache keeps rows for when readers with other windows share it (None with
``window`` set: this layer's own).

Two ways to carry the queries in and the sums out. Few tokens (decode steps) and the 32-bit mode take the small
per-head products as they stand: q = U_q c_q, then U_k,hᵀ q_h; U_v,h (Σ p c), then W_o. Prompt portions in bfloat16
take the same maps multiplied out once when the weights are bound,

    A = stack_h(U_k,hᵀ U_q,h)   [heads·rank, q_rank]        B = concat_h(W_o[:, h] U_v,h)   [hidden, heads·rank]

(products in 32-bit, rounded once to bfloat16), so that both are plain matrix products on the tile kernel: more FLOPs
than the small products, but at the tensor cores' rate instead of a per-head loop.

A third way for prompt steps in which EVERY sequence starts at its position 0 (whole prompts: nothing the step's
queries see lies in the cache only), with heads the tcgen05 attention kernel takes (key size = value size = 64 or
128): the step's own latents, kept as rows [tokens, rank] by the kernel that writes them into their pages (a reader
layer finds its writer's rows in the step's scratch), ARE expanded, K = C U_kᵀ and V = C U_vᵀ as two plain products,
and the attention runs over them with the window and the sinks: 2·(dim + vdim) FLOPs per visible pair and head instead
of 4·rank, on the faster kernel. The cache is written all the same; later steps read it.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .attention import attend_paged, length_bucket
from .base import KVCacheRequest, Mixer, WeightSpec
from .linear import Linear
from .registry import register_part
from ..phases import phase

_UNSET = object()
EXPANDED_FROM_TOKENS = 256   # prompt steps from position 0 with at least this many tokens expand their own keys and values
FOLDED_FROM_TOKENS = 64      # steps of more tokens than this take the multiplied-out maps (bfloat16): below, the weights'
#                              bytes decide, and the small products read a third of them


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    kernel_modules = ("latent",)
    kernel_modules_bf16 = ("attention",)

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, q_rank: int, kv_rank: int,
                 scale: float, eps: float, window=None, cache_window=_UNSET, sink: bool = True, shares_latent: bool = False,
                 prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.q_rank, self.kv_rank = int(q_rank), int(kv_rank)
        self.scale, self.eps = float(scale), float(eps)
        self.window = int(window) if window else None
        self.cache_window = self.window if cache_window is _UNSET else (int(cache_window) if cache_window else None)
        if self.cache_window is not None and (self.window is None or self.window > self.cache_window):
            raise ValueError(f"{prefix}: a window of {self.window} sees rows that a cache of {self.cache_window} has returned")
        self.has_sink, self.shares_latent = bool(sink), bool(shares_latent)
        n = dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", sink="sink", o="o")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.down = self.uq = self.o = self.uk = self.uv = self.sink = self.wq_norm = self.wc_norm = None

    def weight_specs(self):
        W, H, d, vd, qr, r = self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim, self.q_rank, self.kv_rank
        n = self.names
        specs = [WeightSpec(n["dq"], (qr, W)), WeightSpec(n["dq_norm"], (qr,), init="ones"), WeightSpec(n["uq"], (H * d, qr)),
                 WeightSpec(n["uk"], (H * d, r)), WeightSpec(n["uv"], (H * vd, r)), WeightSpec(n["o"], (W, H * vd))]
        if not self.shares_latent:
            specs += [WeightSpec(n["dkv"], (r, W)), WeightSpec(n["dkv_norm"], (r,), init="ones")]
        if self.has_sink:
            specs.append(WeightSpec(n["sink"], (H,)))
        return specs

    def cache_request(self):
        return KVCacheRequest(1, self.kv_rank, self.cache_window, keys_only=True)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        dq = tensors[n["dq"]]
        self.down_q = Linear(dq)
        self.down = None if self.shares_latent else Linear(torch.cat([dq, tensors[n["dkv"]]], dim=0))
        self.wq_norm = tensors[n["dq_norm"]].contiguous()
        self.wc_norm = None if self.shares_latent else tensors[n["dkv_norm"]].contiguous()
        self.uq = Linear(tensors[n["uq"]])
        self.uk = tensors[n["uk"]].contiguous()            # [H·dim, rank]: head h's rows are U_k,h, a matrix [dim, rank]
        self.uv = tensors[n["uv"]].contiguous()            # [H·vdim, rank]
        self.o = Linear(tensors[n["o"]])
        # for steps of a few tokens: U_k,h with the latent's entries as its rows, so that both small products stream
        # rows of a matrix stored [out, in]
        self.uk_t = self.uk.view(self.num_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.sink = tensors[n["sink"]].float().contiguous() if self.has_sink else None     # a score: 32-bit
        self.uk_rows, self.uv_rows = Linear(self.uk), Linear(self.uv)                      # K = C U_kᵀ, V = C U_vᵀ
        self.q_fold = self.o_fold = None
        if rt.act_dtype == torch.bfloat16 and all(w.dtype == torch.bfloat16 for w in (self.uk, self.uv, self.uq.weight, self.o.weight)):
            H, d, vd, qr, r = self.num_heads, self.head_dim, self.v_head_dim, self.q_rank, self.kv_rank
            uk, uq = self.uk.float().view(H, d, r), self.uq.weight.float().view(H, d, qr)
            self.q_fold = Linear(torch.bmm(uk.transpose(1, 2), uq).reshape(H * r, qr).to(torch.bfloat16))
            wo, uv = self.o.weight.float().view(-1, H, vd).permute(1, 0, 2), self.uv.float().view(H, vd, r)
            self.o_fold = Linear(torch.bmm(wo, uv).permute(1, 0, 2).reshape(-1, H * r).to(torch.bfloat16))
        # arrival counters of the split-key decode attention; the kernel returns them to zero
        self.counters = torch.zeros(4096, dtype=torch.int32, device=rt.device)

    def forward(self, x, step, cache, residual):
        H, d, vd, qr, r = self.num_heads, self.head_dim, self.v_head_dim, self.q_rank, self.kv_rank
        T, dev, act = x.shape[0], x.device, self.rt.act_dtype
        writes = cache.writes
        if writes and self.shares_latent:
            raise ValueError(f"{self.prefix}: a layer without a latent projection cannot be the writer of a cache")
        with phase("latent_projection_ms"):
            proj = (self.down if writes else self.down_q)(x, out_dtype=torch.float32)     # the norms read unrounded products
        rows_key = ("latent_rows", cache.k_pool.data_ptr())
        expand = (act == torch.bfloat16 and T >= EXPANDED_FROM_TOKENS and d == vd and self.uk.dtype == torch.bfloat16
                  and step.host.get("seq_len") is not None and step.host["seq_len"] == step.host["new_counts"]
                  and (writes or rows_key in step.scratch) and K.flash_tc_rows_supported(act, H, H, d))
        with phase("latent_norm+append_ms"):
            cq = torch.empty(T, qr, dtype=act, device=dev)
            rows = torch.empty(T, r, dtype=act, device=dev) if expand and writes else None
            K.latent_norm_store(proj, qr, r, self.wq_norm, self.wc_norm if writes else None, self.eps, cq,
                                cache.k_pool if writes else None, cache, rows_out=rows)
            if rows is not None:
                step.scratch[rows_key] = rows          # the layers that read this cache expand the same rows
        if expand:
            rows = step.scratch[rows_key]
            with phase("q_projection_ms"):
                q = self.uq(cq)
            with phase("key_value_expansion_ms"):
                k, v = self.uk_rows(rows), self.uv_rows(rows)
            with phase("latent_attention_ms"):
                ctx = torch.empty_like(q)
                tiles = K.query_tiles(step.host["new_counts"], K.flash_tc_query_tile())
                K.flash_prefill_tc_rows(q, k, v, ctx, step, tiles, H, H, d, self.window, self.scale, self.sink)
            with phase("o_projection+attention_residual_ms"):
                self.o(ctx, out=residual, accumulate=True)
            return
        folded = self.q_fold is not None and T > FOLDED_FROM_TOKENS
        if folded:
            with phase("q_projection_ms"):
                qc = self.q_fold(cq)                                                      # (U_k,hᵀ U_q,h) c_q
        else:
            with phase("q_projection_ms"):
                q = self.uq(cq)
            with phase("query_into_latent_space_ms"):
                qc = torch.empty(T, H * r, dtype=act, device=dev)
                if T <= K.HEADWISE_SMALL_TOKENS:
                    K.headwise_product(q, self.uk_t, qc, H, d, r, w_rows_are_k=False)     # U_k,hᵀ q_h
                else:
                    K.headwise_product(q, self.uk, qc, H, d, r, w_rows_are_k=True)
        with phase("latent_attention_ms"):
            mix = self.attend(qc, step, cache)
        if folded:
            with phase("o_projection+attention_residual_ms"):
                self.o_fold(mix, out=residual, accumulate=True)                           # (W_o,h U_v,h) Σ p c
            return
        with phase("value_expansion_ms"):
            ctx = torch.empty(T, H * vd, dtype=act, device=dev)
            K.headwise_product(mix, self.uv, ctx, H, r, vd, w_rows_are_k=False)           # U_v,h (Σ p c)
        with phase("o_projection+attention_residual_ms"):
            self.o(ctx, out=residual, accumulate=True)

    def attend(self, qc, step, cache):
        """Σ_j p_h(i, j) c_j for queries already in the latent's space: [T, heads·rank]. In bfloat16 the kernel that
        fetches a tile of cached rows once for both products where it is built for the rank; else the cache is read as
        one key/value head of size ``rank`` whose value pool is its key pool, by the grouped-query kernels."""
        H, r = self.num_heads, self.kv_rank
        if qc.dtype == torch.bfloat16 and cache.k_pool.dtype == torch.bfloat16 and K.latent_flash_supported(r, cache.page_size):
            mix = torch.empty_like(qc)
            # the keys of a decode step are shared out for the length's bucket, as the grouped-query kernel's are
            max_len = length_bucket(step.max_len, cache.page_size) if step.all_single else None
            K.latent_flash(qc, cache.k_pool, mix, cache, step, H, r, self.window, self.scale, self.sink, max_len=max_len)
            return mix
        return attend_paged(qc, step, cache, H, 1, r, self.window, self.scale, self.sink, self.counters)


@register_part("mixer", "rotary_latent_attention")
class RotaryLatentAttention(Mixer):
    """Attention through a cached low-rank row plus ONE rotated key part that all heads share, with a gate per head
    (not in the reference).

        q_h = [q_h° (dim) | q_h^r (rot_dim)] = W_q,h x,   q_h^r rotated (neighbouring pairs, the position part's
                                                           frequencies, cos and sin times its amplitude)
        [c° | k^r] = D x,   c = n(c°) ⊙ w_c  (rank),   k^r (rot_dim) rotated the same way: what is cached, ONE page row
        score_h(i, j) = ((U_k,h c_j) · q_i,h° + k_j^r · q_i,h^r) · scale    over i − w < j <= i (``window`` w; None: all)
        y += W_o · concat_h( sigmoid(w_g,h · x) · U_v,h Σ_j p_h(i, j) c_j )

    What is cached is never the expanded keys and values. A page row is r_j = [c_j | k_j^r]; with the per-head map
    E_h = [[U_k,hᵀ, 0], [0, I]] the score is (E_h q_i,h) · r_j, so the query is carried into the rows' space once per
    token, the attention runs over the cached rows as they lie (one row is key and value, for all heads), and the
    weighted sum of rows is expanded once per token by [U_v,h | 0]. A layer built with ``shares_latent`` has no D and
    no norm weight: it reads the rows another layer cached (a run with ``cache.writes`` False), with its own q, U_k,
    U_v, gates and window. ``cache_window``: the window the cache keeps rows for when readers with other windows
    share it.

    Three ways through it, chosen per step (bfloat16; the 32-bit mode takes the last): a step of 256 tokens or more in
    which every sequence starts at its first token expands the step's own rows into keys [U_k,h c | k^r] and values
    U_v,h c (two plain products over the rows) and runs on the tcgen05 prompt kernel, where that takes the sizes; other
    steps of more than 64 tokens take both maps multiplied out into the products before and behind them; short steps
    the small per-head products."""
    graph_safe = True
    kernel_modules = ("sandwich", "latent")
    kernel_modules_bf16 = ("attention",)

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int,
                 scale: float, eps: float, position=None, window=None, cache_window=_UNSET, shares_latent: bool = False,
                 prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank = int(head_dim), int(rot_dim), int(v_head_dim), int(kv_rank)
        self.scale, self.eps = float(scale), float(eps)
        self.window = int(window) if window else None
        self.cache_window = self.window if cache_window is _UNSET else (int(cache_window) if cache_window else None)
        if self.cache_window is not None and (self.window is None or self.window > self.cache_window):
            raise ValueError(f"{prefix}: a window of {self.window} sees rows that a cache of {self.cache_window} has returned")
        self.shares_latent = bool(shares_latent)
        n = dict(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", g="g", o="o")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        from .registry import build_part
        self.position = build_part("position", position) if position is not None else None
        if self.rot_dim and (self.position is None or getattr(self.position, "pairing", "half") != "interleaved"
                             or self.position.rotary_dim != self.rot_dim):
            raise ValueError(f"{prefix}: the rotated part of {self.rot_dim} dims needs a rotary part of that size with pairing 'interleaved'")
        self.proj = self.o = self.wc_norm = self.q_map = self.v_map = None

    def children(self):
        return [self.position] if self.position is not None else []

    def weight_specs(self):
        W, H, d, rd, vd, r = self.hidden_size, self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank
        n = self.names
        specs = [WeightSpec(n["q"], (H * (d + rd), W)), WeightSpec(n["uk"], (H * d, r)), WeightSpec(n["uv"], (H * vd, r)),
                 WeightSpec(n["g"], (H, W)), WeightSpec(n["o"], (W, H * vd))]
        if not self.shares_latent:
            specs += [WeightSpec(n["dkv"], (r + rd, W)), WeightSpec(n["dkv_norm"], (r,), init="ones")]
        return specs

    def cache_request(self):
        return KVCacheRequest(1, self.kv_rank + self.rot_dim, self.cache_window, keys_only=True)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        H, d, rd, vd, r = self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank
        q, g = tensors[n["q"]], tensors[n["g"]]
        stack = [q, g] if self.shares_latent else [q, tensors[n["dkv"]], g]
        if len({p.dtype for p in stack}) != 1:
            raise ValueError(f"{self.prefix}: the projections of one input must share a storage type")
        self.proj = Linear(torch.cat(stack, dim=0))                # rows [q | (c° | k^r) | gates]
        self.wc_norm = None if self.shares_latent else tensors[n["dkv_norm"]].contiguous()
        uk, uv = tensors[n["uk"]], tensors[n["uv"]]
        R = r + rd
        # E_h [R, d + rd]: rows of the cached row's space, stored [out, in] like every weight (exact: ones and zeros)
        q_map = torch.zeros(H, R, d + rd, dtype=uk.dtype, device=uk.device)
        q_map[:, :r, :d] = uk.view(H, d, r).transpose(1, 2)
        if rd:
            q_map[:, r:, d:] = torch.eye(rd, dtype=uk.dtype, device=uk.device)
        self.q_map = q_map.contiguous()
        v_map = torch.zeros(H, vd, R, dtype=uv.dtype, device=uv.device)      # [U_v,h | 0]
        v_map[:, :, :r] = uv.view(H, vd, r)
        self.v_map = v_map.contiguous()
        self.o = Linear(tensors[n["o"]])
        # for steps of many tokens (bfloat16) the per-head maps are multiplied out into the products before and behind
        # them: rows [E_h-part of q | rotated part] per head instead of q, so that the kernel that rotates writes the
        # query in the rows' space, and W_o,h [U_v,h | 0] behind the weighted sums of rows (the gate of a head is one
        # number and passes through the map)
        self.proj_fold = self.o_fold = None
        if rt.act_dtype == torch.bfloat16 and all(w.dtype == torch.bfloat16 for w in (q, uk, uv, self.o.weight)):
            wq = q.float().view(H, d + rd, -1)
            folded = torch.cat([torch.bmm(uk.float().view(H, d, r).transpose(1, 2), wq[:, :d]), wq[:, d:]], dim=1)
            stack[0] = folded.reshape(H * R, -1).to(torch.bfloat16)
            self.proj_fold = Linear(torch.cat(stack, dim=0))
            wo = self.o.weight.float().view(-1, H, vd).permute(1, 0, 2)
            fold = torch.zeros(H, wo.shape[1], R, dtype=torch.float32, device=wo.device)
            fold[:, :, :r] = torch.bmm(wo, uv.float().view(H, vd, r))
            self.o_fold = Linear(fold.permute(1, 0, 2).reshape(-1, H * R).to(torch.bfloat16))
        # whole prompts expand their own rows into keys [U_k,h c | k^r] and values U_v,h c per head and run on the
        # tcgen05 attention kernel where it takes the sizes: the maps as plain products over the rows (E_hᵀ and [U_v,h | 0])
        self.k_rows = self.v_rows = None
        if (rt.act_dtype == torch.bfloat16 and uk.dtype == torch.bfloat16 and uv.dtype == torch.bfloat16
                and K.flash_tc_rows_supported(torch.bfloat16, H, H, d + rd, vd)):
            self.k_rows = Linear(self.q_map.transpose(1, 2).reshape(H * (d + rd), R).contiguous())
            self.v_rows = Linear(self.v_map.reshape(H * vd, R))
        self.counters = torch.zeros(4096, dtype=torch.int32, device=rt.device)

    def forward(self, x, step, cache, residual):
        H, d, rd, vd, r = self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank
        T, dev, act, R = x.shape[0], x.device, self.rt.act_dtype, self.kv_rank + self.rot_dim
        rows_key = ("latent_rows", cache.k_pool.data_ptr())
        if (self.k_rows is not None and T >= EXPANDED_FROM_TOKENS and step.host.get("seq_len") is not None
                and step.host["seq_len"] == step.host["new_counts"] and (cache.writes or rows_key in step.scratch)):
            return self._forward_expanded(x, step, cache, residual, rows_key)
        if self.proj_fold is not None and T > FOLDED_FROM_TOKENS:
            return self._forward_folded(x, step, cache, residual)
        writes = cache.writes
        if writes and self.shares_latent:
            raise ValueError(f"{self.prefix}: a layer without a latent projection cannot be the writer of a cache")
        freq, amp = (self.position.rotary()[0], getattr(self.position, "amplitude", 1.0)) if rd else (None, 1.0)
        with phase("latent_projection_ms"):
            proj = self.proj(x, out_dtype=torch.float32)            # norm and rotation read unrounded products
        with phase("latent_norm+rotary+append_ms"):
            q = torch.empty(T, H * (d + rd), dtype=act, device=dev)
            gates = torch.empty(T, H, dtype=torch.float32, device=dev)
            K.latent_rot_store(proj, self.wc_norm if writes else None, q, cache.k_pool if writes else None, cache, gates, freq,
                               H, d, rd, r, amp, self.eps)
        with phase("query_into_latent_space_ms"):
            qx = torch.empty(T, H * R, dtype=act, device=dev)
            K.headwise_product(q, self.q_map, qx, H, d + rd, R, w_rows_are_k=False)              # E_h q_h
        with phase("latent_attention_ms"):
            mix = self._attend_rows(qx, step, cache)
        with phase("value_expansion_ms"):
            ctx = torch.empty(T, H * vd, dtype=act, device=dev)
            K.headwise_product(mix, self.v_map, ctx, H, R, vd, w_rows_are_k=False)               # U_v,h (Σ p c)
        with phase("head_gate_ms"):
            K.scale_rows_sigmoid(ctx.view(T * H, vd), gates.view(T * H))
        with phase("o_projection+attention_residual_ms"):
            self.o(ctx, out=residual, accumulate=True)

    def _attend_rows(self, qx, step, cache):
        """Σ_j p_h(i, j) [c_j | k_j^r] for queries in the rows' space: [T, heads·(rank + rot_dim)]."""
        H, R, act = self.num_heads, self.kv_rank + self.rot_dim, self.rt.act_dtype
        if act == torch.bfloat16 and cache.k_pool.dtype == torch.bfloat16 and K.latent_flash_supported(R, cache.page_size):
            mix = torch.empty_like(qx)
            max_len = length_bucket(step.max_len, cache.page_size) if step.all_single else None
            K.latent_flash(qx, cache.k_pool, mix, cache, step, H, R, self.window, self.scale, None, max_len=max_len)
            return mix
        return attend_paged(qx, step, cache, H, 1, R, self.window, self.scale, None, self.counters)

    def _forward_expanded(self, x, step, cache, residual, rows_key):
        """A step in which every sequence starts at its first token: the step's own rows, expanded, are all the keys and
        values there are. The writer leaves its rows in the step's scratch for the layers that read its cache."""
        H, d, rd, vd, r = self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank
        T, dev, act, R = x.shape[0], x.device, self.rt.act_dtype, self.kv_rank + self.rot_dim
        writes = cache.writes
        if writes and self.shares_latent:
            raise ValueError(f"{self.prefix}: a layer without a latent projection cannot be the writer of a cache")
        freq, amp = (self.position.rotary()[0], getattr(self.position, "amplitude", 1.0)) if rd else (None, 1.0)
        with phase("latent_projection_ms"):
            proj = self.proj(x, out_dtype=torch.float32)
        with phase("latent_norm+rotary+append_ms"):
            q = torch.empty(T, H * (d + rd), dtype=act, device=dev)
            gates = torch.empty(T, H, dtype=torch.float32, device=dev)
            rows = torch.empty(T, R, dtype=act, device=dev) if writes else None
            K.latent_rot_store(proj, self.wc_norm if writes else None, q, cache.k_pool if writes else None, cache, gates, freq,
                               H, d, rd, r, amp, self.eps, rows_out=rows)
            if writes:
                step.scratch[rows_key] = rows
        rows = step.scratch[rows_key]
        with phase("key_value_expansion_ms"):
            k, v = self.k_rows(rows), self.v_rows(rows)
        with phase("latent_attention_ms"):
            ctx = torch.empty(T, H * vd, dtype=act, device=dev)
            tiles = K.query_tiles(step.host["new_counts"], K.flash_tc_query_tile())
            K.flash_prefill_tc_rows(q, k, v, ctx, step, tiles, H, H, d + rd, self.window, self.scale, None, vd=vd)
        with phase("head_gate_ms"):
            K.scale_rows_sigmoid(ctx.view(T * H, vd), gates.view(T * H))
        with phase("o_projection+attention_residual_ms"):
            self.o(ctx, out=residual, accumulate=True)

    def _forward_folded(self, x, step, cache, residual):
        H, rd, r = self.num_heads, self.rot_dim, self.kv_rank
        T, dev, act, R = x.shape[0], x.device, self.rt.act_dtype, self.kv_rank + self.rot_dim
        writes = cache.writes
        if writes and self.shares_latent:
            raise ValueError(f"{self.prefix}: a layer without a latent projection cannot be the writer of a cache")
        freq, amp = (self.position.rotary()[0], getattr(self.position, "amplitude", 1.0)) if rd else (None, 1.0)
        with phase("latent_projection_ms"):
            proj = self.proj_fold(x, out_dtype=torch.float32)
        with phase("latent_norm+rotary+append_ms"):
            qx = torch.empty(T, H * R, dtype=act, device=dev)
            gates = torch.empty(T, H, dtype=torch.float32, device=dev)
            # the unrotated part of a head's query is already in the rows' space: ``rank`` entries instead of ``dim``
            K.latent_rot_store(proj, self.wc_norm if writes else None, qx, cache.k_pool if writes else None, cache, gates, freq,
                               H, r, rd, r, amp, self.eps)
        with phase("latent_attention_ms"):
            mix = self._attend_rows(qx, step, cache)
        with phase("head_gate_ms"):
            K.scale_rows_sigmoid(mix.view(T * H, R), gates.view(T * H))
        with phase("o_projection+attention_residual_ms"):
            self.o_fold(mix, out=residual, accumulate=True)                                   # (W_o,h [U_v,h | 0]) g_h Σ p r
