"""The Kugirax parts and the whole decoder against the plain implementation in ``plain/kugirax_plain.py``.

Each mechanism alone (kernel against its formula: the norms of a projected row and the latent's page row, the small
per-head products, attention over cached latents with a window and a sink on every kernel that can serve it, sinks in
the grouped-query kernels, values that are the convolved keys, the softmax router with the gate of the shared expert,
the capped logits), then small models with random weights under every way of cutting the work: whole prompts,
token-by-token decoding, portions down to two tokens, batches of unequal requests, slots and pages used again, long
decoding with windows that pass over decoded tokens, greedy generation through ``Engine.generate``, the trace program
and the command line. Where random weights would hide a fault (one key among many, the window's edge, the sink), the
weights or inputs are made so that it shows.
"""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import tiny
import traces
from plain import kugirax_plain as P
from plain.llama_plain import read_model_folder
from spissa_b200 import Engine, SamplingParams
from spissa_b200.config import config_from_dict
from spissa_b200.weights import write_random_model, write_safetensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def conv_mixer(heads, kv, dim, conv=None, rot=None, base=10000.0, scale=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale or 1.0 / math.sqrt(dim))
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    return m


def latent_mixer(heads, dim, vdim, q_rank, kv_rank, window, scale=None, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale or 1.0 / math.sqrt(dim),
             mask=dict(size=window))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, scale=1.0, shared=None):
    out = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale))
    if shared:
        out["shared"] = dict(ff=shared)
    return out


def dense(ff):
    return dict(kind="dense", ff=ff)


def att(mixer, mlp):
    return dict(type="attention", mixer=mixer, mlp=mlp)


def lat(mixer, mlp):
    return dict(type="latent_attention", mixer=mixer, mlp=mlp)


def model(width, vocab, layers, cap=20.0, eps=1e-5):
    out = dict(architecture="Kugirax", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if cap:
        out["logit_softcap"] = cap
    return out


# sizes that differ from one another everywhere: grouped, multi-head and single-kv-head attention; convolutions of 2 to
# 5 taps or none; rotation over a part of the dims, all of them or none; latents of a rank that the tensor-core kernel
# takes (128) and of ranks it does not; key and value sizes of the latent heads equal or not; query and latent ranks
# equal or not; windows of one token, below a page, above a page and above two; readers of another layer's rows with a
# smaller and with a larger window than the writer's, two readers of one writer; dense and routed feed-forwards with
# and without a shared expert, all experts chosen or one; layers without a feed-forward; with and without a cap
CONFIGS = {
    "a": model(64, 200, [lat(latent_mixer(3, 8, 12, 20, 24, 9), dense(56)),
                         att(conv_mixer(4, 2, 16, conv=4, rot=8, base=1000.0), moe(6, 2, 16, 1.5, shared=24)),
                         lat(latent_mixer(2, 16, 4, 10, 24, 70, kv_from=0), None),
                         att(conv_mixer(3, 3, 8), moe(3, 3, 8)),
                         lat(latent_mixer(4, 4, 4, 16, 24, 20, kv_from=0), dense(40))], cap=12.0, eps=1e-4),
    "b": model(128, 333, [att(conv_mixer(4, 1, 32, conv=3, rot=32), dense(96)),
                          lat(latent_mixer(5, 16, 32, 48, 128, 100), moe(8, 3, 32, 2.0, shared=16)),
                          att(conv_mixer(2, 2, 64, conv=2, rot=16, base=50.0), None),
                          lat(latent_mixer(2, 32, 16, 128, 128, 33, kv_from=1), moe(4, 1, 24, 0.5))], cap=30.0),
    # nothing a multiple of four: the paths without wide loads; a window of one token sees the token itself and the sink
    "c": model(50, 97, [lat(latent_mixer(2, 5, 7, 9, 11, 1), moe(5, 2, 10, 1.0, shared=14)),
                        att(conv_mixer(3, 1, 10, conv=5, rot=6, base=300.0), dense(30)),
                        lat(latent_mixer(1, 6, 3, 13, 11, 130, kv_from=0), dense(22))], cap=None, eps=1e-3),
    "d": model(96, 150, [att(conv_mixer(6, 3, 16, rot=16), moe(7, 7, 8, 1.25)),
                         lat(latent_mixer(2, 24, 24, 32, 40, 65), None),
                         lat(latent_mixer(3, 8, 16, 24, 256, 140), dense(64))], cap=8.0),
}
INIT = {"a": dict(seed=5, std=0.1, norm_std=0.2), "b": dict(seed=9, std=0.07, norm_std=0.1),
        "c": dict(seed=13, std=0.12, norm_std=0.3), "d": dict(seed=17, std=0.09, norm_std=0.2)}


def make(cfg, folder, seed, std, norm_std, patch=None):
    write_random_model(config_from_dict(cfg), folder, seed=seed, std=std, norm_std=norm_std)
    pcfg, w = read_model_folder(folder)
    # the random-weights mode gives every tap one value and sinks close to zero: spread them, so that a tap taken from
    # the wrong token, a sink left out or scaled, or a router whose scores lie close together shows
    g = torch.Generator().manual_seed(seed)
    for name in sorted(w):
        last = name.split(".")[-1]
        if last == "conv":
            w[name] = torch.randn(w[name].shape, generator=g).to(w[name].dtype)
        elif last == "sink":
            w[name] = (1.5 * torch.randn(w[name].shape, generator=g)).to(w[name].dtype)
        elif last == "router":
            w[name] = (5.0 * w[name].float()).to(w[name].dtype)
        elif last == "sg":
            w[name] = (4.0 * w[name].float()).to(w[name].dtype)
    if patch:
        patch(w)
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    return read_model_folder(folder)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"kx_{name}")
        pcfg, w = make(cfg, folder, **INIT[name])
        out[name] = SimpleNamespace(folder=str(folder), cfg=pcfg, w=w, vocab=cfg["vocab"])
    return out


def worst(got, ref):
    return float((got.double().cpu() - ref.double()).abs().max() / ref.abs().max())


def logits_of(m, toks):
    return P.forward(m.cfg, m.w, toks)


# ---------------------------------------------------------------------------------------------- each mechanism alone
def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


class Paged:
    """Sequences in scattered pages, fed in steps: the arrays a kernel wants of each step."""

    def __init__(self, pages, n_pages, heads, dim, dtype=torch.float32, with_values=False):
        self.pages, self.at = pages, [0] * len(pages)
        width = max(len(p) for p in pages)
        table = torch.zeros(len(pages) + 1, width, dtype=torch.int32)
        for b, p in enumerate(pages):
            table[b + 1, :len(p)] = torch.tensor(p)                  # row 0 of the table belongs to nobody
        self.table = table.to(DEV)
        self.k_pool = torch.zeros(n_pages, heads, PAGE, dim, dtype=dtype, device=DEV)
        self.v_pool = torch.zeros(n_pages, heads, PAGE, dim, dtype=dtype, device=DEV) if with_values else self.k_pool

    def step(self, counts):
        """``counts[b]`` new tokens of sequence b (0: it sits this step out) -> (step, view, live sequences)."""
        live = [b for b, n in enumerate(counts) if n > 0]
        ns = [counts[b] for b in live]
        starts = [0]
        for n in ns:
            starts.append(starts[-1] + n)
        seq = [i for i, n in enumerate(ns) for _ in range(n)]
        pos = [self.at[b] + t for b, n in zip(live, ns) for t in range(n)]
        for b, n in zip(live, ns):
            self.at[b] += n
        lens = [self.at[b] for b in live]
        step = SimpleNamespace(seq_start=i32(starts), seq_slot=i32(live), token_seq=i32(seq), positions=i32(pos),
                               n_seqs=len(live), all_single=all(n == 1 for n in ns), max_new=max(ns), max_len=max(lens),
                               seq_len=i32(lens), host=dict(new_counts=list(ns)))
        view = SimpleNamespace(k_pool=self.k_pool, v_pool=self.v_pool, page_table=self.table, page_size=PAGE,
                               token_seq=step.token_seq, positions=step.positions, seq_slot=i32([b + 1 for b in live]),
                               window=None, writes=True)
        return step, view, live

    def rows(self, b, n, pool=None):
        pool = self.k_pool if pool is None else pool
        return torch.cat([pool[p].permute(1, 0, 2) for p in self.pages[b]])[:n].cpu()


@pytest.mark.parametrize("qr,rank,dtype", [(20, 24, torch.float32), (9, 11, torch.float32), (128, 128, torch.bfloat16),
                                           (300, 7, torch.float32), (1, 1, torch.float32)])
def test_norms_of_a_projected_row_and_the_latent_in_its_page_row(qr, rank, dtype):
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(qr + rank)
    lengths, eps = [70, 9, 131], 1e-3
    world = Paged([[7, 3], [5], [1, 9, 4]], 12, 1, rank, dtype)
    proj = [3 * torch.randn(n, qr + rank, generator=g) + 0.5 for n in lengths]
    wq, wc = torch.randn(qr, generator=g).to(dtype), torch.randn(rank, generator=g).to(dtype)
    got_q = [[], [], []]
    cuts = [[5, 1, 1, 63, 0], [2, 1, 1, 5, 0], [64, 1, 1, 1, 64]]
    for s in range(5):
        at = list(world.at)
        step, view, live = world.step([c[s] for c in cuts])
        rows = torch.cat([proj[b][at[b]:at[b] + cuts[b][s]] for b in live]).to(DEV)
        cq = torch.empty(rows.shape[0], qr, dtype=dtype, device=DEV)
        K.latent_norm_store(rows, qr, rank, wq.to(DEV), wc.to(DEV), eps, cq, world.k_pool, view)
        o = 0
        for b in live:
            got_q[b].append(cq[o:o + cuts[b][s]].cpu())
            o += cuts[b][s]
    tol = 2e-6 if dtype == torch.float32 else 6e-3
    for b, n in enumerate(lengths):
        x = proj[b].double()
        assert worst(torch.cat(got_q[b]), P.rms_norm(x[:, :qr], wq.double(), eps)) <= tol
        assert worst(world.rows(b, n)[:, 0], P.rms_norm(x[:, qr:], wc.double(), eps)) <= tol
    # a reader of another layer's rows norms its query part only, and writes no page
    before = world.k_pool.clone()
    step, view, live = Paged([[2]], 12, 1, rank, dtype).step([4])
    cq = torch.empty(4, qr, dtype=dtype, device=DEV)
    K.latent_norm_store(proj[0][:4, :qr].contiguous().to(DEV), qr, rank, wq.to(DEV), None, eps, cq, None, view)
    assert worst(cq, P.rms_norm(proj[0][:4, :qr].double(), wq.double(), eps)) <= tol
    assert torch.equal(before, world.k_pool)


@pytest.mark.parametrize("H,Kd,N,dtype", [(3, 8, 24, torch.float32), (2, 5, 7, torch.float32), (6, 32, 128, torch.bfloat16),
                                          (1, 130, 3, torch.float32), (4, 128, 16, torch.bfloat16)])
def test_small_products_head_by_head(H, Kd, N, dtype):
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(H * Kd + N)
    w = torch.randn(H, Kd, N, generator=g).to(dtype)
    tol = 2e-6 if dtype == torch.float32 else 6e-3
    for T in (37, 1, 8, 16, 17):                              # a few tokens take a kernel of their own (a warp per weight row)
        a = torch.randn(T, H, Kd, generator=g).to(dtype)
        ref = torch.einsum("thk,hkn->thn", a.double(), w.double()).reshape(T, H * N)
        for rows_are_k, stored in ((True, w), (False, w.transpose(1, 2))):
            out = torch.empty(T, H * N, dtype=dtype, device=DEV)
            K.headwise_product(a.reshape(T, -1).to(DEV), stored.contiguous().reshape(-1, stored.shape[-1]).to(DEV), out, H, Kd, N,
                               w_rows_are_k=rows_are_k)
            assert worst(out, ref) <= tol, (T, rows_are_k)


def _attention_case(H, r, nkv, dtype, seed, lengths, needle_at):
    """Queries, keys and values with one key per sequence (at ``needle_at``) that every query scores far above the
    rest, so that a window that is one token off, or a page walked wrongly, moves the result by much more than rounding."""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(r, generator=g)
    u = u / u.norm()
    q = [(torch.randn(n, H, r, generator=g) + 4.0 * u).to(dtype) for n in lengths]
    k = [torch.randn(n, nkv, r, generator=g) for n in lengths]
    for b, at in enumerate(needle_at):
        if at is not None:
            k[b][at] = k[b][at] + 5.0 * u
    return q, [x.to(dtype) for x in k]


def _run_attention(world, q, k, cuts, call, v=None):
    """Feed the sequences in steps; rows are written to their pages by hand just before the step that brings them."""
    got = [[] for _ in q]
    for s in range(len(cuts[0])):
        at = list(world.at)
        counts = [c[s] for c in cuts]
        if not any(counts):
            continue
        step, view, live = world.step(counts)
        for b in live:
            for t in range(at[b], at[b] + counts[b]):
                world.k_pool[world.pages[b][t // PAGE], :, t % PAGE] = k[b][t].to(DEV)
                if v is not None:
                    world.v_pool[world.pages[b][t // PAGE], :, t % PAGE] = v[b][t].to(DEV)
        rows = torch.cat([q[b][at[b]:at[b] + counts[b]] for b in live])
        out = call(rows.reshape(rows.shape[0], -1).to(DEV).contiguous(), step, view)
        o = 0
        for b in live:
            got[b].append(out[o:o + counts[b]].cpu())
            o += counts[b]
    return [torch.cat(x) for x in got]


LAT_LENGTHS = [200, 70, 131]
LAT_PAGES = [[7, 3, 11, 2], [5, 8], [1, 9, 4]]
# whole; portions that end and start at page borders; short portions and single tokens, a sequence that ends earlier
LAT_CUTS = ([[200], [70], [131]],
            [[64, 64, 72], [2, 3, 65], [100, 1, 1] + [1] * 8],
            [[150] + [1] * 50, [30] + [1] * 40 + [0] * 10, [81] + [1] * 50])


def _fix_cuts(cuts):
    """Pad the per-sequence lists to one length and let the last step bring what is left of each sequence."""
    n = max(len(c) for c in cuts)
    out = []
    for c, total in zip(cuts, LAT_LENGTHS):
        c = list(c) + [0] * (n - len(c))
        rest = total - sum(c)
        out.append(c + [rest])
    return out


@pytest.mark.parametrize("window", [None, 1, 9, 64, 70, 130])
@pytest.mark.parametrize("kind,H,r", [("generic", 3, 24), ("generic", 2, 11), ("flash", 5, 64), ("latent", 6, 128),
                                      ("latent", 3, 256), ("latent", 17, 128), ("latent", 2, 384), ("latent", 1, 512)])
def test_attention_over_cached_latents_with_a_window_and_a_sink(kind, H, r, window):
    """One row per token is key and value of every head. The needle sits where the last queries see it just inside the
    window (or far back without one); the sinks are large enough to carry a tenth to a half of the weight."""
    from spissa_b200.csrc import lib as K
    from spissa_b200.parts.attention import attend_paged
    dtype = torch.float32 if kind == "generic" else torch.bfloat16
    w = window or 10 ** 6
    needle_at = [max(0, n - 1 - (w - 1)) if window else 1 for n in LAT_LENGTHS]
    needle_at[1] = 63 if window != 1 else needle_at[1]                       # the last row of a page
    q, c = _attention_case(H, r, 1, dtype, 7 * H + r + (window or 0), LAT_LENGTHS, needle_at)
    scale = 0.25
    sink = torch.linspace(1.0, 4.0, H) if window != 1 else torch.linspace(-1.0, 3.0, H)
    refs = [P.sink_softmax_mix(qb.double(), cb.double().expand(-1, H, -1), cb.double().expand(-1, H, -1), scale, window,
                               sink.double()).reshape(qb.shape[0], -1) for qb, cb in zip(q, c)]
    sink_d = sink.to(DEV)
    counters = torch.zeros(4096, dtype=torch.int32, device=DEV)

    def call(rows, step, view, split=True):
        if kind == "latent":
            assert K.latent_flash_supported(r, PAGE)
            out = torch.empty_like(rows)
            # with the step's longest length a decode step's keys are shared out over several blocks per sequence
            K.latent_flash(rows, view.k_pool, out, view, step, H, r, window, scale, sink_d,
                           max_len=step.max_len if step.all_single and split else None)
            return out
        return attend_paged(rows, step, view, H, 1, r, window, scale, sink_d, counters)

    tol = 3e-6 if dtype == torch.float32 else 1.2e-2
    for cuts, split in zip(LAT_CUTS + LAT_CUTS[2:], (True, True, True, False)):
        world = Paged(LAT_PAGES, 12, 1, r, dtype)
        got = _run_attention(world, q, c, _fix_cuts(cuts), lambda *a: call(*a, split=split))
        for b in range(3):
            assert worst(got[b], refs[b]) <= tol, (cuts[b][:4], b, split)
    # the sink matters here: without it the result is far away
    no_sink = P.sink_softmax_mix(q[0].double(), c[0].double().expand(-1, H, -1), c[0].double().expand(-1, H, -1), scale,
                                 window, torch.full((H,), -1e30, dtype=torch.float64)).reshape(LAT_LENGTHS[0], -1)
    assert worst(no_sink, refs[0]) > 0.05


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 64, None), (10, 2, 96, None), (6, 3, 16, 70), (2, 2, 128, None),
                                              (3, 1, 10, None), (4, 4, 32, 9), (4, 2, 64, 70), (2, 1, 128, 128),
                                              (4, 4, 64, 200), (2, 2, 128, 33)])
def test_sinks_in_the_grouped_query_kernels(nh, nkv, hd, window):
    """The same sink on every kernel that serves a grouped-query attention: the generic one (32-bit, any size), the
    mma.sync prompt and split-key decode kernels and, for prompts of 256 tokens and more, the tcgen05 one. A sink of 0
    adds one to the denominator; a sink per head may be anything."""
    from spissa_b200.parts.attention import attend_paged
    lengths, pages = [300, 70, 131], [[7, 3, 11, 2, 12], [5, 8], [1, 9, 4]]
    counters = torch.zeros(4096, dtype=torch.int32, device=DEV)
    for dtype in (torch.float32, torch.bfloat16):
        g = torch.Generator().manual_seed(nh * hd)
        q = [torch.randn(n, nh, hd, generator=g).to(dtype) for n in lengths]
        k = [torch.randn(n, nkv, hd, generator=g).to(dtype) for n in lengths]
        v = [torch.randn(n, nkv, hd, generator=g).to(dtype) for n in lengths]
        scale = 1.0 / math.sqrt(hd)
        for sink in (torch.zeros(nh), torch.linspace(-2.0, 3.0, nh)):
            rep = nh // nkv
            refs = [P.sink_softmax_mix(qb.double(), kb.double().repeat_interleave(rep, 1), vb.double().repeat_interleave(rep, 1),
                                       scale, window, sink.double()).reshape(qb.shape[0], -1) for qb, kb, vb in zip(q, k, v)]
            sd = sink.to(DEV)
            call = lambda rows, step, view: attend_paged(rows, step, view, nh, nkv, hd, window, scale, sd, counters)
            for cuts in ([[300], [70], [131]], [[280] + [1] * 20, [50] + [1] * 20, [111] + [1] * 20],
                         [[2, 62, 64, 172], [3, 1, 66, 0], [64, 64, 2, 1]], [[20, 280], [6, 64], [3, 128]]):
                world = Paged(pages, 14, nkv, hd, dtype, with_values=True)
                got = _run_attention(world, q, k, cuts, call, v=v)
                for b in range(3):
                    assert worst(got[b], refs[b]) <= (3e-6 if dtype == torch.float32 else 1.2e-2), (dtype, cuts[b][:3], b)
            # with scores this small the sink carries weight: leaving it out shows
            none = P.sink_softmax_mix(q[1].double(), k[1].double().repeat_interleave(rep, 1), v[1].double().repeat_interleave(rep, 1),
                                      scale, window, torch.full((nh,), -1e30, dtype=torch.float64)).reshape(70, -1)
            assert worst(none, refs[1]) > 0.05


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 64, None), (4, 4, 64, 70), (2, 1, 128, 128), (3, 3, 64, 1),
                                              (4, 4, 128, 200), (2, 2, 64, 64), (4, 1, 128, 65)])
def test_keys_and_values_as_rows_of_the_steps_own_tokens(nh, nkv, hd, window):
    """The tcgen05 prompt kernel over keys and values that lie in no cache (a latent attention expands a whole prompt's
    own latents): ragged sequences that all start at 0, windows below, at and above a block and a tile, sinks. One key
    of the first sequence is made to stand out, so that a window's edge that is one token off shows."""
    from spissa_b200.csrc import lib as K
    lengths = [300, 64, 129, 5, 410]
    g = torch.Generator().manual_seed(nh * hd + (window or 0))
    q = [torch.randn(n, nh, hd, generator=g).bfloat16() for n in lengths]
    k = [torch.randn(n, nkv, hd, generator=g).bfloat16() for n in lengths]
    v = [torch.randn(n, nkv, hd, generator=g).bfloat16() for n in lengths]
    scale, rep = 1.0 / math.sqrt(hd), nh // nkv
    q[0][:, :, 0] = 6.0
    k[0][150] = 0.0
    k[0][150, :, 0] = 6.0 * math.sqrt(hd) / 8.0              # a score of 4.5 where the others are about 1
    sink = torch.linspace(-2.0, 3.0, nh)
    refs = [P.sink_softmax_mix(qb.double(), kb.double().repeat_interleave(rep, 1), vb.double().repeat_interleave(rep, 1),
                               scale, window, sink.double()).reshape(qb.shape[0], -1) for qb, kb, vb in zip(q, k, v)]
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    step = SimpleNamespace(seq_start=i32(starts), positions=i32([p for n in lengths for p in range(n)]), n_seqs=len(lengths))
    flat = lambda xs, h: torch.cat(xs).reshape(-1, h * hd).to(DEV).contiguous()
    qd, kd, vd = flat(q, nh), flat(k, nkv), flat(v, nkv)
    assert K.flash_tc_rows_supported(torch.bfloat16, nh, nkv, hd)
    for sk, want in ((sink.to(DEV), refs), (None, None)):
        out = torch.full_like(qd, float("nan"))
        K.flash_prefill_tc_rows(qd, kd, vd, out, step, K.query_tiles(lengths, K.flash_tc_query_tile()), nh, nkv, hd, window, scale, sk)
        K.check_status(DEV)
        if want is None:
            want = [P.sink_softmax_mix(qb.double(), kb.double().repeat_interleave(rep, 1), vb.double().repeat_interleave(rep, 1),
                                       scale, window, torch.full((nh,), -1e30, dtype=torch.float64)).reshape(qb.shape[0], -1)
                    for qb, kb, vb in zip(q, k, v)]
        for b, n in enumerate(lengths):
            assert worst(out[starts[b]:starts[b] + n], want[b]) <= 1.2e-2, (b, sk is None)
    if window and 150 + window < 300:
        # the edge shows: with the standing-out key one place further the rows just past its window differ by far more
        rows = slice(150 + window - 1, 150 + window + 1)
        wide = P.sink_softmax_mix(q[0].double(), k[0].double().repeat_interleave(rep, 1), v[0].double().repeat_interleave(rep, 1),
                                  scale, window + 1, sink.double()).reshape(300, -1)
        assert worst(wide[rows], refs[0][rows]) > 0.05


@pytest.mark.parametrize("nh,nkv,d,taps,rd,dtype", [(4, 2, 16, 4, 8, torch.float32), (3, 1, 10, 5, 6, torch.float32),
                                                    (10, 2, 96, 3, 96, torch.bfloat16), (2, 2, 7, 1, 0, torch.float32),
                                                    (6, 3, 16, 2, 16, torch.float32)])
def test_values_are_the_keys_as_they_leave_the_convolution(nh, nkv, d, taps, rd, dtype):
    """Rows [q | k] only: the convolution over the step's rows and the slot's state, q and k rotated, the values the
    convolved keys BEFORE their rotation, across steps of unequal portions over scattered slots and pages."""
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(nh * d + taps)
    C, base = (nh + nkv) * d, 300.0
    lengths = [70, 9, 131]
    u = [torch.randn(n, C, generator=g) for n in lengths]
    conv = torch.randn(C, taps, generator=g) if taps > 1 else None
    inv_freq = torch.tensor([base ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float32) if rd else None
    world = Paged([[7, 3], [5], [1, 9, 4]], 12, nkv, d, dtype, with_values=True)
    state = torch.full((4, max(taps - 1, 1), C), 9.0, device=DEV)
    state[:3] = 0.0                                                # a sequence's state is zero when it starts
    cuts = [[5, 1, 1, 63, 0], [2, 1, 1, 5, 0], [64, 1, 1, 1, 64]]
    q_rows = [[], [], []]
    for s in range(5):
        at = list(world.at)
        step, view, live = world.step([c[s] for c in cuts])
        rows = torch.cat([u[b][at[b]:at[b] + cuts[b][s]] for b in live]).to(DEV)
        q = torch.empty(rows.shape[0], nh * d, dtype=dtype, device=DEV)
        K.conv_qk_store(rows, conv.to(DEV) if conv is not None else None, taps, state if taps > 1 else None, q, world.k_pool,
                        world.v_pool, view, step, inv_freq.to(DEV) if rd else None, nh, nkv, d, d, rd, 0.0, v_scale=1.0,
                        unit_rms=False, v_from_k=True)
        o = 0
        for b in live:
            q_rows[b].append(q[o:o + cuts[b][s]].cpu())
            o += cuts[b][s]
    tol = 3e-6 if dtype == torch.float32 else 6e-3
    for b, n in enumerate(lengths):
        full = P.short_conv(u[b].double(), conv.double()) if conv is not None else u[b].double()
        rq, rk = full[:, :nh * d].view(n, nh, d), full[:, nh * d:].view(n, nkv, d)
        assert worst(torch.cat(q_rows[b]), P.rotate_half(rq, rd, base).reshape(n, -1)) <= tol, b
        assert worst(world.rows(b, n), P.rotate_half(rk, rd, base)) <= tol, b
        assert worst(world.rows(b, n, world.v_pool), rk) <= tol, b
        if taps > 1:
            assert torch.equal(state[b].cpu(), u[b][n - (taps - 1):])
    assert float((state[3] - 9.0).abs().max()) == 0.0               # nobody's slot is left alone


@pytest.mark.parametrize("E,top,scale,gated", [(6, 2, 1.5, True), (3, 3, 1.0, False), (12, 3, 2.5, True), (5, 1, 0.5, False),
                                               (64, 8, 1.0, True), (7, 7, 1.25, False)])
def test_softmax_router_with_the_shared_experts_gate_in_its_product(E, top, scale, gated):
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(E + top)
    T, W, F = 77, 24, 12
    x = torch.randn(T, W, generator=g)
    w = {"router": torch.randn(E, W, generator=g), "shared.sg": torch.randn(1, W, generator=g)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = torch.randn(F, W, generator=g) * 0.4, torch.randn(F, W, generator=g) * 0.4
        w[f"e{e}.down"] = torch.randn(W, F, generator=g) * 0.4
    wd = {k: v.double() for k, v in w.items()}
    r = dict(experts=E, top=top, scale=scale)
    idx, wt = P.route(x.double(), wd, "", r)
    stacked = torch.cat([w["router"], w["shared.sg"]]) if gated else w["router"]
    z = (x @ stacked.T).to(DEV).contiguous()
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    extra = torch.empty(T, device=DEV) if gated else None
    K.moe_select(z, None, ids, wts, top, softmax=True, weight_scale=scale, experts=E, extra=extra)
    assert torch.equal(ids.cpu().long().sort(dim=1).values, idx.sort(dim=1).values)
    order, ref_order = ids.cpu().long().argsort(dim=1), idx.argsort(dim=1)
    assert worst(wts.cpu().gather(1, order), wt.gather(1, ref_order)) <= 2e-6
    assert abs(float(wts.sum(dim=1).mean()) - scale) <= 1e-5 * scale
    if gated:
        assert worst(extra, (x.double() @ wd["shared.sg"].T)[:, 0]) <= 2e-6
    # the experts as plain gated units (a slope of zero), weighted and summed into y
    ref = P.moe_ff(x.double(), wd, "", dict(router=r))
    gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).to(DEV)
    dn = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(DEV)
    y = torch.full((T, W), 0.25, device=DEV)
    K.moe_experts(x.to(DEV), ids, wts, gu, dn, y, top, 0.0, 0.0)
    assert worst(y - 0.25, ref) <= 1e-5
    y1 = torch.zeros(1, W, device=DEV)                              # a token alone: the same row, bit for bit
    K.moe_experts(x[5:6].to(DEV), ids[5:6].contiguous(), wts[5:6].contiguous(), gu, dn, y1, top, 0.0, 0.0)
    y0 = torch.zeros(T, W, device=DEV)
    K.moe_experts(x.to(DEV), ids, wts, gu, dn, y0, top, 0.0, 0.0)
    assert torch.equal(y1[0], y0[5])


def test_a_gate_per_row_and_capped_logits():
    from spissa_b200.csrc import lib as K
    g = torch.Generator().manual_seed(11)
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 5e-3)):
        x = (3 * torch.randn(19, 70, generator=g)).to(dtype)
        z = 2 * torch.randn(19, generator=g)
        xd = x.to(DEV)
        K.scale_rows_sigmoid(xd, z.to(DEV))
        assert worst(xd, x.double() * torch.sigmoid(z.double())[:, None]) <= tol
    logits = 40 * torch.randn(7, 333, generator=g)
    ld = logits.to(DEV)
    K.softcap(ld, 15.0)
    assert worst(ld, 15.0 * torch.tanh(logits.double() / 15.0)) <= 1e-6
    assert float(ld.abs().max()) <= 15.0


# ---------------------------------------------------------------------------------------------- whole models
LENGTHS = {"a": [1, 2, 23, 64, 65, 150], "b": [3, 63, 129, 140, 70, 9], "c": [5, 1, 40, 100, 66, 31],
           "d": [2, 70, 1, 33, 129, 64]}


def refs_of(m, reqs):
    ref = {}
    for rid, toks in reqs.items():
        logits = logits_of(m, toks)
        for p in range(len(toks)):
            ref[(rid, p)] = logits[p]
    return ref


# A router's choice is a step function of its input: where two experts' scores lie closer than bfloat16 rounding moves
# them, the bfloat16 run may choose the other one, and that token's logits (and, fading, those of the tokens that see
# it) differ by far more than rounding. The 32-bit runs must agree everywhere; the bfloat16 runs may leave this share of
# rows outside the tolerance.
CLOSE_CALLS = 0.08
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def compare(got, ref, tol, what, allow=0.0):
    assert set(got) == set(ref), what
    scale = max(float(v.abs().max()) for v in ref.values())
    errs = sorted(((float((row.double() - ref[k].double()).abs().max()) / scale, k) for k, row in got.items()),
                  key=lambda x: x[0] if x[0] == x[0] else 9e9)
    assert all(e == e for e, _ in errs), what
    over = [x for x in errs if x[0] > tol]
    assert len(over) <= allow * len(errs), \
        f"{what}: {len(over)} of {len(errs)} rows beyond {tol:.1e}, the worst {over[-1][0]:.3e} of the largest logit at {over[-1][1]}"


def test_layer_by_layer_the_residual_stream_follows_plain(models):
    """The stream after every layer of a prompt, in 32-bit: the first layer that differs names the mechanism."""
    m = models["a"]
    toks = tiny.random_prompt(m.vocab, 90, 12)
    layers = []
    P.forward(m.cfg, m.w, toks, layers_out=layers)
    eng = Engine.from_folder(m.folder, dtype="float32", max_tokens=128, max_seqs=1)
    seen = []
    hooks = []
    for block in eng.model.layers:
        inner = block.forward

        def run(h, step, cache, inner=inner):
            inner(h, step, cache)
            seen.append(h.detach().float().cpu().clone())
        block.forward = run
        hooks.append((block, inner))
    s = eng.acquire()
    eng.step([(s, toks, [len(toks) - 1])])
    eng.release(s)
    for block, inner in hooks:
        block.forward = inner
    assert len(seen) == len(layers)
    for i, (got, ref) in enumerate(zip(seen, layers)):
        assert worst(got[:len(toks)], ref) <= 1e-5, f"layer {i} ({m.cfg['layers'][i]['type']})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_every_cut_agrees_with_plain(models, name, dtype, tmp_path):
    m = models[name]
    reqs = {f"r{i}": tiny.random_prompt(m.vocab, n, 31 * i + n) for i, n in enumerate(LENGTHS[name])}
    ref = refs_of(m, reqs)
    decode = {rid: d for rid, d in zip(reqs, [0, 1, 22, 40, 3, 90])}
    cuts = {"whole": traces.whole(reqs), "tail": traces.tail_one_by_one(reqs, 45),
            "ragged": traces.ragged_batches(reqs, 3, decode),
            "ragged_pairs": traces.ragged_batches(dict(reversed(list(reqs.items()))), 2, decode)}
    allow = 0.0 if dtype == "float32" else CLOSE_CALLS
    results = {}
    for cut, steps in cuts.items():
        out = tmp_path / cut
        traces.run_in_process(m.folder, dtype, steps, str(out))          # a cache that holds just this trace: slots and pages come back
        results[cut] = traces.collect(steps, str(out), m.vocab)
        compare(results[cut], ref, TOL[dtype], f"{name}/{dtype}/{cut}", allow)
    for cut in ("tail", "ragged", "ragged_pairs"):
        compare(results[cut], results["whole"], TOL[dtype], f"{name}/{dtype}: {cut} against whole", allow)


def test_a_long_prompt_takes_the_grouped_expert_products_and_the_multiplied_out_maps(tmp_path):
    """A width and expert sizes that the tcgen05 tile kernel takes: a prompt of 300 tokens (600 and 900 pairs) runs its
    SwiGLU experts as grouped products and the latent attention's per-head maps multiplied out; the decode steps behind
    it take the small tiles and the small products; the 32-bit mode FFMA kernels. All agree with plain."""
    from spissa_b200.csrc import lib as K
    cfg = model(128, 180, [lat(latent_mixer(4, 32, 16, 64, 128, 100), moe(8, 2, 64, 1.5, shared=64)),
                           att(conv_mixer(2, 1, 64, conv=3, rot=32), moe(4, 3, 128, 1.0)),
                           lat(latent_mixer(2, 16, 48, 32, 128, 140, kv_from=0), dense(192))], cap=10.0)
    pcfg, w = make(cfg, tmp_path, seed=41, std=0.07, norm_std=0.1)
    m = SimpleNamespace(cfg=pcfg, w=w)
    toks = tiny.random_prompt(180, 330, 8)
    ref = logits_of(m, toks)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(str(tmp_path), dtype=dtype, max_tokens=64 * 7, max_seqs=1)
        s = eng.acquire()
        rows = [eng.step([(s, toks[:300], list(range(300)))]).cpu()]
        rows += [eng.step([(s, [t], [0])]).cpu() for t in toks[300:]]
        eng.release(s)
        got = {("p", i): r for i, r in enumerate(torch.cat(rows))}
        compare(got, {("p", i): r for i, r in enumerate(ref)}, TOL[dtype], dtype, 0.0 if dtype == "float32" else CLOSE_CALLS)
        if dtype == "bfloat16":
            assert eng.model.layers[0].ffn.glu_block == 64 and eng.model.layers[1].ffn.glu_block == 128
            assert eng.model.layers[0].mixer.q_fold is not None and eng.model.layers[2].mixer.o_fold.weight.shape == (128, 2 * 128)
        else:
            assert eng.model.layers[0].mixer.q_fold is None
    assert "tc_gemm" in K.loaded_libraries()


def test_whole_prompts_expand_their_own_latents(tmp_path, monkeypatch):
    """Latent heads whose key and value sizes the tcgen05 prompt kernel takes: a step in which every prompt starts at
    its first token expands that step's latents into keys and values (the writer's rows serve its reader too, each
    with its own window, narrower and wider than a block and a tile); a portion behind cached tokens and the decode
    steps attend over the cached rows. All agree with plain, and with each other."""
    from spissa_b200.csrc import lib as K
    cfg = model(128, 150, [lat(latent_mixer(2, 64, 64, 48, 96, 100), dense(64)),
                           att(conv_mixer(2, 1, 32, conv=2, rot=16), None),
                           lat(latent_mixer(1, 128, 128, 32, 96, 270, kv_from=0), moe(4, 2, 64, 1.0)),
                           lat(latent_mixer(3, 64, 64, 40, 64, 30), None)], cap=15.0)
    pcfg, w = make(cfg, tmp_path, seed=43, std=0.07, norm_std=0.1)
    m = SimpleNamespace(cfg=pcfg, w=w)
    reqs = {"p": tiny.random_prompt(150, 336, 5), "r": tiny.random_prompt(150, 296, 6)}
    ref = {(rid, i): row for rid, toks in reqs.items() for i, row in enumerate(logits_of(m, toks))}
    calls = []
    real = K.flash_prefill_tc_rows
    monkeypatch.setattr(K, "flash_prefill_tc_rows", lambda *a, **kw: (calls.append(a[0].shape[0]), real(*a, **kw))[1])
    for dtype in ("float32", "bfloat16"):
        allow = 0.0 if dtype == "float32" else CLOSE_CALLS
        eng = Engine.from_folder(str(tmp_path), dtype=dtype, max_tokens=64 * 14, max_seqs=2)
        calls.clear()
        sp, sr = eng.acquire(), eng.acquire()
        rows = eng.step([(sp, reqs["p"][:330], list(range(330))), (sr, reqs["r"][:290], list(range(290)))]).cpu()
        got = {("p", i): rows[i] for i in range(330)}
        got.update({("r", i): rows[330 + i] for i in range(290)})
        for i in range(6):
            rows = eng.step([(sp, [reqs["p"][330 + i]], [0]), (sr, [reqs["r"][290 + i]], [0])]).cpu()
            got[("p", 330 + i)], got[("r", 290 + i)] = rows[0], rows[1]
        eng.release(sp), eng.release(sr)
        assert calls == ([620] * 3 if dtype == "bfloat16" else []), calls
        compare(got, ref, TOL[dtype], f"{dtype}: two whole prompts", allow)
        # the same prompt behind 40 cached tokens: nothing is expanded, the cached rows are read
        calls.clear()
        s = eng.acquire()
        eng.step([(s, reqs["p"][:40], [])])
        rows = eng.step([(s, reqs["p"][40:330], list(range(290)))]).cpu()
        eng.release(s)
        assert calls == []
        compare({("p", 40 + i): rows[i] for i in range(290)}, {k: v for k, v in ref.items() if k[0] == "p" and 40 <= k[1] < 330},
                TOL[dtype], f"{dtype}: a portion behind cached tokens", allow)


@pytest.mark.parametrize("name", ["a", "c"])
def test_portions_of_a_prompt_down_to_two_tokens(models, name):
    m = models[name]
    toks = tiny.random_prompt(m.vocab, 150, 77)
    ref = logits_of(m, toks)
    other = tiny.random_prompt(m.vocab, 80, 78)
    ref_other = logits_of(m, other)
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 6, max_seqs=3)
    for sizes in ([2, 2, 3, 57, 1, 64, 21], [64, 64, 22], [1, 1, 2, 146]):
        s, s2 = engine.acquire(), engine.acquire()
        at, rows, rows2 = 0, [], []
        for n in sizes:
            entries = [(s, toks[at:at + n], list(range(n)))]
            lo2, hi2 = min(at, 80), min(at + n, 80)                      # the second request's portions end earlier
            if hi2 > lo2:
                entries.append((s2, other[lo2:hi2], list(range(hi2 - lo2))))
            got = engine.step(entries).cpu()
            rows.append(got[:n])
            rows2.append(got[n:])
            at += n
        assert worst(torch.cat(rows), ref) <= 2e-5, sizes
        assert worst(torch.cat(rows2), ref_other) <= 2e-5, sizes
        engine.release(s)
        engine.release(s2)
    engine.cache.check()
    assert engine.cache.slots.held_count == 0


def test_slots_and_pages_that_are_used_again_start_clean(models):
    m = models["a"]
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 3, max_seqs=2)
    for turn in range(3):
        reqs = [tiny.random_prompt(m.vocab, n, 5 * turn + n) for n in ((100, 30), (7, 120), (64, 65))[turn]]
        slots = [engine.acquire() for _ in reqs]
        got = engine.step([(s, r[:-2], [len(r) - 3]) for s, r in zip(slots, reqs)]).cpu()
        for b, r in enumerate(reqs):
            assert worst(got[b], logits_of(m, r[:-2])[-1]) <= 2e-5
        for i in (2, 1):
            got = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
        for b, r in enumerate(reqs):
            assert worst(got[b], logits_of(m, r)[-1]) <= 2e-5
        for s in slots:
            engine.release(s)
        engine.cache.check()


@pytest.mark.parametrize("name", ["a", "b"])
def test_long_decoding_lets_windows_pass_over_decoded_tokens_and_returns_pages(models, name):
    m = models[name]                             # a: windows of 9, 20 and 70 on one cache; b: 100 and 33 on rows of 128
    toks = tiny.random_prompt(m.vocab, 230, 3)
    ref = logits_of(m, toks)
    for dtype in ("float32", "bfloat16"):
        engine = Engine.from_folder(m.folder, dtype=dtype, max_tokens=64 * 4, max_seqs=1)
        s = engine.acquire()
        engine.step([(s, toks[:10], [])])
        rows = torch.cat([engine.step([(s, [t], [0])]).cpu() for t in toks[10:]])
        got = {("long", i): r for i, r in enumerate(rows)}
        compare(got, {("long", i): r for i, r in enumerate(ref[10:])}, TOL[dtype], dtype, 0.0 if dtype == "float32" else CLOSE_CALLS)
        for g in engine.cache.kv_groups.values():
            flags = [p is not None for p in engine.cache.seqs[s].pages[g.name]]
            assert flags[-1]
            assert flags[0] == (g.request.window is None)           # the windowed groups gave their first pages back
        engine.release(s)
        engine.cache.check()


# ---------------------------------------------------------------------------------------------- one key that matters
NEEDLE, DIRECTION, CONST = 7, 0, 1


def _mark_embedding(w, layer):
    """Token ``NEEDLE`` alone has a large entry along ``DIRECTION``; every token the same large one along ``CONST``."""
    w["embed"][:, DIRECTION] = 0.0
    w["embed"][NEEDLE, DIRECTION] = 6.0
    w["embed"][:, CONST] = 5.0
    w[f"l{layer}.norm1"][DIRECTION] = 1.0
    w[f"l{layer}.norm1"][CONST] = 1.0


def latent_needle_model(window, rank=24, q_rank=20, reader_window=None):
    """A latent attention that gives almost all its weight to the row of token ``NEEDLE`` wherever that row is visible,
    and whose values make the needle's presence large in the logits. With ``reader_window`` a second layer reads the
    first one's rows through a window of its own, and only that layer looks for the needle."""
    layers = [lat(latent_mixer(2, 8, 6, q_rank, rank, window, scale=1.0), None)]
    if reader_window:
        layers.append(lat(latent_mixer(3, 4, 8, q_rank, rank, reader_window, scale=1.0, kv_from=0), None))
    cfg = model(32, 64, layers, cap=25.0)
    look = len(layers) - 1                                       # the layer that looks for the needle

    def patch(w):
        _mark_embedding(w, 0)
        if look:
            w["l1.norm1"][DIRECTION] = w["l1.norm1"][CONST] = 1.0
            w["l0.mix.o"][DIRECTION] = w["l0.mix.o"][CONST] = 0.0     # layer 0 leaves the two marks as they are
        p = f"l{look}.mix."
        H, d, vd = (2, 8, 6) if not look else (3, 4, 8)
        for n in ("dq", "dkv"):
            w[f"l{0 if n == 'dkv' else look}.mix.{n}"][:, [DIRECTION, CONST]] = 0.0
        w["l0.mix.dkv"][0] = 0.0
        w["l0.mix.dkv"][0, DIRECTION] = 4.0                       # the needle's latent points along entry 0, nobody else's does
        w[p + "dq"][0] = 0.0
        w[p + "dq"][0, CONST] = 4.0                               # every query's latent has a large entry 0
        w["l0.mix.dkv.norm"][0] = 1.0
        w[p + "dq.norm"][0] = 1.0
        for h in range(H):
            w[p + "uk"][h * d + d - 1] = 0.0
            w[p + "uk"][h * d + d - 1, 0] = 1.0                   # key dim d − 1 reads entry 0 of the latent
            w[p + "uq"][h * d + d - 1] = 0.0
            w[p + "uq"][h * d + d - 1, 0] = 1.0                   # and every query looks along it
        w[p + "uv"][:, 0] = 3.0                                   # the needle's value stands out
        w[p + "sink"][:] = 0.5

    return cfg, patch


def conv_needle_model(dim=16, rot=8, heads=2, kv=1):
    """The same for the convolved attention, which sees every earlier key: the convolutions pass the current token
    only, so that the needle's key stands at the needle's position alone; its value is that key."""
    cfg = model(32, 64, [att(conv_mixer(heads, kv, dim, conv=3, rot=rot, scale=1.0), None)], cap=25.0)

    def patch(w):
        _mark_embedding(w, 0)
        for n in ("q", "k"):
            w[f"l0.mix.{n}.conv"].zero_()
            w[f"l0.mix.{n}.conv"][:, -1] = 1.0
            w[f"l0.mix.{n}"][:, [DIRECTION, CONST]] = 0.0
        j = dim - 1                                               # a dim that is not rotated
        for g in range(kv):
            w["l0.mix.k"][g * dim + j, :] = 0.0
            w["l0.mix.k"][g * dim + j, DIRECTION] = 1.0
        for h in range(heads):
            w["l0.mix.q"][h * dim + j, :] = 0.0
            w["l0.mix.q"][h * dim + j, CONST] = 1.0
        w["l0.mix.o"][:, [h * dim + j for h in range(heads)]] *= 8.0

    return cfg, patch


def _with_needle(base, place):
    toks = list(base)
    toks[place] = NEEDLE
    return toks


def _prompt_and_decoded(eng, toks, tail, tol, ref, what):
    T = len(toks)
    s = eng.acquire()
    got = eng.step([(s, toks, [T - 2, T - 1])]).cpu()                              # in a prompt
    assert worst(got, ref[-2:]) <= tol, (what, "prompt")
    eng.release(s)
    s = eng.acquire()
    eng.step([(s, toks[:T - tail], [])])
    for t in toks[T - tail:T - 2]:
        eng.step([(s, [t], [])])
    got = torch.cat([eng.step([(s, [t], [0])]) for t in toks[T - 2:]]).cpu()       # decoded, pages returned meanwhile
    assert worst(got, ref[-2:]) <= tol, (what, "decoded")
    eng.release(s)


@pytest.mark.parametrize("window,rank", [(20, 24), (64, 24), (70, 128), (130, 128), (1, 24), (2, 128)])
def test_a_row_just_inside_and_just_outside_the_window(tmp_path, window, rank):
    cfg, patch = latent_needle_model(window, rank=rank, q_rank=20 if rank == 24 else 128)
    pcfg, w = make(cfg, tmp_path, seed=21, std=0.05, norm_std=0.0, patch=patch)
    m = SimpleNamespace(cfg=pcfg, w=w)
    T = 200
    base = [t if t != NEEDLE else NEEDLE + 1 for t in tiny.random_prompt(64, T, 99)]
    places = sorted({T - 1 - (window - 1), T - 1 - window, T - 2 - (window - 1), 63, 64, T - 1})
    engines = {dt: Engine.from_folder(str(tmp_path), dtype=dt, max_tokens=64 * 4, max_seqs=1) for dt in ("float32", "bfloat16")}
    last = {}
    for place in places:
        toks = _with_needle(base, place)
        ref = logits_of(m, toks)
        last[place] = ref[-1]
        for dt in ("float32", "bfloat16"):
            _prompt_and_decoded(engines[dt], toks, 40, TOL[dt], ref, (place, dt))
    # the test can see the edge: a needle inside changes the last logits by far more than the tolerance
    inside, outside = last[T - 1 - (window - 1)], last[T - 1 - window]
    assert float((inside - outside).abs().max() / inside.abs().max()) > 0.2


@pytest.mark.parametrize("writer,reader", [(70, 20), (20, 70), (130, 64), (9, 129)])
def test_a_reader_of_another_layers_rows_keeps_its_own_window(tmp_path, writer, reader):
    """The cache keeps rows for the wider of the two windows; each layer sees its own. Only the reader looks for the
    needle: its edge, not the writer's, decides."""
    cfg, patch = latent_needle_model(writer, reader_window=reader)
    pcfg, w = make(cfg, tmp_path, seed=23, std=0.05, norm_std=0.0, patch=patch)
    m = SimpleNamespace(cfg=pcfg, w=w)
    T = 200
    base = [t if t != NEEDLE else NEEDLE + 1 for t in tiny.random_prompt(64, T, 98)]
    engines = {dt: Engine.from_folder(str(tmp_path), dtype=dt, max_tokens=64 * 4, max_seqs=1) for dt in ("float32", "bfloat16")}
    last = {}
    for place in (T - 1 - (reader - 1), T - 1 - reader, T - 1 - (writer - 1), T - 1 - writer):
        toks = _with_needle(base, place)
        ref = logits_of(m, toks)
        last[place] = ref[-1]
        for dt in ("float32", "bfloat16"):
            _prompt_and_decoded(engines[dt], toks, 50, TOL[dt], ref, (place, dt))
    inside, outside = last[T - 1 - (reader - 1)], last[T - 1 - reader]
    assert float((inside - outside).abs().max() / inside.abs().max()) > 0.2


@pytest.mark.parametrize("dim,rot,heads,kv", [(16, 8, 2, 1), (96, 32, 6, 1), (64, 64 - 2, 4, 2)])
def test_a_far_key_among_hundreds(tmp_path, dim, rot, heads, kv):
    cfg, patch = conv_needle_model(dim, rot, heads, kv)
    pcfg, w = make(cfg, tmp_path, seed=22, std=0.05, norm_std=0.0, patch=patch)
    m = SimpleNamespace(cfg=pcfg, w=w)
    T = 700
    base = [t if t != NEEDLE else NEEDLE + 1 for t in tiny.random_prompt(64, T, 5)]
    plain_last = logits_of(m, base)[-1]
    engines = {dt: Engine.from_folder(str(tmp_path), dtype=dt, max_tokens=64 * 11, max_seqs=1) for dt in ("float32", "bfloat16")}
    for place in (0, 1, 64, 383, 640):
        toks = _with_needle(base, place)
        ref = logits_of(m, toks)
        assert float((ref[-1] - plain_last).abs().max() / ref[-1].abs().max()) > 0.2
        for dt, eng in engines.items():
            s = eng.acquire()
            head = eng.step([(s, toks[:-1], [T - 2])]).cpu()
            tail = eng.step([(s, [toks[-1]], [0])]).cpu()
            eng.release(s)
            assert worst(head[0], ref[-2]) <= TOL[dt] and worst(tail[0], ref[-1]) <= TOL[dt], (place, dt)


def test_the_first_tokens_of_a_sequence_see_zeros_before_its_start(models):
    """Tokens 0 … taps−2 convolve over places before the sequence, and the first tokens' windows hold fewer rows than
    their size: a slot whose last sequence left values there must not leak them, neither in a prompt nor when the first
    tokens come one by one."""
    for name in ("a", "c"):
        m = models[name]
        engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 2, max_seqs=1)
        for toks in (tiny.random_prompt(m.vocab, 40, 1), tiny.random_prompt(m.vocab, 6, 2)):
            ref = logits_of(m, toks)
            s = engine.acquire()
            assert worst(engine.step([(s, toks, list(range(len(toks))))]).cpu(), ref) <= 2e-5
            engine.release(s)
            s = engine.acquire()
            rows = [engine.step([(s, [t], [0])]).cpu() for t in toks[:6]]
            assert worst(torch.cat(rows), ref[:6]) <= 2e-5
            engine.release(s)


# ---------------------------------------------------------------------------------------------- generation, the program
def greedy_plain(m, prompt, n):
    return P.generate_greedy(m.cfg, m.w, prompt, n)


@pytest.mark.parametrize("name", ["a", "d"])
def test_greedy_generation_through_the_entry_point(models, name):
    m = models[name]
    prompts = [tiny.random_prompt(m.vocab, n, 7 * n) for n in (1, 9, 70, 30)]
    engine = Engine.from_folder(m.folder, dtype="float32", max_tokens=64 * 8, max_seqs=3)     # two batches
    results, metrics = engine.generate(prompts, 12, SamplingParams(), stop_ids=[])
    for p, r in zip(prompts, results):
        ids = list(p)
        for tok in r.tokens:                                   # along the engine's own tokens: the chosen one is the largest
            row = logits_of(m, ids)[-1]
            assert float(row.max() - row[tok]) <= 2e-5 * float(row.abs().max()), f"prompt of {len(p)}"
            ids.append(tok)
        assert len(r.tokens) == 12 and r.finish_reason == "length"
    assert metrics.generated_tokens == 12 * len(prompts)
    engine.cache.check()
    assert engine.cache.slots.held_count == 0
    # bfloat16 and sampling run through the same loop
    engine = Engine.from_folder(m.folder, dtype="bfloat16", max_tokens=64 * 8)
    results, _ = engine.generate(prompts, 6, SamplingParams(temperature=0.8, top_k=20, seed=3), stop_ids=[])
    assert all(len(r.tokens) == 6 and all(0 <= t < m.vocab for t in r.tokens) for r in results)


def test_trace_program_on_a_model_of_this_design(models, tmp_path):
    m = models["b"]
    reqs = {f"q{i}": tiny.random_prompt(m.vocab, n, n) for i, n in enumerate([40, 3, 90])}
    steps = traces.ragged_batches(reqs, 3, {"q0": 5, "q1": 2, "q2": 30})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("bfloat16", "float32"):
        out = tmp_path / dtype
        proc = subprocess.run(
            [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", m.folder, "--dtype", dtype,
             "--out", str(out), "--max-tokens", str(traces.tokens_needed(steps))],
            input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        compare(traces.collect(steps, str(out), m.vocab), refs_of(m, reqs), TOL[dtype], "trace program",
                CLOSE_CALLS if dtype == "bfloat16" else 0.0)


def test_command_line_generates_from_a_folder_and_from_a_configuration_with_random_weights(models, tmp_path):
    m = models["c"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "bin", "spissa-b200")
    prompt = tiny.random_prompt(m.vocab, 12, 4)
    proc = subprocess.run([sys.executable, exe, "generate", m.folder, "--token-ids", ",".join(map(str, prompt)),
                           "--max-new-tokens", "5", "--dtype", "fp32", "--ctx", "128"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[0])
    assert line["tokens"] == greedy_plain(m, prompt, 5) and line["finish_reason"] == "length"
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["a"]))
    proc = subprocess.run([sys.executable, exe, "generate", "--random", str(cfg_file), "--token-ids", "1,2,3",
                           "--token-ids", "9,8,7,6,5", "--max-new-tokens", "4", "--temp", "0.7", "--seed", "2", "--ctx", "128"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(x) for x in proc.stdout.strip().splitlines()]
    assert [len(x["tokens"]) for x in lines] == [4, 4]
