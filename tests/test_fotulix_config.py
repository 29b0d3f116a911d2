"""Configuration of the Fotulix decoder, its weight list and cache needs, and the plain functions against hand-made
cases (every other test of this design leans on them)."""
import copy
import math

import pytest
import torch

import fotulix_models as M
from plain import fotulix_plain as P
from plain.llama_plain import read_model_folder
from spissa_b200.cache import CacheManager
from spissa_b200.config import ConfigError, FotulixConfig, config_from_dict
from spissa_b200.engine.model import EMBEDDING_CACHE, Model
from spissa_b200.parts import KVCacheRequest, StateRequest
from spissa_b200.weights import write_random_model

CFG = M.model(40, 90, [
    M.layer("latent_attention", M.through_rows(3, 8, 4, 12, 20, 9, base=100.0, scaling=M.RAMP), 56),
    M.layer("attention", M.biased(4, 2, 6, vdim=10, q_temp=(0.35, 16), far=40, rows=12), 48),
    M.layer("latent_attention", M.through_rows(2, 16, 4, 4, 20, 70, base=100.0, scaling=M.RAMP, kv_from=0)),
    M.layer("attention_2", M.turned(3, 3, 8, rot=4, base=50.0, scaling=M.BANDS), 24)],
    mult=0.5, emb_scale=8.0, bigram=(37, 5, 3), side=6, eps=1e-4)


def test_registry_finds_the_architecture_and_the_configuration_round_trips():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, FotulixConfig)
    assert cfg.to_dict() == CFG
    again = config_from_dict(FotulixConfig(**{**cfg.__dict__, "raw": None}).to_dict())
    assert again.layers == cfg.layers and again.bigram == (37, 5, 3) and again.side_dim == 6
    assert again.residual_mult == 0.5 and again.embedding_scale == 8.0
    assert cfg.cache_windows() == {0: 70}                       # the cache keeps rows for the widest reader


def test_absent_keys_mean_not_there():
    bare = dict(architecture="Fotulix", vocab=30, width=16, norm=dict(eps=1e-5),
                layers=[dict(type="attention", mixer=dict(heads=2, dim=8, scale=0.3), mlp=None),
                        dict(type="attention_2", mixer=dict(heads=2, dim=8, scale=0.3), mlp=None),
                        dict(type="latent_attention", mixer=dict(heads=2, dim=8, kv_rank=6, scale=0.3), mlp=None)])
    cfg = config_from_dict(bare)
    assert cfg.residual_mult == 1.0 and cfg.embedding_scale == 1.0 and cfg.bigram is None and cfg.side_dim is None
    shapes = {s.name: tuple(s.shape) for s in Model(cfg.to_spec()).weight_specs()}
    assert "bigram" not in shapes and "side.embed" not in shapes and "l0.mix.rel" not in shapes
    assert shapes["l0.mix.k"] == (16, 16) and shapes["l0.mix.q.b"] == (16,) and shapes["l1.mix.sink"] == (2,)
    assert shapes["l2.mix.q"] == (16, 16) and shapes["l2.mix.dkv"] == (6, 16) and "l0.norm2" not in shapes
    assert Model(cfg.to_spec()).cache_requests()[2] == KVCacheRequest(1, 6, None, keys_only=True)


def test_weight_list():
    model = Model(config_from_dict(CFG).to_spec())
    shapes = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert shapes["embed"] == (90, 40) and shapes["bigram"] == (38, 40) and shapes["side.embed"] == (90, 24)
    assert shapes["head"] == (90, 40) and shapes["final.norm"] == (40,)
    for n in ("norm1", "norm1b", "norm2", "norm2b", "side.norm"):
        assert shapes[f"l0.{n}"] == (40,)
    assert "l2.norm2" not in shapes and "l2.norm2b" not in shapes and shapes["l2.norm1b"] == (40,)
    assert shapes["l0.mix.q"] == (36, 40) and shapes["l0.mix.dkv"] == (24, 40) and shapes["l0.mix.dkv.norm"] == (20,)
    assert shapes["l0.mix.uk"] == (24, 20) and shapes["l0.mix.uv"] == (36, 20) and shapes["l0.mix.g"] == (3, 40)
    assert shapes["l0.mix.o"] == (40, 36)
    assert "l2.mix.dkv" not in shapes and "l2.mix.dkv.norm" not in shapes             # it reads layer 0's rows
    assert shapes["l2.mix.q"] == (40, 40) and shapes["l2.mix.uk"] == (32, 20) and shapes["l2.mix.uv"] == (8, 20)
    assert shapes["l1.mix.q"] == (24, 40) and shapes["l1.mix.k"] == (12, 40) and shapes["l1.mix.v"] == (20, 40)
    assert shapes["l1.mix.q.b"] == (24,) and shapes["l1.mix.k.b"] == (12,) and shapes["l1.mix.v.b"] == (20,)
    assert shapes["l1.mix.rel"] == (-12, 4) and shapes["l1.mix.g"] == (4, 40) and shapes["l1.mix.o"] == (40, 40)
    # (the table's rows are the checkpoint's to choose: −n stands for "any, n when the weights are drawn")
    assert "l1.mix.sink" not in shapes and "l3.mix.rel" not in shapes and "l3.mix.q.b" not in shapes
    assert shapes["l3.mix.sink"] == (3,) and shapes["l3.mix.o"] == (40, 24)
    assert shapes["l1.mlp.gate"] == (48, 40) and shapes["l1.mlp.down"] == (40, 48) and "l2.mlp.up" not in shapes
    assert shapes["l3.side.gate"] == (6, 40) and shapes["l3.side.proj"] == (40, 6)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="recurrent"), "known mixers"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][3]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"]["rot"]["scaling"].update(high=1.0), "high"),
    (lambda c: c["layers"][3]["mixer"]["rot"]["scaling"].pop("original"), "original"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=2), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].pop("every"), "every"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda c: c["token_side"].update(dim=0), "dim"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_bad_configurations_are_refused_with_the_field_named(change, word):
    bad = copy.deepcopy(CFG)
    change(bad)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(bad)


def test_cache_needs_a_word_of_state_for_the_embedding_and_one_pool_for_writer_and_reader():
    model = Model(config_from_dict(CFG).to_spec())
    reqs = model.cache_requests()
    assert sorted(reqs, key=str) == [0, 1, 3, EMBEDDING_CACHE]                          # layer 2 runs on cache 0
    assert reqs[0] == KVCacheRequest(1, 24, 70, keys_only=True)                         # the row and the shared key part
    assert reqs[1] == KVCacheRequest(2, 6, None, v_head_dim=10)
    assert reqs[3] == KVCacheRequest(3, 8, None)
    assert reqs[EMBEDDING_CACHE] == StateRequest((1,), torch.int32)
    assert [(e.layer, e.cache, e.writes_cache) for e in model.spec.schedule] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    cache = CacheManager(reqs, max_tokens=64 * 4, max_seqs=2, page_size=64, dtype=torch.float32, device="cpu")
    step = type("S", (), dict(page_tables={g: None for g in cache.kv_groups}, token_seq=None, positions=None, seq_row=None))
    own, reader = cache.view(0, step, True), cache.view(0, step, False)
    assert own.k_pool.data_ptr() == own.v_pool.data_ptr() and tuple(own.k_pool.shape) == (4, 1, 64, 24)
    assert reader.k_pool.data_ptr() == own.k_pool.data_ptr() and own.writes and not reader.writes
    wide = cache.view(1, step, True)
    assert tuple(wide.k_pool.shape)[-1] == 6 and tuple(wide.v_pool.shape)[-1] == 10
    slot = cache.acquire()
    for n in (150, 1):
        cache.commit(cache.reserve([(slot, n)]))
    held = {g.request.window: [p is not None for p in cache.seqs[slot].pages[g.name]] for g in cache.kv_groups.values()}
    assert held[70] == [False, True, True] and held[None] == [True, True, True]         # rows 81 … 150 are still seen
    cache.check()
    cache.release(slot)


# ---------------------------------------------------------------------------------------------- the plain functions
def test_plain_embedding_rows_and_distance_rows():
    w = {"embed": torch.arange(10.0, dtype=torch.float64)[:, None].repeat(1, 2),
         "bigram": torch.arange(0.0, 600.0, 100.0, dtype=torch.float64)[:, None].repeat(1, 2)}
    x = P.embed([3, 4, 9], w, dict(scale=2.0, bigram=dict(buckets=5, mul_prev=3, mul_cur=2)))
    # first token: the last row (5); then (3·3 + 4·2) mod 5 = 2 and (4·3 + 9·2) mod 5 = 0
    assert x[:, 0].tolist() == [6.0 + 500.0, 8.0 + 200.0, 18.0 + 0.0]
    assert P.embed([3, 4], w, dict(scale=1.0))[:, 0].tolist() == [3.0, 4.0]
    # 8 rows, the last reached at 64: 0 … 3 exact, then a quarter of ln(n / 4) / ln 16 per row
    got = [P.distance_bucket(n, 8, 64.0) for n in (0, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 5000)]
    assert got == [0, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]


def test_plain_rotation_frequencies_and_sink():
    v = torch.zeros(3, 1, 6, dtype=torch.float64)
    v[:, 0, 0] = 1.0
    v[:, 0, 5] = 7.0
    f = torch.tensor([1.0, 0.1], dtype=torch.float64)
    r = torch.cat([P.rotate_pairs(v[..., :4], f), v[..., 4:]], dim=-1)                 # dim 0 pairs with dim 1; 4 and 5 pass
    assert torch.allclose(r[2, 0], torch.tensor([math.cos(2.0), math.sin(2.0), 0.0, 0.0, 0.0, 7.0], dtype=torch.float64))
    assert torch.allclose(P.rotate_pairs(v[..., :2], f[:1], 1.5)[1, 0], torch.tensor([1.5 * math.cos(1.0), 1.5 * math.sin(1.0)], dtype=torch.float64))
    # bands: wavelengths 2π (kept: below 40 / 4), 20π and 200π (above 40 / 1: divided by 4)
    rot = dict(dims=6, base=1000.0, scaling=dict(factor=4.0, low=1.0, high=4.0, original=40))
    fb = P.banded_frequencies(rot)
    assert math.isclose(fb[0], 1.0) and math.isclose(fb[1], 0.1 / 4) and math.isclose(fb[2], 0.01 / 4)
    rot = dict(dims=4, base=4.0, scaling=dict(factor=4.0, low=1.0, high=4.0, original=16))
    s = (16 / (2 * math.pi / 0.5) - 1.0) / 3.0                                         # the pair of wavelength 4π lies between
    assert math.isclose(P.banded_frequencies(rot)[1], (1 - s) * 0.5 / 4 + s * 0.5)
    # ramp: pairs at and below lo keep their frequency, pairs from hi on are divided by the factor
    rot = dict(dims=8, base=10000.0, scaling=dict(factor=2.0, original=64, fast=4.0, slow=2.0))
    fr, amp = P.ramped_frequencies(rot)
    pair = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(pair(4.0)), 0), min(math.ceil(pair(2.0)), 7)
    assert (lo, hi) == (0, 1)
    plain = [10000.0 ** (-2 * i / 8) for i in range(4)]
    assert math.isclose(fr[0], plain[0]) and math.isclose(fr[1], plain[1] / 2) and math.isclose(fr[3], plain[3] / 2)
    assert math.isclose(amp, 0.1 * math.log(2.0) + 1.0)
    # equal scores: with a sink of ln 2 and a window of two, the first row weighs its one key 1/3, later rows 1/4 each
    s = torch.zeros(1, 4, 4, dtype=torch.float64)
    vals = torch.eye(4, dtype=torch.float64)[:, None, :]
    out = P.softmax_mix(s, vals, window=2, sink=torch.tensor([math.log(2.0)], dtype=torch.float64))[:, 0]
    assert torch.allclose(out[0], torch.tensor([1 / 3, 0, 0, 0], dtype=torch.float64))
    assert torch.allclose(out[3], torch.tensor([0, 0, 0.25, 0.25], dtype=torch.float64))
    out = P.softmax_mix(s, vals)[:, 0]
    assert torch.allclose(out[3], torch.full((4,), 0.25, dtype=torch.float64))


def test_plain_model_runs_a_random_folder_and_a_later_token_changes_nothing_earlier(tmp_path):
    write_random_model(config_from_dict(CFG), tmp_path, seed=4, std=0.1, norm_std=0.1)
    cfg, w = read_model_folder(tmp_path)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9]
    layers = []
    full = P.forward(cfg, w, toks, layers_out=layers)
    assert full.shape == (15, 90) and len(layers) == 4
    assert torch.allclose(P.forward(cfg, w, toks[:9]), full[:9], atol=1e-12)
    # the window of nine: with layer 0 alone a change at token 0 reaches token 8 and no later one, except through the
    # pair table (token 1's row is chosen by token 0 too) and only as far as token 9
    other = [8] + toks[1:]
    one_layer = dict(cfg, layers=cfg["layers"][:1])
    assert torch.equal(P.forward(one_layer, w, other)[10:], P.forward(one_layer, w, toks)[10:])
    assert not torch.equal(P.forward(one_layer, w, other)[8], P.forward(one_layer, w, toks)[8])
