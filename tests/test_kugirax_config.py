"""Configuration of the Kugirax decoder, its weight list, and what it brought to the shared parts: a cache whose rows
are key and value at once, a layer that reads the rows another layer cached, one norm for two sublayers. The plain
functions are checked against hand-made cases here as well, since every other test leans on them."""
import copy
import math

import pytest
import torch

from plain import kugirax_plain as P
from plain.llama_plain import read_model_folder
from spissa_b200.cache import CacheManager
from spissa_b200.config import ConfigError, KugiraxConfig, config_from_dict
from spissa_b200.engine.model import Model
from spissa_b200.parts import CacheBundle, KVCacheRequest, StateRequest
from spissa_b200.weights import write_random_model


def conv_mixer(heads, kv, dim, conv=None, rot=None, base=10000.0, scale=0.3):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale)
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    return m


def latent_mixer(heads, dim, vdim, q_rank, kv_rank, window, scale=0.25, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale, mask=dict(size=window))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


CFG = dict(
    architecture="Kugirax", vocab=90, width=40, norm=dict(eps=1e-4), logit_softcap=12.0,
    layers=[
        dict(type="latent_attention", mixer=latent_mixer(3, 8, 12, 20, 24, 9), mlp=dict(kind="dense", ff=56)),
        dict(type="attention", mixer=conv_mixer(4, 2, 6, conv=4, rot=4, base=1000.0),
             mlp=dict(kind="moe", expert=dict(ff=16), shared=dict(ff=24), router=dict(experts=6, top=2, scale=1.5))),
        dict(type="latent_attention", mixer=latent_mixer(2, 16, 4, 10, 24, 70, kv_from=0), mlp=None),
        dict(type="attention", mixer=conv_mixer(3, 3, 8), mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=3, top=3, scale=1.0))),
    ])


def test_registry_finds_the_architecture_and_the_configuration_round_trips():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, KugiraxConfig)
    assert cfg.to_dict() == CFG
    again = config_from_dict(KugiraxConfig(**{**cfg.__dict__, "raw": None}).to_dict())
    assert again.layers == cfg.layers and again.logit_softcap == 12.0
    assert cfg.cache_windows() == {0: 70}                       # the cache keeps rows for the widest reader


def test_weight_list():
    model = Model(config_from_dict(CFG).to_spec())
    shapes = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert shapes["embed"] == (90, 40) and shapes["head"] == (90, 40) and shapes["final.norm"] == (40,)
    assert shapes["l0.norm1"] == (40,) and not any("norm2" in n for n in shapes)
    assert shapes["l0.mix.dq"] == (20, 40) and shapes["l0.mix.dq.norm"] == (20,) and shapes["l0.mix.uq"] == (24, 20)
    assert shapes["l0.mix.dkv"] == (24, 40) and shapes["l0.mix.dkv.norm"] == (24,)
    assert shapes["l0.mix.uk"] == (24, 24) and shapes["l0.mix.uv"] == (36, 24) and shapes["l0.mix.sink"] == (3,)
    assert shapes["l0.mix.o"] == (40, 36)
    assert "l2.mix.dkv" not in shapes and "l2.mix.dkv.norm" not in shapes             # it reads layer 0's rows
    assert shapes["l2.mix.uk"] == (32, 24) and shapes["l2.mix.uv"] == (8, 24) and shapes["l2.mix.o"] == (40, 8)
    assert shapes["l1.mix.q"] == (24, 40) and shapes["l1.mix.k"] == (12, 40) and "l1.mix.v" not in shapes
    assert shapes["l1.mix.q.conv"] == (24, 4) and shapes["l1.mix.k.conv"] == (12, 4) and shapes["l1.mix.o"] == (40, 24)
    assert "l3.mix.q.conv" not in shapes
    assert shapes["l1.mlp.router"] == (6, 40) and shapes["l1.mlp.e5.down"] == (40, 16) and "l1.mlp.correction" not in shapes
    assert shapes["l1.mlp.shared.gate"] == (24, 40) and shapes["l1.mlp.shared.sg"] == (1, 40)
    assert "l3.mlp.shared.sg" not in shapes and "l2.mlp.up" not in shapes and shapes["l0.mlp.down"] == (40, 56)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="recurrent"), "known mixers"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_bad_configurations_are_refused_with_the_field_named(change, word):
    bad = copy.deepcopy(CFG)
    change(bad)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(bad)


def test_a_reader_of_another_layers_rows_has_no_cache_of_its_own():
    model = Model(config_from_dict(CFG).to_spec())
    reqs = model.cache_requests()
    assert sorted(reqs) == [0, 1, 3]                                                    # layer 2 runs on cache 0
    assert reqs[0] == KVCacheRequest(1, 24, 70, keys_only=True)
    assert reqs[1] == CacheBundle((("kv", KVCacheRequest(2, 6, None)), ("conv", StateRequest((3, 36), torch.float32))))
    assert reqs[3] == CacheBundle((("kv", KVCacheRequest(3, 8, None)),))                # no convolution: no state
    assert [(e.layer, e.cache, e.writes_cache) for e in model.spec.schedule] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    cache = CacheManager(reqs, max_tokens=64 * 4, max_seqs=2, page_size=64, dtype=torch.float32, device="cpu")
    step = type("S", (), dict(page_tables={g: None for g in cache.kv_groups}, token_seq=None, positions=None, seq_row=None))
    own, reader = cache.view(0, step, True), cache.view(0, step, False)
    assert own.k_pool.data_ptr() == own.v_pool.data_ptr() and tuple(own.k_pool.shape) == (4, 1, 64, 24)   # one row, key and value at once
    assert reader.k_pool.data_ptr() == own.k_pool.data_ptr() and own.writes and not reader.writes
    slot = cache.acquire()
    for n in (150, 1):
        cache.commit(cache.reserve([(slot, n)]))
    held = {g.request.window: [p is not None for p in cache.seqs[slot].pages[g.name]] for g in cache.kv_groups.values()}
    assert held[70] == [False, True, True]                                              # rows 81 … 150 are still seen
    cache.check()
    cache.release(slot)


# ---------------------------------------------------------------------------------------------- the plain functions
def test_plain_convolution_rotation_and_sink():
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None].repeat(1, 2)               # 1 … 5 in two channels
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 10.0, 100.0]], dtype=torch.float64)
    y = P.short_conv(u, w)
    assert y[:, 0].tolist() == [1, 2, 3, 4, 5]                                          # the last tap is the token itself
    assert y[:, 1].tolist() == [100, 210, 321, 432, 543]                                # zeros before the start
    v = torch.zeros(3, 1, 6, dtype=torch.float64)
    v[:, 0, 0] = 1.0
    v[:, 0, 5] = 7.0
    r = P.rotate_half(v, 4, 100.0)                                                      # dim 0 pairs with dim 2; 4 and 5 pass
    assert torch.allclose(r[2, 0], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0, 0.0, 7.0], dtype=torch.float64))
    assert torch.allclose(P.rotate_half(v, 2, 100.0)[1, 0, :2], torch.tensor([math.cos(1.0), math.sin(1.0)], dtype=torch.float64))
    # equal scores: with a sink of ln 2 and a window of two, the first row weighs its one key 1/3, later rows 1/4 each
    q = torch.zeros(4, 1, 2, dtype=torch.float64)
    vals = torch.eye(4, dtype=torch.float64)[:, None, :]
    out = P.sink_softmax_mix(q, q, vals, 1.0, 2, torch.tensor([math.log(2.0)], dtype=torch.float64))[:, 0]
    assert torch.allclose(out[0], torch.tensor([1 / 3, 0, 0, 0], dtype=torch.float64))
    assert torch.allclose(out[3], torch.tensor([0, 0, 0.25, 0.25], dtype=torch.float64))
    # a sink of 0 adds one to the denominator; no window: every earlier key
    out = P.sink_softmax_mix(q, q, vals, 1.0, None, torch.zeros(1, dtype=torch.float64))[:, 0]
    assert torch.allclose(out[3], torch.full((4,), 0.2, dtype=torch.float64))


def test_plain_router_and_gated_shared_expert():
    w = {"router": torch.zeros(4, 3, dtype=torch.float64)}
    w["router"][:, 0] = torch.tensor([1.0, 3.0, 2.0, -1.0], dtype=torch.float64)
    a = torch.tensor([[1.0, 0.0, 0.0]], dtype=torch.float64)
    idx, wt = P.route(a, w, "", dict(experts=4, top=2, scale=1.5))
    assert sorted(idx[0].tolist()) == [1, 2]
    s = torch.softmax(torch.tensor([1.0, 3.0, 2.0, -1.0], dtype=torch.float64), -1)
    assert torch.allclose(wt[0].sort().values, (s[[2, 1]] / (s[1] + s[2]) * 1.5))       # the chosen scores, renormed, times the scale
    idx, wt = P.route(a, w, "", dict(experts=4, top=4, scale=1.0))
    assert torch.allclose(wt.sum(), torch.tensor(1.0, dtype=torch.float64))
    for e in range(4):
        w[f"e{e}.gate"] = w[f"e{e}.up"] = torch.zeros(2, 3, dtype=torch.float64)
        w[f"e{e}.down"] = torch.zeros(3, 2, dtype=torch.float64)
    w["shared.gate"] = torch.tensor([[2.0, 0, 0]], dtype=torch.float64)
    w["shared.up"] = torch.tensor([[3.0, 0, 0]], dtype=torch.float64)
    w["shared.down"] = torch.tensor([[1.0], [0.0], [0.0]], dtype=torch.float64)
    w["shared.sg"] = torch.tensor([[0.0, 0, 0]], dtype=torch.float64)                  # sigmoid(0) = 1/2
    y = P.moe_ff(a, w, "", dict(router=dict(experts=4, top=2, scale=1.5), shared=dict(ff=1)))
    assert torch.allclose(y[0, 0], torch.tensor(0.5 * 2.0 / (1 + math.exp(-2.0)) * 3.0, dtype=torch.float64))


def test_plain_model_runs_a_random_folder_and_a_later_token_changes_nothing_earlier(tmp_path):
    write_random_model(config_from_dict(CFG), tmp_path, seed=4, std=0.1, norm_std=0.1)
    cfg, w = read_model_folder(tmp_path)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9]
    layers = []
    full = P.forward(cfg, w, toks, layers_out=layers)
    assert full.shape == (15, 90) and len(layers) == 4 and float(full.abs().max()) < 12.0        # the cap bounds the logits
    assert torch.allclose(P.forward(cfg, w, toks[:9]), full[:9], atol=1e-12)
    # the window of nine: a change at token 0 reaches token 12 through layer 2's wider window only
    other = [8] + toks[1:]
    one_layer = dict(cfg, layers=cfg["layers"][:1])
    assert torch.equal(P.forward(one_layer, w, other)[9:], P.forward(one_layer, w, toks)[9:])
    assert not torch.equal(P.forward(one_layer, w, other)[8], P.forward(one_layer, w, toks)[8])
