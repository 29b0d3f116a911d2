"""Measures decoding and prefill of the Llama-3.2-1B shape with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 1b|3b|8b] [--batch B]
                    [--context T] [--profile-phases]
    python bench.py --design duzinex [--design-sizes 1k,2k,4k]      (the Duzinex decoder beside Llama at equal sizes)
    python bench.py --design gozatar [--design-sizes 1k,2k,4k]      (the Gozatar decoder likewise)
    python bench.py --design kugirax [--design-sizes 1k,2k,4k]      (the Kugirax decoder likewise)
    python bench.py --design fotulix [--design-sizes 1k,2k,4k]      (the Fotulix decoder beside Kugirax and Llama)

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 from prompts of
about 2,048 tokens in a cache of 4,096 tokens per sequence, timed on the device with CUDA
events over exactly K decode steps after W warm-up steps; ``e2e`` is the same through the
Python entry point (``Engine.generate``: host token lists in, host token lists out).
``prefill`` is one 2,048-token prompt; ``points`` holds decoding at batch 1 and 64;
``roofline`` compares the decode step with the bytes it has to read. ``--context T`` decodes from prompts of
about T tokens instead (the cache then holds 2T per sequence); the prefill measurement stays at 2,048 tokens.
``--config 3b`` and ``--config 8b`` run the secondary workloads (3B shape: batch 8, prompts uniform in [256, 2048],
256 decode steps, 4,096-token cache per sequence; 8B shape: batch 16, prompts uniform in [512, 4096], 512 steps,
8,192 tokens per sequence) and print the same line. ``--profile-phases`` adds per-phase timings (CUDA events around
the kernel groups of one prompt step and of part-by-part decode steps).
Token ids are synthetic (seeded, uniform over the vocabulary), weights are N(0, 0.02).
Every decode step reads all weights (2.47 GB), far more than the 126 MB L2, so no
flush is needed between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# the Llama 3.2 1B shape: the configuration the headline numbers are quoted on
CONFIG_1B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=16, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072)
CONFIG_3B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=28, hidden_size=3072,
    num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192, vocab_size=128256,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072)
CONFIG_8B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=32, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=False, rms_norm_eps=1e-5, max_position_embeddings=131072)
# name -> configuration, batch, cache per sequence, prompt lengths (mean of a narrow band, or a uniform range), decode
# steps, extra batch sizes: the headline workload and the two secondary ones
WORKLOADS = {
    "1b": dict(cfg=CONFIG_1B, model="llama-3.2-1b-shape", batch=8, context=4096, prompt=2048, span=None, steps=64, points="1,64"),
    "3b": dict(cfg=CONFIG_3B, model="llama-3.2-3b-shape", batch=8, context=4096, prompt=None, span=(256, 2048), steps=256, points=""),
    "8b": dict(cfg=CONFIG_8B, model="llama-3.1-8b-shape", batch=16, context=8192, prompt=None, span=(512, 4096), steps=512, points=""),
}
CONTEXT = 4096
PROMPT = 2048
SPAN = None                                 # (lowest, highest) prompt length when the workload draws them uniformly
PREFILL_TOKENS = 2048                       # the prefill measurement is always of this many tokens
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
        return out
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def model_numbers(cfg, elem_bytes=2):
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    nh, nkv, hd, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.vocab_size
    per_layer = H * nh * hd * 2 + H * nkv * hd * 2 + 3 * H * I
    head = V * H
    return dict(per_layer=per_layer, head=head, kv_bytes_per_token=2 * nkv * hd * elem_bytes * L,
                weight_bytes=(per_layer * L + head) * elem_bytes)


def prefill_flops(cfg, T):
    n = model_numbers(cfg)
    gemm = 2.0 * T * n["per_layer"] * cfg.num_hidden_layers
    attn = 4.0 * (T * (T + 1) / 2) * cfg.head_dim * cfg.num_attention_heads * cfg.num_hidden_layers
    return gemm + attn + 2.0 * n["head"]


def ragged_lengths(batch, seed):
    rng = random.Random(seed)
    if SPAN is not None:
        return [rng.randint(SPAN[0], SPAN[1]) for _ in range(batch)]
    if batch == 1:
        return [PROMPT]
    half = PROMPT // 8
    lens = [PROMPT + rng.randrange(-half, half + 1) for _ in range(batch)]
    lens[0] += PROMPT * batch - sum(lens)         # the mean is PROMPT exactly
    return lens


KERNEL_CASE_LAYERS = 0
KERNEL_CASE_BATCH = 0          # sequences of --kernel-case decode_layers (0: eight)


# ---------------------------------------------------------------------------------------------------------------------
# --design duzinex: the Duzinex decoder beside the Llama decoder at equal layer sizes (random weights)
DESIGN_SIZES = {
    # width, ff, (attention: heads, kv heads, map size, value size), (retention: heads, dim, vdim), Llama heads / kv / head
    "1k": dict(width=1024, ff=4096, att=(8, 2, 64, 128), ret=(4, 128, 256), llama=(16, 4, 64)),
    "2k": dict(width=2048, ff=8192, att=(16, 4, 64, 128), ret=(8, 128, 256), llama=(32, 8, 64)),
    "4k": dict(width=4096, ff=14336, att=(32, 8, 64, 128), ret=(16, 128, 256), llama=(32, 8, 128)),
}
DESIGN_WINDOW = 1024
DESIGN_VOCAB = 32000


def duzinex_config(size: dict, window: int = DESIGN_WINDOW) -> dict:
    W, ff = size["width"], size["ff"]
    h, g, d, vd = size["att"]
    rh, rd, rvd = size["ret"]
    att = dict(type="attention", mixer=dict(heads=h, kv_heads=g, dim=d, vdim=vd, diff=0.5, scale=d ** -0.5, softcap=30.0,
                                            mask=dict(size=window, keep_first=4), rot=dict(dims=d, base=10000.0)))
    ret = dict(type="retention", mixer=dict(heads=rh, dim=rd, vdim=rvd,
                                            decay=[1.0 - 2.0 ** (-5 - i % 4) for i in range(rh)]))
    gru = dict(type="mingru", mixer=dict(width=W))
    mlp = dict(kind="dense", ff=ff)
    layers = [dict(l, mlp=mlp) for l in (ret, gru, att, gru, att, ret)]
    # layers 1 … 4 run twice: ten layer runs (2 of retention, 4 of minGRU, 4 of attention)
    return dict(architecture="Duzinex", vocab=DESIGN_VOCAB, width=W, embedding=dict(scale=W ** 0.5), norm=dict(eps=1e-6),
                layers=layers, loop=dict(start=1, stop=5, times=2))


def llama_config_like(size: dict, layers: int) -> dict:
    nh, nkv, hd = size["llama"]
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=layers, hidden_size=size["width"],
                num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, intermediate_size=size["ff"],
                vocab_size=DESIGN_VOCAB, rope_theta=10000.0, rope_scaling=None, tie_word_embeddings=True,
                rms_norm_eps=1e-6, max_position_embeddings=131072)


# --design gozatar: eight layers of a sliding-window attention (window 1,024, a convolution of four taps, half of each
# head rotated) beside a gated linear attention (heads of 128 x 256); the first and fifth layers have a dense feed-forward
# of ``ff``, the others 32 experts of ff/4 of which a token uses 4 (from 2 of 4 groups) plus a shared expert of ff/4: a
# token's active feed-forward weights are 1.25 times the dense layer's (three matrices instead of two).
GOZATAR_SIZES = {
    "1k": dict(left=(8, 2, 128), right=(4, 128, 256)),
    "2k": dict(left=(16, 4, 128), right=(8, 128, 256)),
    "4k": dict(left=(32, 8, 128), right=(16, 128, 256)),
}
GOZATAR_LAYERS = 8


def gozatar_config(size: dict, goz: dict, window: int = DESIGN_WINDOW) -> dict:
    W, ff = size["width"], size["ff"]
    h, g, d = goz["left"]
    rh, rd, rvd = goz["right"]
    mixer = dict(left=dict(heads=h, kv_heads=g, dim=d, vdim=d, conv=4, scale=d ** -0.5, mask=dict(size=window),
                           rot=dict(dims=d // 2, base=10000.0)), left_scale=0.7,
                 right=dict(heads=rh, dim=rd, vdim=rvd, tau=16.0, rank=16), right_scale=0.7)
    moe = dict(kind="moe", expert=dict(ff=ff // 4, limit=7.0), shared=dict(ff=ff // 4, limit=7.0),
               router=dict(experts=32, top=4, groups=dict(count=4, keep=2)))
    layers = [dict(type="parallel", mixer=mixer, mlp=dict(kind="dense", ff=ff) if i % 4 == 0 else moe)
              for i in range(GOZATAR_LAYERS)]
    return dict(architecture="Gozatar", vocab=DESIGN_VOCAB, width=W, streams=2, norm=dict(eps=1e-6), layers=layers)


# --design kugirax: eight layers with one norm each; six of them a grouped-query attention whose q and k pass a
# convolution of four taps, whose values are the keys, fully rotated, with one added to the softmax's denominator; layers
# 2 and 6 an attention through a cached latent (window 1,024, a sink per head), layer 6 reading the rows layer 2 cached.
# Even layers have a dense feed-forward of ``ff``, odd ones 32 experts of ff/4 of which a token uses 4 plus a gated
# shared expert of ff/4.
KUGIRAX_SIZES = {
    # (attention: heads, kv heads, dim), (latent: heads, dim, vdim, q_rank, kv_rank)
    "1k": dict(att=(8, 2, 128), lat=(8, 128, 128, 512, 256)),
    "2k": dict(att=(16, 4, 128), lat=(16, 128, 128, 768, 256)),
    "4k": dict(att=(32, 8, 128), lat=(32, 128, 128, 1536, 512)),
}
KUGIRAX_LAYERS, KUGIRAX_LATENT = 8, (2, 6)


def kugirax_config(size: dict, kx: dict, window: int = DESIGN_WINDOW) -> dict:
    W, ff = size["width"], size["ff"]
    h, g, d = kx["att"]
    lh, ld, lvd, qr, r = kx["lat"]
    att = dict(heads=h, kv_heads=g, dim=d, vdim=d, conv=4, scale=d ** -0.5, rot=dict(dims=d, base=10000.0))
    lat = dict(heads=lh, dim=ld, vdim=lvd, q_rank=qr, kv_rank=r, scale=ld ** -0.5, mask=dict(size=window))
    moe = dict(kind="moe", expert=dict(ff=ff // 4), shared=dict(ff=ff // 4), router=dict(experts=32, top=4, scale=1.5))
    layers = []
    for i in range(KUGIRAX_LAYERS):
        mlp = dict(kind="dense", ff=ff) if i % 2 == 0 else moe
        if i in KUGIRAX_LATENT:
            m = dict(lat, kv_from=KUGIRAX_LATENT[0]) if i != KUGIRAX_LATENT[0] else lat
            layers.append(dict(type="latent_attention", mixer=m, mlp=mlp))
        else:
            layers.append(dict(type="attention", mixer=att, mlp=mlp))
    return dict(architecture="Kugirax", vocab=DESIGN_VOCAB, width=W, norm=dict(eps=1e-6), logit_softcap=30.0, layers=layers)


# --design fotulix: eight layers, every sublayer between two norms, a pair table and a token side input of 256; layers 0
# and 4 an attention through cached rows (rank + 64 rotated dims shared by the heads, window 1,024), layer 4 reading the
# rows layer 0 cached; layers 2 and 6 a grouped-query attention with half of each head rotated and a sink; the other four
# a grouped-query attention with biases, a query factor and a table of 32 scores by distance. Dense feed-forwards of
# ``ff``. Beside it the closest existing design at equal sizes: a Kugirax decoder of eight layers with its latent
# attention at the same two places (rows of the same size, the same window) and dense feed-forwards, and Llama.
FOTULIX_SIZES = {
    # (attention: heads, kv heads, dim), (latent: heads, dim, rot_dim, vdim, kv_rank), Kugirax's query rank
    "1k": dict(att=(8, 2, 128), lat=(8, 128, 64, 128, 192), q_rank=512),
    "2k": dict(att=(16, 4, 128), lat=(16, 128, 64, 128, 192), q_rank=768),
    "4k": dict(att=(32, 8, 128), lat=(32, 128, 64, 128, 448), q_rank=1536),
}
FOTULIX_LAYERS, FOTULIX_LATENT, FOTULIX_SINK = 8, (0, 4), (2, 6)
FOTULIX_SIDE = 256


def fotulix_config(size: dict, fx: dict, window: int = DESIGN_WINDOW) -> dict:
    W, ff = size["width"], size["ff"]
    h, g, d = fx["att"]
    lh, ld, lrd, lvd, r = fx["lat"]
    biased = dict(heads=h, kv_heads=g, dim=d, vdim=d, scale=d ** -0.5, q_temp=dict(coef=0.2, every=512), bias_max=4096, bias_rows=32)
    turned = dict(heads=h, kv_heads=g, dim=d, vdim=d, scale=d ** -0.5,
                  rot=dict(dims=d // 2, base=500000.0, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    lat = dict(heads=lh, dim=ld, rot_dim=lrd, vdim=lvd, kv_rank=r, scale=(ld + lrd) ** -0.5, mask=dict(size=window),
               rot=dict(dims=lrd, base=10000.0, scaling=dict(factor=8.0, original=4096, fast=32.0, slow=1.0)))
    layers = []
    for i in range(FOTULIX_LAYERS):
        if i in FOTULIX_LATENT:
            m = dict(lat, kv_from=FOTULIX_LATENT[0]) if i != FOTULIX_LATENT[0] else lat
            layers.append(dict(type="latent_attention", mixer=m, mlp=dict(kind="dense", ff=ff)))
        else:
            layers.append(dict(type="attention_2" if i in FOTULIX_SINK else "attention", mixer=turned if i in FOTULIX_SINK else biased,
                               mlp=dict(kind="dense", ff=ff)))
    return dict(architecture="Fotulix", vocab=DESIGN_VOCAB, width=W, norm=dict(eps=1e-6), residual_mult=0.5,
                embedding=dict(scale=W ** 0.5, bigram=dict(buckets=65521, mul_prev=31, mul_cur=17)),
                token_side=dict(dim=FOTULIX_SIDE), layers=layers)


def kugirax_config_like_fotulix(size: dict, fx: dict, window: int = DESIGN_WINDOW) -> dict:
    W, ff = size["width"], size["ff"]
    h, g, d = fx["att"]
    lh, ld, lrd, lvd, r = fx["lat"]
    att = dict(heads=h, kv_heads=g, dim=d, vdim=d, conv=4, scale=d ** -0.5, rot=dict(dims=d, base=10000.0))
    lat = dict(heads=lh, dim=ld, vdim=lvd, q_rank=fx["q_rank"], kv_rank=r + lrd, scale=ld ** -0.5, mask=dict(size=window))
    layers = []
    for i in range(FOTULIX_LAYERS):
        if i in FOTULIX_LATENT:
            m = dict(lat, kv_from=FOTULIX_LATENT[0]) if i != FOTULIX_LATENT[0] else lat
            layers.append(dict(type="latent_attention", mixer=m, mlp=dict(kind="dense", ff=ff)))
        else:
            layers.append(dict(type="attention", mixer=att, mlp=dict(kind="dense", ff=ff)))
    return dict(architecture="Kugirax", vocab=DESIGN_VOCAB, width=W, norm=dict(eps=1e-6), logit_softcap=30.0, layers=layers)


def design_compare(args) -> int:
    """Prefill (one 2,048-token prompt) and decode (batch 8 behind such prompts) of the Duzinex decoder and of the
    Llama decoder with the same width, feed-forward size and number of layer runs; per-phase device times of both
    (CUDA events around kernel groups, steps run part by part), and for the new design's own kernels the bytes or
    FLOPs they have to move against the measured peaks. Prints ONE JSON line."""
    import torch
    from spissa_b200 import Engine
    from spissa_b200.config import config_from_dict
    from spissa_b200.csrc import lib
    peaks = load_peaks()
    torch.cuda.set_device(0)
    T, B = PREFILL_TOKENS, 8
    design = args.design
    out = {"design": design, "beside": "llama", "dtype": args.dtype, "prefill_tokens": T, "decode_batch": B,
           "window": DESIGN_WINDOW, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "sizes": {}}
    names = [n for n in (args.design_sizes.split(",") if args.design_sizes else DESIGN_SIZES) if n in DESIGN_SIZES]
    for name in names:
        size = DESIGN_SIZES[name]
        dz = (duzinex_config(size) if design == "duzinex" else gozatar_config(size, GOZATAR_SIZES[name]) if design == "gozatar"
              else kugirax_config(size, KUGIRAX_SIZES[name]) if design == "kugirax" else fotulix_config(size, FOTULIX_SIZES[name]))
        runs = len(config_from_dict(dz).to_spec().schedule)
        row = {}
        arms = [(design, dz), ("llama", llama_config_like(size, runs))]
        if design == "fotulix":
            arms.insert(1, ("kugirax", kugirax_config_like_fotulix(size, FOTULIX_SIZES[name])))
            out["beside"] = "kugirax, llama"
        for label, cfg_dict in arms:
            cfg = config_from_dict(cfg_dict)
            engine = Engine.from_config(cfg, seed=0, dtype=args.dtype, max_tokens=B * (T + 128), max_seqs=B, device="cuda:0")
            rng = random.Random(7)
            V = DESIGN_VOCAB
            prompt = [rng.randrange(V) for _ in range(T)]

            def prefill_once():
                s = engine.acquire()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                engine.step([(s, prompt, [T - 1])], check=False)
                e1.record()
                torch.cuda.synchronize()
                engine.check()
                engine.release(s)
                return e0.elapsed_time(e1)

            for _ in range(3):
                prefill_once()
            pre_ms = sorted(prefill_once() for _ in range(5))[2]
            slots = [engine.acquire() for _ in range(B)]
            for s in slots:
                engine.step([(s, [rng.randrange(V) for _ in range(T)], [])], check=False)
            engine.check()
            one = lambda: engine.step([(s, [11], [0]) for s in slots], check=False)
            for _ in range(max(3, args.warmup)):
                one()
            torch.cuda.synchronize()
            steps = args.steps or 32
            l0 = lib.launches
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            engine.check()
            dec_ms = e0.elapsed_time(e1) / steps
            launches = (lib.launches - l0) // steps
            # per-phase times, steps run part by part
            engine.profile_phases = True
            engine.phase_totals.clear()
            for sl in slots:
                engine.release(sl)
            for _ in range(2):                                    # the second run's: the first also pays for fresh scratch
                engine.phase_totals.clear()
                s = engine.acquire()
                engine.step([(s, prompt, [T - 1])])
                pre_phases = dict(engine.phase_totals["prefill"]["ms"])
                engine.release(s)
            slots = [engine.acquire() for _ in range(B)]
            engine.step([(sl, prompt[:T - 8], []) for sl in slots])
            engine.phase_totals.pop("decode", None)
            for i in range(4):
                engine.step([(sl, [7 + i], [0]) for sl in slots])
            dec_phases = {k: v / 4 for k, v in engine.phase_totals["decode"]["ms"].items()}
            for sl in slots:
                engine.release(sl)
            engine.profile_phases = False
            weight_bytes = sum(t.numel() * t.element_size() for t in
                               {id(p.weight): p.weight for p in _linears(engine.model)}.values())
            row[label] = dict(layer_runs=runs, prefill_ms=round(pre_ms, 3), prefill_tok_s=round(T / pre_ms * 1e3, 1),
                              decode_ms_per_step=round(dec_ms, 4), decode_tok_s=round(B / dec_ms * 1e3, 1),
                              decode_launches_per_step=launches, weight_gb=round(weight_bytes / 1e9, 3),
                              decode_weight_stream_frac=round(weight_bytes / (dec_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                              prefill_phases_ms={k: round(v, 4) for k, v in sorted(pre_phases.items())},
                              decode_phases_ms={k: round(v, 4) for k, v in sorted(dec_phases.items())})
            del engine
            torch.cuda.empty_cache()
        eb = 4 if args.dtype == "float32" else 2
        row["rooflines"] = (design_rooflines(size, row, T, B, peaks, eb) if design == "duzinex"
                            else gozatar_rooflines(size, GOZATAR_SIZES[name], row, T, peaks, eb) if design == "gozatar"
                            else kugirax_rooflines(size, KUGIRAX_SIZES[name], row, T, peaks, eb) if design == "kugirax"
                            else fotulix_rooflines(size, FOTULIX_SIZES[name], row, T, B, peaks, eb))
        out["sizes"][name] = row
    print(json.dumps(out))
    return 0


def _linears(model):
    found = []

    def walk(p):
        for k, v in vars(p).items():
            if k.endswith("_fold"):
                continue                                  # maps multiplied out for prompt steps: decode steps do not read them
            if hasattr(v, "weight") and hasattr(v, "out_features"):
                found.append(v)
            elif hasattr(v, "plain") and hasattr(v.plain, "out_features"):
                found.append(v.plain)
        for c in p.children():
            walk(c)
    for p in model.parts():
        walk(p)
    return found


def design_rooflines(size, row, T, B, peaks, eb) -> dict:
    """What each kernel group of a prompt step has to do at least, as a fraction of the measured peaks, for the new
    design's own kernels and the Llama kernels that are most like them. Per-phase times are sums over the layer runs."""
    h, g, d, vd = size["att"]
    rh, rd, rvd = size["ret"]
    W, ff = size["width"], size["ff"]
    nh, nkv, hd = size["llama"]
    dz, ll = row["duzinex"]["prefill_phases_ms"], row["llama"]["prefill_phases_ms"]
    tf, bw = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    win = min(T, DESIGN_WINDOW)
    pairs = T * win - win * (win - 1) / 2                       # (query, visible key) pairs of one window, first tokens aside
    frac = lambda work, peak, ms: round(work / (ms * 1e-3) / peak, 4) if ms else None
    out = {}
    # four attention runs: two maps of d MACs per pair for the scores, two maps of vd MACs for the values
    att_flops = 4 * h * pairs * (2 * 2 * d + 2 * 2 * vd)
    out["diff_attention (tensor)"] = dict(ms=dz.get("attention_ms"), frac=frac(att_flops, tf, dz.get("attention_ms")))
    ll_att = ll.get("attention_ms")
    ll_runs = row["llama"]["layer_runs"]
    out["llama attention (tensor)"] = dict(ms=ll_att, frac=frac(ll_runs * 4.0 * (T * (T + 1) / 2) * hd * nh, tf, ll_att))
    # retention: two runs; chunked form: per token and head d·vd MACs for the state, the same for the read, plus the
    # chunk's own pairs; counted as the recurrence's 2·2·d·vd FLOPs per token and head (the least any form does)
    out["retention (tensor)"] = dict(ms=dz.get("retention_ms"), frac=frac(2 * T * rh * 4.0 * rd * rvd, tf, dz.get("retention_ms")))
    out["retention (hbm)"] = dict(ms=dz.get("retention_ms"),
                                  frac=frac(2 * T * (2 * rh * rd + 2 * rh * rvd) * 4.0 + 2 * T * rh * rvd * eb, bw, dz.get("retention_ms")))
    out["mingru (hbm)"] = dict(ms=dz.get("mingru_ms"), frac=frac(4 * T * W * (3 * 4.0 + eb), bw, dz.get("mingru_ms")))
    out["polynorm (hbm)"] = dict(ms=dz.get("activation_ms"), frac=frac(10 * T * ff * (4.0 + eb), bw, dz.get("activation_ms")))
    out["norm+shift (hbm)"] = dict(ms=dz.get("mixer_norm+shift_ms"), frac=frac(10 * T * W * (4.0 + eb), bw, dz.get("mixer_norm+shift_ms")))
    out["llama norm (hbm)"] = dict(ms=ll.get("attention_norm_ms"), frac=frac(T * W * (4.0 + eb), bw, ll.get("attention_norm_ms")))   # one launch: the first layer's
    return out


def gozatar_rooflines(size, goz, row, T, peaks, eb) -> dict:
    """The same for the Gozatar decoder's kernel groups of a prompt step (sums over its eight layers)."""
    W, ff = size["width"], size["ff"]
    h, g, d = goz["left"]
    rh, rd, rvd = goz["right"]
    nh, nkv, hd = size["llama"]
    gz, ll = row["gozatar"]["prefill_phases_ms"], row["llama"]["prefill_phases_ms"]
    tf, bw = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    L, n_moe = GOZATAR_LAYERS, GOZATAR_LAYERS - GOZATAR_LAYERS // 4
    win = min(T, DESIGN_WINDOW)
    pairs = T * win - win * (win - 1) / 2
    frac = lambda work, peak, ms: round(work / (ms * 1e-3) / peak, 4) if ms else None
    out = {}
    out["window attention (tensor)"] = dict(ms=gz.get("attention_ms"), frac=frac(L * 4.0 * pairs * d * h, tf, gz.get("attention_ms")))
    ll_att, ll_runs = ll.get("attention_ms"), row["llama"]["layer_runs"]
    out["llama attention (tensor)"] = dict(ms=ll_att, frac=frac(ll_runs * 4.0 * (T * (T + 1) / 2) * hd * nh, tf, ll_att))
    # the recurrence's 2·2·d·vd FLOPs per token and head (the least any form does), and its 32-bit operands and output
    out["gla (tensor)"] = dict(ms=gz.get("gla_ms"), frac=frac(L * T * rh * 4.0 * rd * rvd, tf, gz.get("gla_ms")))
    out["gla (hbm)"] = dict(ms=gz.get("gla_ms"),
                            frac=frac(L * T * ((2 * rh * rd + 2 * rh * rvd + 16) * 4.0 + rh * rvd * eb), bw, gz.get("gla_ms")))
    # the experts: 4 of 32 per token, three matrices of W x ff/4 each
    out["experts (tensor)"] = dict(ms=gz.get("experts_ms"), frac=frac(n_moe * T * 4 * 3 * 2.0 * W * (ff // 4), tf, gz.get("experts_ms")))
    ll_ff = sum(v for k, v in ll.items() if "gate_projection" in k or "down_projection" in k)
    out["llama feed-forward (tensor)"] = dict(ms=ll_ff, frac=frac(ll_runs * T * 3 * 2.0 * W * ff, tf, ll_ff))
    C = (h + g) * d + g * d
    out["conv+rotary+store (hbm)"] = dict(ms=gz.get("conv+rotary+kv_append_ms"),
                                          frac=frac(L * T * C * (4.0 + eb), bw, gz.get("conv+rotary+kv_append_ms")))
    norm_ms = (gz.get("attention_norm_ms") or 0) + (gz.get("streams_update+mlp_norm_ms") or 0) + (gz.get("streams_update_ms") or 0)
    # per layer: the streams read once for the first norm, read and written by each of the two updates, y read twice
    out["streams+norm (hbm)"] = dict(ms=norm_ms, frac=frac(L * T * W * (2 * 4.0 + 2 * (4 * 4.0 + 4.0) + 2 * eb), bw, norm_ms))
    out["llama norm (hbm)"] = dict(ms=ll.get("attention_norm_ms"), frac=frac(T * W * (4.0 + eb), bw, ll.get("attention_norm_ms")))   # one launch: the first layer's
    act_ms = gz.get("activation_ms")
    out["activations (hbm)"] = dict(ms=act_ms, frac=frac((2 * T * ff + n_moe * T * 3 * (ff // 4)) * (4.0 + eb) * 1.0, bw, act_ms))
    return out


def kugirax_rooflines(size, kx, row, T, peaks, eb) -> dict:
    """The same for the Kugirax decoder's kernel groups of a prompt step (sums over its eight layers)."""
    W, ff = size["width"], size["ff"]
    h, g, d = kx["att"]
    lh, ld, lvd, qr, r = kx["lat"]
    nh, nkv, hd = size["llama"]
    kz, ll = row["kugirax"]["prefill_phases_ms"], row["llama"]["prefill_phases_ms"]
    tf, bw = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    n_lat = len(KUGIRAX_LATENT)
    n_att, n_moe = KUGIRAX_LAYERS - n_lat, KUGIRAX_LAYERS // 2
    win = min(T, DESIGN_WINDOW)
    pairs = T * win - win * (win - 1) / 2
    frac = lambda work, peak, ms: round(work / (ms * 1e-3) / peak, 4) if ms else None
    out = {}
    out["attention with a unit sink (tensor)"] = dict(ms=kz.get("attention_ms"),
                                                      frac=frac(n_att * 4.0 * (T * (T + 1) / 2) * d * h, tf, kz.get("attention_ms")))
    ll_att, ll_runs = ll.get("attention_ms"), row["llama"]["layer_runs"]
    out["llama attention (tensor)"] = dict(ms=ll_att, frac=frac(ll_runs * 4.0 * (T * (T + 1) / 2) * hd * nh, tf, ll_att))
    # a whole prompt expands its own latents: per (query, visible key) pair and head 2·dim FLOPs for the score and
    # 2·vdim for the weighted sum, the least any form does (over the cached rows themselves it is 4·rank)
    out["latent attention (tensor)"] = dict(ms=kz.get("latent_attention_ms"),
                                            frac=frac(n_lat * 2.0 * pairs * (ld + lvd) * lh, tf, kz.get("latent_attention_ms")))
    out["key and value expansion (tensor)"] = dict(ms=kz.get("key_value_expansion_ms"),
                                                   frac=frac(n_lat * T * 2.0 * r * lh * (ld + lvd), tf, kz.get("key_value_expansion_ms")))
    hp = (kz.get("query_into_latent_space_ms") or 0) + (kz.get("value_expansion_ms") or 0)
    if hp:                                                   # only steps that attend over the cached rows run them
        out["per-head products (tensor)"] = dict(ms=hp, frac=frac(n_lat * T * lh * 2.0 * r * (ld + lvd), tf, hp))
    out["latent norms+append (hbm)"] = dict(ms=kz.get("latent_norm+append_ms"),
                                            frac=frac((T * (qr + r) * 4.0 + T * (qr + r) * eb) + T * qr * (4.0 + eb), bw,
                                                      kz.get("latent_norm+append_ms")))
    out["experts (tensor)"] = dict(ms=kz.get("experts_ms"), frac=frac(n_moe * T * 4 * 3 * 2.0 * W * (ff // 4), tf, kz.get("experts_ms")))
    ll_ff = sum(v for k, v in ll.items() if "gate_projection" in k or "down_projection" in k)
    out["llama feed-forward (tensor)"] = dict(ms=ll_ff, frac=frac(ll_runs * T * 3 * 2.0 * W * ff, tf, ll_ff))
    C = (h + g) * d
    out["conv+rotary+store (hbm)"] = dict(ms=kz.get("conv+rotary+kv_append_ms"),
                                          frac=frac(n_att * T * (C * 4.0 + (h + 2 * g) * d * eb), bw, kz.get("conv+rotary+kv_append_ms")))
    out["norm (hbm)"] = dict(ms=kz.get("input_norm_ms"), frac=frac(KUGIRAX_LAYERS * T * W * (4.0 + eb), bw, kz.get("input_norm_ms")))
    # Llama's norms ride in the products' prologues but for the first layer's: one launch
    out["llama norm (hbm)"] = dict(ms=ll.get("attention_norm_ms"), frac=frac(T * W * (4.0 + eb), bw, ll.get("attention_norm_ms")))
    return out


def fotulix_rooflines(size, fx, row, T, B, peaks, eb) -> dict:
    """The same for the Fotulix decoder's kernel groups of a prompt step (sums over its eight layers), beside the like
    groups of the Kugirax decoder at equal sizes and of Llama."""
    W, ff = size["width"], size["ff"]
    h, g, d = fx["att"]
    lh, ld, lrd, lvd, r = fx["lat"]
    nh, nkv, hd = size["llama"]
    fz, kz, ll = row["fotulix"]["prefill_phases_ms"], row["kugirax"]["prefill_phases_ms"], row["llama"]["prefill_phases_ms"]
    tf, bw = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    L, n_lat, n_sink = FOTULIX_LAYERS, len(FOTULIX_LATENT), len(FOTULIX_SINK)
    n_bias = L - n_lat - n_sink
    win = min(T, DESIGN_WINDOW)
    pairs = T * win - win * (win - 1) / 2
    causal = T * (T + 1) / 2
    R = r + lrd
    frac = lambda work, peak, ms: round(work / (ms * 1e-3) / peak, 4) if ms else None
    out = {}
    out["attention with scores by distance (tensor)"] = dict(ms=fz.get("distance_attention_ms"),
                                                             frac=frac(n_bias * 4.0 * causal * d * h, tf, fz.get("distance_attention_ms")))
    out["attention with a sink (tensor)"] = dict(ms=fz.get("attention_ms"), frac=frac(n_sink * 4.0 * causal * d * h, tf, fz.get("attention_ms")))
    out["kugirax attention (tensor)"] = dict(ms=kz.get("attention_ms"), frac=frac((L - n_lat) * 4.0 * causal * d * h, tf, kz.get("attention_ms")))
    ll_att, ll_runs = ll.get("attention_ms"), row["llama"]["layer_runs"]
    out["llama attention (tensor)"] = dict(ms=ll_att, frac=frac(ll_runs * 4.0 * causal * hd * nh, tf, ll_att))
    # per (query, visible key) pair and head 2·(dim + rot_dim) FLOPs for the score and 2·vdim for the weighted sum: the
    # least any form does (over the cached rows themselves it is 4·(rank + rot_dim))
    lat_ms = (fz.get("latent_attention_ms") or 0) + (fz.get("key_value_expansion_ms") or 0)
    out["latent attention (tensor)"] = dict(ms=lat_ms, frac=frac(n_lat * 2.0 * pairs * (ld + lrd + lvd) * lh, tf, lat_ms))
    k_lat = (kz.get("latent_attention_ms") or 0) + (kz.get("key_value_expansion_ms") or 0)
    out["kugirax latent attention (tensor)"] = dict(ms=k_lat, frac=frac(n_lat * 2.0 * pairs * (ld + lvd) * lh, tf, k_lat))
    hp = (fz.get("query_into_latent_space_ms") or 0) + (fz.get("value_expansion_ms") or 0)
    if hp:
        out["per-head products (tensor)"] = dict(ms=hp, frac=frac(n_lat * T * lh * 2.0 * R * (ld + lrd + lvd), tf, hp))
    k_hp = (kz.get("query_into_latent_space_ms") or 0) + (kz.get("value_expansion_ms") or 0)
    if k_hp:
        out["kugirax per-head products (tensor)"] = dict(ms=k_hp, frac=frac(n_lat * T * lh * 2.0 * R * (ld + lvd), tf, k_hp))
    C = (h + g) * d + g * d
    out["bias+factor+rotation+store (hbm)"] = dict(ms=fz.get("rotary+kv_append_ms"),
                                                   frac=frac((L - n_lat) * T * ((C + h) * 4.0 + C * eb + h * 4.0), bw, fz.get("rotary+kv_append_ms")))
    k_store = kz.get("conv+rotary+kv_append_ms")
    out["kugirax conv+rotary+store (hbm)"] = dict(ms=k_store, frac=frac((L - n_lat) * T * ((h + g) * d * 4.0 + (h + 2 * g) * d * eb), bw, k_store))
    q_w = lh * (ld + lrd)
    out["row norm+rotation+store (hbm)"] = dict(ms=fz.get("latent_norm+rotary+append_ms"),
                                                frac=frac(T * ((2 * q_w + R + 2 * lh) * 4.0 + (2 * q_w + R) * eb + 2 * lh * 4.0), bw,
                                                          fz.get("latent_norm+rotary+append_ms")))
    out["kugirax latent norms+append (hbm)"] = dict(ms=kz.get("latent_norm+append_ms"),
                                                    frac=frac(T * (2 * fx["q_rank"] + R) * (4.0 + eb), bw, kz.get("latent_norm+append_ms")))
    # three passes per layer: the stream and the sublayer's sum read, both written (the sum as zeros); each also writes
    # the next reader's input (the last layer's last pass has no reader)
    post = (fz.get("attention_out_norm+mlp_norm_ms") or 0) + (fz.get("out_norm_ms") or 0) + (fz.get("side_out_norm_ms") or 0)
    out["norms into the stream (hbm)"] = dict(ms=post, frac=frac(T * W * (L * (3 * 4 * 4.0 + 2 * eb) + (L - 1) * eb), bw, post))
    # one launch: the first layer's (a layer's last pass over the stream writes the next layer's first norm)
    out["norm (hbm)"] = dict(ms=fz.get("attention_norm_ms"), frac=frac(T * W * (4.0 + eb), bw, fz.get("attention_norm_ms")))
    out["kugirax norm (hbm)"] = dict(ms=kz.get("input_norm_ms"), frac=frac(L * T * W * (4.0 + eb), bw, kz.get("input_norm_ms")))
    out["llama norm (hbm)"] = dict(ms=ll.get("attention_norm_ms"), frac=frac(T * W * (4.0 + eb), bw, ll.get("attention_norm_ms")))
    out["head gates (hbm)"] = dict(ms=fz.get("head_gate_ms"), frac=frac(T * ((L - n_lat) * h * d + n_lat * lh * lvd) * 2 * eb, bw, fz.get("head_gate_ms")))
    side = (fz.get("side_gate_ms") or 0) + (fz.get("side_projection_ms") or 0)
    out["token side input (hbm)"] = dict(ms=side, frac=frac(L * T * (W * eb + 3 * FOTULIX_SIDE * eb + W * 4.0 * 2), bw, side))
    f_ff = sum(v for k, v in fz.items() if "gate_projection" in k or "down_projection" in k)
    k_ff = sum(v for k, v in kz.items() if "gate_projection" in k or "down_projection" in k)
    ll_ff = sum(v for k, v in ll.items() if "gate_projection" in k or "down_projection" in k)
    out["feed-forward (tensor)"] = dict(ms=f_ff, frac=frac(L * T * 3 * 2.0 * W * ff, tf, f_ff))
    out["kugirax feed-forward (tensor)"] = dict(ms=k_ff, frac=frac(L * T * 3 * 2.0 * W * ff, tf, k_ff))
    out["llama feed-forward (tensor)"] = dict(ms=ll_ff, frac=frac(ll_runs * T * 3 * 2.0 * W * ff, tf, ll_ff))
    # a decode step streams every weight once and, per sequence, the cached keys and values (windowed rows: the window's)
    for label, kv_bytes in (("fotulix", B * T * (L - n_lat) * 2 * g * d * eb + B * win * R * eb),
                            ("kugirax", B * T * (L - n_lat) * 2 * g * d * eb + B * win * R * eb),
                            ("llama", B * T * ll_runs * 2 * nkv * hd * eb)):
        ms = row[label]["decode_ms_per_step"]
        out[f"{label} decode step (hbm)"] = dict(ms=ms, frac=frac(row[label]["weight_gb"] * 1e9 + kv_bytes, bw, ms))
    return out


def kernel_case(name: str, reps: int) -> int:
    """One kernel of the step alone, at the 1B shape, on rotating buffers larger than L2.

    Prints one JSON line with its time and its fraction of the measured peak. This is what the
    ncu summaries under profiles/ were captured from (``--kernel-case NAME --reps 3``).
    """
    import math
    import torch
    from types import SimpleNamespace
    from spissa_b200.csrc import lib as K
    peaks = load_peaks()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    H, I, V, nh, nkv, hd, T = 2048, 8192, 128256, 32, 8, 64, PROMPT
    bf = torch.bfloat16

    def rnd(*shape):
        return (torch.randn(*shape, device=dev) * 0.05).to(bf)

    flops = bytes_ = 0.0
    if name == "step_b8":
        # eight 2,048-token prompts one after another, then three decode steps at batch 8, kernel by kernel and
        # part by part (no CUDA graph, no one-kernel decode): the launch list of this run is what
        # profiles/step_b8_launches.md summarises
        from spissa_b200 import Engine, LlamaConfig
        eng = Engine.from_config(LlamaConfig.from_dict(CONFIG_1B), seed=0, dtype="bfloat16", max_tokens=8 * CONTEXT,
                                 max_seqs=8, use_graphs=False, fuse_decode=False)
        rng = random.Random(0)
        slots = [eng.acquire() for _ in range(8)]
        for sl in slots:
            eng.step([(sl, [rng.randrange(V) for _ in range(T)], [T - 1])])
        for i in range(3):
            eng.step([(sl, [5 + i], [0]) for sl in slots])
        torch.cuda.synchronize()
        print(json.dumps({"kernel_case": name, "launches": K.launches}))
        return 0
    if name == "fotulix_step":
        # the Fotulix decoder at the 2k size of --design: one prompt of 2,048 tokens, then three decode steps, kernel by
        # kernel (no CUDA graph): the launch list of this run is what profiles/fotulix_step_and_kernels.md summarises
        from spissa_b200 import Engine
        from spissa_b200.config import config_from_dict
        cfg = config_from_dict(fotulix_config(DESIGN_SIZES["2k"], FOTULIX_SIZES["2k"]))
        eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=T + 128, max_seqs=1, use_graphs=False)
        rng = random.Random(0)
        sl = eng.acquire()
        eng.step([(sl, [rng.randrange(DESIGN_VOCAB) for _ in range(T)], [T - 1])])
        l0 = K.launches
        for i in range(3):
            eng.step([(sl, [5 + i], [0])])
        torch.cuda.synchronize()
        print(json.dumps({"kernel_case": name, "launches": K.launches, "launches_per_decode_step": (K.launches - l0) // 3}))
        return 0
    if name == "prefill":
        # prompts of 2,048 tokens one after another through the engine's own step (the launch list of this run is
        # what profiles/prefill_step_fused_launches.md summarises)
        from spissa_b200 import Engine, LlamaConfig
        cfg = dict(CONFIG_1B)
        if KERNEL_CASE_LAYERS:
            cfg["num_hidden_layers"] = KERNEL_CASE_LAYERS
        eng = Engine.from_config(LlamaConfig.from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=2 * CONTEXT, max_seqs=2)
        rng = random.Random(0)
        times = []
        for i in range(max(2, reps)):
            sl = eng.acquire()
            toks = [rng.randrange(V) for _ in range(T)]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = K.launches
            e0.record()
            eng.step([(sl, toks, [T - 1])], greedy=True, check=False)
            e1.record()
            torch.cuda.synchronize()
            eng.check()
            times.append(e0.elapsed_time(e1))
            eng.release(sl)
        print(json.dumps({"kernel_case": name, "layers": cfg["num_hidden_layers"], "ms": [round(t, 3) for t in times],
                          "launches_per_step": K.launches - l0}))
        return 0
    if name == "decode_layers":
        # the one-kernel decode path alone: eight 2,048-token prompts, then decode steps launched one by one; the
        # last one records the global timer as CTA 0 enters and leaves each grid barrier (phase times per layer)
        import ctypes
        from spissa_b200 import Engine, LlamaConfig
        cfg = dict(CONFIG_1B)
        if KERNEL_CASE_LAYERS:
            cfg["num_hidden_layers"] = KERNEL_CASE_LAYERS
        nl = cfg["num_hidden_layers"]
        n_seqs = KERNEL_CASE_BATCH or 8
        eng = Engine.from_config(LlamaConfig.from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=n_seqs * CONTEXT,
                                 max_seqs=n_seqs, use_graphs=False)
        rng = random.Random(0)
        slots = [eng.acquire() for _ in range(n_seqs)]
        for sl in slots:
            eng.step([(sl, [rng.randrange(V) for _ in range(T)], [T - 1])])
        for i in range(max(1, reps - 1)):
            eng.step([(sl, [5 + i], [0]) for sl in slots])
        trace = torch.zeros(1024, dtype=torch.int64, device=dev)
        lib = K.load("decode_layers")
        lib.sp_decode_layers_set_trace(ctypes.c_void_p(trace.data_ptr()))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([(sl, [9], [0]) for sl in slots], greedy=True)
        e1.record()
        torch.cuda.synchronize()
        lib.sp_decode_layers_set_trace(ctypes.c_void_p(0))
        K.check_status(dev)
        t = trace.cpu().tolist()
        # six grid barriers per layer, or five where the chunks are combined inside the attention phase by CTA pairs
        # (the last layer's last barrier does not exist: the kernel ends there)
        per_layer = ["qkv", "attention", "combine", "output projection", "gate/up", "down"]
        if t[2 * 6 * nl] == 0:
            per_layer = ["qkv", "attention+combine", "output projection", "gate/up", "down"]
        names = ["input statistics"] + per_layer * nl
        work, wait = {}, {}
        for e in range(1, len(per_layer) * nl + 1):              # barrier e: entered at t[2e], left at t[2e + 1]
            work.setdefault(names[e - 1], []).append(t[2 * e] - t[2 * e - 1])
            wait.setdefault(names[e - 1], []).append(t[2 * e + 1] - t[2 * e])
        med = lambda v: sorted(v)[len(v) // 2] / 1e3
        last = len(per_layer) * nl                                # behind the last layer: the final norm and the head, if the kernel ran them
        head_us = round((t[1023] - t[2 * last + 1]) / 1e3, 2) if t[2 * last + 1] else None
        print(json.dumps({"kernel_case": name, "layers": nl, "sequences": n_seqs, "kernel_us": round((t[1023] - t[1]) / 1e3, 1),
                          "head_us": head_us,
                          "step_ms_with_host": round(e0.elapsed_time(e1), 3),
                          "phase_us_median": {k: round(med(v), 2) for k, v in work.items()},
                          "barrier_us_median": {k: round(med(v), 2) for k, v in wait.items()},
                          "fused_steps": eng.model._fused.runs if eng.model._fused else 0}))
        return 0
    if name in ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down"):
        from spissa_b200.parts.linear import tile_width
        N, Kd, mode, bn = {"gemm_qkv": (3072, H, K.TC_STORE, tile_width(T, 3072, 148)), "gemm_o": (H, H, K.TC_ACCUMULATE, tile_width(T, H, 148)),
                           "gemm_gate_up": (2 * I, H, K.TC_SILU_MUL, 256),
                           "gemm_down": (H, I, K.TC_ACCUMULATE, 256)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        a = rnd(T, Kd)
        out = torch.zeros(T, N // 2 if mode == K.TC_SILU_MUL else N,
                          dtype=torch.float32 if mode == K.TC_ACCUMULATE else bf, device=dev)
        run = lambda i: K.tc_gemm(a, ws[i % n_buf], out, mode, bn)
        flops = 2.0 * T * N * Kd
    elif name in ("fused_qkv", "fused_o", "fused_gate_up", "fused_down"):
        # the same products with the epilogues of a fused prompt step (engine/fused_prefill.py)
        from spissa_b200.parts.linear import tile_width
        N, Kd = {"fused_qkv": (3072, H), "fused_o": (H, H), "fused_gate_up": (2 * I, H), "fused_down": (H, I)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        a = rnd(T, Kd)
        ssq = torch.rand(T, 8, device=dev) + 1.0
        flops = 2.0 * T * N * Kd
        if name == "fused_qkv":
            bn = tile_width(T, N, 148)
            pages = T // 64
            kp, vp = rnd(pages, nkv, 64, hd), rnd(pages, nkv, 64, hd)
            q = torch.empty(T, nh * hd, dtype=bf, device=dev)
            cs = torch.rand(T, hd // 2, 2, device=dev)
            pos = torch.arange(T, dtype=torch.int32, device=dev)
            tok_page = (pos // 64).int()
            rope = dict(cs=cs, tok_page=tok_page, positions=pos, q_out=q, k_pool=kp, v_pool=vp, nh=nh, nkv=nkv, hd=hd, page_size=64)
            run = lambda i: K.tc_gemm_fused(a, ws[i % n_buf], None, K.TC_QKV_ROPE, bn, row_ssq=ssq, norm_width=H, eps=1e-5, rope=rope)
        elif name == "fused_gate_up":
            out = torch.empty(T, I, dtype=bf, device=dev)
            run = lambda i: K.tc_gemm_fused(a, ws[i % n_buf], out, K.TC_SILU_MUL, 256, row_ssq=ssq, norm_width=H, eps=1e-5)
        else:
            bn = tile_width(T, N, 148)
            out = torch.zeros(T, N, device=dev)
            xw = torch.empty(T, N, dtype=bf, device=dev)
            nw = rnd(N)
            so = torch.empty(T, K.tc_gemm_n_tiles(N, bn), device=dev)
            run = lambda i: K.tc_gemm_fused(a, ws[i % n_buf], out, K.TC_ACCUMULATE, bn, xw=xw, next_w=nw, ssq_out=so)
    elif name in ("stream_qkv", "stream_o", "stream_gate_up", "stream_down"):
        # the products of a decode step of 64 sequences: tc_stream.cu
        N, Kd, mode, pair = {"stream_qkv": (3072, H, K.TC_STORE, 0), "stream_o": (H, H, K.TC_ACCUMULATE, 0),
                             "stream_gate_up": (2 * I, H, K.TC_SILU_MUL, 128),
                             "stream_down": (H, I, K.TC_ACCUMULATE, 0)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        x = rnd(64, Kd)
        out = torch.zeros(64, N // 2 if mode == K.TC_SILU_MUL else N,
                          dtype=torch.float32 if mode == K.TC_ACCUMULATE else bf, device=dev)
        run = lambda i: K.tc_stream(x, ws[i % n_buf], out, mode, pair)
        bytes_ = N * Kd * 2.0
    elif name in ("stream_fused_qkv", "stream_fused_o", "stream_fused_gate_up", "stream_fused_down"):
        # the same products of 64 tokens with the fused epilogues (engine/fused_prefill.py, 17 to 64 tokens)
        N, Kd = {"stream_fused_qkv": (3072, H), "stream_fused_o": (H, H), "stream_fused_gate_up": (2 * I, H),
                 "stream_fused_down": (H, I)}[name]
        M = 64
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        a = rnd(M, Kd)
        ssq = torch.rand(M, 16, device=dev) + 1.0
        bytes_ = N * Kd * 2.0
        if name == "stream_fused_qkv":
            kp, vp = rnd(M, nkv, 64, hd), rnd(M, nkv, 64, hd)          # every token in a page of its own: a decode step
            q = torch.empty(M, nh * hd, dtype=bf, device=dev)
            cs = torch.rand(M, hd // 2, 2, device=dev)
            pos = torch.full((M,), 2047, dtype=torch.int32, device=dev)
            tok_page = torch.arange(M, dtype=torch.int32, device=dev)
            rope = dict(cs=cs, tok_page=tok_page, positions=pos, q_out=q, k_pool=kp, v_pool=vp, nh=nh, nkv=nkv, hd=hd, page_size=64)
            run = lambda i: K.tc_stream_fused(a, ws[i % n_buf], None, K.TC_QKV_ROPE, 0, row_ssq=ssq, norm_width=H, eps=1e-5, rope=rope)
        elif name == "stream_fused_gate_up":
            out = torch.empty(M, I, dtype=bf, device=dev)
            run = lambda i: K.tc_stream_fused(a, ws[i % n_buf], out, K.TC_SILU_MUL, 128, row_ssq=ssq, norm_width=H, eps=1e-5)
        else:
            out = torch.zeros(M, N, device=dev)
            xw = torch.empty(M, N, dtype=bf, device=dev)
            nw = rnd(N)
            so = torch.empty(M, K.tc_stream_n_tiles(N), device=dev)
            run = lambda i: K.tc_stream_fused(a, ws[i % n_buf], out, K.TC_ACCUMULATE, 0, xw=xw, next_w=nw, ssq_out=so)
    elif name in ("gemv_qkv", "gemv_o", "gemv_gate_up", "gemv_down", "gemv_head"):
        N, Kd, mode = {"gemv_qkv": (3072, H, K.TC_STORE), "gemv_o": (H, H, K.TC_ACCUMULATE),
                       "gemv_gate_up": (2 * I, H, K.TC_SILU_MUL), "gemv_down": (H, I, K.TC_ACCUMULATE),
                       "gemv_head": (V, H, K.TC_STORE)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        x = rnd(8, Kd)
        out = torch.zeros(8, N // 2 if mode == K.TC_SILU_MUL else N,
                          dtype=bf if mode == K.TC_SILU_MUL else torch.float32, device=dev)
        run = lambda i: K.gemv(x, ws[i % n_buf], out, mode, 128)
        bytes_ = N * Kd * 2.0
    elif name in ("flash_prefill", "flash_prefill_tc", "flash_decode", "flash_decode_b64", "flash_prefill_128",
                  "flash_prefill_tc_128"):
        if name.endswith("_128"):          # the 8B shape's attention: 32 heads of 128, 8 kv heads
            hd, name = 128, name[:-4]
        decode_batch = {"flash_decode": 8, "flash_decode_b64": 64}.get(name, 0)
        B = decode_batch or 1
        n_new = 1 if decode_batch else T
        pages = B * (T // 64)
        n_buf = 320 // decode_batch if decode_batch else 1    # 40 x 8.4 MB (5 x 67 MB) of keys and values > L2
        pools = [(rnd(pages, nkv, 64, hd), rnd(pages, nkv, 64, hd)) for _ in range(n_buf)]
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(B, T // 64)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        meta = SimpleNamespace(page_table=table, page_size=64, seq_slot=ar,
                               positions=(torch.arange(n_new, dtype=torch.int32, device=dev) + (T - n_new)).repeat(B),
                               token_seq=ar.repeat_interleave(n_new))
        q = rnd(B * n_new, nh * hd)
        out = torch.empty_like(q)
        scale = 1.0 / math.sqrt(hd)
        if name == "flash_prefill":
            seq_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
            run = lambda i: K.flash_prefill(q, pools[0][0], pools[0][1], out, meta, seq_start, 1, T // 64, nh, nkv,
                                            hd, None, scale)
            flops = 4.0 * (T * (T + 1) / 2) * hd * nh
        elif name == "flash_prefill_tc":
            seq_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
            run = lambda i: K.flash_prefill_tc(q, pools[0][0], pools[0][1], out, meta, seq_start, 1, T // 128, nh, nkv,
                                               hd, None, scale)
            flops = 4.0 * (T * (T + 1) / 2) * hd * nh
        else:
            seq_len = torch.full((B,), T, dtype=torch.int32, device=dev)
            ct, nc = K.flash_decode_plan(B, nkv, T)
            scratch = torch.empty(K.flash_decode_scratch_floats(B, nh, hd, nc), device=dev)
            run = lambda i: K.flash_decode(q, pools[i % n_buf][0], pools[i % n_buf][1], out, meta, seq_len, nh, nkv,
                                           hd, None, scale, ct, nc, scratch)
            bytes_ = B * T * nkv * hd * 2 * 2.0
    elif name in ("diff_flash", "diff_decode"):
        # the Duzinex attention at the 2k size of --design: 16 heads on 4 kv heads, maps of 64, values of 128, window 1,024
        # with 4 kept tokens, cap 30; a 2,048-token prompt, or one query each of 8 sequences with 2,048 cached tokens
        Hq, G, d, vd, win, keep = 16, 4, 64, 128, 1024, 4
        B = 8 if name == "diff_decode" else 1
        n_new = 1 if name == "diff_decode" else T
        pages = B * (T // 64)
        n_buf = 12 if name == "diff_decode" else 1
        pools = [(rnd(pages, G, 64, 2 * d), rnd(pages, G, 64, vd)) for _ in range(n_buf)]
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        meta = SimpleNamespace(page_table=torch.arange(pages, dtype=torch.int32, device=dev).view(B, T // 64), page_size=64,
                               seq_slot=ar, positions=(torch.arange(n_new, dtype=torch.int32, device=dev) + (T - n_new)).repeat(B),
                               token_seq=ar.repeat_interleave(n_new))
        q = rnd(B * n_new, Hq * 2 * d)
        out = torch.empty(B * n_new, Hq * vd, dtype=bf, device=dev)
        consts = (Hq, G, d, vd, win, keep, d ** -0.5, 30.0, 0.4, 1e-6, 0.5)
        if name == "diff_flash":
            seq_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
            run = lambda i: K.diff_flash_prefill(q, pools[0][0], pools[0][1], out, meta, seq_start, 1, T // 64, *consts)
            flops = (T * win - win * (win - 1) / 2) * Hq * (4.0 * d + 4.0 * vd)
        else:
            run = lambda i: K.diff_attention(q, pools[i % n_buf][0], pools[i % n_buf][1], out, meta, *consts)
            bytes_ = B * (win + keep) * G * (2 * d + vd) * 2.0
    elif name in ("retention_chunks", "retention_step", "mingru_chunks", "polynorm", "token_shift"):
        # the other Duzinex kernels at the 2k size of --design (8 retention heads of 128 x 256, width 2,048, ff 8,192)
        rh, rd, rvd, Wd, ff = 8, 128, 256, 2048, 8192
        B = 8 if name == "retention_step" else 1
        n_new = 1 if B > 1 else T
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        step = SimpleNamespace(seq_start=i32([n_new * b for b in range(B + 1)]), seq_slot=i32(list(range(B))),
                               token_seq=torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(n_new), n_seqs=B,
                               all_single=n_new == 1, max_new=n_new, host=dict(new_counts=[n_new] * B))
        if name.startswith("retention"):
            n_buf = 6 if B > 1 else 1
            proj = torch.randn(B * n_new, 2 * rh * rd + 2 * rh * rvd, device=dev)
            states = [torch.zeros(B, rh, rd, rvd, device=dev) for _ in range(n_buf)]
            decay = torch.full((rh,), 0.97, device=dev)
            out = torch.empty(B * n_new, rh * rvd, dtype=bf, device=dev)
            run = lambda i: K.retention(proj, states[i % n_buf], decay, out, step, rh, rd, rvd, 1e-6)
            if B > 1:
                bytes_ = B * rh * rd * rvd * 4 * 2.0
            else:
                flops = T * rh * 4.0 * rd * rvd              # the recurrence's own FLOPs (the chunked form does six times as many)
        elif name == "mingru_chunks":
            proj = torch.randn(T, 3 * Wd, device=dev)
            zb, xb = rnd(Wd), rnd(Wd)
            state = torch.zeros(1, Wd, device=dev)
            out = torch.empty(T, Wd, dtype=bf, device=dev)
            run = lambda i: K.mingru(proj, zb, xb, state, out, step, Wd)
            bytes_ = T * Wd * (2 * 3 * 4 + 2.0)
        elif name == "polynorm":
            zs = [torch.randn(T, ff, device=dev) for _ in range(3)]
            coef = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev).to(bf)
            out = torch.empty(T, ff, dtype=bf, device=dev)
            run = lambda i: K.polynorm(zs[i % 3], coef, out, 1e-6)
            bytes_ = T * ff * (4 + 2.0)
        else:
            xs = [torch.randn(T, Wd, device=dev) for _ in range(6)]
            w, b, al, mu = rnd(Wd), rnd(Wd), torch.full((1,), 0.5, device=dev).to(bf), rnd(Wd)
            state = torch.zeros(1, Wd, device=dev)
            out = torch.empty(T, Wd, dtype=bf, device=dev)
            run = lambda i: K.token_shift(xs[i % 6], mu, state, out, step, dyt=(w, b, al))
            bytes_ = T * Wd * (4 + 2.0)
    elif name in ("gla_chunks", "gla_step", "moe_experts", "moe_experts_b8", "streams_norm", "conv_qk_store"):
        # the Gozatar kernels at the 2k size of --design (8 heads of 128 x 256, width 2,048, 32 experts of 2,048, 4 per token)
        rh, rd, rvd, Wd, rank = 8, 128, 256, 2048, 16
        B = 8 if name in ("gla_step", "moe_experts_b8") else 1
        n_new = 1 if B > 1 else T
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        step = SimpleNamespace(seq_start=i32([n_new * b for b in range(B + 1)]), seq_slot=i32(list(range(B))),
                               token_seq=torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(n_new), n_seqs=B,
                               positions=torch.arange(n_new, dtype=torch.int32, device=dev).repeat(B),
                               all_single=n_new == 1, max_new=n_new, host=dict(new_counts=[n_new] * B))
        if name.startswith("gla"):
            n_buf = 6 if B > 1 else 1
            proj = torch.randn(B * n_new, 2 * rh * rd + 2 * rh * rvd + rank, device=dev)
            states = [torch.zeros(B, rh, rd, rvd, device=dev) for _ in range(n_buf)]
            a2, a2b, nw = rnd(rh * rd, rank), rnd(rh * rd), rnd(rvd)
            out = torch.empty(B * n_new, rh * rvd, dtype=bf, device=dev)
            run = lambda i: K.gla(proj, states[i % n_buf], a2, a2b, nw, out, step, rh, rd, rvd, rank, 16.0, 1e-6, 0.7)
            if B > 1:
                bytes_ = B * rh * rd * rvd * 4 * 2.0
            else:
                flops = T * rh * 4.0 * rd * rvd              # the recurrence's own FLOPs (the chunked form does several times as many)
        elif name.startswith("moe_experts"):
            E, top, F = 32, 4, 2048
            rows = B * n_new
            n_buf = 4 if B > 1 else 1                        # a decode step streams the experts it touches: rotate them
            gus = [rnd(E, 2 * F, Wd) for _ in range(n_buf)]
            dns = [rnd(E, Wd, F) for _ in range(n_buf)]
            x = rnd(rows, Wd)
            ids = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(rows)]).int().contiguous()
            wts = torch.full((rows, top), 1.0 / top, device=dev)
            y = torch.zeros(rows, Wd, device=dev)
            # gate and up rows in blocks of 128 (random weights: the layout only chooses the kernels): the prompt's pairs run
            # as grouped products of the tcgen05 tile kernel, the decode step's on mma.sync tiles
            run = lambda i: K.moe_experts(x, ids, wts, gus[i % n_buf], dns[i % n_buf], y, top, 7.0, glu_block=128)
            if B > 1:
                bytes_ = len(set(ids.flatten().tolist())) * 3.0 * F * Wd * 2
            else:
                flops = rows * top * 3 * 2.0 * Wd * F
        elif name == "streams_norm":
            S = 2
            xs = [torch.randn(T, S * Wd, device=dev) for _ in range(4)]
            ys = [torch.randn(T, Wd, device=dev) for _ in range(4)]
            mix, oc, ic, w = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(S, device=dev) / S, rnd(Wd)
            out = torch.empty(T, Wd, dtype=bf, device=dev)
            run = lambda i: K.streams_norm(xs[i % 4], S, Wd, out=out, weight=w, eps=1e-6, y=ys[i % 4], mix=mix, out_coef=oc, in_coef=ic)
            bytes_ = T * Wd * (2 * S * 4 + 2 * 4 + 2.0)
        else:
            nh, nkv, d = 16, 4, 128
            C = (nh + 2 * nkv) * d
            qkvs = [torch.randn(T, C, device=dev) for _ in range(4)]
            conv = rnd(C, 4)
            state = torch.zeros(1, 3, C, device=dev)
            inv_freq = (10000.0 ** (-torch.arange(0, d // 2, 2, device=dev).float() / (d // 2))).contiguous()
            q = torch.empty(T, nh * d, dtype=bf, device=dev)
            pages = T // 64
            kp, vp = rnd(pages, nkv, 64, d), rnd(pages, nkv, 64, d)
            meta = SimpleNamespace(page_table=torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages), page_size=64,
                                   seq_slot=i32([0]), positions=step.positions, token_seq=step.token_seq)
            run = lambda i: K.conv_qk_store(qkvs[i % 4], conv, 4, state, q, kp, vp, meta, step, inv_freq, nh, nkv, d, d, d // 2, 1e-6)
            bytes_ = T * C * (4 + 2.0)
    elif name in ("latent_flash", "latent_flash_b8", "latent_window_as_gqa", "latent_expanded", "latent_norm_store", "headwise_b8",
                  "headwise"):
        # the Kugirax latent attention at the 2k size of --design (16 heads over rows of 256, a window of 1,024, sinks)
        LH, r, d, qr, win = 16, 256, 128, 768, 1024
        B = 8 if name.endswith("_b8") else 1
        n_new = 1 if B > 1 else T
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        pos = (torch.arange(n_new, dtype=torch.int32, device=dev) + (T - n_new)).repeat(B)
        step = SimpleNamespace(seq_start=i32([n_new * b for b in range(B + 1)]), seq_slot=ar, token_seq=ar.repeat_interleave(n_new),
                               n_seqs=B, positions=pos, all_single=n_new == 1, max_new=n_new, max_len=T,
                               seq_len=i32([T] * B), host=dict(new_counts=[n_new] * B))
        pages = B * (T // 64)
        n_buf = 24 if B > 1 else 1                             # a decode step reads 8 x 1,024 rows of 512 bytes: rotate the pools
        pools = [rnd(pages, 1, 64, r) for _ in range(n_buf)]
        meta = SimpleNamespace(page_table=torch.arange(pages, dtype=torch.int32, device=dev).view(B, T // 64), page_size=64,
                               seq_slot=ar, positions=pos, token_seq=step.token_seq)
        sink = torch.zeros(LH, device=dev)
        rows = B * n_new
        pairs = B * (T * win - win * (win - 1) / 2) if B == 1 else B * win
        if name.startswith("latent_flash"):
            q = rnd(rows, LH * r)
            out = torch.empty_like(q)
            run = lambda i: K.latent_flash(q, pools[i % n_buf], out, meta, step, LH, r, win, d ** -0.5, sink, max_len=T if B > 1 else None)
            if B > 1:
                bytes_ = B * win * r * 2.0
            else:
                flops = 4.0 * pairs * r * LH
        elif name == "latent_window_as_gqa":
            # the grouped-query kernel of the same window on expanded heads of 128 (what a cache of keys and values would run)
            kp, vp = rnd(pages, 4, 64, d), rnd(pages, 4, 64, d)
            q = rnd(rows, LH * d)
            out = torch.empty_like(q)
            run = lambda i: K.flash_prefill(q, kp, vp, out, meta, step.seq_start, 1, T // 64, LH, 4, d, win, d ** -0.5, sink=sink)
            flops = 4.0 * pairs * d * LH
        elif name == "latent_expanded":
            # what a whole prompt runs: the tcgen05 kernel over the prompt's own expanded keys and values, as rows
            ks, vs = [rnd(rows, LH * d) for _ in range(4)], [rnd(rows, LH * d) for _ in range(4)]
            q = rnd(rows, LH * d)
            out = torch.empty_like(q)
            tiles = K.query_tiles([T], K.flash_tc_query_tile())
            run = lambda i: K.flash_prefill_tc_rows(q, ks[i % 4], vs[i % 4], out, step, tiles, LH, LH, d, win, d ** -0.5, sink)
            flops = 4.0 * pairs * d * LH
        elif name == "latent_norm_store":
            projs = [torch.randn(T, qr + r, device=dev) for _ in range(4)]
            wq, wc = rnd(qr), rnd(r)
            cq = torch.empty(T, qr, dtype=bf, device=dev)
            run = lambda i: K.latent_norm_store(projs[i % 4], qr, r, wq, wc, 1e-6, cq, pools[0], meta)
            bytes_ = T * (qr + r) * (4 + 2.0)
        else:
            n_w = 64 if B > 1 else 1
            uks = [rnd(LH * d, r) for _ in range(n_w)]
            a = rnd(rows, LH * d)
            out = torch.empty(rows, LH * r, dtype=bf, device=dev)
            # a decode step streams the stack stored with the outputs as rows, a warp per row
            run = lambda i: K.headwise_product(a, uks[i % n_w], out, LH, d, r, w_rows_are_k=B == 1)
            if B > 1:
                bytes_ = LH * d * r * 2.0
            else:
                flops = rows * LH * 2.0 * d * r
    elif name in ("distance_attention", "distance_attention_plain", "distance_attention_mma", "distance_decode_b8",
                  "distance_decode_b8_plain", "gated_qkv_store", "latent_rot_store", "stream_norm_add", "row_gates",
                  "rows_expanded"):
        # the Fotulix kernels at the 2k size of --design (16 heads of 128 on 4 kv heads, a table of 32 scores by distance
        # that reaches 4,096; width 2,048; 16 latent heads, rows of 192 + 64)
        FH, FG, Fd, Wd, r, rd = 16, 4, 128, 2048, 192, 64
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        B = 8 if "_b8" in name else 1
        n_new = 1 if B > 1 else T
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        pos = (torch.arange(n_new, dtype=torch.int32, device=dev) + (T - n_new)).repeat(B)
        step = SimpleNamespace(seq_start=i32([n_new * b for b in range(B + 1)]), seq_slot=ar, token_seq=ar.repeat_interleave(n_new),
                               n_seqs=B, positions=pos, all_single=n_new == 1, max_new=n_new, max_len=T,
                               seq_len=i32([T] * B), host=dict(new_counts=[n_new] * B))
        pages = B * (T // 64)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(B, T // 64)
        meta = SimpleNamespace(page_table=table, page_size=64, seq_slot=ar, positions=pos, token_seq=step.token_seq)
        rows = B * n_new
        if name.startswith("distance_"):
            from spissa_b200.parts.gated_attention import distance_table
            n_buf = 40 if B > 1 else 1
            pools = [(rnd(pages, FG, 64, Fd), rnd(pages, FG, 64, Fd)) for _ in range(n_buf)]
            dist = None if name.endswith("_plain") else distance_table(torch.randn(32, FH, device=dev), 4096.0)
            q = rnd(rows, FH * Fd)
            out = torch.empty_like(q)
            if B > 1:
                ct, nc = K.flash_decode_plan(B, FG, T)
                scratch = torch.empty(K.flash_decode_scratch_floats(B, FH, Fd, nc), device=dev)
                run = lambda i: K.flash_decode(q, pools[i % n_buf][0], pools[i % n_buf][1], out, meta, step.seq_len, FH, FG, Fd, None,
                                               Fd ** -0.5, ct, nc, scratch, dist_bias=dist)
                bytes_ = B * T * FG * Fd * 2 * 2.0
            elif name == "distance_attention_mma":
                run = lambda i: K.flash_prefill(q, pools[0][0], pools[0][1], out, meta, step.seq_start, 1, T // 64, FH, FG, Fd, None,
                                                Fd ** -0.5, dist_bias=dist)
                flops = 4.0 * (T * (T + 1) / 2) * Fd * FH
            else:
                run = lambda i: K.flash_prefill_tc(q, pools[0][0], pools[0][1], out, meta, step.seq_start, 1, T // 128, FH, FG, Fd,
                                                   None, Fd ** -0.5, dist_bias=dist)
                flops = 4.0 * (T * (T + 1) / 2) * Fd * FH
        elif name == "rows_expanded":
            # what a whole prompt's latent attention runs: the tcgen05 kernel over the prompt's own expanded keys (128 + 64
            # per head) and values (128) as rows, a window of 1,024
            kd, win = Fd + rd, 1024
            ks, vs = [rnd(T, FH * kd) for _ in range(4)], [rnd(T, FH * Fd) for _ in range(4)]
            q = rnd(T, FH * kd)
            out = torch.empty(T, FH * Fd, dtype=bf, device=dev)
            tiles = K.query_tiles([T], K.flash_tc_query_tile())
            run = lambda i: K.flash_prefill_tc_rows(q, ks[i % 4], vs[i % 4], out, step, tiles, FH, FH, kd, win, kd ** -0.5, None, vd=Fd)
            flops = 2.0 * (T * win - win * (win - 1) / 2) * (kd + Fd) * FH
        elif name == "gated_qkv_store":
            C = (FH + FG) * Fd + FG * Fd
            projs = [torch.randn(T, C + FH, device=dev) for _ in range(4)]
            bias = rnd(C)
            q = torch.empty(T, FH * Fd, dtype=bf, device=dev)
            gates = torch.empty(T, FH, device=dev)
            kp, vp = rnd(pages, FG, 64, Fd), rnd(pages, FG, 64, Fd)
            run = lambda i: K.gated_qkv_store(projs[i % 4], bias, q, kp, vp, meta, gates, None, FH, FG, Fd, Fd, 0, temp_coef=0.2,
                                              temp_every=512)
            bytes_ = T * ((C + FH) * 4.0 + C * 2.0 + FH * 4.0)
        elif name == "latent_rot_store":
            R = r + rd
            C = FH * R + R
            projs = [torch.randn(T, C + FH, device=dev) for _ in range(4)]
            wc = rnd(r)
            freq = (10000.0 ** (-torch.arange(0, rd, 2, device=dev).float() / rd)).contiguous()
            q = torch.empty(T, FH * R, dtype=bf, device=dev)
            gates = torch.empty(T, FH, device=dev)
            pool = rnd(pages, 1, 64, R)
            run = lambda i: K.latent_rot_store(projs[i % 4], wc, q, pool, meta, gates, freq, FH, r, rd, r, 1.2, 1e-6)
            bytes_ = T * ((C + FH) * 4.0 + C * 2.0 + FH * 4.0)
        elif name == "stream_norm_add":
            xs = [torch.randn(T, Wd, device=dev) for _ in range(6)]
            ys = [torch.randn(T, Wd, device=dev) for _ in range(6)]
            w1, w2 = torch.randn(Wd, device=dev), torch.randn(Wd, device=dev)
            out = torch.empty(T, Wd, dtype=bf, device=dev)
            run = lambda i: K.stream_norm_add(xs[i % 6], ys[i % 6], w1, 0.5, 1e-6, w_next=w2, out=out)
            bytes_ = T * Wd * (4 * 4.0 + 2.0)
        else:
            xs = [rnd(T * FH, Fd) for _ in range(12)]
            z = torch.randn(T * FH, device=dev)
            run = lambda i: K.scale_rows_sigmoid(xs[i % 12], z)
            bytes_ = T * FH * (Fd * 2 * 2.0 + 4.0)
    elif name in ("sample_b8", "sample_b64", "argmax_b8"):
        # the sampler on rows of 128,256 logits (standard deviation 4 after the temperature): temperature 0.8, top-p 0.95
        B = 64 if name.endswith("b64") else 8
        logits = [torch.randn(B, V, device=dev) * 3.2 for _ in range(4)]
        u = torch.rand(B, device=dev)
        out = torch.empty(B, dtype=torch.int32, device=dev)
        scratch = torch.empty(K.sample_scratch_keys(B, V), dtype=torch.int64, device=dev)
        if name.startswith("argmax"):
            run = lambda i: K.argmax_rows(logits[i % 4], out)
        else:
            run = lambda i: K.sample_rows(logits[i % 4], 0.8, 0, 0.95, u, scratch, out)
        bytes_ = B * V * 4.0
    else:
        print("unknown kernel case", name)
        return 2
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    # the launches are replayed from a CUDA graph so that the host's launch cost is not in the number
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(reps):
            run(3 + i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    K.check_status(dev)
    us = e0.elapsed_time(e1) * 1000.0 / reps
    line = {"kernel_case": name, "us": round(us, 2), "reps": reps, "peaks": peaks["source"]}
    if flops:
        line.update(tflops=round(flops / us / 1e6, 1), frac=round(flops / us / 1e6 / peaks["bf16_tflops"], 4))
    if bytes_:
        line.update(gbs=round(bytes_ / us / 1e3, 1), frac=round(bytes_ / us / 1e3 / peaks["hbm_gbs"], 4))
    print(json.dumps(line))
    return 0


def main() -> int:
    global PROMPT, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed decode steps (default: the workload's: 64, 256 or 512)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="1b", choices=sorted(WORKLOADS), help="the headline workload (1b) or a secondary one")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the true 32-bit path of the whole model (FFMA products, no tensor cores); its prefill "
                         "fraction is of the nominal FFMA rate (148 SMs x 128 lanes x 2 x the maximum SM clock)")
    ap.add_argument("--context", type=int, default=None,
                    help="mean prompt length of the decode runs (the cache holds twice as much per sequence)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--points", default=None, help="extra decode batch sizes, comma separated ('' = none)")
    ap.add_argument("--profile-phases", action="store_true", dest="profile_phases",
                    help="add per-phase timings of one prompt step and of part-by-part decode steps")
    ap.add_argument("--kernel-case", default=None,
                    help="time one kernel alone (gemm_qkv|gemm_o|gemm_gate_up|gemm_down|gemv_qkv|gemv_o|gemv_gate_up|"
                         "gemv_down|gemv_head|diff_flash|diff_decode|retention_chunks|retention_step|mingru_chunks|polynorm|token_shift|gla_chunks|gla_step|moe_experts|moe_experts_b8|streams_norm|conv_qk_store|stream_qkv|stream_o|stream_gate_up|stream_down|stream_fused_qkv|stream_fused_o|stream_fused_gate_up|stream_fused_down|flash_prefill[_128]|flash_prefill_tc[_128]|flash_decode[_b64]|sample_b8|sample_b64|argmax_b8|decode_layers|step_b8|prefill|fused_qkv|fused_o|fused_gate_up|fused_down) instead of the step")
    ap.add_argument("--design", default=None, choices=["duzinex", "gozatar", "kugirax", "fotulix"],
                    help="measure this design beside the Llama decoder at equal layer sizes instead of the headline workload")
    ap.add_argument("--design-sizes", default="", dest="design_sizes", help="which of 1k,2k,4k (default: all)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--case-layers", type=int, default=0, help="layers of the model in --kernel-case decode_layers (0: all)")
    args = ap.parse_args()
    if args.kernel_case:
        global KERNEL_CASE_LAYERS, KERNEL_CASE_BATCH
        KERNEL_CASE_LAYERS = args.case_layers
        KERNEL_CASE_BATCH = args.batch or 0
        return kernel_case(args.kernel_case, args.reps)

    if args.design:
        return design_compare(args)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Erik-cpu-create/spissa is a Rust CPU project with no Python package "
                          "(pip: neither setup.py nor pyproject.toml) and no Rust toolchain is installed"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this library runs on ONE GPU; --gpus %d is not supported" % args.gpus)
        return 2
    if args.warmup < 3:
        args.warmup = 3
    global SPAN
    work = WORKLOADS[args.config]
    args.steps = args.steps or work["steps"]
    args.batch = args.batch or work["batch"]
    args.points = work["points"] if args.points is None else args.points
    CONTEXT, SPAN = work["context"], work["span"]
    PROMPT = work["prompt"] or (SPAN[0] + SPAN[1]) // 2
    if args.context is not None and args.context != PROMPT:
        SPAN = None
        if args.context < 64:
            print("bench.py: --context must be at least 64")
            return 2
        PROMPT, CONTEXT = args.context, max(2 * args.context, PREFILL_TOKENS + 64)

    import torch
    from spissa_b200 import Engine, LlamaConfig, SamplingParams
    from spissa_b200.csrc import lib

    peaks = load_peaks()
    cfg_dict = dict(work["cfg"])
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = LlamaConfig.from_dict(cfg_dict)
    fp32 = args.dtype == "float32"
    nums = model_numbers(cfg, 4 if fp32 else 2)
    points = [int(x) for x in args.points.split(",") if x.strip()]
    max_batch = max([args.batch] + points)
    torch.cuda.set_device(0)
    engine = Engine.from_config(cfg, seed=0, dtype=args.dtype, max_tokens=max_batch * CONTEXT,
                                max_seqs=max_batch, device="cuda:0")
    rng = random.Random(1234)
    V = cfg.vocab_size

    def prompts_for(batch):
        return [[rng.randrange(V) for _ in range(n)] for n in ragged_lengths(batch, 99 + batch)]

    from spissa_b200.sampling import Sampler
    sampler = Sampler(engine.device)
    greedy = SamplingParams()

    def decode_run(batch, steps, warmup):
        """Device-timed decode steps at ``batch`` after a ragged prefill; returns (ms per step, kv tokens, launches)."""
        prompts = prompts_for(batch)
        slots = [engine.acquire() for _ in range(batch)]
        # prompts go in as chunks so that a step never carries more than 8k tokens
        fed = [0] * batch
        while any(f < len(p) for f, p in zip(fed, prompts)):
            ents, room = [], 8192
            for b in range(batch):
                n = min(len(prompts[b]) - fed[b], room)
                if n > 0:
                    ents.append((slots[b], prompts[b][fed[b]:fed[b] + n], []))
                    fed[b] += n
                    room -= n
                if room == 0:
                    break
            engine.step(ents, check=False)
        engine.check()
        toks = [rng.randrange(V) for _ in range(batch)]

        def one():
            # launched back to back: the steps are confirmed (status word read) by ``engine.check()`` after the timing;
            # greedy: the head returns the tokens (no logits are written), as in ``Engine.generate``
            return engine.step([(s, [t], [0]) for s, t in zip(slots, toks)], check=False, greedy=True)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        kv_tokens = sum(engine.length(s) for s in slots) + batch * steps // 2
        l0 = lib.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = lib.launches - l0
        engine.check()
        for s in slots:
            engine.release(s)
        return ms, kv_tokens, launches, [len(p) for p in prompts]

    # ---------------------------------------------------------------- decode, device timed
    clocks = ClockSampler()
    clocks.start()
    ms_step, kv_tokens, launches, prompt_lens = decode_run(args.batch, args.steps, args.warmup)
    clock_info = clocks.stop()
    value = args.batch * 1000.0 / ms_step
    step_bytes = nums["weight_bytes"] + kv_tokens * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # ---------------------------------------------------------------- end to end through Engine.generate
    e2e_prompts = prompts_for(args.batch)
    # long enough that the first steps after the prompts (the SM clock is still under the power cap of the prompt
    # steps: 1.15 ms per step falling to 1.02 within some fifty steps) do not set the number
    e2e_new = max(args.steps, 256)
    engine.generate(e2e_prompts, 4, greedy, stop_ids=[])          # warm the path: the same shapes, so their graphs exist
    torch.cuda.synchronize()
    # three runs, the median one is reported (the host takes part in this number: it varies more than the device's)
    runs = []
    for _ in range(3):
        t0 = time.perf_counter()
        h2d0, steps0 = engine.h2d_bytes, engine.steps_run
        results, metrics = engine.generate(e2e_prompts, e2e_new, greedy, stop_ids=[])
        torch.cuda.synchronize()
        runs.append((metrics.decode_tok_s, (engine.h2d_bytes - h2d0) / max(1, engine.steps_run - steps0),
                     time.perf_counter() - t0))
    runs.sort()
    # every step copies its positions, slots, lengths and (when they changed) page tables to the device and the
    # chosen tokens (int32 per sequence) and the status word (int32) back to the host; the prompt's token ids go up
    # with the first step
    e2e = dict(value=round(runs[1][0], 2), unit="tokens/s", h2d_bytes_per_step=round(runs[1][1]),
               d2h_bytes_per_step=4 * args.batch + 4, new_tokens=e2e_new, wall_s=round(runs[1][2], 3),
               runs=[round(r[0], 1) for r in runs])

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    prompt = [rng.randrange(V) for _ in range(PREFILL_TOKENS)]

    def prefill_once():
        s = engine.acquire()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step([(s, prompt, [PREFILL_TOKENS - 1])], check=False, greedy=True)       # ends with the first token chosen
        e1.record()
        torch.cuda.synchronize()
        engine.check()
        engine.release(s)
        return e0.elapsed_time(e1)

    for _ in range(3):
        prefill_once()
    pre_ms = sorted(prefill_once() for _ in range(5))[2]
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    flop_peak = peaks["bf16_tflops"] * 1e12
    if fp32:
        flop_peak = 148 * 128 * 2 * (clock_info.get("sm_max_mhz") or 1965) * 1e6
    prefill = dict(value=round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), tokens=PREFILL_TOKENS, ms=round(pre_ms, 3),
                   frac=round(flops / (pre_ms * 1e-3) / flop_peak, 4))

    # ---------------------------------------------------------------- other batch sizes
    pts = {}
    for b in points:
        ms_b, _, _, _ = decode_run(b, max(8, args.steps // 2), 3)
        pts[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)

    # ---------------------------------------------------------------- per-phase timings, on request
    phases_out = None
    if args.profile_phases:
        from spissa_b200 import phases as ph
        engine.profile_phases = True
        engine.phase_totals.clear()
        s = engine.acquire()
        engine.step([(s, prompt, [PREFILL_TOKENS - 1])], greedy=True)
        engine.release(s)
        short = [prompts_for(args.batch)[b][:256] for b in range(args.batch)]
        slots = [engine.acquire() for _ in range(args.batch)]
        engine.step([(sl, p, []) for sl, p in zip(slots, short)], check=True)
        engine.phase_totals.pop("decode", None)
        n_dec = 4
        for i in range(n_dec):
            engine.step([(sl, [7 + i], [0]) for sl in slots], greedy=True)
        for sl in slots:
            engine.release(sl)
        engine.profile_phases = False
        L = len(engine.model.spec.schedule)
        pre = engine.phase_totals["prefill"]
        dec = engine.phase_totals["decode"]
        # the prompt entry sums the 2,048-token prompt and the short prompts that the decode steps start from
        phases_out = {"prompt_steps": dict(steps=pre["steps"], tokens=pre["tokens"], **ph.summary(dict(pre["ms"]), L)),
                      "decode_part_by_part_per_step": dict(batch=args.batch, context=256,
                                                           **ph.summary({k: v / n_dec for k, v in dec["ms"].items()}, L))}

    line = {
        "metric": "decode tokens/s (%s, batch %d, ~%d-token prompts)" % (work["model"], args.batch, PROMPT),
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32" if fp32 else "bf16", "data": "synthetic token ids, random N(0,0.02) weights", "impl": "ours",
        "config": {
            "model": work["model"], "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len_mean": round(sum(prompt_lens) / len(prompt_lens)),
            "prompt_len_min": min(prompt_lens), "prompt_len_max": max(prompt_lens), "page_size": engine.page_size,
            "tied_head": bool(cfg_dict.get("tie_word_embeddings")), "decode_steps": args.steps,
            "parallelism": "single-gpu", "l2": "inputs larger than L2 (%.2f GB of weights per step)" % (nums["weight_bytes"] / 1e9),
            "peaks": peaks["source"],
        },
        "clocks": clock_info,
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": pts,
    }
    if phases_out is not None:
        line["phases"] = phases_out
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
