"""Throughput of another design beside the closest existing model at equal size (``bench.py --design NAME``).

For each size the design's model and a Qwen3 dense model of the same width, depth, heads, feed-forward size and vocabulary
(for Megusun and Bumotar: a Topunex model, the closest one, with the same width, depth, projection sizes, experts and vocabulary;
its entry keeps the key "dense") are built with random weights (bfloat16) and timed through the step function:

  prefill   one step of 2,048 prompt tokens (tokens a second, ms)
  decode    steps of single tokens of 8 requests whose context ends at 2,048 (tokens a second, ms per step)

and one prefill step and a few decode steps are run once more with every launch bracketed by CUDA events, which gives
the device time per kernel class.  For the kernels that are the design's own, and for the dense model's like kernels,
the line states the work the kernel must do (bytes it must move, floating-point operations), the time that work takes
at the peaks (copy bandwidth; the bf16 tensor peak for contractions) and the fraction of it that was reached.
"""
from __future__ import annotations

import json
import math
from typing import Dict, List, Tuple

PAGE = 16
PROMPT = 2048
BATCH, CONTEXT = 8, 2048

# Sizes that resemble layers of real models.  A group of four layers: latent attention with its own latent, the
# recurrent mixer (no feed-forward), chunked attention, latent attention on the borrowed latent.
SIZES = {
    "2k": dict(width=2048, groups=2, heads=16, kv_heads=4, dim=128, rot=64, rank=512, inner=4096, state=16, dt_rank=128,
               conv=4, ff=8192, chunk=1024, vocab=32000),
    "4k": dict(width=4096, groups=2, heads=32, kv_heads=8, dim=128, rot=64, rank=512, inner=8192, state=16, dt_rank=256,
               conv=4, ff=12288, chunk=1024, vocab=32000),
}


def bubotar_config(z: dict) -> dict:
    lat = dict(heads=z["heads"], dim=z["dim"], rot_dim=z["rot"], vdim=z["dim"], kv_rank=z["rank"],
               scale=1.0 / math.sqrt(z["dim"] + z["rot"]), rot=dict(base=10000.0, dims=z["rot"]))
    mlp = dict(kind="dense", ff=z["ff"], limit=7.0)
    layers = []
    for g in range(z["groups"]):
        layers += [dict(type="latent_attention", mixer=dict(lat), mlp=dict(mlp)),
                   dict(type="mamba1", mixer=dict(inner=z["inner"], state=z["state"], dt_rank=z["dt_rank"], conv=z["conv"]), mlp=None),
                   dict(type="attention", mixer=dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"],
                                                     scale=1.0 / math.sqrt(z["dim"]), mask=dict(size=z["chunk"])), mlp=dict(mlp)),
                   dict(type="latent_attention", mixer=dict(lat, kv_from=4 * g), mlp=dict(mlp))]
    return dict(architecture="Bubotar", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-6), logit_scale=1.0, layers=layers)


# Topunex at sizes that resemble layers of real models: grouped attention with a window of 1,024 tokens below which the
# first 4 keys stay visible, half of each head rotating; the first layer's feed-forward dense, the others 32 experts of
# which a token uses 4, beside a shared expert.
TOPUNEX_SIZES = {
    "2k": dict(width=2048, layers=8, heads=16, kv_heads=4, dim=128, rot=64, window=1024, keep=4, ff=8192, experts=32, top=4,
               expert_ff=1024, shared_ff=2048, vocab=32000),
    "4k": dict(width=4096, layers=8, heads=32, kv_heads=8, dim=128, rot=64, window=1024, keep=4, ff=12288, experts=32, top=4,
               expert_ff=2048, shared_ff=4096, vocab=32000),
}


def topunex_config(z: dict) -> dict:
    mixer = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"], scale=1.0 / math.sqrt(z["dim"]), softcap=30.0,
                 mask=dict(size=z["window"], keep_first=z["keep"]),
                 rot=dict(base=500000.0, dims=z["rot"], scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    moe = dict(kind="moe", expert=dict(ff=z["expert_ff"], limit=7.0), router=dict(experts=z["experts"], top=z["top"], scale=1.0),
               shared=dict(ff=z["shared_ff"], limit=7.0))
    layers = [dict(type="attention", mixer=dict(mixer), mlp=dict(kind="dense", ff=z["ff"]) if i == 0 else dict(moe))
              for i in range(z["layers"])]
    return dict(architecture="Topunex", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-6), layers=layers)


# Megusun at sizes that resemble layers of real models: of every four layers three have the recurrent mixer and one the
# differential attention (two score maps of 64 per head over values of 128, so a head's query and key rows are as wide as
# a head of 128); the feed-forwards alternate between a dense one and 32 experts of which a token uses 4, beside a gated
# shared expert.  The shape also carries what the model beside it needs (Topunex: a window, kept keys, rotating dimensions).
MEGUSUN_SIZES = {
    "1k": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=128, map_dim=64, vdim=128, gru=1024, rot=64, window=1024, keep=4,
               ff=4096, experts=16, top=2, expert_ff=512, shared_ff=1024, vocab=32000),
    "2k": dict(width=2048, layers=8, heads=16, kv_heads=4, dim=128, map_dim=64, vdim=128, gru=2048, rot=64, window=1024, keep=4,
               ff=8192, experts=32, top=4, expert_ff=1024, shared_ff=2048, vocab=32000),
    "4k": dict(width=4096, layers=8, heads=32, kv_heads=8, dim=128, map_dim=64, vdim=128, gru=4096, rot=64, window=1024, keep=4,
               ff=12288, experts=32, top=4, expert_ff=2048, shared_ff=4096, vocab=32000),
}


def megusun_layers(z: dict):
    """(mixer type, feed-forward kind) per layer: recurrent + dense, recurrent + experts, attention + dense, recurrent + experts."""
    pattern = [("mingru", "dense"), ("mingru", "moe"), ("attention", "dense"), ("mingru", "moe")]
    return [pattern[i % 4] for i in range(z["layers"])]


def megusun_config(z: dict) -> dict:
    att = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["map_dim"], vdim=z["vdim"], scale=1.0 / math.sqrt(z["map_dim"]), diff=0.6,
               q_temp=dict(coef=0.5, every=64))
    moe = dict(kind="moe", expert=dict(ff=z["expert_ff"]), router=dict(experts=z["experts"], top=z["top"]), shared=dict(ff=z["shared_ff"]))
    layers = [dict(type=mixer, mixer=dict(att) if mixer == "attention" else dict(width=z["gru"]),
                   mlp=dict(kind="dense", ff=z["ff"]) if ff == "dense" else dict(moe)) for mixer, ff in megusun_layers(z)]
    return dict(architecture="Megusun", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-6), residual_mult=0.5, layers=layers)


def megusun_work(z: dict, phase: str) -> Dict[str, Tuple[float, float, str]]:
    """Per kernel class of Megusun: (bytes it must move, flops, what the flops run on) summed over the layers of a step."""
    n = PROMPT if phase == "prefill" else BATCH
    seqs = 1 if phase == "prefill" else BATCH
    start = 0 if phase == "prefill" else CONTEXT - 1
    kinds = megusun_layers(z)
    L, w = len(kinds), z["width"]
    La = sum(1 for m, _ in kinds if m == "attention")
    Lg, Ld, Lm = L - La, sum(1 for _, f in kinds if f == "dense"), sum(1 for _, f in kinds if f == "moe")
    H, G, D, V, W = z["heads"], z["kv_heads"], z["map_dim"], z["vdim"], z["gru"]
    E, top, fe, fs = z["experts"], z["top"], z["expert_ff"], z["shared_ff"]
    steps = 1 if phase == "prefill" else 4
    pairs = seqs * _pairs(n // seqs, start)
    keys_read = seqs * (start + n // seqs)
    attention = (La * (keys_read * (2 * G * D + G * V) * 2 + n * 2 * H * (D * 4 + V * 4)), La * 2.0 * 2 * H * 2 * (D + V) * pairs)      # float32 queries in, float32 maps out
    distinct = E * (1.0 - (1.0 - top / E) ** n)
    work = {
        "paged_attention_general_tc": (attention[0], attention[1], "bf16 tensor"),
        "paged_attention_general_tiled": (attention[0], attention[1], "fp32 FMA"),
        "paged_attention_general": (attention[0], attention[1], "fp32 FMA"),
        "qkv_split_write": (La * n * (2 * H * D * (2 + 4) + (2 * G * D + G * V) * 4), 0.0, ""),
        "diff_combine": (La * n * H * V * (2 * 4 + 2), 0.0, ""),                       # two float32 maps in, one head out
        "norm_shift": (n * w * (4 + 2 + 2), 0.0, ""),                                  # the first layer's; the others' ride in parallel_add
        "parallel_add": (n * w * ((L - 1) * (4 + 2 + 2 + 4 + 2 + 2) + (4 + 2 + 2 + 4)), 0.0, ""),
        "activation": (Ld * n * z["ff"] * (4 + 2), 0.0, ""),
        "min_gru": (Lg * (n * W * (12 + 2) + seqs * W * 8), Lg * n * W * 20.0, "fp32 FMA"),
        "moe_route": (Lm * (n * w * 2 + (E + 1) * w * 4), 0.0, ""),
        "moe_grouped": (Lm * (distinct * 3 * w * fe * 2 + n * w * 4 + n * top * (fe * 4 + w * 8)), Lm * 2.0 * n * top * 3 * w * fe, "bf16 tensor"),
        "moe_gate_up": (Lm * (n * top * 2 * fe * w * 2 + n * w * 2), Lm * 4.0 * n * top * fe * w, "fp32 FMA"),
        "moe_down": (Lm * (n * top * fe * w * 2 + n * w * 4), Lm * 2.0 * n * top * fe * w, "fp32 FMA"),
        "silu_mul": (Lm * n * fs * 6, 0.0, ""),
    }
    return {k: (b * steps, f * steps, on) for k, (b, f, on) in work.items()}


# Bumotar at sizes that resemble layers of real models: six layers (parallel, latent, parallel, parallel, latent, parallel) of which
# the second and third are walked twice, eight layer runs in all.  A parallel layer has a window attention (heads of 128, half of
# each rotating, a cap, a window of 1,024) beside a retention (as many heads, keys of 64, values of 128); a latent layer has a latent
# of 512 and a rotated part of 64; every layer has 32 experts of which a token uses 4, beside a gated shared expert.  The shape
# also carries what the model beside it needs (Topunex: eight layers, kept keys, a dense first feed-forward).
BUMOTAR_SIZES = {
    "1k": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=128, rot=64, window=1024, keep=4, ret_dim=64, ret_vdim=128, rank=512,
               ff=4096, experts=16, top=2, expert_ff=512, shared_ff=1024, vocab=32000),
    "2k": dict(width=2048, layers=8, heads=16, kv_heads=4, dim=128, rot=64, window=1024, keep=4, ret_dim=64, ret_vdim=128, rank=512,
               ff=8192, experts=32, top=4, expert_ff=1024, shared_ff=2048, vocab=32000),
    "4k": dict(width=4096, layers=8, heads=32, kv_heads=8, dim=128, rot=64, window=1024, keep=4, ret_dim=64, ret_vdim=128, rank=512,
               ff=12288, experts=32, top=4, expert_ff=2048, shared_ff=4096, vocab=32000),
}
BUMOTAR_RUNS = ["parallel", "latent", "parallel", "latent", "parallel", "parallel", "latent", "parallel"]      # the eight layer runs


def bumotar_config(z: dict) -> dict:
    H = z["heads"]
    left = dict(heads=H, kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"], scale=1.0 / math.sqrt(z["dim"]), softcap=30.0,
                mask=dict(size=z["window"]), rot=dict(base=100000.0, dims=z["rot"], scaling=dict(factor=4.0)))
    right = dict(heads=H, dim=z["ret_dim"], vdim=z["ret_vdim"], decay=[1.0 - 2.0 ** (-5.0 - 5.0 * h / max(1, H - 1)) for h in range(H)],
                 rot=dict(base=10000.0, dims=z["ret_dim"]))
    par = dict(type="parallel", mixer=dict(left=left, right=right, left_scale=0.5, right_scale=1.0))
    lat = dict(type="latent_attention", mixer=dict(heads=H, dim=z["dim"], rot_dim=z["rot"], vdim=z["dim"], kv_rank=z["rank"],
                                                   scale=1.0 / math.sqrt(z["dim"] + z["rot"]),
                                                   rot=dict(base=10000.0, dims=z["rot"], scaling=dict(factor=4.0, original=4096, fast=32.0, slow=1.0))))
    moe = dict(kind="moe", expert=dict(ff=z["expert_ff"]), router=dict(experts=z["experts"], top=z["top"]), shared=dict(ff=z["shared_ff"]))
    order = [par, lat, par, par, lat, par]
    layers = [dict(copy_of, mlp=dict(moe)) for copy_of in order]
    return dict(architecture="Bumotar", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-6), logit_scale=1.0, layers=layers,
                loop=dict(start=1, stop=3, times=2))


def bumotar_work(z: dict, phase: str) -> Dict[str, Tuple[float, float, str]]:
    """Per kernel class of Bumotar: (bytes it must move, flops, what the flops run on) summed over the layer runs of a step."""
    n = PROMPT if phase == "prefill" else BATCH
    seqs = 1 if phase == "prefill" else BATCH
    start = 0 if phase == "prefill" else CONTEXT - 1
    Lp, Ll = BUMOTAR_RUNS.count("parallel"), BUMOTAR_RUNS.count("latent")
    L, w = Lp + Ll, z["width"]
    H, G, d, rot, rank = z["heads"], z["kv_heads"], z["dim"], z["rot"], z["rank"]
    D, V = z["ret_dim"], z["ret_vdim"]
    E, top, fe, fs = z["experts"], z["top"], z["expert_ff"], z["shared_ff"]
    steps = 1 if phase == "prefill" else 4
    row = rank + rot
    win_pairs = seqs * _window_pairs(n // seqs, start, z["window"], 0)
    all_pairs = seqs * _pairs(n // seqs, start)
    keys_read = seqs * min(start + n // seqs, z["window"] + (n // seqs if phase == "prefill" else 0))
    window = (Lp * (keys_read * G * 2 * d * 2 + n * H * d * (4 + 2)), Lp * 4.0 * H * d * win_pairs)
    if phase == "prefill":          # the latent layers expand their keys: heads of their own, keys d + rot wide, values d wide
        latent = (Ll * n * H * ((d + rot) * (4 + 2) + d * 4), Ll * 2.0 * H * (2 * d + rot) * all_pairs)
    else:                           # the absorbed form over the cached rows: keys rank + rot wide, values rank wide
        latent = (Ll * (seqs * (start + 1) * row * 2 + n * H * (row * 4 + rank * 2)), Ll * 2.0 * H * (row + rank) * all_pairs)
    attention = (window[0] + latent[0], window[1] + latent[1])
    chunk = 32
    chunks = n // chunk if phase == "prefill" else 0
    retention = (Lp * (n * (2 * H * (D + V) * 4 + 2 * H * D * 4 * 2 + H * V * 2) + seqs * H * D * V * 8 + chunks * H * D * V * 4 * 3),
                 Lp * n * H * (4.0 * D * V + (chunk * (D + V) if phase == "prefill" else 0.0)))
    distinct = E * (1.0 - (1.0 - top / E) ** n)
    work = {
        "paged_attention_general_tc": (attention[0], attention[1], "bf16 tensor"),
        "paged_attention_general_tiled": (attention[0], attention[1], "fp32 FMA"),
        "paged_attention_general": (attention[0], attention[1], "fp32 FMA"),
        "retention": (retention[0], retention[1], "fp32 FMA"),
        "qk_prepare": (Lp * n * ((H + 2 * G) * d * 4 + H * d * 4 + 2 * G * d * 2), 0.0, ""),
        "sigmoid_gate_strided": (Lp * n * H * d * (4 + 2 + 2) + Ll * n * H * (d * 4 + 2), 0.0, ""),
        "scaled_sum": (Lp * n * w * (4 + 4 + 2), 0.0, ""),
        "concat_streams": (2 * n * w * (4 + 2 + 4 + 4), 0.0, ""),
        "add_bias": (2 * n * w * 8, 0.0, ""),
        "heads_linear": (Ll * (2 * H * d * rank * 2 + n * H * (d * 2 + rank * 4 + rank * 2 + d * 2)), Ll * 2.0 * n * H * d * rank * 2, "fp32 FMA"),
        "latent_prepare": (Ll * (n * H * (rot * 2 + rot * 4) + n * row * 4), 0.0, ""),
        "latent_expand_keys": (Ll * n * H * (2 * d + rot) * 2, 0.0, ""),
        "add_rmsnorm": ((2 * L + 1) * n * w * (4 + 4 + 2 + 2), 0.0, ""),
        "moe_route": (L * (n * w * 2 + (E + 1) * w * 4), 0.0, ""),
        "moe_grouped": (L * (distinct * 3 * w * fe * 2 + n * w * 4 + n * top * (fe * 4 + w * 8)), L * 2.0 * n * top * 3 * w * fe, "bf16 tensor"),
        "moe_gate_up": (L * (n * top * 2 * fe * w * 2 + n * w * 2), L * 4.0 * n * top * fe * w, "fp32 FMA"),
        "moe_down": (L * (n * top * fe * w * 2 + n * w * 4), L * 2.0 * n * top * fe * w, "fp32 FMA"),
        "silu_mul": (L * n * fs * 6, 0.0, ""),
    }
    return {k: (b * steps, f * steps, on) for k, (b, f, on) in work.items()}


def dense_config(z: dict) -> dict:
    n = z["layers"] if "layers" in z else 4 * z["groups"]
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=z["vocab"], hidden_size=z["width"],
                intermediate_size=z["ff"], num_hidden_layers=n, num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
                head_dim=z["dim"], rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
                sliding_window=None, max_window_layers=n, hidden_act="silu", attention_bias=False, initializer_range=0.02,
                eos_token_id=-1)


def build(raw: dict):
    import torch
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.engine.engine import Engine
    from pulsar_b200.models import build_model
    from pulsar_b200.weights import load_random
    cfg = config_from_dict(raw)
    model = build_model(cfg, torch.bfloat16)
    load_random(model, 0, 0.02, "cuda:0")
    pages = BATCH * (-(-(CONTEXT + PAGE) // PAGE)) + PROMPT // PAGE + 8
    engine = Engine.from_model(cfg, model, dict(dtype="bfloat16", device="cuda:0", page_size=PAGE, num_pages=pages,
                                                max_sessions=BATCH + 1, max_running=BATCH + 1, max_chunk_size=PROMPT, eos_id=-1,
                                                temperature=0.0))
    for g in engine.cache.groups:
        for pool in g.pools.values():
            pool.normal_(0.0, 1.0)
    return engine


def profiled(engine, bench) -> Tuple[Dict[str, List[float]], Dict[str, List[float]]]:
    """Device time per kernel class of one prefill step and of four decode steps, launch by launch."""
    import torch
    from pulsar_b200 import ops, profiling
    from pulsar_b200.engine.runner import StepEntry
    runner, cache = engine.runner, engine.cache
    saved = (profiling.ENABLED, runner.cuda_graphs)
    profiling.ENABLED, runner.cuda_graphs = True, False
    ops._fns.clear()
    try:
        gen = torch.Generator().manual_seed(5)
        vocab = engine.model.spec.vocab_size
        prompt = torch.randint(0, vocab, (PROMPT,), generator=gen).tolist()
        out = []
        for phase in ("prefill", "decode"):
            for measured in (False, True):           # once unmeasured: buffers reach their size
                if phase == "prefill":
                    profiling.reset()
                    runner.step([StepEntry("p", prompt, [PROMPT - 1])])
                    runner.finish("p")
                else:
                    rids = [("d", i) for i in range(BATCH)]
                    for rid in rids:
                        cache.open(rid)
                        cache.append(rid, CONTEXT - 5)
                    # every request its own random token: requests that all fed the same one would choose the same experts
                    toks = torch.randint(0, vocab, (5, BATCH), generator=gen).tolist()
                    runner.step([StepEntry(rid, [toks[4][b]], [0]) for b, rid in enumerate(rids)])
                    profiling.reset()
                    for i in range(4):
                        runner.step([StepEntry(rid, [toks[i][b]], [0]) for b, rid in enumerate(rids)])
                    if measured:
                        out.append(profiling.totals()[0])
                    for rid in rids:
                        runner.finish(rid)
                    continue
                if measured:
                    out.append(profiling.totals()[0])
        return out[0], out[1]
    finally:
        profiling.ENABLED, runner.cuda_graphs = saved
        ops._fns.clear()
        profiling.reset()


def _pairs(n_new: int, start: int, chunk: int = 0) -> float:
    """(query, visible key) pairs of n_new tokens that follow `start` cached ones."""
    total = 0.0
    for p in (range(start, start + n_new) if n_new < 64 else ()):
        total += p - (p // chunk * chunk if chunk else 0) + 1
    if n_new >= 64:                                   # a whole prompt from position 0
        if chunk:
            full, rest = divmod(n_new, chunk)
            total = full * chunk * (chunk + 1) / 2.0 + rest * (rest + 1) / 2.0
        else:
            total = n_new * (n_new + 1) / 2.0
    return total


def own_work(z: dict, phase: str) -> Dict[str, Tuple[float, float, str]]:
    """Per kernel class of the design: (bytes it must move, flops, what the flops run on) summed over the layers of a step."""
    n = PROMPT if phase == "prefill" else BATCH
    seqs = 1 if phase == "prefill" else BATCH
    ctx = PROMPT if phase == "prefill" else CONTEXT
    start = 0 if phase == "prefill" else CONTEXT - 1
    g, H, G, d, rot, rank, w = z["groups"], z["heads"], z["kv_heads"], z["dim"], z["rot"], z["rank"], z["width"]
    row = rank + rot
    steps = 1 if phase == "prefill" else 4
    lat_pairs = seqs * _pairs(n // seqs, start)
    att_pairs = seqs * _pairs(n // seqs, start, z["chunk"])
    att_ctx = ctx if phase == "prefill" else (CONTEXT - 1) % z["chunk"] + 1
    work = {
        "paged_attention_general": (
            g * (2 * (seqs * ctx * row * 2 + n * H * (row * 4 + rank * 2)) + seqs * att_ctx * G * 2 * d * 2 + n * H * d * 6),
            g * (2 * 2.0 * H * (row + rank) * lat_pairs + 2.0 * H * 2 * d * att_pairs), "fp32 FMA"),
        "heads_linear": (g * 2 * (2 * H * d * rank * 2 + n * H * (d * 2 + rank * 4 + rank * 2 + d * 2 + d * 2)),
                         g * 2 * 2.0 * n * H * d * rank * 2, "fp32 FMA"),
        "latent_prepare": (g * (2 * n * H * (rot * 2 + rot * 4) + n * row * 4), 0.0, ""),
        "qkv_split_write": (g * n * (H + 2 * G) * d * (2 + 4), 0.0, ""),
        "causal_conv_silu": (g * n * z["inner"] * 4, 0.0, ""),
        "selective_scan": (g * (n * (z["inner"] * 8 + (z["dt_rank"] + 2 * z["state"]) * 2) + seqs * z["inner"] * z["state"] * 8
                                + z["inner"] * (z["dt_rank"] * 2 + z["state"] * 4)),
                           g * n * z["inner"] * (2.0 * z["dt_rank"] + 7.0 * z["state"]), "fp32 FMA"),
        "post_norm_add": (g * 7 * n * w * (4 + 4 + 2 + 2), 0.0, ""),
        "clamped_glu": (g * 3 * n * z["ff"] * 6, 0.0, ""),
    }
    work["paged_attention_general_tiled"] = work["paged_attention_general"]          # the same job, by the other kernel
    # a step of whole prompts: latent attention in its expanded form (keys dim + rot wide, values dim wide, a head of its own
    # each) and the chunked attention, on the tensor cores (useful operations; the kernel issues two MMAs for each)
    work["paged_attention_general_tc"] = (g * (2 * n * H * ((d + rot) * (4 + 2) + d * 4) + n * H * d * 6 + n * G * 2 * d * 2),
                                          g * (2 * 2.0 * H * (2 * d + rot) * lat_pairs + 2.0 * H * 2 * d * att_pairs), "bf16 tensor")
    work["selective_scan_prompt"] = (work["selective_scan"][0] + g * n * z["inner"] * 4, g * n * z["inner"] * 7.0 * z["state"], "fp32 FMA")
    work["selective_scan_chunked"] = (work["selective_scan_prompt"][0], g * n * z["inner"] * 16.0 * z["state"], "fp32 FMA")
    work["latent_expand_keys"] = (g * 2 * n * H * (2 * d + rot) * 2, 0.0, "")
    work["sigmoid_gate"] = (g * 2 * n * H * d * 6, 0.0, "")
    return {k: (b * steps, f * steps, on) for k, (b, f, on) in work.items()}


def _window_pairs(n_new: int, start: int, window: int, keep: int) -> float:
    """(query, visible key) pairs of n_new tokens behind `start` cached ones under a window with kept first keys."""
    total = 0.0
    for p in range(start, start + n_new):
        lo = max(0, p - window + 1)
        total += p - lo + 1 + min(keep, lo)
    return total


def topunex_work(z: dict, phase: str) -> Dict[str, Tuple[float, float, str]]:
    """Per kernel class of Topunex: (bytes it must move, flops, what the flops run on) summed over the layers of a step."""
    n = PROMPT if phase == "prefill" else BATCH
    seqs = 1 if phase == "prefill" else BATCH
    start = 0 if phase == "prefill" else CONTEXT - 1
    L, H, G, d, w = z["layers"], z["heads"], z["kv_heads"], z["dim"], z["width"]
    E, top, fe, fs, moe_layers = z["experts"], z["top"], z["expert_ff"], z["shared_ff"], z["layers"] - 1
    steps = 1 if phase == "prefill" else 4
    pairs = seqs * _window_pairs(n // seqs, start, z["window"], z["keep"])
    keys_read = seqs * min(start + n // seqs, z["window"] + z["keep"] + (n // seqs if phase == "prefill" else 0))
    attention = (L * (keys_read * G * 2 * d * 2 + n * H * d * (4 + 2)), L * 4.0 * H * d * pairs)
    chosen = n * top                                     # the per-token kernels read an expert's weights once per token that chose it
    distinct = E * (1.0 - (1.0 - top / E) ** n)          # different experts that n tokens choose, on average: what the grouped products read
    work = {
        "paged_attention_general_tc": (attention[0], attention[1], "bf16 tensor"),
        "paged_attention_general_tiled": (attention[0], attention[1], "fp32 FMA"),
        "paged_attention_general": (attention[0], attention[1], "fp32 FMA"),
        "qk_prepare": (L * n * ((H + G) * d * 4 + H * d * 4 + 2 * G * d * 2), 0.0, ""),
        "sigmoid_gate_strided": (L * n * H * d * (4 + 2 + 2), 0.0, ""),
        "post_norm_add_bias": (2 * L * n * w * (2 + 4 + 4 + 2), 0.0, ""),
        "glu_bias": (n * z["ff"] * (8 + 2), 0.0, ""),
        "moe_route": (moe_layers * (n * w * 2 + E * w * 4), 0.0, ""),
        "moe_grouped": (moe_layers * (distinct * 3 * w * fe * 2 + n * w * 4 + n * top * (fe * 4 + w * 8)),
                        moe_layers * 2.0 * n * top * 3 * w * fe, "bf16 tensor"),
        "moe_gate_up": (moe_layers * (chosen * 2 * fe * w * 2 + n * w * 2), moe_layers * 4.0 * n * top * fe * w, "fp32 FMA"),
        "moe_down": (moe_layers * (chosen * fe * w * 2 + n * w * 4), moe_layers * 2.0 * n * top * fe * w, "fp32 FMA"),
        "clamped_glu": (moe_layers * n * fs * 6, 0.0, ""),
    }
    return {k: (b * steps, f * steps, on) for k, (b, f, on) in work.items()}


def like_work(z: dict, phase: str) -> Dict[str, Tuple[float, float, str]]:
    """The same for the dense model's kernels that do the like jobs."""
    n = PROMPT if phase == "prefill" else BATCH
    layers, H, G, d, w = z["layers"] if "layers" in z else 4 * z["groups"], z["heads"], z["kv_heads"], z["dim"], z["width"]
    steps = 1 if phase == "prefill" else 4
    if phase == "prefill":
        work = {"paged_attention_prefill_tcgen05": (layers * (PROMPT * (2 * H + 2 * G) * d * 2),
                                                    layers * 4.0 * H * d * PROMPT * (PROMPT + 1) / 2.0, "bf16 tensor"),
                "silu_mul": (0.0, 0.0, "")}
    else:
        work = {"paged_attention_decode_tc": (layers * BATCH * CONTEXT * 2 * G * d * 2, 0.0, ""),
                "paged_attention_decode_tc_qkv": (layers * BATCH * CONTEXT * 2 * G * d * 2, 0.0, "")}
    work["add_rmsnorm"] = ((2 * layers + 1) * n * w * (4 + 4 + 2 + 2), 0.0, "")
    work["qk_norm_rope_write"] = (layers * n * (H + 2 * G) * d * 4, 0.0, "")
    return {k: (b * steps, f * steps, on) for k, (b, f, on) in work.items()}


def rooflines(kernels: Dict[str, List[float]], work: Dict[str, Tuple[float, float, str]], pk: dict) -> dict:
    fp32_tflops = 148 * 128 * 2 * 1.965e9 / 1e12            # FMA lanes x 2 x the maximum SM clock: what float32 arithmetic can reach
    out = {}
    for name, (n, ms) in sorted(kernels.items(), key=lambda kv: -kv[1][1]):
        if name not in work or ms <= 0.0:
            continue
        nbytes, flops, on = work[name]
        if nbytes <= 0.0 and flops <= 0.0:
            continue
        t_mem = nbytes / (pk["hbm_gbs"] * 1e9)
        peak = pk["bf16_tflops"] if on == "bf16 tensor" else fp32_tflops
        t_math = flops / (peak * 1e12) if flops else 0.0
        out[name] = {"launches": int(n), "ms": round(ms, 4), "gbytes": round(nbytes / 1e9, 4), "gflop": round(flops / 1e9, 2),
                     "bound": "memory" if t_mem >= t_math else on, "frac_of_roofline": round(max(t_mem, t_math) * 1e3 / ms, 4)}
    return out


# design -> (sizes, its configuration, its kernels' work, the configuration of the model beside it, that model's kernels' work)
DESIGNS = {"bubotar": (SIZES, bubotar_config, own_work, dense_config, like_work),
           "topunex": (TOPUNEX_SIZES, topunex_config, topunex_work, dense_config, like_work),
           "megusun": (MEGUSUN_SIZES, megusun_config, megusun_work, topunex_config, topunex_work),
           "bumotar": (BUMOTAR_SIZES, bumotar_config, bumotar_work, topunex_config, topunex_work)}


def run(args, bench) -> dict:
    """``bench``: the bench module (its timing functions, peaks and clock sampler are used as they are)."""
    import torch
    pk = bench.peaks()
    table, make_config, design_work, beside_config, beside_work = DESIGNS[args.design]
    sizes = [s for s in (args.sizes.split(",") if args.sizes else table) if s]
    line = {"design": args.design, "dtype": "bf16", "data": "synthetic: random weights, random token ids, random cache contents for decode",
            "prompt_tokens": PROMPT, "decode": {"batch": BATCH, "context": CONTEXT}, "peaks": pk, "sizes": {}}
    for size in sizes:
        z = table[size]
        entry = {"shape": z}
        for who, raw in (("design", make_config(z)), ("dense", beside_config(z))):       # "dense": the model beside it (Qwen3 dense, or Topunex for Megusun)
            engine = build(raw)
            p_seconds = bench.time_prefill(engine, PROMPT)
            d_seconds, _, _ = bench.time_decode(engine, BATCH, CONTEXT, args.steps, max(3, args.warmup))
            prefill_k, decode_k = profiled(engine, bench)
            work = design_work if who == "design" else beside_work
            entry[who] = {
                "model": engine.model.spec.architecture, "weights_gb": round(engine.model.weight_bytes(0) / 1e9, 3),
                "prefill_tokens_per_s": round(PROMPT / p_seconds, 1), "prefill_ms": round(p_seconds * 1e3, 3),
                "decode_tokens_per_s": round(BATCH * args.steps / d_seconds, 1), "decode_ms_per_step": round(d_seconds / args.steps * 1e3, 4),
                "decode_hbm_frac": round(bench.decode_bytes(engine, BATCH, CONTEXT - args.steps / 2.0) / (d_seconds / args.steps) / 1e9
                                         / pk["hbm_gbs"], 4),
                "prefill_kernels": rooflines(prefill_k, work(z, "prefill"), pk),
                "decode_kernels": rooflines(decode_k, work(z, "decode"), pk),
                "prefill_ms_by_class": {k: round(v[1], 3) for k, v in sorted(prefill_k.items(), key=lambda kv: -kv[1][1])[:12]},
                "decode_ms_by_class_4_steps": {k: round(v[1], 3) for k, v in sorted(decode_k.items(), key=lambda kv: -kv[1][1])[:12]},
            }
            del engine
            torch.cuda.empty_cache()
        line["sizes"][size] = entry
    return line
