"""Bumotar through the engine against the plain implementation (tests/plain/bumotar_plain.py): configuration and the
oracle's own mechanisms on the CPU; on a GPU each mechanism alone, prompts against token-by-token decoding, portions
down to two tokens, mixed batches with pages and slots used again, sharpened scores that show every window edge, sink and
far key, the retention state across steps and in chunks, the router, long decoding, and greedy generation through the
public entry point."""
import copy
import json
import math
import os
import random
import subprocess
import sys
import types

import pytest
import torch

import helpers
from plain import bumotar_plain as plain

# Error bars relative to the logits' scale.  float32: three times the bar of the other designs' tests.  A retention head's
# output is divided by its root mean square; at a token where q . k all but cancels, the elements of S^T q are small sums of
# large terms, each element with a rounding of its own in the token-by-token form, and the division magnifies that (seen:
# 3.2e-5 at a sequence's first token where the form in chunks, which takes q . k out of the sum, has 3e-6).  A rounding to
# bfloat16 inside the float32 path (4e-3) stays far above the bar.
# bfloat16: two and a half times the other designs' bar.  The opening of a walk is a product whose operand is the stream itself, rounded to
# 16 bits (in the other designs the stream is never rounded), and the first tokens of a sequence pass through retention
# states of one or two terms (seen: 4.3e-2 at a second token; 1e-2 to 2e-2 elsewhere).  A wrong key, state or expert moves
# the logits by tenths.
TOL = {"float32": 6e-5, "bfloat16": 2.5 * helpers.TOL["bfloat16"]}


def latent(heads, dim, rot_dim, vdim, rank, base=100.0, scaling=None, scale=None):
    rot = dict(base=base, dims=rot_dim)
    if scaling is not None:
        rot["scaling"] = scaling
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, rot=rot,
                                                    scale=scale or 1.0 / math.sqrt(dim + rot_dim)))


def left(heads, kv_heads, dim, vdim, window=None, rot=None, softcap=None, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or 1.0 / math.sqrt(dim))
    if window is not None:
        m["mask"] = dict(size=window)
    if rot is not None:
        m["rot"] = rot
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, dim, vdim, decay, rot=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))
    if rot is not None:
        m["rot"] = rot
    return m


def par(l, r, left_scale=0.7, right_scale=1.2):
    return dict(type="parallel", mixer=dict(left=l, right=r, left_scale=left_scale, right_scale=right_scale))


def moe(experts, top, ff, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared is not None:
        m["shared"] = dict(ff=shared)
    return m


def layer(mixer, mlp=None):
    return dict(mixer, mlp=mlp)


def config(layers, vocab, width, eps=1e-5, loop=None, logit_scale=1.0):
    raw = dict(architecture="Bumotar", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale, layers=layers)
    if loop is not None:
        raw["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return raw


RAMP = dict(factor=4.0, original=64, fast=4.0, slow=0.5)
# Every size differs between the configurations and within them: keys, values and rotating parts of different widths, groups
# of one, two and three query heads, one key/value head, windows shorter than a page and longer than the prompt, layers
# without a window, a cap, a rotation or a feed-forward, retention heads whose keys are wider and narrower than their values
# and rotate wholly, partly or not at all, one expert of one, all experts chosen, walks over one, two and all layers, a walk
# that starts at the first layer, a model without walks.
BUMO_A = config([
    layer(par(left(4, 2, 16, 24, window=9, rot=dict(base=1000.0, dims=8, scaling=dict(factor=4.0)), softcap=20.0),
              right(3, 8, 12, [0.9, 0.97, 0.995], rot=dict(base=50.0, dims=4)), 0.55, 0.8), moe(5, 2, 24, shared=40)),
    layer(latent(3, 12, 6, 10, 20, base=100.0, scaling=RAMP), moe(4, 1, 32)),
    layer(par(left(3, 3, 8, 8, window=5, rot=dict(base=300.0, dims=8)), right(2, 12, 8, [0.8, 0.99], rot=dict(base=20.0, dims=12)),
              1.2, 0.5)),
    layer(latent(2, 8, 4, 16, 12, base=30.0), moe(3, 3, 16, shared=8)),
], vocab=180, width=48, eps=1e-5, loop=(1, 3, 3), logit_scale=0.5)
BUMO_B = config([
    layer(latent(5, 8, 8, 12, 24, base=500.0, scaling=dict(factor=2.0, original=32, fast=8.0, slow=1.0)), moe(1, 1, 48, shared=16)),
    layer(par(left(6, 2, 12, 20, rot=dict(base=200.0, dims=4, scaling=dict(factor=2.0))), right(1, 16, 24, [0.95]), 0.3, 1.1),
          moe(7, 3, 16)),
    layer(par(left(2, 1, 32, 16, window=70, softcap=5.0), right(4, 4, 4, [1.0, 0.5, 0.9, 0.99], rot=dict(base=10.0, dims=2)), 1.0, 1.0)),
], vocab=131, width=40, eps=3e-6, loop=(0, 2, 2), logit_scale=2.0)
# head sizes at which the bfloat16 engine's prompt attention runs on the tensor cores; no walk
BUMO_C = config([
    layer(par(left(4, 2, 64, 64, window=40, rot=dict(base=10000.0, dims=32, scaling=dict(factor=6.0)), softcap=40.0),
              right(2, 32, 64, [0.98, 0.999], rot=dict(base=10000.0, dims=32))), moe(6, 2, 32, shared=48)),
    layer(latent(2, 128, 64, 128, 96, base=10000.0, scaling=dict(factor=2.0, original=64, fast=32.0, slow=1.0)), moe(4, 2, 64)),
    layer(par(left(2, 1, 128, 128, window=33, rot=dict(base=5000.0, dims=128)), right(3, 24, 40, [0.9, 0.95, 0.99]))),
], vocab=150, width=64, eps=1e-6)
# no routed layer: the bfloat16 engine is held to the bar at every position (a router's close call ends the comparison
# of the other configurations early); a walk over the first two layers
BUMO_D = config([
    layer(par(left(4, 2, 32, 16, window=11, rot=dict(base=1000.0, dims=16, scaling=dict(factor=2.0)), softcap=30.0),
              right(2, 16, 24, [0.95, 0.99], rot=dict(base=100.0, dims=8)), 0.7, 0.8)),
    layer(latent(4, 16, 8, 24, 32, base=1000.0, scaling=dict(factor=3.0, original=48, fast=6.0, slow=0.5))),
    layer(par(left(2, 2, 64, 64, window=50, rot=dict(base=1000.0, dims=64)), right(3, 32, 16, [0.9, 0.97, 0.999]), 0.5, 1.0)),
], vocab=140, width=56, eps=2e-6, loop=(0, 2, 2), logit_scale=1.5)
ALONE = {
    "latent": config([layer(latent(3, 12, 6, 10, 20, scaling=RAMP))], vocab=64, width=40),
    "latent_plain_rotation": config([layer(latent(2, 8, 8, 8, 8))], vocab=64, width=40, logit_scale=0.25),
    "parallel": config([layer(par(left(4, 2, 16, 24, window=9, rot=dict(base=1000.0, dims=8, scaling=dict(factor=4.0)), softcap=20.0),
                                  right(3, 8, 12, [0.9, 0.97, 0.995], rot=dict(base=50.0, dims=4))))], vocab=64, width=40),
    "parallel_bare": config([layer(par(left(2, 2, 8, 8), right(2, 8, 8, [0.9, 0.99]), 1.0, 1.0))], vocab=64, width=40),
    "moe": config([layer(latent(2, 8, 4, 8, 8), moe(6, 2, 24))], vocab=64, width=40),
    "moe_shared": config([layer(latent(2, 8, 4, 8, 8), moe(4, 3, 16, shared=32))], vocab=64, width=40),
    "walk": config([layer(latent(2, 8, 4, 8, 8))], vocab=64, width=40, loop=(0, 1, 3)),
}
CONFIGS = {"A": (BUMO_A, 31, 8), "B": (BUMO_B, 32, 4), "C": (BUMO_C, 33, 16), "D": (BUMO_D, 34, 8)}      # config, seed, page size


# ------------------------------------------------------------------ configuration (CPU)
def test_config_becomes_parts():
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.models import build_model
    cfg = config_from_dict(copy.deepcopy(BUMO_A))
    spec = cfg.model_spec()
    # layer 0 once, layers 1 and 2 three times, layer 3 once; a parallel layer has two cache entries per run
    assert [(c.block, c.cache, c.members, c.opens) for c in spec.run_order] == [
        (0, 0, (1,), None), (1, 2, (), 0), (2, 3, (4,), None), (1, 5, (), 1), (2, 6, (7,), None), (1, 8, (), 2), (2, 9, (10,), None),
        (3, 11, (), None)]
    assert spec.walk.times == 3 and spec.logit_scale == 0.5
    assert all(b.kind == "prenorm" for b in spec.blocks)
    assert [b.mixer.kind for b in spec.blocks] == ["side_by_side", "latent_attention", "side_by_side", "latent_attention"]
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].feed_forward_norm is None
    (_, l0, ls), (_, r0, rs) = spec.blocks[0].mixer.option("members")
    assert (ls, rs) == (0.55, 0.8)
    assert (l0.kind, l0.window, l0.softcap, l0.fixed_sink, l0.output_gate, l0.qk_norm_eps, l0.qk_norm_weight) == \
        ("attention", 9, 20.0, 0.0, True, 1e-5, True)
    assert (l0.position.rotary_dim, l0.position.divide, l0.position.ramp, l0.position.magnitude) == (8, 4.0, None, 1.0)
    assert (r0.kind, r0.option("decay"), r0.position.rotary_dim, r0.option("key_scale")) == ("retention", (0.9, 0.97, 0.995), 4, 8 ** -0.5)
    m1 = spec.blocks[1].mixer
    assert (m1.option("kv_rank"), m1.option("rot_dim"), m1.option("head_gate"), m1.sinks, m1.head_dim, m1.value_dim) == (20, 6, True, True, 12, 10)
    assert m1.position.ramp == (4.0, 64.0, 4.0, 0.5) and abs(m1.position.magnitude - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert spec.blocks[3].mixer.position.ramp is None and spec.blocks[3].mixer.position.magnitude == 1.0
    ff0 = spec.blocks[0].feed_forward
    assert (ff0.option("experts"), ff0.option("top"), ff0.option("scoring"), ff0.option("renormalize"), ff0.option("renorm_eps")) == \
        (5, 2, "softmax", True, 1e-20)
    assert ff0.option("shared").intermediate == 40 and ff0.option("shared_gate") == "shared.sg"
    assert spec.blocks[1].feed_forward.option("shared") is None
    assert cfg.to_dict() == BUMO_A
    model = build_model(cfg, torch.float32)
    shapes = {w.name: tuple(w.shape) for w in model.weight_specs()}
    assert shapes["loop.in"] == (48, 96) and shapes["loop.step"] == (3, 48)
    assert shapes["l0.mix.left.q"] == (64, 48) and shapes["l0.mix.left.k"] == (32, 48) and shapes["l0.mix.left.v"] == (48, 48)
    assert shapes["l0.mix.left.g"] == (96, 48) and shapes["l0.mix.left.o"] == (48, 96) and shapes["l0.mix.left.q.norm"] == (16,)
    assert shapes["l0.mix.right.q"] == (24, 48) and shapes["l0.mix.right.v"] == (36, 48) and shapes["l0.mix.right.o"] == (48, 36)
    assert shapes["l1.mix.q"] == (3 * 18, 48) and shapes["l1.mix.dkv"] == (26, 48) and shapes["l1.mix.dkv.norm"] == (20,)
    assert shapes["l1.mix.uk"] == (36, 20) and shapes["l1.mix.uv"] == (30, 20) and shapes["l1.mix.g"] == (3, 48)
    assert shapes["l1.mix.sink"] == (3,) and shapes["l1.mix.o"] == (48, 30) and shapes["l0.mlp.shared.sg"] == (1, 48)
    assert not {"l2.norm2", "l2.mlp.router", "l1.mlp.shared.sg", "l0.mix.left.sink"} & set(shapes)
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["paged_kv", "state", "paged_kv", "paged_kv", "state", "paged_kv", "paged_kv", "state",
                                       "paged_kv", "paged_kv", "state", "paged_kv"]
    assert needs[1].state_shape == (3 * 8 * 12,) and needs[1].state_dtype == torch.float32 and needs[0].window == 9
    assert [(t.name, t.heads, t.width) for t in needs[0].tensors] == [("k", 2, 16), ("v", 2, 24)]
    assert [(t.name, t.heads, t.width) for t in needs[2].tensors] == [("latent", 1, 26)]
    no_walk = config_from_dict(copy.deepcopy(BUMO_C)).model_spec()
    assert no_walk.walk is None and all(c.opens is None for c in no_walk.run_order)
    assert "loop.in" not in {w.name for w in build_model(config_from_dict(copy.deepcopy(BUMO_C)), torch.float32).weight_specs()}


@pytest.mark.parametrize("edit,match", [
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0].update(type="mamba1"), "latent_attention"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors(edit, match):
    from pulsar_b200.config import ConfigError, config_from_dict
    raw = copy.deepcopy(BUMO_A)
    edit(raw)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_rotary_frequencies_of_the_engine_and_of_the_plain_model_agree():
    from pulsar_b200.config.specs import PositionSpec
    from pulsar_b200.parts.rope import RotaryEmbedding
    for rot in (dict(base=100.0, dims=6, scaling=RAMP), dict(base=40000.0, dims=24, scaling=dict(factor=3.0, original=512, fast=16.0, slow=2.0)),
                dict(base=1000.0, dims=8, scaling=dict(factor=4.0)), dict(base=50.0, dims=4), dict(base=7.0, dims=10, scaling=dict(
                    factor=3.0, original=9, fast=0.01, slow=0.001))):
        freqs, magnitude = plain.frequencies_of(rot)
        s = rot.get("scaling") or {}
        ramp = (s["factor"], float(s["original"]), s["fast"], s["slow"]) if "original" in s else None
        enc = RotaryEmbedding(PositionSpec("rope", rot["dims"], rot["dims"], rot["base"], divide=s.get("factor") if ramp is None else None,
                                           ramp=ramp))
        assert [enc.frequency(j) for j in range(rot["dims"] // 2)] == pytest.approx(freqs, rel=1e-15)
        assert magnitude == (1.0 if ramp is None else 0.1 * math.log(s["factor"]) + 1.0)
    # the ramp of RAMP over three pairs: kept, half way, divided
    freqs, _ = plain.frequencies_of(dict(base=100.0, dims=6, scaling=RAMP))
    base = plain.base_frequencies(100.0, 6)
    assert freqs == pytest.approx([base[0], 0.5 * base[1] + 0.5 * base[1] / 4.0, base[2] / 4.0], rel=1e-15)


def test_plain_mechanisms_agree_with_loops_over_single_numbers():
    """The oracle's vectorised forms against the equations written out one token and one pair at a time."""
    g = torch.Generator().manual_seed(3)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=torch.float64)
    L, W = 9, 10
    h = rnd(L, W)
    pos = torch.arange(L)
    # the two layouts of a rotation
    x = rnd(L, 2, 8)
    freqs = [0.7, 0.2, 0.05]
    halves, pairs = plain.rotate_halves(x, pos, freqs, 1.3), plain.rotate_neighbours(x, pos, freqs, 1.3)
    for t in (0, 4, 8):
        for i, f in enumerate(freqs):
            c, s = 1.3 * math.cos(t * f), 1.3 * math.sin(t * f)
            u, v = float(x[t, 1, i]), float(x[t, 1, i + 3])
            assert abs(float(halves[t, 1, i]) - (u * c - v * s)) < 1e-12 and abs(float(halves[t, 1, i + 3]) - (v * c + u * s)) < 1e-12
            u, v = float(x[t, 1, 2 * i]), float(x[t, 1, 2 * i + 1])
            assert abs(float(pairs[t, 1, 2 * i]) - (u * c - v * s)) < 1e-12 and abs(float(pairs[t, 1, 2 * i + 1]) - (v * c + u * s)) < 1e-12
        assert torch.equal(halves[t, :, 6:], x[t, :, 6:]) and torch.equal(pairs[t, :, 6:], x[t, :, 6:])
    # window attention, one query at a time
    m = left(4, 2, 6, 5, window=4, rot=dict(base=10.0, dims=4, scaling=dict(factor=2.0)), softcap=3.0, scale=0.4)
    w = {"q": rnd(24, W), "k": rnd(12, W), "v": rnd(10, W), "g": rnd(20, W), "o": rnd(W, 20), "q.norm": rnd(6), "k.norm": rnd(6)}
    out = plain.window_attention(h, w, m, 1e-6)
    fr = [10.0 ** (-2.0 * i / 4) / 2.0 for i in range(2)]
    unit = lambda v, wt: v / math.sqrt(float((v * v).mean()) + 1e-6) * wt

    def turned(v, t):
        v = v.clone()
        for i, f in enumerate(fr):
            a, b = float(v[i]), float(v[i + 2])
            v[i], v[i + 2] = a * math.cos(t * f) - b * math.sin(t * f), b * math.cos(t * f) + a * math.sin(t * f)
        return v
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    for i in (0, 3, 8):
        heads = []
        for head in range(4):
            kv = head // 2
            qi = turned(unit(q[i, head * 6:(head + 1) * 6], w["q.norm"]), i)
            js = [j for j in range(L) if 0 <= i - j < 4]
            sc = [3.0 * math.tanh(float(qi @ turned(unit(k[j, kv * 6:(kv + 1) * 6], w["k.norm"]), j)) * 0.4 / 3.0) for j in js]
            den = 1.0 + sum(math.exp(s) for s in sc)
            heads.append(sum(math.exp(s) / den * v[j, kv * 5:(kv + 1) * 5] for s, j in zip(sc, js)))
        gate = torch.sigmoid(w["g"] @ h[i])
        assert float(((torch.cat(heads) * gate) @ w["o"].T - out[i]).abs().max()) < 1e-10
    # retention, one head at a time; two halves with a carried state equal the whole
    m = right(2, 4, 3, [0.9, 0.5], rot=dict(base=5.0, dims=2))
    w = {"q": rnd(8, W), "k": rnd(8, W), "v": rnd(6, W), "g": rnd(6, W), "o": torch.eye(6, dtype=torch.float64)}
    out = plain.retention(h, w, m, 1e-6)
    q, k, v, gt = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T, h @ w["g"].T

    def turn2(vec, t):
        vec = vec.clone()
        a, b = float(vec[0]), float(vec[1])
        vec[0], vec[1] = a * math.cos(t) - b * math.sin(t), b * math.cos(t) + a * math.sin(t)
        return vec
    for head, dec in enumerate([0.9, 0.5]):
        S = torch.zeros(4, 3, dtype=torch.float64)
        for t in range(L):
            kt = turn2(k[t, head * 4:(head + 1) * 4], t) * 0.5
            S = dec * S + torch.outer(kt, v[t, head * 3:(head + 1) * 3])
            o = S.T @ turn2(q[t, head * 4:(head + 1) * 4], t)
            o = o / math.sqrt(float((o * o).mean()) + 1e-6)
            gg = gt[t, head * 3:(head + 1) * 3]
            assert float((o * gg * torch.sigmoid(gg) - out[t, head * 3:(head + 1) * 3]).abs().max()) < 1e-10
    # latent attention, one query at a time
    m = latent(2, 3, 4, 5, 6, base=10.0, scaling=dict(factor=2.0, original=8, fast=2.0, slow=0.1), scale=0.3)["mixer"]
    w = {"q": rnd(14, W), "dkv": rnd(10, W), "dkv.norm": rnd(6), "uk": rnd(6, 6), "uv": rnd(10, 6), "sink": rnd(2), "g": rnd(2, W),
         "o": rnd(W, 10)}
    out = plain.latent_attention(h, w, m, 1e-6)
    fr, mag = plain.frequencies_of(m["rot"])

    def turn_pairs(vec, t):
        vec = vec.clone()
        for i, f in enumerate(fr):
            a, b = float(vec[2 * i]), float(vec[2 * i + 1])
            vec[2 * i], vec[2 * i + 1] = mag * (a * math.cos(t * f) - b * math.sin(t * f)), mag * (b * math.cos(t * f) + a * math.sin(t * f))
        return vec
    down = h @ w["dkv"].T
    c = torch.stack([unit(down[t, :6], w["dkv.norm"]) for t in range(L)])
    for i in (0, 5, 8):
        heads = []
        for head in range(2):
            qh = (w["q"] @ h[i])[head * 7:(head + 1) * 7]
            sc = []
            for j in range(i + 1):
                kp = (w["uk"] @ c[j])[head * 3:(head + 1) * 3]
                sc.append((float(qh[:3] @ kp) + float(turn_pairs(qh[3:], i) @ turn_pairs(down[j, 6:], j))) * 0.3)
            den = math.exp(float(w["sink"][head])) + sum(math.exp(s) for s in sc)
            o = sum(math.exp(s) / den * (w["uv"] @ c[j])[head * 5:(head + 1) * 5] for j, s in enumerate(sc))
            heads.append(o * torch.sigmoid(w["g"][head] @ h[i]))
        assert float((torch.cat(heads) @ w["o"].T - out[i]).abs().max()) < 1e-10
    # the mixture: softmax over all experts, the chosen scores divided by their sum
    mlp = dict(router=dict(experts=4, top=2), shared=dict(ff=4))
    wm = {"router": rnd(4, W), "shared.sg": rnd(1, W), "shared.gate": rnd(4, W), "shared.up": rnd(4, W), "shared.down": rnd(W, 4)}
    for e in range(4):
        wm.update({f"e{e}.gate": rnd(5, W), f"e{e}.up": rnd(5, W), f"e{e}.down": rnd(W, 5)})
    out = plain.moe_ff(h, wm, mlp)
    silu = lambda x: x / (1 + torch.exp(-x))
    for t in range(L):
        z = [float(wm["router"][e] @ h[t]) for e in range(4)]
        s = [math.exp(v) / sum(math.exp(u) for u in z) for v in z]
        chosen = sorted(range(4), key=lambda e: -s[e])[:2]
        want = torch.zeros(W, dtype=torch.float64)
        for e in chosen:
            want += s[e] / (s[chosen[0]] + s[chosen[1]] + 1e-20) * (wm[f"e{e}.down"] @ (silu(wm[f"e{e}.gate"] @ h[t]) * (wm[f"e{e}.up"] @ h[t])))
        gate = 1 / (1 + math.exp(-float(wm["shared.sg"][0] @ h[t])))
        want += gate * (wm["shared.down"] @ (silu(wm["shared.gate"] @ h[t]) * (wm["shared.up"] @ h[t])))
        assert float((want - out[t]).abs().max()) < 1e-10
    # the order of the layers and the opening of a walk
    assert plain.walk_order(dict(layers=[0] * 5, loop=dict(start=1, stop=3, times=2))) == [
        (0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (3, None, False), (4, None, False)]
    x, x0, w_in, row = rnd(L, W), rnd(L, W), rnd(W, 2 * W), rnd(W)
    opened = plain.open_walk(x, x0, w_in, row)
    assert float((opened[2] - (w_in[:, :W] @ x[2] + w_in[:, W:] @ x0[2] + row)).abs().max()) < 1e-12


def test_a_random_folder_and_the_plain_model(tmp_path):
    helpers.make_folder(tmp_path, copy.deepcopy(BUMO_B), 7, store_dtype=torch.bfloat16)
    cfg, w = helpers.read_folder(str(tmp_path))
    assert w["loop.in"].shape == (40, 80) and w["loop.step"].shape == (2, 40) and w["l0.mix.sink"].shape == (5,)
    streams = []
    logits = plain.forward(cfg, w, [3, 1, 4, 1, 5, 9, 2, 6], torch.float64, streams=streams)
    assert logits.shape == (8, 131) and bool(torch.isfinite(logits).all()) and len(streams) == 5      # 2 x 2 layers, then one


# ------------------------------------------------------------------ GPU
gpu = pytest.mark.gpu


def _sharpen(folder):
    """Rewrite a folder so that scores are sharp and sinks weigh: every softmax then rests on one or two keys, and a key that
    is wrongly seen or not seen, or a sink left out, moves the logits by much more than rounding."""
    from pulsar_b200.weights import safetensors_io
    cfg, w = helpers.read_folder(folder)
    for name in list(w):
        if name.endswith("mix.q") or name.endswith("mix.left.q"):
            w[name] = (w[name].float() * 6.0).to(w[name].dtype)
        if name.endswith("mix.sink"):
            w[name] = (w[name].float() * 0.0 + 2.0).to(w[name].dtype)
    safetensors_io.write_safetensors(os.path.join(folder, "model.safetensors"), list(w.items()), metadata={"format": "pt"})


EDGES = config([
    layer(par(left(4, 2, 16, 16, window=7, rot=dict(base=1000.0, dims=8, scaling=dict(factor=4.0)), softcap=200.0),
              right(2, 8, 8, [0.9, 0.99], rot=dict(base=50.0, dims=4)), 1.0, 0.3)),
    layer(latent(3, 12, 6, 10, 20, scaling=RAMP)),
    layer(par(left(2, 1, 8, 24, window=16, rot=dict(base=300.0, dims=8)), right(2, 8, 8, [0.5, 0.95]), 1.0, 0.3)),
], vocab=96, width=40, loop=(0, 2, 2))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, raw in list(ALONE.items()) + [(n, c[0]) for n, c in CONFIGS.items()] + [("edges", EDGES)]:
        d = tmp_path_factory.mktemp(f"bumo{name}")
        # bfloat16 values: both precisions hold them exactly.  Wider weights than the default make every sublayer count.
        helpers.make_folder(d, copy.deepcopy(raw), 700 + len(out), store_dtype=torch.bfloat16, std=0.15)
        out[name] = str(d)
    _sharpen(out["edges"])
    return out


CLOSE_CALL = 0.03       # relative margin of a router's choice below which bfloat16 rounding may choose otherwise
CANCELLED = 0.2         # what cancellation leaves of a retention head's output, below which its unit norm magnifies rounding
WIPED_OUT = 0.02        # ... below which the token's stream is off by so much that the tokens behind it, which attend to it, are too


class _Reference(dict):
    """request -> plain logits; ``sure[request]``: the positions before the request's first close call of a router.  A token
    that is routed otherwise moves its own logits and, through its keys and states, those of the tokens behind it, so the
    bfloat16 engine is held to the bar up to there only (the float32 engine everywhere).  ``shaky[request]``: the positions
    at which a retention head's output all but cancels before it is divided by its size (mostly a sequence's first
    tokens, whose state holds one or two terms); the bfloat16 engine is not held to the bar at those."""
    sure = None
    shaky = None


def _reference(folder, requests):
    cfg, w = helpers.read_folder(folder)
    ref = _Reference()
    ref.sure, ref.shaky = {}, {}
    for rid, toks in requests.items():
        margins, cancellations = [], []
        ref[rid] = plain.forward(cfg, w, list(toks), torch.float64, margins=margins, cancellations=cancellations)
        close = [int(torch.nonzero(m < CLOSE_CALL)[0]) for m in margins if bool((m < CLOSE_CALL).any())]
        close += [int(torch.nonzero(c < WIPED_OUT)[0]) for c in cancellations if bool((c < WIPED_OUT).any())]
        ref.sure[rid] = min(close) if close else len(toks)
        ref.shaky[rid] = {int(t) for c in cancellations for t in torch.nonzero(c < CANCELLED).flatten()}
    return ref


def _replay(folder, dtype, trace, max_tokens, page_size, max_running=4):
    from pulsar_b200.replay import Replay
    rp = Replay(folder, dtype, max_tokens, page_size=page_size, max_running=max_running)
    got = {}
    for rec, rows in zip(trace.records, trace.rows):
        logits = rp.run_step(rec)
        for i, key in enumerate(rows):
            got[key] = logits[i]
    rp.cache.check_consistency()
    assert rp.cache.live_requests() == []
    assert all(f == g.allocator.n for f, g in zip(rp.cache.n_free_pages(), rp.cache.groups))
    return got, rp


def _compare(got, ref, dtype, what, tol=None):
    assert got
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        if dtype == "bfloat16" and (pos >= ref.sure[rid] or pos in ref.shaky[rid]):
            continue
        err = helpers.rel_err(row, ref[rid][pos])
        worst = max(worst, err)
        assert err < (tol or TOL[dtype]), f"{what}: request {rid} position {pos}: error {err:.3e} (first wrong place)"
    helpers.report(what, worst, dtype)


def _round64(n):
    return -(-n // 64) * 64


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(folders, name, dtype):
    rng = random.Random(5)
    toks = helpers.random_tokens(rng, 45, 64)
    ref = _reference(folders[name], {"a": toks})
    got, _ = _replay(folders[name], dtype, helpers.trace_whole(toks), 64, 8)
    _compare(got, ref, dtype, f"alone[{name}] whole")
    got, _ = _replay(folders[name], dtype, helpers.trace_portions(toks, [5, 2, 11, 3, 2]), 64, 4)
    _compare(got, ref, dtype, f"alone[{name}] portions")
    got, _ = _replay(folders[name], dtype, helpers.trace_tail(toks, 20), 64, 4)
    _compare(got, ref, dtype, f"alone[{name}] tail")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_tail_and_portions_agree_with_the_plain_logits(folders, name, dtype):
    raw, seed, page = CONFIGS[name]
    rng = random.Random(seed)
    toks = helpers.random_tokens(rng, 93, raw["vocab"])
    ref = _reference(folders[name], {"a": toks})
    for what, trace in (("whole", helpers.trace_whole(toks)), ("tail", helpers.trace_tail(toks, 60)),
                        ("portions", helpers.trace_portions(toks, [7, 2, 13, 2, 5, 17, 3])),
                        ("large portions", helpers.trace_portions(toks, [40, 18, 35])),
                        ("pairs", helpers.trace_portions(toks[:47], [2]))):
        got, _ = _replay(folders[name], dtype, trace, _round64(len(toks)), page)
        _compare(got, ref, dtype, f"{name} {what}")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, dtype):
    raw, seed, page = CONFIGS[name]
    rng = random.Random(seed + 30)
    lengths = [40, 23, 64, 9, 31, 50, 17, 28, 45, 1, 2]
    requests = {f"r{i}": helpers.random_tokens(rng, n, raw["vocab"]) for i, n in enumerate(lengths)}
    ref = _reference(folders[name], requests)
    trace = helpers.trace_mixed(requests, rng, max_live=3)
    budget = sum(sorted(_round64(n) for n in lengths)[-3:])
    got, rp = _replay(folders[name], dtype, trace, budget, page, max_running=3)      # 11 requests through 3 slots
    assert len(got) == sum(lengths)
    _compare(got, ref, dtype, f"{name} mixed")


@gpu
def test_a_batch_of_unequal_requests_equals_each_alone(folders):
    raw, seed, page = CONFIGS["A"]
    rng = random.Random(77)
    requests = {f"q{i}": helpers.random_tokens(rng, n, raw["vocab"]) for i, n in enumerate([37, 5, 22])}
    together = helpers.Trace()
    together.step([(rid, toks[:-4], range(len(toks) - 4)) for rid, toks in requests.items()])
    for k in range(4, 0, -1):
        together.step([(rid, toks[len(toks) - k:len(toks) - k + 1], [0]) for rid, toks in requests.items()],
                      end=list(requests) if k == 1 else [])
    both, _ = _replay(folders["A"], "float32", together, 3 * 64, page)
    for rid, toks in requests.items():
        alone, _ = _replay(folders["A"], "float32", helpers.trace_tail(toks, 4, rid), 64, page)
        for key, row in alone.items():
            assert helpers.rel_err(both[key], row) < 2e-6, f"{key}: a batch changed the logits"


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_long_portions(folders, dtype):
    """230 tokens of which 220 are decoded one by one (from a captured graph; every window passes over decoded tokens), and
    the same prompt in portions long enough for the retention's form that runs in chunks (with ragged last chunks)."""
    for name in ("A", "D"):
        raw, seed, page = CONFIGS[name]
        rng = random.Random(9)
        toks = helpers.random_tokens(rng, 230, raw["vocab"])
        ref = _reference(folders[name], {"a": toks})
        got, rp = _replay(folders[name], dtype, helpers.trace_tail(toks, 220), _round64(len(toks)), page)
        _compare(got, ref, dtype, f"{name} long decoding")
        assert rp.runner.graph_replays > 150          # the steps of single tokens ran from a captured graph
        got, _ = _replay(folders[name], dtype, helpers.trace_portions(toks, [101, 66, 63]), _round64(len(toks)), page)
        _compare(got, ref, dtype, f"{name} long portions")


def test_sharpened_scores_make_every_edge_count():
    """The test below has teeth: with the sharpened weights a window that is one key too long or too short, a sink that
    is left out, a one that is not added, or a far key that is lost moves the plain logits by far more than the bar."""
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        helpers.make_folder(d, copy.deepcopy(EDGES), 713, store_dtype=torch.bfloat16, std=0.15)
        _sharpen(d)
        cfg, w = helpers.read_folder(d)
    rng = random.Random(11)
    toks = helpers.random_tokens(rng, 60, 96)
    ref = plain.forward(cfg, w, toks, torch.float64)
    for edit in (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=8),
                 lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=6),
                 lambda c: c["layers"][2]["mixer"]["left"]["mask"].update(size=17)):
        other = copy.deepcopy(cfg)
        edit(other)
        assert helpers.rel_err(plain.forward(other, w, toks, torch.float64), ref) > 100 * TOL["float32"]
    no_sink = dict(w)
    no_sink["l1.mix.sink"] = w["l1.mix.sink"] - 30.0
    assert helpers.rel_err(plain.forward(cfg, no_sink, toks, torch.float64), ref) > 100 * TOL["float32"]


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_scores_at_window_edges_page_borders_and_far_back(folders, dtype):
    """Sharpened scores: a softmax rests on one or two keys.  Windows of 7 and 16 over pages of 4: their edges fall inside
    pages, on page borders, into the first tokens and into decoded tokens; the latent layers see every key, far ones too."""
    rng = random.Random(11)
    toks = helpers.random_tokens(rng, 330, 96)
    ref = _reference(folders["edges"], {"a": toks})
    tol = TOL[dtype] * (1.5 if dtype == "bfloat16" else 1)       # sharp scores magnify the rounding of queries and keys
    for what, trace, page in (("whole", helpers.trace_whole(toks), 4), ("tail", helpers.trace_tail(toks, 40), 4),
                              ("portions", helpers.trace_portions(toks, [3, 2, 5, 9, 2, 31, 4]), 4),
                              ("tail, pages of 16", helpers.trace_tail(toks[:100], 70), 16)):
        got, _ = _replay(folders["edges"], dtype, trace, _round64(len(toks)), page)
        _compare(got, ref, dtype, f"edges {what}", tol)


def _step_context(q_lens, kv_lens, slots=None):
    """What the kernels' wrappers read of a step: its device arrays, the lengths on the host, scratch memory."""
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return types.SimpleNamespace(cu_q=i32(cu), kv_len=i32(kv_lens), n_seqs=len(q_lens), n_tokens=cu[-1], max_q_len=max(q_lens),
                                 host=types.SimpleNamespace(q_lens=list(q_lens)),
                                 seq_of_token=i32([s for s, n in enumerate(q_lens) for _ in range(n)]),
                                 state_slots=i32(list(range(len(q_lens))) if slots is None else slots),
                                 scratch=lambda tag, shape, dtype=None: torch.empty(shape, dtype=dtype, device="cuda"))


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(2, 8, 8, 8), (3, 12, 20, 4), (1, 33, 7, 0), (4, 64, 64, 64), (2, 128, 128, 32), (5, 6, 50, 6)])
@pytest.mark.parametrize("q_lens", [[1, 1, 1], [7, 1, 30], [150, 2, 65, 33], [32], [97]])
def test_retention_against_its_formula(q_lens, sizes, dtype):
    """Both forms of the kernel (token by token; in chunks) from states that are not zero, in slots out of order: outputs
    and the states left behind."""
    from pulsar_b200 import ops
    H, D, V, rotary = sizes
    g = torch.Generator().manual_seed(sum(q_lens) + D)
    n = sum(q_lens)
    rows = torch.randn(n, 2 * H * (D + V) + 3, generator=g)
    cos_sin = torch.rand(n, max(rotary // 2, 1), generator=g) * 6.28
    cos, sin = torch.cos(cos_sin), torch.sin(cos_sin)
    decay = torch.tensor([0.999, 0.9, 0.5, 1.0, 0.97][:H])
    slots = list(range(len(q_lens) + 2))
    random.Random(n).shuffle(slots)
    slots = slots[:len(q_lens)]
    state0 = 0.3 * torch.randn(len(q_lens) + 2, H * D * V + 5, generator=g)
    k_scale, eps = D ** -0.5, 1e-5
    # the formula, token by token, in float64
    r64, half = rows.double(), rotary // 2
    want = torch.zeros(n, H * V, dtype=torch.float64)
    state_want = state0.double().clone()
    at = 0
    for s, ql in enumerate(q_lens):
        S = state_want[slots[s], :H * D * V].view(H, D, V).clone()
        for t in range(at, at + ql):
            for hd in range(H):
                q, k = r64[t, hd * D:(hd + 1) * D].clone(), r64[t, (H + hd) * D:(H + hd + 1) * D].clone()
                for vec in (q, k):
                    u, v = vec[:half].clone(), vec[half:rotary].clone()
                    vec[:half] = u * cos[t, :half].double() - v * sin[t, :half].double()
                    vec[half:rotary] = v * cos[t, :half].double() + u * sin[t, :half].double()
                k = k * k_scale
                vv = r64[t, 2 * H * D + hd * V:2 * H * D + (hd + 1) * V]
                S[hd] = float(decay[hd]) * S[hd] + torch.outer(k, vv)
                o = S[hd].T @ q
                gg = r64[t, 2 * H * D + H * V + hd * V:2 * H * D + H * V + (hd + 1) * V]
                want[t, hd * V:(hd + 1) * V] = o / torch.sqrt((o * o).mean() + eps) * gg * torch.sigmoid(gg)
        state_want[slots[s], :H * D * V] = S.reshape(-1)
        at += ql
    ctx = _step_context(q_lens, q_lens, slots)
    for chunked in (False, True):
        state = state0.clone().cuda()
        y = torch.empty(n, H * V, dtype=dtype, device="cuda")
        ops.retention(ctx, rows.cuda(), cos.cuda() if rotary else None, sin.cuda() if rotary else None, decay.cuda(), state, y, H, D, V,
                      rotary, k_scale, eps, chunked=chunked)
        err = helpers.rel_err(y.float().cpu(), want)
        assert err < (3e-5 if dtype == torch.float32 else 6e-3), f"retention chunked={chunked}: {err:.3e}"
        assert helpers.rel_err(state.cpu(), state_want) < 3e-5, f"retention chunked={chunked}: the kept state"
        assert torch.equal(state.cpu()[:, H * D * V:], state0[:, H * D * V:])          # nothing behind the mixer's part is touched


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels_against_their_formulas(dtype):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(4)
    tol = 1e-6 if dtype == torch.float32 else 6e-3
    # weighted per-head norm before the rotation, value heads behind the key heads
    n, Hq, Hkv, D, Dv, rotary, page = 11, 4, 2, 12, 20, 8, 4
    rows = torch.randn(n, (Hq + Hkv) * D + Hkv * Dv + 5, generator=g)
    qw, kw = torch.randn(D, generator=g), torch.randn(D, generator=g)
    ang = torch.rand(n, rotary // 2, generator=g) * 6.28
    cos, sin = torch.cos(ang), torch.sin(ang)
    slots = torch.randperm(4 * page, generator=g)[:n].to(torch.int32)
    q_out = torch.empty(n, Hq, D, device="cuda")
    k_pool = torch.zeros(4, Hkv, page, D, dtype=dtype, device="cuda")
    v_pool = torch.zeros(4, Hkv, page, Dv, dtype=dtype, device="cuda")
    ops.qk_prepare(rows.cuda(), q_out, k_pool, v_pool, slots.cuda(), cos.cuda(), sin.cuda(), Hq, Hkv, D, rotary, page,
                   q_norm=qw.cuda(), k_norm=kw.cuda(), norm_eps=1e-5, n_value_heads=Hkv, value_dim=Dv)

    def prepared(x, wt):
        x = x.double()
        x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * wt.double()
        u, v = x[..., :rotary // 2].clone(), x[..., rotary // 2:rotary].clone()
        c, s = cos.double()[:, None, :], sin.double()[:, None, :]
        x[..., :rotary // 2], x[..., rotary // 2:rotary] = u * c - v * s, v * c + u * s
        return x
    assert helpers.rel_err(q_out.cpu(), prepared(rows[:, :Hq * D].view(n, Hq, D), qw)) < 1e-6
    k_want = prepared(rows[:, Hq * D:(Hq + Hkv) * D].view(n, Hkv, D), kw)
    v_want = rows[:, (Hq + Hkv) * D:(Hq + Hkv) * D + Hkv * Dv].view(n, Hkv, Dv)
    for t in range(n):
        p, o = int(slots[t]) // page, int(slots[t]) % page
        assert helpers.rel_err(k_pool[p, :, o].float().cpu(), k_want[t]) < tol
        assert helpers.rel_err(v_pool[p, :, o].float().cpu(), v_want[t]) < tol
    # a gate per head, from a column slice
    x = torch.randn(7, 3 * 10, generator=g).to(dtype)
    gate = torch.randn(7, 9, generator=g)
    xd = x.clone().cuda()
    ops.sigmoid_gate_strided(xd, gate.cuda()[:, 4:7], group=10)
    want = x.double().view(7, 3, 10) * torch.sigmoid(gate[:, 4:7].double())[:, :, None]
    assert helpers.rel_err(xd.float().cpu().view(7, 3, 10), want) < tol
    # two outputs joined with a weight each; two streams side by side
    a, b = torch.randn(5, 24, generator=g).to(dtype), torch.randn(5, 24, generator=g).to(dtype)
    out = torch.empty(5, 24, dtype=dtype, device="cuda")
    ops.scaled_sum(a.cuda(), b.cuda(), out, 0.6, -1.3)
    assert helpers.rel_err(out.float().cpu(), 0.6 * a.double() - 1.3 * b.double()) < tol
    res, origin, delta = torch.randn(5, 24, generator=g), torch.randn(5, 24, generator=g), torch.randn(5, 24, generator=g).to(dtype)
    both = torch.empty(5, 48, dtype=dtype, device="cuda")
    ops.concat_streams(res.cuda(), delta.cuda(), origin.cuda(), both)
    assert helpers.rel_err(both.float().cpu(), torch.cat([res.double() + delta.double(), origin.double()], dim=1)) < tol
    ops.concat_streams(res.cuda(), None, origin.cuda(), both)
    assert helpers.rel_err(both.float().cpu(), torch.cat([res.double(), origin.double()], dim=1)) < tol
    # cosines and sines with a magnitude
    pos = torch.tensor([0, 1, 17, 4000], dtype=torch.int32)
    quad = torch.tensor([0.3, 0.01], dtype=torch.float64) * (2.0 / math.pi)
    c, s = torch.empty(4, 2, device="cuda"), torch.empty(4, 2, device="cuda")
    ops.rope_table(pos.cuda(), quad.cuda(), c, s, 1.25)
    angle = pos.double()[:, None] * torch.tensor([0.3, 0.01], dtype=torch.float64)[None, :]
    assert float((c.cpu() - 1.25 * torch.cos(angle)).abs().max()) < 1e-6 and float((s.cpu() - 1.25 * torch.sin(angle)).abs().max()) < 1e-6


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(1, 40, 6, 2), (3, 48, 16, 4), (40, 72, 5, 5), (300, 64, 33, 1)])
def test_router_with_softmax_scores(sizes, dtype):
    from pulsar_b200 import ops
    n, W, E, top = sizes
    g = torch.Generator().manual_seed(n)
    h = torch.randn(n, W, generator=g).to(dtype)
    router = torch.randn(E + 1, W, generator=g)
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(n, top, device="cuda")
    extra = torch.empty(n, 1, device="cuda")
    ops.moe_route(h.cuda(), router.cuda(), ids, wts, 1.0, True, extra, softmax=True, renorm_eps=1e-20)
    z = h.double() @ router.double().T
    s = torch.softmax(z[:, :E], dim=-1)
    val, idx = torch.topk(s, top, dim=-1)
    assert torch.equal(ids.cpu().long(), idx)
    assert helpers.rel_err(wts.cpu(), val / (val.sum(-1, keepdim=True) + 1e-20)) < 1e-5
    assert helpers.rel_err(extra.cpu(), torch.sigmoid(z[:, E:])) < 1e-5
    assert float((wts.sum(-1).cpu() - 1.0).abs().max()) < 1e-5


@gpu
def test_greedy_generation_through_the_engine(folders):
    from pulsar_b200.api import generate
    raw, seed, page = CONFIGS["A"]
    cfg, w = helpers.read_folder(folders["A"])
    rng = random.Random(41)
    prompts = [helpers.random_tokens(rng, n, raw["vocab"]) for n in (19, 4, 33)]

    def greedy(prompt, n_new):
        seq = list(prompt)
        for _ in range(n_new):
            seq.append(int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax()))
        return seq[len(prompt):]
    got = generate(folders["A"], prompts, 12, dtype="float32", page_size=page, num_pages=40, max_sessions=4, max_running=2,
                   max_chunk_size=7, device="cuda:0")
    assert got == [greedy(p, 12) for p in prompts]
    # bfloat16 on the configuration without routers: every token lies within the bar of the plain model's best one
    raw, seed, page = CONFIGS["D"]
    cfg, w = helpers.read_folder(folders["D"])
    prompts = [helpers.random_tokens(rng, n, raw["vocab"]) for n in (19, 4, 33)]
    got16 = generate(folders["D"], prompts, 5, dtype="bfloat16", page_size=page, num_pages=40, max_sessions=4, max_running=3,
                     max_chunk_size=16, device="cuda:0")
    checked = 0
    for p, new in zip(prompts, got16):
        seq = list(p)
        for tok in new:
            cancellations = []
            row = plain.forward(cfg, w, seq, torch.float64, cancellations=cancellations)[-1]
            # (not where rounding is magnified beyond the bar: at this token, or at one of the few before it that it attends to)
            if all(float(c[-3:].min()) >= WIPED_OUT for c in cancellations):
                assert float(row.max() - row[tok]) <= TOL["bfloat16"] * float(row.abs().max())
                checked += 1
            seq.append(tok)
    assert checked >= 3


@gpu
def test_a_preempted_request_is_recomputed_from_fresh_states(folders):
    """More requests than pages: the scheduler preempts and recomputes; the retention states start again at zero, so the
    tokens are those of undisturbed runs."""
    from pulsar_b200.api import generate
    raw, seed, page = CONFIGS["B"]
    rng = random.Random(43)
    prompts = [helpers.random_tokens(rng, n, raw["vocab"]) for n in (21, 30, 26, 17)]
    calm = generate(folders["B"], prompts, 20, dtype="float32", page_size=page, num_pages=200, max_sessions=4, max_running=4,
                    max_chunk_size=16, device="cuda:0")
    tight = generate(folders["B"], prompts, 20, dtype="float32", page_size=page, num_pages=36, max_sessions=4, max_running=4,
                     max_chunk_size=16, device="cuda:0")
    assert tight == calm


@gpu
def test_command_line_and_trace_program(folders, tmp_path):
    """The framework's two programs on a Bumotar folder: greedy tokens from bin/pulsar-generate, and logits from
    bin/trace_run fed with steps on its standard input (a prompt in two portions, then single tokens)."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    raw, seed, page = CONFIGS["B"]
    cfg, w = helpers.read_folder(folders["B"])
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "pulsar-generate"), "--model", folders["B"], "--dtype", "float32",
                          "--prompt_ids", "5,4,3,2,1,0,7", "--prompt_ids", "9 8", "--gen_tokens", "6", "--max_pages", "64", "--eos_id",
                          "-1", "--json"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["outputs"]
    for prompt, new in zip(([5, 4, 3, 2, 1, 0, 7], [9, 8]), got):
        seq = list(prompt)
        for tok in new:
            assert tok == int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax())
            seq.append(tok)
    rng = random.Random(3)
    toks = helpers.random_tokens(rng, 40, raw["vocab"])
    trace = helpers.Trace()
    trace.step([("x", toks[:21], [20])])
    trace.step([("x", toks[21:37], [0, 15])])
    for i in range(37, 40):
        trace.step([("x", toks[i:i + 1], [0])], end=["x"] if i == 39 else [])
    run = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folders["B"], "--dtype", "float32", "--out", str(tmp_path),
                          "--max-tokens", "64"], input=trace.lines(), capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    assert [ln for ln in run.stdout.splitlines() if ln.startswith("done ")] == [f"done {i}" for i in range(len(trace.records))]
    ref = plain.forward(cfg, w, toks, torch.float64)
    for i, rows in enumerate(trace.rows):
        got = torch.from_file(str(tmp_path / f"{i}.f32"), size=len(rows) * raw["vocab"], dtype=torch.float32).view(len(rows), -1)
        for j, (_, pos) in enumerate(rows):
            assert helpers.rel_err(got[j], ref[pos]) < TOL["float32"]
