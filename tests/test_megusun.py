"""Megusun through the engine against the plain implementation (tests/plain/megusun_plain.py): configuration and the
oracle's own mechanisms on the CPU; on a GPU each mechanism alone, prompts against token-by-token decoding, portions
down to two tokens, mixed batches with pages and slots used again, crafted keys far back, at page borders and among the
first tokens for both score maps, the kept rows of the token shift and of the recurrence across steps, the router and
the experts that weigh their input, long decoding, and greedy generation through the public entry point."""
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
from helpers import TOL
from plain import megusun_plain as plain


def attn(heads, kv_heads, dim, vdim, diff=0.6, temp=None, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, diff=diff, scale=scale or 1.0 / math.sqrt(dim))
    if temp is not None:
        m["q_temp"] = dict(coef=temp[0], every=temp[1])
    return dict(type="attention", mixer=m)


def gru(width):
    return dict(type="mingru", mixer=dict(width=width))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared is not None:
        m["shared"] = dict(ff=shared)
    return m


def layer(mixer, mlp=None):
    return dict(mixer, mlp=mlp)


def config(layers, vocab, width, eps=1e-5, mult=1.0):
    return dict(architecture="Megusun", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, layers=layers)


# Every size differs between the configurations: odd head counts, one key/value head, as many key/value heads as query
# heads, groups of two and three, values narrower than, as wide as and wider than the keys, temperatures whose period is
# shorter than a page and longer than the prompt, layers without a temperature and without a feed-forward, recurrences of
# other widths than the model, one expert of one, all experts chosen, mixtures with and without a shared expert,
# multipliers above and below one.
MEGU_A = config([
    layer(gru(40), dense(72)),
    layer(attn(4, 2, 16, 24, diff=0.3, temp=(0.7, 5)), moe(5, 2, 24, shared=40)),
    layer(gru(56), moe(4, 1, 32)),
    layer(attn(3, 3, 8, 8, diff=0.8)),
    layer(attn(6, 2, 12, 40, diff=0.5, temp=(0.25, 300)), dense(64)),
], vocab=180, width=48, eps=1e-5, mult=0.7)
MEGU_B = config([
    layer(attn(5, 1, 12, 20, diff=0.45, temp=(1.5, 17)), moe(7, 3, 16, shared=24)),
    layer(gru(24)),
    layer(gru(80), moe(3, 3, 20)),
    layer(attn(2, 2, 32, 16, diff=0.2, temp=(0.1, 2)), dense(56)),
    layer(gru(40), moe(1, 1, 48, shared=8)),
], vocab=131, width=40, eps=3e-6, mult=1.3)
# head sizes at which the bfloat16 engine's prompt attention runs on the tensor cores
MEGU_C = config([
    layer(attn(4, 2, 64, 64, diff=0.6, temp=(0.5, 32)), moe(6, 2, 32, shared=48)),
    layer(gru(128), dense(96)),
    layer(attn(2, 1, 64, 128, diff=0.35, temp=(0.4, 9)), dense(96)),
], vocab=150, width=64, eps=1e-6, mult=0.5)
ALONE = {
    "attention": config([layer(attn(4, 2, 16, 24, diff=0.4, temp=(0.6, 4)))], vocab=64, width=40),
    "attention_one_group": config([layer(attn(3, 1, 12, 12, diff=0.7))], vocab=64, width=40, mult=0.5),
    "mingru": config([layer(gru(72))], vocab=64, width=40),
    "dense": config([layer(gru(16), dense(56))], vocab=64, width=40, mult=2.0),
    "moe": config([layer(gru(16), moe(6, 2, 24))], vocab=64, width=40),
    "moe_shared": config([layer(gru(16), moe(4, 3, 16, shared=32))], vocab=64, width=40),
}
CONFIGS = {"A": (MEGU_A, 31, 8), "B": (MEGU_B, 32, 4), "C": (MEGU_C, 33, 16)}      # config, seed, page size


# ------------------------------------------------------------------ configuration (CPU)
def test_config_becomes_parts():
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.models import build_model
    cfg = config_from_dict(copy.deepcopy(MEGU_A))
    spec = cfg.model_spec()
    assert [(c.block, c.cache, c.state) for c in spec.run_order] == [(i, i, 5 + i) for i in range(5)]
    assert all(b.kind == "parallel" and b.token_shift and b.residual_multiplier == 0.7 and b.mixer_norm.scalar for b in spec.blocks)
    assert [b.mixer.kind for b in spec.blocks] == ["min_gru", "attention", "min_gru", "attention", "attention"]
    assert [None if b.feed_forward is None else b.feed_forward.kind for b in spec.blocks] == ["mlp", "moe", "moe", None, "mlp"]
    m1, m3 = spec.blocks[1].mixer, spec.blocks[3].mixer
    assert (m1.differential, m1.q_temperature, m1.head_dim, m1.value_dim, m1.norm_eps) == (0.3, (0.7, 5), 16, 24, 1e-5)
    assert (m3.differential, m3.q_temperature, m3.window, m3.position) == (0.8, None, None, None)
    ff1 = spec.blocks[1].feed_forward
    assert (ff1.option("experts"), ff1.option("top"), ff1.option("weight_input"), ff1.option("renormalize")) == (5, 2, True, False)
    assert ff1.option("shared").intermediate == 40 and ff1.option("shared_gate") == "shared.sg"
    assert spec.blocks[2].feed_forward.option("shared") is None and spec.blocks[2].feed_forward.option("shared_gate") is None
    assert spec.blocks[0].feed_forward.activation == "gelu"
    assert cfg.to_dict() == MEGU_A
    model = build_model(cfg, torch.float32)
    shapes = {w.name: tuple(w.shape) for w in model.weight_specs()}
    assert shapes["l0.norm1"] == () and shapes["final.norm"] == () and shapes["l3.shift"] == (48,)
    assert shapes["l1.mix.q"] == (4 * 2 * 16, 48) and shapes["l1.mix.k"] == (2 * 2 * 16, 48) and shapes["l1.mix.v"] == (2 * 24, 48)
    assert shapes["l1.mix.o"] == (48, 4 * 24) and shapes["l1.mix.lq2"] == (16,) and shapes["l0.mix.z.b"] == (40,)
    assert shapes["l1.mlp.shared.sg"] == (1, 48) and shapes["l1.mlp.e4.gate"] == (24, 48) and shapes["l0.mlp.up"] == (72, 48)
    assert not {"l3.mlp.up", "l2.mlp.shared.sg", "l0.mlp.gate", "l0.norm2", "l1.mix.q.b"} & set(shapes)
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["state", "paged_kv", "state", "paged_kv", "paged_kv"] + ["state"] * 5
    assert needs[0].state_shape == (40,) and needs[7].state_shape == (48,) and needs[0].state_dtype == torch.float32
    # both score maps have key heads of their own and share the value heads
    assert [(t.name, t.heads, t.width) for t in needs[1].tensors] == [("k", 4, 16), ("v", 2, 24)]


@pytest.mark.parametrize("edit,match", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0].update(type="mamba1"), "mingru"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][0]["mixer"].pop("width"), "width"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "dense"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors(edit, match):
    from pulsar_b200.config import ConfigError, config_from_dict
    raw = copy.deepcopy(MEGU_A)
    edit(raw)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_plain_mechanisms_agree_with_loops_over_single_numbers():
    """The oracle's vectorised forms against the equations written out one token and one pair at a time."""
    g = torch.Generator().manual_seed(3)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=torch.float64)
    L, W = 9, 10
    h, mix = rnd(L, W), torch.rand(W, generator=g, dtype=torch.float64)
    hs = plain.token_shift(h, mix)
    for t in range(L):
        for i in range(W):
            before = 0.0 if t == 0 else float(h[t - 1, i])
            assert abs(float(hs[t, i]) - (float(h[t, i]) + (before - float(h[t, i])) * float(mix[i]))) < 1e-12
    temp = plain.query_temperature(12, 0.5, 4, torch.float64)
    assert [round(float(x), 9) for x in temp] == [round(1 + 0.5 * math.log((p + 1) // 4 + 1), 9) for p in range(12)]
    assert float(temp[2]) == 1.0 and float(temp[3]) > 1.0         # the first change comes at position every - 1
    # differential attention, one head at a time, one query at a time
    m = dict(heads=4, kv_heads=2, dim=3, vdim=5, diff=0.3, scale=0.4, q_temp=dict(coef=0.5, every=4))
    w = {"q": rnd(4 * 2 * 3, W), "k": rnd(2 * 2 * 3, W), "v": rnd(2 * 5, W), "o": rnd(W, 4 * 5),
         "lq1": 0.3 * rnd(3), "lk1": 0.3 * rnd(3), "lq2": 0.3 * rnd(3), "lk2": 0.3 * rnd(3)}
    out = plain.differential_attention(h, w, m, 1e-6)
    lam = math.exp(float(w["lq1"] @ w["lk1"])) - math.exp(float(w["lq2"] @ w["lk2"])) + 0.3
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    for i in (0, 3, 8):
        heads = []
        for head in range(4):
            kvh = head // 2
            maps = []
            for which in range(2):
                qv = q[i, (2 * head + which) * 3:(2 * head + which + 1) * 3] * float(temp[i])
                s = torch.tensor([float(qv @ k[j, (2 * kvh + which) * 3:(2 * kvh + which + 1) * 3]) * 0.4 for j in range(i + 1)],
                                 dtype=torch.float64)
                p = torch.exp(s - s.max())
                p = p / p.sum()
                maps.append(sum(float(p[j]) * v[j, kvh * 5:(kvh + 1) * 5] for j in range(i + 1)))
            o = maps[0] - lam * maps[1]
            heads.append(o / math.sqrt(float((o * o).mean()) + 1e-6) * 0.7)
        assert float((torch.cat(heads) @ w["o"].T - out[i]).abs().max()) < 1e-10
    # the recurrence, one channel at a time
    wg = {"z": rnd(6, W), "z.b": rnd(6), "x": rnd(6, W), "x.b": rnd(6), "g": rnd(6, W), "o": torch.eye(6, dtype=torch.float64)}
    y = plain.min_gru(h, wg)
    for c in range(6):
        s = 0.0
        for t in range(L):
            z = 1 / (1 + math.exp(-float(h[t] @ wg["z"][c] + wg["z.b"][c])))
            u = float(h[t] @ wg["x"][c] + wg["x.b"][c])
            cand = u + 0.5 if u >= 0 else 1 / (1 + math.exp(-u))
            s = (1 - z) * s + z * cand
            gv = float(h[t] @ wg["g"][c])
            assert abs(float(y[t, c]) - s * gv / (1 + math.exp(-gv))) < 1e-10
    # carried state: two halves equal the whole
    first = plain.min_gru(h[:4], wg)
    z4 = torch.sigmoid(h[:4] @ wg["z"].T + wg["z.b"])
    s4 = torch.zeros(6, dtype=torch.float64)
    u4 = h[:4] @ wg["x"].T + wg["x.b"]
    for t in range(4):
        s4 = (1 - z4[t]) * s4 + z4[t] * torch.where(u4[t] >= 0, u4[t] + 0.5, torch.sigmoid(u4[t]))
    assert float((torch.cat([first, plain.min_gru(h[4:], wg, s4)]) - y).abs().max()) < 1e-12
    # the mixture: the score multiplies the expert's input
    mlp = dict(router=dict(experts=3, top=2), shared=dict(ff=4))
    wm = {"router": rnd(3, W), "shared.sg": rnd(1, W), "shared.gate": rnd(4, W), "shared.up": rnd(4, W), "shared.down": rnd(W, 4)}
    for e in range(3):
        wm.update({f"e{e}.gate": rnd(5, W), f"e{e}.up": rnd(5, W), f"e{e}.down": rnd(W, 5)})
    out = plain.mixture_ff(h, wm, mlp)
    silu = lambda x: x / (1 + torch.exp(-x))
    for t in range(L):
        s = [1 / (1 + math.exp(-float(wm["router"][e] @ h[t]))) for e in range(3)]
        want = torch.zeros(W, dtype=torch.float64)
        for e in sorted(range(3), key=lambda e: -s[e])[:2]:
            x = s[e] * h[t]
            want += wm[f"e{e}.down"] @ (silu(wm[f"e{e}.gate"] @ x) * (wm[f"e{e}.up"] @ x))
        gate = 1 / (1 + math.exp(-float(wm["shared.sg"][0] @ h[t])))
        want += gate * (wm["shared.down"] @ (silu(wm["shared.gate"] @ h[t]) * (wm["shared.up"] @ h[t])))
        assert float((want - out[t]).abs().max()) < 1e-10


def test_a_model_without_paged_layers_has_state_slots_only():
    from pulsar_b200.cache.manager import CacheManager
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.models import build_model
    model = build_model(config_from_dict(copy.deepcopy(ALONE["mingru"])), torch.float32)
    cache = CacheManager(model.cache_needs(), 8, 4, 2, torch.float32, None)
    assert cache.groups == []
    a, b = cache.open("a"), cache.open("b")
    assert {a, b} == {0, 1}
    cache.close("a")
    assert cache.open("c") == a
    cache.check_consistency()


def test_a_random_folder_holds_single_numbers_and_the_plain_model_reads_it(tmp_path):
    helpers.make_folder(tmp_path, copy.deepcopy(MEGU_B), 7, store_dtype=torch.bfloat16)
    cfg, w = helpers.read_folder(str(tmp_path))
    assert w["l0.norm1"].shape == () and w["final.norm"].shape == () and w["l0.mlp.shared.sg"].shape == (1, 40)
    assert 0.0 <= float(w["l2.shift"].min()) and float(w["l2.shift"].max()) <= 1.0
    logits = plain.forward(cfg, w, [3, 1, 4, 1, 5, 9, 2, 6], torch.float64)
    assert logits.shape == (8, 131) and bool(torch.isfinite(logits).all())


# ------------------------------------------------------------------ GPU
gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, raw in list(ALONE.items()) + [(n, c[0]) for n, c in CONFIGS.items()]:
        d = tmp_path_factory.mktemp(f"megu{name}")
        # bfloat16 values: both precisions hold them exactly.  Wider weights than the default make every sublayer count.
        helpers.make_folder(d, copy.deepcopy(raw), 500 + len(out), store_dtype=torch.bfloat16, std=0.15)
        out[name] = str(d)
    return out


CLOSE_CALL = 0.03       # relative margin of a router's choice below which bfloat16 rounding may choose otherwise


class _Reference(dict):
    """request -> plain logits; ``sure[request]``: the positions before the request's first close call of a router.  A token
    that is routed otherwise moves its own logits and, through its keys and the kept rows, those of the tokens behind it, so
    the bfloat16 engine is held to the bar up to there only (the float32 engine everywhere; the experts' bfloat16 kernels
    are held to their formulas with given routes in tests of their own)."""
    sure = None


def _reference(folder, requests):
    cfg, w = helpers.read_folder(folder)
    ref = _Reference()
    ref.sure = {}
    for rid, toks in requests.items():
        margins = []
        ref[rid] = plain.forward(cfg, w, list(toks), torch.float64, margins=margins)
        close = [int(torch.nonzero(m < CLOSE_CALL)[0]) for m in margins if bool((m < CLOSE_CALL).any())]
        ref.sure[rid] = min(close) if close else len(toks)
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


def _compare(got, ref, dtype, what):
    assert got
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        if dtype == "bfloat16" and pos >= ref.sure[rid]:
            continue
        err = helpers.rel_err(row, ref[rid][pos])
        worst = max(worst, err)
        assert err < TOL[dtype], f"{what}: request {rid} position {pos}: error {err:.3e} (first wrong place)"
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


@gpu
@pytest.mark.parametrize("fused", ["1", "0"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_tail_and_portions_agree_with_the_plain_logits(folders, name, dtype, fused, monkeypatch):
    from pulsar_b200.parts import block
    monkeypatch.setattr(block, "PARALLEL_FUSED", fused == "1")     # a layer boundary as one kernel, and as two
    raw, seed, page = CONFIGS[name]
    rng = random.Random(seed)
    toks = helpers.random_tokens(rng, 93, raw["vocab"])
    ref = _reference(folders[name], {"a": toks})
    for what, trace in (("whole", helpers.trace_whole(toks)), ("tail", helpers.trace_tail(toks, 60)),
                        ("portions", helpers.trace_portions(toks, [7, 2, 13, 2, 5, 17, 3])),
                        ("large portions", helpers.trace_portions(toks, [40, 18, 33])),
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
    """230 tokens of which 220 are decoded one by one (from a captured graph), and the same prompt in portions long enough for
    the recurrence's form that is parallel over tokens (runs of 32 with a ragged last one)."""
    raw, seed, page = CONFIGS["B"]
    rng = random.Random(9)
    toks = helpers.random_tokens(rng, 230, raw["vocab"])
    ref = _reference(folders["B"], {"a": toks})
    got, rp = _replay(folders["B"], dtype, helpers.trace_tail(toks, 220), _round64(len(toks)), page)
    _compare(got, ref, dtype, "long decoding")
    assert rp.runner.graph_replays > 150          # the steps of single tokens ran from a captured graph
    got, _ = _replay(folders["B"], dtype, helpers.trace_portions(toks, [101, 66, 63]), _round64(len(toks)), page)
    _compare(got, ref, dtype, "long portions")


def _paged(rows, page_size, order):
    """rows [L, heads, width] -> pool [pages, heads, page, width] with logical page i at page order[i], and the table."""
    L, heads, width = rows.shape
    n_pages = -(-L // page_size)
    pool = torch.zeros(max(order) + 1, heads, page_size, width, dtype=rows.dtype)
    for lp in range(n_pages):
        part = rows[lp * page_size:(lp + 1) * page_size]
        pool[order[lp], :, :part.shape[0]] = part.transpose(0, 1)
    return pool, torch.tensor([order[:n_pages]], dtype=torch.int32)


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


def _two_maps(q, k, v, scale, lam, eps, gain, first=0):
    """q [Lq, H, 2, D] at positions first .. over k [L, G, 2, D], v [L, G, V]: the head's two softmax maps, their weighted
    difference, the division by its root mean square, the gain."""
    Lq, H = q.shape[:2]
    L, G = k.shape[:2]
    vis = (torch.arange(L)[None, :] <= (first + torch.arange(Lq))[:, None])
    out = []
    for h in range(H):
        g = h // (H // G)
        maps = [torch.softmax(((q[:, h, m] @ k[:, g, m].T) * scale).masked_fill(~vis, float("-inf")), dim=-1) @ v[:, g] for m in range(2)]
        out.append(plain.unit_rms(maps[0] - lam * maps[1], eps) * gain)
    return torch.stack(out, dim=1)


@gpu
@pytest.mark.parametrize("kernel", ["tiled", "plain", "tensor_cores"])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_that_stands_out_in_either_map(decode, kernel):
    """Both score maps of every head through the general attention kernels (key heads of their own, shared value heads) and
    the kernel that subtracts them: one key is made to dominate ONE of the two maps wherever it is visible.  It is put at
    the first tokens, far back among hundreds, on both sides of a page border and of a tile border, and at the query
    itself; a key of the wrong map, a wrong value head or a lost first token moves the whole output."""
    from pulsar_b200 import ops
    dtype = torch.bfloat16 if kernel == "tensor_cores" else torch.float32
    g = torch.Generator().manual_seed(21)
    L, H, G, page = 389, 6, 2, 16
    D, V = (64, 128 if decode else 64) if kernel == "tensor_cores" else (24, 40)
    R = H // G
    order = list(range(40))
    random.Random(4).shuffle(order)
    last = L - 1
    for which in (0, 1):
        for spot in (0, 1, 15, 16, 31, 32, 127, 128, 255, 256, last - 1, last):
            q = torch.randn(L, H, 2, D, generator=g, dtype=torch.float64)
            k = torch.randn(L, G, 2, D, generator=g, dtype=torch.float64)
            v = torch.randn(L, G, V, generator=g, dtype=torch.float64)
            q[..., 0] = 3.0                                   # every query looks along dimension 0 ...
            k[spot, :, which, 0] = 60.0                       # ... where one key of one map is far larger than the rest
            if dtype == torch.bfloat16:
                k, v = k.bfloat16().double(), v.bfloat16().double()
            n_q = 1 if decode else 37
            lam, eps, gain = 0.55, 1e-6, 0.4
            want = _two_maps(q[L - n_q:], k, v, 0.2, lam, eps, gain, first=L - n_q)
            # the engine's layout: query heads ordered (key head, map, head in group); key heads (key head, map)
            q_eng = q.view(L, G, R, 2, D).permute(0, 1, 3, 2, 4).reshape(L, 2 * H, D)
            k_pool, table = _paged(k.reshape(L, 2 * G, D).to(dtype), page, order)
            v_pool, _ = _paged(v.to(dtype), page, order)
            ctx = _step_context([n_q], [L])
            maps = torch.empty(n_q, 2 * H, V, dtype=dtype, device="cuda")
            ops.paged_attention_general(ctx, q_eng[L - n_q:].float().cuda().contiguous(), k_pool.cuda(), v_pool.cuda(), maps, table.cuda(),
                                        0.2, tiled=kernel != "plain", tensor_cores=True if kernel == "tensor_cores" else False,
                                        v_share=2)
            out = torch.empty(n_q, H, V, dtype=dtype, device="cuda")
            ops.diff_combine(maps, out, G, lam, eps, gain)
            err = helpers.rel_err(out.cpu(), want)
            assert err < (2e-2 if dtype == torch.bfloat16 else 2e-5), f"map {which}, key {spot}: {err:.3e}"
            # the dominant key shows: without it the output is another one
            k2 = k.clone()
            k2[spot, :, which, 0] = 0.0
            other = _two_maps(q[L - n_q:], k2, v, 0.2, lam, eps, gain, first=L - n_q)
            assert helpers.rel_err(other, want) > 0.2


@gpu
@pytest.mark.parametrize("kernel", ["tiled", "plain", "tensor_cores"])
@pytest.mark.parametrize("decode", [False, True])
def test_maps_from_bfloat16_pages_stay_unrounded_until_they_are_subtracted(decode, kernel):
    """With a weight near one the difference of the two maps is small beside either, and the norm that follows brings it
    back to size: a rounding of the maps to bfloat16 would come out about twenty times as large.  All three attention
    kernels write float32 rows from bfloat16 pages on request."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(8)
    L, H, G, D, V, page = 301, 4, 2, 64, 128, 16
    R = H // G
    n_q = 1 if decode else 45
    lam, eps, gain, scale = 0.9, 1e-6, 0.1, 0.05
    q = torch.randn(L, H, 2, D, generator=g, dtype=torch.float64)
    k = torch.randn(L, G, 2, D, generator=g, dtype=torch.float64).bfloat16().double()
    v = (1.0 + 0.3 * torch.randn(L, G, V, generator=g, dtype=torch.float64)).bfloat16().double()     # both maps near the same mean
    want = _two_maps(q[L - n_q:], k, v, scale, lam, eps, gain, first=L - n_q)
    q_eng = q.view(L, G, R, 2, D).permute(0, 1, 3, 2, 4).reshape(L, 2 * H, D)
    order = list(range(24))
    random.Random(9).shuffle(order)
    k_pool, table = _paged(k.reshape(L, 2 * G, D).bfloat16(), page, order)
    v_pool, _ = _paged(v.bfloat16(), page, order)
    ctx = _step_context([n_q], [L])
    errs = {}
    for maps_dtype in (torch.float32, torch.bfloat16):
        maps = torch.empty(n_q, 2 * H, V, dtype=maps_dtype, device="cuda")
        ops.paged_attention_general(ctx, q_eng[L - n_q:].float().cuda().contiguous(), k_pool.cuda(), v_pool.cuda(), maps, table.cuda(),
                                    scale, tiled=kernel != "plain", tensor_cores=True if kernel == "tensor_cores" else False, v_share=2)
        out = torch.empty(n_q, H, V, dtype=torch.float32 if maps_dtype == torch.float32 else torch.bfloat16, device="cuda")
        ops.diff_combine(maps, out, G, lam, eps, gain)
        errs[maps_dtype] = helpers.rel_err(out.float().cpu(), want)
    assert errs[torch.float32] < 2e-3, errs
    assert errs[torch.bfloat16] > 4 * errs[torch.float32], errs


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels_against_their_formulas(dtype):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(11)
    tol = 1e-5 if dtype == torch.float32 else 1.2e-2
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=torch.float32)

    def close(got, want, what, bar=tol):
        err = helpers.rel_err(got.float().cpu(), want)
        assert err < bar, f"{what}: {err:.3e}"

    # ---- norm and token shift: three sequences, one of a single token, kept rows in slots that are not in order
    q_lens, slots, W = [5, 1, 9], [2, 0, 3], 40
    ctx = _step_context(q_lens, q_lens, slots)
    n = sum(q_lens)
    x, weight, shift = rnd(n, W), 1.0 + 0.1 * rnd(W), torch.rand(W, generator=g)
    state_full = rnd(4, W + 8)                        # rows with a stride of their own
    state = state_full[:, :W]
    eps = 1e-5
    hd = plain.unit_rms(x.double(), eps) * weight.double()
    want_hs = torch.empty_like(hd)
    at = 0
    for s, ql in enumerate(q_lens):
        before = torch.cat([state[slots[s]].double()[None], hd[at:at + ql - 1]])
        want_hs[at:at + ql] = hd[at:at + ql] + (before - hd[at:at + ql]) * shift.double()
        at += ql
    h, hs = torch.empty(n, W, dtype=dtype, device="cuda"), torch.empty(n, W, dtype=dtype, device="cuda")
    pending = torch.zeros(len(q_lens), W, device="cuda")
    state_d = state_full.cuda()[:, :W]
    assert state_d.stride(0) == W + 8
    ops.norm_shift(ctx, x.cuda(), weight.cuda(), eps, shift.cuda(), state_d, h, hs, pending)
    close(h, hd, "norm_shift h")
    close(hs, want_hs, "norm_shift hs")
    ends = [sum(q_lens[:s + 1]) - 1 for s in range(len(q_lens))]
    close(pending, hd[ends], "norm_shift pending", 1e-5)
    assert torch.equal(state_d.cpu(), state)                       # the kept rows are read only
    plain_h = torch.empty(n, W, dtype=dtype, device="cuda")
    ops.norm_shift(ctx, x.cuda(), weight.cuda(), eps, None, None, plain_h, None, None)
    close(plain_h, hd, "norm without shift")

    # ---- the closing kernel: the sum, the move of the kept rows, and the next layer's opening in the same kernel
    a, b, m = rnd(n, W).to(dtype), rnd(n, W).to(dtype), 0.37
    xs = x.double() + m * (a.double() + b.double())
    res = x.clone().cuda()
    ops.parallel_add(ctx, res, a.cuda(), b.cuda(), m, pending, state_d)
    close(res, xs, "parallel_add", 1e-6)
    kept = state.clone()
    for s in range(len(q_lens)):
        kept[slots[s]] = pending[s].cpu()
    assert torch.equal(state_d.cpu(), kept) and torch.equal(state_d.cpu()[1], state[1])      # slot 1 belongs to nobody
    res2 = x.clone().cuda()
    ops.parallel_add(ctx, res2, a.cuda(), None, m)
    close(res2, x.double() + m * a.double(), "parallel_add of one sublayer", 1e-6)
    weight2, shift2, state2 = 1.0 + 0.1 * rnd(W), torch.rand(W, generator=g), rnd(4, W).cuda()
    out = torch.empty(n, W, device="cuda")
    h2, hs2 = torch.empty(n, W, dtype=dtype, device="cuda"), torch.empty(n, W, dtype=dtype, device="cuda")
    pending2 = torch.zeros(len(q_lens), W, device="cuda")
    state_b = state.contiguous().cuda()
    ops.parallel_add(ctx, x.cuda(), a.cuda(), b.cuda(), m, pending, state_b, out, weight2.cuda(), eps, shift2.cuda(), state2, pending2,
                     h2, hs2)
    assert torch.equal(out, res) and torch.equal(state_b.cpu(), kept)
    h_ref, hs_ref = torch.empty_like(h2), torch.empty_like(hs2)
    pending_ref = torch.zeros_like(pending2)
    ops.norm_shift(ctx, res, weight2.cuda(), eps, shift2.cuda(), state2, h_ref, hs_ref, pending_ref)
    assert torch.equal(h2, h_ref) and torch.equal(hs2, hs_ref) and torch.equal(pending2, pending_ref)      # one kernel or two: the same bits

    # ---- activations
    z = 3.0 * rnd(33, 70)
    for kind, f in (("gelu", lambda t: 0.5 * t * (1 + torch.erf(t / math.sqrt(2.0)))),
                    ("gelu_tanh", lambda t: 0.5 * t * (1 + torch.tanh(math.sqrt(2 / math.pi) * (t + 0.044715 * t ** 3)))),
                    ("silu", lambda t: t * torch.sigmoid(t)), ("relu", lambda t: t.clamp_min(0))):
        o = torch.empty(33, 70, dtype=dtype, device="cuda")
        ops.activation(z.cuda(), o, kind)
        close(o, f(z.double()), kind)
    # (the two gelu forms lie 3.6e-5 apart on this scale: the float32 bar tells them apart)
    assert helpers.rel_err(0.5 * z.double() * (1 + torch.erf(z.double() / math.sqrt(2.0))),
                           0.5 * z.double() * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z.double() + 0.044715 * z.double() ** 3)))) > 2e-5

    # ---- the split of the projection row with a query temperature: positions on both sides of the period's edges
    Hq, Hk, Hv, D, V, page = 6, 4, 2, 12, 20, 4
    positions = [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 33, 34, 35, 36, 699, 700, 701]
    nq = len(positions)
    row = rnd(nq, Hq * D + Hk * D + Hv * V).to(dtype)
    q_out = torch.empty(nq, Hq, D, device="cuda")
    k_pool, v_pool = torch.zeros(8, Hk, page, D, dtype=dtype, device="cuda"), torch.zeros(8, Hv, page, V, dtype=dtype, device="cuda")
    slot = torch.randperm(32, generator=g)[:nq].to(torch.int32)
    ops.qkv_split_write(row.cuda(), q_out, k_pool, v_pool, slot.cuda(), Hq, Hk, D, V, page, n_value_heads=Hv,
                        positions=torch.tensor(positions, dtype=torch.int32).cuda(), q_temperature=(0.8, 7))
    f = torch.tensor([1 + 0.8 * math.log((p + 1) // 7 + 1) for p in positions], dtype=torch.float64)
    assert float(f[5]) == 1.0 and float(f[6]) > 1.5 and float(f[12]) == float(f[6]) and float(f[13]) > float(f[12])
    close(q_out, row[:, :Hq * D].double().view(nq, Hq, D) * f[:, None, None], "queries with their temperature", 1e-6)
    for t in range(nq):
        pg, off = int(slot[t]) // page, int(slot[t]) % page
        assert torch.equal(k_pool[pg, :, off].cpu(), row[t, Hq * D:(Hq + Hk) * D].view(Hk, D))
        assert torch.equal(v_pool[pg, :, off].cpu(), row[t, (Hq + Hk) * D:].view(Hv, V))

    # ---- the weighted difference of the two maps
    Hh, G, V = 6, 3, 40
    maps = rnd(9, 2 * Hh, V).to(dtype)
    o = torch.empty(9, Hh, V, dtype=dtype, device="cuda")
    ops.diff_combine(maps.cuda(), o, G, 0.63, 1e-5, 0.25)
    R = Hh // G
    md = maps.double().view(9, G, 2, R, V)
    want = plain.unit_rms(md[:, :, 0] - 0.63 * md[:, :, 1], 1e-5).reshape(9, Hh, V) * 0.25
    close(o, want, "diff_combine")


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_lens", [[1, 1, 1], [7, 1, 30], [150, 2, 65, 33], [64], [97], [2200, 3, 700]])
def test_the_recurrence_against_its_formula(q_lens, dtype):
    """Both forms of the kernel (token by token; in runs, parallel over tokens) with kept states in slots out of order, and
    a second step that goes on from the states the first one left.  The longest portion has more runs than a block's
    warps keep in registers between their two walks."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(sum(q_lens))
    W, n = 72, sum(q_lens)
    slots = list(range(len(q_lens)))[::-1]
    state_full = torch.randn(len(q_lens) + 1, W + 24, generator=g)
    state = state_full[:, :W]
    bz, bx = torch.randn(W, generator=g), torch.randn(W, generator=g)

    def want(proj, st):
        z = torch.sigmoid(proj[:, :W].double() + bz.double())
        u = proj[:, W:2 * W].double() + bx.double()
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        gate = proj[:, 2 * W:].double()
        gate = gate * torch.sigmoid(gate)
        y, st = torch.empty(n, W, dtype=torch.float64), st.double().clone()
        at = 0
        for s, ql in enumerate(q_lens):
            cur = st[slots[s]]
            for t in range(at, at + ql):
                cur = (1 - z[t]) * cur + z[t] * cand[t]
                y[t] = cur * gate[t]
            st[slots[s]] = cur
            at += ql
        return y, st
    ctx = _step_context(q_lens, q_lens, slots)
    state_d = state_full.cuda()[:, :W]
    ref_state = state
    for step in range(2):
        proj = 2.0 * torch.randn(n, 3 * W, generator=g)
        y = torch.empty(n, W, dtype=dtype, device="cuda")
        ops.min_gru(ctx, proj.cuda(), bz.cuda(), bx.cuda(), state_d, y)
        y_ref, ref_state = want(proj, ref_state)
        assert helpers.rel_err(y.float().cpu(), y_ref) < (1e-5 if dtype == torch.float32 else 1e-2), f"step {step}"
        assert helpers.rel_err(state_d.cpu(), ref_state) < 1e-5, f"kept state after step {step}"
    assert torch.equal(state_d.cpu()[len(q_lens)], state[len(q_lens)])          # a slot nobody holds is untouched


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_and_experts_that_weigh_their_input(dtype):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(13)
    n, W, E, top, ff = 11, 40, 6, 3, 24
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    h = torch.randn(n, W, generator=g).to(dtype)
    router = torch.randn(E + 1, W, generator=g)                      # the last row is the shared expert's gate
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(n, top, device="cuda")
    extra = torch.empty(n, 1, device="cuda")
    ops.moe_route(h.cuda(), router.cuda(), ids, wts, 1.0, False, extra)
    s = torch.sigmoid(h.double() @ router.double().T)
    want_ids, want_w = plain.router_choice(h.double(), router[:E].double(), top)
    assert torch.equal(ids.cpu().long(), want_ids)                  # the row behind the experts' competes for nothing
    assert helpers.rel_err(wts.cpu(), want_w) < 1e-5 and helpers.rel_err(extra.cpu()[:, 0], s[:, E]) < 1e-5
    w_gu = (0.3 * torch.randn(E, 2 * ff, W, generator=g)).to(dtype)
    w_d = (0.3 * torch.randn(E, W, ff, generator=g)).to(dtype)
    add = torch.randn(n, W, generator=g).to(dtype)
    act = torch.empty(n * top, ff, dtype=dtype, device="cuda")
    out = torch.empty(n, W, dtype=dtype, device="cuda")
    ops.moe_gate_up(h.cuda(), w_gu.cuda(), ids, act, (0.0, 1.0, 0.0), wts)
    ops.moe_down(act, w_d.cuda(), ids, None, add.cuda(), out, extra)
    want = torch.zeros(n, W, dtype=torch.float64)
    for t in range(n):
        for c in range(top):
            e, x = int(want_ids[t, c]), float(want_w[t, c]) * h[t].double()
            gu = w_gu[e].double() @ x
            unit = gu[:ff] * torch.sigmoid(gu[:ff]) * gu[ff:]
            if dtype == torch.bfloat16:
                unit = unit.bfloat16().double()
            want[t] += w_d[e].double() @ unit
        want[t] += float(s[t, E]) * add[t].double()
    err = helpers.rel_err(out.float().cpu(), want)
    assert err < tol, f"experts that weigh their input: {err:.3e}"
    # the weight on the input is not the weight on the output
    out2 = torch.empty_like(out)
    ops.moe_gate_up(h.cuda(), w_gu.cuda(), ids, act, (0.0, 1.0, 0.0))
    ops.moe_down(act, w_d.cuda(), ids, wts, add.cuda(), out2, extra)
    assert helpers.rel_err(out2.float().cpu(), want) > 0.05


@gpu
@pytest.mark.parametrize("tcgen05", [False, True])
@pytest.mark.parametrize("sizes", [(150, 40, 7, 3, 24), (37, 64, 3, 1, 72), (300, 72, 5, 5, 8), (700, 320, 6, 2, 136)])
def test_grouped_experts_that_weigh_their_input_equal_the_per_token_kernels(sizes, tcgen05):
    from pulsar_b200 import ops
    n, W, E, top, ff = sizes
    g = torch.Generator().manual_seed(n)
    dev = lambda t: t.cuda()
    h = torch.randn(n, W, generator=g).bfloat16()
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    wts = torch.rand(n, top, generator=g) + 0.2
    w_gu = (0.2 * torch.randn(E, 2 * ff, W, generator=g)).bfloat16()
    w_d = (0.2 * torch.randn(E, W, ff, generator=g)).bfloat16()
    add, scale = torch.randn(n, W, generator=g).bfloat16(), torch.rand(n, generator=g)
    gating = (0.0, 1.0, 0.0)
    act = torch.empty(n * top, ff, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(n * top, W, device="cuda")
    out = torch.empty(n, W, dtype=torch.bfloat16, device="cuda")
    work = torch.empty(ops.moe_grouped_workspace(n, top, E), dtype=torch.int32, device="cuda")
    gathered = torch.empty(n * top, W, dtype=torch.bfloat16, device="cuda") if tcgen05 else None
    ops.moe_grouped(dev(h), dev(w_gu), dev(w_d), dev(ids), dev(wts), dev(add), act, y, out, work, gating, gathered,
                    weight_input=True, add_scale=dev(scale))
    ops.check_wait_words()
    act2 = torch.empty_like(act)
    ref = torch.empty_like(out)
    ops.moe_gate_up(dev(h), dev(w_gu), dev(ids), act2, gating, dev(wts))
    ops.moe_down(act2, dev(w_d), dev(ids), None, dev(add), ref, dev(scale))
    err = helpers.rel_err(out.float().cpu(), ref.float().cpu())
    assert err < 1.2e-2, f"grouped against per-token: {err:.3e}"


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
    got16 = generate(folders["A"], prompts, 5, dtype="bfloat16", page_size=page, num_pages=40, max_sessions=4, max_running=3,
                     max_chunk_size=16, device="cuda:0")
    for p, new in zip(prompts, got16):
        seq = list(p)
        for tok in new:
            row = plain.forward(cfg, w, seq, torch.float64)[-1]
            assert float(row.max() - row[tok]) <= TOL["bfloat16"] * float(row.abs().max())
            seq.append(tok)


@gpu
def test_a_preempted_request_is_recomputed_from_fresh_kept_rows(folders):
    """More requests than pages: the scheduler preempts and recomputes; the kept rows of the token shift and of the
    recurrence start again at zero, so the tokens are those of undisturbed runs."""
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
    """The framework's two programs on a Megusun folder: greedy tokens from bin/pulsar-generate, and logits from
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
