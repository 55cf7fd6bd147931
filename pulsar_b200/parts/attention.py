"""Grouped-query attention over a paged key/value cache."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..cache.manager import CachedTensor, CacheNeed
from ..config.registry import MIXERS, POSITIONS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec
from .norm import RMSNorm, accumulate_and_prepare


@MIXERS.register("attention")
class Attention(Mixer):
    """q/k/v projection without bias (one fused product), optional per-head RMSNorm of
    q and k before rotation, rotation at the tokens' explicit positions, write of k and v
    into the pages, attention over the pages (causal, optional window, grouped heads),
    output projection (pulsar-core/src/model/qwen3.cpp:81-114;
    pulsar-core/src/model/paged_forward.cpp:30-80).

    Keys are stored rotated, once, at their absolute position.  With ``own_kv`` False the
    mixer has no k/v projection and attends over pages another layer wrote this step.

    The general form (``self.general``: value heads of another width than the key heads, a chunk mask, or a
    linear distance bias per head) has no rotation and no per-head norm; positions enter through the bias and
    the masks alone.  Its queries stay float32 from the projection to the scores
    (``ops.qkv_split_write`` / ``ops.paged_attention_general``).

    The general form also carries what further designs ask of an attention layer, each a field of the specification:
    biases of the projections, values that are the projected keys (no v projection), rotation in the rotate-half layout
    followed by a division of q and k by their root mean square (``qk_norm_weight`` False, ``qk_norm_after_rotation``),
    a cap on the scaled scores, first keys that stay visible below a window (``keep_first``), a learned sink per head in
    the softmax's denominator, and a sigmoid gate on the concatenated heads from a projection of the mixer's input.
    With any of these the fused projection (rows q | k | v | gate) is a float32 product, the bias is added in float32,
    and ``ops.qk_prepare`` does what stands between it and the attention kernels.  In that form the per-head norm may
    also be the weighted one in front of the rotation (``qk_norm_weight``, not ``qk_norm_after_rotation``), the mixer may
    have a v projection of its own (value heads of ``value_dim``), and the sink may be one given number for all heads
    (``fixed_sink``; 0 adds one to the softmax's denominator).

    The differential form (``spec.differential`` = d, part of the general form without rotation, biases or per-head norm):
    every head has two score maps over the same values.  Its query rows hold [map 1 | map 2] (``head_dim`` each) and so do
    the key rows of a key/value head; the engine treats the maps as 2 H query heads over 2 G key heads that read G value
    heads (``v_share`` 2), with the query rows re-ordered once at load so that the query heads of one key head are
    neighbours, and ``ops.diff_combine`` gives unit_rms(a1 - lambda a2) * (1 - d) per head, lambda = exp(<lq1, lk1>) -
    exp(<lq2, lk2>) + d.  ``spec.q_temperature`` = (coef, every) multiplies the query at position p by
    1 + coef * ln(floor((p + 1) / every) + 1) (float32, as the queries are split off the projection row).

    ``output_bias`` is the output projection's bias (or None).  ``forward`` adds it unless the block has set
    ``defer_output_bias`` because the kernel behind the mixer takes it along.
    """

    output_bias: Optional[torch.Tensor] = None
    defer_output_bias: bool = False

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        if spec.n_heads <= 0 or spec.n_kv_heads <= 0 or spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"attention: {spec.n_heads} query heads cannot be grouped over {spec.n_kv_heads} kv heads")
        # what only ops.qk_prepare does between the projection and the attention kernels (its rows may be wider than
        # q | k, so the gate's columns ride along in the same product)
        self.prepared = bool(spec.bias or spec.values_from_keys or not spec.qk_norm_weight or spec.qk_norm_after_rotation
                             or spec.output_gate)
        self.maps = 2 if spec.differential is not None else 1          # score maps per head
        self.general = bool(spec.value_dim != spec.head_dim or spec.chunk is not None or spec.distance_bias is not None
                            or spec.keep_first or spec.softcap is not None or spec.sinks or spec.fixed_sink is not None
                            or spec.output_gate or self.prepared
                            or self.maps > 1 or spec.q_temperature is not None)
        if (self.maps > 1 or spec.q_temperature is not None) and (self.prepared or not spec.own_kv):
            raise ValueError("attention: the differential form and the query temperature go with plain projections of its own keys")
        if spec.q_temperature is not None and not (int(spec.q_temperature[1]) > 0):
            raise ValueError("attention: the query temperature's period must be positive")
        if self.general:
            if not self.prepared and (spec.position is not None or spec.qk_norm_eps is not None):
                raise ValueError("attention: the general form (value width, chunk mask, distance bias) has neither rotation nor q/k norm")
            if self.prepared:
                if spec.qk_norm_eps is not None and spec.qk_norm_weight == spec.qk_norm_after_rotation:
                    raise ValueError("attention: the q/k norm is the weighted one before the rotation or the one without a weight behind it")
                if spec.sinks and spec.fixed_sink is not None:
                    raise ValueError("attention: a sink is learned per head or one given number, not both")
                if spec.values_from_keys and spec.value_dim != spec.head_dim:
                    raise ValueError("attention: values that are the keys are as wide as the keys")
            if spec.head_dim <= 0 or spec.value_dim <= 0 or (spec.chunk is not None and spec.chunk <= 0):
                raise ValueError("attention: head sizes and the chunk size must be positive")
            if spec.keep_first < 0 or (spec.softcap is not None and not (spec.softcap > 0.0)):
                raise ValueError("attention: keep_first must not be negative and the cap on the scores must be positive")
        elif spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be a multiple of 16, at most 256")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("attention: window must be positive")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.position = POSITIONS.get(spec.position.kind)(spec.position) if spec.position is not None else None
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.slopes = None
        self.q_bias = self.k_bias = self.sinks = None
        name = spec.tensor_name
        self.names = {"q": name("q", "q_proj.weight"), "k": name("k", "k_proj.weight"), "v": name("v", "v_proj.weight"),
                      "o": name("o", "o_proj.weight"), "q_norm": name("q_norm", "q_norm.weight"),
                      "k_norm": name("k_norm", "k_norm.weight"), "gate": name("gate", "g_proj.weight"),
                      "sinks": name("sinks", "sinks"), "lq1": name("lq1", "lambda_q1"), "lk1": name("lk1", "lambda_k1"),
                      "lq2": name("lq2", "lambda_q2"), "lk2": name("lk2", "lambda_k2")}
        self.diff_lambda = 0.0
        for role in ("q", "k", "o"):          # a bias is named after its weight unless the specification names it
            weight = self.names[role]
            default = weight[:-len(".weight")] + ".bias" if weight.endswith(".weight") else weight + ".b"
            self.names[role + "_bias"] = name(role + "_bias", default)
        self.own_v = spec.own_kv and not spec.values_from_keys

    # ---------------------------------------------------------------- weights
    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        specs = [WeightSpec(p + nm["q"], (s.n_heads * self.maps * s.head_dim, s.hidden))]
        if s.own_kv:
            specs.append(WeightSpec(p + nm["k"], (s.n_kv_heads * self.maps * s.head_dim, s.hidden)))
        if self.own_v:
            specs.append(WeightSpec(p + nm["v"], (s.n_kv_heads * s.value_dim, s.hidden)))
        if s.output_gate:
            specs.append(WeightSpec(p + nm["gate"], (s.n_heads * s.value_dim, s.hidden)))
        specs.append(WeightSpec(p + nm["o"], (s.hidden, s.n_heads * s.value_dim)))
        if s.bias:
            specs.append(WeightSpec(p + nm["q_bias"], (s.n_heads * s.head_dim,), role="vector", init="small"))
            if s.own_kv:
                specs.append(WeightSpec(p + nm["k_bias"], (s.n_kv_heads * s.head_dim,), role="vector", init="small"))
            specs.append(WeightSpec(p + nm["o_bias"], (s.hidden,), role="vector", init="small"))
        if s.sinks:
            specs.append(WeightSpec(p + nm["sinks"], (s.n_heads,), role="vector", init="small"))
        if self.maps > 1:
            specs += [WeightSpec(p + nm[r], (s.head_dim,), role="vector", init="small") for r in ("lq1", "lk1", "lq2", "lk2")]
        if s.qk_norm_eps is not None and s.qk_norm_weight:
            specs.append(WeightSpec(p + nm["q_norm"], (s.head_dim,), role="vector", init="ones_normal"))
            if s.own_kv:
                specs.append(WeightSpec(p + nm["k_norm"], (s.head_dim,), role="vector", init="ones_normal"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s, p, nm = self.spec, self.prefix, self.names
        parts = [tensors[p + nm["q"]]]
        if self.maps > 1:
            # stored head by head as [map 1 | map 2]; the kernels want the query heads of one key head side by side:
            # for key/value head g, map m, head-in-group r:  row block (2 g + m) R + r  <-  stored block 2 (g R + r) + m
            R, D = s.n_heads // s.n_kv_heads, s.head_dim
            blocks = parts[0].view(s.n_kv_heads, R, 2, D, s.hidden)
            parts[0] = blocks.permute(0, 2, 1, 3, 4).reshape(2 * s.n_heads * D, s.hidden).contiguous()
            # one number for the layer, from the float32 vectors
            l1, l2 = (torch.exp((tensors[p + nm[a]].double() * tensors[p + nm[b]].double()).sum()) for a, b in (("lq1", "lk1"), ("lq2", "lk2")))
            self.diff_lambda = float((l1 - l2).item() + float(s.differential))
        if s.own_kv:
            parts.append(tensors[p + nm["k"]])
        if self.own_v:
            parts.append(tensors[p + nm["v"]])
        if s.output_gate:
            parts.append(tensors[p + nm["gate"]])
        self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0]   # rows: q | k | v | gate
        self.w_o = tensors[p + nm["o"]]
        if s.bias:
            self.q_bias, self.k_bias = tensors[p + nm["q_bias"]], tensors.get(p + nm["k_bias"])
            self.output_bias = tensors[p + nm["o_bias"]]
        if s.sinks:
            self.sinks = tensors[p + nm["sinks"]]
        elif s.fixed_sink is not None:
            self.sinks = torch.full((s.n_heads,), float(s.fixed_sink), dtype=torch.float32, device=self.w_o.device)
        if s.qk_norm_eps is not None and s.qk_norm_weight:
            self.q_norm = tensors[p + nm["q_norm"]]
            self.k_norm = tensors.get(p + nm["k_norm"])
        if s.distance_bias is not None:
            slopes = [2.0 ** (-float(s.distance_bias) * (h + 1) / s.n_heads) for h in range(s.n_heads)]
            self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(self.w_o.device)

    def weight_bytes(self) -> int:
        ts = [self.w_qkv, self.w_o, self.q_norm, self.k_norm, self.slopes, self.q_bias, self.k_bias, self.output_bias, self.sinks]
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def cache_need(self) -> CacheNeed:
        s = self.spec
        # Pages behind a window go back to the pool as the queries pass them, except those of the kept first keys.
        if s.value_dim != s.head_dim or self.maps > 1:
            return CacheNeed.paged((CachedTensor("k", s.n_kv_heads * self.maps, s.head_dim), CachedTensor("v", s.n_kv_heads, s.value_dim)),
                                   s.window, s.keep_first)
        return CacheNeed.paged_kv(s.n_kv_heads, s.head_dim, s.window, s.keep_first)

    # ---------------------------------------------------------------- one step
    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        s = self.spec
        n = ctx.n_tokens
        if self.prepared:
            # float32 rows: the biases join before anything is rounded, and the queries are float32 from here on anyway
            qkv = ctx.scratch("attn.qkv32", (n, self.w_qkv.shape[0]), torch.float32)
        else:
            qkv = ctx.scratch("attn.qkv", (n, self.w_qkv.shape[0]))
        ops.linear(h, self.w_qkv, qkv)
        o = self._attend_general(ctx, qkv, cache) if self.general else self._attend(ctx, qkv, cache)
        if s.output_gate:
            at = self.w_qkv.shape[0] - s.n_heads * s.value_dim
            ops.sigmoid_gate_strided(o.view(n, s.n_heads * s.value_dim), qkv[:, at:])
        out = ctx.scratch("attn.out", (n, s.hidden), torch.float32 if self.output_float32 else None)
        ops.linear(o.view(n, s.n_heads * s.value_dim), self.w_o, out)
        if self.output_bias is not None and not self.defer_output_bias:
            ops.add_bias(out, self.output_bias)
        return out

    def _attend_general(self, ctx: StepContext, qkv: torch.Tensor, cache: CacheView) -> torch.Tensor:
        """Queries to float32, keys and values to their pages, then the general kernel: o [N, heads, value_dim]."""
        s = self.spec
        n = ctx.n_tokens
        n_kv = s.n_kv_heads if s.own_kv else 0
        maps = self.maps
        q = ctx.scratch("attn.q32", (n, s.n_heads * maps, s.head_dim), torch.float32)
        if self.prepared:
            cos = sin = None
            rotary = 0
            if self.position is not None:
                cos, sin = self.position.tables(ctx)
                rotary = s.position.rotary_dim
            weighted = s.qk_norm_eps is not None and s.qk_norm_weight          # in front of the rotation, with a weight
            ops.qk_prepare(qkv, q, cache.k_pool if n_kv else None, cache.v_pool if n_kv else None, cache.slots if n_kv else None,
                           cos, sin, s.n_heads, n_kv, s.head_dim, rotary, cache.page_size, self.q_bias, self.k_bias if n_kv else None,
                           None if weighted else s.qk_norm_eps, s.values_from_keys,
                           q_norm=self.q_norm if weighted else None, k_norm=self.k_norm if weighted else None,
                           norm_eps=s.qk_norm_eps if weighted else None,
                           n_value_heads=n_kv if self.own_v else 0, value_dim=s.value_dim if self.own_v else 0)
        else:
            ops.qkv_split_write(qkv, q, cache.k_pool if n_kv else None, cache.v_pool if n_kv else None,
                                cache.slots if n_kv else None, s.n_heads * maps, n_kv * maps, s.head_dim, s.value_dim, cache.page_size,
                                n_value_heads=n_kv, positions=ctx.positions, q_temperature=s.q_temperature)
        if maps > 1:
            # float32 rows: the two maps' outputs are subtracted with a weight near one and the difference is normed, which
            # would magnify a rounding of either by (1 + lambda) / (1 - lambda)
            o = ctx.scratch("attn.o.maps", (n, s.n_heads * maps, s.value_dim), torch.float32)
        else:
            o = ctx.scratch("attn.o", (n, s.n_heads * maps, s.value_dim))
        ops.paged_attention_general(ctx, q, cache.k_pool, cache.v_pool, o, cache.block_table, s.scale, s.window, s.chunk,
                                    self.slopes, keep_first=s.keep_first, softcap=s.softcap, sinks=self.sinks, v_share=maps)
        if maps > 1:
            both, o = o, ctx.scratch("attn.o.diff", (n, s.n_heads, s.value_dim))
            ops.diff_combine(both, o, s.n_kv_heads, self.diff_lambda, s.norm_eps, 1.0 - float(s.differential))
        return o

    def forward_normed(self, ctx: StepContext, residual: torch.Tensor, norm, cache: CacheView, next_norm=None) -> bool:
        s = self.spec
        n = ctx.n_tokens
        if n > 16 or not isinstance(norm, RMSNorm) or self.dtype != torch.bfloat16 or self.general:
            return False
        if not (ops.fused_projection_supported(n, self.w_qkv) and ops.fused_projection_supported(n, self.w_o)):
            return False
        n_kv = s.n_kv_heads if s.own_kv else 0
        qkv = ctx.scratch("attn.qkv", (n, (s.n_heads + 2 * n_kv) * s.head_dim))
        prepared = ctx.prepared_norms.pop(id(norm), None)
        if prepared is None or not ops.linear_prenormed(prepared[0], prepared[1], norm.spec.eps, self.w_qkv, qkv):
            ops.linear(norm.forward(ctx, residual, None), self.w_qkv, qkv)
        o = self._attend(ctx, qkv, cache)
        ctx.prepared_norms.clear()              # the residual changes now
        if not accumulate_and_prepare(ctx, o.view(n, s.n_heads * s.head_dim), self.w_o, residual,
                                      next_norm if ops.FUSED_NORM_MLP else None):
            raise ops.KernelError("attention: the output projection refused sizes it had declared supported")
        return True

    def _attend(self, ctx: StepContext, qkv: torch.Tensor, cache: CacheView) -> torch.Tensor:
        """Per-head norm, rotation and cache write of the projected row, then attention: o [N, heads, head_dim]."""
        s = self.spec
        n = ctx.n_tokens
        n_kv = s.n_kv_heads if s.own_kv else 0
        q = ctx.scratch("attn.q", (n, s.n_heads, s.head_dim))
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary = s.position.rotary_dim
        else:
            cos = sin = ctx.scratch("attn.norope", (n, 0), torch.float32)
            rotary = 0
        # (A lone sequence keeps the kernel of its own: its keys are cut into so many splits that every block's share
        # is short, and the norm and rotation in each block's start then cost more than the launch they save:
        # 2.990 against 2.973 ms per step; with two sequences and more the one kernel is ahead by 1.1 to 1.4 %.)
        if (ctx.all_decode and ctx.n_seqs >= 2 and self.position is not None and qkv.dtype == torch.bfloat16
                and ops.decode_qkv_supported(qkv.dtype, s.n_heads, n_kv, s.head_dim, rotary, cache.page_size)):
            # a step of single tokens: the attention kernel normalises, rotates and writes the cache itself
            o = ctx.scratch("attn.o", (n, s.n_heads, s.head_dim))
            n_splits = ops.decode_splits(ctx.n_seqs, n_kv, cache.block_table.shape[1] * cache.page_size)
            partial = ctx.scratch("attn.partial", (ctx.n_seqs * s.n_heads * n_splits * (s.head_dim + 2),), torch.float32)
            ops.paged_attention_decode_qkv(qkv, self.q_norm, self.k_norm, cos, sin, s.qk_norm_eps or 0.0, cache.slots, cache.k_pool,
                                           cache.v_pool, o, partial, cache.block_table, ctx.kv_len, s.scale, s.window, n_splits)
            return o
        ops.qk_norm_rope_write(qkv, q, cache.k_pool if n_kv else None, cache.v_pool if n_kv else None,
                               cache.slots if n_kv else None, cos, sin, self.q_norm, self.k_norm,
                               s.qk_norm_eps or 0.0, s.n_heads, n_kv, s.head_dim, rotary, cache.page_size)
        o = ctx.scratch("attn.o", (n, s.n_heads, s.head_dim))
        ops.attention(ctx, q, cache, o, s.scale, s.window)
        return o
