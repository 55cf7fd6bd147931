"""Attention over a compressed latent: one cached row per token, expanded per head on the fly."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

from .. import ops
from ..cache.manager import CachedTensor, CacheNeed
from ..config.registry import MIXERS, POSITIONS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec

# PULSAR_LATENT_EXPAND=0: whole prompts too take the absorbed form.
EXPAND_PROMPTS = os.environ.get("PULSAR_LATENT_EXPAND", "1") != "0"


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Every head's query has ``head_dim`` plain dimensions and ``rot_dim`` rotated ones.  A down projection of the
    input gives ``kv_rank`` numbers, RMS-normed into the latent c, and ``rot_dim`` numbers that are rotated at the
    token's position and serve all heads as the rotated key part.  Per head the plain key is W_uk[h] c and the value
    W_uv[h] c; only c and the rotated key part are cached, as one row [c | key_rot] per token.

    The keys and values are never expanded: with q_abs[h] = W_uk[h]^T q_plain[h] the score is
    (q_abs[h] . c + q_rot[h] . key_rot) * scale, and the head's output is W_uv[h] (sum_j p_j c_j).  So the attention
    itself runs with one shared key/value head over the cached rows (key = the whole row, value = its first
    ``kv_rank`` elements) and the two expansions become per-head products on the query and on the output side
    (``ops.heads_linear``).  Queries stay float32 from their rotation to the scores.  A step of whole prompts, whose
    keys are all among its own tokens, expands them instead (see ``forward``); the two forms compute the same function.

    Options (``spec.extra``): ``kv_rank``, ``rot_dim``, ``latent_norm_eps``, ``gated`` (the concatenated heads are
    multiplied by sigmoid(W_g h), h the mixer's input), ``head_gate`` (the same with one gate per head: W_g has a row per
    head and a head's whole output is multiplied by its sigmoid).  ``spec.sinks``: a learned number per head whose
    exponential joins the softmax's denominator (tensor role "sinks").  ``spec.position`` gives the rotation (its table's
    ``rotary_dim`` leading dimensions of the rotated part turn, in neighbouring pairs).  With ``own_kv`` False the
    mixer has no down projection and attends over the rows another layer cached this step, with its own expansions.
    """

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        self.rank = int(spec.option("kv_rank", 0))
        self.rot_dim = int(spec.option("rot_dim", 0))
        self.norm_eps = float(spec.option("latent_norm_eps", 1e-6))
        self.gated = bool(spec.option("gated", False))
        self.head_gate = bool(spec.option("head_gate", False))
        if self.gated and self.head_gate:
            raise ValueError("latent attention: the gate is one per element or one per head, not both")
        if spec.n_heads <= 0 or spec.head_dim <= 0 or spec.value_dim <= 0 or self.rank <= 0 or self.rot_dim < 0:
            raise ValueError("latent attention: heads, head sizes and the latent's rank must be positive")
        if self.rot_dim and spec.position is None:
            raise ValueError("latent attention: a rotated part needs a position encoding")
        if spec.position is not None and spec.position.rotary_dim > self.rot_dim:
            raise ValueError(f"latent attention: {spec.position.rotary_dim} rotating dimensions exceed rot_dim {self.rot_dim}")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.position = POSITIONS.get(spec.position.kind)(spec.position) if spec.position is not None else None
        name = spec.tensor_name
        self.names = {r: name(r, d) for r, d in (("q", "q_proj.weight"), ("down", "kv_down_proj.weight"),
                                                 ("latent_norm", "kv_norm.weight"), ("up_k", "k_up_proj.weight"),
                                                 ("up_v", "v_up_proj.weight"), ("gate", "gate_proj.weight"),
                                                 ("o", "o_proj.weight"), ("sinks", "sinks"))}
        self.sinks = None
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.latent_norm = self.w_uk_rows = self.w_uv_rows = None

    @property
    def row(self) -> int:
        return self.rank + self.rot_dim

    # ---------------------------------------------------------------- weights
    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        specs = [WeightSpec(p + nm["q"], (s.n_heads * (s.head_dim + self.rot_dim), s.hidden))]
        if s.own_kv:
            specs += [WeightSpec(p + nm["down"], (self.row, s.hidden)),
                      WeightSpec(p + nm["latent_norm"], (self.rank,), role="vector", init="ones_normal")]
        specs += [WeightSpec(p + nm["up_k"], (s.n_heads * s.head_dim, self.rank)),
                  WeightSpec(p + nm["up_v"], (s.n_heads * s.value_dim, self.rank))]
        if self.gated or self.head_gate:
            specs.append(WeightSpec(p + nm["gate"], (s.n_heads * (s.value_dim if self.gated else 1), s.hidden)))
        specs.append(WeightSpec(p + nm["o"], (s.hidden, s.n_heads * s.value_dim)))
        if s.sinks:
            specs.append(WeightSpec(p + nm["sinks"], (s.n_heads,), role="vector", init="small"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s, p, nm = self.spec, self.prefix, self.names
        rows = [tensors[p + nm["q"]]]
        if s.own_kv:
            rows.append(tensors[p + nm["down"]])
            self.latent_norm = tensors[p + nm["latent_norm"]]
        if self.gated or self.head_gate:
            rows.append(tensors[p + nm["gate"]])
        if s.sinks:
            self.sinks = tensors[p + nm["sinks"]]
        self.w_in = torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0]      # rows: q | down | gate
        # per head [inputs, outputs]: the key expansion as stored serves the query side (head_dim -> rank), the value
        # expansion is transposed once (rank -> value_dim)
        self.w_uk_t = tensors[p + nm["up_k"]].view(s.n_heads, s.head_dim, self.rank).contiguous()
        self.w_uv = tensors[p + nm["up_v"]].view(s.n_heads, s.value_dim, self.rank).transpose(1, 2).contiguous()
        self.w_uk_rows, self.w_uv_rows = tensors[p + nm["up_k"]], tensors[p + nm["up_v"]]      # as stored: the expanded form's products
        self.w_o = tensors[p + nm["o"]]

    def weight_bytes(self) -> int:
        ts = [self.w_in, self.w_uk_t, self.w_uv, self.w_o, self.latent_norm, self.sinks]      # a step reads one form of the expansions
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def cache_need(self) -> CacheNeed:
        return CacheNeed.paged((CachedTensor("latent", 1, self.row),), self.spec.window)

    # ---------------------------------------------------------------- one step
    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        s, n, H = self.spec, ctx.n_tokens, self.spec.n_heads
        q_width = H * (s.head_dim + self.rot_dim)
        proj = ctx.scratch("latent.in", (n, self.w_in.shape[0]))
        ops.linear(h, self.w_in, proj)
        q = proj[:, :q_width]
        down = proj[:, q_width:q_width + self.row] if s.own_kv else None
        gate = proj[:, self.w_in.shape[0] - H * s.value_dim:] if self.gated else None
        head_gate = proj[:, self.w_in.shape[0] - H:] if self.head_gate else None
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
        else:
            cos = sin = ctx.scratch("latent.norope", (n, 0), torch.float32)
        # A step that brings only whole prompts (every sequence starts at 0) has all its keys among its own tokens: it
        # expands them once (two products for the step) and attends with keys head_dim + rot_dim wide and values value_dim
        # wide, a third of the absorbed form's arithmetic per (query, key) pair.  Every other step (portions behind a
        # cached part, single tokens) attends over the cached rows in the absorbed form.  A captured step is a step of
        # single tokens and always takes the absorbed form, so nothing here goes stale in a replay.
        if EXPAND_PROMPTS and not ctx.all_decode and s.window is None and all(start == 0 for start in ctx.host.starts):
            heads = self._expanded(ctx, q, down, cos, sin, cache)
            if gate is not None:
                ops.sigmoid_gate(heads.view(n, H * s.value_dim), gate)
        else:
            heads = self._absorbed(ctx, q, down, gate, cos, sin, cache)
        if head_gate is not None:
            ops.sigmoid_gate_strided(heads.view(n, H * s.value_dim), head_gate, group=s.value_dim)
        out = ctx.scratch("latent.out", (n, s.hidden), torch.float32 if self.output_float32 else None)
        ops.linear(heads.view(n, H * s.value_dim), self.w_o, out)
        return out

    def _absorbed(self, ctx, q, down, gate, cos, sin, cache) -> torch.Tensor:
        s, n, H = self.spec, ctx.n_tokens, self.spec.n_heads
        pool = cache.pools["latent"]
        q_full = ctx.scratch("latent.q", (n, H, self.row), torch.float32)
        ops.heads_linear(q.view(n, H, s.head_dim + self.rot_dim)[:, :, :s.head_dim], self.w_uk_t, q_full[:, :, :self.rank])
        ops.latent_prepare(q, down, self.latent_norm, self.norm_eps, cos, sin, cache.slots if s.own_kv else None,
                           pool if s.own_kv else None, q_full, H, s.head_dim, self.rot_dim, self.rank, cache.page_size)
        mixed = ctx.scratch("latent.mixed", (n, H, self.rank))
        ops.paged_attention_general(ctx, q_full, pool, pool, mixed, cache.block_table, s.scale, s.window, s.chunk, None,
                                    key_width=self.row, value_width=self.rank, sinks=self.sinks)
        heads = ctx.scratch("latent.heads", (n, H, s.value_dim))
        ops.heads_linear(mixed, self.w_uv, heads, gate)
        return heads

    def _expanded(self, ctx, q, down, cos, sin, cache) -> torch.Tensor:
        s, n, H = self.spec, ctx.n_tokens, self.spec.n_heads
        pool = cache.pools["latent"]
        key = ("latent.rows", pool.data_ptr())            # what the cache's owner wrote this step, for those who borrow it
        q_cat = ctx.scratch("latent.q", (n, H, s.head_dim + self.rot_dim), torch.float32)
        if s.own_kv:
            latent = ctx.scratch(f"latent.rows.{pool.data_ptr()}", (n, self.rank))
            shared = ctx.scratch(f"latent.rot.{pool.data_ptr()}", (n, self.rot_dim))
            ops.latent_prepare(q, down, self.latent_norm, self.norm_eps, cos, sin, cache.slots, pool, q_cat, H, s.head_dim,
                               self.rot_dim, self.rank, cache.page_size, plain_too=True, latent_out=latent, rot_out=shared)
            ctx.shared[key] = (latent, shared)
        else:
            latent, shared = ctx.shared[key]
            ops.latent_prepare(q, None, None, self.norm_eps, cos, sin, None, None, q_cat, H, s.head_dim, self.rot_dim, self.rank,
                               cache.page_size, plain_too=True)
        k_plain = ctx.scratch("latent.k_plain", (n, H * s.head_dim))
        ops.linear(latent, self.w_uk_rows, k_plain)
        values = ctx.scratch("latent.values", (n, H * s.value_dim))
        ops.linear(latent, self.w_uv_rows, values)
        keys = ctx.scratch("latent.keys", (n, H, s.head_dim + self.rot_dim))
        ops.latent_expand_keys(k_plain.view(n, H, s.head_dim), shared, keys)
        # the step's own rows as pages of one token: row t of sequence i is page cu_q[i] + t
        table = ctx.shared.get("rows_as_pages")
        if table is None:
            table = (ctx.cu_q[:-1, None] + torch.arange(ctx.max_q_len, dtype=torch.int32, device=ctx.device)[None, :]).contiguous()
            ctx.shared["rows_as_pages"] = table
        heads = ctx.scratch("latent.heads", (n, H, s.value_dim))
        ops.paged_attention_general(ctx, q_cat, keys.view(n, H, 1, s.head_dim + self.rot_dim), values.view(n, H, 1, s.value_dim),
                                    heads, table, s.scale, None, s.chunk, None, sinks=self.sinks)
        return heads
