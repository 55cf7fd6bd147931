"""Retention: linear attention with a fixed decay per head and a float32 state matrix per sequence."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..cache.manager import CacheNeed
from ..config.registry import MIXERS, POSITIONS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec


@MIXERS.register("retention")
class Retention(Mixer):
    """q = W_q h and k = W_k h have ``n_heads`` heads of ``head_dim``, v = W_v h heads of ``value_dim``; the first rotating
    dimensions of q and k turn at the token's position (rotate-half layout) and k is multiplied by ``key_scale`` afterwards.
    Per head a matrix S [head_dim, value_dim] decays by the head's fixed factor and takes k v^T at every token,
    S_t = decay_h S_(t-1) + k_t v_t^T, and is read with the query, o_t = S_t^T q_t: no softmax, no denominator.  Each head's
    o is divided by its root mean square (``norm_eps`` inside the root, no weight); the concatenated heads are multiplied by
    silu(W_g h) and projected by W_o.

    The state of a sequence (all heads' matrices, float32) lives in the sequence's slot of the cache manager's state arena;
    it starts at zero and is carried from step to step.  The four projections of h are one product with float32 rows
    (q | k | v | g); rotation, scale, recurrence, norm and gate are float32 kernels (``ops.retention``: token by token for
    steps of single tokens and short portions, in chunks that run side by side for longer portions), which take what they
    need to know about the step from the step's device arrays, so a step of single tokens can be replayed from a CUDA graph.

    Options (``spec.extra``): ``decay`` (a tuple with one factor per head), ``key_scale`` (default ``head_dim`` ** -0.5).
    Tensor names by role "q", "k", "v", "g", "o".
    """

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        decay = tuple(float(d) for d in (spec.option("decay", ()) or ()))
        if spec.n_heads <= 0 or spec.head_dim <= 0 or spec.value_dim <= 0:
            raise ValueError("retention: heads and head sizes must be positive")
        if len(decay) != spec.n_heads or any(not (0.0 <= d <= 1.0) for d in decay):
            raise ValueError(f"retention: needs one decay factor between 0 and 1 for each of the {spec.n_heads} heads")
        if spec.position is not None and spec.position.rotary_dim > spec.head_dim:
            raise ValueError(f"retention: {spec.position.rotary_dim} rotating dimensions exceed the head size {spec.head_dim}")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.decay_values = decay
        self.key_scale = float(spec.option("key_scale", spec.head_dim ** -0.5))
        self.position = POSITIONS.get(spec.position.kind)(spec.position) if spec.position is not None else None
        name = spec.tensor_name
        self.names = {r: name(r, d) for r, d in (("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"),
                                                 ("g", "g_proj.weight"), ("o", "o_proj.weight"))}
        self.w_in = self.w_o = self.decay = None

    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        qk, v = s.n_heads * s.head_dim, s.n_heads * s.value_dim
        return [WeightSpec(p + nm["q"], (qk, s.hidden)), WeightSpec(p + nm["k"], (qk, s.hidden)), WeightSpec(p + nm["v"], (v, s.hidden)),
                WeightSpec(p + nm["g"], (v, s.hidden)), WeightSpec(p + nm["o"], (s.hidden, v))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p, nm = self.prefix, self.names
        self.w_in = torch.cat([tensors[p + nm[r]] for r in ("q", "k", "v", "g")], dim=0).contiguous()      # rows: q | k | v | g
        self.w_o = tensors[p + nm["o"]]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(self.w_o.device)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.decay))

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed.state((s.n_heads * s.head_dim * s.value_dim,), torch.float32)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        s, n = self.spec, ctx.n_tokens
        rows = ctx.scratch("retention.rows", (n, self.w_in.shape[0]), torch.float32)
        ops.linear(h, self.w_in, rows)
        cos = sin = None
        rotary = 0
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary = s.position.rotary_dim
        y = ctx.scratch("retention.y", (n, s.n_heads * s.value_dim))
        ops.retention(ctx, rows, cos, sin, self.decay, cache.state, y, s.n_heads, s.head_dim, s.value_dim, rotary, self.key_scale,
                      s.norm_eps)
        out = ctx.scratch("retention.out", (n, s.hidden), torch.float32 if self.output_float32 else None)
        ops.linear(y, self.w_o, out)
        return out
