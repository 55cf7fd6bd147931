"""The minimal gated recurrent mixer: gates that read the current token only, a float32 state per channel."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..cache.manager import CacheNeed
from ..config.registry import MIXERS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec


@MIXERS.register("min_gru")
class MinGRU(Mixer):
    """z = sigmoid(W_z h + b_z), u = W_x h + b_x, both ``width`` channels; the candidate is c = u + 1/2 where u >= 0 and
    sigmoid(u) below; S_t = (1 - z) S_(t-1) + z c element by element; out = W_o (S_t * silu(W_g h)).

    The state S [width] of a sequence is float32 and lives in the sequence's slot of the cache manager's state arena; it
    starts at zero and is carried from step to step.  The three projections of h are one product with float32 rows
    (z | u | g); the biases, the sigmoids, the candidate, the recurrence and the gate are one kernel in float32
    (``ops.min_gru``), which takes what it needs to know about the step (where each sequence's tokens begin, which slot is
    its own) from the step's device arrays, so a step of single tokens can be replayed from a CUDA graph.

    Options (``spec.extra``): ``width``.  Tensor names by role "z", "z_bias", "x", "x_bias", "g", "o".
    """

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        self.width = int(spec.option("width", 0))
        if self.width <= 0:
            raise ValueError("min_gru: width must be positive")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        name = spec.tensor_name
        self.names = {r: name(r, d) for r, d in (("z", "z_proj.weight"), ("z_bias", "z_proj.bias"), ("x", "x_proj.weight"),
                                                 ("x_bias", "x_proj.bias"), ("g", "g_proj.weight"), ("o", "out_proj.weight"))}
        self.w_zxg = self.w_o = self.b_z = self.b_x = None

    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm, w = self.spec, self.prefix, self.names, self.width
        return [WeightSpec(p + nm["z"], (w, s.hidden)), WeightSpec(p + nm["z_bias"], (w,), role="vector", init="small"),
                WeightSpec(p + nm["x"], (w, s.hidden)), WeightSpec(p + nm["x_bias"], (w,), role="vector", init="small"),
                WeightSpec(p + nm["g"], (w, s.hidden)), WeightSpec(p + nm["o"], (s.hidden, w))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p, nm = self.prefix, self.names
        self.w_zxg = torch.cat([tensors[p + nm["z"]], tensors[p + nm["x"]], tensors[p + nm["g"]]], dim=0).contiguous()
        self.w_o = tensors[p + nm["o"]]
        self.b_z, self.b_x = tensors[p + nm["z_bias"]], tensors[p + nm["x_bias"]]

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_zxg, self.w_o, self.b_z, self.b_x))

    def cache_need(self) -> CacheNeed:
        return CacheNeed.state((self.width,), torch.float32)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        n = ctx.n_tokens
        proj = ctx.scratch("gru.proj", (n, 3 * self.width), torch.float32)
        ops.linear(h, self.w_zxg, proj)
        y = ctx.scratch("gru.y", (n, self.width))
        ops.min_gru(ctx, proj, self.b_z, self.b_x, cache.state, y)
        out = ctx.scratch("gru.out", (n, self.spec.hidden))
        ops.linear(y, self.w_o, out)
        return out
