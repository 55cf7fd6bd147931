"""A mixture of gated experts with a sigmoid router and an optional shared expert."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.registry import FEED_FORWARDS
from ..config.specs import FeedForwardSpec
from .base import FeedForward, StepContext, WeightSpec


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    """Every token is sent to the ``top`` experts with the largest router scores s = sigmoid(W_r h) (float32 logits) and
    receives sum over them of w_e * expert_e(h), with w_e = s_e * ``router_scale`` (divided by the chosen scores' sum
    first where ``renormalize`` is set).  An expert is a clamped gated unit without biases,
    W_down (g' * sigmoid(alpha g') * (u' + shift)), g' = min(W_gate h, limit), u' = clamp(W_up h, -limit, limit);
    ``spec.intermediate`` is an expert's inner width.  A shared expert (a feed-forward specification of its own under
    the option ``shared``) runs for every token and is added.

    With ``weight_input`` the weight multiplies the expert's input instead of its output, sum of expert_e(w_e h): the gate
    and up sums are scaled by w_e in float32 before the gating (W (w h) = w (W h)), and the sum over a token's experts
    takes each once.  With ``shared_gate`` (a tensor name behind the prefix, [1, width]) the shared expert's output is
    multiplied by sigmoid(<that row, h>), one number per token; the row rides in the router's product as one more row.

    With ``scoring`` "softmax" the scores are s = softmax(W_r h) over all experts instead of sigmoids, and ``renorm_eps`` is added
    to the chosen scores' sum before a renormalising division.

    Options (``spec.extra``): ``experts``, ``top``, ``router_scale``, ``renormalize``, ``scoring``, ``renorm_eps``, ``limit``, ``alpha``, ``shift``,
    ``weight_input``, ``shared`` (FeedForwardSpec or None), ``shared_prefix`` ("shared."), ``shared_gate``, ``tensor_names``
    by role "router", "gate", "up", "down" (an expert's tensors are ``<prefix>e<i>.<name>``).

    The router's choice stays on the device: the kernels take the chosen ids as an array, so a step of single tokens can
    be captured into a CUDA graph.  Steps of up to ``ops.MOE_GROUPED_MIN`` tokens (and the float32 engine) read each chosen
    expert's weights per token (``ops.moe_gate_up`` / ``ops.moe_down``: a warp per output element, fixed order of addition);
    larger steps in bfloat16 sort the (token, expert) pairs by expert on the device and run each expert's rows through
    tensor-core tiles, reading an expert's weights once (``ops.moe_grouped``)."""

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype: torch.dtype):
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.n_experts, self.top = int(spec.option("experts", 0)), int(spec.option("top", 0))
        if not (0 < self.top <= self.n_experts):
            raise ValueError(f"moe: top ({self.top}) must lie between 1 and the number of experts ({self.n_experts})")
        self.router_scale = float(spec.option("router_scale", 1.0))
        self.renormalize = bool(spec.option("renormalize", False))
        self.scoring = str(spec.option("scoring", "sigmoid"))
        if self.scoring not in ("sigmoid", "softmax"):
            raise ValueError(f"moe: scoring '{self.scoring}' is not one of sigmoid, softmax")
        self.renorm_eps = float(spec.option("renorm_eps", 0.0))
        limit = spec.option("limit", None)
        self.gating = (float(limit) if limit else 0.0, float(spec.option("alpha", 1.702)), float(spec.option("shift", 1.0)))
        names = dict(spec.option("tensor_names", ()))
        self.names = {r: names.get(r, d) for r, d in (("router", "router"), ("gate", "gate"), ("up", "up"), ("down", "down"))}
        self.weight_input = bool(spec.option("weight_input", False))
        shared = spec.option("shared", None)
        self.shared = self.shared_gate_name = None
        if shared is not None:
            self.shared = FEED_FORWARDS.get(shared.kind)(shared, prefix + str(spec.option("shared_prefix", "shared.")), dtype)
            if spec.option("shared_gate", None):
                self.shared_gate_name = prefix + str(spec.option("shared_gate"))
        self.router = self.w_gate_up = self.w_down = None

    def _expert(self, i: int, role: str) -> str:
        return f"{self.prefix}e{i}.{self.names[role]}"

    def weight_specs(self) -> List[WeightSpec]:
        s = self.spec
        specs = []
        for i in range(self.n_experts):
            specs += [WeightSpec(self._expert(i, "gate"), (s.intermediate, s.hidden)),
                      WeightSpec(self._expert(i, "up"), (s.intermediate, s.hidden)),
                      WeightSpec(self._expert(i, "down"), (s.hidden, s.intermediate))]
        specs.append(WeightSpec(self.prefix + self.names["router"], (self.n_experts, s.hidden), role="vector", init="normal"))
        if self.shared is not None:
            specs += self.shared.weight_specs()
        if self.shared_gate_name is not None:
            specs.append(WeightSpec(self.shared_gate_name, (1, s.hidden), role="vector", init="normal"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.n_experts
        self.w_gate_up = torch.stack([torch.cat([tensors[self._expert(i, "gate")], tensors[self._expert(i, "up")]], dim=0)
                                      for i in range(n)]).contiguous()                      # [E, 2 ff, width]
        self.w_down = torch.stack([tensors[self._expert(i, "down")] for i in range(n)]).contiguous()    # [E, width, ff]
        self.router = tensors[self.prefix + self.names["router"]].contiguous()
        if self.shared_gate_name is not None:           # one more row of the router's product: it competes for nothing
            self.router = torch.cat([self.router, tensors[self.shared_gate_name].reshape(1, -1)], dim=0).contiguous()
        if self.shared is not None:
            self.shared.load(tensors)

    def weight_bytes(self) -> int:
        """Bytes a step of one token reads: the router, the chosen experts, the shared expert."""
        per_expert = (self.w_gate_up.numel() + self.w_down.numel()) // self.n_experts * self.w_down.element_size()
        own = self.router.numel() * self.router.element_size() + self.top * per_expert
        return own + (self.shared.weight_bytes() if self.shared is not None else 0)

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        s, n, top = self.spec, ctx.n_tokens, self.top
        ids = ctx.scratch("moe.ids", (n, top), torch.int32)
        weights = ctx.scratch("moe.weights", (n, top), torch.float32)
        shared_scale = ctx.scratch("moe.shared_scale", (n, 1), torch.float32) if self.shared_gate_name is not None else None
        ops.moe_route(h, self.router, ids, weights, self.router_scale, self.renormalize, shared_scale,
                      softmax=self.scoring == "softmax", renorm_eps=self.renorm_eps)
        shared = self.shared.forward(ctx, h) if self.shared is not None else None
        act = ctx.scratch("moe.act", (n * top, s.intermediate))
        out = ctx.scratch("moe.out", (n, s.hidden))
        if n > ops.MOE_GROUPED_MIN and ops.moe_grouped_supported(h.dtype, s.hidden, s.intermediate, self.n_experts):
            y = ctx.scratch("moe.y", (n * top, s.hidden), torch.float32)
            work = ctx.scratch("moe.work", (ops.moe_grouped_workspace(n, top, self.n_experts),), torch.int32)
            gathered = ctx.scratch("moe.gathered", (n * top, s.hidden)) if ops.MOE_TCGEN05 else None
            ops.moe_grouped(h, self.w_gate_up, self.w_down, ids, weights, shared, act, y, out, work, self.gating, gathered,
                            weight_input=self.weight_input, add_scale=shared_scale)
            return out
        ops.moe_gate_up(h, self.w_gate_up, ids, act, self.gating, weights if self.weight_input else None)
        ops.moe_down(act, self.w_down, ids, None if self.weight_input else weights, shared, out, shared_scale)
        return out
