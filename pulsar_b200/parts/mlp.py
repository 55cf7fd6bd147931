"""Dense gated feed-forward."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.registry import FEED_FORWARDS
from ..config.specs import FeedForwardSpec
from .base import FeedForward, StepContext, WeightSpec
from .norm import RMSNorm, accumulate_and_prepare


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """(silu(h Wg^T) * (h Wu^T)) Wd^T without bias (pulsar-core/src/model/qwen3.cpp:117-119).
    Gate and up are one fused product (rows: gate | up); the gating runs in float32 and
    rounds once.

    Options (``spec.extra``): ``tensor_names`` by role "gate", "up", "down"; ``bias`` True: the three projections have
    biases (a weight's name + ".b", or ".bias" in place of ".weight"), added in float32: gate and up inside the gating
    kernel, the down projection's (``output_bias``) here unless the block has set ``defer_output_bias`` because the
    kernel behind the sublayer takes it along."""

    output_bias = None
    defer_output_bias = False

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype: torch.dtype):
        if spec.activation != "silu":
            raise ValueError(f"swiglu: activation '{spec.activation}' is not implemented (only 'silu')")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        names = dict(spec.option("tensor_names", ()))
        self.names = {r: names.get(r, d) for r, d in (("gate", "gate_proj.weight"), ("up", "up_proj.weight"),
                                                      ("down", "down_proj.weight"))}
        self.bias = bool(spec.option("bias", False))
        self.w_gate_up = self.w_down = self.b_gate_up = None

    def _bias_name(self, role: str) -> str:
        weight = self.names[role]
        return weight[:-len(".weight")] + ".bias" if weight.endswith(".weight") else weight + ".b"

    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        specs = [WeightSpec(p + nm["gate"], (s.intermediate, s.hidden)),
                 WeightSpec(p + nm["up"], (s.intermediate, s.hidden)),
                 WeightSpec(p + nm["down"], (s.hidden, s.intermediate))]
        if self.bias:
            specs += [WeightSpec(p + self._bias_name("gate"), (s.intermediate,), role="vector", init="small"),
                      WeightSpec(p + self._bias_name("up"), (s.intermediate,), role="vector", init="small"),
                      WeightSpec(p + self._bias_name("down"), (s.hidden,), role="vector", init="small")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p, nm = self.prefix, self.names
        self.w_gate_up = torch.cat([tensors[p + nm["gate"]], tensors[p + nm["up"]]], dim=0).contiguous()
        self.w_down = tensors[p + nm["down"]]
        if self.bias:
            self.b_gate_up = torch.cat([tensors[p + self._bias_name("gate")], tensors[p + self._bias_name("up")]]).contiguous()
            self.output_bias = tensors[p + self._bias_name("down")]

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down, self.b_gate_up, self.output_bias)
                   if t is not None)

    def forward_normed(self, ctx: StepContext, residual: torch.Tensor, norm, next_norm=None) -> bool:
        s, n = self.spec, ctx.n_tokens
        if n > 16 or not isinstance(norm, RMSNorm) or self.dtype != torch.bfloat16 or self.bias:
            return False
        if not (ops.fused_projection_supported(n, self.w_gate_up, swiglu=True) and ops.fused_projection_supported(n, self.w_down)):
            return False
        act = ctx.scratch("mlp.act", (n, s.intermediate))
        prepared = ctx.prepared_norms.pop(id(norm), None) if ops.FUSED_NORM_MLP else None
        if prepared is None or not ops.linear_prenormed(prepared[0], prepared[1], norm.spec.eps, self.w_gate_up, act, swiglu=True):
            ops.gated_linear(ctx, norm.forward(ctx, residual, None), self.w_gate_up, act)
        ctx.prepared_norms.clear()              # the residual changes now
        if not accumulate_and_prepare(ctx, act, self.w_down, residual, next_norm):
            raise ops.KernelError("swiglu: the down projection refused sizes it had declared supported")
        return True

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        s, n = self.spec, ctx.n_tokens
        act = ctx.scratch("mlp.act", (n, s.intermediate))
        if self.bias:
            # float32 rows of the product, the biases added before anything is rounded
            gate_up = ctx.scratch("mlp.gate_up32", (n, 2 * s.intermediate), torch.float32)
            ops.linear(h, self.w_gate_up, gate_up)
            ops.glu_bias(gate_up, self.b_gate_up, act)
        else:
            ops.gated_linear(ctx, h, self.w_gate_up, act)
        out = ctx.scratch("mlp.out", (n, s.hidden))
        ops.linear(act, self.w_down, out)
        if self.output_bias is not None and not self.defer_output_bias:
            ops.add_bias(out, self.output_bias)
        return out


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """g = min(h Wg^T, limit), u = clamp(h Wu^T, -limit, limit); out = (g * sigmoid(alpha * g) * (u + 1)) Wd^T, without bias.
    Gate and up are one fused product (rows: gate | up); the gating runs in float32 and rounds once.
    Options (``spec.extra``): ``limit``, ``alpha``; tensor names by role "gate", "up", "down"."""

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype: torch.dtype):
        self.limit = float(spec.option("limit", 0.0))
        self.alpha = float(spec.option("alpha", 1.702))
        if not (self.limit > 0.0):
            raise ValueError("clamped_glu: the clamp's limit must be positive")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        names = dict(spec.option("tensor_names", ()))
        self.names = {r: names.get(r, d) for r, d in (("gate", "gate_proj.weight"), ("up", "up_proj.weight"),
                                                      ("down", "down_proj.weight"))}
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        return [WeightSpec(p + nm["gate"], (s.intermediate, s.hidden)),
                WeightSpec(p + nm["up"], (s.intermediate, s.hidden)),
                WeightSpec(p + nm["down"], (s.hidden, s.intermediate))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p, nm = self.prefix, self.names
        self.w_gate_up = torch.cat([tensors[p + nm["gate"]], tensors[p + nm["up"]]], dim=0).contiguous()
        self.w_down = tensors[p + nm["down"]]

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        s, n = self.spec, ctx.n_tokens
        act = ctx.scratch("mlp.act", (n, s.intermediate))
        ops.gated_linear(ctx, h, self.w_gate_up, act, gating=(self.limit, self.alpha, 1.0))     # the gating in the product's epilogue where it fuses
        out = ctx.scratch("mlp.out", (n, s.hidden))
        ops.linear(act, self.w_down, out)
        return out


@FEED_FORWARDS.register("mlp")
class ActivatedMLP(FeedForward):
    """act(h Wu^T) Wd^T without gate and without bias; ``spec.activation``: "gelu" (the erf form), "gelu_tanh", "silu" or
    "relu".  The up product leaves float32 rows, the activation runs in float32 and rounds once (``ops.activation``).
    Options (``spec.extra``): tensor names by role "up", "down"."""

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype: torch.dtype):
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"mlp: activation '{spec.activation}' is not one of {sorted(ops.ACTIVATIONS)}")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        names = dict(spec.option("tensor_names", ()))
        self.names = {r: names.get(r, d) for r, d in (("up", "up_proj.weight"), ("down", "down_proj.weight"))}
        self.w_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        return [WeightSpec(p + nm["up"], (s.intermediate, s.hidden)), WeightSpec(p + nm["down"], (s.hidden, s.intermediate))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = tensors[self.prefix + self.names["up"]], tensors[self.prefix + self.names["down"]]

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        s, n = self.spec, ctx.n_tokens
        up = ctx.scratch("mlp.up32", (n, s.intermediate), torch.float32)
        ops.linear(h, self.w_up, up)
        act = ctx.scratch("mlp.act", (n, s.intermediate))
        ops.activation(up, act, s.activation)
        out = ctx.scratch("mlp.out", (n, s.hidden))
        ops.linear(act, self.w_down, out)
        return out
