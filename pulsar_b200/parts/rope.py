"""Rotary position encoding from an explicit array of positions."""
from __future__ import annotations

import math
from typing import Tuple

import torch

from .. import ops
from ..config.registry import POSITIONS
from ..config.specs import PositionSpec
from .base import PositionEncoding, StepContext


@POSITIONS.register("rope")
class RotaryEmbedding(PositionEncoding):
    """cos/sin of p_t * theta^(-2j/rotary_dim) for the tokens of a step, computed once per
    step and shared by every layer with an equal specification.  The frequency table is
    float64 and carries quadrants per position, as the reference's does
    (pulsar-core/inc/pulsar/rope.hpp:52-69): its relative error is scaled by the position."""

    def __init__(self, spec: PositionSpec):
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and within head_dim {spec.head_dim}")
        if spec.scaling is not None:
            factor, low, high, original = spec.scaling
            if not (factor > 0.0 and original > 0.0 and high > low > 0.0):
                raise ValueError(f"rotary scaling {spec.scaling}: factor and original must be positive and high > low > 0")
        if spec.divide is not None and not (spec.divide > 0.0):
            raise ValueError(f"rotary frequencies cannot be divided by {spec.divide}")
        if spec.ramp is not None:
            factor, original, fast, slow = spec.ramp
            if not (factor > 0.0 and original > 0.0 and fast > 0.0 and slow > 0.0 and spec.theta > 1.0):
                raise ValueError(f"rotary ramp {spec.ramp}: factor, original, fast and slow must be positive and theta above 1")
        self.spec = spec
        self._table = {}
        self._ramp_ends = None
        if spec.ramp is not None:
            factor, original, fast, slow = spec.ramp
            dims = spec.rotary_dim

            def pair_of(turns: float) -> float:
                return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.theta))
            self._ramp_ends = (max(math.floor(pair_of(fast)), 0), min(math.ceil(pair_of(slow)), dims - 1))

    def frequency(self, j: int) -> float:
        """Radians per position of pair j: theta^(-2j / rotary_dim), rescaled by its wavelength where the
        specification says so (``PositionSpec.scaling``), divided by one number (``divide``) or blended along a ramp over the
        pair numbers (``ramp``)."""
        f = self.spec.theta ** (-2.0 * j / self.spec.rotary_dim)
        if self.spec.divide is not None:
            f = f / self.spec.divide
        if self._ramp_ends is not None:
            lo, hi = self._ramp_ends
            ramp = min(max((j - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f = f / self.spec.ramp[0] * ramp + f * (1.0 - ramp)
        if self.spec.scaling is None:
            return f
        factor, low, high, original = self.spec.scaling
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            return f
        if wavelength > original / low:
            return f / factor
        blend = (original / wavelength - low) / (high - low)
        return (1.0 - blend) * f / factor + blend * f

    def quadrants_per_position(self, device) -> torch.Tensor:
        t = self._table.get(device)
        if t is None:
            half = self.spec.rotary_dim // 2
            values = [self.frequency(j) * (2.0 / math.pi) for j in range(half)]
            t = torch.tensor(values, dtype=torch.float64).to(device)
            self._table[device] = t
        return t

    def tables(self, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        key = ("rope", self.spec)
        got = ctx.shared.get(key)
        if got is None:
            half = self.spec.rotary_dim // 2
            tag = f"rope.{self.spec.rotary_dim}.{self.spec.theta}.{self.spec.scaling}.{self.spec.divide}.{self.spec.ramp}.{self.spec.magnitude}"
            cos = ctx.scratch(tag + ".cos", (ctx.n_tokens, half), torch.float32)
            sin = ctx.scratch(tag + ".sin", (ctx.n_tokens, half), torch.float32)
            ops.rope_table(ctx.positions, self.quadrants_per_position(ctx.device), cos, sin, self.spec.magnitude)
            got = ctx.shared[key] = (cos, sin)
        return got
