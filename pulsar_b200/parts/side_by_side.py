"""Two mixers side by side: both read the same input, their outputs join with a weight each."""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .. import ops
from ..cache.manager import CacheNeed
from ..config.registry import MIXERS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    """out = sum over the members of scale_i * member_i(h).  A member is any registered mixer with a specification of its
    own; member i's tensors stand under ``<prefix><member prefix i>``.  Each member keeps its own cache entry: the first
    one's is the layer call's ``cache``, the others' are the call's ``members`` in order (``member_needs``), and reach
    ``forward`` as ``cache.members``.  Members that can (``Mixer.output_float32``) hand over float32 rows, so that the weighted
    sum is rounded once.

    Options (``spec.extra``): ``members`` (a tuple of (member prefix, MixerSpec, scale))."""

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        listed = tuple(spec.option("members", ()) or ())
        if len(listed) < 2:
            raise ValueError("side_by_side: needs at least two members")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.members: List[Mixer] = []
        self.scales: List[float] = []
        for sub_prefix, sub_spec, scale in listed:
            if sub_spec.hidden != spec.hidden:
                raise ValueError("side_by_side: a member reads and writes the width of the whole")
            self.members.append(MIXERS.get(sub_spec.kind)(sub_spec, prefix + sub_prefix, dtype))
            self.members[-1].output_float32 = True
            self.scales.append(float(scale))

    @property
    def graph_safe(self) -> bool:
        return all(getattr(m, "graph_safe", True) for m in self.members)

    def weight_specs(self) -> List[WeightSpec]:
        return [w for m in self.members for w in m.weight_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for m in self.members:
            m.load(tensors)

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in self.members)

    def cache_need(self) -> CacheNeed:
        return self.members[0].cache_need()

    def member_needs(self) -> Tuple[CacheNeed, ...]:
        """What the members behind the first need, one cache entry each."""
        return tuple(m.cache_need() for m in self.members[1:])

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        views = [cache] + list(cache.members or ())
        if len(views) != len(self.members):
            raise ValueError(f"side_by_side: {len(self.members)} members but {len(views)} cache entries (LayerCall.members)")
        total = ctx.scratch("side.sum", (ctx.n_tokens, self.spec.hidden))
        if len(self.members) == 2 and type(self.members[0]) is not type(self.members[1]):
            # two parts of different kinds keep their outputs in buffers of their own: one kernel weighs and adds them
            first = self.members[0].forward(ctx, h, views[0])
            second = self.members[1].forward(ctx, h, views[1])
            if first.dtype == second.dtype:
                ops.scaled_sum(first, second, total, self.scales[0], self.scales[1])
                return total
            outputs = iter((first, second))
        else:
            outputs = None
        # members of one kind write to the same scratch buffer, and members may hand over rows of different dtypes: each
        # output is weighed into float32 rows and added to the running sum before the next member runs
        shape = (ctx.n_tokens, self.spec.hidden)
        running, part = ctx.scratch("side.running", shape, torch.float32), ctx.scratch("side.part", shape, torch.float32)
        for i, (member, view, scale) in enumerate(zip(self.members, views, self.scales)):
            out = next(outputs) if outputs is not None else member.forward(ctx, h, view)
            if i == 0:
                ops.scaled_sum(out, out, running, scale, 0.0)
            else:
                ops.scaled_sum(out, out, part, scale, 0.0)
                ops.scaled_sum(running, part, total if i + 1 == len(self.members) else running, 1.0, 1.0)
        return total
