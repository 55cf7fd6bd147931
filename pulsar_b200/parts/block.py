"""Arrangements of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheNeed
from ..config.registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from ..config.specs import BlockSpec
from .. import ops
from .base import Block, CacheView, StepContext, WeightSpec
from .norm import RMSNorm


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x))
    (pulsar-core/src/model/qwen3.cpp:77-121).  The additions happen inside the norm
    kernels, in float32, on the float32 residual stream.  A block without a feed-forward has
    the first sublayer only and leaves the mixer's contribution pending."""

    def __init__(self, spec: BlockSpec, dtype: torch.dtype):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, spec.sub_prefix("mixer_norm"), dtype, "norm.mixer")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.sub_prefix("mixer"), dtype)
        self.feed_forward_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            if spec.feed_forward_norm is None:
                raise ValueError("a prenorm block with a feed-forward needs the norm before it")
            self.feed_forward_norm = NORMS.get(spec.feed_forward_norm.kind)(
                spec.feed_forward_norm, spec.sub_prefix("feed_forward_norm"), dtype, "norm.ffn")
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, spec.sub_prefix("feed_forward"), dtype)
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None)

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts for w in p.weight_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts)

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                cache: CacheView) -> Optional[torch.Tensor]:
        # With nothing pending, a part may take the norm before it and the addition behind it into its own products
        # (steps of a few tokens); otherwise the norm kernel adds what is pending and normalises.
        after_mixer = self.feed_forward_norm if self.feed_forward is not None else ctx.next_norm
        if delta is not None or not self.mixer.forward_normed(ctx, residual, self.mixer_norm, cache, after_mixer):
            ctx.prepared_norms.clear()
            h = self.mixer_norm.forward(ctx, residual, delta)
            delta = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is None:
            return delta
        if delta is None and self.feed_forward.forward_normed(ctx, residual, self.feed_forward_norm, ctx.next_norm):
            return None
        ctx.prepared_norms.clear()
        h = self.feed_forward_norm.forward(ctx, residual, delta)
        return self.feed_forward.forward(ctx, h)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """x += post1(mixer(norm1(x))); x += post2(feed_forward(norm2(x))): every sublayer is normed before and behind.  A block
    without a feed-forward has the first sublayer only.  All four norms are RMS norms.

    The stream is complete when the block returns (nothing is left pending).  One kernel stands between two sublayers:
    it norms the sublayer's output, adds it to the float32 stream and applies the next sublayer's first norm
    (``ops.post_norm_add``); where the next block's first norm is known (``ctx.next_norm``) the block's last such kernel
    applies it and leaves the result in ``ctx.normed`` for whoever comes next."""

    def __init__(self, spec: BlockSpec, dtype: torch.dtype):
        self.spec = spec

        def norm(norm_spec, part, tag):
            made = NORMS.get(norm_spec.kind)(norm_spec, spec.sub_prefix(part), dtype, tag)
            if not isinstance(made, RMSNorm):
                raise ValueError(f"a sandwich block's norms are RMS norms, '{norm_spec.kind}' is not")
            return made
        if spec.mixer_post_norm is None:
            raise ValueError("a sandwich block needs a norm behind its mixer")
        self.mixer_norm = norm(spec.mixer_norm, "mixer_norm", "norm.mixer")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.sub_prefix("mixer"), dtype)
        self.mixer_post_norm = norm(spec.mixer_post_norm, "mixer_post_norm", "norm.mixer.post")
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            if spec.feed_forward_norm is None or spec.feed_forward_post_norm is None:
                raise ValueError("a sandwich block with a feed-forward needs the norms before and behind it")
            self.feed_forward_norm = norm(spec.feed_forward_norm, "feed_forward_norm", "norm.ffn")
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, spec.sub_prefix("feed_forward"), dtype)
            self.feed_forward_post_norm = norm(spec.feed_forward_post_norm, "feed_forward_post_norm", "norm.ffn.post")
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm,
                                       self.feed_forward, self.feed_forward_post_norm) if p is not None)

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts for w in p.weight_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts)

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                cache: CacheView) -> Optional[torch.Tensor]:
        ctx.prepared_norms.clear()
        h = ctx.normed.pop(id(self.mixer_norm), None) if delta is None else None
        ctx.normed.clear()
        if h is None:
            h = self.mixer_norm.forward(ctx, residual, delta)
        out = self.mixer.forward(ctx, h, cache)
        post = self.mixer_post_norm
        if self.feed_forward is not None:
            nxt = self.feed_forward_norm
            h = ctx.scratch(nxt.tag, residual.shape)
            ops.post_norm_add(residual, out, post.weight, post.spec.eps, nxt.weight, nxt.spec.eps, h)
            out = self.feed_forward.forward(ctx, h)
            post = self.feed_forward_post_norm
        nxt = ctx.next_norm
        if isinstance(nxt, RMSNorm) and nxt.spec.size == residual.shape[1]:
            h = ctx.scratch("norm.ahead", residual.shape)
            ops.post_norm_add(residual, out, post.weight, post.spec.eps, nxt.weight, nxt.spec.eps, h)
            ctx.normed[id(nxt)] = h
        else:
            ops.post_norm_add(residual, out, post.weight, post.spec.eps)
        return None


@BLOCKS.register("postnorm")
class PostNormBlock(Block):
    """x += post1(mixer(x)); x += post2(feed_forward(x)): the sublayers read the stream itself and only their outputs are
    normed (RMS norms; the specification's ``mixer_post_norm`` / ``feed_forward_post_norm``).  A block without a
    feed-forward has the first sublayer only.

    The stream is float32 and complete when the block returns.  One kernel stands behind every sublayer
    (``ops.post_norm_add_bias``): it adds the bias of the sublayer's last projection (where it has one and defers it),
    norms, adds into the stream and leaves the stream's rounding to the activation dtype for the sublayer that reads it
    next (``ctx.normed["stream"]``; a float32 engine reads the stream itself)."""

    def __init__(self, spec: BlockSpec, dtype: torch.dtype):
        self.spec, self.dtype = spec, dtype

        def norm(norm_spec, part, tag):
            made = NORMS.get(norm_spec.kind)(norm_spec, spec.sub_prefix(part), dtype, tag)
            if not isinstance(made, RMSNorm):
                raise ValueError(f"a postnorm block's norms are RMS norms, '{norm_spec.kind}' is not")
            return made
        if spec.mixer_post_norm is None:
            raise ValueError("a postnorm block needs a norm behind its mixer")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.sub_prefix("mixer"), dtype)
        self.mixer_post_norm = norm(spec.mixer_post_norm, "mixer_post_norm", "norm.mixer.post")
        self.feed_forward = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            if spec.feed_forward_post_norm is None:
                raise ValueError("a postnorm block with a feed-forward needs the norm behind it")
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, spec.sub_prefix("feed_forward"), dtype)
            self.feed_forward_post_norm = norm(spec.feed_forward_post_norm, "feed_forward_post_norm", "norm.ffn.post")
        for part in (self.mixer, self.feed_forward):
            if part is not None and hasattr(part, "defer_output_bias"):
                part.defer_output_bias = True          # the kernel behind the sublayer adds it
        self.parts = tuple(p for p in (self.mixer, self.mixer_post_norm, self.feed_forward, self.feed_forward_post_norm)
                           if p is not None)

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts for w in p.weight_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts)

    def _reader(self, ctx: StepContext, residual: torch.Tensor, fresh: bool) -> Optional[torch.Tensor]:
        """Where the kernel behind a sublayer leaves the stream for the next reader (None: the reader takes the float32
        stream itself); ``fresh`` also fills it from the stream as it stands."""
        if self.dtype == torch.float32:
            return None
        h = ctx.scratch("stream.rounded", residual.shape)
        if fresh:
            ops.post_norm_add_bias(residual, None, None, None, 0.0, h)
        return h

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                cache: CacheView) -> Optional[torch.Tensor]:
        ctx.prepared_norms.clear()
        if delta is not None:
            raise ValueError("a postnorm block follows blocks that leave the stream complete")
        h = ctx.normed.pop("stream", None)
        ctx.normed.clear()
        if self.dtype == torch.float32:
            h = residual
        elif h is None:
            h = self._reader(ctx, residual, fresh=True)
        out = self.mixer.forward(ctx, h, cache)
        post = self.mixer_post_norm
        bias = getattr(self.mixer, "output_bias", None)
        if self.feed_forward is not None:
            nxt = self._reader(ctx, residual, fresh=False)
            ops.post_norm_add_bias(residual, out, bias, post.weight, post.spec.eps, nxt)
            out = self.feed_forward.forward(ctx, residual if nxt is None else nxt)
            post = self.feed_forward_post_norm
            bias = getattr(self.feed_forward, "output_bias", None)
        nxt = self._reader(ctx, residual, fresh=False) if ctx.has_following else None
        ops.post_norm_add_bias(residual, out, bias, post.weight, post.spec.eps, nxt)
        if nxt is not None:
            ctx.normed["stream"] = nxt
        return None


# The closing kernel of a parallel block also opens the parallel block that follows (its norm and token shift): one kernel
# at a layer boundary instead of two.  PULSAR_PARALLEL_FUSED=0 keeps them apart.
PARALLEL_FUSED = os.environ.get("PULSAR_PARALLEL_FUSED", "1") != "0"


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """h = norm(x); x += m * (mixer(shift(h)) + feed_forward(h)): one norm, both sublayers read its output, their sum joins the
    float32 stream multiplied by ``residual_multiplier``.  A block without a feed-forward has the mixer only.

    With ``token_shift`` the mixer reads h_t + (h_(t-1) - h_t) * s instead, s a learned vector and h_(t-1) the norm's output
    for the token before in the same sequence as it was before this blend (zeros before the first token); the
    feed-forward reads h as it is.  The last h of a sequence is kept per sequence, in float32, in a state entry that the
    block declares itself (``state_need``) and receives as ``cache.block_state``.

    Two kernels frame the sublayers.  ``ops.norm_shift`` norms a row, blends it with the row above (or, for a portion's
    first token, with the kept row) and leaves the last token's h aside; ``ops.parallel_add`` adds the sublayers' sum into
    the stream and only then moves that h into the kept row, so that no reader of the old row comes too late.  Where the
    block that follows is a parallel block too, the closing kernel does its opening as well; it then writes the stream to
    a second buffer (a row's blend reads the row above as it stood) and hands that buffer on (``ctx.moved_residual``)."""

    def __init__(self, spec: BlockSpec, dtype: torch.dtype):
        self.spec, self.dtype = spec, dtype
        if spec.mixer_norm is None:
            raise ValueError("a parallel block needs its norm")
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, spec.sub_prefix("mixer_norm"), dtype, "norm.parallel")
        if not isinstance(self.mixer_norm, RMSNorm):
            raise ValueError(f"a parallel block's norm is an RMS norm, '{spec.mixer_norm.kind}' is not")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.sub_prefix("mixer"), dtype)
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, spec.sub_prefix("feed_forward"), dtype)
        self.multiplier = float(spec.residual_multiplier)
        self.width = spec.mixer_norm.size
        self.shift_name = spec.sub_prefix("shift") if spec.token_shift else None
        self.shift: Optional[torch.Tensor] = None
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward) if p is not None)

    def weight_specs(self) -> List[WeightSpec]:
        specs = [w for p in self.parts for w in p.weight_specs()]
        if self.shift_name is not None:
            specs.append(WeightSpec(self.shift_name, (self.width,), role="vector", init="unit"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load(tensors)
        if self.shift_name is not None:
            self.shift = tensors[self.shift_name]

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts) + (self.shift.numel() * 4 if self.shift is not None else 0)

    def state_need(self) -> Optional[CacheNeed]:
        return CacheNeed.state((self.width,), torch.float32) if self.shift_name is not None else None

    def _open(self, ctx: StepContext, residual: torch.Tensor, state: Optional[torch.Tensor], which: int):
        """(h, hs, pending) for the stream as it stands; ``which`` picks one of two buffers for the rows left aside."""
        n = residual.shape[0]
        norm = self.mixer_norm
        h = ctx.scratch("parallel.h", (n, self.width))
        if self.shift is None:
            ops.norm_shift(ctx, residual, norm.weight, norm.spec.eps, None, None, h, None, None)
            return h, h, None
        hs = ctx.scratch("parallel.hs", (n, self.width))
        pending = ctx.scratch(f"parallel.pending.{which}", (ctx.n_seqs, self.width), torch.float32)
        ops.norm_shift(ctx, residual, norm.weight, norm.spec.eps, self.shift, state, h, hs, pending)
        return h, hs, pending

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                cache: CacheView) -> Optional[torch.Tensor]:
        ctx.prepared_norms.clear()
        state = cache.block_state
        if self.shift is not None and state is None:
            raise ValueError("a parallel block with a token shift needs its state entry (LayerCall.state)")
        handed = ctx.normed.pop(("parallel", id(self)), None) if delta is None else None
        ctx.normed.clear()
        if handed is not None:
            h, hs, pending, which = handed
        else:
            if delta is not None:                        # a block of another kind left its contribution pending
                ops.parallel_add(ctx, residual, delta, None, 1.0)
            which = 0
            h, hs, pending = self._open(ctx, residual, state, which)
        a = self.mixer.forward(ctx, hs, cache)
        b = self.feed_forward.forward(ctx, h) if self.feed_forward is not None else None
        nxt = ctx.next_block
        if PARALLEL_FUSED and isinstance(nxt, ParallelBlock) and nxt.width == self.width:
            n = residual.shape[0]
            own = ctx.scratch("residual", residual.shape, torch.float32)
            out = ctx.scratch("residual.alt", residual.shape, torch.float32) if own.data_ptr() == residual.data_ptr() else own
            norm = nxt.mixer_norm
            h2 = ctx.scratch("parallel.h", (n, self.width))           # this block's h and hs have been read by now
            hs2 = pending2 = state2 = None
            if nxt.shift is not None:
                hs2 = ctx.scratch("parallel.hs", (n, self.width))
                pending2 = ctx.scratch(f"parallel.pending.{1 - which}", (ctx.n_seqs, self.width), torch.float32)
                state2 = ctx.cache(ctx.next_call.state).state
            ops.parallel_add(ctx, residual, a, b, self.multiplier, pending, state if pending is not None else None, out,
                             norm.weight, norm.spec.eps, nxt.shift, state2, pending2, h2, hs2)
            ctx.normed[("parallel", id(nxt))] = (h2, hs2 if hs2 is not None else h2, pending2, 1 - which)
            ctx.moved_residual = out
            return None
        ops.parallel_add(ctx, residual, a, b, self.multiplier, pending, state if pending is not None else None)
        return None
