"""Specifications of the parts a decoder is assembled from.

A specification is plain data: it carries every size and constant its part needs and
the ``kind`` under which the part's class is registered.  Architectures translate
their ``config.json`` into these; parts never see a ``config.json`` and never know
which model they are in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    kind: str            # "rmsnorm"
    size: int
    eps: float
    suffix: str = "weight"   # the weight's tensor name is the part's prefix + this ("" where the prefix is the whole name)
    scalar: bool = False     # the weight is a single number (a tensor without dimensions) for all coordinates


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # "rope"
    head_dim: int
    rotary_dim: int      # leading dims of each head that rotate (== head_dim for Qwen3)
    theta: float
    # (factor, low, high, original): frequencies are rescaled by wavelength l = 2 pi / f: kept where l < original / high,
    # divided by factor where l > original / low, and blended linearly in original / l between the two.  None: as they are.
    scaling: Optional[Tuple[float, float, float, float]] = None
    divide: Optional[float] = None   # every frequency is divided by this
    # (factor, original, fast, slow): pair i keeps its frequency below a ramp over the pair numbers, has it divided by factor
    # above it and a linear blend on it; the ramp runs from floor(pair(fast)) (at least 0) to ceil(pair(slow)) (at most
    # rotary_dim - 1), pair(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), and is at least 0.001 long.
    ramp: Optional[Tuple[float, float, float, float]] = None
    magnitude: float = 1.0           # cosines and sines are multiplied by this


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of a block.  ``kind`` "attention" is grouped-query attention over
    a paged key/value cache."""
    kind: str
    hidden: int
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0               # softmax scale
    window: Optional[int] = None     # None: all keys; w: keys p-w < j <= p
    qk_norm_eps: Optional[float] = None   # None: no per-head q/k norm
    position: Optional[PositionSpec] = None
    own_kv: bool = True              # False: attends over another layer's cache, has no k/v projection
    v_head_dim: int = 0              # width of a value head; 0: head_dim
    chunk: Optional[int] = None      # c: a query at p sees only keys j with floor(j / c) == floor(p / c), chunks counted from 0
    distance_bias: Optional[float] = None   # r: the score loses 2^(-r (h+1) / n_heads) * (p - j) for head h; None: no bias
    tensor_names: Tuple[Tuple[str, str], ...] = ()   # role ("q", "k", "v", "o", ...) -> name behind the prefix, where not the default
    keep_first: int = 0              # with a window or chunk: the first keep_first keys of a sequence stay visible all the same
    softcap: Optional[float] = None  # c: the scaled score becomes c * tanh(score / c)
    sinks: bool = False              # a learned number per head whose exponential joins the softmax's denominator (no key, no value)
    fixed_sink: Optional[float] = None   # the same with one given number for all heads instead of a learned tensor (0: one is added)
    bias: bool = False               # the q, k, v and o projections have biases (the weight's name + ".b" unless named by role)
    output_gate: bool = False        # the concatenated heads are multiplied by sigmoid(W_g h) before the output projection
    values_from_keys: bool = False   # no v projection: the value is the key as projected (before rotation and norm)
    qk_norm_weight: bool = True      # False: q and k are divided by their root mean square (qk_norm_eps) without a weight
    qk_norm_after_rotation: bool = False   # the per-head norm of q and k follows the rotation instead of preceding it
    # d: differential attention.  Every head has two score maps (its query and key rows hold [map 1 | map 2], head_dim
    # each) over the same values; with a1, a2 their outputs the head gives unit_rms(a1 - lambda a2) * (1 - d), lambda =
    # exp(<lq1, lk1>) - exp(<lq2, lk2>) + d from four learned vectors of head_dim (unit_rms: division by the root mean
    # square over the head's values with ``norm_eps`` inside the root).  None: one map.
    differential: Optional[float] = None
    norm_eps: float = 0.0            # eps of norms inside the mixer (the differential form's norm of a head's output)
    q_temperature: Optional[Tuple[float, int]] = None   # (coef, every): the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form parameters of other kinds

    def option(self, name, default=None):
        return dict(self.extra).get(name, default)

    def tensor_name(self, role: str, default: str) -> str:
        return dict(self.tensor_names).get(role, default)

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str            # "swiglu"
    hidden: int
    intermediate: int
    activation: str = "silu"
    extra: Tuple[Tuple[str, object], ...] = ()

    def option(self, name, default=None):
        return dict(self.extra).get(name, default)


@dataclass(frozen=True)
class BlockSpec:
    """Arrangement of one layer.  ``kind`` "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)).
    ``kind`` "sandwich": x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x))), the second sublayer only where
    ``feed_forward`` is given.  ``kind`` "parallel": h = norm1(x); x += m * (mixer(shift(h)) + ffn(h)) with m =
    ``residual_multiplier`` and shift the blend of neighbouring tokens where ``token_shift`` is set."""
    kind: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: Optional[NormSpec]          # None where the arrangement has no norm before the mixer ("postnorm")
    feed_forward_norm: Optional[NormSpec]
    weight_prefix: str                      # e.g. "model.layers.3."
    names: Tuple[Tuple[str, str], ...] = ()  # sub-prefixes: mixer, feed_forward, mixer_norm, feed_forward_norm (+ the post norms)
    mixer_post_norm: Optional[NormSpec] = None          # norm of the mixer's output before it joins the stream
    feed_forward_post_norm: Optional[NormSpec] = None   # the same behind the feed-forward
    residual_multiplier: float = 1.0                    # "parallel": what the sublayers' sum is multiplied by before it joins the stream
    # "parallel": the mixer reads h_t + (h_(t-1) - h_t) * s with s a learned vector (tensor name under ``names``["shift"]) and
    # h_(t-1) the norm's output for the token before (zeros before the first); the block keeps that row per sequence.
    token_shift: bool = False

    def sub_prefix(self, part: str) -> str:
        return self.weight_prefix + dict(self.names)[part]


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block ``block`` against cache entry ``cache``.
    A block may be named by several entries, and two entries may name one cache entry
    (the later one then reads what the earlier one wrote: its mixer has own_kv False)."""
    block: int
    cache: int
    state: Optional[int] = None      # a further cache entry, of kind "state", that belongs to the block itself (``Block.state_need``)
    members: Tuple[int, ...] = ()    # a composite mixer: the cache entries of its members behind the first (``Mixer.member_needs``)
    opens: Optional[int] = None      # t: this call opens walk number t over a run of layers (``ModelSpec.walk``)


@dataclass(frozen=True)
class WalkSpec:
    """A run of layers that is walked several times in a row with the same weights (the run order names the blocks once per
    walk, each time with cache entries of its own).  Right before the first layer of walk t (``LayerCall.opens`` = t; the
    first walk too) the stream becomes x <- W [x ; x0] + step[t]: x0 the embedding rows, W the tensor ``in_name``
    [width, 2 width] (the stream's columns first), step the tensor ``step_name`` [times, width]."""
    in_name: str
    step_name: str
    times: int


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    blocks: Tuple[BlockSpec, ...]
    run_order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: Optional[str] = "lm_head.weight"   # None: always tied
    tie_word_embeddings: Optional[bool] = None    # None: decided by the head tensor's presence
    init_std: float = 0.02
    eos_token_id: int = -1
    # What sits around the blocks.  Qwen3 dense uses none of it.
    embedding_multiplier: float = 1.0             # the embedding row is scaled by this before the first block
    logit_scale: float = 1.0                      # logits are scaled by this ...
    logit_softcap: Optional[float] = None         # ... and then capped: cap * tanh(logits / cap)
    position_axes: int = 1                        # axes of a token's position; axis 0 is its index in the sequence
    ignore: Tuple[str, ...] = ()                  # tensor-name patterns (fnmatch) that a folder may hold and nobody reads
    walk: Optional["WalkSpec"] = None             # a run of layers walked several times, and what opens each walk

    @property
    def n_cache_entries(self) -> int:
        if not self.run_order:
            return 0
        return 1 + max(max(call.cache, -1 if call.state is None else call.state, *call.members) for call in self.run_order)
