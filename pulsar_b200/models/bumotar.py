"""Bumotar: a pre-norm decoder whose ``config.json`` lists its layers one by one and walks a run of them several times.

A layer is  x += mixer(norm1(x)); x += ff(norm2(x))  (block kind ``prenorm``; the second sublayer only where ``mlp`` is
given).  Layers ``loop.start`` .. ``loop.stop - 1`` are walked ``loop.times`` times in a row with the same weights; every walk
has cache entries of its own and is opened by  x <- W_in [x ; x0] + step[t]  (``ModelSpec.walk``).  The typed configuration
below reads every key, checks it, and states the model as data for the generic decoder:

  * type "latent_attention" -> mixer kind ``latent_attention``: keys and values expanded per head from a normed latent of
    ``kv_rank`` numbers, one rotated key part of ``rot_dim`` for all heads (neighbouring pairs turn; frequencies blended along
    a ramp, cosines and sines multiplied by 0.1 ln(factor) + 1), a learned sink per head in the softmax's denominator, one
    sigmoid gate per head;
  * type "parallel" -> mixer kind ``side_by_side`` with two members whose outputs join as left_scale * left + right_scale *
    right: ``left`` is the general form of kind ``attention`` (grouped heads, weighted norm of q and k per head before the
    rotation, rotate-half layout with every frequency divided by one factor, capped scores, a sliding window, one added
    to the softmax's denominator, a sigmoid gate on every element of the heads), ``right`` is kind ``retention`` (a matrix
    per head that decays by a fixed factor; the keys are multiplied by dim^-1/2 behind the rotation);
  * ``mlp.kind`` "moe" -> feed-forward kind ``moe``: softmax router, ``router.top`` of ``router.experts`` silu-gated experts
    weighted by their scores divided by the chosen scores' sum + 1e-20, plus an optional shared expert (``swiglu``) that is
    multiplied by a sigmoid gate of its own (``shared.sg``);
  * ``mlp`` null -> the layer has its mixer only.

Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1|norm2``, ``l<i>.mix.*`` (``l<i>.mix.left.*`` /
``l<i>.mix.right.*`` for a parallel layer), ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import ConfigError, require
from ..config.registry import register_architecture
from ..config.specs import (BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec, NormSpec, PositionSpec, WalkSpec)

MAGNITUDE_SLOPE = 0.1           # cosines and sines of a ramped rotation are multiplied by 0.1 ln(factor) + 1
RENORM_EPS = 1e-20              # added to the chosen scores' sum before the division
ONE_IN_DENOMINATOR = 0.0        # the window attention's sink: exp(0) joins the softmax's denominator

_LATENT_NAMES = (("q", "q"), ("down", "dkv"), ("latent_norm", "dkv.norm"), ("up_k", "uk"), ("up_v", "uv"), ("gate", "g"),
                 ("o", "o"), ("sinks", "sink"))
_LEFT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm"), ("gate", "g"))
_RIGHT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"))
_FF_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))
_MOE_NAMES = (("router", "router"), ("gate", "gate"), ("up", "up"), ("down", "down"))


def _sub(raw: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


def _positive(raw: Dict[str, Any], key: str, where: str) -> int:
    try:
        value = require(raw, key, int)
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    if value <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be positive, found {value}")
    return value


def _number(raw: Dict[str, Any], key: str, where: str) -> float:
    try:
        return require(raw, key, float)
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None


def _check_rot(rot: Optional[Dict[str, Any]], within: int, where: str) -> None:
    """``rot`` = {base, dims[, scaling]}; scaling {factor} divides every frequency, {factor, original, fast, slow} ramps."""
    if rot is None:
        return
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where}rot must be an object")
    w = where + "rot."
    dims = _positive(rot, "dims", w)
    if dims % 2 or dims > within:
        raise ConfigError(f"config.json: {w}dims ({dims}) must be even and at most {within}")
    if not (_number(rot, "base", w) > 1.0):
        raise ConfigError(f"config.json: {w}base must be above 1")
    scaling = rot.get("scaling")
    if scaling is None:
        return
    if not isinstance(scaling, dict):
        raise ConfigError(f"config.json: {w}scaling must be an object")
    ws = w + "scaling."
    if not (_number(scaling, "factor", ws) > 0.0):
        raise ConfigError(f"config.json: {ws}factor must be positive")
    if any(k in scaling for k in ("original", "fast", "slow")):
        for key in ("original", "fast", "slow"):
            if not (_number(scaling, key, ws) > 0.0):
                raise ConfigError(f"config.json: {ws}{key} must be positive")


def _position(rot: Optional[Dict[str, Any]], head_dim: int) -> Optional[PositionSpec]:
    if rot is None:
        return None
    scaling = rot.get("scaling")
    divide = ramp = None
    magnitude = 1.0
    if scaling is not None:
        factor = float(scaling["factor"])
        if "original" in scaling:
            ramp = (factor, float(scaling["original"]), float(scaling["fast"]), float(scaling["slow"]))
            magnitude = MAGNITUDE_SLOPE * math.log(factor) + 1.0
        else:
            divide = factor
    return PositionSpec(kind="rope", head_dim=head_dim, rotary_dim=int(rot["dims"]), theta=float(rot["base"]), divide=divide,
                        ramp=ramp, magnitude=magnitude)


@dataclass(frozen=True)
class BumotarConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, checked
    loop: Optional[Tuple[int, int, int]]        # (start, stop, times) or None: every layer runs once, nothing is opened
    architecture: str = "Bumotar"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "BumotarConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        loop = None
        if raw.get("loop") is not None:
            lp = _sub(raw, "loop", "")
            try:
                start = require(lp, "start", int)
            except ConfigError as e:
                raise ConfigError(f"{e} (in loop.)") from None
            loop = (start, _positive(lp, "stop", "loop."), _positive(lp, "times", "loop."))
        cfg = cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""),
                  norm_eps=_number(_sub(raw, "norm", ""), "eps", "norm."),
                  logit_scale=_number(raw, "logit_scale", "") if raw.get("logit_scale") is not None else 1.0,
                  layers=tuple(copy.deepcopy(layers)), loop=loop)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0.0):
            raise ConfigError("config.json: norm.eps must be positive")
        if self.loop is not None:
            start, stop, _ = self.loop
            if not (0 <= start < stop <= len(self.layers)):
                raise ConfigError(f"config.json: loop.start ({start}) and loop.stop ({stop}) must bound a run of the "
                                  f"{len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            m = _sub(layer, "mixer", where)
            wm = where + "mixer."
            if kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _positive(m, key, wm)
                if not (_number(m, "scale", wm) > 0.0):
                    raise ConfigError(f"config.json: {wm}scale must be positive")
                _check_rot(_sub(m, "rot", wm), int(m["rot_dim"]), wm)
            elif kind == "parallel":
                left, right = _sub(m, "left", wm), _sub(m, "right", wm)
                wl, wr = wm + "left.", wm + "right."
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive(left, key, wl)
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config.json: {wl}heads ({left['heads']}) is not a multiple of kv_heads ({left['kv_heads']})")
                if not (_number(left, "scale", wl) > 0.0):
                    raise ConfigError(f"config.json: {wl}scale must be positive")
                if left.get("softcap") is not None and not (_number(left, "softcap", wl) > 0.0):
                    raise ConfigError(f"config.json: {wl}softcap must be positive")
                if left.get("mask") is not None:
                    _positive(_sub(left, "mask", wl), "size", wl + "mask.")
                _check_rot(left.get("rot"), int(left["dim"]), wl)
                for key in ("heads", "dim", "vdim"):
                    _positive(right, key, wr)
                decay = right.get("decay")
                if (not isinstance(decay, list) or len(decay) != right["heads"]
                        or any(isinstance(d, bool) or not isinstance(d, (int, float)) or not (0.0 <= d <= 1.0) for d in decay)):
                    raise ConfigError(f"config.json: {wr}decay must list one factor between 0 and 1 for each of the {right['heads']} heads")
                _check_rot(right.get("rot"), int(right["dim"]), wr)
                _number(m, "left_scale", wm)
                _number(m, "right_scale", wm)
            else:
                raise ConfigError(f"config.json: {where}type '{kind}' is not one of latent_attention, parallel")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            wf = where + "mlp."
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"config.json: {wf}kind must be 'moe' (or mlp null)")
            _positive(_sub(mlp, "expert", wf), "ff", wf + "expert.")
            router = _sub(mlp, "router", wf)
            experts, top = _positive(router, "experts", wf + "router."), _positive(router, "top", wf + "router.")
            if top > experts:
                raise ConfigError(f"config.json: {wf}router.top ({top}) exceeds router.experts ({experts})")
            if mlp.get("shared") is not None:
                _positive(_sub(mlp, "shared", wf), "ff", wf + "shared.")

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    # ------------------------------------------------------------------ the model as data
    def _mixer_spec(self, layer: Dict[str, Any]) -> MixerSpec:
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            return MixerSpec(kind="latent_attention", hidden=self.width, n_heads=int(m["heads"]), n_kv_heads=1,
                             head_dim=int(m["dim"]), v_head_dim=int(m["vdim"]), scale=float(m["scale"]), sinks=True,
                             position=_position(m["rot"], int(m["rot_dim"])), tensor_names=_LATENT_NAMES,
                             extra=(("kv_rank", int(m["kv_rank"])), ("rot_dim", int(m["rot_dim"])),
                                    ("latent_norm_eps", self.norm_eps), ("head_gate", True)))
        left, right = m["left"], m["right"]
        mask = left.get("mask")
        left_spec = MixerSpec(kind="attention", hidden=self.width, n_heads=int(left["heads"]), n_kv_heads=int(left["kv_heads"]),
                              head_dim=int(left["dim"]), v_head_dim=int(left["vdim"]), scale=float(left["scale"]),
                              window=None if mask is None else int(mask["size"]), qk_norm_eps=self.norm_eps, qk_norm_weight=True,
                              position=_position(left.get("rot"), int(left["dim"])),
                              softcap=None if left.get("softcap") is None else float(left["softcap"]),
                              fixed_sink=ONE_IN_DENOMINATOR, output_gate=True, tensor_names=_LEFT_NAMES)
        right_spec = MixerSpec(kind="retention", hidden=self.width, n_heads=int(right["heads"]), head_dim=int(right["dim"]),
                               v_head_dim=int(right["vdim"]), norm_eps=self.norm_eps,
                               position=_position(right.get("rot"), int(right["dim"])), tensor_names=_RIGHT_NAMES,
                               extra=(("decay", tuple(float(d) for d in right["decay"])), ("key_scale", int(right["dim"]) ** -0.5)))
        return MixerSpec(kind="side_by_side", hidden=self.width,
                         extra=(("members", (("left.", left_spec, float(m["left_scale"])),
                                             ("right.", right_spec, float(m["right_scale"])))),))

    def _feed_forward_spec(self, mlp: Optional[Dict[str, Any]]) -> Optional[FeedForwardSpec]:
        if mlp is None:
            return None
        expert, router, shared = mlp["expert"], mlp["router"], mlp.get("shared")
        shared_spec = None
        if shared is not None:
            shared_spec = FeedForwardSpec("swiglu", self.width, int(shared["ff"]), "silu", extra=(("tensor_names", _FF_NAMES),))
        # silu-gated experts: the gating g * sigmoid(g) * u, no clamp
        return FeedForwardSpec("moe", self.width, int(expert["ff"]), "silu",
                               extra=(("limit", None), ("alpha", 1.0), ("shift", 0.0), ("experts", int(router["experts"])),
                                      ("top", int(router["top"])), ("router_scale", 1.0), ("renormalize", True),
                                      ("scoring", "softmax"), ("renorm_eps", RENORM_EPS), ("weight_input", False),
                                      ("shared", shared_spec), ("shared_prefix", "shared."),
                                      ("shared_gate", "shared.sg" if shared is not None else None), ("tensor_names", _MOE_NAMES)))

    def walk_order(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, the walk it opens or None) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.width, self.norm_eps, suffix="")
        blocks: List[BlockSpec] = []
        for i, layer in enumerate(self.layers):
            ff = self._feed_forward_spec(layer.get("mlp"))
            blocks.append(BlockSpec(kind="prenorm", mixer=self._mixer_spec(layer), feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff is not None else None, weight_prefix=f"l{i}.",
                                    names=(("mixer", "mix."), ("feed_forward", "mlp."), ("mixer_norm", "norm1"),
                                           ("feed_forward_norm", "norm2"))))
        order: List[LayerCall] = []
        entry = 0
        for i, opens in self.walk_order():             # every run of a layer has cache entries of its own
            if self.layers[i]["type"] == "parallel":
                order.append(LayerCall(i, entry, members=(entry + 1,), opens=opens))
                entry += 2
            else:
                order.append(LayerCall(i, entry, opens=opens))
                entry += 1
        walk = None if self.loop is None else WalkSpec("loop.in", "loop.step", self.loop[2])
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, blocks=tuple(blocks),
                         run_order=tuple(order), final_norm=norm, embed_name="embed", final_norm_name="final.norm", head_name="head",
                         tie_word_embeddings=False, init_std=0.05, logit_scale=self.logit_scale, walk=walk)


@register_architecture("Bumotar")
def bumotar_config(raw: dict) -> BumotarConfig:
    return BumotarConfig.from_dict(raw)
