"""Megusun: a decoder whose ``config.json`` lists its layers one by one; a layer's two sublayers read one norm side by side.

A layer is  h = norm1(x); x += m * (mixer(shift(h)) + ff(h)): one RMS norm whose weight is a single number, a blend of
each token's h with the h of the token before it in front of the mixer (``l<i>.shift``), and the sublayers' sum joins the
stream multiplied by ``residual_mult`` (block kind ``parallel``).  The typed configuration below reads every key, checks
it, and states the model as data for the generic decoder:

  * type "attention" -> the differential form of mixer kind ``attention``: grouped heads without rotation, two softmax maps
    per head over the same values, subtracted with a learned weight (constant ``diff``), normed per head and scaled by
    1 - diff; queries grow with the logarithm of their position (``q_temp``); causal, all keys visible;
  * type "mingru" -> mixer kind ``min_gru`` (``mixer.width`` channels);
  * ``mlp.kind`` "dense" -> feed-forward kind ``mlp`` with the erf gelu;
  * ``mlp.kind`` "moe" -> feed-forward kind ``moe``: sigmoid router, ``router.top`` of ``router.experts`` silu-gated experts,
    each reading the token multiplied by its score (not renormalised), plus an optional shared expert (``swiglu``) that
    is multiplied by a sigmoid gate of its own (``shared.sg``);
  * ``mlp`` null -> the layer has its mixer only.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import ConfigError, require
from ..config.registry import register_architecture
from ..config.specs import BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec, NormSpec

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("lq1", "lq1"), ("lk1", "lk1"), ("lq2", "lq2"), ("lk2", "lk2"))
_GRU_NAMES = (("z", "z"), ("z_bias", "z.b"), ("x", "x"), ("x_bias", "x.b"), ("g", "g"), ("o", "o"))
_MLP_NAMES = (("up", "up"), ("down", "down"))
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


@dataclass(frozen=True)
class MegusunConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, checked
    architecture: str = "Megusun"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MegusunConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        cfg = cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""),
                  norm_eps=_number(_sub(raw, "norm", ""), "eps", "norm."), residual_mult=_number(raw, "residual_mult", ""),
                  layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0.0):
            raise ConfigError("config.json: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            m = _sub(layer, "mixer", where)
            wm = where + "mixer."
            if kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive(m, key, wm)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {wm}heads ({m['heads']}) is not a multiple of kv_heads ({m['kv_heads']})")
                if not (_number(m, "scale", wm) > 0.0):
                    raise ConfigError(f"config.json: {wm}scale must be positive")
                _number(m, "diff", wm)
                if m.get("q_temp") is not None:
                    temp = _sub(m, "q_temp", wm)
                    _number(temp, "coef", wm + "q_temp.")
                    _positive(temp, "every", wm + "q_temp.")
            elif kind == "mingru":
                _positive(m, "width", wm)
            else:
                raise ConfigError(f"config.json: {where}type '{kind}' is not one of attention, mingru")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            wf = where + "mlp."
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config.json: {wf}kind must be 'dense' or 'moe' (or mlp null)")
            if mlp["kind"] == "dense":
                _positive(mlp, "ff", wf)
                continue
            _positive(_sub(mlp, "expert", wf), "ff", wf + "expert.")
            router = _sub(mlp, "router", wf)
            experts, top = _positive(router, "experts", wf + "router."), _positive(router, "top", wf + "router.")
            if top > experts:
                raise ConfigError(f"config.json: {wf}router.top ({top}) exceeds router.experts ({experts})")
            if mlp.get("shared") is not None:
                _positive(_sub(mlp, "shared", wf), "ff", wf + "shared.")

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "layers": copy.deepcopy(list(self.layers))}

    # ------------------------------------------------------------------ the model as data
    def _mixer_spec(self, layer: Dict[str, Any]) -> MixerSpec:
        m = layer["mixer"]
        if layer["type"] == "mingru":
            return MixerSpec(kind="min_gru", hidden=self.width, tensor_names=_GRU_NAMES, extra=(("width", int(m["width"])),))
        temp = m.get("q_temp")
        return MixerSpec(kind="attention", hidden=self.width, n_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]),
                         head_dim=int(m["dim"]), v_head_dim=int(m["vdim"]), scale=float(m["scale"]),
                         differential=float(m["diff"]), norm_eps=self.norm_eps,
                         q_temperature=None if temp is None else (float(temp["coef"]), int(temp["every"])),
                         tensor_names=_ATTENTION_NAMES)

    def _feed_forward_spec(self, mlp: Optional[Dict[str, Any]]) -> Optional[FeedForwardSpec]:
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return FeedForwardSpec("mlp", self.width, int(mlp["ff"]), "gelu", extra=(("tensor_names", _MLP_NAMES),))
        expert, router, shared = mlp["expert"], mlp["router"], mlp.get("shared")
        shared_spec = None
        if shared is not None:
            shared_spec = FeedForwardSpec("swiglu", self.width, int(shared["ff"]), "silu", extra=(("tensor_names", _FF_NAMES),))
        # silu-gated experts: the gating g * sigmoid(g) * u, no clamp
        return FeedForwardSpec("moe", self.width, int(expert["ff"]), "silu",
                               extra=(("limit", None), ("alpha", 1.0), ("shift", 0.0), ("experts", int(router["experts"])),
                                      ("top", int(router["top"])), ("router_scale", 1.0), ("renormalize", False),
                                      ("weight_input", True), ("shared", shared_spec), ("shared_prefix", "shared."),
                                      ("shared_gate", "shared.sg" if shared is not None else None), ("tensor_names", _MOE_NAMES)))

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.width, self.norm_eps, suffix="", scalar=True)
        blocks: List[BlockSpec] = []
        order: List[LayerCall] = []
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            blocks.append(BlockSpec(
                kind="parallel", mixer=self._mixer_spec(layer), feed_forward=self._feed_forward_spec(layer.get("mlp")),
                mixer_norm=norm, feed_forward_norm=None, weight_prefix=f"l{i}.",
                names=(("mixer", "mix."), ("feed_forward", "mlp."), ("mixer_norm", "norm1"), ("shift", "shift")),
                residual_multiplier=self.residual_mult, token_shift=True))
            order.append(LayerCall(i, i, state=n + i))       # the mixer's cache entry, and the block's own kept row
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, blocks=tuple(blocks),
                         run_order=tuple(order), final_norm=norm, embed_name="embed", final_norm_name="final.norm", head_name="head",
                         tie_word_embeddings=False, init_std=0.05)


@register_architecture("Megusun")
def megusun_config(raw: dict) -> MegusunConfig:
    return MegusunConfig.from_dict(raw)
