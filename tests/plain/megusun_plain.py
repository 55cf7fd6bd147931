"""Plain, slow implementation of the Megusun decoder: one function per mechanism, whole sequences only.

Written from the design's equations with dense tensors on the CPU: no cache, no pages, no
portions, no batch.  Nothing here is imported by the product package and nothing of the product is
imported here.  Notation: ``h`` [L, width] is a layer's normed input for the L tokens of one
sequence, positions are 0 .. L-1, weights are stored [out, in] and applied as ``h @ W.T``.

A layer is  x = x + m * (mixer(shift(h)) + ff(h)),  h = N(x),  with N an RMS norm that has a single
learned number, m the model's residual multiplier, and shift a per-coordinate blend of a token's h
with the h of the token before it.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def scalar_rms_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * g, g one number for all coordinates."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * g.reshape(())


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """h_t + (h_(t-1) - h_t) * mix, element by element; the token before the first one is zero."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (before - h) * mix


def query_temperature(L: int, coef: float, every: int, dtype) -> torch.Tensor:
    """[L]: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(L, dtype=torch.int64)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype))


def difference_weight(w: Dict[str, torch.Tensor], diff: float) -> torch.Tensor:
    """exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff: one number for the layer."""
    return torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff


def differential_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values; their outputs are subtracted, normed and scaled."""
    L = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    q = (h @ w["q"].T).view(L, H, 2, D)
    k = (h @ w["k"].T).view(L, G, 2, D)
    v = (h @ w["v"].T).view(L, G, V)
    temp = m.get("q_temp")
    if temp is not None:
        q = q * query_temperature(L, float(temp["coef"]), int(temp["every"]), h.dtype)[:, None, None, None]
    lam = difference_weight(w, diff).to(h.dtype)
    causal = torch.arange(L)[None, :] <= torch.arange(L)[:, None]
    heads = []
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            s = (q[:, head, which] @ k[:, g, which].T) * float(m["scale"])
            p = torch.softmax(s.masked_fill(~causal, float("-inf")), dim=-1)
            maps.append(p @ v[:, g])
        o = maps[0] - lam * maps[1]
        heads.append(unit_rms(o, eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1) @ w["o"].T


def min_gru(h: torch.Tensor, w: Dict[str, torch.Tensor], state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """S_t = (1 - z_t) S_(t-1) + z_t c_t, token by token; the gates read the current token only."""
    z = torch.sigmoid(h @ w["z"].T + w["z.b"])
    u = h @ w["x"].T + w["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = torch.nn.functional.silu(h @ w["g"].T)
    s = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state.clone()
    out = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        out.append(s * gate[t])
    return torch.stack(out) @ w["o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    a = h @ w["up"].T
    return (0.5 * a * (1.0 + torch.erf(a / math.sqrt(2.0)))) @ w["down"].T


def gated_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return (torch.nn.functional.silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def router_choice(h: torch.Tensor, router: torch.Tensor, top: int):
    """(ids [L, top], scores [L, top]): the ``top`` largest sigmoid scores, not renormalised; ties go to the lower index."""
    s = torch.sigmoid(h @ router.T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def choice_margins(h: torch.Tensor, router: torch.Tensor, top: int) -> torch.Tensor:
    """[L]: distance between the logits of the last chosen and the first rejected expert, relative to the largest logit's
    magnitude (infinite where every expert is chosen).  A small margin is a close call that rounding may decide otherwise."""
    z = h @ router.T
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    ordered = torch.sort(z, dim=-1, descending=True).values
    return (ordered[:, top - 1] - ordered[:, top]) / z.abs().max(dim=-1).values.clamp_min(1e-30)


def mixture_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict, margins: Optional[list] = None) -> torch.Tensor:
    """sum over the chosen experts of expert(score * h), plus sigmoid(<sg, h>) * shared(h)."""
    ids, scores = router_choice(h, w["router"], int(mlp["router"]["top"]))
    if margins is not None:
        margins.append(choice_margins(h, w["router"], int(mlp["router"]["top"])))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, sc in zip(ids[t].tolist(), scores[t]):
            out[t] += gated_expert((sc * h[t])[None], w, f"e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * gated_expert(h, w, "shared.")
    return out


def sub(weights: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {n[len(prefix):]: t.to(dtype) for n, t in weights.items() if n.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            streams: Optional[list] = None, margins: Optional[list] = None) -> torch.Tensor:
    """Logits [L, vocab] of one whole sequence.  ``streams``: a list that receives the residual stream behind every layer;
    ``margins``: a list that receives every routed layer's ``choice_margins``."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = weights["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = scalar_rms_norm(x, weights[p + "norm1"].to(dtype), eps)
        hs = token_shift(h, weights[p + "shift"].to(dtype))
        mix = sub(weights, p + "mix.", dtype)
        if layer["type"] == "attention":
            delta = differential_attention(hs, mix, layer["mixer"], eps)
        elif layer["type"] == "mingru":
            delta = min_gru(hs, mix)
        else:
            raise ValueError(f"layer type {layer['type']}")
        mlp = layer.get("mlp")
        if mlp is not None:
            ffw = sub(weights, p + "mlp.", dtype)
            delta = delta + (dense_ff(h, ffw) if mlp["kind"] == "dense" else mixture_ff(h, ffw, mlp, margins))
        x = x + mult * delta
        if streams is not None:
            streams.append(x.clone())
    x = scalar_rms_norm(x, weights["final.norm"].to(dtype), eps)
    return x @ weights["head"].to(dtype).T
