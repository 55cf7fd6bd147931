"""Plain, slow implementation of the Bumotar decoder: one function per mechanism, whole sequences only.

Written from the design's equations with dense tensors on the CPU: no cache, no pages, no portions, no batch.
Nothing here is imported by the product package and nothing of the product is imported here.  Notation: ``h``
[L, width] is a sublayer's input for the L tokens of one sequence, positions are 0 .. L-1, weights are stored
[out, in] and applied as ``h @ W.T``.

A layer is  x = x + mixer(N1(x));  x = x + ff(N2(x))  with N an RMS norm.  Layers ``loop.start`` .. ``loop.stop - 1``
are walked ``loop.times`` times with the same weights; each walk is opened by  x = W_in [x ; x0] + step[t]  with x0 the
embedding rows and t the walk's number.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---------------------------------------------------------------------------------------------- rotation
def base_frequencies(base: float, dims: int) -> List[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def divided_frequencies(base: float, dims: int, factor: float) -> List[float]:
    """Every frequency divided by one factor."""
    return [f / factor for f in base_frequencies(base, dims)]


def ramped_frequencies(base: float, dims: int, factor: float, original: float, fast: float, slow: float):
    """(frequencies, magnitude): pair i keeps its frequency below the ramp, has it divided by ``factor`` above it and a
    blend of both on it.  The ramp's ends are the (fractional) pair numbers whose wave makes ``fast`` and ``slow`` turns
    over ``original`` positions; cosines and sines are multiplied by the magnitude 0.1 ln(factor) + 1."""
    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(base_frequencies(base, dims)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def frequencies_of(rot: dict):
    """(frequencies, magnitude) of a ``rot`` entry: no scaling, one factor, or the ramp."""
    base, dims, scaling = float(rot["base"]), int(rot["dims"]), rot.get("scaling")
    if scaling is None:
        return base_frequencies(base, dims), 1.0
    if "original" in scaling:
        return ramped_frequencies(base, dims, float(scaling["factor"]), float(scaling["original"]), float(scaling["fast"]),
                                  float(scaling["slow"]))
    return divided_frequencies(base, dims, float(scaling["factor"])), 1.0


def _cos_sin(positions: torch.Tensor, freqs: List[float], magnitude: float, dtype):
    angle = positions.to(dtype)[:, None] * torch.tensor(freqs, dtype=dtype)[None, :]
    return torch.cos(angle) * magnitude, torch.sin(angle) * magnitude


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, freqs: List[float], magnitude: float = 1.0) -> torch.Tensor:
    """x [L, heads, D]: element i pairs with element i + n, n = len(freqs); elements from 2n on pass unchanged."""
    n = len(freqs)
    cos, sin = (t[:, None, :] for t in _cos_sin(positions, freqs, magnitude, x.dtype))
    u, v = x[..., :n], x[..., n:2 * n]
    out = x.clone()
    out[..., :n] = u * cos - v * sin
    out[..., n:2 * n] = v * cos + u * sin
    return out


def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, freqs: List[float], magnitude: float = 1.0) -> torch.Tensor:
    """x [L, heads, D]: element 2i pairs with element 2i + 1; elements from 2 len(freqs) on pass unchanged."""
    n = len(freqs)
    cos, sin = (t[:, None, :] for t in _cos_sin(positions, freqs, magnitude, x.dtype))
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = u * cos - v * sin
    out[..., 1:2 * n:2] = v * cos + u * sin
    return out


# ---------------------------------------------------------------------------------------------- mixers
def softmax_with_extra(scores: torch.Tensor, visible: torch.Tensor, extra: torch.Tensor) -> torch.Tensor:
    """scores [H, L, L], extra [H]: the denominator holds one more term per head, exp(extra[h]), without a value."""
    H, L, _ = scores.shape
    scores = scores.masked_fill(~visible, float("-inf"))
    col = extra.to(scores.dtype).view(H, 1, 1).expand(H, L, 1)
    return torch.softmax(torch.cat([scores, col], dim=-1), dim=-1)[..., :-1]


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Keys and values expanded from a normed latent; one rotated key part for all heads; a sink and a gate per head."""
    L = h.shape[0]
    H, D, R, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(L)
    freqs, magnitude = frequencies_of(m["rot"])
    q = (h @ w["q"].T).view(L, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_neighbours(q[..., D:], pos, freqs, magnitude)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :C], w["dkv.norm"], eps)
    k_rot = rotate_neighbours(down[:, None, C:], pos, freqs, magnitude)[:, 0]              # [L, R]
    k_plain = (c @ w["uk"].T).view(L, H, D)
    value = (c @ w["uv"].T).view(L, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * float(m["scale"])
    causal = torch.arange(L)[None, :] <= torch.arange(L)[:, None]
    p = softmax_with_extra(scores, causal[None], w["sink"])
    heads = torch.einsum("hij,jhv->ihv", p, value)
    heads = heads * torch.sigmoid(h @ w["g"].T)[:, :, None]
    return heads.reshape(L, H * V) @ w["o"].T


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Grouped heads, q and k normed per head before the rotation, capped scores, a window, one added to the softmax's
    denominator, a gate on every element of the heads."""
    L = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(L)
    q = rms_norm((h @ w["q"].T).view(L, H, D), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).view(L, G, D), w["k.norm"], eps)
    v = (h @ w["v"].T).view(L, G, V)
    if m.get("rot") is not None:
        freqs, magnitude = frequencies_of(m["rot"])
        q, k = rotate_halves(q, pos, freqs, magnitude), rotate_halves(k, pos, freqs, magnitude)
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    cap = m.get("softcap")
    if cap:
        scores = float(cap) * torch.tanh(scores / float(cap))
    i, j = torch.arange(L)[:, None], torch.arange(L)[None, :]
    visible = j <= i
    if m.get("mask") is not None:
        visible = visible & (i - j < int(m["mask"]["size"]))
    p = softmax_with_extra(scores, visible[None], torch.zeros(H))
    heads = torch.einsum("hij,jhv->ihv", p, v).reshape(L, H * V)
    return (heads * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def retention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, cancellations: Optional[list] = None) -> torch.Tensor:
    """Per head a matrix S that decays by a fixed factor and takes k v^T at every token; read with q; no softmax.
    ``cancellations`` receives, per token, how much of S^T q is left after cancellation (the least over the heads of
    rms(S^T q) / rms(|S|^T |q|)): the division by the root mean square magnifies rounding where little is left."""
    L = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(L)
    q, k, v = (h @ w["q"].T).view(L, H, D), (h @ w["k"].T).view(L, H, D), (h @ w["v"].T).view(L, H, V)
    if m.get("rot") is not None:
        freqs, magnitude = frequencies_of(m["rot"])
        q, k = rotate_halves(q, pos, freqs, magnitude), rotate_halves(k, pos, freqs, magnitude)
    k = k * D ** -0.5
    decay = torch.tensor([float(d) for d in m["decay"]], dtype=h.dtype)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.zeros(L, H, V, dtype=h.dtype)
    left_over = torch.zeros(L, dtype=h.dtype)
    for t in range(L):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
        spread = torch.einsum("hdv,hd->hv", S.abs(), q[t].abs())
        left_over[t] = ((out[t] ** 2).mean(-1).sqrt() / (spread ** 2).mean(-1).sqrt().clamp_min(1e-30)).min()
    if cancellations is not None:
        cancellations.append(left_over)
    out = rms_norm(out, None, eps).reshape(L, H * V)
    g = h @ w["g"].T
    return (out * g * torch.sigmoid(g)) @ w["o"].T


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {n[len(prefix):]: t for n, t in weights.items() if n.startswith(prefix)}


def side_by_side(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, cancellations: Optional[list] = None) -> torch.Tensor:
    left = window_attention(h, sub(w, "left."), m["left"], eps)
    right = retention(h, sub(w, "right."), m["right"], eps, cancellations)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---------------------------------------------------------------------------------------------- feed-forward
def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    g = h @ gate.T
    return (g * torch.sigmoid(g) * (h @ up.T)) @ down.T


def routed(h: torch.Tensor, router: torch.Tensor, top: int):
    """(chosen experts [L, top], weights [L, top]): softmax over all experts, the ``top`` largest, divided by their sum."""
    s = torch.softmax(h @ router.T, dim=-1)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(dim=-1, keepdim=True) + 1e-20)


def route_margins(h: torch.Tensor, router: torch.Tensor, top: int) -> torch.Tensor:
    """[L]: distance between the last chosen and the first rejected logit, relative to the largest magnitude."""
    z = h @ router.T
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    ordered = torch.sort(z, dim=-1, descending=True).values
    return (ordered[:, top - 1] - ordered[:, top]) / z.abs().max(dim=-1).values.clamp_min(1e-30)


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict, margins: Optional[list] = None) -> torch.Tensor:
    top = int(mlp["router"]["top"])
    idx, weight = routed(h, w["router"], top)
    if margins is not None:
        margins.append(route_margins(h, w["router"], top))
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for c in range(top):
            x = int(idx[t, c])
            out[t] += weight[t, c] * expert(h[t:t + 1], w[f"e{x}.gate"], w[f"e{x}.up"], w[f"e{x}.down"])[0]
    if mlp.get("shared") is not None:
        out = out + expert(h, w["shared.gate"], w["shared.up"], w["shared.down"]) * torch.sigmoid(h @ w["shared.sg"].T)
    return out


# ---------------------------------------------------------------------------------------------- the model
def open_walk(x: torch.Tensor, x0: torch.Tensor, w_in: torch.Tensor, step_row: torch.Tensor) -> torch.Tensor:
    return torch.cat([x, x0], dim=-1) @ w_in.T + step_row


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], spec: dict, eps: float, margins: Optional[list] = None,
          cancellations: Optional[list] = None) -> torch.Tensor:
    if spec["type"] == "parallel":
        x = x + side_by_side(rms_norm(x, w["norm1"], eps), sub(w, "mix."), spec["mixer"], eps, cancellations)
    else:
        x = x + latent_attention(rms_norm(x, w["norm1"], eps), sub(w, "mix."), spec["mixer"], eps)
    if spec.get("mlp") is not None:
        x = x + moe_ff(rms_norm(x, w["norm2"], eps), sub(w, "mlp."), spec["mlp"], margins)
    return x


def walk_order(cfg: dict):
    """[(layer, walk number or None, opens a walk)] in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if loop is None:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None, False) for i in range(start)]
    for t in range(times):
        order += [(i, t, i == start) for i in range(start, stop)]
    return order + [(i, None, False) for i in range(stop, n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            streams: Optional[list] = None, margins: Optional[list] = None, cancellations: Optional[list] = None) -> torch.Tensor:
    """Logits [L, vocab] of one whole sequence.  ``streams`` receives the stream after every layer that ran; ``margins``
    receives per-token margins of every routed layer (``route_margins``: a small one marks a token at which rounding to 16
    bits may choose other experts), ``cancellations`` what cancellation leaves of every retention's output (``retention``: a
    small one marks a token at which rounding is magnified)."""
    w = {n: t.to(dtype) for n, t in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"][torch.tensor(list(tokens))]
    x = x0
    for i, t, opens in walk_order(cfg):
        if opens:
            x = open_walk(x, x0, w["loop.in"], w["loop.step"][t])
        x = layer(x, sub(w, f"l{i}."), cfg["layers"][i], eps, margins, cancellations)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T * float(cfg.get("logit_scale", 1.0))
