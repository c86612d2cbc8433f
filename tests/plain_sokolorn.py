"""A plain, slow implementation of the Sokolorn decoder for the tests: whole sequences, float64, no cache, no
batching, one function per mechanism, nothing shared with the package.

    x = table[token]
    layer:   x = x + n1(mixer(x));   x = x + n2(ff(x))        n(y) = y / rms(y) * (1 + w): the norm stands BEHIND a sub-layer
    logits = cap * tanh(table . n(x) / cap)

`weights` maps checkpoint names to float64 tensors; `config` is the dictionary of config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x, weight, eps, one_plus=False):
    """x over its root mean square along the last dimension (eps under the root), times the weight or 1 + weight."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y * (1.0 + weight) if one_plus else y * weight


def scaled_frequencies(base: float, dims: int, scaling: Optional[dict]) -> List[float]:
    """f_i = base^(-2i / dims) for i < dims / 2; long wavelengths are slowed down: with l = 2 pi / f, f stays where
    l < original / high, becomes f / factor where l > original / low, and is blended in between by
    s = (original / l - low) / (high - low): (1 - s) f / factor + s f."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            length = 2.0 * math.pi / f
            if length > original / low:
                f = f / factor
            elif length >= original / high:
                s = (original / length - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_halves(x, positions, freqs):
    """x [T, heads, n]: of the first 2 * len(freqs) values, value i turns with value i + len(freqs) by position * freqs[i]."""
    out = x.clone()
    half = len(freqs)
    for i, f in enumerate(freqs):
        angle = positions.double() * f
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def visible(T: int, window: Optional[int]):
    """[T, T] bool: query i sees key j: j <= i, and with a window also i - j < window."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    return seen


def softmax_with_sink(scores, seen, sink=None):
    """scores [H, T, T]; keys that are not seen get no weight; `sink` [H] adds exp(sink_h) to the denominator only."""
    scores = scores.masked_fill(~seen[None], -math.inf)
    top = scores.max(dim=-1).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None])
    e = torch.exp(scores - top[..., None])
    total = e.sum(dim=-1)
    if sink is not None:
        total = total + torch.exp(sink[:, None] - top)
    return e / total[..., None]


def attend(q, k, v, scale, seen, sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; query head h reads kv head h // (H / G)."""
    H, G = q.shape[1], k.shape[1]
    idx = torch.arange(H) // (H // G)
    scores = torch.einsum("thd,shd->hts", q, k[:, idx]) * scale
    return torch.einsum("hts,shd->thd", softmax_with_sink(scores, seen, sink), v[:, idx])


def windowed_sink_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, kv=None):
    """The mixer `attention`: q and k normed over the WHOLE projection, no rotation, a sliding window, a learned sink in
    the softmax's denominator, every head's result times sigmoid of one gate value per head.  Returns (result, (k, v))."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(T, H, D)
    if kv is None:
        k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(T, G, D)
        v = (h @ w[p + "v"].T).view(T, G, Dv)
    else:
        k, v = kv
    window = m["mask"]["size"] if m.get("mask") else None
    out = attend(q, k, v, m["scale"], visible(T, window), w[p + "sink"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                   # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * Dv) @ w[p + "o"].T, (k, v)


def rotary_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, kv=None):
    """The mixer `attention_2`: biases on q, k, v; q and k normed per head with one weight for all heads; the first
    rot.dims values of each head turned by the position; causal; plain softmax.  With `kv` (keys as cached, after
    norm and rotation, and values, of an earlier layer) the layer makes queries only.  Returns (result, (k, v))."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    freqs = scaled_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling")) if m.get("rot") else []
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    q = rotate_halves(rms_norm(q, w[p + "q.norm"], eps), positions, freqs)
    if kv is None:
        k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
        k = rotate_halves(rms_norm(k, w[p + "k.norm"], eps), positions, freqs)
        v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, Dv)
    else:
        k, v = kv
    out = attend(q, k, v, m["scale"], visible(T, None))
    return out.reshape(T, H * Dv) @ w[p + "o"].T, (k, v)


def squared_relu_ff(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    """g = min(Wg h, limit), u = clamp(Wu h, -limit, limit);  Wd (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, top):
    """Router logits with a bias; the `top` largest are chosen, their weights the softmax over the chosen logits."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    values, chosen = torch.topk(z, top, dim=-1)
    return chosen, torch.softmax(values, dim=-1)


def routing_margin(h, w, p, top):
    """Per token: how far the last chosen logit lies above the first one left out, relative to the largest logit's size
    (infinite when every expert is chosen).  A token with a tiny margin may choose otherwise after any rounding."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    if top >= z.shape[-1]:
        return torch.full(z.shape[:-1], math.inf, dtype=z.dtype)
    values = torch.sort(z, dim=-1, descending=True).values
    return (values[..., top - 1] - values[..., top]) / z.abs().amax(dim=-1)


def routed_experts(h, w, p, mlp, margins_out: Optional[list] = None):
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    chosen, weights = route(h, w, p, top)
    if margins_out is not None:
        margins_out.append(routing_margin(h, w, p, top))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += weights[t, j] * clamped_expert(h[t:t + 1], w, f"{p}e{int(chosen[t, j])}.", limit)[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)       # [T, 1]
        out = out + gate * clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None,
            margins_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence, float64; `layers_out` collects the stream after every layer, `margins_out` the
    routing margins [T] of every layer with experts."""
    w = {k: v.double() for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        mixer = windowed_sink_attention if layer["type"] == "attention" else rotary_attention
        source = m.get("kv_from")
        y, kept[i] = mixer(x, w, p + "mix.", m, eps, kv=kept[source] if source is not None else None)
        x = x + rms_norm(y, w[p + "norm1"], eps, one_plus=True)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = squared_relu_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else routed_experts(x, w, p + "mlp.", mlp, margins_out)
            x = x + rms_norm(y, w[p + "norm2"], eps, one_plus=True)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, w["final.norm"], eps, one_plus=True)
    logits = x @ w["embed"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
