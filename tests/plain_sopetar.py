"""A plain, slow implementation of the Sopetar decoder for the tests: whole sequences, float64, no cache, no
batching, one function per mechanism, nothing shared with the package.

    x_0 = table[token] * scale
    layer i:  u = layer_norm(x);  y = x + (mixer(u) + feed_forward(u));  X_{i+1} = y;  x = sum_{j <= i+1} a_i[j] X_j
    logits = head . layer_norm(x)

`weights` maps checkpoint names to float64 tensors; `config` is the dictionary of config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def layer_norm(x, weight, bias, eps):
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def unit_rms(x, eps):
    """x over its root mean square along the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rotate_pairs(x, positions, base, dims):
    """x [T, heads, n]: of the first `dims` values, value 2i and value 2i + 1 turn by position * base^(-2i / dims)."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.double() * base ** (-2.0 * i / dims)
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def visible(T, window: Optional[int], keep_first: int = 0):
    """[T, T] bool: query i sees key j."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & ((i - j < window) | (j < keep_first))
    return seen


def softmax_with_sink(scores, seen, sink=None):
    """scores [H, T, T]; keys that are not seen get no weight; `sink` [H] adds exp(sink_h) to the denominator."""
    scores = scores.masked_fill(~seen[None], -math.inf)
    top = scores.max(dim=-1).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None])
    e = torch.exp(scores - top[..., None])
    total = e.sum(dim=-1)
    if sink is not None:
        total = total + torch.exp(sink[:, None] - top)
    return e / total[..., None]


def attend(q, k, v, scale, seen, softcap=None, slopes=None, sink=None):
    """q, k [T, H, D], v [T, H, Dv], one key/value head per query head.  The score of query i with key j is
    (q_i . k_j) * scale, then capped, then lowered by slope_h * (i - j); weights by `softmax_with_sink` over the keys `seen`."""
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    if softcap:
        scores = softcap * torch.tanh(scores / softcap)
    if slopes is not None:
        distance = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).double()
        scores = scores - slopes[:, None, None] * distance[None]
    return torch.einsum("hij,jhd->ihd", softmax_with_sink(scores, seen, sink), v)


def latent_attention(m: dict, w: Dict[str, torch.Tensor], p: str, u, eps):
    """Keys and values of every head from one latent per token, plus one rotated key part that all heads share."""
    T = u.shape[0]
    H, D, P, Dv, R = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    q = (u @ w[p + "q"].T).view(T, H, D + P)
    down = u @ w[p + "dkv"].T
    latent = unit_rms(down[:, :R], eps) * w[p + "dkv.norm"]
    q_plain, q_rot = q[..., :D], q[..., D:]
    k_rot = down[:, R:].view(T, 1, P)
    if P:
        q_rot = rotate_pairs(q_rot, positions, m["rot"]["base"], m["rot"]["dims"])
        k_rot = rotate_pairs(k_rot, positions, m["rot"]["base"], m["rot"]["dims"])
    k = (latent @ w[p + "uk"].T).view(T, H, D)
    v = (latent @ w[p + "uv"].T).view(T, H, Dv)
    mask = m.get("mask") or {}
    out = attend(torch.cat([q_plain, q_rot], dim=-1), torch.cat([k, k_rot.expand(T, H, P)], dim=-1), v, m["scale"],
                 visible(T, mask.get("size")), sink=w[p + "sink"])
    out = out * torch.sigmoid(u @ w[p + "g"].T)[..., None]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def distance_slopes(heads: int):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64)


def biased_attention(m: dict, w: Dict[str, torch.Tensor], p: str, u, eps, shared: dict):
    """Grouped-query attention without rotation: biases, unit heads, capped scores, a bias by distance, a window that keeps
    the first tokens, and values mixed with those of the first layer that mixes (`shared` carries them through the layers)."""
    T = u.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = unit_rms((u @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D), eps)
    k = unit_rms((u @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D), eps)
    v = unit_rms((u @ w[p + "v"].T + w[p + "v.b"]).view(T, G, Dv), eps)
    if m.get("v_mix"):
        if "first" in shared:
            lam = w[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["first"]
        else:
            shared["first"] = v
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    mask = m.get("mask") or {}
    out = attend(q, k, v, m["scale"], visible(T, mask.get("size"), mask.get("keep_first", 0)), m.get("softcap"), distance_slopes(H))
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def dense_feed_forward(mlp: dict, w: Dict[str, torch.Tensor], p: str, u):
    g = u @ w[p + "gate"].T + w[p + "gate.b"]
    up = u @ w[p + "up"].T + w[p + "up.b"]
    if mlp.get("limit") is not None:
        g = torch.clamp(g, max=mlp["limit"])
        up = torch.clamp(up, -mlp["limit"], mlp["limit"])
    return (g * torch.sigmoid(1.702 * g) * (up + 1.0)) @ w[p + "down"].T + w[p + "down.b"]


def depth_average(states: List[torch.Tensor], weights):
    return sum(weights[j] * states[j] for j in range(len(states)))


def forward(config: dict, w: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence; `layers_out` collects the stream after every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    states, shared = [x], {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        u = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "latent_attention":
            mixed = latent_attention(layer["mixer"], w, p + "mix.", u, eps)
        else:
            mixed = biased_attention(layer["mixer"], w, p + "mix.", u, eps, shared)
        if layer.get("mlp") is not None:
            mixed = mixed + dense_feed_forward(layer["mlp"], w, p + "mlp.", u)
        states.append(x + mixed)
        x = depth_average(states, w[p + "dwa"])
        if layers_out is not None:
            layers_out.append(x)
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
