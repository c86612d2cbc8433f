"""Small Sokolorn configurations and random weights for the tests.  The configurations differ in every size and option:
width, vocabulary, layer order (starting with either mixer, one kind only), query heads that share key/value heads and heads
of their own in both mixers, key and value sizes that differ, windows of 1, of a few tokens, of more than a tile of keys,
larger than every prompt, and none; rotation of a whole head, of a part of it, and none; frequency scaling whose three
zones (kept, blended, slowed) all occur, and none; layers that read the keys and values of the layer before them and of a
layer further back, two readers of one layer, a windowed reader; dense and routed feed-forwards and none; 1 of n, several of n and all of n
experts, with and without a shared expert, limits that clamp often and never; with and without a cap on the logits."""
from __future__ import annotations

import copy
import math
from typing import Dict

import torch


def _windowed(heads, kv_heads, dim, vdim, scale, mlp, window=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _rotary(heads, kv_heads, dim, vdim, scale, mlp, rot=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        mixer["rot"] = rot
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": mixer, "mlp": mlp}


def _rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


# Starts with the windowed mixer; grouped heads there; a reader of the layer before it; wavelengths in all three zones.
ROT_A = _rot(100.0, 8, (8.0, 1.0, 4.0, 64))
SMALL_A = {
    "architecture": "Sokolorn", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
    "layers": [
        _windowed(4, 2, 8, 12, 0.4, _dense(40), window=9),
        _rotary(6, 3, 8, 16, 0.3, _moe(6, 2, 24, 0.8, shared=(20, 1.5)), rot=ROT_A),
        _rotary(6, 3, 8, 16, 0.5, _dense(24), rot=ROT_A, kv_from=1),
        _windowed(2, 2, 24, 8, 0.2, _moe(5, 5, 16, 100.0), window=5),
        _windowed(3, 1, 16, 4, 0.25, None, window=200),
    ],
}

# Sizes that miss every fast path: a width that is no multiple of 8, heads of 10 and 6, a window of one token, one expert of
# several, a rotation of the whole head without scaling and one of two values, a reader two layers back and a second reader.
ROT_B = _rot(50.0, 10)
SMALL_B = {
    "architecture": "Sokolorn", "vocab": 130, "width": 36, "norm": {"eps": 1e-6},
    "layers": [
        _rotary(5, 5, 10, 6, 0.3, _moe(7, 1, 12, 0.5, shared=(9, 0.3)), rot=ROT_B),
        _windowed(5, 5, 6, 10, 0.5, _dense(28), window=1),
        _rotary(5, 5, 10, 6, 0.2, None, rot=ROT_B, kv_from=0),
        _rotary(3, 1, 6, 10, 0.4, _dense(12), rot=_rot(10000.0, 2, (2.0, 2.0, 8.0, 16))),
        _rotary(10, 5, 10, 6, 0.25, _moe(4, 3, 8, 2.0), rot=ROT_B, kv_from=0),
        _windowed(6, 3, 6, 6, 0.6, _dense(20)),
    ],
}

# Sizes the tensor-core attention kernels take (keys of 32 and 16, values of 16, 8 and 32), windows beyond one tile of 64
# keys and a prompt beyond one tile of rows; no rotation at all in one layer.
ROT_C = _rot(500.0, 16, (4.0, 1.0, 2.0, 32))
SMALL_C = {
    "architecture": "Sokolorn", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
    "layers": [
        _windowed(4, 2, 32, 16, 0.2, _moe(8, 2, 32, 1.0, shared=(48, 1.0)), window=70),
        _rotary(4, 2, 32, 16, 0.25, _dense(64), rot=ROT_C),
        _windowed(8, 8, 16, 8, 0.3, _dense(48), window=100),
        _rotary(8, 2, 32, 16, 0.15, _moe(16, 4, 16, 0.6), rot=ROT_C, kv_from=1),
        _rotary(2, 1, 16, 32, 0.35, _dense(32)),
    ],
}

# Rotated layers whose keys and values have one size, as the tcgen05 prompt kernel and the split-KV kernel take them (heads of 64 and
# 128, the cache rows swizzled), beside one of 32 and one of 24 (no tensor-core size); readers of each; a windowed layer of 64 that stays on the masked kernels.
ROT_D = _rot(5000.0, 48, (2.0, 0.5, 3.0, 96))
SMALL_D = {
    "architecture": "Sokolorn", "vocab": 150, "width": 128, "norm": {"eps": 1e-6}, "logit_softcap": 20.0,
    "layers": [
        _rotary(4, 2, 64, 64, 0.12, _dense(96), rot=ROT_D),
        _windowed(2, 2, 64, 64, 0.15, _moe(6, 2, 32, 1.2, shared=(40, 0.9)), window=40),
        _rotary(2, 2, 64, 64, 0.1, _dense(64), rot=ROT_D, kv_from=0),
        _rotary(2, 1, 128, 128, 0.09, None, rot=_rot(100.0, 128)),
        _rotary(4, 1, 128, 128, 0.08, _dense(48), rot=_rot(100.0, 128), kv_from=3),
        _rotary(4, 4, 32, 32, 0.2, _dense(48)),
        _rotary(6, 2, 24, 24, 0.2, None, rot=_rot(40.0, 12)),
    ],
}

# One kind of mixer only, each in a model of its own.
ONLY_WINDOWED = {
    "architecture": "Sokolorn", "vocab": 61, "width": 32, "norm": {"eps": 1e-5}, "logit_softcap": 5.0,
    "layers": [_windowed(2, 1, 16, 16, 0.3, _dense(16), window=6), _windowed(4, 1, 8, 16, 0.5, None, window=3),
               _windowed(4, 1, 16, 16, 0.4, _dense(24), window=6, kv_from=0)],
}
ONLY_ROTARY = {
    "architecture": "Sokolorn", "vocab": 61, "width": 32, "norm": {"eps": 1e-5},
    "layers": [_rotary(2, 1, 16, 16, 0.3, _moe(3, 2, 8, 0.7), rot=_rot(20.0, 4, (4.0, 1.0, 4.0, 16))),
               _rotary(4, 1, 16, 16, 0.2, _dense(16), rot=_rot(20.0, 4, (4.0, 1.0, 4.0, 16)), kv_from=0)],
}

ALL = {"small_a": SMALL_A, "small_b": SMALL_B, "small_c": SMALL_C, "small_d": SMALL_D, "only_windowed": ONLY_WINDOWED, "only_rotary": ONLY_ROTARY}


def get(name: str) -> dict:
    return copy.deepcopy(ALL[name])


def random_weights(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by their checkpoint names; matrices scaled so that activations stay of order one, router biases and
    gaps between router rows large enough that no choice of experts is a close call."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).bfloat16()

    def vector(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * torch.randn(n, generator=g)).bfloat16()

    def expert(p, ff):
        matrix(p + "gate", ff, W, 2.0)
        matrix(p + "up", ff, W, 2.0)
        matrix(p + "down", W, ff)

    matrix("embed", config["vocab"], W, 4.0)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        own = m.get("kv_from") is None
        vector(p + "norm1", W, 0.0, 0.2)
        matrix(p + "mix.q", H * D, W, 2.0)
        if own:
            matrix(p + "mix.k", G * D, W, 2.0)
            matrix(p + "mix.v", G * Dv, W, 2.0)
        matrix(p + "mix.o", W, H * Dv)
        if layer["type"] == "attention":
            vector(p + "mix.q.norm", H * D, 1.0, 0.2)
            if own:
                vector(p + "mix.k.norm", G * D, 1.0, 0.2)
            vector(p + "mix.sink", H, 0.5, 1.0)
            matrix(p + "mix.g", H, W, 2.0)
        else:
            vector(p + "mix.q.norm", D, 1.0, 0.2)
            vector(p + "mix.q.b", H * D, 0.0, 0.3)
            if own:
                vector(p + "mix.k.norm", D, 1.0, 0.2)
                vector(p + "mix.k.b", G * D, 0.0, 0.3)
                vector(p + "mix.v.b", G * Dv, 0.0, 0.3)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        vector(p + "norm2", W, 0.0, 0.2)
        if mlp["kind"] == "dense":
            matrix(p + "mlp.up", mlp["ff"], W, 2.0)
            matrix(p + "mlp.down", W, mlp["ff"])
            continue
        E = mlp["router"]["experts"]
        matrix(p + "mlp.router", E, W, 6.0)
        vector(p + "mlp.router.b", E, 0.0, 1.0)
        for j in range(E):
            expert(f"{p}mlp.e{j}.", mlp["expert"]["ff"])
        if mlp.get("shared"):
            expert(p + "mlp.shared.", mlp["shared"]["ff"])
            matrix(p + "mlp.shared.sg", 1, W, 2.0)
    vector("final.norm", W, 0.0, 0.2)
    return out
