"""Small Sopetar configurations and random weights for the tests.  The configurations differ in every size and
option: width, vocabulary, embedding scale, layer order (starting with either mixer, one mixer kind only), query
heads that share key/value heads and heads of their own, key and value sizes that differ, rotated parts equal to
and larger than the rotated dimensions, latents that are no multiple of 8, windows of 1, of a few tokens, of more
than a tile of keys, larger than every prompt, and none; kept first tokens fewer than, equal to and more than the
window, and none; layers with and without a cap on the scores, with and without value mixing (none, one, several
such layers), with and without a feed-forward, with and without a clamp in it; one has more than 16 query heads on a kv head."""
from __future__ import annotations

import copy
import math
from typing import Dict

import torch


def _latent(heads, dim, rot_dim, rot_dims, vdim, rank, scale, window, mlp, base=10000.0):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
             "rot": {"base": base, "dims": rot_dims}}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _attention(heads, kv_heads, dim, vdim, scale, mlp, window=None, keep_first=None, softcap=None, v_mix=False):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
        if keep_first is not None:
            mixer["mask"]["keep_first"] = keep_first
    if softcap is not None:
        mixer["softcap"] = softcap
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _dense(ff, limit=None):
    out = {"kind": "dense", "ff": ff}
    if limit is not None:
        out["limit"] = limit
    return out


# Starts with attention; grouped heads; windows of a few tokens; one layer without a feed-forward; three mixing layers.
SMALL_A = {
    "architecture": "Sopetar", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
    "layers": [
        _attention(4, 2, 8, 12, 0.9, _dense(40, 0.7), window=9, keep_first=3, softcap=4.0, v_mix=True),
        _latent(3, 8, 4, 4, 12, 16, 0.35, 7, _dense(24, 2.5)),
        _attention(6, 2, 16, 12, 1.3, None, v_mix=True),
        _latent(2, 16, 8, 6, 8, 24, 0.2, None, _dense(32)),
        _attention(2, 2, 24, 12, 2.0, _dense(16, 1.0), window=5, softcap=30.0, v_mix=True),
        _attention(4, 1, 8, 4, 0.7, _dense(24, 0.4), window=12, keep_first=12),
    ],
}

# Sizes that miss every fast path: a width that is no multiple of 8, heads of 10, a latent of 12 with a rotated part of 6 of
# which 4 turn, a window of one token, more kept tokens than the window is wide.
SMALL_B = {
    "architecture": "Sopetar", "vocab": 130, "width": 36, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.25},
    "layers": [
        _latent(5, 10, 6, 4, 6, 12, 0.3, 1, _dense(20, 1.5), base=100.0),
        _attention(5, 5, 10, 6, 1.1, _dense(28, 3.0), window=3, keep_first=8, softcap=2.0),
        _latent(1, 12, 2, 2, 20, 12, 0.4, 33, None, base=50.0),
        _attention(3, 1, 6, 10, 0.8, _dense(12), window=1, keep_first=2, v_mix=True),
    ],
}

# Sizes the tiled attention kernel takes (keys of 48 + 16 and of 32, values of 48 and 16), windows and kept tokens beyond one
# tile of 64 keys, prompts beyond one tile of rows; only one mixing layer (it keeps its values, nobody reads them).
SMALL_C = {
    "architecture": "Sopetar", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "layers": [
        _latent(4, 16, 16, 16, 8, 48, 0.25, 70, _dense(48, 1.0)),
        _attention(4, 2, 32, 16, 0.6, _dense(64, 2.0), window=40, keep_first=70, softcap=10.0, v_mix=True),
        _latent(2, 32, 32, 16, 16, 32, 0.2, 1000, _dense(32, 0.9), base=500.0),
        _attention(8, 8, 16, 8, 0.9, None, window=100, keep_first=1),
    ],
}

# One kind of mixer only, each in a model of its own.
ONLY_LATENT = {
    "architecture": "Sopetar", "vocab": 61, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [_latent(2, 8, 8, 8, 8, 16, 0.3, 4, _dense(16, 1.2)), _latent(4, 4, 2, 2, 4, 8, 0.5, None, None)],
}
ONLY_ATTENTION = {
    "architecture": "Sopetar", "vocab": 61, "width": 32, "norm": {"eps": 1e-5},
    "layers": [_attention(2, 1, 16, 16, 1.0, _dense(16, 1.2), window=6, keep_first=2, v_mix=True),
               _attention(4, 1, 8, 16, 0.5, None, softcap=5.0, v_mix=True)],
}

# More than 16 query heads on a kv head in both mixers (the latent mixer has one kv head for all of its heads), with sizes the
# tensor-core kernels take: decoded tokens run their heads 16 at a time.
MANY_HEADS = {
    "architecture": "Sopetar", "vocab": 75, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.8},
    "layers": [_latent(18, 16, 16, 8, 8, 32, 0.2, 21, _dense(24, 1.5)),
               _attention(34, 2, 16, 8, 0.5, _dense(24, 2.0), window=30, keep_first=3, softcap=6.0)],
}

ALL = {"small_a": SMALL_A, "many_heads": MANY_HEADS, "small_b": SMALL_B, "small_c": SMALL_C, "only_latent": ONLY_LATENT, "only_attention": ONLY_ATTENTION}


def get(name: str) -> dict:
    return copy.deepcopy(ALL[name])


def random_weights(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by their checkpoint names; matrices scaled so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).bfloat16()

    def vector(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * torch.randn(n, generator=g)).bfloat16()

    matrix("embed", config["vocab"], W, 4.0)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        vector(p + "norm1", W, 1.0, 0.1)
        vector(p + "norm1.b", W, 0.0, 0.1)
        if layer["type"] == "latent_attention":
            H, D, P, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            matrix(p + "mix.q", H * (D + P), W, 2.0)
            matrix(p + "mix.dkv", R + P, W, 2.0)
            vector(p + "mix.dkv.norm", R, 1.0, 0.1)
            matrix(p + "mix.uk", H * D, R, 2.0)
            matrix(p + "mix.uv", H * Dv, R)
            vector(p + "mix.sink", H, 0.5, 1.0)
            matrix(p + "mix.g", H, W, 2.0)
            matrix(p + "mix.o", W, H * Dv)
        else:
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for role, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                matrix(p + f"mix.{role}", rows, W, 2.0)
                vector(p + f"mix.{role}.b", rows, 0.0, 0.3)
            matrix(p + "mix.o", W, H * Dv)
            if m.get("v_mix"):
                out[p + "mix.vmix"] = (0.3 + 0.2 * torch.randn((), generator=g)).bfloat16()
        mlp = layer["mlp"]
        if mlp is not None:
            matrix(p + "mlp.gate", mlp["ff"], W, 2.0)
            matrix(p + "mlp.up", mlp["ff"], W, 2.0)
            matrix(p + "mlp.down", W, mlp["ff"])
            vector(p + "mlp.gate.b", mlp["ff"], 0.0, 0.3)
            vector(p + "mlp.up.b", mlp["ff"], 0.0, 0.3)
            vector(p + "mlp.down.b", W, 0.0, 0.1)
        vector(p + "dwa", i + 2, 1.0 / (i + 2), 0.25)
    vector("final.norm", W, 1.0, 0.1)
    vector("final.norm.b", W, 0.0, 0.1)
    matrix("head", config["vocab"], W)
    return out
