"""Typed configuration of the Sopetar decoder, read from its config.json.

    {"architecture": "Sopetar", "vocab": V, "width": W, "norm": {"eps"}, "embedding": {"scale"},
     "layers": [{"type": "latent_attention" | "attention", "mixer": {...}, "mlp": {"kind": "dense", "ff", "limit"} | null}, ...]}

A "latent_attention" mixer has heads, dim (plain query/key values per head), rot_dim (rotated ones), vdim, kv_rank, scale,
rot = {base, dims} and optionally mask.size (a sliding window).  An "attention" mixer has heads, kv_heads, dim, vdim, scale and
optionally softcap, v_mix and mask = {size, optionally keep_first}.  Every size and constant comes from the file; a missing
required key is an error, and what the file leaves out (a mask, a cap, value mixing, a feed-forward) does not exist.  The design
names no largest position; `max_positions` is this engine's bound on a request's length.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple

from .base import ConfigError
from .gopevik import MAX_POSITIONS, Rotation, _get, _integer, _number


@dataclass(frozen=True)
class LatentRotaryConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Optional[Rotation]
    window: Optional[int]


@dataclass(frozen=True)
class BiasedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    keep_first: int
    v_mix: bool


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: Optional[float]


@dataclass(frozen=True)
class SopetarLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseConfig]


def _window(m: dict, where: str):
    mask = m.get("mask")
    if mask is None:
        return None, 0
    size = _integer(mask, "size", where + "mask.") if mask.get("size") is not None else None
    keep = mask.get("keep_first")
    if keep is None:
        return size, 0
    if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
        raise ConfigError(f"config.json key {where}mask.'keep_first' must be a non-negative integer, got {keep!r}")
    return size, (keep if size is not None else 0)


@dataclass(frozen=True)
class SopetarConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[SopetarLayer, ...]
    max_position_embeddings: int = MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict) -> "SopetarConfig":
        norm = _get(raw, "norm", "")
        emb = raw.get("embedding") or {}
        listed = _get(raw, "layers", "")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(listed):
            where = f"layers[{i}]."
            kind = _get(layer, "type", where)
            m = _get(layer, "mixer", where)
            mw = where + "mixer."
            if kind == "latent_attention":
                rot_dim = _integer(m, "rot_dim", mw) if m.get("rot_dim") else 0
                rot = Rotation.from_dict(m.get("rot"), mw + "rot.", rot_dim) if rot_dim else None
                if rot_dim and rot is None:
                    raise ConfigError(f"config.json lacks required key {mw}'rot' (the mixer has {rot_dim} rotated values)")
                size, keep = _window(m, mw)
                if keep:
                    raise ConfigError(f"config.json key {mw}mask.'keep_first': this mixer's window keeps no first tokens")
                mixer = LatentRotaryConfig(_integer(m, "heads", mw), _integer(m, "dim", mw), rot_dim, _integer(m, "vdim", mw),
                                           _integer(m, "kv_rank", mw), _number(m, "scale", mw), rot, size)
            elif kind == "attention":
                heads = _integer(m, "heads", mw)
                kv_heads = _integer(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
                if heads % kv_heads:
                    raise ConfigError(f"config.json key {mw}'kv_heads' = {kv_heads} does not divide the {heads} heads")
                size, keep = _window(m, mw)
                mixer = BiasedAttentionConfig(heads, kv_heads, _integer(m, "dim", mw), _integer(m, "vdim", mw), _number(m, "scale", mw),
                                              _number(m, "softcap", mw) if m.get("softcap") is not None else None, size, keep,
                                              bool(m.get("v_mix", False)))
            else:
                raise ConfigError(f"config.json key {where}'type' = {kind!r} is not one of 'latent_attention', 'attention'")
            layers.append(SopetarLayer(kind, mixer, cls._mlp(layer.get("mlp"), where + "mlp.")))
        mixing = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        if any((a.kv_heads, a.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for a in mixing):
            raise ConfigError("config.json: layers that mix values must have the same kv_heads and vdim")
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        return cls(architecture=_get(raw, "architecture", ""), vocab_size=_integer(raw, "vocab", ""), width=_integer(raw, "width", ""),
                   norm_eps=_number(norm, "eps", "norm."),
                   embedding_scale=_number(emb, "scale", "embedding.", positive=False) if emb.get("scale") is not None else 1.0,
                   layers=tuple(layers), max_position_embeddings=int(raw.get("max_positions", MAX_POSITIONS)), eos_token_ids=eos)

    @staticmethod
    def _mlp(mlp: Optional[dict], where: str) -> Optional[DenseConfig]:
        if mlp is None:
            return None
        if _get(mlp, "kind", where) != "dense":
            raise ConfigError(f"config.json key {where}'kind' = {mlp['kind']!r}; this design has 'dense'")
        return DenseConfig(_integer(mlp, "ff", where), _number(mlp, "limit", where) if mlp.get("limit") is not None else None)
