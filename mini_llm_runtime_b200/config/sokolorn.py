"""Typed configuration of the Sokolorn decoder, read from its config.json.

    {"architecture": "Sokolorn", "vocab": V, "width": W, "norm": {"eps"}, "logit_softcap": c,
     "layers": [{"type": "attention" | "attention_2", "mixer": {...}, "mlp": {...} | null}, ...]}

An "attention" mixer has heads, kv_heads, dim, vdim, scale and optionally mask.size (a sliding window); an "attention_2"
mixer has heads, kv_heads, dim, vdim, scale and optionally rot = {base, dims, optionally scaling = {factor, low, high, original}}.
Either may name kv_from: the index of an earlier layer of its type whose cached keys and values it reads.  A feed-forward is
{"kind": "dense", "ff"} or {"kind": "moe", "expert": {ff, limit}, "router": {experts, top}, optionally "shared": {ff, limit}}.
Every size and constant comes from the file; a missing required key is an error, and what the file leaves out (a window, a
rotation, its scaling, a shared expert, a cap on the logits, a feed-forward) does not exist.  The design names no largest
position; `max_positions` is this engine's bound on a request's length.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError
from .gopevik import MAX_POSITIONS, _get, _integer, _number


@dataclass(frozen=True)
class FrequencyScaling:
    """Long wavelengths slowed down: see `parts/rotary.py` (`scaled_frequencies`)."""
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class ScaledRotation:
    base: float
    dims: int
    scaling: Optional[FrequencyScaling]

    @classmethod
    def from_dict(cls, raw: Optional[dict], where: str, head: int) -> Optional["ScaledRotation"]:
        if raw is None:
            return None
        dims = _integer(raw, "dims", where)
        if dims % 2 or dims > head:
            raise ConfigError(f"config.json key {where}'dims' = {dims} must be even and at most the head size {head}")
        s = raw.get("scaling")
        scaling = None
        if s is not None:
            sw = where + "scaling."
            scaling = FrequencyScaling(_number(s, "factor", sw), _number(s, "low", sw), _number(s, "high", sw), _number(s, "original", sw))
            if scaling.high <= scaling.low:
                raise ConfigError(f"config.json key {sw}'high' = {scaling.high} must exceed 'low' = {scaling.low}")
        return cls(_number(raw, "base", where), dims, scaling)


@dataclass(frozen=True)
class SokolornMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None                # "attention"
    rot: Optional[ScaledRotation] = None        # "attention_2"
    kv_from: Optional[int] = None               # an earlier layer of the same type whose cached keys and values this one reads


@dataclass(frozen=True)
class ExpertShape:
    ff: int
    limit: Optional[float]


@dataclass(frozen=True)
class SokolornMlp:
    kind: str                       # "dense" | "moe"
    ff: int = 0                     # dense
    expert: Optional[ExpertShape] = None
    experts: int = 0
    top: int = 0
    shared: Optional[ExpertShape] = None


@dataclass(frozen=True)
class SokolornLayer:
    type: str
    mixer: SokolornMixer
    mlp: Optional[SokolornMlp]


def _expert(raw: dict, where: str) -> ExpertShape:
    return ExpertShape(_integer(raw, "ff", where), _number(raw, "limit", where) if raw.get("limit") is not None else None)


@dataclass(frozen=True)
class SokolornConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[SokolornLayer, ...]
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
    def from_dict(cls, raw: dict) -> "SokolornConfig":
        norm = _get(raw, "norm", "")
        listed = _get(raw, "layers", "")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(listed):
            where = f"layers[{i}]."
            kind = _get(layer, "type", where)
            if kind not in ("attention", "attention_2"):
                raise ConfigError(f"config.json key {where}'type' = {kind!r} is not one of 'attention', 'attention_2'")
            m = _get(layer, "mixer", where)
            mw = where + "mixer."
            heads = _integer(m, "heads", mw)
            kv_heads = _integer(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
            if heads % kv_heads:
                raise ConfigError(f"config.json key {mw}'kv_heads' = {kv_heads} does not divide the {heads} heads")
            dim = _integer(m, "dim", mw)
            window = rot = kv_from = None
            if kind == "attention":
                mask = m.get("mask")
                window = _integer(mask, "size", mw + "mask.") if mask is not None and mask.get("size") is not None else None
                if m.get("rot") is not None:
                    raise ConfigError(f"config.json key {mw}'rot' belongs to the mixer 'attention_2'")
            else:
                rot = ScaledRotation.from_dict(m.get("rot"), mw + "rot.", dim)
                if m.get("mask") is not None:
                    raise ConfigError(f"config.json key {mw}'mask' belongs to the mixer 'attention'")
            kv_from = m.get("kv_from")
            if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < i):
                raise ConfigError(f"config.json key {mw}'kv_from' = {kv_from!r} must be the index of an earlier layer")
            mixer = SokolornMixer(heads, kv_heads, dim, _integer(m, "vdim", mw), _number(m, "scale", mw), window, rot, kv_from)
            if kv_from is not None:
                source = layers[kv_from]
                if source.type != kind or source.mixer.kv_from is not None:
                    raise ConfigError(f"config.json key {mw}'kv_from' = {kv_from}: that layer is no '{kind}' layer with keys and values of its own")
                a, b = source.mixer, mixer
                if (a.kv_heads, a.dim, a.vdim, a.rot, a.window) != (b.kv_heads, b.dim, b.vdim, b.rot, b.window):
                    raise ConfigError(f"config.json key {mw}'kv_from' = {kv_from}: key/value heads, sizes, rotation or window of the two layers differ")
            layers.append(SokolornLayer(kind, mixer, cls._mlp(layer.get("mlp"), where + "mlp.")))
        cap = raw.get("logit_softcap")
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        return cls(architecture=_get(raw, "architecture", ""), vocab_size=_integer(raw, "vocab", ""), width=_integer(raw, "width", ""),
                   norm_eps=_number(norm, "eps", "norm."), logit_softcap=_number(raw, "logit_softcap", "") if cap is not None else None,
                   layers=tuple(layers), max_position_embeddings=int(raw.get("max_positions", MAX_POSITIONS)), eos_token_ids=eos)

    @staticmethod
    def _mlp(mlp: Optional[dict], where: str) -> Optional[SokolornMlp]:
        if mlp is None:
            return None
        kind = _get(mlp, "kind", where)
        if kind == "dense":
            return SokolornMlp("dense", ff=_integer(mlp, "ff", where))
        if kind != "moe":
            raise ConfigError(f"config.json key {where}'kind' = {kind!r} is not one of 'dense', 'moe'")
        router = _get(mlp, "router", where)
        experts, top = _integer(router, "experts", where + "router."), _integer(router, "top", where + "router.")
        if top > experts:
            raise ConfigError(f"config.json key {where}router.'top' = {top} exceeds the {experts} experts")
        shared = mlp.get("shared")
        return SokolornMlp("moe", expert=_expert(_get(mlp, "expert", where), where + "expert."), experts=experts, top=top,
                           shared=_expert(shared, where + "shared.") if shared is not None else None)
