"""Sopetar as a model plan: a scaled embedding; layers whose ONE layer norm feeds a mixer and a feed-forward side by side
(`parallel_residual` block), each layer's result averaged with all earlier states of the stream through learned weights
(the block's `states`); mixers of two kinds, latent attention with a rotated key part, a sliding window, a learned sink and a
gate per head, and grouped-query attention with biases, unit-norm heads, a capped score, a distance bias, a window that keeps
the first tokens and values mixed with those of the first such layer; a gated feed-forward with biases and clamps; a last
layer norm and a head of its own.  This module only turns a `SopetarConfig` into data; the parts live in `parts/`.
Tensor names: `embed`, `l<i>.norm1[.b]`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}[.b]`, `l<i>.dwa`, `final.norm[.b]`, `head`.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelPlan, PartSpec, Run
from ..config.registry import register_architecture
from ..config.sopetar import BiasedAttentionConfig, LatentRotaryConfig, SopetarConfig

SWISH_ALPHA = 1.702          # y = g * sigmoid(1.702 g) * (u + 1)
UP_OFFSET = 1.0
SLOPE_EXPONENT = 8.0         # slope of head h of H: 2^(-8 (h + 1) / H)


def sopetar_plan(cfg: SopetarConfig) -> ModelPlan:
    width, count = cfg.width, len(cfg.layers)
    layer_norm = lambda name: PartSpec("layernorm", {"width": width, "eps": cfg.norm_eps}, {"weight": name, "bias": name + ".b"})
    positions, layers, schedule = {}, [], []
    mixing_seen = False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, LatentRotaryConfig):
            position = None
            if m.rot is not None:
                position = f"rot{i}"
                positions[position] = PartSpec("rotary_frequencies", {"base": m.rot.base, "dims": m.rot.dims, "factor": m.rot.factor,
                                                                      "interleaved": True})
            names = {role: f"{p}mix.{role}" for role in ("q", "dkv", "uk", "uv", "o", "sink", "g")}
            names["dkv_norm"] = f"{p}mix.dkv.norm"
            mixer = PartSpec("latent_attention", {"hidden_size": width, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim,
                                                  "rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "own_latent": True,
                                                  "rot_dim": m.rot_dim, "position": position, "window": m.window, "sink": "learned",
                                                  "gate": "sigmoid_head"}, names)
        elif isinstance(m, BiasedAttentionConfig):
            names = {role: f"{p}mix.{role}" for role in ("q", "k", "v", "o")}
            names.update({f"{role}_bias": f"{p}mix.{role}.b" for role in ("q", "k", "v")})
            value_mix = None
            if m.v_mix:
                value_mix = "later" if mixing_seen else "first"
                mixing_seen = True
                names["vmix"] = f"{p}mix.vmix"
            mixer = PartSpec("masked_attention", {"hidden_size": width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                                                  "value_dim": m.vdim, "scale": m.scale, "window": m.window, "keep_first": m.keep_first,
                                                  "softcap": m.softcap, "slopes": [2.0 ** (-SLOPE_EXPONENT * (h + 1) / m.heads) for h in range(m.heads)],
                                                  "bias": True, "unit_qk": True, "unit_v": True, "eps": cfg.norm_eps, "value_mix": value_mix},
                             names)
        else:
            raise TypeError(type(m).__name__)
        schedule.append(Run(i))
        ff = None
        if layer.mlp is not None:
            names = {role: f"{p}mlp.{role}" for role in ("gate", "up", "down")}
            names.update({f"{role}_bias": f"{p}mlp.{role}.b" for role in ("gate", "up", "down")})
            ff = PartSpec("gated_bias", {"hidden_size": width, "intermediate_size": layer.mlp.ff, "activation": "swish", "alpha": SWISH_ALPHA,
                                         "limit": layer.mlp.limit, "up_offset": UP_OFFSET}, names)
        block = PartSpec("parallel_residual", {"width": width, "states": i + 1, "total_states": count + 1}, {"depth": f"{p}dwa"})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ff, norms={"pre": layer_norm(p + "norm1")}))
    embedding = PartSpec("hashed_embedding", {"vocab_size": cfg.vocab_size, "width": width, "streams": 1, "scale": cfg.embedding_scale,
                                              "buckets": 0}, {"weight": "embed"})
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding=embedding, positions=positions, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=layer_norm("final.norm"), lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "width": width}, {"weight": "head"}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture("Sopetar", SopetarConfig, sopetar_plan)
