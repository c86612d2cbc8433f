"""Sokolorn as a model plan: layers whose sub-layers read the residual stream as it is and whose norm stands BEHIND
each sub-layer (`x += norm(mixer(x))`, `x += norm(ff(x))`, the `sandwich` block with `identity` norms in front), an RMS norm
whose weight is stored around zero (`offset` 1); mixers of two kinds, both `masked_attention`: one without rotation, with q
and k normed over the whole projection, a sliding window, a learned sink per head and a sigmoid gate per head; one with
biases, q and k normed per head by one shared weight, rotation of the first values of a head with frequencies whose long
wavelengths are slowed down, causal, which may read the keys and values an earlier layer cached instead of making its own;
a feed-forward that is either `W_down relu(W_up x)^2` or routed experts with a clamped gate, a softmax over the chosen
logits and a gated shared expert; logits from the embedding table, capped by a tanh.  This module only turns a
`SokolornConfig` into data; the parts live in `parts/`.
Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.{q,k,v,o}[.b]`, `l<i>.mix.{q,k}.norm`, `l<i>.mix.{sink,g}`,
`l<i>.mlp.{up,down}`, `l<i>.mlp.{router[.b], e<j>.{gate,up,down}, shared.{gate,up,down,sg}}`, `final.norm`.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelPlan, PartSpec, Run
from ..config.registry import register_architecture
from ..config.sokolorn import SokolornConfig

SWISH_ALPHA = 1.702          # an expert's y = g * sigmoid(1.702 g) * (u + 1)
UP_OFFSET = 1.0
NORM_OFFSET = 1.0            # a norm's weight is stored as its distance from one


def sokolorn_plan(cfg: SokolornConfig) -> ModelPlan:
    width = cfg.width
    norm = lambda name: PartSpec("group_rmsnorm", {"width": width, "groups": 1, "eps": cfg.norm_eps, "offset": NORM_OFFSET}, {"weight": name})
    plain = PartSpec("identity", {"width": width})
    positions, layers, schedule = {}, [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        own_kv = m.kv_from is None
        names = {role: f"{p}mix.{role}" for role in (("q", "k", "v", "o") if own_kv else ("q", "o"))}
        names["q_norm"] = f"{p}mix.q.norm"
        if own_kv:
            names["k_norm"] = f"{p}mix.k.norm"
        params = {"hidden_size": width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                  "scale": m.scale, "eps": cfg.norm_eps, "own_kv": own_kv}
        if layer.type == "attention":
            names.update({"sink": f"{p}mix.sink", "g": f"{p}mix.g"})
            params.update({"qk_norm": "whole", "window": m.window, "sink": "learned", "gate": "sigmoid_head"})
        else:
            names.update({f"{role}_bias": f"{p}mix.{role}.b" for role in (("q", "k", "v") if own_kv else ("q",))})
            params.update({"qk_norm": "head", "bias": True, "dense_kernels": True})
            if m.rot is not None:
                s = m.rot.scaling
                params["position"] = f"rot{i}"
                positions[params["position"]] = PartSpec("rotary_frequencies", {
                    "base": m.rot.base, "dims": m.rot.dims,
                    "scaling": {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original} if s is not None else None})
        mixer = PartSpec("masked_attention", params, names)
        schedule.append(Run(i, m.kv_from))
        ff = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ff = PartSpec("plain", {"hidden_size": width, "intermediate_size": layer.mlp.ff, "activation": "relu2"},
                          {role: f"{p}mlp.{role}" for role in ("up", "down")})
        elif layer.mlp is not None:
            e = layer.mlp
            names = {"router": p + "mlp.router", "router_bias": p + "mlp.router.b"}
            for j in range(e.experts):
                names.update({f"e{j}.{role}": f"{p}mlp.e{j}.{role}" for role in ("gate", "up", "down")})
            if e.shared is not None:
                names.update({f"shared.{role}": f"{p}mlp.shared.{role}" for role in ("gate", "up", "down", "sg")})
            ff = PartSpec("routed_experts", {"hidden_size": width, "intermediate_size": e.expert.ff, "experts": e.experts, "top": e.top,
                                             "router": "softmax_of_chosen", "activation": "swish", "alpha": SWISH_ALPHA,
                                             "up_offset": UP_OFFSET, "limit": e.expert.limit,
                                             "shared_intermediate_size": e.shared.ff if e.shared is not None else None,
                                             "shared_limit": e.shared.limit if e.shared is not None else None}, names)
        norms = {"pre_mixer": plain, "post_mixer": norm(p + "norm1")}
        if ff is not None:
            norms.update({"pre_feed_forward": plain, "post_feed_forward": norm(p + "norm2")})
        layers.append(LayerSpec(block="sandwich", mixer=mixer, feed_forward=ff, norms=norms))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=width, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": width}, {"weight": "embed"}),
        positions=positions, layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "width": width, "softcap": cfg.logit_softcap}, {"weight": "embed"}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture("Sokolorn", SokolornConfig, sokolorn_plan)
