"""Nagavik: from its typed configuration to a model description.

A decoder whose layers are listed one by one in config.json.  Token embedding times a constant plus a learned vector
per position; every sublayer has a norm in front of it and another on what it returns, which is then multiplied by a
learned scale per channel and added (``sandwich_norm``).  Two mixer types: "attention" -- grouped-query attention
without rotation, queries and keys normed over the whole projection with a gain per lane, scores scaled, capped by a
tanh, less a slope per head times the distance, softmax with a silent sink -- and "mamba2", a selective state-space
recurrence with a short convolution in front and a gated norm in groups behind.  Two feed-forwards: a dense one with a
tanh-GELU gate and biases, and routed experts (square-of-ReLU, sigmoid router weights on the experts' input) with a
shared expert.  Final norm, untied head, capped logits.

Tensor names: ``embed``, ``pos``, ``head``, ``final.norm``; layer i under ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``,
``norm2b``, ``ls1``, ``ls2``; attention ``mix.{q,k,v,o}``, ``mix.q.norm``, ``mix.k.norm``; mamba2 ``mix.{in,conv,conv.b,
dt_bias,A_log,D,norm,o}``; dense ``mlp.{gate,up,down}`` (+ ``.b``); experts ``mlp.router``, ``mlp.e<j>.{up,down}``,
``mlp.shared.{up,down}``.  This file only writes data.
"""
from __future__ import annotations

from ..config.base import ConfigError
from ..config.nagavik import NagavikConfig
from ..registry import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture

SLOPE_EXPONENT = 8.0     # slope of head h (from 0) of H: 2^(-8 (h + 1) / H)


def _attention(cfg: NagavikConfig, m) -> PartSpec:
    return PartSpec("conv_window_attention", {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
        "scale": m.scale, "window": 0, "conv_taps": 0, "eps": cfg.norm_eps, "unit_norm": False, "distance_penalty": False,
        "bias": False, "whole_norm": True, "softcap": m.softcap, "slope_exponent": SLOPE_EXPONENT, "sink": True})


def _mamba2(cfg: NagavikConfig, m) -> PartSpec:
    return PartSpec("mamba2", {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.vdim, "state_size": m.state,
                               "groups": m.groups, "conv_taps": m.conv, "norm_groups": m.norm_groups, "eps": cfg.norm_eps})


MIXERS = {"attention": _attention, "mamba2": _mamba2}      # layer type -> its mixer's description


def _feed_forward(cfg: NagavikConfig, mlp) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "activation": "gelu_tanh",
                                      "bias": True})
    return PartSpec("routed_experts", {"hidden_size": cfg.width, "num_experts": mlp.experts, "top": mlp.top,
                                       "expert_size": mlp.ff, "shared_size": mlp.shared_ff, "activation": "relu2",
                                       "router_weights": "sigmoid", "weight_on": "input"})


def describe_nagavik(cfg: NagavikConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "name": ""})
    block = PartSpec("sandwich_norm", {"hidden_size": cfg.width, "layer_scale": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.type not in MIXERS:
            raise ConfigError(f"layer {i}: no mixer of type '{layer.type}' (known: {sorted(MIXERS)})")
        parts = {"norm1": (norm, "norm1"), "mixer": (MIXERS[layer.type](cfg, layer.mixer), "mix."), "norm1b": (norm, "norm1b", "norm")}
        if layer.mlp is not None:
            parts.update({"norm2": (norm, "norm2"), "feed_forward": (_feed_forward(cfg, layer.mlp), "mlp."),
                          "norm2b": (norm, "norm2b", "norm")})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, parts=parts))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions, embed_tensor="embed",
        layers=tuple(layers), order=tuple(LayerRun(layer=i, cache=i, writes=True) for i in range(len(layers))),
        final_norm=norm, final_norm_prefix="final.norm", lm_head_tensor="head",
        embedding=PartSpec("positional_token_embedding", {"tensor": "embed", "position_tensor": "pos", "vocab_size": cfg.vocab,
                                                          "hidden_size": cfg.width, "max_positions": cfg.max_positions,
                                                          "scale": cfg.embedding_scale}),
        head=PartSpec("lm_head", {"tensor": "head", "vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                  "softcap": cfg.logit_softcap}))


register_architecture("Nagavik", NagavikConfig, describe_nagavik)
