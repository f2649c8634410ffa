"""Rimopel: from its typed configuration to a model description.

A decoder whose layers are listed one by one in config.json, each with a mixer of its own sizes and an optional dense
feed-forward.  Token embedding plus a sinusoid of the position; every sublayer reads the residual stream itself, and
what it returns is gated, normed and then added (``gated_postnorm``); the mixer's input passes a causal convolution
first; the one mixer type, "attention", is grouped-query attention without rotation over a sliding window that keeps
a request's first keys, with biased projections, a short convolution on q, k and v, unit-norm queries and keys, a
scale from the configuration and a logarithmic distance penalty per head (``conv_window_attention``).  Final norm,
untied head.

Tensor names: ``embed``, ``head``, ``final.norm``; layer i under ``l<i>.``: ``norm1``, ``norm2``, ``canon1``,
``rg1``(+``.b``), ``rg2``(+``.b``), ``mix.{q,k,v}`` (+``.b``, ``.conv``), ``mix.r1``, ``mix.r2``, ``mix.o``,
``mlp.up``, ``mlp.down``.  This file only writes data.
"""
from __future__ import annotations

from ..config.base import ConfigError
from ..config.rimopel import RimopelConfig
from ..registry import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture

SINUSOID_BASE = 10000.0


def _attention(cfg: RimopelConfig, m) -> PartSpec:
    return PartSpec("conv_window_attention", {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
        "scale": m.scale, "window": m.window, "keep_first": m.keep_first, "conv_taps": m.conv, "eps": cfg.norm_eps,
        "unit_norm": True, "distance_penalty": True, "bias": True})


MIXERS = {"attention": _attention}      # layer type -> its mixer's description


def describe_rimopel(cfg: RimopelConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "name": ""})
    block = PartSpec("gated_postnorm", {"hidden_size": cfg.width, "conv_taps": cfg.canon_taps, "gated": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.type not in MIXERS:
            raise ConfigError(f"layer {i}: no mixer of type '{layer.type}' (known: {sorted(MIXERS)})")
        parts = {"norm1": (norm, "norm1"), "mixer": (MIXERS[layer.type](cfg, layer.mixer), "mix.")}
        if layer.mlp_kind is not None:
            ffn = PartSpec(layer.mlp_kind, {"hidden_size": cfg.width, "intermediate_size": layer.ff, "activation": "gelu_erf",
                                            "up_tensor": "up", "down_tensor": "down"})
            parts.update({"norm2": (norm, "norm2"), "feed_forward": (ffn, "mlp.")})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, parts=parts))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions, embed_tensor="embed",
        layers=tuple(layers), order=tuple(LayerRun(layer=i, cache=i, writes=True) for i in range(len(layers))),
        final_norm=norm, final_norm_prefix="final.norm", lm_head_tensor="head",
        embedding=PartSpec("sinusoidal_token_embedding", {"tensor": "embed", "vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                                          "base": SINUSOID_BASE}))


register_architecture("Rimopel", RimopelConfig, describe_rimopel)
