"""Rimopel configuration, from the keys of its config.json.

The file lists the layers one by one::

    {"architecture": "Rimopel", "vocab": V, "width": W, "norm": {"eps": e}, "canon": {"taps": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s, "conv": n,
                           "mask": {"size": w, "keep_first": f}},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Every size and constant is read from there; a layer may differ from the next in
all of them.  ``canon`` and a mixer's ``conv`` and ``mask`` may be left out (no
input convolution, no short convolution, every earlier key visible).
``max_positions`` (optional) bounds a request's length; the design itself has no
such bound, since positions enter through a sinusoid computed on the fly and
through distances.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, KeyReader, ModelConfig

DEFAULT_MAX_POSITIONS = 1 << 20
MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class RimopelMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int = 0            # taps of the short convolution on q, k, v (0: none)
    window: int = 0          # mask.size (0: every earlier key)
    keep_first: int = 0      # mask.keep_first

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        mask = data.get("mask")
        window = keep = 0
        if mask is not None:
            m = KeyReader(mask, where + ".mask")
            window, keep = m.integer("size", minimum=1), m.integer("keep_first", 0, minimum=0)
        out = cls(heads=r.integer("heads", minimum=1), kv_heads=r.integer("kv_heads", minimum=1), dim=r.integer("dim", minimum=1),
                  vdim=r.integer("vdim", minimum=1), scale=r.number("scale"), conv=r.integer("conv", 0, minimum=0),
                  window=window, keep_first=keep)
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}: 'kv_heads' must divide 'heads'")
        return out

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.conv:
            d["conv"] = self.conv
        if self.window:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return d


@dataclass(frozen=True)
class RimopelLayer:
    type: str
    mixer: RimopelMixer
    mlp_kind: str | None = None     # None: the layer has no feed-forward
    ff: int = 0

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        kind = r.string("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"{where}: layer type '{kind}' is not one of {MIXER_TYPES}")
        if not isinstance(data.get("mixer"), dict):
            raise ConfigError(f"{where}: required key 'mixer' is missing")
        mixer = RimopelMixer.from_dict(data["mixer"], where + ".mixer")
        mlp = data.get("mlp")
        if mlp is None:
            return cls(kind, mixer)
        m = KeyReader(mlp, where + ".mlp")
        mk = m.string("kind")
        if mk not in MLP_KINDS:
            raise ConfigError(f"{where}.mlp: kind '{mk}' is not one of {MLP_KINDS}")
        return cls(kind, mixer, mk, m.integer("ff", minimum=1))

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp_kind is None else {"kind": self.mlp_kind, "ff": self.ff}}


@dataclass(frozen=True)
class RimopelConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple
    norm_eps: float = 1e-5
    canon_taps: int = 0              # taps of the convolution on what a mixer reads (0: none)
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Rimopel"
    extra: dict = field(default_factory=dict, compare=False)

    def __post_init__(self):
        object.__setattr__(self, "layers", tuple(self.layers))
        if not self.layers:
            raise ConfigError("a model needs at least one layer")

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "RimopelConfig":
        r = KeyReader(data)
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = KeyReader(data.get("norm") or {}, "config.json.norm")
        canon = data.get("canon")
        taps = KeyReader(canon, "config.json.canon").integer("taps", minimum=1) if canon is not None else 0
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   layers=tuple(RimopelLayer.from_dict(l, f"config.json.layers[{i}]") for i, l in enumerate(layers)),
                   norm_eps=norm.number("eps", positive=True), canon_taps=taps,
                   max_positions=r.integer("max_positions", DEFAULT_MAX_POSITIONS, minimum=1),
                   architecture=r.string("architecture", "Rimopel"))

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [l.to_dict() for l in self.layers]}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d
