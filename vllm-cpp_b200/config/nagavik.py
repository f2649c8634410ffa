"""Nagavik configuration, from the keys of its config.json.

The file lists the layers one by one::

    {"architecture": "Nagavik", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e},
     "embedding": {"scale": s}, "logit_softcap": c,
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s, "softcap": c},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "mamba2",
                 "mixer": {"heads": H, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": g},
                 "mlp": {"kind": "moe", "router": {"experts": E, "top": k}, "expert": {"ff": F},
                         "shared": {"ff": Fs} | null} | null}, ...]}

Every size and constant is read from there; a layer may differ from the next in all of them.  A cap that is left
out (``logit_softcap``, a mixer's ``softcap``) means no cap, ``embedding.scale`` left out means 1, ``shared`` left
out or null means no shared expert, ``mlp`` null a layer without a feed-forward.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, KeyReader, ModelConfig

MIXER_TYPES = ("attention", "mamba2")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class NagavikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0       # 0: scores are not capped

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        out = cls(heads=r.integer("heads", minimum=1), kv_heads=r.integer("kv_heads", minimum=1), dim=r.integer("dim", minimum=1),
                  vdim=r.integer("vdim", minimum=1), scale=r.number("scale"), softcap=r.number("softcap", 0.0))
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}: 'kv_heads' must divide 'heads'")
        if out.softcap < 0:
            raise ConfigError(f"{where}: 'softcap' must not be negative")
        return out

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class NagavikMamba2:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        out = cls(heads=r.integer("heads", minimum=1), vdim=r.integer("vdim", minimum=1), state=r.integer("state", minimum=1),
                  groups=r.integer("groups", 1, minimum=1), conv=r.integer("conv", minimum=1),
                  norm_groups=r.integer("norm_groups", 1, minimum=1))
        if out.heads % out.groups:
            raise ConfigError(f"{where}: 'groups' must divide 'heads'")
        if (out.heads * out.vdim) % out.norm_groups:
            raise ConfigError(f"{where}: 'norm_groups' must divide heads * vdim")
        return out

    def to_dict(self):
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class NagavikMlp:
    kind: str                  # "dense" or "moe"
    ff: int = 0                # dense: hidden size; moe: an expert's hidden size
    experts: int = 0
    top: int = 0
    shared_ff: int = 0         # 0: no shared expert

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        kind = r.string("kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"{where}: kind '{kind}' is not one of {MLP_KINDS}")
        if kind == "dense":
            return cls(kind, ff=r.integer("ff", minimum=1))
        for key in ("router", "expert"):
            if not isinstance(data.get(key), dict):
                raise ConfigError(f"{where}: required key '{key}' is missing")
        router = KeyReader(data["router"], where + ".router")
        out = cls(kind, ff=KeyReader(data["expert"], where + ".expert").integer("ff", minimum=1),
                  experts=router.integer("experts", minimum=1), top=router.integer("top", minimum=1),
                  shared_ff=KeyReader(data["shared"], where + ".shared").integer("ff", minimum=1) if data.get("shared") else 0)
        if out.top > out.experts:
            raise ConfigError(f"{where}.router: 'top' exceeds 'experts'")
        return out

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff},
                "shared": {"ff": self.shared_ff} if self.shared_ff else None}


@dataclass(frozen=True)
class NagavikLayer:
    type: str
    mixer: Any
    mlp: NagavikMlp | None = None

    @classmethod
    def from_dict(cls, data, where):
        r = KeyReader(data, where)
        kind = r.string("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"{where}: layer type '{kind}' is not one of {MIXER_TYPES}")
        if not isinstance(data.get("mixer"), dict):
            raise ConfigError(f"{where}: required key 'mixer' is missing")
        mixer_cls = NagavikAttention if kind == "attention" else NagavikMamba2
        mlp = data.get("mlp")
        return cls(kind, mixer_cls.from_dict(data["mixer"], where + ".mixer"),
                   None if mlp is None else NagavikMlp.from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class NagavikConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple
    max_positions: int
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0       # 0: logits are not capped
    architecture: str = "Nagavik"
    extra: dict = field(default_factory=dict, compare=False)

    def __post_init__(self):
        object.__setattr__(self, "layers", tuple(self.layers))
        if not self.layers:
            raise ConfigError("a model needs at least one layer")

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "NagavikConfig":
        r = KeyReader(data)
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = KeyReader(data.get("norm") or {}, "config.json.norm")
        emb = KeyReader(data.get("embedding") or {}, "config.json.embedding")
        cap = r.number("logit_softcap", 0.0)
        if cap < 0:
            raise ConfigError("config.json: 'logit_softcap' must not be negative")
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   layers=tuple(NagavikLayer.from_dict(l, f"config.json.layers[{i}]") for i, l in enumerate(layers)),
                   max_positions=r.integer("max_positions", minimum=1), norm_eps=norm.number("eps", positive=True),
                   embedding_scale=emb.number("scale", 1.0), logit_softcap=cap,
                   architecture=r.string("architecture", "Nagavik"))

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
             "layers": [l.to_dict() for l in self.layers]}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d
