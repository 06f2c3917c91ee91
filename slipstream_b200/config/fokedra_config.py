"""Typed configuration of the Fokedra decoder.

The design's ``config.json`` is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, an optional
``streams`` count (hyper-connected residual streams; absent: the ordinary residual sum) and a list ``layers``
whose entries carry ``type`` (the kind of mixer), ``mixer`` (its sizes and constants) and ``mlp`` (the
feed-forward, or null for none).  Every size and every constant that may differ between two models of the design
is read from there; what the file does not mention is off (no mask: every earlier key; no ``rot``: no rotation;
no ``rot.scaling``: the plain frequencies; no ``kv_from``: keys and values of the layer's own).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, ClassVar

from .model_config import ModelConfigBase
from .reader import ConfigError, ConfigReader


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: tuple[float, float, float, float] | None = None  # (factor, original, fast, slow)

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "RotaryConfig":
        r = ConfigReader(data, where=where)
        scaling = r.table("scaling")
        if scaling is not None:
            s = ConfigReader(scaling, where=f"{where}.scaling")
            scaling = (s.number("factor"), s.number("original"), s.number("fast"), s.number("slow"))
        out = cls(base=r.number("base"), dims=r.integer("dims"), scaling=scaling)
        if out.dims < 2 or out.dims % 2 or not out.base > 0.0:
            raise ConfigError(f"{where}: dims must be even and >= 2, base positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return out


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig | None = None
    chunk: int | None = None  # mask.size
    kv_from: int | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "AttentionMixerConfig":
        r = ConfigReader(data, where=where)
        heads = r.integer("heads")
        dim = r.integer("dim")
        rot = r.table("rot")
        mask = r.table("mask")
        chunk = ConfigReader(mask, where=f"{where}.mask").integer("size", None) if mask else None
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", heads), dim=dim, vdim=r.integer("vdim", dim),
                  scale=r.number("scale", dim ** -0.5),
                  rot=RotaryConfig.from_dict(rot, f"{where}.rot") if rot else None, chunk=chunk,
                  kv_from=r.integer("kv_from", None))
        if out.heads < 1 or out.kv_heads < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
        if out.dim < 2 or out.dim % 2 or out.vdim < 1:
            raise ConfigError(f"{where}: dim must be even and >= 2, vdim >= 1")
        if out.rot is not None and out.rot.dims > out.dim:
            raise ConfigError(f"{where}: rot.dims ({out.rot.dims}) exceeds dim ({out.dim})")
        if out.chunk is not None and out.chunk < 1:
            raise ConfigError(f"{where}: mask.size must be >= 1")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                               "vdim": self.vdim}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class DenseFeedForwardConfig:
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "DenseFeedForwardConfig":
        r = ConfigReader(data, where=where)
        kind = r.text("kind", "dense")
        if kind != "dense":
            raise ConfigError(f"{where}: unsupported feed-forward kind {kind!r} (known: dense)")
        out = cls(ff=r.integer("ff"), limit=r.number("limit"))
        if out.ff < 1 or not out.limit > 0.0:
            raise ConfigError(f"{where}: ff must be >= 1 and limit positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"ff": self.ff, "kind": "dense", "limit": self.limit}


@dataclass(frozen=True)
class FokedraLayerConfig:
    type: str
    mixer: AttentionMixerConfig
    mlp: DenseFeedForwardConfig | None

    def to_dict(self) -> dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None, "type": self.type}


@dataclass(frozen=True)
class FokedraConfig(ModelConfigBase):
    architecture: ClassVar[str] = "Fokedra"

    max_position_embeddings: int = 131072  # the design names no limit; this bounds a request for the cache manager
    layers: tuple[FokedraLayerConfig, ...] = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    streams: int | None = None  # hyper-connected residual streams; None: one stream and the plain residual sum
    extra: dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("vocab and width must be >= 1 and there must be a layer")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise ConfigError(f"streams must be between 1 and 8, got {self.streams}")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"unsupported torch_dtype: {self.torch_dtype}")
        for i, layer in enumerate(self.layers):
            src = layer.mixer.kv_from
            if src is None:
                continue
            if not 0 <= src < i or self.layers[src].mixer.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from must name an earlier layer with keys and values of its own")
            a, b = layer.mixer, self.layers[src].mixer
            if (a.kv_heads, a.dim, a.vdim, a.rot) != (b.kv_heads, b.dim, b.vdim, b.rot):
                raise ConfigError(f"layers[{i}] reads layer {src}'s keys and values but differs in kv_heads, dim, vdim or rot")

    @classmethod
    def from_dict(cls, data: dict[str, Any], generation: dict[str, Any] | None = None) -> "FokedraConfig":
        r = ConfigReader(data, behind=generation)
        norm = ConfigReader(r.table("norm") or {}, where="norm")
        embedding = ConfigReader(r.table("embedding") or {}, where="embedding")
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}] must be an object")
            lr = ConfigReader(entry, where=f"layers[{i}]")
            kind = lr.text("type")
            if kind != "attention":
                raise ConfigError(f"layers[{i}].type {kind!r} is not a mixer of this design (known: attention)")
            mixer = lr.table("mixer")
            if mixer is None:
                raise ConfigError(f"layers[{i}] lacks its mixer")
            mlp = lr.table("mlp")
            layers.append(FokedraLayerConfig(
                type=kind, mixer=AttentionMixerConfig.from_dict(mixer, f"layers[{i}].mixer"),
                mlp=DenseFeedForwardConfig.from_dict(mlp, f"layers[{i}].mlp") if mlp is not None else None))
        return cls(
            vocab_size=r.integer("vocab"),
            hidden_size=r.integer("width"),
            num_hidden_layers=len(layers),
            max_position_embeddings=r.integer("max_position_embeddings", 131072),
            torch_dtype=r.precision("torch_dtype", "dtype"),
            eos_token_id=r.token_id("eos_token_id"),
            bos_token_id=r.token_id("bos_token_id"),
            pad_token_id=r.token_id("pad_token_id"),
            layers=tuple(layers),
            norm_eps=norm.number("eps", 1e-6),
            embedding_scale=embedding.number("scale", 1.0),
            streams=r.integer("streams", None),
            extra=r.leftover(also_known=("architecture", "architectures")),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                               "layers": [layer.to_dict() for layer in self.layers], "norm": {"eps": self.norm_eps},
                               "vocab": self.vocab_size, "width": self.hidden_size,
                               "max_position_embeddings": self.max_position_embeddings, "torch_dtype": self.torch_dtype}
        if self.streams is not None:
            out["streams"] = self.streams
        for key in ("eos_token_id", "bos_token_id", "pad_token_id"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        out.update({k: v for k, v in self.extra.items() if k not in out})
        return out
