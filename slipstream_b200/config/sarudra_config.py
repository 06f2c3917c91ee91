"""Typed configuration of the Sarudra decoder.

``config.json`` is nested like the other designs of this family: ``vocab``, ``width``, ``norm.{eps, groups}``,
``embedding.scale``, ``logit_softcap`` and a list ``layers`` whose entries carry ``type`` (``mamba2`` or
``attention``), ``mixer`` (the mixer's sizes and constants) and ``mlp`` (``kind`` ``dense`` or ``moe``, or null
for a layer without feed-forward).  Every size and constant that may differ between two models is read from the
file; what the file does not mention is off (no ``mask``: every earlier key; no ``rot``: no rotation, of
queries, keys or values; no ``softcap`` / ``logit_softcap``: none; no ``shared``: no shared expert).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, ClassVar

from .fokedra_config import RotaryConfig
from .model_config import ModelConfigBase
from .reader import ConfigError, ConfigReader


@dataclass(frozen=True)
class WindowedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig | None = None
    window: int | None = None  # mask.size: a query sees itself and the window - 1 tokens before it
    softcap: float | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "WindowedAttentionConfig":
        r = ConfigReader(data, where=where)
        heads, dim = r.integer("heads"), r.integer("dim")
        rot, mask = r.table("rot"), r.table("mask")
        window = ConfigReader(mask, where=f"{where}.mask").integer("size", None) if mask else None
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", heads), dim=dim, vdim=r.integer("vdim", dim),
                  scale=r.number("scale", dim ** -0.5), rot=RotaryConfig.from_dict(rot, f"{where}.rot") if rot else None,
                  window=window, softcap=r.number("softcap", None))
        if out.heads < 1 or out.kv_heads < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
        if out.dim < 2 or out.dim % 2 or out.vdim < 1:
            raise ConfigError(f"{where}: dim must be even and >= 2, vdim >= 1")
        if out.rot is not None and (out.rot.dims > out.dim or out.rot.scaling is not None):
            raise ConfigError(f"{where}: rot.dims exceeds dim, or rot.scaling is given (this design has none)")
        if out.rot is not None and out.vdim % 2:
            raise ConfigError(f"{where}: rotated values need an even vdim")
        if out.window is not None and out.window < 1:
            raise ConfigError(f"{where}: mask.size must be >= 1")
        if out.softcap is not None and not out.softcap > 0.0:
            raise ConfigError(f"{where}: softcap must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                               "vdim": self.vdim}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "StateSpaceConfig":
        r = ConfigReader(data, where=where)
        out = cls(heads=r.integer("heads"), vdim=r.integer("vdim"), state=r.integer("state"), groups=r.integer("groups", 1),
                  conv=r.integer("conv", 4), norm_groups=r.integer("norm_groups", 1))
        if out.heads < 1 or out.groups < 1 or out.heads % out.groups:
            raise ConfigError(f"{where}: heads ({out.heads}) must be a multiple of groups ({out.groups})")
        if out.vdim < 1 or not 1 <= out.state <= 256 or not 1 <= out.conv <= 8:
            raise ConfigError(f"{where}: vdim >= 1, state 1..256 and conv 1..8 are what the kernels take")
        if out.norm_groups < 1 or (out.heads * out.vdim) % out.norm_groups:
            raise ConfigError(f"{where}: heads * vdim does not split into norm_groups ({out.norm_groups}) equal parts")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" or "moe"
    ff: int  # dense: the hidden size; moe: each expert's
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "FeedForwardConfig":
        r = ConfigReader(data, where=where)
        kind = r.text("kind", "dense")
        if kind == "dense":
            out = cls(kind=kind, ff=r.integer("ff"))
        elif kind == "moe":
            expert = ConfigReader(r.table("expert") or {}, where=f"{where}.expert")
            router = ConfigReader(r.table("router") or {}, where=f"{where}.router")
            shared = r.table("shared")
            out = cls(kind=kind, ff=expert.integer("ff"), experts=router.integer("experts"), top=router.integer("top", 1),
                      shared_ff=ConfigReader(shared, where=f"{where}.shared").integer("ff") if shared else None)
            if not 1 <= out.top <= out.experts or out.experts > 1024:
                raise ConfigError(f"{where}: router.top must be between 1 and router.experts, experts at most 1024")
            if out.shared_ff is not None and out.shared_ff < 1:
                raise ConfigError(f"{where}: shared.ff must be >= 1")
        else:
            raise ConfigError(f"{where}: unsupported feed-forward kind {kind!r} (known: dense, moe)")
        if out.ff < 1:
            raise ConfigError(f"{where}: ff must be >= 1")
        return out

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        out: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class SarudraLayerConfig:
    type: str  # "mamba2" or "attention"
    mixer: "WindowedAttentionConfig | StateSpaceConfig"
    mlp: FeedForwardConfig | None

    def to_dict(self) -> dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None, "type": self.type}


_MIXERS = {"attention": WindowedAttentionConfig, "mamba2": StateSpaceConfig}


@dataclass(frozen=True)
class SarudraConfig(ModelConfigBase):
    architecture: ClassVar[str] = "Sarudra"

    max_position_embeddings: int = 131072  # the design names no limit; this bounds a request for the cache manager
    layers: tuple[SarudraLayerConfig, ...] = ()
    norm_eps: float = 1e-6
    norm_groups: int = 1
    embedding_scale: float = 1.0
    logit_softcap: float | None = None
    extra: dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("vocab and width must be >= 1 and there must be a layer")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
        if self.norm_groups < 1 or self.hidden_size % self.norm_groups:
            raise ConfigError(f"width ({self.hidden_size}) does not split into norm.groups ({self.norm_groups}) equal parts")
        if self.logit_softcap is not None and not self.logit_softcap > 0.0:
            raise ConfigError("logit_softcap must be positive")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"unsupported torch_dtype: {self.torch_dtype}")

    @classmethod
    def from_dict(cls, data: dict[str, Any], generation: dict[str, Any] | None = None) -> "SarudraConfig":
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
            if kind not in _MIXERS:
                raise ConfigError(f"layers[{i}].type {kind!r} is not a mixer of this design (known: {', '.join(sorted(_MIXERS))})")
            mixer = lr.table("mixer")
            if mixer is None:
                raise ConfigError(f"layers[{i}] lacks its mixer")
            mlp = lr.table("mlp")
            layers.append(SarudraLayerConfig(
                type=kind, mixer=_MIXERS[kind].from_dict(mixer, f"layers[{i}].mixer"),
                mlp=FeedForwardConfig.from_dict(mlp, f"layers[{i}].mlp") if mlp is not None else None))
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
            norm_groups=norm.integer("groups", 1),
            embedding_scale=embedding.number("scale", 1.0),
            logit_softcap=r.number("logit_softcap", None),
            extra=r.leftover(also_known=("architecture", "architectures")),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                               "layers": [layer.to_dict() for layer in self.layers],
                               "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                               "vocab": self.vocab_size, "width": self.hidden_size,
                               "max_position_embeddings": self.max_position_embeddings, "torch_dtype": self.torch_dtype}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        for key in ("eos_token_id", "bos_token_id", "pad_token_id"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        out.update({k: v for k, v in self.extra.items() if k not in out})
        return out
