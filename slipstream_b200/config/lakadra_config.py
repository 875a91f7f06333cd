"""Typed configuration of the Lakadra decoder.

``config.json`` is nested like the other designs of this family: ``vocab``, ``width``, ``norm.eps``, ``logit_scale``,
``logit_softcap`` and a list ``layers`` whose entries carry ``type`` (``lightning``, ``latent_attention`` or
``parallel``), ``mixer`` (the mixer's sizes and constants; a ``parallel`` mixer holds a ``left`` attention, a ``right``
recurrence and a scale for each) and ``mlp`` (``kind`` ``moe``, or null for a layer without a feed-forward).  Every
size and every constant that may differ between two models of the design is read from there; what the file does not
name is off (no ``mask``: every earlier key; no ``rot``: no rotation; no ``rot.scaling``: the plain frequencies; no
``groups``: every expert may be chosen; no ``identity``: no identity experts; no ``shared``: no shared expert; no
``logit_scale`` / ``logit_softcap``: the head's output as it is).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, ClassVar

from .bezutar_config import LatentAttentionConfig
from .model_config import ModelConfigBase
from .reader import ConfigError, ConfigReader


@dataclass(frozen=True)
class ScaledRotaryConfig:
    """Rotation of the first ``dims`` elements of a head with frequencies ``base^(-2i/dims) / factor``."""

    base: float
    dims: int
    factor: float = 1.0

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "ScaledRotaryConfig":
        r = ConfigReader(data, where=where)
        scaling = r.table("scaling")
        factor = ConfigReader(scaling, where=f"{where}.scaling").number("factor", 1.0) if scaling else 1.0
        out = cls(base=r.number("base"), dims=r.integer("dims"), factor=factor)
        if out.dims < 2 or out.dims % 2 or not out.base > 0.0 or not out.factor > 0.0:
            raise ConfigError(f"{where}: dims must be even and >= 2, base and scaling.factor positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor != 1.0:
            out["scaling"] = {"factor": self.factor}
        return out


@dataclass(frozen=True)
class DecayedLinearAttentionConfig:
    """``lightning``: ``heads`` heads of ``dim`` query/key elements and ``vdim`` values, one decay per head."""

    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "DecayedLinearAttentionConfig":
        r = ConfigReader(data, where=where)
        dim, decay = r.integer("dim"), r.raw("decay")
        if not isinstance(decay, list) or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"{where}.decay must be a list of numbers")
        out = cls(heads=r.integer("heads"), dim=dim, vdim=r.integer("vdim", dim), decay=tuple(float(d) for d in decay))
        if out.heads < 1 or not 1 <= out.dim <= 256 or out.vdim < 1 or len(out.decay) != out.heads:
            raise ConfigError(f"{where}: heads and vdim must be >= 1, dim between 1 and 256, one decay per head")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class SinkAttentionConfig:
    """The attention side of a ``parallel`` mixer: grouped-query heads with biases, an optional sliding window
    (``mask.size``), a softmax with one more 1 in its denominator and a gate per head."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: ScaledRotaryConfig | None = None
    window: int | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "SinkAttentionConfig":
        r = ConfigReader(data, where=where)
        heads, dim = r.integer("heads"), r.integer("dim")
        rot, mask = r.table("rot"), r.table("mask")
        out = cls(heads=heads, kv_heads=r.integer("kv_heads", heads), dim=dim, vdim=r.integer("vdim", dim),
                  scale=r.number("scale", dim ** -0.5),
                  rot=ScaledRotaryConfig.from_dict(rot, f"{where}.rot") if rot else None,
                  window=ConfigReader(mask, where=f"{where}.mask").integer("size", None) if mask else None)
        if out.heads < 1 or out.kv_heads < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
        if out.dim < 2 or out.dim % 2 or out.dim > 256 or not 1 <= out.vdim <= 256:
            raise ConfigError(f"{where}: dim must be even and between 2 and 256, vdim between 1 and 256")
        if out.rot is not None and out.rot.dims > out.dim:
            raise ConfigError(f"{where}: rot.dims ({out.rot.dims}) exceeds dim ({out.dim})")
        if out.window is not None and out.window < 1:
            raise ConfigError(f"{where}: mask.size must be >= 1")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                               "vdim": self.vdim}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class GatedLinearRecurrenceConfig:
    """The recurrent side of a ``parallel`` mixer: ``width`` channels, gates in ``blocks`` square blocks, a causal
    convolution of ``conv`` taps."""

    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "GatedLinearRecurrenceConfig":
        r = ConfigReader(data, where=where)
        out = cls(width=r.integer("width"), blocks=r.integer("blocks", 1), conv=r.integer("conv", 1))
        if out.width < 1 or out.blocks < 1 or out.width % out.blocks or not 1 <= out.conv <= 8:
            raise ConfigError(f"{where}: width must split into blocks equal parts, conv between 1 and 8")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"blocks": self.blocks, "conv": self.conv, "width": self.width}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SinkAttentionConfig
    right: GatedLinearRecurrenceConfig
    left_scale: float = 1.0
    right_scale: float = 1.0

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "ParallelMixerConfig":
        r = ConfigReader(data, where=where)
        left, right = r.table("left"), r.table("right")
        if left is None or right is None:
            raise ConfigError(f"{where}: a parallel mixer has a left and a right side")
        return cls(left=SinkAttentionConfig.from_dict(left, f"{where}.left"),
                   right=GatedLinearRecurrenceConfig.from_dict(right, f"{where}.right"),
                   left_scale=r.number("left_scale", 1.0), right_scale=r.number("right_scale", 1.0))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class RoutedFeedForwardConfig:
    """``moe``: ``experts`` small feed-forwards and ``identity`` experts that hand their input on, ``top`` chosen per
    token among the best ``group_keep`` of ``group_count`` equal groups of neighbours; an optional shared expert."""

    ff: int
    experts: int
    top: int
    identity: int = 0
    group_count: int | None = None
    group_keep: int | None = None
    shared_ff: int | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "RoutedFeedForwardConfig":
        r = ConfigReader(data, where=where)
        kind = r.text("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}: unsupported feed-forward kind {kind!r} (known: moe)")
        expert = ConfigReader(r.table("expert") or {}, where=f"{where}.expert")
        router = ConfigReader(r.table("router") or {}, where=f"{where}.router")
        groups, shared = router.table("groups"), r.table("shared")
        g = ConfigReader(groups, where=f"{where}.router.groups") if groups else None
        out = cls(ff=expert.integer("ff"), experts=router.integer("experts"), top=router.integer("top", 1),
                  identity=router.integer("identity", 0), group_count=g.integer("count") if g else None,
                  group_keep=g.integer("keep") if g else None,
                  shared_ff=ConfigReader(shared, where=f"{where}.shared").integer("ff") if shared else None)
        slots = out.experts + out.identity
        if out.ff < 1 or out.experts < 1 or out.identity < 0 or slots > 1024 or not 1 <= out.top <= slots:
            raise ConfigError(f"{where}: ff and experts must be >= 1, experts + identity at most 1024, top within them")
        if out.group_count is not None:
            if out.group_count < 1 or slots % out.group_count or not 1 <= out.group_keep <= out.group_count:
                raise ConfigError(f"{where}: experts + identity must split into groups.count groups, keep within them")
            if out.top > out.group_keep * (slots // out.group_count):
                raise ConfigError(f"{where}: router.top exceeds the experts of the groups that are kept")
        if out.shared_ff is not None and out.shared_ff < 1:
            raise ConfigError(f"{where}: shared.ff must be >= 1")
        return out

    def to_dict(self) -> dict[str, Any]:
        router: dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.identity:
            router["identity"] = self.identity
        if self.group_count is not None:
            router["groups"] = {"count": self.group_count, "keep": self.group_keep}
        out: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe", "router": router}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


MIXER_CONFIGS = {"lightning": DecayedLinearAttentionConfig, "latent_attention": LatentAttentionConfig,
                 "parallel": ParallelMixerConfig}


@dataclass(frozen=True)
class LakadraLayerConfig:
    type: str
    mixer: "DecayedLinearAttentionConfig | LatentAttentionConfig | ParallelMixerConfig"
    mlp: RoutedFeedForwardConfig | None

    def to_dict(self) -> dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None, "type": self.type}


@dataclass(frozen=True)
class LakadraConfig(ModelConfigBase):
    architecture: ClassVar[str] = "Lakadra"

    max_position_embeddings: int = 131072  # the design names no limit; this bounds a request for the cache manager
    layers: tuple[LakadraLayerConfig, ...] = ()
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    logit_softcap: float | None = None
    extra: dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("vocab and width must be >= 1 and there must be a layer")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
        if self.logit_softcap is not None and not self.logit_softcap > 0.0:
            raise ConfigError("logit_softcap must be positive")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"unsupported torch_dtype: {self.torch_dtype}")
        for i, layer in enumerate(self.layers):
            src = getattr(layer.mixer, "kv_from", None)
            if src is None:
                continue
            if not 0 <= src < i or getattr(self.layers[src].mixer, "kv_from", 0) is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from must name an earlier latent-attention layer with a latent of its own")
            a, b = layer.mixer, self.layers[src].mixer
            if (a.kv_rank, a.rot_dim, a.rot) != (b.kv_rank, b.rot_dim, b.rot):
                raise ConfigError(f"layers[{i}] reads layer {src}'s latent but differs in kv_rank, rot_dim or rot")

    @classmethod
    def from_dict(cls, data: dict[str, Any], generation: dict[str, Any] | None = None) -> "LakadraConfig":
        r = ConfigReader(data, behind=generation)
        norm = ConfigReader(r.table("norm") or {}, where="norm")
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}] must be an object")
            lr = ConfigReader(entry, where=f"layers[{i}]")
            kind = lr.text("type")
            if kind not in MIXER_CONFIGS:
                raise ConfigError(f"layers[{i}].type {kind!r} is not a mixer of this design (known: {', '.join(MIXER_CONFIGS)})")
            mixer = lr.table("mixer")
            if mixer is None:
                raise ConfigError(f"layers[{i}] lacks its mixer")
            mlp = lr.table("mlp")
            layers.append(LakadraLayerConfig(
                type=kind, mixer=MIXER_CONFIGS[kind].from_dict(mixer, f"layers[{i}].mixer"),
                mlp=RoutedFeedForwardConfig.from_dict(mlp, f"layers[{i}].mlp") if mlp is not None else None))
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
            logit_scale=r.number("logit_scale", 1.0),
            logit_softcap=r.number("logit_softcap", None),
            extra=r.leftover(also_known=("architecture", "architectures")),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
                               "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.hidden_size,
                               "max_position_embeddings": self.max_position_embeddings, "torch_dtype": self.torch_dtype}
        if self.logit_scale != 1.0:
            out["logit_scale"] = self.logit_scale
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        for key in ("eos_token_id", "bos_token_id", "pad_token_id"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        out.update({k: v for k, v in self.extra.items() if k not in out})
        return out
