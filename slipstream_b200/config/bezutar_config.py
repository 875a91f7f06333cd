"""Typed configuration of the Bezutar decoder.

The design's ``config.json`` is nested: ``vocab``, ``width``, ``norm.eps``, an optional ``streams`` count
(hyper-connected residual streams; absent: the ordinary residual sum), an optional ``canon.taps`` (a short causal
convolution laid over every mixer's input; absent: none), an optional ``embedding.bigram`` (a hashed table of token
pairs added to the embedding: ``buckets``, ``mul_prev``, ``mul_cur``), an optional ``max_positions`` (a learned
position table of that many rows added to the embedding) and a list ``layers`` whose entries carry ``type`` (one of
three mixers: ``mlstm``, ``mingru``, ``latent_attention``), ``mixer`` (its sizes and constants) and ``mlp`` (a dense
feed-forward, or null for none).  Every size and every constant that may differ between two models of the design is
read from there; what the file does not mention is off.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, ClassVar

from .fokedra_config import RotaryConfig
from .model_config import ModelConfigBase
from .reader import ConfigError, ConfigReader


@dataclass(frozen=True)
class MatrixMemoryConfig:
    """``mlstm``: heads of ``dim`` query/key elements and ``vdim`` values; gates capped at ``gate_cap``."""

    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "MatrixMemoryConfig":
        r = ConfigReader(data, where=where)
        dim = r.integer("dim")
        out = cls(heads=r.integer("heads"), dim=dim, vdim=r.integer("vdim", dim), gate_cap=r.number("gate_cap"))
        if out.heads < 1 or not 1 <= out.dim <= 256 or out.vdim < 1 or not out.gate_cap > 0.0:
            raise ConfigError(f"{where}: heads and vdim must be >= 1, dim between 1 and 256, gate_cap positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class GatedRecurrenceConfig:
    """``mingru``: a recurrence over ``width`` channels."""

    width: int

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "GatedRecurrenceConfig":
        out = cls(width=ConfigReader(data, where=where).integer("width"))
        if out.width < 1:
            raise ConfigError(f"{where}: width must be >= 1")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"width": self.width}


@dataclass(frozen=True)
class LatentAttentionConfig:
    """``latent_attention``: ``heads`` heads of ``dim`` unrotated and ``rot_dim`` rotated query/key elements and ``vdim``
    values; queries through a latent of ``q_rank``, keys and values up from a cached latent of ``kv_rank``."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: RotaryConfig | None = None
    kv_from: int | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "LatentAttentionConfig":
        r = ConfigReader(data, where=where)
        dim, rot_dim = r.integer("dim"), r.integer("rot_dim", 0)
        rot = r.table("rot")
        out = cls(heads=r.integer("heads"), dim=dim, rot_dim=rot_dim, vdim=r.integer("vdim", dim), q_rank=r.integer("q_rank"),
                  kv_rank=r.integer("kv_rank"), scale=r.number("scale", (dim + rot_dim) ** -0.5),
                  rot=RotaryConfig.from_dict(rot, f"{where}.rot") if rot else None, kv_from=r.integer("kv_from", None))
        if min(out.heads, out.dim, out.vdim, out.q_rank, out.kv_rank) < 1 or out.rot_dim < 0 or out.rot_dim % 2:
            raise ConfigError(f"{where}: heads, dim, vdim, q_rank and kv_rank must be >= 1, rot_dim even and >= 0")
        if out.rot is not None and out.rot.dims != out.rot_dim:
            raise ConfigError(f"{where}: rot.dims ({out.rot.dims}) must equal rot_dim ({out.rot_dim})")
        if out.kv_rank + out.rot_dim > 256:
            raise ConfigError(f"{where}: kv_rank + rot_dim must be at most 256 (what a cached token holds)")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank,
                               "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class ActivatedFeedForwardConfig:
    ff: int

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "ActivatedFeedForwardConfig":
        r = ConfigReader(data, where=where)
        kind = r.text("kind", "dense")
        if kind != "dense":
            raise ConfigError(f"{where}: unsupported feed-forward kind {kind!r} (known: dense)")
        out = cls(ff=r.integer("ff"))
        if out.ff < 1:
            raise ConfigError(f"{where}: ff must be >= 1")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class PairHashConfig:
    """Row ``(previous * mul_prev + current * mul_cur) mod buckets`` of a table of ``buckets + 1`` rows."""

    buckets: int
    mul_prev: int
    mul_cur: int

    @classmethod
    def from_dict(cls, data: dict[str, Any], where: str) -> "PairHashConfig":
        r = ConfigReader(data, where=where)
        out = cls(buckets=r.integer("buckets"), mul_prev=r.integer("mul_prev"), mul_cur=r.integer("mul_cur"))
        if out.buckets < 1 or out.mul_prev < 0 or out.mul_cur < 0:
            raise ConfigError(f"{where}: buckets must be >= 1 and the multipliers >= 0")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"buckets": self.buckets, "mul_cur": self.mul_cur, "mul_prev": self.mul_prev}


MIXER_CONFIGS = {"mlstm": MatrixMemoryConfig, "mingru": GatedRecurrenceConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class BezutarLayerConfig:
    type: str
    mixer: "MatrixMemoryConfig | GatedRecurrenceConfig | LatentAttentionConfig"
    mlp: ActivatedFeedForwardConfig | None

    def to_dict(self) -> dict[str, Any]:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None, "type": self.type}


@dataclass(frozen=True)
class BezutarConfig(ModelConfigBase):
    architecture: ClassVar[str] = "Bezutar"

    max_position_embeddings: int = 131072  # without a position table nothing bounds a request but the cache
    layers: tuple[BezutarLayerConfig, ...] = ()
    norm_eps: float = 1e-6
    streams: int | None = None        # hyper-connected residual streams; None: one stream and the plain residual sum
    canon_taps: int | None = None     # taps of the convolution over every mixer's input; None: no convolution
    pair_hash: PairHashConfig | None = None
    position_rows: int | None = None  # rows of the learned position table; None: no table
    extra: dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("vocab and width must be >= 1 and there must be a layer")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise ConfigError(f"streams must be between 1 and 8, got {self.streams}")
        if self.canon_taps is not None and not 1 <= self.canon_taps <= 8:
            raise ConfigError(f"canon.taps must be between 1 and 8, got {self.canon_taps}")
        if self.position_rows is not None and self.position_rows < 1:
            raise ConfigError("max_positions must be >= 1")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
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
    def from_dict(cls, data: dict[str, Any], generation: dict[str, Any] | None = None) -> "BezutarConfig":
        r = ConfigReader(data, behind=generation)
        norm = ConfigReader(r.table("norm") or {}, where="norm")
        embedding = ConfigReader(r.table("embedding") or {}, where="embedding")
        canon = r.table("canon")
        pair = embedding.table("bigram")
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
            layers.append(BezutarLayerConfig(
                type=kind, mixer=MIXER_CONFIGS[kind].from_dict(mixer, f"layers[{i}].mixer"),
                mlp=ActivatedFeedForwardConfig.from_dict(mlp, f"layers[{i}].mlp") if mlp is not None else None))
        position_rows = r.integer("max_positions", None)
        return cls(
            vocab_size=r.integer("vocab"),
            hidden_size=r.integer("width"),
            num_hidden_layers=len(layers),
            max_position_embeddings=r.integer("max_position_embeddings", position_rows or 131072),
            torch_dtype=r.precision("torch_dtype", "dtype"),
            eos_token_id=r.token_id("eos_token_id"),
            bos_token_id=r.token_id("bos_token_id"),
            pad_token_id=r.token_id("pad_token_id"),
            layers=tuple(layers),
            norm_eps=norm.number("eps", 1e-6),
            streams=r.integer("streams", None),
            canon_taps=ConfigReader(canon, where="canon").integer("taps") if canon else None,
            pair_hash=PairHashConfig.from_dict(pair, "embedding.bigram") if pair else None,
            position_rows=position_rows,
            extra=r.leftover(also_known=("architecture", "architectures")),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
                               "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.hidden_size,
                               "torch_dtype": self.torch_dtype}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.canon_taps is not None:
            out["canon"] = {"taps": self.canon_taps}
        if self.pair_hash is not None:
            out["embedding"] = {"bigram": self.pair_hash.to_dict()}
        if self.position_rows is not None:
            out["max_positions"] = self.position_rows
            if self.max_position_embeddings != self.position_rows:
                out["max_position_embeddings"] = self.max_position_embeddings
        else:
            out["max_position_embeddings"] = self.max_position_embeddings
        for key in ("eos_token_id", "bos_token_id", "pad_token_id"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        out.update({k: v for k, v in self.extra.items() if k not in out})
        return out
