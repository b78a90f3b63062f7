"""Validated configuration of a ``Gegepel`` checkpoint.

The document is nested: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` (one entry
per layer: ``type``, the mixer's sizes under ``mixer``, the feed-forward under ``mlp`` or null) and
``loop`` (``start``, ``stop``, ``times``: layers start .. stop-1 are walked ``times`` times in a row).
Every size and every constant that can differ between checkpoints is read here; nothing is assumed
equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple

from ..config.model_config import ConfigError, RawConfig, missing_field, required_positive_int

ARCHITECTURE = "Gegepel"
#: positions a request may reach when the document gives no limit (every position is exact in 32-bit floats)
DEFAULT_MAX_POSITIONS = 1 << 24


def _section(document: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = document.get(key)
    if not isinstance(value, dict):
        raise ConfigError(ARCHITECTURE, f"{where}`{key}` must be an object")
    return value


def _number(document: Mapping[str, Any], key: str, where: str) -> float:
    value = document.get(key)
    if value is None:
        raise missing_field(ARCHITECTURE, where + key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(ARCHITECTURE, f"`{where}{key}` must be a number, found {value!r}")
    return float(value)


def _count(document: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    value = document.get(key)
    if value is None:
        raise missing_field(ARCHITECTURE, where + key)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(ARCHITECTURE, f"`{where}{key}` must be an integer of at least {least}, found {value!r}")
    return value


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int                 # unrotated query/key entries per head
    rot_dim: int             # rotated query/key entries per head (the key's are shared by all heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int            # leading entries of the rot_dim part that the rotation covers


@dataclass(frozen=True)
class RoutedExpertsSizes:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class LayerSpec:
    kind: str
    mixer: LatentAttentionSizes
    mlp: Optional[RoutedExpertsSizes]


@dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class GegepelConfig:
    ARCHITECTURE = ARCHITECTURE

    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    loop: Optional[LoopSpec]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Sequence[int] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "GegepelConfig":
        doc = raw.document
        vocab = required_positive_int(ARCHITECTURE, doc, "vocab")
        width = required_positive_int(ARCHITECTURE, doc, "width")
        scale = _number(_section(doc, "embedding", ""), "scale", "embedding.")
        eps = _number(_section(doc, "norm", ""), "eps", "norm.")
        if not eps >= 0:
            raise ConfigError(ARCHITECTURE, "`norm.eps` must be non-negative")
        entries = doc.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(ARCHITECTURE, "`layers` must be a list with at least one layer")
        layers = tuple(_layer(entry, f"layers[{i}].") for i, entry in enumerate(entries))
        loop = None
        if doc.get("loop") is not None:
            section = _section(doc, "loop", "")
            loop = LoopSpec(_count(section, "start", "loop.", 0), _count(section, "stop", "loop.", 0),
                            _count(section, "times", "loop."))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(ARCHITECTURE, f"`loop` must name a stretch of the {len(layers)} layers, "
                                                f"found {loop.start} .. {loop.stop}")
        limit = doc.get("max_position_embeddings")
        if limit is not None:
            limit = required_positive_int(ARCHITECTURE, doc, "max_position_embeddings")
        return cls(vocab, width, scale, eps, layers, loop, limit or DEFAULT_MAX_POSITIONS, tuple(raw.eos_token_ids), doc)


def _layer(entry: Any, where: str) -> LayerSpec:
    if not isinstance(entry, dict):
        raise ConfigError(ARCHITECTURE, f"`{where[:-1]}` must be an object")
    kind = entry.get("type")
    if kind != "latent_attention":
        raise ConfigError(ARCHITECTURE, f"`{where}type` {kind!r} is not a mixer of this design (latent_attention)")
    m = _section(entry, "mixer", where)
    inside = where + "mixer."
    rot_dim = _count(m, "rot_dim", inside, 0)
    rot_base, rot_dims = 1.0, 0
    if rot_dim:
        rot = _section(m, "rot", inside)
        rot_base, rot_dims = _number(rot, "base", inside + "rot."), _count(rot, "dims", inside + "rot.", 0)
        if rot_dims % 2 or rot_dims > rot_dim or not rot_base > 0:
            raise ConfigError(ARCHITECTURE, f"`{inside}rot` must rotate an even number of at most {rot_dim} entries "
                                            f"with a positive base")
    mixer = LatentAttentionSizes(
        heads=_count(m, "heads", inside), dim=_count(m, "dim", inside), rot_dim=rot_dim, vdim=_count(m, "vdim", inside),
        q_rank=_count(m, "q_rank", inside), kv_rank=_count(m, "kv_rank", inside), scale=_number(m, "scale", inside),
        rot_base=rot_base, rot_dims=rot_dims)
    mlp = None
    if entry.get("mlp") is not None:
        f = _section(entry, "mlp", where)
        if f.get("kind") != "moe":
            raise ConfigError(ARCHITECTURE, f"`{where}mlp.kind` {f.get('kind')!r} is not a feed-forward of this design (moe)")
        router = _section(f, "router", where + "mlp.")
        mlp = RoutedExpertsSizes(_count(router, "experts", where + "mlp.router."), _count(router, "top", where + "mlp.router."),
                                 _count(_section(f, "expert", where + "mlp."), "ff", where + "mlp.expert."))
        if mlp.top > mlp.experts:
            raise ConfigError(ARCHITECTURE, f"`{where}mlp.router.top` exceeds the number of experts")
    return LayerSpec(kind, mixer, mlp)
