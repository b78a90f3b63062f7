"""Validated configuration of a ``Tosivik`` checkpoint.

The document is nested: ``vocab``, ``width``, ``streams`` (copies of the residual stream; absent: the plain
residual sum), ``logit_softcap`` (absent: none), ``embedding`` (``scale``, and ``bigram`` with ``buckets``,
``mul_prev``, ``mul_cur`` for the table indexed by pairs of tokens; absent: no such table), ``norm.eps`` and
``layers``: one entry per layer with ``type`` (``attention`` or ``lightning``), the mixer's sizes under ``mixer``,
the feed-forward under ``mlp`` (``kind`` ``dense`` or ``moe``; null: none) and optionally ``weights_of``: the
index of the layer whose tensors this layer uses (with a cache or state of its own).  Every size and every
constant that can differ between checkpoints is read here, per layer; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple, Union

from ..config.model_config import ConfigError, RawConfig, missing_field, required_positive_int

ARCHITECTURE = "Tosivik"
#: positions a request may reach when the document gives no limit (every position is exact in 32-bit floats)
DEFAULT_MAX_POSITIONS = 1 << 24


def _section(document: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = document.get(key)
    if not isinstance(value, dict):
        raise ConfigError(ARCHITECTURE, f"`{where}{key}` must be an object")
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
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]             # positions per chunk of the mask; None: every earlier key is seen
    rot_dims: int                    # leading entries of each head that are rotated; 0: none
    rot_base: float
    rot_scaling: Optional[RotaryScaling]


@dataclass(frozen=True)
class LightningSizes:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class DenseSizes:
    ff: int


@dataclass(frozen=True)
class RoutedSizes:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class LayerSpec:
    kind: str
    mixer: Union[AttentionSizes, LightningSizes]
    mlp: Union[DenseSizes, RoutedSizes, None]
    #: the layer whose tensors this layer uses; None: its own
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class TosivikConfig:
    ARCHITECTURE = ARCHITECTURE

    vocab: int
    width: int
    streams: Optional[int]
    embedding_scale: float
    pairs: Optional[PairTable]
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[LayerSpec, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Sequence[int] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "TosivikConfig":
        doc = raw.document
        vocab = required_positive_int(ARCHITECTURE, doc, "vocab")
        width = required_positive_int(ARCHITECTURE, doc, "width")
        streams = None
        if doc.get("streams") is not None:
            streams = _count(doc, "streams", "")
            if streams > 8:
                raise ConfigError(ARCHITECTURE, f"`streams` {streams}: at most 8 copies of the residual stream are taken")
        embedding = _section(doc, "embedding", "")
        scale = _number(embedding, "scale", "embedding.")
        pairs = None
        if embedding.get("bigram") is not None:
            b = _section(embedding, "bigram", "embedding.")
            pairs = PairTable(_count(b, "buckets", "embedding.bigram."), _count(b, "mul_prev", "embedding.bigram.", 0),
                              _count(b, "mul_cur", "embedding.bigram.", 0))
        eps = _number(_section(doc, "norm", ""), "eps", "norm.")
        if not eps >= 0:
            raise ConfigError(ARCHITECTURE, "`norm.eps` must be non-negative")
        cap = None
        if doc.get("logit_softcap") is not None:
            cap = _number(doc, "logit_softcap", "")
            if not cap > 0:
                raise ConfigError(ARCHITECTURE, "`logit_softcap` must be positive")
        entries = doc.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(ARCHITECTURE, "`layers` must be a list with at least one layer")
        layers = tuple(_layer(entry, f"layers[{i}].") for i, entry in enumerate(entries))
        for i, spec in enumerate(layers):
            if spec.weights_of is None:
                continue
            j = spec.weights_of
            if not 0 <= j < len(layers) or j == i or layers[j].weights_of is not None:
                raise ConfigError(ARCHITECTURE, f"`layers[{i}].weights_of` must name another layer that has tensors of its own")
            if (spec.kind, spec.mixer, spec.mlp) != (layers[j].kind, layers[j].mixer, layers[j].mlp):
                raise ConfigError(ARCHITECTURE, f"`layers[{i}]` uses the tensors of layer {j} but differs from it")
        limit = doc.get("max_position_embeddings")
        if limit is not None:
            limit = required_positive_int(ARCHITECTURE, doc, "max_position_embeddings")
        return cls(vocab, width, streams, scale, pairs, eps, cap, layers, limit or DEFAULT_MAX_POSITIONS,
                   tuple(raw.eos_token_ids), doc)


def _attention(m: Mapping[str, Any], inside: str) -> AttentionSizes:
    heads, dim = _count(m, "heads", inside), _count(m, "dim", inside)
    kv_heads = _count(m, "kv_heads", inside) if m.get("kv_heads") is not None else heads
    vdim = _count(m, "vdim", inside) if m.get("vdim") is not None else dim
    if heads % kv_heads:
        raise ConfigError(ARCHITECTURE, f"`{inside}heads` {heads} is not a multiple of `kv_heads` {kv_heads}")
    if vdim != dim:
        raise ConfigError(ARCHITECTURE, f"`{inside}vdim` {vdim} differs from `dim` {dim}: the values are the keys")
    chunk = None
    if m.get("mask") is not None:
        chunk = _count(_section(m, "mask", inside), "size", inside + "mask.")
    rot_dims, rot_base, scaling = 0, 1.0, None
    if m.get("rot") is not None:
        rot = _section(m, "rot", inside)
        rot_dims, rot_base = _count(rot, "dims", inside + "rot.", 0), _number(rot, "base", inside + "rot.")
        if rot_dims % 2 or rot_dims > dim or not rot_base > 0:
            raise ConfigError(ARCHITECTURE, f"`{inside}rot` must rotate an even number of at most {dim} entries with a "
                                            f"positive base")
        if rot_dims and rot.get("scaling") is not None:
            s = _section(rot, "scaling", inside + "rot.")
            where = inside + "rot.scaling."
            scaling = RotaryScaling(_number(s, "factor", where), _number(s, "original", where), _number(s, "fast", where),
                                    _number(s, "slow", where))
            if not (scaling.factor > 0 and scaling.original > 0 and scaling.fast > 0 and scaling.slow > 0 and rot_base > 1):
                raise ConfigError(ARCHITECTURE, f"`{where[:-1]}` needs positive numbers and a base above 1")
    return AttentionSizes(heads, kv_heads, dim, vdim, _number(m, "scale", inside), chunk, rot_dims, rot_base, scaling)


def _lightning(m: Mapping[str, Any], inside: str) -> LightningSizes:
    heads = _count(m, "heads", inside)
    decay = m.get("decay")
    if (not isinstance(decay, list) or len(decay) != heads
            or not all(isinstance(d, (int, float)) and not isinstance(d, bool) and 0.0 <= d <= 1.0 for d in decay)):
        raise ConfigError(ARCHITECTURE, f"`{inside}decay` must list one number between 0 and 1 per head ({heads})")
    return LightningSizes(heads, _count(m, "dim", inside), _count(m, "vdim", inside), tuple(float(d) for d in decay))


def _layer(entry: Any, where: str) -> LayerSpec:
    if not isinstance(entry, dict):
        raise ConfigError(ARCHITECTURE, f"`{where[:-1]}` must be an object")
    kind = entry.get("type")
    m = _section(entry, "mixer", where)
    if kind == "attention":
        mixer = _attention(m, where + "mixer.")
    elif kind == "lightning":
        mixer = _lightning(m, where + "mixer.")
    else:
        raise ConfigError(ARCHITECTURE, f"`{where}type` {kind!r} is not a mixer of this design (attention, lightning)")
    mlp = None
    if entry.get("mlp") is not None:
        f = _section(entry, "mlp", where)
        if f.get("kind") == "dense":
            mlp = DenseSizes(_count(f, "ff", where + "mlp."))
        elif f.get("kind") == "moe":
            router = _section(f, "router", where + "mlp.")
            shared = None
            if f.get("shared") is not None:
                shared = _count(_section(f, "shared", where + "mlp."), "ff", where + "mlp.shared.")
            mlp = RoutedSizes(_count(router, "experts", where + "mlp.router."), _count(router, "top", where + "mlp.router."),
                              _count(_section(f, "expert", where + "mlp."), "ff", where + "mlp.expert."), shared)
            if mlp.top > mlp.experts:
                raise ConfigError(ARCHITECTURE, f"`{where}mlp.router.top` exceeds the number of experts")
        else:
            raise ConfigError(ARCHITECTURE, f"`{where}mlp.kind` {f.get('kind')!r} is not a feed-forward of this design "
                                            f"(dense, moe)")
    weights_of = None
    if entry.get("weights_of") is not None:
        weights_of = _count(entry, "weights_of", where, 0)
    return LayerSpec(kind, mixer, mlp, weights_of)
