"""Gegepel put together from the parts.

A decoder whose layers each hold attention through latents (``parts/latent_attention.py``: a sink per
head, an output gate) and, unless the layer has none, a feed-forward of routed experts
(``parts/moe.py``: softmax over all experts, the scores of the chosen ones as weights), with a layer
norm (weight and bias) ahead of and behind each sublayer (``parts.SandwichBlock``).  The embedding is
scaled.  A stretch of layers may be walked several times with the same weights, each pass with caches of
its own and opened by ``parts.PassEntry``.  The final norm is a layer norm, the head a matrix of its own.

Checkpoint names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), ``loop.in``, ``loop.step``, and per layer
``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b`` (+ ``.b``), ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk,
uv, sink, g, o}``, ``l<i>.mlp.router`` and ``l<i>.mlp.e<j>.{gate, up, down}``.
Fixed by the design, not by config.json: SiLU in the experts, unnormalised router weights, the half-split
pairing of rotated entries, a causal mask without a window.
"""
from __future__ import annotations

from ..config.model_config import ConfigError
from ..config.registry import register_architecture
from ..parts import (GatedMlpNames, LatentAttention, LatentAttentionNames, LayerNorm, OutputHead, PassEntry,
                     RotaryEncoding, RoutedExperts, SandwichBlock, TokenEmbedding)
from .decoder import DecoderModel, LayerCall
from .gegepel_config import ARCHITECTURE, GegepelConfig


def layer_program(config: GegepelConfig):
    """The layer calls of one forward pass: the layers ahead of the stretch, the stretch ``times`` times (the
    first call of each walk opens the pass), the layers behind it."""
    count, loop = len(config.layers), config.loop
    if loop is None:
        return [LayerCall(i) for i in range(count)]
    calls = [LayerCall(i) for i in range(loop.start)]
    for t in range(loop.times):
        for i in range(loop.start, loop.stop):
            calls.append(LayerCall(i, entry=0 if i == loop.start else None, pass_index=t))
    calls += [LayerCall(i) for i in range(loop.stop, count)]
    return calls


def build_gegepel(config: GegepelConfig) -> DecoderModel:
    try:
        return _build(config)
    except ValueError as error:
        if isinstance(error, ConfigError):
            raise
        raise ConfigError(ARCHITECTURE, str(error)) from None


def _build(config: GegepelConfig) -> DecoderModel:
    width, eps = config.width, config.norm_eps
    embedding = TokenEmbedding(config.vocab, width, "embed", scale=config.embedding_scale)

    def norm(name: str) -> LayerNorm:
        return LayerNorm(width, eps, name, name + ".b")
    rotations = {}          # layers with the same rotation share one table of frequencies
    layers = []
    for index, spec in enumerate(config.layers):
        p, m = f"l{index}.", spec.mixer
        rotary = None
        if m.rot_dim and m.rot_dims:
            key = (m.rot_dim, m.rot_base, m.rot_dims)
            rotary = rotations.get(key)
            if rotary is None:
                rotary = rotations[key] = RotaryEncoding(m.rot_dim, m.rot_base, rotary_dim=m.rot_dims)
        mixer = LatentAttention(
            width, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, eps, rotary,
            LatentAttentionNames(q_down=p + "mix.dq", q_norm=p + "mix.dq.norm", q_up=p + "mix.uq", kv_down=p + "mix.dkv",
                                 kv_norm=p + "mix.dkv.norm", k_up=p + "mix.uk", v_up=p + "mix.uv", o=p + "mix.o",
                                 sink=p + "mix.sink", gate=p + "mix.g"))
        if spec.mlp is None:
            layers.append(SandwichBlock(norm(p + "norm1"), mixer, norm(p + "norm1b")))
            continue
        feed_forward = RoutedExperts(
            width, spec.mlp.ff, spec.mlp.experts, spec.mlp.top, "silu", p + "mlp.router",
            lambda e, p=p: GatedMlpNames(gate=f"{p}mlp.e{e}.gate", up=f"{p}mlp.e{e}.up", down=f"{p}mlp.e{e}.down"),
            renormalize=False)
        layers.append(SandwichBlock(norm(p + "norm1"), mixer, norm(p + "norm1b"), norm(p + "norm2"), feed_forward,
                                    norm(p + "norm2b")))
    entries = [PassEntry(width, config.loop.times, "loop.in", "loop.step")] if config.loop is not None else []
    # a layer without a feed-forward has no second pair of norms; checkpoints may carry them all the same
    ignored = [f"l{i}.norm2*" for i, spec in enumerate(config.layers) if spec.mlp is None]
    return DecoderModel(embedding, layers, norm("final.norm"), OutputHead(config.vocab, width, "head"),
                        vocab_size=config.vocab, max_positions=config.max_positions, eos_token_ids=config.eos_token_ids,
                        program=layer_program(config), pass_entries=entries, ignored_tensors=ignored)


register_architecture(ARCHITECTURE, GegepelConfig.from_raw, build_gegepel, replace=True)
