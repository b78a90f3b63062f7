"""Tosivik put together from the parts.

A decoder whose layers each hold one of two mixers and, unless the layer has none, a feed-forward, each behind an
RMS norm, over ``streams`` copies of the residual stream (``parts/hyper.py``).  Mixers: softmax attention whose
values are the unrotated keys, with grouped heads, a rotation of the leading entries of each head with stretched
long wavelengths, and a mask by chunks of positions (``parts/attention.py``); linear attention with a fixed decay
per head over a state per request (``parts/lightning.py``).  Feed-forwards: W_down gelu_tanh(W_up h), or routed
experts W_down relu(W_up h)^2 with a bias on the router's logits, a softmax over the chosen logits and an expert
that every token shares (``parts/moe.py``).  The embedding is scaled and adds a row chosen by the token and the
token before it (``parts.PairTokenEmbedding``).  A layer may use another layer's tensors with a cache or state of
its own: the model's program then calls that layer's block a second time.  The logits are squashed by tanh.

Checkpoint names: ``embed``, ``bigram``, ``head``, ``final.norm`` and per layer ``l<i>.norm1`` / ``norm2``,
``l<i>.hc1.{in, out, mix}`` / ``hc2.*``, ``l<i>.mix.{q, k, o}`` (attention) or ``l<i>.mix.{q, k, v, g, norm, o}``
(lightning), ``l<i>.mlp.{up, down}`` or ``l<i>.mlp.{router, router.b, e<j>.up, e<j>.down, shared.up, shared.down}``.
Fixed by the design, not by config.json: the activations, the half-split pairing of rotated entries, the factor
0.1 ln(factor) + 1 on cosines and sines.
"""
from __future__ import annotations

from ..config.model_config import ConfigError
from ..config.registry import register_architecture
from ..parts import (AttentionNames, GatedMlpNames, GroupedQueryAttention, LightningAttention, LightningNames,
                     NoPositionEncoding, OutputHead, PairTokenEmbedding, PlainMlp, RmsNorm, RotaryEncoding, RoutedExperts,
                     StreamBlock, StreamConnection, StreamNames, StreamSumNorm, WavelengthScaling)
from .decoder import DecoderModel, LayerCall
from .tosivik_config import ARCHITECTURE, AttentionSizes, DenseSizes, TosivikConfig


def build_tosivik(config: TosivikConfig) -> DecoderModel:
    try:
        return _build(config)
    except ValueError as error:
        if isinstance(error, ConfigError):
            raise
        raise ConfigError(ARCHITECTURE, str(error)) from None


def _build(config: TosivikConfig) -> DecoderModel:
    width, eps = config.width, config.norm_eps
    streams = config.streams or 1
    pairs = config.pairs
    embedding = PairTokenEmbedding(
        config.vocab, width, "embed", config.embedding_scale, copies=streams, pair_name="bigram" if pairs else None,
        buckets=pairs.buckets if pairs else 0, mul_prev=pairs.mul_prev if pairs else 0, mul_cur=pairs.mul_cur if pairs else 0)
    rotations = {}          # layers with the same rotation share one table of frequencies

    def rotation(m: AttentionSizes):
        if not m.rot_dims:
            return NoPositionEncoding()
        key = (m.dim, m.rot_dims, m.rot_base, m.rot_scaling)
        if key not in rotations:
            s = m.rot_scaling
            rotations[key] = RotaryEncoding(m.dim, m.rot_base, rotary_dim=m.rot_dims,
                                            scaling=WavelengthScaling(s.factor, s.original, s.fast, s.slow) if s else None)
        return rotations[key]

    def connection(name: str) -> StreamConnection:
        # without `streams` in the document there is one stream and the plain residual sum: no tensors
        return StreamConnection(streams, StreamNames(name + ".in", name + ".out", name + ".mix") if config.streams else None)

    blocks, block_of = [], {}
    for index, spec in enumerate(config.layers):
        if spec.weights_of is not None:
            continue
        p, m = f"l{index}.", spec.mixer
        if spec.kind == "attention":
            mixer = GroupedQueryAttention(width, m.heads, m.kv_heads, m.dim, m.scale, rotation(m),
                                          AttentionNames(q=p + "mix.q", k=p + "mix.k", v=None, o=p + "mix.o"), chunk=m.chunk)
        else:
            mixer = LightningAttention(width, m.heads, m.dim, m.vdim, m.decay, eps,
                                       LightningNames(q=p + "mix.q", k=p + "mix.k", v=p + "mix.v", gate=p + "mix.g",
                                                      norm=p + "mix.norm", o=p + "mix.o"))
        feed_forward = None
        if isinstance(spec.mlp, DenseSizes):
            feed_forward = PlainMlp(width, spec.mlp.ff, "gelu_tanh", p + "mlp.up", p + "mlp.down")
        elif spec.mlp is not None:
            shared = None
            if spec.mlp.shared_ff is not None:
                shared = PlainMlp(width, spec.mlp.shared_ff, "relu2", p + "mlp.shared.up", p + "mlp.shared.down",
                                  float_result=True)
            feed_forward = RoutedExperts(
                width, spec.mlp.ff, spec.mlp.experts, spec.mlp.top, "relu2", p + "mlp.router",
                lambda e, p=p: GatedMlpNames(gate=None, up=f"{p}mlp.e{e}.up", down=f"{p}mlp.e{e}.down"),
                renormalize=True, router_bias_name=p + "mlp.router.b", shared=shared)
        block_of[index] = len(blocks)
        if feed_forward is None:
            blocks.append(StreamBlock(streams, RmsNorm(width, eps, p + "norm1"), mixer, connection(p + "hc1")))
        else:
            blocks.append(StreamBlock(streams, RmsNorm(width, eps, p + "norm1"), mixer, connection(p + "hc1"),
                                      RmsNorm(width, eps, p + "norm2"), feed_forward, connection(p + "hc2")))
    program = [LayerCall(block_of[spec.weights_of if spec.weights_of is not None else index])
               for index, spec in enumerate(config.layers)]
    # a layer without a feed-forward has no second norm and connection; checkpoints may carry them all the same
    ignored = [pattern for i, spec in enumerate(config.layers) if spec.mlp is None and spec.weights_of is None
               for pattern in (f"l{i}.norm2", f"l{i}.hc2.*")]
    return DecoderModel(embedding, blocks, StreamSumNorm(streams, width, eps, "final.norm"),
                        OutputHead(config.vocab, width, "head", softcap=config.logit_softcap),
                        vocab_size=config.vocab, max_positions=config.max_positions, eos_token_ids=config.eos_token_ids,
                        program=program, ignored_tensors=ignored)


register_architecture(ARCHITECTURE, TosivikConfig.from_raw, build_tosivik, replace=True)
