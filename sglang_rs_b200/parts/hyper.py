"""Several copies of the residual stream ("hyper-connections").

Instead of one stream x a model carries ``streams`` copies x_1 .. x_s, all equal to the embedding output at
the start.  A sublayer reads u = sum_s read[s] x_s, computes y = sublayer(norm(u)), and then every copy is
replaced, all at once from the old ones: x_t <- sum_s mix[s, t] x_s + write[t] * y (``mix`` is indexed
[from, to]).  At the end the stream is the sum of the copies.  One copy with read = write = mix = 1 is the plain
pre-norm residual sum.

The copies travel as one float32 tensor [rows, streams * width]; the result of a sublayer travels beside them as a
:class:`StreamUpdate` until the next read, so that "update by the sublayer before, read, norm" is ONE kernel
(``ops.stream_step``), also across the border between two blocks and into the final norm.  All sums are 32-bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import FeedForward, Mixer, Norm, Part, TensorSpec, scale_to
from .norm import RmsNorm


@dataclass(frozen=True)
class StreamNames:
    read: str
    write: str
    mix: str


class StreamConnection(Part):
    """The weights with which one sublayer reads from and writes to the copies.  ``names`` None: constants
    (read 1, write 1, mix the identity) and no tensors, which with one copy is the plain residual sum."""
    graph_safe = True

    def __init__(self, streams: int, names: Optional[StreamNames]):
        if not 1 <= streams <= 8:
            raise ValueError(f"{streams} copies of the residual stream; the kernels take 1 to 8")
        self.streams, self.names = int(streams), names
        self.read = self.write = self.mix = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        if self.names is None:
            return {}
        s = self.streams
        return {self.names.read: TensorSpec((s,), "scale"), self.names.write: TensorSpec((s,), "scale"),
                self.names.mix: TensorSpec((s, s), "scale")}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        if self.names is None:
            self.read = torch.ones(self.streams, dtype=torch.float32, device=device)
            self.write = torch.ones(self.streams, dtype=torch.float32, device=device)
            self.mix = torch.eye(self.streams, dtype=torch.float32, device=device).contiguous()
            return
        self.read = scale_to(tensors[self.names.read], device)
        self.write = scale_to(tensors[self.names.write], device)
        self.mix = scale_to(tensors[self.names.mix], device)


@dataclass
class StreamUpdate:
    """A sublayer's result that the copies have not taken in yet."""
    values: torch.Tensor
    connection: StreamConnection


def read_streams(streams: int, copies: torch.Tensor, pending: Optional[StreamUpdate], connection: Optional[StreamConnection],
                 norm: Optional[RmsNorm], out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None,
                 gather: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Applies the pending update to ``copies`` [rows, streams * width] and returns norm(sum_s read[s] x_s) with the
    read weights of ``connection`` (or ``gather``); None if nothing is to be read."""
    rows, width = copies.shape[0], copies.shape[1] // streams
    x = copies.view(rows, streams, width)
    gather = connection.read if connection is not None else gather
    out = None
    if gather is not None:
        out = torch.empty((rows if row_index is None else row_index.numel(), width), dtype=out_dtype, device=copies.device)
    ops.stream_step(x, pending.values if pending is not None else None,
                    pending.connection.mix if pending is not None else None,
                    pending.connection.write if pending is not None else None, gather,
                    norm.weight if norm is not None else None, norm.eps if norm is not None else 0.0, out,
                    row_index=row_index, norm=norm is not None)
    return out


class StreamBlock(Part):
    """A pre-norm layer over the copies: mixer behind ``norm_1``, then, if the layer has one, the feed-forward
    behind ``norm_2``, each with a :class:`StreamConnection` of its own.  The hidden state travels as
    (copies, pending update)."""

    def __init__(self, streams: int, norm_1: RmsNorm, mixer: Mixer, connection_1: StreamConnection,
                 norm_2: Optional[RmsNorm] = None, feed_forward: Optional[FeedForward] = None,
                 connection_2: Optional[StreamConnection] = None):
        if (feed_forward is None) != (norm_2 is None) or (feed_forward is None) != (connection_2 is None):
            raise ValueError("a feed-forward comes with its norm and its connection, or not at all")
        self.streams = int(streams)
        self.norm_1, self.mixer, self.connection_1 = norm_1, mixer, connection_1
        self.norm_2, self.feed_forward, self.connection_2 = norm_2, feed_forward, connection_2

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def parts(self):
        return tuple(part for part in (self.norm_1, self.mixer, self.connection_1, self.norm_2, self.feed_forward,
                                       self.connection_2) if part is not None)

    def cache_need(self):
        return self.mixer.cache_need()

    def split_scratch(self):
        return self.mixer.split_scratch()

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for part in self.parts():
            specs.update(part.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        for part in self.parts():
            part.load(tensors, device, dtype)

    def forward(self, ctx, cache, copies: torch.Tensor, pending):
        if pending is not None and not isinstance(pending, StreamUpdate):
            raise TypeError("a block over copies of the stream takes a StreamUpdate as the pending term")
        normed = read_streams(self.streams, copies, pending, self.connection_1, self.norm_1, ctx.dtype)
        pending = StreamUpdate(self.mixer.forward(ctx, cache, normed), self.connection_1)
        if self.feed_forward is None:
            return copies, pending
        normed = read_streams(self.streams, copies, pending, self.connection_2, self.norm_2, ctx.dtype)
        return copies, StreamUpdate(self.feed_forward.forward(ctx, normed), self.connection_2)


class StreamSumNorm(Norm):
    """The norm behind the last layer: RMS norm of the sum of the copies, with the last pending update applied
    on the way (only to the rows that are picked, when rows are picked)."""
    graph_safe = True

    def __init__(self, streams: int, width: int, eps: float, weight_name: str):
        self.streams, self.inner = int(streams), RmsNorm(width, eps, weight_name)
        self.ones: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return self.inner.tensor_specs()

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.inner.load(tensors, device, dtype)
        self.ones = torch.ones(self.streams, dtype=torch.float32, device=device)

    def spec(self):
        return self.inner.spec()

    def add_norm(self, residual: torch.Tensor, delta, out_dtype: torch.dtype,
                 row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        if delta is not None and not isinstance(delta, StreamUpdate):
            raise TypeError("the norm over copies of the stream takes a StreamUpdate as the pending term")
        return read_streams(self.streams, residual, delta, None, self.inner, out_dtype, row_index, gather=self.ones)
