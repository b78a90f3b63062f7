"""Linear attention with a fixed decay per head over a state of fixed size ("lightning attention").

q = silu(W_q h), k = silu(W_k h) (heads x dim), v = silu(W_v h) (heads x vdim).  Per head the state
S [dim, vdim] follows S_t = decay_h S_(t-1) + k_t v_t^T and the head's result is o_t = S_t^T q_t; no other
scale.  The heads' results of a row are RMS-normed together (one weight over heads * vdim entries), multiplied
by sigmoid(W_g h) and projected by W_o.  The state starts at zero, is kept in 32-bit floats per request
(``RequestState``) and carried from step to step; the decays, their powers, the scores and the sums are 32-bit
in both dtypes.  W_q, W_k, W_v and W_g read the same input and are one product (rows stacked at load).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Sequence

import torch

from .. import ops
from .base import Mixer, RequestState, TensorSpec, matrix_to, scale_to


@dataclass(frozen=True)
class LightningNames:
    q: str
    k: str
    v: str
    gate: str
    norm: str
    o: str


class LightningAttention(Mixer):
    graph_safe = True
    #: a step in which some request brings more rows than this runs the chunk-parallel kernels (bfloat16, states of 64
    #: or 128 entries a side); steps of decoded tokens walk each request's rows in one block, from its state
    CHUNKED_FROM = 8

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float,
                 names: LightningNames):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        if not all(0.0 <= float(d) <= 1.0 for d in decay):
            raise ValueError("a decay lies between 0 and 1")
        self.hidden, self.heads, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.decay_values, self.eps, self.names = [float(d) for d in decay], float(eps), names
        self.w_in = self.w_o = self.norm = self.decay = None

    def cache_need(self) -> RequestState:
        return RequestState((self.heads, self.dim, self.vdim), torch.float32)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n, qk, vv = self.names, self.heads * self.dim, self.heads * self.vdim
        return {n.q: TensorSpec((qk, self.hidden)), n.k: TensorSpec((qk, self.hidden)), n.v: TensorSpec((vv, self.hidden)),
                n.gate: TensorSpec((vv, self.hidden)), n.norm: TensorSpec((vv,), "scale"), n.o: TensorSpec((self.hidden, vv))}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        n = self.names
        self.w_in = matrix_to(torch.cat([tensors[n.q], tensors[n.k], tensors[n.v], tensors[n.gate]], dim=0), device, dtype)
        self.w_o = matrix_to(tensors[n.o], device, dtype)
        self.norm = scale_to(tensors[n.norm], device)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(device)

    def forward(self, ctx, cache, x: torch.Tensor) -> torch.Tensor:
        rows = x.shape[0]
        qk, vv = self.heads * self.dim, self.heads * self.vdim
        proj = ops.linear(x, self.w_in, error_word=ctx.error_word)
        heads_out = torch.empty((rows, vv), dtype=torch.float32, device=x.device)
        counts = [b - a for a, b in zip(ctx.host_cu_rows, ctx.host_cu_rows[1:])]
        if (len(counts) == ctx.num_requests and max(counts, default=0) > self.CHUNKED_FROM
                and ops.lightning_chunks_takes(proj.dtype, self.dim, self.vdim)):
            # prompt portions: chunks in parallel on the tensor cores
            chunks = sum(-(-count // ops.LIGHTNING_CHUNK_TOKENS) for count in counts)
            ops.lightning_chunks(proj, 0, qk, 2 * qk, ctx.cu_rows, ctx.positions, ctx.state_slots, cache.state, self.decay,
                                 heads_out, ctx.num_requests, chunks, read_only=not cache.writable)
        else:
            ops.lightning_scan(proj, 0, qk, 2 * qk, ctx.cu_rows, ctx.positions, ctx.state_slots, cache.state, self.decay,
                               heads_out, ctx.num_requests, read_only=not cache.writable,
                               single_rows=len(counts) == ctx.num_requests and all(count == 1 for count in counts))
        gated = torch.empty((rows, vv), dtype=x.dtype, device=x.device)
        ops.lightning_gate_norm(heads_out, proj, 2 * qk + vv, self.norm, self.eps, gated)
        return ops.linear(gated, self.w_o, error_word=ctx.error_word, partial_ok=True)
