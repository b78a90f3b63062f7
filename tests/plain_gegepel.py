"""A plain, slow implementation of the Gegepel design, one function per mechanism, in float64 on the host.

It shares no code with the package: it reads the configuration document and a dict of tensors by their
checkpoint names.  The tests compare the engine with it.

Notation: x is the residual stream [tokens, width]; a sequence is processed whole (no cache), so a
token at position i sees the positions 0..i of its own sequence.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def _t(tensors, name):
    return tensors[name].to(F)


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def rotate_half_split(v, positions, base, dims):
    """Rotates the first ``dims`` entries of the last axis: entry i pairs with entry i + dims/2,
    angle = position * base^(-2i/dims).  The design takes positions and angles in 32-bit: the frequency
    and the product are rounded to float32, the cosine and sine are those of that angle."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    freq = torch.pow(torch.tensor(float(base), dtype=F), -2.0 * i / dims)
    angle = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(F)     # [tokens, half]
    while angle.dim() < v.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def softmax_with_sink(scores, sink):
    """scores [heads, queries, keys] (masked entries -inf), sink [heads]: weights whose denominator also
    holds exp(sink)."""
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def latent_attention(h, tensors, prefix, m, eps):
    """h [tokens, width] of one sequence from position 0; m: the mixer's sizes."""
    n = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(n)
    cq = rms_norm(h @ _t(tensors, prefix + "dq").T, _t(tensors, prefix + "dq.norm"), eps)
    q = (cq @ _t(tensors, prefix + "uq").T).view(n, heads, dim + rot)
    kv = h @ _t(tensors, prefix + "dkv").T
    c = rms_norm(kv[:, :rank], _t(tensors, prefix + "dkv.norm"), eps)
    k_rot = rotate_half_split(kv[:, rank:rank + rot], positions, m["rot"]["base"], m["rot"]["dims"])
    q_plain = q[..., :dim]
    q_rot = rotate_half_split(q[..., dim:], positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ _t(tensors, prefix + "uk").T).view(n, heads, dim)
    v = (c @ _t(tensors, prefix + "uv").T).view(n, heads, vdim)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    scores = scores * m["scale"]
    mask = positions[None, :] > positions[:, None]
    scores = scores.masked_fill(mask[None], float("-inf"))
    w = softmax_with_sink(scores, _t(tensors, prefix + "sink"))
    out = torch.einsum("hij,jhd->ihd", w, v)
    gate = torch.sigmoid(h @ _t(tensors, prefix + "g").T)              # [tokens, heads]
    out = out * gate[:, :, None]
    return out.reshape(n, heads * vdim) @ _t(tensors, prefix + "o").T


def routed_experts(h, tensors, prefix, mlp):
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.softmax(h @ _t(tensors, prefix + "router").T, dim=-1)
    chosen = torch.topk(scores, top, dim=-1)
    out = torch.zeros_like(h)
    for e in range(experts):
        gate, up, down = (_t(tensors, f"{prefix}e{e}.{n}") for n in ("gate", "up", "down"))
        z = h @ gate.T
        y = ((z * torch.sigmoid(z)) * (h @ up.T)) @ down.T
        weight = (scores * (chosen.indices == e).any(-1, keepdim=True))[:, e:e + 1]
        out = out + weight * y
    return out


def layer(x, tensors, index, spec, eps):
    p = f"l{index}."

    def norm(name, v):
        return layer_norm(v, _t(tensors, p + name), _t(tensors, p + name + ".b"), eps)
    if spec["type"] != "latent_attention":
        raise ValueError(spec["type"])
    x = x + norm("norm1b", latent_attention(norm("norm1", x), tensors, p + "mix.", spec["mixer"], eps))
    if spec.get("mlp") is not None:
        x = x + norm("norm2b", routed_experts(norm("norm2", x), tensors, p + "mlp.", spec["mlp"]))
    return x


def program(config):
    """The layer runs in order: (layer index, pass number or None, first of its pass)."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(count)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t, i == loop["start"]))
    runs += [(i, None, False) for i in range(loop["stop"], count)]
    return runs


def forward(config, tensors, tokens, return_layers=False):
    """Logits [tokens, vocab] of one sequence (float64); with ``return_layers`` also the residual stream
    after every layer run."""
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = _t(tensors, "embed")[ids] * config["embedding"]["scale"]
    x = x0
    after = []
    for index, t, first in program(config):
        if first:
            x = torch.cat([x, x0], dim=-1) @ _t(tensors, "loop.in").T + _t(tensors, "loop.step")[t]
        x = layer(x, tensors, index, config["layers"][index], eps)
        after.append(x)
    y = layer_norm(x, _t(tensors, "final.norm"), _t(tensors, "final.norm.b"), eps)
    logits = y @ _t(tensors, "head").T
    return (logits, torch.stack(after)) if return_layers else logits
