"""A plain, slow implementation of the Tosivik design, one function per mechanism, in float64 on the host.

It shares no code with the package: it reads the configuration document and a dict of tensors by their
checkpoint names.  The tests compare the engine with it.

Notation: a sequence is processed whole (no cache, no state carried over), so a token at position i sees
positions 0..i of its own sequence; ``xs`` are the copies of the residual stream [streams, tokens, width].
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def _t(tensors, name):
    return tensors[name].to(F)


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def silu(z):
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------- embedding

def bigram_rows(tokens, bigram):
    """Row of the pair table for every token: the last row for a sequence's first token."""
    rows = []
    for i, token in enumerate(tokens):
        if i == 0:
            rows.append(bigram["buckets"])
        else:
            rows.append((tokens[i - 1] * bigram["mul_prev"] + token * bigram["mul_cur"]) % bigram["buckets"])
    return rows


def embed(tokens, tensors, doc):
    e = doc["embedding"]
    x = _t(tensors, "embed")[torch.tensor(tokens)] * e["scale"]
    if e.get("bigram") is not None:
        x = x + _t(tensors, "bigram")[torch.tensor(bigram_rows(tokens, e["bigram"]))]
    return x


# ----------------------------------------------------------------------------- rotation

def rotary_frequencies(rot):
    """Angle per position of every rotated pair, with the stretching of long wavelengths, and the factor on
    cosines and sines.  Positions and angles are 32-bit in the design: the table is rounded once."""
    dims, base = rot["dims"], float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    magnitude = 1.0
    s = rot.get("scaling")
    if s is not None:
        def turn(t):
            return dims * math.log(s["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(turn(s["fast"])), 0)
        hi = min(math.ceil(turn(s["slow"])), dims - 1)
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / s["factor"] * ramp + f[i] * (1.0 - ramp)
        magnitude = 0.1 * math.log(s["factor"]) + 1.0
    return torch.tensor(f, dtype=F), magnitude


def rotate(v, positions, rot):
    """v [tokens, heads, dim]: the first rot.dims entries of each head are rotated, entry i with i + dims/2."""
    if rot is None or not rot.get("dims"):
        return v
    dims = rot["dims"]
    half = dims // 2
    freq, magnitude = rotary_frequencies(rot)
    angle = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(F)[:, None, :]
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


# ----------------------------------------------------------------------------- mixers

def visible(n, chunk):
    """[query, key] True where the query may see the key: causal, and inside the query's own chunk of
    positions (chunks counted from position 0) if there is one."""
    i = torch.arange(n)
    ok = i[None, :] <= i[:, None]
    if chunk:
        ok = ok & ((i[None, :] // chunk) == (i[:, None] // chunk))
    return ok


def attention(h, tensors, prefix, m):
    """Softmax attention whose values are the unrotated keys."""
    n = h.shape[0]
    heads, groups, dim = m["heads"], m["kv_heads"], m["dim"]
    positions = torch.arange(n)
    q = (h @ _t(tensors, prefix + "q").T).view(n, heads, dim)
    k = (h @ _t(tensors, prefix + "k").T).view(n, groups, dim)
    v = k[..., :m["vdim"]]
    q, k = rotate(q, positions, m.get("rot")), rotate(k, positions, m.get("rot"))
    per = heads // groups
    k_of = k[:, torch.arange(heads) // per]
    v_of = v[:, torch.arange(heads) // per]
    scores = torch.einsum("ihd,jhd->hij", q, k_of) * m["scale"]
    chunk = (m.get("mask") or {}).get("size")
    scores = scores.masked_fill(~visible(n, chunk)[None], float("-inf"))
    w = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", w, v_of)
    return out.reshape(n, -1) @ _t(tensors, prefix + "o").T


def lightning(h, tensors, prefix, m, eps):
    """Linear attention with one fixed decay per head, token by token; the state starts at zero."""
    n = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ _t(tensors, prefix + "q").T).view(n, heads, dim)
    k = silu(h @ _t(tensors, prefix + "k").T).view(n, heads, dim)
    v = silu(h @ _t(tensors, prefix + "v").T).view(n, heads, vdim)
    decay = torch.tensor(m["decay"], dtype=F)
    state = torch.zeros(heads, dim, vdim, dtype=F)
    out = torch.zeros(n, heads, vdim, dtype=F)
    for t in range(n):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    o = rms_norm(out.reshape(n, heads * vdim), _t(tensors, prefix + "norm"), eps)
    o = o * torch.sigmoid(h @ _t(tensors, prefix + "g").T)
    return o @ _t(tensors, prefix + "o").T


# ----------------------------------------------------------------------------- feed-forwards

def two_layer(h, tensors, prefix, act):
    return act(h @ _t(tensors, prefix + "up").T) @ _t(tensors, prefix + "down").T


def routed(h, tensors, prefix, mlp):
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ _t(tensors, prefix + "router").T + _t(tensors, prefix + "router.b")
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(z[t, e]), e))[:top]
        w = torch.softmax(z[t, order], dim=0)
        for weight, e in zip(w, order):
            out[t] += weight * two_layer(h[t:t + 1], tensors, f"{prefix}e{e}.", relu_squared)[0]
    if mlp.get("shared") is not None:
        out = out + two_layer(h, tensors, prefix + "shared.", relu_squared)
    return out


def feed_forward(h, tensors, prefix, mlp):
    if mlp["kind"] == "dense":
        return two_layer(h, tensors, prefix, gelu_tanh)
    return routed(h, tensors, prefix, mlp)


# ----------------------------------------------------------------------------- layers

def sublayer(xs, tensors, owner, q, eps, inner, streams):
    """One sublayer behind its norm.  With several copies of the stream: read a weighted sum of the copies,
    then every copy becomes a mixture of the old ones plus its share of the result."""
    norm = _t(tensors, f"{owner}.norm{q}")
    if streams is None:
        return xs + inner(rms_norm(xs[0], norm, eps))[None]
    read, write, mix = (_t(tensors, f"{owner}.hc{q}.{n}") for n in ("in", "out", "mix"))
    u = torch.einsum("s,sik->ik", read, xs)
    y = inner(rms_norm(u, norm, eps))
    return torch.einsum("st,sik->tik", mix, xs) + write[:, None, None] * y[None]


def layer_runs(tokens, tensors, doc):
    """Yields the residual stream (the sum of its copies) after every layer run; the last value is the
    input of the final norm."""
    eps = doc["norm"]["eps"]
    streams = doc.get("streams")
    x = embed(tokens, tensors, doc)
    xs = torch.stack([x] * (streams or 1))
    for index, entry in enumerate(doc["layers"]):
        owner = f"l{entry['weights_of']}" if entry.get("weights_of") is not None else f"l{index}"
        m = entry["mixer"]
        if entry["type"] == "attention":
            mixer = lambda h: attention(h, tensors, owner + ".mix.", m)
        else:
            mixer = lambda h: lightning(h, tensors, owner + ".mix.", m, eps)
        xs = sublayer(xs, tensors, owner, 1, eps, mixer, streams)
        if entry.get("mlp") is not None:
            xs = sublayer(xs, tensors, owner, 2, eps, lambda h: feed_forward(h, tensors, owner + ".mlp.", entry["mlp"]),
                          streams)
        yield xs.sum(0)


def logits(tokens, tensors, doc):
    """[tokens, vocab] for one sequence from its first token."""
    x = None
    for x in layer_runs(tokens, tensors, doc):
        pass
    out = rms_norm(x, _t(tensors, "final.norm"), doc["norm"]["eps"]) @ _t(tensors, "head").T
    cap = doc.get("logit_softcap")
    return cap * torch.tanh(out / cap) if cap else out


# ----------------------------------------------------------------------------- for tests of single kernels

def attend(q, k, v, scale, chunk, first_position):
    """q [rows, heads, d] are the positions first_position .. of a sequence whose keys k and values v
    [keys, kv heads, d] start at position 0; returns [rows, heads, d]."""
    rows, heads, _ = q.shape
    per = heads // k.shape[1]
    out = torch.zeros(rows, heads, v.shape[2], dtype=F)
    for r in range(rows):
        pos = first_position + r
        lo = pos // chunk * chunk if chunk else 0
        for h in range(heads):
            s = (k[lo:pos + 1, h // per] @ q[r, h]) * scale
            out[r, h] = torch.softmax(s, 0) @ v[lo:pos + 1, h // per]
    return out


def linear_attention(q, k, v, decay, state):
    """Token by token from ``state`` [heads, dim, vdim]; q, k [n, heads, dim], v [n, heads, vdim], already
    activated.  Returns the results [n, heads, vdim] and the state after the last token."""
    state = state.clone()
    out = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=F)
    d = torch.tensor(decay, dtype=F)[:, None, None]
    for t in range(q.shape[0]):
        state = d * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    return out, state
