"""Small Tosivik configurations and model folders for the tests.  None has the sizes of a real checkpoint; each makes
unequal what a convenient configuration would make equal or 1 (query and kv heads, the head's width and the rotated part
of it, key and value widths of the linear attention, the copies of the stream, the chosen experts)."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

import plain_tosivik as pt


def attention(heads, kv_heads, dim, chunk=None, rot_dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else dim ** -0.5}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot_dims != 0:
        m["rot"] = {"base": base, "dims": dim if rot_dims is None else rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "attention", "mixer": m}


def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp, weights_of=None):
    entry = dict(mixer, mlp=mlp)
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


def config(width, vocab, layers, streams=2, scale=1.0, eps=1e-5, bigram=(37, 5, 3), softcap=20.0):
    doc = {"architecture": "Tosivik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
           "layers": layers}
    if streams is not None:
        doc["streams"] = streams
    if bigram is not None:
        doc["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    if softcap is not None:
        doc["logit_softcap"] = softcap
    return doc


_A0 = attention(6, 2, 16, chunk=24, rot_dims=8, base=3000.0, scaling=(3.0, 64, 8.0, 1.0))
_L0 = lightning(3, 8, 12, (0.5, 0.97, 1.0))
#: three copies of the stream; grouped heads; half of each head rotated, wavelengths stretched; chunks of 24 positions; a
#: decay of exactly 1; layers 2 and 3 run the tensors of layers 0 and 1 again; dense, routed with and without a shared expert
SMALL_A = config(48, 90, [
    layer(_L0, dense(40)),
    layer(_A0, moe(5, 2, 24, shared=16)),
    layer(_L0, dense(40), weights_of=0),
    layer(_A0, moe(5, 2, 24, shared=16), weights_of=1),
    layer(lightning(2, 16, 8, (0.8, 0.3)), moe(4, 1, 20)),
], streams=3, scale=4.0)
#: no copies of the stream at all (the plain residual sum), no pair table, no cap on the logits, no mask, no rotation in
#: one layer and a whole-head rotation without stretching in the other, every expert chosen, a layer without a feed-forward
SMALL_B = config(40, 70, [
    layer(attention(4, 4, 8, rot_dims=0), moe(3, 3, 16)),
    layer(lightning(1, 24, 24, (0.9,)), None),
    layer(attention(2, 1, 24, base=500.0), dense(56)),
], streams=None, bigram=None, softcap=None, scale=0.7, eps=1e-6)
#: one copy with weights of its own; no size is a multiple of eight (rows off 16-byte borders, ragged tiles in every
#: kernel); a chunk smaller than a page and a chunk that is no multiple of a page
SMALL_C = config(36, 50, [
    layer(attention(3, 3, 10, chunk=5, rot_dims=6, scaling=(2.0, 20, 4.0, 0.5)), dense(28)),
    layer(lightning(3, 6, 10, (0.25, 0.6, 0.999)), moe(7, 3, 12, shared=20)),
    layer(attention(2, 1, 14, chunk=37, rot_dims=14), None),
], streams=1, bigram=(11, 2, 9), scale=2.0)
#: sizes that the tensor-core kernels of the bfloat16 path take (heads of 64 and 128 entries, grouped), four copies, chunks
#: of 96 and of 50 positions, a state of 128 x 128 per head (two slices of value columns)
SMALL_D = config(64, 100, [
    layer(attention(4, 2, 64, chunk=96, rot_dims=32, scaling=(4.0, 128, 16.0, 2.0)), dense(128)),
    layer(lightning(2, 128, 128, (0.99, 0.7)), moe(8, 2, 32, shared=32)),
    layer(attention(2, 2, 128, chunk=50), moe(8, 2, 32)),
    layer(lightning(4, 32, 80, (0.9, 0.95, 0.5, 1.0)), dense(72)),
], streams=4, scale=8.0, bigram=(101, 31, 7))


def make_folder(tmp_path, name: str, doc: dict, seed: int, dtype: torch.dtype, sharpen: float = 8.0) -> str:
    """A model folder from the engine's random-weights mode, changed so that faults show: query and key matrices are
    scaled up (peaked attention; linear attention whose state matters beside the norm's eps), the weights of the copies
    of the stream are spread, routers separate their experts and have biases that change the choice, the pair table is
    as large as the embedding."""
    from sglang_rs_b200.weights import read_model_dir, write_file, write_model_folder
    folder = write_model_folder(str(tmp_path / name), doc, seed=seed, dtype=dtype)
    tensors = {k: v.clone() for k, v in read_model_dir(folder).items()}
    generator = torch.Generator().manual_seed(seed)
    for key in tensors:
        shape = tensors[key].shape
        if key.endswith(("mix.q", "mix.k", "mix.v", "mix.g")):
            tensors[key] = (tensors[key].float() * sharpen).to(dtype)
        elif ".hc" in key:
            spread = torch.randn(shape, generator=generator) * 0.25
            tensors[key] = (spread + (torch.eye(shape[0]) if key.endswith("mix") else 0.7)).to(dtype)
        elif key.endswith("mlp.router"):
            tensors[key] = (tensors[key].float() * 60).to(dtype)
        elif key.endswith("router.b"):
            tensors[key] = (torch.randn(shape, generator=generator) * 1.5).to(dtype)
        elif key == "bigram":
            tensors[key] = (tensors[key].float() * doc["embedding"]["scale"]).to(dtype)
    write_file(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def load_folder(folder: str):
    from sglang_rs_b200.weights import read_model_dir
    with open(os.path.join(folder, "config.json")) as handle:
        doc = json.load(handle)
    return doc, read_model_dir(folder)


def random_requests(doc: dict, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(doc["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


def oracle(folder: str, requests: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    doc, tensors = load_folder(folder)
    return {rid: pt.logits(tokens, tensors, doc).numpy() for rid, tokens in requests.items()}


def plain_greedy(doc, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(torch.argmax(pt.logits(tokens, tensors, doc)[-1])))
    return tokens[len(prompt):]


MARK = 41          # the token that the made-up models below look for
FILL = 40          # what stands where the mark would be, in sequences without it


def marked_folder(tmp_path, dtype: torch.dtype, mixer: str, chunk: Optional[int] = None) -> str:
    """One layer that looks for the one position holding ``MARK``.

    Only that token's embedding has an entry in channel 0; channel 1 is the same constant in every embedding.
    ``attention``: head 0's key reads channel 0 into an unrotated entry, its query reads the constant into the same
    entry, so the mark's score stands far above all others wherever it is visible; the value is that key, and W_o
    carries the entry on.  ``lightning``: head 0 decays by 0.999 only, its key and value read channel 0 and its query
    the constant, so the state keeps the mark for hundreds of tokens and every later result holds it."""
    from sglang_rs_b200.weights import read_model_dir, write_file
    if mixer == "attention":
        first = attention(2, 1, 16, chunk=chunk, rot_dims=8, base=10000.0)
    else:
        first = lightning(2, 8, 8, (0.999, 0.5))
    doc = config(32, 60, [layer(first, dense(24))], streams=2, scale=1.0, bigram=None, softcap=None)
    folder = make_folder(tmp_path, f"marked_{mixer}", doc, seed=7, dtype=dtype, sharpen=8.0)
    t = {k: v.float().clone() for k, v in read_model_dir(folder).items()}
    t["embed"][:, 0] = 0
    t["embed"][MARK, 0] = 6.0
    t["embed"][:, 1] = 3.0
    t["l0.norm1"][:] = 1.0
    t["l0.hc1.in"][:] = torch.tensor([0.6, 0.4])
    entry = 15 if mixer == "attention" else 7                # head 0's last entry (outside the rotated ones)
    t["l0.mix.k"][entry] = 0
    t["l0.mix.k"][entry, 0] = 4.0
    t["l0.mix.q"][entry] = 0
    t["l0.mix.q"][entry, 1] = 6.0
    if mixer == "lightning":
        t["l0.mix.v"][:8] = 0
        t["l0.mix.v"][:8, 0] = 3.0
        t["l0.mix.g"][:8] = 0                                 # head 0's gates are one half, its results are carried on
        t["l0.mix.o"][:, :8] *= 40.0
    write_file(os.path.join(folder, "model.safetensors"), {k: v.to(dtype) for k, v in t.items()})
    return folder


def assert_rows_close(rows, expected, tolerance, dtype_name, what=""):
    """32-bit: every row within ``tolerance`` (largest difference over the largest |logit|).  bfloat16: a router's close
    call can go the other way once its input is rounded to 8 bits, which changes that row by far more than rounding does
    elsewhere; so there the rule is on the set of rows: at least 97 in 100 within ``tolerance`` and the median within a
    third of it.  A fault of a mechanism (a lost state, a key missed, a stale page) moves most rows and fails both."""
    errors, where = [], []
    for rid, by_pos in rows.items():
        scale = float(np.abs(expected[rid]).max())
        for pos, row in sorted(by_pos.items()):
            error = float(np.abs(row.astype(np.float64) - expected[rid][pos]).max()) / scale
            errors.append(error if np.isfinite(error) else float("inf"))
            where.append((rid, pos))
    errors = np.asarray(errors)
    worst = int(np.argmax(errors))
    if dtype_name == "float32":
        assert errors[worst] <= tolerance, (what, where[worst], float(errors[worst]))
        return
    over = int((errors > tolerance).sum())
    assert over <= 0.03 * len(errors) and float(np.median(errors)) <= tolerance / 3, \
        (what, over, len(errors), float(np.median(errors)), where[worst], float(errors[worst]))
