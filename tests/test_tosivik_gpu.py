"""Tosivik on the GPU against the plain implementation: each mechanism alone, whole prompts, prompts with a tail decoded
token by token, portions down to two tokens, mixed batches over a small pool (pages and state slots are used again), keys
just inside and just outside a chunk of the mask, a state that must survive hundreds of tokens, long decoding from captured
graphs, and greedy generation through the entry point, the command line and the trace program."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_tosivik as pt
import replay_helpers as rh
import tosivik_helpers as th

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 1e-4), ("bfloat16", torch.bfloat16, 4e-2)]
BOTH = [torch.float32, torch.bfloat16]


def seen(tensor, dtype):
    """What the kernel sees of a tensor: rounded to the storage type, as float64."""
    return tensor.to(dtype).to(torch.float64)


def close(got, want, dtype, what, fraction=None):
    tolerance = fraction if fraction is not None else (2e-5 if dtype == torch.float32 else 2e-2)
    scale = float(want.abs().max()) or 1.0
    error = float((got.detach().cpu().to(torch.float64) - want).abs().max()) / scale
    assert error <= tolerance, (what, error)


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("streams", [1, 3, 8])
def test_copies_of_the_stream_update_read_and_norm_in_one_kernel(dtype, streams):
    from sglang_rs_b200 import ops
    torch.manual_seed(streams)
    rows, width = 9, 70
    x = torch.randn(rows, streams, width) * 2
    y = torch.randn(rows, width) * 3
    mix, spread, gather = torch.randn(streams, streams), torch.randn(streams), torch.randn(streams)
    weight = torch.rand(width) + 0.5
    fresh = torch.einsum("st,rsk->rtk", mix.double(), x.double()) + spread.double()[None, :, None] * seen(y, dtype)[:, None, :]
    u = torch.einsum("t,rtk->rk", gather.double(), fresh)
    want = pt.rms_norm(u, weight.double(), 1e-5)
    on = x.to(DEV)
    out = torch.empty((rows, width), dtype=dtype, device=DEV)
    ops.stream_step(on, y.to(DEV, dtype), mix.to(DEV), spread.to(DEV), gather.to(DEV), weight.to(DEV), 1e-5, out)
    close(on, fresh, torch.float32, "all copies replaced at once from the old ones")
    close(out, want, dtype, "norm of what is read")
    # the result as 32-bit partial sums; picked rows leave the copies as they are
    parts = torch.randn(3, rows, width)
    fresh = torch.einsum("st,rsk->rtk", mix.double(), x.double()) + spread.double()[None, :, None] * parts.double().sum(0)[:, None, :]
    on = x.to(DEV)
    index = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    picked = torch.empty((3, width), dtype=dtype, device=DEV)
    ops.stream_step(on, parts.to(DEV), mix.to(DEV), spread.to(DEV), gather.to(DEV), weight.to(DEV), 1e-5, picked, row_index=index)
    close(picked, pt.rms_norm(torch.einsum("t,rtk->rk", gather.double(), fresh), weight.double(), 1e-5)[[7, 0, 3]], dtype, "picked rows")
    assert torch.equal(on.cpu(), x)
    # a read without an update before it
    ops.stream_step(on, None, None, None, gather.to(DEV), weight.to(DEV), 1e-5, out)
    close(out, pt.rms_norm(torch.einsum("t,rtk->rk", gather.double(), x.double()), weight.double(), 1e-5), dtype, "read alone")


@pytest.mark.parametrize("dtype", BOTH)
def test_embedding_with_a_row_chosen_by_two_tokens(dtype):
    """Three requests in one step (a first portion, a later portion, one decoded token), then the next step: the token
    before a portion's first row comes from the slot that the step before wrote."""
    from sglang_rs_b200 import ops
    torch.manual_seed(3)
    vocab, width, buckets, mp, mc, copies = 50, 24, 13, 31, 7, 3
    table, pairs = torch.randn(vocab, width), torch.randn(buckets + 1, width)
    last = torch.full((6,), 49, dtype=torch.int32, device=DEV)             # slots 1, 4, 2 are used; what they hold is stale
    last[4], last[2] = 17, 33
    sequences = {1: ([], [5, 9, 9, 2]), 4: ([0] * 6 + [17], [8, 1]), 2: ([3] * 10 + [33], [44])}
    word = ops.new_error_word(DEV)

    def step(chunks, slots):
        ids = [t for c in chunks for t in c[1]]
        positions = [len(c[0]) + i for c in chunks for i in range(len(c[1]))]
        row_request = [r for r, c in enumerate(chunks) for _ in c[1]]
        cu = np.cumsum([0] + [len(c[1]) for c in chunks]).tolist()
        def dev(values):
            return torch.tensor(values, dtype=torch.int32, device=DEV)
        out = torch.empty((len(ids), copies * width), device=DEV)
        ops.embedding_pairs(dev(ids), table.to(DEV, dtype), out, word, scale=2.5, copies=copies, pairs=pairs.to(DEV, dtype),
                            buckets=buckets, mul_prev=mp, mul_cur=mc, positions=dev(positions), row_request=dev(row_request),
                            cu_rows=dev(cu), state_slots=dev(slots), last_token=last)
        ops.remember_tokens(dev(ids), dev(cu), dev(slots), last, len(chunks))
        want = []
        for before, tokens in chunks:
            whole = before + tokens
            rows = pt.bigram_rows(whole, {"buckets": buckets, "mul_prev": mp, "mul_cur": mc})[len(before):]
            want.append(seen(table, dtype)[tokens] * 2.5 + seen(pairs, dtype)[rows])
        want = torch.cat(want)
        for c in range(copies):
            close(out.view(-1, copies, width)[:, c], want, torch.float32, f"copy {c}", 1e-6)
    step([sequences[1], sequences[4], sequences[2]], [1, 4, 2])
    assert last.tolist() == [49, 2, 44, 49, 1, 49]
    step([([3] * 10 + [33, 44], [6]), ([5, 9, 9, 2], [7, 7, 30])], [2, 1])
    assert int(word.item()) == 0


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows,n_q,n_kv,d,rot", [(5, 3, 1, 24, 8), (70, 4, 2, 16, 16), (300, 4, 2, 128, 128), (300, 2, 2, 128, 64)])
def test_rotation_with_a_magnitude_and_values_that_are_the_unrotated_keys(dtype, rows, n_q, n_kv, d, rot):
    """Few rows, many rows and the kernel for heads of 128 entries (which the last case, rotating half a head, does not
    take) give the same: q and k rotated and scaled, the value pool holding k as projected."""
    from sglang_rs_b200 import ops
    from sglang_rs_b200.parts import RotaryEncoding, WavelengthScaling
    g = torch.Generator().manual_seed(rows + rot)
    page = 8
    pages = -(-rows // page) + 1
    qk = torch.randn(rows, (n_q + n_kv) * d, generator=g)
    slots = torch.randperm(pages * page, generator=g)[:rows].to(torch.int32)
    positions = torch.randint(0, 5000, (rows,), generator=g, dtype=torch.int32)
    positions[0] = 0
    rotary = {"dims": rot, "base": 5000.0, "scaling": {"factor": 3.0, "original": 256, "fast": 16.0, "slow": 2.0}}
    part = RotaryEncoding(d, 5000.0, rotary_dim=rot, scaling=WavelengthScaling(3.0, 256, 16.0, 2.0))
    part.load({}, DEV, dtype)
    table = part.fused_rotary()
    k_pool = torch.zeros(pages, n_kv, page, d, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty(rows, n_q, d, device=DEV, dtype=dtype)
    word = ops.new_error_word(DEV)
    ops.qk_norm_rope_kv(qk.to(DEV, dtype), q_out, k_pool, v_pool, positions.to(DEV), slots.to(DEV), None, None, 0.0,
                        table.inv_freq, rot, False, n_q, n_kv, d, word, magnitude=table.magnitude, values_from_keys=True)
    ops.raise_on_error_word(word)
    x = seen(qk, dtype)
    q = pt.rotate(x[:, :n_q * d].view(rows, n_q, d), positions, rotary)
    k_plain = x[:, n_q * d:].view(rows, n_kv, d)
    close(q_out, q, dtype, "q")
    at = (slots.long() // page, slots.long() % page)
    close(k_pool.cpu()[at[0], :, at[1]], pt.rotate(k_plain, positions, rotary), dtype, "rotated keys")
    close(v_pool.cpu()[at[0], :, at[1]], k_plain, dtype, "values: the keys as projected", 1e-6)
    assert table.magnitude > 1.05


def attention_case(dtype, n_q, n_kv, d, page, lengths, rows_per_request, seed, boost=None):
    """Requests whose keys lie scattered over shuffled pages; the last ``rows`` positions of each are the step's rows.
    ``boost`` = (request, key position, factor): that key is made to stand out for the request's last row."""
    g = torch.Generator().manual_seed(seed)
    total = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(total, generator=g).tolist()
    k_pool, v_pool = torch.randn(total, n_kv, page, d, generator=g), torch.randn(total, n_kv, page, d, generator=g)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    case = dict(ks=[], vs=[], qs=[], lengths=lengths, rows=rows_per_request, dtype=dtype)
    positions, row_request = [], []
    for r, (n, rows) in enumerate(zip(lengths, rows_per_request)):
        k, v, q = torch.randn(n, n_kv, d, generator=g), torch.randn(n, n_kv, d, generator=g), torch.randn(rows, n_q, d, generator=g)
        if boost is not None and boost[0] == r:
            k[boost[1]] = q[-1, ::n_q // n_kv] * boost[2]
        for j in range(-(-n // page)):
            p = order.pop()
            table[r, j] = p
            part = slice(j * page, min(n, (j + 1) * page))
            k_pool[p, :, :part.stop - part.start] = k[part].transpose(0, 1)
            v_pool[p, :, :part.stop - part.start] = v[part].transpose(0, 1)
        case["ks"].append(k); case["vs"].append(v); case["qs"].append(q)
        positions += list(range(n - rows, n))
        row_request += [r] * rows
    case.update(k_pool=k_pool.to(DEV, dtype), v_pool=v_pool.to(DEV, dtype), table=table.to(DEV), q=torch.cat(case["qs"]).to(DEV, dtype),
                positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                row_request=torch.tensor(row_request, dtype=torch.int32, device=DEV))
    return case


def plain_case(case, scale, chunk):
    return torch.cat([pt.attend(seen(q, case["dtype"]), seen(k, case["dtype"]), seen(v, case["dtype"]), scale, chunk, n - rows)
                      for k, v, q, n, rows in zip(case["ks"], case["vs"], case["qs"], case["lengths"], case["rows"])])


def run_generic(case, scale, chunk, split):
    from sglang_rs_b200 import ops
    rows, n_q, d = case["q"].shape
    out = torch.full_like(case["q"], float("nan"))
    splits = int(case["positions"].max()) // split + 1 if split else 1
    acc = torch.full((rows * n_q * splits * d,), float("nan"), device=DEV)
    ml = torch.full((rows * n_q * splits * 2,), float("nan"), device=DEV)
    word = ops.new_error_word(DEV)
    ops.paged_attention(case["q"], case["k_pool"], case["v_pool"], out, case["positions"], case["row_request"], case["table"],
                        scale=scale, window=0, split_size=split, max_splits=splits, scratch_acc=acc, scratch_ml=ml,
                        error_word=word, chunk=chunk)
    ops.raise_on_error_word(word)
    return out


def tiles_of(case, tile_rows):
    tiles, first = [], 0
    for r, (n, rows) in enumerate(zip(case["lengths"], case["rows"])):
        for begin in range(0, rows, tile_rows):
            tiles.append([first + begin, min(tile_rows, rows - begin), r, n - rows + begin])
        first += rows
    return torch.tensor(tiles, dtype=torch.int32, device=DEV)


def run_tensor_core(case, scale, chunk, kind):
    from sglang_rs_b200 import ops
    q = case["q"]
    out = torch.full_like(q, float("nan"))
    word = ops.new_error_word(DEV)
    if kind == "decode":
        rows, n_q, d = q.shape
        n_kv = case["k_pool"].shape[1]
        splits = ops.decode_splits(rows, n_kv, None)
        acc = torch.full((rows * n_q * splits * d,), float("nan"), device=DEV)
        ml = torch.full((rows * n_q * splits * 2,), float("nan"), device=DEV)
        counters = torch.zeros(rows * n_kv, dtype=torch.int32, device=DEV)
        ops.decode_attention(q, case["k_pool"], case["v_pool"], out, case["positions"], case["row_request"], case["table"],
                             scale=scale, window=0, scratch_acc=acc, scratch_ml=ml, counters=counters, error_word=word, chunk=chunk)
    elif kind == "tiles":
        ops.tiled_attention(q, case["k_pool"], case["v_pool"], out, tiles_of(case, 64), case["table"], scale=scale, window=0,
                            error_word=word, chunk=chunk)
    else:
        ops.tiled_attention_tc(q, case["k_pool"], case["v_pool"], out, tiles_of(case, 128), case["table"], scale=scale, window=0,
                               error_word=word, chunk=chunk)
    ops.raise_on_error_word(word)
    return out


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("n_q,n_kv,d,page,chunk", [(4, 2, 16, 16, 24), (3, 3, 10, 8, 5), (6, 1, 48, 16, 96), (2, 2, 40, 4, 37)])
@pytest.mark.parametrize("split", [0, 32])
def test_attention_inside_chunks_of_positions(dtype, n_q, n_kv, d, page, chunk, split):
    lengths, rows = (1, 33, 300, chunk, chunk + 1, 2 * chunk, 257), (1, 5, 130, 1, 1, chunk + 3, 70)
    case = attention_case(dtype, n_q, n_kv, d, page, lengths, rows, seed=d + chunk)
    scale = 0.8 / math.sqrt(d)
    close(run_generic(case, scale, chunk, split), plain_case(case, scale, chunk), dtype, "chunked attention")


@pytest.mark.parametrize("kind,rows", [("decode", (1, 1, 1, 1, 1, 1)), ("tiles", (1, 5, 130, 64, 70, 200)), ("tensor memory", (1, 5, 130, 64, 70, 200))])
@pytest.mark.parametrize("n_q,n_kv,d,page,chunk", [(4, 2, 64, 16, 96), (6, 3, 128, 8, 50), (4, 4, 128, 16, 64), (2, 1, 64, 32, 200)])
def test_tensor_core_attention_inside_chunks_of_positions(kind, rows, n_q, n_kv, d, page, chunk):
    lengths = (1, 33, 300, chunk, 2 * chunk + 1, 700)
    case = attention_case(torch.bfloat16, n_q, n_kv, d, page, lengths, tuple(min(r, n) for r, n in zip(rows, lengths)), seed=d + chunk)
    scale = 1.0 / math.sqrt(d)
    close(run_tensor_core(case, scale, chunk, kind), plain_case(case, scale, chunk), torch.bfloat16, kind)


@pytest.mark.parametrize("kind", ["generic32", "generic", "split", "decode", "tiles", "tensor memory"])
def test_a_key_just_inside_and_just_outside_the_chunk(kind):
    """The last row's query is made to stand out against one key: the first key of its chunk (seen: the result is that
    key's value) or the last key of the chunk before (not seen), with the chunk's edge off every page border."""
    dtype = torch.float32 if kind == "generic32" else torch.bfloat16
    chunk, n, d = 44, 150, 64                                 # the last row is at 149: its chunk starts at 132
    for key, visible in ((132, True), (131, False), (148, True), (87, False), (0, False)):
        rows = 1 if kind in ("decode", "split") else 5
        case = attention_case(dtype, 2, 1, d, 16, (70, n), (3 if rows > 1 else 1, rows), seed=5, boost=(1, key, 4.0))
        scale = 1.0 / 8.0
        if kind in ("generic32", "generic", "split"):
            out = run_generic(case, scale, chunk, 32 if kind == "split" else 0)
        else:
            out = run_tensor_core(case, scale, chunk, kind)
        close(out, plain_case(case, scale, chunk), dtype, f"key {key}")
        near = float((out[-1, 0].double().cpu() - seen(case["vs"][1][key, 0], dtype)).abs().max()) < 0.05
        assert near == visible, (key, kind)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 8, 12), (2, 128, 128), (1, 24, 70), (5, 6, 10)])
def test_linear_attention_over_states_in_slots(dtype, heads, dim, vdim):
    """Three requests in one step (a prompt from position 0 in a slot that holds rubbish, a later portion from a given
    state, one decoded token), then a second step that continues the first two from the states the first step left."""
    from sglang_rs_b200 import ops
    torch.manual_seed(dim + vdim)
    decay = [1.0, 0.2, 0.97, 0.5, 0.999][:heads]
    counts, starts, slots = [45, 33, 1], [0, 70, 9], [2, 0, 3]
    total = sum(counts)
    width = heads * (2 * dim + 2 * vdim) + 3
    proj = torch.randn(total + 40, width)
    state = torch.randn(5, heads, dim, vdim, device=DEV)
    given = state.cpu().double()
    offsets = (1, 1 + heads * dim, 1 + 2 * heads * dim)

    def parts(rows):
        x = seen(proj[rows], dtype)
        return (pt.silu(x[:, offsets[0]:offsets[0] + heads * dim]).view(-1, heads, dim),
                pt.silu(x[:, offsets[1]:offsets[1] + heads * dim]).view(-1, heads, dim),
                pt.silu(x[:, offsets[2]:offsets[2] + heads * vdim]).view(-1, heads, vdim))

    def dev(values):
        return torch.tensor(values, dtype=torch.int32, device=DEV)
    cu = np.cumsum([0] + counts).tolist()
    positions = [s + i for s, c in zip(starts, counts) for i in range(c)]
    out = torch.full((total, heads * vdim), float("nan"), device=DEV)
    ops.lightning_scan(proj[:total].to(DEV, dtype), *offsets, dev(cu), dev(positions), dev(slots), state,
                       torch.tensor(decay, device=DEV), out, 3)
    after = {}
    for r in range(3):
        rows = slice(cu[r], cu[r + 1])
        begin = torch.zeros(heads, dim, vdim, dtype=torch.float64) if starts[r] == 0 else given[slots[r]]
        want, after[r] = pt.linear_attention(*parts(rows), decay, begin)
        close(out[rows], want.reshape(-1, heads * vdim), torch.float32, f"request {r}", 3e-5)
        close(state[slots[r]], after[r], torch.float32, f"state of request {r}", 3e-5)
    close(state[1], given[1], torch.float32, "a slot that no request holds", 0.0)
    # the next step: two tokens of request 0, 38 of request 1; a read-only run leaves the states alone
    counts2, rows2 = [2, 38], slice(total, total + 40)
    cu2 = [0, 2, 40]
    positions2 = [45, 46] + list(range(103, 141))
    out2 = torch.full((40, heads * vdim), float("nan"), device=DEV)
    before = state.clone()
    ops.lightning_scan(proj[rows2].to(DEV, dtype), *offsets, dev(cu2), dev(positions2), dev(slots[:2]), state,
                       torch.tensor(decay, device=DEV), out2, 2, read_only=True)
    assert torch.equal(state, before)
    q, k, v = parts(rows2)
    for r in range(2):
        part = slice(cu2[r], cu2[r + 1])
        want, _ = pt.linear_attention(q[part], k[part], v[part], decay, after[r])
        close(out2[part], want.reshape(-1, heads * vdim), torch.float32, f"second step, request {r}", 3e-5)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 8, 12), (2, 128, 128), (1, 24, 70), (5, 6, 10), (4, 33, 32)])
def test_linear_attention_of_a_step_of_decoded_tokens(dtype, heads, dim, vdim):
    """Every request brings one row: one pass over the states.  One request is at position 0 in a slot that holds
    rubbish; a read-only run leaves the states alone and gives the same results."""
    from sglang_rs_b200 import ops
    torch.manual_seed(dim * vdim)
    decay = [1.0, 0.2, 0.97, 0.5, 0.999][:heads]
    slots, positions = [3, 0, 5, 1], [17, 0, 400, 1]
    width = heads * (2 * dim + vdim) + 5
    proj = torch.randn(4, width)
    state = torch.randn(6, heads, dim, vdim, device=DEV)
    given = state.cpu().double()
    offsets = (2, 2 + heads * dim, 2 + 2 * heads * dim)
    x = seen(proj, dtype)
    q = pt.silu(x[:, offsets[0]:offsets[0] + heads * dim]).view(4, heads, dim)
    k = pt.silu(x[:, offsets[1]:offsets[1] + heads * dim]).view(4, heads, dim)
    v = pt.silu(x[:, offsets[2]:offsets[2] + heads * vdim]).view(4, heads, vdim)

    def dev(values):
        return torch.tensor(values, dtype=torch.int32, device=DEV)
    for read_only in (True, False):
        out = torch.full((4, heads * vdim), float("nan"), device=DEV)
        ops.lightning_scan(proj.to(DEV, dtype), *offsets, dev([0, 1, 2, 3, 4]), dev(positions), dev(slots), state,
                           torch.tensor(decay, device=DEV), out, 4, read_only=read_only, single_rows=True)
        for r in range(4):
            begin = torch.zeros(heads, dim, vdim, dtype=torch.float64) if positions[r] == 0 else given[slots[r]]
            want, after = pt.linear_attention(q[r:r + 1], k[r:r + 1], v[r:r + 1], decay, begin)
            close(out[r:r + 1], want.reshape(1, -1), torch.float32, f"request {r}", 3e-5)
            close(state[slots[r]], given[slots[r]] if read_only else after, torch.float32, f"state of request {r}", 3e-5)
    close(state[2], given[2], torch.float32, "a slot that no request holds", 0.0)


@pytest.mark.parametrize("heads,dim,vdim", [(3, 64, 128), (2, 128, 128), (2, 128, 64), (5, 64, 64)])
def test_linear_attention_in_parallel_chunks_on_the_tensor_cores(heads, dim, vdim):
    """Four requests in one step: a prompt of three chunks and a bit from position 0 in a slot that holds rubbish, a
    portion that ends exactly at a chunk's end from a given state, a single token, and two tokens; then the next step
    continues two of them.  q, k and v are the rounded activations; everything else is held to 32-bit accuracy."""
    from sglang_rs_b200 import ops
    torch.manual_seed(dim + vdim)
    decay = [1.0, 0.3, 0.97, 0.999, 0.9][:heads]
    counts, starts, slots = [401, 256, 1, 2], [0, 70, 9, 500], [2, 0, 3, 4]
    total = sum(counts)
    offsets = (8, 8 + heads * dim, 8 + 2 * heads * dim)
    width = 8 + heads * (2 * dim + vdim) + 16
    proj = torch.randn(total + 90, width)
    state = torch.randn(6, heads, dim, vdim, device=DEV) * 0.5
    given = state.cpu().double()

    def parts(rows):
        x = seen(proj[rows], torch.bfloat16)
        def act(lo, n, d):
            return seen(pt.silu(x[:, lo:lo + heads * d]), torch.bfloat16).view(-1, heads, d)
        return act(offsets[0], heads, dim), act(offsets[1], heads, dim), act(offsets[2], heads, vdim)

    def dev(values):
        return torch.tensor(values, dtype=torch.int32, device=DEV)

    def run(rows, counts, starts, slots, begin_states, read_only=False):
        cu = np.cumsum([0] + counts).tolist()
        positions = [s + i for s, c in zip(starts, counts) for i in range(c)]
        out = torch.full((sum(counts), heads * vdim), float("nan"), device=DEV)
        chunks = sum(-(-c // ops.LIGHTNING_CHUNK_TOKENS) for c in counts)
        ops.lightning_chunks(proj[rows].to(DEV, torch.bfloat16), *offsets, dev(cu), dev(positions), dev(slots), state,
                             torch.tensor(decay, device=DEV), out, len(counts), chunks, read_only=read_only)
        q, k, v = parts(rows)
        after = []
        for r in range(len(counts)):
            part = slice(cu[r], cu[r + 1])
            want, last = pt.linear_attention(q[part], k[part], v[part], decay, begin_states[r])
            close(out[part], want.reshape(-1, heads * vdim), torch.float32, f"request {r}", 1e-4)
            after.append(last)
        return after
    zero = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    after = run(slice(0, total), counts, starts, slots, [zero, given[0], given[3], given[4]])
    for r in range(4):
        close(state[slots[r]], after[r], torch.float32, f"state of request {r}", 1e-4)
    close(state[1], given[1], torch.float32, "a slot that no request holds", 0.0)
    before = state.clone()
    run(slice(total, total + 90), [70, 20], [401, 326], [2, 0], [after[0], after[1]], read_only=True)
    assert torch.equal(state, before)


def test_linear_attention_with_a_decay_whose_powers_vanish():
    """600 tokens at a decay of 0.01: powers of the decay underflow to zero, and nothing becomes infinite or NaN."""
    from sglang_rs_b200 import ops
    torch.manual_seed(0)
    heads, dim, vdim, n = 2, 8, 8, 600
    proj = torch.randn(n, heads * (2 * dim + vdim))
    state = torch.zeros(1, heads, dim, vdim, device=DEV)
    out = torch.empty((n, heads * vdim), device=DEV)
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.lightning_scan(proj.to(DEV), 0, heads * dim, 2 * heads * dim, torch.tensor([0, n], dtype=torch.int32, device=DEV),
                       torch.arange(n, dtype=torch.int32, device=DEV), zero, state, torch.tensor([0.01, 0.0], device=DEV), out, 1)
    x = proj.double()
    want, _ = pt.linear_attention(pt.silu(x[:, :16]).view(n, 2, 8), pt.silu(x[:, 16:32]).view(n, 2, 8), pt.silu(x[:, 32:]).view(n, 2, 8),
                                  [0.01, 0.0], torch.zeros(2, 8, 8, dtype=torch.float64))
    assert bool(torch.isfinite(out).all())
    close(out, want.reshape(n, -1), torch.float32, "vanishing decay", 3e-5)


@pytest.mark.parametrize("dtype", BOTH)
def test_heads_normed_together_and_gated(dtype):
    from sglang_rs_b200 import ops
    torch.manual_seed(2)
    rows, width = 11, 36
    o, proj, weight = torch.randn(rows, width) * 4, torch.randn(rows, width + 9) * 2, torch.rand(width) + 0.5
    out = torch.empty((rows, width), dtype=dtype, device=DEV)
    ops.lightning_gate_norm(o.to(DEV), proj.to(DEV, dtype), 9, weight.to(DEV), 1e-5, out)
    close(out, pt.rms_norm(o.double(), weight.double(), 1e-5) * torch.sigmoid(seen(proj, dtype)[:, 9:]), dtype, "norm and gate")


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("experts,top,rows,shared", [(5, 2, 150, True), (3, 3, 9, False), (4, 1, 1, True), (70, 4, 40, True), (3, 2, 500, True)])
def test_experts_without_a_gate_with_a_router_bias_and_a_shared_expert(dtype, experts, top, rows, shared):
    from sglang_rs_b200 import ops
    torch.manual_seed(5)
    width, inner = 40, 24
    h = torch.randn(rows, width)
    tensors = {"p.router": torch.randn(experts, width) * 0.6, "p.router.b": torch.randn(experts) * 2,
               "p.shared.up": torch.randn(16, width) * 0.2, "p.shared.down": torch.randn(width, 16) * 0.2}
    for e in range(experts):
        tensors.update({f"p.e{e}.up": torch.randn(inner, width) * 0.2, f"p.e{e}.down": torch.randn(width, inner) * 0.2})
    stacked = {n: torch.stack([tensors[f"p.e{e}.{n}"] for e in range(experts)]).to(DEV, dtype) for n in ("up", "down")}
    word = ops.new_error_word(DEV)
    rounded = {k: seen(v, dtype) if k != "p.router.b" else v.double() for k, v in tensors.items()}
    base = None
    if shared:
        base = (pt.two_layer(seen(h, dtype), rounded, "p.shared.", pt.relu_squared)).to(torch.float32).to(DEV)
    out = ops.routed_experts(h.to(DEV, dtype), tensors["p.router"].to(DEV, dtype), stacked["up"], stacked["down"], top, "relu2", True,
                             word, gated=False, router_bias=tensors["p.router.b"].to(DEV), base=base)
    mlp = {"router": {"experts": experts, "top": top}}
    want = pt.routed(seen(h, dtype), rounded, "p.", mlp)
    if shared:
        want = want + base.cpu().double()
    assert out.dtype == torch.float32 and int(word.item()) == 0
    close(out, want, dtype, "weighted sum of the chosen experts")
    # the bias decides: without it other experts are chosen for some row
    z = seen(h, dtype) @ rounded["p.router"].T
    if top < experts and rows >= 9:
        assert not torch.equal(torch.topk(z, top).indices.sort().values, torch.topk(z + rounded["p.router.b"], top).indices.sort().values)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows", [3, 64, 200, 1500])
def test_feed_forward_without_a_gate_and_the_cap_on_logits(dtype, rows):
    from sglang_rs_b200 import ops
    from sglang_rs_b200.parts import PlainMlp
    torch.manual_seed(rows)
    width, inner = 48, 72
    x = torch.randn(rows, width)
    tensors = {"f.up": torch.randn(inner, width) * 0.3, "f.down": torch.randn(width, inner) * 0.3}
    word = ops.new_error_word(DEV)

    class Ctx:
        error_word = word
    for activation, plain in (("gelu_tanh", pt.gelu_tanh), ("relu2", pt.relu_squared)):
        part = PlainMlp(width, inner, activation, "f.up", "f.down", float_result=activation == "relu2")
        part.load(tensors, DEV, dtype)
        out = part.forward(Ctx, x.to(DEV, dtype))
        if out.dim() == 3:
            out = out.sum(0)
        hidden = plain(seen(x, dtype) @ seen(tensors["f.up"], dtype).T)
        if dtype == torch.bfloat16:
            hidden = seen(hidden, dtype)
        close(out, hidden @ seen(tensors["f.down"], dtype).T, dtype, activation)
    logits = torch.randn(rows, 70, device=DEV) * 40
    want = 25.0 * torch.tanh(logits.double().cpu() / 25.0)
    ops.softcap(logits, 25.0)
    close(logits, want, torch.float32, "cap", 1e-6)
    assert int(word.item()) == 0


# ------------------------------------------------------------------------------ whole models, every way of cutting
@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
@pytest.mark.parametrize("doc", [th.SMALL_A, th.SMALL_B, th.SMALL_C, th.SMALL_D], ids=["a", "b", "c", "d"])
def test_prompts_tails_portions_and_mixed_batches(tmp_path, doc, dtype_name, stored, tolerance):
    folder = th.make_folder(tmp_path, "m", doc, seed=5, dtype=stored)
    requests = th.random_requests(doc, (1, 2, 23, 64, 65, 150, 131), seed=3)
    expected = th.oracle(folder, requests)
    worst = {}
    for name, trace, page in (("whole", rh.trace_whole(requests), 16), ("tail", rh.trace_tail_by_one(requests, tail=20), 16),
                              ("portions", rh.trace_portions(requests), 8), ("mixed", rh.trace_mixed(requests, seed=9), 16)):
        # the pool holds what is live at any time and no more, so pages and state slots go from one request to the next
        rows, session = rh.run_in_process(folder, dtype_name, trace, page_size=page)
        assert all(len(rows[rid]) == len(tokens) for rid, tokens in requests.items())
        worst[name] = rh.worst_error(rows, expected)
        th.assert_rows_close(rows, expected, tolerance, dtype_name, name)
        if name == "mixed":
            assert any(len(owners) > 1 for owners in session.page_owners.values()), "no page was used again"
            assert len(requests) > session.cache.max_requests, "no state slot was used again"
    print(doc["width"], dtype_name, worst)


def test_the_cut_and_the_batch_change_nothing_beyond_rounding(tmp_path):
    """In 32-bit the logits of a position agree to rounding whatever the portions, the pages, the slots and the requests
    beside it."""
    folder = th.make_folder(tmp_path, "m", th.SMALL_A, seed=6, dtype=torch.float32)
    requests = th.random_requests(th.SMALL_A, (40, 97, 130, 5, 61), seed=4)
    whole, _ = rh.run_in_process(folder, "float32", rh.trace_whole(requests), page_size=16)
    for trace, page in ((rh.trace_portions(requests, sizes=(2, 2, 3, 33, 2, 15)), 4), (rh.trace_mixed(requests, seed=2, max_live=3), 32)):
        rows, _ = rh.run_in_process(folder, "float32", trace, page_size=page)
        for rid in requests:
            for pos, row in rows[rid].items():
                assert float(np.abs(row - whole[rid][pos]).max()) <= 1e-4 * float(np.abs(whole[rid][pos]).max()), (rid, pos)


def _with_mark(doc, length, place, seed):
    tokens = [th.FILL if t == th.MARK else t for t in th.random_requests(doc, (length,), seed=seed)["r0"]]
    tokens[place] = th.MARK
    return tokens


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_a_key_at_the_edge_of_a_chunk_decides_the_logits(tmp_path, dtype_name, stored, tolerance):
    """A model whose head looks for one token (``tosivik_helpers.marked_folder``).  Chunks of 40 positions over pages of
    16: the mark is the first position of the last chunk (seen from the end) or the last one of the chunk before (not
    seen), in whole prompts, in decoded tokens and in portions that are cut inside the chunk."""
    folder = th.marked_folder(tmp_path, stored, "attention", chunk=40)
    doc, tensors = th.load_folder(folder)
    for place, seen_from_the_end in ((120, True), (119, False), (133, True)):
        tokens = _with_mark(doc, 135, place, seed=place)
        requests = {"r0": tokens}
        expected = th.oracle(folder, requests)
        without = pt.logits(tokens[:place] + [th.FILL] + tokens[place + 1:], tensors, doc).numpy()
        decides = np.abs(without[-1] - expected["r0"][-1]).max() > 0.2 * np.abs(expected["r0"]).max()
        assert decides == seen_from_the_end, place
        for trace in (rh.trace_whole(requests), rh.trace_tail_by_one(requests, tail=25), rh.trace_portions(requests, sizes=(17, 2, 30))):
            rows, _ = rh.run_in_process(folder, dtype_name, trace, page_size=16)
            th.assert_rows_close(rows, expected, tolerance, dtype_name, place)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_a_state_keeps_a_token_from_hundreds_of_positions_back(tmp_path, dtype_name, stored, tolerance):
    """The mark at position 3 of 420 tokens, in a model whose linear attention decays by 0.999 only: the last logits
    hang on it.  A state that is lost between steps, zeroed with a slot or mixed up in a batch shows."""
    folder = th.marked_folder(tmp_path, stored, "lightning")
    doc, tensors = th.load_folder(folder)
    tokens = _with_mark(doc, 420, 3, seed=1)
    other = _with_mark(doc, 90, 50, seed=2)
    requests = {"r0": tokens, "r1": other, "r2": tokens[:200]}
    expected = th.oracle(folder, requests)
    without = pt.logits(tokens[:3] + [th.FILL] + tokens[4:], tensors, doc).numpy()
    assert np.abs(without[-1] - expected["r0"][-1]).max() > 0.2 * np.abs(expected["r0"]).max(), "the far token decides nothing"
    for trace in (rh.trace_whole(requests), rh.trace_tail_by_one(requests, tail=40), rh.trace_portions(requests, sizes=(17, 2, 30, 64, 3)),
                  rh.trace_mixed(requests, seed=4, max_live=2)):
        rows, _ = rh.run_in_process(folder, dtype_name, trace, page_size=16)
        th.assert_rows_close(rows, expected, tolerance, dtype_name)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_long_decoding_from_the_first_token(tmp_path, dtype_name, stored, tolerance):
    """Two tokens of prompt, then 400 decoded one by one (several key splits, pages and chunks of the mask); beside it a
    request that is fed token by token from position 0.  The decode steps replay captured graphs."""
    folder = th.make_folder(tmp_path, "m", th.SMALL_A, seed=8, dtype=stored)
    requests = th.random_requests(th.SMALL_A, (402, 9), seed=5)
    expected = th.oracle(folder, requests)
    long, short = requests["r0"], requests["r1"]
    trace = [{"entries": [{"id": "r0", "tokens": long[:2], "want": [0, 1]}], "end": []}]
    for p in range(2, len(long)):
        entries = [{"id": "r0", "tokens": [long[p]], "want": [0]}]
        if p - 2 < len(short):
            entries.append({"id": "r1", "tokens": [short[p - 2]], "want": [0]})
        trace.append({"entries": entries, "end": ["r1"] if p - 2 == len(short) - 1 else []})
    trace[-1]["end"] = ["r0"]
    for i, step in enumerate(trace):
        step["step"] = i
    rows, session = rh.run_in_process(folder, dtype_name, trace)
    th.assert_rows_close(rows, expected, tolerance, dtype_name)
    assert len(rows["r0"]) == 402 and len(rows["r1"]) == 9
    assert session.runner.graphs is not None and session.runner.graphs.replays > 300


@pytest.mark.parametrize("dtype_name,stored", [("float32", torch.float32), ("bfloat16", torch.bfloat16)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype_name, stored):
    from sglang_rs_b200 import Engine
    folder = th.make_folder(tmp_path, "m", th.SMALL_A, seed=11, dtype=stored)
    doc, tensors = th.load_folder(folder)
    prompts = list(th.random_requests(th.SMALL_A, (5, 17, 33, 70), seed=8).values())
    engine = Engine(model_path=folder, dtype=dtype_name, page_size=16, max_total_tokens=400, max_running_requests=3,
                    chunked_prefill_size=16)
    results = engine.generate(prompts, {"max_new_tokens": 12})
    for prompt, result in zip(prompts, results):
        assert result["finished"] and len(result["output_ids"]) == 12
        tokens = list(prompt)
        for token in result["output_ids"]:
            logits = pt.logits(tokens, tensors, doc)[-1]
            best = int(torch.argmax(logits))
            limit = 0.0 if dtype_name == "float32" else 4e-2
            assert float(logits[best] - logits[token]) <= limit * float(logits.abs().max()), (prompt[:4], token, best)
            tokens.append(token)
    again = Engine(model_path=folder, dtype=dtype_name, page_size=8, max_total_tokens=400, max_running_requests=1,
                   chunked_prefill_size=7, disable_cuda_graph=True)
    if dtype_name == "float32":
        assert [again.generate(p, {"max_new_tokens": 12})["output_ids"] for p in prompts] == [r["output_ids"] for r in results]
    engine.cache.check_invariants()
    assert engine.flush_cache()
    assert all(a.free_count == a.num_pages for a in engine.cache.allocators.values())
    assert engine.cache.state_pool.free_count == engine.cache.max_requests


def test_preemption_on_a_small_pool_gives_the_same_tokens(tmp_path):
    """Three requests on a pool that cannot hold them: a request is preempted, gives its pages and its state slot back
    and is computed again from its first token, in other portions and another slot; every token stays what the plain
    implementation gives (32-bit)."""
    from sglang_rs_b200 import Engine
    folder = th.make_folder(tmp_path, "m", th.SMALL_A, seed=4, dtype=torch.float32)
    doc, tensors = th.load_folder(folder)
    prompts = list(th.random_requests(th.SMALL_A, (40, 35, 50), seed=2).values())
    engine = Engine(model_path=folder, dtype="float32", page_size=16, max_total_tokens=160, max_running_requests=3,
                    chunked_prefill_size=64)
    results = engine.generate(prompts, {"max_new_tokens": 40})
    assert engine.scheduler.stats["preemptions"] >= 1
    assert [r["output_ids"] for r in results] == [th.plain_greedy(doc, tensors, p, 40) for p in prompts]
    assert engine.cache.state_pool.free_count == engine.cache.max_requests


def test_the_command_line_and_the_trace_program_take_the_design(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(th.SMALL_C))
    folder = str(tmp_path / "written")
    made = subprocess.run([sys.executable, os.path.join(root, "bin", "sglang-rs"), "random-model", "--config", str(config_path),
                           "--out", folder, "--seed", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    doc, tensors = th.load_folder(folder)
    command = [sys.executable, os.path.join(root, "bin", "sglang-rs"), "generate", f"--model-path={folder}", "--device", "cuda",
               "--dtype", "float32", "--input-ids", "5,17,3", "--input-ids", "9 8 7 6", "--max-new-tokens", "5",
               "--max-total-tokens", "256"]
    process = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    lines = [json.loads(line) for line in process.stdout.strip().splitlines()]
    assert [l["output_ids"] for l in lines] == [th.plain_greedy(doc, tensors, p, 5) for p in ([5, 17, 3], [9, 8, 7, 6])]
    tokens = th.random_requests(doc, (37,), seed=1)["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[30:], "want": [6]}], "end": ["a"]}]
    out = tmp_path / "out"
    replay = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                             "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                            capture_output=True, text=True, timeout=600)
    assert replay.returncode == 0 and replay.stdout.split() == ["done", "0", "done", "1"], replay.stderr[-2000:]
    want = pt.logits(tokens, tensors, doc).numpy()
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    last = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    for got, pos in ((first[0], 0), (first[1], 29), (last[0], 36)):
        assert float(np.abs(got - want[pos]).max()) <= 2e-5 * float(np.abs(want).max())
