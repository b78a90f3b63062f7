"""Gegepel on the GPU against the plain implementation: each mechanism alone, whole prompts, prompts with a tail
decoded token by token, portions down to two tokens, mixed batches over a small pool (pages are used again), keys at
page borders and far away, long decoding, and greedy generation through the entry point."""
import math

import numpy as np
import pytest
import torch

import gegepel_helpers as gh
import plain_gegepel as pg
import replay_helpers as rh

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 4e-2)]


def seen(tensor, dtype):
    """What the kernel sees of a tensor: rounded to the storage type, as float64."""
    return tensor.to(dtype).to(torch.float64)


def close(got, want, dtype, what, fraction=None):
    tolerance = fraction if fraction is not None else (2e-5 if dtype == torch.float32 else 2e-2)
    scale = float(want.abs().max()) or 1.0
    error = float((got.detach().cpu().to(torch.float64) - want).abs().max()) / scale
    assert error <= tolerance, (what, error)


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,outer", [("layer", "layer"), ("layer", "none"), ("rms", "layer"), ("none", "rms"), (None, "layer")])
def test_norm_sum_norm_in_one_kernel(dtype, inner, outer):
    from sglang_rs_b200 import ops
    torch.manual_seed(1)
    rows, width = 7, 70
    residual = torch.randn(rows, width) * 3 + 1
    delta = torch.randn(rows, width) * 5 - 2
    w1, b1, w2, b2 = (torch.rand(width) + 0.5, torch.randn(width), torch.rand(width) + 0.5, torch.randn(width))
    extra = torch.randn(rows, width)

    def plain(kind, v, w, b):
        if kind == "layer":
            return pg.layer_norm(v, w.double(), b.double(), 1e-5)
        if kind == "rms":
            return pg.rms_norm(v, w.double(), 1e-5)
        return v
    x = residual.double() + (plain(inner, seen(delta, dtype), w1, b1) if inner is not None else 0)
    want = plain(outer, x, w2, b2)
    res = residual.to(DEV)
    out = torch.zeros((rows, 2 * width + 3), dtype=dtype, device=DEV)
    ops.norm_add_norm(res, delta.to(DEV, dtype) if inner is not None else None,
                      None if inner in (None, "none") else (inner, w1.to(DEV), b1.to(DEV), 1e-5),
                      None if outer == "none" else (outer, w2.to(DEV), b2.to(DEV), 1e-5), out, extra=extra.to(DEV))
    close(res, x, torch.float32, "sum")
    close(out[:, :width], want, dtype, "norm of the sum")
    close(out[:, width:2 * width], seen(extra, dtype), dtype, "the rows beside it", 1e-6)
    assert float(out[:, 2 * width:].abs().max()) == 0
    # picked rows, a 32-bit pending term, no output
    res = residual.to(DEV)
    index = torch.tensor([5, 0, 2], dtype=torch.int32, device=DEV)
    picked = torch.empty((3, width), dtype=dtype, device=DEV)
    ops.norm_add_norm(res, delta.to(DEV), ("layer", w1.to(DEV), b1.to(DEV), 1e-5), ("layer", w2.to(DEV), b2.to(DEV), 1e-5),
                      picked, row_index=index, write_residual=False)
    x32 = residual.double() + pg.layer_norm(delta.double(), w1.double(), b1.double(), 1e-5)
    close(picked, pg.layer_norm(x32, w2.double(), b2.double(), 1e-5)[[5, 0, 2]], dtype, "picked rows")
    assert torch.equal(res.cpu(), residual)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latents_rotation_and_cache_rows(dtype):
    from sglang_rs_b200 import ops
    from sglang_rs_b200.parts import RotaryEncoding
    torch.manual_seed(2)
    rows, q_rank, kv_rank, rot_dim, rot_dims, heads, dim = 9, 12, 20, 10, 6, 3, 14
    proj = torch.randn(rows, q_rank + kv_rank + rot_dim + 5) * 2
    qw, kw = torch.rand(q_rank) + 0.5, torch.rand(kv_rank) + 0.5
    positions = torch.tensor([0, 1, 2, 3, 100, 101, 5000, 70000, 7], dtype=torch.int32)
    rotary = RotaryEncoding(rot_dim, 777.0, rotary_dim=rot_dims)
    rotary.load({}, DEV, dtype)
    inv_freq = rotary.fused_rotary().inv_freq
    pool = torch.zeros((4, 1, 8, kv_rank + rot_dim), dtype=dtype, device=DEV)
    slots = torch.tensor([31, 0, 8, 9, 17, 2, 3, 30, 16], dtype=torch.int32, device=DEV)
    q_latent = torch.empty((rows, q_rank), dtype=dtype, device=DEV)
    word = ops.new_error_word(DEV)
    ops.latent_prepare(proj.to(DEV, dtype), q_rank, kv_rank, rot_dim, qw.to(DEV), kw.to(DEV), 1e-5, positions.to(DEV), inv_freq,
                       rot_dims, q_latent, pool, slots, word)
    p = seen(proj, dtype)
    close(q_latent, pg.rms_norm(p[:, :q_rank], qw.double(), 1e-5), dtype, "query latent")
    stored = pool.view(-1, kv_rank + rot_dim)[slots.long()]
    close(stored[:, :kv_rank], pg.rms_norm(p[:, q_rank:q_rank + kv_rank], kw.double(), 1e-5), dtype, "latent")
    rotated = pg.rotate_half_split(p[:, q_rank + kv_rank:q_rank + kv_rank + rot_dim], positions, 777.0, rot_dims)
    close(stored[:, kv_rank:], rotated, dtype, "shared key part", 2e-4 if dtype == torch.float32 else None)
    assert int(word.item()) == 0
    # the same rotation on a slice of every head
    q = torch.randn(rows, heads, dim + rot_dim)
    out = torch.zeros((rows, heads, kv_rank + rot_dim), dtype=dtype, device=DEV)
    ops.rope_slice(q.to(DEV, dtype), dim, out, kv_rank, rot_dim, rot_dims, positions.to(DEV), inv_freq)
    close(out[:, :, kv_rank:], pg.rotate_half_split(seen(q, dtype)[..., dim:], positions, 777.0, rot_dims), dtype, "rotated slice",
          2e-4 if dtype == torch.float32 else None)
    assert float(out[:, :, :kv_rank].abs().max()) == 0
    # a slot outside the pool is flagged, not written
    ops.latent_prepare(proj.to(DEV, dtype), q_rank, kv_rank, rot_dim, qw.to(DEV), kw.to(DEV), 1e-5, positions.to(DEV), inv_freq,
                       rot_dims, q_latent, pool, torch.full((rows,), 32, dtype=torch.int32, device=DEV), word)
    assert int(word.item()) == 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_matrix_per_head_with_a_gate(dtype):
    from sglang_rs_b200 import ops
    torch.manual_seed(3)
    for rows, heads, n_in, n_out, spare in ((70, 3, 21, 67, 4), (300, 2, 40, 72, 8)):        # odd sizes; rows on 16-byte borders
        one_matrix_per_head(dtype, rows, heads, n_in, n_out, spare)


def one_matrix_per_head(dtype, rows, heads, n_in, n_out, spare):
    from sglang_rs_b200 import ops
    x = torch.randn(rows, heads, n_in + spare)
    w = torch.randn(heads, n_out, n_in)
    gate = torch.randn(rows, heads + 2) * 3
    out = torch.zeros((rows, heads, n_out + 3), dtype=dtype, device=DEV)
    ops.head_linear(x.to(DEV, dtype), w.to(DEV, dtype), out, gate=gate.to(DEV, dtype)[:, 1:])
    want = torch.einsum("rhi,hoi->rho", seen(x, dtype)[..., :n_in], seen(w, dtype)) * torch.sigmoid(seen(gate, dtype)[:, 1:1 + heads])[..., None]
    close(out[..., :n_out], want, dtype, "gated per-head product")
    assert float(out[..., n_out:].abs().max()) == 0
    plain = torch.empty((rows, heads, n_out), dtype=dtype, device=DEV)
    ops.head_linear(x.to(DEV, dtype), w.to(DEV, dtype), plain)
    close(plain, torch.einsum("rhi,hoi->rho", seen(x, dtype)[..., :n_in], seen(w, dtype)), dtype, "per-head product")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,split", [(3, 0), (3, 16), (34, 0), (34, 16)])
def test_attention_over_shared_rows_with_a_sink(dtype, heads, split):
    """Rows that serve as key (all of them) and as value (their head), a sink per head, more heads than one block takes;
    one query is made to stand out against a single far key, so that a key that is missed shows."""
    from sglang_rs_b200 import ops
    torch.manual_seed(4)
    width, value_dim, page, length = 24, 16, 8, 75
    keys = torch.randn(length, width)
    q = torch.randn(2, heads, width)
    keys[3] = 4.0 * q[0, 0] / q[0, 0].norm()                   # head 0 of row 0 looks at key 3, far back
    sinks = torch.randn(heads) * 2
    positions = torch.tensor([length - 1, 40], dtype=torch.int32)
    pages = torch.randperm(12)[:math.ceil(length / page)]
    pool = torch.zeros((12, 1, page, width), dtype=dtype, device=DEV)
    for p in range(length):
        pool[pages[p // page], 0, p % page] = keys[p].to(dtype)
    table = pages.to(torch.int32).view(1, -1).to(DEV)
    out = torch.empty((2, heads, value_dim), dtype=dtype, device=DEV)
    splits = max(1, math.ceil(length / split)) if split else 1
    acc = torch.empty(2 * heads * splits * value_dim, device=DEV)
    ml = torch.empty(2 * heads * splits * 2, device=DEV)
    word = ops.new_error_word(DEV)
    ops.paged_attention(q.to(DEV, dtype), pool, None, out, positions.to(DEV), torch.zeros(2, dtype=torch.int32, device=DEV), table,
                        scale=0.3, window=0, split_size=split, max_splits=splits, scratch_acc=acc, scratch_ml=ml,
                        error_word=word, sinks=sinks.to(DEV))
    k = seen(keys, dtype)
    for r, pos in enumerate(positions.tolist()):
        scores = torch.einsum("hd,jd->hj", seen(q, dtype)[r], k[:pos + 1]) * 0.3
        w = pg.softmax_with_sink(scores[:, None, :], sinks.double())[:, 0]
        close(out[r], w @ k[:pos + 1, :value_dim], dtype, f"row {r}")
        if r == 0:
            assert float(w[0, 3]) > 0.5
    assert int(word.item()) == 0
    # values in a pool of their own, narrower than the keys, without a sink
    values = torch.randn(length, value_dim)
    v_pool = torch.zeros((12, 1, page, value_dim), dtype=dtype, device=DEV)
    for p in range(length):
        v_pool[pages[p // page], 0, p % page] = values[p].to(dtype)
    ops.paged_attention(q.to(DEV, dtype), pool, v_pool, out, positions.to(DEV), torch.zeros(2, dtype=torch.int32, device=DEV), table,
                        scale=0.3, window=0, split_size=split, max_splits=splits, scratch_acc=acc, scratch_ml=ml, error_word=word)
    for r, pos in enumerate(positions.tolist()):
        scores = torch.einsum("hd,jd->hj", seen(q, dtype)[r], k[:pos + 1]) * 0.3
        close(out[r], torch.softmax(scores, -1) @ seen(values, dtype)[:pos + 1], dtype, f"row {r}, own values")


@pytest.mark.parametrize("heads,width,value_dim", [(3, 48, 32), (8, 80, 64), (16, 144, 96), (34, 32, 32), (5, 160, 128), (2, 528, 512)])
def test_tensor_core_attention_over_shared_rows(heads, width, value_dim):
    """The bfloat16 kernel for rows that are key and value: prompt portions given as tiles (several requests, a portion
    that starts in the middle of a page and of a 64-key block, rows outside the tiles untouched) and decoded rows whose
    keys are split; one head looks at a single far key."""
    from sglang_rs_b200 import ops
    torch.manual_seed(6)
    dtype, page = torch.bfloat16, 8
    lengths = [150, 70]                                     # two requests; their last 41 and 70 tokens are this step's rows
    portions = [(0, 109, 41), (1, 0, 70)]                   # (request, first position, rows)
    keys = [torch.randn(n, width) for n in lengths]
    rows = sum(n for _, _, n in portions)
    q = torch.randn(rows + 2, heads, width)                 # two rows behind the portions that no tile names
    keys[0][5] = 5.0 * q[40, 0] / q[40, 0].norm()           # the last row of request 0, head 0, looks at key 5
    sinks = torch.randn(heads) * 2
    pages = torch.randperm(40)
    pool = torch.zeros((40, 1, page, width), dtype=dtype, device=DEV)
    table = torch.full((2, 24), -1, dtype=torch.int32)
    used = 0
    for r, k in enumerate(keys):
        for pos in range(len(k)):
            if pos % page == 0:
                table[r, pos // page] = pages[used]
                used += 1
            pool[table[r, pos // page], 0, pos % page] = k[pos].to(dtype)
    tiles, positions, row_request, first = [], [], [], 0
    for request, start, count in portions:
        for offset in range(0, count, 64):
            tiles.append([first + offset, min(64, count - offset), request, start + offset])
        positions += list(range(start, start + count))
        row_request += [request] * count
        first += count
    positions += [0, 0]
    row_request += [0, 0]
    word = ops.new_error_word(DEV)
    out = torch.full((rows + 2, heads, value_dim), 7.0, dtype=dtype, device=DEV)
    ops.latent_attention(q.to(DEV, dtype), pool, out, torch.tensor(positions, dtype=torch.int32, device=DEV),
                         torch.tensor(row_request, dtype=torch.int32, device=DEV), table.to(DEV), scale=0.25, sinks=sinks.to(DEV),
                         error_word=word, tiles=torch.tensor(tiles, dtype=torch.int32, device=DEV))

    def plain(row):
        k = seen(keys[row_request[row]], dtype)[:positions[row] + 1]
        scores = torch.einsum("hd,jd->hj", seen(q, dtype)[row], k) * 0.25
        w = pg.softmax_with_sink(scores[:, None, :], sinks.double())[:, 0]
        return w, w @ k[:, :value_dim]
    for row in range(rows):
        w, want = plain(row)
        close(out[row], want, dtype, f"portion row {row}")
        if row == 40:
            assert float(w[0, 5]) > 0.5
    assert float((out[rows:] - 7.0).abs().max()) == 0 and int(word.item()) == 0
    # the same rows as decoded tokens, keys cut every 64 positions
    picks = [40, 0, rows - 1, 41]
    splits = 3
    acc = torch.empty(len(picks) * heads * splits * value_dim, device=DEV)
    ml = torch.empty(len(picks) * heads * splits * 2, device=DEV)
    single = torch.empty((len(picks), heads, value_dim), dtype=dtype, device=DEV)
    ops.latent_attention(q[picks].to(DEV, dtype), pool, single, torch.tensor([positions[r] for r in picks], dtype=torch.int32, device=DEV),
                         torch.tensor([row_request[r] for r in picks], dtype=torch.int32, device=DEV), table.to(DEV), scale=0.25,
                         sinks=sinks.to(DEV), error_word=word, split_size=64, max_splits=splits, scratch_acc=acc, scratch_ml=ml)
    for i, row in enumerate(picks):
        close(single[i], plain(row)[1], dtype, f"decoded row {row}")
    assert int(word.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,rows", [(5, 2, 150), (3, 3, 9), (4, 1, 1), (70, 4, 40), (3, 2, 500)])
def test_routed_experts(dtype, experts, top, rows):
    from sglang_rs_b200 import ops
    torch.manual_seed(5)
    width, inner = 40, 24
    h = torch.randn(rows, width)
    tensors = {"p.router": torch.randn(experts, width) * 0.6}
    for e in range(experts):
        tensors.update({f"p.e{e}.gate": torch.randn(inner, width) * 0.2, f"p.e{e}.up": torch.randn(inner, width) * 0.2,
                        f"p.e{e}.down": torch.randn(width, inner) * 0.2})
    stacked = {n: torch.stack([tensors[f"p.e{e}.{n}"] for e in range(experts)]).to(DEV, dtype) for n in ("gate", "up", "down")}
    word = ops.new_error_word(DEV)
    out = ops.routed_experts(h.to(DEV, dtype), tensors["p.router"].to(DEV, dtype), torch.cat([stacked["gate"], stacked["up"]], dim=1),
                             stacked["down"], top, "silu", False, word)
    rounded = {k: seen(v, dtype) for k, v in tensors.items()}
    want = pg.routed_experts(seen(h, dtype), rounded, "p.", {"router": {"experts": experts, "top": top}})
    assert out.dtype == torch.float32 and int(word.item()) == 0
    close(out, want, dtype, "weighted sum of the chosen experts")
    chosen, weights = ops.route(h.to(DEV, dtype), tensors["p.router"].to(DEV, dtype), top)
    scores = torch.softmax(seen(h, dtype) @ rounded["p.router"].T, -1)
    best = torch.topk(scores, top, -1)
    assert torch.equal(chosen.cpu().long(), best.indices)
    close(weights, best.values, torch.float32, "weights are the scores themselves", 1e-5)
    _, renormed = ops.route(h.to(DEV, dtype), tensors["p.router"].to(DEV, dtype), top, renormalize=True)
    close(renormed, best.values / best.values.sum(-1, keepdim=True), torch.float32, "weights divided by their sum", 1e-5)


# ------------------------------------------------------------------------------ whole models, every way of cutting
@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
@pytest.mark.parametrize("doc", [gh.SMALL_A, gh.SMALL_B, gh.SMALL_C, gh.SMALL_D, gh.SMALL_E], ids=["a", "b", "c", "d", "e"])
def test_prompts_tails_portions_and_mixed_batches(tmp_path, doc, dtype_name, stored, tolerance):
    folder = gh.make_folder(tmp_path, "m", doc, seed=5, dtype=stored)
    requests = gh.random_requests(doc, (1, 2, 23, 64, 65, 150, 131), seed=3)
    expected = gh.oracle(folder, requests)
    worst = {}
    for name, trace, page in (("whole", rh.trace_whole(requests), 16), ("tail", rh.trace_tail_by_one(requests, tail=20), 16),
                              ("portions", rh.trace_portions(requests), 8), ("mixed", rh.trace_mixed(requests, seed=9), 16)):
        # the pool holds what is live at any time and no more, so pages go from one request to the next
        rows, session = rh.run_in_process(folder, dtype_name, trace, page_size=page)
        assert all(len(rows[rid]) == len(tokens) for rid, tokens in requests.items())
        worst[name] = rh.worst_error(rows, expected)
        gh.assert_rows_close(rows, expected, tolerance, dtype_name, name)
        if name == "mixed":
            assert any(len(owners) > 1 for owners in session.page_owners.values()), "no page was used again"
    print(doc["width"], dtype_name, worst)


def test_the_cut_and_the_batch_change_nothing_beyond_rounding(tmp_path):
    """In 32-bit the logits of a position agree to rounding whatever the portions, the pages and the requests beside it."""
    folder = gh.make_folder(tmp_path, "m", gh.SMALL_A, seed=6, dtype=torch.float32)
    requests = gh.random_requests(gh.SMALL_A, (40, 97, 130), seed=4)
    whole, _ = rh.run_in_process(folder, "float32", rh.trace_whole(requests), page_size=16)
    for trace, page in ((rh.trace_portions(requests, sizes=(2, 2, 3, 33, 2, 15)), 4), (rh.trace_mixed(requests, seed=2, max_live=3), 32)):
        rows, _ = rh.run_in_process(folder, "float32", trace, page_size=page)
        for rid in requests:
            for pos, row in rows[rid].items():
                assert float(np.abs(row - whole[rid][pos]).max()) <= 2e-5 * float(np.abs(whole[rid][pos]).max()), (rid, pos)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_a_far_key_at_a_page_border_decides_the_logits(tmp_path, dtype_name, stored, tolerance):
    """A model made so that head 0 looks at one early position only (``gegepel_helpers.far_key_folder``): the logits of
    late positions hang on a key 240 tokens back, the last one of a page or the first one of the next, in whole prompts,
    in decoded tokens and in portions."""
    folder = gh.far_key_folder(tmp_path, stored)
    doc, tensors = gh.load_folder(folder)
    for target in (15, 16):
        tokens = [58 if t == gh.FAR_KEY_TOKEN else t for t in gh.random_requests(doc, (260,), seed=target)["r0"]]
        tokens[target] = gh.FAR_KEY_TOKEN
        requests = {"r0": tokens}
        expected = gh.oracle(folder, requests)
        without = pg.forward(doc, tensors, tokens[:target] + [58] + tokens[target + 1:]).numpy()
        assert np.abs(without[-1] - expected["r0"][-1]).max() > 0.3 * np.abs(expected["r0"]).max(), "the far key decides nothing"
        for trace in (rh.trace_whole(requests), rh.trace_tail_by_one(requests, tail=40), rh.trace_portions(requests, sizes=(17, 2, 30))):
            rows, _ = rh.run_in_process(folder, dtype_name, trace, page_size=16)
            gh.assert_rows_close(rows, expected, tolerance, dtype_name, target)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_long_decoding_from_the_first_token(tmp_path, dtype_name, stored, tolerance):
    """Two tokens of prompt, then 400 decoded one by one (several key splits and pages); beside it a request that is fed
    token by token from position 0.  The decode steps replay captured graphs."""
    folder = gh.make_folder(tmp_path, "m", gh.SMALL_B, seed=8, dtype=stored)
    requests = gh.random_requests(gh.SMALL_B, (402, 9), seed=5)
    expected = gh.oracle(folder, requests)
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
    gh.assert_rows_close(rows, expected, tolerance, dtype_name)
    assert len(rows["r0"]) == 402 and len(rows["r1"]) == 9
    assert session.runner.graphs is not None and session.runner.graphs.replays > 300


@pytest.mark.parametrize("dtype_name,stored", [("float32", torch.float32), ("bfloat16", torch.bfloat16)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype_name, stored):
    from sglang_rs_b200 import Engine
    folder = gh.make_folder(tmp_path, "m", gh.SMALL_A, seed=11, dtype=stored)
    doc, tensors = gh.load_folder(folder)
    prompts = list(gh.random_requests(gh.SMALL_A, (5, 17, 33, 70), seed=8).values())
    engine = Engine(model_path=folder, dtype=dtype_name, page_size=16, max_total_tokens=400, max_running_requests=3,
                    chunked_prefill_size=16)
    results = engine.generate(prompts, {"max_new_tokens": 12})
    for prompt, result in zip(prompts, results):
        assert result["finished"] and len(result["output_ids"]) == 12
        tokens = list(prompt)
        for token in result["output_ids"]:
            logits = pg.forward(doc, tensors, tokens)[-1]
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


def test_the_command_line_and_the_trace_program_take_the_design(tmp_path):
    """`sglang-rs random-model` writes a folder from a configuration, `sglang-rs generate` decodes from it (greedy, and with
    temperature and top-k from a seed), and `trace_run` replays steps on it: the same programs as for every model."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(gh.SMALL_D))
    folder = str(tmp_path / "written")
    made = subprocess.run([sys.executable, os.path.join(root, "bin", "sglang-rs"), "random-model", "--config", str(config_path),
                           "--out", folder, "--seed", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    doc, tensors = gh.load_folder(folder)
    command = [sys.executable, os.path.join(root, "bin", "sglang-rs"), "generate", f"--model-path={folder}", "--device", "cuda",
               "--dtype", "float32", "--input-ids", "5,17,3", "--input-ids", "9 8 7 6", "--max-new-tokens", "5",
               "--max-total-tokens", "256"]
    process = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    lines = [json.loads(line) for line in process.stdout.strip().splitlines()]
    assert [l["output_ids"] for l in lines] == [gh.plain_greedy(doc, tensors, p, 5) for p in ([5, 17, 3], [9, 8, 7, 6])]
    sampled = [subprocess.run(command + ["--temperature", "0.9", "--top-k", "8", "--sampling-seed", "3"], capture_output=True,
                              text=True, timeout=600) for _ in range(2)]
    assert sampled[0].returncode == 0 and sampled[0].stdout == sampled[1].stdout
    assert all(0 <= t < doc["vocab"] for line in sampled[0].stdout.strip().splitlines() for t in json.loads(line)["output_ids"])
    tokens = gh.random_requests(doc, (37,), seed=1)["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[30:], "want": [6]}], "end": ["a"]}]
    out = tmp_path / "out"
    replay = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                             "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                            capture_output=True, text=True, timeout=600)
    assert replay.returncode == 0 and replay.stdout.split() == ["done", "0", "done", "1"], replay.stderr[-2000:]
    want = pg.forward(doc, tensors, tokens).numpy()
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    last = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    for got, pos in ((first[0], 0), (first[1], 29), (last[0], 36)):
        assert float(np.abs(got - want[pos]).max()) <= 2e-5 * float(np.abs(want).max())
