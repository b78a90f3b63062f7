"""Gegepel on the host: the configuration reader, the order of layer calls, the checkpoint names, and the plain
implementation against itself (a sequence and its prefixes; the sink; the choice of experts)."""
import copy

import pytest
import torch

import gegepel_helpers as gh
import plain_gegepel as pg
from sglang_rs_b200.config import ConfigError, RawConfig, resolve_architecture
from sglang_rs_b200.weights import build_model, random_tensors


def test_the_design_is_found_by_its_name_in_the_singular_and_in_the_list():
    import sglang_rs_b200.models  # noqa: F401
    doc = copy.deepcopy(gh.SMALL_A)
    assert resolve_architecture(RawConfig.from_dict(doc)).name == "Gegepel"
    doc["architectures"] = [doc.pop("architecture")]
    assert resolve_architecture(RawConfig.from_dict(doc)).name == "Gegepel"


def test_layer_calls_follow_the_stretch_and_each_call_has_a_cache_of_its_own():
    model, config = build_model(gh.SMALL_A)
    assert [(c.layer, c.entry, c.pass_index) for c in model.program] == [(0, 0, 0), (1, None, 0), (0, 0, 1), (1, None, 1), (2, None, 0)]
    assert [(i, t, first) for i, t, first in pg.program(gh.SMALL_A)] == [(0, 0, True), (1, 0, False), (0, 1, True), (1, 1, False), (2, None, False)]
    needs = model.cache_needs()
    assert len(needs) == 5 and all(need is not None and not need.values and need.num_kv_heads == 1 for need in needs)
    assert [need.head_dim for need in needs] == [56, 48, 56, 48, 56]
    model, _ = build_model(gh.SMALL_C)
    assert [(c.layer, c.entry, c.pass_index) for c in model.program] == [(0, None, 0), (1, 0, 0), (1, 0, 1), (1, 0, 2)]
    model, _ = build_model(gh.SMALL_B)
    assert [c.layer for c in model.program] == [0, 1] and not model.pass_entries


def test_tensor_names_and_shapes():
    model, _ = build_model(gh.SMALL_A)
    specs = {name: spec.shape for name, spec in model.tensor_specs().items()}
    assert specs["embed"] == (96, 64) and specs["head"] == (96, 64) and specs["final.norm.b"] == (64,)
    assert specs["loop.in"] == (64, 128) and specs["loop.step"] == (2, 64)
    assert specs["l0.mix.dq"] == (40, 64) and specs["l0.mix.uq"] == (3 * 24, 40) and specs["l0.mix.dkv"] == (56, 64)
    assert specs["l0.mix.uk"] == (48, 48) and specs["l0.mix.uv"] == (72, 48) and specs["l0.mix.o"] == (64, 72)
    assert specs["l0.mix.sink"] == (3,) and specs["l0.mix.g"] == (3, 64) and specs["l0.mix.dkv.norm"] == (48,)
    assert specs["l1.mlp.router"] == (4, 64) and specs["l1.mlp.e3.down"] == (64, 24) and "l1.mlp.e4.up" not in specs
    assert "l2.norm2" not in specs and "l2.mlp.router" not in specs and specs["l2.norm1b.b"] == (64,)


@pytest.mark.parametrize("change,message", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["layers"][0].update(type="window"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5), "rot"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["loop"].update(stop=7), "loop"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_documents_that_cannot_describe_a_model_are_refused(change, message):
    doc = copy.deepcopy(gh.SMALL_A)
    change(doc)
    with pytest.raises(ConfigError, match=message):
        build_model(doc)


def test_plain_implementation_is_causal_and_counts_the_sink_once():
    model, _ = build_model(gh.SMALL_A)
    tensors = random_tensors(model.tensor_specs(), 3, "cpu", torch.float32)
    tokens = [5, 9, 77, 3, 3, 41, 8, 60, 2]
    whole = pg.forward(gh.SMALL_A, tensors, tokens)
    for n in (1, 4, 8):
        assert torch.allclose(pg.forward(gh.SMALL_A, tensors, tokens[:n]), whole[:n], atol=1e-9)
    scores = torch.tensor([[[0.3, -1.0, 2.0]]], dtype=torch.float64)
    w = pg.softmax_with_sink(scores, torch.tensor([0.5], dtype=torch.float64))
    e = torch.exp(scores[0, 0])
    assert torch.allclose(w[0, 0], e / (e.sum() + torch.exp(torch.tensor(0.5, dtype=torch.float64))))
    # a very low sink is no sink; a very high one takes all the weight
    assert torch.allclose(pg.softmax_with_sink(scores, torch.tensor([-80.0], dtype=torch.float64)).sum(), torch.tensor(1.0, dtype=torch.float64))
    assert float(pg.softmax_with_sink(scores, torch.tensor([80.0], dtype=torch.float64)).sum()) < 1e-30


def test_plain_experts_use_the_scores_of_the_chosen_ones_as_they_are():
    torch.manual_seed(0)
    h = torch.randn(6, 8, dtype=torch.float64)
    tensors = {"p.router": torch.randn(3, 8)}
    for e in range(3):
        tensors.update({f"p.e{e}.gate": torch.randn(4, 8), f"p.e{e}.up": torch.randn(4, 8), f"p.e{e}.down": torch.randn(8, 4)})
    every = pg.routed_experts(h, tensors, "p.", {"router": {"experts": 3, "top": 3}})
    scores = torch.softmax(h @ tensors["p.router"].double().T, -1)
    by_hand = torch.zeros_like(h)
    for e in range(3):
        z = h @ tensors[f"p.e{e}.gate"].double().T
        by_hand += scores[:, e:e + 1] * (((z * torch.sigmoid(z)) * (h @ tensors[f"p.e{e}.up"].double().T)) @ tensors[f"p.e{e}.down"].double().T)
    assert torch.allclose(every, by_hand)
    one = pg.routed_experts(h, tensors, "p.", {"router": {"experts": 3, "top": 1}})
    best = scores.argmax(-1)
    for r in range(6):
        e = int(best[r])
        z = h[r] @ tensors[f"p.e{e}.gate"].double().T
        y = ((z * torch.sigmoid(z)) * (h[r] @ tensors[f"p.e{e}.up"].double().T)) @ tensors[f"p.e{e}.down"].double().T
        assert torch.allclose(one[r], scores[r, e] * y)
