"""Tosivik on the host: the configuration reader, the order of layer calls, the checkpoint names, the needs for cache
and state, and the plain implementation against itself."""
import copy
import math

import pytest
import torch

import plain_tosivik as pt
import tosivik_helpers as th
from sglang_rs_b200.config import ConfigError, RawConfig, resolve_architecture
from sglang_rs_b200.parts import PagedKV, RequestState
from sglang_rs_b200.weights import build_model, random_tensors


def test_the_design_is_found_by_its_name():
    import sglang_rs_b200.models  # noqa: F401
    assert resolve_architecture(RawConfig.from_dict(copy.deepcopy(th.SMALL_A))).name == "Tosivik"


def test_a_layer_that_uses_another_layers_tensors_is_a_second_call_with_a_cache_of_its_own():
    model, config = build_model(th.SMALL_A)
    assert [c.layer for c in model.program] == [0, 1, 0, 1, 2] and len(model.layers) == 3
    needs = model.cache_needs()
    assert len(needs) == 6                                   # five calls and the embedding's remembered token
    assert needs[0] == needs[2] == RequestState((3, 8, 12), torch.float32)
    assert needs[1] == needs[3] == PagedKV(2, 16, None)
    assert needs[4] == RequestState((2, 16, 8), torch.float32) and needs[5] == RequestState((1,), torch.int32)
    model, _ = build_model(th.SMALL_B)                       # no pair table: the embedding keeps nothing
    assert len(model.cache_needs()) == 3


def test_tensor_names_and_shapes():
    model, _ = build_model(th.SMALL_A)
    specs = {name: spec.shape for name, spec in model.tensor_specs().items()}
    assert specs["embed"] == (90, 48) and specs["bigram"] == (38, 48) and specs["head"] == (90, 48) and specs["final.norm"] == (48,)
    assert specs["l0.mix.q"] == (24, 48) and specs["l0.mix.v"] == (36, 48) and specs["l0.mix.g"] == (36, 48)
    assert specs["l0.mix.norm"] == (36,) and specs["l0.mix.o"] == (48, 36) and specs["l0.mlp.up"] == (40, 48)
    assert specs["l1.mix.q"] == (96, 48) and specs["l1.mix.k"] == (32, 48) and "l1.mix.v" not in specs
    assert specs["l1.mlp.router"] == (5, 48) and specs["l1.mlp.router.b"] == (5,) and specs["l1.mlp.e4.down"] == (48, 24)
    assert specs["l1.mlp.shared.up"] == (16, 48) and "l4.mlp.shared.up" not in specs
    assert specs["l0.hc1.in"] == (3,) and specs["l1.hc2.mix"] == (3, 3)
    assert not any(name.startswith(("l2.", "l3.")) for name in specs)
    model, _ = build_model(th.SMALL_B)
    specs = model.tensor_specs()
    assert "bigram" not in specs and not any(".hc" in name for name in specs) and "l1.norm2" not in specs


@pytest.mark.parametrize("change,message", [
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][0].update(type="window"), "type"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=5), "rot"),
    (lambda d: d["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][2].update(weights_of=3), "weights_of"),
    (lambda d: d["layers"][2].update(mlp={"kind": "dense", "ff": 8}), "differs"),
    (lambda d: d.update(streams=20), "streams"),
    (lambda d: d["embedding"]["bigram"].pop("buckets"), "buckets"),
])
def test_documents_that_cannot_describe_a_model_are_refused(change, message):
    doc = copy.deepcopy(th.SMALL_A)
    change(doc)
    with pytest.raises(ConfigError, match=message):
        build_model(doc)


def test_stretched_wavelengths_of_the_part_equal_the_plain_ones():
    from sglang_rs_b200.parts import RotaryEncoding, WavelengthScaling
    for dims, base, s in ((8, 3000.0, (3.0, 64, 8.0, 1.0)), (6, 10000.0, (2.0, 20, 4.0, 0.5)), (32, 50000.0, (4.0, 128, 16.0, 2.0))):
        rot = {"dims": dims, "base": base, "scaling": dict(zip(("factor", "original", "fast", "slow"), s))}
        plain, magnitude = pt.rotary_frequencies(rot)
        part = RotaryEncoding(dims + 2, base, rotary_dim=dims, scaling=WavelengthScaling(*s))
        assert torch.equal(part.inverse_frequencies(), plain.to(torch.float32))
        assert part.scaling.magnitude == magnitude == 0.1 * math.log(s[0]) + 1.0
        unscaled = RotaryEncoding(dims + 2, base, rotary_dim=dims).inverse_frequencies()
        assert not torch.equal(unscaled, plain.to(torch.float32)), "the scaling changes nothing here"


def _tensors(doc, seed=3):
    model, _ = build_model(doc)
    return random_tensors(model.tensor_specs(), seed, "cpu", torch.float32)


def test_plain_implementation_is_causal():
    for doc in (th.SMALL_A, th.SMALL_B, th.SMALL_C):
        tensors = _tensors(doc)
        tokens = [5, 9, 47, 3, 3, 41, 8, 30, 2, 11, 17, 6, 6]
        whole = pt.logits(tokens, tensors, doc)
        for n in (1, 4, 12):
            assert torch.allclose(pt.logits(tokens[:n], tensors, doc), whole[:n], atol=1e-9)


def test_plain_mask_pairs_and_experts():
    ok = pt.visible(7, 3)
    assert ok[5].tolist() == [False, False, False, True, True, True, False] and ok[3].tolist() == [False] * 3 + [True] + [False] * 3
    assert pt.visible(4, None)[3].tolist() == [True] * 4
    b = {"buckets": 7, "mul_prev": 3, "mul_cur": 5}
    assert pt.bigram_rows([2, 4, 6], b) == [7, (2 * 3 + 4 * 5) % 7, (4 * 3 + 6 * 5) % 7]
    torch.manual_seed(0)
    h = torch.randn(6, 8, dtype=torch.float64)
    tensors = {"p.router": torch.randn(3, 8), "p.router.b": torch.tensor([0.0, 5.0, -5.0])}
    for e in range(3):
        tensors.update({f"p.e{e}.up": torch.randn(4, 8), f"p.e{e}.down": torch.randn(8, 4)})
    z = h @ tensors["p.router"].double().T + tensors["p.router.b"].double()
    one = pt.routed(h, tensors, "p.", {"router": {"experts": 3, "top": 1}})
    for r in range(6):
        e = int(z[r].argmax())
        assert torch.allclose(one[r], pt.two_layer(h[r:r + 1], tensors, f"p.e{e}.", pt.relu_squared)[0])   # the only weight is 1
    two = pt.routed(h, tensors, "p.", {"router": {"experts": 3, "top": 2}})
    for r in range(6):
        a, c = sorted(range(3), key=lambda e: -float(z[r, e]))[:2]
        wa = 1.0 / (1.0 + math.exp(float(z[r, c] - z[r, a])))
        want = wa * pt.two_layer(h[r:r + 1], tensors, f"p.e{a}.", pt.relu_squared)[0] + \
            (1 - wa) * pt.two_layer(h[r:r + 1], tensors, f"p.e{c}.", pt.relu_squared)[0]
        assert torch.allclose(two[r], want)


def test_plain_linear_attention_in_closed_form():
    torch.manual_seed(1)
    n, heads, dim, vdim = 9, 2, 4, 3
    h = torch.randn(n, 6, dtype=torch.float64)
    tensors = {"m.q": torch.randn(heads * dim, 6), "m.k": torch.randn(heads * dim, 6), "m.v": torch.randn(heads * vdim, 6),
               "m.g": torch.randn(heads * vdim, 6), "m.norm": torch.rand(heads * vdim) + 0.5, "m.o": torch.eye(heads * vdim)}
    decay = [0.5, 1.0]
    out = pt.lightning(h, tensors, "m.", {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, 1e-5)
    q = pt.silu(h @ tensors["m.q"].double().T).view(n, heads, dim)
    k = pt.silu(h @ tensors["m.k"].double().T).view(n, heads, dim)
    v = pt.silu(h @ tensors["m.v"].double().T).view(n, heads, vdim)
    o = torch.zeros(n, heads, vdim, dtype=torch.float64)
    for t in range(n):
        for j in range(t + 1):
            for a in range(heads):
                o[t, a] += decay[a] ** (t - j) * float(q[t, a] @ k[j, a]) * v[j, a]
    want = pt.rms_norm(o.reshape(n, -1), tensors["m.norm"].double(), 1e-5) * torch.sigmoid(h @ tensors["m.g"].double().T)
    assert torch.allclose(out, want)
