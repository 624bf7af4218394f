"""Poselorn: reading config.json, what it refuses, the model spec it produces (the loop as a
schedule, parts, tensor names, cache and state needs); the plain implementation's mechanisms
against cases written out by hand."""

import copy
import json
import math

import pytest
import torch

from somi_inference_b200.config import ConfigError, PoselornConfig, load_config
from somi_inference_b200.parts import declared_tensors
from somi_inference_b200.weights.random_init import random_tensors
from tests.poselorn_tiny import TINY, TINY_A, TINY_B, TINY_C, random_tokens, random_weights, stored_values
from tests.plain import poselorn_plain as plain


def test_round_trip_and_registry(tmp_path):
    for raw in TINY.values():
        cfg = PoselornConfig.from_dict(raw)
        assert PoselornConfig.from_dict(cfg.to_dict()) == cfg
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, PoselornConfig) and cfg.vocab_size == 131 and cfg.loop == (1, 3, 2)
    assert cfg.hidden_size == 48 and cfg.residual_mult == 0.6


def test_spec_schedule_parts_and_names():
    cfg = PoselornConfig.from_dict(TINY_A)
    spec = cfg.to_model_spec()
    assert [r.layer for r in spec.schedule] == [0, 1, 2, 1, 2, 3]
    assert [r.add_embedding for r in spec.schedule] == [False, False, False, True, False, False]
    assert all(r.cache_of is None for r in spec.schedule)         # every run has a cache of its own
    assert [l.mixer.kind for l in spec.layers] == ["delta_rule", "side_by_side", "delta_rule", "side_by_side"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        ["dense_ff", "routed_moe", None, "routed_moe"]
    assert all(l.arrangement == "parallel_branches" for l in spec.layers)
    assert set(spec.layers[2].norms) == {"mixer"} and set(spec.layers[0].norms) == {"mixer", "feed_forward"}
    left = spec.layers[1].mixer.params["left"].params
    assert left["mask"] == {"kind": "window", "size": 9} and left["rotary"] == {"dims": 8, "base": 10000.0}
    assert spec.layers[1].mixer.params["right"].params["decay"] == [0.5, 0.9, 0.99]
    assert spec.layers[1].feed_forward.params["groups"] == {"count": 3, "keep": 2}
    assert spec.layers[3].feed_forward.params["groups"] is None
    assert spec.embedding.params["scale"] == 3.0
    assert spec.layers[0].extras["branch_factor"].params["value"] == 0.6
    names = declared_tensors(spec)
    assert names["l0.mix.q"].shape == (24, 48) and names["l0.mix.v"].shape == (80, 48)
    assert names["l0.mix.k.conv"].shape == (24, 3) and names["l0.mix.a2"].shape == (48, 6)
    assert names["l0.mix.g1"].shape == (5, 48) and names["l0.mix.g2"].shape == (80, 5)
    assert names["l0.mix.b"].shape == (4, 48) and names["l0.mix.norm"].shape == (20,)
    assert names["l1.mix.left.q"].shape == (48, 48) and names["l1.mix.left.v.b"].shape == (40,)
    assert names["l1.mix.left.k.norm"].shape == (12,) and names["l1.mix.left.o"].shape == (48, 80)
    assert names["l1.mix.right.k"].shape == (30, 48) and names["l1.mix.right.g"].shape == (18, 48)
    assert names["l1.mix.right.norm"].shape == (18,) and names["l1.mix.right.out"].shape == (48,)
    assert names["l1.mlp.router"].shape == (6, 48) and names["l1.mlp.correction"].shape == (6,)
    assert names["l1.mlp.e4.down"].shape == (48, 24) and "l1.mlp.e5.up" not in names
    assert "l2.norm2" not in names and "l2.ls2" not in names and "l2.mlp.up" not in names
    assert names["l0.mlp.up.b"].shape == (72,) and names["head"].shape == (131, 48)
    no_loop = PoselornConfig.from_dict(TINY_B)
    assert [i for i, _ in no_loop.runs()] == [0, 1, 2, 3] and not any(a for _, a in no_loop.runs())
    thrice = PoselornConfig.from_dict(TINY_C)
    assert thrice.runs() == [(0, False), (1, False), (0, True), (1, False), (0, True), (1, False), (2, False)]


def test_ranks_come_from_the_tensors_shapes():
    raw = copy.deepcopy(TINY_A)
    for key in ("decay_rank", "gate_rank"):
        raw["layers"][0]["mixer"].pop(key)
    cfg = PoselornConfig.from_dict(raw).with_shapes({"l0.mix.a1": (7, 48), "l0.mix.g1": (3, 48)})
    names = declared_tensors(cfg.to_model_spec())
    assert names["l0.mix.a2"].shape == (48, 7) and names["l0.mix.g2"].shape == (80, 3)
    assert names["l2.mix.a1"].shape == (6, 48)               # stated in the file: kept


def test_random_tensors_cover_every_declared_name():
    cfg = PoselornConfig.from_dict(TINY_C)
    w = random_tensors(cfg, 5)
    assert set(w) == set(declared_tensors(cfg.to_model_spec()))
    assert w["l0.mlp.correction"].shape == (8,) and w["l0.mix.q.conv"].shape == (32, 5)


@pytest.mark.parametrize("change, message", [
    (lambda d: d.pop("vocab"), "lacks"),
    (lambda d: d["norm"].pop("eps"), "norm.eps"),
    (lambda d: d["embedding"].pop("scale"), "embedding.scale"),
    (lambda d: d.update(residual_mult="much"), "residual_mult"),
    (lambda d: d["layers"][0].update(type="mystery"), "not a mixer"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "dense"),
    (lambda d: d["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=14), "at most dim"),
    (lambda d: d["layers"][1]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(decay=[0.5, 0.9]), "one number per head"),
    (lambda d: d["layers"][1]["mixer"].pop("right"), "right"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=3) or
               d["layers"][1]["mlp"]["router"].update(top=3), "kept groups"),
    (lambda d: d["loop"].update(stop=9), "loop"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(TINY_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        PoselornConfig.from_dict(raw)


# ------------------------------------------------------------------ the plain mechanisms by hand
def test_plain_short_conv_and_unit_vector():
    u = torch.tensor([[1.0, 2.0], [3.0, -1.0], [0.5, 4.0]], dtype=torch.float64)
    taps = torch.tensor([[10.0, 100.0, 1.0], [0.0, -1.0, 2.0]], dtype=torch.float64)
    y = plain.short_conv(u, taps)
    assert torch.equal(y, torch.tensor([[1.0, 4.0], [103.0, -4.0], [310.5, 9.0]], dtype=torch.float64))
    assert torch.equal(plain.short_conv(u, taps[:, 2:]), u * taps[:, 2])
    x = torch.tensor([3.0, 4.0], dtype=torch.float64)
    assert torch.allclose(plain.unit_vector(x, 0.0), x / 5.0)
    assert torch.allclose(plain.unit_vector(x, 11.0), x / 6.0)


def test_plain_delta_rule_by_hand():
    """Two tokens of one head with two key channels and one value channel, written out."""
    q = torch.tensor([[[1.0, 0.0]], [[1.0, 1.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.0, 0.0]], [[0.5, 1.0]]], dtype=torch.float64)
    v = torch.tensor([[[2.0]], [[3.0]]], dtype=torch.float64)
    beta = torch.tensor([[0.5], [1.0]], dtype=torch.float64)
    g = torch.tensor([[[0.9, 0.8]], [[0.5, 0.25]]], dtype=torch.float64)
    o = plain.gated_delta_rule(q, k, v, beta, g)
    # token 0: M = 0; u = 0.5 * 2 = 1; M = [[1], [0]]; o = 1
    # token 1: M = [[0.5], [0]]; M^T k = 0.25; u = 3 - 0.25 = 2.75; M = [[0.5 + 1.375], [2.75]]; o = 4.625
    assert torch.allclose(o[:, 0, 0], torch.tensor([1.0, 4.625], dtype=torch.float64))
    # beta = 1, no decay, the same unit key twice: the second write replaces the first value
    k1 = torch.tensor([[[0.6, 0.8]], [[0.6, 0.8]]], dtype=torch.float64)
    one = torch.ones_like(g)
    o2 = plain.gated_delta_rule(k1, k1, v, torch.ones_like(beta), one)
    assert torch.allclose(o2[:, 0, 0], torch.tensor([2.0, 3.0], dtype=torch.float64))


def test_plain_decayed_sum_is_a_weighted_causal_sum():
    g = torch.Generator().manual_seed(2)
    q, k = torch.randn(9, 2, 3, generator=g).double(), torch.randn(9, 2, 3, generator=g).double()
    v = torch.randn(9, 2, 4, generator=g).double()
    decay = torch.tensor([0.5, 1.0], dtype=torch.float64)
    o = plain.decayed_outer_sum(q, k, v, decay)
    for t in (0, 4, 8):
        for h in range(2):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(o[t, h], want, atol=1e-12)


def test_plain_rotation_and_window():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0
    x[:, 0, 5] = 7.0
    y = plain.rotate_halves(x, 4, 100.0)
    # entry 0 pairs with entry 2 at frequency 1; entry 1 with entry 3 at 100^(-1/2); 4 and 5 pass
    assert torch.allclose(y[2, 0], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0, 0.0, 7.0],
                                                dtype=torch.float64))
    x[:, 0, :] = 0.0
    x[:, 0, 1] = 1.0
    y = plain.rotate_halves(x, 4, 100.0)
    assert torch.allclose(y[2, 0, [1, 3]], torch.tensor([math.cos(0.2), math.sin(0.2)], dtype=torch.float64))
    assert torch.equal(plain.rotate_halves(x, 0, 100.0), x)
    g = torch.Generator().manual_seed(3)
    q, k = torch.randn(11, 4, 6, generator=g).double(), torch.randn(11, 2, 6, generator=g).double()
    v = torch.randn(11, 2, 5, generator=g).double()
    vv = v.repeat_interleave(2, dim=1)
    a = plain.window_softmax_attention(q, k, v, 0.4, None)
    assert torch.equal(a, plain.window_softmax_attention(q, k, v, 0.4, 50))
    assert torch.allclose(plain.window_softmax_attention(q, k, v, 0.4, 1), vv, atol=1e-12)
    three = plain.window_softmax_attention(q, k, v, 0.4, 3)
    assert torch.allclose(three[:3], a[:3], atol=1e-12) and not torch.allclose(three[3], a[3])
    # a huge key three back is seen by a window of 4 and not by a window of 3
    k2 = k.clone()
    k2[4] = 50.0 * torch.sign(q[7, 0])[None, :]
    four = plain.window_softmax_attention(q, k2, v, 0.4, 4)
    assert torch.allclose(four[7, 0], vv[4, 0], atol=1e-6)
    assert (plain.window_softmax_attention(q, k2, v, 0.4, 3)[7, 0] - vv[4, 0]).abs().max() > 1e-2


def test_plain_choice_of_experts():
    z = torch.log(torch.tensor([[0.05, 0.30, 0.10, 0.20, 0.25, 0.10]], dtype=torch.float64))
    none = torch.zeros(6, dtype=torch.float64)
    chosen, weight = plain.choose_experts(z, none, None, 2)
    assert chosen.tolist() == [[1, 4]] and torch.allclose(weight, torch.tensor([[0.30, 0.25]], dtype=torch.float64))
    # the correction decides and does not weigh
    corr = torch.tensor([0.5, 0.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64)
    chosen, weight = plain.choose_experts(z, corr, None, 2)
    assert chosen.tolist() == [[0, 1]] and torch.allclose(weight, torch.tensor([[0.05, 0.30]], dtype=torch.float64))
    # three groups of two, one kept: the group of output 1 wins and both choices come from it
    chosen, _ = plain.choose_experts(z, none, (3, 1), 2)
    assert chosen.tolist() == [[1, 0]]
    # negative choice scores still beat an output outside the kept groups
    low = torch.tensor([-2.0, -0.1, -3.0, -3.0, -3.0, -3.0], dtype=torch.float64)
    chosen, _ = plain.choose_experts(z, low, (3, 1), 2)
    assert chosen.tolist() == [[1, 0]]
    chosen, _ = plain.choose_experts(z, none, (3, 2), 3)
    assert sorted(chosen.tolist()[0]) == [1, 4, 5]            # groups {0,1} and {4,5} are kept: 0.30, 0.25, then 0.10 of 5 over 0.05 of 0


def test_plain_identity_expert_and_weights_not_renormalised():
    raw = {"router": {"experts": 1, "identity": 1, "top": 2}, "expert": {"ff": 2}, "kind": "moe"}
    h = torch.tensor([[1.0, -2.0, 0.5]], dtype=torch.float64)
    w = {"m.mlp.router": torch.zeros(2, 3, dtype=torch.float64),
         "m.mlp.correction": torch.zeros(2, dtype=torch.float64),
         "m.mlp.e0.gate": torch.zeros(2, 3, dtype=torch.float64),
         "m.mlp.e0.up": torch.ones(2, 3, dtype=torch.float64),
         "m.mlp.e0.down": torch.ones(3, 2, dtype=torch.float64)}
    # silu(0) = 0: the real expert gives nothing; the identity expert hands on h times s = 1/2
    assert torch.allclose(plain.moe_ff(h, w, "m", raw), 0.5 * h)


def test_plain_prefix_property_and_loop():
    """Causality of the whole plain model, and the loop: with `times` = 1 nothing is added in
    front of a pass, with 2 the embedding's output enters again."""
    w = stored_values(random_weights(TINY_A, 4))
    toks = random_tokens(30, 131, 1)
    full = plain.forward(TINY_A, w, toks)
    assert torch.allclose(plain.forward(TINY_A, w, toks[:17]), full[:17], atol=1e-9)
    once = copy.deepcopy(TINY_A)
    once["loop"]["times"] = 1
    flat = copy.deepcopy(TINY_A)
    flat.pop("loop")
    assert torch.equal(plain.forward(once, w, toks), plain.forward(flat, w, toks))
    res = []
    plain.forward(TINY_A, w, toks, residuals=res)
    assert len(res) == 6
