"""Gikarax: reading config.json, what it refuses, the model spec it produces (the loop as a
schedule with the stream re-mixed in front of every pass, parts, tensor names); the plain
implementation's mechanisms against cases written out by hand, and the engine's frequency tables
against the plain ones."""

import copy
import json
import math

import pytest
import torch

from somi_inference_b200.config import ConfigError, GikaraxConfig, load_config
from somi_inference_b200.parts import declared_tensors
from somi_inference_b200.parts.position import rotary_frequencies
from somi_inference_b200.weights.random_init import random_tensors
from tests.gikarax_tiny import TINY, TINY_A, TINY_B, TINY_C, random_tokens, random_weights, stored_values
from tests.plain import gikarax_plain as plain


def test_round_trip_and_registry(tmp_path):
    for raw in TINY.values():
        cfg = GikaraxConfig.from_dict(raw)
        assert GikaraxConfig.from_dict(cfg.to_dict()) == cfg
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, GikaraxConfig) and cfg.vocab_size == 131 and cfg.loop == (1, 4, 2)
    assert cfg.hidden_size == 48 and cfg.norm_eps == 1e-5


def test_spec_schedule_parts_and_names():
    spec = GikaraxConfig.from_dict(TINY_A).to_model_spec()
    assert [r.layer for r in spec.schedule] == [0, 1, 2, 3, 1, 2, 3, 4]
    assert [r.remix for r in spec.schedule] == [None, "loop_in", None, None, "loop_in", None, None, None]
    assert all(r.cache_of is None and not r.add_embedding for r in spec.schedule)
    assert spec.stream_parts["loop_in"].kind == "embedding_remix"
    assert [l.mixer.kind for l in spec.layers] == ["normed_attention", "side_by_side", "latent_attention",
                                                    "normed_attention", "latent_attention"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        ["routed_moe", "routed_moe", None, "routed_moe", "routed_moe"]
    assert all(l.arrangement == "shared_norm" and set(l.norms) == {"shared"} for l in spec.layers)
    assert all(l.norms["shared"].kind == "layernorm" for l in spec.layers) and spec.final_norm.kind == "layernorm"
    a = spec.layers[0].mixer.params
    assert a["mask"] == {"kind": "window", "size": 9} and a["softcap"] == 3.0 and a["sink"] == "zero"
    assert a["head_gate"] and a["head_norm"] and not a["qkv_bias"]
    assert a["rotary"] == {"dims": 8, "base": 10000.0,
                           "scaling": {"kind": "bands", "factor": 4.0, "low": 1.0, "high": 3.0, "original": 64.0}}
    left, right = (spec.layers[1].mixer.params[k].params for k in ("left", "right"))
    assert left["qkv_bias"] and left["o_bias"] and not left["head_norm"] and left["mask"] is None
    assert left.get("sink") is None and left.get("softcap") is None and not left.get("head_gate")
    assert left["rotary"]["scaling"]["kind"] == "ramp" and left["rotary"]["scaling"]["fast"] == 8.0
    assert right["tau"] == 4.0 and right["decay_rank"] == 5 and right["q_scale"] == 10 ** -0.5
    ff = spec.layers[0].feed_forward.params
    assert ff["weights"] == "softmax_chosen" and ff["activation"] == "gelu" and ff["top"] == 2
    names = declared_tensors(spec)
    assert names["loop.in"].shape == (48, 96)
    assert names["l0.mix.q"].shape == (48, 48) and names["l0.mix.v"].shape == (40, 48)
    assert names["l0.mix.q.norm"].shape == (12,) and names["l0.mix.g"].shape == (4, 48)
    assert names["l0.mix.o"].shape == (48, 80) and "l0.mix.q.b" not in names
    assert names["l1.mix.left.q.b"].shape == (48,) and names["l1.mix.left.o.b"].shape == (48,)
    assert names["l1.mix.left.v"].shape == (40, 48) and "l1.mix.left.q.norm" not in names
    assert names["l1.mix.right.k"].shape == (30, 48) and names["l1.mix.right.g"].shape == (18, 48)
    assert names["l1.mix.right.a1"].shape == (5, 48) and names["l1.mix.right.a2"].shape == (30, 5)
    assert names["l1.mix.right.a2.b"].shape == (30,) and names["l1.mix.right.norm"].shape == (6,)
    assert names["l1.mix.right.out"].shape == (48,) and names["l1.mix.left.out"].shape == (48,)
    assert names["l2.mix.dq"].shape == (20, 48) and names["l2.mix.uq"].shape == (24, 20)
    assert names["l2.mix.dkv.norm"].shape == (16,) and names["l2.mix.uv"].shape == (36, 16)
    assert names["l2.mix.g"].shape == (36, 48) and names["l2.mix.o"].shape == (48, 36)
    assert "l2.mlp.router" not in names and "l0.mlp.e0.gate" not in names and "l0.norm2" not in names
    assert names["l0.mlp.router"].shape == (5, 48) and names["l0.mlp.e4.down"].shape == (48, 24)
    no_loop = GikaraxConfig.from_dict(TINY_B)
    assert no_loop.runs() == [(i, False) for i in range(4)] and not no_loop.to_model_spec().stream_parts
    assert "loop.in" not in declared_tensors(no_loop.to_model_spec())
    thrice = GikaraxConfig.from_dict(TINY_C)
    assert thrice.runs() == [(0, True), (1, False), (2, False)] * 3
    assert plain.layer_runs(TINY_A) == GikaraxConfig.from_dict(TINY_A).runs()
    assert plain.layer_runs(TINY_C) == thrice.runs()


def test_rank_comes_from_the_tensors_shapes():
    raw = copy.deepcopy(TINY_A)
    raw["layers"][1]["mixer"]["right"].pop("decay_rank")
    cfg = GikaraxConfig.from_dict(raw).with_shapes({"l1.mix.right.a1": (7, 48)})
    names = declared_tensors(cfg.to_model_spec())
    assert names["l1.mix.right.a2"].shape == (30, 7) and names["l1.mix.right.a1"].shape == (7, 48)


def test_random_tensors_cover_every_declared_name():
    cfg = GikaraxConfig.from_dict(TINY_C)
    w = random_tensors(cfg, 5)
    assert set(w) == set(declared_tensors(cfg.to_model_spec()))


@pytest.mark.parametrize("change, what", [
    (lambda d: d.pop("width"), "lacks"),
    (lambda d: d["layers"][0].update(type="mamba"), "not a mixer"),
    (lambda d: d["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind 'moe'"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(tau=0), "tau"),
    (lambda d: d["layers"][1]["mixer"].pop("left"), "left"),
    (lambda d: d["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["norm"].update(eps=0.0), "eps"),
])
def test_refusals(change, what):
    raw = copy.deepcopy(TINY_A)
    change(raw)
    with pytest.raises(ConfigError, match=what):
        GikaraxConfig.from_dict(raw)


# --------------------------------------------------------------- plain mechanisms by hand
def test_frequency_tables():
    f, mag = plain.banded_frequencies(8, 10000.0, 4.0, 1.0, 3.0, 64)
    base = [10000.0 ** (-2 * i / 8) for i in range(4)]
    # wavelengths 6.3, 63, 628, 6283 against 64 / 3 = 21.3 and 64 / 1: kept, blended, slowed, slowed
    assert f[0] == base[0] and f[2] == base[2] / 4 and f[3] == base[3] / 4 and mag == 1.0
    s = (64 / (2 * math.pi / base[1]) - 1.0) / 2.0
    assert abs(f[1] - ((1 - s) * base[1] / 4 + s * base[1])) < 1e-15 and 0 < s < 1
    f, mag = plain.ramped_frequencies(8, 300.0, 6.0, 40, 8.0, 1.0)
    base = [300.0 ** (-2 * i / 8) for i in range(4)]
    lo = max(math.floor(8 * math.log(40 / (2 * math.pi * 8.0)) / (2 * math.log(300.0))), 0)
    hi = min(math.ceil(8 * math.log(40 / (2 * math.pi * 1.0)) / (2 * math.log(300.0))), 7)
    assert (lo, hi) == (0, 2) and mag == 0.1 * math.log(6.0) + 1.0
    assert f[0] == base[0] and abs(f[1] - (base[1] / 6 * 0.5 + base[1] * 0.5)) < 1e-15
    assert f[2] == base[2] / 6 and f[3] == base[3] / 6
    # the engine's tables are the plain ones
    for raw in TINY.values():
        spec = GikaraxConfig.from_dict(raw).to_model_spec()
        for layer, lc in zip(spec.layers, raw["layers"]):
            pairs = [(layer.mixer.params, lc["mixer"])] if lc["type"] == "attention" else \
                [(layer.mixer.params["left"].params, lc["mixer"]["left"])] if lc["type"] == "parallel" else []
            for params, m in pairs:
                if m.get("rot") is None:
                    continue
                got, got_mag = rotary_frequencies(params["rotary"])
                want, want_mag = plain.rotation_table(m["rot"])
                assert got.tolist() == pytest.approx(want, rel=1e-15) and got_mag == pytest.approx(want_mag)


def test_rotation_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64).repeat(3, 1, 1)
    y = plain.rotate_halves(x, {"dims": 4, "base": 100.0})
    for p in range(3):
        for i, f in enumerate((1.0, 0.1)):
            c, s = math.cos(p * f), math.sin(p * f)
            assert abs(y[p, 0, i] - (x[p, 0, i] * c - x[p, 0, i + 2] * s)) < 1e-12
            assert abs(y[p, 0, i + 2] - (x[p, 0, i + 2] * c + x[p, 0, i] * s)) < 1e-12
        assert y[p, 0, 4] == 5.0


def test_attention_masks_cap_and_sink_by_hand():
    q = torch.ones((4, 1, 1), dtype=torch.float64)
    k = torch.tensor([2.0, 0.0, 1.0, 3.0], dtype=torch.float64).reshape(4, 1, 1)
    v = torch.tensor([1.0, 10.0, 100.0, 1000.0], dtype=torch.float64).reshape(4, 1, 1)
    o = plain.masked_attention(q, k, v, 1.0, window=2)
    e = math.exp
    assert abs(o[2, 0, 0] - (e(0) * 10 + e(1) * 100) / (e(0) + e(1))) < 1e-12       # key 0 is out
    assert abs(o[0, 0, 0] - 1.0) < 1e-12
    o = plain.masked_attention(q, k, v, 1.0, window=2, sink=True)
    assert abs(o[2, 0, 0] - (e(0) * 10 + e(1) * 100) / (1 + e(0) + e(1))) < 1e-12
    assert abs(o[0, 0, 0] - e(2) / (1 + e(2))) < 1e-12
    o = plain.masked_attention(q, k, v, 2.0, softcap=1.5)
    s = [1.5 * math.tanh(2 * x / 1.5) for x in (2.0, 0.0, 1.0, 3.0)]
    want = sum(e(a) * b for a, b in zip(s, (1.0, 10.0, 100.0, 1000.0))) / sum(e(a) for a in s)
    assert abs(o[3, 0, 0] - want) < 1e-9
    # grouped heads: query heads 0, 1 read key head 0; 2, 3 read key head 1
    g = torch.Generator().manual_seed(0)
    q4, k2, v2 = (torch.randn(s, generator=g, dtype=torch.float64) for s in ((5, 4, 3), (5, 2, 3), (5, 2, 2)))
    o = plain.masked_attention(q4, k2, v2, 0.5)
    alone = plain.masked_attention(q4[:, 2:3], k2[:, 1:2], v2[:, 1:2], 0.5)
    assert torch.allclose(o[:, 2:3], alone)


def test_channel_decayed_sum_by_hand():
    q = torch.ones((3, 1, 2), dtype=torch.float64)
    k = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=torch.float64).reshape(3, 1, 2)
    v = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64).reshape(3, 1, 1)
    alpha = torch.tensor([[0.5, 0.25]] * 3, dtype=torch.float64).reshape(3, 1, 2)
    o = plain.channel_decayed_sum(q, k, v, alpha)
    # channel 0 holds 1, then .5, then .25 + 100; channel 1 holds 0, 10, 2.5 + 100
    assert o.flatten().tolist() == [1.0, 10.5, 202.75]


def test_choice_of_experts_by_hand():
    z = torch.tensor([[1.0, 3.0, 2.0, 3.0], [0.0, -1.0, -2.0, -3.0]], dtype=torch.float64)
    idx, wt = plain.choose_experts(z, 2)
    assert idx.tolist() == [[1, 3], [0, 1]]                       # a tie goes to the lower index
    assert wt[0].tolist() == [0.5, 0.5]
    assert abs(wt[1, 0] - 1 / (1 + math.exp(-1))) < 1e-12 and abs(wt[1].sum() - 1) < 1e-12
    idx, wt = plain.choose_experts(z, 1)
    assert wt.flatten().tolist() == [1.0, 1.0]
    assert plain.choice_margin(z, 2)[1] == 1.0 and plain.choice_margin(z, 4)[0] == float("inf")


def test_the_prefix_property_and_the_loop():
    """Logits of a position do not change when tokens follow it; the re-mix in front of each pass
    matters (a model whose re-mix is the identity on the stream differs from one that is not)."""
    w = stored_values(random_weights(TINY_A, 3))
    toks = random_tokens(30, 131, 4)
    full = plain.forward(TINY_A, w, toks)
    assert torch.allclose(plain.forward(TINY_A, w, toks[:17]), full[:17], atol=1e-10)
    streams = []
    plain.forward(TINY_A, w, toks, streams=streams)
    assert len(streams) == 8
    w2 = dict(w)
    w2["loop.in"] = torch.cat([torch.eye(48, dtype=torch.float64), torch.zeros((48, 48), dtype=torch.float64)], 1)
    assert not torch.allclose(plain.forward(TINY_A, w2, toks), full, atol=1e-3)
