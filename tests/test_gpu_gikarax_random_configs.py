"""Gikarax models of random sizes, layer orders, windows, constants and loops through the engine
under two ways of cutting the work, against the plain implementation: float32 row by row;
bfloat16 by the root mean square over all rows (a single row may rest on a close call of a
router, or on the sign of one head's q.k at a sequence's first positions, which the gated linear
attention's norm turns into the sign of that head's whole output)."""

import json
import os
import random

import pytest
import torch

from somi_inference_b200.weights.safetensors_io import save_safetensors
from tests import replay
from tests.gikarax_tiny import (causal, gated_linear, latent, layer, moe, pair, random_tokens,
                                random_weights, stored_values, windowed)
from tests.plain import gikarax_plain as plain

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random) -> dict:
    width = rng.choice([64, 96, 160, 192, 256, 104])

    def grouped():
        heads = rng.choice([2, 4, 6, 8, 3])
        kv = rng.choice([g for g in (1, 2, 3, 4, heads) if heads % g == 0])
        d = rng.choice([16, 32, 48, 64, 96, 128, 24])
        dv = rng.choice([d, d, 16, 32, 64, 128])
        rot = None
        if rng.random() < 0.8:
            dims = rng.choice([d, d // 2, 8])
            rot = (dims - dims % 2, rng.choice([1e4, 5e5, 100.0]))
        return heads, kv, d, dv, rot

    def mixer(kind):
        if kind == "attention":
            heads, kv, d, dv, rot = grouped()
            bands = ((rng.choice([2.0, 6.0]), 1.0, rng.choice([2.0, 3.0]), rng.choice([32, 1024]))
                     if rot and rng.random() < 0.7 else None)
            return windowed(heads, kv, d, dv, d ** -0.5, rng.choice([None, 1, 7, 33, 100, 64]),
                            rng.choice([None, 10.0, 35.0]), rot, bands)
        if kind == "latent_attention":
            return latent(rng.choice([1, 3, 5, 8]), rng.choice([16, 32, 40]), rng.choice([16, 32, 24]),
                          rng.choice([24, 80, 160]), rng.choice([16, 40, 64, 136, 200, 36]), rng.choice([0.2, 0.15]))
        heads, kv, d, dv, rot = grouped()
        ramp = ((rng.choice([4.0, 6.0]), rng.choice([64, 1024]), 24.0, 2.0) if rot and rng.random() < 0.7 else None)
        return pair(causal(heads, kv, d, dv, d ** -0.5, rot, ramp),
                    gated_linear(rng.choice([1, 2, 5]), rng.choice([8, 40, 64, 128, 20]),
                                 rng.choice([8, 64, 96, 20]), rng.choice([1.0, 4.0, 12.0, 20.5]),
                                 rank=rng.choice([4, 12, 24])))

    n = rng.choice([3, 4, 5])
    layers = []
    for _ in range(n):
        kind = rng.choice(["attention", "latent_attention", "parallel"])
        experts = rng.choice([2, 4, 7, 12, 5])
        mlp = None if rng.random() < 0.15 else moe(experts, rng.randint(1, experts), rng.choice([16, 64, 96, 128, 20]))
        layers.append(layer(kind, mixer(kind), mlp))
    cfg = dict(architecture="Gikarax", vocab=rng.choice([100, 513, 333]), width=width,
               norm={"eps": rng.choice([1e-6, 1e-5])}, layers=layers)
    if rng.random() < 0.8:
        start = rng.randint(0, n - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, n), "times": rng.choice([1, 2, 3])}
    return cfg


@pytest.mark.parametrize("seed", range(8))
def test_random_models_in_portions_and_mixed_batches(tmp_path, seed):
    from somi_inference_b200.engine import Engine
    raw = random_config(random.Random(100 + seed))
    reqs = {f"r{i}": random_tokens(n, raw["vocab"], 50 + i) for i, n in enumerate([120, 37, 70, 1, 64, 5])}
    for dt, dtype in ((torch.float32, "float32"), (torch.bfloat16, "bfloat16")):
        d = str(tmp_path / dtype)
        os.makedirs(d)
        w = random_weights(raw, seed, dt)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(raw, f)
        save_safetensors(w, os.path.join(d, "model.safetensors"))
        ref = {rid: plain.forward(raw, stored_values(w), toks) for rid, toks in reqs.items()}
        scale = max(v.abs().max().item() for v in ref.values())
        for cut in (replay.portions, replay.mixed):
            steps, max_tokens = cut(reqs)
            eng = Engine(d, dtype=dtype, page_size=16, max_tokens=max_tokens, max_requests=4)
            got = replay.run_steps(eng, steps)
            eng.ops.check_errors()
            assert len(got) >= 100
            diffs = {k: (row.double() - ref[k[0]][k[1]]) for k, row in got.items()}
            if dtype == "float32":
                worst = max((v.abs().max().item(), k) for k, v in diffs.items())
                assert worst[0] < 2e-4 * scale, (json.dumps(raw), worst)
            else:
                rms = (sum((v ** 2).mean().item() for v in diffs.values()) / len(diffs)) ** 0.5
                assert rms < 3e-2 * scale, (json.dumps(raw), rms)
            assert all(f == eng.num_pages for f in eng.cache.free_pages()), "pages were lost"
