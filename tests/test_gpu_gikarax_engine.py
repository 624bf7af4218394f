"""Gikarax through the engine, against the plain implementation, under every way of cutting the
work: whole prompts; most of a prompt and then token by token; portions of changing size down to
two tokens; up to four live requests in one batch with so few pages and slots that both are
used again; long decoding past every window; greedy generation through `LLM` and the command
line.  float32 and bfloat16, four small configurations (tests/gikarax_tiny.py)."""

import json
import os

import pytest
import torch

from somi_inference_b200.config import GikaraxConfig
from somi_inference_b200.weights.safetensors_io import save_safetensors
from tests import replay
from tests.gikarax_tiny import PAGE_SIZES, TINY, random_tokens, random_weights, stored_values
from tests.plain import gikarax_plain as plain

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 97, 40, 70, 1, 33, 100, 64, 81, 2], "B": [3, 50, 17, 64, 1, 30],
           "C": [150, 5, 129, 71, 200, 16, 90], "D": [300, 70, 1, 180, 33, 257]}
# float32: logits are of size 3-8 here; bfloat16: every activation between two kernels is rounded
# to 8 bits.  A wrong key, a window that is off by one or a lost state moves a logit by its own size.
ATOL = {"float32": lambda s: 4e-5 * max(1.0, s), "bfloat16": lambda s: 8e-2 * s}
RMS = {"float32": lambda s: 1e-5 * max(1.0, s), "bfloat16": lambda s: 1.2e-2 * s}
# bfloat16 only: a token whose choice of experts hangs on less than this (in router logits, with a
# weight of more than 0.02 at stake) may be routed otherwise after rounding, which is no fault;
# such rows are left out of the comparison.  float32 compares every row.
CLOSE_CALL = 0.3
MODES = {"whole": replay.whole, "last32": replay.last_one_by_one, "portions": replay.portions,
         "mixed": replay.mixed}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("gikarax")
    out = {}
    for k, (name, raw) in enumerate(TINY.items()):
        for dt in (torch.float32, torch.bfloat16):
            d = str(root / f"{name}_{str(dt).split('.')[-1]}")
            os.makedirs(d)
            w = random_weights(raw, 20 + k, dt)
            with open(os.path.join(d, "config.json"), "w") as f:
                json.dump(raw, f)
            save_safetensors(w, os.path.join(d, "model.safetensors"))
            reqs = {f"r{i}": random_tokens(n, raw["vocab"], 50 + i) for i, n in enumerate(LENGTHS[name])}
            ref = plain_logits(raw, w, reqs, dt)
            scale = max(v.abs().max().item() for v in ref.values())
            out[(name, str(dt).split(".")[-1])] = (d, raw, w, reqs, ref, scale)
    return out


class Logits(dict):
    """request -> plain logits [S, vocab], with the rows that rest on a close call."""
    close: set


def plain_logits(raw, w, reqs, dt) -> Logits:
    ref = Logits()
    ref.close = set()
    for rid, toks in reqs.items():
        margins = []
        ref[rid] = plain.forward(raw, stored_values(w), toks, margins=margins)
        if dt == torch.bfloat16 and margins:
            low = torch.stack(margins).min(dim=0).values < CLOSE_CALL
            ref.close |= {(rid, int(p)) for p in low.nonzero().flatten()}
    assert len(ref.close) * 5 < sum(len(t) for t in reqs.values()) + 10
    return ref


def settled(got: dict, ref: Logits) -> dict:
    return {key: row for key, row in got.items() if key not in ref.close}


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_in_process(models, name, dtype, mode):
    from somi_inference_b200.engine import Engine
    d, raw, w, reqs, ref, scale = models[(name, dtype)]
    steps, max_tokens = MODES[mode](reqs)
    eng = Engine(d, dtype=dtype, page_size=PAGE_SIZES[name], max_tokens=max_tokens, max_requests=4)
    got = replay.run_steps(eng, steps)
    eng.ops.check_errors()
    assert len(got) >= len(reqs)
    replay.compare(settled(got, ref), ref, ATOL[dtype](scale), f"{name}/{dtype}/{mode}", RMS[dtype](scale))
    assert all(f == eng.num_pages for f in eng.cache.free_pages()), "pages were lost"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(models, tmp_path, dtype):
    d, raw, w, reqs, ref, scale = models[("A", dtype)]
    for mode in ("mixed", "last32"):
        steps, max_tokens = MODES[mode](reqs)
        got = replay.run_trace_program(d, dtype, steps, max_tokens, str(tmp_path / mode), raw["vocab"])
        replay.compare(settled(got, ref), ref, ATOL[dtype](scale), f"trace_run A/{dtype}/{mode}", RMS[dtype](scale))


@pytest.mark.parametrize("name", ["A", "C"])
def test_cut_independence_float32(models, name):
    """The same position whole, token by token and in portions: equal beyond rounding, and the
    first tokens of a sequence (before any window or state is full) among them."""
    from somi_inference_b200.engine import Engine
    d, raw, w, reqs, ref, scale = models[(name, "float32")]
    sub = {"r0": reqs["r0"], "r1": reqs["r1"]}
    outs = []
    for mode in ("whole", "last32", "portions"):
        steps, mt = MODES[mode](sub)
        eng = Engine(d, dtype="float32", page_size=PAGE_SIZES[name], max_tokens=mt, max_requests=4)
        outs.append(replay.run_steps(eng, steps))
    for key in outs[0]:
        for o in outs[1:]:
            assert (outs[0][key] - o[key]).abs().max().item() < 2e-5 * max(1.0, scale)


def test_token_by_token_from_the_first_token(models):
    """Every token in a step of its own from position 0 on, two requests side by side, with graph
    replay: the matrix states, the latents and the windows start from nothing."""
    from somi_inference_b200.engine import Engine, StepEntry
    d, raw, w, reqs, ref, scale = models[("A", "float32")]
    eng = Engine(d, dtype="float32", page_size=8, max_tokens=256, max_requests=2)
    toks = {"r1": reqs["r1"][:60], "r3": reqs["r3"][:45]}
    got = {}
    for i in range(60):
        entries = [StepEntry(k, [v[i]], [0]) for k, v in toks.items() if i < len(v)]
        for e, row in zip(entries, eng.step(entries).float().cpu()):
            got[(e.request, i)] = row
    eng.ops.check_errors()
    assert eng._graphs.hits > 0
    replay.compare(got, ref, ATOL["float32"](scale), "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_in_a_small_pool(models, dtype):
    """Token by token from the first token on, far past every window, two requests side by side
    in a pool that holds a fraction of their length: caches give the pages behind their windows
    back as they go and take them again; the state slots carry the recurrences all the way."""
    from somi_inference_b200.engine import Engine, StepEntry
    d, raw, w, _, _, _ = models[("C", dtype)]
    toks = {"x": random_tokens(260, raw["vocab"], 1), "y": random_tokens(190, raw["vocab"], 2)}
    want = plain_logits(raw, w, toks, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    s2 = max(v.abs().max().item() for v in want.values())
    # the windowed caches give pages back; the latents and the causal half keep every position
    eng = Engine(d, dtype=dtype, page_size=16, num_pages=34, max_requests=2)
    got = {}
    for i in range(260):
        entries = [StepEntry(k, [v[i]], [0]) for k, v in toks.items() if i < len(v)]
        logits = eng.step(entries).float().cpu()
        for e, row in zip(entries, logits):
            got[(e.request, i)] = row
        for k, v in toks.items():
            if i == len(v) - 1:
                eng.end(k)
        eng.cache.check_consistency()
    eng.ops.check_errors()
    replay.compare(settled(got, want), want, ATOL[dtype](s2), f"long decoding/{dtype}", RMS[dtype](s2))
    assert all(f == 34 for f in eng.cache.free_pages())


def test_slots_that_are_used_again_start_from_nothing(models):
    """A request that takes over the slot and pages of a finished one gives the logits it gives
    alone: the recurrent state of the slot was cleared."""
    from somi_inference_b200.engine import Engine, StepEntry
    d, raw, w, reqs, ref, scale = models[("A", "float32")]
    eng = Engine(d, dtype="float32", page_size=8, max_tokens=128, max_requests=1)
    for rid in ("r1", "r3", "r2"):
        toks = reqs[rid]
        lg = eng.step([StepEntry(rid, toks, range(len(toks)))]).float().cpu()
        eng.end(rid)
        assert (lg - ref[rid].float()).abs().max().item() < ATOL["float32"](scale), rid


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_llm(models, name):
    """Greedy continuations through the scheduler (prompts in portions, several requests at once)
    equal the plain model's, which recomputes the whole sequence for every token."""
    from somi_inference_b200.engine import LLM
    from somi_inference_b200.sampling import SamplingParams
    d, raw, w, reqs, ref, scale = models[(name, "float32")]
    prompts = [random_tokens(n, raw["vocab"], 90 + n) for n in (3, 41, 18, 1, 66)]
    llm = LLM(d, num_blocks=64, block_size=PAGE_SIZES[name], dtype="float32", max_concurrent=3,
              chunk_size=16, max_num_batched_tokens=40)
    outs = llm.generate_many(prompts, max_new_tokens=12,
                             sampling_params=[SamplingParams(temperature=0.0)] * len(prompts),
                             ignore_eos=True)
    for p, o in zip(prompts, outs):
        assert list(o) == plain.greedy(raw, stored_values(w), p, 12), len(p)


def test_command_line_from_config_and_seed(tmp_path, capsys):
    from somi_inference_b200.entrypoints.generate import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY["A"]))
    rc = main(["--config", str(cfg), "--random-weights", "--seed", "3", "--prompt-lens", "4", "19",
               "--max-new-tokens", "5", "--temperature", "0", "--dtype", "float32", "--std", "0.2"])
    assert rc == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
    assert [r["prompt_len"] for r in lines] == [4, 19] and all(len(r["output_ids"]) == 5 for r in lines)
    # the same weights written to a folder and read back give the same tokens
    folder = tmp_path / "model"
    assert main(["--write-random-model", str(folder), "--config", str(cfg), "--seed", "3",
                 "--std", "0.2"]) == 0
    capsys.readouterr()
    assert GikaraxConfig.from_json(str(folder)).to_dict() == GikaraxConfig.from_dict(TINY["A"]).to_dict()
