"""Small Gikarax configurations for the tests, with random weights that make faults show.

A: a loop of three layers (one of each mixer) run twice behind a first layer, grouped heads,
   values wider than keys, rotation on part of the head with both frequency scalings, windows (9,
   21) that are no multiple of the page (8), a layer without a feed-forward, a layer whose tokens
   choose one expert, a cap low enough to bend the scores.
B: an odd width, one head, key and value widths that are no multiple of 2 or 4, no rotation, a
   window of one (a token sees only itself) beside an attention without window and cap, no loop,
   a router whose tokens take every expert (nothing to choose), tau of one.
C: a loop from the first layer on run three times and nothing behind it, keys and values of equal
   width, a window of 64 over pages of 16, rotation on the whole head without scaling, ranks of
   the latents larger than the width.
D: head sizes of 64 and 128, key widths of 128 in the recurrence, windows (48, 200) that are no
   multiple of a key tile, a page or a query tile, a latent of 256.
"""

from __future__ import annotations

import torch

from somi_inference_b200.config import GikaraxConfig
from somi_inference_b200.parts import declared_tensors


def latent(heads, dim, vdim, q_rank, kv_rank, scale):
    return dict(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale)


def windowed(heads, kv_heads, dim, vdim, scale, window=None, softcap=None, rot=None, bands=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if bands is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return m


def causal(heads, kv_heads, dim, vdim, scale, rot=None, ramp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if ramp is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), ramp))
    return m


def gated_linear(heads, dim, vdim, tau, rank=5):
    return dict(heads=heads, dim=dim, vdim=vdim, tau=tau, decay_rank=rank)


def pair(left, right):
    return {"left": left, "right": right}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


TINY_A = dict(architecture="Gikarax", vocab=131, width=48, norm={"eps": 1e-5},
              loop={"start": 1, "stop": 4, "times": 2},
              layers=[layer("attention", windowed(4, 2, 12, 20, 0.9, 9, 3.0, (8, 10000.0), (4.0, 1.0, 3.0, 64)),
                            moe(5, 2, 24)),
                      layer("parallel", pair(causal(4, 2, 12, 20, 0.6, (8, 300.0), (6.0, 40, 8.0, 1.0)),
                                             gated_linear(3, 10, 6, 4.0)), moe(3, 1, 20)),
                      layer("latent_attention", latent(3, 8, 12, 20, 16, 0.7), None),
                      layer("attention", windowed(2, 1, 16, 8, 0.7, 21, 30.0, (16, 500.0)), moe(4, 3, 16)),
                      layer("latent_attention", latent(2, 16, 8, 12, 24, 0.5), moe(6, 2, 8))])
TINY_B = dict(architecture="Gikarax", vocab=67, width=45, norm={"eps": 1e-4},
              layers=[layer("attention", windowed(1, 1, 5, 3, 1.2, 1, 7.0), moe(2, 2, 9)),
                      layer("parallel", pair(causal(1, 1, 5, 3, 1.1), gated_linear(1, 3, 5, 1.0, rank=1)),
                            moe(3, 2, 33)),
                      layer("attention", windowed(3, 3, 10, 6, 0.8), None),
                      layer("latent_attention", latent(1, 7, 3, 9, 5, 0.9), moe(4, 1, 21))])
TINY_C = dict(architecture="Gikarax", vocab=257, width=96, norm={"eps": 1e-6},
              loop={"start": 0, "stop": 3, "times": 3},
              layers=[layer("latent_attention", latent(4, 24, 24, 128, 104, 0.3), moe(6, 3, 32)),
                      layer("attention", windowed(4, 2, 32, 32, 0.5, 64, 20.0, (32, 1e6), (6.0, 1.0, 3.0, 128)),
                            moe(4, 2, 40)),
                      layer("parallel", pair(causal(6, 6, 16, 16, 0.75, (16, 100.0)),
                                             gated_linear(6, 8, 8, 12.0, rank=8)), moe(8, 5, 24))])
TINY_D = dict(architecture="Gikarax", vocab=300, width=128, norm={"eps": 1e-6},
              loop={"start": 1, "stop": 2, "times": 2},
              layers=[layer("attention", windowed(4, 2, 64, 64, 0.3, 48, 35.0, (48, 1e4), (4.0, 1.0, 2.0, 256)),
                            moe(4, 2, 64)),
                      layer("parallel", pair(causal(4, 2, 128, 128, 0.2, (64, 2e4), (5.0, 256, 24.0, 2.0)),
                                             gated_linear(2, 128, 32, 8.0, rank=16)), moe(4, 2, 64)),
                      layer("latent_attention", latent(4, 32, 64, 96, 256, 0.25), None),
                      layer("attention", windowed(2, 1, 128, 128, 0.2, 200, 15.0, (128, 1e4)), moe(3, 2, 48))])
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
PAGE_SIZES = {"A": 8, "B": 4, "C": 16, "D": 16}


def random_weights(raw: dict, seed: int, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Tensors for `raw`, by name: matrices spread widely enough that attention is peaked and the
    recurrence forgets at a visible rate; norm weights around one; biases of order one; the
    branches' last matrices smaller, so that a branch moves the stream by a fraction of its size
    and the rounding of bfloat16 is not multiplied from run to run.  Routers are made decisive, so
    that a comparison in bfloat16 does not rest on a close call: their logits spread over tens;
    a decisive router multiplies a small change of its input, so the experts' last matrices are
    smaller still."""
    g = torch.Generator().manual_seed(seed)
    cfg = GikaraxConfig.from_dict(raw)
    out = {}
    for name, decl in declared_tensors(cfg.to_model_spec()).items():
        shape = tuple(decl.shape)
        last = name.split(".")[-1]
        if last == "router":
            t = torch.randn(shape, generator=g) * (8.0 / shape[1] ** 0.5)
        elif last in ("norm", "norm1"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "out":
            t = 0.4 + 0.1 * torch.randn(shape, generator=g)
        elif last == "b" and name.endswith("a2.b"):
            t = 2.0 + 1.5 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name == "loop.in":
            t = torch.randn(shape, generator=g) * (1.0 / shape[1] ** 0.5)
        elif last in ("o", "down"):
            t = torch.randn(shape, generator=g) * ((0.25 if last == "down" else 0.6) / shape[1] ** 0.5)
        else:
            t = torch.randn(shape, generator=g) * (1.6 / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def stored_values(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The weights as float64 (integer tables as they are), exactly the values that were stored."""
    return {k: (v.double() if v.is_floating_point() else v) for k, v in weights.items()}


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
