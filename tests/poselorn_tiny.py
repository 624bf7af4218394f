"""Small Poselorn configurations for the tests, with random weights that make faults show.

A: a loop of two layers run twice (the embedding's output is added again in front of the second
   pass), grouped heads in both kinds of mixer, values wider than keys, rotation on part of the
   head, windows (9, 21) that are no multiple of the page (8), five experts and one identity
   expert in three groups of which two are kept, a layer without a feed-forward, a layer whose
   tokens choose one expert.
B: an odd width, one head, key and value widths that are no multiple of 2 or 4, one tap (no
   convolution state), no rotation, a window of one (a token sees only itself) beside no window at
   all, no loop, a branch factor and an embedding scale of one, a router whose tokens take every
   output (nothing to choose), groups that are all kept.
C: keys and values of equal width (one cache tensor), a window of 64 over pages of 16, a loop from
   the first layer on run three times, six experts and two identity experts in four groups, five
   taps, rotation on the whole head.
D: head sizes of 64 and 128, which the tensor-core attention kernels take in bfloat16, under
   windows (48, 200) that are no multiple of a key tile, a page or a query tile; key widths of 128
   in the recurrences.
"""

from __future__ import annotations

import torch

from somi_inference_b200.config import PoselornConfig
from somi_inference_b200.parts import declared_tensors


def delta(heads, kv_heads, dim, vdim, conv, ranks=(6, 5)):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv,
                decay_rank=ranks[0], gate_rank=ranks[1])


def window_attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def decayed(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))


def moe(experts, identity, top, ff, groups=None):
    r = {"experts": experts, "identity": identity, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def pair(left, right):
    return {"left": left, "right": right}


TINY_A = dict(architecture="Poselorn", vocab=131, width=48, norm={"eps": 1e-5}, embedding={"scale": 3.0},
              residual_mult=0.6, loop={"start": 1, "stop": 3, "times": 2},
              layers=[layer("channel_delta", delta(4, 2, 12, 20, 3), dense(72)),
                      layer("parallel", pair(window_attention(4, 2, 12, 20, 0.9, 9, rot=(8, 10000.0)),
                                             decayed(3, 10, 6, (0.5, 0.9, 0.99))), moe(5, 1, 2, 24, (3, 2))),
                      layer("channel_delta", delta(2, 2, 16, 8, 2), None),
                      layer("parallel", pair(window_attention(2, 1, 16, 8, 0.7, 21, rot=(16, 500.0)),
                                             decayed(2, 7, 9, (0.8, 1.0))), moe(3, 0, 1, 20))])
TINY_B = dict(architecture="Poselorn", vocab=67, width=45, norm={"eps": 1e-4}, embedding={"scale": 1.0},
              residual_mult=1.0,
              layers=[layer("parallel", pair(window_attention(1, 1, 5, 3, 1.2, 1), decayed(1, 3, 5, (0.7,))),
                            dense(33)),
                      layer("channel_delta", delta(3, 1, 5, 7, 1, ranks=(1, 3)), None),
                      layer("parallel", pair(window_attention(3, 3, 10, 6, 0.8), decayed(5, 2, 3, (0.3, 0.6, 0.9, 0.95, 0.2))),
                            moe(2, 0, 2, 9, (2, 2))),
                      layer("channel_delta", delta(1, 1, 9, 3, 4), dense(21))])
TINY_C = dict(architecture="Poselorn", vocab=257, width=96, norm={"eps": 1e-6}, embedding={"scale": 7.5},
              residual_mult=0.25, loop={"start": 0, "stop": 2, "times": 3},
              layers=[layer("channel_delta", delta(8, 4, 8, 16, 5), moe(6, 2, 3, 32, (4, 2))),
                      layer("parallel", pair(window_attention(4, 2, 32, 32, 0.5, 64, rot=(32, 1e6)),
                                             decayed(2, 32, 16, (0.9, 0.999))), dense(160)),
                      layer("parallel", pair(window_attention(6, 6, 16, 16, 0.75, 16, rot=(4, 100.0)),
                                             decayed(6, 8, 8, (0.1, 0.5, 0.8, 0.9, 0.97, 0.995))),
                            moe(4, 4, 2, 40, (2, 1)))])
TINY_D = dict(architecture="Poselorn", vocab=300, width=128, norm={"eps": 1e-6}, embedding={"scale": 2.0},
              residual_mult=0.5,
              layers=[layer("parallel", pair(window_attention(4, 2, 64, 64, 0.3, 48, rot=(32, 1e4)),
                                             decayed(2, 128, 32, (0.95, 0.99))), dense(256)),
                      layer("channel_delta", delta(2, 1, 128, 48, 4, ranks=(16, 8)), moe(4, 0, 2, 64)),
                      layer("parallel", pair(window_attention(2, 1, 128, 128, 0.2, 200, rot=(128, 1e4)),
                                             decayed(4, 16, 64, (0.5, 0.9, 0.99, 0.999))), dense(192))])
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
PAGE_SIZES = {"A": 8, "B": 4, "C": 16, "D": 16}


def random_weights(raw: dict, seed: int, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Tensors for `raw`, by name: matrices spread widely enough that attention is peaked and the
    recurrences forget at a visible rate; norm weights and channel scales around one; biases, taps,
    step biases and decay rates of order one.  Routers are made decisive, so that a comparison in
    bfloat16 does not rest on a close call: their logits spread over tens (the softmax is close to
    one-hot, and a token's further choices weigh next to nothing), the corrections are distinct
    values a fixed step apart, and where a token takes one expert only, the correction names it."""
    g = torch.Generator().manual_seed(seed)
    cfg = PoselornConfig.from_dict(raw)
    tops = {f"l{i}.mlp.correction": l.mlp["router"]["top"] for i, l in enumerate(cfg.layers)
            if l.mlp is not None and l.mlp["kind"] == "moe"}
    out = {}
    for name, decl in declared_tensors(cfg.to_model_spec()).items():
        shape = tuple(decl.shape)
        last = name.split(".")[-1]
        if last == "correction":
            n = shape[0]
            t = torch.linspace(-0.2, 0.2, n)[torch.randperm(n, generator=g)] if n > 1 else torch.zeros(1)
            if tops[name] == 1:
                t[int(torch.randint(0, n, (1,), generator=g))] = 4.0
        elif last == "router":
            t = torch.randn(shape, generator=g) * (12.0 / shape[1] ** 0.5)
        elif last in ("norm", "norm1", "norm2", "out", "ls1", "ls2"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif len(shape) == 1 and last in ("b", "dt_bias"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "A_log":
            t = 0.7 * torch.randn(shape, generator=g)
        elif last == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
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
