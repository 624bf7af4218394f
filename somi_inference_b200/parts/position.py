"""Position encodings that act on queries and keys before they reach the cache.

Rotary encoding as the reference computes it (somi_inference/models/qwen2.py:65-113):
inv_freq[i] = 1 / theta^(2i/d) for i in [0, d/2), angle = position * inv_freq[i]
in float32, and the rotation pairs element i with element i + d/2 ("rotate half"):
    out[i]       = x[i] * cos - x[i + d/2] * sin
    out[i + d/2] = x[i + d/2] * cos + x[i] * sin
Values are left untouched.  inv_freq is computed here once, on the host, in
float32 with the reference's expression; angles, sines and cosines are computed
in float32 inside the kernel, which also writes the rotated keys and the values
to their cache slots.

A position encoding answers
    encode_and_store(qkv, num_heads, num_kv_heads, head_dim, batch, paged, write)
where `qkv` is [T, (num_heads + 2 num_kv_heads) * head_dim], rotated in place.  One that sets
`takes_partial_sums = True` also accepts `partials=` (float32 [splits, T, width] partial sums of
the projection) and `bias=`, adds them up itself and leaves the queries in `qkv`.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl
from .registry import POSITION_ENCODINGS


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return []

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.ctx = ctx
        exponent = torch.arange(0, self.rotary_dim, 2) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(torch.float32).to(ctx.device)

    takes_partial_sums = True     # encode_and_store accepts `partials=` and `bias=`

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, batch, paged, write,
                         partials=None, bias=None):
        group = batch.groups[paged.group] if paged is not None else None
        self.ctx.ops.rope_store(
            qkv, batch.positions, self.inv_freq, num_heads, num_kv_heads, head_dim,
            self.rotary_dim,
            group.slot_map if (write and group is not None) else None,
            paged.keys if paged is not None else None,
            paged.values if paged is not None else None, partials=partials, bias=bias)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding:
    """Stores keys and values as they are (rotary_dim 0)."""

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return []

    takes_partial_sums = True

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=ctx.device)

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, batch, paged, write,
                         partials=None, bias=None):
        group = batch.groups[paged.group] if paged is not None else None
        self.ctx.ops.rope_store(
            qkv, batch.positions, self.inv_freq, num_heads, num_kv_heads, head_dim, 0,
            group.slot_map if (write and group is not None) else None,
            paged.keys if paged is not None else None,
            paged.values if paged is not None else None, partials=partials, bias=bias)


def rotary_frequencies(rotary) -> tuple[torch.Tensor, float]:
    """(float64 frequencies of the dims / 2 pairs, factor on every sine and cosine) of a rotation
    {"dims", "base", "scaling": None | {...}}.  Pair i turns by position * base^(-2i / dims) where
    nothing is scaled.  Scalings, by `kind`:

    "bands" {factor, low, high, original}: with wavelength l = 2 pi / f, pairs with
        l < original / high keep f, pairs with l > original / low get f / factor, and between
        the two s = (original / l - low) / (high - low) blends (1 - s) f / factor + s f.
    "ramp" {factor, original, fast, slow}: with index(t) = dims ln(original / (2 pi t)) /
        (2 ln base), lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), dims - 1) and
        r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i gets f / factor * r_i +
        f * (1 - r_i), and sines and cosines are multiplied by 0.1 ln(factor) + 1.
    """
    import math
    dims = int(rotary.get("dims", 0)) if rotary else 0
    if dims == 0:
        return torch.zeros(1, dtype=torch.float64), 1.0
    base = float(rotary["base"])
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rotary.get("scaling")
    if not scaling:
        return torch.tensor(freq, dtype=torch.float64), 1.0
    kind, factor, original = scaling["kind"], float(scaling["factor"]), float(scaling["original"])
    if kind == "bands":
        low, high = float(scaling["low"]), float(scaling["high"])
        out = []
        for f in freq:
            wave = 2.0 * math.pi / f
            if wave < original / high:
                out.append(f)
            elif wave > original / low:
                out.append(f / factor)
            else:
                s = (original / wave - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        return torch.tensor(out, dtype=torch.float64), 1.0
    if kind == "ramp":
        def index(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(index(float(scaling["fast"]))), 0)
        hi = min(math.ceil(index(float(scaling["slow"]))), dims - 1)
        out = []
        for i, f in enumerate(freq):
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * r + f * (1.0 - r))
        return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0
    raise ValueError(f"unknown rotary scaling {kind!r} (kinds: 'bands', 'ramp')")
