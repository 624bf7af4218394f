"""Layer extras: parts of a layer that are neither mixer, feed-forward nor norm.

* `sigmoid_gate`: logits = W h + b; the branch it gates is multiplied by sigmoid(logits) when
  the next norm adds it to the residual stream (the sigmoid and the product are float32, in the
  norm's kernel).
* `channel_scale`: a per-channel factor of a residual branch (one weight per channel of the
  model width); the arrangement hands it to the kernel that adds the branch.
* `constant`: a number of the layer that its arrangement reads (`value`); it has no tensors.
* `causal_taps`: h <- h + conv(h), a causal convolution over time on every channel,
  conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j) with zeros before a sequence's start.  The last
  taps - 1 inputs of every request are kept in a state slot, so a sequence may arrive in portions
  of any size.
"""

from __future__ import annotations

import torch

from .base import BranchSum, BuildContext, StateNeeds, TensorDecl, names_of
from .linear import Linear
from .registry import LAYER_EXTRAS, STREAM_PARTS


@LAYER_EXTRAS.register("sigmoid_gate")
class SigmoidGate:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        return [TensorDecl(n["weight"], (int(params["out_features"]), int(params["in_features"]))),
                TensorDecl(n["bias"], (int(params["out_features"]),), init="zeros", matrix=False)]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.weight = tensors[n["weight"]]
        self.bias = tensors[n["bias"]].float()
        self.proj = Linear(self.weight, self.bias, ctx.ops)

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        """[T, out], or (a step of few tokens) the float32 partial sums [splits, T, out] of the
        split-K product, which the norm's kernel adds up before the sigmoid."""
        partial = self.proj.partial_sums(h)
        return partial if partial is not None else self.proj(h)


@LAYER_EXTRAS.register("causal_taps")
class CausalTaps:
    STATE = "taps"

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"], (int(params["channels"]), int(params["taps"])),
                           matrix=False)]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.channels = int(params["channels"])
        self.taps = int(params["taps"])
        ctx.ops.check_taps(self.taps)
        # [taps, channels] float32: a thread reads the taps of four neighbouring channels at once
        self.weight = tensors[names_of(params)["weight"]].float().t().contiguous()

    def state_needs(self) -> StateNeeds:
        """The last taps - 1 inputs of a request, oldest first, in the compute dtype."""
        if self.taps == 1:
            return StateNeeds({})
        return StateNeeds({self.STATE: ((self.taps - 1, self.channels), self.ctx.dtype)})

    def forward(self, h: torch.Tensor, batch, state: dict) -> torch.Tensor:
        out = torch.empty_like(h)
        self.ctx.ops.causal_taps(h, self.weight, state.get(self.STATE), batch, out)
        return out


@LAYER_EXTRAS.register("channel_scale")
class ChannelScale:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"], (int(params["size"]),), init="ones",
                           matrix=False)]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.weight = tensors[names_of(params)["weight"]]


@LAYER_EXTRAS.register("constant")
class Constant:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return []

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.value = float(params["value"])


@STREAM_PARTS.register("embedding_remix")
class EmbeddingRemix:
    """A product that makes a new residual stream out of the stream and the embedding's output:
        x <- W [x; x0]          W: [H, 2 H], the stream's columns first.
    What the run before left pending is added to the stream first.  The sums are float32; the
    product reads [x; x0] in the compute dtype and leaves a float32 stream."""

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        hidden = int(params["hidden_size"])
        return [TensorDecl(names_of(params)["weight"], (hidden, 2 * hidden))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.hidden = int(params["hidden_size"])
        self.proj = Linear(tensors[names_of(params)["weight"]], None, ctx.ops)

    def forward(self, residual: torch.Tensor, pending, start: torch.Tensor) -> torch.Tensor:
        delta = extra = None
        if isinstance(pending, BranchSum):
            delta, extra = pending.a, pending.b
            if extra is not None and extra.dtype != torch.float32:
                extra = extra.float()
        elif pending is None or isinstance(pending, torch.Tensor):
            delta = pending
        else:
            raise ValueError("the stream is re-mixed behind a layer that hands on a tensor or a "
                             f"BranchSum, not {type(pending).__name__}")
        both = torch.empty((residual.shape[0], 2 * self.hidden), dtype=self.ctx.dtype,
                           device=residual.device)
        self.ctx.ops.add_concat(residual, delta, extra, start, both)
        return self.proj.to_float32(both)
