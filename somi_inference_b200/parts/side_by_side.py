"""Two mixers side by side: both read the same input, and the result is half the sum of their
outputs, each first RMS-normed over the model width with a weight of its own:

    out = (rmsnorm(left(h)) * w_left + rmsnorm(right(h)) * w_right) / 2

`left` and `right` are mixer specs of any registered kind.  At most one of them may keep paged
keys and values; the state tensors of both live in the layer's state slot side by side (their
names must differ).  The norms and the sum are float32, in one kernel.
"""

from __future__ import annotations

import torch

from .base import BuildContext, CacheNeeds, StateNeeds, TensorDecl, names_of
from .registry import MIXERS


@MIXERS.register("side_by_side")
class SideBySideMixer:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden = int(params["hidden_size"])
        return [*MIXERS.declare(params["left"]), *MIXERS.declare(params["right"]),
                TensorDecl(n["left_norm"], (hidden,), init="ones", matrix=False),
                TensorDecl(n["right_norm"], (hidden,), init="ones", matrix=False)]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.hidden = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.left = MIXERS.build(params["left"], tensors, ctx)
        self.right = MIXERS.build(params["right"], tensors, ctx)
        self.left_norm = tensors[n["left_norm"]]
        self.right_norm = tensors[n["right_norm"]]
        self.graph_safe = bool(getattr(self.left, "graph_safe", False)
                               and getattr(self.right, "graph_safe", False))
        self.cache_needs()

    def cache_needs(self) -> CacheNeeds:
        a, b = self.left.cache_needs(), self.right.cache_needs()
        if a.paged is not None and b.paged is not None:
            raise ValueError("only one of two mixers side by side may keep paged keys and values")
        sa = {} if a.state is None else dict(a.state.tensors)
        sb = {} if b.state is None else dict(b.state.tensors)
        clash = set(sa) & set(sb)
        if clash:
            raise ValueError(f"state names used by both mixers of a layer: {sorted(clash)}")
        state = {**sa, **sb}
        return CacheNeeds(paged=a.paged if a.paged is not None else b.paged,
                          state=StateNeeds(state) if state else None)

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        # either result may be the float32 partial sums [splits, T, H] of a split-K product (a
        # step of few tokens): the kernel adds them up
        a = self.left.forward(x, batch, cache, owns_cache)
        b = self.right.forward(x, batch, cache, owns_cache)
        out = torch.empty((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        self.ctx.ops.rmsnorm_pair_mean(a, b, self.left_norm, self.right_norm, self.eps, out)
        return out
