"""RMS normalisation over the last dimension, fused with the residual sum.

Formula (somi_inference/models/qwen2.py:46-62): x32 = float(x);
y = x32 * rsqrt(mean(x32^2) + eps); out = weight * y.  The reference casts y to
the input dtype before the weight multiply; here the residual stream stays in
float32 and the product is rounded once, at the end.
"""

from __future__ import annotations

import torch

from .base import (BranchSum, BuildContext, GatedDelta, NormedDelta, ScaledBranches, TensorDecl,
                   names_of)
from .registry import NORMS


@NORMS.register("rmsnorm")
class RMSNorm:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"], (int(params["size"]),), init="ones",
                           matrix=False)]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.ctx = ctx
        self.weight = tensors[names_of(params)["weight"]]

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """`delta` is [T, size], or float32 [splits, T, size] partial sums that are added up; or a
        `NormedDelta`: the branch's result passes an RMS norm of its own before it is added."""
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=residual.device)
        if isinstance(delta, BranchSum):
            delta = ScaledBranches(delta.a, None, delta.b, None, 1.0)
        if isinstance(delta, ScaledBranches):
            self.ctx.ops.add_scaled_rmsnorm(residual, delta.a, delta.scale_a, delta.b, delta.scale_b,
                                            delta.mult, delta.extra, self.weight, None, self.eps,
                                            out, None, rows)
        elif isinstance(delta, NormedDelta):
            self.ctx.ops.add_normed_rmsnorm(residual, delta.delta, delta.weight, delta.eps,
                                            self.weight, self.eps, out, rows)
        else:
            self.ctx.ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
        return out

    def forward_pair(self, residual: torch.Tensor, delta, other: "RMSNorm | None"):
        """Add `delta` (a `ScaledBranches`, a tensor, partial sums or None) to the residual
        stream and normalise it twice, with this norm's weight and with `other`'s (None: once),
        in one pass over the rows.  Returns the two results (the second None without `other`)."""
        if delta is not None and not isinstance(delta, ScaledBranches):
            if isinstance(delta, (NormedDelta, GatedDelta)):
                raise ValueError("a layer of parallel branches cannot follow one whose result "
                                 "passes a norm or a gate of its own")
            delta = ScaledBranches(delta, None, None, None, 1.0)
        if other is not None and other.weight.dtype != self.weight.dtype:
            raise ValueError("the two norms of a layer hold their weights in one precision")
        shape = (residual.shape[0], self.size)
        out1 = torch.empty(shape, dtype=self.ctx.dtype, device=residual.device)
        out2 = None if other is None else torch.empty(shape, dtype=self.ctx.dtype, device=residual.device)
        d = delta
        self.ctx.ops.add_scaled_rmsnorm(
            residual, None if d is None else d.a, None if d is None else d.scale_a,
            None if d is None else d.b, None if d is None else d.scale_b,
            1.0 if d is None else d.mult, None if d is None else d.extra, self.weight,
            None if other is None else other.weight, self.eps, out1, out2, None)
        return out1, out2


@NORMS.register("layernorm")
class LayerNorm:
    """(x - mean) / sqrt(var + eps) * weight, var the mean of the squared deviations; a weight and
    no bias.  Mean, variance and the residual sum are float32.  `delta` may be a `GatedDelta`:
    the branch's result is then multiplied by sigmoid(gate logits) as it is added; or a
    `BranchSum`: both results of the layer before are added."""

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"], (int(params["size"]),), init="ones",
                           matrix=False)]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.ctx = ctx
        self.weight = tensors[names_of(params)["weight"]]

    def forward(self, residual: torch.Tensor, delta=None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        gate = extra = None
        if isinstance(delta, GatedDelta):
            delta, gate = delta.delta, delta.gate_logits
        elif isinstance(delta, BranchSum):
            delta, extra = delta.a, delta.b
            if extra is not None and extra.dtype != torch.float32:
                extra = extra.float()
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=residual.device)
        self.ctx.ops.add_layernorm(residual, delta, gate, self.weight, self.eps, out, rows,
                                   extra=extra)
        return out
