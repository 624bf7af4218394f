"""Dense gated feed-forward (SwiGLU).

Formula (somi_inference/models/qwen2.py:209-229): gu = h W_gu^T with
W_gu = cat(gate_proj, up_proj) on the output dimension
(somi_inference/models/qwen2_adapter.py:182-189,244-248); gate, up = the two
halves; y = (silu(gate) * up) W_down^T; silu(z) = z * sigmoid(z), in float32.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl, names_of
from .linear import Linear
from .registry import FEED_FORWARDS


@FEED_FORWARDS.register("swiglu")
class SwiGLU:
    graph_safe = True     # launches kernels only; nothing is decided on the host per step

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, inter = int(params["hidden_size"]), int(params["intermediate_size"])
        return [TensorDecl(n["gate_weight"], (inter, hidden)),
                TensorDecl(n["up_weight"], (inter, hidden)),
                TensorDecl(n["down_weight"], (hidden, inter))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.inter = int(params["intermediate_size"])
        # rows alternate gate_i, up_i, so that one thread pair of the product's epilogue (or one
        # vector load of the activation kernel) holds a matching gate and up
        gate, up = tensors[n["gate_weight"]], tensors[n["up_weight"]]
        self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.inter, -1).contiguous(),
                              None, ctx.ops)
        self.down = Linear(tensors[n["down_weight"]], None, ctx.ops)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        act = self.gate_up.swiglu(x)
        if act is None:
            gu = self.gate_up(x)
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            self.ctx.ops.silu_mul(gu, act, interleaved=True)
        partial = self.down.partial_sums(act)
        return partial if partial is not None else self.down(act)


@FEED_FORWARDS.register("dense_ff")
class DenseFF:
    """y = W_down act(W_up h + b_up) + b_down with an activation that has parameters of its own.

    `activation` "xielu": with (p, q) the two numbers of the tensor `act`,
    act(z) = softplus(p) z^2 + z/2 for z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2
    otherwise, evaluated in float32.  `activation` "relu2": act(z) = max(z, 0)^2; it has no tensor.
    `forward(x, batch, side=...)` lets the caller ride a second
    projection of the same input (a gate of the residual branch) on the up projection's product:
    the side matrix's rows are appended to W_up's, and its output comes back as a view."""

    graph_safe = True

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, inter = int(params["hidden_size"]), int(params["intermediate_size"])
        decl = [TensorDecl(n["up"], (inter, hidden)), TensorDecl(n["down"], (hidden, inter))]
        if params.get("activation") == "xielu":
            decl.append(TensorDecl(n["act"], (2,), matrix=False))
        if params.get("bias"):
            decl += [TensorDecl(n["up_bias"], (inter,), init="zeros", matrix=False),
                     TensorDecl(n["down_bias"], (hidden,), init="zeros", matrix=False)]
        return decl

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.activation = params.get("activation")
        if self.activation not in ("xielu", "relu2"):
            raise ValueError(f"unknown activation {self.activation!r} (known: 'xielu', 'relu2')")
        self.ctx = ctx
        self.inter = int(params["intermediate_size"])
        bias = bool(params.get("bias"))
        self.up_weight = tensors[n["up"]]
        self.up_bias = tensors[n["up_bias"]].float() if bias else None
        self.up = Linear(self.up_weight, self.up_bias, ctx.ops)
        self.down = Linear(tensors[n["down"]], tensors[n["down_bias"]].float() if bias else None,
                           ctx.ops)
        self.act = tensors[n["act"]].float().contiguous() if self.activation == "xielu" else None
        self._with_side = None

    def attach_side(self, weight: torch.Tensor, bias: torch.Tensor | None) -> None:
        """Append a second projection of the same input to the up projection."""
        w = torch.cat([self.up_weight, weight], 0).contiguous()
        b = None
        if self.up_bias is not None or bias is not None:
            zeros = lambda k: torch.zeros(k, dtype=torch.float32, device=w.device)
            b = torch.cat([self.up_bias if self.up_bias is not None else zeros(self.inter),
                           bias.float() if bias is not None else zeros(weight.shape[0])], 0)
        self._with_side = Linear(w, b, self.ctx.ops)

    def forward(self, x: torch.Tensor, batch, side: bool = False):
        proj = self._with_side if side else self.up
        fused = None
        if self.activation == "xielu":
            fused = proj.xielu_side(x, self.act, self.inter)  # few tokens: in the product's epilogue
        if fused is not None:
            act, rest = fused
        else:
            z = proj(x)                                 # [T, inter (+ side)]
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            if self.activation == "xielu":
                self.ctx.ops.xielu(z, self.inter, self.act, act)
            elif z.shape[1] == self.inter:
                self.ctx.ops.relu2(z, act)
            else:
                self.ctx.ops.relu2(z[:, :self.inter].contiguous(), act)
            rest = z[:, self.inter:]
        partial = self.down.partial_sums(act)
        y = partial if partial is not None else self.down(act)
        return (y, rest) if side else y
