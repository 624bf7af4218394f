"""Mixtures of experts: routed by a table (`table_moe`) or by a router (`routed_moe`, at the end).

`table_moe`: a token's id names its experts.

    experts of token t: table[id_t, 0..top-1] (distinct), each weighted 1 / top
    expert(h) = W_down (g * sigmoid(alpha * g) * (u + 1)),
                g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)
    y_t = (1 / top) * sum of its experts' outputs (+ a shared expert of the same form, with
          sizes and limit of its own, that every token passes)
There is no router product.  Gate and up rows are interleaved, so that the activation can be a
product's epilogue.  Three ways through the routed experts, by the step's size and dtype:
  * few (token, expert) pairs, bfloat16: every pair streams the rows of its own expert (a
    matrix-vector kernel; nothing is sorted);
  * many pairs, bfloat16: the pairs are grouped by expert on the device, the rows gathered in that
    order, and the library's grouped product runs over them, as the engine's prompt-sized products
    run in the library; the activation is a kernel between the two products;
  * float32, and sizes the others refuse: the engine's own grouped product (float32 FMAs, every
    output summed over K in ascending order whatever the step).
The shared expert is two ordinary products with the activation's kernel between them.  The
weighted sum is float32.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl, names_of
from .linear import Linear
from .registry import FEED_FORWARDS


def _interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[..., ff, K] twice -> [..., 2 ff, K] with rows gate_0, up_0, gate_1, up_1, ..."""
    return torch.stack([gate, up], dim=-2).reshape(*gate.shape[:-2], 2 * gate.shape[-2], gate.shape[-1])


@FEED_FORWARDS.register("table_moe")
class TableMoE:
    graph_safe = True

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, E, top = int(params["hidden_size"]), int(params["experts"]), int(params["top"])
        ff = int(params["expert_ff"])
        decl = [TensorDecl(n["table"], (int(params["vocab_size"]), top), init=f"distinct:{E}",
                           matrix=False)]
        for e in range(E):
            decl += [TensorDecl(n["gate"][e], (ff, hidden)), TensorDecl(n["up"][e], (ff, hidden)),
                     TensorDecl(n["down"][e], (hidden, ff))]
        shared = params.get("shared")
        if shared:
            sff = int(shared["ff"])
            decl += [TensorDecl(n["shared_gate"], (sff, hidden)), TensorDecl(n["shared_up"], (sff, hidden)),
                     TensorDecl(n["shared_down"], (hidden, sff))]
        return decl

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.experts, self.top = int(params["experts"]), int(params["top"])
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"top = {self.top} of {self.experts} experts")
        self.gated = (float(params["limit"]), float(params["alpha"]))
        self.table = tensors[n["table"]].contiguous()
        if self.table.numel() and not (0 <= int(self.table.min()) and int(self.table.max()) < self.experts):
            raise ValueError(f"the routing table names experts outside 0..{self.experts - 1}")
        E = range(self.experts)
        self.w_gate_up = _interleave(torch.stack([tensors[n["gate"][e]] for e in E]),
                                     torch.stack([tensors[n["up"][e]] for e in E])).contiguous()
        self.w_down = torch.stack([tensors[n["down"][e]] for e in E]).contiguous()
        shared = params.get("shared")
        self.shared = None
        if shared:
            self.shared = (Linear(_interleave(tensors[n["shared_gate"]], tensors[n["shared_up"]]).contiguous(),
                                  None, ctx.ops),
                           Linear(tensors[n["shared_down"]], None, ctx.ops),
                           (float(shared["limit"]), float(params["alpha"])))

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        ops, top, E = self.ctx.ops, self.top, self.experts
        extra = None
        if self.shared is not None:
            gate_up, down, (limit, alpha) = self.shared
            extra = down.to_float32(ops.clamped_gate_up(gate_up(x), limit, alpha))
        n_entries = x.shape[0] * top
        if ops.moe_gemv_supported(n_entries, x.shape[1], x.dtype) and self.w_down.shape[2] % 8 == 0:
            act = ops.moe_gemv(x, self.w_gate_up, batch.token_ids, self.table, per_token=True,
                               gated=self.gated)
            y = ops.moe_gemv(act, self.w_down, batch.token_ids, self.table, per_token=False)
            return ops.moe_combine(y, extra, 1.0 / top, top)
        route = ops.moe_route(batch.token_ids, self.table, E)
        if x.dtype == torch.bfloat16:
            rows = ops.moe_gather_rows(x, route, E, top)
            gu = ops.library_grouped_product(rows, self.w_gate_up, route)
            if gu is not None:
                y = ops.library_grouped_product(ops.clamped_gate_up(gu, *self.gated), self.w_down, route)
                if y is not None:
                    return ops.moe_combine(y, extra, 1.0 / top, top, place=ops._route_parts(route, E)[2])
        act = ops.grouped_product(x, self.w_gate_up, route=route, top=top, gather=True, gated=self.gated)
        y = ops.grouped_product(act, self.w_down, route=route, top=top, scatter=True, out_float32=True)
        return ops.moe_combine(y, extra, 1.0 / top, top)


@FEED_FORWARDS.register("routed_moe")
class RoutedMoE:
    """A mixture of experts whose router is a product over the token:

        s = softmax(W_router h) over all n = experts + identity outputs           (float32)
        choice = s + correction                  (a stored vector; it decides, it does not weigh)
        the n outputs form `groups.count` equal groups of neighbours; a group's score is its best
        choice; only members of the `groups.keep` best groups can be chosen
        the `top` best choices are the token's experts, each weighted by its s (not renormalised)
        expert(h) = W_down (silu(W_gate h) * (W_up h)); the last `identity` outputs are identity
        experts without tensors: expert(h) = h
        y = sum of weight * expert(h) over the chosen

    Two parameters change the form.  `weights` = "softmax_chosen": the `top` largest logits are
    chosen (no correction, no groups) and the weights are the softmax over the chosen logits only.
    `activation` (a name of the kernel table's `ACTIVATIONS`, e.g. "gelu"): experts without a gate,
    expert(h) = W_down act(W_up h), and no gate tensors.

    The router's logits are a float32 product; one kernel makes softmax, choice and weights and
    leaves a table row per token, from which the experts run like those of `table_moe`: entry by
    entry for a step of few tokens, grouped by expert otherwise.  The weighted sum is float32."""

    graph_safe = True

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, E = int(params["hidden_size"]), int(params["experts"])
        ff, outputs = int(params["expert_ff"]), E + int(params.get("identity", 0))
        decl = [TensorDecl(n["router"], (outputs, hidden))]
        if params.get("correction"):
            decl.append(TensorDecl(n["correction"], (outputs,), init="zeros", matrix=False))
        for e in range(E):
            if not params.get("activation"):
                decl.append(TensorDecl(n["gate"][e], (ff, hidden)))
            decl += [TensorDecl(n["up"][e], (ff, hidden)), TensorDecl(n["down"][e], (hidden, ff))]
        return decl

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.experts, self.top = int(params["experts"]), int(params["top"])
        self.outputs = self.experts + int(params.get("identity", 0))
        self.over_chosen = params.get("weights", "softmax_all") == "softmax_chosen"
        if params.get("weights", "softmax_all") not in ("softmax_all", "softmax_chosen"):
            raise ValueError(f"unknown router weights {params['weights']!r}")
        if self.over_chosen and (params.get("correction") or params.get("groups")):
            raise ValueError("a softmax over the chosen logits goes with no correction and no groups")
        self.act = params.get("activation")
        if self.act is not None and self.act not in ctx.ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.act!r}; known: {sorted(ctx.ops.ACTIVATIONS)}")
        groups = params.get("groups") or {}
        self.group_count = int(groups.get("count", 1))
        self.group_keep = int(groups.get("keep", self.group_count))
        if self.experts < 1 or not 1 <= self.top <= self.outputs:
            raise ValueError(f"top = {self.top} of {self.outputs} router outputs")
        if self.outputs % self.group_count or not 1 <= self.group_keep <= self.group_count:
            raise ValueError(f"{self.outputs} router outputs in {self.group_count} groups, of which "
                             f"{self.group_keep} are kept")
        if self.top > self.group_keep * (self.outputs // self.group_count):
            raise ValueError("the kept groups hold fewer outputs than a token chooses")
        self.router = Linear(tensors[n["router"]], None, ctx.ops)
        self.correction = (tensors[n["correction"]].float().contiguous()
                           if params.get("correction") else None)
        E = range(self.experts)
        if self.act is None:
            self.w_gate_up = _interleave(torch.stack([tensors[n["gate"][e]] for e in E]),
                                         torch.stack([tensors[n["up"][e]] for e in E])).contiguous()
            self.gated = (float("inf"), 1.0, 0.0)           # silu(gate) * up
        else:
            self.w_gate_up = torch.stack([tensors[n["up"][e]] for e in E]).contiguous()
            self.gated = None
        self.w_down = torch.stack([tensors[n["down"][e]] for e in E]).contiguous()

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        ops, top, E = self.ctx.ops, self.top, self.experts
        logits = self.router.to_float32(x)
        chosen, weight = ops.moe_router_select(logits, self.correction, self.group_count,
                                               self.group_keep, top, over_chosen=self.over_chosen)
        n_entries = x.shape[0] * top
        if ops.moe_gemv_supported(n_entries, x.shape[1], x.dtype) and self.w_down.shape[2] % 8 == 0:
            act = ops.moe_gemv(x, self.w_gate_up, None, chosen, per_token=True, gated=self.gated,
                               act=self.act)
            y = ops.moe_gemv(act, self.w_down, None, chosen, per_token=False)
            return ops.moe_combine_weighted(y, None, chosen, weight, x, E)
        route = ops.moe_route(None, chosen, E, self.outputs)
        if x.dtype == torch.bfloat16:
            rows = ops.moe_gather_rows(x, route, E, top)
            gu = ops.library_grouped_product(rows, self.w_gate_up, route)
            if gu is not None:
                mid = (ops.clamped_gate_up(gu, *self.gated) if self.act is None
                       else ops.unary_act(gu, self.act))
                y = ops.library_grouped_product(mid, self.w_down, route)
                if y is not None:
                    return ops.moe_combine_weighted(y, ops._route_parts(route, E)[2], chosen, weight, x, E)
        act = ops.grouped_product(x, self.w_gate_up, route=route, top=top, gather=True, gated=self.gated,
                                  act=self.act)
        y = ops.grouped_product(act, self.w_down, route=route, top=top, scatter=True, out_float32=True)
        return ops.moe_combine_weighted(y, None, chosen, weight, x, E)
