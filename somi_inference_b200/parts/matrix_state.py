"""Mixers that carry a matrix per head from token to token instead of a cache of keys.

Both keep, per request and head, a float32 state M [key width, value width] (stored column by
column) that starts at zero, lives in the request's state slot and is read out by the token's query:

`delta_rule` (the gated delta rule with a decay per key channel).  With h the mixer's input,
H heads over G query/key heads (head i reads query/key head i // (H / G)):
    q = silu(conv(Wq h)), k = silu(conv(Wk h)), v = silu(conv(Wv h))   (short causal convolutions
        per channel, zeros before the start; their last taps - 1 inputs are state too)
    q <- q / sqrt(|q|^2 + unit_eps) * key_width^-1/2,  k <- k / sqrt(|k|^2 + unit_eps)   per head
    beta = sigmoid(Wb h)                                                  one per head
    g = exp(-exp(A_log) * softplus(Wa2 (Wa1 h) + dt_bias))                per head and key channel
    M <- g[:, None] * M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q      (in this order)
    out = Wo (rmsnorm_per_head(o) * norm * sigmoid(Wg2 (Wg1 h)))
`decay_sum` (linear attention with a constant decay per head):
    q = silu(Wq h), k = silu(Wk h), v = silu(Wv h)
    M <- decay * M + k v^T;  o = M^T q
    out = Wo (rmsnorm_over_all_heads(o) * norm * sigmoid(Wg h))

`gated_linear_attention` (at the end of the file): a decay per key channel and token from a
sigmoid, no correction, a SiLU gate.

Products run in the compute dtype with float32 accumulation; unit norms, beta, the decays with
their softplus and exponentials, the recurrence, the norms and the gates' sigmoids are float32 in
the kernels.  One kernel walks through a request's rows of the step, so a sequence may arrive
in portions of any size.
"""

from __future__ import annotations

import torch

from .base import BuildContext, CacheNeeds, StateNeeds, TensorDecl, names_of
from .linear import Linear
from .registry import MIXERS


def _block_diagonal(a: torch.Tensor, b: torch.Tensor, tail: int) -> torch.Tensor:
    """[[a, 0, 0], [0, b, 0]] with `tail` zero columns at the end."""
    out = torch.zeros((a.shape[0] + b.shape[0], a.shape[1] + b.shape[1] + tail), dtype=a.dtype,
                      device=a.device)
    out[:a.shape[0], :a.shape[1]] = a
    out[a.shape[0]:, a.shape[1]:a.shape[1] + b.shape[1]] = b
    return out


@MIXERS.register("delta_rule")
class DeltaRuleMixer:
    graph_safe = True
    STATE, STATE_CONV = "delta_state", "delta_taps"

    @staticmethod
    def _sizes(params):
        H, G = int(params["heads"]), int(params["qk_heads"])
        return H, G, int(params["key_dim"]), int(params["value_dim"])

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, taps = int(params["hidden_size"]), int(params["taps"])
        H, G, d, dv = DeltaRuleMixer._sizes(params)
        ra, rg = int(params["decay_rank"]), int(params["gate_rank"])
        decl = []
        for part, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
            decl.append(TensorDecl(n[part + "_weight"], (rows, hidden)))
            decl.append(TensorDecl(n[part + "_taps"], (rows, taps), init="taps", matrix=False))
        return decl + [
            TensorDecl(n["beta_weight"], (H, hidden)),
            TensorDecl(n["a_log"], (H,), init="zeros", matrix=False),
            TensorDecl(n["decay_down"], (ra, hidden)), TensorDecl(n["decay_up"], (H * d, ra)),
            TensorDecl(n["dt_bias"], (H * d,), init="zeros", matrix=False),
            TensorDecl(n["gate_down"], (rg, hidden)), TensorDecl(n["gate_up"], (H * dv, rg)),
            TensorDecl(n["norm"], (dv,), init="ones", matrix=False),
            TensorDecl(n["o_weight"], (hidden, H * dv))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.heads, self.qk_heads, self.key_dim, self.value_dim = self._sizes(params)
        ctx.ops.check_matrix_state_geometry(self.heads, self.qk_heads, self.key_dim, self.value_dim)
        self.taps = int(params["taps"])
        ctx.ops.check_conv_taps(self.taps)
        self.eps = float(params["eps"])
        self.unit_eps = float(params["unit_eps"])
        self.q_scale = float(params.get("q_scale", self.key_dim ** -0.5))
        parts = ("q", "k", "v")
        self.qk_width = self.qk_heads * self.key_dim
        self.conv_width = 2 * self.qk_width + self.heads * self.value_dim
        self.proj = Linear(torch.cat([tensors[n[p + "_weight"]] for p in parts], 0).contiguous(),
                           None, ctx.ops)
        self.taps_weight = torch.cat([tensors[n[p + "_taps"]].float() for p in parts], 0).t().contiguous()
        # one narrow product makes [decay rank | gate rank | beta logits]; one wide product over
        # that (its two matrices on the diagonal, zeros under the beta columns) makes the decay
        # logits per key channel and the gate logits per value channel, in float32
        down = torch.cat([tensors[n["decay_down"]], tensors[n["gate_down"]], tensors[n["beta_weight"]]], 0)
        self.narrow = Linear(down.contiguous(), None, ctx.ops)
        self.beta_at = down.shape[0] - self.heads
        self.wide = Linear(_block_diagonal(tensors[n["decay_up"]], tensors[n["gate_up"]],
                                           self.heads).contiguous(), None, ctx.ops)
        self.decay_width = self.heads * self.key_dim
        self.dt_bias = tensors[n["dt_bias"]].float().contiguous()
        self.a_log = tensors[n["a_log"]].float().contiguous()
        self.norm_weight = tensors[n["norm"]]
        self.out = Linear(tensors[n["o_weight"]], None, ctx.ops)

    def cache_needs(self) -> CacheNeeds:
        state = {self.STATE: ((self.heads, self.value_dim, self.key_dim), torch.float32)}
        if self.taps > 1:
            state[self.STATE_CONV] = ((self.taps - 1, self.conv_width), self.ctx.dtype)
        return CacheNeeds(paged=None, state=StateNeeds(state))

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        ops = self.ctx.ops
        T = x.shape[0]
        qkv = torch.empty((T, self.conv_width), dtype=x.dtype, device=x.device)
        ops.causal_conv(self.proj(x), self.conv_width, self.taps_weight, None,
                        cache.state.get(self.STATE_CONV), batch, qkv, act="silu")
        small = self.narrow(x)                                  # [T, decay rank | gate rank | beta]
        logits = self.wide.to_float32(small)                    # [T, heads * key | heads * value]
        y = torch.empty((T, self.heads * self.value_dim), dtype=torch.float32, device=x.device)
        ops.matrix_state_scan(qkv[:, :self.qk_width], qkv[:, self.qk_width:2 * self.qk_width],
                              qkv[:, 2 * self.qk_width:], cache.state[self.STATE], batch, y,
                              self.heads, self.qk_heads, self.key_dim, self.value_dim,
                              unit_eps=self.unit_eps, q_scale=self.q_scale,
                              beta=small[:, self.beta_at:], decay_logits=logits[:, :self.decay_width],
                              dt_bias=self.dt_bias, a_log=self.a_log)
        gated = torch.empty((T, self.heads * self.value_dim), dtype=x.dtype, device=x.device)
        ops.group_rmsnorm_gate(y, logits[:, self.decay_width:], self.norm_weight, self.eps,
                               self.heads, gated)
        partial = self.out.partial_sums(gated)
        return partial if partial is not None else self.out(gated)


@MIXERS.register("decay_sum")
class DecaySumMixer:
    graph_safe = True
    STATE = "decay_state"

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, H = int(params["hidden_size"]), int(params["heads"])
        d, dv = int(params["key_dim"]), int(params["value_dim"])
        return [TensorDecl(n["q_weight"], (H * d, hidden)), TensorDecl(n["k_weight"], (H * d, hidden)),
                TensorDecl(n["v_weight"], (H * dv, hidden)), TensorDecl(n["gate_weight"], (H * dv, hidden)),
                TensorDecl(n["norm"], (H * dv,), init="ones", matrix=False),
                TensorDecl(n["o_weight"], (hidden, H * dv))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.heads = int(params["heads"])
        self.key_dim, self.value_dim = int(params["key_dim"]), int(params["value_dim"])
        ctx.ops.check_matrix_state_geometry(self.heads, self.heads, self.key_dim, self.value_dim)
        decay = [float(v) for v in params["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=ctx.device)
        self.eps = float(params["eps"])
        self.qk_width = self.heads * self.key_dim
        self.inner = self.heads * self.value_dim
        self.proj = Linear(torch.cat([tensors[n["q_weight"]], tensors[n["k_weight"]],
                                      tensors[n["v_weight"]], tensors[n["gate_weight"]]], 0).contiguous(),
                           None, ctx.ops)
        self.norm_weight = tensors[n["norm"]]
        self.out = Linear(tensors[n["o_weight"]], None, ctx.ops)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=None, state=StateNeeds(
            {self.STATE: ((self.heads, self.value_dim, self.key_dim), torch.float32)}))

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        ops = self.ctx.ops
        T, w = x.shape[0], self.qk_width
        proj = self.proj(x)                                     # [T, q | k | v | gate logits]
        y = torch.empty((T, self.inner), dtype=torch.float32, device=x.device)
        ops.matrix_state_scan(proj[:, :w], proj[:, w:2 * w], proj[:, 2 * w:2 * w + self.inner],
                              cache.state[self.STATE], batch, y, self.heads, self.heads,
                              self.key_dim, self.value_dim, act_silu=True, decay=self.decay)
        gated = torch.empty((T, self.inner), dtype=x.dtype, device=x.device)
        ops.group_rmsnorm_gate(y, proj[:, 2 * w + self.inner:], self.norm_weight, self.eps, 1, gated)
        partial = self.out.partial_sums(gated)
        return partial if partial is not None else self.out(gated)


@MIXERS.register("gated_linear_attention")
class GatedLinearAttentionMixer:
    """Linear attention with a learned decay per key channel and token:

        q = Wq h * q_scale, k = Wk h, v = Wv h                        (heads x key / value width)
        alpha = sigmoid(Wa2 (Wa1 h) + ba)^(1 / tau)                   per head and key channel
        M <- alpha[:, None] * M + k v^T;  o = M^T q
        out = Wo (rmsnorm_per_head(o) * norm * silu(Wg h))            (`norm`: one head's width)

    alpha = exp(-softplus(-z) / tau), which is the matrix-state kernel's channel decay
    exp(-rate * softplus(a + bias)) with a = -z, bias = -ba and rate = 1 / tau: the second decay
    matrix and its bias are held negated (exact in every dtype).  The decay's logits are a float32
    product; softplus, the exponential, the recurrence, the norm and the gate's SiLU are float32."""

    graph_safe = True
    STATE = "gla_state"

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, H = int(params["hidden_size"]), int(params["heads"])
        d, dv, r = int(params["key_dim"]), int(params["value_dim"]), int(params["decay_rank"])
        return [TensorDecl(n["q_weight"], (H * d, hidden)), TensorDecl(n["k_weight"], (H * d, hidden)),
                TensorDecl(n["v_weight"], (H * dv, hidden)), TensorDecl(n["gate_weight"], (H * dv, hidden)),
                TensorDecl(n["decay_down"], (r, hidden)), TensorDecl(n["decay_up"], (H * d, r)),
                TensorDecl(n["decay_bias"], (H * d,), init="zeros", matrix=False),
                TensorDecl(n["norm"], (dv,), init="ones", matrix=False),
                TensorDecl(n["o_weight"], (hidden, H * dv))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        import math
        n = names_of(params)
        self.ctx = ctx
        self.heads = int(params["heads"])
        self.key_dim, self.value_dim = int(params["key_dim"]), int(params["value_dim"])
        ctx.ops.check_matrix_state_geometry(self.heads, self.heads, self.key_dim, self.value_dim)
        tau = float(params["tau"])
        if not tau > 0.0:
            raise ValueError("tau must be positive")
        self.eps = float(params["eps"])
        self.q_scale = float(params.get("q_scale", self.key_dim ** -0.5))
        self.qk_width = self.heads * self.key_dim
        self.inner = self.heads * self.value_dim
        self.proj = Linear(torch.cat([tensors[n["q_weight"]], tensors[n["k_weight"]],
                                      tensors[n["v_weight"]], tensors[n["gate_weight"]]], 0).contiguous(),
                           None, ctx.ops)
        self.narrow = Linear(tensors[n["decay_down"]], None, ctx.ops)
        self.wide = Linear((-tensors[n["decay_up"]]).contiguous(), None, ctx.ops)
        self.neg_bias = (-tensors[n["decay_bias"]].float()).contiguous()
        self.log_rate = torch.full((self.heads,), -math.log(tau), dtype=torch.float32, device=ctx.device)
        self.norm_weight = tensors[n["norm"]]
        self.out = Linear(tensors[n["o_weight"]], None, ctx.ops)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=None, state=StateNeeds(
            {self.STATE: ((self.heads, self.value_dim, self.key_dim), torch.float32)}))

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        ops = self.ctx.ops
        T, w = x.shape[0], self.qk_width
        proj = self.proj(x)                                     # [T, q | k | v | gate logits]
        logits = self.wide.to_float32(self.narrow(x))           # [T, heads * key]: -z
        y = torch.empty((T, self.inner), dtype=torch.float32, device=x.device)
        ops.matrix_state_scan(proj[:, :w], proj[:, w:2 * w], proj[:, 2 * w:2 * w + self.inner],
                              cache.state[self.STATE], batch, y, self.heads, self.heads,
                              self.key_dim, self.value_dim, q_scale=self.q_scale,
                              decay_logits=logits, dt_bias=self.neg_bias, a_log=self.log_rate)
        gated = torch.empty((T, self.inner), dtype=x.dtype, device=x.device)
        ops.group_rmsnorm_gate(y, proj[:, 2 * w + self.inner:], self.norm_weight, self.eps,
                               self.heads, gated, gate_act="silu")
        partial = self.out.partial_sums(gated)
        return partial if partial is not None else self.out(gated)
