"""Attention whose queries and keys pass an RMS norm per head before they are rotated.

Per token, with h the mixer's input:
    q = Wq h + bq, k = Wk h + bk, v = Wv h + bv                    (`qkv_bias`)
    q, k: every head divided by its root mean square over the head (eps inside the root) and
          multiplied by a weight of the head's width that all heads share     (`head_norm`)
    q, k: entry i < dims / 2 of a head is paired with entry i + dims / 2; the pair of the token at
          position p turns by p * base^(-2i / dims); entries from `dims` on pass      (`rotary`;
          its `scaling` changes the frequencies: `position.rotary_frequencies`)
    scores q.k * scale, then cap * tanh(score / cap) where there is a `softcap`, over the keys the
          mask leaves: all earlier ones, or the token's own and the `size` - 1 before it
          (`mask` = {"kind": "window", "size"}); softmax, with `sink` = "zero" one more term
          exp(0) in its denominator that has no value ("learned": exp of a stored score per head)
    head i's output times sigmoid(Wg h)_i, one logit per head                      (`head_gate`)
    out = Wo heads (+ bo: `o_bias`)
Key and value widths may differ; query head i reads key/value head i // (heads / kv_heads).

One product makes q, k and v; one kernel normalises, rotates and writes keys and values to their
pages; attention reads everything, old and new, from the pages.  Norms, scores and softmax are
float32; angles are formed in float64 (their sines and cosines are float32).
"""

from __future__ import annotations

import torch

from .base import BuildContext, CacheNeeds, PagedKVNeeds, TensorDecl, names_of
from .linear import Linear
from .position import rotary_frequencies
from .registry import MIXERS


@MIXERS.register("normed_attention")
class NormedAttentionMixer:
    graph_safe = True

    @staticmethod
    def _sizes(params):
        return (int(params["num_heads"]), int(params["num_kv_heads"]), int(params["key_dim"]),
                int(params["value_dim"]))

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden = int(params["hidden_size"])
        heads, kv_heads, d, dv = NormedAttentionMixer._sizes(params)
        decl = []
        for part, rows in (("q", heads * d), ("k", kv_heads * d), ("v", kv_heads * dv)):
            decl.append(TensorDecl(n[part + "_weight"], (rows, hidden)))
            if params.get("qkv_bias"):
                decl.append(TensorDecl(n[part + "_bias"], (rows,), init="zeros", matrix=False))
        if params.get("head_norm"):
            decl += [TensorDecl(n["q_norm"], (d,), init="ones", matrix=False),
                     TensorDecl(n["k_norm"], (d,), init="ones", matrix=False)]
        if params.get("head_gate"):
            decl.append(TensorDecl(n["gate_weight"], (heads, hidden)))
        if params.get("sink") == "learned":
            decl.append(TensorDecl(n["sink"], (heads,), init="zeros", matrix=False))
        decl.append(TensorDecl(n["o_weight"], (hidden, heads * dv)))
        if params.get("o_bias"):
            decl.append(TensorDecl(n["o_bias"], (hidden,), init="zeros", matrix=False))
        return decl

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.heads, self.kv_heads, self.key_dim, self.value_dim = self._sizes(params)
        if self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot be grouped over {self.kv_heads} "
                             "key/value heads")
        if not (1 <= self.key_dim <= 256 and 1 <= self.value_dim <= 256):
            raise ValueError("key and value widths of 1 to 256 are supported")
        self.scale = float(params["scale"])
        self.eps = float(params.get("eps", 0.0))
        mask = params.get("mask") or {}
        kind, size = mask.get("kind"), mask.get("size")
        if kind not in (None, "window") or (kind is not None and not (size and size > 0)):
            raise ValueError(f"unknown mask {mask!r} (kinds: 'window' with a size)")
        self.window = int(size) if kind == "window" else None
        rotary = params.get("rotary") or {}
        self.rotary_dim = int(rotary.get("dims", 0))
        if self.rotary_dim % 2 or self.rotary_dim > self.key_dim:
            raise ValueError("rotary dims must be even and at most the key width")
        inv, self.magnitude = rotary_frequencies(rotary)
        self.inv_freq = inv.to(ctx.device)
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        sink = params.get("sink")
        if sink not in (None, "zero", "learned"):
            raise ValueError(f"unknown sink {sink!r} (kinds: 'zero', 'learned')")
        self.sinks = None
        if sink == "zero":
            self.sinks = torch.zeros(self.heads, dtype=torch.float32, device=ctx.device)
        elif sink == "learned":
            self.sinks = tensors[n["sink"]].float().contiguous()
        parts = ("q", "k", "v")
        bias = None
        if params.get("qkv_bias"):
            bias = torch.cat([tensors[n[p + "_bias"]].float() for p in parts], 0)
        weights = [tensors[n[p + "_weight"]] for p in parts]
        # the gate's logits are further columns of the same product
        self.head_gate = bool(params.get("head_gate"))
        self.gate_at = sum(w.shape[0] for w in weights)
        if self.head_gate:
            # (rows of zeros behind them keep the product's rows a multiple of 16 bytes, which the
            # tensor-core attention kernels need to fetch the queries)
            gate_w = tensors[n["gate_weight"]]
            pad = -(self.gate_at + self.heads) % 8
            weights += [gate_w, gate_w.new_zeros((pad, gate_w.shape[1]))]
            if bias is not None:
                bias = torch.cat([bias, torch.zeros(self.heads + pad, dtype=bias.dtype, device=bias.device)])
        self.proj = Linear(torch.cat(weights, 0).contiguous(), bias, ctx.ops)
        self.q_norm = tensors[n["q_norm"]] if params.get("head_norm") else None
        self.k_norm = tensors[n["k_norm"]] if params.get("head_norm") else None
        self.out = Linear(tensors[n["o_weight"]],
                          tensors[n["o_bias"]].float() if params.get("o_bias") else None, ctx.ops)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVNeeds(
            self.kv_heads, self.key_dim, self.window,
            None if self.value_dim == self.key_dim else self.value_dim))

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        ops, paged = self.ctx.ops, cache.paged
        qkv = self.proj(x)
        group = batch.groups[paged.group]
        ops.headnorm_rotary_store(qkv, batch.positions, self.inv_freq, self.heads, self.kv_heads,
                                  self.key_dim, self.value_dim, self.rotary_dim, self.q_norm,
                                  self.k_norm, self.eps, group.slot_map if owns_cache else None,
                                  paged.keys, paged.values, magnitude=self.magnitude)
        out = torch.empty((x.shape[0], self.heads * self.value_dim), dtype=x.dtype, device=x.device)
        ops.paged_attention(qkv, paged.keys, paged.values, batch, group, self.heads, self.kv_heads,
                            self.key_dim, self.scale, self.window, out, storage=paged.storage,
                            value_dim=self.value_dim,
                            gate=qkv[:, self.gate_at:self.gate_at + self.heads] if self.head_gate else None,
                            gate_per_head=self.head_gate, softcap=self.softcap, sinks=self.sinks)
        partial = self.out.partial_sums(out)
        return partial if partial is not None else self.out(out)
