"""Latent attention: queries, keys and values all pass through narrow latents, and only the
key/value latent is cached.

With h the mixer's input, per token:
    c_q = rmsnorm(W_dq h) * g_q          (q_rank wide)        q_h = W_uq,h c_q     (key_dim per head)
    c   = rmsnorm(W_dkv h) * g_kv        (kv_rank wide, cached)
    k_h = W_uk,h c,  v_h = W_uv,h c      for every head h, from the cached c of each position
    s   = scale * q_h . k_h  over the window's positions; softmax with a sink per head in the
          denominator (a learned score without a key or value)
    out = W_o (concat_h(sum_j p_j v_h,j) * sigmoid(W_g h))    (the gate only where `gate` is set)
No position encoding acts on queries or keys.  A mixer with `own_latent` false has no W_dkv: its
run reads the cache of an earlier run (same kv_rank) with its own W_uk, W_uv, window and sink.

Because k and v are linear in c, the expansions are moved to the query side and behind the sum:
    q_h . k_h = (W_uk,h^T q_h) . c,        sum_j p_j v_h,j = W_uv,h (sum_j p_j c_j),
so the attention kernel is multi-query attention over the latent cache itself (key = value = c,
kv_rank wide), and no step ever expands cached positions again.  The two per-head products are
batched products over heads.  The norms, scores, softmax and sink are float32.
"""

from __future__ import annotations

import torch

from .base import BuildContext, CacheNeeds, PagedKVNeeds, TensorDecl, names_of
from .linear import Linear
from .registry import MIXERS


@MIXERS.register("latent_attention")
class LatentAttentionMixer:
    graph_safe = True

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        D, H = int(params["hidden_size"]), int(params["heads"])
        dk, dv = int(params["key_dim"]), int(params["value_dim"])
        rq, rkv = int(params["q_rank"]), int(params["kv_rank"])
        decl = [TensorDecl(n["q_down"], (rq, D)),
                TensorDecl(n["q_norm"], (rq,), init="ones", matrix=False),
                TensorDecl(n["q_up"], (H * dk, rq)),
                TensorDecl(n["k_up"], (H * dk, rkv)), TensorDecl(n["v_up"], (H * dv, rkv)),
                TensorDecl(n["out"], (D, H * dv))]
        if params.get("own_latent", True):
            decl += [TensorDecl(n["kv_down"], (rkv, D)),
                     TensorDecl(n["kv_norm"], (rkv,), init="ones", matrix=False)]
        if params.get("sink"):
            decl.append(TensorDecl(n["sink"], (H,), init="zeros", matrix=False))
        if params.get("gate"):
            decl.append(TensorDecl(n["gate"], (H * dv, D)))
        return decl

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.heads = H = int(params["heads"])
        self.key_dim, self.value_dim = int(params["key_dim"]), int(params["value_dim"])
        self.q_rank, self.kv_rank = int(params["q_rank"]), int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        self.window = params.get("window")
        self.cache_window = params.get("cache_window", self.window)
        if self.cache_window is not None and (self.window is None or self.window > self.cache_window):
            raise ValueError("a mixer's window cannot reach further back than its cache is kept")
        self.own_latent = bool(params.get("own_latent", True))
        ctx.ops.check_latent_geometry(H, self.kv_rank)
        # one product for both latents of a layer that makes its own
        down = [tensors[n["q_down"]]] + ([tensors[n["kv_down"]]] if self.own_latent else [])
        self.down = Linear(torch.cat(down, 0).contiguous(), None, ctx.ops)
        self.q_norm = tensors[n["q_norm"]]
        self.kv_norm = tensors[n["kv_norm"]] if self.own_latent else None
        self.q_up = Linear(tensors[n["q_up"]], None, ctx.ops)
        # W_uk,h^T as rows [kv_rank, key_dim] (q'_h = q_h @ W_uk,h), W_uv,h as rows [value_dim, kv_rank]
        self.k_up_t = tensors[n["k_up"]].view(H, self.key_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.v_up = tensors[n["v_up"]].view(H, self.value_dim, self.kv_rank).contiguous()
        self.out = Linear(tensors[n["out"]], None, ctx.ops)
        self.sinks = tensors[n["sink"]].float().contiguous() if params.get("sink") else None
        self.gate = Linear(tensors[n["gate"]], None, ctx.ops) if params.get("gate") else None

    def cache_needs(self) -> CacheNeeds:
        # one "head" of kv_rank elements per position, read as key and as value: no value tensor
        return CacheNeeds(paged=PagedKVNeeds(1, self.kv_rank, self.cache_window, value_dim=0))

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        if owns_cache != self.own_latent:
            raise ValueError("a latent-attention mixer without a latent of its own must read "
                             "another run's cache, and one with its own must not")
        ops, T, H, R = self.ctx.ops, x.shape[0], self.heads, self.kv_rank
        paged = cache.paged
        group = batch.groups[paged.group]
        lat = self.down.partial_sums(x)           # few tokens: split-K partial sums, added up below
        if lat is None:
            lat = self.down(x)                                      # [T, q_rank (+ kv_rank)]
        cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
        ops.latent_norm_store(lat, self.q_rank, R if self.own_latent else 0, self.q_norm,
                              self.kv_norm, self.eps, cq,
                              group.slot_map if self.own_latent else None,
                              paged.keys if self.own_latent else None)
        q = self.q_up(cq)                                           # [T, H * key_dim]
        qa = ops.head_product(q.view(T, H, self.key_dim), self.k_up_t, heads_first=True)   # [H, T, R]
        o_lat = torch.empty_like(qa)
        ops.latent_attention(qa, paged.keys, batch, group, H, R, self.scale, self.window,
                             self.sinks, o_lat)
        o = ops.head_product(o_lat, self.v_up, heads_first=False)    # [T, H, value_dim]
        o = o.view(T, H * self.value_dim)
        if self.gate is not None:
            ops.sigmoid_gate_mul(o, self.gate(x))
        partial = self.out.partial_sums(o)
        return partial if partial is not None else self.out(o)
