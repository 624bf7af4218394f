"""A plain, slow restatement of the Poselorn decoder, one function per mechanism.

Written from the design's equations with whole-sequence tensors and Python loops over time.  It
shares nothing with the engine (no cache, no pages, no kernels, no portions) and is the oracle of
the engine's tests.  `cfg` is the dictionary of a model's config.json, `w` maps tensor names to
tensors; all arithmetic runs in `dtype` (float64 by default).

Notation: S tokens of one sequence at positions 0..S-1, D the model width, x the residual stream.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight` where there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def short_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [S, C], taps [C, n]: y[t] = sum_j taps[:, j] * u[t - (n - 1) + j]; inputs before the
    sequence's start are zero.  The last column of `taps` multiplies the current token."""
    S, _ = u.shape
    n = taps.shape[1]
    y = torch.zeros_like(u)
    for j in range(n):
        back = n - 1 - j
        if back < S:
            y[back:] += taps[:, j] * u[:S - back]
    return y


def unit_vector(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(sum(x^2) + eps) over the last axis (a sum, not a mean)."""
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


# ------------------------------------------------------------------ recurrences
def gated_delta_rule(q, k, v, beta, g):
    """q, k [S, H, d], v [S, H, dv], beta [S, H], g [S, H, d] (decay per key channel, in (0, 1]).
    Per head a state M [d, dv] from zero; per token, in this order:
        M <- g_t[:, None] * M;  u = beta_t (v_t - M^T k_t);  M <- M + k_t u^T;  o_t = M^T q_t."""
    S, H, d = q.shape
    dv = v.shape[2]
    M = torch.zeros((H, d, dv), dtype=q.dtype)
    out = torch.zeros((S, H, dv), dtype=q.dtype)
    for t in range(S):
        M = g[t][:, :, None] * M
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", M, k[t]))
        M = M + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", M, q[t])
    return out


def decayed_outer_sum(q, k, v, decay):
    """q, k [S, H, d], v [S, H, dv], decay [H]: M_t = decay M_(t-1) + k_t v_t^T, o_t = M_t^T q_t."""
    S, H, d = q.shape
    dv = v.shape[2]
    M = torch.zeros((H, d, dv), dtype=q.dtype)
    out = torch.zeros((S, H, dv), dtype=q.dtype)
    for t in range(S):
        M = decay[:, None, None] * M + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", M, q[t])
    return out


# ----------------------------------------------------------------------- mixers
def channel_delta_mixer(h, w, prefix, m, eps):
    """Projections, a short convolution and SiLU on each of q, k, v, unit-length queries and keys,
    a sigmoid step size per head, a decay per head and key channel through a narrow pair of
    projections, the gated delta rule, a per-head RMS norm with a gate through a second narrow
    pair, the output projection."""
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    p = prefix + ".mix."
    proj = {}
    for name in ("q", "k", "v"):
        proj[name] = silu(short_conv(h @ w[p + name].T, w[p + name + ".conv"]))
    q = unit_vector(proj["q"].reshape(S, G, d), 1e-6) * d ** -0.5
    k = unit_vector(proj["k"].reshape(S, G, d), 1e-6)
    v = proj["v"].reshape(S, H, dv)
    share = H // G
    q = q.repeat_interleave(share, dim=1)          # head i reads q/k head i // (H / G)
    k = k.repeat_interleave(share, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(S, H, d)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)
    o = gated_delta_rule(q, k, v, beta, g)
    o = rms_norm(o, w[p + "norm"], eps)
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(S, H, dv)
    return (o * gate).reshape(S, H * dv) @ w[p + "o"].T


def rotate_halves(x, dims, base):
    """x [S, heads, d]: entry i < dims/2 is paired with entry i + dims/2; the pair of the token at
    position p turns by p * base^(-2i/dims).  Entries from `dims` on pass unchanged."""
    S = x.shape[0]
    half = dims // 2
    if half == 0:
        return x
    pos = torch.arange(S, dtype=x.dtype)
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = pos[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def window_softmax_attention(q, k, v, scale, window):
    """q [S, H, d], k [S, G, d], v [S, G, dv] -> [S, H, dv].  Token i reads j with
    0 <= i - j < window (no window: all j <= i); query head h reads key/value head h // (H / G)."""
    S, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((S, H, v.shape[2]), dtype=q.dtype)
    for i in range(S):
        lo = 0 if window is None else max(0, i - window + 1)
        for hd in range(H):
            g = hd // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale
            out[i, hd] = torch.softmax(s, dim=0) @ v[lo:i + 1, g]
    return out


def window_attention_branch(h, w, p, m, eps):
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(S, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(S, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(S, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate_halves(q, rot["dims"], rot["base"])
        k = rotate_halves(k, rot["dims"], rot["base"])
    mask = m.get("mask")
    a = window_softmax_attention(q, k, v, m["scale"], mask["size"] if mask else None)
    return a.reshape(S, H * dv) @ w[p + "o"].T


def decay_attention_branch(h, w, p, m, eps):
    S = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(S, H, d)
    k = silu(h @ w[p + "k"].T).reshape(S, H, d)
    v = silu(h @ w[p + "v"].T).reshape(S, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    o = decayed_outer_sum(q, k, v, decay).reshape(S, H * dv)
    o = rms_norm(o, w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def parallel_mixer(h, w, prefix, m, eps):
    """Two branches read the same input; each result is RMS-normed over the model width with a
    weight of its own; the mixer returns half their sum."""
    p = prefix + ".mix."
    left = window_attention_branch(h, w, p + "left.", m["left"], eps)
    right = decay_attention_branch(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ---------------------------------------------------------------- feed-forwards
def dense_ff(h, w, prefix):
    p = prefix + ".mlp."
    z = torch.clamp(h @ w[p + "up"].T + w[p + "up.b"], min=0)
    return (z * z) @ w[p + "down"].T + w[p + "down.b"]


def choose_experts(z, correction, groups, top):
    """z [S, n] router logits -> (chosen [S, top], weights [S, top]).  s = softmax(z); the choice
    is made on s + correction; with `groups` = (count, keep) the n outputs are cut into `count`
    equal runs of neighbours, a run's score is its largest choice, and outputs outside the `keep`
    best runs cannot be chosen; the weights are the chosen outputs' s."""
    s = torch.softmax(z, dim=-1)
    choice = s + correction
    if groups:
        count, keep = groups
        size = z.shape[-1] // count
        best = choice.reshape(-1, count, size).max(dim=-1).values
        kept = best.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        choice = torch.where(allowed.repeat_interleave(size, dim=1), choice,
                             torch.full_like(choice, -math.inf))
    chosen = choice.topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen)


def choice_margin(z, correction, groups, top, least_weight: float = 0.0):
    """How far a token's choice is from another one [S]: the smallest distance between two choice
    scores where the order of the two decides who is chosen (the last chosen output against the
    best one left out, and with groups the last kept group against the best one dropped).
    Infinite where there is nothing to decide, or where neither side of the decision holds an
    output whose weight s exceeds `least_weight` (the other choice would change next to nothing)."""
    s = torch.softmax(z, dim=-1)
    choice = s + correction
    inf = torch.full((z.shape[0],), math.inf, dtype=z.dtype)
    margin = inf
    if groups:
        count, keep = groups
        size = z.shape[-1] // count
        best = choice.reshape(-1, count, size).max(dim=-1).values
        order = best.sort(dim=-1, descending=True)
        if keep < count:
            heaviest = s.reshape(-1, count, size).max(dim=-1).values
            stake = torch.maximum(heaviest.gather(1, order.indices[:, keep - 1:keep]),
                                  heaviest.gather(1, order.indices[:, keep:keep + 1]))[:, 0]
            margin = torch.where(stake > least_weight, order.values[:, keep - 1] - order.values[:, keep], inf)
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, order.indices[:, :keep], True)
        choice = torch.where(allowed.repeat_interleave(size, dim=1), choice,
                             torch.full_like(choice, -math.inf))
    if top < z.shape[-1]:
        order = choice.sort(dim=-1, descending=True)
        gap = order.values[:, top - 1] - order.values[:, top]
        stake = torch.maximum(s.gather(1, order.indices[:, top - 1:top]),
                              s.gather(1, order.indices[:, top:top + 1]))[:, 0]
        gap = torch.where(torch.isfinite(gap) & (stake > least_weight), gap, inf)
        margin = torch.minimum(margin, gap)
    return margin


def route(h, w, prefix, mlp):
    """-> (chosen [S, top] indices into experts + identity experts, their weights [S, top])."""
    p = prefix + ".mlp."
    r = mlp["router"]
    groups = r.get("groups")
    return choose_experts(h @ w[p + "router"].T, w[p + "correction"],
                          (groups["count"], groups["keep"]) if groups else None, r["top"])


def moe_ff(h, w, prefix, mlp, margins: list | None = None, least_weight: float = 0.02):
    p = prefix + ".mlp."
    E = mlp["router"]["experts"]
    chosen, weight = route(h, w, prefix, mlp)
    if margins is not None:
        r = mlp["router"]
        groups = r.get("groups")
        margins.append(choice_margin(h @ w[p + "router"].T, w[p + "correction"],
                                     (groups["count"], groups["keep"]) if groups else None, r["top"],
                                     least_weight))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t].tolist(), weight[t]):
            if e >= E:                      # an identity expert hands its input on
                out[t] += c * h[t]
            else:
                pe = f"{p}e{e}."
                out[t] += c * ((silu(w[pe + "gate"] @ h[t]) * (w[pe + "up"] @ h[t])) @ w[pe + "down"].T)
    return out


# -------------------------------------------------------------------- the model
def layer_order(cfg):
    """(layer, whether the embedding output is added in front of it) for every run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for turn in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, turn > 0 and i == loop["start"]))
    return runs + [(i, False) for i in range(loop["stop"], n)]


def layer(x, w, i, lc, cfg, margins: list | None = None):
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    p = f"l{i}"
    h = rms_norm(x, w[p + ".norm1"], eps)
    if lc["type"] == "channel_delta":
        branch = channel_delta_mixer(h, w, p, lc["mixer"], eps)
    else:
        branch = parallel_mixer(h, w, p, lc["mixer"], eps)
    total = branch * w[p + ".ls1"]
    mlp = lc.get("mlp")
    if mlp:
        h2 = rms_norm(x, w[p + ".norm2"], eps)
        f = dense_ff(h2, w, p) if mlp["kind"] == "dense" else moe_ff(h2, w, p, mlp, margins)
        total = total + f * w[p + ".ls2"]
    return x + mult * total


def forward(cfg, w, tokens, dtype=torch.float64, residuals: list | None = None,
            margins: list | None = None):
    """Logits [S, vocab] of one sequence; `residuals` collects x after every layer run, `margins`
    one tensor [S] per routed feed-forward that ran (see `choice_margin`)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    start = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x = start
    for i, again in layer_order(cfg):
        if again:
            x = x + start
        x = layer(x, w, i, cfg["layers"][i], cfg, margins)
        if residuals is not None:
            residuals.append(x)
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def greedy(cfg: dict, weights: dict, prompt, n_new: int, dtype=torch.float64) -> list[int]:
    """Greedy continuation by recomputing the whole sequence for every new token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, weights, seq, dtype)[-1].argmax()))
    return seq[len(prompt):]
