"""A plain, slow restatement of the Gikarax decoder, one function per mechanism.

Written from the design's equations with whole-sequence tensors and Python loops over time.  It
shares nothing with the engine (no cache, no pages, no kernels, no portions) and is the oracle of
the engine's tests.  `cfg` is the dictionary of a model's config.json, `w` maps tensor names to
tensors; all arithmetic runs in `dtype` (float64 by default).

Notation: S tokens of one sequence at positions 0..S-1, D the model width, x the residual stream.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------ norms
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight` where there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight; no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * weight


def silu(z):
    return z / (1.0 + torch.exp(-z))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


# -------------------------------------------------------------------- positions
def plain_frequencies(dims, base):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def banded_frequencies(dims, base, factor, low, high, original):
    """Long wavelengths are slowed by `factor`, short ones kept, the band between them blended:
    with l = 2 pi / f: l < original / high keeps f; l > original / low gives f / factor; else
    s = (original / l - low) / (high - low) and (1 - s) f / factor + s f."""
    out = []
    for f in plain_frequencies(dims, base):
        l = 2.0 * math.pi / f
        if l < original / high:
            out.append(f)
        elif l > original / low:
            out.append(f / factor)
        else:
            s = (original / l - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out, 1.0


def ramped_frequencies(dims, base, factor, original, fast, slow):
    """A linear ramp over the pair index between the pairs that make `fast` and `slow` turns in
    `original` positions: turns(t) -> index dims ln(original / (2 pi t)) / (2 ln base);
    frequency f / factor * ramp + f (1 - ramp); sines and cosines grow by 0.1 ln(factor) + 1."""
    def index(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index(fast)), 0)
    hi = min(math.ceil(index(slow)), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotation_table(rot):
    """(frequencies per pair, factor on sines and cosines) of a mixer's `rot` entry."""
    dims, base, sc = rot["dims"], rot["base"], rot.get("scaling")
    if sc is None:
        return plain_frequencies(dims, base), 1.0
    if "fast" in sc:
        return ramped_frequencies(dims, base, sc["factor"], sc["original"], sc["fast"], sc["slow"])
    return banded_frequencies(dims, base, sc["factor"], sc["low"], sc["high"], sc["original"])


def rotate_halves(x, rot, first=0):
    """x [S, heads, d]: entry i < dims/2 is paired with entry i + dims/2; the pair (u, v) of the
    token at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * frequency_i.
    Entries from `dims` on pass unchanged.  `first`: the position of row 0."""
    if rot is None or rot["dims"] == 0:
        return x
    dims, half = rot["dims"], rot["dims"] // 2
    freq, mag = rotation_table(rot)
    pos = torch.arange(first, first + x.shape[0], dtype=x.dtype)
    angle = pos[:, None] * torch.tensor(freq, dtype=x.dtype)[None, :]
    c, s = (torch.cos(angle) * mag)[:, None, :], (torch.sin(angle) * mag)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# -------------------------------------------------------------------- attention
def masked_attention(q, k, v, scale, window=None, softcap=None, sink=False):
    """q [S, H, d], k [S, G, d], v [S, G, dv]; query head h reads key/value head h // (H / G).
    Position i sees j <= i, with `window` only those with i - j < window.  Scores q.k * scale,
    then cap * tanh(score / cap) where there is a cap; softmax over the visible keys, with `sink`
    one more term exp(0) in the denominator that has no value."""
    S, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    out = torch.zeros((S, H, dv), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(S):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            m = s.max()
            if sink:
                m = torch.clamp(m, min=0.0)
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(-m) if sink else 0.0)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def gated_window_attention(h, w, p, m, eps):
    """The 'attention' mixer: per-head RMS norm of queries and keys (one weight for all heads),
    rotation, capped scores under a sliding window, a sink in the denominator, one sigmoid gate
    per head from the mixer's input, the output projection."""
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w[p + "q"].T).reshape(S, H, d), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T).reshape(S, G, d), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).reshape(S, G, dv)
    q, k = rotate_halves(q, m.get("rot")), rotate_halves(k, m.get("rot"))
    mask = m.get("mask")
    o = masked_attention(q, k, v, m["scale"], None if mask is None else mask["size"],
                         m.get("softcap"), sink=True)
    gate = torch.sigmoid(h @ w[p + "g"].T)                     # [S, H]
    return (o * gate[:, :, None]).reshape(S, H * dv) @ w[p + "o"].T


def biased_attention(h, w, p, m):
    """The left half of the 'parallel' mixer: projections with biases, rotation, plain causal
    softmax attention, an output projection with a bias."""
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(S, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(S, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(S, G, dv)
    q, k = rotate_halves(q, m.get("rot")), rotate_halves(k, m.get("rot"))
    o = masked_attention(q, k, v, m["scale"])
    return o.reshape(S, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def latent_attention(h, w, p, m, eps):
    """Queries through a normed latent; keys and values of every head expanded from one normed
    latent per position; causal softmax; a sigmoid gate per output element; output projection."""
    S = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(S, H, d)
    c = rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).reshape(S, H, d)
    v = (c @ w[p + "uv"].T).reshape(S, H, dv)
    o = masked_attention(q, k, v, m["scale"]).reshape(S, H * dv)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ------------------------------------------------------------------- recurrence
def channel_decayed_sum(q, k, v, alpha):
    """q, k, alpha [S, H, d], v [S, H, dv]: per head a matrix M [d, dv] from zero,
    M_t = alpha_t[:, None] * M_(t-1) + k_t v_t^T, o_t = M_t^T q_t."""
    S, H, d = q.shape
    dv = v.shape[2]
    M = torch.zeros((H, d, dv), dtype=q.dtype)
    out = torch.zeros((S, H, dv), dtype=q.dtype)
    for t in range(S):
        M = alpha[t][:, :, None] * M + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", M, q[t])
    return out


def gated_linear_attention(h, w, p, m, eps):
    """The right half of the 'parallel' mixer: a decay per key channel sigmoid(z)^(1 / tau) from a
    narrow pair of projections with a bias, the decayed sum of outer products, an RMS norm per
    head (one weight for all heads), a SiLU gate, the output projection."""
    S = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(S, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(S, H, d)
    v = (h @ w[p + "v"].T).reshape(S, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).reshape(S, H, d)
    o = rms_norm(channel_decayed_sum(q, k, v, alpha), w[p + "norm"], eps).reshape(S, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def side_by_side(h, w, p, m, eps):
    """Half the sum of the two halves' outputs, each RMS-normed over the model width."""
    a = biased_attention(h, w, p + "left.", m["left"])
    b = gated_linear_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(a, w[p + "left.out"], eps) + rms_norm(b, w[p + "right.out"], eps))


# ----------------------------------------------------------------- feed-forward
def choose_experts(logits, top):
    """logits [S, E] -> (indices [S, top], weights [S, top]): the `top` largest logits (ties to
    the lower index), weighted by the softmax over the chosen logits only."""
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :top]
    picked = torch.gather(logits, 1, order)
    e = torch.exp(picked - picked.max(dim=-1, keepdim=True).values)
    return order, e / e.sum(dim=-1, keepdim=True)


def choice_margin(logits, top, least_weight=0.02):
    """[S]: by how much the last chosen logit beats the best one left out, infinite where nothing
    is left out or where the last chosen weighs less than `least_weight` (a swap changes little)."""
    S, E = logits.shape
    if top >= E:
        return torch.full((S,), float("inf"), dtype=logits.dtype)
    ordered = torch.sort(logits, dim=-1, descending=True).values
    _, wt = choose_experts(logits, top)
    gap = ordered[:, top - 1] - ordered[:, top]
    return torch.where(wt[:, top - 1] < least_weight, torch.full_like(gap, float("inf")), gap)


def expert_mixture(h, w, p, mlp, margins=None):
    """y_t = sum over the chosen experts of weight * W_down gelu(W_up h_t)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wt = choose_experts(h @ w[p + "router"].T, top)
    if margins is not None:
        margins.append(choice_margin(h @ w[p + "router"].T, top))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wt[t, j] * (w[f"{p}e{e}.down"] @ gelu_erf(w[f"{p}e{e}.up"] @ h[t]))
    return out


# ------------------------------------------------------------------------ model
def layer_runs(cfg):
    """[(layer, opens a pass)]: layers before the loop once, the looped layers `times` times in a
    row (each pass opened by the re-mix with the embedding's output), then the rest."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, False) for i in range(start)]
    for _ in range(times):
        out += [(i, i == start) for i in range(start, stop)]
    return out + [(i, False) for i in range(stop, n)]


def mixer(kind, h, w, p, m, eps):
    if kind == "attention":
        return gated_window_attention(h, w, p, m, eps)
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps)
    if kind == "parallel":
        return side_by_side(h, w, p, m, eps)
    raise ValueError(kind)


def forward(cfg, w, tokens, dtype=torch.float64, streams=None, margins=None):
    """Logits [S, vocab] of one sequence.  `streams`: a list that receives the residual stream
    after every layer run; `margins`: one that receives a tensor [S] per mixture of experts that
    ran (see `choice_margin`)."""
    w = {n: t.to(dtype) if t.is_floating_point() else t for n, t in w.items()}
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    for i, opens in layer_runs(cfg):
        if opens:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        layer = cfg["layers"][i]
        h = layer_norm(x, w[f"l{i}.norm1"], eps)
        y = mixer(layer["type"], h, w, f"l{i}.mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + expert_mixture(h, w, f"l{i}.mlp.", layer["mlp"], margins)
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg, weights, prompt, n_new, dtype=torch.float64):
    """Greedy continuation by recomputing the whole sequence for every new token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, weights, seq, dtype)[-1].argmax()))
    return seq[len(prompt):]
