"""Gikarax's mechanisms one at a time: each kernel and each part against the plain function of
the same mechanism.

Attention cases plant one dominating key (a key and one query are scaled so that its score stands
out) far back, on either side of the window's edge and at page borders, in prompt portions and in
single-token steps; the matrix states are carried over several steps of unequal requests and must
still hold a token written hundreds of steps before; routers are given logits that make the
choice clear."""

import math

import pytest
import torch

from somi_inference_b200.config import GikaraxConfig
from somi_inference_b200.parts import (FEED_FORWARDS, MIXERS, STREAM_PARTS, BranchSum, BuildContext,
                                       declared_tensors)
from somi_inference_b200.parts.base import PagedKVNeeds, StateNeeds
from somi_inference_b200.parts.position import rotary_frequencies
from tests.gikarax_tiny import causal, gated_linear, latent, layer, moe, pair, random_weights, windowed
from tests.gpu_util import Steps, gather_cache
from tests.plain import gikarax_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
STEPS = ({"a": 9, "b": 1}, {"a": 1, "b": 1, "c": 30}, {"c": 1, "a": 2, "b": 40}, {"a": 1, "c": 1},
         {"a": 17, "b": 2, "c": 8})


@pytest.fixture(scope="module")
def ops():
    from somi_inference_b200.ops import cuda_ops
    return cuda_ops()


def tol(dtype, f32=2e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def one_layer_model(kind, mixer, mlp, width=40, eps=1e-5):
    return dict(architecture="Gikarax", vocab=11, width=width, norm={"eps": eps},
                layers=[layer(kind, mixer, mlp)])


def build_parts(raw, ops, dtype, seed):
    """(mixer, feed-forward or None, weights by name as float64) of the only layer of `raw`."""
    w = random_weights(raw, seed, dtype)
    model = GikaraxConfig.from_dict(raw).to_model_spec()
    spec, decl = model.layers[0], declared_tensors(model)
    ctx = BuildContext(dtype=dtype, device=torch.device("cuda"), ops=ops)
    placed = {k: ctx.place(v, matrix=decl[k].matrix) for k, v in w.items()}
    mixer = MIXERS.build(spec.mixer, placed, ctx)
    ff = None if spec.feed_forward is None else FEED_FORWARDS.build(spec.feed_forward, placed, ctx)
    return mixer, ff, {k: v.double() for k, v in w.items()}


def summed(t):
    return t.double().sum(0) if t.dim() == 3 else t.double()


# ------------------------------------------------------------------ the layer's sums and norm
@pytest.mark.parametrize("width", [48, 256, 1030, 37])
@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_adds_both_branches(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    T = 9
    res = torch.randn((T, width), generator=g).cuda() * 3 + 1
    w = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype).cuda()
    a2 = (torch.randn((T, width), generator=g) * 4).to(dtype).cuda()
    a3 = torch.randn((3, T, width), generator=g).cuda()
    b = torch.randn((T, width), generator=g).cuda()
    for a, extra in ((a2, b), (a3, b), (a2, None), (a3, None)):
        r = res.clone()
        out = torch.empty((T, width), dtype=dtype, device="cuda")
        ops.add_layernorm(r, a, None, w, 1e-5, out, extra=extra)
        want_r = res.double() + summed(a) + (0.0 if extra is None else extra.double())
        assert (r.double() - want_r).abs().max().item() < 1e-5
        assert (out.double() - plain.layer_norm(want_r, w.double(), 1e-5)).abs().max().item() < tol(dtype, 1e-5, 3e-2)
        rows = torch.tensor([4, 0, 7], dtype=torch.int32, device="cuda")
        r2 = res.clone()
        o3 = torch.empty((3, width), dtype=dtype, device="cuda")
        ops.add_layernorm(r2, a, None, w, 1e-5, o3, rows, extra=extra)
        assert torch.equal(r2, res)                              # chosen rows: the stream stays
        want = plain.layer_norm(want_r, w.double(), 1e-5)[rows.long()]
        assert (o3.double() - want).abs().max().item() < tol(dtype, 1e-5, 3e-2)


@pytest.mark.parametrize("width", [48, 37, 256])
@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_remixed_with_the_embedding(ops, dtype, width):
    """The part that opens a pass: [x + what is pending; x0] through one product, float32 out."""
    g = torch.Generator().manual_seed(width)
    T = 11
    ctx = BuildContext(dtype=dtype, device=torch.device("cuda"), ops=ops)
    wm = (torch.randn((width, 2 * width), generator=g) / width ** 0.5).to(dtype)
    part = STREAM_PARTS.get("embedding_remix")({"hidden_size": width, "names": {"weight": "w"}},
                                               {"w": wm.cuda()}, ctx)
    res, x0 = torch.randn((T, width), generator=g).cuda(), torch.randn((T, width), generator=g).cuda()
    a2 = torch.randn((T, width), generator=g).to(dtype).cuda()
    a3 = torch.randn((2, T, width), generator=g).cuda()
    b = torch.randn((T, width), generator=g).cuda()
    for pending in (None, a2, BranchSum(a2, b), BranchSum(a3, b), BranchSum(a3, None)):
        before = res.clone()
        got = part.forward(res, pending, x0)
        assert got.dtype == torch.float32 and torch.equal(res, before)
        x = res.double()
        if isinstance(pending, BranchSum):
            x = x + summed(pending.a) + (0.0 if pending.b is None else pending.b.double())
        elif pending is not None:
            x = x + pending.double()
        both = torch.cat([x, x0.double()], 1)
        if dtype == torch.bfloat16:
            both = both.bfloat16().double()                       # the product reads rounded rows
        want = both @ wm.double().cuda().T
        assert (got.double() - want).abs().max().item() < tol(dtype, 2e-5, 2e-3) * max(1.0, want.abs().max().item())


# ------------------------------------------------------------------ rotation with scaled frequencies
@pytest.mark.parametrize("rot", [
    {"dims": 8, "base": 10000.0, "scaling": {"kind": "bands", "factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}},
    {"dims": 12, "base": 300.0, "scaling": {"kind": "ramp", "factor": 6.0, "original": 40, "fast": 8.0, "slow": 1.0}},
    {"dims": 16, "base": 500.0}])
@pytest.mark.parametrize("dtype", DTYPES)
def test_rotation_with_scaled_frequencies(ops, dtype, rot):
    nq, nkv, hd, vd = 3, 1, 16, 6
    g = torch.Generator().manual_seed(rot["dims"])
    steps = Steps(ops, 2, paged=PagedKVNeeds(nkv, hd, None, vd), dtype=dtype, page_size=4)
    steps.step({"a": 30})
    batch, where = steps.step({"a": 5, "b": 7})
    width = (nq + nkv) * hd + nkv * vd
    qkv0 = torch.randn((batch.num_tokens, width), generator=g).to(dtype).cuda()
    qkv = qkv0.clone()
    inv, mag = rotary_frequencies(rot)
    view = steps.mgr.view(0).paged
    ops.headnorm_rotary_store(qkv, batch.positions, inv.cuda(), nq, nkv, hd, vd, rot["dims"], None, None,
                              0.0, batch.groups[0].slot_map, view.keys, view.values, magnitude=mag)
    sc = rot.get("scaling")
    plain_rot = {"dims": rot["dims"], "base": rot["base"],
                 "scaling": None if sc is None else {k: v for k, v in sc.items() if k != "kind"}}
    for r, (first, q, c) in where.items():
        x = qkv0[first:first + q, :nq * hd].double().cpu().reshape(q, nq, hd)
        want = plain.rotate_halves(x, plain_rot, first=c)
        got = qkv[first:first + q, :nq * hd].double().cpu().reshape(q, nq, hd)
        assert (got - want).abs().max().item() < tol(dtype, 1e-5, 3e-2)
    if sc is not None and sc["kind"] == "ramp":
        assert mag > 1.0


# ------------------------------------------------------------------ capped scores, sink, gate per head
@pytest.mark.parametrize("case", [
    # (heads, kv heads, key width, value width, window, page size, cap)
    (4, 2, 12, 20, 9, 8, 30.0), (2, 1, 16, 16, 21, 4, 200.0), (3, 3, 5, 3, 1, 4, 25.0), (2, 2, 32, 8, 64, 16, 45.0),
    (1, 1, 40, 40, None, 16, None), (6, 3, 64, 64, 36, 16, 35.0), (2, 1, 128, 128, 130, 64, 40.0),
    (8, 2, 64, 64, 44, 16, 2.0)])
@pytest.mark.parametrize("aligned", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_capped_attention_with_a_sink_and_planted_keys(ops, dtype, case, aligned):
    """Prompt portions and single tokens whose queries point at one scaled key each: the oldest
    key the window keeps, the one just before it (which must not be seen), the key a page border
    back, the very first key of the sequence, the token itself.  Scores are capped, the softmax
    has one more in its denominator and every head's output is gated.  `aligned`: rows of a
    multiple of 16 bytes, which lets bfloat16 heads of 64 and 128 run the tensor-core kernels
    (prompt portions fed by TMA, single tokens split over their keys); else the kernel for any size."""
    nq, nkv, hd, vd, window, ps, cap = case
    g = torch.Generator().manual_seed(window or 7)
    reach = window or 10 ** 6
    steps = Steps(ops, 6, paged=PagedKVNeeds(nkv, hd, window, vd if vd != hd else None), dtype=dtype,
                  page_size=ps, max_len=400)
    steps.step({"a": 130, "b": 2 * reach + 3 if reach < 100 else 77, "c": 1, "d": min(reach, 300)})
    batch, where = steps.step({"a": 19, "b": 1, "c": 2, "d": 1, "e": 37, "f": 290})
    view = steps.mgr.view(0).paged
    for t in (view.keys, view.values):
        t.copy_(torch.randn(t.shape, generator=g).to(dtype))
    gate_at = (nq + nkv) * hd + nkv * vd                          # the gate's logits behind v
    width = gate_at + nq
    width += (-width % 8) if aligned else (1 if width % 8 == 0 else 0)
    qkv = torch.randn((batch.num_tokens, width), generator=g).to(dtype)
    table = batch.groups[0].block_table.cpu()
    planted = 0
    for j, r in enumerate(batch.host.requests):
        first, q, c = where[r]
        for i in range(q):
            p = c + i
            oldest = max(0, p - reach + 1)
            target = [oldest, oldest - 1, p - p % ps - 1, 0, p][(i + j) % 5]
            if target < 0 or (cap is not None and cap < 10):
                continue
            page = int(table[j, target // ps])
            if page < 0:          # given back: it lies behind the window and must not be read anyway
                continue
            sign = torch.where(torch.randn(hd, generator=g) > 0, 1.0, -1.0)
            view.keys[page, :, target % ps] = (min(6.0, 20.0 / (0.4 * hd)) * sign).to(dtype).cuda()
            qkv[first + i, :nq * hd] = sign.repeat(nq).to(dtype)
            planted += 1
    assert planted > 10 or (cap is not None and cap < 10)
    qkv = qkv.cuda()
    sinks = torch.zeros(nq, dtype=torch.float32, device="cuda")
    gate = qkv[:, gate_at:gate_at + nq]
    wants = {}
    for j, r in enumerate(batch.host.requests):
        first, q, c = where[r]
        keys, values = gather_cache(view, table[j], c + q, ps)
        qs = torch.zeros((c + q, nq, hd), dtype=torch.float64)
        qs[c:] = qkv[first:first + q, :nq * hd].double().cpu().reshape(q, nq, hd)
        want = plain.masked_attention(qs, keys, values, 0.4, window, cap, sink=True)[c:]
        wants[r] = (want * torch.sigmoid(gate[first:first + q].double().cpu())[:, :, None]).reshape(q, nq * vd)
    # the tcgen05 kernel, then the one that TMA feeds (sizes that neither takes run the kernel for
    # any size whatever the switch says)
    saved = ops.use_tc_prefill
    for use_tc in ((True, False) if aligned and dtype == torch.bfloat16 and hd in (64, 128) else (True,)):
        out = torch.empty((batch.num_tokens, nq * vd), dtype=dtype, device="cuda")
        ops.use_tc_prefill = use_tc
        try:
            ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], nq, nkv, hd, 0.4, window,
                                out, storage=view.storage, value_dim=vd, gate=gate, gate_per_head=True,
                                softcap=cap, sinks=sinks)
        finally:
            ops.use_tc_prefill = saved
        ops.check_errors()
        for r, (first, q, c) in where.items():
            err = (out[first:first + q].double().cpu() - wants[r]).abs().max().item()
            assert err < tol(dtype, 4e-5, 4e-2), (r, c, q, err, use_tc)


def test_a_learned_sink_joins_the_denominator(ops):
    """One key, score 0: the output is value / (1 + exp(sink)) per head."""
    steps = Steps(ops, 1, paged=PagedKVNeeds(1, 4, None, None), dtype=torch.float32, page_size=4)
    batch, _ = steps.step({"a": 1})
    view = steps.mgr.view(0).paged
    view.keys.zero_()
    view.values.fill_(1.0)
    qkv = torch.zeros((1, 2 * 4 + 2 * 4), device="cuda")
    sinks = torch.tensor([0.0, 1.5], device="cuda")
    out = torch.empty((1, 8), device="cuda")
    ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], 2, 1, 4, 1.0, None, out,
                        storage=view.storage, sinks=sinks)
    assert torch.allclose(out[0, :4].cpu(), torch.full((4,), 0.5))
    assert torch.allclose(out[0, 4:].cpu(), torch.full((4,), 1 / (1 + math.exp(1.5))))


# ------------------------------------------------------------------ the gated linear recurrence
def carry_over_steps(steps, seqs, run, counts_list):
    """Feed `seqs` (request -> per-token inputs, a dict of tensors [L, ...]) in the steps of
    `counts_list`; `run(batch, rows)` gets the step's rows of every input.  -> request -> [L, out]."""
    got = {r: [] for r in seqs}
    for counts in counts_list:
        batch, where = steps.step(counts)
        rows = {}
        for name in next(iter(seqs.values())):
            some = next(iter(seqs.values()))[name]
            buf = torch.zeros((batch.num_tokens, *some.shape[1:]), dtype=some.dtype)
            for r, (first, q, c) in where.items():
                buf[first:first + q] = seqs[r][name][c:c + q]
            rows[name] = buf.cuda()
        y = run(batch, rows)
        for r, (first, q, c) in where.items():
            assert c == sum(len(t) for t in got[r])
            got[r].append(y[first:first + q].double().cpu())
    return {r: torch.cat(v) for r, v in got.items() if v}


@pytest.mark.parametrize("geometry", [(3, 10, 6, 4.0), (4, 64, 64, 16.0), (1, 3, 5, 1.0), (2, 128, 32, 8.0),
                                      (5, 2, 3, 2.5), (2, 16, 100, 16.0), (6, 56, 40, 12.0)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_channel_decay_from_a_sigmoid_over_steps(ops, dtype, geometry):
    """The scan with alpha = sigmoid(z)^(1 / tau) per key channel, handed over as the negated
    logits and bias with the rate 1 / tau, q scaled, inputs that are views of wider rows."""
    H, d, dv, tau = geometry
    g = torch.Generator().manual_seed(d)
    steps = Steps(ops, 3, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=dtype)
    L = 60
    seqs = {r: {"qkv": torch.randn((L, 2 * H * d + H * dv + 3), generator=g).to(dtype),
                "z": 2.0 * torch.randn((L, H * d + 1), generator=g)} for r in "abc"}
    bias = 2.0 + torch.randn(H * d, generator=g)
    scale = d ** -0.5
    want = {}
    for r, s in seqs.items():
        x = s["qkv"].double()
        q = x[:, 1:1 + H * d].reshape(L, H, d) * scale
        k = x[:, 1 + H * d:1 + 2 * H * d].reshape(L, H, d)
        v = x[:, 1 + 2 * H * d:1 + 2 * H * d + H * dv].reshape(L, H, dv)
        alpha = torch.sigmoid(s["z"][:, :H * d].double() + bias.double()).pow(1.0 / tau).reshape(L, H, d)
        want[r] = plain.channel_decayed_sum(q, k, v, alpha).reshape(L, H * dv)
    rate = torch.full((H,), -math.log(tau), dtype=torch.float32, device="cuda")
    for prepare in (None, True, False):
        steps = Steps(ops, 3, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=dtype)
        state = steps.mgr.view(0).state["m"]

        def run(batch, rows):
            y = torch.empty((batch.num_tokens, H * dv), dtype=torch.float32, device="cuda")
            x = rows["qkv"]
            ops.matrix_state_scan(x[:, 1:1 + H * d], x[:, 1 + H * d:1 + 2 * H * d], x[:, 1 + 2 * H * d:-2],
                                  state, batch, y, H, H, d, dv, q_scale=scale,
                                  decay_logits=(-rows["z"])[:, :H * d], dt_bias=(-bias).cuda(), a_log=rate,
                                  prepare=prepare)
            return y

        got = carry_over_steps(steps, seqs, run, STEPS)
        for r in "abc":
            ref = want[r][:len(got[r])]
            assert len(ref) >= 28
            assert (got[r] - ref).abs().max().item() < 3e-5 * max(1.0, ref.abs().max().item()), (r, prepare)


def test_a_state_keeps_a_token_for_hundreds_of_steps(ops):
    """A channel whose decay is one to rounding holds what token 0 wrote through 400 single-token
    steps; a channel that decays loses it."""
    H, d, dv = 1, 4, 3
    steps = Steps(ops, 1, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=torch.float32)
    state = steps.mgr.view(0).state["m"]
    rate = torch.zeros(H, device="cuda")                          # tau = 1
    z = torch.tensor([[40.0, 40.0, -1.0, 0.0]])                   # sigmoid: 1, 1, 0.27, 0.5
    y = None
    for t in range(401):
        batch, _ = steps.step({"a": 1})
        k = torch.tensor([[1.0, 0.0, 1.0, 0.0]]) if t == 0 else torch.zeros((1, 4))
        v = torch.tensor([[1.0, 2.0, 3.0]]) if t == 0 else torch.zeros((1, 3))
        q = torch.tensor([[1.0, 0.0, 0.0, 0.0]]) if t < 400 else torch.tensor([[0.0, 0.0, 1.0, 0.0]])
        y = torch.empty((1, 3), device="cuda")
        ops.matrix_state_scan(q.cuda(), k.cuda(), v.cuda(), state, batch, y, H, H, d, dv,
                              decay_logits=(-z).cuda(), dt_bias=torch.zeros(4, device="cuda"), a_log=rate)
        if t == 399:
            assert torch.allclose(y.cpu(), torch.tensor([[1.0, 2.0, 3.0]]), atol=1e-5)
    assert y.abs().max().item() < 1e-30                           # channel 2 forgot it


@pytest.mark.parametrize("groups, shared", [(1, False), (6, True), (3, False), (4, True)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_in_parts_with_silu_gate(ops, dtype, groups, shared):
    g = torch.Generator().manual_seed(groups)
    T, C = 5, 60
    y = torch.randn((T, C), generator=g).cuda() * 3
    wide = torch.randn((T, C + 9), generator=g).to(dtype).cuda()
    z = wide[:, 4:4 + C]
    w = (1 + 0.3 * torch.randn(C // groups if shared else C, generator=g)).to(dtype).cuda()
    out = torch.empty((T, C), dtype=dtype, device="cuda")
    ops.group_rmsnorm_gate(y, z, w, 1e-5, groups, out, gate_act="silu")
    normed = plain.rms_norm(y.double().reshape(T, groups, C // groups), None, 1e-5)
    weight = w.double().reshape(1, 1, -1) if shared else w.double().reshape(1, groups, -1)
    want = (normed * weight).reshape(T, C) * plain.silu(z.double())
    assert (out.double() - want).abs().max().item() < tol(dtype, 1e-5, 4e-2)


# ------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("n, top", [(9, 4), (5, 1), (3, 3), (64, 6), (2, 1)])
def test_router_softmax_over_the_chosen(ops, n, top):
    g = torch.Generator().manual_seed(n)
    T = 37
    logits = torch.randn((T, n), generator=g).cuda() * 4
    logits[0, :] = 1.0                                             # all equal: the lowest indices
    if n > 2:
        logits[1, :3] = 90.0                                       # large and tied
    chosen, weight = ops.moe_router_select(logits, None, 1, 1, top, over_chosen=True)
    idx, wt = plain.choose_experts(logits.double().cpu(), top)
    assert torch.equal(chosen.cpu().long(), idx)
    assert (weight.double().cpu() - wt).abs().max().item() < 1e-6
    assert (weight.sum(1) - 1).abs().max().item() < 1e-6


@pytest.mark.parametrize("tokens", [1, 5, 16, 130])
@pytest.mark.parametrize("experts, top, ff", [(7, 4, 24), (3, 1, 20), (2, 2, 9), (6, 3, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_without_gates(ops, dtype, tokens, experts, top, ff):
    """One token to many (every way through the experts: entry by entry, the library's grouped
    product, the engine's own), against the plain mixture; rows whose choice is a close call in
    bfloat16 are left out."""
    raw = one_layer_model("latent_attention", latent(1, 4, 4, 4, 4, 1.0), moe(experts, top, ff))
    _, part, w = build_parts(raw, ops, dtype, experts)
    steps = Steps(ops, 1, dtype=dtype, max_len=256)
    batch, _ = steps.step({"a": tokens})
    x = torch.randn((tokens, 40), generator=torch.Generator().manual_seed(tokens)).to(dtype)
    got = summed(part.forward(x.cuda(), batch)).cpu()
    margins = []
    want = plain.expert_mixture(x.double(), w, "l0.mlp.", raw["layers"][0]["mlp"], margins)
    keep = margins[0] > (0.3 if dtype == torch.bfloat16 else 1e-4)
    assert keep.sum().item() * 2 >= tokens
    err = (got - want)[keep].abs().max().item()
    assert err < tol(dtype, 3e-5, 6e-2) * max(1.0, want.abs().max().item())


# ------------------------------------------------------------------ whole mixers over steps
MIXER_CASES = {
    "attention": ("attention", windowed(4, 2, 12, 20, 0.9, 9, 3.0, (8, 10000.0), (4.0, 1.0, 3.0, 64))),
    "attention_64": ("attention", windowed(4, 2, 64, 64, 0.3, 21, 35.0, (48, 1e4), (6.0, 1.0, 3.0, 32))),
    "attention_plain": ("attention", windowed(3, 3, 10, 6, 0.8)),
    "latent": ("latent_attention", latent(3, 8, 12, 20, 16, 0.7)),
    "latent_wide": ("latent_attention", latent(2, 32, 16, 48, 72, 0.3)),
    "parallel": ("parallel", pair(causal(4, 2, 12, 20, 0.6, (8, 300.0), (6.0, 40, 8.0, 1.0)),
                                  gated_linear(3, 10, 6, 4.0))),
    "parallel_wide": ("parallel", pair(causal(2, 1, 80, 48, 0.2, (40, 2e4), (5.0, 64, 24.0, 2.0)),
                                       gated_linear(2, 40, 72, 12.0, rank=12))),
}


@pytest.mark.parametrize("case", list(MIXER_CASES))
@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_alone_over_steps(ops, dtype, case):
    """Each mixer by itself, three requests in five steps of unequal portions and single tokens,
    against the plain mixer on whole sequences."""
    kind, m = MIXER_CASES[case]
    raw = one_layer_model(kind, m, None)
    mixer, _, w = build_parts(raw, ops, dtype, 7)
    needs = mixer.cache_needs()
    steps = Steps(ops, 3, paged=needs.paged, state=needs.state, dtype=dtype, page_size=8)
    g = torch.Generator().manual_seed(3)
    L = 60
    seqs = {r: {"h": torch.randn((L, 40), generator=g).to(dtype)} for r in "abc"}
    view = steps.mgr.view(0)

    def run(batch, rows):
        return summed(mixer.forward(rows["h"], batch, view, True))

    got = carry_over_steps(steps, seqs, run, STEPS)
    ops.check_errors()
    for r in "abc":
        want = plain.mixer(kind, seqs[r]["h"].double(), w, "l0.mix.", m, 1e-5)[:len(got[r])]
        err = (got[r] - want).abs().max().item()
        assert err < tol(dtype, 5e-5, 8e-2) * max(1.0, want.abs().max().item()), (r, err)
