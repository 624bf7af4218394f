"""Poselorn's mechanisms one at a time: each kernel and each part against the plain function of
the same mechanism.

Attention cases plant one dominating key (a key and one query are scaled so that its score stands
out) far back, on either side of the window's edge and at page borders, in prompt portions and in
single-token steps; the matrix states are carried over several steps of unequal requests and must
still hold a token written hundreds of steps before; routers are given scores that make the
correction, the groups and the identity experts decide."""

import pytest
import torch

from somi_inference_b200.config import PoselornConfig
from somi_inference_b200.parts import FEED_FORWARDS, MIXERS, BuildContext, declared_tensors
from somi_inference_b200.parts.base import PagedKVNeeds, StateNeeds
from tests.gpu_util import Steps, gather_cache
from tests.plain import poselorn_plain as plain
from tests.poselorn_tiny import (decayed, delta, dense, layer, moe, pair, random_weights,
                                 window_attention)

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from somi_inference_b200.ops import cuda_ops
    return cuda_ops()


def tol(dtype, f32=2e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def one_layer_model(kind, mixer, mlp, width=40, eps=1e-5):
    return dict(architecture="Poselorn", vocab=11, width=width, norm={"eps": eps},
                embedding={"scale": 1.0}, residual_mult=1.0, layers=[layer(kind, mixer, mlp)])


def build_parts(raw, ops, dtype, seed):
    """(mixer, feed-forward or None, weights by name) of the only layer of `raw`."""
    w = random_weights(raw, seed, dtype)
    model = PoselornConfig.from_dict(raw).to_model_spec()
    spec, decl = model.layers[0], declared_tensors(model)
    ctx = BuildContext(dtype=dtype, device=torch.device("cuda"), ops=ops)
    placed = {k: ctx.place(v, matrix=decl[k].matrix) for k, v in w.items()}
    mixer = MIXERS.build(spec.mixer, placed, ctx)
    ff = None if spec.feed_forward is None else FEED_FORWARDS.build(spec.feed_forward, placed, ctx)
    return mixer, ff, {k: v.double() for k, v in w.items()}


# ------------------------------------------------------------------ the layer's sum and norms
@pytest.mark.parametrize("width", [48, 256, 1030, 37])
@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_branches_and_two_norms(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    T = 9
    res = torch.randn((T, width), generator=g).cuda()
    extra = torch.randn((T, width), generator=g).cuda()
    s1, s2, w1, w2 = ((1 + 0.3 * torch.randn(width, generator=g)).to(dtype).cuda() for _ in range(4))
    a2 = torch.randn((T, width), generator=g).to(dtype).cuda() * 4
    a3 = torch.randn((3, T, width), generator=g).cuda()
    b2 = torch.randn((T, width), generator=g).cuda()
    for a, b, sa, sb, ex in ((a2, b2, s1, s2, None), (a3, None, s1, None, extra), (a2, a3, None, s2, extra),
                             (None, None, None, None, None), (a3, a3, s1, s2, None)):
        r = res.clone()
        o1 = torch.empty((T, width), dtype=dtype, device="cuda")
        o2 = torch.empty((T, width), dtype=dtype, device="cuda")
        ops.add_scaled_rmsnorm(r, a, sa, b, sb, 0.45, ex, w1, w2, 1e-5, o1, o2)

        def branch(d, s):
            if d is None:
                return 0.0
            d = d.double() if d.dim() == 2 else d.double().sum(0)
            return d if s is None else d * s.double()

        want_r = res.double() + 0.45 * (branch(a, sa) + branch(b, sb)) + (0.0 if ex is None else ex.double())
        assert (r.double() - want_r).abs().max().item() < 1e-5
        assert (o1.double() - plain.rms_norm(want_r, w1.double(), 1e-5)).abs().max().item() < tol(dtype, 1e-5)
        assert (o2.double() - plain.rms_norm(want_r, w2.double(), 1e-5)).abs().max().item() < tol(dtype, 1e-5)
        # chosen rows and one norm only: the stream stays as it is
        rows = torch.tensor([4, 0, 7], dtype=torch.int32, device="cuda")
        r2 = res.clone()
        o3 = torch.empty((3, width), dtype=dtype, device="cuda")
        ops.add_scaled_rmsnorm(r2, a, sa, b, sb, 0.45, ex, w2, None, 1e-5, o3, None, rows)
        assert torch.equal(r2, res)
        want = plain.rms_norm(want_r, w2.double(), 1e-5)[rows.long()]
        assert (o3.double() - want).abs().max().item() < tol(dtype, 1e-5)


@pytest.mark.parametrize("groups, shared", [(1, False), (6, True), (3, False), (4, True)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_in_parts_with_sigmoid_gate(ops, dtype, groups, shared):
    g = torch.Generator().manual_seed(groups)
    T, C = 5, 60
    y = torch.randn((T, C), generator=g).cuda() * 3
    wide = torch.randn((T, C + 9), generator=g).to(dtype).cuda()
    z = wide[:, 4:4 + C]
    w = (1 + 0.3 * torch.randn(C // groups if shared else C, generator=g)).to(dtype).cuda()
    out = torch.empty((T, C), dtype=dtype, device="cuda")
    ops.group_rmsnorm_gate(y, z, w, 1e-5, groups, out)
    normed = plain.rms_norm(y.double().reshape(T, groups, C // groups), None, 1e-5)
    weight = w.double().reshape(1, 1, -1) if shared else w.double().reshape(1, groups, -1)
    want = (normed * weight).reshape(T, C) * torch.sigmoid(z.double())
    assert (out.double() - want).abs().max().item() < tol(dtype, 1e-5, 3e-2)
    ops.group_rmsnorm_gate(y, None, w, 1e-5, groups, out)
    assert (out.double() - (normed * weight).reshape(T, C)).abs().max().item() < tol(dtype, 1e-5, 3e-2)


@pytest.mark.parametrize("width", [45, 128, 1030])
@pytest.mark.parametrize("dtype", DTYPES)
def test_mean_of_two_normed_rows(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    T = 7
    wa, wb = ((1 + 0.3 * torch.randn(width, generator=g)).to(dtype).cuda() for _ in range(2))
    a2 = (torch.randn((T, width), generator=g) * 5).to(dtype).cuda()
    b2 = (torch.randn((T, width), generator=g) * 0.01).to(dtype).cuda()
    a3 = torch.randn((4, T, width), generator=g).cuda()
    for a, b in ((a2, b2), (a3, b2), (a2, a3)):
        out = torch.empty((T, width), dtype=torch.float32, device="cuda")
        ops.rmsnorm_pair_mean(a, b, wa, wb, 1e-5, out)
        da, db = (d.double() if d.dim() == 2 else d.double().sum(0) for d in (a, b))
        want = 0.5 * (plain.rms_norm(da, wa.double(), 1e-5) + plain.rms_norm(db, wb.double(), 1e-5))
        assert (out.double() - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("tokens", [1, 5, 130])
@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward_with_squared_relu_and_biases(ops, dtype, tokens):
    raw = one_layer_model("channel_delta", delta(1, 1, 4, 4, 2), dense(56))
    _, ff, w = build_parts(raw, ops, dtype, 3)
    steps = Steps(ops, 1, dtype=dtype, max_len=256)
    batch, _ = steps.step({"a": tokens})
    x = torch.randn((tokens, 40), generator=torch.Generator().manual_seed(tokens)).to(dtype)
    got = ff.forward(x.cuda(), batch)
    got = got.double().sum(0) if got.dim() == 3 else got.double()
    want = plain.dense_ff(x.double(), w, "l0")
    assert (got.cpu() - want).abs().max().item() < tol(dtype, 3e-5, 8e-2) * max(1.0, want.abs().max().item())


# ------------------------------------------------------------------ head norm, rotation, cache write
@pytest.mark.parametrize("geometry", [(3, 1, 12, 20, 8), (2, 2, 5, 3, 0), (4, 2, 32, 32, 32), (1, 1, 70, 6, 2),
                                      (6, 2, 80, 80, 48), (2, 1, 128, 64, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_head_norm_rotation_of_halves_and_store(ops, dtype, geometry):
    nq, nkv, hd, vd, rot = geometry
    g = torch.Generator().manual_seed(hd)
    steps = Steps(ops, 3, paged=PagedKVNeeds(nkv, hd, None, vd if vd != hd else None), dtype=dtype,
                  page_size=4)
    batch, _ = steps.step({"a": 30, "b": 2})
    batch, where = steps.step({"a": 3, "b": 1, "c": 6})
    width = (nq + nkv) * hd + nkv * vd
    qkv0 = torch.randn((batch.num_tokens, width + 5), generator=g).to(dtype).cuda()
    qw, kw = ((1 + 0.3 * torch.randn(hd, generator=g)).to(dtype).cuda() for _ in range(2))
    inv = (77.0 ** (-torch.arange(0, max(rot, 2), 2, dtype=torch.float64) / max(rot, 2))).cuda()
    view = steps.mgr.view(0).paged
    group = batch.groups[0]
    for normed in (True, False):
        qkv = qkv0.clone()
        ops.headnorm_rotary_store(qkv, batch.positions, inv, nq, nkv, hd, vd, rot, qw if normed else None,
                                  kw if normed else None, 1e-5, group.slot_map, view.keys, view.values)
        assert torch.equal(qkv[:, nq * hd:], qkv0[:, nq * hd:])          # k, v and what lies beside stay
        slots = group.slot_map.cpu()
        ps = steps.mgr.page_size
        for r, (first, q, c) in where.items():
            full = torch.zeros((c + q, width), dtype=torch.float64)
            full[c:] = qkv0[first:first + q, :width].double().cpu()
            qk = full[:, :(nq + nkv) * hd].reshape(c + q, nq + nkv, hd)
            if normed:      # the norm comes before the rotation
                qk = torch.cat([plain.rms_norm(qk[:, :nq], qw.double().cpu(), 1e-5),
                                plain.rms_norm(qk[:, nq:], kw.double().cpu(), 1e-5)], 1)
            qk = plain.rotate_halves(qk, rot, 77.0)[c:]
            got_q = qkv[first:first + q, :nq * hd].double().cpu().reshape(q, nq, hd)
            assert (got_q - qk[:, :nq]).abs().max().item() < tol(dtype, 1e-5, 3e-2)
            for i in range(q):
                page, off = int(slots[first + i]) // ps, int(slots[first + i]) % ps
                got_k = view.keys[page, :, off].double().cpu()
                got_v = view.values[page, :, off].double().cpu()
                assert (got_k - qk[i, nq:]).abs().max().item() < tol(dtype, 1e-5, 3e-2)
                assert torch.equal(got_v, full[c + i, (nq + nkv) * hd:].reshape(nkv, vd))


def test_rotation_at_far_positions_float32(ops):
    """Angles of thousands of radians: the kernel's sines and cosines stay those of the exact
    product position x frequency."""
    nq, nkv, hd, rot = 1, 1, 16, 16
    T = 6
    qkv = torch.randn((T, 3 * hd), generator=torch.Generator().manual_seed(0)).cuda()
    before = qkv.clone()
    pos = torch.tensor([0, 1, 4097, 50001, 131071, 999983], dtype=torch.int32, device="cuda")
    inv = (10000.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).cuda()
    ops.headnorm_rotary_store(qkv, pos, inv, nq, nkv, hd, hd, rot, None, None, 0.0, None, None, None)
    x = before[:, :hd].double().cpu()
    angle = pos.double().cpu()[:, None] * inv.cpu()[None, :]
    a, b = x[:, :rot // 2], x[:, rot // 2:]
    want = torch.cat([a * torch.cos(angle) - b * torch.sin(angle), b * torch.cos(angle) + a * torch.sin(angle)], 1)
    assert (qkv[:, :hd].double().cpu() - want).abs().max().item() < 2e-6


# ------------------------------------------------------------------ window attention
@pytest.mark.parametrize("case", [
    # (heads, kv heads, key width, value width, window, page size)
    (4, 2, 12, 20, 9, 8), (2, 1, 16, 16, 21, 4), (3, 3, 5, 3, 1, 4), (2, 2, 32, 8, 64, 16),
    (1, 1, 40, 40, None, 16), (6, 3, 80, 80, 36, 16), (2, 1, 96, 48, 130, 64),
    # head sizes of the tensor-core kernels (bfloat16)
    (4, 2, 64, 64, 96, 16), (8, 1, 128, 128, 300, 16), (4, 4, 128, 128, 50, 8), (2, 2, 64, 64, 5, 16)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_window_attention_with_planted_keys(ops, dtype, case):
    """Prompt portions and single tokens whose queries point at one scaled key each: the oldest
    key the window keeps, the one just before it (which must not be seen), the key a page border
    back, the very first key of the sequence, the token itself."""
    nq, nkv, hd, vd, window, ps = case
    g = torch.Generator().manual_seed(window or 7)
    reach = window or 10 ** 6
    steps = Steps(ops, 6, paged=PagedKVNeeds(nkv, hd, window, vd if vd != hd else None), dtype=dtype,
                  page_size=ps, max_len=400)
    steps.step({"a": 130, "b": 2 * reach + 3 if reach < 100 else 77, "c": 1, "d": min(reach, 300)})
    batch, where = steps.step({"a": 19, "b": 1, "c": 2, "d": 1, "e": 37, "f": 290})
    view = steps.mgr.view(0).paged
    for t in (view.keys, view.values):
        t.copy_(torch.randn(t.shape, generator=g).to(dtype))
    width = (nq + nkv) * hd + nkv * vd
    qkv = torch.randn((batch.num_tokens, width), generator=g).to(dtype)
    table = batch.groups[0].block_table.cpu()
    planted = 0
    for j, r in enumerate(batch.host.requests):
        first, q, c = where[r]
        for i in range(q):
            p = c + i
            oldest = max(0, p - reach + 1)
            target = [oldest, oldest - 1, p - p % ps - 1, 0, p][(i + j) % 5]
            if target < 0:
                continue
            page = int(table[j, target // ps])
            if page < 0:          # given back: it lies behind the window and must not be read anyway
                continue
            sign = torch.where(torch.randn(hd, generator=g) > 0, 1.0, -1.0)
            # a score of at most 100: far above the others, and its float32 rounding stays small
            view.keys[page, :, target % ps] = (min(6.0, 100.0 / (0.4 * hd)) * sign).to(dtype).cuda()
            qkv[first + i, :nq * hd] = sign.repeat(nq).to(dtype)
            planted += 1
    assert planted > 10
    qkv = qkv.cuda()
    # every prompt kernel in turn: two query tiles per CTA, one, mma.sync fed by TMA, by cp.async
    # (sizes that none of them takes run the kernel for any size whatever the switches say)
    switches = [(True, 1, True, True), (False, 1, True, True), (False, 1, False, True),
                (False, 1, False, False)]
    saved = (ops.use_pp_prefill, ops.pp_prefill_min_ctas, ops.use_tc_prefill, ops.use_tma_prefill)
    for k in range(4 if dtype == torch.bfloat16 and hd in (64, 128) else 1):
        out = torch.empty((batch.num_tokens, nq * vd), dtype=dtype, device="cuda")
        ops.use_pp_prefill, ops.pp_prefill_min_ctas, ops.use_tc_prefill, ops.use_tma_prefill = switches[k]
        try:
            ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], nq, nkv, hd, 0.4,
                                window, out, storage=view.storage, value_dim=vd)
        finally:
            ops.use_pp_prefill, ops.pp_prefill_min_ctas, ops.use_tc_prefill, ops.use_tma_prefill = saved
        ops.check_errors()
        for j, r in enumerate(batch.host.requests):
            first, q, c = where[r]
            keys, values = gather_cache(view, table[j], c + q, ps)
            qs = torch.zeros((c + q, nq, hd), dtype=torch.float64)
            qs[c:] = qkv[first:first + q, :nq * hd].double().cpu().reshape(q, nq, hd)
            want = plain.window_softmax_attention(qs, keys, values, 0.4, window)[c:].reshape(q, nq * vd)
            err = (out[first:first + q].double().cpu() - want).abs().max().item()
            assert err < tol(dtype, 4e-5, 4e-2), (r, c, q, err)


# ------------------------------------------------------------------ matrix states
def carry_over_steps(ops, steps, seqs, run, counts_list, width_out):
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
    return {r: torch.cat(v) if v else torch.zeros((0, width_out), dtype=torch.float64) for r, v in got.items()}


STEPS = ({"a": 9, "b": 1}, {"a": 1, "b": 1, "c": 30}, {"c": 1, "a": 2, "b": 40}, {"a": 1, "c": 1},
         {"a": 17, "b": 2, "c": 8})


@pytest.mark.parametrize("geometry", [(3, 3, 10, 12), (4, 2, 6, 40), (1, 1, 5, 70), (8, 2, 128, 16), (2, 1, 7, 3),
                                      (2, 2, 200, 20), (6, 3, 64, 48)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_rule_over_steps(ops, dtype, geometry):
    """The scan with unit norms, a step size per head and a decay per key channel, heads grouped
    over fewer query/key heads, inputs that are views of wider rows."""
    H, G, d, dv = geometry
    g = torch.Generator().manual_seed(d)
    steps = Steps(ops, 3, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=dtype)
    L = 60
    seqs = {r: {"qkv": torch.randn((L, 2 * G * d + H * dv + 3), generator=g).to(dtype),
                "beta": torch.randn((L, H + 2), generator=g).to(dtype),
                "a": torch.randn((L, H * d + 1), generator=g)} for r in "abc"}
    dt_bias, a_log = 0.5 * torch.randn(H * d, generator=g), 0.7 * torch.randn(H, generator=g)
    want = {}
    for r, s in seqs.items():
        x = s["qkv"].double()
        q = plain.unit_vector(x[:, 1:1 + G * d].reshape(L, G, d), 1e-6) * 0.37
        k = plain.unit_vector(x[:, 1 + G * d:1 + 2 * G * d].reshape(L, G, d), 1e-6)
        v = x[:, 1 + 2 * G * d:1 + 2 * G * d + H * dv].reshape(L, H, dv)
        step = plain.softplus(s["a"][:, :H * d].double() + dt_bias.double()).reshape(L, H, d)
        decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * step)
        want[r] = plain.gated_delta_rule(q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1), v,
                                         torch.sigmoid(s["beta"][:, 1:1 + H].double()), decay).reshape(L, H * dv)
    state = steps.mgr.view(0).state["m"]

    def run(batch, rows):
        y = torch.empty((batch.num_tokens, H * dv), dtype=torch.float32, device="cuda")
        x = rows["qkv"]
        ops.matrix_state_scan(x[:, 1:1 + G * d], x[:, 1 + G * d:1 + 2 * G * d], x[:, 1 + 2 * G * d:-2],
                              state, batch, y, H, G, d, dv, unit_eps=1e-6, q_scale=0.37,
                              beta=rows["beta"][:, 1:1 + H], decay_logits=rows["a"][:, :H * d],
                              dt_bias=dt_bias.cuda(), a_log=a_log.cuda())
        return y

    got = carry_over_steps(ops, steps, seqs, run, STEPS, H * dv)
    for r in "abc":
        ref = want[r][:len(got[r])]
        assert len(ref) >= 28
        assert (got[r] - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item()), r


@pytest.mark.parametrize("geometry", [(3, 10, 6), (4, 64, 64), (1, 3, 5), (2, 128, 32), (5, 2, 3), (2, 16, 100)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_decayed_sum_over_steps(ops, dtype, geometry):
    H, d, dv = geometry
    g = torch.Generator().manual_seed(d)
    steps = Steps(ops, 3, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=dtype)
    L = 60
    seqs = {r: {"qkv": torch.randn((L, 2 * H * d + 2 * H * dv), generator=g).to(dtype)} for r in "abc"}
    decay = torch.tensor([0.3, 0.9, 1.0, 0.999, 0.6][:H])
    want = {}
    for r, s in seqs.items():
        x = plain.silu(s["qkv"].double())
        want[r] = plain.decayed_outer_sum(x[:, :H * d].reshape(L, H, d), x[:, H * d:2 * H * d].reshape(L, H, d),
                                          x[:, 2 * H * d:2 * H * d + H * dv].reshape(L, H, dv),
                                          decay.double()).reshape(L, H * dv)
    state = steps.mgr.view(0).state["m"]

    def run(batch, rows):
        y = torch.empty((batch.num_tokens, H * dv), dtype=torch.float32, device="cuda")
        x = rows["qkv"]
        ops.matrix_state_scan(x[:, :H * d], x[:, H * d:2 * H * d], x[:, 2 * H * d:2 * H * d + H * dv],
                              state, batch, y, H, H, d, dv, act_silu=True, decay=decay.cuda())
        return y

    got = carry_over_steps(ops, steps, seqs, run, STEPS, H * dv)
    for r in "abc":
        ref = want[r][:len(got[r])]
        assert (got[r] - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item()), r


@pytest.mark.parametrize("delta", [False, True])
def test_scan_staging_does_not_change_the_sums(ops, delta):
    """A step in which no request has more than four rows stages fewer rows at a time; y and the
    state are bit for bit those of the long staging."""
    import dataclasses
    H, d, dv = 3, 24, 20
    g = torch.Generator().manual_seed(5)
    outs = []
    for known in (True, False):
        steps = Steps(ops, 3, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=torch.float32)
        state = steps.mgr.view(0).state["m"]
        g.manual_seed(5)
        ys = []
        for counts in ({"a": 4, "b": 1, "c": 3}, {"a": 2, "b": 4}, {"c": 1, "a": 1}):
            batch, _ = steps.step(counts)
            assert batch.max_q_len <= 4
            if not known:
                batch = dataclasses.replace(batch, max_q_len=0)
            n = batch.num_tokens
            q, k = torch.randn((n, H * d), generator=g).cuda(), torch.randn((n, H * d), generator=g).cuda()
            v, beta = torch.randn((n, H * dv), generator=g).cuda(), torch.randn((n, H), generator=g).cuda()
            y = torch.empty((n, H * dv), dtype=torch.float32, device="cuda")
            ops.matrix_state_scan(q, k, v, state, batch, y, H, H, d, dv, unit_eps=1e-6,
                                  beta=beta if delta else None, decay=torch.tensor([0.9, 1.0, 0.5]).cuda())
            ys.append(y.cpu())
        outs.append((torch.cat(ys), state.cpu().clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert outs[0][0].abs().max().item() > 0.1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("delta", [False, True])
def test_rows_made_ready_ahead_do_not_change_the_sums(ops, dtype, delta):
    """A long step has q, k and the decays of its rows computed once by a kernel of their own;
    y and the state are bit for bit those of the scan that computes them as it goes."""
    H, G, d, dv = (6, 3, 40, 24) if delta else (3, 3, 24, 20)
    outs = []
    for prepare in (True, False):
        steps = Steps(ops, 3, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=dtype)
        state = steps.mgr.view(0).state["m"]
        g = torch.Generator().manual_seed(11)
        dt_bias, a_log = 0.5 * torch.randn(H * d, generator=g), 0.7 * torch.randn(H, generator=g)
        ys = []
        for counts in ({"a": 37, "b": 5, "c": 20}, {"a": 2, "b": 33}):
            batch, _ = steps.step(counts)
            n = batch.num_tokens
            x = torch.randn((n, 2 * G * d + H * dv + 1), generator=g).to(dtype).cuda()
            beta = torch.randn((n, H), generator=g).to(dtype).cuda()
            a = torch.randn((n, H * d), generator=g).cuda()
            y = torch.empty((n, H * dv), dtype=torch.float32, device="cuda")
            q, k, v = x[:, :G * d], x[:, G * d:2 * G * d], x[:, 2 * G * d:-1]
            if delta:
                ops.matrix_state_scan(q, k, v, state, batch, y, H, G, d, dv, unit_eps=1e-6, q_scale=0.3,
                                      beta=beta, decay_logits=a, dt_bias=dt_bias.cuda(), a_log=a_log.cuda(),
                                      prepare=prepare)
            else:
                ops.matrix_state_scan(q, k, v, state, batch, y, H, G, d, dv, act_silu=True,
                                      decay=torch.tensor([0.9, 1.0, 0.5]).cuda(), prepare=prepare)
            ys.append(y.cpu())
        outs.append((torch.cat(ys), state.cpu().clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert outs[0][0].abs().max().item() > 0.1


def test_a_state_keeps_a_token_written_long_before(ops):
    """A key along one axis, written once, is read back 400 single-token steps later through a
    state that forgets nothing on that axis (decay 1), while every other token writes along other
    axes; with a decay below one on the second head the same token has faded to decay^400."""
    H, d, dv = 2, 8, 4
    steps = Steps(ops, 2, state=StateNeeds({"m": ((H, dv, d), torch.float32)}), dtype=torch.float32,
                  max_len=512)
    state = steps.mgr.view(0).state["m"]
    decay = torch.tensor([1.0, 0.99])
    g = torch.Generator().manual_seed(0)
    mark = torch.tensor([1.0, -2.0, 3.0, 0.5])
    out = None
    for t in range(402):
        batch, _ = steps.step({"a": 1, "b": 1} if t % 3 else {"a": 1})
        n = batch.num_tokens
        k = torch.zeros((n, H, d))
        k[:, :, 1:] = torch.randn((n, H, d - 1), generator=g)
        q, v = torch.randn((n, H, d), generator=g), torch.randn((n, H, dv), generator=g)
        if t == 1:
            k[0], v[0] = 0.0, mark
            k[0, :, 0] = 1.0
        if t == 401:
            q[0] = 0.0
            q[0, :, 0] = 1.0
        y = torch.empty((n, H * dv), dtype=torch.float32, device="cuda")
        ops.matrix_state_scan(q.reshape(n, -1).cuda(), k.reshape(n, -1).cuda(), v.reshape(n, -1).cuda(),
                              state, batch, y, H, H, d, dv, decay=decay.cuda())
        out = y[0].cpu().reshape(H, dv)
    assert (out[0] - mark).abs().max().item() < 1e-5
    assert (out[1] - mark * 0.99 ** 400).abs().max().item() < 1e-5


# ------------------------------------------------------------------ routers and experts
@pytest.mark.parametrize("shape", [(6, None, 2), (6, (3, 1), 2), (6, (3, 2), 3), (10, (5, 3), 4), (8, (8, 3), 3),
                                   (5, (1, 1), 5), (4, (2, 2), 1), (64, (8, 4), 8)])
def test_router_choice(ops, shape):
    n, groups, top = shape
    g = torch.Generator().manual_seed(n + top)
    T = 300
    z = torch.randn((T, n + 3), generator=g) * 1.5
    corr = torch.randn(n, generator=g) * 0.3 - 0.5        # mostly negative choice scores
    zc = z[:, 1:1 + n].contiguous().cuda()
    count, keep = groups or (1, 1)
    chosen, weight = ops.moe_router_select(zc, corr.cuda(), count, keep, top)
    want_c, want_w = plain.choose_experts(z[:, 1:1 + n].double(), corr.double(), groups, top)
    margin = plain.choice_margin(z[:, 1:1 + n].double(), corr.double(), groups, top)
    clear = margin > 1e-5
    assert clear.sum() > T - 5
    assert torch.equal(chosen.cpu().long().sort(-1).values[clear], want_c.sort(-1).values[clear])
    order = chosen.cpu().long()
    s = torch.softmax(z[:, 1:1 + n].double(), -1)
    assert (weight.cpu().double() - s.gather(1, order)).abs().max().item() < 1e-6
    # no correction: the plain softmax decides
    chosen, _ = ops.moe_router_select(zc, None, count, keep, top)
    want_c, _ = plain.choose_experts(z[:, 1:1 + n].double(), torch.zeros(n, dtype=torch.float64), groups, top)
    clear = plain.choice_margin(z[:, 1:1 + n].double(), torch.zeros(n, dtype=torch.float64), groups, top) > 1e-5
    assert torch.equal(chosen.cpu().long().sort(-1).values[clear], want_c.sort(-1).values[clear])


@pytest.mark.parametrize("tokens", [1, 3, 50, 200])
@pytest.mark.parametrize("shape", [(5, 1, 2, 24, (3, 2)), (3, 0, 1, 20, None), (4, 4, 3, 8, (2, 1)), (2, 3, 5, 16, None),
                                   (6, 3, 3, 40, (3, 2))])
@pytest.mark.parametrize("dtype", DTYPES)
def test_routed_experts_with_identity_experts(ops, dtype, shape, tokens):
    E, identity, top, ff, groups = shape
    raw = one_layer_model("channel_delta", delta(1, 1, 4, 4, 2), moe(E, identity, top, ff, groups), width=44)
    _, part, w = build_parts(raw, ops, dtype, tokens + E)
    g = torch.Generator().manual_seed(tokens + E)
    steps = Steps(ops, 1, dtype=dtype, max_len=256)
    batch, _ = steps.step({"a": tokens})
    x = torch.randn((tokens, 44), generator=g).to(dtype)
    if tokens == 200:             # most experts get no token at all, some a full tile and more
        first = []
        plain.moe_ff(x.double(), w, "l0", raw["layers"][0]["mlp"], first, 0.0)
        x[:150] = x[int(first[0].argmax())]
    got = part.forward(x.cuda(), batch)
    assert got.dtype == torch.float32
    margins = []
    want = plain.moe_ff(x.double(), w, "l0", raw["layers"][0]["mlp"], margins, 0.0)
    clear = margins[0] > (1e-4 if dtype == torch.float32 else 2e-2)
    assert clear.sum() * 10 >= 7 * tokens or tokens < 5
    err = (got.double().cpu() - want).abs().amax(1)
    assert err[clear].max().item() < tol(dtype, 3e-5, 6e-2) * max(1.0, want.abs().max().item()) if clear.any() else True


# ------------------------------------------------------------------ whole mixers over steps
def mixer_over_steps(ops, dtype, raw, seed, page_size=8):
    mixer, _, w = build_parts(raw, ops, dtype, seed)
    needs = mixer.cache_needs()
    steps = Steps(ops, 3, paged=needs.paged, state=needs.state, dtype=dtype, page_size=page_size)
    g = torch.Generator().manual_seed(seed)
    L, D = 60, raw["width"]
    seqs = {r: {"h": torch.randn((L, D), generator=g).to(dtype)} for r in "abc"}
    cache = steps.mgr.view(0)

    def run(batch, rows):
        y = mixer.forward(rows["h"], batch, cache, True)
        return y.sum(0) if y.dim() == 3 else y

    got = carry_over_steps(ops, steps, seqs, run, STEPS, D)
    ops.check_errors()
    return got, seqs, w


@pytest.mark.parametrize("sizes", [(4, 2, 12, 20, 3), (3, 1, 5, 7, 1), (2, 2, 64, 64, 4), (6, 6, 16, 8, 2)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_rule_mixer(ops, dtype, sizes):
    raw = one_layer_model("channel_delta", delta(*sizes), None)
    got, seqs, w = mixer_over_steps(ops, dtype, raw, sizes[2])
    for r in "abc":
        want = plain.channel_delta_mixer(seqs[r]["h"].double(), w, "l0", raw["layers"][0]["mixer"], 1e-5)
        ref = want[:len(got[r])]
        assert (got[r] - ref).abs().max().item() < tol(dtype, 3e-5, 5e-2) * max(1.0, ref.abs().max().item()), r


@pytest.mark.parametrize("sizes", [
    (window_attention(4, 2, 12, 20, 0.9, 9, rot=(8, 10000.0)), decayed(3, 10, 6, (0.5, 0.9, 0.99))),
    (window_attention(1, 1, 5, 3, 1.2, 1), decayed(1, 3, 5, (0.7,))),
    (window_attention(3, 3, 10, 6, 0.8), decayed(5, 2, 3, (0.3, 0.6, 0.9, 0.95, 1.0))),
    (window_attention(2, 1, 64, 64, 0.3, 20, rot=(64, 1e4)), decayed(2, 32, 16, (0.9, 0.999)))])
@pytest.mark.parametrize("dtype", DTYPES)
def test_two_mixers_side_by_side(ops, dtype, sizes):
    raw = one_layer_model("parallel", pair(*sizes), None)
    got, seqs, w = mixer_over_steps(ops, dtype, raw, 5)
    for r in "abc":
        want = plain.parallel_mixer(seqs[r]["h"].double(), w, "l0", raw["layers"][0]["mixer"], 1e-5)
        ref = want[:len(got[r])]
        assert (got[r] - ref).abs().max().item() < tol(dtype, 3e-5, 6e-2) * max(1.0, ref.abs().max().item()), r
