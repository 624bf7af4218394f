"""Dapozen's mechanisms one at a time: each kernel against the plain function of the same name.

Attention cases plant one dominating key (a key and one query are scaled so that its score
stands out) far back in a chunk, on either side of a chunk's edge and at page borders, in prompt
portions and in single-token steps; the recurrence is carried over several steps of unequal
requests; convolutions start inside a request's history and at its very beginning."""

import pytest
import torch

from somi_inference_b200.config.spec import PartSpec
from somi_inference_b200.parts import FEED_FORWARDS, BuildContext
from somi_inference_b200.parts.base import PagedKVNeeds, StateNeeds
from tests.gpu_util import Steps, gather_cache
from tests.plain import dapozen_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from somi_inference_b200.ops import cuda_ops
    return cuda_ops()


def tol(dtype, f32=2e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


# ------------------------------------------------------------------ embedding, norms, cap
@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding_and_soft_cap(ops, dtype):
    g = torch.Generator().manual_seed(1)
    table = torch.randn((50, 37), generator=g).to(dtype).cuda()
    ids = torch.randint(0, 50, (11,), generator=g).to(torch.int32).cuda()
    out = torch.empty((11, 37), dtype=torch.float32, device="cuda")
    ops.embed_scaled(ids, table, 2.5, out)
    assert torch.equal(out, table.float()[ids.long()] * 2.5)
    x = (torch.randn((7, 91), generator=g) * 30).cuda()
    want = 12.0 * torch.tanh(x.double() / 12.0)
    ops.softcap(x, 12.0)
    assert (x.double() - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("width", [48, 256, 1030, 37])
@pytest.mark.parametrize("dtype", DTYPES)
def test_sandwich_norm(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    T = 9
    res = torch.randn((T, width), generator=g).cuda()
    wb = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype).cuda()
    w = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype).cuda()
    for delta in (torch.randn((T, width), generator=g).to(dtype).cuda() * 4,
                  torch.randn((3, T, width), generator=g).cuda(), None):
        r = res.clone()
        out = torch.empty((T, width), dtype=dtype, device="cuda")
        ops.add_normed_rmsnorm(r, delta, wb if delta is not None else None, 1e-5, w, 1e-6, out)
        d = None if delta is None else (delta.double() if delta.dim() == 2 else delta.double().sum(0))
        want_r = res.double() if d is None else res.double() + plain.rms_norm(d, wb.double(), 1e-5)
        want = plain.rms_norm(want_r, w.double(), 1e-6)
        assert (r.double() - want_r).abs().max().item() < 1e-5
        assert (out.double() - want).abs().max().item() < tol(dtype, 1e-5)
        # chosen rows only: the residual stream stays as it is
        rows = torch.tensor([4, 0, 7], dtype=torch.int32, device="cuda")
        r2 = res.clone()
        out2 = torch.empty((3, width), dtype=dtype, device="cuda")
        ops.add_normed_rmsnorm(r2, delta, wb if delta is not None else None, 1e-5, w, 1e-6, out2, rows)
        assert torch.equal(r2, res)
        assert (out2.double() - want[rows.long()]).abs().max().item() < tol(dtype, 1e-5)


@pytest.mark.parametrize("groups", [1, 2, 6])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_group_norm(ops, dtype, groups):
    g = torch.Generator().manual_seed(groups)
    T, C = 5, 60
    y = torch.randn((T, C), generator=g).cuda() * 3
    wide = torch.randn((T, C + 9), generator=g).to(dtype).cuda()
    z = wide[:, 4:4 + C]
    w = (1 + 0.3 * torch.randn(C, generator=g)).to(dtype).cuda()
    out = torch.empty((T, C), dtype=dtype, device="cuda")
    ops.gated_group_rmsnorm(y, z, w, 1e-5, groups, out)
    want = plain.grouped_rms_norm(y.double() * plain.silu(z.double()), w.double(), groups, 1e-5)
    assert (out.double() - want).abs().max().item() < tol(dtype, 1e-5, 3e-2)


# ------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("taps", [1, 2, 4])
@pytest.mark.parametrize("dtype", DTYPES)
def test_causal_conv_over_steps(ops, dtype, taps):
    """Three steps of unequal requests (one arrives late, one brings single tokens): every
    step's rows equal the convolution over the whole sequence, from its very first token on."""
    g = torch.Generator().manual_seed(taps)
    C, wide = 23, 31
    state = None if taps == 1 else StateNeeds({"s": ((taps - 1, C), dtype)})
    steps = Steps(ops, 4, state=state, dtype=dtype)
    seqs = {r: torch.randn((40, wide), generator=g).to(dtype) for r in "abcd"}
    w = torch.randn((C, taps), generator=g)
    bias = torch.randn(C, generator=g)
    for use_bias, act in ((False, None), (True, "silu")):
        want = {r: plain.short_conv(s[:, 3:3 + C].double(), w.double(), bias.double() if use_bias else None)
                for r, s in seqs.items()}
        if act:
            want = {r: plain.silu(v) for r, v in want.items()}
        steps = Steps(ops, 4, state=state, dtype=dtype)
        st = steps.mgr.view(0).state.get("s")
        for counts in ({"a": 7, "b": 1, "c": 2}, {"a": 1, "b": 1, "c": 16, "d": 3}, {"d": 1, "a": 5, "b": 2}):
            batch, where = steps.step(counts)
            u = torch.zeros((batch.num_tokens, wide), dtype=dtype)
            for r, (first, q, c) in where.items():
                u[first:first + q] = seqs[r][c:c + q]
            u = u.cuda()
            out = torch.full((batch.num_tokens, C + 2), 7.0, dtype=dtype, device="cuda")
            ops.causal_conv(u[:, 3:], C, w.t().contiguous().cuda(), bias.cuda() if use_bias else None,
                            st, batch, out, act=act)
            for r, (first, q, c) in where.items():
                err = (out[first:first + q, :C].double().cpu() - want[r][c:c + q]).abs().max().item()
                assert err < tol(dtype, 1e-5, 5e-2), (r, counts, err)
            assert (out[:, C:] == 7.0).all()


# ------------------------------------------------------------------ rotation, unit norm, cache write
@pytest.mark.parametrize("geometry", [(3, 1, 12, 20, 8), (2, 2, 5, 3, 0), (4, 2, 32, 32, 32), (1, 1, 70, 6, 2)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_rotary_pairs_store(ops, dtype, geometry):
    nq, nkv, hd, vd, rot = geometry
    g = torch.Generator().manual_seed(hd)
    steps = Steps(ops, 3, paged=PagedKVNeeds(nkv, hd, None, vd if vd != hd else None), dtype=dtype,
                  page_size=4)
    batch, _ = steps.step({"a": 30, "b": 2})
    batch, where = steps.step({"a": 3, "b": 1, "c": 6})
    width = (nq + nkv) * hd + nkv * vd
    qkv0 = torch.randn((batch.num_tokens, width + 5), generator=g).to(dtype).cuda()
    qkv = qkv0.clone()
    inv = (77.0 ** (-torch.arange(0, max(rot, 2), 2, dtype=torch.float64) / max(rot, 2))).cuda()
    view = steps.mgr.view(0).paged
    group = batch.groups[0]
    ops.rotary_pairs_store(qkv, batch.positions, inv, nq, nkv, hd, vd, rot, True, 1e-5,
                           group.slot_map, view.keys, view.values)
    assert torch.equal(qkv[:, nq * hd:], qkv0[:, nq * hd:])          # k, v and what lies beside stay
    slots = group.slot_map.cpu()
    ps = steps.mgr.page_size
    for r, (first, q, c) in where.items():
        full = torch.zeros((c + q, width), dtype=torch.float64)
        full[c:] = qkv0[first:first + q, :width].double().cpu()
        qk = full[:, :(nq + nkv) * hd].reshape(c + q, nq + nkv, hd)
        if rot:
            qk = plain.rotate_pairs(qk, rot, 77.0)
        qk = plain.rms_norm(qk, None, 1e-5)[c:]
        got_q = qkv[first:first + q, :nq * hd].double().cpu().reshape(q, nq, hd)
        assert (got_q - qk[:, :nq]).abs().max().item() < tol(dtype, 1e-5)
        for i in range(q):
            page, off = int(slots[first + i]) // ps, int(slots[first + i]) % ps
            got_k = view.keys[page, :, off].double().cpu()
            got_v = view.values[page, :, off].double().cpu()
            assert (got_k - qk[i, nq:]).abs().max().item() < tol(dtype, 1e-5)
            assert torch.equal(got_v, full[c + i, (nq + nkv) * hd:].reshape(nkv, vd))


# ------------------------------------------------------------------ chunked attention
@pytest.mark.parametrize("case", [
    # (heads, kv heads, key width, value width, chunk, page size)
    (4, 2, 12, 20, 9, 8), (2, 1, 16, 16, 21, 4), (3, 3, 5, 3, 1, 4), (2, 2, 32, 8, 64, 16),
    (1, 1, 40, 40, 300, 16),
    # head sizes of the tensor-core kernels (bfloat16): the same mask as one signed number
    (4, 2, 64, 64, 96, 16), (8, 1, 128, 128, 300, 16), (4, 4, 128, 128, 50, 8), (2, 2, 64, 64, 5, 16)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_chunked_attention_with_planted_keys(ops, dtype, case):
    """Prompt portions and single tokens whose queries point at one scaled key each: the chunk's
    first key, the key just before the chunk (which must not be seen), the key a page border
    back, the token itself."""
    nq, nkv, hd, vd, chunk, ps = case
    g = torch.Generator().manual_seed(chunk)
    steps = Steps(ops, 6, paged=PagedKVNeeds(nkv, hd, chunk, vd if vd != hd else None), dtype=dtype,
                  page_size=ps, max_len=400)
    steps.step({"a": 130, "b": 2 * chunk + 3 if chunk < 100 else 77, "c": 1, "d": chunk})
    batch, where = steps.step({"a": 19, "b": 1, "c": 2, "d": 1, "e": 37, "f": 290})
    view = steps.mgr.view(0).paged
    for t in (view.keys, view.values):
        t.copy_(torch.randn(t.shape, generator=g).to(dtype))
    width = (nq + nkv) * hd + nkv * vd
    qkv = torch.randn((batch.num_tokens, width), generator=g).to(dtype)
    table = batch.groups[0].block_table.cpu()
    planted = []
    for j, r in enumerate(batch.host.requests):
        first, q, c = where[r]
        for i in range(q):
            p = c + i
            start = (p // chunk) * chunk
            target = [start, start - 1, p - p % ps - 1, p][(i + j) % 4]
            if target < 0:
                continue
            page = int(table[j, target // ps])
            if page < 0:          # given back: it lies before the chunk and must not be read anyway
                continue
            sign = torch.where(torch.randn(hd, generator=g) > 0, 1.0, -1.0)
            # a score of at most 100: far above the others, and its float32 rounding stays small
            view.keys[page, :, target % ps] = (min(6.0, 100.0 / (0.4 * hd)) * sign).to(dtype).cuda()
            qkv[first + i, :nq * hd] = sign.repeat(nq).to(dtype)
            planted.append((r, p, target))
    assert len(planted) > 10
    qkv = qkv.cuda()
    gate = torch.randn((batch.num_tokens, nq * vd + 3), generator=g).to(dtype).cuda()
    # every prompt kernel in turn: two query tiles per CTA, one, mma.sync fed by TMA, by cp.async
    # (sizes that none of them takes run the kernel for any size whatever the switches say)
    switches = [(True, 1, True, True), (False, 1, True, True), (False, 1, False, True),
                (False, 1, False, False)]
    saved = (ops.use_pp_prefill, ops.pp_prefill_min_ctas, ops.use_tc_prefill, ops.use_tma_prefill)
    for k, use_gate in enumerate((False, True, False, True)):
        out = torch.empty((batch.num_tokens, nq * vd), dtype=dtype, device="cuda")
        ops.use_pp_prefill, ops.pp_prefill_min_ctas, ops.use_tc_prefill, ops.use_tma_prefill = switches[k]
        try:
            ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], nq, nkv, hd, 0.4,
                                None, out, storage=view.storage, value_dim=vd, chunk=chunk,
                                gate=gate[:, :nq * vd] if use_gate else None)
        finally:
            ops.use_pp_prefill, ops.pp_prefill_min_ctas, ops.use_tc_prefill, ops.use_tma_prefill = saved
        ops.check_errors()
        for j, r in enumerate(batch.host.requests):
            first, q, c = where[r]
            keys, values = gather_cache(view, table[j], c + q, ps)
            qs = torch.zeros((c + q, nq, hd), dtype=torch.float64)
            qs[c:] = qkv[first:first + q, :nq * hd].double().cpu().reshape(q, nq, hd)
            want = plain.chunked_softmax_attention(qs, keys, values, 0.4, chunk)[c:].reshape(q, nq * vd)
            if use_gate:
                want = want * torch.sigmoid(gate[first:first + q, :nq * vd].double().cpu())
            err = (out[first:first + q].double().cpu() - want).abs().max().item()
            assert err < tol(dtype, 4e-5, 4e-2), (r, c, q, err)


# ------------------------------------------------------------------ the recurrence
@pytest.mark.parametrize("geometry", [(3, 10, 12, 1), (4, 6, 40, 2), (1, 5, 70, 1), (8, 16, 128, 4), (2, 7, 3, 2),
                                      (2, 20, 300, 1)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_state_space_recurrence_over_steps(ops, dtype, geometry):
    heads, P, N, G = geometry
    g = torch.Generator().manual_seed(N)
    inner, wide = heads * P, heads * P + 2 * G * N
    steps = Steps(ops, 3, state=StateNeeds({"m": ((heads, P, N), torch.float32)}), dtype=dtype)
    L = 60
    xbc = {r: torch.randn((L, wide), generator=g).to(dtype) for r in "abc"}
    dt = {r: torch.randn((L, heads + 2), generator=g).to(dtype) for r in "abc"}
    dt_bias, a_log, skip = (torch.randn(heads, generator=g) * 0.5 for _ in range(3))
    want = {}
    for r in "abc":
        x64 = xbc[r].double()
        want[r] = plain.ssm_scan(x64[:, :inner].reshape(L, heads, P),
                                 plain.softplus(dt[r][:, 1:1 + heads].double() + dt_bias.double()),
                                 a_log.double(), x64[:, inner:inner + G * N].reshape(L, G, N),
                                 x64[:, inner + G * N:].reshape(L, G, N), skip.double()).reshape(L, inner)
    state = steps.mgr.view(0).state["m"]
    for counts in ({"a": 9, "b": 1}, {"a": 1, "b": 1, "c": 30}, {"c": 1, "a": 2, "b": 40}, {"a": 1, "c": 1}):
        batch, where = steps.step(counts)
        xs = torch.zeros((batch.num_tokens, wide), dtype=dtype)
        ds = torch.zeros((batch.num_tokens, heads + 2), dtype=dtype)
        for r, (first, q, c) in where.items():
            xs[first:first + q] = xbc[r][c:c + q]
            ds[first:first + q] = dt[r][c:c + q]
        xs, ds = xs.cuda(), ds.cuda()
        y = torch.empty((batch.num_tokens, inner), dtype=torch.float32, device="cuda")
        ops.ssm_scan(xs, ds[:, 1:1 + heads], dt_bias.cuda(), a_log.cuda(), skip.cuda(), state, batch, y,
                     heads, G, N, P)
        for r, (first, q, c) in where.items():
            ref = want[r][c:c + q]
            err = (y[first:first + q].double().cpu() - ref).abs().max().item()
            assert err < 2e-5 * max(1.0, ref.abs().max().item()), (r, counts, err)


# ------------------------------------------------------------------ experts by table
@pytest.mark.parametrize("tokens", [1, 3, 50, 200])
@pytest.mark.parametrize("shape", [(5, 2, 24, 16), (3, 1, 20, None), (9, 9, 7, 5)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_table_routed_experts(ops, dtype, shape, tokens):
    E, top, ff, shared_ff = shape
    H, vocab = 44, 31
    g = torch.Generator().manual_seed(tokens + E)
    mlp = {"expert": {"ff": ff, "limit": 1.5}, "router": {"experts": E, "top": top}}
    names = {"table": "m.mlp.table", "gate": [f"m.mlp.e{e}.gate" for e in range(E)],
             "up": [f"m.mlp.e{e}.up" for e in range(E)], "down": [f"m.mlp.e{e}.down" for e in range(E)],
             "shared_gate": "m.mlp.shared.gate", "shared_up": "m.mlp.shared.up",
             "shared_down": "m.mlp.shared.down"}
    params = {"hidden_size": H, "vocab_size": vocab, "experts": E, "top": top, "expert_ff": ff,
              "limit": 1.5, "alpha": 1.702, "shared": None, "names": names}
    if shared_ff:
        mlp["shared"] = params["shared"] = {"ff": shared_ff, "limit": 0.8}
    spec = PartSpec("table_moe", params)
    w = {}
    for d in FEED_FORWARDS.declare(spec):
        if d.name.endswith("table"):
            w[d.name] = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(vocab)]).to(torch.int32)
        else:
            w[d.name] = (torch.randn(d.shape, generator=g) * (1.6 / d.shape[1] ** 0.5)).to(dtype)
    ctx = BuildContext(dtype=dtype, device=torch.device("cuda"), ops=ops)
    part = FEED_FORWARDS.build(spec, {k: ctx.place(v, matrix=True) for k, v in w.items()}, ctx)
    steps = Steps(ops, 1, dtype=dtype, max_len=256)
    batch, _ = steps.step({"a": tokens})
    ids = torch.randint(0, vocab, (tokens,), generator=g)
    if tokens == 200:
        ids[:150] = 7          # most experts get no token at all, some a full tile and more
    batch.token_ids.copy_(ids.to(torch.int32))
    x = torch.randn((tokens, H), generator=g).to(dtype)
    got = part.forward(x.cuda(), batch)
    want = plain.table_moe_ff(x.double(), ids, {k: (v.double() if v.is_floating_point() else v)
                                               for k, v in w.items()}, "m", mlp)
    assert got.dtype == torch.float32
    assert (got.double().cpu() - want).abs().max().item() < tol(dtype, 3e-5, 6e-2)
