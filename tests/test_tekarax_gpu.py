"""Tekarax on the GPU: every new mechanism alone against the plain implementation's function for it, each mixer alone
through the package's cache manager and step context (batches of unequal entries, portions, slots and pages used
again), then the engine through the replay loop and through ``Engine.generate`` against the plain implementation of
the whole model, in 32-bit and in bfloat16, for four small configurations that differ in every size and option."""

import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import tekarax_helpers as TH
from plain import tekarax_plain as TP

pytestmark = pytest.mark.gpu

BOTH = [torch.float32, torch.bfloat16]
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from pyre_b200.kernels import build, ops as o
    build.ensure_built(["wkv", "blockops", "grouped", "elementwise", "gemm_f32", "gemm_tc", "attention_generic", "attention_mma",
                        "attention_prefill", "attention_tc", "latent_attention"])
    return o


def close(got, want, dtype, what="", atol32=3e-6, rel16=1.6e-2):
    tol = dict(rtol=3e-5, atol=atol32) if dtype == torch.float32 else dict(rtol=rel16, atol=rel16)
    torch.testing.assert_close(got.double().cpu(), want.double().cpu(), msg=lambda m: f"{what}: {m}", **tol)


def close_part(got, want, dtype, what="", roundings=4):
    """A whole part: the largest error against the size of its output.  float32: sums in another order, 1e-5 of the
    largest output.  bfloat16: every tensor that the part rounds on the way (``roundings`` of them) may be off by
    2^-8 relative."""
    bound = (1e-5 if dtype == torch.float32 else roundings * 2.0 ** -8) * float(want.abs().max())
    err = float((got.double().cpu() - want.double()).abs().max())
    assert err <= bound, f"{what}: max error {err:.3e} > {bound:.3e} (largest output {float(want.abs().max()):.3f})"


def bf16_exact(*shape, scale=1.0, seed=0):
    """Random fp64 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).double()


# --------------------------------------------------------------------------- the small kernels, each alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("Hn,d,W", [(3, 16, 40), (2, 20, 92), (4, 32, 96), (2, 64, 128), (1, 128, 72), (5, 24, 33)])
def test_blend_and_recurrence_over_state_slots(ops, dtype, Hn, d, W):
    """Entries of unequal lengths in one launch (a single token, two tokens, a long portion), cut into two steps,
    over state slots in scrambled order: every token against the plain recurrence run over
    the whole sequence.  One channel of one head decays almost at once and one almost never, and the bonus of one
    head is large: a state that is lost, a decay applied before the output, or a bonus that leaks into the state shows
    at once."""
    lens = [[1, 7, 2, 40], [3, 1, 30, 2]]          # tokens of the four requests in step one and step two
    n_req, n_slots, HD = 4, 6, Hn * d
    floats = ops.wkv_state_floats(Hn, d, W)
    state = torch.zeros(n_slots, floats, dtype=torch.float32, device="cuda")
    slots = [4, 0, 5, 2]
    u = bf16_exact(Hn, d, scale=0.5, seed=1)
    u[0] = 3.0
    w0 = bf16_exact(HD, scale=0.7, seed=2) - 1.0
    w0[0], w0[1] = 3.0, -9.0                       # decay exp(-e^3): gone after a token; exp(-e^-9): kept
    norm_w = bf16_exact(HD, scale=0.1, seed=3) + 1.0
    mu = bf16_exact(5, W, scale=0.2, seed=4) + 0.5
    total = [sum(l[b] for l in lens) for b in range(n_req)]
    seq = [dict(h=bf16_exact(total[b], W, seed=10 + b), r=bf16_exact(total[b], HD, seed=20 + b), k=bf16_exact(total[b], HD, scale=0.5, seed=30 + b),
                v=bf16_exact(total[b], HD, seed=40 + b), g=bf16_exact(total[b], HD, seed=50 + b),
                dlog=bf16_exact(total[b], HD, scale=0.8, seed=60 + b)) for b in range(n_req)]
    want_mix, want_out = [], []
    for b in range(n_req):
        s = seq[b]
        want_mix.append(torch.stack([TP.token_blend(s["h"], mu[i]) for i in range(5)]))
        decay = torch.exp(-torch.exp(s["dlog"] + w0)).view(-1, Hn, d)
        o, S_end = TP.wkv_recurrence(s["r"].view(-1, Hn, d), s["k"].view(-1, Hn, d), s["v"].view(-1, Hn, d), decay, u)
        s["S_end"] = S_end
        want_out.append(TP.unit_rms(o, 1e-5).reshape(-1, HD) * norm_w * TP.silu(s["g"]))
    at = [0] * n_req
    for step in lens:
        cu = torch.tensor([0] + list(np.cumsum(step)), dtype=torch.int32, device="cuda")
        seq_of = torch.tensor(sum(([b] * n for b, n in enumerate(step)), []), dtype=torch.int32, device="cuda")
        cat = lambda key, dt: torch.cat([seq[b][key][at[b]:at[b] + n] for b, n in enumerate(step)]).to(dt).cuda()
        h = cat("h", dtype)
        sl = torch.tensor(slots, dtype=torch.int32, device="cuda")
        x = ops.token_shift_mix(h, state, Hn * d * d, sl, seq_of, cu, mu.float().cuda())
        wm = torch.cat([want_mix[b][:, at[b]:at[b] + n] for b, n in enumerate(step)], dim=1)
        close(x, wm, dtype, "blends", atol32=2e-6)
        out = ops.wkv_scan(cat("r", dtype), cat("k", dtype), cat("v", dtype), cat("g", dtype), cat("dlog", torch.float32), w0.float().cuda(),
                           u.reshape(-1).float().cuda(), norm_w.float().cuda(), state, Hn * d * d, sl, cu, h, Hn, d, 1e-5)
        wo = torch.cat([want_out[b][at[b]:at[b] + n] for b, n in enumerate(step)])
        close(out, wo, dtype, "recurrence", atol32=2e-5, rel16=2e-2)
        at = [a + n for a, n in zip(at, step)]
    for b in range(n_req):
        close(state[slots[b], :Hn * d * d], seq[b]["S_end"].reshape(-1), torch.float32, "state left in the slot", atol32=2e-5)
        close(state[slots[b], Hn * d * d:Hn * d * d + W], seq[b]["h"][-1], torch.float32, "last input row")
    assert (state[[1, 3]] == 0).all(), "a slot of no request was written"


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,Hn,parts,gated,bias,center", [(1, 96, 0, True, False, True), (5, 92, 0, True, True, True), (37, 1024, 3, True, False, True),
                                                          (3, 4100, 2, False, True, True), (9, 128, 0, True, False, False)])
def test_gated_norm_of_a_sublayers_result(ops, dtype, T, Hn, parts, gated, bias, center):
    y = bf16_exact(max(parts, 1), T, Hn, seed=1)
    gate, gb, yb, w = bf16_exact(T, Hn, seed=2), bf16_exact(Hn, seed=3), bf16_exact(Hn, seed=4), bf16_exact(Hn, scale=0.2, seed=5) + 1
    v = y.sum(0) + (yb if bias else 0)
    if gated:
        v = v * torch.sigmoid(gate + gb)
    want = TP.layer_norm(v, w, 1e-5) if center else TP.unit_rms(v, 1e-5) * w
    src = ops.PartialSums(y.float().cuda(), dtype) if parts else y[0].to(dtype).cuda()
    got = ops.gated_norm(src, yb.float().cuda() if bias else None, gate.to(dtype).cuda() if gated else None,
                         gb.float().cuda() if gated else None, w.float().cuda(), 1e-5, dtype, center=center)
    assert got.dtype == torch.float32
    close(got, want, torch.float32, "gated norm", atol32=2e-5)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("kind,fn", [("relu2", TP.relu2), ("tanh", torch.tanh), ("silu", TP.silu), (None, lambda z: z)])
@pytest.mark.parametrize("T,Hn", [(7, 50), (3, 320), (1, 67)])
def test_bias_and_activation(ops, dtype, kind, fn, T, Hn):
    x, b = bf16_exact(T, Hn, scale=2.0, seed=6), bf16_exact(Hn, seed=7)
    close(ops.bias_act(x.to(dtype).cuda(), b.float().cuda(), kind), fn(x + b), dtype, str(kind), atol32=1e-5)
    close(ops.bias_act(x.to(dtype).cuda(), None, kind), fn(x), dtype, f"{kind}, no bias", atol32=1e-5)


def test_vector_added_to_every_row_of_the_stream(ops):
    for T, Hn in ((1, 96), (13, 92), (5, 2048)):
        x, v = torch.randn(T, Hn, device="cuda"), torch.randn(Hn, device="cuda")
        want = x + v
        assert ops.add_row_vector(x, v) is x and torch.equal(x, want)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("nh,nkv,dk,dv,rot,page", [(4, 2, 16, 24, 8, 16), (5, 5, 20, 12, 12, 8), (8, 2, 64, 64, 64, 32), (6, 1, 128, 64, 32, 16)])
def test_values_turn_with_their_position_and_sums_turn_back(ops, dtype, nh, nkv, dk, dv, rot, page):
    """The write: queries and keys turn over their leading dims by stretched frequencies, values over all their dims
    by plain ones, and are cached so.  The gate kernel: a head's sum is turned by minus the token's own angles, then
    one gate per head.  A value that is cached at position j and read back at position j comes out as it was."""
    T, n_pages, base = 9, 6, 500.0
    pos = torch.tensor([0, 1, 2, 3, 77, 78, 500, 511, 600])
    row = ops.attention_row_dim(dk, dv, dtype)
    W = nh * dk + nkv * dk + nkv * dv + nh
    proj = bf16_exact(T, W, seed=11)
    scaling = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    fq, fv = TP.scaled_frequencies(base, rot, scaling), TP.scaled_frequencies(base, dv)
    cos, sin = ops.rope_table(pos.int().cuda(), fq.float().cuda())
    vcos, vsin = ops.rope_table(pos.int().cuda(), fv.float().cuda())
    slots = torch.randperm(page * n_pages, generator=torch.Generator().manual_seed(dk))[:T]
    cache = torch.full((n_pages, 2, nkv, page, row), 7.0, dtype=dtype, device="cuda")
    k_col, v_col, g_col = nh * dk, nh * dk + nkv * dk, nh * dk + nkv * dk + nkv * dv
    q = ops.qk_norm_rope_write(proj.to(dtype).cuda(), 0, k_col, v_col, None, None, 0.0, cos, sin, cache, slots.int().cuda(), nh, nkv, dk, dv,
                               row, rot, page, v_cos=vcos, v_sin=vsin)
    tol = dict(atol32=3e-4)      # angles are fp32 in the engine: 600 x 2^-24 of error
    close(q.view(T, nh, row)[..., :dk], TP.rotate_halves(proj[:, :k_col].view(T, nh, dk), pos, fq), dtype, "queries", **tol)
    assert (q.view(T, nh, row)[..., dk:] == 0).all()
    pg, off = (slots // page).cuda(), (slots % page).cuda()
    close(cache[pg, 0, :, off, :dk], TP.rotate_halves(proj[:, k_col:v_col].view(T, nkv, dk), pos, fq), dtype, "cached keys", **tol)
    want_v = TP.rotate_halves(proj[:, v_col:g_col].view(T, nkv, dv), pos, fv)
    close(cache[pg, 1, :, off, :dv], want_v, dtype, "cached values", **tol)
    assert (cache[pg, 0, :, off, dk:] == 0).all() and (cache[pg, 1, :, off, dv:] == 0).all(), "the rest of a row is zero"
    untouched = torch.ones(page * n_pages, dtype=torch.bool)
    untouched[slots] = False
    assert (cache.permute(0, 3, 1, 2, 4).reshape(page * n_pages, -1)[untouched.cuda()] == 7.0).all(), "a row of no token was written"
    # the way back, with one gate per head
    a = bf16_exact(T, nh, row, seed=12)
    want = TP.rotate_halves(a[..., :dv], pos, fv, sign=-1.0) * torch.sigmoid(proj[:, g_col:])[:, :, None]
    got = ops.head_gate(a.reshape(T, nh * row).to(dtype).cuda(), row, proj.to(dtype).cuda(), g_col, nh, dv, vcos, vsin)
    close(got.view(T, nh, dv), want, dtype, "turned back and gated", **tol)
    got = ops.head_gate(a.reshape(T, nh * row).to(dtype).cuda(), row, None, 0, nh, dv, None, None)
    close(got.view(T, nh, dv), a[..., :dv], dtype, "narrowed only")
    back = ops.head_gate(cache[pg, 1, :, off, :].reshape(T, nkv * row).contiguous(), row, None, 0, nkv, dv, vcos, vsin)
    close(back.view(T, nkv, dv), proj[:, v_col:g_col].view(T, nkv, dv), dtype, "there and back", **tol)


def plain_paged_attention_with_sinks(q, cache, table, seq_of_token, positions, nh, nkv, D, scale, sinks):
    page = cache.shape[3]
    out = torch.zeros(q.shape, dtype=F64)
    c = cache.double()
    for t in range(q.shape[0]):
        b, p = int(seq_of_token[t]), int(positions[t])
        at = torch.arange(p + 1)
        pages = table[b].long()[at // page]
        keys, vals = c[pages, 0, :, at % page], c[pages, 1, :, at % page]      # [keys, nkv, D]
        for n in range(nh):
            s = (keys[:, n // (nh // nkv)] @ q[t].double().view(nh, D)[n]) * scale
            out[t, n * D:(n + 1) * D] = TP.softmax_with_sink(s, sinks[n]) @ vals[:, n // (nh // nkv)]
    return out


@pytest.mark.parametrize("nh,nkv,D,page", [(4, 2, 64, 16), (6, 1, 128, 8), (5, 5, 32, 16)])
def test_a_learned_sink_per_head_in_every_attention_kernel(ops, nh, nkv, D, page):
    """Prompt portions beside decoded tokens in one step; the heads' sinks differ widely (one so low that it changes
    nothing, one so high that it takes most of every row), so a kernel that reads another head's sink, scales it, or
    leaves it out of one of its partial sums is off by the whole output."""
    from pyre_b200.engine.context import StepContext
    g = torch.Generator(device="cuda").manual_seed(D + page)
    ctx_lens, new = [300, 100, 64, 200, 40, 1], [130, 100, 64, 1, 20, 1]
    B = len(new)
    n_pages = sum(-(-c // page) for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(2)).tolist()
    table = torch.full((B, max(-(-c // page) for c in ctx_lens)), -1, dtype=torch.int32)
    for s_, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s_, lp] = perm.pop()
    cache16 = torch.randn(n_pages, 2, nkv, page, D, device="cuda", generator=g).to(torch.bfloat16)
    seq_of_token = torch.tensor(sum(([s_] * n for s_, n in enumerate(new)), []), dtype=torch.int32)
    positions = torch.tensor(sum((list(range(c - n, c)) for c, n in zip(ctx_lens, new)), []), dtype=torch.int32)
    cu_host = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    T = int(seq_of_token.shape[0])
    q16 = (torch.randn(T, nh * D, device="cuda", generator=g) * 1.5).to(torch.bfloat16)
    scale = 0.9 * D ** -0.5
    sinks = torch.linspace(-2.0, 2.0, nh, dtype=F64)
    sinks[0], sinks[-1] = -40.0, 9.0
    want = plain_paged_attention_with_sinks(q16.cpu(), cache16.cpu(), table, seq_of_token, positions, nh, nkv, D, scale, sinks)
    none = plain_paged_attention_with_sinks(q16.cpu(), cache16.cpu(), table, seq_of_token, positions, nh, nkv, D, scale, [None] * nh)
    assert (want[:, :D] - none[:, :D]).abs().max() < 1e-9 and (want[:, -D:].abs().max() < 0.2 * none[:, -D:].abs().max())
    sink_d = sinks.float().cuda()
    table_d, seq_d, pos_d, cu = table.cuda(), seq_of_token.cuda(), positions.cuda(), torch.from_numpy(cu_host).cuda()

    def check(got, rows, what):
        assert torch.isfinite(got[rows]).all(), what
        err = (got[rows].double().cpu() - want[rows]).abs()
        bad = (err > 1.2e-2 + 1.6e-2 * want[rows].abs()).any(dim=1)
        assert not bad.any(), f"{what}: first wrong row {int(torch.where(bad)[0][0])}, max error {float(err.max()):.3e}"

    z = torch.zeros(T, dtype=torch.int32, device="cuda")
    ctx = StepContext(dtype=torch.bfloat16, device=torch.device("cuda"), num_tokens=T, num_seqs=B, num_logit_rows=0,
                      token_ids=z, positions=pos_d, seq_of_token=seq_d, cu_seqlens=cu, logit_rows=z[:0],
                      cu_seqlens_host=cu_host, start_pos_host=np.asarray([c - n for c, n in zip(ctx_lens, new)]))
    everything, long_rows = slice(0, T), slice(0, 294)
    check(ops.paged_attention_bf16(ctx, q16, cache16, table_d, nh, nkv, D, scale, None, sink=sink_d), everything, "dispatch")
    if D in ops.PREFILL_HEAD_DIMS:
        out = torch.full_like(q16, 7.0)
        ops.attention_prefill(q16, cache16, table_d, cu, pos_d, B, 294, nh, nkv, D, scale, None, out, sink=sink_d)
        check(out, long_rows, "mma.sync prompt kernel")
        for splits in (1, 3):
            out = torch.full_like(q16, 7.0)
            ops.attention_prefill_tc(q16, cache16, table_d, cu, pos_d, B, 294, nh, nkv, D, scale, None, out, 64, splits, sink=sink_d)
            check(out, long_rows, f"tcgen05 prompt kernel, {splits} share(s) of the keys")
    for splits, scratch in ((1, None), (4, None), (5, "scratch")):
        out = torch.full_like(q16, 7.0)
        sc = torch.empty(T * nh * splits * (D + 2), dtype=torch.float32, device="cuda") if scratch else None
        ops.paged_attention_mma(q16, cache16, table_d, cu, pos_d, B, nh, nkv, D, scale, None, splits, out=out, scratch=sc, sink=sink_d)
        check(out, everything, f"split-KV kernel, {splits} split(s){' through scratch' if scratch else ''}")
    check(ops.paged_attention_generic(q16, cache16, table_d, seq_d, pos_d, nh, nkv, D, scale, None, sink=sink_d), everything, "exact kernel, bf16 storage")
    got32 = ops.paged_attention_generic(q16.float(), cache16.float(), table_d, seq_d, pos_d, nh, nkv, D, scale, None, sink=sink_d)
    torch.testing.assert_close(got32.double().cpu(), want, rtol=2e-5, atol=2e-6)
    ops.check_device_errors()


# --------------------------------------------------------------------------- the feed-forwards, each alone
def load_part_from(part, w, prefix, dtype):
    from pyre_b200.parts.base import collect_tensors, load_part
    tensors = {}
    for name, spec in collect_tensors(part).items():
        t = w[prefix + name]
        tensors[name] = t.to(torch.float32 if spec.role == "vector" else dtype).cuda()
    load_part(part, tensors)
    return part


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("mma", [False, True])
@pytest.mark.parametrize("T,Hn,ff,E,top,shared", [(1, 96, 64, 5, 2, 48), (77, 92, 24, 3, 3, 0), (300, 256, 128, 8, 2, 256), (9, 64, 32, 4, 1, 0),
                                                  (40, 128, 16, 1, 1, 64), (700, 128, 192, 16, 1, 128)])
def test_experts_that_read_weighted_inputs(ops, dtype, mma, T, Hn, ff, E, top, shared, monkeypatch):
    """Sigmoid scores (each output's own, so they do not sum to one), the ``top`` largest chosen, the weight on the
    expert's INPUT (a gated expert is not linear, so a weight on its output gives another result), no
    renormalising, a shared expert for every token; inputs are drawn again until no choice is a close call."""
    from pyre_b200.parts.base import PartSpec, make_part
    monkeypatch.setattr(ops, "USE_GROUPED_MMA", mma)
    mlp = {"router": {"experts": E, "top": top}}
    for seed in range(50):
        w = {"p.router": bf16_exact(E, Hn, scale=0.15, seed=seed)}
        h = bf16_exact(T, Hn, seed=seed + 200)
        ranked = TP.router_scores(h, w, "p.").sort(dim=-1, descending=True).values
        margins = (ranked[:, top - 1] - ranked[:, top]).tolist() if top < E else []
        if not margins or min(margins) > 2e-3:
            break
    for e in range(E):
        w[f"p.e{e}.gate"], w[f"p.e{e}.up"], w[f"p.e{e}.down"] = (bf16_exact(ff, Hn, scale=0.12, seed=7 * e + 1), bf16_exact(ff, Hn, scale=0.12, seed=7 * e + 2),
                                                                bf16_exact(Hn, ff, scale=0.12, seed=7 * e + 3))
    if shared:
        mlp["shared"] = {"ff": shared}
        w["p.shared.gate"], w["p.shared.up"], w["p.shared.down"] = (bf16_exact(shared, Hn, scale=0.1, seed=91), bf16_exact(shared, Hn, scale=0.1, seed=92),
                                                                    bf16_exact(Hn, shared, scale=0.1, seed=93))
    hd = h.to(dtype).cuda()
    idx, wt = ops.route(hd, w["p.router"].float().cuda(), None, top, 1.0, sigmoid=True)
    scores = TP.router_scores(h, w, "p.")
    pick = scores.topk(top, dim=-1).indices
    assert torch.equal(idx.cpu().long().sort(-1).values, pick.sort(-1).values), "the chosen experts"
    close(wt.cpu().gather(-1, idx.cpu().long().argsort(-1)), scores.gather(-1, pick.sort(-1).values), torch.float32, "weights: the plain scores", atol32=1e-6)
    offsets, place_of, _src = ops.group_pairs(idx, E)
    x = ops.scale_to_places(hd, place_of, wt, T * top)
    want_x = torch.zeros(T * top, Hn, dtype=F64)
    po = place_of.cpu().long()
    for t in range(T):
        for k in range(top):
            want_x[po[t, k]] = wt[t, k].double().cpu() * h[t]
    close(x, want_x, dtype, "weighted inputs by place", atol32=1e-6)
    part = make_part("ffn", PartSpec("routed_mlp", {"width": Hn, "intermediate": ff, "n_experts": E, "top": top, "correction": False,
                                                    "scores": "sigmoid", "weight_on": "input", "shared": shared or None}), dtype, "cuda")
    got = ops.materialize(load_part_from(part, w, "p.", dtype).forward(None, hd))
    want = TP.moe_mlp(h, w, "p.", mlp)
    close_part(got, want, dtype, "routed feed-forward", roundings=5)      # weighted input, gate and up, activation, result, shared
    if top < E or E == 1:      # the other reading (weights on outputs) is a different function on these inputs
        other = sum(scores[:, e:e + 1] * TP.gated_expert(h, w, f"p.e{e}.") * (pick == e).any(-1, keepdim=True) for e in range(E))
        assert (other + (TP.gated_expert(h, w, "p.shared.") if shared else 0) - want).abs().max() > 0.1 * want.abs().max()


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,Hn,ff", [(1, 96, 160), (33, 92, 66), (200, 256, 512), (5, 128, 72)])
def test_dense_feed_forward_with_biases_and_squared_relu(ops, dtype, T, Hn, ff):
    from pyre_b200.parts.base import PartSpec, make_part
    w = {"p.up": bf16_exact(ff, Hn, scale=0.2, seed=1), "p.up.b": bf16_exact(ff, scale=0.5, seed=2), "p.down": bf16_exact(Hn, ff, scale=0.2, seed=3),
         "p.down.b": bf16_exact(Hn, scale=0.5, seed=4)}
    h = bf16_exact(T, Hn, seed=5)
    part = make_part("ffn", PartSpec("dense_mlp", {"width": Hn, "intermediate": ff, "activation": "relu2", "bias": True,
                                                   "names": {"up": "up", "down": "down", "up_bias": "up.b", "down_bias": "down.b"}}), dtype, "cuda")
    got = ops.materialize(load_part_from(part, w, "p.", dtype).forward(None, h.to(dtype).cuda()))
    close_part(got, TP.dense_mlp(h, w, "p."), dtype, "dense feed-forward", roundings=3)


# --------------------------------------------------------------------------- each mixer alone, through the cache manager
def run_mixer_alone(tmp_path, layer, width, eps, dtype, page, steps, inputs, seed=0):
    """A model of this one layer is loaded (registry, loader, cache and state groups as ever), and its MIXER is called
    with inputs of the test's own on the step contexts that the package's stepper builds for ``steps`` (lists of
    (request, tokens) per step; a request begins at its first entry and ends after its last).  Returns the mixer's
    rows per request and the weights."""
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import ops
    from pyre_b200.models.model import load_model
    from safetensors.torch import load_file
    raw = {"architecture": "Tekarax", "vocab": 32, "width": width, "norm": {"eps": eps}, "layers": [dict(layer, mlp=None)]}
    TH.make_tekarax_dir(tmp_path, raw, seed=seed)
    model, _ = load_model(tmp_path, "cuda", dtype)
    as_trace = [{"entries": [{"id": r, "tokens": [0] * n} for r, n in st],
                 "end": [r for r, _ in st if all(r != x for later in steps[i + 1:] for x, _ in later)]} for i, st in enumerate(steps)]
    cache, stepper = runtime_for_model(model, H.max_live_tokens(as_trace), page, max_requests=max(len(st) for st in steps), poison=True,
                                       cuda_graphs=False)
    mixer, call = model.blocks[0].mixer, model.calls[0]
    at, out = {}, {}
    for i, step in enumerate(steps):
        for r, _ in step:
            if r not in at:
                cache.begin(r)
                at[r], out[r] = 0, []
        ctx = stepper.build_context([StepEntry(r, [0] * n, []) for r, n in step])
        h = torch.cat([inputs[r][at[r]:at[r] + n] for r, n in step]).to(model.dtype).cuda()
        rows = ops.materialize(mixer.forward(ctx, h, call)).float().cpu()
        k = 0
        for (r, n), new_len in zip(step, ctx.new_lens):
            cache.commit(r, new_len)
            out[r].append(rows[k:k + n])
            at[r], k = at[r] + n, k + n
        later = {x for st in steps[i + 1:] for x, _ in st}
        for r, _ in step:
            if r not in later:
                cache.end(r)
    ops.check_device_errors()
    cache.check()
    assert not cache.live()
    return {r: torch.cat(v) for r, v in out.items()}, load_file(str(tmp_path / "model.safetensors"))


def mixer_schedule(lengths, seed):
    """Steps of up to three live requests: a first portion, then portions of 2 to 9 tokens or single tokens, until
    each request has had all of its tokens; six requests in all, so slots and pages are used again."""
    rng = np.random.default_rng(seed)
    waiting, live, left, steps = list(lengths.items()), [], {}, []
    while waiting or live:
        while waiting and len(live) < 3:
            r, n = waiting.pop(0)
            live.append(r)
            left[r] = n
        step = []
        for r in list(live):
            n = min(left[r], int(rng.choice([1, 1, 2, 5, 9, 30])))
            step.append((r, n))
            left[r] -= n
            if not left[r]:
                live.remove(r)
        steps.append(step)
    return steps


MIXER_LENGTHS = {"a": 1, "b": 2, "c": 50, "d": 33, "e": 90, "f": 17}


def check_mixer(tmp_path, layer, width, eps, dtype, page, plain, seed):
    inputs = {r: bf16_exact(n, width, seed=seed + i) for i, (r, n) in enumerate(MIXER_LENGTHS.items())}
    got, w = run_mixer_alone(tmp_path, layer, width, eps, dtype, page, mixer_schedule(MIXER_LENGTHS, seed), inputs, seed)
    for r, h in inputs.items():
        want = plain(h, w)
        err = (got[r].double() - want).abs()
        bound = (2e-5 if dtype == "float32" else 4e-2) * (1.0 + want.abs())
        bad = (err > bound).any(dim=1)
        assert not bad.any(), f"request {r}: first wrong token {int(torch.where(bad)[0][0])} of {h.shape[0]}, max error {float(err.max()):.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,dk,dv,rot,page,width", [(4, 2, 16, 24, 8, 16, 96), (5, 5, 20, 12, 12, 8, 92), (8, 4, 64, 64, 64, 32, 256),
                                                            (6, 1, 128, 64, 32, 16, 128), (2, 2, 32, 32, 0, 16, 64)])
def test_attention_mixer_alone(tmp_path, dtype, heads, kv, dk, dv, rot, page, width):
    layer = TH._attn(heads, kv, dk, dv, 0.8 / math.sqrt(dk), rot, 100.0, (8.0, 1.0, 4.0, 32))
    if not rot:
        layer["mixer"].pop("rot")
    check_mixer(tmp_path, layer, width, 1e-5, dtype, page, lambda h, w: TP.attention(h, w, "l0.mix.", layer["mixer"]), seed=heads)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dk,dv,rank,window,page,width", [(3, 16, 24, 24, 11, 16, 96), (5, 20, 12, 36, 7, 8, 92), (8, 64, 64, 192, 64, 32, 256),
                                                                 (2, 48, 40, 64, 0, 16, 128), (4, 32, 32, 64, 1, 16, 64), (6, 32, 24, 80, 37, 16, 160)])
def test_latent_mixer_alone(tmp_path, dtype, heads, dk, dv, rank, window, page, width):
    """Windows of 1 (a token sees itself only), smaller and larger than a page, and none at all."""
    layer = TH._latent(heads, dk, dv, rank, 0.8 / math.sqrt(dk), window)
    check_mixer(tmp_path, layer, width, 1e-5, dtype, page, lambda h, w: TP.latent_attention(h, w, "l0.mix.", layer["mixer"], 1e-5), seed=heads)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,d,rank,width", [(3, 16, 8, 96), (4, 20, 12, 92), (4, 64, 32, 256), (1, 128, 24, 128), (6, 32, 16, 160)])
def test_wkv_mixer_alone(tmp_path, dtype, heads, d, rank, width):
    layer = TH._wkv(heads, d, rank)
    check_mixer(tmp_path, layer, width, 1e-5, dtype, 16, lambda h, w: TP.wkv(h, w, "l0.mix.", layer["mixer"], 1e-5), seed=heads)


# --------------------------------------------------------------------------- the engine against the plain model
LENGTHS = {"A": [1, 2, 17, 33, 70, 130], "B": [5, 31, 97, 150], "C": [3, 63, 64, 65, 200], "D": [2, 47, 129]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for n, (name, raw) in enumerate(TH.TEK.items()):
        d = tmp_path_factory.mktemp(f"tekarax_{name}")
        TH.make_tekarax_dir(d, raw, seed=700 + n)
        reqs = {f"{name}{i}": TH.decided_ids(d, L, seed=13 * n + i) for i, L in enumerate(LENGTHS[name])}
        plain = {rid: TH.plain_logits(d, ids) for rid, ids in reqs.items()}
        lowp = {rid: TH.plain_logits(d, ids, lowp=True) for rid, ids in reqs.items()}
        sq = sum(float(((lowp[rid] - plain[rid]) ** 2).sum()) for rid in reqs)
        out[name] = (d, reqs, plain, math.sqrt(sq / sum(p.size for p in plain.values())), lowp)
    return out


def run(models, name, dtype, steps, what, rename=None):
    d, reqs, plain, lowp_rms, lowp = models[name]
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), TH.TEK_PAGE_SIZE[name])
    if rename:
        plain, lowp = ({new: src[old] for new, old in rename.items()} for src in (plain, lowp))
    TH.compare(got, plain, dtype, what, lowp_rms, lowp)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_stream_after_every_layer_run(models, name):
    """In 32-bit, the stream after each run of a layer (a repeated layer counts each time) against the plain
    implementation's: the first run that differs names the layer."""
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import ops
    from pyre_b200.models.model import load_model
    from safetensors.torch import load_file
    d, reqs = models[name][:2]
    ids = max(reqs.values(), key=len)[:48]
    with torch.inference_mode():
        _logits, want = TP.forward(TH.TEK[name], load_file(str(d / "model.safetensors")), ids, keep_layers=True)
    model, _ = load_model(d, "cuda", "float32")
    cache, stepper = runtime_for_model(model, 64, TH.TEK_PAGE_SIZE[name], max_requests=1, cuda_graphs=False)
    cache.begin("r")
    ctx = stepper.build_context([StepEntry("r", ids, [])])
    x, pending = model.embed.forward(ctx), None
    for n, call in enumerate(model.calls):
        if call.add_vector is not None:
            ops.add_row_vector(x, model.vectors[call.add_vector[0]][call.add_vector[1]])
        x, pending = model.blocks[call.block].forward(ctx, x, pending, call)
        now = x + ops.materialize(pending).float() if pending is not None else x
        err = (now.double().cpu() - want[n]).abs().max()
        assert err < 2e-4 * (1 + want[n].abs().max()), f"run {n} (layer {call.block}, {TH.TEK[name]['layers'][call.block]['type']}): off by {float(err):.3e}"
    cache.end("r")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts(models, name, dtype):
    run(models, name, dtype, H.trace_whole(models[name][1]), "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prefill_then_token_by_token(models, name, dtype):
    steps = []
    for k, (rid, ids) in enumerate(models[name][1].items()):
        # most of it in one step and the rest one by one (a window passes over decoded tokens); every third request
        # one by one from its first token
        steps += H.trace_decode_tail(rid, ids, len(ids) if k % 3 == 2 else 32, first_step=len(steps))
    run(models, name, dtype, steps, "decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_down_to_two_tokens(models, name, dtype):
    steps = []
    for k, (rid, ids) in enumerate(models[name][1].items()):
        sizes = [[2, 9, 3, 17, 2, 31], [5, 2, 16, 8, 64], [24, 2, 2, 7, 1, 70]][k % 3]
        steps += H.trace_portions(rid, ids, sizes, first_step=len(steps))
    run(models, name, dtype, steps, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Every request twice under other names, at most four alive: later ones get the pages (filled with NaN when
    they were given back, by a window or at the end) and the state slots that earlier ones held, and must come out as
    each alone."""
    reqs = models[name][1]
    many = {f"{rid}r{rep}": ids for rep in range(2) for rid, ids in reqs.items()}
    steps = H.trace_mixed(many, seed=21, max_live=4, portion=(2, 40))
    run(models, name, dtype, steps, "mixed", rename={f"{rid}r{rep}": rid for rep in range(2) for rid in reqs})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(models, name, dtype):
    """220 tokens, the last 150 or more one by one (captured decode steps), two requests side by side: every window
    passes over decoded tokens several times and gives pages back on the way, and the recurrent state is carried
    through every step."""
    d, lowp_rms = models[name][0], models[name][3]
    reqs = {f"long{i}": TH.decided_ids(d, n, seed=90 + i) for i, n in enumerate([220, 190])}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:70 - 30 * i], "want": [0]} for i, (r, ids) in enumerate(reqs.items())], "end": []}]
    at = {r: 70 - 30 * i for i, r in enumerate(reqs)}
    while any(at[r] < len(reqs[r]) for r in reqs):
        entries = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in reqs if at[r] < len(reqs[r])]
        for e in entries:
            at[e["id"]] += 1
        steps.append({"step": len(steps), "entries": entries, "end": [e["id"] for e in entries if at[e["id"]] == len(reqs[e["id"]])]})
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), TH.TEK_PAGE_SIZE[name])
    want, lowp = {}, {}
    for i, (r, ids) in enumerate(reqs.items()):
        for dst, full in ((want, TH.plain_logits(d, ids)), (lowp, TH.plain_logits(d, ids, lowp=True))):
            dst[r] = np.concatenate([full[:1], full[70 - 30 * i:]])
    TH.compare(got, want, dtype, "long decoding", lowp_rms, lowp)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(models, name):
    """``Engine.generate`` (scheduler, portions of prompts, captured decode steps, sampler) gives the tokens that
    the plain implementation's argmax gives, in 32-bit; a cache too small for all requests at once makes the
    scheduler preempt and recompute, state slots included."""
    from pyre_b200.engine.engine import Engine
    from pyre_b200.sampling import SamplingParams
    d = models[name][0]
    raw = TH.TEK[name]
    prompts = [H.random_ids(raw["vocab"], n, seed=40 + n) for n in (15, 16, 3, 30)]
    new = 12
    engine = Engine(str(d), dtype="float32", page_size=16, num_pages=5, max_num_seqs=3, max_num_batched_tokens=32, prefill_chunk=20)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, return_logits=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for k in range(new):
            logits = TH.plain_logits(d, ids)[-1]
            top2 = np.sort(logits)[-2:]
            np.testing.assert_allclose(o.logits[k], logits, rtol=2e-4, atol=3e-5)
            if top2[1] - top2[0] > 1e-4:
                assert o.token_ids[k] == int(logits.argmax()), f"token {k} of a prompt of {len(p)}"
            ids.append(o.token_ids[k])
    assert json.dumps(engine.stats())
