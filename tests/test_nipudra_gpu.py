"""Nipudra on the GPU: every new mechanism alone against the plain implementation's function for it, each mixer alone
through the package's cache manager and step context (batches of unequal entries, portions, slots and pages used
again), then the engine through the replay loop and through ``Engine.generate`` against the plain implementation of
the whole model, in 32-bit and in bfloat16, for four small configurations that differ in every size and option."""

import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import nipudra_helpers as NH
from plain import nipudra_plain as NP

pytestmark = pytest.mark.gpu

BOTH = [torch.float32, torch.bfloat16]
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from pyre_b200.kernels import build, ops as o
    build.ensure_built(["seqmix", "blockops", "grouped", "parallel_block", "elementwise"])
    return o


def close(got, want, dtype, what="", atol32=3e-6, rel16=1.6e-2):
    tol = dict(rtol=3e-5, atol=atol32) if dtype == torch.float32 else dict(rtol=rel16, atol=rel16)
    torch.testing.assert_close(got.double().cpu(), want.double().cpu(), msg=lambda m: f"{what}: {m}", **tol)


def bf16_exact(*shape, scale=1.0, seed=0):
    """Random fp64 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).double()


def batch(lens):
    """seq_of_token and cu_seqlens of a step whose entries bring ``lens`` tokens."""
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    seq = np.repeat(np.arange(len(lens), dtype=np.int32), lens)
    return torch.from_numpy(seq).cuda(), torch.from_numpy(cu).cuda()


# Three sequences walked in steps of unequal portions (one token, fewer tokens than the history holds, many), the third
# one starting later in the slot that the first one leaves: (sequence, tokens) per step.
SEQ_LENS = {"a": 9, "b": 41, "c": 23}
STEPS = [[("a", 1), ("b", 7)], [("a", 2), ("b", 1)], [("a", 1), ("b", 1)], [("b", 30), ("a", 5)], [("c", 1), ("b", 2)], [("c", 2)],
         [("c", 20)]]
SLOT = {"a": 2, "b": 0, "c": 2}


# --------------------------------------------------------------------------- the small kernels, each alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("C,taps,col,extra,silu,bias,in_bias", [(5, 2, 0, 0, False, False, True), (33, 4, 3, 6, True, True, False),
                                                               (64, 3, 0, 0, False, False, False), (20, 5, 7, 1, True, True, True), (130, 8, 2, 0, False, True, False), (48, 4, 8, 8, True, True, True), (256, 2, 16, 0, False, False, False),
                                                               (7, 9, 0, 3, True, False, True)])
def test_short_convolution_over_state_slots(ops, dtype, C, taps, col, extra, silu, bias, in_bias):
    """Portions of every size against the convolution of the whole sequence; the history continues from the slot, a
    request that begins finds zeros where an earlier one left its inputs, and the floats beside the history stay."""
    W, off = col + C + extra, 11
    u = {r: bf16_exact(n, W, seed=i + taps) for i, (r, n) in enumerate(SEQ_LENS.items())}
    w, b, ib = bf16_exact(C, taps, seed=7), bf16_exact(C, seed=8) if bias else None, bf16_exact(C, seed=9) if in_bias else None
    want = {}
    for r in u:
        y = NP.short_convolution(u[r][:, col:col + C] + (ib if in_bias else 0.0), w, b)
        want[r] = NP.silu(y) if silu else y
    floats = off + (taps - 1) * C + 5
    state = torch.full((4, floats), float("nan"), device="cuda")
    state[:, :off], state[:, off + (taps - 1) * C:] = 3.0, 4.0
    at, got = {r: 0 for r in u}, {r: [] for r in u}
    for step in STEPS:
        for r, _ in step:
            if at[r] == 0:
                state[SLOT[r], off:off + (taps - 1) * C] = 0.0          # what the cache manager does when a request begins
        rows = torch.cat([u[r][at[r]:at[r] + n] for r, n in step]).to(dtype).cuda()
        seq, cu = batch([n for _, n in step])
        slots = torch.tensor([SLOT[r] for r, _ in step], dtype=torch.int32, device="cuda")
        y = ops.short_conv(rows, col, C, w.float().cuda(), b.float().cuda() if bias else None, state, off, slots, seq, cu, silu=silu,
                           in_bias=ib.float().cuda() if in_bias else None)
        k = 0
        for r, n in step:
            got[r].append(y[k:k + n].float().cpu())
            at[r], k = at[r] + n, k + n
    for r in u:
        close(torch.cat(got[r]), want[r], dtype, f"sequence {r}", atol32=2e-5)
    assert bool((state[:, :off] == 3.0).all()) and bool((state[:, off + (taps - 1) * C:] == 4.0).all())
    last = (u["b"][-(taps - 1):, col:col + C] + (ib if in_bias else 0.0)).float()
    assert torch.equal(state[SLOT["b"], off:off + (taps - 1) * C].cpu().view(taps - 1, C), last)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("wide", [None, False, True])
@pytest.mark.parametrize("Hn,G,P,N", [(3, 1, 16, 12), (4, 4, 20, 20), (8, 2, 64, 64), (2, 2, 40, 128), (2, 1, 33, 200), (6, 3, 8, 5)])
def test_state_space_recurrence_over_state_slots(ops, dtype, Hn, G, P, N, wide):
    """Step sizes from softplus of large and small arguments, decays from nearly one to nearly zero; the kernel's variant
    for single tokens, the one for prompt portions, and the choice by the step (a state that one left, the other takes up)."""
    cols = Hn * P + 2 * G * N
    xbc = {r: bf16_exact(n, cols, scale=0.7, seed=i) for i, (r, n) in enumerate(SEQ_LENS.items())}
    raw = {r: bf16_exact(n, 3 + Hn, scale=3.0, seed=10 + i) for i, (r, n) in enumerate(SEQ_LENS.items())}
    dt_bias, a_log, d_skip = bf16_exact(Hn, seed=20), bf16_exact(Hn, scale=1.5, seed=21), bf16_exact(Hn, seed=22)
    want = {}
    for r in xbc:
        T = SEQ_LENS[r]
        x = xbc[r][:, :Hn * P].reshape(T, Hn, P)
        B = xbc[r][:, Hn * P:Hn * P + G * N].reshape(T, G, N).repeat_interleave(Hn // G, dim=1)
        C = xbc[r][:, Hn * P + G * N:].reshape(T, G, N).repeat_interleave(Hn // G, dim=1)
        want[r] = NP.selective_scan(x, NP.softplus(raw[r][:, 3:] + dt_bias), torch.exp(a_log), B, C, d_skip).reshape(T, Hn * P)
    floats = Hn * N * P + 6
    state = torch.full((4, floats), float("nan"), device="cuda")
    state[:, Hn * N * P:] = 5.0
    at, got = {r: 0 for r in xbc}, {r: [] for r in xbc}
    for step in STEPS:
        for r, _ in step:
            if at[r] == 0:
                state[SLOT[r], :Hn * N * P] = 0.0
        rows = torch.cat([xbc[r][at[r]:at[r] + n] for r, n in step]).to(dtype).cuda()
        proj = torch.cat([raw[r][at[r]:at[r] + n] for r, n in step]).to(dtype).cuda()
        _, cu = batch([n for _, n in step])
        slots = torch.tensor([SLOT[r] for r, _ in step], dtype=torch.int32, device="cuda")
        y = ops.ssm_scan(rows, proj, 3, dt_bias.float().cuda(), a_log.float().cuda(), d_skip.float().cuda(), state, slots, cu, Hn, G, P, N, wide=wide)
        assert y.dtype == torch.float32
        k = 0
        for r, n in step:
            got[r].append(y[k:k + n].cpu())
            at[r], k = at[r] + n, k + n
    for r in xbc:
        err = (torch.cat(got[r]).double() - want[r]).abs().max()
        assert err <= 2e-5 * (1 + want[r].abs().max()), f"sequence {r}: off by {float(err):.3e}"
    assert bool((state[:, Hn * N * P:] == 5.0).all())


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,W,groups,gate,first,weight,post", [(5, 96, 3, "silu", True, True, 1.0), (3, 72, 3, "silu", False, False, 1.0),
                                                              (7, 92, 1, "sigmoid", False, True, 0.5), (2, 2048, 2, "silu", True, True, 1.0),
                                                              (4, 40, 5, None, False, False, 0.7)])
def test_unit_norm_over_parts_with_a_gate(ops, dtype, T, W, groups, gate, first, weight, post):
    y, proj, w = bf16_exact(T, W, seed=1), bf16_exact(T, W + 9, seed=2), bf16_exact(W, seed=3) + 1.0
    g = None if gate is None else (NP.silu if gate == "silu" else torch.sigmoid)(proj[:, 4:4 + W])
    v = y * g if (g is not None and first) else y
    want = NP.unit_rms(v.reshape(T, groups, W // groups), 1e-5).reshape(T, W) * (w if weight else 1.0) * post
    if g is not None and not first:
        want = want * g
    got = ops.group_norm_gate(y.float().cuda(), groups, w.float().cuda() if weight else None, 1e-5,
                              proj.to(dtype).cuda() if gate else None, 4, dtype, gate=gate or "silu", gate_first=first, post=post)
    assert got.dtype == dtype
    close(got, want, dtype, "gated unit norm", atol32=1e-5)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("Hn,G,dv,a_dim,lam,diff", [(4, 2, 24, 32, 0.8, 0.25), (5, 5, 12, 16, -0.3, 0.1), (6, 1, 40, 64, 1.7, 0.6), (3, 3, 64, 64, 0.05, 0.0)])
def test_two_maps_combined_per_head(ops, dtype, Hn, G, dv, a_dim, lam, diff):
    T, rep = 7, Hn // G
    a = bf16_exact(T, G, 2, rep, a_dim, seed=Hn)          # the kernels' order of the maps: (key/value head, map, query head of the group)
    o = (a[:, :, 0] - lam * a[:, :, 1]).reshape(T, Hn, a_dim)[..., :dv]
    want = (NP.unit_rms(o, 1e-6) * (1.0 - diff)).reshape(T, Hn * dv)
    got = ops.diff_combine(a.reshape(T, -1).to(dtype).cuda(), a_dim, lam, 1.0 - diff, Hn, G, dv, 1e-6)
    close(got, want, dtype, "a1 - lambda a2", atol32=1e-5)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("Hn,dim,rot,col,factor,amp", [(3, 16, 16, 0, 0.25, 1.0), (5, 20, 12, 7, 1.0, 1.2), (1, 128, 0, 3, 128 ** -0.5, 1.0), (4, 64, 32, 64, 0.125, 1.0)])
def test_heads_rotated_in_the_projection_row(ops, dtype, Hn, dim, rot, col, factor, amp):
    T, W = 9, col + Hn * dim + 5
    proj = bf16_exact(T, W, seed=dim)
    pos = torch.tensor([0, 1, 2, 50, 51, 100, 255, 7, 300], dtype=torch.int32)      # fp32 angles: a position beyond a few hundred shows in the fifth digit
    freqs = [10000.0 ** (-2.0 * i / rot) for i in range(rot // 2)] if rot else []
    want = proj.clone()
    heads = NP.rotate_halves(proj[:, col:col + Hn * dim].reshape(T, Hn, dim), pos, freqs, amp) * factor
    want[:, col:col + Hn * dim] = heads.reshape(T, Hn * dim)
    cos = sin = None
    if rot:
        cos, sin = ops.rope_table(pos.cuda(), torch.tensor(freqs, dtype=F64).float().cuda())
        ops.scale_cap(cos, amp), ops.scale_cap(sin, amp)
    got = ops.rotate_heads(proj.to(dtype).cuda(), col, Hn, dim, cos, sin, rot, factor)
    close(got, want, dtype, "rotated heads", atol32=2e-5)


@pytest.mark.parametrize("dtype", BOTH)
def test_side_slice_gate_shared_gate_and_cap(ops, dtype):
    T, dim, V, Wn = 6, 12, 50, 40
    pre, table = bf16_exact(T, dim, scale=2.0, seed=1), bf16_exact(V, 3 * dim, seed=2)
    ids = torch.tensor([0, 49, 7, 7, 13, 21], dtype=torch.int32)
    got = ops.side_gate(pre.to(dtype).cuda(), table.to(dtype).cuda(), dim, ids.cuda())
    close(got, NP.gelu_tanh(pre) * table[ids.long()][:, dim:2 * dim], dtype, "side slice", atol32=1e-5)
    acc, h, w, y = bf16_exact(T, Wn, seed=3), bf16_exact(T, 92, seed=4), bf16_exact(92, scale=0.1, seed=5), bf16_exact(T, Wn, seed=6)
    got = ops.token_gate_add(acc.float().cuda(), h.to(dtype).cuda(), w.float().cuda(), y.to(dtype).cuda())
    close(got, acc + torch.sigmoid(h @ w)[:, None] * y, torch.float32, "one gate per token", atol32=1e-5)
    x = bf16_exact(T, Wn, scale=30.0, seed=7)
    close(ops.scale_cap(x.float().cuda(), 0.5, 20.0), 20.0 * torch.tanh(x * 0.5 / 20.0), torch.float32, "cap", atol32=1e-5)
    close(ops.scale_cap(x.float().cuda(), 3.0), x * 3.0, torch.float32, "factor")


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("E,top", [(5, 2), (3, 3), (1, 1), (10, 4), (40, 1)])
def test_router_with_bias_and_weights_over_the_chosen(ops, dtype, E, top):
    T, Hn = 11, 92
    h, w, b = bf16_exact(T, Hn, seed=E), bf16_exact(E, Hn, scale=0.3, seed=E + 1), bf16_exact(E, scale=2.0, seed=E + 2)
    z = h @ w.T + b
    order = torch.argsort(z, dim=-1, descending=True, stable=True)[:, :top]
    want = torch.softmax(torch.gather(z, 1, order), dim=-1)
    idx, wt = ops.route(h.to(dtype).cuda(), w.float().cuda(), None, top, 1.0, bias=b.float().cuda(), renormalise=True)
    assert torch.equal(idx.cpu().long(), order), "the bias decides the choice too"
    close(wt, want, torch.float32, "softmax over the chosen logits", atol32=1e-5)


@pytest.mark.parametrize("dtype", BOTH)
def test_layer_norm_with_a_bias(ops, dtype):
    T, Hn = 5, 92
    x, d, w, b = bf16_exact(T, Hn, seed=1), bf16_exact(T, Hn, seed=2), bf16_exact(Hn, seed=3) + 1.0, bf16_exact(Hn, seed=4)
    xd = x.float().cuda()
    got = ops.add_layernorm(xd, d.to(dtype).cuda(), w.float().cuda(), 1e-5, dtype, bias=b.float().cuda())
    close(got, NP.layer_norm(x + d, w, b, 1e-5), dtype, "norm before a sublayer", atol32=2e-5)
    close(xd, x + d, torch.float32, "the stream")
    got = ops.gated_norm(d.to(dtype).cuda(), None, None, None, w.float().cuda(), 1e-5, dtype, center=True, out_bias=b.float().cuda())
    close(got, NP.layer_norm(d, w, b, 1e-5), torch.float32, "norm after a sublayer", atol32=2e-5)


# --------------------------------------------------------------------------- each mixer alone through the cache manager
def run_mixer_alone(tmp_path, layer, width, eps, dtype, page, steps, inputs, seed):
    """A model of this one layer is loaded (registry, loader, cache and state groups as ever), and its MIXER is called
    with inputs of the test's own on the step contexts that the package's stepper builds for ``steps`` (lists of
    (request, tokens) per step; a request begins at its first entry and ends after its last).  Returns the mixer's
    rows per request and the weights."""
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import ops
    from pyre_b200.models.model import load_model
    from safetensors.torch import load_file
    raw = {"architecture": "Nipudra", "vocab": 32, "width": width, "norm": {"eps": eps}, "layers": [dict(layer, mlp=None)]}
    NH.make_nipudra_dir(tmp_path, raw, seed=seed)
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
    """Steps of up to three live requests: portions of 1 to 30 tokens until each request has had all of its tokens;
    six requests in all, so slots and pages are used again."""
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


def check_mixer(tmp_path, layer, width, eps, dtype, page, plain, seed, wrong=None):
    inputs = {r: bf16_exact(n, width, seed=seed + i) for i, (r, n) in enumerate(MIXER_LENGTHS.items())}
    got, w = run_mixer_alone(tmp_path, layer, width, eps, dtype, page, mixer_schedule(MIXER_LENGTHS, seed), inputs, seed)
    for r, h in inputs.items():
        want = plain(h, w)
        err = (got[r].double() - want).abs()
        bound = (2e-5 if dtype == "float32" else 5e-2) * (1.0 + want.abs())
        bad = (err > bound).any(dim=1)
        assert not bad.any(), f"request {r}: first wrong token {int(torch.where(bad)[0][0])} of {h.shape[0]}, max error {float(err.max()):.3e}"
    if wrong is not None:     # the test can see the fault it is there for: the plain result with it is far outside the bound
        h = inputs["e"]
        want = plain(h, w)
        for other in wrong:
            assert ((other(h, w) - want).abs() > 2 * 5e-2 * (1.0 + want.abs())).any(), "this case would not show a window that is one off"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,dk,dv,conv,window,rot,page,width", [
    (4, 2, 16, 24, 3, 11, 8, 16, 96), (5, 5, 20, 12, 0, 0, 0, 8, 92), (4, 2, 64, 64, 4, 64, 64, 32, 256), (6, 1, 48, 40, 4, 100000, 16, 16, 128),
    (2, 2, 32, 32, 2, 1, 0, 16, 64), (6, 3, 12, 20, 5, 7, 12, 8, 92), (2, 1, 16, 16, 4, 16, 16, 16, 64), (3, 1, 32, 16, 2, 17, 32, 16, 72),
    (2, 1, 64, 128, 3, 40, 32, 16, 128), (4, 4, 128, 96, 4, 33, 64, 32, 256)])
def test_differential_attention_alone(tmp_path, dtype, heads, kv, dk, dv, conv, window, rot, page, width):
    """Windows of 1 (a token sees itself only), of a page, one more than a page, smaller and larger than a page, and none
    at all; the keys just inside and just outside: the plain result with a window one shorter or longer is far off."""
    layer = NH.attn(heads, kv, dk, dv, 0.8 / math.sqrt(dk), 0.35, conv, window, rot, 100.0, (8.0, 32, 4.0, 1.0) if rot else None)
    mixer = layer["mixer"]

    def plain(h, w, m=mixer):
        keys, values = NP.attention_keys_values(h, w, "l0.mix.", m, torch.arange(h.shape[0]))
        return NP.differential_attention(h, w, "l0.mix.", m, 1e-5, keys, values)
    wrong = None
    if 1 < window < 90:
        wrong = [lambda h, w, d=d: plain(h, w, dict(mixer, mask={"size": window + d})) for d in (-1, 1)]
    check_mixer(tmp_path, layer, width, 1e-5, dtype, page, plain, seed=heads, wrong=wrong)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,P,N,G,conv,parts,width", [(3, 16, 12, 1, 4, 3, 96), (4, 20, 20, 4, 2, 1, 92), (8, 64, 64, 2, 4, 2, 256),
                                                           (2, 40, 128, 2, 3, 4, 128), (1, 24, 8, 1, 6, 1, 40)])
def test_state_space_mixer_alone(tmp_path, dtype, heads, P, N, G, conv, parts, width):
    layer = NH.mamba(heads, P, N, G, conv, parts)
    check_mixer(tmp_path, layer, width, 1e-5, dtype, 16, lambda h, w: NP.mamba2(h, w, "l0.mix.", layer["mixer"], 1e-5), seed=heads)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dk,dv,rot,width", [(3, 16, 24, 16, 96), (5, 20, 12, 12, 92), (4, 64, 64, 32, 256), (1, 128, 64, 0, 128), (2, 32, 48, 8, 64)])
def test_retention_mixer_alone(tmp_path, dtype, heads, dk, dv, rot, width):
    decay = [1.0 - 2.0 ** (-2 - i) for i in range(heads)]
    layer = NH.retention(heads, dk, dv, decay, rot, 1000.0)
    check_mixer(tmp_path, layer, width, 1e-5, dtype, 16, lambda h, w: NP.retention(h, w, "l0.mix.", layer["mixer"], 1e-5), seed=heads)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("T,Hn,ff,E,top,shared", [(9, 96, 32, 5, 2, 48), (7, 92, 20, 3, 3, 0), (300, 256, 128, 8, 2, 256), (4, 128, 64, 1, 1, 0)])
def test_routed_feed_forward_of_plain_experts(ops, dtype, T, Hn, ff, E, top, shared):
    """Experts up / relu squared / down, the softmax over the chosen logits, a shared expert behind one gate per token;
    inputs on which no router decision is a close call."""
    from pyre_b200.parts.base import PartSpec, load_part, make_part
    g = torch.Generator().manual_seed(E)
    w = {f"p.e{e}.{n}": bf16_exact(*s, scale=0.2, seed=10 * e + i) for e in range(E) for i, (n, s) in enumerate((("up", (ff, Hn)), ("down", (Hn, ff))))}
    w["p.router"], w["p.router.b"] = bf16_exact(E, Hn, scale=0.5, seed=91), bf16_exact(E, seed=92)
    if shared:
        w.update({"p.shared.up": bf16_exact(shared, Hn, scale=0.2, seed=93), "p.shared.down": bf16_exact(Hn, shared, scale=0.2, seed=94),
                  "p.shared.sg": bf16_exact(1, Hn, scale=0.2, seed=95)})
    mlp = NH.moe(ff, E, top, shared)
    rows = []
    while len(rows) < T:
        h = (torch.randn(1, Hn, generator=g)).to(torch.bfloat16).double()
        margins = []
        NP.moe_mlp(h, w, "p.", mlp, margins=margins)
        if not margins or margins[0] > 0.05:
            rows.append(h)
    h = torch.cat(rows)
    want = NP.moe_mlp(h, w, "p.", mlp)
    part = make_part("ffn", PartSpec("routed_mlp", {"width": Hn, "intermediate": ff, "n_experts": E, "top": top, "activation": "relu2", "gated": False,
                                                    "correction": False, "renormalise": True, "router_bias": True, "shared": shared or None,
                                                    "shared_gate": bool(shared)}), dtype, "cuda")
    from pyre_b200.weights.loader import target_dtype
    table = {}
    from pyre_b200.parts.base import collect_tensors
    for name, spec in collect_tensors(part, "p.").items():
        table[name] = w[name].to(target_dtype(spec, torch.float32, dtype)).cuda()
    load_part(part, table, "p.")
    got = ops.materialize(part.forward(None, h.to(dtype).cuda())).float()
    bound = (2e-5 if dtype == torch.float32 else 3e-2) * float(want.abs().max())
    assert float((got.double().cpu() - want).abs().max()) <= bound


# --------------------------------------------------------------------------- the engine against the plain model
LENGTHS = {"A": [1, 2, 17, 33, 70, 130], "B": [5, 31, 97, 120], "C": [3, 63, 64, 65, 130], "D": [2, 47, 129]}
LONG = {"A": [220, 190], "C": [150, 120]}      # decoded one by one from token 70 (40) on


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for n, (name, raw) in enumerate(NH.NIP.items()):
        d = tmp_path_factory.mktemp(f"nipudra_{name}")
        NH.make_nipudra_dir(d, raw, seed=700 + n)
        reqs = {f"{name}{i}": NH.decided_ids(d, L, seed=13 * n + i) for i, L in enumerate(LENGTHS[name])}
        plain = {rid: NH.plain_logits(d, ids) for rid, ids in reqs.items()}
        lowp = {rid: NH.plain_logits(d, ids, lowp=True) for rid, ids in reqs.items()}
        sq = sum(float(((lowp[rid] - plain[rid]) ** 2).sum()) for rid in reqs)
        long_reqs = {f"long{i}": NH.decided_ids(d, L, seed=90 + i) for i, L in enumerate(LONG.get(name, []))}
        long_plain = {r: (NH.plain_logits(d, ids), NH.plain_logits(d, ids, lowp=True)) for r, ids in long_reqs.items()}
        out[name] = (d, reqs, plain, math.sqrt(sq / sum(p.size for p in plain.values())), lowp, long_reqs, long_plain)
    return out


def run(models, name, dtype, steps, what, rename=None):
    d, reqs, plain, lowp_rms, lowp = models[name][:5]
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), NH.NIP_PAGE_SIZE[name])
    if rename:
        plain, lowp = ({new: src[old] for new, old in rename.items()} for src in (plain, lowp))
    NH.compare(got, plain, dtype, what, lowp_rms, lowp)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_stream_after_every_layer(models, name):
    """In 32-bit, the stream after each layer against the plain implementation's: the first layer that differs is named."""
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import ops
    from pyre_b200.models.model import load_model
    from safetensors.torch import load_file
    d, reqs = models[name][:2]
    ids = max(reqs.values(), key=len)[:48]
    with torch.inference_mode():
        _logits, want = NP.forward(NH.NIP[name], load_file(str(d / "model.safetensors")), ids, keep_layers=True)
    model, _ = load_model(d, "cuda", "float32")
    cache, stepper = runtime_for_model(model, 64, NH.NIP_PAGE_SIZE[name], max_requests=1, cuda_graphs=False)
    cache.begin("r")
    ctx = stepper.build_context([StepEntry("r", ids, [])])
    x, pending = model.embed.forward(ctx), None
    for n, call in enumerate(model.calls):
        x, pending = model.blocks[call.block].forward(ctx, x, pending, call)
        now = x + ops.materialize(pending).float() if pending is not None else x
        err = (now.double().cpu() - want[n]).abs().max()
        assert err < 2e-4 * (1 + want[n].abs().max()), f"layer {call.block} ({NH.NIP[name]['layers'][call.block]['type']}): off by {float(err):.3e}"
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
    """Up to 220 tokens, the last 80 to 150 one by one (captured decode steps), two requests side by side: every window
    passes over decoded tokens several times and gives pages back on the way, and the recurrent states and the
    convolutions' histories are carried through every step."""
    d, lowp_rms, reqs, long_plain = models[name][0], models[name][3], models[name][5], models[name][6]
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:70 - 30 * i], "want": [0]} for i, (r, ids) in enumerate(reqs.items())], "end": []}]
    at = {r: 70 - 30 * i for i, r in enumerate(reqs)}
    while any(at[r] < len(reqs[r]) for r in reqs):
        entries = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in reqs if at[r] < len(reqs[r])]
        for e in entries:
            at[e["id"]] += 1
        steps.append({"step": len(steps), "entries": entries, "end": [e["id"] for e in entries if at[e["id"]] == len(reqs[e["id"]])]})
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), NH.NIP_PAGE_SIZE[name])
    want, lowp = {}, {}
    for i, r in enumerate(reqs):
        for dst, full in ((want, long_plain[r][0]), (lowp, long_plain[r][1])):
            dst[r] = np.concatenate([full[:1], full[70 - 30 * i:]])
    NH.compare(got, want, dtype, "long decoding", lowp_rms, lowp)


@pytest.mark.parametrize("name,seqs,pages", [("A", 3, 5), ("C", 3, 5), ("A", 6, 14)])
def test_greedy_generation_through_the_engine(models, name, seqs, pages):
    """``Engine.generate`` (scheduler, portions of prompts, captured decode steps, sampler) gives the tokens that
    the plain implementation's argmax gives, in 32-bit; a cache too small for all requests at once makes the
    scheduler preempt and recompute, state slots included; six requests side by side decode in captured steps that are
    padded with rows of no request (the scratch page and the scratch state slot)."""
    from pyre_b200.engine.engine import Engine
    from pyre_b200.sampling import SamplingParams
    d = models[name][0]
    raw = NH.NIP[name]
    prompts = [H.random_ids(raw["vocab"], n, seed=40 + n) for n in ((15, 16, 3, 30) if seqs == 3 else (15, 16, 3, 30, 7, 11))]
    new = 12
    engine = Engine(str(d), dtype="float32", page_size=16, num_pages=pages, max_num_seqs=seqs, max_num_batched_tokens=32, prefill_chunk=20)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, return_logits=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for k in range(new):
            logits = NH.plain_logits(d, ids)[-1]
            top2 = np.sort(logits)[-2:]
            np.testing.assert_allclose(o.logits[k], logits, rtol=2e-4, atol=3e-5)
            if top2[1] - top2[0] > 1e-4:
                assert o.token_ids[k] == int(logits.argmax()), f"token {k} of a prompt of {len(p)}"
            ids.append(o.token_ids[k])
    assert json.dumps(engine.stats())
