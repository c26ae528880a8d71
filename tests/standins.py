"""Plain torch stand-ins for the CUDA kernels, for tests without a GPU.

They state each kernel's contract (arguments, layouts, what is written where) in the simplest
terms and share no code with the kernels.  With them in place of ``pyre_b200.kernels.ops`` the
package's own parts, model, cache manager, step function and replay loop run on the CPU, so the
host side of the engine (the batch's layout, the block tables, the order of the schedule, the
bookkeeping of lengths and pages) is tested against the plain implementation where no GPU is."""

from __future__ import annotations

import torch


def embedding(table, ids, out=None, err_flag=None):
    return table[ids.long()].float()


def add_rmsnorm(x, delta, weight, eps, out_dtype, rows=None, update_x=True, out=None, scaled_ok=False):
    v = x if delta is None else x + delta.float()
    if rows is None and update_x and delta is not None:
        x.copy_(v)
    if rows is not None:
        v = v[rows.long()]
    h = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight
    return h.to(out_dtype)


def add_residual(x, delta):
    x.add_(delta.float())
    return x


def rope_table(positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def qkv_rope_write(qkv, bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads, head_dim, rotary_dim,
                   page_size, q_out=None):
    T = qkv.shape[0]
    x = qkv.float()
    if bias is not None:
        x = x + bias
    q, k, v = x.split([n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim], dim=1)
    q, k, v = q.reshape(T, n_heads, head_dim), k.reshape(T, n_kv_heads, head_dim), v.reshape(T, n_kv_heads, head_dim)

    def rotate(t):
        if not rotary_dim:
            return t
        half = rotary_dim // 2
        a, b, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        c, s = cos[:, None, :], sin[:, None, :]
        return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)

    q, k = rotate(q), rotate(k)
    if cache_layer is not None:
        for t in range(T):
            page, off = divmod(int(slot_mapping[t]), page_size)
            cache_layer[page, 0, :, off, :] = k[t].to(cache_layer.dtype)
            cache_layer[page, 1, :, off, :] = v[t].to(cache_layer.dtype)
    return q.reshape(T, n_heads * head_dim).to(qkv.dtype)


def paged_attention_generic(q, cache_layer, block_table, seq_of_token, positions, n_heads, n_kv_heads, head_dim, scale,
                            window=None, out=None, sink=None):
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    n_rep = n_heads // n_kv_heads
    result = torch.empty_like(q)
    for t in range(T):
        b, p = int(seq_of_token[t]), int(positions[t])
        lo = 0 if not window else max(0, p - window + 1)
        pos = torch.arange(lo, p + 1)
        pages = block_table[b].long()[pos // page_size]
        assert (pages >= 0).all(), f"token {t}: a key in its window lies on a page that was given back"
        keys = cache_layer[pages, 0, :, pos % page_size, :].float()          # [keys, kv heads, head_dim]
        vals = cache_layer[pages, 1, :, pos % page_size, :].float()
        qt = q[t].float().reshape(n_kv_heads, n_rep, head_dim)
        scores = torch.einsum("grd,kgd->grk", qt, keys) * scale
        if sink is None:
            probs = torch.softmax(scores, dim=-1)
        else:       # one more term in the denominator, with no value; a tensor holds a score per query head
            sk = sink.float().reshape(n_kv_heads, n_rep, 1) if isinstance(sink, torch.Tensor) else torch.full((1, 1, 1), float(sink))
            top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sk)
            e = torch.exp(scores - top)
            probs = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sk - top))
        result[t] = torch.einsum("grk,kgd->grd", probs, vals).reshape(-1).to(q.dtype)
    return result


def cast_rows(x, dtype):
    return x if dtype == torch.float32 else x.to(dtype)


def norm_add(x, y, weight, eps, act_dtype, want_next=False):
    v = _partial_sums_or_tensor(y)
    x.add_(v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight)
    if not want_next:
        return None
    return x if act_dtype == torch.float32 else x.to(act_dtype)


def activation(x, kind):
    z = x.float()
    if kind == "silu":
        return torch.nn.functional.silu(z).to(x.dtype)
    assert kind == "gelu_tanh"
    return torch.nn.functional.gelu(z, approximate="tanh").to(x.dtype)


def linear_act(x, w, kind):
    from pyre_b200.kernels import ops
    return ops.activation(ops.materialize(ops.linear(x, w)), kind)


def qk_norm_rope_write(proj, q_col, k_col, v_col, q_weight, k_weight, eps, cos, sin, cache_layer, slot_mapping, n_heads,
                       n_kv_heads, qk_dim, v_dim, row_dim, rotary_dim, page_size, v_cos=None, v_sin=None):
    T = proj.shape[0]
    x = proj.float()

    def heads(col, n, d, w):
        t = x[:, col:col + n * d].reshape(T, n, d)
        if w is not None:
            t = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w
        if rotary_dim:
            half = rotary_dim // 2
            a, b, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
            c, s = cos[:, None, :], sin[:, None, :]
            t = torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)
        return torch.nn.functional.pad(t, (0, row_dim - d))

    q = heads(q_col, n_heads, qk_dim, q_weight)
    if cache_layer is not None:
        k = heads(k_col, n_kv_heads, qk_dim, k_weight)
        v = x[:, v_col:v_col + n_kv_heads * v_dim].reshape(T, n_kv_heads, v_dim)
        if v_cos is not None:      # the values turn over all their dims, by tables of their own
            a, b = v[..., :v_dim // 2], v[..., v_dim // 2:]
            c, sn = v_cos[:, None, :], v_sin[:, None, :]
            v = torch.cat([a * c - b * sn, b * c + a * sn], dim=-1)
        v = torch.nn.functional.pad(v, (0, row_dim - v_dim))
        for t in range(T):
            page, off = divmod(int(slot_mapping[t]), page_size)
            cache_layer[page, 0, :, off, :] = k[t].to(cache_layer.dtype)
            cache_layer[page, 1, :, off, :] = v[t].to(cache_layer.dtype)
    return q.reshape(T, n_heads * row_dim).to(proj.dtype)


def sigmoid_gate(a, a_dim, proj, g_col, n_heads, v_dim):
    T = a.shape[0]
    out = a.float().reshape(T, n_heads, a_dim)[..., :v_dim].reshape(T, n_heads * v_dim)
    if proj is not None:
        out = out * torch.sigmoid(proj[:, g_col:g_col + n_heads * v_dim].float())
    return out.to(a.dtype)


def head_gate(a, a_dim, proj, g_col, n_heads, v_dim, cos=None, sin=None):
    T = a.shape[0]
    out = a.float().reshape(T, n_heads, a_dim)[..., :v_dim]
    if cos is not None:      # turned back: minus the token's angles
        x, y = out[..., :v_dim // 2], out[..., v_dim // 2:]
        c, sn = cos[:, None, :], sin[:, None, :]
        out = torch.cat([x * c + y * sn, y * c - x * sn], dim=-1)
    if proj is not None:
        out = out * torch.sigmoid(proj[:, g_col:g_col + n_heads].float())[:, :, None]
    return out.reshape(T, n_heads * v_dim).to(a.dtype)


def bias_act(x, bias, kind):
    z = x.float() if bias is None else x.float() + bias
    fn = {"silu": torch.nn.functional.silu, "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
          "relu2": lambda t: torch.relu(t) ** 2, "tanh": torch.tanh, None: lambda t: t}[kind]
    return fn(z).to(x.dtype)


def add_row_vector(x, v):
    x.add_(v)
    return x


def gated_norm(y, y_bias, gate, gate_bias, weight, eps, act_dtype, center=True, out_bias=None):
    v = _partial_sums_or_tensor(y)
    if y_bias is not None:
        v = v + y_bias
    if gate is not None:
        v = v * torch.sigmoid(gate.float() + (gate_bias if gate_bias is not None else 0.0))
    if center:
        v = v - v.mean(-1, keepdim=True)
    out = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight
    return out if out_bias is None else out + out_bias


def scale_to_places(h, place_of, weight, n_places):
    out = torch.full((n_places, h.shape[1]), float("nan"), dtype=h.dtype)
    for t in range(h.shape[0]):
        for k in range(place_of.shape[1]):
            if int(place_of[t, k]) >= 0:
                out[int(place_of[t, k])] = (weight[t, k] * h[t].float()).to(h.dtype)
    return out


def token_shift_mix(h, state_layer, prev_off, slots, seq_of_token, cu_seqlens, mu):
    T, W = h.shape
    x = h.float()
    prev = torch.empty_like(x)
    for t in range(T):
        b = int(seq_of_token[t])
        prev[t] = state_layer[int(slots[b]), prev_off:prev_off + W] if t == int(cu_seqlens[b]) else x[t - 1]
    return (x[None] + (prev - x)[None] * mu[:, None, :]).to(h.dtype)


def wkv_scan(r, k, v, g, dlog, w0, u, norm_w, state_layer, prev_off, slots, cu_seqlens, h, n_heads, dim, eps):
    T = r.shape[0]
    shape = (T, n_heads, dim)
    rf, kf, vf = r.float().reshape(shape), k.float().reshape(shape), v.float().reshape(shape)
    decay = torch.exp(-torch.exp(dlog + w0)).reshape(shape)
    bonus = u.reshape(n_heads, dim)
    out = torch.empty(shape)
    for b in range(cu_seqlens.shape[0] - 1):
        slot = int(slots[b])
        S = state_layer[slot, :prev_off].reshape(n_heads, dim, dim).clone()
        for t in range(int(cu_seqlens[b]), int(cu_seqlens[b + 1])):
            kv = kf[t][:, :, None] * vf[t][:, None, :]
            out[t] = torch.einsum("hi,hij->hj", rf[t], S + bonus[:, :, None] * kv)
            S = decay[t][:, :, None] * S + kv
        state_layer[slot, :prev_off] = S.reshape(-1)
        if int(cu_seqlens[b + 1]) > int(cu_seqlens[b]):
            state_layer[slot, prev_off:prev_off + h.shape[1]] = h[int(cu_seqlens[b + 1]) - 1].float()
    out = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + eps)
    return (out.reshape(T, -1) * norm_w * torch.nn.functional.silu(g.float())).to(r.dtype)


def rmsnorm_gate(o, weight, eps, proj, g_col, out_dtype):
    v = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * weight
    if proj is not None:
        v = v * torch.sigmoid(proj[:, g_col:g_col + o.shape[1]].float())
    return v.to(out_dtype)


def linear_attention(proj, q_col, k_col, v_col, state_layer, slots, cu_seqlens, decay, n_heads, qk_dim, v_dim,
                     activation="silu", lens=None):
    T = proj.shape[0]
    x = proj.float()
    act = torch.nn.functional.silu if activation == "silu" else (lambda z: z)
    q = act(x[:, q_col:q_col + n_heads * qk_dim]).reshape(T, n_heads, qk_dim)
    k = act(x[:, k_col:k_col + n_heads * qk_dim]).reshape(T, n_heads, qk_dim)
    v = act(x[:, v_col:v_col + n_heads * v_dim]).reshape(T, n_heads, v_dim)
    out = torch.empty((T, n_heads, v_dim), dtype=torch.float32)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        S = state_layer[int(slots[b])]            # [heads, qk_dim, v_dim], updated in place
        for t in range(cu[b], cu[b + 1]):
            S.mul_(decay[:, None, None]).add_(k[t][:, :, None] * v[t][:, None, :])
            out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out.reshape(T, n_heads * v_dim)


def sgemm_nt(a, w, bias=None, out=None):
    y = a @ w.t()
    return y if bias is None else y + bias


def silu_mul(gate_up, out=None, block=0):
    assert block == 0, "the float32 path stacks all gates before all ups"
    inter = gate_up.shape[1] // 2
    return torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]


def sample(logits, temperature=None, seeds=None, token_index=None, out=None):
    assert temperature is None, "the stand-in samples greedily only"
    return logits.argmax(dim=-1).to(torch.int32)


def feed_tokens(token_ids, dst, src, prev):
    for d, s in zip(dst.tolist(), src.tolist()):
        if d >= 0:
            token_ids[d] = prev[s]



# --------------------------------------------------------------------------- layers whose branches share one norm
def _branch(t):
    from pyre_b200.kernels import ops
    if isinstance(t, ops.PartialSums):
        return t.parts.sum(0)
    return t.float()


def add_layernorm(x, delta, weight, eps, out_dtype, rows=None, update_x=True, act_dtype=None, bias=None):
    from pyre_b200.kernels import ops
    v = x
    if delta is not None:
        terms = delta.terms if isinstance(delta, ops.ScaledSum) else [(delta, torch.ones_like(weight))]
        add = sum(g * _branch(t) for t, g in terms)
        v = x + add
        if rows is None and update_x:
            x.copy_(v)
    if rows is not None:
        v = v[rows.long()]
    dev = v - v.mean(-1, keepdim=True)
    out = dev * torch.rsqrt(dev.pow(2).mean(-1, keepdim=True) + eps) * weight
    return (out if bias is None else out + bias).to(out_dtype)


def act_mul(gate_up, kind):
    g, u = gate_up.float().chunk(2, dim=1)
    a = torch.nn.functional.silu(g) if kind == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    return (a * u).to(gate_up.dtype)


def _turn_pairs(v, cos, sin, rot):
    """Neighbouring pairs of the first ``rot`` entries of the last axis turn by the token's angles; v [T, ..., n]."""
    if not rot:
        return v
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [rot // 2]
    c, s = cos.view(shape), sin.view(shape)
    a, b = v[..., 0:rot:2], v[..., 1:rot:2]
    out = v.clone()
    out[..., 0:rot:2] = a * c - b * s
    out[..., 1:rot:2] = b * c + a * s
    return out


def latent_prepare(proj, q_col, q_rank, c_col, rank, rope, rot, wq, wc, eps, cos, sin, cache_layer, slot_mapping, page_size,
                   act_dtype):
    x = _branch(proj)
    T = x.shape[0]
    rms = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w
    cq = rms(x[:, q_col:q_col + q_rank], wq).to(act_dtype) if q_rank else None
    if cache_layer is not None:
        c = rms(x[:, c_col:c_col + rank], wc)
        r = _turn_pairs(x[:, c_col + rank:c_col + rank + rope], cos, sin, rot)
        assert cache_layer.shape[1:3] == (1, 1)
        for t in range(T):
            page, off = divmod(int(slot_mapping[t]), page_size)
            cache_layer[page, 0, 0, off, :] = 0
            cache_layer[page, 0, 0, off, :rank + rope] = torch.cat([c[t], r[t]]).to(cache_layer.dtype)
    return cq


def latent_rotate_q(q, qa, cos, sin, n_heads, dq, rope, rot, rank):
    T = q.shape[0]
    tail = _turn_pairs(q.float().view(T, n_heads, dq + rope)[..., dq:], cos, sin, rot)
    qa[..., rank:] = 0
    qa[..., rank:rank + rope] = tail.to(qa.dtype)


def latent_attention(ctx, qa, cache_layer, block_table, rank, rope, scale, window):
    T, nh, row = qa.shape
    page_size = cache_layer.shape[3]
    out = torch.empty((T, nh, rank), dtype=qa.dtype)
    for t in range(T):
        b, p = int(ctx.seq_of_token[t]), int(ctx.positions[t])
        lo = 0 if not window else max(0, p - window + 1)
        pos = torch.arange(lo, p + 1)
        pages = block_table[b].long()[pos // page_size]
        assert (pages >= 0).all(), f"token {t}: a key in its window lies on a page that was given back"
        rows = cache_layer[pages, 0, 0, pos % page_size, :].float()             # [keys, row]
        scores = qa[t].float()[:, :rank + rope] @ rows[:, :rank + rope].t() * scale
        out[t] = (torch.softmax(scores, dim=-1) @ rows[:, :rank]).to(qa.dtype)
    return out


def headwise_linear(x, w, out=None):
    T, H, _ = x.shape
    N, K = w.shape[1:]
    y = torch.einsum("thk,hnk->thn", x.float()[..., :K], w.float()).to(x.dtype).contiguous()
    if out is None:
        return y
    out[..., :N] = y
    return out


def route(h, w, correction, top, scale, sigmoid=False, bias=None, renormalise=False):
    z = h.float() @ w.t()
    if bias is not None:
        z = z + bias
    s = torch.sigmoid(z) if sigmoid else torch.softmax(z, dim=-1)
    choice = s if correction is None else s + correction
    idx = choice.topk(top, dim=-1).indices
    weight = s.gather(-1, idx) * scale
    if renormalise:
        weight = weight / weight.sum(-1, keepdim=True)
    return idx.to(torch.int32), weight


# --------------------------------------------------------------------------- short histories and recurrent states
def scale_cap(x, scale=1.0, cap=0.0):
    x.mul_(scale)
    if cap > 0:
        x.copy_(cap * torch.tanh(x / cap))
    return x


def short_conv(inp, col, n_ch, weight, bias, state_layer, state_off, slots, seq_of_token, cu_seqlens, silu=False, in_bias=None):
    T = inp.shape[0]
    taps = weight.shape[1]
    u = inp[:, col:col + n_ch].float()
    if in_bias is not None:
        u = u + in_bias
    out = torch.empty((T, n_ch), dtype=torch.float32)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        if cu[b + 1] == cu[b]:
            continue
        hist = state_layer[int(slots[b]), state_off:state_off + (taps - 1) * n_ch].view(taps - 1, n_ch)
        seq = torch.cat([hist, u[cu[b]:cu[b + 1]]], dim=0)
        n = cu[b + 1] - cu[b]
        y = sum(seq[j:j + n] * weight[:, j] for j in range(taps))
        out[cu[b]:cu[b + 1]] = y if bias is None else y + bias
        hist.copy_(seq[n:].clone())
    if silu:
        out = torch.nn.functional.silu(out)
    return out.to(inp.dtype)


def ssm_scan(xbc, proj, dt_col, dt_bias, a_log, d_skip, state_layer, slots, cu_seqlens, n_heads, n_groups, p_dim, n_state, wide=None):
    T = xbc.shape[0]
    H, G, P, N = n_heads, n_groups, p_dim, n_state
    v = xbc.float()
    x = v[:, :H * P].reshape(T, H, P)
    B = v[:, H * P:H * P + G * N].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    C = v[:, H * P + G * N:].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    dt = torch.nn.functional.softplus(proj[:, dt_col:dt_col + H].float() + dt_bias, threshold=20.0)
    dec = torch.exp(-torch.exp(a_log) * dt)
    y = torch.empty((T, H, P), dtype=torch.float32)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        S = state_layer[int(slots[b]), :H * N * P].view(H, N, P)      # updated in place
        for t in range(cu[b], cu[b + 1]):
            S.mul_(dec[t][:, None, None]).add_((dt[t][:, None] * x[t])[:, None, :] * B[t][:, :, None])
            y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + d_skip[:, None] * x[t]
    return y.reshape(T, H * P)


def group_norm_gate(y, groups, weight, eps, proj, g_col, out_dtype, gate="silu", gate_first=False, post=1.0):
    T, W = y.shape
    act = torch.nn.functional.silu if gate == "silu" else torch.sigmoid
    g = act(proj[:, g_col:g_col + W].float()) if proj is not None else None
    v = y * g if (g is not None and gate_first) else y
    v = v.reshape(T, groups, W // groups)
    v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).reshape(T, W)
    if weight is not None:
        v = v * weight
    v = v * post
    if g is not None and not gate_first:
        v = v * g
    return v.to(out_dtype)


def diff_combine(a, a_dim, lam, post, n_heads, n_kv_heads, v_dim, eps):
    T = a.shape[0]
    rep = n_heads // n_kv_heads
    maps = a.float().reshape(T, n_kv_heads, 2, rep, a_dim)[..., :v_dim]
    o = (maps[:, :, 0] - lam * maps[:, :, 1]).reshape(T, n_heads, v_dim)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * post
    return o.reshape(T, n_heads * v_dim).to(a.dtype)


def rotate_heads(proj, col, n_heads, dim, cos, sin, rotary_dim, factor=1.0):
    T = proj.shape[0]
    v = proj[:, col:col + n_heads * dim].float().reshape(T, n_heads, dim)
    if rotary_dim:
        half = rotary_dim // 2
        a, b, rest = v[..., :half], v[..., half:rotary_dim], v[..., rotary_dim:]
        c, sn = cos[:, None, :], sin[:, None, :]
        v = torch.cat([a * c - b * sn, b * c + a * sn, rest], dim=-1)
    proj[:, col:col + n_heads * dim] = (v * factor).reshape(T, n_heads * dim).to(proj.dtype)
    return proj


def side_gate(pre, table, col, token_ids, err_flag=None):
    e = table[token_ids.long()][:, col:col + pre.shape[1]].float()
    return (torch.nn.functional.gelu(pre.float(), approximate="tanh") * e).to(pre.dtype)


def token_gate_add(acc, h, w, y):
    acc.add_(torch.sigmoid(h.float() @ w)[:, None] * y.float())
    return acc


def group_pairs(idx, n_experts):
    T, top = idx.shape
    flat = idx.reshape(-1).long()
    order = [p for e in range(n_experts) for p in range(T * top) if flat[p] == e]
    counts = [int((flat == e).sum()) for e in range(n_experts)]
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    place_of = torch.full((T * top,), -1, dtype=torch.int32)
    src = torch.zeros(T * top, dtype=torch.int32)
    for place, p in enumerate(order):
        place_of[p] = place
        src[place] = p // top
    return offsets, place_of.view(T, top), src


def expert_linear(x, w, offsets, src, n_places, out_dtype=None):
    E, N, K = w.shape
    out = torch.full((n_places, N), float("nan"), dtype=out_dtype or x.dtype)      # places that no expert owns are never read
    for e in range(E):
        for p in range(int(offsets[e]), int(offsets[e + 1])):
            r = int(src[p]) if src is not None else p
            out[p] = (x[r].float() @ w[e].float().t()).to(out.dtype)
    return out


def combine_pairs(y, h, place_of, weight):
    T, H = h.shape
    out = torch.zeros((T, H), dtype=torch.float32)
    for t in range(T):
        for k in range(place_of.shape[1]):
            p = int(place_of[t, k])
            out[t] += weight[t, k] * (y[p] if p >= 0 else h[t].float())
    return out


def install(monkeypatch) -> None:
    """Put the stand-ins in place of the kernels for one test (float32 models on the CPU)."""
    from pyre_b200.engine import step
    from pyre_b200.kernels import build, ops

    monkeypatch.setattr(build, "ensure_built", lambda names, **kw: None)     # the stand-ins need no library
    flag = torch.zeros(1, dtype=torch.int32)
    for name, fn in dict(embedding=embedding, add_rmsnorm=add_rmsnorm, add_residual=add_residual, rope_table=rope_table,
                         qkv_rope_write=qkv_rope_write, paged_attention_generic=paged_attention_generic,
                         sgemm_nt=sgemm_nt, silu_mul=silu_mul, sample=sample, feed_tokens=feed_tokens, cast_rows=cast_rows,
                         norm_add=norm_add, activation=activation, linear_act=linear_act, qk_norm_rope_write=qk_norm_rope_write,
                         sigmoid_gate=sigmoid_gate, rmsnorm_gate=rmsnorm_gate, linear_attention=linear_attention,
                         add_layernorm=add_layernorm, act_mul=act_mul, latent_prepare=latent_prepare, latent_rotate_q=latent_rotate_q,
                         latent_attention=latent_attention, headwise_linear=headwise_linear, route=route, group_pairs=group_pairs,
                         expert_linear=expert_linear, combine_pairs=combine_pairs, head_gate=head_gate, bias_act=bias_act,
                         add_row_vector=add_row_vector, gated_norm=gated_norm, scale_to_places=scale_to_places,
                         token_shift_mix=token_shift_mix, wkv_scan=wkv_scan, scale_cap=scale_cap, short_conv=short_conv,
                         ssm_scan=ssm_scan, group_norm_gate=group_norm_gate, diff_combine=diff_combine, rotate_heads=rotate_heads,
                         side_gate=side_gate, token_gate_add=token_gate_add).items():
        monkeypatch.setattr(ops, name, fn)
    monkeypatch.setattr(ops, "device_error_flag", lambda device: flag)
    monkeypatch.setattr(ops, "check_device_errors", lambda device="cpu": None)
    monkeypatch.setattr(step._Staging, "upload", lambda self, flat: torch.from_numpy(flat.copy()))
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)


# --------------------------------------------------------------------------- the bfloat16 path
# Stand-ins for the tensor-core kernels: bf16 operands, fp32 arithmetic, results rounded where the
# kernels round them.  The products honour the package's own plan (orientation, width, split of K), so
# split-K partial sums travel to their consumers as they do on the device; the attention stand-ins
# write only the rows of the entries that the kernel they stand for would take.

def _partial_sums_or_tensor(t):
    from pyre_b200.kernels import ops
    if isinstance(t, ops.DeferredProduct):      # a product not launched yet: the stand-ins never fold, they run it plainly
        t = t.partials()
    return t.parts.sum(0) if isinstance(t, ops.PartialSums) else t.float()


def add_rmsnorm_any(x, delta, weight, eps, out_dtype, rows=None, update_x=True, out=None, scaled_ok=False):
    return add_rmsnorm(x, None if delta is None else _partial_sums_or_tensor(delta), weight, eps, out_dtype, rows, update_x)


def qkv_rope_write_any(qkv, bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads, head_dim, rotary_dim,
                       page_size, q_out=None):
    act = qkv.dtype          # of the activations, for a tensor and for partial sums alike
    q = qkv_rope_write(_partial_sums_or_tensor(qkv), bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads,
                       head_dim, rotary_dim, page_size)
    return q.to(act)


def materialize(t):
    from pyre_b200.kernels import ops
    if isinstance(t, ops.DeferredProduct):
        t = t.partials()
    return t.parts.sum(0).to(t.dtype) if isinstance(t, ops.PartialSums) else t


def gemm_tc(x, w, out_dtype=torch.bfloat16, plan=None, reduce=True, gated=False, pair=None, checked=False):
    from pyre_b200.kernels import ops
    assert x.dtype == w.dtype == torch.bfloat16 and x.shape[1] == w.shape[1]
    M, K = x.shape
    N = w.shape[0]
    _rows, _bn, splits = plan or ops.tc_gemm_plan(M, N, K)
    kb = -(-K // 64)
    splits = max(1, min(splits, kb))
    if gated:
        assert N % (2 * ops.GATED_BLOCK) == 0
        y = (x.float() @ w.float().t()).view(M, N // (2 * ops.GATED_BLOCK), 2, ops.GATED_BLOCK)
        return (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(M, N // 2).to(torch.bfloat16)
    per = -(-kb // splits) * 64
    parts = torch.stack([x[:, s * per:(s + 1) * per].float() @ w[:, s * per:(s + 1) * per].float().t() for s in range(splits)])
    if splits == 1 and reduce:
        return parts[0].to(out_dtype)
    if not reduce:
        return ops.PartialSums(parts.contiguous(), out_dtype)
    return parts.sum(0).to(out_dtype)


def silu_mul_any(gate_up, out=None, block=0):
    if block == 0:
        return silu_mul(gate_up.float()).to(gate_up.dtype)
    T, two_i = gate_up.shape
    y = gate_up.float().view(T, two_i // (2 * block), 2, block)
    return (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(T, two_i // 2).to(gate_up.dtype)


def _attend_entries(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale, window,
                    out, takes, sink=None):
    cu = cu_seqlens.tolist()
    taken = 0
    for b in range(n_seqs):
        n = cu[b + 1] - cu[b]
        if not takes(n):
            continue
        taken += n
        rows = slice(cu[b], cu[b + 1])
        out[rows] = paged_attention_generic(q[rows], cache_layer, block_table[b:b + 1], torch.zeros(n, dtype=torch.int32),
                                            positions[rows], n_heads, n_kv_heads, head_dim, scale, window, sink=sink)
    return taken


def paged_attention_mma(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale,
                        window=None, n_splits=1, out=None, scratch=None, max_len=0, uniform_len=0, sink=None):
    from pyre_b200.kernels import ops
    assert q.dtype == cache_layer.dtype == torch.bfloat16 and head_dim <= ops.MMA_MAX_HEAD_DIM
    assert 1 <= n_splits <= ops.MAX_SCRATCH_SPLITS
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    assert not uniform_len or all(n == uniform_len for n in lens), "uniform_len promises entries of one length"
    if out is None:
        out = torch.empty_like(q)
    _attend_entries(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale, window,
                    out, lambda n: not (max_len > 0 and n > max_len), sink=sink)
    return out


def attention_prefill(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_long_tokens, n_heads, n_kv_heads,
                      head_dim, scale, window, out, min_len=32, sink=None):
    from pyre_b200.kernels import ops
    assert head_dim in ops.PREFILL_HEAD_DIMS
    taken = _attend_entries(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale,
                            window, out, lambda n: n >= min_len, sink=sink)
    assert taken == n_long_tokens, "n_long_tokens must count the tokens of the entries this kernel takes"
    return out


def attention_prefill_tc(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_long_tokens, n_heads, n_kv_heads,
                         head_dim, scale, window, out, min_len, key_splits=1, sink=None):
    page_size = cache_layer.shape[3]
    assert 1 <= key_splits <= 32
    assert page_size & (page_size - 1) == 0 and page_size >= 4, "the tcgen05 attention takes power-of-two pages"
    return attention_prefill(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_long_tokens, n_heads, n_kv_heads,
                             head_dim, scale, window, out, min_len, sink=sink)


def install_bf16(monkeypatch, calls: "dict | None" = None) -> None:
    """The float32 stand-ins plus those of the bfloat16 path.  ``calls`` (optional) counts how often
    each attention kernel's stand-in ran."""
    from pyre_b200.kernels import ops

    install(monkeypatch)

    def counted(name, fn):
        def wrapper(*a, **k):
            if calls is not None:
                calls[name] = calls.get(name, 0) + 1
            return fn(*a, **k)
        return wrapper

    for name, fn in dict(add_rmsnorm=add_rmsnorm_any, qkv_rope_write=qkv_rope_write_any, materialize=materialize,
                         gemm_tc=gemm_tc, silu_mul=silu_mul_any).items():
        monkeypatch.setattr(ops, name, fn)
    for name, fn in dict(paged_attention_mma=paged_attention_mma, attention_prefill=attention_prefill,
                         attention_prefill_tc=attention_prefill_tc).items():
        monkeypatch.setattr(ops, name, counted(name, fn))
