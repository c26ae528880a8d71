"""A plain, slow evaluation of the Nipudra decoder in float64, one function per mechanism, written from the
design's equations and sharing no code with the package.  A whole sequence at a time, no cache, no state carried:
every token's keys, values, convolution inputs and recurrent state are recomputed from the layer's input.

Weights are a dict name -> torch tensor (any dtype; widened here), the configuration is the dict that
``config.json`` holds.  ``lowp=True`` rounds to bfloat16 where an engine's bfloat16 path may (operands and results
of matrix products, short convolutions and their activations, cached keys and values, the heads' outputs); norms,
angles, scores, softmax weights, routers, decays, step sizes, the recurrences and the stream stay exact.  It measures
what rounding alone costs.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _r(x, lowp):
    return x.to(torch.bfloat16).to(F64) if lowp else x


def matmul(x, w, lowp=False, bias=None):
    """x W^T (+ bias) for a weight stored [out, in]."""
    y = _r(x, lowp) @ w.to(F64).T
    if bias is not None:
        y = y + bias.to(F64)
    return _r(y, lowp)


def layer_norm(x, gain, bias, eps):
    """(x - mean) / sqrt(var + eps) * gain + bias over the last axis; var is the mean squared deviation."""
    dev = x - x.mean(-1, keepdim=True)
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * gain.to(F64) + bias.to(F64)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_convolution(u, taps_w, bias=None):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j) per channel, zeros before the first token.  u [T, C], w [C, taps]."""
    T, C = u.shape
    w = taps_w.to(F64)
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), u], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias.to(F64)
    return y


def rotary_frequencies(base, dims, scaling=None):
    """(f_i for i < dims / 2, amplitude).  Plain: f_i = base^(-2i / dims), amplitude 1.  With ``scaling`` {factor,
    original, fast, slow}: the pair index at which a wave turns t times within ``original`` positions is
    d(t) = dims ln(original / (2 pi t)) / (2 ln base); between lo = floor(d(fast)) and hi = ceil(d(slow)) (clipped to
    the pairs' range) a ramp from 0 to 1 blends f_i into f_i / factor; cos and sin are multiplied by
    0.1 ln(factor) + 1."""
    freqs = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return freqs, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_index(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(float(base)))
    lo = max(math.floor(turn_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_index(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(v, positions, freqs, amplitude=1.0):
    """v [T, n, d]: dim i pairs with dim i + R/2 over the leading R = 2 len(freqs) dims; the rest pass."""
    half = len(freqs)
    ang = positions.to(F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    cos, sin = (torch.cos(ang) * amplitude)[:, None, :], (torch.sin(ang) * amplitude)[:, None, :]
    a, b = v[..., :half], v[..., half:2 * half]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., 2 * half:]], dim=-1)


def windowed_softmax(scores, window):
    """scores [T, T]: row i keeps columns j with 0 <= i - j < window."""
    T = scores.shape[0]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & (i - j < window)
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)


def projected(h, w, name, lowp):
    """A biased projection, then its short convolution when the layer has one (``<name>.conv``)."""
    y = matmul(h, w[name], lowp, w[name + ".b"])
    return _r(short_convolution(y, w[name + ".conv"]), lowp) if name + ".conv" in w else y


def map_frequencies(mixer):
    rot = mixer.get("rot") or {}
    return rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling")) if rot.get("dims") else ([], 1.0)


def attention_keys_values(h, w, prefix, mixer, positions, lowp=False):
    """What a layer caches: keys after convolution and rotation [T, G, 2, dim], values after convolution [T, G, vdim]."""
    G, dim, vdim = mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    k, v = projected(h, w, prefix + "k", lowp), projected(h, w, prefix + "v", lowp)
    freqs, amp = map_frequencies(mixer)
    k = rotate_halves(k.reshape(T, 2 * G, dim), positions, freqs, amp).reshape(T, G, 2, dim)
    return _r(k, lowp), v.reshape(T, G, vdim)


def differential_attention(h, w, prefix, mixer, eps, keys, values, lowp=False):
    """Two softmax maps per head over the same values: o = a1 - lambda a2, unit norm over the head's values,
    times (1 - diff).  ``keys`` / ``values``: what this layer or the layer it reads from caches."""
    H, G, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    positions = torch.arange(T)
    q = projected(h, w, prefix + "q", lowp)
    freqs, amp = map_frequencies(mixer)
    q = _r(rotate_halves(q.reshape(T, 2 * H, dim), positions, freqs, amp), lowp).reshape(T, H, 2, dim)
    f = lambda name: w[prefix + name].to(F64)
    lam = math.exp(float((f("lq1") * f("lk1")).sum())) - math.exp(float((f("lq2") * f("lk2")).sum())) + mixer["diff"]
    heads = []
    for n in range(H):
        g = n // (H // G)
        maps = []
        for m in range(2):
            p = windowed_softmax(q[:, n, m] @ keys[:, g, m].T * mixer["scale"], (mixer.get("mask") or {}).get("size") or T)
            maps.append(_r(p, lowp) @ values[:, g])
        o = maps[0] - lam * maps[1]
        heads.append(unit_rms(o, eps) * (1.0 - mixer["diff"]))
    return matmul(torch.cat(heads, dim=-1), w[prefix + "o"], lowp, w[prefix + "o.b"])


def retention(h, w, prefix, mixer, eps, lowp=False):
    """S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head; unit norm per head; silu gate; projection."""
    H, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    positions = torch.arange(T)
    freqs, _ = map_frequencies(mixer)
    q = _r(rotate_halves(matmul(h, w[prefix + "q"], lowp).reshape(T, H, dim), positions, freqs), lowp)
    k = _r(rotate_halves(matmul(h, w[prefix + "k"], lowp).reshape(T, H, dim), positions, freqs) * dim ** -0.5, lowp)
    v = matmul(h, w[prefix + "v"], lowp).reshape(T, H, vdim)
    out = torch.zeros(T, H, vdim, dtype=F64)
    for n in range(H):
        S = torch.zeros(dim, vdim, dtype=F64)
        for t in range(T):
            S = float(mixer["decay"][n]) * S + k[t, n][:, None] * v[t, n][None, :]
            out[t, n] = S.T @ q[t, n]
    out = unit_rms(out, eps).reshape(T, H * vdim) * silu(matmul(h, w[prefix + "g"], lowp))
    return matmul(out, w[prefix + "o"], lowp)


def selective_scan(x, dt, A, B, C, D):
    """Per head: S_t = exp(-A dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t.
    x [T, H, P], dt [T, H], A, D [H], B, C [T, H, N] (already spread from groups to heads)."""
    T, H, P = x.shape
    y = torch.zeros(T, H, P, dtype=F64)
    for n in range(H):
        S = torch.zeros(B.shape[-1], P, dtype=F64)
        for t in range(T):
            S = torch.exp(-A[n] * dt[t, n]) * S + dt[t, n] * B[t, n][:, None] * x[t, n][None, :]
            y[t, n] = S.T @ C[t, n] + D[n] * x[t, n]
    return y


def mamba2(h, w, prefix, mixer, eps, lowp=False):
    H, P, N, G = mixer["heads"], mixer["vdim"], mixer["state"], mixer["groups"]
    inner, T = H * P, h.shape[0]
    proj = matmul(h, w[prefix + "in"], lowp)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = _r(silu(short_convolution(xbc, w[prefix + "conv"], w[prefix + "conv.b"])), lowp)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    dt = softplus(dt + w[prefix + "dt_bias"].to(F64))
    y = selective_scan(x, dt, torch.exp(w[prefix + "A_log"].to(F64)), B, C, w[prefix + "D"].to(F64))
    y = y.reshape(T, inner) * silu(z)
    parts = mixer["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[prefix + "norm"].to(F64)
    return matmul(y, w[prefix + "o"], lowp)


def relu2(z):
    return torch.relu(z) ** 2


def expert(x, w, prefix, lowp=False):
    return matmul(_r(relu2(matmul(x, w[prefix + "up"], lowp)), lowp), w[prefix + "down"], lowp)


def router_logits(h, w, prefix):
    return h @ w[prefix + "router"].to(F64).T + w[prefix + "router.b"].to(F64)


def moe_mlp(h, w, prefix, mlp, lowp=False, margins=None):
    """The ``top`` largest router logits choose; the weights are the softmax over the chosen logits; a shared
    expert times sigmoid(w_sg . h) is added.  ``margins``: a list that receives, per token, the gap between the
    last chosen and the first refused logit."""
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = router_logits(_r(h, lowp), w, prefix)
    order = torch.argsort(z, dim=-1, descending=True, stable=True)
    if margins is not None and top < n:
        zs = torch.gather(z, 1, order)
        margins.extend((zs[:, top - 1] - zs[:, top]).tolist())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = order[t, :top]
        weights = torch.softmax(z[t, chosen], dim=-1)
        for e, wt in zip(chosen.tolist(), weights):
            out[t] = out[t] + wt * expert(h[t:t + 1], w, f"{prefix}e{e}.", lowp)[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(_r(h, lowp) @ w[prefix + "shared.sg"].to(F64).T)
        out = out + gate * expert(h, w, prefix + "shared.", lowp)
    return out


def token_side_input(x, tokens, w, prefix, layer, dim, eps, lowp=False):
    """x + unit_rms(W_proj (gelu_tanh(W_gate x) * e)) * gain, e the layer's slice of the token's side embedding."""
    e = w["side.embed"].to(F64)[tokens][:, layer * dim:(layer + 1) * dim]
    g = _r(gelu_tanh(matmul(x, w[prefix + "gate"], lowp)) * e, lowp)
    y = matmul(g, w[prefix + "proj"], lowp)
    return x + unit_rms(y, eps) * w[prefix + "norm"].to(F64)


def forward(config, w, tokens, lowp=False, keep_layers=False, margins=None):
    """Logits [T, vocab] of one sequence (and the stream after every layer with ``keep_layers``)."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    x = w["embed"].to(F64)[tokens] * (config.get("embedding") or {}).get("scale", 1.0)
    side = config.get("token_side")
    cached, streams = {}, []
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        norm = lambda name, v: layer_norm(v, w[p + name], w[p + name + ".b"], eps)
        h = norm("norm1", x)
        mixer = L["mixer"]
        if L["type"] == "attention":
            src = mixer.get("kv_from")
            if src is None:
                cached[i] = attention_keys_values(h, w, p + "mix.", mixer, positions, lowp)
                src = i
            y = differential_attention(h, w, p + "mix.", mixer, eps, *cached[src], lowp=lowp)
        elif L["type"] == "mamba2":
            y = mamba2(h, w, p + "mix.", mixer, eps, lowp)
        elif L["type"] == "retention":
            y = retention(h, w, p + "mix.", mixer, eps, lowp)
        else:
            raise ValueError(f"layer {i}: unknown type {L['type']!r}")
        x = x + norm("norm1b", y)
        if L.get("mlp"):
            x = x + norm("norm2b", moe_mlp(norm("norm2", x), w, p + "mlp.", L["mlp"], lowp, margins))
        if side:
            x = token_side_input(x, tokens, w, p + "side.", i, side["dim"], eps, lowp)
        streams.append(x.clone())
    h = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = matmul(h, w["embed"], lowp) * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if keep_layers else logits
