"""A plain, slow evaluation of the Tekarax decoder in float64, one function per mechanism, written from the
design's equations and sharing no code with the package.  A whole sequence at a time, no cache, no state carried:
every token's keys, values and recurrent state are recomputed from the layer's input.

Weights are a dict name -> torch tensor (any dtype; widened here), the configuration is the dict that
``config.json`` holds.  ``lowp=True`` rounds to bfloat16 where an engine's bfloat16 path may (operands and results
of matrix products and their activations, cached keys, values and latents, the heads' outputs); norms, angles,
scores, softmax weights, routers, decays, the recurrence and the stream stay exact.  It measures what rounding
alone costs.
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


def layer_norm(x, gain, eps):
    """(x - mean) / sqrt(var + eps) * gain over the last axis; var is the mean squared deviation; no bias."""
    dev = x - x.mean(-1, keepdim=True)
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * gain.to(F64)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def scaled_frequencies(base, dims, scaling=None):
    """f_i = base^(-2i / dims), i < dims / 2; with ``scaling`` {factor, low, high, original} a frequency whose
    wavelength 2 pi / f is longer than original / low is divided by factor, one shorter than original / high is
    kept, and the ones between are blended linearly in original / wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave > orig / lo:
                f = f / fac
            elif wave >= orig / hi:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_halves(v, positions, freqs, sign=1.0):
    """Pairs (v[i], v[i + n]) with n = len(freqs) turn by sign * p * freqs[i]; entries from 2 n on stay.
    ``v`` [T, ..., d], ``positions`` [T]."""
    n = freqs.shape[0]
    ang = sign * positions.to(F64)[:, None] * freqs[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [n]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = v[..., :n], v[..., n:2 * n]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., 2 * n:]], dim=-1)


def softmax_with_sink(scores, sink=None):
    """Softmax over the last axis whose denominator holds one more term, exp(sink): a sink has a score (as it is, not
    scaled) and no value, so the weights of a row sum to less than one."""
    m = scores.max(-1, keepdim=True).values
    if sink is None:
        e = torch.exp(scores - m)
        return e / e.sum(-1, keepdim=True)
    m = torch.maximum(m, torch.as_tensor(sink, dtype=scores.dtype).expand_as(m))
    e = torch.exp(scores - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def attention(h, w, prefix, mixer, lowp=False):
    """Grouped-query softmax attention, causal, with rotated queries and keys (leading dims, scaled frequencies),
    values rotated by their own position over all their dims and each head's sum turned back by the query's position,
    a learned sink per head in the denominator, and one sigmoid gate per head.  ``h`` [T, width] from position 0."""
    T = h.shape[0]
    H, dk = mixer["heads"], mixer["dim"]
    G = int(mixer.get("kv_heads") or H)
    dv = int(mixer.get("vdim") or dk)
    g = lambda n: w[prefix + n].to(F64)
    pos = torch.arange(T)
    q = matmul(h, g("q"), lowp).view(T, H, dk)
    k = matmul(h, g("k"), lowp).view(T, G, dk)
    v = matmul(h, g("v"), lowp).view(T, G, dv)
    rot = mixer.get("rot")
    if rot:
        fq = scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        fv = scaled_frequencies(rot["base"], dv)
        q, k, v = rotate_halves(q, pos, fq), rotate_halves(k, pos, fq), rotate_halves(v, pos, fv)
    q, k, v = _r(q, lowp), _r(k, lowp), _r(v, lowp)
    sink = g("sink") if prefix + "sink" in w else None
    out = torch.zeros(T, H, dv, dtype=F64)
    causal = pos[:, None] >= pos[None, :]
    for n in range(H):
        kv = n // (H // G)
        s = (q[:, n] @ k[:, kv].T) * mixer["scale"]
        s = s.masked_fill(~causal, -math.inf)
        out[:, n] = softmax_with_sink(s, sink[n] if sink is not None else None) @ v[:, kv]
    if rot:
        out = rotate_halves(out, pos, fv, sign=-1.0)
    if prefix + "g" in w:
        out = out * torch.sigmoid(matmul(h, g("g"), lowp))[:, :, None]
    return matmul(_r(out, lowp).reshape(T, H * dv), g("o"), lowp)


def latent_attention(h, w, prefix, mixer, eps, lowp=False):
    """Softmax attention over a sliding window, without positions, whose keys and values are expanded per head
    from one normed low-rank latent per token."""
    T = h.shape[0]
    H, dk = mixer["heads"], mixer["dim"]
    dv = int(mixer.get("vdim") or dk)
    g = lambda n: w[prefix + n].to(F64)
    q = matmul(h, g("q"), lowp).view(T, H, dk)
    c = _r(unit_rms(matmul(h, g("dkv"), lowp), eps) * g("dkv.norm"), lowp)
    k = matmul(c, g("uk"), lowp).view(T, H, dk)
    v = matmul(c, g("uv"), lowp).view(T, H, dv)
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    size = (mixer.get("mask") or {}).get("size")
    if size:
        seen = seen & (dist < int(size))
    out = torch.zeros(T, H, dv, dtype=F64)
    for n in range(H):
        s = ((q[:, n] @ k[:, n].T) * mixer["scale"]).masked_fill(~seen, -math.inf)
        out[:, n] = torch.softmax(s, dim=-1) @ v[:, n]
    return matmul(_r(out, lowp).reshape(T, H * dv), g("o"), lowp)


def token_blend(h, mu, before=None):
    """h_t + (h_(t-1) - h_t) * mu; the row before the first is ``before`` (zeros when a sequence begins)."""
    first = torch.zeros(1, h.shape[1], dtype=h.dtype) if before is None else before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], dim=0)
    return h + (prev - h) * mu


def wkv_recurrence(r, k, v, decay, u, S=None):
    """Per head n: o_t = (S + diag(u) k_t v_t^T)^T r_t, then S = diag(decay_t) S + k_t v_t^T.  r, k, v, decay
    [T, H, d]; u [H, d]; S [H, d, d] (zeros when a sequence begins).  Returns (o [T, H, d], the state after)."""
    T, H, d = r.shape
    S = torch.zeros(H, d, d, dtype=r.dtype) if S is None else S.clone()
    out = torch.zeros(T, H, d, dtype=r.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    return out, S


def wkv(h, w, prefix, mixer, eps, lowp=False):
    """Time mixing with a matrix state per head: each of r, k, v, g, w reads its own blend of the token's input and
    the previous token's; a decay per head and key channel from a small two-layer map; the current token's key-value
    product enters the output with a bonus u and the state without."""
    T, width = h.shape
    H, d = mixer["heads"], mixer["dim"]
    g = lambda n: w[prefix + n].to(F64)
    mix = lambda s: _r(token_blend(h, g("mu." + s)), lowp)
    r = matmul(mix("r"), g("r"), lowp).view(T, H, d)
    k = matmul(mix("k"), g("k"), lowp).view(T, H, d)
    v = matmul(mix("v"), g("v"), lowp).view(T, H, d)
    gate = _r(silu(matmul(mix("g"), g("g"), lowp)), lowp)
    inner = _r(torch.tanh(matmul(mix("w"), g("w1"), lowp)), lowp)
    decay = torch.exp(-torch.exp(_r(inner, lowp) @ g("w2").T + g("w0"))).view(T, H, d)
    u = g("u").view(H, d)
    out, _ = wkv_recurrence(r, k, v, decay, u)
    out = unit_rms(out, eps).reshape(T, H * d) * g("norm") * gate
    return matmul(_r(out, lowp), g("o"), lowp)


def relu2(z):
    return torch.relu(z) ** 2


def dense_mlp(h, w, prefix, lowp=False):
    a = _r(relu2(matmul(h, w[prefix + "up"], lowp, bias=w[prefix + "up.b"])), lowp)
    return matmul(a, w[prefix + "down"], lowp, bias=w[prefix + "down.b"])


def gated_expert(x, w, prefix, lowp=False):
    a = _r(silu(matmul(x, w[prefix + "gate"], lowp)) * matmul(x, w[prefix + "up"], lowp), lowp)
    return matmul(a, w[prefix + "down"], lowp)


def router_scores(h, w, prefix):
    return torch.sigmoid(h @ w[prefix + "router"].to(F64).T)


def moe_mlp(h, w, prefix, mlp, lowp=False, margins=None):
    """Each token's ``top`` experts by sigmoid score; the score multiplies the expert's INPUT; a shared expert runs
    for every token.  ``margins`` (a list) receives, per token, the gap between the last chosen score and the first
    one left out."""
    scores = router_scores(_r(h, lowp), w, prefix)
    top = int(mlp["router"]["top"])
    choice = scores.topk(top, dim=-1).indices
    if margins is not None and top < scores.shape[-1]:
        ranked = scores.sort(dim=-1, descending=True).values
        margins.extend((ranked[:, top - 1] - ranked[:, top]).tolist())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in choice[t].tolist():
            out[t] += gated_expert((scores[t, e] * h[t])[None], w, f"{prefix}e{e}.", lowp)[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, w, prefix + "shared.", lowp)
    return out


def layer_order(config):
    """(layer, pass number or None) in the order the layers run; the first layer of each pass carries the number."""
    n = len(config["layers"])
    loop = config.get("loop") or {}
    start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
    if not loop or stop <= start:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(config, w, tokens, lowp=False, keep_layers=False, margins=None):
    """Logits [T, vocab] of one sequence from position 0 (and, with ``keep_layers``, the stream after every layer run)."""
    eps = float(config["norm"]["eps"])
    x = w["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    kept = []
    for i, step in layer_order(config):
        L = config["layers"][i]
        p = f"l{i}."
        if step is not None:
            x = x + w["loop.step"].to(F64)[step]
        h = _r(layer_norm(x, w[p + "norm1"], eps), lowp)
        if L["type"] == "attention":
            m = attention(h, w, p + "mix.", L["mixer"], lowp)
        elif L["type"] == "latent_attention":
            m = latent_attention(h, w, p + "mix.", L["mixer"], eps, lowp)
        elif L["type"] == "wkv":
            m = wkv(h, w, p + "mix.", L["mixer"], eps, lowp)
        else:
            raise ValueError(L["type"])
        m = m * torch.sigmoid(matmul(h, w[p + "rg1"], lowp, bias=w[p + "rg1.b"]))
        x = x + layer_norm(m, w[p + "norm1b"], eps)
        mlp = L.get("mlp")
        if mlp:
            h = _r(layer_norm(x, w[p + "norm2"], eps), lowp)
            f = dense_mlp(h, w, p + "mlp.", lowp) if mlp.get("kind", "dense") == "dense" else moe_mlp(h, w, p + "mlp.", mlp, lowp, margins)
            f = f * torch.sigmoid(matmul(h, w[p + "rg2"], lowp, bias=w[p + "rg2.b"]))
            x = x + layer_norm(f, w[p + "norm2b"], eps)
        if keep_layers:
            kept.append(x.clone())
    logits = matmul(_r(layer_norm(x, w["final.norm"], eps), lowp), w["head"], lowp)
    return (logits, torch.stack(kept)) if keep_layers else logits
