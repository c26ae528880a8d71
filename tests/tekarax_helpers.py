"""Fixtures of the Tekarax tests: small configurations that differ in every size and option, model folders with
random weights, and the plain implementation's logits."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import load_file, save_file

import math

from plain import tekarax_plain


def _attn(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}}


def _latent(heads, dim, vdim, kv_rank, scale, window):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def _wkv(heads, dim, decay_rank):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}}


def _with(layer, mlp=None):
    return dict(layer, mlp=mlp)


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# A: a span in the middle (layers 1-2: a recurrent and a windowed layer) that runs three times; value heads wider than
#    key heads; a rotation of half of each head whose stretching already matters at a few dozen tokens (original 32);
#    a window of 11 on pages of 16; one layer without a feed-forward; two of five experts plus a shared one.
TEK_A = {"architecture": "Tekarax", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
         "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    _with(_attn(4, 2, 16, 24, 0.3, 8, 100.0, (8.0, 1.0, 4.0, 32)), _dense(160)),
    _with(_wkv(3, 16, 8), _moe(32, 5, 2, 48)),
    _with(_latent(3, 16, 24, 24, 0.3, 11)),
    _with(_wkv(2, 24, 16), _dense(72)),
]}
# B: no size is a multiple of 8 (width 92: the library product for odd K and the scalar paths), as many key/value
#    heads as query heads, value heads smaller than key heads, no stretching, a decay map of 12, heads x dim of the
#    recurrent layer below and above the width, a window of 7 on pages of 8, all three experts chosen, no span.
TEK_B = {"architecture": "Tekarax", "vocab": 333, "width": 92, "norm": {"eps": 3e-6}, "layers": [
    _with(_wkv(4, 20, 12), _moe(20, 3, 3)),
    _with(_attn(5, 5, 20, 12, 0.25, 12, 500.0), _dense(66)),
    _with(_latent(5, 20, 12, 36, 0.2, 7), _moe(28, 4, 1, 20)),
    _with(_wkv(5, 28, 12)),
]}
# C: sizes of the tensor-core paths: heads of 64 over four key/value heads, a latent of 192, recurrent heads of 64, a
#    window of 64 on pages of 32, the first two layers twice, feed-forwards wide enough for the fused products.
TEK_C = {"architecture": "Tekarax", "vocab": 640, "width": 256, "norm": {"eps": 1e-6},
         "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
    _with(_latent(8, 64, 64, 192, 0.12, 64), _moe(128, 8, 2, 256)),
    _with(_attn(8, 4, 64, 64, 0.12, 64, 500000.0, (3.0, 1.0, 4.0, 256)), _dense(512)),
    _with(_wkv(4, 64, 32), _dense(512)),
]}
# D: one key/value head under six query heads of 128 with values of 64 and a rotation of a quarter of the head; one
#    expert of which one is chosen; recurrent heads of 128 (the largest the recurrence takes); a window wider than any
#    request; the last layer alone repeated.
TEK_D = {"architecture": "Tekarax", "vocab": 256, "width": 128, "norm": {"eps": 1e-5},
         "loop": {"start": 2, "stop": 3, "times": 2}, "layers": [
    _with(_attn(6, 1, 128, 64, 0.09, 32, 10000.0, (2.0, 1.0, 2.0, 64)), _moe(64, 1, 1)),
    _with(_latent(2, 48, 40, 64, 0.15, 100000), _dense(128)),
    _with(_wkv(1, 128, 24), _moe(32, 6, 2, 64)),
]}
TEK = {"A": TEK_A, "B": TEK_B, "C": TEK_C, "D": TEK_D}
TEK_PAGE_SIZE = {"A": 16, "B": 8, "C": 32, "D": 16}
NEIGHBOURS = 8
ROUTER_MARGIN = 2e-2     # a router decision closer than this could fall either way under bfloat16 rounding of the stream


def make_tekarax_dir(path: Path, raw: dict, seed: int, sharpen: float = 4.0, matrix_scale: float = 2.0) -> dict:
    """config.json + model.safetensors (fp32 values that bfloat16 holds exactly) from the package's random mode.
    The maps that make queries and keys are scaled up so that attention is peaked (with small random weights every
    score is near zero and a wrong key would change nothing), the router's so that its scores differ without
    saturating."""
    from pyre_b200.config import config_from_dict
    from pyre_b200.weights import random_state

    path.mkdir(parents=True, exist_ok=True)
    state = random_state(config_from_dict(raw), seed)
    kinds = {f"l{i}.": L["type"] for i, L in enumerate(raw["layers"])}
    for name in state:
        kind = kinds.get(name.split("mix.")[0]) if ".mix." in name else None
        if kind in ("attention", "latent_attention") and name.endswith((".mix.q", ".mix.k", ".mix.dkv")):
            state[name] = state[name] * sharpen
        elif name.endswith(".mlp.router"):
            state[name] = state[name] * (30.0 / raw["width"] ** 0.5)      # logits of order one: sigmoid scores that differ
        elif name.endswith(".mix.w2") or name == "loop.step":
            pass
        elif state[name].dim() == 2 and not name.endswith(".mix.u"):
            state[name] = state[name] * matrix_scale
        state[name] = state[name].to(torch.bfloat16).to(torch.float32)
    (path / "config.json").write_text(json.dumps(raw))
    save_file({k: v.contiguous() for k, v in state.items()}, str(path / "model.safetensors"))
    return state


def decided_ids(path: Path, length: int, seed: int, chunk: int = 4) -> list:
    """Random token ids on which no router decision of the model is a close call: grown a few tokens at a time, a
    piece drawn again while any decision at its positions is closer than ROUTER_MARGIN (a decision depends on the
    tokens up to its own only).  A model without routers gets plain random ids."""
    raw = json.loads((Path(path) / "config.json").read_text())
    rng = np.random.default_rng(seed)
    routed = [L for L in raw["layers"] if (L.get("mlp") or {}).get("kind") == "moe"
              and L["mlp"]["router"]["top"] < L["mlp"]["router"]["experts"]]
    if not routed:
        return [int(x) for x in rng.integers(0, raw["vocab"], length)]
    w = load_file(str(Path(path) / "model.safetensors"))
    ids: list = []
    while len(ids) < length:
        n = min(chunk, length - len(ids))
        for _ in range(200):
            piece = [int(x) for x in rng.integers(0, raw["vocab"], n)]
            margins: list = []
            with torch.inference_mode():
                tekarax_plain.forward(raw, w, ids + piece, margins=margins)
            T = len(ids) + n
            per_run = np.asarray(margins).reshape(-1, T)[:, -n:]       # one row per run of a routed layer
            if per_run.size == 0 or per_run.min() > ROUTER_MARGIN:
                break
        else:
            raise AssertionError("no piece of tokens gave decided router choices")
        ids += piece
    return ids


def plain_logits(path: Path, ids, lowp: bool = False) -> np.ndarray:
    raw = json.loads((Path(path) / "config.json").read_text())
    w = load_file(str(Path(path) / "model.safetensors"))
    with torch.inference_mode():
        return tekarax_plain.forward(raw, w, list(ids), lowp=lowp).numpy()


def compare(got: dict, want: dict, dtype: str, what: str, lowp_rms: float = 0.0, lowp: "dict | None" = None):
    """float32: every logit within rounding of the plain implementation (sums in another order through up to eight
    layer runs).  bfloat16: the engine's rms error against the plain implementation is at most twice that of the plain
    implementation rounded to bfloat16 where the engine may round (``lowp``, its logits per request), and no logit is
    off by more than sixteen times that rms plus three times the rounded plain implementation's own largest error at
    that position or one of its eight neighbours on either side (what rounding does at one position is a matter of
    chance; its neighbours show what it can do in that part of the sequence): where a sublayer's result is small (the first tokens of a recurrent layer, whose state is still
    nearly empty) the norm after it enlarges every rounding, for both alike, while a wrong key, page, slot or
    position moves logits by their whole spread at positions of every kind."""
    assert set(got) == set(want), f"{what}: requests differ"
    sq, cnt = 0.0, 0
    for rid in want:
        g, w = got[rid], want[rid]
        assert g.shape == w.shape, f"{what} {rid}: shape {g.shape} != {w.shape}"
        assert np.isfinite(g).all(), f"{what} {rid}: non-finite logits at rows {np.unique(np.where(~np.isfinite(g))[0])[:8]}"
        err = np.abs(g - w)
        if dtype == "float32":
            bound = 1e-4 + 2e-4 * np.abs(w)
        else:
            own = 0.0
            if lowp is not None:
                rows = np.abs(lowp[rid] - w).max(axis=1)
                own = np.array([rows[max(0, i - NEIGHBOURS):i + NEIGHBOURS + 1].max() for i in range(len(rows))])[:, None]
            bound = np.broadcast_to(16.0 * lowp_rms + 3.0 * own, w.shape)
        sq, cnt = sq + float((err.astype(np.float64) ** 2).sum()), cnt + err.size
        bad = err > bound
        if bad.any():
            row = int(np.where(bad.any(axis=1))[0][0])
            raise AssertionError(f"{what} {rid} ({dtype}): first wrong token at position {row} of {g.shape[0]}; "
                                 f"max |diff| there {err[row].max():.3e}, bound {bound[row].max():.3e}, "
                                 f"overall max {err.max():.3e}, logits std {w.std():.3f}")
    if dtype == "bfloat16":
        rms = math.sqrt(sq / cnt)
        assert rms <= 2.0 * lowp_rms, f"{what} (bfloat16): rms error {rms:.3e} against {lowp_rms:.3e} of plain rounding"
