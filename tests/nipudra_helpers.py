"""Fixtures of the Nipudra tests: small configurations that differ in every size and option, model folders with
random weights, and the plain implementation's logits."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import load_file, save_file

from plain import nipudra_plain
from tekarax_helpers import compare  # noqa: F401  (the same bounds serve: see its docstring)


def attn(heads, kv_heads, dim, vdim, scale, diff, conv=0, window=0, rot_dims=0, base=10000.0, scaling=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if conv:
        m["conv"] = conv
    if window:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def retention(heads, dim, vdim, decay, rot_dims=0, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "retention", "mixer": m}


def with_mlp(layer, mlp=None):
    return dict(layer, mlp=mlp)


def moe(ff, experts, top, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# A: value heads wider than key heads; a rotation of half of each map whose stretching already matters at a few dozen
#    tokens; a window of 11 on pages of 16 whose reader (layer 3) looks back 29; convolutions of 3 and 2 taps; a
#    state-space layer without a feed-forward; two of five experts plus a shared one; a side table of 8 per layer.
NIP_A = {"architecture": "Nipudra", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
         "logit_scale": 0.5, "logit_softcap": 20.0, "token_side": {"dim": 8}, "layers": [
    with_mlp(attn(4, 2, 16, 24, 0.3, 0.25, 3, 11, 8, 100.0, (8.0, 32, 4.0, 1.0)), moe(32, 5, 2, 48)),
    with_mlp(mamba(3, 16, 12, 1, 4, 3)),
    with_mlp(retention(3, 16, 24, (0.9, 0.97, 0.995), 16, 1000.0), moe(24, 4, 1)),
    with_mlp(attn(4, 2, 16, 24, 0.35, 0.4, 2, 29, 8, 100.0, (8.0, 32, 4.0, 1.0), kv_from=0), moe(40, 3, 2, 16)),
]}
# B: no size is a multiple of 8 (width 92: the library product for odd K and the scalar paths); as many key/value heads
#    as query heads; value heads smaller than key heads; attention without convolution, window or rotation beside
#    attention with a window of 7 on pages of 8; a state of 20 rows (no multiple of 4) in four groups; all three experts
#    chosen; no side table, no cap, factors of one.
NIP_B = {"architecture": "Nipudra", "vocab": 333, "width": 92, "norm": {"eps": 3e-6}, "layers": [
    with_mlp(retention(5, 20, 12, (0.5, 0.8, 0.9, 0.99, 1.0), 12, 500.0), moe(20, 3, 3)),
    with_mlp(attn(5, 5, 20, 12, 0.25, 0.1), moe(28, 4, 1, 20)),
    with_mlp(mamba(4, 20, 20, 4, 2, 1), moe(28, 6, 3)),
    with_mlp(attn(6, 3, 12, 20, 0.3, 0.5, 5, 7, 12, 50.0)),
]}
# C: sizes of the tensor-core paths: maps of 64 over two key/value heads, retention heads of 64, a state of 64 rows under
#    heads of 64, a window of 64 on pages of 32, feed-forwards wide enough for the fused products; the reader's window
#    is smaller than the writer's.
NIP_C = {"architecture": "Nipudra", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 16.0},
         "logit_scale": 0.125, "logit_softcap": 50.0, "token_side": {"dim": 16}, "layers": [
    with_mlp(mamba(8, 64, 64, 2, 4, 2), moe(128, 8, 2, 256)),
    with_mlp(attn(4, 2, 64, 64, 0.12, 0.2, 4, 64, 64, 500000.0, (3.0, 256, 16.0, 2.0)), moe(128, 8, 2, 256)),
    with_mlp(retention(4, 64, 64, (0.96, 0.98, 0.99, 0.999), 32, 10000.0), moe(64, 4, 2)),
    with_mlp(attn(4, 2, 64, 64, 0.12, 0.2, 4, 48, 64, 500000.0, (3.0, 256, 16.0, 2.0), kv_from=1), moe(128, 8, 2, 256)),
]}
# D: one key/value head under six query heads with maps of 48 and values of 40; one expert of which one is chosen; a
#    state of 128 rows; one retention head of 128; a window wider than any request; a side table of 12.
NIP_D = {"architecture": "Nipudra", "vocab": 256, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
         "logit_scale": 2.0, "token_side": {"dim": 12}, "layers": [
    with_mlp(attn(6, 1, 48, 40, 0.09, 0.6, 4, 100000, 16, 10000.0, (2.0, 64, 8.0, 0.5)), moe(64, 1, 1)),
    with_mlp(retention(1, 128, 64, (0.98,)), moe(32, 6, 2, 64)),
    with_mlp(mamba(2, 40, 128, 2, 3, 4), moe(32, 6, 2, 64)),
]}
NIP = {"A": NIP_A, "B": NIP_B, "C": NIP_C, "D": NIP_D}
NIP_PAGE_SIZE = {"A": 16, "B": 8, "C": 32, "D": 16}
ROUTER_MARGIN = 0.15     # a router decision closer than this could fall either way under bfloat16 rounding of the stream


def make_nipudra_dir(path: Path, raw: dict, seed: int, sharpen: float = 4.0, matrix_scale: float = 2.0) -> dict:
    """config.json + model.safetensors (fp32 values that bfloat16 holds exactly) from the package's random mode.
    The maps that make queries and keys are scaled up so that attention is peaked (with small random weights every
    score is near zero and a wrong key would change nothing), the router's so that its logits differ."""
    from pyre_b200.config import config_from_dict
    from pyre_b200.weights import random_state

    path.mkdir(parents=True, exist_ok=True)
    state = random_state(config_from_dict(raw), seed)
    kinds = {f"l{i}.": L["type"] for i, L in enumerate(raw["layers"])}
    for name in state:
        kind = kinds.get(name.split("mix.")[0]) if ".mix." in name else None
        if kind == "attention" and name.endswith((".mix.q", ".mix.k")):
            state[name] = state[name] * sharpen
        elif name.endswith(".mlp.router"):
            state[name] = state[name] * (60.0 / raw["width"] ** 0.5)      # logits that lie well apart
        elif state[name].dim() == 2 and not name.endswith((".conv", "side.embed", ".shared.sg")):
            state[name] = state[name] * matrix_scale
        state[name] = state[name].to(torch.bfloat16).to(torch.float32)
    (path / "config.json").write_text(json.dumps(raw))
    save_file({k: v.contiguous() for k, v in state.items()}, str(path / "model.safetensors"))
    return state


def decided_ids(path: Path, length: int, seed: int, chunk: int = 4) -> list:
    """Random token ids on which no router decision of the model is a close call: grown a few tokens at a time, a
    piece drawn again while any decision at its positions is closer than ROUTER_MARGIN (a decision depends on the
    tokens up to its own only)."""
    raw = json.loads((Path(path) / "config.json").read_text())
    rng = np.random.default_rng(seed)
    w = load_file(str(Path(path) / "model.safetensors"))
    ids: list = []
    while len(ids) < length:
        n = min(chunk, length - len(ids))
        for _ in range(200):
            piece = [int(x) for x in rng.integers(0, raw["vocab"], n)]
            margins: list = []
            with torch.inference_mode():
                nipudra_plain.forward(raw, w, ids + piece, margins=margins)
            T = len(ids) + n
            per_run = np.asarray(margins).reshape(-1, T)[:, -n:]       # one row per routed layer that has a choice
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
        return nipudra_plain.forward(raw, w, list(ids), lowp=lowp).numpy()
