"""The Nipudra decoder as data: a scaled embedding; layers with a layer norm (gain and bias) before and after each
sublayer; three kinds of mixer in any order; a routed feed-forward (or none); a per-layer input from the token's row
of a side table after the sublayers; a final layer norm and a head tied to the embedding, its logits scaled and
soft-capped.

* mixer ``attention``: differential softmax attention over a sliding window: two maps per head over the same values,
  the second subtracted with a learned factor; biased projections; a short causal convolution on q, k and v; a
  rotation of the leading dims of each map whose slow frequencies are stretched; a layer may read the keys and values
  that an earlier layer cached.
* mixer ``mamba2``: a selective state-space recurrence with a matrix state per head.
* mixer ``retention``: linear attention with a constant decay per head, rotated queries and keys, a unit norm per
  head and a silu gate.
* feed-forward: experts up / relu squared / down, the softmax over the chosen router logits, a shared expert let in
  by one sigmoid gate per token.

This file only turns the configuration into a ModelSpec, layer by layer; all the computing is in ``pyre_b200.parts``.
"""

from __future__ import annotations

from ..config.model_config import NipudraConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec

SIDE_TABLE = "side.embed"      # [vocab, layers * side_dim]: layer i reads columns i * side_dim .. (i + 1) * side_dim


def build_nipudra(cfg: NipudraConfig) -> ModelSpec:
    def norm():
        return PartSpec("layer_norm", {"width": cfg.width, "eps": cfg.norm_eps, "tensor_name": "", "bias_name": ".b"})

    # a cache layer keeps what the widest window among its writer and its readers shows (None: every key)
    keep: dict = {}
    for i, L in enumerate(cfg.layers):
        if L.kind == "attention":
            src = L.kv_from if L.kv_from >= 0 else i
            seen = keep.get(src, 0)
            keep[src] = None if (seen is None or not L.window) else max(seen, L.window)
    blocks, schedule = [], []
    for i, L in enumerate(cfg.layers):
        call = LayerCall(i)
        if L.kind == "attention":
            position = None
            if L.rot_dims:
                scaling = dict(zip(("factor", "original", "fast", "slow"), L.rot_scaling)) if L.rot_scaling else None
                position = PartSpec("rotary", {"head_dim": L.dim, "theta": L.rot_base, "rotary_dim": L.rot_dims,
                                               "exact_frequencies": True, "scaling": scaling})
            shares = L.kv_from >= 0
            mixer = PartSpec("differential_attention", {
                "width": cfg.width, "n_heads": L.heads, "n_kv_heads": L.kv_heads, "head_dim": L.dim, "v_head_dim": L.vdim,
                "diff": L.diff, "eps": cfg.norm_eps, "scale": L.scale, "window": L.window or None, "position": position,
                "conv_taps": L.conv, "qkv_bias": True, "o_bias": True, "own_kv": not shares,
                "cache_window": keep[L.kv_from if shares else i]})
            call = LayerCall(i, cache=("layer", L.kv_from if shares else i), write=not shares)
        elif L.kind == "mamba2":
            mixer = PartSpec("mamba2", {"width": cfg.width, "n_heads": L.heads, "p_dim": L.vdim, "n_state": L.state,
                                        "n_groups": L.groups, "conv_taps": L.conv, "norm_groups": L.norm_groups,
                                        "eps": cfg.norm_eps})
        else:
            position = PartSpec("rotary", {"head_dim": L.dim, "theta": L.rot_base, "rotary_dim": L.rot_dims,
                                           "exact_frequencies": True}) if L.rot_dims else None
            mixer = PartSpec("decay_linear_attention", {
                "width": cfg.width, "n_heads": L.heads, "head_dim": L.dim, "v_head_dim": L.vdim, "decay": tuple(L.decay),
                "eps": cfg.norm_eps, "activation": None, "out_gate": True, "position": position, "k_scale": L.dim ** -0.5,
                "norm": "head", "norm_weight": False, "gate": "silu",
                "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}})
        params = {"width": cfg.width, "norm1": norm(), "mixer": mixer, "norm1b": norm(), "gated": False,
                  "names": {"norm1": "norm1", "norm1b": "norm1b", "mixer": "mix.", "norm2": "norm2", "norm2b": "norm2b",
                            "ffn": "mlp.", "after": "side."}}
        if L.mlp_kind == "moe":
            params["ffn"] = PartSpec("routed_mlp", {
                "width": cfg.width, "intermediate": L.ff, "n_experts": L.experts, "top": L.top, "activation": "relu2",
                "gated": False, "correction": False, "scores": "softmax", "renormalise": True, "router_bias": True,
                "shared": L.shared_ff or None, "shared_gate": bool(L.shared_ff)})
            params["norm2"], params["norm2b"] = norm(), norm()
        if cfg.side_dim:
            params["after"] = PartSpec("token_side_input", {
                "width": cfg.width, "dim": cfg.side_dim, "vocab": cfg.vocab, "table_name": SIDE_TABLE,
                "table_width": len(cfg.layers) * cfg.side_dim, "col": i * cfg.side_dim, "eps": cfg.norm_eps})
        blocks.append(PartSpec("sandwich", params))
        schedule.append(call)
    return ModelSpec(
        embed=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": "", "scale": cfg.embedding_scale}),
        blocks=blocks,
        final_norm=norm(),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": "", "tied_to": "embed",
                                      "logit_scale": cfg.logit_scale, "softcap": cfg.logit_softcap}),
        schedule=schedule,
        embed_prefix="embed", block_prefix="l{i}.", final_norm_prefix="final.norm", head_prefix="head",
        vocab_size=cfg.vocab,
        max_positions=0,
        width=cfg.width,
    )


register_architecture(NipudraConfig.architecture, NipudraConfig, build_nipudra)
