"""The Tekarax decoder as data: layers with a layer norm before and after each sublayer and a sigmoid gate per feature
on the sublayer's result; three kinds of mixer in any order; a span of layers that runs several times in a row with
the same weights, every pass with a cache or state of its own and a learned vector added to the stream before it; a
final layer norm and a head.

* mixer ``attention``: grouped-query softmax attention with a rotation of the leading dims of queries and keys whose
  slow frequencies are stretched, values that are rotated too (by their own position; each head's sum is turned back
  by the query's), a learned sink per head, one output gate per head.
* mixer ``wkv``: time mixing with a matrix state per head, a decay per channel that depends on the token, a bonus for
  the current token.
* mixer ``latent_attention``: softmax attention over a sliding window, without positions, whose keys and values are
  maps of one cached low-rank latent per token.
* feed-forward: dense with biases and the square of relu, or routed (gated silu experts; sigmoid scores; the weights
  multiply the experts' inputs and are not renormalised; a shared expert), or none.

This file only turns the configuration into a ModelSpec, layer by layer; all the computing is in ``pyre_b200.parts``.
"""

from __future__ import annotations

from ..config.model_config import ConfigError, TekaraxConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec

PASS_VECTORS = "loop.step"      # [passes, width]: row t is added to the stream before pass t of the repeated span


def build_tekarax(cfg: TekaraxConfig) -> ModelSpec:
    def norm():
        return PartSpec("layer_norm", {"width": cfg.width, "eps": cfg.norm_eps, "tensor_name": ""})

    blocks = []
    for i, L in enumerate(cfg.layers):
        if L.kind == "attention":
            position = value_position = None
            if L.rot_dims:
                scaling = dict(zip(("factor", "low", "high", "original"), L.rot_scaling)) if L.rot_scaling else None
                position = PartSpec("rotary", {"head_dim": L.dim, "theta": L.rot_base, "rotary_dim": L.rot_dims,
                                               "exact_frequencies": True, "scaling": scaling})
                # the values turn over all their dims, with the plain frequencies of the same base
                value_position = PartSpec("rotary", {"head_dim": L.vdim, "theta": L.rot_base, "rotary_dim": L.vdim,
                                                     "exact_frequencies": True})
            mixer = PartSpec("attention", {
                "width": cfg.width, "n_heads": L.heads, "n_kv_heads": L.kv_heads, "head_dim": L.dim, "v_head_dim": L.vdim,
                "qkv_bias": False, "o_bias": False, "scale": L.scale, "window": None, "position": position,
                "value_position": value_position, "sink": "learned", "out_gate": "head", "weight_suffix": "",
                "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "sink": "sink"}})
        elif L.kind == "wkv":
            if not L.decay_rank:
                raise ConfigError(f"config.json: layers[{i}].mixer: the inner size of the decay map is given neither by "
                                  f"'decay_rank' nor by the weights")
            mixer = PartSpec("wkv", {"width": cfg.width, "n_heads": L.heads, "head_dim": L.dim, "decay_rank": L.decay_rank,
                                     "eps": cfg.norm_eps})
        else:
            mixer = PartSpec("latent_attention", {
                "width": cfg.width, "n_heads": L.heads, "head_dim": L.dim, "rope_dim": 0, "v_head_dim": L.vdim,
                "q_rank": None, "kv_rank": L.kv_rank, "scale": L.scale, "eps": cfg.norm_eps, "window": L.window or None,
                "position": None})
        params = {"width": cfg.width, "norm1": norm(), "mixer": mixer, "norm1b": norm(), "gated": True,
                  "names": {"norm1": "norm1", "norm1b": "norm1b", "mixer": "mix.", "norm2": "norm2", "norm2b": "norm2b",
                            "ffn": "mlp.", "gate1": "rg1", "gate1_bias": "rg1.b", "gate2": "rg2", "gate2_bias": "rg2.b"}}
        if L.mlp_kind == "dense":
            params["ffn"] = PartSpec("dense_mlp", {"width": cfg.width, "intermediate": L.ff, "activation": "relu2", "bias": True,
                                                   "names": {"up": "up", "down": "down", "up_bias": "up.b", "down_bias": "down.b"}})
        elif L.mlp_kind == "moe":
            params["ffn"] = PartSpec("routed_mlp", {"width": cfg.width, "intermediate": L.ff, "n_experts": L.experts,
                                                    "top": L.top, "activation": "silu", "correction": False,
                                                    "scores": "sigmoid", "weight_on": "input", "shared": L.shared_ff or None})
        if L.mlp_kind:
            params["norm2"], params["norm2b"] = norm(), norm()
        blocks.append(PartSpec("sandwich", params))
    # a layer of the repeated span appears once per pass; every appearance has a cache or state layer of its own
    schedule = [LayerCall(i, add_vector=(PASS_VECTORS, t) if t is not None else None) for i, t in cfg.layer_order()]
    return ModelSpec(
        embed=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": ""}),
        blocks=blocks,
        final_norm=norm(),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "tensor_name": ""}),
        schedule=schedule,
        embed_prefix="embed", block_prefix="l{i}.", final_norm_prefix="final.norm", head_prefix="head",
        vocab_size=cfg.vocab,
        max_positions=0,
        vectors={PASS_VECTORS: cfg.loop_times} if cfg.has_loop() else {},
        width=cfg.width,
    )


register_architecture(TekaraxConfig.architecture, TekaraxConfig, build_tekarax)
