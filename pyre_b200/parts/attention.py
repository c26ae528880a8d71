"""Grouped-query attention over the paged cache (pyre/model.py:75-125 for the math,
pyre/model.py:296-342 and pyre/kernels/paged_attn.py for reading pages in place)."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import HeadGeometry, PagedKVSpec, Part, PartSpec, ProjectionLayout, make_part, register_part


def attention_libraries(dtype, row_dim: int) -> list[str]:
    """The kernel libraries that ``attend`` needs for cache rows of ``row_dim`` in ``dtype``."""
    if dtype == torch.bfloat16 and row_dim <= ops.MMA_MAX_HEAD_DIM:
        return ["attention_mma"] + (["attention_prefill", "attention_tc"] if row_dim in ops.PREFILL_HEAD_DIMS else [])
    return ["attention_generic"]


def attend(ctx, dtype, q, layer, kv, n_heads: int, n_kv_heads: int, row_dim: int, scale: float, window, sink=None):
    """Softmax attention of every token of the step over its sequence's cached keys and values in ``layer``, by the
    package's kernels: bfloat16 rows up to 128 on the tensor cores, everything else on the exact fp32 kernel."""
    if dtype == torch.bfloat16 and row_dim <= ops.MMA_MAX_HEAD_DIM:
        return ops.paged_attention_bf16(ctx, q, layer, kv.block_table, n_heads, n_kv_heads, row_dim, scale, window, sink=sink)
    return ops.paged_attention_generic(q, layer, kv.block_table, ctx.seq_of_token, ctx.positions, n_heads, n_kv_heads, row_dim,
                                       scale, window, sink=sink)


class Attention(Part):
    """q, k, v projections (stacked into one product); the position encoding (a sub-part, which adds the
    bias, encodes positions into q and k in its own way and writes keys and values to the pages of this
    call's cache layer); attention of every token of the step over its sequence's cached keys; output projection.

    Parameters: ``width`` (model width), ``n_heads``, ``n_kv_heads``, ``head_dim``
    (``n_heads * head_dim`` need not equal ``width``), ``qkv_bias`` / ``o_bias``,
    ``scale`` (default head_dim^-0.5, pyre/model.py:82), ``window`` (None = all keys),
    ``position``, the PartSpec of the position encoding applied to q and k, and ``names``, the checkpoint's
    names of the four projections (default q_proj, k_proj, v_proj, o_proj: an architecture whose checkpoint
    calls them otherwise says so in its builder, no new part needed).
    A query at position p sees keys max(0, p - window + 1)..p.

    Further parameters, all off by default (the stacked, fused path above is untouched by them):
    ``v_head_dim``: a value head's size when it differs from ``head_dim`` (the cache's rows then have one size that
    holds both, ``ops.attention_row_dim``, the rest zero);
    ``qk_norm``: an RMS norm per head over the ``head_dim`` dims of queries and keys before the position encoding,
    ``{"eps": e}``, with weights of ``head_dim`` entries shared by the heads (names ``q_norm`` / ``k_norm``);
    ``sink``: the score of a sink that has no value: exp(sink) joins every softmax denominator; ``"learned"``: a score
    per query head read from the checkpoint (name ``sink``, [n_heads]);
    ``out_gate``: the concatenated heads are multiplied by sigmoid(W_g h) before the output projection (name ``g``);
    ``"head"``: ONE gate per head (W_g has ``n_heads`` rows);
    ``value_position``: the PartSpec of a rotation (half-split pairs over all ``v_head_dim`` dims) by which each
    token's VALUES are turned by the token's own position before they are cached; each head's weighted sum is turned
    back by the query's position before the gate (the sum then depends on position differences only);
    ``own_kv=False``: the mixer has no key and value projections (and no key norm): it reads the cache layer that
    another entry of the schedule writes (``LayerCall(cache=..., write=False)``);
    ``weight_suffix``: what follows a projection's name in the checkpoint (".weight").
    """

    DEFAULT_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "g": "g_proj", "q_norm": "q_norm.weight",
                     "k_norm": "k_norm.weight", "sink": "sink"}

    graph_safe = True
    takes_scaled_rows = True      # ``h`` may be ``ops.ScaledRows``: the q/k/v product applies the norm's 1/rms itself

    def __init__(self, dtype, device, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: "PartSpec | None" = None, qkv_bias: bool = True, o_bias: bool = False,
                 scale: "float | None" = None, window: "int | None" = None, names: "dict[str, str] | None" = None,
                 v_head_dim: "int | None" = None, qk_norm: "dict | None" = None, sink: "float | None" = None,
                 out_gate: "bool | str" = False, own_kv: bool = True, weight_suffix: str = ".weight",
                 value_position: "PartSpec | None" = None):
        super().__init__(dtype, device)
        self.v_head_dim = int(v_head_dim) if v_head_dim is not None else int(head_dim)
        self.qk_norm_eps = float(qk_norm["eps"]) if qk_norm is not None else None
        self.learned_sink = sink == "learned"
        self.sink = None if sink is None or self.learned_sink else float(sink)
        if out_gate not in (False, True, "head"):
            raise ValueError(f"out_gate {out_gate!r}: False, True (a gate per entry) or 'head' (one per head)")
        self.head_gate = out_gate == "head"
        self.out_gate, self.own_kv, self.suffix = bool(out_gate), bool(own_kv), str(weight_suffix)
        self.value_position = make_part("position", value_position, dtype, device) if value_position is not None else None
        if self.value_position is not None and (self.v_head_dim % 2 or getattr(self.value_position, "pairing", "half") != "half"):
            raise ops.UnsupportedSize("rotated values: an even value size and half-split pairs")
        # the general path: projections laid out by a ProjectionLayout, unfused small kernels
        self.general = (self.v_head_dim != int(head_dim) or qk_norm is not None or self.out_gate or not self.own_kv
                        or self.value_position is not None or self.learned_sink)
        if self.general and qkv_bias:
            raise ops.UnsupportedSize("projection biases together with v_head_dim, qk_norm, out_gate or own_kv=False are not implemented")
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = int(width), int(n_heads), int(n_kv_heads), int(head_dim)
        if self.n_heads % self.n_kv_heads:
            raise ops.UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
        # the size of a cache row: the head size itself, or (general path) one size that holds keys and values
        self.row_dim = ops.attention_row_dim(self.head_dim, self.v_head_dim, dtype) if self.general else self.head_dim
        if self.row_dim % 16 or not 16 <= self.row_dim <= 256:
            raise ops.UnsupportedSize(f"head_dim {head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        if o_bias:
            raise ops.UnsupportedSize("an output-projection bias is not implemented")
        if window is not None and window <= 0:
            raise ValueError("window must be positive or None")
        self.qkv_bias = bool(qkv_bias)
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.window = window
        self.heads = HeadGeometry(self.n_heads, self.n_kv_heads, self.head_dim)
        self.position = make_part("position", position or PartSpec("none"), dtype, device)
        self.w_qkv = self.b_qkv = self.w_o = None
        self.w_proj = self.q_norm_w = self.k_norm_w = None
        q_cols, kv_cols = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.layout = ProjectionLayout(self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim, self.row_dim, 0,
                                       q_cols if self.own_kv else -1, q_cols + kv_cols if self.own_kv else -1)
        self.g_col = q_cols + (kv_cols + self.n_kv_heads * self.v_head_dim if self.own_kv else 0)

    def children(self):
        # a position encoding with tensors of its own would find them under the mixer's prefix
        return {"": self.position} if self.value_position is None else {"": self.position, "value.": self.value_position}

    def tensors(self):
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        n = self.names
        t = {}
        if self.general:
            sfx = self.suffix
            vq, vkv = self.n_heads * self.v_head_dim, self.n_kv_heads * self.v_head_dim
            t[n["q"] + sfx] = TensorSpec((q, self.width))
            if self.own_kv:
                t[n["k"] + sfx] = TensorSpec((kv, self.width))
                t[n["v"] + sfx] = TensorSpec((vkv, self.width))
            if self.qk_norm_eps is not None:
                t[n["q_norm"]] = TensorSpec((self.head_dim,), role="vector", init=("normal", 1.0, 0.1))
                if self.own_kv:
                    t[n["k_norm"]] = TensorSpec((self.head_dim,), role="vector", init=("normal", 1.0, 0.1))
            if self.out_gate:
                t[n["g"] + sfx] = TensorSpec((self.n_heads if self.head_gate else vq, self.width))
            if self.learned_sink:
                t[n["sink"]] = TensorSpec((self.n_heads,), role="vector", init=("normal", 0.0, 1.0))
            t[n["o"] + sfx] = TensorSpec((self.width, vq))
            return t
        # checkpoint order: weight then bias per projection, the output projection last
        for key, rows in (("q", q), ("k", kv), ("v", kv)):
            t[f"{n[key]}.weight"] = TensorSpec((rows, self.width))
            if self.qkv_bias:
                t[f"{n[key]}.bias"] = TensorSpec((rows,), role="vector")
        t[f"{n['o']}.weight"] = TensorSpec((self.width, q))
        return t

    def load(self, tensors):
        n = self.names
        if self.general:
            sfx = self.suffix
            stack = [tensors[n["q"] + sfx]] + ([tensors[n["k"] + sfx], tensors[n["v"] + sfx]] if self.own_kv else [])
            if self.out_gate:
                stack.append(tensors[n["g"] + sfx])
            self.w_proj = torch.cat(stack, dim=0).contiguous() if len(stack) > 1 else stack[0]
            if self.qk_norm_eps is not None:
                self.q_norm_w = tensors[n["q_norm"]]
                self.k_norm_w = tensors[n["k_norm"]] if self.own_kv else None
            self.w_o = tensors[n["o"] + sfx]
            if self.learned_sink:
                self.sink = tensors[n["sink"]]
            return
        self.w_qkv = torch.cat([tensors[f"{n[k]}.weight"] for k in "qkv"], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[f"{n[k]}.bias"] for k in "qkv"]).contiguous()
        self.w_o = tensors[f"{n['o']}.weight"]

    def kernel_libraries(self):
        libs = ["elementwise"]      # the position encoding, a sub-part, names its own
        if self.general:
            libs.append("blockops")
        libs += attention_libraries(self.dtype, self.row_dim)
        libs.append("gemm_f32" if self.dtype == torch.float32 else "gemm_tc")
        return libs

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.row_dim, self.window)

    def state_spec(self):
        return None

    def launch_key(self, n_rows, max_context):
        # the tensor-core kernel's split count is chosen on the host from these numbers
        return (ops.attention_splits(n_rows, n_rows, self.n_heads, self.n_kv_heads, max_context, self.window),)

    def _attend(self, ctx, q, layer, kv):
        return attend(ctx, self.dtype, q, layer, kv, self.n_heads, self.n_kv_heads, self.row_dim, self.scale, self.window,
                      sink=self.sink)

    def _forward_general(self, ctx, h, call):
        """Projections in one product [q | k | v | gate]; norm, position encoding and the paged write by the
        encoding's ``apply_layout``; attention over cache rows of ``row_dim``; the gate; the output projection."""
        kv = ctx.kv_group(call.kv_group)
        layer = kv.pool[call.kv_layer]
        if self.own_kv != bool(call.kv_write):
            raise ValueError("a mixer with its own keys and values writes its cache layer; one without reads another's")
        with lib.section("qkv"):
            proj = ops.materialize(ops.linear(h, self.w_proj))
        kw, vcos, vsin = {}, None, None
        if self.value_position is not None:
            vcos, vsin, _ = self.value_position.rotation(ctx, self.v_head_dim)
            kw["value_tables"] = (vcos, vsin)
        q = self.position.apply_layout(ctx, proj, self.layout, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0, kv,
                                       layer if call.kv_write else None, **kw)
        a = self._attend(ctx, q, layer, kv)
        if self.head_gate or vcos is not None:
            if self.out_gate and not self.head_gate:
                raise ops.UnsupportedSize("rotated values with a gate per entry are not implemented")
            a = ops.head_gate(a, self.row_dim, proj if self.head_gate else None, self.g_col, self.n_heads, self.v_head_dim, vcos, vsin)
        elif self.out_gate or self.row_dim != self.v_head_dim:
            a = ops.sigmoid_gate(a, self.row_dim, proj if self.out_gate else None, self.g_col, self.n_heads, self.v_head_dim)
        with lib.section("o"):
            return ops.linear(a, self.w_o, partials_ok=True)

    def forward(self, ctx, h, call):
        if self.general:
            return self._forward_general(ctx, h, call)
        kv = ctx.kv_group(call.kv_group)
        layer = kv.pool[call.kv_layer]
        with lib.section("qkv"):
            qkv = ops.linear(h, self.w_qkv, partials_ok=True, deferred_ok=("rope", self.head_dim))
        # the position encoding owns the step from projections to cache: bias, its transformation of q and k,
        # the paged write of k and v; the queries come back
        q = self.position.apply(ctx, qkv, self.b_qkv, self.heads, kv, layer if call.kv_write else None)
        a = self._attend(ctx, q, layer, kv)
        with lib.section("o"):
            return ops.linear(a, self.w_o, partials_ok=True, deferred_ok="residual")


register_part("mixer", "attention", Attention)
