"""Differential attention over the paged cache: two softmax maps per head over the same values, one subtracted from
the other, with an optional short causal convolution on the projections."""

from __future__ import annotations

import math

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .attention import attend, attention_libraries
from .base import PagedKVSpec, Part, PartSpec, ProjectionLayout, StateSpec, make_part, register_part


class DifferentialAttention(Part):
    """Per query head h (key/value head g = h // (n_heads / n_kv_heads)) two attention maps m = 1, 2 with queries
    q_(h,m) and keys k_(g,m) of ``head_dim`` entries and the SAME values v_g of ``v_head_dim``:

        a_m = softmax(scale q_(h,m) . k_(g,m), over the keys the window shows) v_g
        o_h = a_1 - lambda a_2;   o_h / sqrt(mean(o_h^2) + eps) * (1 - diff);   out = W_o [o_1 .. o_H] (+ bias)
        lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff          one number per layer, from four vectors of ``head_dim``

    The projections W_q [n_heads * 2 * head_dim], W_k [n_kv_heads * 2 * head_dim] (head by head, [map 1 | map 2]) and
    W_v are one product; ``qkv_bias`` adds their biases.  ``conv_taps`` > 0: a causal convolution of that many taps
    over time on every channel of q, k and v, right after the projection (names ``<projection>.conv``); the last
    ``conv_taps - 1`` projected rows of a request live in its state slot.  Then the position encoding (a sub-part)
    turns each map's queries and keys and keys and values go to the cache.  ``own_kv=False``: the mixer projects
    queries only and reads the cache layer another schedule entry writes.  ``cache_window``: how far back the cache
    layer must keep keys (default: ``window``); a layer whose cache is read by layers with other windows names the
    widest of them (None: everything), and so do its readers, so that all of them ask the same of the cache manager.

    For the package's attention kernels a map is a head of its own: 2 n_heads query heads over 2 n_kv_heads key/value
    heads, the query maps ordered (g, m, r) so that the kernels' grouping sends map m of head g * rep + r to key head
    (g, m); key head (g, m) carries a copy of v_g.  The maps' sums meet again in ``ops.diff_combine``."""

    DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "bias": ".b", "conv": ".conv", "lq1": "lq1", "lk1": "lk1",
                     "lq2": "lq2", "lk2": "lk2"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, diff: float,
                 eps: float, scale: "float | None" = None, window: "int | None" = None, position: "PartSpec | None" = None,
                 conv_taps: int = 0, qkv_bias: bool = True, o_bias: bool = True, own_kv: bool = True,
                 names: "dict[str, str] | None" = None, cache_window: "int | None | str" = "window"):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        if self.n_heads % self.n_kv_heads:
            raise ops.UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
        if window is not None and window <= 0:
            raise ValueError("window must be positive or None")
        self.rep = self.n_heads // self.n_kv_heads
        self.diff, self.eps = float(diff), float(eps)
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.window, self.conv_taps = window, int(conv_taps)
        self.cache_window = window if cache_window == "window" else cache_window
        if self.cache_window is not None and (window is None or self.cache_window < window):
            raise ValueError("the cache must keep at least the keys that the window shows")
        if self.conv_taps == 1 or self.conv_taps < 0:
            raise ops.UnsupportedSize("a convolution over time has at least two taps (0: none)")
        self.qkv_bias, self.o_bias, self.own_kv = bool(qkv_bias), bool(o_bias), bool(own_kv)
        self.row_dim = ops.attention_row_dim(self.head_dim, self.v_head_dim, dtype)
        self.position = make_part("position", position or PartSpec("none"), dtype, device)
        self.q_cols = 2 * self.n_heads * self.head_dim
        self.k_cols = 2 * self.n_kv_heads * self.head_dim if self.own_kv else 0
        self.v_cols = 2 * self.n_kv_heads * self.v_head_dim if self.own_kv else 0       # every key head has its copy
        self.n_ch = self.q_cols + self.k_cols + self.v_cols
        self.layout = ProjectionLayout(2 * self.n_heads, 2 * self.n_kv_heads, self.head_dim, self.v_head_dim, self.row_dim, 0,
                                       self.q_cols if self.own_kv else -1, self.q_cols + self.k_cols if self.own_kv else -1)
        self.w_proj = self.b_proj = self.w_conv = self.w_o = self.b_o = None
        self.lam = 0.0

    def children(self):
        return {"": self.position}

    def _projections(self):
        """(name, rows) of the projections this mixer owns, in the order of the stacked product."""
        n = self.names
        out = [(n["q"], self.q_cols)]
        if self.own_kv:
            out += [(n["k"], self.k_cols), (n["v"], self.n_kv_heads * self.v_head_dim)]
        return out

    def tensors(self):
        n, t = self.names, {}
        for name, rows in self._projections():
            t[name] = TensorSpec((rows, self.width))
            if self.qkv_bias:
                t[name + n["bias"]] = TensorSpec((rows,), role="vector", init=("normal", 0.0, 0.1))
            if self.conv_taps:
                t[name + n["conv"]] = TensorSpec((rows, self.conv_taps), role="vector", init=("normal", 0.3, 0.3))
        for v in ("lq1", "lk1", "lq2", "lk2"):
            t[n[v]] = TensorSpec((self.head_dim,), role="vector", init=("normal", 0.0, 0.1))
        t[n["o"]] = TensorSpec((self.width, self.n_heads * self.v_head_dim))
        if self.o_bias:
            t[n["o"] + n["bias"]] = TensorSpec((self.width,), role="vector", init=("normal", 0.0, 0.1))
        return t

    def _arrange(self, tensors, suffix: str):
        """The rows of q, k and v tensors (weights, biases or taps) in the order of the stacked product: the query maps
        grouped (g, m, r), the keys as stored, the values once per map."""
        n = self.names
        q = tensors[n["q"] + suffix]
        tail = q.shape[1:]
        q = q.reshape(self.n_kv_heads, self.rep, 2, self.head_dim, *tail).transpose(1, 2).reshape(self.q_cols, *tail)
        if not self.own_kv:
            return q.contiguous()
        v = tensors[n["v"] + suffix]
        v = v.reshape(self.n_kv_heads, 1, self.v_head_dim, *tail).expand(self.n_kv_heads, 2, self.v_head_dim, *tail)
        return torch.cat([q, tensors[n["k"] + suffix], v.reshape(self.v_cols, *tail)], dim=0).contiguous()

    def load(self, tensors):
        n = self.names
        self.w_proj = self._arrange(tensors, "")
        self.b_proj = self._arrange(tensors, n["bias"]) if self.qkv_bias else None
        self.w_conv = self._arrange(tensors, n["conv"]) if self.conv_taps else None
        self.w_o = tensors[n["o"]]
        self.b_o = tensors[n["o"] + n["bias"]] if self.o_bias else None
        dot = lambda a, b: float((tensors[n[a]].double() * tensors[n[b]].double()).sum())
        self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff

    def kernel_libraries(self):
        return ["elementwise", "blockops", "seqmix"] + attention_libraries(self.dtype, self.row_dim) + \
            (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def cache_spec(self):
        return PagedKVSpec(2 * self.n_kv_heads, self.row_dim, self.cache_window)

    def state_spec(self):
        return StateSpec(((self.conv_taps - 1) * self.n_ch,), torch.float32) if self.conv_taps > 1 else None

    def launch_key(self, n_rows, max_context):
        return (ops.attention_splits(n_rows, n_rows, 2 * self.n_heads, 2 * self.n_kv_heads, max_context, self.window),)

    def forward(self, ctx, h, call):
        kv = ctx.kv_group(call.kv_group)
        layer = kv.pool[call.kv_layer]
        if self.own_kv != bool(call.kv_write):
            raise ValueError("a mixer with its own keys and values writes its cache layer; one without reads another's")
        with lib.section("qkv"):
            proj = ops.materialize(ops.linear(h, self.w_proj))
        if self.conv_taps > 1:
            st = ctx.state_group(call.state_group)
            proj = ops.short_conv(proj, 0, self.n_ch, self.w_conv, None, st.buffer[call.state_layer], 0, st.slots,
                                  ctx.seq_of_token, ctx.cu_seqlens, in_bias=self.b_proj)
        elif self.b_proj is not None:
            proj = ops.bias_act(proj, self.b_proj, None)
        q = self.position.apply_layout(ctx, proj, self.layout, None, None, 0.0, kv, layer if call.kv_write else None)
        a = attend(ctx, self.dtype, q, layer, kv, 2 * self.n_heads, 2 * self.n_kv_heads, self.row_dim, self.scale, self.window)
        o = ops.diff_combine(a, self.row_dim, self.lam, 1.0 - self.diff, self.n_heads, self.n_kv_heads, self.v_head_dim, self.eps)
        with lib.section("o"):
            if self.b_o is None:
                return ops.linear(o, self.w_o, partials_ok=True)
            return ops.bias_act(ops.materialize(ops.linear(o, self.w_o)), self.b_o, None)


register_part("mixer", "differential_attention", DifferentialAttention)
