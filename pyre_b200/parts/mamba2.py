"""A selective state-space mixer (Mamba-2 form): a recurrent mixer whose memory is a matrix of fixed size per request
and head plus the last inputs of a short convolution, kept in a state slot of the cache manager."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, StateSpec, register_part


class Mamba2Mixer(Part):
    """With inner = n_heads * p_dim, N = n_state and G = n_groups, one product W_in h gives a row
    [z: inner | x: inner | B: G N | C: G N | dt: n_heads].  x, B and C together pass a causal convolution of
    ``conv_taps`` taps per channel (with bias) and silu; per head (group h // (n_heads / G)):

        dt = softplus(dt + dt_bias)                  no clamp
        S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T          S [N, p_dim]
        y_t = S_t^T C_t + D x_t

    y (heads concatenated) is multiplied by silu(z), unit-normed in ``norm_groups`` equal parts, multiplied by a gain
    and projected by W_o.  The gate comes before the norm.  S and the convolution's last ``conv_taps - 1`` inputs live
    in fp32 in the request's state slot (zeros when a request begins).  Step sizes, decays, the recurrence, the gate's
    product and the norm are fp32 in both precisions; the two projections and the convolution's results are in the
    compute dtype.

    ``names``: the checkpoint's local names."""

    DEFAULT_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
                     "norm": "norm", "o": "o"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, n_heads: int, p_dim: int, n_state: int, n_groups: int, conv_taps: int,
                 norm_groups: int, eps: float, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.p_dim, self.n_state = int(width), int(n_heads), int(p_dim), int(n_state)
        self.n_groups, self.conv_taps, self.norm_groups, self.eps = int(n_groups), int(conv_taps), int(norm_groups), float(eps)
        if min(self.width, self.n_heads, self.p_dim, self.n_state, self.n_groups, self.norm_groups) <= 0 or self.conv_taps < 2:
            raise ValueError("the sizes of a state-space mixer are positive and its convolution has at least two taps")
        self.inner = self.n_heads * self.p_dim
        if self.n_heads % self.n_groups or self.inner % self.norm_groups:
            raise ValueError(f"{n_heads} heads do not divide into {n_groups} groups, or rows of {self.inner} into {norm_groups} parts")
        if self.n_state > ops.SSM_MAX_STATE:
            raise ops.UnsupportedSize(f"a state of {n_state} rows per head: the recurrence takes up to {ops.SSM_MAX_STATE}")
        self.conv_ch = self.inner + 2 * self.n_groups * self.n_state
        self.row = 2 * self.inner + 2 * self.n_groups * self.n_state + self.n_heads
        self.hist_off = self.n_heads * self.n_state * self.p_dim
        self.w_in = self.w_conv = self.b_conv = self.dt_bias = self.a_log = self.d_skip = self.norm_w = self.w_o = None

    def tensors(self):
        n, H = self.names, self.n_heads
        return {n["in"]: TensorSpec((self.row, self.width)),
                n["conv"]: TensorSpec((self.conv_ch, self.conv_taps), role="vector", init=("normal", 0.3, 0.3)),
                n["conv_bias"]: TensorSpec((self.conv_ch,), role="vector", init=("normal", 0.0, 0.1)),
                n["dt_bias"]: TensorSpec((H,), role="vector", init=("normal", -1.0, 1.0)),
                n["A_log"]: TensorSpec((H,), role="vector", init=("normal", 0.0, 0.7)),
                n["D"]: TensorSpec((H,), role="vector", init=("normal", 1.0, 0.3)),
                n["norm"]: TensorSpec((self.inner,), role="vector", init=("normal", 1.0, 0.1)),
                n["o"]: TensorSpec((self.width, self.inner))}

    def load(self, tensors):
        n = self.names
        self.w_in, self.w_conv, self.b_conv = tensors[n["in"]], tensors[n["conv"]], tensors[n["conv_bias"]]
        self.dt_bias, self.a_log, self.d_skip = tensors[n["dt_bias"]], tensors[n["A_log"]], tensors[n["D"]]
        self.norm_w, self.w_o = tensors[n["norm"]], tensors[n["o"]]

    def kernel_libraries(self):
        return ["seqmix", "elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def cache_spec(self):
        return None

    def state_spec(self):
        return StateSpec((self.hist_off + (self.conv_taps - 1) * self.conv_ch,), torch.float32)

    def forward(self, ctx, h, call):
        st = ctx.state_group(call.state_group)
        state = st.buffer[call.state_layer]
        with lib.section("qkv"):
            proj = ops.materialize(ops.linear(h, self.w_in))
        xbc = ops.short_conv(proj, self.inner, self.conv_ch, self.w_conv, self.b_conv, state, self.hist_off, st.slots,
                             ctx.seq_of_token, ctx.cu_seqlens, silu=True)
        y = ops.ssm_scan(xbc, proj, self.inner + self.conv_ch, self.dt_bias, self.a_log, self.d_skip, state, st.slots,
                         ctx.cu_seqlens, self.n_heads, self.n_groups, self.p_dim, self.n_state)
        a = ops.group_norm_gate(y, self.norm_groups, self.norm_w, self.eps, proj, 0, self.dtype, gate="silu", gate_first=True)
        with lib.section("o"):
            return ops.linear(a, self.w_o, partials_ok=True)


register_part("mixer", "mamba2", Mamba2Mixer)
