"""Time mixing with a matrix state per head (an RWKV-style mixer): a recurrent mixer whose memory is a matrix of
fixed size per request and head plus the last token's input, kept in a state slot of the cache manager."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, StateSpec, register_part


class WKVMixer(Part):
    """Per token, with h the mixer's input and h' the input of the token before it (zeros at a sequence's start):

        x_s = h + (h' - h) * mu_s                      one blend per stream s in (r, k, v, g, w)
        r, k, v = W_r x_r, W_k x_k, W_v x_v            ``n_heads`` heads of ``head_dim``
        gate = silu(W_g x_g)
        w = exp(-exp(W_w2 tanh(W_w1 x_w) + w0))        a decay per head and key channel, ``decay_rank`` inner size
        head n:  o_t = (S + diag(u) k_t v_t^T)^T r_t;   S = diag(w_t) S + k_t v_t^T
        out = W_o [ (o / rms(o) per head) * norm * gate ]

    The bonus u counts for the current token only.  S [head_dim, head_dim] per head and h' live in fp32 in the
    request's state slot (``StateSpec``): zeros when a request begins, carried from step to step.  The blends, the
    decay from its logits on, the recurrence, the unit norm and the gate's product are fp32 in both precisions; the
    five projections and the decay's second product are matrix products in the compute dtype (the decay's logits
    leave theirs in fp32).

    ``names``: the checkpoint's local names; the blends are ``mu`` + stream letter."""

    DEFAULT_NAMES = {"r": "r", "k": "k", "v": "v", "g": "g", "o": "o", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u",
                     "norm": "norm", "mu": "mu."}
    STREAMS = ("r", "k", "v", "g", "w")

    graph_safe = True

    def __init__(self, dtype, device, width: int, n_heads: int, head_dim: int, decay_rank: int, eps: float,
                 names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.head_dim, self.decay_rank = int(width), int(n_heads), int(head_dim), int(decay_rank)
        self.eps = float(eps)
        if min(self.width, self.n_heads, self.head_dim, self.decay_rank) <= 0:
            raise ValueError("the sizes of a wkv mixer are positive")
        if self.head_dim > ops.WKV_MAX_DIM:
            raise ops.UnsupportedSize(f"heads of {head_dim}: the recurrence takes up to {ops.WKV_MAX_DIM}")
        self.prev_off = self.n_heads * self.head_dim * self.head_dim
        self.mu = self.w = self.w_o = self.w0 = self.u = self.norm_w = None

    def tensors(self):
        n, HD, W = self.names, self.n_heads * self.head_dim, self.width
        t = {n["mu"] + s: TensorSpec((W,), role="vector", init=("normal", 0.5, 0.15)) for s in self.STREAMS}
        for s in ("r", "k", "v", "g"):
            t[n[s]] = TensorSpec((HD, W))
        t[n["w1"]] = TensorSpec((self.decay_rank, W))
        t[n["w2"]] = TensorSpec((HD, self.decay_rank), init=("normal", 0.0, 0.1))
        t[n["w0"]] = TensorSpec((HD,), role="vector", init=("normal", -1.0, 0.7))
        t[n["u"]] = TensorSpec((self.n_heads, self.head_dim), role="vector", init=("normal", 0.3, 0.3))
        t[n["norm"]] = TensorSpec((HD,), role="vector", init=("normal", 1.0, 0.1))
        t[n["o"]] = TensorSpec((W, HD))
        return t

    def load(self, tensors):
        n = self.names
        self.mu = torch.stack([tensors[n["mu"] + s] for s in self.STREAMS]).contiguous()
        self.w = {s: tensors[n[s]] for s in ("r", "k", "v", "g", "w1", "w2")}
        self.w0, self.u, self.norm_w = tensors[n["w0"]], tensors[n["u"]].reshape(-1).contiguous(), tensors[n["norm"]]
        self.w_o = tensors[n["o"]]

    def kernel_libraries(self):
        return ["wkv", "blockops", "elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def cache_spec(self):
        return None

    def state_spec(self):
        return StateSpec((ops.wkv_state_floats(self.n_heads, self.head_dim, self.width),), torch.float32)

    def forward(self, ctx, h, call):
        st = ctx.state_group(call.state_group)
        state = st.buffer[call.state_layer]
        h = ops.materialize(h)
        x = ops.token_shift_mix(h, state, self.prev_off, st.slots, ctx.seq_of_token, ctx.cu_seqlens, self.mu)
        with lib.section("qkv"):
            r, k, v, g = (ops.materialize(ops.linear(x[i], self.w[s])) for i, s in enumerate(("r", "k", "v", "g")))
        with lib.section("decay"):
            inner = ops.bias_act(ops.materialize(ops.linear(x[4], self.w["w1"])), None, "tanh")
            dlog = ops.linear(inner, self.w["w2"], out_dtype=torch.float32)
        a = ops.wkv_scan(r, k, v, g, dlog, self.w0, self.u, self.norm_w, state, self.prev_off, st.slots, ctx.cu_seqlens, h,
                         self.n_heads, self.head_dim, self.eps)
        with lib.section("o"):
            return ops.linear(a, self.w_o, partials_ok=True)


register_part("mixer", "wkv", WKVMixer)
