"""Linear attention with a constant decay per head: a mixer whose memory is a matrix of fixed size per request
and head, kept in a state slot of the cache manager instead of pages."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, PartSpec, StateSpec, make_part, register_part


class DecayLinearAttention(Part):
    """Per head, with q_t, k_t of ``head_dim`` and v_t of ``v_head_dim`` entries (each act(W h), ``activation``
    silu or None):

        S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t        (no other scale)

    The state S [head_dim, v_head_dim] is fp32, starts at zero when a request begins and is carried from token
    to token in the request's state slot; the decays are constants of the model (``decay``, one per head).  The
    concatenated heads then pass an RMS norm over the whole row (plain weight, ``eps``; name ``norm``), are
    multiplied by sigmoid(W_g h) when ``out_gate`` and projected by W_o.  The recurrence, the norm and the gate are
    computed in fp32; the four projections are one product [q | k | v | gate].

    Further parameters: ``position``: the PartSpec of a rotation applied to queries and keys (per head, by the token's
    position) before the recurrence; ``k_scale``: a factor on the keys after it; ``norm="head"``: the unit norm runs
    over each head's ``v_head_dim`` values instead of the whole row; ``norm_weight=False``: the norm has no gain;
    ``gate``: ``"sigmoid"`` or ``"silu"`` of W_g h.

    ``names``: the checkpoint's full local names of the tensors."""

    DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                     "o": "o_proj.weight", "norm": "norm.weight"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, n_heads: int, head_dim: int, v_head_dim: int, decay, eps: float,
                 activation: "str | None" = "silu", out_gate: bool = True, names: "dict[str, str] | None" = None,
                 position: "PartSpec | None" = None, k_scale: float = 1.0, norm: str = "row", norm_weight: bool = True,
                 gate: str = "sigmoid"):
        super().__init__(dtype, device)
        if norm not in ("row", "head") or gate not in ("sigmoid", "silu"):
            raise ValueError(f"norm {norm!r} / gate {gate!r}: 'row' or 'head', 'sigmoid' or 'silu'")
        self.position = make_part("position", position, dtype, device) if position is not None else None
        self.k_scale, self.norm, self.norm_weight, self.gate = float(k_scale), norm, bool(norm_weight), gate
        # the plain form (a gained norm over the row, a sigmoid gate) has a kernel of its own
        self.grouped_norm = norm == "head" or not self.norm_weight or gate != "sigmoid"
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.head_dim, self.v_head_dim = int(width), int(n_heads), int(head_dim), int(v_head_dim)
        decay = [float(d) for d in decay]
        if len(decay) != self.n_heads:
            raise ValueError(f"{len(decay)} decays for {self.n_heads} heads")
        if not 1 <= self.head_dim <= 256:
            raise ops.UnsupportedSize(f"linear attention takes query/key sizes up to 256, got {head_dim}")
        if activation not in (None, "silu"):
            raise ops.UnsupportedSize(f"linear attention: activation {activation!r} is not implemented")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(self.device)
        self.eps, self.activation, self.out_gate = float(eps), activation, bool(out_gate)
        qk, vv = self.n_heads * self.head_dim, self.n_heads * self.v_head_dim
        self.q_col, self.k_col, self.v_col, self.g_col = 0, qk, 2 * qk, 2 * qk + vv
        self.w_proj = self.w_o = self.norm_w = None

    def tensors(self):
        n = self.names
        qk, vv = self.n_heads * self.head_dim, self.n_heads * self.v_head_dim
        t = {n["q"]: TensorSpec((qk, self.width)), n["k"]: TensorSpec((qk, self.width)), n["v"]: TensorSpec((vv, self.width))}
        if self.out_gate:
            t[n["g"]] = TensorSpec((vv, self.width))
        t[n["o"]] = TensorSpec((self.width, vv))
        if self.norm_weight:
            t[n["norm"]] = TensorSpec((vv,), role="vector", init=("normal", 1.0, 0.1))
        return t

    def children(self):
        return {"": self.position} if self.position is not None else {}

    def load(self, tensors):
        n = self.names
        stack = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["g"]]] if self.out_gate else [])
        self.w_proj = torch.cat(stack, dim=0).contiguous()
        self.w_o, self.norm_w = tensors[n["o"]], tensors[n["norm"]] if self.norm_weight else None

    def kernel_libraries(self):
        return ["blockops", "linear_attention", "elementwise"] + (["seqmix"] if self.grouped_norm or self.position is not None
                                                                  or self.k_scale != 1.0 else []) + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def cache_spec(self):
        return None

    def state_spec(self):
        return StateSpec((self.n_heads, self.head_dim, self.v_head_dim), torch.float32)

    def forward(self, ctx, h, call):
        st = ctx.state_group(call.state_group)
        with lib.section("qkv"):
            proj = ops.materialize(ops.linear(h, self.w_proj))
        if self.position is not None or self.k_scale != 1.0:
            cos, sin, rot = self.position.rotation(ctx, self.head_dim) if self.position is not None else (None, None, 0)
            if rot:
                ops.rotate_heads(proj, self.q_col, self.n_heads, self.head_dim, cos, sin, rot)
            ops.rotate_heads(proj, self.k_col, self.n_heads, self.head_dim, cos, sin, rot, self.k_scale)
        o = ops.linear_attention(proj, self.q_col, self.k_col, self.v_col, st.buffer[call.state_layer], st.slots,
                                 ctx.cu_seqlens, self.decay, self.n_heads, self.head_dim, self.v_head_dim, self.activation,
                                 lens=ctx.cu_seqlens_host[1:] - ctx.cu_seqlens_host[:-1])
        if self.grouped_norm:
            a = ops.group_norm_gate(o, self.n_heads if self.norm == "head" else 1, self.norm_w, self.eps,
                                    proj if self.out_gate else None, self.g_col, self.dtype, gate=self.gate)
        else:
            a = ops.rmsnorm_gate(o, self.norm_w, self.eps, proj if self.out_gate else None, self.g_col, self.dtype)
        with lib.section("o"):
            return ops.linear(a, self.w_o, partials_ok=True)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
