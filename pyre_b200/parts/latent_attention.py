"""Softmax attention whose keys and values are linear maps of ONE low-rank latent per token: the paged cache holds
a row [latent | rotated key part] per token, shared by all heads, instead of keys and values per head."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import PagedKVSpec, Part, PartSpec, make_part, register_part


class LatentAttention(Part):
    """Per token, with h the mixer's input:

        cq = rmsnorm(W_dq h) * g_q                      the query latent, ``q_rank`` entries
        q  = W_uq cq                                     per head [``head_dim`` plain | ``rope_dim`` rotated]
        [c' | r'] = W_dkv h;  c = rmsnorm(c') * g_c      the key/value latent, ``kv_rank`` entries
        r  = rotate(r')                                  one rotated key part of ``rope_dim`` entries for all heads
        head n:  k_n = U_k,n c,  v_n = U_v,n c
        score(i, j) = (q_plain,i . k_n,j + rotate(q_rot,i) . r_j) * scale,  softmax over the visible j
        out = W_o [heads' sum_j p_ij v_n,j]

    Only c and r are cached (``PagedKVSpec(1, row, window, planes=1)``).  The kernels use the absorbed form:
    q~_n = U_k,n^T q_plain,n (a product per head), scores against the cached rows themselves, the weighted sum of
    the latents per head, and then the head's value map (a second product per head).  Keys and values are never
    expanded, in prompts or in decoding.  ``window``: a query at position p sees p - window + 1 .. p (None: all).
    ``position``: the PartSpec of a rotation that gives tables (``rotation(ctx, rope_dim)``) and pairs neighbours
    (None with ``rope_dim`` 0: attention without positions).  ``q_rank`` None: the queries have no latent of their own,
    q = W_q h (name ``q``).  Norms, angles, scores and the softmax are fp32."""

    DEFAULT_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                     "uv": "uv", "o": "o", "q": "q"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, n_heads: int, head_dim: int, rope_dim: int, v_head_dim: int,
                 q_rank: "int | None", kv_rank: int, scale: float, eps: float, position: "PartSpec | None" = None,
                 window: "int | None" = None, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.head_dim, self.rope_dim = int(width), int(n_heads), int(head_dim), int(rope_dim)
        self.v_head_dim, self.q_rank, self.kv_rank = int(v_head_dim), int(q_rank) if q_rank is not None else 0, int(kv_rank)
        self.q_latent = q_rank is not None
        self.scale, self.eps = float(scale), float(eps)
        if window is not None and window <= 0:
            raise ValueError("window must be positive or None")
        self.window = window
        if min(self.n_heads, self.head_dim, self.v_head_dim, self.q_rank if self.q_latent else 1, self.kv_rank) <= 0 or self.rope_dim < 0:
            raise ValueError("the sizes of a latent attention are positive")
        if self.kv_rank > ops.LATENT_MAX_RANK:
            raise ops.UnsupportedSize(f"kv_rank {kv_rank}: the latent attention kernels take up to {ops.LATENT_MAX_RANK}")
        # a cache row: latent, rotated key part, zeros up to a multiple of 16 entries (whole k-steps of the MMA)
        self.row = -(-(self.kv_rank + self.rope_dim) // 16) * 16
        if position is None and self.rope_dim:
            raise ValueError("a rotated key part needs a position encoding")
        self.position = make_part("position", position or PartSpec("none"), dtype, device)
        if self.rope_dim and getattr(self.position, "pairing", "interleaved") != "interleaved":
            raise ops.UnsupportedSize("the latent attention kernels rotate neighbouring pairs")
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = self.g_q = self.g_c = None

    def children(self):
        return {"": self.position}

    def tensors(self):
        n, H = self.names, self.n_heads
        queries = {
            n["dq"]: TensorSpec((self.q_rank, self.width)),
            n["dq_norm"]: TensorSpec((self.q_rank,), role="vector", init=("normal", 1.0, 0.1)),
            n["uq"]: TensorSpec((H * (self.head_dim + self.rope_dim), self.q_rank)),
        } if self.q_latent else {n["q"]: TensorSpec((H * (self.head_dim + self.rope_dim), self.width))}
        return {
            **queries,
            n["dkv"]: TensorSpec((self.kv_rank + self.rope_dim, self.width)),
            n["dkv_norm"]: TensorSpec((self.kv_rank,), role="vector", init=("normal", 1.0, 0.1)),
            n["uk"]: TensorSpec((H * self.head_dim, self.kv_rank)),
            n["uv"]: TensorSpec((H * self.v_head_dim, self.kv_rank)),
            n["o"]: TensorSpec((self.width, H * self.v_head_dim)),
        }

    def load(self, tensors):
        n, H = self.names, self.n_heads
        if self.q_latent:
            self.w_down = torch.cat([tensors[n["dq"]], tensors[n["dkv"]]], dim=0).contiguous()
            self.w_uq, self.g_q = tensors[n["uq"]], tensors[n["dq_norm"]]
        else:
            self.w_down, self.w_uq = tensors[n["dkv"]], tensors[n["q"]]
        # the key map moves to the query: per head [kv_rank, head_dim], the layout of a linear layer from
        # head_dim to kv_rank
        self.w_uk_t = tensors[n["uk"]].view(H, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(H, self.v_head_dim, self.kv_rank).contiguous()
        self.w_o = tensors[n["o"]]
        self.g_c = tensors[n["dkv_norm"]]

    def kernel_libraries(self):
        return ["latent_attention", "grouped", "elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def cache_spec(self):
        return PagedKVSpec(1, self.row, self.window, planes=1)

    def state_spec(self):
        return None

    def launch_key(self, n_rows, max_context):
        # the tensor-core kernel's split count is chosen on the host from these numbers
        if not ops.latent_mma_ok(self.dtype, self.row):
            return ()
        tq = ops.LATENT_MMA_ROWS // min(self.n_heads, ops.LATENT_MMA_ROWS)
        span = max_context if not self.window else min(max_context, self.window + tq)
        return (ops.latent_attention_splits(n_rows, self.n_heads, self.kv_rank, span, self.row),)

    def forward(self, ctx, h, call):
        kv = ctx.kv_group(call.kv_group)
        layer = kv.pool[call.kv_layer]
        T, H = ctx.num_tokens, self.n_heads
        with lib.section("qkv"):
            down = ops.linear(h, self.w_down, partials_ok=True)
        cos, sin, rot = self.position.rotation(ctx, self.rope_dim) if self.rope_dim else (None, None, 0)
        cq = ops.latent_prepare(down, 0, self.q_rank, self.q_rank, self.kv_rank, self.rope_dim, rot, self.g_q, self.g_c,
                                self.eps, cos, sin, layer if call.kv_write else None, kv.slot_mapping, kv.page_size, self.dtype)
        with lib.section("q_up"):
            q = ops.materialize(ops.linear(cq if self.q_latent else h, self.w_uq))
        qa = torch.empty((T, H, self.row), dtype=self.dtype, device=q.device)
        with lib.section("absorb"):
            ops.headwise_linear(q.view(T, H, self.head_dim + self.rope_dim), self.w_uk_t, out=qa)
        if self.row > self.kv_rank:      # the rotated tail of the rows, and zeros up to the row size
            ops.latent_rotate_q(q, qa, cos, sin, H, self.head_dim, self.rope_dim, rot, self.kv_rank)
        lat = ops.latent_attention(ctx, qa, layer, kv.block_table, self.kv_rank, self.rope_dim, self.scale, self.window)
        with lib.section("v_up"):
            heads = ops.headwise_linear(lat, self.w_uv)
        with lib.section("o"):
            return ops.linear(heads.view(T, H * self.v_head_dim), self.w_o, partials_ok=True)


register_part("mixer", "latent_attention", LatentAttention)
