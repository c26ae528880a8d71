"""A per-layer input derived from the step's token ids, added to the residual stream after a layer's sublayers."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, register_part


class TokenSideInput(Part):
    """With e the token's row of a side table restricted to this layer's ``dim`` columns (from ``col``):

        g = gelu_tanh(W_gate x) * e;   y = W_proj g;   x <- x + y / sqrt(mean(y^2) + eps) * gain

    x is the fp32 stream after the layer's sublayers (a branch output still pending is added first, unrounded).  The
    table [vocab, table_width] belongs to the model (``table_name`` is its full checkpoint name; every layer reads its
    own columns of the one tensor).  The two small products run in the compute dtype; the sum and the norm are fp32.
    ``names``: local names of the two projections and the gain."""

    DEFAULT_NAMES = {"gate": "gate", "proj": "proj", "norm": "norm"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, dim: int, vocab: int, table_name: str, table_width: int, col: int, eps: float,
                 names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.dim, self.vocab, self.table_name = int(width), int(dim), int(vocab), str(table_name)
        self.table_width, self.col, self.eps = int(table_width), int(col), float(eps)
        if self.dim <= 0 or self.col < 0 or self.col + self.dim > self.table_width:
            raise ValueError(f"columns {col}..{col + dim} do not lie inside table rows of {table_width}")
        self.table = self.w_gate = self.w_proj = self.norm_w = None

    def tensors(self):
        n = self.names
        return {n["gate"]: TensorSpec((self.dim, self.width)), n["proj"]: TensorSpec((self.width, self.dim)),
                n["norm"]: TensorSpec((self.width,), role="vector", init=("normal", 1.0, 0.1))}

    def shared_tensors(self):
        return {self.table_name: TensorSpec((self.vocab, self.table_width), init=("normal", 0.0, 1.0))}

    def load(self, tensors):
        n = self.names
        self.table, self.w_gate, self.w_proj, self.norm_w = tensors[self.table_name], tensors[n["gate"]], tensors[n["proj"]], tensors[n["norm"]]

    def kernel_libraries(self):
        return ["seqmix", "blockops", "elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def forward(self, ctx, x, pending):
        if pending is not None:
            if isinstance(pending, ops.PartialSums):
                for i in range(pending.n):
                    ops.add_residual(x, pending.parts[i])          # fp32 parts enter the stream unrounded
            else:
                ops.add_residual(x, ops.materialize(pending))
        with lib.section("side"):
            pre = ops.materialize(ops.linear(ops.cast_rows(x, self.dtype), self.w_gate))
            g = ops.side_gate(pre, self.table, self.col, ctx.token_ids, err_flag=ctx.error_flag)
            y = ops.linear(g, self.w_proj, partials_ok=True)
        ops.norm_add(x, y, self.norm_w, self.eps, self.dtype)
        return x, None


register_part("stream", "token_side_input", TokenSideInput)
