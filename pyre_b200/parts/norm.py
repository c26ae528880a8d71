"""RMSNorm (pyre/model.py:22-38) and a layer norm, each fused with the residual add that precedes it."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.specs import TensorSpec
from .base import Part, register_part


class RMSNorm(Part):
    """h = (v / sqrt(mean(v^2) + eps)) * gain with v = x + delta, all in fp32; ``x`` is
    the fp32 residual stream and receives the sum.

    ``offset``: the checkpoint stores ``gain - offset`` (a weight kept around zero has offset 1; the sum is
    formed once, in fp32, at load).  ``tensor_name``: the local name of the weight ("" when the prefix is the
    whole name).  Beside the pre-norm use (``forward``) the same norm can sit on a branch's output:
    ``add_normed`` adds norm(y) * gain to the stream."""

    graph_safe = True
    fuses_into_product = True     # forward takes ``scaled_ok``: with it, the norm may run as the fix-up of the product
                                  # that ``delta`` stands for and hand its consumer ``ops.ScaledRows``

    def __init__(self, dtype, device, width: int, eps: float, offset: float = 0.0, tensor_name: str = "weight"):
        super().__init__(dtype, device)
        self.width, self.eps, self.offset, self.tensor_name = int(width), float(eps), float(offset), str(tensor_name)
        self.weight = None

    def tensors(self):
        return {self.tensor_name: TensorSpec((self.width,), role="vector", init=("normal", 1.0 - self.offset, 0.1))}

    def load(self, tensors):
        w = tensors[self.tensor_name]
        self.weight = w + self.offset if self.offset else w

    def kernel_libraries(self):
        return ["elementwise"]

    def forward(self, ctx, x, delta=None, rows=None, update_x=True, scaled_ok=False):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, self.dtype, rows=rows, update_x=update_x, scaled_ok=scaled_ok)

    def add_normed(self, ctx, x, y, want_next: bool = False):
        """x += norm(y) * gain on the fp32 stream, ``y`` a branch's output; with ``want_next`` the new stream comes
        back as activations for the branch that reads it next."""
        return ops.norm_add(x, y, self.weight, self.eps, self.dtype, want_next=want_next)

    def gated_output(self, ctx, y, gate=None, gate_bias=None):
        """norm(y * sigmoid(gate + gate_bias)) * gain for a sublayer's result ``y`` that is not added to the stream
        here: it comes back as an fp32 branch output (one unrounded part in bfloat16) for the next norm to add."""
        out = ops.gated_norm(y, None, gate, gate_bias, self.weight, self.eps, self.dtype, center=False)
        return out if self.dtype == torch.float32 else ops.PartialSums(out.unsqueeze(0), self.dtype)


register_part("norm", "rms_norm", RMSNorm)


class LayerNorm(Part):
    """h = (v - mean(v)) / sqrt(var(v) + eps) * gain (+ bias) with v = x + delta, all in fp32; var is the mean
    squared deviation.  ``bias_name``: the local name of a bias per feature (None: the norm has none).  ``x`` is the fp32 residual stream and receives the sum.  ``delta`` may be an
    ``ops.ScaledSum`` (several branch outputs, each with a gain per feature): the kernel adds its terms itself.
    ``tensor_name``: the local name of the weight ("" when the prefix is the whole name).
    ``normalize_stream`` applies the norm to the stream itself (fp32 in, fp32 out): a norm right after the
    embedding."""

    graph_safe = True
    takes_scaled_sum = True

    def __init__(self, dtype, device, width: int, eps: float, tensor_name: str = "weight", bias_name: "str | None" = None):
        super().__init__(dtype, device)
        self.width, self.eps, self.tensor_name = int(width), float(eps), str(tensor_name)
        self.bias_name = None if bias_name is None else str(bias_name)
        self.weight = self.bias = None

    def tensors(self):
        t = {self.tensor_name: TensorSpec((self.width,), role="vector", init=("normal", 1.0, 0.1))}
        if self.bias_name is not None:
            t[self.bias_name] = TensorSpec((self.width,), role="vector", init=("normal", 0.0, 0.1))
        return t

    def load(self, tensors):
        self.weight = tensors[self.tensor_name]
        self.bias = tensors[self.bias_name] if self.bias_name is not None else None

    def kernel_libraries(self):
        return ["parallel_block", "blockops"]

    def forward(self, ctx, x, delta=None, rows=None, update_x=True, scaled_ok=False):
        return ops.add_layernorm(x, delta, self.weight, self.eps, self.dtype, rows=rows, update_x=update_x, bias=self.bias)

    def gated_output(self, ctx, y, gate=None, gate_bias=None):
        """norm(y * sigmoid(gate + gate_bias)) * gain for a sublayer's result ``y`` that is not added to the stream
        here: it comes back as an fp32 branch output (one unrounded part in bfloat16) for the next norm to add."""
        out = ops.gated_norm(y, None, gate, gate_bias, self.weight, self.eps, self.dtype, center=True, out_bias=self.bias)
        return out if self.dtype == torch.float32 else ops.PartialSums(out.unsqueeze(0), self.dtype)

    def normalize_stream(self, ctx, x):
        return ops.add_layernorm(x, None, self.weight, self.eps, torch.float32, act_dtype=self.dtype, bias=self.bias)


register_part("norm", "layer_norm", LayerNorm)
