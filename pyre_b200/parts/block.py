"""Arrangements of a layer's parts: the pre-norm residual block (pyre/model.py:142-153), a block whose norms
sit on the branches' outputs, and a block whose branches read one norm's output side by side."""

from __future__ import annotations

from .base import Part, PartSpec, make_part, register_part


class PreNormBlock(Part):
    """x = x + mixer(norm1(x)); x = x + ffn(norm2(x)).

    The residual stream ``x`` is fp32.  A branch output is not added at once: it
    travels as ``pending`` to the next norm, whose kernel adds it to x while it
    normalises (one pass over the row instead of three).  The block therefore returns
    (x, pending) with the feed-forward's output still pending.

    ``names`` gives the prefix of each sub-part's tensors inside the layer."""

    graph_safe = True

    DEFAULT_NAMES = {"norm1": "input_layernorm.", "mixer": "self_attn.",
                     "norm2": "post_attention_layernorm.", "ffn": "mlp."}

    def __init__(self, dtype, device, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec,
                 names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.norm1 = make_part("norm", norm1, dtype, device)
        self.mixer = make_part("mixer", mixer, dtype, device)
        self.norm2 = make_part("norm", norm2, dtype, device)
        self.ffn = make_part("ffn", ffn, dtype, device)
        # A norm that can run as the fix-up of the product before it hands its consumer activations that still lack
        # the 1/rms factor (``ops.ScaledRows``); it may do so only for a consumer that says it takes them.  Both are
        # opt-in attributes of the parts; parts without them see plain tensors.

        def lazy(norm, consumer):
            ok = getattr(norm, "fuses_into_product", False) and getattr(consumer, "takes_scaled_rows", False)
            return {"scaled_ok": True} if ok else {}
        self._kw1, self._kw2 = lazy(self.norm1, self.mixer), lazy(self.norm2, self.ffn)

    def children(self):
        return {self.names["norm1"]: self.norm1, self.names["mixer"]: self.mixer,
                self.names["norm2"]: self.norm2, self.names["ffn"]: self.ffn}

    def forward(self, ctx, x, pending, call):
        h = self.norm1.forward(ctx, x, delta=pending, **self._kw1)
        a = self.mixer.forward(ctx, h, call)
        h = self.norm2.forward(ctx, x, delta=a, **self._kw2)
        return x, self.ffn.forward(ctx, h)


register_part("block", "prenorm", PreNormBlock)


class OutputNormBlock(Part):
    """x = x + norm1(mixer(x)); x = x + norm2(ffn(x)): the norms sit on the branches' OUTPUTS and the branches
    read the stream itself.  ``norm2`` and ``ffn`` may both be None: a layer with one branch.

    The residual stream ``x`` is fp32 and is updated in place by the norm's kernel, which also leaves the new
    stream as activations for the branch that reads it next (one pass over the row); the block therefore never
    leaves anything pending.  A branch output still pending from a block before it is added first.

    ``names`` gives the prefix of each sub-part's tensors inside the layer."""

    graph_safe = True

    DEFAULT_NAMES = {"norm1": "norm1.", "mixer": "mixer.", "norm2": "norm2.", "ffn": "ffn."}
    _STREAM = "stream_as_activations"      # ctx.scratch: (the stream tensor, its activations) left by the last norm

    def __init__(self, dtype, device, norm1: PartSpec, mixer: PartSpec, norm2: "PartSpec | None" = None,
                 ffn: "PartSpec | None" = None, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        if (norm2 is None) != (ffn is None):
            raise ValueError("a second branch needs both its norm and its feed-forward")
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.norm1 = make_part("norm", norm1, dtype, device)
        self.mixer = make_part("mixer", mixer, dtype, device)
        self.norm2 = make_part("norm", norm2, dtype, device) if norm2 is not None else None
        self.ffn = make_part("ffn", ffn, dtype, device) if ffn is not None else None
        for n in (self.norm1, self.norm2):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError(f"{type(n).__name__} cannot sit on a branch's output: it has no add_normed")

    def children(self):
        out = {self.names["norm1"]: self.norm1, self.names["mixer"]: self.mixer}
        if self.ffn is not None:
            out[self.names["norm2"]] = self.norm2
            out[self.names["ffn"]] = self.ffn
        return out

    def kernel_libraries(self):
        return ["elementwise", "blockops"]

    def forward(self, ctx, x, pending, call):
        from ..kernels import ops
        left = ctx.scratch.pop(self._STREAM, None)
        if pending is not None:
            ops.add_residual(x, ops.materialize(pending))
            left = None
        h = left[1] if left is not None and left[0] is x else ops.cast_rows(x, self.dtype)
        h = self.norm1.add_normed(ctx, x, self.mixer.forward(ctx, h, call), want_next=True)
        if self.ffn is not None:
            h = self.norm2.add_normed(ctx, x, self.ffn.forward(ctx, h), want_next=True)
        ctx.scratch[self._STREAM] = (x, h)
        return x, None


register_part("block", "output_norm", OutputNormBlock)


class ParallelBlock(Part):
    """x = x + m * (g1 * mixer(h) + g2 * ffn(h)) with h = norm1(x): ONE norm, both branches read its output, and
    their results enter the stream together.  ``residual_mult`` is m; ``layer_scale``: g1 and g2 are gains per
    feature read from the checkpoint (names ``ls1`` / ``ls2``), else ones.  ``ffn`` None: the layer has the mixer
    only.

    Nothing is added here: the branches travel as ``ops.ScaledSum`` (each with its gain times m, formed once in
    fp32 at load) to the next norm, whose kernel adds them to the fp32 stream while it normalises."""

    graph_safe = True

    DEFAULT_NAMES = {"norm1": "norm1.", "mixer": "mixer.", "ffn": "ffn.", "ls1": "ls1", "ls2": "ls2"}

    def __init__(self, dtype, device, width: int, norm1: PartSpec, mixer: PartSpec, ffn: "PartSpec | None" = None,
                 residual_mult: float = 1.0, layer_scale: bool = False, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.residual_mult, self.layer_scale = int(width), float(residual_mult), bool(layer_scale)
        self.norm1 = make_part("norm", norm1, dtype, device)
        self.mixer = make_part("mixer", mixer, dtype, device)
        self.ffn = make_part("ffn", ffn, dtype, device) if ffn is not None else None
        self.gain1 = self.gain2 = None

    def children(self):
        out = {self.names["norm1"]: self.norm1, self.names["mixer"]: self.mixer}
        if self.ffn is not None:
            out[self.names["ffn"]] = self.ffn
        return out

    def tensors(self):
        from ..weights.specs import TensorSpec
        if not self.layer_scale:
            return {}
        t = {self.names["ls1"]: TensorSpec((self.width,), role="vector", init=("normal", 1.0, 0.1))}
        # a layer without a feed-forward has no use for the second gain; a checkpoint may hold it all the same
        t[self.names["ls2"]] = TensorSpec((self.width,), role="vector", init=("normal", 1.0, 0.1), optional=self.ffn is None)
        return t

    def load(self, tensors):
        import torch
        m = self.residual_mult
        ones = torch.ones(self.width, dtype=torch.float32, device=self.device) if not self.layer_scale else None
        self.gain1 = (tensors[self.names["ls1"]] if self.layer_scale else ones) * m
        if self.ffn is not None:
            self.gain2 = (tensors[self.names["ls2"]] if self.layer_scale else ones) * m

    def kernel_libraries(self):
        return ["parallel_block"]

    def forward(self, ctx, x, pending, call):
        from ..kernels import ops
        if pending is not None and isinstance(pending, ops.ScaledSum) and not getattr(self.norm1, "takes_scaled_sum", False):
            pending = ops.materialize(pending)
        h = self.norm1.forward(ctx, x, delta=pending)
        terms = [(self.mixer.forward(ctx, h, call), self.gain1)]
        if self.ffn is not None:
            terms.append((self.ffn.forward(ctx, h), self.gain2))
        return x, ops.ScaledSum(terms, self.dtype)


register_part("block", "parallel", ParallelBlock)


class SandwichBlock(Part):
    """A norm before AND after each sublayer, and a gate per feature on the sublayer's result:

        h = norm1(x);  x = x + norm1b(mixer(h) * sigmoid(W_g1 h + b_g1))
        h = norm2(x);  x = x + norm2b(ffn(h)   * sigmoid(W_g2 h + b_g2))

    The gate reads what the sublayer reads and comes before the norm of the sublayer's result.  ``gated=False``: no
    gates (a plain sandwich of norms).  ``ffn`` None (with ``norm2`` and ``norm2b`` None): the layer has the mixer only.

    The stream ``x`` is fp32.  A sublayer's gated, normed result is formed in fp32 by one kernel (``gated_output`` of
    the norm part) and travels unadded, as ``pending``, to the next norm before a sublayer, whose kernel adds it to
    the stream while it normalises.  ``after``: a ``stream`` part that runs once the sublayers are done (a per-layer
    input from the step's token ids); it gets the stream and what is pending.  ``names``: the prefixes of the
    sub-parts' tensors and the names of the gates' weights and biases."""

    graph_safe = True

    DEFAULT_NAMES = {"norm1": "norm1.", "norm1b": "norm1b.", "mixer": "mixer.", "norm2": "norm2.", "norm2b": "norm2b.",
                     "ffn": "ffn.", "gate1": "gate1.weight", "gate1_bias": "gate1.bias", "gate2": "gate2.weight",
                     "gate2_bias": "gate2.bias", "after": "after."}

    def __init__(self, dtype, device, width: int, norm1: PartSpec, mixer: PartSpec, norm1b: PartSpec,
                 norm2: "PartSpec | None" = None, ffn: "PartSpec | None" = None, norm2b: "PartSpec | None" = None,
                 gated: bool = True, names: "dict[str, str] | None" = None, after: "PartSpec | None" = None):
        super().__init__(dtype, device)
        self.after = make_part("stream", after, dtype, device) if after is not None else None
        if len({norm2 is None, ffn is None, norm2b is None}) != 1:
            raise ValueError("a second sublayer needs its feed-forward and both of its norms")
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.gated = int(width), bool(gated)
        self.norm1 = make_part("norm", norm1, dtype, device)
        self.mixer = make_part("mixer", mixer, dtype, device)
        self.norm1b = make_part("norm", norm1b, dtype, device)
        self.norm2 = make_part("norm", norm2, dtype, device) if norm2 is not None else None
        self.ffn = make_part("ffn", ffn, dtype, device) if ffn is not None else None
        self.norm2b = make_part("norm", norm2b, dtype, device) if norm2b is not None else None
        for n in (self.norm1b, self.norm2b):
            if n is not None and not hasattr(n, "gated_output"):
                raise ValueError(f"{type(n).__name__} cannot sit on a sublayer's result: it has no gated_output")
        self.w_g1 = self.b_g1 = self.w_g2 = self.b_g2 = None

    def children(self):
        n = self.names
        out = {n["norm1"]: self.norm1, n["mixer"]: self.mixer, n["norm1b"]: self.norm1b}
        if self.ffn is not None:
            out.update({n["norm2"]: self.norm2, n["ffn"]: self.ffn, n["norm2b"]: self.norm2b})
        if self.after is not None:
            out[n["after"]] = self.after
        return out

    def tensors(self):
        from ..weights.specs import TensorSpec
        if not self.gated:
            return {}
        n, W = self.names, self.width
        t = {n["gate1"]: TensorSpec((W, W)), n["gate1_bias"]: TensorSpec((W,), role="vector")}
        if self.ffn is not None:
            t.update({n["gate2"]: TensorSpec((W, W)), n["gate2_bias"]: TensorSpec((W,), role="vector")})
        return t

    def load(self, tensors):
        if not self.gated:
            return
        n = self.names
        self.w_g1, self.b_g1 = tensors[n["gate1"]], tensors[n["gate1_bias"]]
        if self.ffn is not None:
            self.w_g2, self.b_g2 = tensors[n["gate2"]], tensors[n["gate2_bias"]]

    def kernel_libraries(self):
        import torch
        return ["blockops"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def _sublayer(self, ctx, h, branch, w_gate, b_gate, norm_b):
        from ..kernels import lib, ops
        gate = None
        if self.gated:
            with lib.section("residual_gate"):
                gate = ops.materialize(ops.linear(h, w_gate))
        return norm_b.gated_output(ctx, branch, gate, b_gate)

    def forward(self, ctx, x, pending, call):
        h = self.norm1.forward(ctx, x, delta=pending)
        pending = self._sublayer(ctx, h, self.mixer.forward(ctx, h, call), self.w_g1, self.b_g1, self.norm1b)
        if self.ffn is not None:
            h = self.norm2.forward(ctx, x, delta=pending)
            pending = self._sublayer(ctx, h, self.ffn.forward(ctx, h), self.w_g2, self.b_g2, self.norm2b)
        if self.after is not None:
            return self.after.forward(ctx, x, pending)
        return x, pending


register_part("block", "sandwich", SandwichBlock)
