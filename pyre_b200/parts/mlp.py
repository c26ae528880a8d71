"""Dense feed-forwards: the gated one (SwiGLU, pyre/model.py:128-139) and the plain one (up, activation, down)."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, PartSpec, make_part, register_part


class GatedMLP(Part):
    """down(act(gate(h)) * up(h)) without biases.  The gate and up weights are stacked
    into one [2 I, width] matrix at load, so one product feeds the activation; in bfloat16,
    when I is a multiple of 128, their rows alternate in blocks of 64 features so that one
    output tile of the product holds both halves and the activation runs in its epilogue.
    ``names``: the checkpoint's names of the three projections (default gate_proj, up_proj, down_proj);
    ``weight_suffix``: what follows a projection's name (".weight").  ``activation``: ``silu``, or ``gelu_tanh``
    (product, then the activation kernel on the stacked [gates | ups])."""

    DEFAULT_NAMES = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}

    graph_safe = True
    takes_scaled_rows = True      # ``h`` may be ``ops.ScaledRows``: the gate/up product applies the norm's 1/rms itself

    def __init__(self, dtype, device, width: int, intermediate: int, activation: str = "silu",
                 names: "dict[str, str] | None" = None, weight_suffix: str = ".weight"):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.suffix = str(weight_suffix)
        self.width, self.intermediate = int(width), int(intermediate)
        if activation not in ops.ACTIVATIONS:
            raise ops.UnsupportedSize(f"activation {activation!r}: implemented are {sorted(ops.ACTIVATIONS)}")
        self.activation = activation
        self.w_gate_up = self.w_down = None
        # the product's epilogue knows silu; another activation runs after the product on [gates | ups]
        self.interleaved = activation == "silu" and dtype == torch.bfloat16 and self.intermediate % (2 * ops.GATED_BLOCK) == 0
        if activation != "silu":
            self.takes_scaled_rows = False

    def tensors(self):
        n, sfx = self.names, self.suffix
        return {
            n["gate"] + sfx: TensorSpec((self.intermediate, self.width)),
            n["up"] + sfx: TensorSpec((self.intermediate, self.width)),
            n["down"] + sfx: TensorSpec((self.width, self.intermediate)),
        }

    def load(self, tensors):
        n, sfx = self.names, self.suffix
        gate, up = tensors[n["gate"] + sfx], tensors[n["up"] + sfx]
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[n["down"] + sfx]

    def kernel_libraries(self):
        return ["elementwise"] + (["parallel_block"] if self.activation != "silu" else []) + \
            (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def forward(self, ctx, h):
        with lib.section("gate_up"):
            if self.activation == "silu":
                act = ops.gated_linear(h, self.w_gate_up, self.interleaved)
            else:
                act = ops.act_mul(ops.materialize(ops.linear(h, self.w_gate_up)), self.activation)
        with lib.section("down"):
            return ops.linear(act, self.w_down, partials_ok=True, deferred_ok="residual")


register_part("ffn", "gated_mlp", GatedMLP)


class DenseMLP(Part):
    """down(act(up(h))): a feed-forward with one product before the activation.
    ``activation``: ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))), ``silu`` or ``relu2`` (the
    square of relu), computed in fp32 on the product's result.  ``bias``: both projections have one (names ``up_bias``
    / ``down_bias``); the first is added before the activation, the second to the result.  ``names``: the
    checkpoint's full local names of the tensors."""

    DEFAULT_NAMES = {"up": "up_proj.weight", "down": "down_proj.weight", "up_bias": "up_proj.bias", "down_bias": "down_proj.bias"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, intermediate: int, activation: str = "gelu_tanh",
                 names: "dict[str, str] | None" = None, bias: bool = False):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.intermediate, self.bias = int(width), int(intermediate), bool(bias)
        if activation not in ops.BIAS_ACTIVATIONS or activation is None:
            raise ops.UnsupportedSize(f"activation {activation!r}: implemented are {sorted(k for k in ops.BIAS_ACTIVATIONS if k)}")
        self.activation = activation
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def tensors(self):
        t = {self.names["up"]: TensorSpec((self.intermediate, self.width)),
             self.names["down"]: TensorSpec((self.width, self.intermediate))}
        if self.bias:
            t[self.names["up_bias"]] = TensorSpec((self.intermediate,), role="vector")
            t[self.names["down_bias"]] = TensorSpec((self.width,), role="vector")
        return t

    def load(self, tensors):
        self.w_up, self.w_down = tensors[self.names["up"]], tensors[self.names["down"]]
        if self.bias:
            self.b_up, self.b_down = tensors[self.names["up_bias"]], tensors[self.names["down_bias"]]

    def kernel_libraries(self):
        return ["blockops", "elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def forward(self, ctx, h):
        with lib.section("up"):
            if self.bias or self.activation not in ops.ACTIVATIONS:
                a = ops.bias_act(ops.materialize(ops.linear(h, self.w_up)), self.b_up, self.activation)
            else:
                a = ops.linear_act(h, self.w_up, self.activation)
        with lib.section("down"):
            y = ops.linear(a, self.w_down, partials_ok=not self.bias)
            return ops.bias_act(ops.materialize(y), self.b_down, None) if self.bias else y


register_part("ffn", "dense_mlp", DenseMLP)


class RoutedMLP(Part):
    """A routed feed-forward: ``n_experts`` small gated feed-forwards (down(act(gate(h)) * up(h)), no biases) and
    ``n_identity`` further router outputs without weights whose "expert" returns h itself; each token uses ``top``
    of them.  The router's logits W_r h are fp32, the scores a softmax over ALL router outputs; the choice takes
    the ``top`` largest of score + correction (a tensor per router output, ``correction=True``), the weights are the
    chosen outputs' plain scores times ``scale``, not renormalised.  The result is the weighted sum.
    ``scores="sigmoid"``: each router output's score is its own sigmoid instead of the softmax over all.
    ``weight_on="input"``: the weight multiplies what the expert READS (the result is the plain sum of
    expert(weight * h); needs ``n_identity`` 0); ``"output"``: what it returns.
    ``shared``: the intermediate size of one more feed-forward of the same form that runs for every token and
    is added (names under ``shared``), or None.
    ``gated=False``: an expert is down(act(up(h))) with ``activation`` silu, gelu_tanh or relu2 (no gate projection).
    ``router_bias``: a bias per router output added to the logits (name ``router_bias``).  ``renormalise``: the chosen
    weights are divided by their sum (with softmax scores: the softmax over the chosen logits alone).
    ``shared_gate``: the shared expert's result is multiplied by sigmoid(w_sg . h), one number per token (name
    ``shared_gate``, a tensor [1, width]).

    On the device throughout (no host reads): the router kernel, a sort of the (token, choice) pairs by expert,
    two products with one weight matrix per expert over the sorted pairs with the activation between them, and the
    weighted sum per token in fp32.  ``names``: the prefix of expert e's tensors (``expert``, formatted with e), the
    local names of its three projections, the router's and the correction's names."""

    DEFAULT_NAMES = {"expert": "e{e}.", "gate": "gate", "up": "up", "down": "down", "router": "router", "correction": "correction",
                     "shared": "shared.", "router_bias": "router.b", "shared_gate": "shared.sg"}

    graph_safe = True

    def __init__(self, dtype, device, width: int, intermediate: int, n_experts: int, top: int, scale: float = 1.0,
                 n_identity: int = 0, activation: str = "silu", correction: bool = True, names: "dict[str, str] | None" = None,
                 scores: str = "softmax", weight_on: str = "output", shared: "int | None" = None, gated: bool = True,
                 router_bias: bool = False, renormalise: bool = False, shared_gate: bool = False):
        super().__init__(dtype, device)
        self.gated, self.router_bias, self.renormalise = bool(gated), bool(router_bias), bool(renormalise)
        self.shared_gate = bool(shared_gate) and bool(shared)
        if self.router_bias and int(n_identity):
            raise ValueError("a router bias and router outputs without weights do not go together")
        if scores not in ("softmax", "sigmoid") or weight_on not in ("output", "input"):
            raise ValueError(f"router scores {scores!r} / weight_on {weight_on!r}: 'softmax' or 'sigmoid', 'output' or 'input'")
        if weight_on == "input" and n_identity:
            raise ValueError("weights on the experts' inputs and router outputs without weights do not go together")
        self.sigmoid, self.weight_on_input = scores == "sigmoid", weight_on == "input"
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.intermediate = int(width), int(intermediate)
        self.n_experts, self.n_identity, self.top, self.scale = int(n_experts), int(n_identity), int(top), float(scale)
        known = ops.ACTIVATIONS if self.gated else {k: v for k, v in ops.BIAS_ACTIVATIONS.items() if k not in (None, "tanh")}
        if activation not in known:
            raise ops.UnsupportedSize(f"activation {activation!r}: implemented are {sorted(known)}")
        if self.n_experts <= 0 or self.n_identity < 0 or not 0 < self.top <= self.n_experts + self.n_identity:
            raise ValueError(f"a routed feed-forward of {n_experts} + {n_identity} experts cannot choose {top}")
        self.activation, self.has_correction = activation, bool(correction)
        self.w_gate_up = self.w_down = self.w_router = self.correction = self._ones = self.b_router = self.w_shared_gate = None
        n = self.names
        if not shared:
            self.shared = None
        elif self.gated:
            self.shared = make_part("ffn", PartSpec("gated_mlp", {
                "width": self.width, "intermediate": int(shared), "activation": activation, "weight_suffix": "",
                "names": {"gate": n["gate"], "up": n["up"], "down": n["down"]}}), dtype, device)
        else:
            self.shared = make_part("ffn", PartSpec("dense_mlp", {
                "width": self.width, "intermediate": int(shared), "activation": activation,
                "names": {"up": n["up"], "down": n["down"]}}), dtype, device)

    def children(self):
        return {self.names["shared"]: self.shared} if self.shared is not None else {}

    def tensors(self):
        n, t = self.names, {}
        for e in range(self.n_experts):
            pre = n["expert"].format(e=e)
            if self.gated:
                t[pre + n["gate"]] = TensorSpec((self.intermediate, self.width))
            t[pre + n["up"]] = TensorSpec((self.intermediate, self.width))
            t[pre + n["down"]] = TensorSpec((self.width, self.intermediate))
        outs = self.n_experts + self.n_identity
        t[n["router"]] = TensorSpec((outs, self.width), role="vector", init=("normal", 0.0, 0.05))
        if self.has_correction:
            t[n["correction"]] = TensorSpec((outs,), role="vector", init=("normal", 0.0, 0.02))
        if self.router_bias:
            t[n["router_bias"]] = TensorSpec((outs,), role="vector", init=("normal", 0.0, 0.05))
        if self.shared_gate:
            t[n["shared_gate"]] = TensorSpec((1, self.width), role="vector", init=("normal", 0.0, 0.05))
        return t

    def load(self, tensors):
        n = self.names
        pres = [n["expert"].format(e=e) for e in range(self.n_experts)]
        if self.gated:
            self.w_gate_up = torch.stack([torch.cat([tensors[p + n["gate"]], tensors[p + n["up"]]], dim=0) for p in pres]).contiguous()
        else:
            self.w_gate_up = torch.stack([tensors[p + n["up"]] for p in pres]).contiguous()
        self.w_down = torch.stack([tensors[p + n["down"]] for p in pres]).contiguous()
        self.w_router = tensors[n["router"]]
        self.correction = tensors[n["correction"]] if self.has_correction else None
        self.b_router = tensors[n["router_bias"]] if self.router_bias else None
        self.w_shared_gate = tensors[n["shared_gate"]].reshape(-1).contiguous() if self.shared_gate else None

    def kernel_libraries(self):
        return ["grouped", "parallel_block"] + ([] if self.gated else ["blockops"]) + (["seqmix"] if self.shared_gate else [])

    def forward(self, ctx, h):
        h = ops.materialize(h)
        T = h.shape[0]
        idx, weight = ops.route(h, self.w_router, self.correction, self.top, self.scale, sigmoid=self.sigmoid,
                                bias=self.b_router, renormalise=self.renormalise)
        offsets, place_of, src = ops.group_pairs(idx, self.n_experts)
        places = T * self.top
        x = h
        if self.weight_on_input:
            # the experts read weight * h, laid out by place; their results are summed unweighted
            x, src = ops.scale_to_places(h, place_of, weight, places), None
            weight = torch.ones_like(weight)
        with lib.section("experts_gate_up"):
            gu = ops.expert_linear(x, self.w_gate_up, offsets, src, places)
        act = ops.act_mul(gu, self.activation) if self.gated else ops.bias_act(gu, None, self.activation)
        with lib.section("experts_down"):
            y = ops.expert_linear(act, self.w_down, offsets, None, places, out_dtype=torch.float32)
        out = ops.combine_pairs(y, h, place_of, weight)
        if self.shared is not None and self.shared_gate:
            ops.token_gate_add(out, h, self.w_shared_gate, ops.materialize(self.shared.forward(ctx, h)))
        elif self.shared is not None:
            ops.add_residual(out, ops.materialize(self.shared.forward(ctx, h)))
        # fp32 [T, width]: in bfloat16 it travels as the one part of a split product, which every norm adds unrounded
        return out if self.dtype == torch.float32 else ops.PartialSums(out.unsqueeze(0), self.dtype)


register_part("ffn", "routed_mlp", RoutedMLP)
