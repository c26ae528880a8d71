"""The vocabulary of model parts.

A model is put together from parts of nine categories: ``embed``, ``norm``,
``position``, ``mixer``, ``ffn``, ``block``, ``stream``, ``head`` and ``tail``.  A part

* is described by data: ``PartSpec(kind, params)``; ``kind`` is looked up in the
  registry of its category, ``params`` are the sizes and constants it is built with
  (a part never reads a model configuration and never knows which model it is in);
* lists the checkpoint tensors it owns (``tensors()``: local name -> ``TensorSpec``);
* takes them on the device (``load``), packing them as its kernels want;
* computes on a ``StepContext`` (``pyre_b200.engine.context``), the flat batch of one step.

Interfaces by category (``ctx`` is the StepContext, T its number of tokens):

    embed     forward(ctx) -> x                     fp32 residual stream [T, width]
    norm      forward(ctx, x, delta=None, rows=None, update_x=True) -> h
              h = norm(x + delta) in the activation dtype; writes the sum back to x
              when update_x; with rows, only those rows (gathered), x untouched
    position  apply(ctx, qkv, bias, heads, kv, cache_layer) -> q
              ``qkv``: the stacked projections of the step's tokens [T, (nh + 2 nkv) hd] (a tensor or
              ``kernels.ops.PartialSums``), ``bias`` fp32 or None, ``heads`` a HeadGeometry, ``kv`` the KVView
              of the mixer's cache group.  The part adds the bias, encodes the tokens' positions into the
              queries and keys in whatever way is its own, stores every token's key and value at
              ``kv.slot_mapping`` in ``cache_layer`` (None: store nothing) and returns the queries
              [T, nh hd].  ``PositionEncoding.store`` does the storing for encodings that bring no fused kernel
    mixer     forward(ctx, h, call) -> [T, width]    ``call`` (BoundCall) names the cache
              layer or state layer of this use of the mixer; cache_spec()/state_spec()
              say what it needs from the cache manager
    ffn       forward(ctx, h) -> [T, width]
    block     forward(ctx, x, pending, call) -> (x, pending)   ``pending`` is a branch
              output not yet added to x; the next norm adds it (fused).  A branch output
              (what a mixer or a feed-forward returns, hence ``delta`` and ``pending``) is a
              tensor [T, width] in the activation dtype, or ``kernels.ops.PartialSums`` (fp32
              partial sums that the built-in norm adds up), or ``kernels.ops.DeferredProduct`` (a
              product of few tokens that the built-in norm launches with the residual add folded
              in); a part that needs a plain tensor calls ``kernels.ops.materialize`` on it.
              Likewise a norm may hand a consumer that declares ``takes_scaled_rows``
              ``kernels.ops.ScaledRows`` instead of a tensor (see ``PreNormBlock``)
    stream    forward(ctx, x, pending) -> (x, pending)   a step of a layer that works on the residual stream itself
              after the sublayers (a per-layer input derived from the step's token ids); a block that has one
              calls it last
    head      forward(ctx, h_rows) -> fp32 logits [R, vocab]
    tail      forward(ctx, x, pending) -> fp32 logits [R, vocab] at ``ctx.logit_rows``: everything after the last
              block (the built-in one: a norm over the wanted rows, then a head)

A new part is a class with these methods and one ``register_part`` call; nothing else
in the package has to change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch

from ..weights.specs import TensorSpec

CATEGORIES = ("embed", "norm", "position", "mixer", "ffn", "block", "stream", "head", "tail")


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class PagedKVSpec:
    """What an attention-like mixer needs from the paged cache: per token and layer,
    keys and values of ``n_kv_heads * head_dim`` elements each.  ``window``: only the
    last ``window`` positions are ever read (None = all), so older pages may be given back.
    ``planes``: 2 = a plane of keys and a plane of values per page; 1 = one plane of rows that serve as both (a
    cache of latent rows from which keys and values are derived)."""

    n_kv_heads: int
    head_dim: int
    window: int | None = None
    planes: int = 2

    def bytes_per_token(self, element_size: int) -> int:
        """Bytes of one token's keys and values in one layer of the group."""
        return self.planes * self.n_kv_heads * self.head_dim * element_size

    def tokens_held(self, step_tokens: int) -> "int | None":
        """The most tokens of one request whose pages are held at a time, when a step brings it at most
        ``step_tokens`` new ones: None = all of them (no window); with a window, the window of the step's first
        token and the step's own tokens."""
        return None if self.window is None else self.window - 1 + step_tokens


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per request and per use of the mixer, kept across steps in a
    slot of the cache manager; it starts as zeros when a request begins."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def bytes_per_request(self) -> int:
        """Bytes of one request's state in one layer of the group."""
        n = 1
        for d in self.shape:
            n *= int(d)
        return n * torch.empty((), dtype=self.dtype).element_size()


@dataclass(frozen=True)
class HeadGeometry:
    """How the columns of stacked q, k, v projections divide into heads: ``n_heads`` query heads, then
    ``n_kv_heads`` key heads, then as many value heads, ``head_dim`` columns each."""

    n_heads: int
    n_kv_heads: int
    head_dim: int

    @property
    def width(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim


@dataclass(frozen=True)
class ProjectionLayout:
    """Where a token's queries, keys and values lie in a row of stacked projections when a head's query/key size
    ``qk_dim`` and value size ``v_dim`` are not the cache's row size ``row_dim`` (>= both): ``n_heads`` query heads
    from column ``q_col``, ``n_kv_heads`` key heads from ``k_col`` and as many value heads from ``v_col``
    (``k_col`` < 0: the row holds no keys or values).  The row may hold more columns (a gate)."""

    n_heads: int
    n_kv_heads: int
    qk_dim: int
    v_dim: int
    row_dim: int
    q_col: int = 0
    k_col: int = -1
    v_col: int = -1


@dataclass(frozen=True)
class BoundCall:
    """One entry of the layer schedule, resolved against the cache manager's groups."""

    index: int                 # position in the schedule
    block: int                 # which block's weights
    kv_group: int | None = None
    kv_layer: int = 0          # layer index inside the group's pool
    kv_write: bool = True      # False: read what another call wrote
    state_group: int | None = None
    state_layer: int = 0
    add_embedding: bool = False   # the embedding's output is added to the stream before this entry runs
    add_vector: "tuple | None" = None   # (tensor name, row): that row is added to every token's stream before the entry


class Part:
    category: str = ""
    # True if forward() only launches work on the current stream from device-side inputs
    # (no host reads of the step's arrays, no host synchronisation): such a part may be
    # captured in a CUDA graph and replayed for later steps of the same shape.
    graph_safe: bool = False

    def __init__(self, dtype: torch.dtype, device: torch.device):
        self.dtype = dtype
        self.device = device

    def tensors(self) -> dict[str, TensorSpec]:
        return {}

    def shared_tensors(self) -> dict[str, TensorSpec]:
        """Checkpoint tensors that the part reads but that belong to the model as a whole (a table that every layer
        takes a slice of): FULL checkpoint name -> ``TensorSpec``.  Several parts may name the same tensor; it is
        read once and ``load`` gets it under its full name."""
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take the tensors named by ``tensors()`` (already on the device, already in
        their roles' dtypes) and by ``shared_tensors()``."""

    def kernel_libraries(self) -> list[str]:
        return []

    def children(self) -> "dict[str, Part]":
        """Sub-parts by the name prefix of their tensors."""
        return {}

    def launch_key(self, n_rows: int, max_context: int) -> tuple:
        """What this part's launches take from host-side facts of a step of single tokens
        (``n_rows`` of them, the longest sequence ``max_context`` tokens long) beyond the
        shapes of the step's arrays: a split count, a choice between kernels.  A captured
        step is replayed only for steps whose parts give the same keys.  Hashable items."""
        return ()


class PositionEncoding(Part):
    """Base of the ``position`` parts.  The encoding owns what happens between the q/k/v projections and the
    cache: a mixer hands it the stacked projections and gets the queries back, with keys and values stored.
    The mixer assumes nothing about the encoding (no tables, no rotary width)."""

    category = "position"

    def apply(self, ctx, qkv, bias, heads: HeadGeometry, kv, cache_layer):
        """No encoding at all: bias added, keys and values stored as projected."""
        return self.store(qkv, bias, heads, kv, cache_layer)

    def rotation(self, ctx, qk_dim: int):
        """(cos, sin, rotary_dim) of the step's tokens for heads of ``qk_dim`` dims, or (None, None, 0) for an
        encoding that does not rotate.  Used by ``apply_layout``."""
        return None, None, 0

    def apply_layout(self, ctx, proj, layout: ProjectionLayout, q_norm, k_norm, norm_eps: float, kv, cache_layer,
                     value_tables=None):
        """The same step for projections laid out by a ``ProjectionLayout`` (key and value sizes that differ, rows
        padded to the cache's row size), with an optional RMS norm per head over the query and key dims before
        the encoding (``q_norm`` / ``k_norm``: fp32 weights [qk_dim] or None).  Stores keys and values in
        ``cache_layer`` (None: nothing) and returns the queries [T, n_heads * row_dim].  An encoding that is a
        rotation of leading dims only has to give ``rotation``.  ``value_tables``: (cos, sin) [T, v_dim / 2] of a
        rotation that the mixer wants on the VALUES before they are cached (given only by a mixer that has one)."""
        from ..kernels import ops
        cos, sin, rotary_dim = self.rotation(ctx, layout.qk_dim)
        return ops.qk_norm_rope_write(proj, layout.q_col, layout.k_col, layout.v_col, q_norm, k_norm, norm_eps, cos, sin,
                                      cache_layer, kv.slot_mapping, layout.n_heads, layout.n_kv_heads, layout.qk_dim,
                                      layout.v_dim, layout.row_dim, rotary_dim, kv.page_size,
                                      *(value_tables or ()))

    @staticmethod
    def store(qkv, bias, heads: HeadGeometry, kv, cache_layer):
        """For an encoding without a fused kernel of its own: it transforms the projections first (any way it
        likes) and calls this to add ``bias`` (or None), write every token's key and value to the pages and
        split off the queries."""
        from ..kernels import ops
        return ops.qkv_rope_write(qkv, bias, None, None, cache_layer, kv.slot_mapping, heads.n_heads, heads.n_kv_heads,
                                  heads.head_dim, 0, kv.page_size)


_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: Callable[..., Part], *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; categories: {CATEGORIES}")
    if kind in _REGISTRY[category] and not replace:
        raise ValueError(f"{category} part {kind!r} is already registered")
    _REGISTRY[category][kind] = cls


def registered_parts(category: str) -> list[str]:
    return sorted(_REGISTRY[category])


def make_part(category: str, spec: PartSpec, dtype: torch.dtype, device) -> Part:
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise ValueError(f"unknown {category} part {spec.kind!r}; registered: {registered_parts(category)}") from None
    part = cls(dtype=dtype, device=torch.device(device), **dict(spec.params))
    part.category = category
    return part


def collect_tensors(part: Part, prefix: str = "") -> dict[str, TensorSpec]:
    """Full names of a part's tensors and of its sub-parts', under ``prefix``."""
    out = {prefix + name: spec for name, spec in part.tensors().items()}
    out.update(part.shared_tensors())
    for sub_prefix, child in part.children().items():
        out.update(collect_tensors(child, prefix + sub_prefix))
    return out


def load_part(part: Part, tensors: Mapping[str, torch.Tensor], prefix: str = "") -> None:
    own = {name: tensors[prefix + name] for name, spec in part.tensors().items()
           if prefix + name in tensors or not getattr(spec, "optional", False)}
    own.update({name: tensors[name] for name in part.shared_tensors()})
    part.load(own)
    for sub_prefix, child in part.children().items():
        load_part(child, tensors, prefix + sub_prefix)


def all_graph_safe(part: Part) -> bool:
    return bool(part.graph_safe) and all(all_graph_safe(c) for c in part.children().values())


def collect_launch_keys(part: Part, n_rows: int, max_context: int) -> set:
    """The launch keys of a part and of its sub-parts for a step of single tokens."""
    key = getattr(part, "launch_key", None)
    out = {tuple(key(n_rows, max_context))} if key is not None else set()
    for child in part.children().values():
        out |= collect_launch_keys(child, n_rows, max_context)
    out.discard(())
    return out


def collect_libraries(part: Part) -> list[str]:
    libs = list(part.kernel_libraries())
    for child in part.children().values():
        libs += collect_libraries(child)
    return libs
