"""The kernels as Python functions over torch tensors.

Each function checks shapes, dtypes, contiguity and device, then launches the CUDA
kernel on torch's current stream.  A size the kernels do not take is refused with a
clear error; nothing here computes on the CPU or falls back to a library.

The matrix products are the package's own kernels too (``gemm_tc`` on the tcgen05 tensor
cores for bfloat16, ``sgemm_nt`` for float32).  One case goes to a library (cuBLAS through
``torch``): a bfloat16 product whose rows are no multiple of 16 bytes, which a TMA copy
cannot fetch; the reference's engine uses a library for every projection (``nn.Linear``,
pyre/model.py:84-87,133-135,172).  See ``linear``.
"""

from __future__ import annotations

import ctypes

import torch

from . import lib

_DT = {torch.float32: 0, torch.bfloat16: 1}


class UnsupportedSize(ValueError):
    """A configuration whose sizes the kernels refuse."""


class PartialSums:
    """fp32 partial sums [n, T, N] of a matrix product whose inner dimension was split over
    CTAs.  The kernels that consume a product (``add_rmsnorm``, ``qkv_rope_write``) add the n
    parts themselves, in index order, so no separate reduction runs; anything else calls
    ``materialize``."""

    def __init__(self, parts: torch.Tensor, dtype: torch.dtype):
        self.parts = parts          # contiguous [n, T, N] float32
        self.dtype = dtype          # what materialize() rounds to

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def n(self) -> int:
        return self.parts.shape[0]


class ScaledRows:
    """Activations that carry a norm's weight but not yet its 1/rms: ``rows`` [T, H] bf16 and, per token, the
    sums of squares of the normalised vector's elements in tiles of 128 features (``ssq`` [tiles, T] fp32).  The
    normalised activations are ``rows[t] / sqrt(sum(ssq[:, t]) / H + eps)``.  A product that takes them applies the
    factor to its result rows in its epilogue (the factor is a scalar per row, so it commutes with the product);
    anything else calls ``materialize``."""

    def __init__(self, rows: torch.Tensor, ssq: torch.Tensor, eps: float):
        self.rows, self.ssq, self.eps = rows, ssq, float(eps)

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    @property
    def device(self):
        return self.rows.device


class DeferredProduct:
    """y = x w^T of a linear layer over few tokens, not launched yet.  The kernel that consumes it decides how it
    runs: the built-in norm launches it with a fix-up that adds the result to the residual stream and prepares the
    normalised activations (no norm kernel), the rotary position encoding with one that adds the bias, rotates and
    writes keys and values to the pages (no rotary kernel); anything else calls ``partials`` or ``materialize``."""

    def __init__(self, x: "torch.Tensor | ScaledRows", w: torch.Tensor, dtype: torch.dtype):
        self.x, self.w, self.dtype = x, w, dtype
        self.section = lib.current_section()      # the kernel class its launch counts for, whoever launches it

    @property
    def shape(self):
        return (self.x.shape[0], self.w.shape[0])

    @property
    def device(self):
        return self.w.device

    def partials(self) -> "torch.Tensor | PartialSums":
        """Launch the plain product: a tensor, or partial sums where K is split."""
        with lib.section(self.section):
            return gemm_tc(self.x, self.w, self.dtype, reduce=False)


def materialize(t: "torch.Tensor | PartialSums | DeferredProduct | ScaledRows | ScaledSum") -> torch.Tensor:
    """A plain tensor in the activation dtype from a tensor or any of the lazy forms a branch output or a
    norm's output may take."""
    if isinstance(t, ScaledSum):
        return t.tensor()
    if isinstance(t, DeferredProduct):
        t = t.partials()
    if isinstance(t, ScaledRows):
        out = torch.empty_like(t.rows)
        T, H = t.rows.shape
        lib.call("pyre_scale_rows", t.rows.data_ptr(), t.ssq.data_ptr(), t.ssq.shape[0], out.data_ptr(), T, H, t.eps, _stream())
        return out
    if not isinstance(t, PartialSums):
        return t
    out = torch.empty(tuple(t.shape), dtype=t.dtype, device=t.parts.device)
    n = t.parts[0].numel()
    lib.call("pyre_sum_partials", t.parts.data_ptr(), t.n, n, out.data_ptr(), n, _dt(t.dtype), _stream())
    return out


# A step of prompt portions is a few hundred launches from Python, so the two questions every launch asks (which
# stream, which device) go to torch's C layer directly where it offers that (a fraction of a microsecond instead of
# several); the public calls stand in where it does not.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _current_device() -> int:
    return _raw_device() if _raw_device is not None else torch.cuda.current_device()


def _stream() -> int:
    """The current stream of the current device.  Kernels are launched in the current device's
    context, so the tensors of a call must live there (``_check`` refuses others)."""
    if _raw_stream is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def require_current_device(device, what: str = "a tensor") -> None:
    """Raise on the host if ``device`` (a CUDA device) is not the current one.  A kernel launched
    on another device's stream with this device's pointers would fault on the GPU instead."""
    current = _current_device()
    index = device.index if device.index is not None else current
    if index != current:
        raise ValueError(f"{what} is on cuda:{index} but the current device is cuda:{current}; "
                         f"enter torch.cuda.device({index}) around the call")


def _ptr(t: "torch.Tensor | None") -> "int | None":
    return None if t is None else t.data_ptr()


def _check(t: torch.Tensor, name: str, dtype=None, dim: "int | None" = None) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (pyre_b200 has no CPU path)")
    require_current_device(t.device, name)
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise ValueError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


def _dt(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise ValueError(f"activations must be float32 or bfloat16, got {dtype}") from None


def embedding(table: torch.Tensor, ids: torch.Tensor, out: "torch.Tensor | None" = None,
              err_flag: "torch.Tensor | None" = None) -> torch.Tensor:
    """x[t] = float32(table[ids[t]]); ids int32 [T]; returns the fp32 residual stream [T, H]."""
    _check(table, "table", dim=2)
    _check(ids, "ids", torch.int32, 1)
    V, H = table.shape
    T = ids.shape[0]
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    else:
        _check(out, "out", torch.float32, 2)
    lib.call("pyre_embedding", table.data_ptr(), _dt(table.dtype), ids.data_ptr(), out.data_ptr(), T, H, V,
             _ptr(err_flag), _stream())
    return out


def add_rmsnorm(x: torch.Tensor, delta: "torch.Tensor | None", weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: "torch.Tensor | None" = None, update_x: bool = True,
                out: "torch.Tensor | None" = None, scaled_ok: bool = False) -> "torch.Tensor | ScaledRows":
    """out[r] = rmsnorm(x[src] + delta[src]) * weight with src = rows[r] (or r).

    ``x`` is the fp32 residual stream [T, H]; with ``update_x`` (and no ``rows``) the sum is
    written back to it.  ``delta`` has the activation dtype, or is a ``PartialSums`` whose
    parts the kernel adds, or a ``DeferredProduct``.  ``weight`` is fp32 [H].

    ``scaled_ok``: the caller's consumer takes ``ScaledRows``.  Then a deferred product is launched with the
    residual add and the norm's preparation as its fix-up, and no norm kernel runs at all."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    T, H = x.shape
    if weight.shape[0] != H:
        raise ValueError(f"norm weight has {weight.shape[0]} entries, rows have {H}")
    if isinstance(delta, DeferredProduct):
        if tuple(delta.shape) != (T, H):
            raise ValueError(f"delta shape {tuple(delta.shape)} != x shape {(T, H)}")
        if scaled_ok and rows is None and update_x and out is None and out_dtype == torch.bfloat16 and H % 8 == 0 \
                and H <= 128 * _MAX_FIX_TILES and folds_residual(T, H, delta.x.shape[1]):
            return gemm_residual_norm(delta, x, weight, eps)
        delta = delta.partials()
    parts, n_parts, part_stride = None, 0, 0
    if isinstance(delta, PartialSums):
        if tuple(delta.shape) != (T, H):
            raise ValueError(f"delta shape {tuple(delta.shape)} != x shape {(T, H)}")
        parts, n_parts, part_stride, delta = delta.parts, delta.n, T * H, None
    elif delta is not None:
        _check(delta, "delta", out_dtype, 2)
        if tuple(delta.shape) != (T, H):
            raise ValueError(f"delta shape {tuple(delta.shape)} != x shape {(T, H)}")
    n_rows = T
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
        update_x = False
    if out is None:
        out = torch.empty((n_rows, H), dtype=out_dtype, device=x.device)
    else:
        _check(out, "out", out_dtype, 2)
    lib.call("pyre_add_rmsnorm", x.data_ptr(), _ptr(delta), _ptr(parts), n_parts, part_stride, weight.data_ptr(),
             out.data_ptr(), _ptr(rows), n_rows, H, float(eps),
             int(bool(update_x and (delta is not None or parts is not None))), _dt(out_dtype), _stream())
    return out


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += float32(delta) in place on the fp32 residual stream: for a block arrangement in which no
    norm follows a branch (the built-in pre-norm block adds its branches inside the next norm's kernel)."""
    _check(x, "x", torch.float32)
    _check(delta, "delta")
    if x.shape != delta.shape:
        raise ValueError("x and delta differ in shape")
    lib.call("pyre_add_residual", x.data_ptr(), delta.data_ptr(), x.numel(), _dt(delta.dtype), _stream())
    return x


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor):
    """cos, sin fp32 [T, rot/2] of float(position) * inv_freq."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    T, half = positions.shape[0], inv_freq.shape[0]
    cos = torch.empty((T, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    lib.call("pyre_rope_table", positions.data_ptr(), inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, half,
             _stream())
    return cos, sin


def qkv_rope_write(qkv: torch.Tensor, bias: "torch.Tensor | None", cos: torch.Tensor, sin: torch.Tensor,
                   cache_layer: "torch.Tensor | None", slot_mapping: "torch.Tensor | None",
                   n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                   q_out: "torch.Tensor | None" = None) -> torch.Tensor:
    """Bias, rotary and the paged K/V write in one pass; returns rotated q [T, nh*hd].

    ``cache_layer``: [pages, 2, nkv, page_size, hd] of the activation dtype, or None to
    store nothing (a layer that reads another layer's cache)."""
    if isinstance(qkv, DeferredProduct):
        width = (n_heads + 2 * n_kv_heads) * head_dim
        few = qkv.shape[0] <= 128 and 128 % head_dim == 0 and head_dim % 8 == 0 and width <= 128 * _MAX_FIX_TILES
        many = qkv.shape[0] > 128 and folds_rope(qkv.shape[0], width, qkv.x.shape[1], head_dim)
        if q_out is None and qkv.shape[1] == width and rotary_dim in (0, head_dim) and (few or many):
            return gemm_rope_write(qkv, bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads, head_dim,
                                   rotary_dim, page_size)
        qkv = qkv.partials()
    parts, n_parts = None, 0
    if isinstance(qkv, PartialSums):
        parts, n_parts, act_dtype, device = qkv.parts, qkv.n, qkv.dtype, qkv.parts.device
    else:
        _check(qkv, "qkv", dim=2)
        act_dtype, device = qkv.dtype, qkv.device
    T = qkv.shape[0]
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise ValueError(f"qkv has {qkv.shape[1]} columns, expected (nh + 2 nkv) * hd = {width}")
    if head_dim % 8 or rotary_dim % 8 or not 0 <= rotary_dim <= head_dim:
        raise UnsupportedSize(f"head_dim ({head_dim}) and rotary_dim ({rotary_dim}) must be multiples of 8, "
                              f"rotary_dim <= head_dim")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != width:
            raise ValueError(f"qkv bias has {bias.shape[0]} entries, expected {width}")
    half = rotary_dim // 2
    if rotary_dim:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, half) or tuple(sin.shape) != (T, half):
            raise ValueError(f"cos/sin must be [{T}, {half}], got {tuple(cos.shape)}")
    if cache_layer is not None:
        _check(cache_layer, "cache_layer", act_dtype, 5)
        if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match "
                             f"[pages, 2, {n_kv_heads}, {page_size}, {head_dim}]")
        if slot_mapping is None:
            raise ValueError("slot_mapping is required with a cache")
        _check(slot_mapping, "slot_mapping", torch.int32, 1)
        if slot_mapping.shape[0] != T:
            raise ValueError("slot_mapping must have one entry per token")
    if q_out is None:
        q_out = torch.empty((T, n_heads * head_dim), dtype=act_dtype, device=device)
    lib.call("pyre_qkv_rope_write", None if parts is not None else qkv.data_ptr(), _ptr(parts), n_parts, T * width,
             _ptr(bias), _ptr(cos) if rotary_dim else None,
             _ptr(sin) if rotary_dim else None, q_out.data_ptr(), _ptr(cache_layer),
             _ptr(slot_mapping) if cache_layer is not None else None, T, n_heads, n_kv_heads, head_dim,
             rotary_dim, page_size, _dt(act_dtype), cache_layer.shape[0] if cache_layer is not None else 0,
             device_error_flag(device).data_ptr(), _stream())
    return q_out


def silu_mul(gate_up: torch.Tensor, out: "torch.Tensor | None" = None, block: int = 0) -> torch.Tensor:
    """out[t, i] = silu(gate[t, i]) * up[t, i].  ``block == 0``: gate_up = [all gates | all ups];
    ``block == n``: gates and ups alternate in blocks of n features (n gates, their n ups, ...)."""
    _check(gate_up, "gate_up", dim=2)
    T, two_i = gate_up.shape
    if two_i % 2:
        raise ValueError("gate_up must have an even number of columns")
    inter = two_i // 2
    if block and (block % 8 or inter % block):
        raise UnsupportedSize(f"silu_mul: blocks of {block} features do not tile {inter} features in steps of 8")
    if out is None:
        out = torch.empty((T, inter), dtype=gate_up.dtype, device=gate_up.device)
    lib.call("pyre_silu_mul", gate_up.data_ptr(), out.data_ptr(), T, inter, int(block), _dt(gate_up.dtype), _stream())
    return out


def feed_tokens(token_ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """token_ids[dst[i]] = prev[src[i]] where dst[i] >= 0 (all int32, on the device): tokens sampled by
    the last step enter the next one without a trip through the host."""
    for t, name in ((token_ids, "token_ids"), (dst, "dst"), (src, "src"), (prev, "prev")):
        _check(t, name, torch.int32, 1)
    if dst.shape[0] != src.shape[0]:
        raise ValueError("dst and src must have one entry each per fed token")
    lib.call("pyre_feed_tokens", token_ids.data_ptr(), dst.data_ptr(), src.data_ptr(), prev.data_ptr(), dst.shape[0], _stream())


def delay(milliseconds: float) -> None:
    """Queue a kernel that idles for ``milliseconds`` (at most 1,000) on the current stream: a measured region
    queued behind it is in the stream in full before the GPU starts on it."""
    lib.call("pyre_delay", int(milliseconds * 1e6), _stream())


def sample(logits: torch.Tensor, temperature: "torch.Tensor | None" = None, seeds: "torch.Tensor | None" = None,
           token_index: "torch.Tensor | None" = None, out: "torch.Tensor | None" = None) -> torch.Tensor:
    """One token id per row of fp32 logits [R, V]: argmax where temperature is 0, else Gumbel-max."""
    if logits.dim() != 2 or logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise ValueError("logits must be a CUDA float32 matrix with contiguous rows")
    R, V = logits.shape
    if temperature is not None:
        _check(temperature, "temperature", torch.float32, 1)
        if seeds is None or token_index is None:
            raise ValueError("temperature sampling needs seeds and token_index")
        _check(seeds, "seeds", torch.int64, 1)
        _check(token_index, "token_index", torch.int32, 1)
        if not (temperature.shape[0] == seeds.shape[0] == token_index.shape[0] == R):
            raise ValueError("temperature, seeds and token_index need one entry per row")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    slices = lib.call_value("pyre_sample_slices", V)
    scratch = torch.empty(R * slices * 2, dtype=torch.int32, device=logits.device) if slices else None
    lib.call("pyre_sample", logits.data_ptr(), logits.stride(0), _ptr(temperature), _ptr(seeds), _ptr(token_index),
             out.data_ptr(), R, V, _ptr(scratch), _stream())
    return out


def paged_attention_generic(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor, n_heads: int, n_kv_heads: int,
                            head_dim: int, scale: float, window: "int | None" = None,
                            out: "torch.Tensor | None" = None, sink: "float | None" = None) -> torch.Tensor:
    """Exact fp32-arithmetic attention of every query token over its sequence's pages.  ``sink``: the score of a
    sink that has no value: exp(sink) joins every softmax denominator (None: no sink; a float32 tensor [n_heads]: a
    score per query head)."""
    _check(q, "q", dim=2)
    _check(cache_layer, "cache_layer", q.dtype, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T = q.shape[0]
    if q.shape[1] != n_heads * head_dim:
        raise ValueError(f"q has {q.shape[1]} columns, expected nh * hd = {n_heads * head_dim}")
    if head_dim % 16 or head_dim > 256:
        raise UnsupportedSize(f"head_dim {head_dim}: the attention kernels take multiples of 16 up to 256")
    if n_heads % n_kv_heads:
        raise UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
        raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match the head sizes")
    if out is None:
        out = torch.empty_like(q)
    lib.call("pyre_paged_attention_generic", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(), T,
             n_heads, n_kv_heads, head_dim, page_size, int(window or 0), float(scale), _sink_args(sink, n_heads)[0], _sink_args(sink, n_heads)[1], _dt(q.dtype), cache_layer.shape[0],
             device_error_flag(q.device).data_ptr(), _stream())
    return out


def _sink(sink: "float | None") -> float:
    """The kernels' encoding of 'no sink': a score of minus infinity, whose term in the denominator is zero."""
    return float("-inf") if sink is None else float(sink)


def _sink_args(sink, n_heads: int) -> tuple:
    """(one score for all heads, pointer to a score per query head or None) as the attention kernels take them:
    ``sink`` is None, a number, or a float32 tensor [n_heads] on the device."""
    if isinstance(sink, torch.Tensor):
        _check(sink, "sink", torch.float32, 1)
        if sink.shape[0] != n_heads:
            raise ValueError(f"{sink.shape[0]} sink scores for {n_heads} query heads")
        return float("-inf"), sink.data_ptr()
    return _sink(sink), None


MMA_MAX_HEAD_DIM = 128
CLUSTER_MAX_SPLITS = 16      # splits of one group merge through a thread-block cluster up to this many
MAX_SCRATCH_SPLITS = 64      # beyond a cluster: partial results through scratch memory and the combining kernel
_DEFAULT_SM_COUNT = 148     # a B200; used only where no device can be asked (planning on a host without a GPU)
_sm_counts: dict = {}
_have_cuda: "bool | None" = None


def sm_count(device=None) -> int:
    """Multiprocessors of ``device`` (default: the current one), as the launch code asks the device
    too; the planners below size splits and rounds of tiles by it."""
    global _have_cuda
    if _have_cuda is None:
        _have_cuda = torch.cuda.is_available()
    if not _have_cuda:
        return _DEFAULT_SM_COUNT
    index = _current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count) or _DEFAULT_SM_COUNT
    return n


def attention_splits(n_tokens: int, n_seqs: int, n_heads: int, n_kv_heads: int, max_context: int,
                     window: "int | None", n_groups: "int | None" = None) -> int:
    """How many ways the tensor-core kernel splits each sequence's keys: enough CTAs for
    about one and a half per SM, at least two 16-key tiles per split, at most 16 (the
    splits of a group form one thread-block cluster), or 24 to 64 through scratch memory for
    one or two sequences with long contexts."""
    _SM_COUNT = sm_count()
    n_rep = n_heads // n_kv_heads
    hpg = min(n_rep, 16)
    tpg = 16 // hpg
    if n_groups is None:     # one token per entry (decode) when the counts agree, else an upper bound
        n_groups = n_seqs if n_tokens == n_seqs else n_tokens // tpg + n_seqs
    ctas = n_groups * n_kv_heads * (-(-n_rep // hpg))
    span = max_context if not window else min(max_context, window + tpg)
    tiles = -(-span // 16) + 1
    # Measured inside whole decode steps (7B shape, contexts of 2-3 thousand tokens): about one and a half CTAs per
    # SM in all is best (batch 8: 7 splits, 16: 4, 32: 2, 64: 1); with two per SM the product that follows
    # finds no SM on which to prefetch its weights while the attention runs.
    # One or two sequences with long contexts: a cluster's 16 CTAs per group leave most SMs idle and give every warp
    # dozens of tiles (0.6 us of dependent work each).  Many small CTAs (about 256 in all, at least 16 tiles each)
    # through scratch memory and the combining kernel win there: alone, 8,192 keys 10.9 -> 8.9 us, 16,384 keys
    # 16.9 -> 12.3, 32,768 keys 25.7 -> 17.0 (one sequence); 34.0 -> 25.9 for two sequences of 32,768.
    # Four sequences of 32,768 keys: 16 splits through scratch 47.4 us, 32: 49.3, clusters of 8 or 16: 62-68.
    many = min(256 // max(ctas, 1), tiles // 16, MAX_SCRATCH_SPLITS)
    if many >= 24 or (many >= 16 and tiles >= 512):
        return max(24, many // 8 * 8)
    want = max(1, min(int(1.57 * _SM_COUNT / max(ctas, 1) + 0.5), -(-tiles // 2), CLUSTER_MAX_SPLITS))
    if want > 8:
        # a cluster of 16 CTAs must sit in one GPC: it pays only while all of them fit on the chip at once
        if ctas * 16 > _SM_COUNT:
            return min(want, 10)
        # one or two sequences with tens of thousands of keys: 16 CTAs per group leave most SMs idle; 32 splits
        # through scratch memory and the combining kernel win from about 24 thousand keys on
        if ctas * 32 <= _SM_COUNT and tiles >= 1536:
            return 32
        return 16
    return int(want)


def paged_attention_mma(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor,
                        cu_seqlens: torch.Tensor, positions: torch.Tensor, n_seqs: int, n_heads: int,
                        n_kv_heads: int, head_dim: int, scale: float, window: "int | None" = None,
                        n_splits: int = 1, out: "torch.Tensor | None" = None,
                        scratch: "torch.Tensor | None" = None, max_len: int = 0, uniform_len: int = 0,
                        sink: "float | None" = None) -> torch.Tensor:
    """bfloat16 attention on the tensor cores over the block table (decode tokens and
    prompt portions alike); ``n_splits`` > 1 splits each sequence's keys over CTAs and needs
    ``T * nh * n_splits * (hd + 2)`` floats of scratch (allocated here if not given)."""
    _check(q, "q", torch.bfloat16, 2)
    _check(cache_layer, "cache_layer", torch.bfloat16, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T = q.shape[0]
    if q.shape[1] != n_heads * head_dim:
        raise ValueError(f"q has {q.shape[1]} columns, expected nh * hd = {n_heads * head_dim}")
    if head_dim % 16 or not 16 <= head_dim <= MMA_MAX_HEAD_DIM:
        raise UnsupportedSize(f"head_dim {head_dim}: the tensor-core attention takes multiples of 16 up to {MMA_MAX_HEAD_DIM}")
    if n_heads % n_kv_heads:
        raise UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
        raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match the head sizes")
    if cu_seqlens.shape[0] != n_seqs + 1 or positions.shape[0] != T or block_table.shape[0] < n_seqs:
        raise ValueError("cu_seqlens, positions and block_table do not match the batch")
    if out is None:
        out = torch.empty_like(q)
    n_splits = int(n_splits)
    if n_splits > 1 and not (scratch is None and n_splits <= CLUSTER_MAX_SPLITS):
        need = T * n_heads * n_splits * (head_dim + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        elif scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_contiguous():
            raise ValueError(f"scratch must be {need} contiguous floats")
    lib.call("pyre_paged_attention_mma", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), _ptr(scratch),
             block_table.data_ptr(), block_table.stride(0), cu_seqlens.data_ptr(), positions.data_ptr(), T, n_seqs,
             n_heads, n_kv_heads, head_dim, page_size, int(window or 0), float(scale), _sink_args(sink, n_heads)[0], _sink_args(sink, n_heads)[1], n_splits, int(max_len),
             cache_layer.shape[0], int(uniform_len), device_error_flag(q.device).data_ptr(), _stream())
    return out


PREFILL_HEAD_DIMS = (64, 128)
PREFILL_MIN_LEN = 32     # entries with at least this many tokens go to the prompt-portion kernel


def attention_prefill(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                      positions: torch.Tensor, n_seqs: int, n_long_tokens: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, scale: float, window: "int | None", out: torch.Tensor,
                      min_len: int = PREFILL_MIN_LEN, sink: "float | None" = None) -> torch.Tensor:
    """bfloat16 attention of the entries with at least ``min_len`` tokens (64 queries of a head
    per CTA, keys and values tiled through shared memory); writes only those entries' rows of ``out``."""
    _check(q, "q", torch.bfloat16, 2)
    _check(cache_layer, "cache_layer", torch.bfloat16, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    _check(out, "out", torch.bfloat16, 2)
    if head_dim not in PREFILL_HEAD_DIMS:
        raise UnsupportedSize(f"head_dim {head_dim}: the prompt-portion attention kernel takes {PREFILL_HEAD_DIMS}")
    if n_heads % n_kv_heads:
        raise UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim) or q.shape[1] != n_heads * head_dim:
        raise ValueError("q or the cache layer do not match the head sizes")
    if out.shape != q.shape or cu_seqlens.shape[0] != n_seqs + 1 or positions.shape[0] != q.shape[0]:
        raise ValueError("out, cu_seqlens and positions do not match the batch")
    lib.call("pyre_attention_prefill", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), cu_seqlens.data_ptr(), positions.data_ptr(), int(n_long_tokens), n_seqs, n_heads,
             n_kv_heads, head_dim, page_size, int(window or 0), float(scale), _sink_args(sink, n_heads)[0], _sink_args(sink, n_heads)[1], int(min_len), cache_layer.shape[0],
             device_error_flag(q.device).data_ptr(), _stream())
    return out


USE_TC_ATTENTION = True
TC_ATTENTION_MIN_LEN = 64    # entries with at least this many tokens go to the tcgen05 kernel (128-query tiles)


MAX_KEY_SPLITS = 8
KEY_SPLIT_SCRATCH_BYTES = 128 << 20      # of partial outputs per launch (fewer items than SMs keep it below this anyway)


def prefill_key_splits(n_items: int, mean_tiles: float, n_tokens: int, n_heads: int, head_dim: int) -> int:
    """Into how many shares of the keys the prompt attention cuts every (128-query tile, head).  Shares pay only
    while SMs would stand idle: an SM runs the tiles of one CTA alone as fast as those of two together, so what
    counts is that every SM has a CTA, and a share costs its partial output's trip through memory and a second
    kernel (measured: 2,048 tokens after 8,192, 448 items, 292 us whole, 350 in two shares; 512 tokens after 30,720,
    112 items, 492 us whole, 294 in two shares, 269 in five).  So: only with fewer items than SMs, as many shares as
    fill two CTAs per SM, each of at least 16 key tiles (1,024 keys); or as many as fill them twice over, if every
    share then still has 80 key tiles (two rounds of 97 tiles beat one round of 242; two rounds of 65 lose to one of
    131: 640 tokens after 16,384, 191 us in four shares against 186 in two)."""
    sms = sm_count()
    if n_items >= sms:
        return 1
    s = min(MAX_KEY_SPLITS, 2 * sms // max(n_items, 1), int(mean_tiles // 16))
    twice = min(MAX_KEY_SPLITS, 4 * sms // max(n_items, 1))
    if twice > s and mean_tiles / twice >= 80:
        s = twice
    while s > 1 and n_tokens * n_heads * s * head_dim * 4 > KEY_SPLIT_SCRATCH_BYTES:
        s -= 1
    return max(1, s)


def attention_prefill_tc(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                         positions: torch.Tensor, n_seqs: int, n_long_tokens: int, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: "int | None", out: torch.Tensor, min_len: int,
                         key_splits: int = 1, sink: "float | None" = None) -> torch.Tensor:
    """bfloat16 attention of the entries with at least ``min_len`` tokens on the tcgen05 tensor
    cores (scores and output in tensor memory, Q/K/V tiles by TMA); writes only those entries' rows.
    ``key_splits`` > 1: that many CTAs share the keys of every (query tile, head); a second kernel combines them."""
    _check(q, "q", torch.bfloat16, 2)
    _check(cache_layer, "cache_layer", torch.bfloat16, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    _check(out, "out", torch.bfloat16, 2)
    page_size = cache_layer.shape[3]
    if head_dim not in PREFILL_HEAD_DIMS or page_size & (page_size - 1) or page_size < 4:
        raise UnsupportedSize(f"the tcgen05 attention takes head sizes {PREFILL_HEAD_DIMS} and power-of-two pages")
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim) or q.shape[1] != n_heads * head_dim:
        raise ValueError("q or the cache layer do not match the head sizes")
    if out.shape != q.shape or cu_seqlens.shape[0] != n_seqs + 1 or positions.shape[0] != q.shape[0]:
        raise ValueError("out, cu_seqlens and positions do not match the batch")
    key_splits = int(key_splits)
    if not 1 <= key_splits <= 32:
        raise ValueError(f"key_splits must be 1 to 32, got {key_splits}")
    part_o = part_ml = None
    if key_splits > 1:
        part_o = torch.empty((q.shape[0], n_heads, key_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((q.shape[0], n_heads, key_splits, 2), dtype=torch.float32, device=q.device)
    lib.call("pyre_attention_prefill_tc", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), cu_seqlens.data_ptr(), positions.data_ptr(), q.shape[0], int(n_long_tokens), n_seqs,
             n_heads, n_kv_heads, head_dim, page_size, cache_layer.shape[0], int(window or 0), float(scale), _sink_args(sink, n_heads)[0], _sink_args(sink, n_heads)[1], int(min_len),
             key_splits, _ptr(part_o), _ptr(part_ml), device_error_flag(q.device).data_ptr(), _stream())
    return out


def paged_attention_bf16(ctx, q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, n_heads: int,
                         n_kv_heads: int, head_dim: int, scale: float, window: "int | None",
                         sink: "float | None" = None) -> torch.Tensor:
    """Attention of a whole step in bfloat16: entries with many tokens go to the
    prompt-portion kernel, the others (decoded tokens, short portions) to the split-KV kernel."""
    lens = ctx.cu_seqlens_host[1:] - ctx.cu_seqlens_host[:-1]
    page_size = cache_layer.shape[3]
    use_tc = USE_TC_ATTENTION and head_dim in PREFILL_HEAD_DIMS and page_size & (page_size - 1) == 0 and page_size >= 4
    min_len = TC_ATTENTION_MIN_LEN if use_tc else PREFILL_MIN_LEN
    long_mask = lens >= min_len if head_dim in PREFILL_HEAD_DIMS else lens < 0
    n_long = int(lens[long_mask].sum())
    n_short_seqs = int((~long_mask).sum())
    out = torch.empty_like(q)
    if n_long and use_tc:
        long_lens, long_starts = lens[long_mask], ctx.start_pos_host[long_mask]
        q_tiles = -(-long_lens // 128)
        # key tiles of 64 that a query tile walks, averaged over the tiles: from position 0 (or the window's start)
        # to the tile's last row
        keys = long_starts + long_lens / 2.0 + 64.0
        if window:
            keys = keys.clip(max=window + 192.0)
        mean_tiles = float((keys / 64.0 * q_tiles).sum() / q_tiles.sum())
        key_splits = prefill_key_splits(int(q_tiles.sum()) * n_heads, mean_tiles, q.shape[0], n_heads, head_dim)
        attention_prefill_tc(q, cache_layer, block_table, ctx.cu_seqlens, ctx.positions, ctx.num_seqs, n_long, n_heads,
                             n_kv_heads, head_dim, scale, window, out, min_len, key_splits, sink=sink)
    elif n_long:
        attention_prefill(q, cache_layer, block_table, ctx.cu_seqlens, ctx.positions, ctx.num_seqs, n_long, n_heads,
                          n_kv_heads, head_dim, scale, window, out, sink=sink)
    if n_short_seqs:
        n_short = ctx.num_tokens - n_long
        short_ctx = int((ctx.start_pos_host + lens)[~long_mask].max())
        tpg = max(1, 16 // min(n_heads // n_kv_heads, 16))
        groups = int((-(-lens[~long_mask] // tpg)).sum())
        splits = attention_splits(n_short, n_short_seqs, n_heads, n_kv_heads, short_ctx, window, groups)
        uniform = int(lens[0]) if not n_long and bool((lens == lens[0]).all()) else 0
        paged_attention_mma(q, cache_layer, block_table, ctx.cu_seqlens, ctx.positions, ctx.num_seqs, n_heads,
                            n_kv_heads, head_dim, scale, window, splits, out=out,
                            max_len=min_len - 1 if n_long else 0, uniform_len=uniform, sink=sink)
    return out


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, bias: "torch.Tensor | None" = None,
             out: "torch.Tensor | None" = None) -> torch.Tensor:
    """C = A W^T (+ bias) in IEEE fp32 on the CUDA cores; a [M, K], w [N, K]."""
    for t, n in ((a, "a"), (w, "w")):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{n} must be a CUDA float32 matrix with contiguous rows")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise ValueError(f"inner sizes differ: a is [{M}, {K}], w is [{N}, {K2}]")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    lib.call("pyre_sgemm_nt", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
             _ptr(bias), M, N, K, _stream())
    return out


_error_flags: dict = {}


def device_error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels raise when a bounded wait runs out or an index is out of range."""
    key = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    flag = _error_flags.get(key)
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=device)
        _error_flags[key] = flag
    return flag


DEVICE_ERROR_MESSAGES = {
    1: "a kernel met an index outside its range (token id outside the vocabulary)",
    2: "a tensor-core GEMM gave up waiting on its pipeline (bounded wait ran out)",
    3: "the attention kernel gave up waiting for a tile copy (bounded wait ran out)",
    4: "the tcgen05 attention kernel gave up waiting on its pipeline (bounded wait ran out)",
    5: "the tcgen05 attention kernel found its shared memory misaligned",
    6: "a kernel met a cache page or slot outside the pool (debug checks): a block table or slot mapping names "
       "a page that was given back or never existed",
}


def device_error_message(code: int) -> str:
    """What a value of the device's error word means."""
    return DEVICE_ERROR_MESSAGES.get(int(code), f"a kernel raised error code {int(code)}")


def check_device_errors(device="cuda") -> None:
    flag = device_error_flag(device)
    code = int(flag.item())
    if code:
        flag.zero_()
        counters = _fix_counters.get(torch.device(device).index or 0)
        if counters is not None:
            counters.zero_()      # a product that gave up may have left arrivals uncounted
        raise lib.KernelError(device_error_message(code))


def tc_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The TMA-fed tcgen05 kernel takes bf16 operands whose rows are 16-byte multiples and 16-byte aligned."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


CTA_PAIRS = True     # prompt portions: two CTAs of a cluster share each 256-row tile (tcgen05 cta_group::2)


def tc_gemm_plan(M: int, N: int, K: int) -> tuple[bool, int, int]:
    """(weights_as_rows, bn, splits) for y[M, N] = a[M, K] w[N, K]^T.

    Up to 128 tokens the weights take the 128-row side of the MMA and the tokens the
    narrow side (bn = tokens rounded up to 16/32/64/128); K is split so that about one
    CTA lands on every SM, each split keeping at least four 64-wide K blocks.  Beyond
    that the tokens take the rows and 128 to 256 output features form a tile, whichever
    width fills the rounds of the persistent CTAs best."""
    _SM_COUNT = sm_count()
    kb = -(-K // 64)
    if M <= 128 or N % 8:
        bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
        tiles = -(-N // 128) * -(-M // bn)
        splits = max(1, min(_SM_COUNT // tiles if tiles < _SM_COUNT else 1, kb // 4, 16))
        # 33 to 128 tokens and few tiles (a split K): one 128-row tile of tokens against 128 weight rows per CTA, the
        # same tiles and splits with the operands' roles exchanged, is faster: the narrow operand then costs 16 KB per K
        # block whatever the token count.  Timed alone at 128 tokens (28 weight matrices in turn): down 34.4 -> 30.4 us,
        # q/k/v 16.6 -> 12.2, output 15.3 -> 11.3; the decode step of 128 requests 7.03 -> 6.66 ms.  From 33 tokens it
        # pays inside the step too since the fp32 partial sums leave the epilogue in whole lines (64 requests 4.71 ->
        # 4.67 ms, 40 requests 4.22 -> 4.19); up to 32 tokens the weights stay on the rows (16 requests: 3.51 against 3.61).
        if 32 < M <= 128 and N % 8 == 0 and splits > 1:
            return False, 128, splits
        return True, bn, splits
    # The tile width and the split of K with the least estimated time on the persistent CTAs (microseconds).
    # Measured on products of 256-2,048 tokens: the main loop is bound by loads, not by the MMAs.  One SM pulls
    # what its ring holds in flight (all stages but the one being multiplied) per memory latency, 1.1 us when
    # many row tiles share each weight tile in L2 and 1.6 us when few do; all SMs together pull about 18 TB/s
    # from L2 into shared memory.  Wide tiles move the fewest bytes, narrow ones fill the CTAs' rounds better,
    # and a split K fills the SMs when there are few tiles (512 tokens x 3,584 features over K = 18,944:
    # 224 wide with K in two takes 63 us, 112 tiles of 128 take 88 us).
    # With CTA pairs (two CTAs of a cluster on a 256-row tile, each loading half of the tile's weight rows) an SM
    # loads 128 (128 + bn / 2) bytes per K block, its ring is deeper, and the workers are the 74 pairs.
    pair = CTA_PAIRS
    workers = _SM_COUNT // 2 if pair else _SM_COUNT
    rows = -(-M // (256 if pair else 128))
    latency = 1.7 - 0.035 * min(-(-M // 128), 16)
    widths = ((256, 6), (224, 6), (208, 7), (192, 7), (160, 7), (128, 8)) if pair else \
        ((256, 4), (224, 5), (208, 5), (192, 5), (160, 5), (128, 6))
    best = [None, None]      # without and with a split K
    for cand, stages in widths:
        if cand > 128 and N < cand:
            continue
        cols = -(-N // cand)
        nbytes = ((256 + cand) if pair else (128 + cand)) * 128       # one K block of both operands, per worker
        per_block = max(cand * 2 / 1900.0, latency / (stages - 1))
        for sp in (1, 2, 3, 4):
            if sp > 1 and kb // sp < 8:
                break
            items = rows * cols * sp
            per_worker = -(-items // workers)
            blocks = -(-kb // sp)
            cost = max(per_worker * blocks * per_block, items * blocks * nbytes / 18e6) \
                + per_worker * (1.5 + cand / 64.0 * (2 if sp > 1 else 1))
            # near-ties go to the wider tile; a split K (fp32 partials, estimated less surely) has to gain a tenth
            if best[sp > 1] is None or cost < best[sp > 1][0] * 0.98:
                best[sp > 1] = (cost, cand, sp)
    whole, split = best
    if split is not None and split[0] < 0.9 * whole[0]:
        return False, split[1], split[2]
    return False, whole[1], whole[2]


GATED_BLOCK = 64     # gate and up rows of a fused feed-forward weight alternate in blocks of this many features


_MAX_FIX_TILES = 4096       # arrival counters per device: tiles of 128 features of one folded product
_fix_counters: dict = {}


def _tile_counters(device) -> torch.Tensor:
    """Arrival counters of the products with a fix-up (zero between launches: the kernel resets what it counts)."""
    key = torch.device(device).index or 0
    c = _fix_counters.get(key)
    if c is None:
        c = _fix_counters[key] = torch.zeros(_MAX_FIX_TILES, dtype=torch.int32, device=device)
    return c


def _scale_fields(fx: "lib.GemmFix", x: "ScaledRows") -> None:
    fx.scale_ssq, fx.scale_tiles = x.ssq.data_ptr(), x.ssq.shape[0]
    fx.scale_n, fx.scale_eps = float(x.rows.shape[1]), x.eps


def gemm_tc(x: "torch.Tensor | ScaledRows", w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
            plan: "tuple[bool, int, int] | None" = None, reduce: bool = True, gated: bool = False,
            pair: "bool | None" = None, checked: bool = False) -> torch.Tensor:
    """y = x w^T on the tensor cores (tcgen05, TMEM accumulators, TMA-fed), bf16 in, fp32 accumulate.

    With a split K the kernel leaves fp32 partial sums [splits, M, N]; ``reduce`` adds
    them up here (fixed order) and converts to ``out_dtype``.  ``reduce=False`` returns them
    as ``PartialSums`` for a consumer kernel that adds them itself.

    ``gated``: w holds gate and up rows alternating in blocks of ``GATED_BLOCK`` features; the
    result is silu(x gate^T) * (x up^T), [M, N / 2] bf16.  The activation runs in the product's
    epilogue (whole tiles, one split: the usual case in both orientations), otherwise after it.

    ``x`` may be ``ScaledRows``: the result rows are scaled by the tokens' 1/rms in the epilogue, before the
    activation of a gated product."""
    scaled = x if isinstance(x, ScaledRows) else None
    if scaled is not None:
        x = scaled.rows
    if not checked and not tc_gemm_supported(x, w):      # ``checked``: the caller has asked already
        raise UnsupportedSize("gemm_tc needs bf16 operands with K and leading dimensions that are multiples of 8")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise ValueError(f"inner sizes differ: x is [{M}, {K}], w is [{N}, {K2}]")
    weights_as_rows, bn, splits = plan or tc_gemm_plan(M, N, K)
    if gated and plan is None and M == 128 and N % 256 == 0:
        # exactly 128 tokens: 58.6 us with the weights on the rows, 52.4 so; with 72-120 tokens (a tile of token rows
        # that is not full) this orientation takes 66 us and the other 54-58
        weights_as_rows, bn, splits = False, 256, 1
    if scaled is not None and weights_as_rows and (M > bn or bn > 128):      # more than one tile of at most 128 tokens on the narrow side: not served
        x, scaled = materialize(scaled), None
    splits = max(1, min(splits, -(-K // 64)))
    if pair is None:
        pair = CTA_PAIRS
    pair = int(bool(pair) and not weights_as_rows and M > 128 and bn in (128, 160, 192, 208, 224, 256))
    err = device_error_flag(x.device)
    fx = None
    if scaled is not None:
        fold = lib.GemmFix()
        _scale_fields(fold, scaled)
        fx = ctypes.byref(fold)

    if gated:
        if N % (2 * GATED_BLOCK) or out_dtype != torch.bfloat16:
            raise UnsupportedSize("a gated product needs whole blocks of gate and up rows and a bfloat16 result")
        if not weights_as_rows and plan is None and N % 256 == 0:
            bn, splits = 256, 1      # the fused activation needs whole 256-wide tiles and saves more than a better fit
        if not weights_as_rows and bn == 256 and splits == 1 and N % 256 == 0:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
            lib.call("pyre_gemm_tc", x.data_ptr(), M, x.stride(0), w.data_ptr(), N, w.stride(0), K, out.data_ptr(), 0,
                     N // 2, 1, 0, 1, bn, 0, 1, pair, err.data_ptr(), fx, _stream())
            return out
        if weights_as_rows and bn <= 128 and splits == 1 and N % 128 == 0:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
            lib.call("pyre_gemm_tc", w.data_ptr(), N, w.stride(0), x.data_ptr(), M, x.stride(0), K, out.data_ptr(), 0,
                     1, N // 2, 0, 1, bn, 1, 1, 0, err.data_ptr(), fx, _stream())
            return out
        return silu_mul(gemm_tc(scaled if scaled is not None else x, w, torch.bfloat16, (weights_as_rows, bn, splits), pair=bool(pair)),
                        block=GATED_BLOCK)
    if splits == 1 and reduce:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        target, split_stride = out, 0
    else:
        target = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        split_stride = M * N
    f32 = int(target.dtype == torch.float32)
    if weights_as_rows:
        lib.call("pyre_gemm_tc", w.data_ptr(), N, w.stride(0), x.data_ptr(), M, x.stride(0), K, target.data_ptr(), f32,
                 1, N, split_stride, splits, bn, 1, 0, 0, err.data_ptr(), fx, _stream())
    else:
        lib.call("pyre_gemm_tc", x.data_ptr(), M, x.stride(0), w.data_ptr(), N, w.stride(0), K, target.data_ptr(), f32,
                 N, 1, split_stride, splits, bn, 0, 0, pair, err.data_ptr(), fx, _stream())
    if target.dim() == 2:
        return target
    if not reduce:
        return PartialSums(target, out_dtype)
    return materialize(PartialSums(target, out_dtype))


def _launch_with_fixup(prod: DeferredProduct, fx: "lib.GemmFix", rows_out: "torch.Tensor | None" = None,
                       row_plan: "tuple[bool, int, int] | None" = None) -> None:
    """The product of a ``DeferredProduct`` with work folded in.  Few tokens (weights on the MMA's rows, all tokens
    in one tile, K split as the plan says): fp32 partial sums that only the kernel's own fix-up reads.  Many tokens
    (tokens on the rows, one split): the epilogue itself folds, and what it stores is ``rows_out``."""
    x = prod.x
    if isinstance(x, ScaledRows):
        _scale_fields(fx, x)
        x = x.rows
    w = prod.w
    M, K = x.shape
    N = w.shape[0]
    weights_as_rows, bn, splits = row_plan or tc_gemm_plan(M, N, K)
    if M <= 128 and not weights_as_rows:
        # the fix-up lives in the orientation with the weights on the rows; the same tiles and splits serve it
        weights_as_rows, bn = True, 128
    err = device_error_flag(x.device).data_ptr()
    with lib.section(prod.section):
        if weights_as_rows:
            splits = max(1, min(splits, -(-K // 64)))
            parts = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
            fx.tile_counters = _tile_counters(x.device).data_ptr()
            lib.call("pyre_gemm_tc", w.data_ptr(), N, w.stride(0), x.data_ptr(), M, x.stride(0), K, parts.data_ptr(), 1,
                     1, N, M * N, splits, bn, 1, 0, 0, err, ctypes.byref(fx), _stream())
        else:
            if splits != 1 or rows_out is None:
                raise UnsupportedSize("a product of many tokens folds only with one split and the residual fix-up")
            pair = int(CTA_PAIRS and bn in (128, 160, 192, 208, 224, 256))
            lib.call("pyre_gemm_tc", x.data_ptr(), M, x.stride(0), w.data_ptr(), N, w.stride(0), K, rows_out.data_ptr(), 0,
                     N, 1, 0, 1, bn, 0, 0, pair, err, ctypes.byref(fx), _stream())


def folds_residual(M: int, N: int, K: int) -> bool:
    """Does a product of this shape take the residual add and the next norm's preparation as folded work?  Very few
    tokens (the fix-up of the last CTA per tile), or many tokens in one split (the epilogue's threads own token rows)."""
    if not FOLD_SMALL_KERNELS or N % 8:
        return False
    if M <= FOLD_MAX_TOKENS:
        return True
    if M <= 128:
        return False
    weights_as_rows, _bn, splits = tc_gemm_plan(M, N, K)
    return not weights_as_rows and splits == 1


def rope_fold_width(N: int, head_dim: int) -> int:
    """The tile width with which a q/k/v product of many tokens carries bias, rotary and the cache write in its
    epilogue (tiles of whole heads), or 0."""
    for bn in (256, 128):
        if N % bn == 0 and bn % head_dim == 0 and head_dim % 32 == 0:
            return bn
    return 0


def folds_rope(M: int, N: int, K: int, head_dim: int) -> bool:
    """Does the stacked q/k/v product of this shape take bias, rotary and the paged write as folded work?  Very few
    tokens (the fix-up of the last CTA per tile), or a prompt portion whose plan is one split of the row store."""
    if not FOLD_SMALL_KERNELS or N % 8:
        return False
    if M <= FOLD_MAX_TOKENS:
        return True
    if M <= 128 or not rope_fold_width(N, head_dim):
        return False
    weights_as_rows, _bn, splits = tc_gemm_plan(M, N, K)
    return not weights_as_rows and splits == 1


def gemm_residual_norm(prod: DeferredProduct, x: torch.Tensor, weight: torch.Tensor, eps: float) -> ScaledRows:
    """x += prod (the fp32 residual stream, in place), and the activations of the RMSNorm that follows as
    ``ScaledRows``: one kernel, the product; the CTA that finishes a tile of 128 features last adds the splits'
    partial sums and the residual, stores bf16(x * weight) and the tile's sums of squares per token."""
    T, H = x.shape
    rows = torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
    ssq = torch.empty((-(-H // 128), T), dtype=torch.float32, device=x.device)
    fx = lib.GemmFix()
    fx.fix = 1
    fx.resid, fx.norm_w, fx.h_out, fx.ssq_out = x.data_ptr(), weight.data_ptr(), rows.data_ptr(), ssq.data_ptr()
    if T > 128:
        # tokens on the rows: a tile is up to 256 features wide, so the sums of squares come per such tile
        _rows, bn, _splits = tc_gemm_plan(T, H, prod.x.shape[1])
        ssq = torch.empty((-(-H // bn), T), dtype=torch.float32, device=x.device)
        fx.ssq_out = ssq.data_ptr()
    _launch_with_fixup(prod, fx, rows)
    return ScaledRows(rows, ssq, eps)


def gemm_rope_write(prod: DeferredProduct, bias, cos, sin, cache_layer, slot_mapping, n_heads: int, n_kv_heads: int,
                    head_dim: int, rotary_dim: int, page_size: int) -> torch.Tensor:
    """The stacked q/k/v projection with bias, rotary and the paged K/V write as its fix-up (what
    ``qkv_rope_write`` does in a kernel of its own); returns the queries [T, nh * hd]."""
    T = prod.shape[0]
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    if rotary_dim:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, rotary_dim // 2) or tuple(sin.shape) != (T, rotary_dim // 2):
            raise ValueError(f"cos/sin must be [{T}, {rotary_dim // 2}], got {tuple(cos.shape)}")
    q_out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=prod.device)
    fx = lib.GemmFix()
    fx.fix = 2
    fx.bias = _ptr(bias)
    fx.cos_t, fx.sin_t = (_ptr(cos), _ptr(sin)) if rotary_dim else (None, None)
    fx.q_out = q_out.data_ptr()
    fx.nh, fx.nkv, fx.hd, fx.rot, fx.page_size = n_heads, n_kv_heads, head_dim, rotary_dim, page_size
    if cache_layer is not None:
        _check(cache_layer, "cache_layer", torch.bfloat16, 5)
        if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match "
                             f"[pages, 2, {n_kv_heads}, {page_size}, {head_dim}]")
        _check(slot_mapping, "slot_mapping", torch.int32, 1)
        if slot_mapping.shape[0] != T:
            raise ValueError("slot_mapping must have one entry per token")
        fx.kv_cache, fx.slot_mapping, fx.n_pages = cache_layer.data_ptr(), slot_mapping.data_ptr(), cache_layer.shape[0]
    if T > 128:
        # tokens on the rows: the epilogue thread that owns a token row rotates and stores whole heads
        _launch_with_fixup(prod, fx, q_out, (False, rope_fold_width(prod.shape[1], head_dim), 1))
    else:
        _launch_with_fixup(prod, fx)
    return q_out


USE_TC_GEMM = True


# Very few tokens (a decode step of one to four requests): residual add + norm and bias + rotary + K/V write run as
# fix-ups of the products before them instead of kernels of their own.  Measured inside whole decode steps of the 7B
# shape: 4 % faster at one request; at eight requests the fix-up's chain of global round trips (store, fence, arrival
# counter, reload) is longer than the small kernel it replaces, and at 64 its loop over the tokens in the one CTA per
# tile that arrives last costs several times what the norm kernel's one CTA per token does.
FOLD_SMALL_KERNELS = True
FOLD_MAX_TOKENS = 4


def linear(x: "torch.Tensor | ScaledRows", w: torch.Tensor, out_dtype: "torch.dtype | None" = None, partials_ok: bool = False,
           deferred_ok: "bool | str | tuple" = False):
    """y = x W^T for a weight in the linear-layer layout [out, in].

    float32: the package's own fp32 kernel (no reduced-precision matrix mode).
    bfloat16: the package's tcgen05 kernel (``gemm_tc``); rows that are no 16-byte multiple
    (K not a multiple of 8) go to a library product instead, as the reference uses a library
    for every projection.  ``out_dtype=torch.float32`` keeps the accumulator's precision
    (used for the logits).  ``partials_ok``: the caller's consumer adds split-K partial
    sums itself, so a ``PartialSums`` may come back instead of a tensor.  ``deferred_ok``: the caller's
    consumer is one of the kernels that take a ``DeferredProduct`` (the built-in norm, ``qkv_rope_write``) or
    calls ``materialize``; for very few tokens (``FOLD_MAX_TOKENS``) the product is then not launched here.
    ``deferred_ok="residual"`` says that the consumer is the norm (the product is a branch output): then a product
    of many tokens in one split is deferred too, since its epilogue can fold the residual add (``folds_residual``).
    ``deferred_ok=("rope", head_dim)``: the consumer is a position encoding that may fold bias, rotation and the cache
    write into the stacked q/k/v product (``folds_rope``)."""
    if x.dtype == torch.float32:
        return sgemm_nt(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ValueError(f"linear: unsupported dtypes {x.dtype} x {w.dtype}")
    rows = x.rows if isinstance(x, ScaledRows) else x
    if USE_TC_GEMM and tc_gemm_supported(rows, w):
        if deferred_ok and FOLD_SMALL_KERNELS and out_dtype in (None, torch.bfloat16) and w.shape[0] % 4 == 0:
            M = rows.shape[0]
            if M <= FOLD_MAX_TOKENS or (deferred_ok == "residual" and folds_residual(M, w.shape[0], w.shape[1])) or \
                    (isinstance(deferred_ok, tuple) and deferred_ok[0] == "rope" and folds_rope(M, w.shape[0], w.shape[1], deferred_ok[1])):
                return DeferredProduct(x, w, torch.bfloat16)
        return gemm_tc(x, w, out_dtype or torch.bfloat16, reduce=not partials_ok, checked=True)
    x = materialize(x)
    if out_dtype is None or out_dtype == torch.bfloat16:
        if partials_ok:     # the consumer adds fp32 partial sums: hand it the accumulator unrounded, as one part
            return PartialSums(torch.mm(x, w.t(), out_dtype=torch.float32).unsqueeze(0), torch.bfloat16)
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = GATED_BLOCK) -> torch.Tensor:
    """[2 I, K]: ``block`` gate rows, the up rows of the same features, the next gate rows, ... (I % block == 0)."""
    inter, K = gate.shape
    if up.shape != gate.shape or inter % block:
        raise UnsupportedSize(f"cannot interleave {tuple(gate.shape)} and {tuple(up.shape)} in blocks of {block}")
    return torch.stack([gate.view(inter // block, block, K), up.view(inter // block, block, K)], dim=1).reshape(2 * inter, K).contiguous()


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for the stacked weight of a gated feed-forward: [gates | ups] rows, or
    (``interleaved``) blocks of ``GATED_BLOCK`` gate rows and up rows in turn, which lets the bfloat16
    tensor-core product apply the activation in its epilogue."""
    rows = x.rows if isinstance(x, ScaledRows) else x
    if interleaved and x.dtype == torch.bfloat16 and USE_TC_GEMM and tc_gemm_supported(rows, w_gate_up):
        return gemm_tc(x, w_gate_up, torch.bfloat16, gated=True, checked=True)
    return silu_mul(linear(x, w_gate_up), block=GATED_BLOCK if interleaved else 0)


# ---------------------------------------------------------------------------------- layers that are no pre-norm block
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The fp32 residual stream as the activations a branch reads: rounded to ``dtype``; for float32 the stream
    itself (a branch reads it before the stream is updated)."""
    _check(x, "x", torch.float32)
    if dtype == torch.float32:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    lib.call("pyre_cast_rows", x.data_ptr(), out.data_ptr(), x.numel(), _dt(dtype), _stream())
    return out


def norm_add(x: torch.Tensor, y: "torch.Tensor | PartialSums | DeferredProduct", weight: torch.Tensor, eps: float,
             act_dtype: torch.dtype, want_next: bool = False) -> "torch.Tensor | None":
    """x[t] += rmsnorm(y[t]) * weight in place on the fp32 stream ``x`` [T, H]: the norm sits on a branch's OUTPUT
    ``y`` (activation dtype, or fp32 partial sums that the kernel adds).  ``want_next``: also return the new stream
    as activations (what the next branch reads), written in the same pass."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    T, H = x.shape
    if weight.shape[0] != H:
        raise ValueError(f"norm weight has {weight.shape[0]} entries, rows have {H}")
    if isinstance(y, DeferredProduct):
        y = y.partials()
    parts, n_parts = None, 0
    if isinstance(y, PartialSums):
        parts, n_parts, y = y.parts, y.n, None
        if tuple(parts.shape[1:]) != (T, H):
            raise ValueError(f"branch output {tuple(parts.shape[1:])} != stream {(T, H)}")
    else:
        _check(y, "y", act_dtype, 2)
        if tuple(y.shape) != (T, H):
            raise ValueError(f"branch output {tuple(y.shape)} != stream {(T, H)}")
    nxt = None
    if want_next and act_dtype != torch.float32:
        nxt = torch.empty((T, H), dtype=act_dtype, device=x.device)
    lib.call("pyre_norm_add", x.data_ptr(), _ptr(y), _ptr(parts), n_parts, T * H, weight.data_ptr(), _ptr(nxt), T, H,
             float(eps), _dt(act_dtype), _stream())
    if want_next and nxt is None:
        return x      # float32 activations are the stream itself
    return nxt


def linear_act(x: torch.Tensor, w: torch.Tensor, kind: str) -> torch.Tensor:
    """act(x W^T) in the activation dtype.  A bfloat16 prompt portion whose plan is a row store in one split gets
    ``gelu_tanh`` in the product's epilogue (on the product rounded to bfloat16, so the result is that of the two
    kernels); everything else runs the product and then ``activation``."""
    if kind not in ACTIVATIONS:
        raise UnsupportedSize(f"activation {kind!r}: implemented are {sorted(ACTIVATIONS)}")
    if FUSE_ACTIVATION and kind == "gelu_tanh" and x.dtype == torch.bfloat16 and USE_TC_GEMM and tc_gemm_supported(x, w):
        M, K = x.shape
        N = w.shape[0]
        weights_as_rows, bn, splits = tc_gemm_plan(M, N, K)
        if M > 128 and not weights_as_rows and splits == 1 and N % 8 == 0:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
            pair = int(CTA_PAIRS and bn in (128, 160, 192, 208, 224, 256))
            lib.call("pyre_gemm_tc", x.data_ptr(), M, x.stride(0), w.data_ptr(), N, w.stride(0), K, out.data_ptr(), 0,
                     N, 1, 0, 1, bn, 0, 2, pair, device_error_flag(x.device).data_ptr(), None, _stream())
            return out
    return activation(materialize(linear(x, w)), kind)


FUSE_ACTIVATION = True


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """act(x) elementwise, fp32 arithmetic: ``silu`` or ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))."""
    _check(x, "x")
    if kind not in ACTIVATIONS:
        raise UnsupportedSize(f"activation {kind!r}: implemented are {sorted(ACTIVATIONS)}")
    out = torch.empty_like(x)
    lib.call("pyre_activation", x.data_ptr(), out.data_ptr(), x.numel(), ACTIVATIONS[kind], _dt(x.dtype), _stream())
    return out


def qk_norm_rope_write(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, q_weight: "torch.Tensor | None",
                       k_weight: "torch.Tensor | None", eps: float, cos: "torch.Tensor | None", sin: "torch.Tensor | None",
                       cache_layer: "torch.Tensor | None", slot_mapping: "torch.Tensor | None", n_heads: int,
                       n_kv_heads: int, qk_dim: int, v_dim: int, row_dim: int, rotary_dim: int, page_size: int,
                       v_cos: "torch.Tensor | None" = None, v_sin: "torch.Tensor | None" = None) -> torch.Tensor:
    """Per-head RMS norm of queries and keys (weights [qk_dim], shared by the heads; None: no norm), rotation of
    the first ``rotary_dim`` dims of each head, and the paged write, for heads whose query/key size ``qk_dim`` and
    value size ``v_dim`` differ from the cache's row size ``row_dim`` (the rest of a row is zero).
    ``proj`` [T, W] holds the token's projections: queries at column ``q_col``, keys at ``k_col``, values at ``v_col``.
    ``cache_layer`` None: nothing is stored and no keys or values are read from ``proj`` (a layer that reads another
    layer's cache).  ``v_cos`` / ``v_sin`` [T, v_dim / 2]: the values are turned too, over all their dims in
    half-split pairs, by these tables, and cached so (``head_gate`` turns a head's weighted sum back).
    Returns the queries [T, n_heads * row_dim]."""
    _check(proj, "proj", dim=2)
    T, W = proj.shape
    D = int(row_dim)
    if (v_cos is None) != (v_sin is None):
        raise ValueError("value tables come in pairs")
    if v_cos is not None:
        _check(v_cos, "v_cos", torch.float32, 2)
        _check(v_sin, "v_sin", torch.float32, 2)
        if v_dim % 2 or tuple(v_cos.shape) != (T, v_dim // 2) or tuple(v_sin.shape) != (T, v_dim // 2):
            raise ValueError(f"v_cos/v_sin must be [{T}, {v_dim // 2}] for values of an even size")
    write = cache_layer is not None
    if write:
        _check(cache_layer, "cache_layer", proj.dtype, 5)
        if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, D):
            raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match [pages, 2, {n_kv_heads}, {page_size}, {D}]")
        if slot_mapping is None:
            raise ValueError("slot_mapping is required with a cache")
        _check(slot_mapping, "slot_mapping", torch.int32, 1)
        if slot_mapping.shape[0] != T:
            raise ValueError("slot_mapping must have one entry per token")
        if k_col < 0 or v_col < 0 or k_col + n_kv_heads * qk_dim > W or v_col + n_kv_heads * v_dim > W:
            raise ValueError("the keys or values do not lie inside the projection row")
    if qk_dim > D or v_dim > D:
        raise ValueError(f"heads of {qk_dim} / {v_dim} do not fit cache rows of {D}")
    if rotary_dim % 2 or not 0 <= rotary_dim <= qk_dim:
        raise UnsupportedSize(f"rotary_dim {rotary_dim} must be even and at most the query/key size {qk_dim}")
    if q_col < 0 or q_col + n_heads * qk_dim > W:
        raise ValueError("the queries do not lie inside the projection row")
    for w, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _check(w, name, torch.float32, 1)
            if w.shape[0] != qk_dim:
                raise ValueError(f"{name} has {w.shape[0]} entries, a head has {qk_dim}")
    half = rotary_dim // 2
    if rotary_dim:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, half) or tuple(sin.shape) != (T, half):
            raise ValueError(f"cos/sin must be [{T}, {half}], got {tuple(cos.shape)}")
    q_out = torch.empty((T, n_heads * D), dtype=proj.dtype, device=proj.device)
    lib.call("pyre_qk_norm_rope_write", proj.data_ptr(), W, int(q_col), int(k_col) if write else -1, int(v_col) if write else -1,
             _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos) if rotary_dim else None, _ptr(sin) if rotary_dim else None,
             _ptr(v_cos), _ptr(v_sin), q_out.data_ptr(), _ptr(cache_layer), _ptr(slot_mapping) if write else None, T, n_heads,
             n_kv_heads, qk_dim, v_dim, D, rotary_dim, page_size, _dt(proj.dtype),
             cache_layer.shape[0] if write else 0, device_error_flag(proj.device).data_ptr(), _stream())
    return q_out


def sigmoid_gate(a: torch.Tensor, a_dim: int, proj: "torch.Tensor | None", g_col: int, n_heads: int, v_dim: int) -> torch.Tensor:
    """out[t, h, j] = a[t, h, j] * sigmoid(proj[t, g_col + h v_dim + j]) for j < v_dim; a head of ``a`` has ``a_dim``
    columns, of which the first ``v_dim`` count.  ``proj`` None: no gate, the heads are only narrowed.
    Returns [T, n_heads * v_dim]."""
    _check(a, "a", dim=2)
    T = a.shape[0]
    if a.shape[1] != n_heads * a_dim or a_dim < v_dim:
        raise ValueError("the heads do not match the tensor")
    if proj is not None:
        _check(proj, "proj", a.dtype, 2)
        if proj.shape[0] != T or g_col < 0 or g_col + n_heads * v_dim > proj.shape[1]:
            raise ValueError("the gate does not lie inside the projection row")
    out = torch.empty((T, n_heads * v_dim), dtype=a.dtype, device=a.device)
    lib.call("pyre_sigmoid_gate", a.data_ptr(), int(a_dim), _ptr(proj), proj.shape[1] if proj is not None else 0,
             int(g_col) if proj is not None else -1, out.data_ptr(), T, n_heads, v_dim, _dt(a.dtype), _stream())
    return out


def head_gate(a: torch.Tensor, a_dim: int, proj: "torch.Tensor | None", g_col: int, n_heads: int, v_dim: int,
              cos: "torch.Tensor | None" = None, sin: "torch.Tensor | None" = None) -> torch.Tensor:
    """out[t, h, :] = turn_back(a[t, h, :v_dim]) * sigmoid(proj[t, g_col + h]): ONE gate per head (``proj`` None: no
    gate); with ``cos`` / ``sin`` [T, v_dim / 2] the half-split pairs of a head are turned by minus the token's
    angles first (the sum of values that were cached rotated).  A head of ``a`` has ``a_dim`` columns, of which the
    first ``v_dim`` count.  Returns [T, n_heads * v_dim]."""
    _check(a, "a", dim=2)
    T = a.shape[0]
    if a.shape[1] != n_heads * a_dim or a_dim < v_dim:
        raise ValueError("the heads do not match the tensor")
    if proj is not None:
        _check(proj, "proj", a.dtype, 2)
        if proj.shape[0] != T or g_col < 0 or g_col + n_heads > proj.shape[1]:
            raise ValueError("the gates do not lie inside the projection row")
    if (cos is None) != (sin is None):
        raise ValueError("tables come in pairs")
    if cos is not None:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if v_dim % 2 or tuple(cos.shape) != (T, v_dim // 2) or tuple(sin.shape) != (T, v_dim // 2):
            raise ValueError(f"cos/sin must be [{T}, {v_dim // 2}] for values of an even size")
    out = torch.empty((T, n_heads * v_dim), dtype=a.dtype, device=a.device)
    lib.call("pyre_head_gate", a.data_ptr(), int(a_dim), _ptr(proj), proj.shape[1] if proj is not None else 0,
             int(g_col) if proj is not None else -1, _ptr(cos), _ptr(sin), out.data_ptr(), T, n_heads, v_dim, _dt(a.dtype), _stream())
    return out


BIAS_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu2": 2, "tanh": 3, None: 4}


def bias_act(x: torch.Tensor, bias: "torch.Tensor | None", kind: "str | None") -> torch.Tensor:
    """act(x + bias) over rows, fp32 arithmetic on a product's result: ``silu``, ``gelu_tanh``, ``relu2`` (the square
    of relu), ``tanh`` or None (the bias only); ``bias`` fp32 [H] or None."""
    _check(x, "x", dim=2)
    if kind not in BIAS_ACTIVATIONS:
        raise UnsupportedSize(f"activation {kind!r}: implemented are {sorted(k for k in BIAS_ACTIVATIONS if k)}")
    T, H = x.shape
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != H:
            raise ValueError(f"bias has {bias.shape[0]} entries, rows have {H}")
    out = torch.empty_like(x)
    lib.call("pyre_bias_act", x.data_ptr(), _ptr(bias), out.data_ptr(), T, H, BIAS_ACTIVATIONS[kind], _dt(x.dtype), _stream())
    return out


def add_row_vector(x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """x[t] += v for every row of the fp32 stream ``x`` [T, H], in place."""
    _check(x, "x", torch.float32, 2)
    _check(v, "v", torch.float32, 1)
    if v.shape[0] != x.shape[1]:
        raise ValueError(f"a vector of {v.shape[0]} entries for rows of {x.shape[1]}")
    lib.call("pyre_add_row_vector", x.data_ptr(), v.data_ptr(), x.shape[0], x.shape[1], _stream())
    return x


def gated_norm(y: "torch.Tensor | PartialSums | DeferredProduct", y_bias: "torch.Tensor | None", gate: "torch.Tensor | None",
               gate_bias: "torch.Tensor | None", weight: torch.Tensor, eps: float, act_dtype: torch.dtype,
               center: bool = True, out_bias: "torch.Tensor | None" = None) -> torch.Tensor:
    """norm((y + y_bias) * sigmoid(gate + gate_bias)) * weight per row, as fp32 [T, H]: a branch's output (activation
    dtype, or fp32 partial sums that the kernel adds) gated element by element and normed, ready to be added to the
    stream.  ``center``: a layer norm without bias (mean taken off, variance of the deviations); else an RMS norm.
    ``gate`` None: no gate.  ``out_bias`` fp32 [H]: added after the gain (a norm with a bias)."""
    _check(weight, "weight", torch.float32, 1)
    H = weight.shape[0]
    if isinstance(y, DeferredProduct):
        y = y.partials()
    parts, n_parts, stride = None, 0, 0
    if isinstance(y, PartialSums):
        parts, n_parts, y = y.parts, y.n, None
        T = parts.shape[1]
        stride, device = T * H, parts.device
        if parts.shape[2] != H:
            raise ValueError(f"branch output rows of {parts.shape[2]}, norm weight of {H}")
    else:
        _check(y, "y", act_dtype, 2)
        T, device = y.shape[0], y.device
        if y.shape[1] != H:
            raise ValueError(f"branch output rows of {y.shape[1]}, norm weight of {H}")
    for b, name in ((y_bias, "y_bias"), (gate_bias, "gate_bias"), (out_bias, "out_bias")):
        if b is not None:
            _check(b, name, torch.float32, 1)
            if b.shape[0] != H:
                raise ValueError(f"{name} has {b.shape[0]} entries, rows have {H}")
    if gate is not None:
        _check(gate, "gate", act_dtype, 2)
        if tuple(gate.shape) != (T, H):
            raise ValueError(f"gate {tuple(gate.shape)} != branch output {(T, H)}")
    if H * 4 > 48 * 1024:
        raise UnsupportedSize(f"rows of {H}: the gated norm takes up to 12,288 entries")
    out = torch.empty((T, H), dtype=torch.float32, device=device)
    lib.call("pyre_gated_norm", _ptr(y), _ptr(parts), n_parts, stride, _ptr(y_bias), _ptr(gate),
             _ptr(gate_bias) if gate is not None else None, weight.data_ptr(), _ptr(out_bias), out.data_ptr(), T, H, float(eps),
             int(bool(center)),
             _dt(act_dtype), _stream())
    return out


def rmsnorm_gate(o: torch.Tensor, weight: torch.Tensor, eps: float, proj: "torch.Tensor | None", g_col: int,
                 out_dtype: torch.dtype) -> torch.Tensor:
    """rmsnorm(o[t]) * weight * sigmoid(proj[t, g_col:g_col + H]) over whole rows of fp32 ``o`` [T, H]
    (``proj`` None: no gate); returns the activation dtype."""
    _check(o, "o", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    T, H = o.shape
    if weight.shape[0] != H:
        raise ValueError(f"norm weight has {weight.shape[0]} entries, rows have {H}")
    if proj is not None:
        _check(proj, "proj", out_dtype, 2)
        if proj.shape[0] != T or g_col < 0 or g_col + H > proj.shape[1]:
            raise ValueError("the gate does not lie inside the projection row")
    out = torch.empty((T, H), dtype=out_dtype, device=o.device)
    lib.call("pyre_rmsnorm_gate", o.data_ptr(), weight.data_ptr(), _ptr(proj), proj.shape[1] if proj is not None else 0,
             int(g_col) if proj is not None else -1, out.data_ptr(), T, H, float(eps), _dt(out_dtype), _stream())
    return out


def linear_attention(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, state_layer: torch.Tensor,
                     slots: torch.Tensor, cu_seqlens: torch.Tensor, decay: torch.Tensor, n_heads: int, qk_dim: int,
                     v_dim: int, activation: "str | None" = "silu", lens=None) -> torch.Tensor:
    """Linear attention with a constant decay per head over the step's entries, continuing each request's state:
    S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, with q, k, v = act(columns of ``proj``).
    ``state_layer`` [slots, n_heads, qk_dim, v_dim] fp32 is read and left updated at ``slots[b]`` for entry b.
    Returns fp32 [T, n_heads * v_dim].

    ``lens``: the entries' token counts on the host.  With them, bfloat16 entries of ``LINEAR_CHUNK_MIN_LEN`` tokens
    or more run on the tensor cores in chunks of 64 tokens (query/key sizes 64 and 128, value sizes that are
    multiples of 32, 16-byte aligned columns); everything else, and all of float32, walks token by token in fp32,
    bit-identical under any cutting."""
    _check(proj, "proj", dim=2)
    _check(state_layer, "state_layer", torch.float32, 4)
    _check(slots, "slots", torch.int32, 1)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(decay, "decay", torch.float32, 1)
    T, W = proj.shape
    n_seqs = cu_seqlens.shape[0] - 1
    if tuple(state_layer.shape[1:]) != (n_heads, qk_dim, v_dim) or decay.shape[0] != n_heads or slots.shape[0] < n_seqs:
        raise ValueError("state, decay or slots do not match the heads and the batch")
    if qk_dim > 256:
        raise UnsupportedSize(f"linear attention takes query/key sizes up to 256, got {qk_dim}")
    if min(q_col, k_col, v_col) < 0 or max(q_col, k_col) + n_heads * qk_dim > W or v_col + n_heads * v_dim > W:
        raise ValueError("q, k or v do not lie inside the projection row")
    if activation not in (None, "silu"):
        raise UnsupportedSize(f"linear attention: activation {activation!r} is not implemented")
    out = torch.empty((T, n_heads * v_dim), dtype=torch.float32, device=proj.device)
    act = 1 if activation == "silu" else 0
    max_len = 0
    if lens is not None and USE_LINEAR_CHUNKS and proj.dtype == torch.bfloat16 and linear_chunks_ok(W, q_col, k_col, v_col, qk_dim, v_dim) \
            and int(max(lens)) >= LINEAR_CHUNK_MIN_LEN:
        lib.call("pyre_linear_attention_chunked", proj.data_ptr(), W, int(q_col), int(k_col), int(v_col), state_layer.data_ptr(),
                 slots.data_ptr(), cu_seqlens.data_ptr(), decay.data_ptr(), out.data_ptr(), T, n_seqs, n_heads, qk_dim, v_dim,
                 act, LINEAR_CHUNK_MIN_LEN, _stream())
        if int(min(lens)) >= LINEAR_CHUNK_MIN_LEN:
            return out
        max_len = LINEAR_CHUNK_MIN_LEN - 1
    lib.call("pyre_linear_attention_scan", proj.data_ptr(), W, int(q_col), int(k_col), int(v_col), state_layer.data_ptr(),
             slots.data_ptr(), cu_seqlens.data_ptr(), decay.data_ptr(), out.data_ptr(), T, n_seqs, n_heads, qk_dim, v_dim,
             act, _dt(proj.dtype), max_len, _stream())
    return out


USE_LINEAR_CHUNKS = True
LINEAR_CHUNK_MIN_LEN = 32     # entries with at least this many tokens go to the tensor-core kernel


def linear_chunks_ok(row_width: int, q_col: int, k_col: int, v_col: int, qk_dim: int, v_dim: int) -> bool:
    """The sizes the tensor-core linear attention takes (as its launcher checks them)."""
    return qk_dim in (64, 128) and v_dim % 32 == 0 and row_width % 8 == 0 and q_col % 8 == 0 and k_col % 8 == 0 and v_col % 8 == 0


def attention_row_dim(qk_dim: int, v_dim: int, dtype: torch.dtype) -> int:
    """The row size of a paged cache whose heads have ``qk_dim`` query/key dims and ``v_dim`` value dims: one size
    for keys and values, so that every attention kernel of the package serves them (the columns beyond a head's own
    are zero and change neither scores nor outputs).  A multiple of 16; for bfloat16 the head sizes of the
    prompt-portion kernels (64, 128) where the heads are larger than 32."""
    d = -(-max(int(qk_dim), int(v_dim)) // 16) * 16
    if dtype == torch.bfloat16:
        if 32 < d <= 64:
            d = 64
        elif 64 < d <= 128:
            d = 128
    if d > 256:
        raise UnsupportedSize(f"heads of {qk_dim} / {v_dim} dims: the attention kernels take up to 256")
    return d


# ---------------------------------------------------------------------------------- layers whose branches share one norm
class ScaledSum:
    """The branch outputs of a layer that adds all of them to the stream at once, each with a gain per feature:
    ``sum_k scale_k * term_k``, not formed yet.  ``terms``: one or two of (branch output, fp32 gain [H]); a branch
    output is a tensor [T, H] in the activation dtype, an fp32 tensor [T, H] (taken as one part of a split
    product) or ``PartialSums``.  A norm that knows this type adds the terms to the fp32 stream in its own kernel
    (``add_layernorm``); anything else calls ``materialize``."""

    def __init__(self, terms, dtype: torch.dtype):
        if not 1 <= len(terms) <= 2:
            raise ValueError("a ScaledSum holds one or two terms")
        self.terms = [(materialize(t) if isinstance(t, (DeferredProduct, ScaledRows)) else t, s) for t, s in terms]
        self.dtype = dtype

    @property
    def shape(self):
        return tuple(self.terms[0][0].shape)

    def _args(self, act_dtype):
        """Per term (tensor pointer, parts pointer, number of parts, gain pointer), two terms, and the parts' stride."""
        out, stride = [], 0
        T, H = self.shape
        for t, s in self.terms:
            _check(s, "gain", torch.float32, 1)
            if s.shape[0] != H:
                raise ValueError(f"a gain of {s.shape[0]} entries for rows of {H}")
            if isinstance(t, PartialSums):
                out += [None, t.parts.data_ptr(), t.n, s.data_ptr()]
                stride = T * H
            elif t.dtype == torch.float32 and act_dtype != torch.float32:
                _check(t, "branch output", torch.float32, 2)
                out += [None, t.data_ptr(), 1, s.data_ptr()]
                stride = T * H
            else:
                _check(t, "branch output", act_dtype, 2)
                out += [t.data_ptr(), None, 0, s.data_ptr()]
            if tuple(t.shape) != (T, H):
                raise ValueError("the branch outputs differ in shape")
        if len(self.terms) == 1:
            out += [None, None, 0, None]
        return out, stride

    def tensor(self) -> torch.Tensor:
        T, H = self.shape
        args, stride = self._args(self.dtype)
        out = torch.empty((T, H), dtype=self.dtype, device=self.terms[0][1].device)
        a = args
        lib.call("pyre_scaled_sum", a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], stride, out.data_ptr(), T, H, _dt(self.dtype),
                 _stream())
        return out


def add_layernorm(x: torch.Tensor, delta: "ScaledSum | torch.Tensor | PartialSums | None", weight: torch.Tensor, eps: float,
                  out_dtype: torch.dtype, rows: "torch.Tensor | None" = None, update_x: bool = True,
                  act_dtype: "torch.dtype | None" = None, bias: "torch.Tensor | None" = None) -> torch.Tensor:
    """out[r] = layernorm(x[src] + delta[src]) * weight (+ bias) with src = rows[r] (or r): the mean is taken off, the
    variance is the mean squared deviation; ``bias`` fp32 [H] or None.  ``x`` is the fp32 residual stream [T, H]; with ``update_x``
    (and no ``rows``) the sum is written back to it.  ``delta``: a ``ScaledSum`` (each term times its gain), a
    plain branch output or partial sums (gain one), or None.  ``out_dtype`` float32 with bfloat16 activations
    (``act_dtype``) gives the normalised rows in fp32: a norm applied to the stream itself."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    T, H = x.shape
    act = act_dtype or out_dtype
    if weight.shape[0] != H:
        raise ValueError(f"norm weight has {weight.shape[0]} entries, rows have {H}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != H:
            raise ValueError(f"norm bias has {bias.shape[0]} entries, rows have {H}")
    if H * 4 > 48 * 1024:
        raise UnsupportedSize(f"layer norm over rows of {H}: the kernel holds a row of at most 12,288 in shared memory")
    if delta is not None and not isinstance(delta, ScaledSum):
        delta = ScaledSum([(delta, _ones(H, x.device))], act)
    args, stride = ([None, None, 0, None] * 2, 0)
    if delta is not None:
        if delta.shape != (T, H):
            raise ValueError(f"delta shape {delta.shape} != x shape {(T, H)}")
        args, stride = delta._args(act)
    n_rows = T
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_rows, update_x = rows.shape[0], False
    out = torch.empty((n_rows, H), dtype=out_dtype, device=x.device)
    a = args
    lib.call("pyre_add_layernorm", x.data_ptr(), a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], stride, weight.data_ptr(), _ptr(bias), out.data_ptr(),
             int(out_dtype == torch.float32 and act != torch.float32), _ptr(rows), n_rows, H, float(eps),
             int(bool(update_x and delta is not None)), _dt(act), _stream())
    return out


_ones_cache: dict = {}


def _ones(n: int, device) -> torch.Tensor:
    key = (n, str(device))
    t = _ones_cache.get(key)
    if t is None:
        t = _ones_cache[key] = torch.ones(n, dtype=torch.float32, device=device)
    return t


def act_mul(gate_up: torch.Tensor, kind: str) -> torch.Tensor:
    """out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i] for rows [gates | ups]; ``kind`` as in ``ACTIVATIONS``."""
    _check(gate_up, "gate_up", dim=2)
    if kind not in ACTIVATIONS:
        raise UnsupportedSize(f"activation {kind!r}: implemented are {sorted(ACTIVATIONS)}")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise ValueError("gate_up must have an even number of columns")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    lib.call("pyre_act_mul", gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, ACTIVATIONS[kind], _dt(gate_up.dtype), _stream())
    return out


# ---------------------------------------------------------------------------------- attention over a cache of latent rows
LATENT_MAX_RANK = 512


def latent_prepare(proj: "torch.Tensor | PartialSums", q_col: int, q_rank: int, c_col: int, rank: int, rope: int, rot: int,
                   wq: "torch.Tensor | None", wc: torch.Tensor, eps: float, cos: "torch.Tensor | None", sin: "torch.Tensor | None",
                   cache_layer: "torch.Tensor | None", slot_mapping: "torch.Tensor | None", page_size: int,
                   act_dtype: torch.dtype) -> "torch.Tensor | None":
    """From a token's down-projections ``proj`` [T, W] (columns ``q_col``: the query latent of ``q_rank`` entries,
    0 for none; ``c_col``: the key/value latent of ``rank`` entries followed by the shared key part of ``rope``):
    returns rmsnorm(query latent) * wq [T, q_rank] and writes [rmsnorm(latent) * wc | rotate(key part)] to the
    token's row of ``cache_layer`` [pages, 1, 1, page_size, row].  The rotation turns neighbouring pairs of the
    first ``rot`` entries by the angles whose cos/sin are given [T, rot / 2]."""
    parts, n_parts, stride, tensor = None, 0, 0, None
    if isinstance(proj, PartialSums):
        parts, n_parts, stride = proj.parts, proj.n, proj.parts[0].numel()
        T, W = proj.shape
        device = proj.parts.device
    else:
        _check(proj, "proj", act_dtype, 2)
        tensor, (T, W), device = proj, proj.shape, proj.device
    if q_col < 0 or q_col + q_rank > W or c_col < 0 or c_col + rank + rope > W:
        raise ValueError("the latents do not lie inside the projection row")
    if rot % 2 or not 0 <= rot <= rope:
        raise UnsupportedSize(f"rotated dims ({rot}) must be even and at most the rotated key part ({rope})")
    _check(wc, "wc", torch.float32, 1)
    if wc.shape[0] != rank or (q_rank and (wq is None or wq.shape[0] != q_rank)):
        raise ValueError("a norm weight does not match its latent")
    if rot:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, rot // 2) or tuple(sin.shape) != (T, rot // 2):
            raise ValueError(f"cos/sin must be [{T}, {rot // 2}], got {tuple(cos.shape)}")
    row = n_pages = 0
    if cache_layer is not None:
        _check(cache_layer, "cache_layer", act_dtype, 5)
        row, n_pages = cache_layer.shape[4], cache_layer.shape[0]
        if tuple(cache_layer.shape[1:4]) != (1, 1, page_size) or row < rank + rope:
            raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match [pages, 1, 1, {page_size}, >= {rank + rope}]")
        _check(slot_mapping, "slot_mapping", torch.int32, 1)
        if slot_mapping.shape[0] != T:
            raise ValueError("slot_mapping must have one entry per token")
    cq = torch.empty((T, q_rank), dtype=act_dtype, device=device) if q_rank else None
    lib.call("pyre_latent_prepare", _ptr(tensor), _ptr(parts), n_parts, stride, W, int(q_col), int(q_rank), int(c_col), int(rank),
             int(rope), int(rot), _ptr(wq), wc.data_ptr(), float(eps), _ptr(cos) if rot else None, _ptr(sin) if rot else None,
             _ptr(cq), _ptr(cache_layer), _ptr(slot_mapping) if cache_layer is not None else None, T, max(row, rank + rope),
             n_pages, int(page_size), _dt(act_dtype), device_error_flag(device).data_ptr(), _stream())
    return cq


def latent_rotate_q(q: torch.Tensor, qa: torch.Tensor, cos, sin, n_heads: int, dq: int, rope: int, rot: int, rank: int) -> None:
    """qa[t, h, rank + i] = rotate(q[t, h, dq + i]) for i < rope (zeros beyond): the rotated tail of the absorbed
    query rows ``qa`` [T, n_heads, row]; ``q`` [T, n_heads * (dq + rope)]."""
    _check(q, "q", dim=2)
    _check(qa, "qa", q.dtype, 3)
    T, row = q.shape[0], qa.shape[2]
    if q.shape[1] != n_heads * (dq + rope) or tuple(qa.shape[:2]) != (T, n_heads) or row < rank + rope:
        raise ValueError("q or qa do not match the head sizes")
    lib.call("pyre_latent_rotate_q", q.data_ptr(), qa.data_ptr(), _ptr(cos) if rot else None, _ptr(sin) if rot else None, T,
             n_heads, int(dq), int(rope), int(rot), int(rank), row, _dt(q.dtype), _stream())


def latent_attention_exact(qa: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, seq_of_token: torch.Tensor,
                           positions: torch.Tensor, rank: int, rope: int, scale: float, window: "int | None") -> torch.Tensor:
    """Exact fp32-arithmetic attention of absorbed queries ``qa`` [T, nh, row] over the latent rows of their
    sequences' pages: score = qa . row[: rank + rope] * scale, output = sum of probabilities times row[: rank];
    returns [T, nh, rank]."""
    _check(qa, "qa", dim=3)
    _check(cache_layer, "cache_layer", qa.dtype, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T, nh, row = qa.shape
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (1, 1, page_size, row) or row < rank + rope:
        raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match rows of {row}")
    if rank > LATENT_MAX_RANK or (rank + rope) * 16 > 48 * 1024:
        raise UnsupportedSize(f"latent rows of {rank} + {rope}: the kernel takes latents up to {LATENT_MAX_RANK}")
    out = torch.empty((T, nh, rank), dtype=qa.dtype, device=qa.device)
    lib.call("pyre_latent_attention_exact", qa.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(), T, nh, int(rank), int(rope), row, page_size,
             int(window or 0), float(scale), _dt(qa.dtype), cache_layer.shape[0], device_error_flag(qa.device).data_ptr(), _stream())
    return out


# ---------------------------------------------------------------------------------- one weight matrix per group
USE_GROUPED_MMA = True


def _grouped_mma_ok(x: torch.Tensor, w: torch.Tensor, x_row_stride: int, x_group_stride: int, K: int) -> int:
    return int(USE_GROUPED_MMA and x.dtype == torch.bfloat16 and K % 8 == 0 and x_row_stride % 8 == 0
               and x_group_stride % 8 == 0 and (w.shape[1] * w.shape[2]) % 8 == 0 and x.data_ptr() % 16 == 0
               and w.data_ptr() % 16 == 0)


def headwise_linear(x: torch.Tensor, w: torch.Tensor, out: "torch.Tensor | None" = None) -> torch.Tensor:
    """out[t, h, :N] = x[t, h, :K] . w[h]^T for ``x`` [T, H, >= K] and ``w`` [H, N, K]: a product per head.  ``out``
    [T, H, >= N] may be given (rows wider than N keep their other columns); else [T, H, N] is returned."""
    _check(x, "x", dim=3)
    _check(w, "w", x.dtype, 3)
    T, H, xs = x.shape
    _, N, K = w.shape
    if w.shape[0] != H or xs < K:
        raise ValueError(f"x {tuple(x.shape)} and w {tuple(w.shape)} do not match head by head")
    if out is None:
        out = torch.empty((T, H, N), dtype=x.dtype, device=x.device)
    else:
        _check(out, "out", x.dtype, 3)
        if tuple(out.shape[:2]) != (T, H) or out.shape[2] < N:
            raise ValueError("out does not match the heads")
    lib.call("pyre_grouped_linear", x.data_ptr(), H * xs, xs, w.data_ptr(), N * K, out.data_ptr(), H * out.shape[2], out.shape[2],
             None, None, None, T, N, K, H, 0, 0, _dt(x.dtype), _grouped_mma_ok(x, w, H * xs, xs, K), _stream())
    return out


def expert_linear(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, src: "torch.Tensor | None", n_places: int,
                  out_dtype: "torch.dtype | None" = None) -> torch.Tensor:
    """out[p] = x[src[p]] . w[e]^T for every sorted place p of expert e (``offsets`` [E + 1] on the device; places
    beyond ``offsets[E]`` are not written); ``x`` [rows, K], ``w`` [E, N, K]; ``src`` None: place p reads row p.
    Returns [n_places, N] in ``out_dtype`` (the activation dtype, or float32)."""
    _check(x, "x", dim=2)
    _check(w, "w", x.dtype, 3)
    _check(offsets, "offsets", torch.int32, 1)
    E, N, K = w.shape
    if x.shape[1] != K or offsets.shape[0] != E + 1:
        raise ValueError("x, w and offsets do not match")
    if src is not None:
        _check(src, "src", torch.int32, 1)
    out_dtype = out_dtype or x.dtype
    if out_dtype not in (x.dtype, torch.float32):
        raise ValueError("the result is in the activation dtype or float32")
    out = torch.empty((n_places, N), dtype=out_dtype, device=x.device)
    lib.call("pyre_grouped_linear", x.data_ptr(), K, 0, w.data_ptr(), N * K, out.data_ptr(), N, 0, offsets.data_ptr(), _ptr(src),
             None, 0, N, K, E, int(n_places), int(out_dtype == torch.float32), _dt(x.dtype), _grouped_mma_ok(x, w, K, 0, K), _stream())
    return out


def route(h: torch.Tensor, w: torch.Tensor, correction: "torch.Tensor | None", top: int, scale: float, sigmoid: bool = False,
          bias: "torch.Tensor | None" = None, renormalise: bool = False):
    """Router of a routed feed-forward: fp32 logits w h (+ ``bias``) over all router outputs, softmax scores s
    (``sigmoid``: each output's own sigmoid instead); the ``top`` outputs with the largest s + correction are chosen
    (lowest index on ties), weights s * scale; ``renormalise``: divided by their sum over the chosen (with softmax
    scores that is the softmax over the chosen logits alone).
    Returns (idx int32 [T, top], weight fp32 [T, top])."""
    _check(h, "h", dim=2)
    _check(w, "w", torch.float32, 2)
    T, H = h.shape
    n_out = w.shape[0]
    if w.shape[1] != H or not 0 < top <= n_out:
        raise ValueError("router weight or top do not match")
    if correction is not None:
        _check(correction, "correction", torch.float32, 1)
        if correction.shape[0] != n_out:
            raise ValueError("one correction per router output")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != n_out:
            raise ValueError("one bias per router output")
    if n_out * 8 > 48 * 1024:
        raise UnsupportedSize(f"{n_out} router outputs: the kernel takes up to 6,144")
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=h.device)
    lib.call("pyre_route", h.data_ptr(), w.data_ptr(), _ptr(correction), _ptr(bias), idx.data_ptr(), weight.data_ptr(), T, H, n_out,
             int(top), float(scale), int(bool(sigmoid)), int(bool(renormalise)), _dt(h.dtype), _stream())
    return idx, weight


def group_pairs(idx: torch.Tensor, n_experts: int):
    """Sort the (token, choice) pairs ``idx`` [T, top] by expert; outputs >= ``n_experts`` get no place.
    Returns (offsets int32 [n_experts + 1], place_of int32 [T, top], src int32 [T * top])."""
    _check(idx, "idx", torch.int32, 2)
    T, top = idx.shape
    if n_experts * 4 > 48 * 1024:
        raise UnsupportedSize(f"{n_experts} experts: the kernel takes up to 12,288")
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=idx.device)
    place_of = torch.empty((T, top), dtype=torch.int32, device=idx.device)
    src = torch.empty(T * top, dtype=torch.int32, device=idx.device)
    lib.call("pyre_group_pairs", idx.data_ptr(), T * top, top, int(n_experts), offsets.data_ptr(), place_of.data_ptr(),
             src.data_ptr(), _stream())
    return offsets, place_of, src


def combine_pairs(y: torch.Tensor, h: torch.Tensor, place_of: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_k weight[t, k] * (y[place_of[t, k]], or h[t] where the place is -1), fp32 [T, H]."""
    _check(y, "y", torch.float32, 2)
    _check(h, "h", dim=2)
    _check(place_of, "place_of", torch.int32, 2)
    _check(weight, "weight", torch.float32, 2)
    T, H = h.shape
    if y.shape[1] != H or place_of.shape != weight.shape or place_of.shape[0] != T:
        raise ValueError("y, h, place_of and weight do not match")
    out = torch.empty((T, H), dtype=torch.float32, device=h.device)
    lib.call("pyre_combine_pairs", y.data_ptr(), h.data_ptr(), place_of.data_ptr(), weight.data_ptr(), out.data_ptr(), T, H,
             place_of.shape[1], _dt(h.dtype), _stream())
    return out


def scale_to_places(h: torch.Tensor, place_of: torch.Tensor, weight: torch.Tensor, n_places: int) -> torch.Tensor:
    """out[place_of[t, k]] = weight[t, k] * h[t] for every pair with a place: the experts' inputs of a routed
    feed-forward whose weights multiply what an expert reads, in the order of the sorted places [n_places, H]."""
    _check(h, "h", dim=2)
    _check(place_of, "place_of", torch.int32, 2)
    _check(weight, "weight", torch.float32, 2)
    T, H = h.shape
    if place_of.shape != weight.shape or place_of.shape[0] != T:
        raise ValueError("h, place_of and weight do not match")
    out = torch.empty((int(n_places), H), dtype=h.dtype, device=h.device)
    lib.call("pyre_scale_to_places", h.data_ptr(), place_of.data_ptr(), weight.data_ptr(), out.data_ptr(), T, H, place_of.shape[1],
             _dt(h.dtype), _stream())
    return out


# ---------------------------------------------------------------------------------- time mixing with a matrix state
WKV_MAX_DIM = 128


def wkv_state_floats(n_heads: int, dim: int, width: int) -> int:
    """Floats of one request's state slot: [n_heads, dim, dim] matrices, then the last token's input [width]."""
    return n_heads * dim * dim + width


def token_shift_mix(h: torch.Tensor, state_layer: torch.Tensor, prev_off: int, slots: torch.Tensor, seq_of_token: torch.Tensor,
                    cu_seqlens: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """out[s, t] = h[t] + (prev[t] - h[t]) * mu[s] for each of the blends ``mu`` [S, W] (fp32): prev[t] is the row
    before t inside an entry of the step, and for an entry's first token the vector kept at ``prev_off`` of the
    request's slot of ``state_layer`` [slots, floats] (zeros for a new request).  Returns [S, T, W]."""
    _check(h, "h", dim=2)
    _check(state_layer, "state_layer", torch.float32, 2)
    _check(slots, "slots", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(mu, "mu", torch.float32, 2)
    T, W = h.shape
    if mu.shape[1] != W or prev_off < 0 or prev_off + W > state_layer.shape[1] or seq_of_token.shape[0] != T:
        raise ValueError("mu, the state or the batch do not match the rows")
    out = torch.empty((mu.shape[0], T, W), dtype=h.dtype, device=h.device)
    lib.call("pyre_token_shift_mix", h.data_ptr(), state_layer.data_ptr(), state_layer.shape[1], int(prev_off), slots.data_ptr(),
             seq_of_token.data_ptr(), cu_seqlens.data_ptr(), mu.data_ptr(), out.data_ptr(), T, W, mu.shape[0], _dt(h.dtype), _stream())
    return out


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, dlog: torch.Tensor, w0: torch.Tensor,
             u: torch.Tensor, norm_w: torch.Tensor, state_layer: torch.Tensor, prev_off: int, slots: torch.Tensor,
             cu_seqlens: torch.Tensor, h: torch.Tensor, n_heads: int, dim: int, eps: float) -> torch.Tensor:
    """The recurrence of a time-mixing layer with a matrix state per head, token by token in fp32, continuing each
    request's state: with w = exp(-exp(dlog + w0)) per key channel,
    o_t = (S + diag(u) k_t v_t^T)^T r_t, then S = diag(w_t) S + k_t v_t^T; each head's o_t is divided by its root mean
    square (``eps`` inside the root), multiplied by ``norm_w`` and by silu(g).  ``r, k, v, g`` [T, n_heads * dim] in
    the activation dtype, ``dlog`` fp32.  ``state_layer`` [slots, floats] holds [n_heads, dim, dim] per request and,
    at ``prev_off``, the last input row ``h`` [T, W] of each entry, which this call leaves there.
    Returns [T, n_heads * dim] in the activation dtype."""
    _check(r, "r", dim=2)
    T, HD = r.shape
    for t, name in ((k, "k"), (v, "v"), (g, "g")):
        _check(t, name, r.dtype, 2)
        if tuple(t.shape) != (T, HD):
            raise ValueError(f"{name} {tuple(t.shape)} != r {(T, HD)}")
    _check(dlog, "dlog", torch.float32, 2)
    _check(h, "h", r.dtype, 2)
    _check(state_layer, "state_layer", torch.float32, 2)
    _check(slots, "slots", torch.int32, 1)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    for t, name in ((w0, "w0"), (u, "u"), (norm_w, "norm_w")):
        _check(t, name, torch.float32, 1)
        if t.shape[0] != HD:
            raise ValueError(f"{name} has {t.shape[0]} entries, expected {HD}")
    W = h.shape[1]
    n_seqs = cu_seqlens.shape[0] - 1
    if HD != n_heads * dim or tuple(dlog.shape) != (T, HD) or h.shape[0] != T or slots.shape[0] < n_seqs:
        raise ValueError("the heads, the decay or the batch do not match")
    if dim > WKV_MAX_DIM:
        raise UnsupportedSize(f"heads of {dim}: the recurrence takes up to {WKV_MAX_DIM}")
    if prev_off < n_heads * dim * dim or prev_off + W > state_layer.shape[1]:
        raise ValueError("the state slot does not hold the matrices and the input row")
    out = torch.empty((T, HD), dtype=r.dtype, device=r.device)
    raw = torch.empty((T, HD), dtype=torch.float32, device=r.device)      # o before the unit norm, between the two kernels
    lib.call("pyre_wkv_scan", r.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), dlog.data_ptr(), w0.data_ptr(), u.data_ptr(),
             norm_w.data_ptr(), state_layer.data_ptr(), state_layer.shape[1], int(prev_off), slots.data_ptr(), cu_seqlens.data_ptr(),
             h.data_ptr(), raw.data_ptr(), out.data_ptr(), T, n_seqs, n_heads, dim, W, float(eps), _dt(r.dtype), _stream())
    return out


LATENT_MMA_ROWS = 64          # (token, head) rows of a CTA of the tensor-core kernel
LATENT_MMA_KEYS = 32          # cached rows per key tile
LATENT_MMA_COLS = 128         # output columns per warp; up to four such groups of warps per CTA
USE_LATENT_MMA = True


def latent_mma_ok(dtype: torch.dtype, row: int) -> bool:
    """The sizes the tensor-core latent attention takes (as its launcher checks them)."""
    return USE_LATENT_MMA and dtype == torch.bfloat16 and row % 16 == 0 and (LATENT_MMA_ROWS + 2 * LATENT_MMA_KEYS) * (row + 8) * 2 + 32 * 1024 <= 200 * 1024


def latent_attention_splits(n_tiles: int, n_heads: int, rank: int, span: int, row: "int | None" = None) -> int:
    """Into how many shares the tensor-core latent attention cuts the keys of every row tile: as many as fill the CTAs
    that are resident at once (its shared memory and threads allow one to a few per SM: whole rounds, since a second
    round of CTAs costs as much as the first), at least four key tiles per share, at most 16.  ``span``: the most keys
    a tile walks; ``row``: entries of a cached row (default: the latent and a rotated part of a quarter of it)."""
    ctas = max(1, n_tiles * -(-n_heads // LATENT_MMA_ROWS))      # the column groups of a wide latent are warps of one CTA
    groups = -(-rank // LATENT_MMA_COLS)
    row = row if row is not None else -(-(rank + rank // 4) // 16) * 16
    smem = (LATENT_MMA_ROWS + 2 * LATENT_MMA_KEYS) * (row + 8) * 2 + (4 * groups * 16 * 32 * 4 if groups > 1 else 0)
    resident = sm_count() * max(1, min(227 * 1024 // smem, 2048 // (128 * groups), 4))
    tiles = -(-span // LATENT_MMA_KEYS) + 1
    return int(max(1, min(resident // ctas, tiles // 4, 16)))


def latent_attention_mma(qa: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                         positions: torch.Tensor, n_tiles: int, rank: int, scale: float, window: "int | None", n_splits: int = 1,
                         max_len: int = 0, out: "torch.Tensor | None" = None) -> torch.Tensor:
    """bfloat16 attention of absorbed queries ``qa`` [T, nh, row] over latent rows on the tensor cores; ``n_tiles``:
    an upper bound of the row tiles (64 // min(nh, 64) tokens each) of the entries taken (``max_len`` > 0: those of
    at most that many tokens).  Returns [T, nh, rank]."""
    _check(qa, "qa", torch.bfloat16, 3)
    _check(cache_layer, "cache_layer", torch.bfloat16, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T, nh, row = qa.shape
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (1, 1, page_size, row) or row < rank or not latent_mma_ok(qa.dtype, row):
        raise UnsupportedSize(f"latent rows of {row} entries in {tuple(cache_layer.shape)}: the tensor-core kernel takes multiples of 16")
    n_seqs = cu_seqlens.shape[0] - 1
    if positions.shape[0] != T or block_table.shape[0] < n_seqs:
        raise ValueError("cu_seqlens, positions and block_table do not match the batch")
    if out is None:
        out = torch.empty((T, nh, rank), dtype=qa.dtype, device=qa.device)
    n_splits = int(n_splits)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((T, nh, n_splits, rank), dtype=torch.float32, device=qa.device)
        part_ml = torch.empty((T, nh, n_splits, 2), dtype=torch.float32, device=qa.device)
    lib.call("pyre_latent_attention_mma", qa.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), _ptr(part_o), _ptr(part_ml),
             block_table.data_ptr(), block_table.stride(0), cu_seqlens.data_ptr(), positions.data_ptr(), T, n_seqs, int(n_tiles), nh,
             int(rank), row, page_size, int(window or 0), float(scale), n_splits, int(max_len), cache_layer.shape[0],
             device_error_flag(qa.device).data_ptr(), _stream())
    return out


def latent_attention(ctx, qa: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, rank: int, rope: int,
                     scale: float, window: "int | None") -> torch.Tensor:
    """Attention of a whole step's absorbed queries over their sequences' latent rows; [T, nh, rank].  bfloat16 with
    rows of a multiple of 16 entries: the tensor-core kernel; everything else: the exact one."""
    T, nh, row = qa.shape
    if not latent_mma_ok(qa.dtype, row):
        return latent_attention_exact(qa, cache_layer, block_table, ctx.seq_of_token, ctx.positions, rank, rope, scale, window)
    tq = LATENT_MMA_ROWS // min(nh, LATENT_MMA_ROWS)
    lens = ctx.cu_seqlens_host[1:] - ctx.cu_seqlens_host[:-1]
    n_tiles = int((-(-lens // tq)).sum())
    span = ctx.max_context if not window else min(ctx.max_context, window + tq)
    return latent_attention_mma(qa, cache_layer, block_table, ctx.cu_seqlens, ctx.positions, n_tiles, rank, scale, window,
                                latent_attention_splits(n_tiles, nh, rank, span, row))


# ---------------------------------------------------------------------------------- short histories and recurrent states
def scale_cap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """x = scale * x, then cap * tanh(x / cap) where ``cap`` > 0; fp32, in place (a scaled embedding, rotary tables
    with an amplitude, logits with a factor and a soft cap)."""
    _check(x, "x", torch.float32)
    lib.call("pyre_scale_cap", x.data_ptr(), x.numel(), float(scale), float(cap), _stream())
    return x


def short_conv(inp: torch.Tensor, col: int, n_ch: int, weight: torch.Tensor, bias: "torch.Tensor | None", state_layer: torch.Tensor,
               state_off: int, slots: torch.Tensor, seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor, silu: bool = False,
               in_bias: "torch.Tensor | None" = None) -> torch.Tensor:
    """A short causal convolution over time per channel, continuing each request's history:
    y[t, c] = act(bias[c] + sum_j weight[c, j] u[t - taps + 1 + j, c]) with u the ``n_ch`` columns of ``inp`` from
    ``col``; the last tap is the token's own.  ``state_layer`` [slots, floats] fp32 holds, ``state_off`` floats into
    slot ``slots[b]``, entry b's last ``taps - 1`` inputs [taps - 1, n_ch] (oldest first; zeros when a request begins)
    and is left moved on by the step's tokens.  ``in_bias`` fp32 [n_ch]: added to every input as it is read from ``inp``
    (a projection's bias; the history holds inputs with it).  Returns [T, n_ch] in the dtype of ``inp``."""
    _check(inp, "inp", dim=2)
    _check(weight, "weight", torch.float32, 2)
    _check(state_layer, "state_layer", torch.float32, 2)
    _check(slots, "slots", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    T, W = inp.shape
    taps = weight.shape[1]
    n_seqs = cu_seqlens.shape[0] - 1
    if weight.shape[0] != n_ch or col < 0 or col + n_ch > W or taps < 1:
        raise ValueError("the convolution's channels do not lie inside the row, or its weight does not match them")
    if state_off < 0 or state_off + (taps - 1) * n_ch > state_layer.shape[1] or slots.shape[0] < n_seqs or seq_of_token.shape[0] < T:
        raise ValueError("the history does not lie inside the state slot, or slots do not match the batch")
    for v, name in ((bias, "bias"), (in_bias, "in_bias")):
        if v is not None:
            _check(v, name, torch.float32, 1)
            if v.shape[0] != n_ch:
                raise ValueError(f"{name}: one entry per channel")
    out = torch.empty((T, n_ch), dtype=inp.dtype, device=inp.device)
    lib.call("pyre_short_conv", inp.data_ptr(), W, int(col), _ptr(in_bias), weight.data_ptr(), _ptr(bias), state_layer.data_ptr(),
             state_layer.shape[1], int(state_off), slots.data_ptr(), seq_of_token.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(),
             T, n_seqs, int(n_ch), int(taps), int(bool(silu)), _dt(inp.dtype), _stream())
    return out


SSM_MAX_STATE = 256
SSM_WIDE_MEAN_LEN = 8      # steps that bring this many tokens per entry or more, on average, take the variant for prompt portions


def ssm_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state_layer: torch.Tensor, slots: torch.Tensor, cu_seqlens: torch.Tensor, n_heads: int, n_groups: int, p_dim: int,
             n_state: int, wide: "bool | None" = None) -> torch.Tensor:
    """The selective state-space recurrence over the step's entries, continuing each request's state.  Per head h of
    group h // (n_heads / n_groups), with x_t [p_dim], B_t and C_t [n_state] columns of ``xbc`` ([x: heads * p_dim |
    B: groups * n_state | C: groups * n_state]) and the raw step size column ``dt_col + h`` of ``proj``:
    dt = softplus(raw + dt_bias), S_t = exp(-exp(a_log) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + d_skip x_t.
    ``state_layer`` [slots, floats] fp32 holds S [heads, n_state, p_dim] at the start of slot ``slots[b]``.
    Token by token in fp32.  ``wide``: the kernel variant for prompt portions (a quarter of the rows per thread, four
    times the warps) instead of the one for single tokens (whole sectors of the state per warp); None: chosen by
    the mean number of tokens per entry (``SSM_WIDE_MEAN_LEN``).  With one variant results are bit-identical under
    any cutting; between the two the order of a column's partial sums differs.  Returns fp32 [T, heads * p_dim]."""
    _check(xbc, "xbc", dim=2)
    _check(proj, "proj", xbc.dtype, 2)
    _check(state_layer, "state_layer", torch.float32, 2)
    _check(slots, "slots", torch.int32, 1)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    T = xbc.shape[0]
    n_seqs = cu_seqlens.shape[0] - 1
    for v, name in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        _check(v, name, torch.float32, 1)
        if v.shape[0] != n_heads:
            raise ValueError(f"{name}: one entry per head")
    if n_state > SSM_MAX_STATE:
        raise UnsupportedSize(f"a state of {n_state} rows per head: the recurrence takes up to {SSM_MAX_STATE}")
    if n_heads % n_groups or xbc.shape[1] != n_heads * p_dim + 2 * n_groups * n_state or proj.shape[0] != T \
            or dt_col < 0 or dt_col + n_heads > proj.shape[1]:
        raise ValueError("x, B, C or the step sizes do not match the heads and groups")
    if n_heads * n_state * p_dim > state_layer.shape[1] or slots.shape[0] < n_seqs:
        raise ValueError("the state does not lie inside the slot, or slots do not match the batch")
    if wide is None:
        wide = T >= SSM_WIDE_MEAN_LEN * max(n_seqs, 1)
    y = torch.empty((T, n_heads * p_dim), dtype=torch.float32, device=xbc.device)
    lib.call("pyre_ssm_scan", xbc.data_ptr(), xbc.shape[1], proj.data_ptr(), proj.shape[1], int(dt_col), dt_bias.data_ptr(),
             a_log.data_ptr(), d_skip.data_ptr(), state_layer.data_ptr(), state_layer.shape[1], slots.data_ptr(),
             cu_seqlens.data_ptr(), y.data_ptr(), T, n_seqs, int(n_heads), int(n_groups), int(p_dim), int(n_state), int(bool(wide)),
             _dt(xbc.dtype), _stream())
    return y


GATE_ACTIVATIONS = {"silu": 1, "sigmoid": 2}


def group_norm_gate(y: torch.Tensor, groups: int, weight: "torch.Tensor | None", eps: float, proj: "torch.Tensor | None", g_col: int,
                    out_dtype: torch.dtype, gate: str = "silu", gate_first: bool = False, post: float = 1.0) -> torch.Tensor:
    """A unit norm over each of ``groups`` equal parts of the rows of fp32 ``y`` [T, W], times ``weight`` (fp32 [W] or
    None) and ``post``, with a gate act(proj[t, g_col:g_col + W]) (``gate`` silu or sigmoid; ``proj`` None: none) that
    multiplies ``y`` BEFORE the norm (``gate_first``) or its result.  Returns [T, W] in ``out_dtype``."""
    _check(y, "y", torch.float32, 2)
    T, W = y.shape
    if groups <= 0 or W % groups:
        raise ValueError(f"rows of {W} do not divide into {groups} equal parts")
    if weight is not None:
        _check(weight, "weight", torch.float32, 1)
        if weight.shape[0] != W:
            raise ValueError(f"norm weight has {weight.shape[0]} entries, rows have {W}")
    if gate not in GATE_ACTIVATIONS:
        raise UnsupportedSize(f"gate {gate!r}: implemented are {sorted(GATE_ACTIVATIONS)}")
    if proj is not None:
        _check(proj, "proj", out_dtype, 2)
        if proj.shape[0] != T or g_col < 0 or g_col + W > proj.shape[1]:
            raise ValueError("the gate does not lie inside the projection row")
    out = torch.empty((T, W), dtype=out_dtype, device=y.device)
    lib.call("pyre_group_norm_gate", y.data_ptr(), _ptr(proj), proj.shape[1] if proj is not None else 0,
             int(g_col) if proj is not None else -1, GATE_ACTIVATIONS[gate], int(bool(gate_first)), _ptr(weight), float(post),
             out.data_ptr(), T, W, int(groups), float(eps), _dt(out_dtype), _stream())
    return out


def diff_combine(a: torch.Tensor, a_dim: int, lam: float, post: float, n_heads: int, n_kv_heads: int, v_dim: int, eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values: o = a1 - lam * a2, then o / sqrt(mean(o^2) + eps) * post over
    the head's ``v_dim`` values.  ``a`` [T, 2 * n_heads * a_dim] holds the maps' sums grouped by key/value head: for
    head h = g * rep + r (rep = n_heads / n_kv_heads) map m is row (g * 2 + m) * rep + r of ``a_dim`` >= ``v_dim``
    columns.  Returns [T, n_heads * v_dim] in the heads' own order."""
    _check(a, "a", dim=2)
    T = a.shape[0]
    if n_heads % n_kv_heads or a.shape[1] != 2 * n_heads * a_dim or a_dim < v_dim:
        raise ValueError("the maps do not match the heads")
    out = torch.empty((T, n_heads * v_dim), dtype=a.dtype, device=a.device)
    lib.call("pyre_diff_combine", a.data_ptr(), int(a_dim), float(lam), float(post), out.data_ptr(), T, int(n_heads), int(n_kv_heads),
             int(v_dim), float(eps), _dt(a.dtype), _stream())
    return out


def rotate_heads(proj: torch.Tensor, col: int, n_heads: int, dim: int, cos: "torch.Tensor | None", sin: "torch.Tensor | None",
                 rotary_dim: int, factor: float = 1.0) -> torch.Tensor:
    """In place on ``proj`` [T, W]: the ``n_heads`` heads of ``dim`` columns from ``col`` turn their pairs
    (i, i + rotary_dim / 2) by the token's angle (cos, sin fp32 [T, rotary_dim / 2]) and are multiplied by ``factor``."""
    _check(proj, "proj", dim=2)
    T, W = proj.shape
    if col < 0 or col + n_heads * dim > W or rotary_dim % 2 or not 0 <= rotary_dim <= dim:
        raise ValueError("the heads do not lie inside the row, or the rotated dims do not fit a head")
    if rotary_dim:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, rotary_dim // 2) or tuple(sin.shape) != (T, rotary_dim // 2):
            raise ValueError(f"cos/sin must be [{T}, {rotary_dim // 2}]")
    lib.call("pyre_rotate_heads", proj.data_ptr(), W, int(col), _ptr(cos) if rotary_dim else None, _ptr(sin) if rotary_dim else None,
             T, int(n_heads), int(dim), int(rotary_dim), float(factor), _dt(proj.dtype), _stream())
    return proj


def side_gate(pre: torch.Tensor, table: torch.Tensor, col: int, token_ids: torch.Tensor, err_flag: "torch.Tensor | None" = None) -> torch.Tensor:
    """out[t, j] = gelu_tanh(pre[t, j]) * table[token_ids[t], col + j]: a token's slice of a side table, gated."""
    _check(pre, "pre", dim=2)
    _check(table, "table", pre.dtype, 2)
    _check(token_ids, "token_ids", torch.int32, 1)
    T, dim = pre.shape
    if token_ids.shape[0] != T or col < 0 or col + dim > table.shape[1]:
        raise ValueError("the slice does not lie inside the table's rows, or the ids do not match the tokens")
    out = torch.empty_like(pre)
    lib.call("pyre_side_gate", pre.data_ptr(), table.data_ptr(), table.shape[1], int(col), token_ids.data_ptr(), table.shape[0],
             out.data_ptr(), T, dim, _dt(pre.dtype), _ptr(err_flag), _stream())
    return out


def token_gate_add(acc: torch.Tensor, h: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """acc[t] += sigmoid(w . h[t]) * y[t] in place on fp32 ``acc`` [T, W]: a branch let in by one gate per token
    (``w`` fp32 [K], ``h`` [T, K] and ``y`` [T, W] activations)."""
    _check(acc, "acc", torch.float32, 2)
    _check(h, "h", dim=2)
    _check(y, "y", h.dtype, 2)
    _check(w, "w", torch.float32, 1)
    T, W = acc.shape
    if h.shape[0] != T or tuple(y.shape) != (T, W) or w.shape[0] != h.shape[1]:
        raise ValueError("acc, h, w and y do not match")
    lib.call("pyre_token_gate_add", acc.data_ptr(), h.data_ptr(), w.data_ptr(), y.data_ptr(), T, h.shape[1], W, _dt(h.dtype), _stream())
    return acc
