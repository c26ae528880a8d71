"""Typed model configurations, read from an architecture's own ``config.json`` keys.

``Qwen2Config`` holds exactly the keys that the reference's ``ModelConfig`` reads
(pyre/config.py:15-62): five required sizes and six defaulted values.  No size or
constant that ``config.json`` gives appears anywhere else in the package; parts get
them as constructor parameters from the architecture's builder.
"""

from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: names the key at fault."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations.

    A subclass lists its fields, names its architecture string and implements
    ``from_dict``; ``to_dict`` must write keys that ``from_dict`` reads back to an
    equal object, because the random-weights mode writes a model folder from it.
    """

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        out = dataclasses.asdict(self)
        out["architectures"] = [self.architecture]
        return out

    @classmethod
    def from_json(cls, path: str | Path) -> "ModelConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_json(self, path: str | Path) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=2) + "\n")


def _require(raw: dict[str, Any], key: str, kind=int):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    try:
        value = kind(raw[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: key {key!r} must be {kind.__name__}, got {raw[key]!r}") from None
    return value


def _positive(name: str, value: int) -> int:
    if value <= 0:
        raise ConfigError(f"config.json: {name} must be positive, got {value}")
    return value


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """The Qwen2.5 dense decoder as the reference computes it (pyre/model.py).

    Keys and defaults follow pyre/config.py:45-61: ``num_key_value_heads`` defaults
    to the number of heads, ``rms_norm_eps`` to 1e-6, ``rope_theta`` to 10000,
    ``tie_word_embeddings`` to False, ``max_position_embeddings`` to 32768 and
    ``head_dim`` to ``hidden_size // num_attention_heads`` (a null or zero
    ``head_dim`` falls back too, pyre/config.py:48).

    The reference silently ignores ``rope_scaling`` and the sliding-window keys; a
    checkpoint that switches them on would then be computed wrongly, so they are
    refused here with an error that names the key.
    """

    architecture: ClassVar[str] = "Qwen2ForCausalLM"

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    head_dim: int = 0

    def __post_init__(self):
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "vocab_size",
                     "max_position_embeddings"):
            _positive(name, getattr(self, name))
        if not self.head_dim:
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)
        _positive("head_dim", self.head_dim)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a "
                f"multiple of num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")

    @property
    def n_rep(self) -> int:
        """Query heads per key/value head (pyre/config.py:29-32)."""
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen2Config":
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is set; scaled rotary frequencies are not implemented")
        if raw.get("use_sliding_window"):
            raise ConfigError("config.json: use_sliding_window is true; this architecture is built without a window")
        hidden = _require(raw, "hidden_size")
        heads = _require(raw, "num_attention_heads")
        _positive("num_attention_heads", heads)
        return cls(
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size"),
            num_hidden_layers=_require(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(raw.get("num_key_value_heads") or heads),
            vocab_size=_require(raw, "vocab_size"),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            head_dim=int(raw.get("head_dim") or hidden // heads),
        )


@dataclass(frozen=True)
class ModovikLayer:
    """One layer of a Modovik model: ``kind`` "attention" (softmax attention with a sink over the paged cache) or
    "lightning" (linear attention with a decay per head over a state), the mixer's sizes, and the size of the
    dense feed-forward (0: the layer has none)."""

    kind: str
    heads: int
    dim: int                       # query/key entries per head
    vdim: int                      # value entries per head
    kv_heads: int = 0              # attention: key/value heads
    scale: float = 0.0             # attention: factor on q . k
    rot_dims: int = 0              # attention: leading dims of a head that are rotated
    rot_base: float = 10000.0
    kv_from: int = -1              # attention: the layer whose cached keys and values this one reads (-1: its own)
    decay: tuple = ()              # lightning: one constant per head
    ff: int = 0


@dataclass(frozen=True)
class ModovikConfig(ModelConfig):
    """A Modovik decoder: an embedding, layers in the order of ``layers`` whose norms sit on the branch outputs,
    a final norm and a head.  ``config.json`` keys: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list of
    ``{"type", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null}`` with the mixer's keys ``heads``, ``dim``,
    ``vdim`` and, for attention, ``kv_heads``, ``scale``, ``rot: {"dims", "base"}``, optionally ``kv_from``; for
    lightning, ``decay``."""

    architecture: ClassVar[str] = "Modovik"

    vocab: int
    width: int
    norm_eps: float
    layers: tuple

    def __post_init__(self):
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        for i, L in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            if L.kind not in ("attention", "lightning"):
                raise ConfigError(f"{where}.type {L.kind!r}: known are 'attention' and 'lightning'")
            for name in ("heads", "dim", "vdim"):
                if getattr(L, name) <= 0:
                    raise ConfigError(f"{where}.mixer.{name} must be positive")
            if L.ff < 0:
                raise ConfigError(f"{where}.mlp.ff must be positive")
            if L.kind == "lightning":
                if len(L.decay) != L.heads:
                    raise ConfigError(f"{where}.mixer.decay has {len(L.decay)} entries for {L.heads} heads")
                continue
            if L.kv_heads <= 0 or L.heads % L.kv_heads:
                raise ConfigError(f"{where}.mixer: heads ({L.heads}) must be a multiple of kv_heads ({L.kv_heads})")
            if L.rot_dims < 0 or L.rot_dims % 2 or L.rot_dims > L.dim:
                raise ConfigError(f"{where}.mixer.rot.dims ({L.rot_dims}) must be even and at most dim ({L.dim})")
            if L.rot_dims and not L.rot_base > 0:
                raise ConfigError(f"{where}.mixer.rot.base must be positive")
            if L.kv_from >= 0:
                src = self.layers[L.kv_from] if L.kv_from < len(self.layers) else None
                if src is None or L.kv_from >= i or src.kind != "attention" or src.kv_from >= 0:
                    raise ConfigError(f"{where}.mixer.kv_from ({L.kv_from}) must name an earlier attention layer with "
                                      f"keys and values of its own")
                if (src.kv_heads, src.dim, src.vdim, src.rot_dims, src.rot_base) != (L.kv_heads, L.dim, L.vdim, L.rot_dims, L.rot_base):
                    raise ConfigError(f"{where}.mixer: head sizes and rotation must equal those of layer {L.kv_from}, "
                                      f"whose keys and values it reads")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModovikConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: required key 'norm' (with 'eps') is missing")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)):
            raise ConfigError("config.json: required key 'layers' is missing")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and 'mixer'")
            m = entry["mixer"]
            kind = str(entry.get("type"))
            mlp = entry.get("mlp")
            ff = 0
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r}: only 'dense' is known")
                ff = _positive(f"{where}.mlp.ff", _require(mlp, "ff"))
            fields = dict(kind=kind, heads=_require(m, "heads"), dim=_require(m, "dim"), vdim=_require(m, "vdim"), ff=ff)
            if kind == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)):
                    raise ConfigError(f"config.json: {where}.mixer.decay is missing")
                fields["decay"] = tuple(float(d) for d in decay)
            elif kind == "attention":
                rot = m.get("rot") or {}
                fields.update(kv_heads=int(m.get("kv_heads") or fields["heads"]), scale=_require(m, "scale", float),
                              rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                              kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else -1)
            layers.append(ModovikLayer(**fields))
        return cls(vocab=_require(raw, "vocab"), width=_require(raw, "width"), norm_eps=_require(norm, "eps", float),
                   layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            if L.kind == "lightning":
                mixer = {"heads": L.heads, "dim": L.dim, "vdim": L.vdim, "decay": list(L.decay)}
            else:
                mixer = {"heads": L.heads, "kv_heads": L.kv_heads, "dim": L.dim, "vdim": L.vdim, "scale": L.scale,
                         "rot": {"dims": L.rot_dims, "base": L.rot_base}}
                if L.kv_from >= 0:
                    mixer["kv_from"] = L.kv_from
            layers.append({"type": L.kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": L.ff} if L.ff else None})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": layers}


@dataclass(frozen=True)
class PivinexLayer:
    """One layer of a Pivinex model: a latent-attention mixer (its sizes) and its feed-forward: ``mlp_kind`` "dense"
    (gated, ``ff`` wide), "moe" (``experts`` gated experts of ``ff`` plus ``identity`` router outputs without weights,
    ``top`` per token, weights scaled by ``router_scale``) or "" (none)."""

    kind: str
    heads: int
    dim: int                       # unrotated query/key entries per head
    rot_dim: int                   # rotated query/key entries per head (the key's are shared by the heads)
    vdim: int                      # value entries per head
    q_rank: int                    # size of the query latent
    kv_rank: int                   # size of the cached key/value latent
    scale: float                   # factor on q . k
    window: int = 0                # a position sees itself and window - 1 before it (0: all)
    rot_dims: int = 0              # leading entries of the rotated part that are rotated
    rot_base: float = 10000.0
    mlp_kind: str = ""
    ff: int = 0
    experts: int = 0
    identity: int = 0
    top: int = 0
    router_scale: float = 1.0


@dataclass(frozen=True)
class PivinexConfig(ModelConfig):
    """A Pivinex decoder: an embedding followed by a layer norm; layers that read ONE layer norm and add
    ``residual_mult`` times (mixer and feed-forward, each with a gain per feature) to the stream; a span of layers
    ``loop_start .. loop_stop - 1`` that runs ``loop_times`` times in a row with the same weights, each pass with a
    cache of its own, the embedding's output added to the stream before every pass but the first; a final layer norm
    and a head.  ``config.json`` keys: ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``loop: {start, stop,
    times}`` (optional) and ``layers``, a list of ``{"type": "latent_attention", "mixer": {heads, dim, rot_dim, vdim,
    q_rank, kv_rank, scale, mask: {size}, rot: {dims, base}}, "mlp": {"kind": "dense", "ff"} | {"kind": "moe", "expert":
    {"ff"}, "router": {experts, identity, top, scale}} | null}``."""

    architecture: ClassVar[str] = "Pivinex"

    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    def __post_init__(self):
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
            raise ConfigError(f"config.json: loop {{start: {self.loop_start}, stop: {self.loop_stop}, times: {self.loop_times}}} "
                              f"must name a span of the {len(self.layers)} layers and run it at least once")
        for i, L in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            if L.kind != "latent_attention":
                raise ConfigError(f"{where}.type {L.kind!r}: known is 'latent_attention'")
            for name in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                if getattr(L, name) <= 0:
                    raise ConfigError(f"{where}.mixer.{name} must be positive")
            if L.rot_dim < 0 or L.rot_dims < 0 or L.rot_dims % 2 or L.rot_dims > L.rot_dim:
                raise ConfigError(f"{where}.mixer.rot.dims ({L.rot_dims}) must be even and at most rot_dim ({L.rot_dim})")
            if L.rot_dims and not L.rot_base > 0:
                raise ConfigError(f"{where}.mixer.rot.base must be positive")
            if L.window < 0:
                raise ConfigError(f"{where}.mixer.mask.size must be positive")
            if L.mlp_kind not in ("", "dense", "moe"):
                raise ConfigError(f"{where}.mlp.kind {L.mlp_kind!r}: known are 'dense' and 'moe'")
            if L.mlp_kind and L.ff <= 0:
                raise ConfigError(f"{where}.mlp: ff must be positive")
            if L.mlp_kind == "moe" and (L.experts <= 0 or L.identity < 0 or not 0 < L.top <= L.experts + L.identity):
                raise ConfigError(f"{where}.mlp.router: {L.experts} experts + {L.identity} identity cannot give top {L.top}")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "PivinexConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: required key 'norm' (with 'eps') is missing")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)):
            raise ConfigError("config.json: required key 'layers' is missing")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and 'mixer'")
            m = entry["mixer"]
            rot = m.get("rot") or {}
            mask = m.get("mask") or {}
            rot_dim = int(m.get("rot_dim") or 0)
            fields = dict(kind=str(entry.get("type")), heads=_require(m, "heads"), dim=_require(m, "dim"), rot_dim=rot_dim,
                          vdim=_require(m, "vdim"), q_rank=_require(m, "q_rank"), kv_rank=_require(m, "kv_rank"),
                          scale=_require(m, "scale", float), window=int(mask.get("size") or 0),
                          rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)))
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                kind = str(mlp.get("kind", "dense"))
                fields["mlp_kind"] = kind
                if kind == "moe":
                    expert, router = mlp.get("expert"), mlp.get("router")
                    if not isinstance(expert, dict) or not isinstance(router, dict):
                        raise ConfigError(f"config.json: {where}.mlp needs 'expert' and 'router'")
                    fields.update(ff=_require(expert, "ff"), experts=_require(router, "experts"),
                                  identity=int(router.get("identity") or 0), top=_require(router, "top"),
                                  router_scale=float(router.get("scale", 1.0)))
                else:
                    fields["ff"] = _require(mlp, "ff")
            layers.append(PivinexLayer(**fields))
        loop = raw.get("loop") or {}
        start = int(loop.get("start", 0))
        return cls(vocab=_require(raw, "vocab"), width=_require(raw, "width"), norm_eps=_require(norm, "eps", float),
                   residual_mult=float(raw.get("residual_mult", 1.0)), layers=tuple(layers), loop_start=start,
                   loop_stop=int(loop.get("stop", start)), loop_times=int(loop.get("times", 1)))

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            mixer = {"heads": L.heads, "dim": L.dim, "rot_dim": L.rot_dim, "vdim": L.vdim, "q_rank": L.q_rank,
                     "kv_rank": L.kv_rank, "scale": L.scale, "rot": {"dims": L.rot_dims, "base": L.rot_base}}
            if L.window:
                mixer["mask"] = {"size": L.window}
            mlp = None
            if L.mlp_kind == "dense":
                mlp = {"kind": "dense", "ff": L.ff}
            elif L.mlp_kind == "moe":
                mlp = {"kind": "moe", "expert": {"ff": L.ff},
                       "router": {"experts": L.experts, "identity": L.identity, "top": L.top, "scale": L.router_scale}}
            layers.append({"type": L.kind, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult,
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}, "layers": layers}

    def layer_order(self) -> list:
        """(layer index, first layer of a repeated pass?) in the order the layers run."""
        order = [(i, False) for i in range(self.loop_start)]
        for rep in range(self.loop_times):
            order += [(i, rep > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, False) for i in range(self.loop_stop, len(self.layers))]


@dataclass(frozen=True)
class TekaraxLayer:
    """One layer of a Tekarax model: which mixer (``kind``: "attention", "wkv" or "latent_attention") with its sizes,
    and its feed-forward: ``mlp_kind`` "dense" (``ff`` wide, biases, squared relu), "moe" (``experts`` gated experts of
    ``ff``, ``top`` per token, plus a shared one of ``shared_ff`` when that is positive) or "" (none)."""

    kind: str
    heads: int
    dim: int                       # query/key entries per head (wkv: key and value entries per head)
    vdim: int = 0                  # value entries per head (attention, latent_attention)
    kv_heads: int = 0              # attention: key/value heads
    scale: float = 0.0             # factor on q . k
    rot_dims: int = 0              # attention: leading entries of a head that are rotated (0: no rotation at all)
    rot_base: float = 10000.0
    rot_scaling: "tuple | None" = None      # (factor, low, high, original) or None
    kv_rank: int = 0               # latent_attention: size of the cached latent
    window: int = 0                # latent_attention: a position sees itself and window - 1 before it (0: all)
    decay_rank: int = 0            # wkv: inner size of the decay's two-layer map (0: read from the tensor's shape)
    mlp_kind: str = ""
    ff: int = 0
    experts: int = 0
    top: int = 0
    shared_ff: int = 0


@dataclass(frozen=True)
class TekaraxConfig(ModelConfig):
    """A Tekarax decoder: layers with a layer norm before AND after each sublayer and a sigmoid gate per feature on the
    sublayer's result, x += norm_b(sublayer(norm(x)) * sigmoid(W norm(x) + b)); three kinds of mixer in any order; a
    span of layers ``loop_start .. loop_stop - 1`` that runs ``loop_times`` times in a row with the same weights, each
    pass with a cache or state of its own and a learned vector per pass added to the stream before it; a final layer
    norm and a head.  ``config.json`` keys: ``vocab``, ``width``, ``norm.eps``, ``loop: {start, stop, times}``
    (optional) and ``layers``, a list of ``{"type", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | {"kind": "moe",
    "expert": {"ff"}, "router": {experts, top}, "shared": {"ff"}} | null}`` with the mixers
    ``attention {heads, kv_heads, dim, vdim, scale, rot: {dims, base, scaling: {factor, low, high, original}}}``,
    ``wkv {heads, dim}`` and ``latent_attention {heads, dim, vdim, kv_rank, scale, mask: {size}}``.  A size that the
    file does not give (the inner size of a wkv layer's decay map) is read from the shape of the layer's tensor
    (``with_tensor_shapes``)."""

    architecture: ClassVar[str] = "Tekarax"
    KINDS: ClassVar[tuple] = ("attention", "wkv", "latent_attention")

    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    def __post_init__(self):
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
            raise ConfigError(f"config.json: loop {{start: {self.loop_start}, stop: {self.loop_stop}, times: {self.loop_times}}} "
                              f"must name a span of the {len(self.layers)} layers and run it at least once")
        for i, L in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            if L.kind not in self.KINDS:
                raise ConfigError(f"{where}.type {L.kind!r}: known are {', '.join(self.KINDS)}")
            if L.heads <= 0 or L.dim <= 0:
                raise ConfigError(f"{where}.mixer: heads and dim must be positive")
            if L.kind != "wkv" and (L.vdim <= 0 or not L.scale > 0):
                raise ConfigError(f"{where}.mixer: vdim and scale must be positive")
            if L.kind == "attention":
                if L.kv_heads <= 0 or L.heads % L.kv_heads:
                    raise ConfigError(f"{where}.mixer.kv_heads ({L.kv_heads}) must divide heads ({L.heads})")
                if L.rot_dims < 0 or L.rot_dims % 2 or L.rot_dims > L.dim:
                    raise ConfigError(f"{where}.mixer.rot.dims ({L.rot_dims}) must be even and at most dim ({L.dim})")
                if L.rot_dims and (not L.rot_base > 0 or L.vdim % 2):
                    raise ConfigError(f"{where}.mixer.rot: base must be positive and vdim even (the values are rotated too)")
            if L.kind == "latent_attention" and (L.kv_rank <= 0 or L.window < 0):
                raise ConfigError(f"{where}.mixer: kv_rank must be positive and mask.size not negative")
            if L.kind == "wkv" and L.decay_rank < 0:
                raise ConfigError(f"{where}.mixer.decay_rank must not be negative")
            if L.mlp_kind not in ("", "dense", "moe"):
                raise ConfigError(f"{where}.mlp.kind {L.mlp_kind!r}: known are 'dense' and 'moe'")
            if L.mlp_kind and L.ff <= 0:
                raise ConfigError(f"{where}.mlp: ff must be positive")
            if L.mlp_kind == "moe" and (L.experts <= 0 or not 0 < L.top <= L.experts or L.shared_ff < 0):
                raise ConfigError(f"{where}.mlp.router: {L.experts} experts cannot give top {L.top}")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "TekaraxConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: required key 'norm' (with 'eps') is missing")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)):
            raise ConfigError("config.json: required key 'layers' is missing")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and 'mixer'")
            m, kind = entry["mixer"], str(entry.get("type"))
            fields = dict(kind=kind, heads=_require(m, "heads"), dim=_require(m, "dim"))
            if kind == "attention":
                rot = m.get("rot") or {}
                sc = rot.get("scaling")
                if sc is not None:
                    if not isinstance(sc, dict):
                        raise ConfigError(f"config.json: {where}.mixer.rot.scaling must be an object or null")
                    sc = tuple(_require(sc, k, float) for k in ("factor", "low", "high", "original"))
                fields.update(vdim=int(m.get("vdim") or fields["dim"]), kv_heads=int(m.get("kv_heads") or fields["heads"]),
                              scale=_require(m, "scale", float), rot_dims=int(rot.get("dims", 0)),
                              rot_base=float(rot.get("base", 10000.0)), rot_scaling=sc)
            elif kind == "latent_attention":
                mask = m.get("mask") or {}
                fields.update(vdim=int(m.get("vdim") or fields["dim"]), kv_rank=_require(m, "kv_rank"),
                              scale=_require(m, "scale", float), window=int(mask.get("size") or 0))
            elif kind == "wkv":
                fields["decay_rank"] = int(m.get("decay_rank") or 0)
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                mk = str(mlp.get("kind", "dense"))
                fields["mlp_kind"] = mk
                if mk == "moe":
                    expert, router = mlp.get("expert"), mlp.get("router")
                    if not isinstance(expert, dict) or not isinstance(router, dict):
                        raise ConfigError(f"config.json: {where}.mlp needs 'expert' and 'router'")
                    shared = mlp.get("shared") or {}
                    fields.update(ff=_require(expert, "ff"), experts=_require(router, "experts"), top=_require(router, "top"),
                                  shared_ff=int(shared.get("ff") or 0))
                else:
                    fields["ff"] = _require(mlp, "ff")
            layers.append(TekaraxLayer(**fields))
        loop = raw.get("loop") or {}
        start = int(loop.get("start", 0))
        return cls(vocab=_require(raw, "vocab"), width=_require(raw, "width"), norm_eps=_require(norm, "eps", float),
                   layers=tuple(layers), loop_start=start, loop_stop=int(loop.get("stop", start)),
                   loop_times=int(loop.get("times", 1)))

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            if L.kind == "attention":
                mixer = {"heads": L.heads, "kv_heads": L.kv_heads, "dim": L.dim, "vdim": L.vdim, "scale": L.scale}
                if L.rot_dims:
                    mixer["rot"] = {"dims": L.rot_dims, "base": L.rot_base}
                    if L.rot_scaling:
                        mixer["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), L.rot_scaling))
            elif L.kind == "latent_attention":
                mixer = {"heads": L.heads, "dim": L.dim, "vdim": L.vdim, "kv_rank": L.kv_rank, "scale": L.scale}
                if L.window:
                    mixer["mask"] = {"size": L.window}
            else:
                mixer = {"heads": L.heads, "dim": L.dim}
                if L.decay_rank:
                    mixer["decay_rank"] = L.decay_rank
            mlp = None
            if L.mlp_kind == "dense":
                mlp = {"kind": "dense", "ff": L.ff}
            elif L.mlp_kind == "moe":
                mlp = {"kind": "moe", "expert": {"ff": L.ff}, "router": {"experts": L.experts, "top": L.top}}
                if L.shared_ff:
                    mlp["shared"] = {"ff": L.shared_ff}
            layers.append({"type": L.kind, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": layers}
        if self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    def layer_order(self) -> list:
        """(layer index, number of the pass that starts here or None) in the order the layers run."""
        if not self.has_loop():
            return [(i, None) for i in range(len(self.layers))]
        order = [(i, None) for i in range(self.loop_start)]
        for rep in range(self.loop_times):
            order += [(i, rep if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, None) for i in range(self.loop_stop, len(self.layers))]

    def needs_tensor_shapes(self) -> bool:
        return any(L.kind == "wkv" and not L.decay_rank for L in self.layers)

    def with_tensor_shapes(self, shape_of) -> "TekaraxConfig":
        """The configuration with the sizes that only the weights give filled in; ``shape_of(name)`` returns the
        shape of a checkpoint tensor (or None)."""
        layers = []
        for i, L in enumerate(self.layers):
            if L.kind == "wkv" and not L.decay_rank:
                shape = shape_of(f"l{i}.mix.w1")
                if shape is None or len(shape) != 2:
                    raise ConfigError(f"config.json: layers[{i}] gives no decay_rank and the weights hold no l{i}.mix.w1 to read it from")
                L = dataclasses.replace(L, decay_rank=int(shape[0]))
            layers.append(L)
        return dataclasses.replace(self, layers=tuple(layers))


@dataclass(frozen=True)
class NipudraLayer:
    """One layer of a Nipudra model: which mixer (``kind``: "attention", "mamba2" or "retention") with its sizes, and
    its feed-forward: ``mlp_kind`` "moe" (``experts`` experts of ``ff``, ``top`` per token, plus a shared one of
    ``shared_ff`` when that is positive) or "" (none)."""

    kind: str
    heads: int
    vdim: int                      # value entries per head (mamba2: entries of x per head)
    dim: int = 0                   # query/key entries per head and map (attention, retention)
    kv_heads: int = 0              # attention: key/value heads
    scale: float = 0.0             # attention: factor on q . k
    diff: float = 0.0              # attention: the constant of lambda and of the heads' final factor 1 - diff
    window: int = 0                # attention: a position sees itself and window - 1 before it (0: all)
    kv_from: int = -1              # attention: the layer whose cached keys and values this one reads (-1: its own)
    conv: int = 0                  # attention, mamba2: taps of the short convolution (attention: 0 = none)
    rot_dims: int = 0              # attention, retention: leading entries of a head that are rotated
    rot_base: float = 10000.0
    rot_scaling: "tuple | None" = None      # attention: (factor, original, fast, slow) or None
    decay: tuple = ()              # retention: one decay per head
    state: int = 0                 # mamba2: rows of a head's state
    groups: int = 0                # mamba2: groups that share B and C
    norm_groups: int = 0           # mamba2: equal parts of the gated row, each with its own unit norm
    mlp_kind: str = ""
    ff: int = 0
    experts: int = 0
    top: int = 0
    shared_ff: int = 0


@dataclass(frozen=True)
class NipudraConfig(ModelConfig):
    """A Nipudra decoder: a scaled embedding; layers with a layer norm (gain and bias) before AND after each sublayer,
    x += norm_b(sublayer(norm(x))); three kinds of mixer in any order (differential softmax attention over a sliding
    window with short convolutions on q, k and v; a selective state-space recurrence; retention with a constant decay
    per head); a routed feed-forward or none; a per-layer input from the token's row of a side table; a final layer
    norm and a head tied to the embedding whose logits are scaled and soft-capped.  ``config.json`` keys: ``vocab``,
    ``width``, ``norm.eps``, ``embedding.scale``, ``logit_scale``, ``logit_softcap``, ``token_side.dim`` and ``layers``,
    a list of ``{"type", "mixer": {...}, "mlp": {"kind": "moe", "expert": {"ff"}, "router": {experts, top}, "shared":
    {"ff"}} | null}`` with the mixers ``attention {heads, kv_heads, dim, vdim, scale, diff, conv, mask: {size}, kv_from,
    rot: {dims, base, scaling: {factor, original, fast, slow}}}``, ``mamba2 {heads, vdim, state, groups, conv,
    norm_groups}`` and ``retention {heads, dim, vdim, decay: [...], rot: {dims, base}}``.  The taps of a convolution
    that the file leaves out are read from the shape of the layer's tensor (``with_tensor_shapes``)."""

    architecture: ClassVar[str] = "Nipudra"
    KINDS: ClassVar[tuple] = ("attention", "mamba2", "retention")

    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    side_dim: int = 0

    def __post_init__(self):
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        if self.side_dim < 0 or self.logit_softcap < 0 or not self.logit_scale > 0:
            raise ConfigError("config.json: token_side.dim and logit_softcap must not be negative, logit_scale positive")
        for i, L in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            if L.kind not in self.KINDS:
                raise ConfigError(f"{where}.type {L.kind!r}: known are {', '.join(self.KINDS)}")
            if L.heads <= 0 or L.vdim <= 0:
                raise ConfigError(f"{where}.mixer: heads and vdim must be positive")
            if L.kind in ("attention", "retention"):
                if L.dim <= 0:
                    raise ConfigError(f"{where}.mixer.dim must be positive")
                if L.rot_dims < 0 or L.rot_dims % 2 or L.rot_dims > L.dim or (L.rot_dims and not L.rot_base > 1):
                    raise ConfigError(f"{where}.mixer.rot: dims ({L.rot_dims}) must be even and at most dim ({L.dim}), base above 1")
            if L.kind == "attention":
                if L.kv_heads <= 0 or L.heads % L.kv_heads:
                    raise ConfigError(f"{where}.mixer.kv_heads ({L.kv_heads}) must divide heads ({L.heads})")
                if not L.scale > 0 or L.window < 0 or L.conv < 0 or L.conv == 1:
                    raise ConfigError(f"{where}.mixer: scale must be positive, mask.size not negative, conv 0 or at least 2")
                if L.kv_from >= 0:
                    src = self.layers[L.kv_from] if L.kv_from < i else None
                    if src is None or src.kind != "attention" or src.kv_from >= 0:
                        raise ConfigError(f"{where}.mixer.kv_from ({L.kv_from}) must name an earlier attention layer with keys and values of its own")
                    if (src.kv_heads, src.dim, src.vdim, src.rot_dims, src.rot_base, src.rot_scaling) != \
                            (L.kv_heads, L.dim, L.vdim, L.rot_dims, L.rot_base, L.rot_scaling):
                        raise ConfigError(f"{where}.mixer: head sizes and rotation must equal those of layer {L.kv_from}, whose keys and values it reads")
            if L.kind == "retention" and len(L.decay) != L.heads:
                raise ConfigError(f"{where}.mixer.decay: {len(L.decay)} decays for {L.heads} heads")
            if L.kind == "mamba2":
                if L.state <= 0 or L.groups <= 0 or L.heads % L.groups or L.norm_groups <= 0 or (L.heads * L.vdim) % L.norm_groups:
                    raise ConfigError(f"{where}.mixer: state, groups and norm_groups must be positive, groups divide heads and "
                                      f"norm_groups divide heads * vdim")
                if L.conv < 0 or L.conv == 1:
                    raise ConfigError(f"{where}.mixer.conv must be at least 2")
            if L.mlp_kind not in ("", "moe"):
                raise ConfigError(f"{where}.mlp.kind {L.mlp_kind!r}: known is 'moe'")
            if L.mlp_kind == "moe" and (L.ff <= 0 or L.experts <= 0 or not 0 < L.top <= L.experts or L.shared_ff < 0):
                raise ConfigError(f"{where}.mlp: ff must be positive and {L.experts} experts cannot give top {L.top}")

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "NipudraConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: required key 'norm' (with 'eps') is missing")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)):
            raise ConfigError("config.json: required key 'layers' is missing")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and 'mixer'")
            m, kind = entry["mixer"], str(entry.get("type"))
            fields = dict(kind=kind, heads=_require(m, "heads"), vdim=_require(m, "vdim"))
            rot = m.get("rot") or {}
            if kind in ("attention", "retention"):
                fields.update(dim=_require(m, "dim"), rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)))
            if kind == "attention":
                sc = rot.get("scaling")
                if sc is not None:
                    if not isinstance(sc, dict):
                        raise ConfigError(f"config.json: {where}.mixer.rot.scaling must be an object or null")
                    sc = tuple(_require(sc, k, float) for k in ("factor", "original", "fast", "slow"))
                mask = m.get("mask") or {}
                kv_from = m.get("kv_from")
                fields.update(kv_heads=int(m.get("kv_heads") or fields["heads"]), scale=_require(m, "scale", float),
                              diff=_require(m, "diff", float), window=int(mask.get("size") or 0),
                              kv_from=-1 if kv_from is None else int(kv_from), conv=int(m.get("conv") or 0), rot_scaling=sc)
            elif kind == "retention":
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)):
                    raise ConfigError(f"config.json: {where}.mixer.decay must be a list with one decay per head")
                fields["decay"] = tuple(float(d) for d in decay)
            elif kind == "mamba2":
                fields.update(state=_require(m, "state"), groups=int(m.get("groups") or 1), conv=int(m.get("conv") or 0),
                              norm_groups=int(m.get("norm_groups") or 1))
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                fields["mlp_kind"] = str(mlp.get("kind", "moe"))
                expert, router = mlp.get("expert"), mlp.get("router")
                if not isinstance(expert, dict) or not isinstance(router, dict):
                    raise ConfigError(f"config.json: {where}.mlp needs 'expert' and 'router'")
                shared = mlp.get("shared") or {}
                fields.update(ff=_require(expert, "ff"), experts=_require(router, "experts"), top=_require(router, "top"),
                              shared_ff=int(shared.get("ff") or 0))
            layers.append(NipudraLayer(**fields))
        emb, side = raw.get("embedding") or {}, raw.get("token_side") or {}
        return cls(vocab=_require(raw, "vocab"), width=_require(raw, "width"), norm_eps=_require(norm, "eps", float),
                   layers=tuple(layers), embedding_scale=float(emb.get("scale", 1.0)), logit_scale=float(raw.get("logit_scale") or 1.0),
                   logit_softcap=float(raw.get("logit_softcap") or 0.0), side_dim=int(side.get("dim") or 0))

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            rot = {"dims": L.rot_dims, "base": L.rot_base} if L.rot_dims else None
            if L.kind == "attention":
                mixer = {"heads": L.heads, "kv_heads": L.kv_heads, "dim": L.dim, "vdim": L.vdim, "scale": L.scale, "diff": L.diff}
                if L.conv:
                    mixer["conv"] = L.conv
                if L.window:
                    mixer["mask"] = {"size": L.window}
                if L.kv_from >= 0:
                    mixer["kv_from"] = L.kv_from
                if rot:
                    if L.rot_scaling:
                        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), L.rot_scaling))
                    mixer["rot"] = rot
            elif L.kind == "retention":
                mixer = {"heads": L.heads, "dim": L.dim, "vdim": L.vdim, "decay": list(L.decay)}
                if rot:
                    mixer["rot"] = rot
            else:
                mixer = {"heads": L.heads, "vdim": L.vdim, "state": L.state, "groups": L.groups, "conv": L.conv,
                         "norm_groups": L.norm_groups}
            mlp = None
            if L.mlp_kind == "moe":
                mlp = {"kind": "moe", "expert": {"ff": L.ff}, "router": {"experts": L.experts, "top": L.top}}
                if L.shared_ff:
                    mlp["shared"] = {"ff": L.shared_ff}
            layers.append({"type": L.kind, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "layers": layers}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out

    def needs_tensor_shapes(self) -> bool:
        return any(L.kind == "mamba2" and not L.conv for L in self.layers)

    def with_tensor_shapes(self, shape_of) -> "NipudraConfig":
        """The configuration with the sizes that only the weights give filled in; ``shape_of(name)`` returns the
        shape of a checkpoint tensor (or None)."""
        layers = []
        for i, L in enumerate(self.layers):
            if L.kind == "mamba2" and not L.conv:
                shape = shape_of(f"l{i}.mix.conv")
                if shape is None or len(shape) != 2:
                    raise ConfigError(f"config.json: layers[{i}] gives no conv and the weights hold no l{i}.mix.conv to read it from")
                L = dataclasses.replace(L, conv=int(shape[1]))
            layers.append(L)
        return dataclasses.replace(self, layers=tuple(layers))
