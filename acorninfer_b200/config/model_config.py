"""Typed model configurations, read from an architecture's own ``config.json`` keys.

Every size and constant of a model comes from here; nothing downstream carries a
default for a size.  A configuration class knows two things: how to read itself
from the raw ``config.json`` dictionary (``from_dict``) and how to write itself
back (``to_dict``), so that the random-weights mode can produce a model folder.

Reference behaviour: ``acorninfer/config.py:16-48`` reads twelve required keys with
``raw[...]`` and ignores every other key.  Here a missing key is an error that names
the key, and keys that would change the computation but are not implemented
(``attention_bias``, ``rope_scaling``, an active sliding window) are refused instead
of being ignored.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import ClassVar


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a model: names the key at fault."""


_MISSING = object()


def _take(raw: dict, key: str, kind, default=_MISSING):
    """Read ``raw[key]`` as ``kind``; a missing key without default is a ConfigError."""
    if key not in raw or raw[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    value = raw[key]
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config.json: key '{key}' must be true/false, got {value!r}")
        return value
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: key '{key}' must be an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: key '{key}' must be a number, got {value!r}")
        return float(value)
    return value


@dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations.

    ``architecture`` is the name under which the model is registered
    (``config.json``'s ``architectures[0]``).
    """

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:
        out = {"architectures": [self.architecture]}
        out.update(asdict(self))
        return out


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder: GQA attention with per-head q/k RMSNorm, half-rotate
    RoPE, SwiGLU feed-forward, pre-norm residual blocks, optionally tied output head.

    Keys as in ``acorninfer/config.py:33-48``.  ``head_dim`` may be absent (then
    ``hidden_size / num_attention_heads``), ``tie_word_embeddings`` defaults to
    false, ``bos_token_id``/``eos_token_id`` are optional and only stored.
    """

    architecture: ClassVar[str] = "Qwen3ForCausalLM"

    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    vocab_size: int
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        for f in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"):
            if getattr(self, f) < 1:
                raise ConfigError(f"config.json: '{f}' must be >= 1, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "config.json: 'num_attention_heads' "
                f"({self.num_attention_heads}) must be a multiple of 'num_key_value_heads' "
                f"({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' must be even for rotary pairs, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"config.json: 'rms_norm_eps' must be > 0, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"config.json: 'rope_theta' must be > 0, got {self.rope_theta}")

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        n_heads = _take(raw, "num_attention_heads", int)
        hidden = _take(raw, "hidden_size", int)
        if "head_dim" in raw and raw["head_dim"] is not None:
            head_dim = _take(raw, "head_dim", int)
        else:
            if hidden % n_heads != 0:
                raise ConfigError(
                    "config.json: 'head_dim' is absent and 'hidden_size' is not a multiple of "
                    "'num_attention_heads'")
            head_dim = hidden // n_heads
        # Keys that change the computation and are not implemented are refused.
        if _take(raw, "attention_bias", bool, False):
            raise ConfigError("config.json: 'attention_bias' = true is not supported by Qwen3ForCausalLM here")
        if raw.get("rope_scaling") is not None:
            raise ConfigError("config.json: 'rope_scaling' is not supported (only plain RoPE)")
        if _take(raw, "use_sliding_window", bool, False):
            raise ConfigError("config.json: 'use_sliding_window' = true is not supported for Qwen3ForCausalLM")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu', got {act!r}")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        bos = raw.get("bos_token_id")
        return cls(
            num_hidden_layers=_take(raw, "num_hidden_layers", int),
            hidden_size=hidden,
            num_attention_heads=n_heads,
            num_key_value_heads=_take(raw, "num_key_value_heads", int),
            head_dim=head_dim,
            intermediate_size=_take(raw, "intermediate_size", int),
            rms_norm_eps=_take(raw, "rms_norm_eps", float),
            rope_theta=_take(raw, "rope_theta", float),
            vocab_size=_take(raw, "vocab_size", int),
            tie_word_embeddings=_take(raw, "tie_word_embeddings", bool, False),
            bos_token_id=None if bos is None else int(bos),
            eos_token_id=eos_ids,
        )

    def to_dict(self) -> dict:
        out = super().to_dict()
        out["eos_token_id"] = list(self.eos_token_id)
        out["hidden_act"] = "silu"
        out["attention_bias"] = False
        out["model_type"] = "qwen3"
        return out


# --------------------------------------------------------------------------- Kogonex


def _sub(raw: dict, key: str, where: str, required: bool = True):
    """``raw[key]`` as a JSON object (None if absent and not required)."""
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: {where}'{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class RotaryScaling:
    """Frequency scaling of rotary positions for contexts beyond the trained one: pairs that turn
    more than ``fast`` times over ``original`` positions keep their frequency, pairs that turn less
    than ``slow`` times are slowed by ``factor``, a linear ramp between."""

    factor: float
    original: int
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentAttentionConfig:
    """Attention whose keys and values are up-projections of one cached latent per token."""

    kind: ClassVar[str] = "latent_attention"
    heads: int
    dim: int                     # unrotated query/key entries per head
    rot_dim: int                 # rotated entries per head; the rotated key part is shared by all heads
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int                # entries of the rotated part that are really rotated
    rot_base: float
    scaling: RotaryScaling | None = None
    window: int | None = None    # a query sees itself and the window - 1 tokens before it
    kv_from: int | None = None   # layer whose cached latent and key part this layer reads
    q_rank: int | None = None    # size of a latent the queries come through (None: projected directly)

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "LatentAttentionConfig":
        rot = _sub(m, "rot", where)
        sc = _sub(rot, "scaling", where + "rot.", required=False)
        mask = _sub(m, "mask", where, required=False)
        return cls(
            heads=_take(m, "heads", int), dim=_take(m, "dim", int), rot_dim=_take(m, "rot_dim", int),
            vdim=_take(m, "vdim", int), kv_rank=_take(m, "kv_rank", int), scale=_take(m, "scale", float),
            rot_dims=_take(rot, "dims", int), rot_base=_take(rot, "base", float),
            scaling=None if sc is None else RotaryScaling(_take(sc, "factor", float), _take(sc, "original", int),
                                                          _take(sc, "fast", float), _take(sc, "slow", float)),
            window=None if mask is None else _take(mask, "size", int),
            kv_from=_take(m, "kv_from", int, None), q_rank=_take(m, "q_rank", int, None))

    def to_dict(self) -> dict:
        rot: dict = {"base": self.rot_base, "dims": self.rot_dims}
        if self.scaling is not None:
            rot["scaling"] = asdict(self.scaling)
        out: dict = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot": rot, "rot_dim": self.rot_dim,
                     "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        if self.q_rank is not None:
            out["q_rank"] = self.q_rank
        return out


@dataclass(frozen=True)
class ChannelDeltaConfig:
    """Gated delta rule with a decay per key channel and short convolutions on q, k, v."""

    kind: ClassVar[str] = "channel_delta"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    # Inner sizes of the decay's and the gate's low-rank projections.  A checkpoint's tensors fix them;
    # they are needed (and written as "decay_rank" / "gate_rank") only to make a model from nothing.
    decay_rank: int | None = None
    gate_rank: int | None = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "ChannelDeltaConfig":
        return cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                   vdim=_take(m, "vdim", int), conv=_take(m, "conv", int),
                   decay_rank=_take(m, "decay_rank", int, None), gate_rank=_take(m, "gate_rank", int, None))

    def to_dict(self) -> dict:
        out = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            out["gate_rank"] = self.gate_rank
        return out


@dataclass(frozen=True)
class RoutedExpertsConfig:
    """A routed mixture of small SwiGLU experts; the last ``identity`` router outputs return their input."""

    ff: int
    experts: int
    identity: int
    top: int
    groups: int = 1
    keep: int = 1

    @classmethod
    def from_dict(cls, f: dict, where: str) -> "RoutedExpertsConfig":
        kind = f.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"config.json: {where}'kind' must be 'moe', got {kind!r}")
        r = _sub(f, "router", where)
        g = _sub(r, "groups", where + "router.", required=False)
        return cls(ff=_take(_sub(f, "expert", where), "ff", int), experts=_take(r, "experts", int),
                   identity=_take(r, "identity", int, 0), top=_take(r, "top", int),
                   groups=1 if g is None else _take(g, "count", int), keep=1 if g is None else _take(g, "keep", int))

    def to_dict(self) -> dict:
        return {"expert": {"ff": self.ff}, "kind": "moe",
                "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep},
                           "identity": self.identity, "top": self.top}}


_KOGONEX_MIXERS = {c.kind: c for c in (LatentAttentionConfig, ChannelDeltaConfig)}


@dataclass(frozen=True)
class KogonexLayer:
    mixer: LatentAttentionConfig | ChannelDeltaConfig
    mlp: RoutedExpertsConfig | None


@dataclass(frozen=True)
class KogonexConfig(ModelConfig):
    """Kogonex: a token table plus hashed bigram rows; layers that add the RMS norm of each
    sublayer's output to the stream (``x += norm(mixer(x))``, ``x += norm(ff(x))``), with a mixer that
    is either attention through a cached latent (sliding window, sink, scaled rotary positions,
    optionally reading an earlier layer's cache) or a gated delta rule, and routed experts as
    feed-forward (or none); a final norm and an output matrix.  ``config.json`` lists the layers
    in order, each with its own sizes."""

    architecture: ClassVar[str] = "Kogonex"

    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[KogonexLayer, ...]
    bigram_buckets: int | None = None
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' must be >= 1 and 'layers' non-empty")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm 'eps' must be > 0, got {self.norm_eps}")
        if self.bigram_buckets is not None and self.bigram_buckets < 1:
            raise ConfigError("config.json: bigram 'buckets' must be >= 1")
        for i, layer in enumerate(self.layers):
            m, w = layer.mixer, f"layers[{i}].mixer."
            if isinstance(m, LatentAttentionConfig):
                if min(m.heads, m.dim, m.vdim, m.kv_rank) < 1 or m.rot_dim < 0:
                    raise ConfigError(f"config.json: {w}sizes must be >= 1")
                if m.rot_dims % 2 or not (0 <= m.rot_dims <= m.rot_dim):
                    raise ConfigError(f"config.json: {w}rot.dims must be even and at most rot_dim, got {m.rot_dims}")
                if m.window is not None and m.window < 1:
                    raise ConfigError(f"config.json: {w}mask.size must be >= 1, got {m.window}")
                if m.kv_from is not None:
                    src = self.layers[m.kv_from].mixer if 0 <= m.kv_from < i else None
                    if not isinstance(src, LatentAttentionConfig) or src.kv_from is not None:
                        raise ConfigError(f"config.json: {w}kv_from must name an earlier latent_attention layer "
                                          "that keeps its own cache")
                    if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base, src.scaling) != \
                            (m.kv_rank, m.rot_dim, m.rot_dims, m.rot_base, m.scaling):
                        raise ConfigError(f"config.json: {w}kv_rank, rot_dim and rot must equal those of layer {m.kv_from}")
            else:
                if min(m.heads, m.kv_heads, m.dim, m.vdim, m.conv) < 1 or m.heads % m.kv_heads:
                    raise ConfigError(f"config.json: {w}sizes must be >= 1 and 'heads' a multiple of 'kv_heads'")
            f = layer.mlp
            if f is not None:
                n = f.experts + f.identity
                if min(f.ff, f.top, f.groups, f.keep) < 1 or f.experts < 0 or f.identity < 0 or n < 1:
                    raise ConfigError(f"config.json: layers[{i}].mlp sizes must be positive")
                if n % f.groups or f.keep > f.groups or f.top > f.keep * (n // f.groups):
                    raise ConfigError(f"config.json: layers[{i}].mlp: {n} router outputs do not split into {f.groups} groups "
                                      f"of which {f.keep} hold {f.top} choices")

    @classmethod
    def from_dict(cls, raw: dict) -> "KogonexConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = lr.get("type") if isinstance(lr, dict) else None
            if kind not in _KOGONEX_MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {sorted(_KOGONEX_MIXERS)}, got {kind!r}")
            mixer = _KOGONEX_MIXERS[kind].from_dict(_sub(lr, "mixer", where), where + "mixer.")
            mlp = _sub(lr, "mlp", where, required=False)
            layers.append(KogonexLayer(mixer, None if mlp is None else RoutedExpertsConfig.from_dict(mlp, where + "mlp.")))
        emb = _sub(raw, "embedding", "", required=False) or {}
        big = _sub(emb, "bigram", "embedding.", required=False)
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab_size=_take(raw, "vocab", int), hidden_size=_take(raw, "width", int),
                   norm_eps=_take(_sub(raw, "norm", ""), "eps", float), layers=tuple(layers),
                   bigram_buckets=None if big is None else _take(big, "buckets", int),
                   bigram_mul_prev=0 if big is None else _take(big, "mul_prev", int),
                   bigram_mul_cur=0 if big is None else _take(big, "mul_cur", int), eos_token_id=eos_ids)

    def to_dict(self) -> dict:
        out: dict = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                     "norm": {"eps": self.norm_eps}}
        if self.bigram_buckets is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram_buckets, "mul_cur": self.bigram_mul_cur,
                                           "mul_prev": self.bigram_mul_prev}}
        out["layers"] = [{"type": l.mixer.kind, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                         for l in self.layers]
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out


# --------------------------------------------------------------------------- Vagulorn


@dataclass(frozen=True)
class MaskedAttentionConfig:
    """Grouped-query attention with q/k norm and rotary positions on the first ``rot_dims`` entries of a head.
    ``mask_size`` None: every earlier key is read; else the rule its place in the model gives it (blocks of
    positions for a layer of its own, a window with ``keep_first`` kept keys beside a recurrent mixer)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int = 0
    rot_base: float = 10000.0
    mask_size: int | None = None
    keep_first: int = 0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "MaskedAttentionConfig":
        rot = _sub(m, "rot", where, required=False)
        mask = _sub(m, "mask", where, required=False)
        return cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                   vdim=_take(m, "vdim", int), scale=_take(m, "scale", float),
                   rot_dims=0 if rot is None else _take(rot, "dims", int),
                   rot_base=10000.0 if rot is None else _take(rot, "base", float),
                   mask_size=None if mask is None else _take(mask, "size", int, None),
                   keep_first=0 if mask is None else _take(mask, "keep_first", int, 0))

    def check(self, where: str) -> None:
        if min(self.heads, self.kv_heads, self.dim, self.vdim) < 1 or self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}sizes must be >= 1 and 'heads' a multiple of 'kv_heads'")
        if self.rot_dims % 2 or not (0 <= self.rot_dims <= self.dim):
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, got {self.rot_dims}")
        if self.rot_dims and not self.rot_base > 0:
            raise ConfigError(f"config.json: {where}rot.base must be > 0, got {self.rot_base}")
        if self.mask_size is not None and self.mask_size < 1:
            raise ConfigError(f"config.json: {where}mask.size must be >= 1, got {self.mask_size}")
        if self.keep_first < 0:
            raise ConfigError(f"config.json: {where}mask.keep_first must be >= 0, got {self.keep_first}")

    def to_dict(self) -> dict:
        out: dict = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.mask_size is not None:
            out["mask"] = {"size": self.mask_size}
            if self.keep_first:
                out["mask"]["keep_first"] = self.keep_first
        return out


@dataclass(frozen=True)
class DecayLinearAttentionConfig:
    """Linear attention with one fixed decay per head."""

    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "DecayLinearAttentionConfig":
        decay = m.get("decay")
        if not isinstance(decay, list) or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            raise ConfigError(f"config.json: {where}'decay' must be a list of numbers, one per head")
        return cls(heads=_take(m, "heads", int), dim=_take(m, "dim", int), vdim=_take(m, "vdim", int),
                   decay=tuple(float(d) for d in decay))

    def check(self, where: str) -> None:
        if min(self.heads, self.dim, self.vdim) < 1 or len(self.decay) != self.heads:
            raise ConfigError(f"config.json: {where}sizes must be >= 1 and 'decay' hold one number per head")

    def to_dict(self) -> dict:
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class SideBySideConfig:
    """Attention (left) and linear attention (right) on the same input, their results scaled and added."""

    left: MaskedAttentionConfig
    right: DecayLinearAttentionConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "SideBySideConfig":
        return cls(left=MaskedAttentionConfig.from_dict(_sub(m, "left", where), where + "left."),
                   right=DecayLinearAttentionConfig.from_dict(_sub(m, "right", where), where + "right."),
                   left_scale=_take(m, "left_scale", float), right_scale=_take(m, "right_scale", float))

    def check(self, where: str) -> None:
        self.left.check(where + "left.")
        self.right.check(where + "right.")
        if self.left.vdim != self.left.dim:
            raise ConfigError(f"config.json: {where}left.vdim must equal left.dim (the values are the keys)")

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class StateSpaceConfig:
    """A selective state space layer (state-space duality form)."""

    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "StateSpaceConfig":
        return cls(heads=_take(m, "heads", int), vdim=_take(m, "vdim", int), state=_take(m, "state", int),
                   groups=_take(m, "groups", int), conv=_take(m, "conv", int), norm_groups=_take(m, "norm_groups", int))

    def check(self, where: str) -> None:
        if min(self.heads, self.vdim, self.state, self.groups, self.conv, self.norm_groups) < 1:
            raise ConfigError(f"config.json: {where}sizes must be >= 1")
        if self.heads % self.groups or (self.heads * self.vdim) % self.norm_groups:
            raise ConfigError(f"config.json: {where}'groups' must divide 'heads' and 'norm_groups' must divide heads * vdim")

    def to_dict(self) -> dict:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


_VAGULORN_MIXERS = {"attention": MaskedAttentionConfig, "parallel": SideBySideConfig, "mamba2": StateSpaceConfig}


@dataclass(frozen=True)
class VagulornLayer:
    type: str                   # "attention", "parallel" or "mamba2"
    mixer: MaskedAttentionConfig | SideBySideConfig | StateSpaceConfig
    ff: int | None              # inner width of the dense gated feed-forward; None: the layer has none


@dataclass(frozen=True)
class VagulornConfig(ModelConfig):
    """Vagulorn: token rows times a scale; layers ``h = LayerNorm(x); x += mixer(h) + ff(h)`` whose mixer is
    attention within blocks of positions, attention with a window and kept first keys beside linear attention
    with fixed decays, or a selective state space layer, and whose feed-forward is gated with the tanh form of
    gelu (or absent); a final LayerNorm and the token table as output matrix.  ``config.json`` lists the layers in
    order, each with its own sizes."""

    architecture: ClassVar[str] = "Vagulorn"

    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[VagulornLayer, ...]
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' must be >= 1 and 'layers' non-empty")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm 'eps' must be > 0, got {self.norm_eps}")
        for i, layer in enumerate(self.layers):
            layer.mixer.check(f"layers[{i}].mixer.")
            if layer.ff is not None and layer.ff < 1:
                raise ConfigError(f"config.json: layers[{i}].mlp.ff must be >= 1, got {layer.ff}")

    @classmethod
    def from_dict(cls, raw: dict) -> "VagulornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = lr.get("type") if isinstance(lr, dict) else None
            if kind not in _VAGULORN_MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {sorted(_VAGULORN_MIXERS)}, got {kind!r}")
            mixer = _VAGULORN_MIXERS[kind].from_dict(_sub(lr, "mixer", where), where + "mixer.")
            mlp = _sub(lr, "mlp", where, required=False)
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where}mlp.kind must be 'dense', got {mlp.get('kind')!r}")
            layers.append(VagulornLayer(kind, mixer, None if mlp is None else _take(mlp, "ff", int)))
        emb = _sub(raw, "embedding", "", required=False) or {}
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab_size=_take(raw, "vocab", int), hidden_size=_take(raw, "width", int),
                   norm_eps=_take(_sub(raw, "norm", ""), "eps", float),
                   embedding_scale=_take(emb, "scale", float, 1.0), layers=tuple(layers), eos_token_id=eos_ids)

    def to_dict(self) -> dict:
        out: dict = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                     "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}}
        out["layers"] = [{"type": l.type, "mixer": l.mixer.to_dict(),
                          "mlp": None if l.ff is None else {"ff": l.ff, "kind": "dense"}} for l in self.layers]
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out


# --------------------------------------------------------------------------- Tedenex


@dataclass(frozen=True)
class ConvAttentionConfig:
    """Grouped-query attention with biased projections, a short convolution over time on q, k and v, q/k norm,
    no rotation, a penalty per head on the distance to the key and, with ``mask_size``, blocks of positions."""

    kind: ClassVar[str] = "attention"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int | None = None
    mask_size: int | None = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "ConvAttentionConfig":
        mask = _sub(m, "mask", where, required=False)
        return cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                   vdim=_take(m, "vdim", int), scale=_take(m, "scale", float), conv=_take(m, "conv", int, None),
                   mask_size=None if mask is None else _take(mask, "size", int, None))

    def check(self, where: str) -> None:
        if min(self.heads, self.kv_heads, self.dim, self.vdim) < 1 or self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}sizes must be >= 1 and 'heads' a multiple of 'kv_heads'")
        if self.conv is not None and self.conv < 1:
            raise ConfigError(f"config.json: {where}conv must be >= 1, got {self.conv}")
        if self.mask_size is not None and self.mask_size < 1:
            raise ConfigError(f"config.json: {where}mask.size must be >= 1, got {self.mask_size}")

    def to_dict(self) -> dict:
        out: dict = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.conv is not None:
            out["conv"] = self.conv
        if self.mask_size is not None:
            out["mask"] = {"size": self.mask_size}
        return out


@dataclass(frozen=True)
class TimeMixConfig:
    """Time mixing with a matrix state per head.  ``decay_rank``, the inner size of the decay's low-rank
    projection, is fixed by a checkpoint's tensors; it is needed (and written) only to make a model from nothing."""

    kind: ClassVar[str] = "wkv"
    heads: int
    dim: int
    decay_rank: int | None = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "TimeMixConfig":
        return cls(heads=_take(m, "heads", int), dim=_take(m, "dim", int), decay_rank=_take(m, "decay_rank", int, None))

    def check(self, where: str) -> None:
        if min(self.heads, self.dim) < 1 or (self.decay_rank is not None and self.decay_rank < 1):
            raise ConfigError(f"config.json: {where}sizes must be >= 1")

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        return out


@dataclass(frozen=True)
class LayerLoop:
    """Layers ``start .. stop - 1`` run ``times`` times in a row with the same weights."""

    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TedenexLayer:
    type: str                   # "attention", "wkv" or "latent_attention"
    mixer: "ConvAttentionConfig | TimeMixConfig | LatentAttentionConfig"
    ff: int | None              # inner width of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class TedenexConfig(ModelConfig):
    """Tedenex: layers ``x += norm(mixer(norm(x))); x += norm(ff(norm(x)))`` (RMS norms whose weights are stored
    as distances from one) followed by a token's side rows, with a mixer that is convolved attention in blocks of
    positions, time mixing with a matrix state, or attention through cached latents; a span of the layers may run
    several times in a row, each pass with a cache of its own, the token rows added again before each pass but the
    first; a final norm and the token table as output matrix.  ``config.json`` lists the layers in order."""

    architecture: ClassVar[str] = "Tedenex"

    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[TedenexLayer, ...]
    loop: LayerLoop | None = None
    side_dim: int | None = None
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' must be >= 1 and 'layers' non-empty")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm 'eps' must be > 0, got {self.norm_eps}")
        if self.side_dim is not None and self.side_dim < 1:
            raise ConfigError(f"config.json: token_side 'dim' must be >= 1, got {self.side_dim}")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start < lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError(f"config.json: loop must name layers start < stop <= {len(self.layers)} and times >= 1, "
                                  f"got start {lp.start}, stop {lp.stop}, times {lp.times}")
        for i, layer in enumerate(self.layers):
            m, w = layer.mixer, f"layers[{i}].mixer."
            if isinstance(m, LatentAttentionConfig):
                if min(m.heads, m.dim, m.vdim, m.kv_rank) < 1 or m.rot_dim < 0 or (m.q_rank is not None and m.q_rank < 1):
                    raise ConfigError(f"config.json: {w}sizes must be >= 1")
                if m.rot_dims % 2 or not (0 <= m.rot_dims <= m.rot_dim):
                    raise ConfigError(f"config.json: {w}rot.dims must be even and at most rot_dim, got {m.rot_dims}")
                if m.kv_from is not None or m.scaling is not None or m.window is not None:
                    raise ConfigError(f"config.json: {w}kv_from, rot.scaling and mask are not part of this architecture")
            else:
                m.check(w)
            if layer.ff is not None and layer.ff < 1:
                raise ConfigError(f"config.json: layers[{i}].mlp.ff must be >= 1, got {layer.ff}")

    @classmethod
    def from_dict(cls, raw: dict) -> "TedenexConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = lr.get("type") if isinstance(lr, dict) else None
            if kind not in _TEDENEX_MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {sorted(_TEDENEX_MIXERS)}, got {kind!r}")
            mixer = _TEDENEX_MIXERS[kind].from_dict(_sub(lr, "mixer", where), where + "mixer.")
            mlp = _sub(lr, "mlp", where, required=False)
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where}mlp.kind must be 'dense', got {mlp.get('kind')!r}")
            layers.append(TedenexLayer(kind, mixer, None if mlp is None else _take(mlp, "ff", int)))
        loop = _sub(raw, "loop", "", required=False)
        side = _sub(raw, "token_side", "", required=False)
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab_size=_take(raw, "vocab", int), hidden_size=_take(raw, "width", int),
                   norm_eps=_take(_sub(raw, "norm", ""), "eps", float), layers=tuple(layers),
                   loop=None if loop is None else LayerLoop(_take(loop, "start", int), _take(loop, "stop", int),
                                                            _take(loop, "times", int)),
                   side_dim=None if side is None else _take(side, "dim", int), eos_token_id=eos_ids)

    def to_dict(self) -> dict:
        out: dict = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                     "norm": {"eps": self.norm_eps}}
        out["layers"] = [{"type": l.type, "mixer": l.mixer.to_dict(),
                          "mlp": None if l.ff is None else {"ff": l.ff, "kind": "dense"}} for l in self.layers]
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out


_TEDENEX_MIXERS = {"attention": ConvAttentionConfig, "wkv": TimeMixConfig, "latent_attention": LatentAttentionConfig}


# --------------------------------------------------------------------------- Zigolix


@dataclass(frozen=True)
class SinkAttentionConfig:
    """Grouped-query attention whose values are the keys as projected; a part of each head rotated
    (neighbouring pairs, optionally with stretched frequencies); q and k brought to unit root mean square
    after the rotation; a sliding window; a learned sink per head in the softmax denominator."""

    kind: ClassVar[str] = "attention"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask_size: int | None = None
    rot_dims: int = 0
    rot_base: float = 10000.0
    scaling: RotaryScaling | None = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "SinkAttentionConfig":
        mask = _sub(m, "mask", where, required=False)
        rot = _sub(m, "rot", where, required=False)
        sc = None if rot is None else _sub(rot, "scaling", where + "rot.", required=False)
        return cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                   vdim=_take(m, "vdim", int), scale=_take(m, "scale", float),
                   mask_size=None if mask is None else _take(mask, "size", int, None),
                   rot_dims=0 if rot is None else _take(rot, "dims", int), rot_base=1e4 if rot is None else _take(rot, "base", float),
                   scaling=None if sc is None else RotaryScaling(_take(sc, "factor", float), _take(sc, "original", int),
                                                                 _take(sc, "fast", float), _take(sc, "slow", float)))

    def check(self, where: str) -> None:
        if min(self.heads, self.kv_heads, self.dim) < 1 or self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}sizes must be >= 1 and 'heads' a multiple of 'kv_heads'")
        if self.vdim != self.dim:
            raise ConfigError(f"config.json: {where}vdim must equal dim (the values are the keys), got {self.vdim} and {self.dim}")
        if self.rot_dims % 2 or not (0 <= self.rot_dims <= self.dim):
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, got {self.rot_dims}")
        if self.mask_size is not None and self.mask_size < 1:
            raise ConfigError(f"config.json: {where}mask.size must be >= 1, got {self.mask_size}")

    def to_dict(self) -> dict:
        out: dict = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.mask_size is not None:
            out["mask"] = {"size": self.mask_size}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.scaling is not None:
                out["rot"]["scaling"] = asdict(self.scaling)
        return out


@dataclass(frozen=True)
class DiffAttentionConfig:
    """Differential attention: two score maps per head over the same values, combined as ``a1 - lambda a2``;
    biased projections, no rotation, capped scores, a sliding window, a gate on the heads' outputs."""

    kind: ClassVar[str] = "attention_2"
    heads: int
    kv_heads: int
    dim: int                    # entries of ONE score map of a head (a query head holds two)
    vdim: int
    scale: float
    diff: float
    softcap: float | None = None
    mask_size: int | None = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "DiffAttentionConfig":
        mask = _sub(m, "mask", where, required=False)
        return cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                   vdim=_take(m, "vdim", int), scale=_take(m, "scale", float), diff=_take(m, "diff", float),
                   softcap=_take(m, "softcap", float, None),
                   mask_size=None if mask is None else _take(mask, "size", int, None))

    def check(self, where: str) -> None:
        if min(self.heads, self.kv_heads, self.dim, self.vdim) < 1 or self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}sizes must be >= 1 and 'heads' a multiple of 'kv_heads'")
        if self.softcap is not None and not self.softcap > 0:
            raise ConfigError(f"config.json: {where}softcap must be > 0, got {self.softcap}")
        if self.mask_size is not None and self.mask_size < 1:
            raise ConfigError(f"config.json: {where}mask.size must be >= 1, got {self.mask_size}")

    def to_dict(self) -> dict:
        out: dict = {"diff": self.diff, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                     "scale": self.scale, "vdim": self.vdim}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.mask_size is not None:
            out["mask"] = {"size": self.mask_size}
        return out


@dataclass(frozen=True)
class CappedExpertsConfig:
    """A routed mixture of small experts of the capped form (``limit``), the chosen experts' softmax scores
    divided by their sum, and optionally a shared expert of the same form that every token takes."""

    ff: int
    limit: float
    experts: int
    top: int
    shared_ff: int | None = None
    shared_limit: float | None = None

    @classmethod
    def from_dict(cls, f: dict, where: str) -> "CappedExpertsConfig":
        e, r = _sub(f, "expert", where), _sub(f, "router", where)
        sh = _sub(f, "shared", where, required=False)
        return cls(ff=_take(e, "ff", int), limit=_take(e, "limit", float), experts=_take(r, "experts", int),
                   top=_take(r, "top", int), shared_ff=None if sh is None else _take(sh, "ff", int),
                   shared_limit=None if sh is None else _take(sh, "limit", float))

    def check(self, where: str) -> None:
        if self.ff < 1 or self.experts < 1 or not (1 <= self.top <= self.experts) or (self.shared_ff is not None and self.shared_ff < 1):
            raise ConfigError(f"config.json: {where}sizes must be >= 1 and 1 <= router.top <= router.experts")
        if not self.limit > 0 or (self.shared_limit is not None and not self.shared_limit > 0):
            raise ConfigError(f"config.json: {where}'limit' must be > 0")

    def to_dict(self) -> dict:
        out: dict = {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
                     "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


@dataclass(frozen=True)
class ZigolixLayer:
    type: str                                   # "attention" or "attention_2"
    mixer: "SinkAttentionConfig | DiffAttentionConfig"
    ff: "int | CappedExpertsConfig | None"      # inner width of the dense gated feed-forward; routed experts; none


@dataclass(frozen=True)
class ZigolixConfig(ModelConfig):
    """Zigolix: pre-norm layers ``x += mixer(norm1(x)); x += ff(norm2(x))`` whose mixer is attention with a sink
    and keys as values, or differential attention; the feed-forward is gated with the tanh form of gelu or a routed
    mixture of capped experts beside a shared one.  A span of the layers may run several times in a row, each pass
    with a cache of its own; every pass opens with ``x <- W_in [x; x0] + step[pass]`` (x0 the token rows).  A final
    norm, an output matrix of its own and a factor on the logits.  ``config.json`` lists the layers in order."""

    architecture: ClassVar[str] = "Zigolix"

    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[ZigolixLayer, ...]
    loop: LayerLoop | None = None
    logit_scale: float = 1.0
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        if self.vocab_size < 1 or self.hidden_size < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' must be >= 1 and 'layers' non-empty")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm 'eps' must be > 0, got {self.norm_eps}")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start < lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError(f"config.json: loop must name layers start < stop <= {len(self.layers)} and times >= 1, "
                                  f"got start {lp.start}, stop {lp.stop}, times {lp.times}")
        for i, layer in enumerate(self.layers):
            layer.mixer.check(f"layers[{i}].mixer.")
            if isinstance(layer.ff, CappedExpertsConfig):
                layer.ff.check(f"layers[{i}].mlp.")
            elif layer.ff is not None and layer.ff < 1:
                raise ConfigError(f"config.json: layers[{i}].mlp.ff must be >= 1, got {layer.ff}")

    @classmethod
    def from_dict(cls, raw: dict) -> "ZigolixConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = lr.get("type") if isinstance(lr, dict) else None
            if kind not in _ZIGOLIX_MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {sorted(_ZIGOLIX_MIXERS)}, got {kind!r}")
            mixer = _ZIGOLIX_MIXERS[kind].from_dict(_sub(lr, "mixer", where), where + "mixer.")
            mlp = _sub(lr, "mlp", where, required=False)
            if mlp is None:
                ff = None
            elif mlp.get("kind", "dense") == "dense":
                ff = _take(mlp, "ff", int)
            elif mlp.get("kind") == "moe":
                ff = CappedExpertsConfig.from_dict(mlp, where + "mlp.")
            else:
                raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' or 'moe', got {mlp.get('kind')!r}")
            layers.append(ZigolixLayer(kind, mixer, ff))
        loop = _sub(raw, "loop", "", required=False)
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab_size=_take(raw, "vocab", int), hidden_size=_take(raw, "width", int),
                   norm_eps=_take(_sub(raw, "norm", ""), "eps", float), layers=tuple(layers),
                   loop=None if loop is None else LayerLoop(_take(loop, "start", int), _take(loop, "stop", int),
                                                            _take(loop, "times", int)),
                   logit_scale=_take(raw, "logit_scale", float, 1.0), eos_token_id=eos_ids)

    def to_dict(self) -> dict:
        out: dict = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                     "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale}
        out["layers"] = [{"type": l.type, "mixer": l.mixer.to_dict(),
                          "mlp": None if l.ff is None else l.ff.to_dict() if isinstance(l.ff, CappedExpertsConfig)
                          else {"ff": l.ff, "kind": "dense"}} for l in self.layers]
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out


_ZIGOLIX_MIXERS = {c.kind: c for c in (SinkAttentionConfig, DiffAttentionConfig)}


def read_config_json(model_dir: str | Path) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw


def architecture_name(raw: dict) -> str:
    if isinstance(raw.get("architecture"), str):         # designs that name themselves with one string
        return raw["architecture"]
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]


def config_field_names(cls) -> list[str]:
    return [f.name for f in fields(cls)]


def dump_config(cfg: ModelConfig, model_dir: str | Path) -> None:
    Path(model_dir).mkdir(parents=True, exist_ok=True)
    (Path(model_dir) / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1) + "\n")
