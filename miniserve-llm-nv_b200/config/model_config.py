"""Typed configuration of the Qwen3 dense decoder, read from its own ``config.json`` keys.

Follows the contract of miniserve/config/model_config.py:59-215: every size is required and
must be an integer (booleans are refused), ``head_dim`` is read and never inferred from
``hidden_size / num_attention_heads``, the float constants must be finite and positive, and
every option the model code does not implement (biases, dropout, scaled or interleaved RoPE,
sliding windows, another activation) is refused with a message that names the key.  Unlike
that contract, untied output embeddings are accepted (``tie_word_embeddings`` false needs
``lm_head.weight`` in the checkpoint).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .registry import UnsupportedModelError


def _integer(data: Mapping[str, Any], key: str) -> int:
    value = data.get(key)
    if not isinstance(value, int) or isinstance(value, bool):
        raise ValueError(f"{key} must be an integer in the model config, got {value!r}")
    if value <= 0:
        raise ValueError(f"{key} must be positive, got {value}")
    return value


def _number(data: Mapping[str, Any], key: str) -> float:
    value = data.get(key)
    if not isinstance(value, (int, float)) or isinstance(value, bool):
        raise ValueError(f"{key} must be numeric in the model config, got {value!r}")
    return float(value)


def _boolean(data: Mapping[str, Any], key: str, default: bool = False) -> bool:
    value = data.get(key, default)
    if not isinstance(value, bool):
        raise ValueError(f"{key} must be boolean in the model config, got {value!r}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    """Sizes and constants of one Qwen3 dense checkpoint; immutable."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"
    hidden_act: str = "silu"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen3Config":
        architectures = data.get("architectures") or ()
        if list(architectures) != ["Qwen3ForCausalLM"] or str(data.get("model_type", "")) != "qwen3":
            raise UnsupportedModelError(
                "UNSUPPORTED_MODEL_CONFIGURATION: expected architectures ['Qwen3ForCausalLM'] with model_type "
                f"'qwen3', got {list(architectures)!r} with {data.get('model_type')!r}")
        if "head_dim" not in data:
            raise ValueError("Qwen3 model config must define integer head_dim (it is not hidden_size / heads)")
        config = cls(
            hidden_size=_integer(data, "hidden_size"),
            intermediate_size=_integer(data, "intermediate_size"),
            num_hidden_layers=_integer(data, "num_hidden_layers"),
            num_attention_heads=_integer(data, "num_attention_heads"),
            num_key_value_heads=_integer(data, "num_key_value_heads"),
            head_dim=_integer(data, "head_dim"),
            vocab_size=_integer(data, "vocab_size"),
            max_position_embeddings=_integer(data, "max_position_embeddings"),
            rms_norm_eps=_number(data, "rms_norm_eps"),
            rope_theta=_number(data, "rope_theta"),
            tie_word_embeddings=_boolean(data, "tie_word_embeddings"),
            hidden_act=str(data.get("hidden_act", "")),
        )
        if config.hidden_act != "silu":
            raise ValueError(f"hidden_act must be 'silu' (the only gated activation implemented), got {config.hidden_act!r}")
        if _boolean(data, "attention_bias") or _boolean(data, "mlp_bias"):
            raise ValueError("attention_bias and mlp_bias must be false: only bias-free projections are implemented")
        if "attention_dropout" in data and _number(data, "attention_dropout") != 0.0:
            raise ValueError("attention_dropout must be 0.0")
        if _boolean(data, "rope_interleaved") or data.get("rope_scaling") is not None:
            raise ValueError("rope_scaling must be null and rope_interleaved false: scaled or interleaved RoPE is not implemented")
        if _boolean(data, "use_sliding_window"):
            raise ValueError("use_sliding_window must be false: this architecture is implemented without a window")
        config.validate()
        return config

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise ValueError(f"head_dim {self.head_dim} is odd; the rotation pairs the elements of a head")
        from ..kernels import MAX_HEAD_DIM      # a number, no device work: the largest head the attention kernels take

        if self.head_dim > MAX_HEAD_DIM:
            raise ValueError(f"head_dim {self.head_dim} exceeds {MAX_HEAD_DIM}, the largest head size the attention "
                             "kernels of this engine take")
        for name in ("rms_norm_eps", "rope_theta"):
            value = getattr(self, name)
            if not math.isfinite(value) or value <= 0:
                raise ValueError(f"{name} must be finite and positive, got {value}")

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        return {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "attention_dropout": 0.0,
            "rope_scaling": None,
            "sliding_window": None,
            "use_sliding_window": False,
        }


# --------------------------------------------------------------------------- Vesidra


def _section(data: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = data.get(key)
    if not isinstance(value, Mapping):
        raise ValueError(f"{where}{key} must be an object in the model config, got {value!r}")
    return value


def _positive(data: Mapping[str, Any], key: str, where: str) -> float:
    value = _number(data, key)
    if not math.isfinite(value) or value <= 0:
        raise ValueError(f"{where}{key} must be finite and positive, got {value}")
    return value


@dataclass(frozen=True)
class RotationConfig:
    """A rotary position encoding: ``dims`` rotated entries with base ``base``; ``scaling`` is None or the YaRN
    constants (factor, original context, fast and slow turn counts)."""

    base: float
    dims: int
    scaling: Any = None      # None or a tuple (factor, original, fast, slow)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "RotationConfig":
        scaling = data.get("scaling")
        if scaling is not None:
            scaling = _section(data, "scaling", where)
            scaling = tuple(_positive(scaling, key, where + "scaling.") for key in ("factor", "original", "fast", "slow"))
        config = cls(base=_positive(data, "base", where), dims=_integer(data, "dims"), scaling=scaling)
        if config.dims % 2:
            raise ValueError(f"{where}dims {config.dims} is odd; the rotation turns pairs of entries")
        if config.base == 1.0:
            raise ValueError(f"{where}base must differ from 1")
        return config

    def scaling_dict(self):
        return None if self.scaling is None else dict(zip(("factor", "original", "fast", "slow"), self.scaling))


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationConfig

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        config = cls(heads=_integer(data, "heads"), dim=_integer(data, "dim"), rot_dim=_integer(data, "rot_dim"),
                     vdim=_integer(data, "vdim"), kv_rank=_integer(data, "kv_rank"), scale=_positive(data, "scale", where),
                     rot=RotationConfig.from_dict(_section(data, "rot", where), where + "rot."))
        if config.rot.dims > config.rot_dim:
            raise ValueError(f"{where}rot.dims {config.rot.dims} exceeds the rotated part rot_dim {config.rot_dim}")
        return config


@dataclass(frozen=True)
class VesidraFeedForwardConfig:
    """``kind`` "dense": a gated feed-forward of inner size ``ff``.  ``kind`` "moe": ``experts`` experts of inner size
    ``ff`` of which a token uses ``top``, and a shared expert of inner size ``shared_ff`` (None: no shared expert)."""

    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    shared_ff: Any = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "VesidraFeedForwardConfig":
        kind = data.get("kind")
        if kind == "dense":
            return cls(kind="dense", ff=_integer(data, "ff"))
        if kind == "moe":
            router = _section(data, "router", where)
            shared = data.get("shared")
            config = cls(kind="moe", ff=_integer(_section(data, "expert", where), "ff"), experts=_integer(router, "experts"),
                         top=_integer(router, "top"), shared_ff=None if shared is None else _integer(_section(data, "shared", where), "ff"))
            if config.top > config.experts:
                raise ValueError(f"{where}router.top {config.top} exceeds router.experts {config.experts}")
            return config
        raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}kind {kind!r} is not implemented (dense, moe)")


@dataclass(frozen=True)
class VesidraLayerConfig:
    type: str
    mixer: LatentAttentionConfig
    mlp: Any      # VesidraFeedForwardConfig or None


@dataclass(frozen=True)
class VesidraConfig:
    """The Vesidra decoder: ``config.json`` holds ``architecture``, ``vocab``, ``width``, ``embedding.scale``,
    ``norm.eps`` and ``layers``, a list whose entries give each layer's mixer ``type``, the mixer's sizes and
    constants (``mixer``) and its feed-forward (``mlp``, or null).  Every size and constant is read; nothing is
    inferred from another."""

    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: tuple
    architecture: str = "Vesidra"

    MIXERS = ("latent_attention",)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "VesidraConfig":
        if data.get("architecture") != "Vesidra":
            raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: expected architecture 'Vesidra', got {data.get('architecture')!r}")
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ValueError("layers must be a non-empty list in the model config")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"layers[{index}]."
            if not isinstance(raw, Mapping):
                raise ValueError(f"layers[{index}] must be an object")
            kind = raw.get("type")
            if kind not in cls.MIXERS:
                raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}type {kind!r} is not implemented "
                                            f"({', '.join(cls.MIXERS)})")
            mixer = LatentAttentionConfig.from_dict(_section(raw, "mixer", where), where + "mixer.")
            mlp = None if raw.get("mlp") is None else VesidraFeedForwardConfig.from_dict(_section(raw, "mlp", where), where + "mlp.")
            layers.append(VesidraLayerConfig(kind, mixer, mlp))
        return cls(vocab=_integer(data, "vocab"), width=_integer(data, "width"),
                   embedding_scale=_positive(_section(data, "embedding", ""), "scale", "embedding."),
                   eps=_positive(_section(data, "norm", ""), "eps", "norm."), layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer = dict(heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
                         rot=dict(base=m.rot.base, dims=m.rot.dims, scaling=m.rot.scaling_dict()))
            mlp = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                mlp = dict(kind="dense", ff=layer.mlp.ff)
            elif layer.mlp is not None:
                mlp = dict(kind="moe", expert=dict(ff=layer.mlp.ff), router=dict(experts=layer.mlp.experts, top=layer.mlp.top),
                           shared=None if layer.mlp.shared_ff is None else dict(ff=layer.mlp.shared_ff))
            layers.append(dict(type=layer.type, mixer=mixer, mlp=mlp))
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width,
                    embedding=dict(scale=self.embedding_scale), norm=dict(eps=self.eps), layers=layers)


# --------------------------------------------------------------------------- Zozezen


def _count(data: Mapping[str, Any], key: str, default: int) -> int:
    """An integer that may be absent or null (then ``default``) and may be zero."""
    value = data.get(key)
    if value is None:
        return default
    if not isinstance(value, int) or isinstance(value, bool) or value < 0:
        raise ValueError(f"{key} must be a non-negative integer in the model config, got {value!r}")
    return value


@dataclass(frozen=True)
class GatedAttentionConfig:
    """Grouped-query attention with query/key heads of ``dim`` and value heads of ``vdim`` entries, a rotation over the
    first ``rot.dims`` entries, a sink in the softmax and a gate per head.  ``kv_from``: the index of the layer whose
    keys and values this layer reads instead of making its own (None: its own)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig
    kv_from: Any = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "GatedAttentionConfig":
        rot = _section(data, "rot", where)
        if _count(rot, "dims", 0) == 0:
            rotation = RotationConfig(base=_positive(rot, "base", where + "rot."), dims=0)      # nothing is rotated
        else:
            rotation = RotationConfig.from_dict(rot, where + "rot.")
        config = cls(heads=_integer(data, "heads"), kv_heads=_integer(data, "kv_heads"), dim=_integer(data, "dim"),
                     vdim=_integer(data, "vdim"), scale=_positive(data, "scale", where), rot=rotation,
                     kv_from=None if data.get("kv_from") is None else _count(data, "kv_from", 0))
        if config.heads % config.kv_heads:
            raise ValueError(f"{where}heads {config.heads} is not a multiple of kv_heads {config.kv_heads}")
        if config.rot.dims > config.dim:
            raise ValueError(f"{where}rot.dims {config.rot.dims} exceeds the head size dim {config.dim}")
        if config.rot.scaling is not None:
            raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}rot.scaling is not part of this design")
        return config

    def to_dict(self) -> dict[str, Any]:
        out = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                   rot=dict(base=self.rot.base, dims=self.rot.dims))
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class StateSpaceConfig:
    """The selective state-space mixer: ``heads`` heads of ``vdim`` channels, a state of ``state`` numbers per channel,
    ``groups`` groups of input and output maps shared by ``heads / groups`` heads each, a causal convolution of ``conv``
    taps, and a gated norm in ``norm_groups`` equal parts."""

    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "StateSpaceConfig":
        config = cls(heads=_integer(data, "heads"), vdim=_integer(data, "vdim"), state=_integer(data, "state"),
                     groups=_integer(data, "groups"), conv=_integer(data, "conv"), norm_groups=_integer(data, "norm_groups"))
        if config.heads % config.groups:
            raise ValueError(f"{where}heads {config.heads} is not a multiple of groups {config.groups}")
        if (config.heads * config.vdim) % config.norm_groups:
            raise ValueError(f"{where}norm_groups {config.norm_groups} does not divide heads * vdim = {config.heads * config.vdim}")
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, vdim=self.vdim, state=self.state, groups=self.groups, conv=self.conv,
                    norm_groups=self.norm_groups)


@dataclass(frozen=True)
class GroupedMixtureConfig:
    """A mixture of ``experts`` clamped gated experts of inner size ``ff`` plus ``identity`` identity experts, of which a
    token uses ``top``; the router's outputs form ``group_count`` equal groups of neighbours of which the best
    ``group_keep`` can be chosen from; a shared expert of inner size ``shared_ff`` (None: no shared expert)."""

    ff: int
    limit: float
    experts: int
    identity: int
    top: int
    group_count: int
    group_keep: int
    shared_ff: Any = None
    shared_limit: Any = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "GroupedMixtureConfig":
        kind = data.get("kind", "moe")
        if kind != "moe":
            raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}kind {kind!r} is not implemented (moe)")
        expert, router = _section(data, "expert", where), _section(data, "router", where)
        groups = router.get("groups")
        count, keep = 1, 1
        if groups is not None:
            groups = _section(router, "groups", where + "router.")
            count, keep = _integer(groups, "count"), _integer(groups, "keep")
        shared = data.get("shared")
        if shared is not None:
            shared = _section(data, "shared", where)
        config = cls(ff=_integer(expert, "ff"), limit=_positive(expert, "limit", where + "expert."),
                     experts=_integer(router, "experts"), identity=_count(router, "identity", 0), top=_integer(router, "top"),
                     group_count=count, group_keep=keep,
                     shared_ff=None if shared is None else _integer(shared, "ff"),
                     shared_limit=None if shared is None else _positive(shared, "limit", where + "shared."))
        total = config.experts + config.identity
        if total % config.group_count or not 1 <= config.group_keep <= config.group_count:
            raise ValueError(f"{where}router.groups: {total} router outputs in {config.group_count} groups, {config.group_keep} kept")
        if config.top > config.group_keep * (total // config.group_count):
            raise ValueError(f"{where}router.top {config.top} exceeds the {config.group_keep} kept groups of {total // config.group_count}")
        return config

    def to_dict(self) -> dict[str, Any]:
        router = dict(experts=self.experts, identity=self.identity, top=self.top,
                      groups=dict(count=self.group_count, keep=self.group_keep))
        shared = None if self.shared_ff is None else dict(ff=self.shared_ff, limit=self.shared_limit)
        return dict(kind="moe", expert=dict(ff=self.ff, limit=self.limit), router=router, shared=shared)


@dataclass(frozen=True)
class ZozezenLayerConfig:
    type: str       # "attention" or "mamba2"
    mixer: Any      # GatedAttentionConfig or StateSpaceConfig
    mlp: Any        # GroupedMixtureConfig or None


@dataclass(frozen=True)
class ZozezenConfig:
    """The Zozezen decoder: ``config.json`` holds ``architecture``, ``vocab``, ``width``, ``norm.eps`` and ``layers``, a
    list whose entries give each layer's mixer ``type`` (``attention`` or ``mamba2``), the mixer's sizes and constants
    (``mixer``) and its feed-forward (``mlp``, or null).  Every size and constant is read; nothing is inferred."""

    vocab: int
    width: int
    eps: float
    layers: tuple
    architecture: str = "Zozezen"

    MIXERS = {"attention": GatedAttentionConfig, "mamba2": StateSpaceConfig}

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ZozezenConfig":
        if data.get("architecture") != "Zozezen":
            raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: expected architecture 'Zozezen', got {data.get('architecture')!r}")
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ValueError("layers must be a non-empty list in the model config")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"layers[{index}]."
            if not isinstance(raw, Mapping):
                raise ValueError(f"layers[{index}] must be an object")
            kind = raw.get("type")
            if kind not in cls.MIXERS:
                raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}type {kind!r} is not implemented "
                                            f"({', '.join(cls.MIXERS)})")
            mixer = cls.MIXERS[kind].from_dict(_section(raw, "mixer", where), where + "mixer.")
            mlp = None if raw.get("mlp") is None else GroupedMixtureConfig.from_dict(_section(raw, "mlp", where), where + "mlp.")
            layers.append(ZozezenLayerConfig(kind, mixer, mlp))
        for index, layer in enumerate(layers):
            source = getattr(layer.mixer, "kv_from", None)
            if source is None:
                continue
            where = f"layers[{index}].mixer.kv_from"
            if not source < index or layers[source].type != "attention" or layers[source].mixer.kv_from is not None:
                raise ValueError(f"{where} {source} must name an earlier attention layer that has keys and values of its own")
            lender, m = layers[source].mixer, layer.mixer
            if (lender.kv_heads, lender.dim, lender.vdim, lender.rot) != (m.kv_heads, m.dim, m.vdim, m.rot):
                raise ValueError(f"{where}: layer {source}'s key/value heads, sizes and rotation differ from this layer's")
        return cls(vocab=_integer(data, "vocab"), width=_integer(data, "width"),
                   eps=_positive(_section(data, "norm", ""), "eps", "norm."), layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        layers = [dict(type=layer.type, mixer=layer.mixer.to_dict(), mlp=None if layer.mlp is None else layer.mlp.to_dict())
                  for layer in self.layers]
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.eps), layers=layers)


# --------------------------------------------------------------------------- Kivurax


@dataclass(frozen=True)
class MatrixMemoryConfig:
    """The matrix-memory mixer (mLSTM): ``heads`` heads with queries and keys of ``dim`` and values of ``vdim`` entries; the
    log gates are soft-capped at ``gate_cap``."""

    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "MatrixMemoryConfig":
        return cls(heads=_integer(data, "heads"), dim=_integer(data, "dim"), vdim=_integer(data, "vdim"),
                   gate_cap=_positive(data, "gate_cap", where))

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, dim=self.dim, vdim=self.vdim, gate_cap=self.gate_cap)


@dataclass(frozen=True)
class WindowAttentionConfig:
    """Grouped-query attention over a sliding window of ``window`` keys whose values are its keys as projected, with a
    sink in the softmax, a norm per query and key head and an interleaved rotation of the first ``rot.dims`` entries."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot: RotationConfig

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "WindowAttentionConfig":
        rot = _section(data, "rot", where)
        if _count(rot, "dims", 0) == 0:
            rotation = RotationConfig(base=_positive(rot, "base", where + "rot."), dims=0)
        else:
            rotation = RotationConfig.from_dict(rot, where + "rot.")
        config = cls(heads=_integer(data, "heads"), kv_heads=_integer(data, "kv_heads"), dim=_integer(data, "dim"),
                     vdim=_integer(data, "vdim"), scale=_positive(data, "scale", where),
                     window=_integer(_section(data, "mask", where), "size"), rot=rotation)
        if config.heads % config.kv_heads:
            raise ValueError(f"{where}heads {config.heads} is not a multiple of kv_heads {config.kv_heads}")
        if config.vdim != config.dim:
            raise ValueError(f"{where}vdim {config.vdim} differs from dim {config.dim}, but the values are the keys")
        if config.rot.dims > config.dim:
            raise ValueError(f"{where}rot.dims {config.rot.dims} exceeds the head size dim {config.dim}")
        return config

    def to_dict(self) -> dict[str, Any]:
        rot = dict(base=self.rot.base, dims=self.rot.dims)
        if self.rot.scaling is not None:
            rot["scaling"] = self.rot.scaling_dict()
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                    mask=dict(size=self.window), rot=rot)


@dataclass(frozen=True)
class LinearRecurrenceConfig:
    """The gated linear recurrence (a real-gated linear recurrent unit behind a short convolution): ``width`` channels whose
    two gates are block-diagonal maps in ``blocks`` equal parts; a causal convolution of ``conv`` taps."""

    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "LinearRecurrenceConfig":
        config = cls(width=_integer(data, "width"), blocks=_integer(data, "blocks"), conv=_integer(data, "conv"))
        if config.width % config.blocks:
            raise ValueError(f"{where}blocks {config.blocks} does not divide width {config.width}")
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(width=self.width, blocks=self.blocks, conv=self.conv)


@dataclass(frozen=True)
class SideBySideConfig:
    """Two mixers that read the same input; the result is ``left_scale * left + right_scale * right``."""

    left: WindowAttentionConfig
    right: LinearRecurrenceConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "SideBySideConfig":
        return cls(left=WindowAttentionConfig.from_dict(_section(data, "left", where), where + "left."),
                   right=LinearRecurrenceConfig.from_dict(_section(data, "right", where), where + "right."),
                   left_scale=_number(data, "left_scale"), right_scale=_number(data, "right_scale"))

    def to_dict(self) -> dict[str, Any]:
        return dict(left=self.left.to_dict(), right=self.right.to_dict(), left_scale=self.left_scale, right_scale=self.right_scale)


@dataclass(frozen=True)
class DeltaRuleConfig:
    """The gated delta rule: ``heads`` value heads of ``vdim`` entries over ``kv_heads`` query/key heads of ``dim`` entries;
    queries, keys and values pass a causal convolution of ``conv`` taps."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "DeltaRuleConfig":
        config = cls(heads=_integer(data, "heads"), kv_heads=_integer(data, "kv_heads"), dim=_integer(data, "dim"),
                     vdim=_integer(data, "vdim"), conv=_integer(data, "conv"))
        if config.heads % config.kv_heads:
            raise ValueError(f"{where}heads {config.heads} is not a multiple of kv_heads {config.kv_heads}")
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, conv=self.conv)


@dataclass(frozen=True)
class KivuraxFeedForwardConfig:
    """``kind`` "dense": a gated feed-forward of inner size ``ff`` whose three projections have biases.  ``kind`` "moe":
    ``experts`` gated experts of inner size ``ff`` without biases, of which a token uses ``top``."""

    kind: str
    ff: int
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "KivuraxFeedForwardConfig":
        kind = data.get("kind")
        if kind == "dense":
            return cls(kind="dense", ff=_integer(data, "ff"))
        if kind == "moe":
            router = _section(data, "router", where)
            config = cls(kind="moe", ff=_integer(_section(data, "expert", where), "ff"), experts=_integer(router, "experts"),
                         top=_integer(router, "top"))
            if config.top > config.experts:
                raise ValueError(f"{where}router.top {config.top} exceeds router.experts {config.experts}")
            return config
        raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}kind {kind!r} is not implemented (dense, moe)")

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        return dict(kind="moe", expert=dict(ff=self.ff), router=dict(experts=self.experts, top=self.top))


@dataclass(frozen=True)
class KivuraxLayerConfig:
    type: str       # "mlstm", "parallel" or "delta"
    mixer: Any
    mlp: Any        # KivuraxFeedForwardConfig or None


@dataclass(frozen=True)
class KivuraxConfig:
    """The Kivurax decoder: ``config.json`` holds ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` and
    ``layers``, a list whose entries give each layer's mixer ``type`` (``mlstm``, ``parallel`` or ``delta``), the mixer's
    sizes and constants (``mixer``) and its feed-forward (``mlp``, or null).  Every size and constant is read."""

    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: tuple
    architecture: str = "Kivurax"

    MIXERS = {"mlstm": MatrixMemoryConfig, "parallel": SideBySideConfig, "delta": DeltaRuleConfig}

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "KivuraxConfig":
        if data.get("architecture") != "Kivurax":
            raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: expected architecture 'Kivurax', got {data.get('architecture')!r}")
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ValueError("layers must be a non-empty list in the model config")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"layers[{index}]."
            if not isinstance(raw, Mapping):
                raise ValueError(f"layers[{index}] must be an object")
            kind = raw.get("type")
            if kind not in cls.MIXERS:
                raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}type {kind!r} is not implemented "
                                            f"({', '.join(cls.MIXERS)})")
            mixer = cls.MIXERS[kind].from_dict(_section(raw, "mixer", where), where + "mixer.")
            mlp = None if raw.get("mlp") is None else KivuraxFeedForwardConfig.from_dict(_section(raw, "mlp", where), where + "mlp.")
            layers.append(KivuraxLayerConfig(kind, mixer, mlp))
        mult = _number(data, "residual_mult")
        if not math.isfinite(mult):
            raise ValueError(f"residual_mult must be finite, got {mult}")
        return cls(vocab=_integer(data, "vocab"), width=_integer(data, "width"),
                   eps=_positive(_section(data, "norm", ""), "eps", "norm."), residual_mult=mult, layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        layers = [dict(type=layer.type, mixer=layer.mixer.to_dict(), mlp=None if layer.mlp is None else layer.mlp.to_dict())
                  for layer in self.layers]
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.eps),
                    residual_mult=self.residual_mult, layers=layers)


# --------------------------------------------------------------------------- Bafavik


def _rotation_or_none(data: Mapping[str, Any], where: str) -> RotationConfig:
    rot = _section(data, "rot", where)
    if _count(rot, "dims", 0) == 0:
        return RotationConfig(base=_positive(rot, "base", where + "rot."), dims=0)
    return RotationConfig.from_dict(rot, where + "rot.")


@dataclass(frozen=True)
class RotaryAttentionConfig:
    """Grouped-query softmax attention with a rotation of the first ``rot.dims`` entries of a head, values of their own size
    and, where ``conv`` is given, a short causal convolution of that many taps on queries, keys and values."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig
    conv: Any = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str, conv: bool = False) -> "RotaryAttentionConfig":
        config = cls(heads=_integer(data, "heads"), kv_heads=_integer(data, "kv_heads"), dim=_integer(data, "dim"),
                     vdim=_integer(data, "vdim"), scale=_positive(data, "scale", where), rot=_rotation_or_none(data, where),
                     conv=_integer(data, "conv") if conv else None)
        if config.heads % config.kv_heads:
            raise ValueError(f"{where}heads {config.heads} is not a multiple of kv_heads {config.kv_heads}")
        if config.rot.dims > config.dim:
            raise ValueError(f"{where}rot.dims {config.rot.dims} exceeds the head size dim {config.dim}")
        return config

    def to_dict(self) -> dict[str, Any]:
        out = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                   rot=dict(base=self.rot.base, dims=self.rot.dims))
        if self.conv is not None:
            out["conv"] = self.conv
        return out


@dataclass(frozen=True)
class LinearAttentionConfig:
    """Linear attention with a constant decay per head (``decay``: one number per head)."""

    heads: int
    dim: int
    vdim: int
    decay: tuple

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "LinearAttentionConfig":
        decay = data.get("decay")
        if not isinstance(decay, (list, tuple)) or not all(isinstance(v, (int, float)) and not isinstance(v, bool) for v in decay):
            raise ValueError(f"{where}decay must be a list of numbers, got {decay!r}")
        config = cls(heads=_integer(data, "heads"), dim=_integer(data, "dim"), vdim=_integer(data, "vdim"),
                     decay=tuple(float(v) for v in decay))
        if len(config.decay) != config.heads or not all(math.isfinite(v) for v in config.decay):
            raise ValueError(f"{where}decay must hold one finite number for each of the {config.heads} heads")
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, dim=self.dim, vdim=self.vdim, decay=list(self.decay))


@dataclass(frozen=True)
class ChannelDeltaRuleConfig:
    """The gated delta rule with a decay per head and key channel; the decay's and the output gate's projections are products
    of two matrices through ``decay_rank`` and ``gate_rank`` numbers, which a checkpoint's tensor shapes give where
    ``config.json`` does not."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Any = None
    gate_rank: Any = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "ChannelDeltaRuleConfig":
        config = cls(heads=_integer(data, "heads"), kv_heads=_integer(data, "kv_heads"), dim=_integer(data, "dim"),
                     vdim=_integer(data, "vdim"), conv=_integer(data, "conv"),
                     decay_rank=_integer(data, "decay_rank") if "decay_rank" in data else None,
                     gate_rank=_integer(data, "gate_rank") if "gate_rank" in data else None)
        if config.heads % config.kv_heads:
            raise ValueError(f"{where}heads {config.heads} is not a multiple of kv_heads {config.kv_heads}")
        return config

    def to_dict(self) -> dict[str, Any]:
        out = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, conv=self.conv)
        for key in ("decay_rank", "gate_rank"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        return out


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    """Differential attention without rotation under a chunked mask of ``chunk`` positions."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    chunk: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "DifferentialAttentionConfig":
        config = cls(heads=_integer(data, "heads"), kv_heads=_integer(data, "kv_heads"), dim=_integer(data, "dim"),
                     vdim=_integer(data, "vdim"), scale=_positive(data, "scale", where), diff=_number(data, "diff"),
                     chunk=_integer(_section(data, "mask", where), "size"))
        if config.heads % config.kv_heads:
            raise ValueError(f"{where}heads {config.heads} is not a multiple of kv_heads {config.kv_heads}")
        if not math.isfinite(config.diff):
            raise ValueError(f"{where}diff must be finite, got {config.diff}")
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale, diff=self.diff,
                    mask=dict(size=self.chunk))


@dataclass(frozen=True)
class BafavikPairConfig:
    """Two mixers that read the same input.  ``parallel``: rotary attention beside linear attention, summed with a scale each.
    ``parallel_2``: convolved rotary attention beside the channel delta rule, each output normed, half their sum."""

    left: Any
    right: Any
    left_scale: Any = None
    right_scale: Any = None

    @classmethod
    def scaled(cls, data: Mapping[str, Any], where: str) -> "BafavikPairConfig":
        return cls(left=RotaryAttentionConfig.from_dict(_section(data, "left", where), where + "left."),
                   right=LinearAttentionConfig.from_dict(_section(data, "right", where), where + "right."),
                   left_scale=_number(data, "left_scale"), right_scale=_number(data, "right_scale"))

    @classmethod
    def normed(cls, data: Mapping[str, Any], where: str) -> "BafavikPairConfig":
        return cls(left=RotaryAttentionConfig.from_dict(_section(data, "left", where), where + "left.", conv=True),
                   right=ChannelDeltaRuleConfig.from_dict(_section(data, "right", where), where + "right."))

    def to_dict(self) -> dict[str, Any]:
        out = dict(left=self.left.to_dict(), right=self.right.to_dict())
        if self.left_scale is not None:
            out.update(left_scale=self.left_scale, right_scale=self.right_scale)
        return out


@dataclass(frozen=True)
class BafavikLayerConfig:
    type: str       # "parallel", "attention" or "parallel_2"
    mixer: Any
    ff: Any         # inner size of the dense feed-forward, or None


@dataclass(frozen=True)
class TokenPairConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class BafavikConfig:
    """The Bafavik decoder: ``config.json`` holds ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult``,
    ``logit_scale``, ``embedding`` (``scale`` and, optionally, ``bigram`` with ``buckets``, ``mul_prev``, ``mul_cur``), ``loop``
    (``start``, ``stop``, ``times``: those layers run that often in a row, or null) and ``layers``, a list whose entries give each
    layer's mixer ``type`` (``parallel``, ``attention`` or ``parallel_2``), the mixer's sizes and constants (``mixer``) and its
    feed-forward (``mlp`` with ``kind`` "dense" and ``ff``, or null).  Every size and constant is read."""

    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    embedding_scale: float
    bigram: Any
    loop: Any       # None or (start, stop, times)
    layers: tuple
    architecture: str = "Bafavik"

    MIXERS = {"parallel": BafavikPairConfig.scaled, "attention": DifferentialAttentionConfig.from_dict,
              "parallel_2": BafavikPairConfig.normed}

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "BafavikConfig":
        if data.get("architecture") != "Bafavik":
            raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: expected architecture 'Bafavik', got {data.get('architecture')!r}")
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ValueError("layers must be a non-empty list in the model config")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"layers[{index}]."
            if not isinstance(raw, Mapping):
                raise ValueError(f"layers[{index}] must be an object")
            kind = raw.get("type")
            if kind not in cls.MIXERS:
                raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}type {kind!r} is not implemented "
                                            f"({', '.join(cls.MIXERS)})")
            mixer = cls.MIXERS[kind](_section(raw, "mixer", where), where + "mixer.")
            ff = None
            if raw.get("mlp") is not None:
                mlp = _section(raw, "mlp", where)
                if mlp.get("kind") != "dense":
                    raise UnsupportedModelError(f"UNSUPPORTED_MODEL_CONFIGURATION: {where}mlp.kind {mlp.get('kind')!r} is not implemented (dense)")
                ff = _integer(mlp, "ff")
            layers.append(BafavikLayerConfig(kind, mixer, ff))
        embedding = _section(data, "embedding", "")
        bigram = None
        if embedding.get("bigram") is not None:
            raw = _section(embedding, "bigram", "embedding.")
            bigram = TokenPairConfig(_integer(raw, "buckets"), _count(raw, "mul_prev", 0), _count(raw, "mul_cur", 0))
        loop = None
        if data.get("loop") is not None:
            raw = _section(data, "loop", "")
            loop = (_count(raw, "start", 0), _integer(raw, "stop"), _integer(raw, "times"))
            if not loop[0] < loop[1] <= len(layers):
                raise ValueError(f"loop: layers {loop[0]} .. {loop[1]} - 1 are not a run of the model's {len(layers)} layers")
        mult, logit_scale = _number(data, "residual_mult"), _number(data, "logit_scale")
        if not math.isfinite(mult) or not math.isfinite(logit_scale):
            raise ValueError(f"residual_mult and logit_scale must be finite, got {mult} and {logit_scale}")
        return cls(vocab=_integer(data, "vocab"), width=_integer(data, "width"),
                   eps=_positive(_section(data, "norm", ""), "eps", "norm."), residual_mult=mult, logit_scale=logit_scale,
                   embedding_scale=_number(embedding, "scale"), bigram=bigram, loop=loop, layers=tuple(layers))

    def with_stored_shapes(self, shapes: Mapping[str, tuple]) -> "BafavikConfig":
        """The configuration with the sizes that only a checkpoint's tensor shapes give: the inner sizes of the two-step
        projections of the delta rule (the rows of ``l<i>.mix.right.a1`` and ``l<i>.mix.right.g1``)."""
        from dataclasses import replace

        layers = []
        for index, layer in enumerate(self.layers):
            if layer.type == "parallel_2":
                right = layer.mixer.right
                found = {}
                for key, name in (("decay_rank", "a1"), ("gate_rank", "g1")):
                    stored = shapes.get(f"l{index}.mix.right.{name}")
                    if getattr(right, key) is None and stored is not None and len(stored) == 2:
                        found[key] = int(stored[0])
                if found:
                    layer = replace(layer, mixer=replace(layer.mixer, right=replace(right, **found)))
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        layers = [dict(type=layer.type, mixer=layer.mixer.to_dict(), mlp=None if layer.ff is None else dict(kind="dense", ff=layer.ff))
                  for layer in self.layers]
        embedding: dict[str, Any] = dict(scale=self.embedding_scale)
        if self.bigram is not None:
            embedding["bigram"] = dict(buckets=self.bigram.buckets, mul_prev=self.bigram.mul_prev, mul_cur=self.bigram.mul_cur)
        loop = None if self.loop is None else dict(start=self.loop[0], stop=self.loop[1], times=self.loop[2])
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.eps),
                    residual_mult=self.residual_mult, logit_scale=self.logit_scale, embedding=embedding, loop=loop, layers=layers)
