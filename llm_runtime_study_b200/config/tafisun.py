"""Typed configuration of the Tafisun decoder.

``config.json`` gives the vocabulary, the width, the norms' epsilon, the bigram embedding's hash and the list of layers;
each layer names the type of its mixer (``attention`` or ``mingru``), the mixer's sizes and constants, and its
feed-forward (dense, a mixture of experts, or ``null``).  Every size and constant is read from there; nothing about a
particular model is written in the code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..errors import ConfigError
from .fields import optional, required

NUMBER = (int, float)


@dataclass(frozen=True)
class ChunkedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int | None        # positions of one block of the mask; None: every earlier position is seen


@dataclass(frozen=True)
class MinGru:
    width: int


@dataclass(frozen=True)
class Dense:
    ff: int


@dataclass(frozen=True)
class Shared:
    ff: int
    limit: float


@dataclass(frozen=True)
class Experts:
    experts: int         # real experts (with tensors)
    identity: int        # further router outputs that return their input
    top: int
    groups: int
    keep: int
    scale: float
    ff: int
    limit: float
    shared: Shared | None


@dataclass(frozen=True)
class TafisunLayer:
    type: str
    mixer: ChunkedAttention | MinGru
    mlp: Dense | Experts | None


@dataclass(frozen=True)
class Bigram:
    buckets: int
    mul_prev: int
    mul_cur: int


def _positive(raw: Mapping[str, Any], name: str, where: str) -> int:
    value = required(raw, name, int)
    if value <= 0:
        raise ConfigError(f"{where}.{name} must be positive, got {value}")
    return value


def _limit(raw: Mapping[str, Any], where: str) -> float:
    value = float(required(raw, "limit", NUMBER))
    if value <= 0:
        raise ConfigError(f"{where}.limit must be positive, got {value}")
    return value


def _mixer(kind: str, mixer: Mapping[str, Any], where: str):
    if kind == "attention":
        heads = _positive(mixer, "heads", where)
        kv_heads = _positive(mixer, "kv_heads", where) if "kv_heads" in mixer else heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
        dim = _positive(mixer, "dim", where)
        vdim = _positive(mixer, "vdim", where) if "vdim" in mixer else dim
        if vdim != dim:
            raise ConfigError(f"{where}: the values are the projected keys, so vdim {vdim} must equal dim {dim}")
        mask = optional(mixer, "mask", (dict, type(None)), None)
        chunk = optional(mask, "size", (int, type(None)), None) if mask is not None else None
        if chunk is not None and chunk <= 0:
            raise ConfigError(f"{where}.mask.size must be positive, got {chunk}")
        return ChunkedAttention(heads, kv_heads, dim, vdim, float(required(mixer, "scale", NUMBER)), chunk)
    if kind == "mingru":
        return MinGru(_positive(mixer, "width", where))
    raise ConfigError(f"{where}: type {kind!r} is not a layer of this design; expected attention or mingru")


def _mlp(raw: Mapping[str, Any] | None, where: str):
    if raw is None:
        return None
    kind = required(raw, "kind", str)
    if kind == "dense":
        return Dense(_positive(raw, "ff", where))
    if kind != "moe":
        raise ConfigError(f"{where}.kind {kind!r} is not a feed-forward of this design; expected dense or moe")
    router, expert = required(raw, "router", dict), required(raw, "expert", dict)
    rw = f"{where}.router"
    experts, top = _positive(router, "experts", rw), _positive(router, "top", rw)
    identity = optional(router, "identity", int, 0)
    if identity < 0:
        raise ConfigError(f"{rw}.identity must not be negative, got {identity}")
    groups_raw = optional(router, "groups", (dict, type(None)), None)
    groups = _positive(groups_raw, "count", f"{rw}.groups") if groups_raw else 1
    keep = _positive(groups_raw, "keep", f"{rw}.groups") if groups_raw else 1
    outputs = experts + identity
    if outputs % groups:
        raise ConfigError(f"{rw}: {outputs} router outputs do not form {groups} equal groups")
    if keep > groups:
        raise ConfigError(f"{rw}.groups: keep {keep} exceeds count {groups}")
    if top > keep * (outputs // groups):
        raise ConfigError(f"{rw}: top {top} exceeds the {keep * (outputs // groups)} outputs of the groups that are kept")
    shared_raw = optional(raw, "shared", (dict, type(None)), None)
    shared = Shared(_positive(shared_raw, "ff", f"{where}.shared"), _limit(shared_raw, f"{where}.shared")) if shared_raw else None
    return Experts(experts, identity, top, groups, keep, float(optional(router, "scale", NUMBER, 1.0)),
                   _positive(expert, "ff", f"{where}.expert"), _limit(expert, f"{where}.expert"), shared)


def _layer(raw: Any, index: int) -> TafisunLayer:
    where = f"layers[{index}]"
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} must be an object")
    kind = required(raw, "type", str)
    typed = _mixer(kind, required(raw, "mixer", dict), f"{where}.mixer")
    return TafisunLayer(kind, typed, _mlp(optional(raw, "mlp", (dict, type(None)), None), f"{where}.mlp"))


@dataclass(frozen=True)
class TafisunConfig:
    vocab: int
    width: int
    eps: float
    bigram: Bigram | None
    layers: tuple[TafisunLayer, ...]

    ARCHITECTURE = "Tafisun"
    MODEL_TYPE = "tafisun"
    # positions enter through the sinusoid and the masks only; the engine still wants a bound for its own bookkeeping
    MAX_POSITIONS = 1 << 24

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TafisunConfig":
        norm = required(raw, "norm", dict)
        eps = float(required(norm, "eps", NUMBER))
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        layers_raw = required(raw, "layers", list)
        if not layers_raw:
            raise ConfigError("layers must not be empty")
        layers = tuple(_layer(item, i) for i, item in enumerate(layers_raw))
        width = _positive(raw, "width", "config")
        for i, layer in enumerate(layers):
            if isinstance(layer.mixer, MinGru) and layer.mixer.width <= 0:
                raise ConfigError(f"layers[{i}].mixer.width must be positive")
        embedding = optional(raw, "embedding", (dict, type(None)), None) or {}
        bigram_raw = optional(embedding, "bigram", (dict, type(None)), None)
        bigram = None
        if bigram_raw is not None:
            bigram = Bigram(_positive(bigram_raw, "buckets", "embedding.bigram"), required(bigram_raw, "mul_prev", int),
                            required(bigram_raw, "mul_cur", int))
            if bigram.mul_prev < 0 or bigram.mul_cur < 0:
                raise ConfigError("embedding.bigram: the multipliers must not be negative")
        return cls(_positive(raw, "vocab", "config"), width, eps, bigram, layers)

    def validate_context_length(self, max_seq_len: int) -> None:
        if max_seq_len <= 0:
            raise ConfigError(f"max_seq_len must be positive, got {max_seq_len}")
        if max_seq_len > self.MAX_POSITIONS:
            raise ConfigError(f"max_seq_len {max_seq_len} exceeds the engine's bound {self.MAX_POSITIONS}")
