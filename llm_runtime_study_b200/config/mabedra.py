"""Typed configuration of the Mabedra decoder.

``config.json`` gives the vocabulary, the width, the norms' epsilon, the taps of the short convolution on the sublayers'
inputs and the list of layers; each layer names the type of its mixer (``attention``: differential attention), the
mixer's sizes and constants, and its feed-forward (``dense``, ``moe`` or ``null``).  Every size and constant is read from
there; nothing about a particular model is written in the code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..errors import ConfigError
from .fields import optional, required

NUMBER = (int, float)


@dataclass(frozen=True)
class FrequencyScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class DifferentialAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: int | None
    rot_base: float
    rot_dims: int                       # 0: no rotation
    rot_scaling: FrequencyScaling | None


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class ExpertsFF:
    experts: int
    top: int
    ff: int
    shared_ff: int | None


@dataclass(frozen=True)
class MabedraLayer:
    type: str
    mixer: DifferentialAttention
    mlp: DenseFF | ExpertsFF | None


def _positive(raw: Mapping[str, Any], name: str, where: str) -> int:
    value = required(raw, name, int)
    if value <= 0:
        raise ConfigError(f"{where}.{name} must be positive, got {value}")
    return value


def _window(mixer: Mapping[str, Any], where: str) -> int | None:
    mask = optional(mixer, "mask", (dict, type(None)), None)
    if mask is None:
        return None
    size = optional(mask, "size", (int, type(None)), None)
    if size is not None and size <= 0:
        raise ConfigError(f"{where}.mask.size must be positive, got {size}")
    return size


def _scaling(rot: Mapping[str, Any], where: str) -> FrequencyScaling | None:
    raw = optional(rot, "scaling", (dict, type(None)), None)
    if raw is None:
        return None
    s = FrequencyScaling(*(float(required(raw, k, NUMBER)) for k in ("factor", "low", "high", "original")))
    if s.factor <= 0 or s.original <= 0 or s.low <= 0 or s.high <= s.low:
        raise ConfigError(f"{where}.rot.scaling needs factor > 0, original > 0 and 0 < low < high, got {s}")
    return s


def _attention(mixer: Mapping[str, Any], where: str) -> DifferentialAttention:
    heads = _positive(mixer, "heads", where)
    kv_heads = _positive(mixer, "kv_heads", where) if "kv_heads" in mixer else heads
    if heads % kv_heads:
        raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    dim = _positive(mixer, "dim", where)
    vdim = _positive(mixer, "vdim", where) if "vdim" in mixer else dim
    diff = float(required(mixer, "diff", NUMBER))
    rot = optional(mixer, "rot", (dict, type(None)), None)
    rot_dims = required(rot, "dims", int) if rot else 0
    if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{where}.rot.dims must be even and at most dim {dim}, got {rot_dims}")
    base = float(required(rot, "base", NUMBER)) if rot else 1.0
    if base <= 0:
        raise ConfigError(f"{where}.rot.base must be positive, got {base}")
    return DifferentialAttention(heads, kv_heads, dim, vdim, float(required(mixer, "scale", NUMBER)), diff, _window(mixer, where),
                                 base, rot_dims, _scaling(rot, where) if rot and rot_dims else None)


def _mlp(raw: Mapping[str, Any] | None, where: str) -> DenseFF | ExpertsFF | None:
    if raw is None:
        return None
    kind = required(raw, "kind", str)
    if kind == "dense":
        return DenseFF(_positive(raw, "ff", where))
    if kind == "moe":
        router, expert = required(raw, "router", dict), required(raw, "expert", dict)
        shared = optional(raw, "shared", (dict, type(None)), None)
        mlp = ExpertsFF(_positive(router, "experts", f"{where}.router"), _positive(router, "top", f"{where}.router"),
                        _positive(expert, "ff", f"{where}.expert"), _positive(shared, "ff", f"{where}.shared") if shared else None)
        if mlp.top > mlp.experts:
            raise ConfigError(f"{where}.router: top {mlp.top} exceeds experts {mlp.experts}")
        return mlp
    raise ConfigError(f"{where}.kind {kind!r} is not a feed-forward of this design; expected dense or moe")


def _layer(raw: Any, index: int) -> MabedraLayer:
    where = f"layers[{index}]"
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} must be an object")
    kind = required(raw, "type", str)
    if kind != "attention":
        raise ConfigError(f"{where}: type {kind!r} is not a layer of this design; expected attention")
    return MabedraLayer(kind, _attention(required(raw, "mixer", dict), f"{where}.mixer"),
                        _mlp(optional(raw, "mlp", (dict, type(None)), None), f"{where}.mlp"))


@dataclass(frozen=True)
class MabedraConfig:
    vocab: int
    width: int
    eps: float
    taps: int                           # of the convolution on the sublayers' inputs; 1: none
    layers: tuple[MabedraLayer, ...]

    ARCHITECTURE = "Mabedra"
    MODEL_TYPE = "mabedra"
    # positions enter through rotations and masks only; the engine still wants a bound for its own bookkeeping
    MAX_POSITIONS = 1 << 24

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MabedraConfig":
        norm = required(raw, "norm", dict)
        eps = float(required(norm, "eps", NUMBER))
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        canon = optional(raw, "canon", (dict, type(None)), None)
        taps = _positive(canon, "taps", "canon") if canon else 1
        layers_raw = required(raw, "layers", list)
        if not layers_raw:
            raise ConfigError("layers must not be empty")
        layers = tuple(_layer(item, i) for i, item in enumerate(layers_raw))
        return cls(_positive(raw, "vocab", "config"), _positive(raw, "width", "config"), eps, taps, layers)

    def validate_context_length(self, max_seq_len: int) -> None:
        if max_seq_len <= 0:
            raise ConfigError(f"max_seq_len must be positive, got {max_seq_len}")
        if max_seq_len > self.MAX_POSITIONS:
            raise ConfigError(f"max_seq_len {max_seq_len} exceeds the engine's bound {self.MAX_POSITIONS}")
