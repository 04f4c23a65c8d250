"""Rotary position encoding (half-split convention)."""

from __future__ import annotations

import math
from typing import Mapping

import torch

from .base import POSITION_ENCODINGS, PositionEncoding, Runtime


@POSITION_ENCODINGS.register("rope")
class RotaryEmbedding(PositionEncoding):
    """``inv_freq[i] = 1 / theta^(2i / rotary_dim)``, built in float32 on the host
    with the same expression as the reference (mini_llm/nn/rope.py:37-40); the
    angle ``float32(position) * inv_freq[i]`` and its sine and cosine are formed
    in float32 inside the fused kernel (mini_llm/nn/rope.py:74-80).  Pairs are
    ``(i, i + rotary_dim/2)`` (mini_llm/nn/rope.py:110-114).  ``rotary_dim``
    smaller than the head size leaves the remaining columns unrotated.

    ``scaling`` (``factor``, ``low``, ``high``, ``original``) stretches long wavelengths: with ``l = 2 pi / f`` a frequency
    is kept where ``l < original / high``, divided by ``factor`` where ``l > original / low``, and in between blended as
    ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)`` (formed in float64, kept in float32)."""

    graph_safe = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None,
                 scaling: Mapping[str, float] | None = None) -> None:
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if head_dim <= 0 or rotary_dim <= 0 or rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"rope needs an even rotary_dim in (0, head_dim], got {rotary_dim}, {head_dim}")
        if theta <= 0:
            raise ValueError(f"rope theta must be positive, got {theta}")
        self.head_dim, self.theta, self.rotary_dim = head_dim, float(theta), rotary_dim
        self.scaling = None
        if scaling:
            self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
            if self.scaling["factor"] <= 0 or self.scaling["original"] <= 0 or not 0 < self.scaling["low"] < self.scaling["high"]:
                raise ValueError(f"rope scaling needs factor > 0, original > 0 and 0 < low < high, got {self.scaling}")
        self.inv_freq: torch.Tensor | None = None

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        dims = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        if self.scaling is None:
            self.inv_freq = (1.0 / (self.theta ** (dims / self.rotary_dim))).to(runtime.device)
            return
        s = self.scaling
        f = self.theta ** (-dims.to(torch.float64) / self.rotary_dim)
        wavelength = 2.0 * math.pi / f
        blend = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
        blended = (1.0 - blend) * f / s["factor"] + blend * f
        f = torch.where(wavelength < s["original"] / s["high"], f,
                        torch.where(wavelength > s["original"] / s["low"], f / s["factor"], blended))
        self.inv_freq = f.to(torch.float32).to(runtime.device)

    def rotary_parameters(self) -> tuple[torch.Tensor, int]:
        return self.inv_freq, self.rotary_dim
