"""Gated feed-forward (SwiGLU)."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import block_steps as B
from ..ops import functional as F
from ..weights.checkpoint import TensorSpec
from .base import FEED_FORWARDS, FeedForward, Runtime
from .linear import Projection


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """``down(silu(gate(x)) * up(x))`` without biases (mini_llm/nn/mlp.py:80-87).
    gate and up are one stacked product; the activation and the product with
    ``up`` are computed in float32 and rounded once."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int) -> None:
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("swiglu sizes must be positive")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        gate, up = runtime.place_matrix(tensors["gate_proj.weight"]), runtime.place_matrix(tensors["up_proj.weight"])
        # When the width allows, gate and up rows are interleaved in blocks of eight
        # ([g0..g7, u0..u7, g8..g15, ...]): a projection kernel then holds matching gate and
        # up features in one tile and can apply SiLU * up before it writes anything.
        self.interleaved = self.intermediate_size % 8 == 0
        if self.interleaved:
            blocks = self.intermediate_size // 8
            stacked = torch.stack((gate.view(blocks, 8, -1), up.view(blocks, 8, -1)), dim=1).reshape(2 * self.intermediate_size, -1)
            del gate, up
            self.gate_up_proj = Projection([stacked], None, runtime)
            del stacked
        else:
            self.gate_up_proj = Projection([gate, up], None, runtime)
        self.down_proj = Projection([tensors["down_proj.weight"]], None, runtime)

    adds_to_residual = True
    fuses_norms = True

    def forward(self, x: Any, ctx: Any, residual: torch.Tensor | None = None, next_norm: Any = None):
        hidden = self.gate_up_proj.swiglu(x) if self.interleaved else F.silu_mul(self.gate_up_proj(x))
        return self.down_proj(hidden, torch.float32, add_to=residual, next_norm=next_norm)


@FEED_FORWARDS.register("limited_glu")
class LimitedGLU(FeedForward):
    """``g = min(W_gate x + b_gate, limit)``, ``u = clamp(W_up x + b_up, -limit, limit)``,
    ``y = g * sigmoid(alpha g) * (u + 1)``, output ``W_down y + b_down``.  gate and up are one stacked
    product.  Tensors: ``gate``, ``gate.b``, ``up``, ``up.b``, ``down``, ``down.b``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702) -> None:
        if hidden_size <= 0 or intermediate_size <= 0 or limit <= 0:
            raise ValueError("limited_glu sizes and its limit must be positive")
        self.hidden_size, self.intermediate_size, self.limit, self.alpha = hidden_size, intermediate_size, float(limit), float(alpha)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate": TensorSpec((i, h)), "gate.b": TensorSpec((i,)), "up": TensorSpec((i, h)), "up.b": TensorSpec((i,)),
            "down": TensorSpec((h, i)), "down.b": TensorSpec((h,)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.gate_up_proj = Projection([tensors["gate"], tensors["up"]], [tensors["gate.b"], tensors["up.b"]], runtime)
        self.down_proj = Projection([tensors["down"]], [tensors["down.b"]], runtime)

    adds_to_residual = True

    def forward(self, x: Any, ctx: Any, residual: torch.Tensor | None = None):
        hidden = F.glu_limit(self.gate_up_proj(x), self.limit, self.alpha)
        return self.down_proj(hidden, torch.float32, add_to=residual)


@FEED_FORWARDS.register("relu2_mlp")
class SquaredReluMLP(FeedForward):
    """``W_down relu(W_up x)^2`` without biases.  Tensors: ``up``, ``down``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int) -> None:
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("relu2_mlp sizes must be positive")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"up": TensorSpec((self.intermediate_size, self.hidden_size)), "down": TensorSpec((self.hidden_size, self.intermediate_size))}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.up_proj = Projection([tensors["up"]], None, runtime)
        self.down_proj = Projection([tensors["down"]], None, runtime)

    adds_to_residual = True
    fuses_norms = True

    def forward(self, x: Any, ctx: Any, residual: torch.Tensor | None = None, next_norm: Any = None):
        return self.down_proj(F.relu2(self.up_proj(x)), torch.float32, add_to=residual, next_norm=next_norm)


@FEED_FORWARDS.register("poly_norm_mlp")
class PolyNormMLP(FeedForward):
    """``W_down act(W_up x)`` without biases, ``act(z) = a u(z) + b u(z^2) + c u(z^3) + e`` with element-wise powers and
    ``u(y) = y / sqrt(mean(y^2) + eps)`` over a token's ``intermediate_size`` values (statistics in float32).  Tensors:
    ``up``, ``down``, ``act`` (the four numbers a, b, c, e)."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int, eps: float) -> None:
        if hidden_size <= 0 or intermediate_size <= 0 or eps <= 0:
            raise ValueError("poly_norm_mlp sizes and eps must be positive")
        self.hidden_size, self.intermediate_size, self.eps = hidden_size, intermediate_size, float(eps)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {"up": TensorSpec((i, h)), "down": TensorSpec((h, i)), "act": TensorSpec((4,), init="normal", std=0.5)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.up_proj = Projection([tensors["up"]], None, runtime)
        self.down_proj = Projection([tensors["down"]], None, runtime)
        self.coef = runtime.place_vector_f32(tensors["act"])

    def forward(self, x: Any, ctx: Any) -> torch.Tensor:
        return self.down_proj(B.poly_norm(self.up_proj(x), self.coef, self.eps), torch.float32)
