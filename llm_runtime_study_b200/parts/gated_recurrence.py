"""Mixers that keep one float32 number per channel and request: a gated linear recurrence behind a short convolution, and minGRU."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import grouped as G
from ..ops import mixer_steps as M
from ..ops import sequence_state as S
from ..weights.checkpoint import TensorSpec
from .base import MIXERS, FixedState, Mixer, Runtime
from .linear import Projection


@MIXERS.register("gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """Two branches of ``width`` channels: ``y = gelu_tanh(W_y x + b_y)`` and ``u = conv(W_x x + b_x)``, a causal convolution
    over time per channel (``taps`` taps, the last one the current token's, zeros before the start, a bias, no activation).
    ``u`` is cut into ``blocks`` equal parts; in part b ``r = sigmoid(ra[b] u_b + ra.b[b])`` and ``i = sigmoid(ri[b] u_b + ri.b[b])``
    with square matrices ``[out, in]``.  ``log a = -decay_scale * r * softplus(lam)``, ``S_t = a S_(t-1) + sqrt(1 - a^2) i u_t``
    from ``S = 0``; output ``W_o (S * y)``.

    Per request: the float32 state ``[width]`` and the last ``taps - 1`` inputs of the convolution.  Tensors: ``x``, ``x.b``,
    ``y``, ``y.b`` (one stacked product), ``conv``, ``conv.b``, ``ra``, ``ra.b``, ``ri``, ``ri.b``, ``lam``, ``o``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, width: int, blocks: int, taps: int, decay_scale: float = 8.0) -> None:
        if min(hidden_size, width, blocks, taps) <= 0 or width % blocks:
            raise ValueError("recurrence sizes must be positive and the width a multiple of the number of blocks")
        self.hidden_size, self.width, self.blocks, self.taps = hidden_size, width, blocks, taps
        self.block_width = width // blocks
        self.decay_scale = float(decay_scale)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, w, b, bw = self.hidden_size, self.width, self.blocks, self.block_width
        small = dict(init="normal", std=0.5)
        return {
            "x": TensorSpec((w, h)), "x.b": TensorSpec((w,), **small), "y": TensorSpec((w, h)), "y.b": TensorSpec((w,), **small),
            "conv": TensorSpec((w, self.taps), **small), "conv.b": TensorSpec((w,), **small),
            "ra": TensorSpec((b, bw, bw), init="normal", std=bw ** -0.5), "ra.b": TensorSpec((b, bw), **small),
            "ri": TensorSpec((b, bw, bw), init="normal", std=bw ** -0.5), "ri.b": TensorSpec((b, bw), **small),
            "lam": TensorSpec((w,), **small), "o": TensorSpec((h, w)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.in_proj = Projection([tensors["x"], tensors["y"]], [tensors["x.b"], tensors["y.b"]], runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)
        self.conv_taps = runtime.place_vector_f32(tensors["conv"])
        self.conv_bias = runtime.place_vector_f32(tensors["conv.b"])
        # per block: the rows of ra, then the rows of ri (one product gives both gates' logits)
        self.gate_weight = torch.cat([runtime.place_matrix(tensors["ra"]), runtime.place_matrix(tensors["ri"])], dim=1).contiguous()
        self.gate_bias = torch.cat([runtime.place_vector_f32(tensors["ra.b"]), runtime.place_vector_f32(tensors["ri.b"])], dim=1).contiguous()
        self.lam = runtime.place_vector_f32(tensors["lam"])

    def cache_requirement(self):
        needs = [FixedState((self.width,), torch.float32, name="state")]
        if self.taps > 1:
            needs.append(FixedState((self.taps - 1, self.width), torch.float32, name="conv"))
        return tuple(needs)

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        proj = self.in_proj(x)                      # [N, x | y]
        kept = cache.states.get("conv")
        u = M.conv_taps(proj, self.conv_taps, self.conv_bias, kept, q_start=ctx.q_start, slots=ctx.slots, token_entry=ctx.token_entry)
        if self.taps > 1:
            S.conv_state_update(proj, kept, ctx.q_start, ctx.slots)      # its first `width` columns: the x branch
        gates = G.batched_linear(u, self.gate_weight, batch=self.blocks, k=self.block_width, n_out=2 * self.block_width,
                                 a_batch_stride=self.block_width, bias=self.gate_bias, out_dtype=torch.float32)
        out = M.gated_recurrence(gates.view(-1, self.blocks, 2 * self.block_width), u, proj, y_offset=self.width, lam=self.lam,
                                 decay_scale=self.decay_scale, state=cache.states["state"], q_start=ctx.q_start, slots=ctx.slots,
                                 block_width=self.block_width)
        return self.o_proj(out, torch.float32)


@MIXERS.register("min_gru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read the current token only: ``z = sigmoid(W_z x + b_z)``, ``u = W_x x + b_x`` (``width``
    channels each), candidate ``c = u + 1/2`` where ``u >= 0`` and ``sigmoid(u)`` where ``u < 0``, ``S_t = (1 - z_t) S_(t-1) + z_t c_t``
    per channel from ``S = 0``; output ``W_o (S_t * silu(W_g x))``.

    Per request: the float32 state ``[width]``.  Tensors: ``z``, ``z.b``, ``x``, ``x.b``, ``g`` (one stacked product), ``o``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, width: int) -> None:
        if min(hidden_size, width) <= 0:
            raise ValueError("recurrence sizes must be positive")
        self.hidden_size, self.width = hidden_size, width

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, w = self.hidden_size, self.width
        small = dict(init="normal", std=0.5)
        return {"z": TensorSpec((w, h)), "z.b": TensorSpec((w,), **small), "x": TensorSpec((w, h)), "x.b": TensorSpec((w,), **small),
                "g": TensorSpec((w, h)), "o": TensorSpec((h, w))}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        # g has no bias; zero rows bring the number of outputs to a multiple of eight (rows of results then start on 16 bytes)
        pad = -3 * self.width % 8
        weights = [tensors["z"], tensors["x"], tensors["g"]]
        biases = [tensors["z.b"], tensors["x.b"], torch.zeros(self.width + pad, dtype=torch.float32)]
        if pad:
            weights.append(torch.zeros((pad, self.hidden_size), dtype=weights[0].dtype))
        self.in_proj = Projection(weights, biases, runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)

    def cache_requirement(self):
        return FixedState((self.width,), torch.float32, name="state")

    adds_to_residual = True
    fuses_norms = True

    def forward(self, x: Any, ctx: Any, cache: Any, residual: torch.Tensor | None = None, next_norm: Any = None):
        proj = self.in_proj(x)                      # [N, z | u | g]
        segments = None
        # long portions in bfloat16: the scan in segments (its sums are grouped by segment, which the 32-bit path, whose
        # bits do not depend on the cut, must not do); the map is made once a step and shared by the layers
        if (proj.dtype == torch.bfloat16 and not getattr(ctx, "captured", False) and ctx.entry_slots is not None
                and 0 < M.MINGRU_SEGMENT_MIN <= ctx.max_q_len):
            maps = ctx.__dict__.setdefault("_segment_maps", {})
            if "mingru" not in maps:
                maps["mingru"] = M.mingru_segment_map(ctx.q_lens, ctx.entry_slots, proj.device)
            segments = maps["mingru"]
        out = M.mingru_scan(proj, width=self.width, z_offset=0, u_offset=self.width, g_offset=2 * self.width,
                            state=cache.states["state"], q_start=ctx.q_start, slots=ctx.slots, segments=segments)
        return self.o_proj(out, torch.float32, add_to=residual, next_norm=next_norm)
