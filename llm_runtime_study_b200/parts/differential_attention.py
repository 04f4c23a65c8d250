"""Differential attention: two softmax maps per head over the same values, the second subtracted."""

from __future__ import annotations

import math
from typing import Any, Mapping

import torch

from ..ops import attention_diff as A
from ..weights.checkpoint import TensorSpec
from .base import MIXERS, POSITION_ENCODINGS, Mixer, PagedTensors, Runtime
from .linear import Projection


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """Grouped-query causal attention in which every head has two score maps (the differential attention of the
    Differential Transformer).  ``q = W_q x + b_q`` has ``heads * 2 * head_dim`` rows and ``k = W_k x + b_k`` has
    ``kv_heads * 2 * head_dim``, laid out head by head as ``[map 1 | map 2]``; ``v = W_v x + b_v`` has ``kv_heads * value_dim``.
    Every map of q and of k is RMS-normed over ``head_dim`` (weights ``q.norm`` / ``k.norm`` shared by all heads and maps),
    then rotated (``position``: a rotary encoding over the map's leading columns; ``None``: none).  ``S_m = scale * q_m . k_m``;
    position i sees j with ``0 <= i - j < window`` (``None``: all before it); ``a_m = softmax(S_m) v``.  With
    ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` (one number for the layer, float32) the head's output is
    ``o = a_1 - lambda a_2``, divided by its root mean square over ``value_dim`` (``eps`` inside the root, no weight) and
    scaled by ``1 - diff``; then ``W_o`` on the heads side by side.  Query head h reads key/value head
    ``h // (heads / kv_heads)``.

    The pages hold one key row of both maps (``2 * head_dim`` columns) and one value row per token and kv head, so one pass
    over the keys and one over the values serve both maps.  Tensors: ``q``, ``k``, ``v`` (one stacked product) with biases
    ``q.b``, ``k.b``, ``v.b``; ``q.norm``, ``k.norm``; ``lq1``, ``lk1``, ``lq2``, ``lk2``; ``o``."""

    graph_safe = True
    MAPS = 2

    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int | None = None,
                 scale: float | None = None, diff: float, eps: float, window: int | None = None,
                 position: Mapping[str, Any] | None = None, bias: bool = True) -> None:
        value_dim = head_dim if value_dim is None else value_dim
        if min(hidden_size, num_heads, num_kv_heads, head_dim, value_dim) <= 0:
            raise ValueError("attention sizes must be positive")
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if window is not None and window <= 0:
            raise ValueError("a window must be positive")
        if head_dim > 512 or value_dim > 256:
            raise ValueError(f"head sizes {head_dim} and {value_dim} exceed 512 and 256: no kernel takes larger ones")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.diff, self.eps, self.window, self.bias = float(diff), float(eps), window, bool(bias)
        self.position = POSITION_ENCODINGS.build(position) if position else None

    def children(self):
        return (self.position,) if self.position is not None else ()

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, d = self.hidden_size, self.head_dim
        q_out, k_out, v_out = self.num_heads * self.MAPS * d, self.num_kv_heads * self.MAPS * d, self.num_kv_heads * self.value_dim
        specs = {
            "q": TensorSpec((q_out, h)), "k": TensorSpec((k_out, h)), "v": TensorSpec((v_out, h)),
            "q.norm": TensorSpec((d,), init="one_plus_normal", std=0.05), "k.norm": TensorSpec((d,), init="one_plus_normal", std=0.05),
            "o": TensorSpec((h, self.num_heads * self.value_dim)),
        }
        if self.bias:
            small = dict(init="normal", std=0.1)
            specs.update({"q.b": TensorSpec((q_out,), **small), "k.b": TensorSpec((k_out,), **small), "v.b": TensorSpec((v_out,), **small)})
        for name in ("lq1", "lk1", "lq2", "lk2"):
            specs[name] = TensorSpec((d,), init="normal", std=0.1)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        names = ("q", "k", "v")
        self.qkv_proj = Projection([tensors[n] for n in names], [tensors[f"{n}.b"] for n in names] if self.bias else None, runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)
        self.q_weight = runtime.place_vector_f32(tensors["q.norm"])
        self.k_weight = runtime.place_vector_f32(tensors["k.norm"])
        # one number for the layer, formed once in float32
        l = {n: tensors[n].to(torch.float32).cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
        lam = torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum()) + torch.tensor(self.diff, dtype=torch.float32)
        self.lam = float(lam)
        if self.position is not None:
            self.position.load({}, runtime)

    def cache_requirement(self) -> PagedTensors:
        return PagedTensors(
            tensors=(("keys", (self.num_kv_heads, self.MAPS * self.head_dim)), ("values", (self.num_kv_heads, self.value_dim))),
            window=self.window,
        )

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        qkv = self.qkv_proj(x)
        table = ctx.block_table(cache.group)
        rotary = self.position.rotary_parameters() if self.position is not None else None
        if self.position is not None and rotary is None:
            raise ValueError("differential_attention rotates with a rotary encoding only")
        q = A.map_norm_rope_write(
            qkv, num_q_heads=self.num_heads, num_kv_heads=self.num_kv_heads, maps=self.MAPS, head_dim=self.head_dim,
            value_dim=self.value_dim, q_weight=self.q_weight, k_weight=self.k_weight, eps=self.eps,
            inv_freq=rotary[0] if rotary else None, rotary_dim=rotary[1] if rotary else 0, positions=ctx.positions,
            token_entry=ctx.token_entry, block_table=table, page_size=cache.page_size, k_pool=cache.keys, v_pool=cache.values,
        )
        out = A.diff_attention(q, cache, ctx, table, scale=self.scale, window=self.window or 0, lam=self.lam,
                               out_scale=1.0 - self.diff, eps=self.eps)
        return self.o_proj(out.view(out.shape[0], -1), torch.float32)
