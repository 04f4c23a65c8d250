"""Softmax attention mixers with a sigmoid gate on their read-out: one over keys and values per head, one over a low-rank
latent per token that all heads share."""

from __future__ import annotations

import math
from typing import Any, Mapping

import torch

from ..ops import attention_latent
from ..ops import attention_rules
from ..ops import functional as F
from ..ops import grouped as G
from ..ops import mixer_steps as M
from ..weights.checkpoint import TensorSpec
from .base import MIXERS, POSITION_ENCODINGS, Mixer, PagedTensors, Runtime
from .linear import Projection
from .linear_state import _padded


@MIXERS.register("gated_attention")
class GatedAttention(Mixer):
    """Grouped-query causal attention without rotation: ``q = W_q x``, ``k = W_k x`` (heads of ``head_dim``), ``v = W_v x``
    (heads of ``value_dim``); every q and k head is divided by its root mean square (``unit_eps`` inside the root, no weight;
    ``None``: left as they are); ``S = scale * q.k``; position i sees j with ``0 <= i - j < window`` (``None``: all before
    it); ordinary softmax; head h's output is multiplied by ``sigmoid(W_g x)_h`` (one number per head); then ``W_o``.
    Query head h reads key/value head ``h // (heads / kv_heads)``.  Tensors: ``q``, ``k``, ``v``, ``g`` (one stacked
    product), ``o``.  Positions enter through the mask only, so the pages hold k and v as they leave the norm."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int | None = None,
                 scale: float | None = None, unit_eps: float | None = None, window: int | None = None) -> None:
        value_dim = head_dim if value_dim is None else value_dim
        if min(hidden_size, num_heads, num_kv_heads, head_dim, value_dim) <= 0:
            raise ValueError("attention sizes must be positive")
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if window is not None and window <= 0:
            raise ValueError("a window must be positive")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.unit_eps = None if unit_eps is None else float(unit_eps)
        self.window = window

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h = self.hidden_size
        return {
            "q": TensorSpec((self.num_heads * self.head_dim, h)), "k": TensorSpec((self.num_kv_heads * self.head_dim, h)),
            "v": TensorSpec((self.num_kv_heads * self.value_dim, h)), "g": TensorSpec((self.num_heads, h)),
            "o": TensorSpec((h, self.num_heads * self.value_dim)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.in_proj = _padded([tensors[n] for n in ("q", "k", "v", "g")], runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)

    def cache_requirement(self) -> PagedTensors:
        return PagedTensors(
            tensors=(("keys", (self.num_kv_heads, self.head_dim)), ("values", (self.num_kv_heads, self.value_dim))),
            window=self.window,
        )

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        proj = self.in_proj(x)
        table = ctx.block_table(cache.group)
        q = M.head_norm_write(
            proj, num_q_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, value_dim=self.value_dim,
            eps=self.unit_eps or 0.0, normalise=self.unit_eps is not None, positions=ctx.positions, token_entry=ctx.token_entry,
            block_table=table, page_size=cache.page_size, k_pool=cache.keys, v_pool=cache.values,
        )
        if self.head_dim == self.value_dim and self.head_dim % 16 == 0:
            out = ctx.attention(q, cache, scale=self.scale, window=self.window or 0)
        else:
            out = F.paged_attention_simt_rules(q, cache.keys, cache.values, positions=ctx.positions, token_entry=ctx.token_entry,
                                               block_table=table, scale=self.scale, window=self.window or 0)
        gate_offset = self.num_heads * self.head_dim + self.num_kv_heads * (self.head_dim + self.value_dim)
        gated = M.sigmoid_gate(out.view(out.shape[0], -1), proj, gate_offset=gate_offset, group=self.value_dim)
        return self.o_proj(gated, torch.float32)


@MIXERS.register("chunked_attention")
class ChunkedAttention(Mixer):
    """Grouped-query causal attention without rotation or value projection: ``q = W_q x``, ``k = W_k x`` (heads of ``head_dim``); the
    values are the keys as projected; then every q and k head is RMS-normed with one weight of ``head_dim`` numbers for all
    heads (``q.norm``, ``k.norm``; ``eps`` inside the root).  ``S = scale * q.k - r1_h ln(1 + r2_h (i - j))`` with two numbers per query
    head (``log_bias``; off: no such term and no ``r1``, ``r2``); position i sees ``j <= i`` in its own block of ``chunk`` positions
    counted from position 0 (``None``: all before it); ordinary softmax; the heads side by side are multiplied element by
    element with ``sigmoid(W_g x)``; then ``W_o``.  Query head h reads key/value head ``h // (heads / kv_heads)``.

    The pages hold the normed keys and, as values, the keys before their norm.  Tensors: ``q``, ``k``, ``g`` (one stacked
    product), ``q.norm``, ``k.norm``, ``r1``, ``r2``, ``o``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, eps: float, scale: float | None = None,
                 chunk: int | None = None, log_bias: bool = True) -> None:
        if min(hidden_size, num_heads, num_kv_heads, head_dim) <= 0:
            raise ValueError("attention sizes must be positive")
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if chunk is not None and chunk <= 0:
            raise ValueError("a chunk must be positive")
        if head_dim > 256:
            raise ValueError(f"head size {head_dim} must be at most 256: no kernel takes a larger one")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.eps, self.chunk, self.log_bias = float(eps), chunk, bool(log_bias)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, d = self.hidden_size, self.head_dim
        specs = {
            "q": TensorSpec((self.num_heads * d, h)), "k": TensorSpec((self.num_kv_heads * d, h)), "g": TensorSpec((self.num_heads * d, h)),
            "q.norm": TensorSpec((d,), init="one_plus_normal", std=0.05), "k.norm": TensorSpec((d,), init="one_plus_normal", std=0.05),
            "o": TensorSpec((h, self.num_heads * d)),
        }
        if self.log_bias:
            specs["r1"] = TensorSpec((self.num_heads,), init="normal", std=0.5)
            specs["r2"] = TensorSpec((self.num_heads,), init="abs_normal", std=0.5)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.in_proj = _padded([tensors[n] for n in ("q", "k", "g")], runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)
        self.q_weight = runtime.place_vector_f32(tensors["q.norm"])
        self.k_weight = runtime.place_vector_f32(tensors["k.norm"])
        self.bias = (runtime.place_vector_f32(tensors["r1"]), runtime.place_vector_f32(tensors["r2"])) if self.log_bias else None

    def cache_requirement(self) -> PagedTensors:
        # a block of the mask is never read from behind its end: what lies a whole block back may be given up
        shape = (self.num_kv_heads, self.head_dim)
        return PagedTensors(tensors=(("keys", shape), ("values", shape)), window=self.chunk)

    adds_to_residual = True
    fuses_norms = True

    def forward(self, x: Any, ctx: Any, cache: Any, residual: torch.Tensor | None = None, next_norm: Any = None):
        proj = self.in_proj(x)                      # [N, q | k | g]
        table = ctx.block_table(cache.group)
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        q = M.head_norm_write(
            proj, num_q_heads=nq, num_kv_heads=nkv, head_dim=d, value_dim=d, eps=self.eps, q_weight=self.q_weight,
            k_weight=self.k_weight, positions=ctx.positions, token_entry=ctx.token_entry, block_table=table,
            page_size=cache.page_size, k_pool=cache.keys, v_pool=cache.values, value_offset=nq * d,
        )
        out = attention_rules.paged_attention_rules(q, cache, ctx, table, scale=self.scale, chunk=self.chunk or 0, log_bias=self.bias)
        gated = M.sigmoid_gate(out.view(out.shape[0], -1), proj, gate_offset=(nq + nkv) * d, group=1)
        return self.o_proj(gated, torch.float32, add_to=residual, next_norm=next_norm)


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Attention whose keys and values are made from one low-rank latent per token (the latent attention of DeepSeek-V2).

    ``c_q = rms_norm(W_dq x)`` (weight ``dq.norm``), ``q = W_uq c_q`` laid out head by head as ``[head_dim plain | rot_dim rotated]``.
    ``W_dkv x`` has ``kv_rank + rot_dim`` rows: the first ``kv_rank``, RMS-normed with ``dkv.norm``, are the latent ``c``; the rest
    is one key part shared by all heads, rotated by the position (``position``: a rotary encoding over the first columns of the
    ``rot_dim``; ``None``: no rotation).  Per
    head the plain key is ``W_uk c`` and the value ``W_uv c``; ``S = scale * (q_plain . k_plain + q_rot . k_rot)``; a window as in
    ``gated_attention``; softmax; the heads side by side are multiplied element by element with ``sigmoid(W_g x)``; then ``W_o``.

    Only ``c`` and the rotated key part are kept per token (one row of ``kv_rank + rot_dim`` columns).  The products with
    ``W_uk`` and ``W_uv`` are moved to the query's side: ``q_plain . (W_uk c) = (W_uk^T q_plain) . c`` and
    ``sum_j p_j W_uv c_j = W_uv sum_j p_j c_j``, so every head attends over the same rows, whose first ``kv_rank`` columns
    are also the values.  ``shares_kv``: the layer has no ``W_dkv`` and reads the rows another layer wrote.  ``keep_window``:
    how far back the kept rows are read by this layer or by any layer that borrows them (``None``: everything).

    Tensors: ``dq``, ``dkv``, ``g`` (one stacked product), ``dq.norm``, ``dkv.norm``, ``uq``, ``uk``, ``uv``, ``o``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int, q_rank: int,
                 eps: float, position: Mapping[str, Any] | None = None, scale: float | None = None, window: int | None = None,
                 shares_kv: bool = False, keep_window: int | None = None) -> None:
        if min(hidden_size, num_heads, head_dim, value_dim, kv_rank, q_rank) <= 0 or rot_dim < 0:
            raise ValueError("latent attention sizes must be positive")
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.value_dim, self.kv_rank, self.q_rank, self.eps = value_dim, kv_rank, q_rank, float(eps)
        self.scale = 1.0 / math.sqrt(head_dim + rot_dim) if scale is None else float(scale)
        self.window, self.shares_kv, self.keep_window = window, bool(shares_kv), keep_window
        self.position = POSITION_ENCODINGS.build(position) if position else None

    def children(self):
        return (self.position,) if self.position is not None else ()

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, H = self.hidden_size, self.num_heads
        specs = {
            "dq": TensorSpec((self.q_rank, h)), "dq.norm": TensorSpec((self.q_rank,), init="one_plus_normal", std=0.05),
            "uq": TensorSpec((H * (self.head_dim + self.rot_dim), self.q_rank)),
            "dkv": TensorSpec((self.kv_rank + self.rot_dim, h)),
            "dkv.norm": TensorSpec((self.kv_rank,), init="one_plus_normal", std=0.05),
            "uk": TensorSpec((H * self.head_dim, self.kv_rank)), "uv": TensorSpec((H * self.value_dim, self.kv_rank)),
            "g": TensorSpec((H * self.value_dim, h)), "o": TensorSpec((h, H * self.value_dim)),
        }
        if self.shares_kv:
            del specs["dkv"], specs["dkv.norm"]
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        names = ("dq", "g") if self.shares_kv else ("dq", "dkv", "g")
        self.in_proj = _padded([tensors[n] for n in names], runtime)
        self.q_weight = runtime.place_vector_f32(tensors["dq.norm"])
        self.kv_weight = None if self.shares_kv else runtime.place_vector_f32(tensors["dkv.norm"])
        self.uq_proj = Projection([tensors["uq"]], None, runtime)
        H = self.num_heads
        # per head: W_uk^T as [kv_rank, head_dim] (the product with it is moved to the query's side), and W_uv [value_dim, kv_rank]
        self.uk = runtime.place_matrix(tensors["uk"]).view(H, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = runtime.place_matrix(tensors["uv"]).view(H, self.value_dim, self.kv_rank)
        self.o_proj = Projection([tensors["o"]], None, runtime)
        if self.position is not None:
            self.position.load({}, runtime)

    def cache_requirement(self) -> PagedTensors | None:
        if self.shares_kv:
            return None
        return PagedTensors(tensors=(("latent", (self.kv_rank + self.rot_dim,)),), window=self.keep_window)

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        proj = self.in_proj(x)
        table = ctx.block_table(cache.group)
        pool = cache.tensors["latent"]
        inv_freq, rot_dims = self.position.rotary_parameters() if self.position is not None else (None, 0)
        own = not self.shares_kv
        cq = M.latent_prepare(
            proj, q_offset=0, q_rank=self.q_rank, q_weight=self.q_weight, eps=self.eps, positions=ctx.positions,
            token_entry=ctx.token_entry, kv_offset=self.q_rank, kv_rank=self.kv_rank if own else 0, kv_weight=self.kv_weight,
            rot=self.rot_dim, rot_dims=rot_dims, inv_freq=inv_freq, block_table=table, page_size=cache.page_size, pool=pool,
        )
        q = self.uq_proj(cq)
        n, H, row = q.shape[0], self.num_heads, self.kv_rank + self.rot_dim
        q_head = self.head_dim + self.rot_dim
        absorbed = torch.empty((n, H * row), dtype=q.dtype, device=q.device)
        G.batched_linear(q, self.uk, batch=H, k=self.head_dim, n_out=self.kv_rank, a_batch_stride=q_head,
                         out=absorbed, out_batch_stride=row)
        if self.rot_dim:
            M.rope_slice(q, absorbed, heads=H, src_head=q_head, src_offset=self.head_dim, dst_head=row, dst_offset=self.kv_rank,
                         rot=self.rot_dim, rot_dims=rot_dims, inv_freq=inv_freq, positions=ctx.positions)
        mixed = attention_latent.latent_attention(absorbed.view(n, H, row), pool, ctx, table, value_dim=self.kv_rank, scale=self.scale,
                                                  window=self.window or 0)
        out = G.batched_linear(mixed.view(n, H * self.kv_rank), self.uv, batch=H, k=self.kv_rank, n_out=self.value_dim,
                               a_batch_stride=self.kv_rank)
        gate_offset = self.q_rank + (self.kv_rank + self.rot_dim if own else 0)
        gated = M.sigmoid_gate(out, proj, gate_offset=gate_offset, group=1)
        return self.o_proj(gated, torch.float32)
