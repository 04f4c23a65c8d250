"""Choice of the kernel for attention with rules on the scores (soft cap, bias by distance, sink)."""

from __future__ import annotations

import os
from typing import Any

import torch

from . import attention_bf16, native
from . import functional as F

# "tcgen05": the tensor-core kernels wherever they take the shape (tcgen05 for prompt portions of head size 64 and
# 128, mma.sync otherwise); "mma": mma.sync only; "simt": the CUDA-core kernel everywhere
BACKEND = os.environ.get("LLM_RUNTIME_STUDY_B200_ATTENTION_RULES", "tcgen05")


def tensor_core_supported(q: torch.Tensor, cache: Any) -> bool:
    """bfloat16, keys and values of one head size that the mma.sync kernels are built for."""

    d = q.shape[2]
    return (q.dtype == torch.bfloat16 and cache.values.shape[3] == d and attention_bf16.supported(d))


def paged_attention_rules(q: torch.Tensor, cache: Any, ctx: Any, table: torch.Tensor, *, scale: float, window: int = 0,
                          softcap: float = 0.0, slopes: torch.Tensor | None = None, sink: bool = False, chunk: int = 0,
                          log_bias: "tuple[torch.Tensor, torch.Tensor] | None" = None) -> torch.Tensor:
    """Causal attention of the batch's query tokens ``[N, heads, d]`` over their requests' pages with
    ``S <- cap * tanh(S / cap)``, ``S <- S - slope_h * distance``, ``S <- S - r1_h ln(1 + r2_h * distance)`` (``log_bias = (r1, r2)``),
    the sink's ``1 +`` in the denominator, and a mask in blocks (``chunk > 0``: a position sees its own block of ``chunk``
    positions, counted from 0, only).

    float32 runtime, and shapes no tensor-core kernel takes (values of another head size than the keys): the
    CUDA-core kernel (one warp per token and head, float32 arithmetic, tiles of 32 keys from key 0, so the order
    of every sum depends on the token's position alone).  bfloat16 runtime: the kernels of the plain attention,
    built a second time with the rules applied to the score tile: for batches that hold prompt portions the tcgen05
    kernel with one row tile per CTA (head sizes 64 and 128, portions of 32 tokens and more, no window) or the
    mma.sync kernel; for batches of single decoded tokens the split-sequence mma.sync kernel with its merge."""

    if chunk or log_bias is not None:
        return _masked(q, cache, ctx, table, scale=scale, window=window, softcap=softcap, slopes=slopes, sink=sink, chunk=chunk,
                       log_bias=log_bias)
    if BACKEND in ("mma", "tcgen05") and tensor_core_supported(q, cache):
        n, nq, d = q.shape
        keys, values = cache.keys, cache.values
        _, _, _, nkv, page_size, gs, slices = attention_bf16._geometry(q, keys)
        lib = attention_bf16.library_name(d)
        out = torch.empty_like(q)
        if ctx.all_decode and n == ctx.num_entries:
            splits = attention_bf16.decode_splits(n, nkv, slices, ctx.max_kv_len, head_dim=d)
            floats = native.query("b200_attention_decode_scratch_floats", n, nq, splits, library=lib)
            scratch = torch.empty(max(floats, 1), dtype=torch.float32, device=q.device)
            native.call(
                "b200_attention_decode_rules_bf16", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
                ctx.kv_len.data_ptr(), table.data_ptr(), table.shape[1], page_size, n, nq, nkv, float(scale), int(window),
                float(softcap), native.ptr(slopes), 1 if sink else 0, splits, scratch.data_ptr(), floats, native.stream_ptr(),
                library=lib, launches=2 if splits > 1 else 1)
            return out
        maps = ctx.__dict__.setdefault("_tile_maps", {})
        if (BACKEND == "tcgen05" and attention_bf16.PREFILL_BACKEND == "tcgen05" and attention_bf16.tc_supported(d, page_size, window)
                and ctx.max_q_len >= attention_bf16.TC_MIN_PORTION):
            per_tile = 128 // gs
            key = ("tc", per_tile)
            if key not in maps:
                maps[key] = attention_bf16.tile_map(ctx.q_lens, per_tile, q.device, ctx.kv_lens)
            tiles, count = maps[key]
            native.call(
                "b200_attention_prefill_tcgen05_rules", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
                ctx.positions.data_ptr(), table.data_ptr(), table.shape[1], page_size, keys.shape[0], n, nq, nkv, float(scale),
                float(softcap), native.ptr(slopes), 1 if sink else 0, tiles[0].data_ptr(), tiles[1].data_ptr(), tiles[2].data_ptr(),
                count, native.stream_ptr(), library=attention_bf16.tc_library_name(d))
            return out
        per_tile = 64 // gs
        if per_tile not in maps:
            maps[per_tile] = attention_bf16.tile_map(ctx.q_lens, per_tile, q.device, ctx.kv_lens)
        tiles, count = maps[per_tile]
        native.call(
            "b200_attention_prefill_rules_bf16", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
            ctx.positions.data_ptr(), table.data_ptr(), table.shape[1], page_size, nq, nkv, float(scale), int(window),
            float(softcap), native.ptr(slopes), 1 if sink else 0, tiles[0].data_ptr(), tiles[1].data_ptr(), tiles[2].data_ptr(),
            count, native.stream_ptr(), library=lib)
        return out
    return F.paged_attention_simt_rules(
        q, cache.keys, cache.values, positions=ctx.positions, token_entry=ctx.token_entry, block_table=table,
        scale=scale, window=window, softcap=softcap, slopes=slopes, sink=sink,
    )


def _masked(q: torch.Tensor, cache: Any, ctx: Any, table: torch.Tensor, *, scale: float, window: int, softcap: float,
            slopes: torch.Tensor | None, sink: bool, chunk: int, log_bias) -> torch.Tensor:
    """The forms with a mask in blocks or a bias by the logarithm of the distance: the mma.sync kernels with rules (bfloat16,
    one head size for keys and values that they are built for), the split-sequence kernel for batches of single tokens (a
    token reads its own block at most, so the parts are sized for the block), else the CUDA-core kernel."""

    r1, r2 = log_bias if log_bias is not None else (None, None)
    if BACKEND in ("mma", "tcgen05") and tensor_core_supported(q, cache):
        n, nq, d = q.shape
        keys, values = cache.keys, cache.values
        _, _, _, nkv, page_size, gs, slices = attention_bf16._geometry(q, keys)
        lib = attention_bf16.library_name(d)
        out = torch.empty_like(q)
        if ctx.all_decode and n == ctx.num_entries:
            reach = min(ctx.max_kv_len, chunk) if chunk else ctx.max_kv_len
            splits = attention_bf16.decode_splits(n, nkv, slices, reach, head_dim=d)
            floats = native.query("b200_attention_decode_scratch_floats", n, nq, splits, library=lib)
            scratch = torch.empty(max(floats, 1), dtype=torch.float32, device=q.device)
            native.call(
                "b200_attention_decode_masked_bf16", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
                ctx.kv_len.data_ptr(), table.data_ptr(), table.shape[1], page_size, n, nq, nkv, float(scale), int(window),
                float(softcap), native.ptr(slopes), 1 if sink else 0, int(chunk), native.ptr(r1), native.ptr(r2), splits,
                scratch.data_ptr(), floats, native.stream_ptr(), library=lib, launches=2 if splits > 1 else 1)
            return out
        maps = ctx.__dict__.setdefault("_tile_maps", {})
        per_tile = 64 // gs
        if per_tile not in maps:
            maps[per_tile] = attention_bf16.tile_map(ctx.q_lens, per_tile, q.device, ctx.kv_lens)
        tiles, count = maps[per_tile]
        native.call(
            "b200_attention_prefill_masked_bf16", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
            ctx.positions.data_ptr(), table.data_ptr(), table.shape[1], page_size, nq, nkv, float(scale), int(window),
            float(softcap), native.ptr(slopes), 1 if sink else 0, int(chunk), native.ptr(r1), native.ptr(r2),
            tiles[0].data_ptr(), tiles[1].data_ptr(), tiles[2].data_ptr(), count, native.stream_ptr(), library=lib)
        return out
    return F.paged_attention_simt_rules(
        q, cache.keys, cache.values, positions=ctx.positions, token_entry=ctx.token_entry, block_table=table,
        scale=scale, window=window, softcap=softcap, slopes=slopes, sink=sink, chunk=chunk, log_bias=log_bias,
    )
