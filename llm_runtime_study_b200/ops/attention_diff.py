"""Differential attention over the paged cache: the preparation of q, k and v and the choice of the attention kernel."""

from __future__ import annotations

import ctypes
import os
from typing import Any

import torch

from ..errors import KernelError
from . import native
from .native import c_float, c_int, c_void_p, call, ptr, require, stream_ptr, tag

# "mma": the tensor-core kernel wherever it takes the sizes; "simt": the CUDA-core kernel everywhere
BACKEND = os.environ.get("LLM_RUNTIME_STUDY_B200_ATTENTION_DIFF", "mma")
ROWS_PER_TILE = 64
SINGLE_ROWS = 16          # a single token with at most this many heads a key/value head runs the kernel's second form

_TABLE = {
    "b200_attention_diff_dim": [],
    "b200_attention_diff_vdim": [],
    "b200_attention_diff_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int,
                                 c_float, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, ctypes.c_long,
                                 c_void_p],
}
_SOURCES = ("attention_diff_mma.cu",)


def library_name(head_dim: int, value_dim: int) -> str:
    name = f"b200_attention_diff_d{head_dim}_v{value_dim}"
    if name not in native.library_specs():
        native.register_library(name, _SOURCES, _TABLE, defines=(f"DIFF_DIM={head_dim}", f"DIFF_VDIM={value_dim}"))
    return name


def supported(head_dim: int, value_dim: int) -> bool:
    """Both widths in steps of 16 up to 256: what the tensor-core kernel is built for."""

    return head_dim % 16 == 0 and value_dim % 16 == 0 and 16 <= head_dim <= 256 and 16 <= value_dim <= 256


def build(head_dim: int, value_dim: int) -> None:
    from ..csrc.build import build_library

    name = library_name(head_dim, value_dim)
    build_library(name, _SOURCES, native.library_defines(name))


def map_norm_rope_write(
    rows: torch.Tensor, *, num_q_heads: int, num_kv_heads: int, maps: int, head_dim: int, value_dim: int,
    q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, inv_freq: torch.Tensor | None, rotary_dim: int,
    positions: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor, page_size: int, k_pool: torch.Tensor,
    v_pool: torch.Tensor,
) -> torch.Tensor:
    """Rows ``[q | k | v]`` where every q and k head holds ``maps`` maps of ``head_dim`` columns: each map is RMS-normed
    (weights of ``head_dim`` floats shared by all heads and maps; ``None``: no norm), its first ``rotary_dim`` columns rotated by
    the token's position (pairs ``(i, i + rotary_dim / 2)``; ``inv_freq`` ``None``: no rotation); q is returned
    ``[N, nq, maps * d]``, k goes into the pages ``[pages, nkv, page_size, maps * d]`` and v into ``[pages, nkv, page_size, dv]``."""

    require(rows, "rows", dims=2)
    n, ld = rows.shape
    dt = rows.dtype
    if ld < (num_q_heads + num_kv_heads) * maps * head_dim + num_kv_heads * value_dim:
        raise KernelError(f"rows of width {ld} do not hold (nq + nkv) * maps * d + nkv * dv")
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    for w, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            require(w, name, dtype=torch.float32, shape=(head_dim,))
    if inv_freq is not None:
        require(inv_freq, "inv_freq", dtype=torch.float32, shape=(rotary_dim // 2,))
    require(k_pool, "k_pool", dtype=dt, dims=4)
    require(v_pool, "v_pool", dtype=dt, dims=4)
    if (tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, maps * head_dim)
            or tuple(v_pool.shape[1:]) != (num_kv_heads, page_size, value_dim)):
        raise KernelError(f"pools have shapes {tuple(k_pool.shape)} and {tuple(v_pool.shape)}, expected "
                          f"[pages, {num_kv_heads}, {page_size}, {maps * head_dim} | {value_dim}]")
    q_out = torch.empty((n, num_q_heads, maps * head_dim), dtype=dt, device=rows.device)
    call("b200_map_norm_rope_write", ptr(rows), ld, ptr(q_out), ptr(q_weight), ptr(k_weight), float(eps), ptr(inv_freq),
         rotary_dim if inv_freq is not None else 0, ptr(positions), ptr(token_entry), ptr(block_table), block_table.shape[1],
         page_size, ptr(k_pool), ptr(v_pool), n, num_q_heads, num_kv_heads, maps, head_dim, value_dim, tag(dt), stream_ptr())
    return q_out


def diff_attention_simt(
    q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *, positions: torch.Tensor, token_entry: torch.Tensor,
    block_table: torch.Tensor, scale: float, window: int, lam: float, out_scale: float, eps: float, normalise: bool = True,
) -> torch.Tensor:
    """``o = softmax(S1) V - lam * softmax(S2) V`` per head with ``S_m = scale * q_m . k_m`` over the keys the causal mask and the
    window let through; then ``o / sqrt(mean(o^2) + eps) * out_scale`` over the head's value columns (``normalise``).  q
    ``[N, nq, 2 d]``, keys ``[pages, nkv, page, 2 d]``, values ``[pages, nkv, page, dv]``; result ``[N, nq, dv]``.  32-bit
    arithmetic; the order of every sum depends on the token's position alone."""

    require(q, "q", dims=3)
    n, nq, two_d = q.shape
    require(k_pool, "k_pool", dtype=q.dtype, dims=4)
    require(v_pool, "v_pool", dtype=q.dtype, dims=4)
    _, nkv, page_size, kd = k_pool.shape
    dv = v_pool.shape[3]
    if kd != two_d or two_d % 2 or tuple(v_pool.shape[:3]) != tuple(k_pool.shape[:3]):
        raise KernelError(f"q {tuple(q.shape)}, key pool {tuple(k_pool.shape)} and value pool {tuple(v_pool.shape)} do not fit")
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    out = torch.empty((n, nq, dv), dtype=q.dtype, device=q.device)
    call("b200_diff_attention_simt", ptr(q), ptr(k_pool), ptr(v_pool), ptr(out), ptr(positions), ptr(token_entry), ptr(block_table),
         block_table.shape[1], page_size, n, nq, nkv, two_d // 2, dv, float(scale), int(window), float(lam), float(out_scale),
         float(eps), 1 if normalise else 0, tag(q.dtype), stream_ptr())
    return out


def diff_attention_mma(
    q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx: Any, table: torch.Tensor, *, scale: float, window: int, lam: float,
    out_scale: float, eps: float, normalise: bool = True, splits: int | None = None,
) -> torch.Tensor:
    """The same on tensor cores (bfloat16, both widths in steps of 16): prompt portions and single tokens alike; a tile is up
    to ``64 // min(64, nq // nkv)`` consecutive tokens of one request times the query heads of one key/value head.  A batch of
    single tokens has every token's keys cut into ``splits`` parts (``None``: chosen from the batch), merged by a second launch."""

    require(q, "q", dtype=torch.bfloat16, dims=3)
    n, nq, two_d = q.shape
    require(k_pool, "k_pool", dtype=q.dtype, dims=4)
    require(v_pool, "v_pool", dtype=q.dtype, dims=4)
    _, nkv, page_size, kd = k_pool.shape
    d, dv = two_d // 2, v_pool.shape[3]
    if kd != two_d or two_d % 2 or tuple(v_pool.shape[:3]) != tuple(k_pool.shape[:3]) or nq % nkv:
        raise KernelError(f"q {tuple(q.shape)}, key pool {tuple(k_pool.shape)} and value pool {tuple(v_pool.shape)} do not fit")
    if not supported(d, dv):
        raise KernelError(f"the tensor-core kernel takes widths in steps of 16 up to 256, not {d} and {dv}")
    group_heads = min(nq // nkv, ROWS_PER_TILE)
    slices = -(-(nq // nkv) // group_heads)
    per_tile = max(1, ROWS_PER_TILE // group_heads)
    decode = ctx.all_decode and n == ctx.num_entries
    maps = ctx.__dict__.setdefault("_tile_maps", {})
    key = ("diff", per_tile)
    if key not in maps:
        from . import attention_bf16, attention_latent

        if decode:
            maps[key] = (attention_latent._single_token_tiles(n, q.device), n)      # one tile a request
        else:
            maps[key] = attention_bf16.tile_map(ctx.q_lens, per_tile, q.device, ctx.kv_lens)
    tiles, count = maps[key]
    out = torch.empty((n, nq, dv), dtype=q.dtype, device=q.device)
    scratch, floats = None, 0
    if not decode:
        splits = 1
    elif splits is None:
        splits = decode_splits(n * nkv * slices, min(window, ctx.max_kv_len) if window else ctx.max_kv_len)
    if splits > 1 or (decode and nq // nkv <= SINGLE_ROWS):
        # parts in scratch memory and a merging launch; single tokens with few heads take this way with one part too,
        # since their form of the kernel (every warp on a share of the value columns) leaves parts only
        floats = n * nq * 2 * splits * (dv + 2)
        scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
    native.call("b200_attention_diff_bf16", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), ctx.positions.data_ptr(),
                table.data_ptr(), table.shape[1], page_size, nq, nkv, float(scale), int(window), float(lam), float(out_scale), float(eps),
                1 if normalise else 0, tiles[0].data_ptr(), tiles[1].data_ptr(), tiles[2].data_ptr(), count, splits, ptr(scratch), floats,
                stream_ptr(), library=library_name(d, dv), launches=2 if scratch is not None else 1)
    return out


def decode_splits(ctas: int, keys: int, per_sm: int = 2) -> int:
    """Into how many parts a single token's keys are cut, at most 32: the count for which the launch's waves over the
    multiprocessors (``per_sm`` CTAs each) times the tiles of 32 keys a CTA walks (and three tile times to start and end a
    CTA) is least; the fewest parts among equals."""

    tiles = max(1, -(-keys // 32))
    places = per_sm * native.sm_count()
    best, least = 1, None
    for parts in range(1, min(32, tiles) + 1):
        waves = -(-max(ctas, 1) * parts // places)
        cost = waves * (-(-tiles // parts) + 3)
        if least is None or cost < least:
            best, least = parts, cost
    return best


def diff_attention(q: torch.Tensor, cache, ctx, table: torch.Tensor, *, scale: float, window: int, lam: float, out_scale: float,
                   eps: float) -> torch.Tensor:
    """The differential attention of the batch's query tokens over their requests' pages; chooses the kernel: bfloat16 with
    both widths in steps of 16 runs on tensor cores, float32 and every other size on CUDA cores in 32-bit arithmetic."""

    if BACKEND == "mma" and q.dtype == torch.bfloat16 and supported(q.shape[2] // 2, cache.values.shape[3]):
        return diff_attention_mma(q, cache.keys, cache.values, ctx, table, scale=scale, window=window, lam=lam, out_scale=out_scale, eps=eps)
    return diff_attention_simt(q, cache.keys, cache.values, positions=ctx.positions, token_entry=ctx.token_entry, block_table=table,
                               scale=scale, window=window, lam=lam, out_scale=out_scale, eps=eps)
