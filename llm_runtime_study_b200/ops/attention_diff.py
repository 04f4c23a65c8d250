"""Differential attention over the paged cache: the preparation of q, k and v and the choice of the attention kernel."""

from __future__ import annotations

import torch

from ..errors import KernelError
from .native import call, ptr, require, stream_ptr, tag


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


def diff_attention(q: torch.Tensor, cache, ctx, table: torch.Tensor, *, scale: float, window: int, lam: float, out_scale: float,
                   eps: float) -> torch.Tensor:
    """The differential attention of the batch's query tokens over their requests' pages; chooses the kernel."""

    return diff_attention_simt(q, cache.keys, cache.values, positions=ctx.positions, token_entry=ctx.token_entry, block_table=table,
                               scale=scale, window=window, lam=lam, out_scale=out_scale, eps=eps)
