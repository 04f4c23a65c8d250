"""Small kernels around mixers: per-head norm and page write, what a latent attention keeps per token, rotation of a
slice of every head, sigmoid gates on a read-out, the norm on a sublayer's output, and the gated linear recurrence
behind a short convolution.  Statistics, angles, gates and states are float32 in both run types."""

from __future__ import annotations

import os

import torch

from dataclasses import dataclass

from ..errors import KernelError
from .native import call, ptr, query, require, stream_ptr, tag


@dataclass
class PairedRows:
    """A sublayer's output given in pieces: row ``t`` is ``sum_j weights[t, j] * rows[pair_row[t * top + j]]`` (what the experts a
    router chose returned for token ``t``).  A consumer that reads the rows anyway forms the sum itself."""

    rows: torch.Tensor          # float32 [sorted rows, width]
    pair_row: torch.Tensor      # int32 [N * top]
    weights: torch.Tensor       # float32 [N, top]



def head_norm_write(
    rows: torch.Tensor, *, num_q_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, eps: float,
    q_weight: torch.Tensor | None = None, k_weight: torch.Tensor | None = None, normalise: bool = True,
    positions: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor, page_size: int,
    k_pool: torch.Tensor, v_pool: torch.Tensor, value_offset: int | None = None,
) -> torch.Tensor:
    """Rows ``[q | k | v | ...]``: every q and k head divided by its root mean square (``eps`` inside the root), times a
    weight of ``head_dim`` floats where given; q is returned ``[N, nq, d]``, k and v go into the pages
    ``[pages, nkv, page_size, d | dv]`` at each token's position.  ``value_offset``: the column at which the values' heads
    start (default: behind the keys); ``nq * d`` makes the values the keys as projected, before their norm."""

    require(rows, "rows", dims=2)
    n, ld = rows.shape
    if value_offset is None:
        value_offset = (num_q_heads + num_kv_heads) * head_dim
    if ld < (num_q_heads + num_kv_heads) * head_dim or value_offset < 0 or ld < value_offset + num_kv_heads * value_dim:
        raise KernelError(f"rows of width {ld} do not hold nq*d + nkv*d and the values at column {value_offset}")
    dt = rows.dtype
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    for w, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            require(w, name, dtype=torch.float32, shape=(head_dim,))
    require(k_pool, "k_pool", dtype=dt, dims=4)
    require(v_pool, "v_pool", dtype=dt, dims=4)
    if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or tuple(v_pool.shape[1:]) != (num_kv_heads, page_size, value_dim):
        raise KernelError(f"pools have shapes {tuple(k_pool.shape)} and {tuple(v_pool.shape)}, expected "
                          f"[pages, {num_kv_heads}, {page_size}, {head_dim} | {value_dim}]")
    q_out = torch.empty((n, num_q_heads, head_dim), dtype=dt, device=rows.device)
    call("b200_head_norm_write_at", ptr(rows), ld, ptr(q_out), ptr(q_weight), ptr(k_weight), float(eps), 1 if normalise else 0,
         ptr(positions), ptr(token_entry), ptr(block_table), block_table.shape[1], page_size, ptr(k_pool), ptr(v_pool), n,
         num_q_heads, num_kv_heads, head_dim, value_dim, int(value_offset), tag(dt), stream_ptr())
    return q_out


def latent_prepare(
    rows: torch.Tensor, *, q_offset: int, q_rank: int, q_weight: torch.Tensor, eps: float, positions: torch.Tensor,
    token_entry: torch.Tensor, kv_offset: int = 0, kv_rank: int = 0, kv_weight: torch.Tensor | None = None, rot: int = 0,
    rot_dims: int = 0, inv_freq: torch.Tensor | None = None, block_table: torch.Tensor | None = None, page_size: int = 0,
    pool: torch.Tensor | None = None,
) -> torch.Tensor:
    """From rows of a stacked projection: columns ``q_offset .. + q_rank`` RMS-normed with ``q_weight`` are returned
    ``[N, q_rank]``; with ``kv_rank > 0`` columns ``kv_offset .. + kv_rank`` RMS-normed with ``kv_weight`` and the ``rot``
    columns behind them (the first ``rot_dims`` rotated by the position, pairs ``(i, i + rot_dims/2)``) are written into
    the pages ``[pages, page_size, kv_rank + rot]``."""

    require(rows, "rows", dims=2)
    n, ld = rows.shape
    dt = rows.dtype
    require(q_weight, "q_weight", dtype=torch.float32, shape=(q_rank,))
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    stride = 0
    if kv_rank > 0:
        require(kv_weight, "kv_weight", dtype=torch.float32, shape=(kv_rank,))
        require(block_table, "block_table", dtype=torch.int32, dims=2)
        stride = block_table.shape[1]
        require(pool, "pool", dtype=dt, dims=3)
        if tuple(pool.shape[1:]) != (page_size, kv_rank + rot):
            raise KernelError(f"pool has shape {tuple(pool.shape)}, expected [pages, {page_size}, {kv_rank + rot}]")
        if rot_dims:
            require(inv_freq, "inv_freq", dtype=torch.float32, shape=(rot_dims // 2,))
    out = torch.empty((n, q_rank), dtype=dt, device=rows.device)
    call("b200_latent_prepare", ptr(rows), ld, q_offset, q_rank, ptr(q_weight), ptr(out), kv_offset, kv_rank, ptr(kv_weight), rot,
         rot_dims, ptr(inv_freq), float(eps), ptr(positions), ptr(token_entry), ptr(block_table), stride, page_size, ptr(pool), n,
         tag(dt), stream_ptr())
    return out


def rope_slice(src: torch.Tensor, dst: torch.Tensor, *, heads: int, src_head: int, src_offset: int, dst_head: int,
               dst_offset: int, rot: int, rot_dims: int, inv_freq: torch.Tensor, positions: torch.Tensor) -> None:
    """Columns ``src_offset .. + rot`` of every head of ``src`` (``[N, heads * src_head]``), the first ``rot_dims`` of them
    rotated by the token's position, are written to columns ``dst_offset ..`` of every head of ``dst``."""

    require(src, "src", dims=2)
    require(dst, "dst", dtype=src.dtype, dims=2)
    n = src.shape[0]
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    if rot_dims:
        require(inv_freq, "inv_freq", dtype=torch.float32, shape=(rot_dims // 2,))
    if src.shape[1] < heads * src_head or dst.shape[1] < heads * dst_head or dst.shape[0] != n:
        raise KernelError("rope_slice: the heads do not fit the rows")
    call("b200_rope_slice", ptr(src), src.shape[1], src_head, src_offset, ptr(dst), dst.shape[1], dst_head, dst_offset, heads, rot,
         rot_dims, ptr(inv_freq), ptr(positions), n, tag(src.dtype), stream_ptr())


def sigmoid_gate(x: torch.Tensor, gate_rows: torch.Tensor, *, gate_offset: int, group: int) -> torch.Tensor:
    """``x[t, c] * sigmoid(gate_rows[t, gate_offset + c // group])``: one gate per ``group`` columns, read out of the rows of a
    stacked projection.  ``x`` ``[N, width]`` in the activation type; a new tensor of that type is returned."""

    require(x, "x", dims=2)
    require(gate_rows, "gate_rows", dtype=x.dtype, dims=2)
    n, width = x.shape
    if gate_rows.shape[0] != n or gate_offset + -(-width // group) > gate_rows.shape[1]:
        raise KernelError("sigmoid_gate: the gate's columns lie outside gate_rows")
    out = torch.empty_like(x)
    call("b200_sigmoid_gate", ptr(x), gate_rows.data_ptr() + gate_offset * gate_rows.element_size(), gate_rows.shape[1], group,
         ptr(out), n, width, tag(x.dtype), stream_ptr())
    return out


def norm_accumulate_round(x: "torch.Tensor | PairedRows | None", weight: torch.Tensor | None, eps: float, resid: torch.Tensor,
                          rounded_dtype: torch.dtype | None) -> torch.Tensor | None:
    """``resid += x * rsqrt(mean(x^2) + eps) * weight`` in place on float32 rows (nothing is added when ``x`` is ``None``);
    with ``rounded_dtype`` the updated rows are also returned in that type, for the sublayer that reads them next.  ``x`` may be
    ``PairedRows``: then row ``t`` of the sublayer's output is ``sum_j weights[t, j] * rows[pair_row[t, j]]``, formed inside the
    kernel.  The width is at most 12,288 (a row is kept in shared memory)."""

    require(resid, "resid", dtype=torch.float32, dims=2)
    n, hidden = resid.shape
    pair_row = pair_w = None
    top = 0
    if isinstance(x, PairedRows):
        pair_row, pair_w, top, x = x.pair_row, x.weights, x.weights.shape[1], x.rows
        require(x, "rows", dtype=torch.float32, dims=2)
        if x.shape[1] != hidden or pair_w.shape[0] != n:
            raise KernelError("norm_accumulate_round: the paired rows do not fit the residual rows")
    elif x is not None:
        require(x, "x", dtype=torch.float32, shape=resid.shape)
    if x is not None:
        require(weight, "weight", dtype=torch.float32, shape=(hidden,))
    rounded = None
    if rounded_dtype is not None:
        rounded = torch.empty((n, hidden), dtype=rounded_dtype, device=resid.device)
    if x is None and rounded is None:
        return None
    call("b200_norm_accumulate_round", ptr(x), ptr(weight), ptr(resid), ptr(rounded), n, hidden, float(eps), ptr(pair_row), ptr(pair_w),
         top, tag(rounded_dtype or torch.float32), stream_ptr())
    return rounded


def conv_taps(proj: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor, conv_state: torch.Tensor | None, *,
              q_start: torch.Tensor, slots: torch.Tensor, token_entry: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time of the first ``channels`` columns of ``proj``: ``u[t, c] = bias[c] + sum_j taps[c, j] *
    x[t - (K - 1 - j), c]``; inputs before the step come from the slot's kept rows ``[slots, K - 1, channels]`` (oldest
    first; zeros for a new request).  Returned in ``proj``'s type."""

    require(proj, "proj", dims=2)
    require(taps, "taps", dtype=torch.float32, dims=2)
    width, ntaps = taps.shape
    require(bias, "bias", dtype=torch.float32, shape=(width,))
    n = proj.shape[0]
    if ntaps > 1:
        require(conv_state, "conv_state", dtype=torch.float32, dims=3)
        if tuple(conv_state.shape[1:]) != (ntaps - 1, width):
            raise KernelError(f"conv_state has shape {tuple(conv_state.shape)}, expected [slots, {ntaps - 1}, {width}]")
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    u = torch.empty((n, width), dtype=proj.dtype, device=proj.device)
    call("b200_conv_taps", ptr(proj), proj.shape[1], ptr(taps), ptr(bias), ntaps, ptr(conv_state) if ntaps > 1 else None,
         ptr(q_start), ptr(slots), ptr(token_entry), ptr(u), n, width, tag(proj.dtype), stream_ptr())
    return u


def gated_recurrence(gates: torch.Tensor, u: torch.Tensor, proj: torch.Tensor, *, y_offset: int, lam: torch.Tensor,
                     decay_scale: float, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, block_width: int) -> torch.Tensor:
    """Per request (entry ``e`` owns rows ``q_start[e] .. q_start[e+1]-1`` and the state row ``slots[e]``) and channel, token after
    token: ``r, i = sigmoid(gates)``, ``log a = -decay_scale r softplus(lam)``, ``S <- a S + sqrt(1 - a^2) i u``; the result is
    ``S * gelu_tanh(proj[:, y_offset + c])`` in ``u``'s type.  Two launches: everything that does not depend on the state for all
    (token, channel) at once, then the chain of multiply-adds per channel.  ``gates`` float32 ``[N, blocks, 2 * block_width]`` (r logits, then i
    logits, per block); ``state`` ``[slots, width]`` float32, updated in place."""

    require(u, "u", dims=2)
    n, width = u.shape
    require(gates, "gates", dtype=torch.float32, shape=(n, width // block_width, 2 * block_width))
    require(proj, "proj", dtype=u.dtype, dims=2)
    require(lam, "lam", dtype=torch.float32, shape=(width,))
    require(state, "state", dtype=torch.float32, dims=2)
    if state.shape[1] != width:
        raise KernelError(f"state has shape {tuple(state.shape)}, expected [slots, {width}]")
    entries = q_start.shape[0] - 1
    require(slots, "slots", dtype=torch.int32, shape=(entries,))
    out = torch.empty_like(u)
    scratch = torch.empty((2, n, width), dtype=torch.float32, device=u.device)      # a and b of every (token, channel)
    call("b200_gated_recurrence", ptr(gates), ptr(u), ptr(proj), proj.shape[1], y_offset, ptr(lam), float(decay_scale), ptr(state),
         ptr(q_start), ptr(slots), ptr(out), ptr(scratch[0]), ptr(scratch[1]), n, entries, width, block_width, tag(u.dtype),
         stream_ptr(), launches=2)
    return out


# Longest portion of a step from which the minGRU scan runs in segments (three launches over all segments and channels
# instead of one chain per request and channel); LLM_RUNTIME_STUDY_B200_MINGRU_SEGMENTS=0: never.
MINGRU_SEGMENT_MIN = int(os.environ.get("LLM_RUNTIME_STUDY_B200_MINGRU_SEGMENTS", "128"))


def mingru_segment_map(q_lens, slots, device) -> tuple[torch.Tensor, int]:
    """Every entry cut into segments of tokens for ``mingru_scan``: one int32 tensor holding ``seg_first``, ``seg_count``,
    ``seg_slot`` (``[segments]`` each; the slot for an entry's last segment, else -1) and ``entry_seg`` (``[entries + 1]``)."""

    size = query("b200_mingru_segment_tokens")
    first, count, slot, entry_seg, at = [], [], [], [0], 0
    for n, s in zip(q_lens, slots):
        for start in range(0, n, size):
            first.append(at + start)
            count.append(min(size, n - start))
            slot.append(s if start + size >= n else -1)
        entry_seg.append(len(first))
        at += n
    packed = torch.tensor(first + count + slot + entry_seg, dtype=torch.int32)
    return packed.to(device), len(first)


def mingru_scan(proj: torch.Tensor, *, width: int, z_offset: int, u_offset: int, g_offset: int, state: torch.Tensor,
                q_start: torch.Tensor, slots: torch.Tensor, segments: "tuple[torch.Tensor, int] | None" = None) -> torch.Tensor:
    """The minGRU recurrence over the rows of one stacked projection (columns ``z_offset``, ``u_offset``, ``g_offset``, each
    ``width`` wide): ``z = sigmoid(zl)``, candidate ``u + 1/2`` where ``u >= 0`` else ``sigmoid(u)``,
    ``S_t = (1 - z_t) S_(t-1) + z_t c_t`` continued from ``state[slot]`` (float32 ``[slots, width]``, updated in place), output
    ``S_t * silu(g_t)`` ``[N, width]`` in the type of ``proj``.  ``segments`` (from ``mingru_segment_map``): the form in three
    launches for long portions, whose results differ from the chain's by rounding."""

    require(proj, "proj", dims=2)
    n, ld = proj.shape
    require(state, "state", dtype=torch.float32, dims=2)
    require(q_start, "q_start", dtype=torch.int32, dims=1)
    entries = q_start.shape[0] - 1
    require(slots, "slots", dtype=torch.int32, shape=(entries,))
    if state.shape[1] != width or max(z_offset, u_offset, g_offset) + width > ld:
        raise KernelError("mingru_scan: the columns lie outside the rows, or the state has another width")
    out = torch.empty((n, width), dtype=proj.dtype, device=proj.device)
    if segments is not None:
        packed, count = segments
        require(packed, "segments", dtype=torch.int32, shape=(3 * count + entries + 1,))
        scratch = torch.empty((2, count, width), dtype=torch.float32, device=proj.device)
        base, step = packed.data_ptr(), 4 * count
        call("b200_mingru_scan_segments", ptr(proj), ld, z_offset, u_offset, g_offset, ptr(out), ptr(state), ptr(slots), base, base + step,
             base + 2 * step, base + 3 * step, ptr(scratch), n, entries, count, width, tag(proj.dtype), stream_ptr(), launches=3)
        return out
    call("b200_mingru_scan", ptr(proj), ld, z_offset, u_offset, g_offset, ptr(out), ptr(state), ptr(q_start), ptr(slots), n, entries, width,
         tag(proj.dtype), stream_ptr())
    return out
