"""The kernels as functions over torch tensors (device memory only).

Activations are ``float32`` or ``bfloat16``; the residual stream, norm weights,
rotary frequencies and logits are always ``float32``.
"""

from __future__ import annotations

import torch

from ..errors import KernelError
from . import native
from .native import call, ptr, require, stream_ptr, tag


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``out[n] = table[ids[n]] * scale`` as float32 (the residual stream's type)."""

    require(ids, "ids", dtype=torch.int32, dims=1)
    require(table, "table", dims=2)
    n, (vocab, hidden) = ids.shape[0], table.shape
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    call("b200_embedding", ptr(ids), ptr(table), ptr(out), n, hidden, vocab, float(scale),
         tag(table.dtype), stream_ptr())
    return out


def embedding_weighted(ids: torch.Tensor, table: torch.Tensor, scale: float, norm_weight: torch.Tensor, eps: float):
    """For at most 16 tokens: the embedding rows as float32, the same rows times ``norm_weight`` in bfloat16,
    and each row's factor ``rsqrt(mean of squares + eps)`` (``[16]`` floats, what ``gemm_bf16.linear_skinny``
    takes as ``row_scale``).  The row width must be a multiple of a 16-byte vector of the table's type."""

    require(ids, "ids", dtype=torch.int32, dims=1)
    require(table, "table", dims=2)
    n, (vocab, hidden) = ids.shape[0], table.shape
    require(norm_weight, "norm_weight", dtype=torch.float32, shape=(hidden,))
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    weighted = torch.empty((n, hidden), dtype=torch.bfloat16, device=table.device)
    row_scale = torch.empty(16, dtype=torch.float32, device=table.device)
    call("b200_embedding_weighted", ptr(ids), ptr(table), ptr(out), ptr(norm_weight), ptr(weighted), ptr(row_scale), n, hidden,
         vocab, float(scale), float(eps), tag(table.dtype), stream_ptr())
    return out, weighted, row_scale


def add_rmsnorm(
    resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
    out_dtype: torch.dtype, *, rows: torch.Tensor | None = None,
) -> torch.Tensor:
    """``resid += delta`` (in place, float32) and return ``rms_norm(resid) * weight``.

    With ``rows`` the given rows are gathered, normalised and returned, and
    ``resid`` is left as it is (used for the rows whose logits are wanted).
    """

    require(resid, "resid", dtype=torch.float32, dims=2)
    n_src, hidden = resid.shape
    if delta is not None:
        require(delta, "delta", dtype=torch.float32, shape=resid.shape)
    require(weight, "weight", dtype=torch.float32, shape=(hidden,))
    if rows is not None:
        require(rows, "rows", dtype=torch.int32, dims=1)
    n = n_src if rows is None else rows.shape[0]
    out = torch.empty((n, hidden), dtype=out_dtype, device=resid.device)
    call("b200_add_rmsnorm", ptr(resid), ptr(delta), ptr(weight), ptr(out), ptr(rows), n, hidden,
         float(eps), 1 if (rows is None and delta is not None) else 0, tag(out_dtype), stream_ptr())
    return out


def linear_f32(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` in true float32 (FFMA only)."""

    require(x, "x", dtype=torch.float32, dims=2)
    require(weight, "weight", dtype=torch.float32, dims=2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x has width {k}, weight expects {weight.shape[1]}")
    if bias is not None:
        require(bias, "bias", dtype=torch.float32, shape=(n,))
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    call("b200_gemm_f32", ptr(x), ptr(weight), ptr(bias), ptr(out), m, n, k, k, n, stream_ptr())
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for rows laid out as ``[gate | up]``."""

    require(gate_up, "gate_up", dims=2)
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("silu_mul: row width must be even ([gate | up])")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("b200_silu_mul", ptr(gate_up), ptr(out), n, two_i // 2, tag(gate_up.dtype), stream_ptr())
    return out


def silu_mul_interleaved(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for rows laid out in blocks of eight, ``[g0..g7 | u0..u7 | g8..g15 | ...]``
    (the layout of a stacked gate/up projection whose kernels can apply the activation themselves)."""

    require(gate_up, "gate_up", dims=2)
    n, two_i = gate_up.shape
    if two_i % 16:
        raise KernelError("silu_mul_interleaved: row width must be a multiple of 16")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("b200_silu_mul_interleaved", ptr(gate_up), ptr(out), n, two_i // 2, tag(gate_up.dtype), stream_ptr())
    return out


def qk_norm_rope_write(
    qkv: torch.Tensor, *, num_q_heads: int, num_kv_heads: int, head_dim: int,
    q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
    inv_freq: torch.Tensor | None, rotary_dim: int, positions: torch.Tensor,
    token_entry: torch.Tensor, block_table: torch.Tensor | None, page_size: int,
    k_pool: torch.Tensor | None, v_pool: torch.Tensor | None,
) -> torch.Tensor:
    """Per-head RMS norm of q and k (optional), rotary rotation (optional), then q is
    returned as ``[N, nq, d]`` and k, v are written into the paged pools
    ``[pages, nkv, page_size, d]`` at each token's position.  ``num_kv_heads = 0``
    with no pools handles a layer that only reads another layer's cache."""

    require(qkv, "qkv", dims=2)
    n, width = qkv.shape
    if width != (num_q_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv width {width} != (nq + 2 nkv) * d")
    dev, dt = qkv.device, qkv.dtype
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    for w, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            require(w, name, dtype=torch.float32, shape=(head_dim,))
    if inv_freq is not None:
        require(inv_freq, "inv_freq", dtype=torch.float32, shape=(rotary_dim // 2,))
    table_stride = 0
    if num_kv_heads > 0:
        require(block_table, "block_table", dtype=torch.int32, dims=2)
        table_stride = block_table.shape[1]
        for pool, name in ((k_pool, "k_pool"), (v_pool, "v_pool")):
            require(pool, name, dtype=dt, dims=4)
            if tuple(pool.shape[1:]) != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name} has shape {tuple(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
    q_out = torch.empty((n, num_q_heads, head_dim), dtype=dt, device=dev)
    call("b200_qk_norm_rope_write", ptr(qkv), ptr(q_out), ptr(q_weight), ptr(k_weight), float(eps),
         ptr(inv_freq), rotary_dim if inv_freq is not None else 0, ptr(positions), ptr(token_entry),
         ptr(block_table), table_stride, page_size, ptr(k_pool), ptr(v_pool), n, num_q_heads,
         num_kv_heads, head_dim, width, tag(dt), stream_ptr())
    return q_out


def paged_attention_simt(
    q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *, positions: torch.Tensor,
    token_entry: torch.Tensor, block_table: torch.Tensor, scale: float, window: int = 0,
) -> torch.Tensor:
    """Causal attention of every query token over keys ``0..position`` of its request,
    32-bit arithmetic, reduction order fixed by the token's position alone."""

    require(q, "q", dims=3)
    n, nq, d = q.shape
    require(k_pool, "k_pool", dtype=q.dtype, dims=4)
    require(v_pool, "v_pool", dtype=q.dtype, shape=k_pool.shape)
    _, nkv, page_size, dk = k_pool.shape
    if dk != d:
        raise KernelError(f"q head size {d} != cache head size {dk}")
    if d % 16:
        raise KernelError(f"head size {d} is not a multiple of 16")
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    out = torch.empty_like(q)
    call("b200_paged_attention_simt", ptr(q), ptr(k_pool), ptr(v_pool), ptr(out), ptr(positions),
         ptr(token_entry), ptr(block_table), block_table.shape[1], page_size, n, nq, nkv, d,
         float(scale), int(window), tag(q.dtype), stream_ptr())
    return out


def qk_rownorm_write(
    qkv: torch.Tensor, *, num_q_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
    q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, temp_coef: float, temp_every: int,
    positions: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor, page_size: int,
    k_pool: torch.Tensor, v_pool: torch.Tensor,
) -> torch.Tensor:
    """Rows ``[q | k | v]``: RMS norm of q and of k over the whole projection (all heads at once, weights of that
    width), q times the position's temperature ``1 + coef * ln(floor((p + 1) / every) + 1)`` (``every = 0``: none);
    q is returned as ``[N, nq, d]``, k and v are written into the pages ``[pages, nkv, page_size, d | dv]``."""

    require(qkv, "qkv", dims=2)
    n, width = qkv.shape
    qw, kw = num_q_heads * head_dim, num_kv_heads * head_dim
    if width < qw + kw + num_kv_heads * value_dim:
        raise KernelError(f"qkv width {width} is less than nq*d + nkv*(d + dv)")
    dt = qkv.dtype
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    if q_weight is not None:
        require(q_weight, "q_weight", dtype=torch.float32, shape=(qw,))
    if k_weight is not None:
        require(k_weight, "k_weight", dtype=torch.float32, shape=(kw,))
    require(k_pool, "k_pool", dtype=dt, dims=4)
    require(v_pool, "v_pool", dtype=dt, dims=4)
    if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or tuple(v_pool.shape[1:]) != (num_kv_heads, page_size, value_dim):
        raise KernelError(f"pools have shapes {tuple(k_pool.shape)} and {tuple(v_pool.shape)}, expected "
                          f"[pages, {num_kv_heads}, {page_size}, {head_dim} | {value_dim}]")
    q_out = torch.empty((n, num_q_heads, head_dim), dtype=dt, device=qkv.device)
    call("b200_qk_rownorm_write", ptr(qkv), width, ptr(q_out), ptr(q_weight), ptr(k_weight), float(eps), float(temp_coef),
         int(temp_every), ptr(positions), ptr(token_entry), ptr(block_table), block_table.shape[1], page_size, ptr(k_pool),
         ptr(v_pool), n, num_q_heads, num_kv_heads, head_dim, value_dim, tag(dt), stream_ptr())
    return q_out


def paged_attention_simt_rules(
    q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *, positions: torch.Tensor, token_entry: torch.Tensor,
    block_table: torch.Tensor, scale: float, window: int = 0, softcap: float = 0.0, slopes: torch.Tensor | None = None,
    sink: bool = False, chunk: int = 0, log_bias: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> torch.Tensor:
    """``paged_attention_simt`` with rules on the scores: ``S <- cap * tanh(S / cap)`` (``softcap > 0``), then
    ``S <- S - slopes[head] * (p - t)``, ``S <- S - r1[head] * ln(1 + r2[head] * (p - t))`` (``log_bias = (r1, r2)``), and with
    ``sink`` the weights ``exp(S) / (1 + sum exp(S))``.  ``chunk > 0``: position p sees t only inside its own block of ``chunk``
    positions (counted from 0).  Values may have a head size of their own: q ``[N, nq, d]``, keys ``[pages, nkv, page, d]``,
    values ``[pages, nkv, page, dv]``, result ``[N, nq, dv]``."""

    require(q, "q", dims=3)
    n, nq, d = q.shape
    require(k_pool, "k_pool", dtype=q.dtype, dims=4)
    require(v_pool, "v_pool", dtype=q.dtype, dims=4)
    _, nkv, page_size, dk = k_pool.shape
    dv = v_pool.shape[3]
    if dk != d or tuple(v_pool.shape[:3]) != tuple(k_pool.shape[:3]):
        raise KernelError(f"q head size {d}, key pool {tuple(k_pool.shape)} and value pool {tuple(v_pool.shape)} do not fit")
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    if slopes is not None:
        require(slopes, "slopes", dtype=torch.float32, shape=(nq,))
    r1 = r2 = None
    if log_bias is not None:
        r1, r2 = log_bias
        require(r1, "log_bias[0]", dtype=torch.float32, shape=(nq,))
        require(r2, "log_bias[1]", dtype=torch.float32, shape=(nq,))
    if d > 256 or dv > 256:
        raise KernelError(f"head sizes {d} and {dv} must be at most 256")
    out = torch.empty((n, nq, dv), dtype=q.dtype, device=q.device)
    call("b200_paged_attention_simt_masked", ptr(q), ptr(k_pool), ptr(v_pool), ptr(out), ptr(positions), ptr(token_entry),
         ptr(block_table), block_table.shape[1], page_size, n, nq, nkv, d, dv, dv, float(scale), int(window), float(softcap),
         ptr(slopes), 1 if sink else 0, int(chunk), ptr(r1), ptr(r2), tag(q.dtype), stream_ptr())
    return out


def relu2(x: torch.Tensor) -> torch.Tensor:
    """``relu(x)^2`` element by element, in the type of ``x``."""

    require(x, "x")
    out = torch.empty_like(x)
    call("b200_relu2", ptr(x), ptr(out), x.numel(), tag(x.dtype), stream_ptr())
    return out


def embedding_sum(ids: torch.Tensor, table: torch.Tensor, bigram: torch.Tensor | None, *, positions: torch.Tensor,
                  token_entry: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, previous: torch.Tensor | None,
                  freq: torch.Tensor | None, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0, scale: float = 1.0) -> torch.Tensor:
    """``table[id] * scale + bigram[row] + pos(p)`` as float32 rows: ``row = (previous token * mul_prev + id * mul_cur) mod buckets``,
    row ``buckets`` at position 0; ``pos(p)``: column ``2i`` is ``sin(p * freq[i])``, column ``2i + 1`` the cosine (``freq`` float64).
    The token before a step's first token of a request is read from ``previous[slot]`` (int32 per request slot), which then
    receives the entry's last token.  ``bigram`` and ``freq`` may each be ``None``."""

    require(ids, "ids", dtype=torch.int32, dims=1)
    require(table, "table", dims=2)
    n, (vocab, hidden) = ids.shape[0], table.shape
    for t, name in ((positions, "positions"), (token_entry, "token_entry")):
        require(t, name, dtype=torch.int32, shape=(n,))
    require(q_start, "q_start", dtype=torch.int32, dims=1)
    entries = q_start.shape[0] - 1
    require(slots, "slots", dtype=torch.int32, shape=(entries,))
    if bigram is not None:
        require(bigram, "bigram", dtype=table.dtype, shape=(buckets + 1, hidden))
        require(previous, "previous", dtype=torch.int32)
    if freq is not None:
        require(freq, "freq", dtype=torch.float64, shape=((hidden + 1) // 2,))
    out = torch.empty((n, hidden), dtype=torch.float32, device=ids.device)
    call("b200_embedding_sum", ptr(ids), ptr(table), ptr(bigram), ptr(out), ptr(positions), ptr(token_entry), ptr(q_start), ptr(slots),
         ptr(previous), ptr(freq), n, entries, hidden, vocab, int(buckets), int(mul_prev), int(mul_cur), float(scale), tag(table.dtype),
         stream_ptr())
    return out


def glu_limit(gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """Rows ``[gate | up]``: ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, ``g * sigmoid(alpha g) * (u + 1)``."""

    require(gate_up, "gate_up", dims=2)
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("glu_limit: row width must be even ([gate | up])")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("b200_glu_limit", ptr(gate_up), ptr(out), n, two_i // 2, float(limit), float(alpha), tag(gate_up.dtype), stream_ptr())
    return out


def rmsnorm_accumulate(x: torch.Tensor, weight: torch.Tensor, eps: float, factor: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out (+)= factor * rms_norm(x) * weight`` on float32 rows; a fresh ``out`` is made (and not read) when none is given."""

    require(x, "x", dtype=torch.float32, dims=2)
    n, hidden = x.shape
    require(weight, "weight", dtype=torch.float32, shape=(hidden,))
    accumulate = out is not None
    if out is None:
        out = torch.empty_like(x)
    else:
        require(out, "out", dtype=torch.float32, shape=x.shape)
    call("b200_rmsnorm_accumulate", ptr(x), ptr(weight), ptr(out), n, hidden, float(eps), float(factor), 1 if accumulate else 0,
         stream_ptr())
    return out


def add_rows(resid: torch.Tensor, a: torch.Tensor | None = None, b: torch.Tensor | None = None,
             vector: torch.Tensor | None = None) -> None:
    """``resid += a + b + vector`` in place on float32 rows (each term optional; ``vector`` is one row for all)."""

    require(resid, "resid", dtype=torch.float32, dims=2)
    n, hidden = resid.shape
    for t, name in ((a, "a"), (b, "b")):
        if t is not None:
            require(t, name, dtype=torch.float32, shape=resid.shape)
    if vector is not None:
        require(vector, "vector", dtype=torch.float32, shape=(hidden,))
    call("b200_add_rows", ptr(resid), ptr(a), ptr(b), ptr(vector), n, hidden, stream_ptr())


def paged_attention_simt_latent(
    q: torch.Tensor, pool: torch.Tensor, *, value_dim: int, positions: torch.Tensor, token_entry: torch.Tensor,
    block_table: torch.Tensor, scale: float, window: int = 0,
) -> torch.Tensor:
    """Causal attention of every query head over one shared row per token whose leading ``value_dim`` columns are also the
    value: q ``[N, heads, d]``, pool ``[pages, page_size, d]``, result ``[N, heads, value_dim]``.  32-bit arithmetic, tiles
    of 32 keys from key 0 of the window's first tile, so the order of every sum depends on the token's position alone."""

    require(q, "q", dims=3)
    n, nq, d = q.shape
    require(pool, "pool", dtype=q.dtype, dims=3)
    page_size = pool.shape[1]
    if pool.shape[2] != d or not 0 < value_dim <= d:
        raise KernelError(f"q head size {d}, pool {tuple(pool.shape)} and value size {value_dim} do not fit")
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    out = torch.empty((n, nq, value_dim), dtype=q.dtype, device=q.device)
    call("b200_paged_attention_simt_strided", ptr(q), ptr(pool), ptr(pool), ptr(out), ptr(positions), ptr(token_entry),
         ptr(block_table), block_table.shape[1], page_size, n, nq, 1, d, value_dim, d, float(scale), int(window), 0.0, None, 0,
         tag(q.dtype), stream_ptr())
    return out
