"""Kernels of a layer whose sublayers read one normalised copy of the stream side by side: layer norm, the short
convolution added to each sublayer's input, the scaled sum of the sublayers' outputs with the average over all layers'
results, the polynomial activation of normalised powers, and the gated unit of rows whose router weight multiplies the
expert's input.  Statistics and sums are float32 in both run types."""

from __future__ import annotations

import torch

from ..errors import KernelError
from .native import call, ptr, require, stream_ptr, tag


def layer_norm(resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out_dtype: torch.dtype, *,
               rows: torch.Tensor | None = None) -> torch.Tensor:
    """``resid += delta`` (in place, float32; only without ``rows``) and return ``(x - mean) / sqrt(var + eps) * weight`` of every
    row, the variance being the mean of the squared deviations.  With ``rows`` the given rows (plus ``delta``'s) are gathered and
    ``resid`` is left as it is."""

    require(resid, "resid", dtype=torch.float32, dims=2)
    hidden = resid.shape[1]
    if delta is not None:
        require(delta, "delta", dtype=torch.float32, shape=resid.shape)
    require(weight, "weight", dtype=torch.float32, shape=(hidden,))
    if rows is not None:
        require(rows, "rows", dtype=torch.int32, dims=1)
    n = resid.shape[0] if rows is None else rows.shape[0]
    out = torch.empty((n, hidden), dtype=out_dtype, device=resid.device)
    call("b200_layer_norm", ptr(resid), ptr(delta), ptr(weight), ptr(out), ptr(rows), n, hidden, float(eps),
         1 if (rows is None and delta is not None) else 0, tag(out_dtype), stream_ptr())
    return out


def taps_pair(h: torch.Tensor, taps_a: torch.Tensor, taps_b: torch.Tensor | None, kept: torch.Tensor | None, *, q_start: torch.Tensor,
              slots: torch.Tensor, token_entry: torch.Tensor, out_dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor | None]:
    """``h + conv_a(h)`` and ``h + conv_b(h)`` for float32 rows ``h`` ``[N, C]``: ``conv(h)[t] = sum_j taps[:, j] * h[t - (K - 1) + j]``
    per channel, over time within each request; inputs before the step come from ``kept`` ``[slots, K - 1, C]`` (oldest first,
    zeros for a new request).  Both results in ``out_dtype``; ``taps_b`` may be ``None``."""

    require(h, "h", dtype=torch.float32, dims=2)
    n, width = h.shape
    require(taps_a, "taps_a", dtype=torch.float32, dims=2)
    ntaps = taps_a.shape[1]
    if taps_a.shape[0] != width:
        raise KernelError(f"taps have shape {tuple(taps_a.shape)}, expected [{width}, taps]")
    if taps_b is not None:
        require(taps_b, "taps_b", dtype=torch.float32, shape=taps_a.shape)
    if ntaps > 1:
        require(kept, "kept", dtype=torch.float32, dims=3)
        if tuple(kept.shape[1:]) != (ntaps - 1, width):
            raise KernelError(f"kept rows have shape {tuple(kept.shape)}, expected [slots, {ntaps - 1}, {width}]")
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    out_a = torch.empty((n, width), dtype=out_dtype, device=h.device)
    out_b = torch.empty((n, width), dtype=out_dtype, device=h.device) if taps_b is not None else None
    call("b200_taps_pair", ptr(h), ptr(taps_a), ptr(taps_b), ptr(kept) if ntaps > 1 else None, ptr(q_start), ptr(slots), ptr(token_entry),
         ptr(out_a), ptr(out_b), n, width, ntaps, tag(out_dtype), stream_ptr())
    return out_a, out_b


def scale_sum_average(x: torch.Tensor, a: torch.Tensor, scale_a: torch.Tensor | None, b: torch.Tensor | None,
                      scale_b: torch.Tensor | None, results: torch.Tensor | None, mix: torch.Tensor | None, index: int) -> None:
    """In place on the float32 stream ``x`` ``[N, C]``: the layer's result ``x + scale_a * a + scale_b * b`` is stored as
    ``results[index + 1]`` and ``x`` becomes ``sum_{j <= index + 1} mix[j] * results[j]``.  Without ``mix`` the stream becomes the
    layer's result and nothing is stored."""

    require(x, "x", dtype=torch.float32, dims=2)
    n, width = x.shape
    require(a, "a", dtype=torch.float32, shape=x.shape)
    if b is not None:
        require(b, "b", dtype=torch.float32, shape=x.shape)
    for s, name in ((scale_a, "scale_a"), (scale_b, "scale_b")):
        if s is not None:
            require(s, name, dtype=torch.float32, shape=(width,))
    if mix is not None:
        require(mix, "mix", dtype=torch.float32, shape=(index + 2,))
        require(results, "results", dtype=torch.float32, dims=3)
        if results.shape[0] < index + 2 or tuple(results.shape[1:]) != (n, width):
            raise KernelError(f"results have shape {tuple(results.shape)}, expected [>= {index + 2}, {n}, {width}]")
    call("b200_scale_sum_average", ptr(x), ptr(a), ptr(scale_a), ptr(b), ptr(scale_b), ptr(results) if mix is not None else None,
         ptr(mix), index, n, width, stream_ptr())


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """``coef[0] u(z) + coef[1] u(z^2) + coef[2] u(z^3) + coef[3]`` with element-wise powers and ``u(y) = y / sqrt(mean(y^2) + eps)``
    over each row; in ``z``'s type."""

    require(z, "z", dims=2)
    require(coef, "coef", dtype=torch.float32, shape=(4,))
    out = torch.empty_like(z)
    call("b200_poly_norm", ptr(z), ptr(coef), ptr(out), z.shape[0], z.shape[1], float(eps), tag(z.dtype), stream_ptr())
    return out


def silu_mul_scaled(gate_up: torch.Tensor, pair_row: torch.Tensor | None = None, scale: torch.Tensor | None = None) -> torch.Tensor:
    """Rows ``[gate | up]``: ``silu(s * gate) * (s * up)`` with one factor per row.  With ``pair_row`` (``[pairs]`` int32) and
    ``scale`` (``[pairs]`` float32) only the rows that pairs own are computed, each with its pair's factor."""

    require(gate_up, "gate_up", dims=2)
    rows, two_f = gate_up.shape
    if two_f % 2:
        raise KernelError("silu_mul_scaled: row width must be even ([gate | up])")
    count = rows
    if pair_row is not None:
        require(pair_row, "pair_row", dtype=torch.int32, dims=1)
        count = pair_row.shape[0]
    if scale is not None:
        require(scale, "scale", dtype=torch.float32)
        if scale.numel() != count:
            raise KernelError("silu_mul_scaled: one factor per row (or pair) is needed")
    out = torch.empty((rows, two_f // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("b200_silu_mul_scaled", ptr(gate_up), ptr(pair_row), ptr(scale), ptr(out), count, two_f // 2, tag(gate_up.dtype), stream_ptr())
    return out
