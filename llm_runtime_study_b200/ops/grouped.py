"""Matrix products in groups (one weight per head or diagonal block; one weight per expert for the rows a router sent
there) and the router's kernels.  Nothing here asks the device how many rows an expert received: the launch is sized for
the worst case and tiles without rows leave at once, so a step can be replayed from a CUDA graph."""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ..errors import KernelError
from .native import call, ptr, query, require, stream_ptr, tag

# Rows of (token, choice) pairs from which the experts' products go to the tcgen05 kernel (tiles of 128 rows an expert);
# below that, and wherever a width is no multiple of eight, the mma.sync kernel with tiles of 64 rows.
# LLM_RUNTIME_STUDY_B200_EXPERTS=mma keeps every size on the latter.
TC_MIN_PAIRS = 512
TC_TILE_ROWS = 128
EXPERTS_BACKEND = os.environ.get("LLM_RUNTIME_STUDY_B200_EXPERTS", "tcgen05")


def batched_linear(
    a: torch.Tensor, weight: torch.Tensor, *, batch: int, k: int, n_out: int, a_batch_stride: int, weight_k_major: bool = False,
    bias: torch.Tensor | None = None, out: torch.Tensor | None = None, out_batch_stride: int | None = None,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """For ``z`` in ``range(batch)``: ``out[:, z * out_batch_stride : + n_out] = a[:, z * a_batch_stride : + k] @ W[z]^T (+ bias[z])``.
    ``weight`` is ``[batch, n_out, k]`` or, with ``weight_k_major``, ``[batch, k, n_out]`` (then ``W[z]^T`` is the stored matrix
    itself).  ``a`` and ``out`` are rows ``[M, ...]`` with unit column stride; ``out`` may be given (a column block of a wider
    tensor is fine).  float accumulation in ascending ``k``."""

    require(a, "a", dims=2)
    require(weight, "weight", dtype=a.dtype, dims=3)
    m = a.shape[0]
    expect = (batch, k, n_out) if weight_k_major else (batch, n_out, k)
    if tuple(weight.shape) != expect:
        raise KernelError(f"weight has shape {tuple(weight.shape)}, expected {expect}")
    if (batch - 1) * a_batch_stride + k > a.shape[1]:
        raise KernelError("batched_linear: a batch entry's columns lie outside a")
    if bias is not None:
        require(bias, "bias", dtype=torch.float32, shape=(batch, n_out))
    out_dtype = out_dtype or a.dtype
    if out is None:
        out_batch_stride = n_out if out_batch_stride is None else out_batch_stride
        out = torch.empty((m, batch * out_batch_stride), dtype=out_dtype, device=a.device)
    else:
        if out.dim() != 2 or out.shape[0] != m or out.stride(1) != 1 or out.device != a.device:
            raise KernelError("batched_linear: out must be rows on the same device with unit column stride")
        if out_batch_stride is None or (batch - 1) * out_batch_stride + n_out > out.shape[1]:
            raise KernelError("batched_linear: a batch entry's results lie outside out")
    call("b200_gemm_grouped", ptr(a), a.stride(0), a_batch_stride, None, 0, ptr(weight), weight.stride(1), weight.stride(0),
         1 if weight_k_major else 0, ptr(bias), n_out, out.data_ptr(), out.stride(0), out_batch_stride, None, 0, m, n_out, k, batch, 0,
         tag(a.dtype), tag(out.dtype), stream_ptr())
    return out


@dataclass
class Routing:
    """Where a router sent the tokens.  ``ids``/``weights`` ``[N, top]``; ``pair_row[N * top]``: the row of each (token, choice)
    pair in the expert-sorted order; ``sorted_token[rows]``: the token of a sorted row (-1: padding up to whole tiles);
    ``tile_group[tiles]``: the expert of each tile of rows (-1: unused)."""

    ids: torch.Tensor
    weights: torch.Tensor
    pair_row: torch.Tensor
    sorted_token: torch.Tensor
    tile_group: torch.Tensor
    top: int
    tile_rows: int = 64
    extra: torch.Tensor | None = None      # float32 [N, extra]: sigmoids of the router's further rows (gates for every token)

    @property
    def rows(self) -> int:
        return self.sorted_token.shape[0]


def tile_rows() -> int:
    return query("b200_moe_tile_rows")


SCORES = {"softmax_chosen": 0, "sigmoid": 1, "softmax_all": 2}


def route(h: torch.Tensor, router: torch.Tensor, bias: torch.Tensor | None, *, top: int, wide_tiles: bool = False,
          score: str = "softmax_chosen", correction: torch.Tensor | None = None, groups: int = 1, keep: int = 1,
          scale: float = 1.0, identity: int = 0, extra: int = 0) -> Routing:
    """Logits ``router @ h + bias`` in float32 (``router`` float32 ``[outputs + extra, width]``; ``h`` in the activation type), the
    ``top`` largest chosen (the lower index wins a tie); weights by ``score``: the softmax over the chosen logits, each chosen
    logit's sigmoid (not renormalised), or (``softmax_all``) the chosen outputs' shares ``s`` of the softmax over all outputs
    times ``scale``, where the choice goes by ``s + correction`` among the outputs of the ``keep`` best of ``groups`` equal
    groups of neighbours (a group scores its largest choice score).  The last ``identity`` outputs have no expert behind them
    (their pairs get no row: ``pair_row`` -1).  ``extra`` further rows of ``router`` give one number per token each, whose
    sigmoids are returned in ``Routing.extra``.  Then the pairs sorted by expert, each expert's rows padded to whole tiles
    (of 128 rows with ``wide_tiles``, what the tcgen05 kernel takes; else of 64)."""

    require(h, "h", dims=2)
    n, width = h.shape
    require(router, "router", dtype=torch.float32, dims=2)
    outputs = router.shape[0] - extra
    experts = outputs - identity
    if experts <= 0 or identity < 0 or extra < 0:
        raise KernelError(f"router of {router.shape[0]} rows does not hold {identity} identity outputs and {extra} further rows")
    if router.shape[1] != width:
        raise KernelError(f"router has shape {tuple(router.shape)}, expected [experts, {width}]")
    if bias is not None:
        require(bias, "bias", dtype=torch.float32, shape=(outputs + extra,))
    if correction is not None:
        require(correction, "correction", dtype=torch.float32, shape=(outputs,))
    dev = h.device
    ids = torch.empty((n, top), dtype=torch.int32, device=dev)
    weights = torch.empty((n, top), dtype=torch.float32, device=dev)
    extra_out = torch.empty((n, extra), dtype=torch.float32, device=dev) if extra else None
    if score not in SCORES:
        raise KernelError(f"unknown router score {score!r}; expected one of {sorted(SCORES)}")
    call("b200_moe_route_grouped", ptr(h), ptr(router), ptr(bias), ptr(correction), ptr(ids), ptr(weights), ptr(extra_out), n, width,
         outputs, top, SCORES[score], int(groups), int(keep), float(scale), int(extra), tag(h.dtype), stream_ptr())
    tile = TC_TILE_ROWS if wide_tiles else tile_rows()
    max_tiles = min(-(-n * top // tile) + experts, n * top)       # a tile holds one expert's rows only
    pair_row = torch.empty(n * top, dtype=torch.int32, device=dev)
    sorted_token = torch.empty(max_tiles * tile, dtype=torch.int32, device=dev)
    tile_group = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    call("b200_moe_plan", ptr(ids), n * top, top, experts, ptr(sorted_token), ptr(pair_row), ptr(tile_group), max_tiles, tile, stream_ptr())
    return Routing(ids, weights, pair_row, sorted_token, tile_group, top, tile, extra_out)


def wide_tiles_pay(n: int, top: int, dtype: torch.dtype, *widths: int) -> bool:
    """Whether the experts' products of ``n`` tokens go to the tcgen05 kernel."""

    return (EXPERTS_BACKEND == "tcgen05" and dtype == torch.bfloat16 and n * top >= TC_MIN_PAIRS and all(w % 8 == 0 for w in widths))


def gather_sorted(x: torch.Tensor, routing: Routing) -> torch.Tensor:
    """``x``'s rows in the sorted order, zeros in the padding (bfloat16, a width in steps of eight)."""

    require(x, "x", dtype=torch.bfloat16, dims=2)
    out = torch.empty((routing.rows, x.shape[1]), dtype=x.dtype, device=x.device)
    call("b200_gather_rows_bf16", ptr(x), ptr(routing.sorted_token), ptr(out), routing.rows, x.shape[1], stream_ptr())
    return out


def expert_linear(a: torch.Tensor, weight: torch.Tensor, routing: Routing, *, gather: bool, act: str | None = None,
                  out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``out[row] = act(W[expert of row] @ a[source of row])`` for every sorted row.  ``weight`` ``[experts, n_out, k]``.  With
    ``gather`` the source is the row's token (``a`` is ``[N, k]``); otherwise ``a`` is already in sorted order (``[rows, k]``).
    ``act``: ``"relu2"`` (the square of relu) or ``None``.  Rows of the padding are not written, or hold zeros.

    A routing made with tiles of 128 rows (bfloat16, widths in steps of eight) goes to the tcgen05 kernel, which fetches its
    operands by TMA: the gathered rows are then laid out first (one more launch).  Everything else runs on mma.sync tiles
    (bfloat16) or FFMA (float32) with the gather inside the kernel."""

    require(a, "a", dims=2)
    require(weight, "weight", dtype=a.dtype, dims=3)
    experts, n_out, k = weight.shape
    if a.shape[1] != k or (not gather and a.shape[0] != routing.rows):
        raise KernelError(f"expert_linear: a {tuple(a.shape)} does not fit the weight {tuple(weight.shape)} and {routing.rows} sorted rows")
    out = torch.empty((routing.rows, n_out), dtype=out_dtype or a.dtype, device=a.device)
    code = {None: 0, "relu2": 1}[act]
    if (routing.tile_rows == TC_TILE_ROWS and a.dtype == torch.bfloat16 and k % 8 == 0 and weight.is_contiguous()
            and EXPERTS_BACKEND == "tcgen05"):
        from . import gemm_bf16  # noqa: F401  (registers the library)

        rows = gather_sorted(a, routing) if gather else a
        call("b200_gemm_tcgen05_grouped", ptr(rows), ptr(weight), ptr(out), routing.rows, n_out, k, out.stride(0),
             1 if out.dtype == torch.float32 else 0, code, ptr(routing.tile_group), experts, 256 if n_out >= 256 else 128, stream_ptr(),
             launches=2 if gather else 1)
        return out
    call("b200_gemm_grouped", ptr(a), a.stride(0), 0, ptr(routing.sorted_token), 1 if gather else 0, ptr(weight), weight.stride(1),
         weight.stride(0), 0, None, 0, ptr(out), out.stride(0), 0, ptr(routing.tile_group), routing.tile_rows, routing.rows, n_out, k, 1,
         code, tag(a.dtype), tag(out.dtype), stream_ptr())
    return out


def combine(rows: torch.Tensor, routing: Routing, *, weighted: bool = True) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * rows[pair_row[t, j]]`` (float32, ``j`` ascending); without ``weighted`` the plain sum
    (the weights went into the experts' inputs)."""

    require(rows, "rows", dtype=torch.float32, dims=2)
    n = routing.ids.shape[0]
    out = torch.empty((n, rows.shape[1]), dtype=torch.float32, device=rows.device)
    call("b200_moe_combine", ptr(rows), ptr(routing.pair_row), ptr(routing.weights) if weighted else None, ptr(out), n, rows.shape[1],
         routing.top, stream_ptr())
    return out


def combine_mixed(rows: torch.Tensor, routing: Routing, x: torch.Tensor, *, extra: torch.Tensor | None = None,
                  extra_scale: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * r_j + extra_scale[t] * extra[t]`` with ``r_j = rows[pair_row[t, j]]``, or ``x[t]`` (the token's
    own input row, activation type) where the pair has no row (an output that returns its input).  float32, ``j`` ascending."""

    require(rows, "rows", dtype=torch.float32, dims=2)
    n, width = routing.ids.shape[0], rows.shape[1]
    require(x, "x", shape=(n, width))
    if extra is not None:
        require(extra, "extra", dtype=torch.float32, shape=(n, width))
        require(extra_scale, "extra_scale", dtype=torch.float32)
        if extra_scale.numel() != n:
            raise KernelError("combine_mixed: one factor per token is expected")
    out = torch.empty((n, width), dtype=torch.float32, device=rows.device)
    call("b200_moe_combine_mixed", ptr(rows), ptr(routing.pair_row), ptr(routing.weights), ptr(x), ptr(extra), ptr(extra_scale), ptr(out),
         n, width, routing.top, tag(x.dtype), stream_ptr())
    return out
