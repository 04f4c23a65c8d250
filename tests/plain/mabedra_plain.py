"""Plain, slow Mabedra forward pass: whole sequences, no cache, CPU.

One function per mechanism, elementary torch operations only, nothing shared with the engine.  It takes a
``config.json`` dict and ``{tensor name: tensor}`` with the checkpoint's own names.  ``dtype`` is the arithmetic
type (float64 separates rounding from faults).

``store`` (optional) is applied wherever a serving engine with 16-bit activations keeps a tensor in memory
between two operations: the rows a sublayer reads, the results of projections, q and k as they enter the
attention, the attention's read-out, the hidden rows of a feed-forward.  The residual stream, the statistics,
the router and the logits stay in ``dtype`` either way.

Notation: ``T`` tokens at positions ``0..T-1``; ``unit(x) = x / sqrt(mean(x^2) + eps)`` over the last axis;
every linear map is ``x @ W.T`` with ``W`` stored ``[out, in]``.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch


# ----------------------------------------------------------------- elementary
def keep(x: torch.Tensor) -> torch.Tensor:
    return x


def round_bfloat16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``(x - mean) / sqrt(var + eps) * w`` with the variance as the mean of squared deviations; no bias."""

    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(dim=-1, keepdim=True) + eps) * w


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * sigmoid(x)


# ------------------------------------------------------------ short convolution
def causal_taps(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_j w[:, j] * h[t - (K - 1) + j]`` per channel, zeros before the sequence's start.  ``h`` ``[T, C]``,
    ``w`` ``[C, K]``."""

    T, K = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for j in range(K):
        back = K - 1 - j
        if back < T:
            out[back:] += w[:, j] * h[: T - back]
    return out


# ------------------------------------------------------------------- rotation
def scaled_frequencies(dims: int, base: float, scaling: Mapping | None, dtype) -> torch.Tensor:
    """``f_i = base^(-2i / dims)`` for ``i < dims / 2``; with ``scaling`` long wavelengths are stretched: a wavelength
    below ``original / high`` keeps its frequency, one above ``original / low`` gets ``f / factor``, and in between the two
    are blended by ``s = (original / wavelength - low) / (high - low)``."""

    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    if scaling:
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wavelength = 2.0 * math.pi / f
        s = (original / wavelength - low) / (high - low)
        blended = (1.0 - s) * f / factor + s * f
        f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blended))
    return f.to(dtype)


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """``x`` ``[T, ..., d]``: the first ``2 * len(freqs)`` columns are rotated, column i paired with ``i + len(freqs)``."""

    half = freqs.shape[0]
    if half == 0:
        return x
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    angle = (positions.to(freqs.dtype)[:, None] * freqs[None, :]).reshape(shape)
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, v = x[..., :half], x[..., half : 2 * half]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half :]], dim=-1)


# ------------------------------------------------------------------ attention
def window_mask(T: int, window: int | None) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    return seen


def one_map(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, seen: torch.Tensor) -> torch.Tensor:
    s = (q @ k.T) * scale
    s = s.masked_fill(~seen, -math.inf)
    return torch.softmax(s, dim=-1) @ v


def differential_read_out(q, k, v, *, scale: float, window: int | None, lam: float, out_scale: float, eps: float,
                          normalise: bool = True) -> torch.Tensor:
    """``q`` ``[T, H, 2, d]``, ``k`` ``[T, G, 2, d]``, ``v`` ``[T, G, dv]`` at positions ``0..T-1``: per head
    ``o = softmax(S_1) v - lam * softmax(S_2) v`` with ``S_m = scale * q_m k_m^T`` under the causal mask and the window,
    then ``unit(o) * out_scale``.  Result ``[T, H, dv]``."""

    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    seen = window_mask(T, window)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        a1 = one_map(q[:, head, 0], k[:, g, 0], v[:, g], scale, seen)
        a2 = one_map(q[:, head, 1], k[:, g, 1], v[:, g], scale, seen)
        o = a1 - lam * a2
        out[:, head] = (unit(o, eps) if normalise else o) * out_scale
    return out


def lambda_of(W, diff: float) -> torch.Tensor:
    return torch.exp((W["lq1"] * W["lk1"]).sum()) - torch.exp((W["lq2"] * W["lk2"]).sum()) + diff


def differential_attention(h, W, m: Mapping, eps: float, store=keep) -> torch.Tensor:
    """Two softmax maps per head over the same values, the second subtracted ``lambda`` times; the difference divided by
    its root mean square per head and scaled by ``1 - diff``."""

    T = h.shape[0]
    H, d = int(m["heads"]), int(m["dim"])
    G, dv = int(m.get("kv_heads", H)), int(m.get("vdim", d))
    diff = float(m["diff"])
    q = store(h @ W["q"].T + W["q.b"]).reshape(T, H, 2, d)
    k = store(h @ W["k"].T + W["k.b"]).reshape(T, G, 2, d)
    v = store(h @ W["v"].T + W["v.b"]).reshape(T, G, dv)
    q = unit(q, eps) * W["q.norm"]
    k = unit(k, eps) * W["k.norm"]
    positions = torch.arange(T)
    rot = m.get("rot")
    if rot:
        freqs = scaled_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"), h.dtype)
        q, k = rotate(q, positions, freqs), rotate(k, positions, freqs)
    q, k = store(q), store(k)
    mask = m.get("mask")
    out = differential_read_out(q, k, v, scale=float(m["scale"]), window=int(mask["size"]) if mask and mask.get("size") else None,
                                lam=float(lambda_of(W, diff)), out_scale=1.0 - diff, eps=eps)
    return store(out).reshape(T, H * dv) @ W["o"].T


# --------------------------------------------------------------- feed-forward
def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """``a unit(z) + b unit(z^2) + c unit(z^3) + e`` with element-wise powers and the unit taken over a token's row."""

    return coef[0] * unit(z, eps) + coef[1] * unit(z * z, eps) + coef[2] * unit(z * z * z, eps) + coef[3]


def dense_ff(h, W, eps: float, store=keep) -> torch.Tensor:
    return store(poly_norm(store(h @ W["up"].T), W["act"], eps)) @ W["down"].T


def gated_expert(h, W, prefix: str, store=keep) -> torch.Tensor:
    return store(silu(store(h @ W[prefix + "gate"].T)) * store(h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def routed_ff(h, W, mlp: Mapping, store=keep, margins=None) -> torch.Tensor:
    """Sigmoid scores, the ``top`` largest chosen, the score multiplies the chosen expert's *input*; a shared expert
    runs for every token.  ``margins`` (a list) receives, per token, the gap between the last chosen logit and the first
    one left out (infinite when every expert is used)."""

    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ W["router"].T
    scores = sigmoid(logits)
    chosen = torch.topk(logits, top, dim=-1).indices          # the sigmoid keeps the order of the logits
    if margins is not None:
        ordered = torch.sort(logits, dim=-1, descending=True).values
        margins.append(ordered[:, top - 1] - ordered[:, top] if top < experts else torch.full((h.shape[0],), math.inf, dtype=h.dtype))
    out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += gated_expert(store(scores[t, e] * h[t : t + 1]), W, f"e{e}.", store)[0]
    if mlp.get("shared"):
        out += gated_expert(h, W, "shared.", store)
    return out


# ---------------------------------------------------------------------- model
def sub(weights: Mapping[str, torch.Tensor], prefix: str, dtype) -> dict:
    return {n[len(prefix):]: t.to(dtype) for n, t in weights.items() if n.startswith(prefix)}


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens, dtype=torch.float64, store=keep, layers_out=None, margins=None):
    """Logits ``[T, vocab]``.  ``layers_out`` (a list) receives the stream after every layer, ``margins`` every router's."""

    eps = float(config["norm"]["eps"])
    x = weights["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    history = [x]
    for i, layer in enumerate(config["layers"]):
        L = sub(weights, f"l{i}.", dtype)
        h = layer_norm(x, L["norm1"], eps)
        h_mix = store(h + causal_taps(h, L["canon1"])) if "canon1" in L else store(h)
        new = x + L["ls1"] * differential_attention(h_mix, sub(L, "mix.", dtype), layer["mixer"], eps, store)
        mlp = layer.get("mlp")
        if mlp:
            h_ff = store(h + causal_taps(h, L["canon2"])) if "canon2" in L else store(h)
            M = sub(L, "mlp.", dtype)
            ff = dense_ff(h_ff, M, eps, store) if mlp["kind"] == "dense" else routed_ff(h_ff, M, mlp, store, margins)
            new = new + L["ls2"] * ff
        history.append(new)
        x = sum(L["dwa"][j] * history[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    x = layer_norm(x, weights["final.norm"].to(dtype), eps)
    return store(x) @ weights["head"].to(dtype).T
