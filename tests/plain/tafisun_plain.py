"""Plain, slow Tafisun forward pass: whole sequences, no cache, CPU.

One function per mechanism, elementary torch operations only, nothing shared with the engine.  It takes a
``config.json`` dict and ``{tensor name: tensor}`` with the checkpoint's own names.  ``dtype`` is the arithmetic
type (float64 separates rounding from faults).

``store`` (optional) is applied wherever a serving engine with 16-bit activations keeps a tensor in memory
between two operations: the rows a sublayer reads, the results of projections, q and k as they enter the
attention, the gated read-outs, the hidden rows of a feed-forward.  The residual stream, the statistics, the
recurrent state, the router and the logits stay in ``dtype`` either way.

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


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit(x, eps) * w


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * sigmoid(x)


# ------------------------------------------------------------------ embedding
def bigram_rows(tokens: list[int], *, buckets: int, mul_prev: int, mul_cur: int) -> list[int]:
    """The row of the bigram table for every position: a hash of (previous token, token); the table's last row
    (number ``buckets``) where there is no previous token."""

    rows = []
    for t, token in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + token * mul_cur) % buckets)
    return rows


def sinusoid(T: int, width: int, dtype) -> torch.Tensor:
    """``[T, width]``: column ``2i`` is ``sin(p * 10000^(-2i / width))``, column ``2i + 1`` the cosine of the same angle."""

    out = torch.zeros(T, width, dtype=dtype)
    p = torch.arange(T, dtype=dtype)
    for c in range(width):
        i = c // 2
        angle = p * (10000.0 ** (-2.0 * i / width))
        out[:, c] = torch.sin(angle) if c % 2 == 0 else torch.cos(angle)
    return out


def embed(tokens: list[int], weights: Mapping[str, torch.Tensor], config: Mapping, dtype) -> torch.Tensor:
    x = weights["embed"].to(dtype)[tokens]
    bigram = (config.get("embedding") or {}).get("bigram")
    if bigram:
        rows = bigram_rows(tokens, buckets=bigram["buckets"], mul_prev=bigram["mul_prev"], mul_cur=bigram["mul_cur"])
        x = x + weights["bigram"].to(dtype)[rows]
    return x + sinusoid(len(tokens), config["width"], dtype)


# ------------------------------------------------------------------ attention
def chunk_mask(T: int, size: int) -> torch.Tensor:
    """``[T, T]`` True where query i sees key j: ``j <= i`` and both in the same block of ``size`` positions counted from 0."""

    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def distance_bias(T: int, r1: float, r2: float, dtype) -> torch.Tensor:
    """``[T, T]``: ``r1 * ln(1 + r2 * (i - j))`` (what is taken off the score; entries with j > i are masked anyway)."""

    i = torch.arange(T, dtype=dtype)[:, None]
    j = torch.arange(T, dtype=dtype)[None, :]
    return r1 * torch.log(1.0 + r2 * torch.clamp(i - j, min=0.0))


def chunked_attention(q, k, v, *, scale: float, size: int, r1: torch.Tensor, r2: torch.Tensor) -> torch.Tensor:
    """q ``[T, H, d]``, k ``[T, G, d]``, v ``[T, G, dv]`` -> ``[T, H, dv]``; query head h reads key/value head ``h // (H / G)``;
    ``S = scale * q.k - r1_h ln(1 + r2_h (i - j))``; ordinary softmax over the keys of the query's own block."""

    T, H, _ = q.shape
    G = k.shape[1]
    seen = chunk_mask(T, size)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale - distance_bias(T, float(r1[h]), float(r2[h]), q.dtype)
        s = s.masked_fill(~seen, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention_mixer(h, w: Mapping[str, torch.Tensor], m: Mapping, eps: float, dtype, store) -> torch.Tensor:
    """``w``: the mixer's tensors by their short names (``q``, ``k``, ``q.norm``, ``k.norm``, ``r1``, ``r2``, ``g``, ``o``)."""

    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", d)
    q = store(h @ w["q"].to(dtype).T).view(T, H, d)
    k = store(h @ w["k"].to(dtype).T).view(T, G, d)
    v = k                                                       # the values are the keys as projected
    qn = store(rms_norm(q, w["q.norm"].to(dtype), eps))
    kn = store(rms_norm(k, w["k.norm"].to(dtype), eps))
    size = (m.get("mask") or {}).get("size") or max(T, 1)
    a = chunked_attention(qn, kn, v.reshape(T, G, dv), scale=m["scale"], size=size,
                          r1=w["r1"].to(dtype), r2=w["r2"].to(dtype))
    gate = sigmoid(store(h @ w["g"].to(dtype).T))
    return store(store(a).reshape(T, H * dv) * gate) @ w["o"].to(dtype).T


# --------------------------------------------------------------------- minGRU
def mingru_candidate(u: torch.Tensor) -> torch.Tensor:
    """``u + 1/2`` where ``u >= 0``, ``sigmoid(u)`` where ``u < 0`` (continuous, positive)."""

    return torch.where(u >= 0, u + 0.5, sigmoid(u))


def mingru_scan(z: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """``S_t = (1 - z_t) S_(t-1) + z_t c_t`` per channel from ``S = 0``; returns every ``S_t``."""

    S = torch.zeros(z.shape[1], dtype=z.dtype)
    out = torch.zeros_like(z)
    for t in range(z.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S
    return out


def mingru_mixer(h, w: Mapping[str, torch.Tensor], dtype, store) -> torch.Tensor:
    z = sigmoid(store(h @ w["z"].to(dtype).T + w["z.b"].to(dtype)))
    u = store(h @ w["x"].to(dtype).T + w["x.b"].to(dtype))
    S = mingru_scan(z, mingru_candidate(u))
    g = store(h @ w["g"].to(dtype).T)
    return store(S * silu(g)) @ w["o"].to(dtype).T


# --------------------------------------------------------------- feed-forward
def dense_ff(h, w: Mapping[str, torch.Tensor], dtype, store) -> torch.Tensor:
    up = store(h @ w["up"].to(dtype).T)
    return store(torch.relu(up) ** 2) @ w["down"].to(dtype).T


def limited_unit(h, gate_w, up_w, down_w, limit: float, dtype, store) -> torch.Tensor:
    """``W_down (g sigmoid(1.702 g) (u + 1))`` with ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``."""

    g = torch.clamp(store(h @ gate_w.to(dtype).T), max=limit)
    u = torch.clamp(store(h @ up_w.to(dtype).T), min=-limit, max=limit)
    return store(g * sigmoid(1.702 * g) * (u + 1.0)) @ down_w.to(dtype).T


def route(h, router_w, correction, r: Mapping, dtype, margins: list | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """For every token the ids ``[T, top]`` of the chosen router outputs and their weights ``[T, top]``.  ``margins`` (a list)
    receives ``[T]``: by how much the choice was clear (the last chosen score over the first one left out, the last kept
    group over the first one dropped; the smaller of the two).

    ``s = softmax(W_router h)`` over all outputs; the choice goes by ``s + correction``: outputs form ``groups.count`` equal
    groups of neighbours, a group scores the largest choice score in it, only outputs of the ``groups.keep`` best groups
    may be chosen; of those the ``top`` largest.  Weights: ``s`` (without the correction) times ``scale``."""

    s = torch.softmax(h @ router_w.to(dtype).T, dim=-1)
    choice = s + correction.to(dtype)
    T, n = choice.shape
    count, keep_groups = r["groups"]["count"], r["groups"]["keep"]
    per = n // count
    best = choice.view(T, count, per).max(dim=-1).values
    kept = torch.topk(best, keep_groups, dim=-1).indices
    allowed = torch.zeros(T, count, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(T, count, per).reshape(T, n)
    masked = choice.masked_fill(~allowed, -math.inf)
    ids = torch.topk(masked, r["top"], dim=-1).indices
    if margins is not None:
        ranked = torch.sort(masked, dim=-1, descending=True).values
        gap = ranked[:, r["top"] - 1] - ranked[:, r["top"]] if r["top"] < n else torch.full((T,), math.inf, dtype=dtype)
        groups_ranked = torch.sort(best, dim=-1, descending=True).values
        if keep_groups < count:
            gap = torch.minimum(gap, groups_ranked[:, keep_groups - 1] - groups_ranked[:, keep_groups])
        margins.append(gap)
    return ids, torch.gather(s, 1, ids) * r["scale"]


def moe_ff(h, w: Mapping[str, torch.Tensor], mlp: Mapping, dtype, store, router_input=None, margins: list | None = None) -> torch.Tensor:
    """``w``: the feed-forward's tensors by their short names.  The last ``router.identity`` router outputs return their
    input; the shared unit runs for every token, times ``sigmoid(W_sg h)`` (one number a token)."""

    r = mlp["router"]
    experts = r["experts"]
    rh = h if router_input is None else router_input
    r = {"identity": 0, "scale": 1.0, "groups": {"count": 1, "keep": 1}, **r}
    ids, weights = route(rh, w["router"], w["correction"], r, dtype, margins)
    out = torch.zeros(h.shape[0], w["router"].shape[1], dtype=dtype)
    for t in range(h.shape[0]):
        for e, weight in zip(ids[t].tolist(), weights[t]):
            if e >= experts:
                out[t] += weight * h[t]
            else:
                out[t] += weight * limited_unit(h[t : t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                                mlp["expert"]["limit"], dtype, store)[0]
    if mlp.get("shared"):
        shared = limited_unit(h, w["shared.gate"], w["shared.up"], w["shared.down"], mlp["shared"]["limit"], dtype, store)
        out = out + sigmoid(rh @ w["shared.sg"].to(dtype).T) * shared
    return out


# ---------------------------------------------------------------------- model
def sub(weights: Mapping[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    return {name[len(prefix) + 1 :]: t for name, t in weights.items() if name.startswith(prefix + ".")}


def forward(weights: Mapping[str, torch.Tensor], config: Mapping, tokens: list[int], dtype=torch.float64, *, store=keep,
            layers_out: list | None = None, margins: list | None = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence.  ``layers_out`` (a list) receives the residual rows after every layer,
    ``margins`` one ``[T]`` tensor per router (see ``route``)."""

    eps = config["norm"]["eps"]
    x = embed(tokens, weights, config, dtype)
    for i, layer in enumerate(config["layers"]):
        h = store(rms_norm(x, weights[f"l{i}.norm1"].to(dtype), eps))
        mix = sub(weights, f"l{i}.mix")
        if layer["type"] == "attention":
            x = x + attention_mixer(h, mix, layer["mixer"], eps, dtype, store)
        elif layer["type"] == "mingru":
            x = x + mingru_mixer(h, mix, dtype, store)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        mlp = layer.get("mlp")
        if mlp:
            h = store(rms_norm(x, weights[f"l{i}.norm2"].to(dtype), eps))
            ff = sub(weights, f"l{i}.mlp")
            x = x + (dense_ff(h, ff, dtype, store) if mlp["kind"] == "dense" else moe_ff(h, ff, mlp, dtype, store, margins=margins))
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, weights["final.norm"].to(dtype), eps)
    return x @ weights["head"].to(dtype).T
