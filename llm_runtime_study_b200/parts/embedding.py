"""Token embedding and output head."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import functional as F
from ..weights.checkpoint import TensorSpec
from .base import EMBEDDINGS, HEADS, FixedState, Part, Runtime, WeightedRows
from .linear import Projection


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """``h = E[token] * scale`` (mini_llm/model/base.py:72-74; Qwen3 uses scale 1)."""

    graph_safe = True

    def __init__(self, *, vocab_size: int, hidden_size: int, scale: float = 1.0) -> None:
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.weight = runtime.place_matrix(tensors["weight"])

    fuses_norms = True    # takes a keyword ``next_norm`` and may return (rows, WeightedRows for that norm)

    def forward(self, token_ids: torch.Tensor, next_norm: Any = None):
        fusable = next_norm.fusable() if next_norm is not None and Projection.FUSE_NORMS else None
        if (fusable is not None and self.runtime.dtype == torch.bfloat16 and token_ids.shape[0] <= 16
                and fusable[0].shape[0] == self.hidden_size and self.hidden_size % 8 == 0 and self.hidden_size <= 8 * 2048):
            rows, weighted, row_scale = F.embedding_weighted(token_ids, self.weight, self.scale, *fusable)
            return rows, WeightedRows(weighted, row_scale)
        return F.embedding(token_ids, self.weight, self.scale)


@EMBEDDINGS.register("summed_embedding")
class SummedEmbedding(Part):
    """``h = E[token] * scale + B[row] + pos(p)``: a token table, a table of hashed bigrams and a sinusoidal position vector,
    each of the last two optional.

    * ``bigram = (buckets, mul_prev, mul_cur)``: ``row = (previous token * mul_prev + token * mul_cur) mod buckets``; a
      sequence's first token reads row ``buckets``, the table's last.  The token before a step's first one is kept per
      request slot (an int32 a request), so a prompt may be cut anywhere.
    * ``sinusoid_base``: column ``2i`` of ``pos(p)`` is ``sin(p * base^(-2i / hidden))``, column ``2i + 1`` the cosine of the same
      angle; frequencies, angles and their sines are formed in float64 and rounded once.

    Tensors: ``weight`` ``[vocab, hidden]`` and ``bigram`` ``[buckets + 1, hidden]`` (``table_name`` and ``bigram_name`` rename
    them)."""

    graph_safe = True
    takes_context = True     # forward(ctx, cache): it reads positions, entries and slots, and keeps state per request

    def __init__(self, *, vocab_size: int, hidden_size: int, scale: float = 1.0, bigram: tuple[int, int, int] | None = None,
                 sinusoid_base: float | None = None, table_name: str = "weight", bigram_name: str = "bigram") -> None:
        if vocab_size <= 0 or hidden_size <= 0:
            raise ValueError("embedding sizes must be positive")
        if bigram is not None and (len(bigram) != 3 or int(bigram[0]) <= 0 or min(int(bigram[1]), int(bigram[2])) < 0):
            raise ValueError("bigram is (buckets > 0, mul_prev >= 0, mul_cur >= 0)")
        if sinusoid_base is not None and sinusoid_base <= 0:
            raise ValueError("the sinusoid's base must be positive")
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.bigram = None if bigram is None else tuple(int(v) for v in bigram)
        self.sinusoid_base = None if sinusoid_base is None else float(sinusoid_base)
        self.table_name, self.bigram_name = table_name, bigram_name
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {self.table_name: TensorSpec((self.vocab_size, self.hidden_size))}
        if self.bigram is not None:
            specs[self.bigram_name] = TensorSpec((self.bigram[0] + 1, self.hidden_size))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.weight = runtime.place_matrix(tensors[self.table_name])
        self.bigram_table = runtime.place_matrix(tensors[self.bigram_name]) if self.bigram is not None else None
        self.freq = None
        if self.sinusoid_base is not None:
            pairs = (self.hidden_size + 1) // 2
            freq = [self.sinusoid_base ** (-2.0 * i / self.hidden_size) for i in range(pairs)]
            self.freq = torch.tensor(freq, dtype=torch.float64).to(runtime.device)

    def cache_requirement(self):
        return FixedState((1,), torch.int32, name="previous_token") if self.bigram is not None else None

    def forward(self, ctx: Any, cache: Any) -> torch.Tensor:
        buckets, mul_prev, mul_cur = self.bigram or (0, 0, 0)
        previous = cache.states["previous_token"] if self.bigram is not None else None
        return F.embedding_sum(ctx.token_ids, self.weight, self.bigram_table, positions=ctx.positions, token_entry=ctx.token_entry,
                               q_start=ctx.q_start, slots=ctx.slots, previous=previous, freq=self.freq, buckets=buckets,
                               mul_prev=mul_prev, mul_cur=mul_cur, scale=self.scale)


@HEADS.register("linear_head")
class OutputHead(Part):
    """``logits = h W^T`` in float32, no bias (mini_llm/model/qwen.py:112).  With
    ``tied`` the weight may be absent from the checkpoint; the embedding matrix
    is used then.  A stored ``lm_head.weight`` is always used when present."""

    graph_safe = True

    def __init__(self, *, vocab_size: int, hidden_size: int, tied: bool = False) -> None:
        self.vocab_size, self.hidden_size, self.tied = vocab_size, hidden_size, bool(tied)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime, *, embedding: TokenEmbedding | None = None) -> None:
        self.runtime = runtime
        if "weight" in tensors:
            self.proj = Projection([tensors["weight"]], None, runtime)
        elif self.tied and embedding is not None:
            self.proj = Projection.__new__(Projection)
            self.proj.runtime, self.proj.weight, self.proj.bias = runtime, embedding.weight, None
            self.proj.out_features, self.proj.in_features = embedding.weight.shape
        else:
            raise KeyError("output head has no weight and is not tied to the embedding")

    fuses_norms = True    # takes ``WeightedRows`` prepared for the final norm

    def forward(self, x: "torch.Tensor | WeightedRows") -> torch.Tensor:
        return self.proj(x, torch.float32)
