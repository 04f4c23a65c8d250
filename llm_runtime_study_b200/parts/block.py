"""Arrangement of norm, mixer and feed-forward in one layer."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..weights.checkpoint import TensorSpec
from ..weights.view import TensorView
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, ResidualStream, Runtime

_DEFAULT_NAMES = {
    "mixer_norm": "input_layernorm",
    "mixer": "self_attn",
    "ffn_norm": "post_attention_layernorm",
    "feed_forward": "mlp",
}


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``h = h + mixer(norm_1(h)); h = h + ffn(norm_2(h))``
    (mini_llm/model/qwen.py:58-72).  The additions are carried out by the *next*
    norm, in float32, while it reads the rows anyway.  ``names`` gives the
    checkpoint's name of each sub-part below the layer's prefix.  A layer
    without a feed-forward (``feed_forward=None``) is its first half only."""

    def __init__(
        self, *, mixer: Mapping[str, Any], feed_forward: Mapping[str, Any] | None, mixer_norm: Mapping[str, Any],
        ffn_norm: Mapping[str, Any] | None = None, names: Mapping[str, str] | None = None,
    ) -> None:
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self.mixer = MIXERS.build(mixer)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward else None
        self.ffn_norm = NORMS.build(ffn_norm) if feed_forward else None
        if feed_forward and not ffn_norm:
            raise ValueError("a pre_norm block with a feed-forward needs the norm before it (ffn_norm)")

    graph_safe = True

    def children(self):
        return tuple(part for _, part in self._parts())

    def _parts(self):
        parts = [(self.names["mixer_norm"], self.mixer_norm), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            parts += [(self.names["ffn_norm"], self.ffn_norm), (self.names["feed_forward"], self.feed_forward)]
        return tuple(parts)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {f"{prefix}.{n}": s for prefix, part in self._parts() for n, s in part.tensor_specs().items()}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        view = TensorView.of(tensors)
        for prefix, part in self._parts():
            part.load(view.sub(prefix), runtime)

    fuses_norms = True

    def first_norm(self):
        return self.mixer_norm

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any, next_norm: Any = None) -> None:
        x = stream.take_rows(self.mixer_norm, self.mixer)
        after_mixer = self.ffn_norm if self.feed_forward is not None else next_norm
        stream.put(self._run(self.mixer, (x, ctx, cache), stream.resid, after_mixer), after_mixer)
        if self.feed_forward is None:
            return
        x = stream.take_rows(self.ffn_norm, self.feed_forward)
        stream.put(self._run(self.feed_forward, (x, ctx), stream.resid, next_norm), next_norm)

    @staticmethod
    def _run(part: Any, args: tuple, resid: torch.Tensor, next_norm: Any):
        """Call a mixer or feed-forward with as much as it says it can take."""

        if not part.adds_to_residual:
            return part.forward(*args)
        if part.fuses_norms:
            return part.forward(*args, residual=resid, next_norm=next_norm)
        return part.forward(*args, residual=resid)


@BLOCKS.register("output_norm")
class OutputNormBlock(Block):
    """``h = h + norm_1(mixer(h)); h = h + norm_2(ffn(h))``: the sublayers read the residual rows themselves (rounded to
    the activation type where that is not float32) and the norm sits on their output only.  The kernel that normalises a
    sublayer's output adds it into the float32 rows and hands the next sublayer its rounded copy in the same pass.
    ``names`` as for ``pre_norm``; a layer without a feed-forward is its first half only."""

    graph_safe = True

    def __init__(
        self, *, mixer: Mapping[str, Any], feed_forward: Mapping[str, Any] | None, mixer_norm: Mapping[str, Any],
        ffn_norm: Mapping[str, Any] | None = None, names: Mapping[str, str] | None = None,
    ) -> None:
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self.mixer = MIXERS.build(mixer)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward else None
        self.ffn_norm = NORMS.build(ffn_norm) if feed_forward else None
        if feed_forward and not ffn_norm:
            raise ValueError("an output_norm block with a feed-forward needs the norm behind it (ffn_norm)")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and norm.fusable() is None:
                raise ValueError("an output_norm block normalises with a norm of the form w * x * rsqrt(mean(x^2) + eps)")

    def children(self):
        return tuple(part for _, part in self._parts())

    _parts = PreNormBlock._parts
    tensor_specs = PreNormBlock.tensor_specs
    load = PreNormBlock.load

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        from ..ops import mixer_steps as M

        resid = stream.resid
        if stream.delta is not None:
            resid += stream.delta
            stream.put(None, None)
        act = self.runtime.dtype
        rounds = act != torch.float32
        # what the block before this one left for its reader, if it was a block of this kind
        x = stream.rounded
        stream.put(None, None)
        if x is None:
            x = M.norm_accumulate_round(None, None, 0.0, resid, act) if rounds else resid
        out = self.mixer.forward(x, ctx, cache)
        weight, eps = self.mixer_norm.fusable()
        x = M.norm_accumulate_round(out, weight, eps, resid, act if rounds else None)
        if self.feed_forward is not None:
            # a feed-forward that can hand over its experts' rows unsummed does: the norm's kernel forms the sum
            pieces = {"pieces": True} if getattr(self.feed_forward, "returns_pieces", False) else {}
            out = self.feed_forward.forward(x if rounds else resid, ctx, **pieces)
            weight, eps = self.ffn_norm.fusable()
            x = M.norm_accumulate_round(out, weight, eps, resid, act if rounds else None)
        if rounds:
            stream.rounded = x


_PARALLEL_NAMES = {
    "norm": "norm1", "mixer": "mix", "feed_forward": "mlp", "mixer_scale": "ls1", "ffn_scale": "ls2",
    "mixer_taps": "canon1", "ffn_taps": "canon2", "average": "dwa",
}


@BLOCKS.register("parallel_sublayers")
class ParallelSublayersBlock(Block):
    """One norm, both sublayers read its output: with ``h = norm(x)``,
    ``x_new = x + s1 * mixer(h + conv1(h)) + s2 * ff(h + conv2(h))``.

    * ``taps`` > 1: each sublayer's input is ``h + conv(h)``, a causal convolution over time per channel with weights
      ``[width, taps]`` of its own (``conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j)``, zeros before the sequence's start).  The
      last ``taps - 1`` rows of ``h`` are kept per request (float32), one array for both sublayers since they read the same ``h``.
    * ``layer_scale``: ``s1`` and ``s2`` are vectors of the width (otherwise 1).
    * ``average_over = k``: the block's result is kept beside the results of all blocks before it and the embedding's
      output (``k`` rows of the stream in all), and the stream handed on is ``sum_j a[j] * result_j`` with the block's
      own ``k`` weights.  ``None``: the stream is the block's result.  ``average_capacity``: the largest ``k`` among the model's
      blocks (room for all results is made once per step, by the first block).

    The norm's output, the convolution's sums and the stream stay float32; the sublayers get their inputs in the run type.
    ``names`` gives the checkpoint's name of each sub-part below the layer's prefix."""

    graph_safe = True
    KEPT = "kept_inputs"

    def __init__(
        self, *, hidden_size: int, mixer: Mapping[str, Any], feed_forward: Mapping[str, Any] | None, norm: Mapping[str, Any],
        taps: int = 1, layer_scale: bool = False, average_over: int | None = None, average_capacity: int | None = None,
        names: Mapping[str, str] | None = None,
    ) -> None:
        if hidden_size <= 0 or taps <= 0 or (average_over is not None and average_over < 2):
            raise ValueError("a parallel_sublayers block needs a positive width and taps, and an average over at least two results")
        self.names = {**_PARALLEL_NAMES, **(names or {})}
        self.hidden_size, self.taps, self.layer_scale, self.average_over = hidden_size, int(taps), bool(layer_scale), average_over
        # how many results the model's deepest block of this kind averages over: room for them is made once per step
        self.average_capacity = max(average_capacity or 0, average_over or 0)
        self.norm = NORMS.build(norm)
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward else None

    def children(self):
        return tuple(part for _, part in self._parts())

    def _parts(self):
        parts = [(self.names["norm"], self.norm), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            parts.append((self.names["feed_forward"], self.feed_forward))
        return tuple(parts)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {f"{prefix}.{n}": s for prefix, part in self._parts() for n, s in part.tensor_specs().items()}
        w, ff = self.hidden_size, self.feed_forward is not None
        if self.layer_scale:
            specs[self.names["mixer_scale"]] = TensorSpec((w,), init="one_plus_normal", std=0.2)
            if ff:
                specs[self.names["ffn_scale"]] = TensorSpec((w,), init="one_plus_normal", std=0.2)
        if self.taps > 1:
            specs[self.names["mixer_taps"]] = TensorSpec((w, self.taps), init="normal", std=0.3)
            if ff:
                specs[self.names["ffn_taps"]] = TensorSpec((w, self.taps), init="normal", std=0.3)
        if self.average_over is not None:
            specs[self.names["average"]] = TensorSpec((self.average_over,), init="normal", std=0.6)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        view = TensorView.of(tensors)
        for prefix, part in self._parts():
            part.load(view.sub(prefix), runtime)
        ff = self.feed_forward is not None
        f32 = runtime.place_vector_f32
        self.mixer_scale = f32(tensors[self.names["mixer_scale"]]) if self.layer_scale else None
        self.ffn_scale = f32(tensors[self.names["ffn_scale"]]) if self.layer_scale and ff else None
        self.mixer_taps = f32(tensors[self.names["mixer_taps"]]) if self.taps > 1 else None
        self.ffn_taps = f32(tensors[self.names["ffn_taps"]]) if self.taps > 1 and ff else None
        self.average = f32(tensors[self.names["average"]]) if self.average_over is not None else None

    def first_norm(self):
        return self.norm

    def cache_requirement(self):
        needs = self.mixer.cache_requirement()
        needs = () if needs is None else (tuple(needs) if isinstance(needs, (tuple, list)) else (needs,))
        if self.taps > 1:
            from .base import FixedState

            needs += (FixedState((self.taps - 1, self.hidden_size), torch.float32, name=self.KEPT),)
        return needs or None

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        from ..ops import block_steps as B
        from ..ops import sequence_state as S

        resid, act = stream.resid, self.runtime.dtype
        delta = stream.delta
        stream.put(None, None)
        if self.average_over is not None and stream.results is None:
            # the first block of this kind: the rows it starts from are result 0 (the embedding's output)
            if delta is not None:
                resid += delta
                delta = None
            stream.results = torch.empty((self.average_capacity, *resid.shape), dtype=torch.float32, device=resid.device)
            stream.results[0].copy_(resid)
        if self.taps > 1:
            h = self.norm.add_norm(resid, delta, torch.float32)
            kept = cache.states[self.KEPT]
            x_mix, x_ff = B.taps_pair(h, self.mixer_taps, self.ffn_taps, kept, q_start=ctx.q_start, slots=ctx.slots,
                                      token_entry=ctx.token_entry, out_dtype=act)
            S.conv_state_update(h, kept, ctx.q_start, ctx.slots)
        else:
            x_mix = x_ff = self.norm.add_norm(resid, delta)
        out_mix = self.mixer.forward(x_mix, ctx, cache)
        out_ff = self.feed_forward.forward(x_ff, ctx) if self.feed_forward is not None else None
        results = stream.results
        if self.average_over is not None and results.shape[0] < self.average_over:
            # blocks further down average over more results than the first one made room for
            grown = torch.empty((self.average_over, *resid.shape), dtype=torch.float32, device=resid.device)
            grown[: results.shape[0]].copy_(results)
            results = stream.results = grown
        B.scale_sum_average(resid, out_mix, self.mixer_scale, out_ff, self.ffn_scale, results, self.average,
                            (self.average_over or 2) - 2)
