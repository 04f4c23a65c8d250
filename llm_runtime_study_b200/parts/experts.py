"""A feed-forward made of several small ones, of which a router picks a few per token."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import block_steps as B
from ..ops import functional as F
from ..ops import grouped as G
from ..ops.mixer_steps import PairedRows
from ..weights.checkpoint import TensorSpec
from .base import FEED_FORWARDS, FeedForward, Runtime
from .linear import Projection

ACTS = ("relu2", "silu_glu", "limited_glu")
GATED = ("silu_glu", "limited_glu")


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """``experts`` feed-forward layers without biases, of which each token uses the ``top`` with the largest router logits
    ``z = W_router x (+ b_router)`` (float32).  Every choice is a parameter:

    * ``act``: ``relu2``: an expert is ``W_down relu(W_up x)^2``; ``silu_glu``: ``W_down (silu(W_gate x) * (W_up x))``;
      ``limited_glu``: ``W_down (g sigmoid(alpha g) (u + 1))`` with ``g = min(W_gate x, limit)``, ``u = clamp(W_up x, -limit, limit)``.
    * ``score``: ``softmax_chosen``: the weights are the softmax over the chosen logits only; ``sigmoid``: each chosen
      expert's ``sigmoid(z)``, not renormalised; ``softmax_all``: ``s = softmax(z)`` over all router outputs, the choice goes
      by ``s + correction`` (``correction``: a stored vector) among the outputs of the ``keep`` best of ``groups`` equal groups of
      neighbours (a group scores its largest choice score), the weights are ``weight_scale * s`` of the chosen, not renormalised.
    * ``identity``: that many further router outputs behind the experts' that have no tensors and return their input.
    * ``weight_on``: ``output``: the result is ``sum w_e expert_e(x)``; ``input``: ``sum expert_e(w_e x)``.
    * ``shared_size``: a further expert of that inner size (same form; ``shared_limit``) that runs for every token and is
      added; with ``shared_gate`` it is multiplied by ``sigmoid(W_sg x)``, one number per token.

    Tensors: ``router`` (``router.b``), ``correction``, ``e<j>.up`` ``[ff, hidden]`` (``e<j>.gate``), ``e<j>.down`` ``[hidden, ff]``,
    ``shared.gate|up|down``, ``shared.sg`` ``[1, hidden]``.

    The (token, choice) pairs are sorted by expert on the device and every expert's rows are padded to whole tiles, so the
    two products run as one launch each over all experts, sized without the host knowing the counts.  With ``input`` weights
    the factor is applied where the gated unit is formed: ``W (w x) = w (W x)``, so ``silu(w g) * (w u)`` of the unweighted
    products ``g`` and ``u`` is the same expert on the weighted input."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int, experts: int, top: int, act: str = "relu2",
                 router_bias: bool = True, score: str = "softmax_chosen", weight_on: str = "output",
                 shared_size: int | None = None, limit: float | None = None, alpha: float = 1.702, correction: bool = False,
                 groups: int = 1, keep: int = 1, weight_scale: float = 1.0, identity: int = 0, shared_limit: float | None = None,
                 shared_gate: bool = False) -> None:
        if min(hidden_size, intermediate_size, experts, top) <= 0 or top > experts:
            raise ValueError("expert sizes must be positive and top at most the number of experts")
        if act not in ACTS:
            raise ValueError(f"unknown expert activation {act!r}; expected one of {ACTS}")
        if score not in G.SCORES:
            raise ValueError(f"unknown router score {score!r}; expected one of {sorted(G.SCORES)}")
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on is 'output' or 'input', got {weight_on!r}")
        if weight_on == "input" and act != "silu_glu":
            raise ValueError("weights on the experts' inputs are built for the gated unit only")
        if shared_size is not None and (shared_size <= 0 or act not in GATED):
            raise ValueError("a shared expert needs a positive size and a gated unit")
        if act == "limited_glu" and (limit is None or limit <= 0 or (shared_size is not None and (shared_limit is None or shared_limit <= 0))):
            raise ValueError("the limited unit needs a positive limit (and one for the shared expert)")
        outputs = experts + identity
        if identity < 0 or groups <= 0 or outputs % groups or not 0 < keep <= groups or top > keep * (outputs // groups):
            raise ValueError("router outputs must form equal groups, and the kept groups must hold at least `top` outputs")
        if (groups > 1 or correction or identity or weight_scale != 1.0) and score != "softmax_all":
            raise ValueError("groups, a correction, identity outputs and a weight scale belong to the score 'softmax_all'")
        if identity and weight_on != "output":
            raise ValueError("identity outputs are weighted on the output")
        if shared_gate and shared_size is None:
            raise ValueError("a gate on the shared expert needs a shared expert")
        self.hidden_size, self.intermediate_size, self.experts, self.top = hidden_size, intermediate_size, experts, top
        self.act, self.router_bias, self.score, self.weight_on, self.shared_size = act, bool(router_bias), score, weight_on, shared_size
        self.limit, self.alpha, self.correction, self.groups, self.keep = limit, float(alpha), bool(correction), groups, keep
        self.weight_scale, self.identity, self.shared_limit, self.shared_gate = float(weight_scale), identity, shared_limit, bool(shared_gate)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, f = self.hidden_size, self.intermediate_size
        outputs = self.experts + self.identity
        specs = {"router": TensorSpec((outputs, h), init="normal", std=h ** -0.5 * 2)}
        if self.router_bias:
            specs["router.b"] = TensorSpec((outputs,), init="normal", std=0.5)
        if self.correction:
            specs["correction"] = TensorSpec((outputs,), init="normal", std=0.1)
        if self.shared_gate:
            specs["shared.sg"] = TensorSpec((1, h), init="normal", std=h ** -0.5 * 2)
        for e in range(self.experts):
            if self.act in GATED:
                specs[f"e{e}.gate"] = TensorSpec((f, h))
            specs[f"e{e}.up"] = TensorSpec((f, h))
            specs[f"e{e}.down"] = TensorSpec((h, f))
        if self.shared_size is not None:
            specs.update({"shared.gate": TensorSpec((self.shared_size, h)), "shared.up": TensorSpec((self.shared_size, h)),
                          "shared.down": TensorSpec((h, self.shared_size))})
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.router = tensors["router"].to(device=runtime.device).to(torch.float32).contiguous()
        self.router_b = runtime.place_vector_f32(tensors["router.b"]) if self.router_bias else None
        self.correction_b = runtime.place_vector_f32(tensors["correction"]) if self.correction else None
        if self.shared_gate:            # the gate's row rides behind the router's: one pass over the token's row gives both
            gate_row = tensors["shared.sg"].to(device=runtime.device).to(torch.float32).reshape(1, -1)
            self.router = torch.cat([self.router, gate_row]).contiguous()
            if self.router_b is not None:
                self.router_b = torch.cat([self.router_b, torch.zeros(1, dtype=torch.float32, device=runtime.device)])
        if self.act in GATED:      # per expert: the rows of gate, then the rows of up (one product gives both)
            self.up = torch.stack([torch.cat([runtime.place_matrix(tensors[f"e{e}.gate"]), runtime.place_matrix(tensors[f"e{e}.up"])])
                                   for e in range(self.experts)])
        else:
            self.up = torch.stack([runtime.place_matrix(tensors[f"e{e}.up"]) for e in range(self.experts)])
        self.down = torch.stack([runtime.place_matrix(tensors[f"e{e}.down"]) for e in range(self.experts)])
        self.shared_up = self.shared_down = None
        if self.shared_size is not None:
            self.shared_up = Projection([tensors["shared.gate"], tensors["shared.up"]], None, runtime)
            self.shared_down = Projection([tensors["shared.down"]], None, runtime)

    # the weighted sum over a token's experts may be left to the consumer (``PairedRows``): see ``forward``
    @property
    def returns_pieces(self) -> bool:
        return self.shared_size is None and self.weight_on == "output" and not self.identity

    def forward(self, x: torch.Tensor, ctx: Any, *, pieces: bool = False) -> "torch.Tensor | PairedRows":
        """``pieces``: return the experts' rows with the pairing instead of their weighted sum, for a consumer that forms the
        sum while it reads the rows anyway (the norm behind this part does)."""

        wide = G.wide_tiles_pay(x.shape[0], self.top, x.dtype, self.hidden_size, self.intermediate_size)
        routing = G.route(x, self.router, self.router_b, top=self.top, wide_tiles=wide, score=self.score, correction=self.correction_b,
                          groups=self.groups, keep=self.keep, scale=self.weight_scale, identity=self.identity,
                          extra=1 if self.shared_gate else 0)
        if self.act == "limited_glu":
            on_input = False
            hidden = F.glu_limit(G.expert_linear(x, self.up, routing, gather=True), self.limit, self.alpha)
        elif self.act == "silu_glu":
            gate_up = G.expert_linear(x, self.up, routing, gather=True)
            on_input = self.weight_on == "input"
            hidden = B.silu_mul_scaled(gate_up, routing.pair_row, routing.weights.view(-1) if on_input else None)
        else:
            on_input = False
            hidden = G.expert_linear(x, self.up, routing, gather=True, act=self.act)
        rows = G.expert_linear(hidden, self.down, routing, gather=False, out_dtype=torch.float32)
        if pieces and self.returns_pieces:
            return PairedRows(rows, routing.pair_row, routing.weights)
        if self.identity or self.shared_gate:
            # one pass forms the weighted sum, hands an identity output the token's own row, and adds the gated shared expert
            shared = self.shared_down(self._shared_hidden(x), torch.float32) if self.shared_gate else None
            out = G.combine_mixed(rows, routing, x, extra=shared, extra_scale=routing.extra)
            if self.shared_gate:
                return out
        else:
            out = G.combine(rows, routing, weighted=not on_input)
        if self.shared_down is not None:
            shared = self.shared_down(self._shared_hidden(x), torch.float32, add_to=out)
            if shared is not None:
                out += shared
        return out

    def _shared_hidden(self, x: torch.Tensor) -> torch.Tensor:
        if self.act == "limited_glu":
            return F.glu_limit(self.shared_up(x), self.shared_limit, self.alpha)
        return B.silu_mul_scaled(self.shared_up(x))
