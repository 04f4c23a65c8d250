"""Tafisun, described as parts.

A pre-norm decoder (``x <- x + mixer(norm1(x))``, ``x <- x + ff(norm2(x))``, RMS norms with plain weights) whose embedding is the
sum of a token table, a table of hashed bigrams and a sinusoidal position vector, and whose layers carry one of two
mixers: ``attention`` (grouped-query softmax attention without rotation or value projection: the values are the keys as
projected; per-head RMS norm of q and k; a bias by the logarithm of the distance; a mask in blocks of positions; an
element-wise sigmoid gate on the read-out) or ``mingru`` (a gated recurrence per channel whose gates read the current
token only).  The feed-forward is dense (``W_down relu(W_up x)^2``), a mixture of limited gated units (router: softmax over
all outputs, a correction for the choice only, groups of neighbours, outputs that return their input, a shared unit behind
a sigmoid gate per token), or absent.  The output head has a matrix of its own.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head``; a layer's tensors start with ``l<i>.``: ``norm1``, ``norm2``, ``mix.*``,
``mlp.*``; a linear map's weight is stored under the map's own name (no ``.weight``), its bias under ``<name>.b``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.tafisun import ChunkedAttention, Dense, Experts, MinGru, TafisunConfig, TafisunLayer
from .description import LayerDescription, ModelDescription

# Fixed by the design (not in config.json): the sinusoid's base and the slope inside the experts' sigmoid.
SINUSOID_BASE = 10000.0
GLU_ALPHA = 1.702


def stored_name(name: str) -> str:
    """The parts of this package call a norm's or an embedding's tensor ``<part>.weight``; the checkpoint stores it under the
    part's own name.  The bigram table belongs to the embedding part and is stored at the root."""

    if name == "embed.bigram":
        return "bigram"
    return name[: -len(".weight")] if name.endswith(".weight") else name


def _mixer(layer: TafisunLayer, config: TafisunConfig) -> dict:
    m = layer.mixer
    if isinstance(m, ChunkedAttention):
        return {"kind": "chunked_attention", "hidden_size": config.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
                "head_dim": m.dim, "eps": config.eps, "scale": m.scale, "chunk": m.chunk, "log_bias": True}
    assert isinstance(m, MinGru)
    return {"kind": "min_gru", "hidden_size": config.width, "width": m.width}


def _feed_forward(layer: TafisunLayer, config: TafisunConfig) -> dict | None:
    mlp = layer.mlp
    if mlp is None:
        return None
    if isinstance(mlp, Dense):
        return {"kind": "relu2_mlp", "hidden_size": config.width, "intermediate_size": mlp.ff}
    assert isinstance(mlp, Experts)
    return {
        "kind": "routed_experts", "hidden_size": config.width, "intermediate_size": mlp.ff, "experts": mlp.experts, "top": mlp.top,
        "act": "limited_glu", "limit": mlp.limit, "alpha": GLU_ALPHA, "router_bias": False, "score": "softmax_all",
        "correction": True, "groups": mlp.groups, "keep": mlp.keep, "weight_scale": mlp.scale, "identity": mlp.identity,
        "shared_size": mlp.shared.ff if mlp.shared else None, "shared_limit": mlp.shared.limit if mlp.shared else None,
        "shared_gate": mlp.shared is not None,
    }


def describe_tafisun(config: TafisunConfig) -> ModelDescription:
    norm = {"kind": "rms_norm", "dim": config.width, "eps": config.eps}
    layers = []
    for i, layer in enumerate(config.layers):
        ff = _feed_forward(layer, config)
        block = {
            "kind": "pre_norm", "mixer_norm": norm, "mixer": _mixer(layer, config), "ffn_norm": norm if ff else None,
            "feed_forward": ff, "names": {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "feed_forward": "mlp"},
        }
        layers.append(LayerDescription(block=block, prefix=f"l{i}"))
    bigram = config.bigram
    return ModelDescription(
        architecture=TafisunConfig.ARCHITECTURE, vocab_size=config.vocab, hidden_size=config.width,
        max_positions=TafisunConfig.MAX_POSITIONS, eos_token_ids=(),
        embedding={"prefix": "embed", "kind": "summed_embedding", "vocab_size": config.vocab, "hidden_size": config.width,
                   "bigram": (bigram.buckets, bigram.mul_prev, bigram.mul_cur) if bigram else None, "sinusoid_base": SINUSOID_BASE},
        layers=tuple(layers), order=tuple(range(len(layers))),
        final_norm={"prefix": "final.norm", **norm},
        head={"prefix": "head", "vocab_size": config.vocab, "hidden_size": config.width},
        stored_name=stored_name,
    )


TAFISUN = Architecture(
    name=TafisunConfig.ARCHITECTURE, model_type=TafisunConfig.MODEL_TYPE,
    config_from_dict=TafisunConfig.from_dict, describe=describe_tafisun,
)
register_architecture(TAFISUN, replace=True)
