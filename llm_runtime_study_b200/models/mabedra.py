"""Mabedra, described as parts.

A decoder whose two sublayers read one layer-normed copy of the stream side by side
(``x <- x + s1 * mixer(h + conv1(h)) + s2 * ff(h + conv2(h))`` with ``h = layer_norm(x)``, a short causal convolution over time
on each sublayer's input and a scale per channel on each output), and whose stream after every layer is a weighted
average of the results of all layers so far and the embedding's output.  The mixer is differential attention (two
softmax maps per head over the same values, the second subtracted; per-map RMS norm of q and k, a rotation with stretched
long wavelengths on the leading columns, a sliding window); the feed-forward is dense with a polynomial activation of
normalised powers, or a mixture of gated experts whose sigmoid router weight multiplies the expert's input, beside a
shared expert.  The output head has a matrix of its own.

Tensor names: a layer's tensors start with ``l<i>.``; ``norm1``, ``mix.*``, ``mlp.*``, ``ls1``, ``ls2``, ``canon1``, ``canon2``,
``dwa``; a linear map's weight is stored under the map's own name (no ``.weight``), its bias under ``<name>.b``.
"""

from __future__ import annotations

from ..config.mabedra import DenseFF, ExpertsFF, MabedraConfig, MabedraLayer
from ..config.registry import Architecture, register_architecture
from .description import LayerDescription, ModelDescription
from .sorulix import stored_name


def _mixer(layer: MabedraLayer, config: MabedraConfig) -> dict:
    m = layer.mixer
    position = None
    if m.rot_dims:
        scaling = m.rot_scaling
        position = {"kind": "rope", "head_dim": m.dim, "theta": m.rot_base, "rotary_dim": m.rot_dims,
                    "scaling": None if scaling is None else {"factor": scaling.factor, "low": scaling.low, "high": scaling.high,
                                                             "original": scaling.original}}
    return {"kind": "differential_attention", "hidden_size": config.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
            "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale, "diff": m.diff, "eps": config.eps, "window": m.window,
            "position": position}


def _feed_forward(layer: MabedraLayer, config: MabedraConfig) -> dict | None:
    mlp = layer.mlp
    if mlp is None:
        return None
    if isinstance(mlp, DenseFF):
        return {"kind": "poly_norm_mlp", "hidden_size": config.width, "intermediate_size": mlp.ff, "eps": config.eps}
    assert isinstance(mlp, ExpertsFF)
    return {"kind": "routed_experts", "hidden_size": config.width, "intermediate_size": mlp.ff, "experts": mlp.experts,
            "top": mlp.top, "act": "silu_glu", "score": "sigmoid", "weight_on": "input", "router_bias": False,
            "shared_size": mlp.shared_ff}


def describe_mabedra(config: MabedraConfig) -> ModelDescription:
    norm = {"kind": "layer_norm", "dim": config.width, "eps": config.eps}
    layers = []
    for i, layer in enumerate(config.layers):
        block = {
            "kind": "parallel_sublayers", "hidden_size": config.width, "norm": norm, "mixer": _mixer(layer, config),
            "feed_forward": _feed_forward(layer, config), "taps": config.taps, "layer_scale": True, "average_over": i + 2,
            "average_capacity": len(config.layers) + 1,
        }
        layers.append(LayerDescription(block=block, prefix=f"l{i}"))
    return ModelDescription(
        architecture=MabedraConfig.ARCHITECTURE, vocab_size=config.vocab, hidden_size=config.width,
        max_positions=MabedraConfig.MAX_POSITIONS, eos_token_ids=(),
        embedding={"prefix": "embed", "vocab_size": config.vocab, "hidden_size": config.width},
        layers=tuple(layers), order=tuple(range(len(layers))),
        final_norm={"prefix": "final.norm", **norm},
        head={"prefix": "head", "vocab_size": config.vocab, "hidden_size": config.width, "tied": False},
        stored_name=stored_name,
    )


MABEDRA = Architecture(
    name=MabedraConfig.ARCHITECTURE, model_type=MabedraConfig.MODEL_TYPE,
    config_from_dict=MabedraConfig.from_dict, describe=describe_mabedra,
)
register_architecture(MABEDRA, replace=True)
