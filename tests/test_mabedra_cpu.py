"""Mabedra without a GPU: configuration, description, tensor names, cache layout, and the plain implementation's own
mechanisms against closed forms."""

import copy
import math

import pytest
import torch

from llm_runtime_study_b200.cache.manager import CacheLayout
from llm_runtime_study_b200.config import MabedraConfig, architecture_for
from llm_runtime_study_b200.errors import ConfigError
from llm_runtime_study_b200.models.description import tensor_schema
from llm_runtime_study_b200.models.mabedra import describe_mabedra
from llm_runtime_study_b200.models.model import DecoderModel
from llm_runtime_study_b200.parts import FixedState, PagedTensors
from tests import helpers
from tests.plain import mabedra_plain as plain


def test_the_registry_finds_the_design_by_its_architecture_key():
    assert architecture_for(helpers.MABEDRA_A).name == "Mabedra"


def test_every_size_and_constant_is_read_from_the_dict():
    cfg = MabedraConfig.from_dict(helpers.MABEDRA_A)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.taps, len(cfg.layers)) == (157, 48, 1e-5, 3, 4)
    first, second, third, last = (layer.mixer for layer in cfg.layers)
    assert (first.heads, first.kv_heads, first.dim, first.vdim, first.diff, first.scale, first.window) == (3, 1, 8, 12, 0.2, 0.4, 7)
    assert (first.rot_base, first.rot_dims) == (500.0, 4)
    assert (first.rot_scaling.factor, first.rot_scaling.low, first.rot_scaling.high, first.rot_scaling.original) == (4.0, 1.0, 3.0, 32.0)
    assert second.window is None and (second.rot_dims, second.rot_scaling.original) == (16, 64.0)
    assert third.rot_dims == 0 and third.rot_scaling is None and last.rot_scaling is None and last.rot_dims == 24
    assert cfg.layers[0].mlp.ff == 40 and cfg.layers[2].mlp is None
    moe = cfg.layers[1].mlp
    assert (moe.experts, moe.top, moe.ff, moe.shared_ff) == (5, 2, 24, 16) and cfg.layers[3].mlp.shared_ff is None
    assert MabedraConfig.from_dict(helpers.MABEDRA_C).taps == 1          # no convolution where the key is absent


@pytest.mark.parametrize("patch,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.__setitem__("width", True), "width must be int, got bool"),
    (lambda c: c["canon"].__setitem__("taps", 0), "canon.taps"),
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "not a layer of this design"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 2), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "not a feed-forward of this design"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "exceeds experts"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].__setitem__("high", 0.5), "scaling"),
    (lambda c: c.__setitem__("layers", []), "layers must not be empty"),
])
def test_a_bad_config_is_refused_with_the_key_named(patch, match):
    raw = copy.deepcopy(helpers.MABEDRA_A)
    patch(raw)
    with pytest.raises(ConfigError, match=match):
        MabedraConfig.from_dict(raw)


def test_tensor_names_and_shapes():
    schema = tensor_schema(describe_mabedra(MabedraConfig.from_dict(helpers.MABEDRA_A)))
    shapes = {name: tuple(spec.shape) for name, spec in schema.items() if not spec.optional}
    assert shapes["embed"] == (157, 48) and shapes["head"] == (157, 48) and shapes["final.norm"] == (48,) and shapes["l0.norm1"] == (48,)
    assert shapes["l0.mix.q"] == (3 * 2 * 8, 48) and shapes["l0.mix.q.b"] == (48,) and shapes["l0.mix.k"] == (16, 48)
    assert shapes["l0.mix.v"] == (12, 48) and shapes["l0.mix.v.b"] == (12,) and shapes["l0.mix.o"] == (48, 36)
    assert shapes["l0.mix.q.norm"] == (8,) and shapes["l0.mix.lk2"] == (8,)
    assert shapes["l0.mlp.up"] == (40, 48) and shapes["l0.mlp.down"] == (48, 40) and shapes["l0.mlp.act"] == (4,)
    assert shapes["l0.ls1"] == (48,) and shapes["l0.canon2"] == (48, 3) and shapes["l0.dwa"] == (2,) and shapes["l3.dwa"] == (5,)
    assert shapes["l1.mlp.router"] == (5, 48) and "l1.mlp.router.b" not in shapes
    assert shapes["l1.mlp.e4.gate"] == (24, 48) and shapes["l1.mlp.e0.down"] == (48, 24) and shapes["l1.mlp.shared.up"] == (16, 48)
    assert "l2.ls2" not in shapes and "l2.canon2" not in shapes and "l2.norm2" not in shapes and shapes["l2.canon1"] == (48, 3)
    assert "l3.mlp.shared.gate" not in shapes and "l3.mlp.e3.up" not in shapes
    no_taps = tensor_schema(describe_mabedra(MabedraConfig.from_dict(helpers.MABEDRA_C)))
    assert "l0.canon1" not in no_taps and "l0.ls1" in no_taps


def test_cache_layout_follows_the_layers():
    """Every layer keeps one key row of both maps and one value row per token and key/value head, with its own window, and
    the last inputs of its convolution (none where there is a single tap)."""

    model = DecoderModel(describe_mabedra(MabedraConfig.from_dict(helpers.MABEDRA_A)))
    layout = model.cache_layout()
    by_layers = {group.layers: group.requirement for group in layout.groups}
    assert by_layers[(0,)] == PagedTensors(tensors=(("keys", (1, 16)), ("values", (1, 12))), window=7)
    assert by_layers[(1,)] == PagedTensors(tensors=(("keys", (2, 32)), ("values", (2, 8))), window=None)
    assert by_layers[(3,)] == PagedTensors(tensors=(("keys", (1, 48)), ("values", (1, 40))), window=33)
    states = {(s.layer, s.requirement.name): s.requirement for s in layout.states}
    assert states == {(i, "kept_inputs"): FixedState((2, 48), torch.float32, "kept_inputs") for i in range(4)}
    other = DecoderModel(describe_mabedra(MabedraConfig.from_dict(helpers.MABEDRA_C))).cache_layout()
    assert not other.states and [g.requirement.window for g in other.groups] == [24, 50, None]
    assert isinstance(layout, CacheLayout)


# ------------------------------------------------------------- the plain implementation against closed forms
def test_plain_layer_norm_and_taps():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    out = plain.layer_norm(x, torch.tensor([1.0, 1.0, 2.0, 1.0], dtype=torch.float64), 0.0)
    sd = math.sqrt((4 + 1 + 0 + 9) / 4)
    assert torch.allclose(out[0], torch.tensor([-2 / sd, -1 / sd, 0.0, 3 / sd], dtype=torch.float64))
    h = torch.arange(1.0, 5.0, dtype=torch.float64).view(4, 1)
    assert plain.causal_taps(h, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)).flatten().tolist() == [1.0, 12.0, 123.0, 234.0]
    assert plain.causal_taps(h[:1], torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)).flatten().tolist() == [1.0]


def test_plain_frequencies_and_rotation():
    f = plain.scaled_frequencies(8, 100.0, None, torch.float64)
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=torch.float64))
    s = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 100.0}
    g = plain.scaled_frequencies(8, 100.0, s, torch.float64)
    # wavelengths 6.3, 19.9, 62.8, 198.7 against 25 and 100: two kept, one blended, one divided
    assert g[0] == f[0] and g[1] == f[1] and abs(float(g[3]) - float(f[3]) / 4) < 1e-15
    blend = (100.0 / (2 * math.pi / 0.1) - 1.0) / 3.0
    assert abs(float(g[2]) - ((1 - blend) * 0.1 / 4 + blend * 0.1)) < 1e-15
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0]], dtype=torch.float64)
    out = plain.rotate(x, torch.tensor([3]), torch.tensor([1.0, 0.1], dtype=torch.float64))
    want = [1 * math.cos(3.0) - 3 * math.sin(3.0), 2 * math.cos(0.3) - 4 * math.sin(0.3), 3 * math.cos(3.0) + 1 * math.sin(3.0),
            4 * math.cos(0.3) + 2 * math.sin(0.3), 5.0]
    assert torch.allclose(out[0], torch.tensor(want, dtype=torch.float64))


def test_plain_differential_attention_with_equal_maps():
    """Both maps alike and lambda known: the difference is (1 - lambda) times one map's output, whose unit norm is that
    output's own; with zero queries a map's output is the mean of the values the window lets through."""

    d, dv, T = 2, 2, 5
    W = {"q": torch.zeros(2 * d, 1), "q.b": torch.zeros(2 * d), "k": torch.zeros(2 * d, 1), "k.b": torch.ones(2 * d),
         "v": torch.tensor([[1.0], [2.0]]), "v.b": torch.zeros(dv), "q.norm": torch.ones(d), "k.norm": torch.ones(d),
         "lq1": torch.zeros(d), "lk1": torch.zeros(d), "lq2": torch.tensor([1.0, 0.0]), "lk2": torch.tensor([math.log(0.5), 0.0]),
         "o": torch.eye(dv)}
    W = {k: v.double() for k, v in W.items()}
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "diff": 0.25, "scale": 1.0, "mask": {"size": 2}}
    h = torch.arange(1.0, T + 1, dtype=torch.float64).view(T, 1)
    out = plain.differential_attention(h, W, m, 1e-30)
    lam = 1.0 - 0.5 + 0.25
    means = torch.tensor([1.0, 1.5, 2.5, 3.5, 4.5], dtype=torch.float64)
    o = (1 - lam) * means[:, None] * torch.tensor([1.0, 2.0], dtype=torch.float64)
    want = o / o.pow(2).mean(dim=1, keepdim=True).sqrt() * 0.75
    assert torch.allclose(out, want)


def test_plain_feed_forwards():
    z = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    out = plain.poly_norm(z, torch.tensor([1.0, 10.0, 100.0, 0.5], dtype=torch.float64), 0.0)
    r1, r2, r3 = math.sqrt(2.5), math.sqrt(8.5), math.sqrt(32.5)
    assert torch.allclose(out[0], torch.tensor([1 / r1 + 10 / r2 + 100 / r3 + 0.5, -2 / r1 + 40 / r2 - 800 / r3 + 0.5], dtype=torch.float64))
    # experts: the two largest of three logits are chosen; the score multiplies the input, so a gated unit sees it twice
    W = {"router": torch.tensor([[1.0], [3.0], [2.0]]), "shared.gate": torch.tensor([[1.0]]), "shared.up": torch.tensor([[1.0]]),
         "shared.down": torch.tensor([[10.0]])}
    for e in range(3):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = torch.tensor([[1.0]]), torch.tensor([[float(e + 1)]]), torch.tensor([[1.0]])
    W = {k: v.double() for k, v in W.items()}
    mlp = {"router": {"experts": 3, "top": 2}, "shared": {"ff": 1}}
    margins = []
    out = plain.routed_ff(torch.tensor([[1.0]], dtype=torch.float64), W, mlp, margins=margins)
    silu = lambda v: v / (1 + math.exp(-v))
    s1, s2 = 1 / (1 + math.exp(-3.0)), 1 / (1 + math.exp(-2.0))
    assert abs(float(out) - (silu(s1) * 2 * s1 + silu(s2) * 3 * s2 + silu(1.0) * 10)) < 1e-12
    assert abs(float(margins[0]) - 1.0) < 1e-12
