"""Tafisun without a GPU: configuration, description, tensor names, cache layout, and the plain implementation's own
mechanisms against closed forms."""

import copy
import math

import pytest
import torch

from llm_runtime_study_b200.cache.manager import CacheLayout
from llm_runtime_study_b200.config import TafisunConfig, architecture_for
from llm_runtime_study_b200.errors import ConfigError
from llm_runtime_study_b200.models.description import tensor_schema
from llm_runtime_study_b200.models.model import DecoderModel
from llm_runtime_study_b200.models.tafisun import describe_tafisun
from llm_runtime_study_b200.parts import FixedState, PagedTensors
from tests import helpers
from tests.plain import tafisun_plain as plain


def test_the_registry_finds_the_design_by_its_architecture_key():
    assert architecture_for(helpers.TAFISUN_A).name == "Tafisun"


def test_every_size_and_constant_is_read_from_the_dict():
    cfg = TafisunConfig.from_dict(helpers.TAFISUN_A)
    assert (cfg.vocab, cfg.width, cfg.eps, len(cfg.layers)) == (211, 64, 1e-5, 4)
    assert (cfg.bigram.buckets, cfg.bigram.mul_prev, cfg.bigram.mul_cur) == (13, 40_000_003, 11)
    attention, recurrence, second, last = (layer.mixer for layer in cfg.layers)
    assert (attention.heads, attention.kv_heads, attention.dim, attention.vdim, attention.chunk, attention.scale) == (4, 1, 16, 16, 5, 0.3)
    assert recurrence.width == 96 and last.width == 40 and second.chunk == 7
    moe = cfg.layers[0].mlp
    assert (moe.experts, moe.identity, moe.top, moe.groups, moe.keep, moe.scale, moe.ff, moe.limit) == (5, 1, 2, 3, 2, 2.5, 40, 1.5)
    assert (moe.shared.ff, moe.shared.limit) == (24, 0.75)
    assert cfg.layers[1].mlp is None and cfg.layers[2].mlp.ff == 72


@pytest.mark.parametrize("patch,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.__setitem__("width", True), "width must be int, got bool"),
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "not a layer of this design"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("vdim", 8), "values are the projected keys"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "not a feed-forward of this design"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "exceeds"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("keep", 4), "keep"),
    (lambda c: c["layers"][0]["mlp"]["expert"].__setitem__("limit", 0), "limit"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("width", 0), "width"),
    (lambda c: c["embedding"]["bigram"].__setitem__("buckets", 0), "buckets"),
    (lambda c: c.__setitem__("layers", []), "layers must not be empty"),
])
def test_a_bad_config_is_refused_with_the_key_named(patch, match):
    raw = copy.deepcopy(helpers.TAFISUN_A)
    patch(raw)
    with pytest.raises(ConfigError, match=match):
        TafisunConfig.from_dict(raw)


def test_tensor_names_and_shapes_follow_the_description():
    schema = tensor_schema(describe_tafisun(TafisunConfig.from_dict(helpers.TAFISUN_A)))
    assert schema["embed"].shape == (211, 64) and schema["bigram"].shape == (14, 64) and schema["head"].shape == (211, 64)
    assert schema["final.norm"].shape == (64,) and "l1.norm2" not in schema and schema["l2.norm2"].shape == (64,)
    assert schema["l0.mix.q"].shape == (64, 64) and schema["l0.mix.k"].shape == (16, 64) and "l0.mix.v" not in schema
    assert schema["l0.mix.q.norm"].shape == (16,) and schema["l0.mix.r1"].shape == (4,) and schema["l0.mix.g"].shape == (64, 64)
    assert schema["l1.mix.z"].shape == (96, 64) and schema["l1.mix.x.b"].shape == (96,) and schema["l1.mix.o"].shape == (64, 96)
    assert "l1.mix.g.b" not in schema
    assert schema["l0.mlp.router"].shape == (6, 64) and schema["l0.mlp.correction"].shape == (6,)
    assert "l0.mlp.e5.up" not in schema and schema["l0.mlp.e4.gate"].shape == (40, 64) and schema["l0.mlp.e4.down"].shape == (64, 40)
    assert schema["l0.mlp.shared.sg"].shape == (1, 64) and schema["l0.mlp.shared.up"].shape == (24, 64)
    assert schema["l2.mlp.up"].shape == (72, 64) and schema["l2.mlp.down"].shape == (64, 72)


def test_the_cache_layout_comes_from_the_mixers_and_the_embedding():
    model = DecoderModel(describe_tafisun(TafisunConfig.from_dict(helpers.TAFISUN_A)))
    layout = model.cache_layout()
    assert isinstance(layout, CacheLayout)
    needs = {group.requirement: group.layers for group in layout.groups}
    assert all(isinstance(need, PagedTensors) for need in needs)
    assert sorted((need.window, layers) for need, layers in needs.items()) == [(5, (0,)), (7, (2,))]
    states = {(s.layer, s.requirement.name): s.requirement for s in layout.states}
    assert states[(1, "state")] == FixedState((96,), torch.float32, "state") and states[(3, "state")].shape == (40,)
    # the embedding keeps the token before a step's first one: an int32 a request, behind the last layer's entries
    assert states[(4, "previous_token")] == FixedState((1,), torch.int32, "previous_token")


def test_the_plain_hash_mask_bias_and_candidate():
    assert plain.bigram_rows([3, 5, 5], buckets=7, mul_prev=2, mul_cur=3) == [7, (6 + 15) % 7, (10 + 15) % 7]
    pos = plain.sinusoid(3, 6, torch.float64)
    assert pos[0].tolist() == [0, 1, 0, 1, 0, 1]
    assert abs(float(pos[2, 2]) - math.sin(2 * 10000 ** (-2 / 6))) < 1e-12 and abs(float(pos[2, 5]) - math.cos(2 * 10000 ** (-4 / 6))) < 1e-12
    seen = plain.chunk_mask(7, 3)
    assert seen[2].tolist() == [True, True, True, False, False, False, False]
    assert seen[3].tolist() == [False, False, False, True, False, False, False]
    assert seen[6].tolist() == [False] * 6 + [True]
    bias = plain.distance_bias(4, 2.0, 0.5, torch.float64)
    assert abs(float(bias[3, 1]) - 2.0 * math.log(2.0)) < 1e-12 and float(bias[2, 2]) == 0.0
    c = plain.mingru_candidate(torch.tensor([-2.0, 0.0, 1.5], dtype=torch.float64))
    assert abs(float(c[0]) - 1 / (1 + math.exp(2.0))) < 1e-12 and c[1:].tolist() == [0.5, 2.0]
    z = torch.tensor([[1.0], [0.25], [0.0]], dtype=torch.float64)
    S = plain.mingru_scan(z, torch.tensor([[4.0], [8.0], [100.0]], dtype=torch.float64))
    assert S[:, 0].tolist() == [4.0, 5.0, 5.0]


def test_the_plain_router_groups_correction_and_identity():
    """Six outputs in three groups of which two are kept: the correction moves the choice but not the weights; an output of a
    dropped group is never chosen however large; the identity output returns its input times its weight."""

    r = {"experts": 5, "identity": 1, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    router = torch.zeros(6, 4, dtype=torch.float64)
    h = torch.tensor([[1.0, 0.0, 0.0, 0.0]], dtype=torch.float64)
    router[:, 0] = torch.tensor([0.0, 3.0, 0.5, 0.0, 2.0, 2.5])
    s = torch.softmax(router[:, 0], dim=0)
    ids, w = plain.route(h, router, torch.zeros(6), r, torch.float64)
    assert sorted(ids[0].tolist()) == [1, 5] and abs(float(w.sum()) - 2.0 * float(s[1] + s[5])) < 1e-12
    # a correction lifts output 2 over output 5's group: groups {0,1} and {2,3} are kept, the choice is 1 and 2, weights without it
    correction = torch.tensor([0.0, 0.0, 1.0, 0.0, 0.0, 0.0], dtype=torch.float64)
    ids, w = plain.route(h, router, correction, r, torch.float64)
    assert sorted(ids[0].tolist()) == [1, 2]
    assert abs(float(w[0, ids[0].tolist().index(2)]) - 2.0 * float(s[2])) < 1e-12
    # negative choice scores everywhere: a dropped group counts as minus infinity, not as zero
    ids, _ = plain.route(h, router, torch.tensor([-5.0, -5.0, -5.0, -5.0, -9.0, -9.0], dtype=torch.float64), r, torch.float64)
    assert all(i < 4 for i in ids[0].tolist())
    mlp = {"expert": {"ff": 2, "limit": 1.0}, "router": {**r, "top": 1, "groups": {"count": 1, "keep": 1}}}
    w_id = {"router": router.clone(), "correction": torch.tensor([0.0, 0, 0, 0, 0, 9.0], dtype=torch.float64)}
    out = plain.moe_ff(h, w_id, mlp, torch.float64, plain.keep)
    assert torch.allclose(out, 2.0 * s[5] * h)
