"""Tafisun under random configurations: head sizes on and off the tensor-core kernels' steps, any number of heads and
groups, widths and vocabularies that are no power of two, blocks of the mask from one position to longer than the prompts,
any order of layers, routers of every shape.  Each configuration is replayed whole, in portions and mixed, in both run
types, against the plain implementation."""

import random

import numpy as np
import pytest
import torch

from tests import helpers
from tests.plain import tafisun_plain as plain

pytestmark = pytest.mark.gpu

TOL32 = (3e-5, 2e-4)
BF16_USUAL, BF16_WORST, CLOSE_CALL = 6e-2, 5e-1, 0.02


def _router(rng: random.Random) -> dict:
    groups = rng.choice([1, 1, 2, 3, 4])
    per = rng.choice([1, 2, 3, 5])
    outputs = groups * per
    identity = rng.randrange(0, max(1, outputs // 2))
    keep = rng.randrange(1, groups + 1)
    top = rng.randrange(1, min(keep * per, 4) + 1)
    return {"experts": outputs - identity, "identity": identity, "top": top, "scale": rng.choice([0.5, 1.0, 2.5]),
            "groups": {"count": groups, "keep": keep}}


def _configuration(case: int):
    rng = random.Random(case)
    width = rng.choice([48, 64, 72, 104, 136, 200, 256])
    layers = []
    for _ in range(rng.choice([1, 2, 3, 4])):
        if rng.random() < 0.55:
            kv = rng.choice([1, 2, 3])
            d = rng.choice([8, 16, 24, 32, 40, 48, 64, 64, 96, 128])
            mixer = {"heads": kv * rng.choice([1, 2, 3, 5]), "kv_heads": kv, "dim": d, "vdim": d, "scale": rng.choice([0.1, 0.2, d ** -0.5]),
                     "mask": {"size": rng.choice([1, 3, 16, 17, 64, 100, 128, 1000])}}
            kind = "attention"
        else:
            mixer = {"width": rng.choice([width, 40, 88, 130])}
            kind = "mingru"
        pick = rng.random()
        if pick < 0.2:
            mlp = None
        elif pick < 0.45:
            mlp = {"kind": "dense", "ff": rng.choice([56, 96, 130, 272])}
        else:
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([16, 24, 64, 72]), "limit": rng.choice([0.5, 2.0, 7.0])}, "router": _router(rng),
                   "shared": {"ff": rng.choice([8, 64, 80]), "limit": rng.choice([1.0, 3.0])}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    raw = {"architecture": "Tafisun", "vocab": rng.choice([97, 256, 503, 1000, 2049]), "width": width,
           "norm": {"eps": rng.choice([1e-6, 1e-5, 3e-6])},
           "embedding": {"bigram": {"buckets": rng.choice([1, 37, 1013, 65521]), "mul_prev": rng.choice([0, 1, 29, 1_000_003]),
                                    "mul_cur": rng.choice([0, 1, 5, 999_983])}},
           "layers": layers}
    lengths = [rng.choice([1, 2, 5, 33, 64, 65, 130, 200, 300]) for _ in range(5)]
    return raw, lengths, rng


# Sizes that no kernel's vector width divides: a width of 100 and of 63, heads of 20 and of 7 columns, hidden sizes of 9, 31 and
# 50, a recurrence of 33 channels, 48 router outputs in six groups of which six are used, a layer without a mask.
ODD = {
    "width-100": ({"architecture": "Tafisun", "vocab": 333, "width": 100, "norm": {"eps": 1e-5},
                   "embedding": {"bigram": {"buckets": 50, "mul_prev": 3, "mul_cur": 2}},
                   "layers": [
                       {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 20, "vdim": 20, "mask": {"size": 10}, "scale": 0.2},
                        "mlp": {"kind": "moe", "expert": {"ff": 20, "limit": 2.0},
                                "router": {"experts": 3, "identity": 1, "top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}},
                                "shared": {"ff": 36, "limit": 1.0}}},
                       {"type": "mingru", "mixer": {"width": 50}, "mlp": {"kind": "dense", "ff": 50}},
                       {"type": "attention", "mixer": {"heads": 2, "dim": 16, "vdim": 16, "scale": 0.25}, "mlp": None}]},
                  [1, 2, 33, 130, 65]),
    "width-63": ({"architecture": "Tafisun", "vocab": 97, "width": 63, "norm": {"eps": 1e-6},
                  "embedding": {"bigram": {"buckets": 5, "mul_prev": 1, "mul_cur": 1}},
                  "layers": [
                      {"type": "mingru", "mixer": {"width": 33},
                       "mlp": {"kind": "moe", "expert": {"ff": 9, "limit": 2.0},
                               "router": {"experts": 40, "identity": 8, "top": 6, "scale": 3, "groups": {"count": 6, "keep": 2}},
                               "shared": {"ff": 7, "limit": 1}}},
                      {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 7, "vdim": 7, "mask": {"size": 300}, "scale": 1},
                       "mlp": {"kind": "dense", "ff": 31}}]},
                 [5, 64, 200, 1, 17]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, "width-100", "width-63"])
def test_random_configuration(case, dtype, tmp_path):
    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.engine.runtime import load

    if isinstance(case, str):
        (raw, lengths), rng, case = ODD[case], random.Random(len(case)), len(case)
    else:
        raw, lengths, rng = _configuration(case)
    path, weights = helpers.make_tafisun_dir(tmp_path / "model", raw, case, torch_dtype=dtype)
    requests = {f"r{i}": helpers.random_tokens(rng, raw["vocab"], n) for i, n in enumerate(lengths)}
    store = plain.round_bfloat16 if dtype == "bfloat16" else plain.keep
    expected, clear = {}, {}
    for rid, tokens in requests.items():
        margins = []
        expected[rid] = plain.forward(weights, raw, tokens, store=store, margins=margins)
        clear[rid] = torch.stack(margins).min(dim=0).values > CLOSE_CALL if margins else torch.ones(len(tokens), dtype=torch.bool)
    loaded = load(path, device="cuda:0", dtype=dtype, strict_dtype=False)
    traces = {
        "whole": helpers.trace_whole(requests),
        "mixed": helpers.trace_mixed(requests, random.Random(case), sizes=(2, 3, 8, 40, 130, 260)),
        "portions": helpers.trace_chunked(requests, random.Random(case), sizes=(2, 17, 64, 128, 129, 250)),
    }
    for kind, steps in traces.items():
        replayer = TraceReplayer(loaded, max_tokens=helpers.pool_tokens(steps), max_requests=4)
        outputs = {}
        for record in steps:
            rows = replayer.run_step(record)
            if rows is not None:
                outputs[record["step"]] = torch.from_numpy(np.array(rows))
        replayer.runner.manager.check()
        got = helpers.collect_logits(steps, outputs)
        for rid, tokens in requests.items():
            rows = torch.stack([got[rid][p] for p in range(len(tokens))]).double()
            want = expected[rid]
            if dtype == "float32":
                bad, err, top = helpers.first_wrong_row(rows, want, TOL32)
                assert bad is None, f"{kind}, request {rid}: first wrong position {bad} of {len(tokens)}, {err:.3e}, {top:.3e}; configuration {raw}"
                continue
            err = (rows - want).pow(2).mean(dim=1).sqrt() / want.pow(2).mean(dim=1).sqrt()
            assert torch.isfinite(err).all(), (kind, rid, raw)
            err = torch.where(clear[rid], err, torch.zeros_like(err))
            assert float(err.max()) <= BF16_WORST, (kind, rid, int(err.argmax()), float(err.max()), raw)
            assert int((err > BF16_USUAL).sum()) <= max(1, len(tokens) // 10), (kind, rid, err, raw)
