"""Shared test material: two tiny Qwen3 configurations that differ in every
size and option, model folders with random weights, and trace builders."""

from __future__ import annotations

import json
import random
from pathlib import Path

import torch

from tests.plain import qwen3_plain

# Tiny A: 2 layers, hidden 64, 4 q heads / 2 kv heads, head 16 (q width = hidden),
# tied head, theta 1e4, eps 1e-6, page size 4.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "hidden_act": "silu", "attention_bias": False, "attention_dropout": 0.0,
    "tie_word_embeddings": True, "torch_dtype": "float32", "bos_token_id": 1, "eos_token_id": 2,
}
# Tiny B: 3 layers, hidden 96, 6 q heads / 1 kv head (MQA), head 32 (q width 192 != hidden),
# intermediate 272 and vocab 503 (no powers of two), untied head, theta 1e6, eps 1e-5, page size 8.
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 503, "hidden_size": 96, "intermediate_size": 272, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32,
    "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "hidden_act": "silu", "attention_bias": False, "attention_dropout": 0.0,
    "tie_word_embeddings": False, "torch_dtype": "float32", "bos_token_id": 0, "eos_token_id": [501, 502],
}
# Tiny C: biases on q/k/v, head 48 (a multiple of 16 that is no power of two), 5 q / 5 kv heads.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 131, "hidden_size": 80, "intermediate_size": 112, "num_hidden_layers": 1,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "max_position_embeddings": 384, "rms_norm_eps": 3e-6, "rope_theta": 50000.0,
    "hidden_act": "silu", "attention_bias": True, "attention_dropout": 0.0,
    "tie_word_embeddings": False, "torch_dtype": "float32", "bos_token_id": 0, "eos_token_id": 1,
}
TINY = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16)}  # config, seed, page size


def make_model_dir(path: Path, config: dict, seed: int, *, torch_dtype: str | None = None, shards: int = 1):
    """Write a model folder; return (path, {name: CPU tensor as stored})."""

    from llm_runtime_study_b200.weights import Checkpoint, write_random_model

    cfg = dict(config)
    if torch_dtype is not None:
        cfg["torch_dtype"] = torch_dtype
    write_random_model(path, cfg, seed, shards=shards)
    return path, Checkpoint.from_model_dir(path).get_tensors()


def plain_logits(weights: dict, config: dict, token_ids, dtype=torch.float64, *, rows=None, rounded: bool = False) -> torch.Tensor:
    """``rounded``: the plain model keeps its activations as a bfloat16 engine stores them."""

    store = qwen3_plain.round_bfloat16 if rounded else qwen3_plain._keep
    return qwen3_plain.forward(weights, config, token_ids, dtype=dtype, rows=rows, store=store)


# How far a row of logits may be from the plain model's, as fractions of the row's root mean square:
# (the root mean square of the differences, the largest difference).
# float32: the engine in 32-bit against the plain model in 64-bit (32-bit at real sizes): only the order of
# the sums differs; seen: 6e-6 and 2.7e-5.
# bfloat16: the plain model (64-bit arithmetic) rounds its activations to bfloat16 where the engine
# stores them, so what is left is the order of the sums, the rounding of the attention weights, and
# roundings that fall the other way here and there (one bfloat16 step is 2^-8 of a value).  The root
# mean square over a row is a steady figure (a wrong key, position or page moves it by tens of per
# cent); the largest of up to 151,936 differences is a tail value of the same noise and gets more room.
# Seen over all rows these tests compare, tiny models and real sizes alike: rms up to 1.35e-2 (median
# 0.6e-2 to 0.9e-2), largest up to 6.2e-2; the bounds are one and a half times that.
REPLAY_TOL = {"float32": (2e-5, 1e-4), "bfloat16": (2e-2, 1e-1)}


def plain_for(dtype: str, weights: dict, config: dict, token_ids, **kw) -> torch.Tensor:
    """The plain logits an engine of run type ``dtype`` is compared with."""

    return plain_logits(weights, config, token_ids, rounded=dtype == "bfloat16", **kw)


def first_wrong_row(got: torch.Tensor, want: torch.Tensor, tol: tuple[float, float]):
    """(index of the first row that is too far off, or None; the worst rms error / rms; the worst error / rms).
    A NaN anywhere in a row makes it wrong."""

    rms = want.pow(2).mean(dim=1, keepdim=True).sqrt().clamp_min(1e-30)
    diff = (got - want).abs() / rms
    worst, mean = diff.max(dim=1).values, diff.pow(2).mean(dim=1).sqrt()
    bad = (~((mean <= tol[0]) & (worst <= tol[1]))).nonzero()
    return (int(bad[0]) if bad.numel() else None), float(mean.max()), float(worst.max())


def random_tokens(rng: random.Random, vocab: int, length: int) -> list[int]:
    return [rng.randrange(vocab) for _ in range(length)]


# ----------------------------------------------------------------- traces
def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole: one step holding all its tokens."""

    steps = []
    for step, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [rid]})
    return steps


def trace_decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, its last ``tail`` tokens one by one."""

    steps, step = [], 0
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        step += 1
        for i in range(head, len(tokens)):
            steps.append({"step": step, "entries": [{"id": rid, "tokens": [tokens[i]], "want": [0]}],
                          "end": [rid] if i == len(tokens) - 1 else []})
            step += 1
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def trace_chunked(requests: dict[str, list[int]], rng: random.Random, sizes=(2, 3, 5, 7, 13, 16, 17, 31)) -> list[dict]:
    """Each request in portions of changing size, down to two tokens."""

    steps, step = [], 0
    for rid, tokens in requests.items():
        at = 0
        while at < len(tokens):
            n = min(rng.choice(sizes), len(tokens) - at)
            steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(tokens) else []})
            at += n
            step += 1
    return steps


def trace_mixed(requests: dict[str, list[int]], rng: random.Random, *, live_max: int = 4, tail: int = 8,
                sizes=(2, 3, 5, 8, 13)) -> list[dict]:
    """Up to ``live_max`` live requests; portions of some beside single tokens
    of others; a request may sit a step out.  Requests are admitted as others
    end, so pages are used again."""

    waiting = list(requests.items())
    live: dict[str, int] = {}  # id -> tokens fed so far
    steps, step = [], 0
    while waiting or live:
        while waiting and len(live) < live_max:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        ids = list(live)
        rng.shuffle(ids)
        for rid in ids:
            tokens = requests[rid]
            at = live[rid]
            if len(ids) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            decode_from = max(1, len(tokens) - tail)
            n = 1 if at >= decode_from else min(rng.choice(sizes), decode_from - at)
            entries.append({"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))})
            live[rid] = at + n
            if live[rid] == len(tokens):
                ended.append(rid)
        if not entries:
            continue
        for rid in ended:
            del live[rid]
        steps.append({"step": step, "entries": entries, "end": ended})
        step += 1
    return steps


def collect_logits(steps: list[dict], outputs: dict[int, "torch.Tensor"]) -> dict[str, dict[int, torch.Tensor]]:
    """Key replayed logits by (request, absolute position)."""

    fed: dict[str, int] = {}
    result: dict[str, dict[int, torch.Tensor]] = {}
    for record in steps:
        rows = outputs.get(record["step"])
        r = 0
        for entry in record["entries"]:
            base = fed.get(entry["id"], 0)
            for w in entry["want"]:
                result.setdefault(entry["id"], {})[base + w] = rows[r]
                r += 1
            fed[entry["id"]] = base + len(entry["tokens"])
    return result


def pool_tokens(steps: list[dict]) -> int:
    """Most tokens live requests hold at any time, each rounded up to 64."""

    held: dict[str, int] = {}
    worst = 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-v // 64) * 64 for v in held.values()))
        for rid in record["end"]:
            held.pop(rid, None)
    return worst


def dump_trace(steps: list[dict]) -> str:
    return "".join(json.dumps(s) + "\n" for s in steps)


# ----------------------------------------------------------------- Sorulix
# Two small configurations that differ in every size and option.  A: a loop over layers 1..2 (three passes), a
# layer without a feed-forward, grouped heads in both attention and delta rule, key and value sizes that differ,
# a soft cap and a query temperature that both bite.  B: no loop, no soft cap, no temperature, one head here and
# there, a period-2 convolution, sizes that are no multiples of 16.
SORULIX_A = {
    "architecture": "Sorulix", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "conv": 3},
         "mlp": {"kind": "dense", "ff": 80, "limit": 1.5}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.9, "softcap": 1.0, "q_temp": {"coef": 0.5, "every": 3}},
            "right": {"heads": 2, "dim": 8, "vdim": 40, "decay": [0.9, 0.5]}},
         "mlp": {"kind": "dense", "ff": 80, "limit": 1.5}},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "conv": 3}, "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.5, "softcap": 2.0, "q_temp": {"coef": 0.2, "every": 1}},
            "right": {"heads": 3, "dim": 16, "vdim": 16, "decay": [0.99, 0.7, 0.2]}},
         "mlp": {"kind": "dense", "ff": 48, "limit": 0.7}},
    ],
}
SORULIX_A_RANKS = {0: (5, 7), 2: (8, 3)}
SORULIX_B = {
    "architecture": "Sorulix", "vocab": 131, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "parallel", "mixer": {
            "left": {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 8, "scale": 1.0},
            "right": {"heads": 1, "dim": 40, "vdim": 8, "decay": [0.97]}},
         "mlp": {"kind": "dense", "ff": 56, "limit": 0.7}},
        {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 40, "vdim": 48, "conv": 2},
         "mlp": {"kind": "dense", "ff": 56, "limit": 2.5}},
    ],
}
SORULIX_B_RANKS = {1: (16, 1)}
SORULIX = {"A": (SORULIX_A, SORULIX_A_RANKS, 11, 4), "B": (SORULIX_B, SORULIX_B_RANKS, 12, 16)}   # config, ranks, seed, page size


def make_sorulix_dir(path: Path, config: dict, ranks: dict, seed: int, *, torch_dtype: str = "float32", gain: float = 8.0):
    """Write a Sorulix model folder with random weights; return (path, {name: CPU tensor as stored}).  The matrices
    are drawn ``gain`` times larger than the framework's default so that limits, caps and gates bite."""

    from llm_runtime_study_b200.config import SorulixConfig
    from llm_runtime_study_b200.models.description import tensor_schema
    from llm_runtime_study_b200.models.sorulix import describe_sorulix
    from llm_runtime_study_b200.weights.random_init import random_state
    from llm_runtime_study_b200.weights.safetensors_io import write_file

    schema = tensor_schema(describe_sorulix(SorulixConfig.from_dict(config), ranks))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[torch_dtype]
    state = random_state(schema, seed, dtype=torch.float32, include_optional=False)
    for name, tensor in state.items():
        if tensor.dim() == 2 and not name.endswith(".conv") and name not in ("loop.step",):
            tensor *= gain
    state = {name: tensor.to(dtype) for name, tensor in state.items()}
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config, indent=1), encoding="utf-8")
    write_file(path / "model.safetensors", state)
    return path, state


# ----------------------------------------------------------------- Ropulix
# Two small configurations that differ in every size and option.  A: a latent attention layer whose rows a later layer
# borrows with a wider window, grouped heads sharing one key/value head, key and value sizes that differ and are no
# multiples of 16, a layer without a feed-forward, experts of which one, two or all are used.  B: a recurrence without a
# convolution and with one block, attention with as many key/value heads as query heads, latent attention without a
# window and with a query rank that is no multiple of eight, a period-2 convolution.
ROPULIX_A = {
    "architecture": "Ropulix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "q_rank": 48,
                                               "mask": {"size": 9}, "rot": {"base": 1000.0, "dims": 8}, "scale": 0.35},
         "mlp": {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 5, "top": 2}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 16, "mask": {"size": 5}, "scale": 0.3}, "mlp": None},
        {"type": "rglru", "mixer": {"width": 96, "blocks": 3, "conv": 4},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 3, "top": 3}}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 8, "vdim": 8, "kv_rank": 40, "q_rank": 16, "kv_from": 0,
                                               "mask": {"size": 13}, "rot": {"base": 1000.0, "dims": 8}, "scale": 0.5},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 4, "top": 1}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "scale": 0.2},
         "mlp": {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 5, "top": 2}}},
    ],
}
ROPULIX_B = {
    "architecture": "Ropulix", "vocab": 131, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "rglru", "mixer": {"width": 48, "blocks": 1, "conv": 1},
         "mlp": {"kind": "moe", "expert": {"ff": 56}, "router": {"experts": 2, "top": 1}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 32, "mask": {"size": 33}, "scale": 0.18},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 6, "top": 3}}},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 24, "rot_dim": 16, "vdim": 40, "kv_rank": 24, "q_rank": 12,
                                               "rot": {"base": 10000.0, "dims": 16}, "scale": 0.16}, "mlp": None},
        {"type": "rglru", "mixer": {"width": 80, "blocks": 5, "conv": 2},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 6, "top": 3}}},
    ],
}
# C: sizes in steps of 16 throughout, which is what the tensor-core kernels of the bfloat16 run type take: latent rows of
# 32 + 16 columns shared by two layers with windows of 24 and 50, heads of 32 and 64, experts of 64 hidden units.
ROPULIX_C = {
    "architecture": "Ropulix", "vocab": 151, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "mask": {"size": 20}, "scale": 0.2},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 6, "top": 2}}},
        {"type": "latent_attention", "mixer": {"heads": 5, "dim": 16, "rot_dim": 16, "vdim": 32, "kv_rank": 32, "q_rank": 48,
                                               "mask": {"size": 50}, "rot": {"base": 5000.0, "dims": 16}, "scale": 0.25},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 6, "top": 2}}},
        {"type": "rglru", "mixer": {"width": 128, "blocks": 2, "conv": 3},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 6, "top": 2}}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 64, "rot_dim": 16, "vdim": 16, "kv_rank": 32, "q_rank": 32, "kv_from": 1,
                                               "mask": {"size": 24}, "rot": {"base": 5000.0, "dims": 16}, "scale": 0.12},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 6, "top": 2}}},
    ],
}
# D: no window anywhere (every key since the first token is read, through the kernels that take no mask), heads of 64 with
# grouped key/value heads, a latent whose value size differs from the rows' width by 16, experts in two passes of eight.
ROPULIX_D = {
    "architecture": "Ropulix", "vocab": 173, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 32, "rot_dim": 16, "vdim": 48, "kv_rank": 64, "q_rank": 64,
                                               "rot": {"base": 30000.0, "dims": 16}, "scale": 0.15},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 10, "top": 4}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 10, "top": 4}}},
        {"type": "rglru", "mixer": {"width": 160, "blocks": 5, "conv": 5}, "mlp": None},
    ],
}
ROPULIX = {"A": (ROPULIX_A, 21, 4), "B": (ROPULIX_B, 22, 16), "C": (ROPULIX_C, 23, 16), "D": (ROPULIX_D, 24, 16)}   # config, seed, page size


def make_ropulix_dir(path: Path, config: dict, seed: int, *, torch_dtype: str = "float32", gain: float = 6.0):
    """Write a Ropulix model folder with random weights; return (path, {name: CPU tensor as stored}).  The matrices are
    drawn ``gain`` times larger than the framework's default, so that gates, decays and routers are not all alike."""

    from llm_runtime_study_b200.config import RopulixConfig
    from llm_runtime_study_b200.models.description import tensor_schema
    from llm_runtime_study_b200.models.ropulix import describe_ropulix
    from llm_runtime_study_b200.weights.random_init import random_state
    from llm_runtime_study_b200.weights.safetensors_io import write_file

    schema = tensor_schema(describe_ropulix(RopulixConfig.from_dict(config)))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[torch_dtype]
    state = random_state(schema, seed, dtype=torch.float32, include_optional=False)
    for name, tensor in state.items():
        if tensor.dim() == 2 and not name.endswith((".conv", ".ra.b", ".ri.b", ".router")):
            tensor *= gain
    state = {name: tensor.to(dtype) for name, tensor in state.items()}
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config, indent=1), encoding="utf-8")
    write_file(path / "model.safetensors", state)
    return path, state


# ----------------------------------------------------------------- Mabedra
# A: sizes that are no multiples of 16, grouped heads sharing one key/value head, value sizes larger and smaller than the
# key size, a rotation over part of a map and over all of it, stretched wavelengths of which some are kept, some blended
# and some divided, a layer without a window, one without a rotation, one without a feed-forward, a dense feed-forward,
# experts of which two of five or all three are used, with and without a shared expert, three taps.
MABEDRA_A = {
    "architecture": "Mabedra", "vocab": 157, "width": 48, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
    "layers": [
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 8, "vdim": 12, "diff": 0.2, "scale": 0.4, "mask": {"size": 7},
                                        "rot": {"base": 500.0, "dims": 4, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 32}}},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 8, "diff": 0.35, "scale": 0.25,
                                        "rot": {"base": 100.0, "dims": 16, "scaling": {"factor": 2.0, "low": 1.0, "high": 4.0, "original": 64}}},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 16}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "diff": 0.5, "scale": 0.35, "mask": {"size": 5}},
         "mlp": None},
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 24, "vdim": 40, "diff": 0.1, "scale": 0.2, "mask": {"size": 33},
                                        "rot": {"base": 10000.0, "dims": 24}},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 3}}},
    ],
}
# B: two taps, one expert of six used, as many key/value heads as query heads, a window of one page.
MABEDRA_B = {
    "architecture": "Mabedra", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "canon": {"taps": 2},
    "layers": [
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 16, "diff": 0.25, "scale": 0.18, "mask": {"size": 16},
                                        "rot": {"base": 3000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}}},
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 16, "diff": 0.4, "scale": 0.25, "mask": {"size": 40},
                                        "rot": {"base": 3000.0, "dims": 8}},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 6, "top": 1}, "shared": {"ff": 48}}},
    ],
}
# C: sizes in steps of 16 throughout (what the tensor-core kernels of the bfloat16 run type take), no convolution on the
# sublayers' inputs, windows of 24 and 50 and none, heads of 32 with values of 64 and heads of 64 with values of 32.
MABEDRA_C = {
    "architecture": "Mabedra", "vocab": 151, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 64, "diff": 0.3, "scale": 0.18, "mask": {"size": 24},
                                        "rot": {"base": 5000.0, "dims": 32}},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 32}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 32, "diff": 0.15, "scale": 0.125, "mask": {"size": 50},
                                        "rot": {"base": 5000.0, "dims": 16}},
         "mlp": {"kind": "dense", "ff": 192}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 48, "vdim": 48, "diff": 0.3, "scale": 0.14,
                                        "rot": {"base": 20000.0, "dims": 48, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}}},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 32}}},
    ],
}
MABEDRA = {"A": (MABEDRA_A, 31, 4), "B": (MABEDRA_B, 32, 16), "C": (MABEDRA_C, 33, 16)}   # config, seed, page size


def make_mabedra_dir(path: Path, config: dict, seed: int, *, torch_dtype: str = "float32", gain: float = 6.0):
    """Write a Mabedra model folder with random weights; return (path, {name: CPU tensor as stored}).  The matrices are
    drawn ``gain`` times larger than the framework's default, so that scores and routers are not all alike."""

    from llm_runtime_study_b200.config import MabedraConfig
    from llm_runtime_study_b200.models.description import tensor_schema
    from llm_runtime_study_b200.models.mabedra import describe_mabedra
    from llm_runtime_study_b200.weights.random_init import random_state
    from llm_runtime_study_b200.weights.safetensors_io import write_file

    schema = tensor_schema(describe_mabedra(MabedraConfig.from_dict(config)))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[torch_dtype]
    state = random_state(schema, seed, dtype=torch.float32, include_optional=False)
    for name, tensor in state.items():
        if tensor.dim() == 2 and not name.endswith((".canon1", ".canon2", ".router")):
            tensor *= gain
    state = {name: tensor.to(dtype) for name, tensor in state.items()}
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config, indent=1), encoding="utf-8")
    write_file(path / "model.safetensors", state)
    return path, state


# ----------------------------------------------------------------- Tafisun
# A: sizes that are no multiples of 16, grouped heads sharing one key/value head, a recurrence wider than the model, blocks
# of the mask of 5 and 7 positions beside pages of 4, routers with one and with three groups, with and without outputs that
# return their input, one that uses all of its outputs, a dense feed-forward and a layer without one, a bigram table of 13
# rows (many pairs collide), multipliers that overflow 32 bits with the vocabulary's ids.
TAFISUN_A = {
    "architecture": "Tafisun", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 13, "mul_prev": 40_000_003, "mul_cur": 11}},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 16, "mask": {"size": 5}, "scale": 0.3},
         "mlp": {"kind": "moe", "expert": {"ff": 40, "limit": 1.5},
                 "router": {"experts": 5, "identity": 1, "top": 2, "scale": 2.5, "groups": {"count": 3, "keep": 2}},
                 "shared": {"ff": 24, "limit": 0.75}}},
        {"type": "mingru", "mixer": {"width": 96}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 24, "mask": {"size": 7}, "scale": 0.2},
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "mingru", "mixer": {"width": 40},
         "mlp": {"kind": "moe", "expert": {"ff": 24, "limit": 3.0},
                 "router": {"experts": 3, "identity": 0, "top": 3, "scale": 1.0, "groups": {"count": 1, "keep": 1}},
                 "shared": {"ff": 8, "limit": 2.0}}},
    ],
}
# B: one layer of each kind in the other order, as many key/value heads as query heads, a block of the mask that is no
# power of two and no multiple of the page, more identity outputs than a group holds, a single router output chosen, no
# shared unit.
TAFISUN_B = {
    "architecture": "Tafisun", "vocab": 131, "width": 48, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 257, "mul_prev": 1, "mul_cur": 0}},
    "layers": [
        {"type": "mingru", "mixer": {"width": 48},
         "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 2.0},
                 "router": {"experts": 5, "identity": 3, "top": 1, "scale": 0.7, "groups": {"count": 4, "keep": 1}},
                 "shared": None}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 32, "mask": {"size": 33}, "scale": 0.18},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "mask": {"size": 2}, "scale": 0.5}, "mlp": None},
    ],
}
# C: sizes in steps of 16 throughout, which is what the tensor-core kernels of the bfloat16 run type take: heads of 32 and 64,
# blocks of the mask of one page, of three pages and of 20 positions, experts of 64 hidden units.
TAFISUN_C = {
    "architecture": "Tafisun", "vocab": 151, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 29, "mul_cur": 5}},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "mask": {"size": 16}, "scale": 0.2},
         "mlp": {"kind": "moe", "expert": {"ff": 64, "limit": 2.5},
                 "router": {"experts": 6, "identity": 2, "top": 2, "scale": 1.25, "groups": {"count": 4, "keep": 2}},
                 "shared": {"ff": 64, "limit": 1.5}}},
        {"type": "mingru", "mixer": {"width": 128}, "mlp": {"kind": "dense", "ff": 256}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 64, "vdim": 64, "mask": {"size": 48}, "scale": 0.125},
         "mlp": {"kind": "moe", "expert": {"ff": 64, "limit": 2.5},
                 "router": {"experts": 6, "identity": 2, "top": 2, "scale": 1.25, "groups": {"count": 4, "keep": 2}},
                 "shared": {"ff": 64, "limit": 1.5}}},
        {"type": "attention", "mixer": {"heads": 10, "kv_heads": 1, "dim": 16, "vdim": 16, "mask": {"size": 20}, "scale": 0.25}, "mlp": None},
    ],
}
# D: a block of the mask longer than every sequence (every key since the first token is read: far keys), heads of 64 with
# grouped key/value heads, four of twelve outputs in two passes of eight, a recurrence between them.
TAFISUN_D = {
    "architecture": "Tafisun", "vocab": 173, "width": 128, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 1009, "mul_prev": 5, "mul_cur": 29}},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "mask": {"size": 4096}, "scale": 0.125},
         "mlp": {"kind": "moe", "expert": {"ff": 32, "limit": 2.0},
                 "router": {"experts": 10, "identity": 2, "top": 4, "scale": 1.0, "groups": {"count": 3, "keep": 2}},
                 "shared": {"ff": 32, "limit": 2.0}}},
        {"type": "mingru", "mixer": {"width": 160}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "mask": {"size": 100}, "scale": 0.2},
         "mlp": {"kind": "dense", "ff": 64}},
    ],
}
TAFISUN = {"A": (TAFISUN_A, 41, 4), "B": (TAFISUN_B, 42, 16), "C": (TAFISUN_C, 43, 16), "D": (TAFISUN_D, 44, 16)}   # config, seed, page size


def make_tafisun_dir(path: Path, config: dict, seed: int, *, torch_dtype: str = "float32", gain: float = 6.0):
    """Write a Tafisun model folder with random weights; return (path, {name: CPU tensor as stored}).  The matrices are
    drawn ``gain`` times larger than the framework's default, so that gates and routers are not all alike; the tables of
    the embedding are drawn of the size of the position vector's entries."""

    from llm_runtime_study_b200.config import TafisunConfig
    from llm_runtime_study_b200.models.description import tensor_schema
    from llm_runtime_study_b200.models.tafisun import describe_tafisun
    from llm_runtime_study_b200.weights.random_init import random_state
    from llm_runtime_study_b200.weights.safetensors_io import write_file

    schema = tensor_schema(describe_tafisun(TafisunConfig.from_dict(config)))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[torch_dtype]
    state = random_state(schema, seed, dtype=torch.float32, include_optional=False)
    for name, tensor in state.items():
        if name in ("embed", "bigram"):
            tensor *= 40.0
        elif tensor.dim() == 2 and not name.endswith((".router", ".sg")):
            tensor *= gain
    state = {name: tensor.to(dtype) for name, tensor in state.items()}
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config, indent=1), encoding="utf-8")
    write_file(path / "model.safetensors", state)
    return path, state
