"""Decode and prefill throughput of the engine at Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line: ``value`` is decoded tokens per second at batch 8 with 2,048
cached tokens per request (device time, CUDA events around K decode steps as
generation runs them: slot records in, drawn tokens out, ids copied to the host);
``e2e`` is the same through the scheduler the Python entry point uses, host token
ids in and out, by the wall clock (batch 1 and 64 under its ``points``); ``prefill`` is one
2,048-token prompt; ``points`` holds decode at batch 1 and 64; ``roofline`` is the
bytes a decode step must read (every weight once plus the live requests' cache)
over its time.  Weights are random (N(0, 0.02); norms 1 + N(0, 0.05)) and token
ids uniform random: there is no network for checkpoints or datasets.  Every
decode step reads far more than the 126 MB L2 holds (16 GB of weights), so no
separate L2 flush is needed between timed iterations.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 4096,
    "intermediate_size": 12288, "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "hidden_act": "silu", "attention_bias": False, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    "bos_token_id": 151643, "eos_token_id": 151645,
}
CONTEXT = 2048          # cached tokens per request when decoding
PREFILL_TOKENS = 2048
PAGE_SIZE = 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.lines: list[str] = []
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None

    def _read(self) -> None:
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def stop(self, start: int = 0) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        rows = [l.split(", ") for l in self.lines[start:] if l.count(",") >= 7] or [l.split(", ") for l in self.lines if l.count(",") >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[4:8]) if v.strip().lower() == "active"})
        mhz = [float(r[0]) for r in rows]
        return {"sm_mhz": statistics.median(mhz), "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "power_w": statistics.median(float(r[2]) for r in rows), "samples": len(rows)}


def model_bytes(cfg: dict, layers: int) -> int:
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * h + h * q + 3 * h * i + 2 * h + 2 * cfg["head_dim"]
    # a decode step reads every layer, the final norm, the head, and one embedding row per token
    return 2 * (layers * per_layer + h + v * h)


def kv_bytes_per_token(cfg: dict, layers: int) -> int:
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg: dict, layers: int, tokens: int) -> float:
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    gemm = 2.0 * tokens * layers * ((q + 2 * kv) * h + h * q + 3 * h * i)
    attention = 4.0 * layers * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    return gemm + attention + 2.0 * v * h


def run_ours(args) -> dict:
    import torch

    from llm_runtime_study_b200.cache.slots import SlotRecord
    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.engine.step import StepEntry
    from llm_runtime_study_b200.ops import native

    cfg = dict(QWEN3_8B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    torch.cuda.set_device(0)
    generator = torch.Generator().manual_seed(0)

    def ids(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=generator).tolist()

    max_batch = max(args.batch, 64)
    context = CONTEXT
    if args.only == "decode" and args.context:     # profiling aid: another context length, its own pool size
        context, max_batch = args.context, args.batch
        cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], context + 1024)
    engine = Engine.from_random_weights(
        cfg, seed=0, device="cuda:0", dtype="bfloat16", max_seq_len=cfg["max_position_embeddings"],
        max_batch_size=max_batch, page_size=PAGE_SIZE,
        max_cache_tokens=max_batch * (context + args.steps + max_batch + max(args.warmup, 3) + 2 * PAGE_SIZE),
        max_tokens_per_step=PREFILL_TOKENS, use_cuda_graph=True)
    runner, manager = engine.runner, engine.cache_manager
    sampler = engine._sampler
    greedy = SlotRecord(position=0)          # temperature 0: the largest logit

    def timed(fn, repeat):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeat):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / repeat

    # ------------------------------------------------------------- prefill
    def one_prefill():
        request = manager.admit()
        handle = runner.step_sampled([StepEntry(request, prompt, [PREFILL_TOKENS - 1], greedy)], sampler)
        handle.tokens()
        manager.release(request)

    prompt = ids(PREFILL_TOKENS)
    if args.only == "prefill":  # profiling aid: nothing but prefills of one prompt
        for _ in range(max(args.warmup, 1)):
            one_prefill()
        return {"only": "prefill", "layers": layers, "ms": round(timed(one_prefill, args.steps), 3)}
    prefill_ms = 0.0
    if args.only != "decode":
        for _ in range(max(args.warmup, 3)):
            one_prefill()
        prefill_ms = statistics.median(timed(one_prefill, 1) for _ in range(5))

    # -------------------------------------------------------------- decode
    def decode_point(batch, steps, warmup, sample_clocks=False):
        """The decode step as generation runs it: slot records in, drawn tokens out, replayed from
        a CUDA graph, the drawn ids copied to pinned host memory after every step."""

        requests = [manager.admit() for _ in range(batch)]
        for request in requests:
            for at in range(0, context, PREFILL_TOKENS):
                n = min(PREFILL_TOKENS, context - at)
                last = at + n == context
                runner.step_sampled([StepEntry(request, ids(n), [n - 1] if last else [], greedy if last else None)], sampler)
        handles = []

        def one_step():
            handles.append(runner.decode_sampled(requests, sampler))

        for _ in range(max(warmup, 3)):
            one_step()
        handles.pop().tokens()
        handles.clear()
        clocks = ClockSampler() if sample_clocks else None
        mark = clocks.mark() if clocks else 0
        before = native.launch_count()
        ms = timed(one_step, steps)
        launches = native.launch_count() - before
        info = clocks.stop(mark) if clocks else None
        handles[-1].tokens()
        for request in requests:
            manager.release(request)
        return ms, launches, info

    if args.only == "decode":   # profiling aid: nothing but the decode steps of one batch size
        ms, launches, _ = decode_point(args.batch, args.steps, args.warmup)
        return {"only": "decode", "layers": layers, "batch": args.batch, "context": context, "ms_per_step": round(ms, 4),
                "gpu_launches": launches}
    ms_b8, launches, clocks = decode_point(args.batch, args.steps, args.warmup, sample_clocks=True)
    ms_b1, _, _ = decode_point(1, args.steps, args.warmup)
    ms_b64, _, _ = decode_point(64, args.steps, args.warmup)

    # ------------------------------------- end to end through the scheduler
    def end_to_end(batch):
        """Tokens per second by the wall clock through the scheduler that ``Engine.generate`` drives:
        requests in as host token ids, events with token ids out.  Every step copies its slots and block
        tables from pinned host memory to the device and the drawn ids back into pinned host memory."""

        engine.max_batch_size = batch
        scheduler = engine.create_scheduler()
        for _ in range(batch):
            scheduler.add_request(ids(CONTEXT), max_new_tokens=1024)
        while scheduler.num_waiting or any(r.prefilling for r in scheduler._running):
            scheduler.step()
        for _ in range(max(args.warmup, 3)):
            scheduler.step()
        graph = runner._graphs.graph_for(batch) if runner._graphs else None
        if graph is not None:
            graph.always_send = True          # copy the step's inputs every step, changed or not
        gc.collect()                          # a collection of the host's garbage inside a 60 ms region is milliseconds of noise
        gc.disable()
        try:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            produced = 0
            for _ in range(args.steps):
                produced += len(scheduler.step())
            torch.cuda.synchronize()
            seconds = time.perf_counter() - t0
        finally:
            gc.enable()
        scheduler.abort_all()
        torch.cuda.synchronize()
        return produced / seconds, (graph.sent * 4 if graph else 0), batch * 4

    e2e_b8, h2d, d2h = end_to_end(args.batch)
    e2e_b1, _, _ = end_to_end(1)
    e2e_b64, _, _ = end_to_end(64)

    pk = peaks()
    step_bytes = model_bytes(cfg, layers) + args.batch * CONTEXT * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (ms_b8 * 1e-3) / 1e9
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    value = args.batch / (ms_b8 * 1e-3)
    return {
        "metric": "decode tok/s at batch 8 (2,048 cached tokens each), Qwen3-8B shape",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_b8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids", "impl": "ours",
        "config": {
            "model": "Qwen3-8B shape", "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
            "seq_len": CONTEXT, "context_limit": cfg["max_position_embeddings"], "page_size": PAGE_SIZE,
            "parallelism": "none (1 GPU)", "cuda_graph": True, "sampling": "greedy, inside the captured step",
            "l2": "inputs larger than L2 (16 GB of weights per step)", "peaks": pk["source"],
        },
        "e2e": {"value": round(e2e_b8, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "points": {"decode_b1": round(e2e_b1, 1), "decode_b64": round(e2e_b64, 1)}},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(1 / (ms_b1 * 1e-3), 1), "decode_b64": round(64 / (ms_b64 * 1e-3), 1)},
        "clocks": clocks,
    }


class _IdsTokenizer:
    """Stands in for the tokenizer files, which cannot be had offline: a prompt's
    "text" is its token ids separated by spaces.  It implements the reference's
    ``RuntimeTokenizer`` protocol (mini_llm/tokenizer.py:27-41) and is the only
    object on the reference arm that is not the reference's own."""

    def encode(self, text):
        return [int(t) for t in text.split()]

    def decode(self, token_ids, *, skip_special_tokens=False):
        return " ".join(str(t) for t in token_ids)

    def format_chat(self, messages, *, enable_thinking=False):
        return messages[-1].content


QWEN3_14B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 17408, "num_hidden_layers": 40,
             "num_attention_heads": 40, "num_key_value_heads": 8, "max_position_embeddings": 8192}
QWEN3_32B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 25600, "num_hidden_layers": 64,
             "num_attention_heads": 64, "num_key_value_heads": 8, "max_position_embeddings": 4096}


def _reference_model(cfg: dict):
    """The reference's own Qwen3ForCausalLM with random weights on the GPU (N(0, 0.02); norms 1 + N(0, 0.05))."""

    import torch

    from mini_llm.config import Qwen3Config
    from mini_llm.model.qwen import Qwen3ForCausalLM

    config = Qwen3Config.from_dict({**cfg, "attention_dropout": 0.0})
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    with torch.device("meta"):
        model = Qwen3ForCausalLM(config)
    model.to_empty(device=device)
    generator = torch.Generator(device=device).manual_seed(0)
    with torch.no_grad():
        for name, parameter in model.named_parameters():
            values = torch.empty(parameter.shape, dtype=torch.float32, device=device)
            if name.endswith("norm.weight") or "layernorm" in name:
                values.normal_(1.0, 0.05, generator=generator)
            else:
                values.normal_(0.0, 0.02, generator=generator)
            parameter.data = values.to(torch.bfloat16)
            del values
    model.materialize_derived_buffers(device)
    model.eval().requires_grad_(False)
    return model, device


class _Arm:
    """One implementation behind the two larger workloads: how to open an engine for a configuration, how to
    hand its scheduler a prompt of token ids, and how many tokens its cache holds at the moment.  Everything
    else (arrival times, prompts, what is timed) is the same code for both arms."""

    def __init__(self, impl: str, cfg: dict, *, max_seq_len: int, max_batch: int, pool_tokens: int, budget: int) -> None:
        import torch

        self.impl, self.cfg = impl, cfg
        if impl == "ours":
            from llm_runtime_study_b200.engine.engine import Engine

            self.engine = Engine.from_random_weights(
                cfg, seed=0, device="cuda:0", dtype="bfloat16", max_seq_len=max_seq_len, max_batch_size=max_batch,
                page_size=PAGE_SIZE, max_cache_tokens=pool_tokens, max_tokens_per_step=budget, use_cuda_graph=True)
        else:
            sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
            from mini_llm.engine import Engine

            model, device = _reference_model(cfg)
            # the reference sizes its pool itself: max_seq_len x max_batch_size tokens (mini_llm/engine.py:273-282)
            self.engine = Engine(model=model, tokenizer=_IdsTokenizer(), device=device, dtype=torch.bfloat16,
                                 max_seq_len=max_seq_len, load_seconds=0.0, max_batch_size=max_batch)
        self.torch = torch

    def scheduler(self):
        return self.engine.create_scheduler()

    def add(self, scheduler, token_ids, new_tokens: int) -> int:
        if self.impl == "ours":
            return scheduler.add_request(token_ids, max_new_tokens=new_tokens)
        from mini_llm.tokenizer import ChatMessage

        return scheduler.add_request([ChatMessage(role="user", content=" ".join(map(str, token_ids)))], max_new_tokens=new_tokens)

    def cached_tokens(self) -> int:
        manager = self.engine.cache_manager
        return int(manager.used_tokens) if manager is not None else 0

    def prefilling(self, scheduler) -> bool:
        if self.impl == "ours":
            return bool(scheduler.num_waiting or any(r.prefilling for r in scheduler._running))
        return bool(scheduler.num_waiting)

    def synchronize(self) -> None:
        self.torch.cuda.synchronize()

    def warm(self, prompt, sizes: int) -> None:
        """Requests that end one after the other, so that every batch size up to ``sizes`` has run once
        (kernels built and loaded, every decode graph captured)."""

        scheduler = self.scheduler()
        for i in range(sizes):
            self.add(scheduler, prompt, 3 + i)
        while scheduler.has_unfinished:
            scheduler.step()
        self.synchronize()


def _unavailable(reason: str) -> dict:
    return {"impl": "reference", "unavailable": reason}


def run_staggered_14b(args) -> dict:
    """Qwen3-14B shape: 32 requests arriving 50 ms apart, prompt lengths uniform in [128, 4096], 256 new
    tokens each, continuous batching of at most 16 (the reference's staggered benchmark,
    benchmarks/staggered.py:99-130 and doc/batch.md:45-53, at this model size).  Wall-clock figures through
    each implementation's own scheduler; the reference prefills whole prompts, which is its stock path."""

    import random

    import torch

    cfg = dict(QWEN3_14B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "mini_llm")):
        return _unavailable("the reference is not installed under baseline/_ref")
    torch.cuda.set_device(0)
    rng = random.Random(0)
    generator = torch.Generator().manual_seed(0)
    requests, new_tokens, interval, max_batch = 32, 256, 0.050, 16
    prompts = [torch.randint(0, cfg["vocab_size"], (rng.randint(128, 4096),), generator=generator).tolist()
               for _ in range(requests)]
    try:
        arm = _Arm(args.impl, cfg, max_seq_len=8192, max_batch=max_batch, pool_tokens=max_batch * (4096 + new_tokens + PAGE_SIZE),
                   budget=4096)
        arm.warm(prompts[0][:128], max_batch)
        scheduler = arm.scheduler()
        clocks = ClockSampler()
        arm.synchronize()
        start = time.perf_counter()
        arrival, first, done, index_of = {}, {}, {}, {}
        submitted = produced = steps = 0
        bytes_read = 0.0
        weights, per_token = model_bytes(cfg, layers), kv_bytes_per_token(cfg, layers)
        while submitted < requests or scheduler.has_unfinished:
            now = time.perf_counter() - start
            while submitted < requests and now >= submitted * interval:
                index_of[arm.add(scheduler, prompts[submitted], new_tokens)] = submitted
                arrival[submitted] = submitted * interval
                submitted += 1
            if not scheduler.has_unfinished:
                time.sleep(max(0.0, submitted * interval - now))
                continue
            bytes_read += weights + arm.cached_tokens() * per_token      # what this step has to read at least
            steps += 1
            for index, event in scheduler.step():
                stamp = time.perf_counter() - start
                r = index_of[index]
                first.setdefault(r, stamp)
                produced += event.token_id is not None
                if event.finish_reason is not None:
                    done[r] = stamp
        arm.synchronize()
        makespan = time.perf_counter() - start
        clock_info = clocks.stop()
    except Exception as exc:
        if args.impl == "reference":
            return _unavailable(f"{type(exc).__name__}: {exc}".splitlines()[0][:300])
        raise

    def pct(values, q):
        values = sorted(values)
        return values[min(len(values) - 1, int(round(q * (len(values) - 1))))]

    pk = peaks()
    ttft = [first[r] - arrival[r] for r in range(requests)]
    latency = [done[r] - arrival[r] for r in range(requests)]
    achieved = bytes_read / makespan / 1e9
    config = {"model": "Qwen3-14B shape", "layers": layers, "layers_full": 40, "requests": requests,
              "prompt_tokens": "uniform 128..4096", "new_tokens": new_tokens, "arrival_interval_ms": 50,
              "max_batch_size": max_batch, "page_size": PAGE_SIZE, "steps": steps, "peaks": pk["source"]}
    if args.impl == "ours":
        config.update({"max_tokens_per_step": 4096, "preemptions": scheduler.stats["preemptions"]})
    return {
        "metric": "staggered arrivals, continuous batching: output tok/s (Qwen3-14B shape)", "impl": args.impl,
        "value": round(produced / makespan, 1), "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids", "makespan_s": round(makespan, 3),
        "ttft_ms": {"p50": round(pct(ttft, 0.5) * 1e3, 1), "p95": round(pct(ttft, 0.95) * 1e3, 1)},
        "latency_ms": {"p50": round(pct(latency, 0.5) * 1e3, 1), "p95": round(pct(latency, 0.95) * 1e3, 1)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4),
                     "note": "every step's weights plus the cache live at that step, over the makespan (prompt steps are compute-bound)"},
        "clocks": clock_info, "config": config,
    }


def run_decode_32b(args) -> dict:
    """Qwen3-32B shape: decode at batch 1 and 16 after 1,024-token prompts, 128 new tokens, CUDA-graph decode
    step, through each implementation's own scheduler by the wall clock."""

    import torch

    cfg = dict(QWEN3_32B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "mini_llm")):
        return _unavailable("the reference is not installed under baseline/_ref")
    torch.cuda.set_device(0)
    generator = torch.Generator().manual_seed(0)
    pk = peaks()
    out = {}
    try:
        arm = _Arm(args.impl, cfg, max_seq_len=4096, max_batch=16, pool_tokens=16 * (1024 + 128 + 64), budget=2048)
        clocks = ClockSampler()
        for batch in (1, 16):
            scheduler = arm.scheduler()
            for _ in range(batch):
                arm.add(scheduler, torch.randint(0, cfg["vocab_size"], (1024,), generator=generator).tolist(), 129)
            while arm.prefilling(scheduler):
                scheduler.step()
            for _ in range(8):
                scheduler.step()
            arm.synchronize()
            started = time.perf_counter()
            produced, steps = 0, 0
            while scheduler.has_unfinished and steps < 100:
                produced += len(scheduler.step())
                steps += 1
            arm.synchronize()
            seconds = time.perf_counter() - started
            scheduler.abort_all()
            step_bytes = model_bytes(cfg, layers) + batch * 1088 * kv_bytes_per_token(cfg, layers)
            achieved = step_bytes / (seconds / steps) / 1e9
            out[f"decode_b{batch}"] = {"tokens_per_s": round(produced / seconds, 1), "ms_per_step": round(seconds / steps * 1e3, 3),
                                       "hbm_gbs": round(achieved, 1), "hbm_frac": round(achieved / pk["hbm_gbs"], 4)}
        clock_info = clocks.stop()
    except Exception as exc:
        if args.impl == "reference":
            return _unavailable(f"{type(exc).__name__}: {exc}".splitlines()[0][:300])
        raise
    return {"metric": "decode tok/s at batch 1 and 16 (Qwen3-32B shape, 1,024-token prompts, CUDA-graph decode)", "impl": args.impl,
            "value": out["decode_b16"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic: random weights, uniform random token ids", "points": out,
            "roofline": {"bound": "hbm", "achieved": out["decode_b16"]["hbm_gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": out["decode_b16"]["hbm_frac"]},
            "clocks": clock_info,
            "config": {"model": "Qwen3-32B shape", "layers": layers, "layers_full": 64, "prompt_tokens": 1024, "new_tokens": 128,
                       "page_size": PAGE_SIZE, "timing": "wall clock through the scheduler", "peaks": pk["source"]}}


# ------------------------------------------------------------------------------ Sorulix beside Qwen3
SORULIX_SIZES = {
    # name: (width, feed-forward, heads, kv heads, head size, pairs of layers, vocabulary)
    "2k": (2048, 8192, 16, 4, 128, 2, 32000),
    "4k": (4096, 12288, 32, 8, 128, 2, 32000),
}


def _sorulix_config(width, ff, heads, kv_heads, d, pairs, vocab) -> dict:
    parallel = {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": d, "scale": d ** -0.5, "softcap": 50.0,
                 "q_temp": {"coef": 0.3, "every": 64}},
        "right": {"heads": heads, "dim": d, "vdim": d, "decay": [1.0 - 2.0 ** (-5 - 3 * h / heads) for h in range(heads)]}},
        "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}}
    delta = {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": heads, "dim": d, "vdim": d, "conv": 4},
             "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}}
    return {"architecture": "Sorulix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "torch_dtype": "bfloat16",
            "layers": [parallel, delta] * pairs}


def _qwen3_like(width, ff, heads, kv_heads, d, pairs, vocab) -> dict:
    cfg = dict(QWEN3_8B)
    cfg.update(vocab_size=vocab, hidden_size=width, intermediate_size=ff, num_hidden_layers=2 * pairs, num_attention_heads=heads,
               num_key_value_heads=kv_heads, head_dim=d, max_position_embeddings=16384, tie_word_embeddings=True,
               bos_token_id=1, eos_token_id=2)
    return cfg


def _engine_measurer(args):
    """(peaks, timed, measure) behind the workloads that set a design beside another at equal sizes: ``measure(cfg, vocab)``
    opens an engine with seeded random weights and times a prefill of PREFILL_TOKENS tokens and decode steps at batch 1, 8
    and 32 with CONTEXT cached tokens per request, from a CUDA graph."""

    import torch

    from llm_runtime_study_b200.cache.slots import SlotRecord
    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.engine.step import StepEntry
    from llm_runtime_study_b200.ops import native

    torch.cuda.set_device(0)
    peak = peaks()
    generator = torch.Generator().manual_seed(0)
    greedy = SlotRecord(position=0)
    context, prefill_tokens = CONTEXT, PREFILL_TOKENS

    def timed(fn, repeat):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeat):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / repeat

    def measure(cfg, vocab):
        def ids(n):
            return torch.randint(0, vocab, (n,), generator=generator).tolist()

        batches = (1, 8, 32)
        engine = Engine.from_random_weights(
            cfg, seed=0, device="cuda:0", dtype="bfloat16", max_seq_len=8192, max_batch_size=max(*batches, args.batch), page_size=PAGE_SIZE,
            max_cache_tokens=max(*batches, args.batch) * (context + args.steps + 64), max_tokens_per_step=prefill_tokens, use_cuda_graph=True)
        runner, manager, sampler = engine.runner, engine.cache_manager, engine._sampler
        prompt = ids(prefill_tokens)

        def one_prefill():
            request = manager.admit()
            runner.step_sampled([StepEntry(request, prompt, [prefill_tokens - 1], greedy)], sampler).tokens()
            manager.release(request)

        out = {}
        if args.only != "decode":
            for _ in range(3):
                one_prefill()
            out = {"prefill_tokens": prefill_tokens, "prefill_ms": round(statistics.median(timed(one_prefill, 1) for _ in range(5)), 3)}
            out["prefill_tok_s"] = round(prefill_tokens / out["prefill_ms"] * 1e3)
        for batch in (() if args.only == "prefill" else (args.batch,) if args.only == "decode" else batches):
            requests = [manager.admit() for _ in range(batch)]
            for request in requests:
                runner.step_sampled([StepEntry(request, ids(context), [context - 1], greedy)], sampler)
            handles = []
            for _ in range(max(args.warmup, 3)):
                handles.append(runner.decode_sampled(requests, sampler))
            handles.pop().tokens()
            before = native.launch_count()
            ms = timed(lambda: handles.append(runner.decode_sampled(requests, sampler)), args.steps)
            out[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tok_s": round(batch / ms * 1e3),
                                       "launches_per_step": (native.launch_count() - before) // args.steps}
            handles[-1].tokens()
            for request in requests:
                manager.release(request)
        del engine, runner, manager, sampler
        gc.collect()
        torch.cuda.empty_cache()
        return out

    return peak, timed, measure


def run_sorulix(args) -> dict:
    """Prefill and decode of Sorulix at layer sizes of real models (random weights), beside Qwen3 at equal width,
    feed-forward, heads, head size and depth, through the same engine; then the new kernels alone, each against
    the bytes or flops it must move, beside the kernel of the Qwen3 path that does the like work."""

    peak, timed, measure = _engine_measurer(args)
    context = CONTEXT
    results = {}
    for name in (() if args.only == "kernels" else args.size.split(",") if args.size else SORULIX_SIZES):
        shape = SORULIX_SIZES[name]
        results[name] = {"shape": dict(zip(("width", "ff", "heads", "kv_heads", "head_dim", "layer_pairs", "vocab"), shape)),
                         "sorulix": measure(_sorulix_config(*shape), shape[-1])}
        if args.only not in ("prefill", "decode"):      # those two are profiling aids: the new design alone
            results[name]["qwen3_equal_size"] = measure(_qwen3_like(*shape), shape[-1])
    kernels = _sorulix_kernels(peak, timed) if args.only in ("all", "kernels") else {}
    return {"workload": "sorulix", "context": context, "steps": args.steps, "warmup": max(args.warmup, 3), "dtype": "bfloat16",
            "data": "synthetic token ids, seeded random weights", "peaks": peak, "models": results, "kernels": kernels}


def _sorulix_kernels(peak, timed) -> dict:
    """Each new kernel alone at the 4k shape (32 heads of 128, 8 KV heads), back to back, inputs larger than L2 where
    the kernel is bound by memory; beside it the kernel of the plain attention path at the same shape."""

    import torch
    from types import SimpleNamespace

    from llm_runtime_study_b200.ops import attention_bf16, attention_rules
    from llm_runtime_study_b200.ops import functional as F
    from llm_runtime_study_b200.ops import sequence_state as S

    dev = "cuda:0"
    heads, kv_heads, d, page = 32, 8, 128, PAGE_SIZE
    out = {}
    cold = timed

    def timed(fn, repeat):        # the first calls build and load libraries and size workspaces
        fn()
        fn()
        return cold(fn, repeat)

    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float32, device=dev)

    def attention_case(lengths, q_lens):
        pages = sum(-(-n // page) for n in lengths)
        table = torch.full((len(lengths), max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
        at = 0
        for r, n in enumerate(lengths):
            count = -(-n // page)
            table[r, :count] = torch.arange(at, at + count, dtype=torch.int32)
            at += count
        keys = torch.randn(pages, kv_heads, page, d, device=dev).bfloat16()
        values = torch.randn(pages, kv_heads, page, d, device=dev).bfloat16()
        q = torch.randn(sum(q_lens), heads, d, device=dev).bfloat16()
        positions = torch.cat([torch.arange(n - m, n) for n, m in zip(lengths, q_lens)]).int().to(dev)
        entry = torch.cat([torch.full((m,), i) for i, m in enumerate(q_lens)]).int().to(dev)
        ctx = SimpleNamespace(all_decode=max(q_lens) == 1, num_entries=len(lengths), max_kv_len=max(lengths), max_q_len=max(q_lens),
                              q_lens=list(q_lens), kv_lens=list(lengths), kv_len=torch.tensor(lengths, dtype=torch.int32, device=dev),
                              positions=positions, token_entry=entry, live_parts=None)
        return q, SimpleNamespace(keys=keys, values=values), ctx, table.to(dev)

    for tokens in (2048, 8192):
        q, cache, ctx, table = attention_case([tokens], [tokens])
        flops = 4.0 * heads * d * tokens * (tokens + 1) / 2
        rules = timed(lambda: attention_rules.paged_attention_rules(q, cache, ctx, table, scale=d ** -0.5, softcap=50.0, slopes=slopes, sink=True), 5)
        ctx.__dict__.pop("_tile_maps", None)
        plain_mma = timed(lambda: attention_bf16.prefill_attention(q, cache.keys, cache.values, positions=ctx.positions, block_table=table,
                                                                   q_lens=ctx.q_lens, scale=d ** -0.5), 5)
        plain_tc = timed(lambda: attention_bf16.try_paged_attention(q, cache, ctx, table, scale=d ** -0.5, window=0), 5)
        out[f"prefill_attention_{tokens}"] = {
            "with_rules_ms": round(rules, 3), "plain_mma_ms": round(plain_mma, 3), "plain_tcgen05_ms": round(plain_tc, 3),
            "with_rules_tflops": round(flops / rules / 1e9, 1), "plain_mma_tflops": round(flops / plain_mma / 1e9, 1),
            "plain_tcgen05_tflops": round(flops / plain_tc / 1e9, 1),
            "of_measured_bf16_burst": {"with_rules": round(flops / rules / 1e9 / peak["bf16_tflops"], 3),
                                       "plain_tcgen05": round(flops / plain_tc / 1e9 / peak["bf16_tflops"], 3)}}
    for batch, length in ((8, 2048), (32, 8192)):
        q, cache, ctx, table = attention_case([length] * batch, [1] * batch)
        moved = 2.0 * batch * length * kv_heads * d * 2
        rules = timed(lambda: attention_rules.paged_attention_rules(q, cache, ctx, table, scale=d ** -0.5, softcap=50.0, slopes=slopes, sink=True), 20)
        plain_tma = timed(lambda: attention_bf16.try_paged_attention(q, cache, ctx, table, scale=d ** -0.5, window=0), 20)
        out[f"decode_attention_b{batch}_ctx{length}"] = {
            "with_rules_us": round(rules * 1e3, 1), "plain_tma_us": round(plain_tma * 1e3, 1), "cache_mb": round(moved / 1e6, 1),
            "of_measured_copy": {"with_rules": round(moved / rules / 1e6 / peak["hbm_gbs"], 3),
                                 "plain_tma": round(moved / plain_tma / 1e6 / peak["hbm_gbs"], 3)}}
    # the scans: decoding moves every request's state in and out; a prompt is a chain of dependent steps
    for batch in (8, 64):
        n = batch
        q, k, v = (torch.randn(n, heads * d, device=dev) for _ in range(3))
        gate, beta = torch.rand(n, heads * d, device=dev), torch.rand(n, heads, device=dev)
        state = torch.zeros(batch + 1, heads, d, d, device=dev)
        q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        slots = torch.arange(batch, dtype=torch.int32, device=dev)
        decay = torch.full((heads,), 0.97, device=dev)
        moved = 2.0 * batch * heads * d * d * 4
        plain_ms = timed(lambda: S.linear_scan(q, k, v, heads=heads, qk_heads=heads, dim=d, vdim=d, state=state, q_start=q_start, slots=slots, decay=decay, silu=True), 20)
        delta_ms = timed(lambda: S.linear_scan(q, k, v, heads=heads, qk_heads=heads, dim=d, vdim=d, state=state, q_start=q_start, slots=slots, gate=gate, beta=beta), 20)
        out[f"scan_decode_b{batch}"] = {"decay_us": round(plain_ms * 1e3, 1), "delta_us": round(delta_ms * 1e3, 1), "state_mb": round(moved / 1e6, 1),
                                        "of_measured_copy": {"decay": round(moved / plain_ms / 1e6 / peak["hbm_gbs"], 3),
                                                             "delta": round(moved / delta_ms / 1e6 / peak["hbm_gbs"], 3)}}
    n = 2048
    q, k, v = (torch.randn(n, heads * d, device=dev) for _ in range(3))
    gate, beta = torch.rand(n, heads * d, device=dev) * 0.1 + 0.9, torch.rand(n, heads, device=dev)
    state = torch.zeros(2, heads, d, d, device=dev)
    q_start = torch.tensor([0, n], dtype=torch.int32, device=dev)
    slots = torch.zeros(1, dtype=torch.int32, device=dev)
    kn = torch.nn.functional.normalize(k.view(n, heads, d), dim=-1).reshape(n, -1)
    delta_ms = timed(lambda: S.linear_scan(q, kn, v, heads=heads, qk_heads=heads, dim=d, vdim=d, state=state, q_start=q_start, slots=slots, gate=gate, beta=beta), 3)
    state.zero_()
    decay_ms = timed(lambda: S.linear_scan(q, kn, v, heads=heads, qk_heads=heads, dim=d, vdim=d, state=state, q_start=q_start, slots=slots,
                                           decay=torch.full((heads,), 0.97, device=dev)), 3)
    out["scan_prefill_2048"] = {"delta_ms": round(delta_ms, 3), "decay_ms": round(decay_ms, 3),
                                "delta_us_per_token": round(delta_ms * 1e3 / n, 3), "decay_us_per_token": round(decay_ms * 1e3 / n, 3)}
    # element-wise kernels at 2,048 rows (inputs of tens of MB; the figure is bytes moved over the copy rate)
    rows, ff = 2048, 12288
    gate_up = torch.randn(rows, 2 * ff, device=dev).bfloat16()
    ms = timed(lambda: F.glu_limit(gate_up, 7.0, 1.702), 20)
    ref = timed(lambda: F.silu_mul(gate_up), 20)
    moved = rows * ff * 2 * 3
    out["glu_limit_2048x12288"] = {"us": round(ms * 1e3, 1), "silu_mul_us": round(ref * 1e3, 1),
                                   "of_measured_copy": {"glu_limit": round(moved / ms / 1e6 / peak["hbm_gbs"], 3),
                                                        "silu_mul": round(moved / ref / 1e6 / peak["hbm_gbs"], 3)}}
    return out


# ------------------------------------------------------------------------------ Ropulix beside Sorulix and Qwen3
ROPULIX_EXPERTS, ROPULIX_TOP, ROPULIX_WINDOW = 8, 2, 1024


def _ropulix_config(width, ff, heads, kv_heads, d, pairs, vocab) -> dict:
    """Four kinds of layers in turn (recurrence, latent attention, windowed attention, latent attention on borrowed rows);
    every token uses ROPULIX_TOP experts whose hidden sizes add up to the dense feed-forward's."""

    moe = {"kind": "moe", "expert": {"ff": ff // ROPULIX_TOP}, "router": {"experts": ROPULIX_EXPERTS, "top": ROPULIX_TOP}}
    latent = {"heads": heads, "dim": d, "rot_dim": d // 2, "vdim": d, "kv_rank": 4 * d, "q_rank": width // 2, "mask": {"size": ROPULIX_WINDOW},
              "rot": {"base": 10000.0, "dims": d // 2}, "scale": (d + d // 2) ** -0.5}
    layers = []
    for pair in range(pairs):
        at = len(layers)
        layers += [
            {"type": "rglru", "mixer": {"width": width, "blocks": heads, "conv": 4}, "mlp": moe},
            {"type": "latent_attention", "mixer": dict(latent), "mlp": moe},
            {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": d, "mask": {"size": ROPULIX_WINDOW},
                                            "scale": d ** -0.5}, "mlp": moe},
            {"type": "latent_attention", "mixer": dict(latent, kv_from=at + 1), "mlp": moe},
        ]
    return {"architecture": "Ropulix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "torch_dtype": "bfloat16",
            "layers": layers[: 2 * pairs]}


def run_ropulix(args) -> dict:
    """Prefill and decode of Ropulix at layer sizes of real models (random weights), beside Sorulix (the closest design:
    attention beside mixers with a state per request) and Qwen3 at equal width, active feed-forward size, heads, head size
    and depth, through the same engine; then the new kernels alone against the bytes or flops they must move."""

    peak, timed, measure = _engine_measurer(args)
    results = {}
    for name in (() if args.only == "kernels" else args.size.split(",") if args.size else SORULIX_SIZES):
        shape = SORULIX_SIZES[name]
        results[name] = {"shape": dict(zip(("width", "ff", "heads", "kv_heads", "head_dim", "layer_pairs", "vocab"), shape)),
                         "experts": ROPULIX_EXPERTS, "top": ROPULIX_TOP, "window": ROPULIX_WINDOW,
                         "ropulix": measure(_ropulix_config(*shape), shape[-1])}
        if args.only not in ("prefill", "decode"):
            results[name]["sorulix_equal_size"] = measure(_sorulix_config(*shape), shape[-1])
            results[name]["qwen3_equal_size"] = measure(_qwen3_like(*shape), shape[-1])
    kernels = _ropulix_kernels(peak, timed) if args.only in ("all", "kernels") else {}
    return {"workload": "ropulix", "context": CONTEXT, "steps": args.steps, "warmup": max(args.warmup, 3), "dtype": "bfloat16",
            "data": "synthetic token ids, seeded random weights", "peaks": peak, "models": results, "kernels": kernels}


def _ropulix_kernels(peak, timed) -> dict:
    """Each new kernel alone at the 4k shape (width 4096, 32 heads of 128), back to back, beside the kernel of an existing
    path that does the like work."""

    import torch
    from types import SimpleNamespace

    from llm_runtime_study_b200.ops import attention_latent
    from llm_runtime_study_b200.ops import functional as F
    from llm_runtime_study_b200.ops import gemm_bf16
    from llm_runtime_study_b200.ops import grouped as G
    from llm_runtime_study_b200.ops import mixer_steps as M
    from llm_runtime_study_b200.ops import sequence_state as S

    dev = "cuda:0"
    width, heads, d, ff = 4096, 32, 128, 12288 // ROPULIX_TOP
    out = {}
    cold = timed

    def timed(fn, repeat):
        """Replayed from a CUDA graph, so that what is timed is the device's work and not the host's preparation of a launch of
        a few microseconds; the first calls build and load libraries and make the maps a capture must not make."""

        fn()
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        return cold(graph.replay, repeat)

    bf = lambda *shape: (0.05 * torch.randn(*shape, device=dev)).bfloat16()
    # experts: sorted rows through both products, against one dense projection of the same flops
    router, up, down = torch.randn(ROPULIX_EXPERTS, width, device=dev), bf(ROPULIX_EXPERTS, ff, width), bf(ROPULIX_EXPERTS, width, ff)
    for n in (2048, 8):
        x = bf(n, width)
        wide = G.wide_tiles_pay(n, ROPULIX_TOP, x.dtype, width, ff)
        routing = G.route(x, router, None, top=ROPULIX_TOP, wide_tiles=wide)
        hidden = G.expert_linear(x, up, routing, gather=True, act="relu2")
        t_route = timed(lambda: G.route(x, router, None, top=ROPULIX_TOP, wide_tiles=wide), 10)
        t_up = timed(lambda: G.expert_linear(x, up, routing, gather=True, act="relu2"), 10)
        t_down = timed(lambda: G.expert_linear(hidden, down, routing, gather=False, out_dtype=torch.float32), 10)
        rows = n * ROPULIX_TOP
        dense_x, dense_w = bf(rows, width), bf(ff, width)
        t_dense = timed(lambda: gemm_bf16.linear(dense_x, dense_w, None, torch.bfloat16) if rows >= 128
                        else gemm_bf16.linear_skinny(dense_x, dense_w, None, torch.bfloat16), 10)
        flops = 2.0 * rows * width * ff
        touched = min(ROPULIX_EXPERTS, rows) * ff * width * 2
        out[f"experts_{n}_tokens"] = {
            "route_and_sort_us": round(t_route * 1e3, 1), "up_us": round(t_up * 1e3, 1), "down_us": round(t_down * 1e3, 1),
            "dense_projection_of_equal_flops_us": round(t_dense * 1e3, 1),
            "up_tflops": round(flops / t_up / 1e9, 1), "dense_tflops": round(flops / t_dense / 1e9, 1),
            "of_measured_bf16_burst": {"up": round(flops / t_up / 1e9 / peak["bf16_tflops"], 3), "dense": round(flops / t_dense / 1e9 / peak["bf16_tflops"], 3)},
            "of_measured_copy": {"up": round(touched / t_up / 1e6 / peak["hbm_gbs"], 3), "dense": round(ff * width * 2 / t_dense / 1e6 / peak["hbm_gbs"], 3)}}
    # latent attention over shared rows (CUDA cores) beside the plain windowed attention of equal heads (tensor cores)
    rank, rot, page = 4 * d, d // 2, PAGE_SIZE
    for n, new in ((2048, 2048), (8 * 2048, 8)):
        length = 2048
        seqs = n // length if new == n else 8
        lengths = [length] * seqs
        q_lens = [length] * seqs if new == n else [1] * seqs
        pages = sum(-(-m // page) for m in lengths)
        table = torch.arange(pages, dtype=torch.int32).view(seqs, -1).to(dev)
        pool = bf(pages, page, rank + rot)
        q = bf(sum(q_lens), heads, rank + rot)
        positions = torch.cat([torch.arange(m - k, m) for m, k in zip(lengths, q_lens)]).int().to(dev)
        entry = torch.cat([torch.full((k,), i) for i, k in enumerate(q_lens)]).int().to(dev)
        ctx = SimpleNamespace(positions=positions, token_entry=entry, all_decode=max(q_lens) == 1, num_entries=seqs, q_lens=q_lens,
                              kv_lens=lengths, max_kv_len=max(lengths))
        t = timed(lambda: attention_latent.latent_attention(q, pool, ctx, table, value_dim=rank, scale=0.07, window=ROPULIX_WINDOW), 3)
        t_simt = cold(lambda: F.paged_attention_simt_latent(q, pool, value_dim=rank, positions=positions, token_entry=entry,
                                                            block_table=table, scale=0.07, window=ROPULIX_WINDOW), 1)
        seen = sum(min(ROPULIX_WINDOW, p + 1) for p in positions.tolist())
        flops = 2.0 * heads * seen * (2 * rank + rot)
        out[f"latent_attention_{'prefill' if new == n else 'decode_b8'}_{length}"] = {
            "ms": round(t, 3), "cuda_core_kernel_ms": round(t_simt, 3), "tflops": round(flops / t / 1e9, 2),
            "of_measured_bf16_burst": round(flops / t / 1e9 / peak["bf16_tflops"], 4),
            "rows_read_mb": round(seqs * min(length, ROPULIX_WINDOW + (length if new == n else 0)) * (rank + rot) * 2 / 1e6, 2)}
    # the recurrence: a prompt portion is a chain per channel; decoding moves the state in and out
    for n, entries in ((2048, 1), (32, 32)):
        bw = width // heads
        proj, u = bf(n, 2 * width), bf(n, width)
        gates = torch.randn(n, heads, 2 * bw, device=dev)
        lam = torch.randn(width, device=dev)
        state = torch.zeros(entries + 1, width, device=dev)
        q_start = torch.arange(0, n + 1, n // entries, dtype=torch.int32, device=dev)
        slots = torch.arange(entries, dtype=torch.int32, device=dev)
        gate_w = bf(heads, 2 * bw, bw)
        t_scan = timed(lambda: M.gated_recurrence(gates, u, proj, y_offset=width, lam=lam, decay_scale=8.0, state=state, q_start=q_start,
                                                  slots=slots, block_width=bw), 5)
        t_gates = timed(lambda: G.batched_linear(u, gate_w, batch=heads, k=bw, n_out=2 * bw, a_batch_stride=bw, out_dtype=torch.float32), 5)
        moved = n * width * (8 + 2 + 2 + 2)
        out[f"recurrence_{n}_tokens_{entries}_requests"] = {
            "scan_us": round(t_scan * 1e3, 1), "gate_product_us": round(t_gates * 1e3, 1),
            "scan_of_measured_copy": round(moved / t_scan / 1e6 / peak["hbm_gbs"], 3),
            "gate_product_tflops": round(2.0 * n * width * 2 * bw / t_gates / 1e9, 1)}
    # the norm on a sublayer's output beside the pre-norm's add-and-normalise
    rows = 2048
    x, w, resid = torch.randn(rows, width, device=dev), torch.randn(width, device=dev), torch.randn(rows, width, device=dev)
    t_new = timed(lambda: M.norm_accumulate_round(x, w, 1e-6, resid, torch.bfloat16), 20)
    t_old = timed(lambda: F.add_rmsnorm(resid, x, w, 1e-6, torch.bfloat16), 20)
    out["norm_on_output_2048x4096"] = {"us": round(t_new * 1e3, 1), "add_rmsnorm_us": round(t_old * 1e3, 1),
                                       "of_measured_copy": {"norm_on_output": round(rows * width * 14 / t_new / 1e6 / peak["hbm_gbs"], 3),
                                                            "add_rmsnorm": round(rows * width * 14 / t_old / 1e6 / peak["hbm_gbs"], 3)}}
    return out


# ------------------------------------------------------------------------------ Mabedra beside Ropulix and Qwen3
MABEDRA_EXPERTS, MABEDRA_TOP, MABEDRA_WINDOW, MABEDRA_TAPS = 8, 2, 1024, 4


def _mabedra_config(width, ff, heads, kv_heads, d, pairs, vocab) -> dict:
    """Half as many heads as the plain attention of equal size, each with two maps of ``d`` columns and values of ``2 d``
    (projections and cache rows of equal size); a dense layer whose two matrices hold what the gated unit's three do, then a
    layer of experts: every token uses MABEDRA_TOP of ``ff / 4`` beside a shared one of ``ff / 2``."""

    mixer = {"heads": heads // 2, "kv_heads": kv_heads // 2, "dim": d, "vdim": 2 * d, "diff": 0.3, "scale": d ** -0.5,
             "mask": {"size": MABEDRA_WINDOW},
             "rot": {"base": 10000.0, "dims": d, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    dense = {"kind": "dense", "ff": ff * 3 // 2}
    moe = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": MABEDRA_EXPERTS, "top": MABEDRA_TOP}, "shared": {"ff": ff // 2}}
    layers = [{"type": "attention", "mixer": dict(mixer), "mlp": dense}, {"type": "attention", "mixer": dict(mixer), "mlp": moe}] * pairs
    return {"architecture": "Mabedra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": MABEDRA_TAPS},
            "torch_dtype": "bfloat16", "layers": layers}


def run_mabedra(args) -> dict:
    """Prefill and decode of Mabedra at layer sizes of real models (random weights), beside Qwen3 (the closest design: every
    layer is softmax attention over paged keys and values with normed, rotated heads) and Ropulix (windows and routed
    experts) at equal width, active feed-forward size, attention columns and depth, through the same engine; then the new
    kernels alone against the bytes or flops they must move, each beside the like kernel of those paths."""

    peak, timed, measure = _engine_measurer(args)
    results = {}
    for name in (() if args.only == "kernels" else args.size.split(",") if args.size else SORULIX_SIZES):
        shape = SORULIX_SIZES[name]
        results[name] = {"shape": dict(zip(("width", "ff", "heads", "kv_heads", "head_dim", "layer_pairs", "vocab"), shape)),
                         "experts": MABEDRA_EXPERTS, "top": MABEDRA_TOP, "window": MABEDRA_WINDOW, "taps": MABEDRA_TAPS,
                         "mabedra": measure(_mabedra_config(*shape), shape[-1])}
        if args.only not in ("prefill", "decode"):
            results[name]["qwen3_equal_size"] = measure(_qwen3_like(*shape), shape[-1])
            results[name]["ropulix_equal_size"] = measure(_ropulix_config(*shape), shape[-1])
    kernels = _mabedra_kernels(peak, timed) if args.only in ("all", "kernels") else {}
    return {"workload": "mabedra", "context": CONTEXT, "steps": args.steps, "warmup": max(args.warmup, 3), "dtype": "bfloat16",
            "data": "synthetic token ids, seeded random weights", "peaks": peak, "models": results, "kernels": kernels}


def _mabedra_kernels(peak, timed) -> dict:
    """Each new kernel alone at the 4k shape (width 4096; 16 heads of two maps of 128 with values of 256, 4 key/value heads),
    replayed from a CUDA graph, beside the kernel of an existing path that does the like work (32 heads of 128, 8 key/value
    heads: projections and cache rows of equal size)."""

    import torch
    from types import SimpleNamespace

    from llm_runtime_study_b200.ops import attention_bf16, attention_diff
    from llm_runtime_study_b200.ops import block_steps as B
    from llm_runtime_study_b200.ops import functional as F
    from llm_runtime_study_b200.ops import sequence_state as S

    dev = "cuda:0"
    width, heads, kv_heads, d, page, window = 4096, 32, 8, 128, PAGE_SIZE, MABEDRA_WINDOW
    dh, dkv, dv = heads // 2, kv_heads // 2, 2 * d
    out = {}
    cold = timed

    def timed(fn, repeat):
        fn()
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        return cold(graph.replay, repeat)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed_cold(fn, repeat):
        """The same with the L2 overwritten before every replay (256 MB of zeros), each replay between events of its own: a kernel
        whose arrays would stay in the L2 from one replay to the next is then measured from memory like one whose arrays do not."""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        total = 0.0
        for _ in range(repeat):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            total += start.elapsed_time(end)
        return total / repeat

    bf = lambda *shape: torch.randn(*shape, device=dev).bfloat16()

    def case(lengths, q_lens):
        seqs = len(lengths)
        per = -(-max(lengths) // page)
        table = torch.arange(seqs * per, dtype=torch.int32).view(seqs, per).to(dev)
        positions = torch.cat([torch.arange(m - k, m) for m, k in zip(lengths, q_lens)]).int().to(dev)
        entry = torch.cat([torch.full((k,), i) for i, k in enumerate(q_lens)]).int().to(dev)
        ctx = SimpleNamespace(positions=positions, token_entry=entry, all_decode=max(q_lens) == 1, num_entries=seqs, q_lens=list(q_lens),
                              kv_lens=list(lengths), max_kv_len=max(lengths), max_q_len=max(q_lens),
                              kv_len=torch.tensor(lengths, dtype=torch.int32, device=dev), live_parts=None)
        pools = dict(diff_k=bf(seqs * per, dkv, page, 2 * d), diff_v=bf(seqs * per, dkv, page, dv),
                     keys=bf(seqs * per, kv_heads, page, d), values=bf(seqs * per, kv_heads, page, d))
        return ctx, table, pools, positions

    def run_diff(q, pools, ctx, table):
        return attention_diff.diff_attention_mma(q, pools["diff_k"], pools["diff_v"], ctx, table, scale=d ** -0.5, window=window, lam=0.4,
                                                 out_scale=0.7, eps=1e-6)

    for tokens in (2048, 8192):
        ctx, table, pools, positions = case([tokens], [tokens])
        seen = sum(min(window, p + 1) for p in positions.tolist())
        q, q_plain = bf(tokens, dh, 2 * d), bf(tokens, heads, d)
        t = timed(lambda: run_diff(q, pools, ctx, table), 5)
        plain_tiles = attention_bf16.tile_map(ctx.q_lens, 64 // min(heads // kv_heads, 16), dev, ctx.kv_lens)
        t_plain = timed(lambda: attention_bf16.prefill_attention(q_plain, pools["keys"], pools["values"], positions=ctx.positions, block_table=table,
                                                                 q_lens=ctx.q_lens, scale=d ** -0.5, window=window, tiles=plain_tiles), 5)
        flops, flops_plain = 2.0 * dh * seen * 2 * (d + dv), 2.0 * heads * seen * 2 * d
        out[f"differential_attention_prefill_{tokens}_window_{window}"] = {
            "ms": round(t, 3), "plain_windowed_mma_ms": round(t_plain, 3), "tflops": round(flops / t / 1e9, 1),
            "plain_windowed_mma_tflops": round(flops_plain / t_plain / 1e9, 1),
            "of_measured_bf16_burst": {"differential": round(flops / t / 1e9 / peak["bf16_tflops"], 4),
                                       "plain_windowed_mma": round(flops_plain / t_plain / 1e9 / peak["bf16_tflops"], 4)}}
    for batch, length in ((8, 2048), (32, 8192)):
        ctx, table, pools, _ = case([length] * batch, [1] * batch)
        q, q_plain = bf(batch, dh, 2 * d), bf(batch, heads, d)
        t = timed(lambda: run_diff(q, pools, ctx, table), 20)
        cache = SimpleNamespace(keys=pools["keys"], values=pools["values"])
        t_plain = timed(lambda: attention_bf16.try_paged_attention(q_plain, cache, ctx, table, scale=d ** -0.5, window=window), 20)
        moved = 2.0 * batch * min(length, window) * (dkv * (2 * d + dv))        # equal to the plain cache's rows
        out[f"differential_attention_decode_b{batch}_ctx{length}_window_{window}"] = {
            "us": round(t * 1e3, 1), "plain_windowed_us": round(t_plain * 1e3, 1), "rows_read_mb": round(moved / 1e6, 2),
            "of_measured_copy": {"differential": round(moved / t / 1e6 / peak["hbm_gbs"], 3),
                                 "plain_windowed": round(moved / t_plain / 1e6 / peak["hbm_gbs"], 3)}}
    # the head of a layer: the norm, both sublayers' inputs with their convolutions, the kept inputs; beside add-and-normalise
    rows, taps = 2048, MABEDRA_TAPS
    resid, delta, w = torch.randn(rows, width, device=dev), torch.randn(rows, width, device=dev), torch.randn(width, device=dev)
    wa, wb = torch.randn(width, taps, device=dev), torch.randn(width, taps, device=dev)
    kept = torch.zeros(2, taps - 1, width, device=dev)
    q_start = torch.tensor([0, rows], dtype=torch.int32, device=dev)
    slots, entry = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(rows, dtype=torch.int32, device=dev)

    def head_of_layer():
        h = B.layer_norm(resid, delta, w, 1e-6, torch.float32)
        pair = B.taps_pair(h, wa, wb, kept, q_start=q_start, slots=slots, token_entry=entry, out_dtype=torch.bfloat16)
        S.conv_state_update(h, kept, q_start, slots)
        return pair

    t_norm = timed(lambda: B.layer_norm(resid, delta, w, 1e-6, torch.float32), 20)
    t_head = timed(head_of_layer, 20)
    t_old = timed(lambda: F.add_rmsnorm(resid, delta, w, 1e-6, torch.bfloat16), 20)
    cell = rows * width
    c_norm = timed_cold(lambda: B.layer_norm(resid, delta, w, 1e-6, torch.float32), 10)
    c_head = timed_cold(head_of_layer, 10)
    c_old = timed_cold(lambda: F.add_rmsnorm(resid, delta, w, 1e-6, torch.bfloat16), 10)
    out["layer_head_2048x4096"] = {
        "layer_norm_us": round(t_norm * 1e3, 1), "norm_taps_kept_us": round(t_head * 1e3, 1), "add_rmsnorm_us": round(t_old * 1e3, 1),
        "of_measured_copy": {"layer_norm": round(cell * 16 / t_norm / 1e6 / peak["hbm_gbs"], 3),
                             "norm_taps_kept": round(cell * (16 + 4 + 4) / t_head / 1e6 / peak["hbm_gbs"], 3),
                             "add_rmsnorm": round(cell * 14 / t_old / 1e6 / peak["hbm_gbs"], 3)},
        "l2_flushed_us": {"layer_norm": round(c_norm * 1e3, 1), "norm_taps_kept": round(c_head * 1e3, 1), "add_rmsnorm": round(c_old * 1e3, 1)},
        "l2_flushed_of_measured_copy": {"layer_norm": round(cell * 16 / c_norm / 1e6 / peak["hbm_gbs"], 3),
                                        "norm_taps_kept": round(cell * (16 + 4 + 4) / c_head / 1e6 / peak["hbm_gbs"], 3),
                                        "add_rmsnorm": round(cell * 14 / c_old / 1e6 / peak["hbm_gbs"], 3)}}
    # the tail of a layer: both sublayers' results scaled and added, the result kept, the average over all results so far
    a, b, sa, sb = torch.randn(rows, width, device=dev), torch.randn(rows, width, device=dev), torch.randn(width, device=dev), torch.randn(width, device=dev)
    for index in (0, 3):
        results, mix = torch.randn(index + 2, rows, width, device=dev), torch.randn(index + 2, device=dev)
        t = timed(lambda: B.scale_sum_average(resid, a, sa, b, sb, results, mix, index), 20)
        moved = cell * 4 * (3 + 1 + (index + 1) + 1)       # x, a, b read; the result written; earlier results read; x written
        out[f"layer_tail_2048x4096_over_{index + 2}"] = {"us": round(t * 1e3, 1), "of_measured_copy": round(moved / t / 1e6 / peak["hbm_gbs"], 3)}
    # the activations: normalised powers over a row of the dense feed-forward; the gated unit with a factor per row
    ff = 12288 * 3 // 2
    z = bf(rows, ff)
    coef = torch.tensor([0.9, -0.4, 0.3, 0.1], device=dev)
    gate_up = bf(rows, 2 * 12288)
    factor = torch.rand(rows, device=dev)
    t_poly = timed(lambda: B.poly_norm(z, coef, 1e-6), 20)
    t_scaled = timed(lambda: B.silu_mul_scaled(gate_up, None, factor), 20)
    t_silu = timed(lambda: F.silu_mul(gate_up), 20)
    out["activations_2048_rows"] = {
        "poly_norm_us": round(t_poly * 1e3, 1), "silu_mul_scaled_us": round(t_scaled * 1e3, 1), "silu_mul_us": round(t_silu * 1e3, 1),
        "of_measured_copy": {"poly_norm": round(rows * ff * 4 / t_poly / 1e6 / peak["hbm_gbs"], 3),
                             "silu_mul_scaled": round(rows * 12288 * 6 / t_scaled / 1e6 / peak["hbm_gbs"], 3),
                             "silu_mul": round(rows * 12288 * 6 / t_silu / 1e6 / peak["hbm_gbs"], 3)}}
    # norm, rotation and page write of both maps beside the plain heads' (rows of equal width)
    ctx, table, pools, positions = case([rows], [rows])
    qkv, qkv_plain = bf(rows, (dh + dkv) * 2 * d + dkv * dv), bf(rows, (heads + 2 * kv_heads) * d)
    hw = torch.ones(d, device=dev)
    inv_freq = (10000.0 ** (-torch.arange(0, d, 2, dtype=torch.float32) / d)).to(dev)
    t_maps = timed(lambda: attention_diff.map_norm_rope_write(
        qkv, num_q_heads=dh, num_kv_heads=dkv, maps=2, head_dim=d, value_dim=dv, q_weight=hw, k_weight=hw, eps=1e-6, inv_freq=inv_freq,
        rotary_dim=d, positions=positions, token_entry=ctx.token_entry, block_table=table, page_size=page, k_pool=pools["diff_k"],
        v_pool=pools["diff_v"]), 20)
    t_heads = timed(lambda: F.qk_norm_rope_write(
        qkv_plain, num_q_heads=heads, num_kv_heads=kv_heads, head_dim=d, q_weight=hw, k_weight=hw, eps=1e-6, inv_freq=inv_freq, rotary_dim=d,
        positions=positions, token_entry=ctx.token_entry, block_table=table, page_size=page, k_pool=pools["keys"], v_pool=pools["values"]), 20)
    moved = rows * (heads + 2 * kv_heads) * d * 4
    out["norm_rotate_write_2048_tokens"] = {"maps_us": round(t_maps * 1e3, 1), "plain_heads_us": round(t_heads * 1e3, 1),
                                            "of_measured_copy": {"maps": round(moved / t_maps / 1e6 / peak["hbm_gbs"], 3),
                                                                 "plain_heads": round(moved / t_heads / 1e6 / peak["hbm_gbs"], 3)}}
    return out


# ------------------------------------------------------------------------------ Tafisun beside Ropulix and Qwen3
TAFISUN_EXPERTS, TAFISUN_IDENTITY, TAFISUN_TOP, TAFISUN_GROUPS, TAFISUN_KEEP, TAFISUN_CHUNK = 8, 2, 2, 5, 3, 1024


def _tafisun_config(width, ff, heads, kv_heads, d, pairs, vocab) -> dict:
    """A minGRU layer and a chunked attention layer in turn; the first layer's feed-forward is dense, every other one a
    mixture: every token uses TAFISUN_TOP of eight experts of ``ff / 4`` hidden units (or of two outputs that return their
    input) beside a shared unit of ``ff / 4``."""

    moe = {"kind": "moe", "expert": {"ff": ff // 4, "limit": 7.0},
           "router": {"experts": TAFISUN_EXPERTS, "identity": TAFISUN_IDENTITY, "top": TAFISUN_TOP, "scale": 2.0,
                      "groups": {"count": TAFISUN_GROUPS, "keep": TAFISUN_KEEP}},
           "shared": {"ff": ff // 4, "limit": 7.0}}
    layers = []
    for pair in range(pairs):
        layers += [
            {"type": "mingru", "mixer": {"width": width}, "mlp": {"kind": "dense", "ff": ff} if pair == 0 else moe},
            {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": d, "mask": {"size": TAFISUN_CHUNK},
                                            "scale": d ** -0.5}, "mlp": moe},
        ]
    return {"architecture": "Tafisun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "torch_dtype": "bfloat16",
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 131, "mul_cur": 17}}, "layers": layers}


def run_tafisun(args) -> dict:
    """Prefill and decode of Tafisun at layer sizes of real models (random weights), beside Ropulix (the closest design:
    masked attention beside a recurrence per channel, and experts) and Qwen3 at equal width, heads, head size and depth,
    through the same engine; then the new kernels alone against the bytes or flops they must move, each beside the like
    kernel of an existing path."""

    peak, timed, measure = _engine_measurer(args)
    results = {}
    for name in (() if args.only == "kernels" else args.size.split(",") if args.size else SORULIX_SIZES):
        shape = SORULIX_SIZES[name]
        results[name] = {"shape": dict(zip(("width", "ff", "heads", "kv_heads", "head_dim", "layer_pairs", "vocab"), shape)),
                         "experts": TAFISUN_EXPERTS, "identity": TAFISUN_IDENTITY, "top": TAFISUN_TOP, "chunk": TAFISUN_CHUNK,
                         "tafisun": measure(_tafisun_config(*shape), shape[-1])}
        if args.only not in ("prefill", "decode"):
            results[name]["ropulix_equal_size"] = measure(_ropulix_config(*shape), shape[-1])
            results[name]["qwen3_equal_size"] = measure(_qwen3_like(*shape), shape[-1])
    kernels = _tafisun_kernels(peak, timed) if args.only in ("all", "kernels") else {}
    return {"workload": "tafisun", "context": CONTEXT, "steps": args.steps, "warmup": max(args.warmup, 3), "dtype": "bfloat16",
            "data": "synthetic token ids, seeded random weights", "peaks": peak, "models": results, "kernels": kernels}


def _tafisun_kernels(peak, timed) -> dict:
    """Each new kernel alone at the 4k shape (width 4096, 32 heads of 128 over 8 key/value heads), replayed from a CUDA
    graph, beside the kernel of an existing path that does the like work; fractions are of the measured copy bandwidth
    for the bytes a kernel must move."""

    import torch
    from types import SimpleNamespace

    from llm_runtime_study_b200.ops import attention_bf16, attention_rules
    from llm_runtime_study_b200.ops import block_steps as B
    from llm_runtime_study_b200.ops import functional as F
    from llm_runtime_study_b200.ops import grouped as G
    from llm_runtime_study_b200.ops import mixer_steps as M

    dev = "cuda:0"
    width, heads, kv_heads, d, ff = 4096, 32, 8, 128, 12288 // 4
    out = {}
    cold = timed

    def timed(fn, repeat):
        fn()
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        return cold(graph.replay, repeat)

    def frac(moved, ms):
        return round(moved / ms / 1e6 / peak["hbm_gbs"], 3)

    bf = lambda *shape: (0.05 * torch.randn(*shape, device=dev)).bfloat16()
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=dev)
    # the embedding's sum beside the plain table lookup
    vocab, buckets = 32000, 65521
    table, bigram = bf(vocab, width), bf(buckets + 1, width)
    freq = torch.tensor([10000.0 ** (-2.0 * i / width) for i in range(width // 2)], dtype=torch.float64, device=dev)
    for n, entries in ((2048, 1), (32, 32)):
        ids = torch.randint(0, vocab, (n,), dtype=torch.int32, device=dev)
        per = n // entries
        positions = ints([2048 * (entries > 1) + j for _ in range(entries) for j in range(per)])
        entry = ints([e for e in range(entries) for _ in range(per)])
        q_start, slots = ints(list(range(0, n + 1, per))), ints(list(range(entries)))
        previous = torch.zeros(entries + 1, 1, dtype=torch.int32, device=dev)
        t_new = timed(lambda: F.embedding_sum(ids, table, bigram, positions=positions, token_entry=entry, q_start=q_start, slots=slots,
                                              previous=previous, freq=freq, buckets=buckets, mul_prev=131, mul_cur=17), 20)
        t_old = timed(lambda: F.embedding(ids, table), 20)
        out[f"embedding_{n}_tokens"] = {"summed_us": round(t_new * 1e3, 1), "table_only_us": round(t_old * 1e3, 1),
                                        "of_measured_copy": {"summed": frac(n * width * 8, t_new), "table_only": frac(n * width * 6, t_old)}}
    # minGRU beside the gated linear recurrence's two kernels (gates' arithmetic, chain)
    for n, entries in ((2048, 1), (8192, 4), (32, 32)):
        proj = bf(n, 3 * width)
        state = torch.zeros(entries + 1, width, device=dev)
        q_start, slots = ints(list(range(0, n + 1, n // entries))), ints(list(range(entries)))
        t_chain = timed(lambda: M.mingru_scan(proj, width=width, z_offset=0, u_offset=width, g_offset=2 * width, state=state, q_start=q_start,
                                              slots=slots), 5)
        t_new = t_chain
        if n // entries >= M.MINGRU_SEGMENT_MIN > 0:      # the form the model runs for portions of this length
            segments = M.mingru_segment_map([n // entries] * entries, list(range(entries)), dev)
            t_new = timed(lambda: M.mingru_scan(proj, width=width, z_offset=0, u_offset=width, g_offset=2 * width, state=state,
                                                q_start=q_start, slots=slots, segments=segments), 5)
        bw = width // heads
        proj2, u = bf(n, 2 * width), bf(n, width)
        gates, lam = torch.randn(n, heads, 2 * bw, device=dev), torch.randn(width, device=dev)
        t_old = timed(lambda: M.gated_recurrence(gates, u, proj2, y_offset=width, lam=lam, decay_scale=8.0, state=state, q_start=q_start,
                                                 slots=slots, block_width=bw), 5)
        out[f"recurrence_{n}_tokens_{entries}_requests"] = {
            "mingru_us": round(t_new * 1e3, 1), "mingru_one_chain_us": round(t_chain * 1e3, 1), "gated_linear_recurrence_us": round(t_old * 1e3, 1),
            "of_measured_copy": {"mingru": frac(n * width * 8, t_new), "gated_linear_recurrence": frac(n * width * 14, t_old)}}
    # attention under the block mask with the logarithmic bias beside the plain attention under a window of equal reach
    page = PAGE_SIZE
    r1, r2 = torch.rand(heads, device=dev), torch.rand(heads, device=dev)
    for seqs, length, new in ((1, 2048, 2048), (4, 2048, 2048), (8, 2048, 1), (32, 2048, 1)):
        lengths, q_lens = [length] * seqs, [new] * seqs
        pages = seqs * (length // page)
        table_ = torch.arange(pages, dtype=torch.int32).view(seqs, -1).to(dev)
        keys, values = bf(pages, kv_heads, page, d), bf(pages, kv_heads, page, d)
        q = bf(seqs * new, heads, d)
        positions = ints([p for m, k in zip(lengths, q_lens) for p in range(m - k, m)])
        entry = ints([i for i, k in enumerate(q_lens) for _ in range(k)])
        ctx = SimpleNamespace(positions=positions, token_entry=entry, all_decode=new == 1, num_entries=seqs, q_lens=q_lens, kv_lens=lengths,
                              max_kv_len=length, max_q_len=new, kv_len=ints(lengths), runtime=None, manager=None)
        cache = SimpleNamespace(keys=keys, values=values, page_size=page, group=0)
        t_new = timed(lambda: attention_rules.paged_attention_rules(q, cache, ctx, table_, scale=0.09, chunk=TAFISUN_CHUNK, log_bias=(r1, r2)), 5)
        ctx2 = SimpleNamespace(**vars(ctx))
        ctx2.tables = [table_]
        ctx2.block_table = lambda group: table_
        t_old = timed(lambda: attention_bf16.try_paged_attention(q, cache, ctx2, table_, scale=0.09, window=TAFISUN_CHUNK), 5)
        seen = sum(p % TAFISUN_CHUNK + 1 for p in positions.tolist())
        seen_window = sum(min(p + 1, TAFISUN_CHUNK) for p in positions.tolist())
        name = f"attention_{'prefill' if new > 1 else 'decode'}_{seqs}x{length}"
        out[name] = {"chunked_ms": round(t_new, 4), "windowed_ms": round(t_old, 4),
                     "tflops": {"chunked": round(4.0 * heads * d * seen / t_new / 1e9, 1), "windowed": round(4.0 * heads * d * seen_window / t_old / 1e9, 1)}}
        if new == 1:
            moved = seqs * kv_heads * 2 * d * 2
            out[name]["of_measured_copy"] = {"chunked": frac(moved * (seen // seqs), t_new), "windowed": frac(moved * (seen_window // seqs), t_old)}
    # the router with groups, a correction, identity outputs and the shared unit's gate beside the plain router; the sums
    outputs = TAFISUN_EXPERTS + TAFISUN_IDENTITY
    router, correction = torch.randn(outputs + 1, width, device=dev), torch.randn(outputs, device=dev) * 0.1
    plain_router = torch.randn(ROPULIX_EXPERTS, width, device=dev)
    for n in (2048, 8):
        x = bf(n, width)
        wide = G.wide_tiles_pay(n, TAFISUN_TOP, x.dtype, width, ff)
        route_new = lambda: G.route(x, router, None, top=TAFISUN_TOP, wide_tiles=wide, score="softmax_all", correction=correction,
                                    groups=TAFISUN_GROUPS, keep=TAFISUN_KEEP, scale=2.0, identity=TAFISUN_IDENTITY, extra=1)
        routing = route_new()
        routing_old = G.route(x, plain_router, None, top=ROPULIX_TOP, wide_tiles=wide)
        t_route = timed(route_new, 10)
        t_route_old = timed(lambda: G.route(x, plain_router, None, top=ROPULIX_TOP, wide_tiles=wide), 10)
        rows, rows_old = torch.randn(routing.rows, width, device=dev), torch.randn(routing_old.rows, width, device=dev)
        shared = torch.randn(n, width, device=dev)
        t_sum = timed(lambda: G.combine_mixed(rows, routing, x, extra=shared, extra_scale=routing.extra), 10)
        t_sum_old = timed(lambda: G.combine(rows_old, routing_old), 10)
        gate_up = bf(routing.rows, 2 * ff)
        t_glu = timed(lambda: F.glu_limit(gate_up, 7.0, 1.702), 10)
        t_silu = timed(lambda: B.silu_mul_scaled(gate_up), 10)
        out[f"experts_{n}_tokens"] = {
            "route_and_sort_us": {"grouped": round(t_route * 1e3, 1), "plain": round(t_route_old * 1e3, 1)},
            "weighted_sum_us": {"with_identity_and_shared": round(t_sum * 1e3, 1), "plain": round(t_sum_old * 1e3, 1)},
            "weighted_sum_of_measured_copy": {"with_identity_and_shared": frac(n * width * (4 * TAFISUN_TOP + 4 + 4 + 2), t_sum),
                                              "plain": frac(n * width * (4 * ROPULIX_TOP + 4), t_sum_old)},
            "gated_unit_us": {"limited": round(t_glu * 1e3, 1), "silu": round(t_silu * 1e3, 1)},
            "gated_unit_of_measured_copy": {"limited": frac(routing.rows * ff * 6, t_glu), "silu": frac(routing.rows * ff * 6, t_silu)}}
    # the per-head norm with weights and the keys written twice, and the element-wise gate; squared relu beside SiLU * up
    n = 2048
    rows_ = bf(n, (2 * heads + kv_heads) * d)
    qw, kw = torch.ones(d, device=dev), torch.ones(d, device=dev)
    positions, entry = ints(list(range(n))), ints([0] * n)
    table_ = torch.arange(n // page, dtype=torch.int32).view(1, -1).to(dev)
    keys, values = bf(n // page, kv_heads, page, d), bf(n // page, kv_heads, page, d)
    t_norm = timed(lambda: M.head_norm_write(rows_, num_q_heads=heads, num_kv_heads=kv_heads, head_dim=d, value_dim=d, eps=1e-6, q_weight=qw,
                                             k_weight=kw, positions=positions, token_entry=entry, block_table=table_, page_size=page,
                                             k_pool=keys, v_pool=values, value_offset=heads * d), 10)
    attn = bf(n, heads * d)
    t_gate = timed(lambda: M.sigmoid_gate(attn, rows_, gate_offset=(heads + kv_heads) * d, group=1), 10)
    hidden = bf(n, 12288)
    t_relu2 = timed(lambda: F.relu2(hidden), 10)
    both = bf(n, 2 * 12288)
    t_silu = timed(lambda: F.silu_mul(both), 10)
    out["small_steps_2048_tokens"] = {
        "head_norm_write_us": round(t_norm * 1e3, 1), "head_norm_write_of_measured_copy": frac(n * d * (heads * 4 + kv_heads * 6), t_norm),
        "sigmoid_gate_us": round(t_gate * 1e3, 1), "sigmoid_gate_of_measured_copy": frac(n * heads * d * 6, t_gate),
        "relu2_us": round(t_relu2 * 1e3, 1), "relu2_of_measured_copy": frac(n * 12288 * 4, t_relu2),
        "silu_mul_us": round(t_silu * 1e3, 1), "silu_mul_of_measured_copy": frac(n * 12288 * 6, t_silu)}
    return out


def run_reference(args) -> dict:
    """The unmodified reference from baseline/_ref: its own Qwen3ForCausalLM, paged cache,
    CUDA-graph decode and BatchScheduler, driven through Engine.create_scheduler()."""

    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "mini_llm")):
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}
    sys.path.insert(0, ref)
    try:
        import torch

        from mini_llm.engine import Engine
        from mini_llm.tokenizer import ChatMessage

        cfg = dict(QWEN3_8B)
        layers = args.layers or cfg["num_hidden_layers"]
        full_layers = cfg["num_hidden_layers"]
        cfg["num_hidden_layers"] = layers
        model, device = _reference_model(cfg)
        host = torch.Generator().manual_seed(0)

        def prompt(n):
            ids = torch.randint(0, cfg["vocab_size"], (n,), generator=host).tolist()
            return [ChatMessage(role="user", content=" ".join(str(t) for t in ids))]

        def engine_for(batch):
            return Engine(model=model, tokenizer=_IdsTokenizer(), device=device, dtype=torch.bfloat16,
                          max_seq_len=cfg["max_position_embeddings"], load_seconds=0.0, max_batch_size=batch)

        def decode_rate(batch, steps, warmup):
            scheduler = engine_for(batch).create_scheduler()
            for _ in range(batch):
                scheduler.add_request(prompt(CONTEXT), max_new_tokens=1024)
            while scheduler.num_waiting:
                scheduler.step()
            for _ in range(max(warmup, 3)):
                scheduler.step()
            torch.cuda.synchronize()
            started = time.perf_counter()
            produced = 0
            for _ in range(steps):
                produced += len(scheduler.step())
            torch.cuda.synchronize()
            seconds = time.perf_counter() - started
            scheduler.abort_all()
            return produced / seconds, seconds / steps * 1e3

        def prefill_ms():
            times = []
            for _ in range(max(args.warmup, 3) + 5):
                scheduler = engine_for(1).create_scheduler()
                scheduler.add_request(prompt(PREFILL_TOKENS), max_new_tokens=1)
                torch.cuda.synchronize()
                started = time.perf_counter()
                scheduler.step()
                torch.cuda.synchronize()
                times.append((time.perf_counter() - started) * 1e3)
                scheduler.abort_all()
            return statistics.median(times[-5:])

        pre = prefill_ms()
        clocks = ClockSampler()
        rate8, ms8 = decode_rate(args.batch, args.steps, args.warmup)
        clock_info = clocks.stop()
        rate1, _ = decode_rate(1, args.steps, args.warmup)
        rate64, _ = decode_rate(64, args.steps, args.warmup)
        pk = peaks()
        step_bytes = model_bytes(cfg, layers) + args.batch * CONTEXT * kv_bytes_per_token(cfg, layers)
        achieved = step_bytes / (ms8 * 1e-3) / 1e9
        flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
        return {
            "metric": "decode tok/s at batch 8 (2,048 cached tokens each), Qwen3-8B shape", "impl": "reference",
            "value": round(rate8, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids",
            "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": full_layers, "global_batch": args.batch,
                       "seq_len": CONTEXT, "context_limit": cfg["max_position_embeddings"], "page_size": 16,
                       "parallelism": "none (1 GPU)", "cuda_graph": True,
                       "timing": "wall clock around BatchScheduler.step, synchronised", "peaks": pk["source"]},
            "e2e": {"value": round(rate8, 1), "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 8 * 2,
                    "d2h_bytes_per_step": args.batch * 8},
            "gpu_launches": 0,
            "prefill": {"value": round(PREFILL_TOKENS / (pre * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre, 3),
                        "frac": round(flops / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
            "points": {"decode_b1": round(rate1, 1), "decode_b64": round(rate64, 1)},
            "clocks": clock_info,
        }
    except Exception as exc:  # the reference or one of its dependencies does not run here
        reason = f"{type(exc).__name__}: {exc}".splitlines()[0][:300]
        return {"impl": "reference", "unavailable": reason}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=0, help="with --only decode: cached tokens per request (default 2048)")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in config)")
    parser.add_argument("--workload", choices=("default", "staggered14b", "decode32b", "sorulix", "ropulix", "mabedra", "tafisun"), default="default",
                        help="default: Qwen3-8B decode/prefill; staggered14b, decode32b: the larger configurations (either --impl); "
                             "sorulix: the Sorulix design beside Qwen3 at equal sizes, and its kernels alone; "
                             "ropulix: the Ropulix design beside Sorulix and Qwen3 at equal sizes, and its kernels alone; "
                             "mabedra: the Mabedra design beside Qwen3 and Ropulix at equal sizes, and its kernels alone; "
                             "tafisun: the Tafisun design beside Ropulix and Qwen3 at equal sizes, and its kernels alone")
    parser.add_argument("--size", default="", help="with --workload sorulix, ropulix, mabedra or tafisun: sizes to run, with commas (2k, 4k; default both)")
    parser.add_argument("--only", choices=("all", "decode", "prefill", "kernels", "models"), default="all",
                        help="run only the decode steps or only the prefill (for profiler captures of a small case); "
                             "with --workload sorulix: only the kernels alone, or only the whole models")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU: --gpus {args.gpus} is not supported by this engine (single-GPU tier)")
        return 2
    if args.workload == "staggered14b":
        result = run_staggered_14b(args)
    elif args.workload == "decode32b":
        result = run_decode_32b(args)
    elif args.workload == "sorulix":
        if args.impl == "reference":
            result = _unavailable("the reference has no model of this design")
        else:
            result = run_sorulix(args)
    elif args.workload == "ropulix":
        if args.impl == "reference":
            result = _unavailable("the reference has no model of this design")
        else:
            result = run_ropulix(args)
    elif args.workload == "mabedra":
        if args.impl == "reference":
            result = _unavailable("the reference has no model of this design")
        else:
            result = run_mabedra(args)
    elif args.workload == "tafisun":
        if args.impl == "reference":
            result = _unavailable("the reference has no model of this design")
        else:
            result = run_tafisun(args)
    else:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
