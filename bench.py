"""Decode and prefill throughput of the engine at Qwen2.5-7B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line is printed.  A "step" is one decode step of the whole batch (forward,
sampling, the sampled tokens back on the host).  `value` is decoded tokens per second
at batch 8 and a context of 1,024 tokens, timed with CUDA events around exactly K
steps; `e2e` is the same measured through `LLMEngine.step()`, host token ids in and
out; `prefill` is one 2,048-token prompt in one step; `roofline` relates the bytes a
decode step must read (every weight once, the cache of the live requests) to its time;
`points` holds decoding at batch 1 and 64; `mixed` the scheduler end to end (64 requests of mixed
lengths at Qwen2.5-1.5B widths, `--workload mixed` alone).  Weights are random (seeded), token ids
uniform random: no checkpoint and no dataset is read.  Peaks come from
MEASURED_PEAKS.json beside this file when present, else from an earlier measurement
on the same GPU pool.  `--shape 14b --context 8192` (and the like) time the same
workload at other layer sizes and context lengths; the default line is the 7B one.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

def _shapes() -> dict:
    """The layer sizes of the Qwen2.5 dense family, read from the package's shape files; the
    larger ones run with --layers (or in --case timeline)."""
    from shrike_b200.shapes import shape_config

    return {key: (f"Qwen2.5-{key.upper()} shape", shape_config(f"qwen2.5-{key}"))
            for key in ("0.5b", "1.5b", "3b", "7b", "14b", "32b", "72b")}


SHAPES = _shapes()
MODEL_7B = SHAPES["7b"][1]
MODEL_1_5B = SHAPES["1.5b"][1]
DEVICE_BYTES_LIMIT = 120e9   # weights and cache pool together stay under this, whatever the options
CONTEXT = 1024
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
                elif isinstance(node, list):
                    for item in node:
                        walk(item)

            walk(raw)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat["source"] = "measured"
                return flat
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return

        def read():
            for line in self.process.stdout:
                self.samples.append((time.perf_counter(), line.strip()))

        self.thread = threading.Thread(target=read, daemon=True)
        self.thread.start()

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self, windows) -> dict:
        clocks, max_clock, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for stamp, line in self.samples:
            if not any(lo <= stamp <= hi for lo, hi in windows):
                continue
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 6:
                continue
            try:
                clocks.append(int(fields[0]))
                max_clock = max(max_clock, int(fields[1]))
            except ValueError:
                continue
            for name, flag in zip(names, fields[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None, "sm_max_mhz": max_clock or None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(raw: dict, layers: int) -> dict:
    h, inter, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    heads, kv, d = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    matrices = h * (heads + 2 * kv) * d + heads * d * h + 3 * h * inter
    vectors = (heads + 2 * kv) * d + 2 * h
    return dict(
        layer_matrix_params=matrices, layer_params=matrices + vectors, head_params=v * h,
        kv_bytes_per_token=layers * 2 * kv * d * 2,
        weight_bytes_per_step=2 * (layers * (matrices + vectors) + v * h + h),
    )


def decode_bytes(numbers: dict, batch: int, context: float) -> float:
    return numbers["weight_bytes_per_step"] + batch * context * numbers["kv_bytes_per_token"]


def prefill_flops(raw: dict, layers: int, tokens: int) -> float:
    numbers = model_numbers(raw, layers)
    heads, d = raw["num_attention_heads"], raw["head_dim"]
    linear = 2.0 * tokens * layers * numbers["layer_matrix_params"]
    attention = layers * 4.0 * heads * d * (tokens * (tokens + 1) / 2)
    head = 2.0 * raw["vocab_size"] * raw["hidden_size"]
    return linear + attention + head


def run_ours(args) -> dict:
    import numpy as np
    import torch

    import shrike_b200.models  # noqa: F401
    from shrike_b200 import SamplingParams
    from shrike_b200.config import parse_config
    from shrike_b200.engine.batch import StepEntry
    from shrike_b200.engine.llm_engine import LLMEngine
    from shrike_b200.weights.random_init import random_tensors

    torch.cuda.set_device(0)
    device = torch.device("cuda:0")
    shape_name, shape = SHAPES[args.shape]
    raw = dict(shape)
    context = args.context
    full_layers = raw["num_hidden_layers"]
    raw["num_hidden_layers"] = args.layers or full_layers
    layers = raw["num_hidden_layers"]
    config = parse_config(raw)
    numbers = model_numbers(raw, layers)
    if numbers["weight_bytes_per_step"] > 0.8 * DEVICE_BYTES_LIMIT:
        raise SystemExit(f"{shape_name} with {layers} layers holds {numbers['weight_bytes_per_step'] / 1e9:.0f} GB "
                         "of weights: give --layers")
    tensors = random_tensors(config, seed=0, device=device, dtype=torch.bfloat16)
    budget = 4096   # the engine's tokens per step: long prompts are cut, and finish their prefill steps apart
    spread = args.batch * -(-context // budget)   # steps from the first request's first token to the last one's
    pages_per_request = -(-(context + args.steps + args.warmup + 8 + spread) // BLOCK_SIZE)
    page_bytes = BLOCK_SIZE * numbers["kv_bytes_per_token"]
    large = 64   # the large batch of `points`: 64, or what the memory limit leaves at this shape and context
    while large > 1 and numbers["weight_bytes_per_step"] + large * pages_per_request * page_bytes > DEVICE_BYTES_LIMIT:
        large //= 2
    if args.batch > large:
        raise SystemExit(f"--batch {args.batch} at --context {context} needs more than {DEVICE_BYTES_LIMIT / 1e9:.0f} GB")
    pages = large * pages_per_request + -(-PREFILL_TOKENS // BLOCK_SIZE) + 64
    engine = LLMEngine(None, block_size=BLOCK_SIZE, num_blocks=pages, max_tokens_per_step=budget, max_running=64,
                       dtype="bfloat16", config=config, tensors=tensors)
    del tensors
    runner, ops = engine.runner, engine.ops
    rng = np.random.default_rng(0)
    vocab = raw["vocab_size"]
    peaks = load_peaks()
    sampler = ClockSampler()
    sampler.start()
    windows = []

    def fill(batch: int):
        """`batch` requests with context - 1 tokens in the cache (untimed)."""
        caches = []
        for _ in range(batch):
            cache = runner.cache.open()
            ids = rng.integers(0, vocab, context - 1).tolist()
            runner.cache.append(cache, 0, len(ids))
            runner.step([StepEntry(cache, ids, 0, [])])
            caches.append(cache)
        torch.cuda.synchronize()
        return caches

    def decode_run(batch: int, steps: int, warmup: int):
        """Device-timed decode through the step function and the sampling kernel."""
        caches = fill(batch)
        tokens = rng.integers(0, vocab, batch).tolist()
        fed = context - 1
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def launch(fed, tokens=None):
            """Launches the step that feeds position `fed`.  Without tokens the step takes them on
            the device from what the step before it draws (id -1 - row), as the engine does in
            steady decoding: the host has not seen them yet."""
            entries = []
            for index, cache in enumerate(caches):
                runner.cache.append(cache, fed, 1)
                entries.append(StepEntry(cache, [tokens[index] if tokens else -1 - index], fed, [0], (0.0, 1.0, 0)))
            _logits, drawn = runner.step(entries, sample=True)
            return runner.fetch(drawn)

        def run(count, in_flight, fed):
            """`count` steps, one launched and one read back per round; the device never waits."""
            for _ in range(count):
                fed += 1
                following = launch(fed)
                runner.wait(in_flight)          # this step's tokens reach the host
                in_flight = following
            return in_flight, fed

        in_flight, fed = run(warmup - 1, launch(fed, tokens), fed)
        tokens = runner.wait(in_flight)
        torch.cuda.synchronize()
        launches_before = ops.launches
        t0 = time.perf_counter()
        start.record()
        fed += 1
        in_flight, fed = run(steps - 1, launch(fed, tokens), fed)   # `steps` launches ...
        runner.wait(in_flight)                                       # ... and `steps` read-backs
        stop.record()
        torch.cuda.synchronize()
        windows.append((t0, time.perf_counter()))
        ms = start.elapsed_time(stop) / steps
        launches = ops.launches - launches_before
        for cache in caches:
            runner.cache.free(cache)
        mean_context = context + warmup + (steps - 1) / 2.0
        return ms, launches, mean_context

    # ---- decode at the headline batch, device-timed -------------------------
    ms, launches, mean_context = decode_run(args.batch, args.steps, args.warmup)
    value = args.batch * 1000.0 / ms
    bytes_step = decode_bytes(numbers, args.batch, mean_context)
    achieved = bytes_step / (ms * 1e-3) / 1e9

    # ---- the same through the public entry point ------------------------------
    def e2e_run(batch: int, steps: int, warmup: int):
        prompts = [rng.integers(0, vocab, context - 1).tolist() for _ in range(batch)]
        # every request decodes through all timed steps, although the prompts finish their prefill steps apart
        params = SamplingParams(max_new_tokens=steps + warmup + 8 + spread, ignore_eos=True)
        for prompt in prompts:
            engine.add_request(prompt, params)
        while any(not r.prefill_done for r in engine.requests.values()) or engine.scheduler.waiting:
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        copied = runner.builder.copied_bytes
        t0 = time.perf_counter()
        start.record()
        produced = 0
        for _ in range(steps):
            produced += len(engine.step())
        stop.record()
        torch.cuda.synchronize()
        windows.append((t0, time.perf_counter()))
        e2e_ms = start.elapsed_time(stop) / steps
        for req_id in list(engine.requests):
            engine.abort(req_id)
        assert engine.block_manager.whole()
        h2d = (runner.builder.copied_bytes - copied) // steps   # the packed metadata block of each step
        return produced / steps * 1000.0 / e2e_ms, h2d, 4 * batch

    e2e_value, h2d, d2h = e2e_run(args.batch, args.steps, args.warmup)

    # ---- prefill of 2,048 tokens in one step ----------------------------------
    def prefill_run(repeats: int, warmup: int):
        times = []
        for index in range(warmup + repeats):
            cache = runner.cache.open()
            ids = rng.integers(0, vocab, PREFILL_TOKENS).tolist()
            runner.cache.append(cache, 0, PREFILL_TOKENS)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            logits = runner.step([StepEntry(cache, ids, 0, [PREFILL_TOKENS - 1])])
            stop.record()
            torch.cuda.synchronize()
            if index >= warmup:
                times.append(start.elapsed_time(stop))
                windows.append((t0, time.perf_counter()))
            runner.cache.free(cache)
        return statistics.median(times)

    # the step function replays a batch shape as a CUDA graph once it has come a few times (a long
    # prompt cut into equal portions does that; a benchmark's repeats too).  Both figures are given:
    # the first sightings, launched kernel by kernel, and the replayed sequence.
    use_graphs = runner.use_graphs
    runner.use_graphs = False
    prefill_uncaptured_ms = prefill_run(5, 3)
    runner.use_graphs = use_graphs
    prefill_ms = prefill_run(5, 6)   # warm-up long enough for the step's launch sequence to be captured
    flops = prefill_flops(raw, layers, PREFILL_TOKENS)
    peak_flops = peaks["bf16_tflops"] * 1e12

    def prefill_through_engine(budget: int, repeats: int, warmup: int):
        """One 2,048-token prompt through `LLMEngine.step()` under a token budget (four portions at
        the stock 512), host token ids in, the first generated token out: wall clock around it,
        as the reference arm's prefill figure is taken."""
        stock = engine.scheduler.max_tokens_per_step
        engine.scheduler.max_tokens_per_step = budget
        times, steps_taken = [], 0
        try:
            for index in range(warmup + repeats):
                prompt = rng.integers(0, vocab, PREFILL_TOKENS).tolist()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                engine.add_request(prompt, SamplingParams(max_new_tokens=1, ignore_eos=True))
                steps_taken = 0
                while engine.has_work:
                    engine.step()
                    steps_taken += 1
                torch.cuda.synchronize()
                t1 = time.perf_counter()
                if index >= warmup:
                    times.append((t1 - t0) * 1000.0)
                    windows.append((t0, t1))
        finally:
            engine.scheduler.max_tokens_per_step = stock
        return statistics.median(times), steps_taken

    budget512_ms, budget512_steps = prefill_through_engine(512, 5, 3)

    points = {}
    for batch in (1, large):
        point_ms, _, _ = decode_run(batch, max(10, args.steps // 2), 3)
        points[f"decode_b{batch}"] = round(batch * 1000.0 / point_ms, 1)

    kernels = dominant_kernels(ops, raw, args.batch, peaks, context) if not args.layers else {}
    sampler.stop()
    clocks = sampler.summary(windows)
    return {
        "metric": f"decode_tokens_per_second_qwen2.5-{args.shape}_b{args.batch}_ctx{context}",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "impl": "ours",
        "config": {
            "model": shape_name, "layers": layers, "layers_full": full_layers, "hidden": raw["hidden_size"],
            "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
            "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "global_batch": args.batch,
            "seq_len": context, "block_size": BLOCK_SIZE, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single_gpu", "l2": f"inputs larger than L2 (weights read per step: {numbers['weight_bytes_per_step'] / 1e9:.1f} GB)",
            "peaks": peaks["source"],
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms * 1e-3) / peak_flops, 4),
                    "uncaptured_ms": round(prefill_uncaptured_ms, 3),
                    "uncaptured_frac": round(flops / (prefill_uncaptured_ms * 1e-3) / peak_flops, 4),
                    "budget512": {"value": round(PREFILL_TOKENS * 1000.0 / budget512_ms, 1), "ms": round(budget512_ms, 3),
                                  "steps": budget512_steps,
                                  "note": "through LLMEngine.step() with a 512-token budget, wall clock"}},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernels,
        "clocks": clocks,
    }


def dominant_kernels(ops, raw: dict, batch: int, peaks: dict, context: int = 0) -> dict:
    """Each dominant decode kernel at the headline batch, as a stream of back-to-back launches
    over rotated operands (so every launch reads HBM) in one captured graph: the time the
    stream takes divided by its launches, and the bandwidth that is.  Under programmatic
    dependent launch a launch streams its weights while the one before it drains, so this is
    the rate the kernel sustains in a chain, not the duration of one launch alone (those are
    in profiles/, from ncu: longer, since a lone launch has nothing to overlap with)."""
    import torch

    dev = "cuda"
    h, inter, vocab = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    heads, kv, d = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]

    def graph_us(fn, reps):
        fn(0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(5):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / (5 * reps)

    out = {}
    shapes = {"qkv": ((heads + 2 * kv) * d, h, 8), "o": (h, heads * d, 8), "gate_up": (2 * inter, h, 4),
              "down": (h, inter, 4), "lm_head": (vocab, h, 2)}
    for name, (n, k, copies) in shapes.items():
        weights = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
        x = torch.randn(batch, k, device=dev, dtype=torch.bfloat16)
        result = torch.empty(batch, n, device=dev, dtype=torch.bfloat16 if name == "gate_up" else torch.float32)
        partial = name in ("qkv", "o", "down")
        us = graph_us(lambda i: ops.linear(x, weights[i % copies], result, allow_partials=partial), 2 * copies)
        gbs = n * k * 2 / us / 1e3
        out[name] = {"us": round(us, 1), "GBps": round(gbs, 0), "frac": round(gbs / peaks["hbm_gbs"], 3)}
        del weights
    context = context or CONTEXT
    blocks = -(-context // BLOCK_SIZE)
    sets = 4   # rotated key/value pools, so that a launch does not find its keys in L2
    pools = [(torch.randn(batch * blocks, BLOCK_SIZE, kv, d, device=dev, dtype=torch.bfloat16),
              torch.randn(batch * blocks, BLOCK_SIZE, kv, d, device=dev, dtype=torch.bfloat16)) for _ in range(sets)]
    q = torch.randn(batch, heads * d, device=dev, dtype=torch.bfloat16)
    width = max(8, 1 << (blocks - 1).bit_length())
    table = torch.full((batch, width), -1, dtype=torch.int32, device=dev)
    table[:, :blocks] = torch.arange(batch * blocks, dtype=torch.int32, device=dev).view(batch, blocks)
    q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    ctx = torch.full((batch,), context, dtype=torch.int32, device=dev)
    seq_of = torch.arange(batch, dtype=torch.int32, device=dev)
    attn = torch.empty_like(q)
    us = graph_us(lambda i: ops.paged_attention(q, pools[i % sets][0], pools[i % sets][1], table, q_start, ctx, seq_of,
                                                heads, kv, d, d ** -0.5, None, attn, max_q_len=1, min_q_len=1), 2 * sets)
    gbs = batch * context * 2 * kv * d * 2 / us / 1e3
    out["attention"] = {"us": round(us, 1), "GBps": round(gbs, 0), "frac": round(gbs / peaks["hbm_gbs"], 3)}
    out["note"] = "back-to-back launches in one graph, time per launch of the stream (launches overlap): a sustained rate, not one kernel's duration"
    return out


def run_mixed(args) -> dict:
    """The scheduler end to end at Qwen2.5-1.5B shape: 64 requests, random-id prompts of 32 to
    2,048 tokens, 32 to 256 output tokens each (lengths drawn as shrike's bench/workload.py:15-22
    does, `random.Random(20260718).randint`), greedy, fixed lengths, chunked-prefill budget 512,
    through `LLMEngine.generate`.  Wall-clock, as shrike's bench/bench_engine.py:54-62 measures."""
    import random

    import torch

    import shrike_b200.models  # noqa: F401
    from shrike_b200 import SamplingParams
    from shrike_b200.config import parse_config
    from shrike_b200.engine.llm_engine import LLMEngine
    from shrike_b200.weights.random_init import random_tensors

    torch.cuda.set_device(0)
    raw = dict(MODEL_1_5B)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    config = parse_config(raw)
    tensors = random_tensors(config, seed=0, device="cuda", dtype=torch.bfloat16)
    engine = LLMEngine(None, block_size=BLOCK_SIZE, num_blocks=args.num_blocks or 12000, max_tokens_per_step=512,
                       max_running=256, dtype="bfloat16", config=config, tensors=tensors)
    del tensors
    rng = random.Random(20260718)
    outputs = [rng.randint(32, 256) for _ in range(64)]
    prompts = [[rng.randrange(raw["vocab_size"]) for _ in range(rng.randint(32, 2048))] for _ in range(64)]
    params = [SamplingParams(max_new_tokens=n, temperature=0.0, ignore_eos=True) for n in outputs]
    engine.generate(prompts[:4], params[:4])   # warm-up: builds, graphs for small batches
    torch.cuda.synchronize()
    steps_before = engine.stats.steps
    began = time.perf_counter()
    results = engine.generate(prompts, params)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    engine.ops.check_status()
    generated = sum(len(r) for r in results)
    assert [len(r) for r in results] == outputs and engine.block_manager.whole()
    return {
        "workload": "mixed", "model": "Qwen2.5-1.5B shape", "layers": raw["num_hidden_layers"], "requests": 64,
        "prompt_tokens": sum(len(p) for p in prompts), "generated_tokens": generated, "seconds": round(seconds, 3),
        "value": round(generated / seconds, 1), "unit": "generated tok/s",
        "total_tokens_per_second": round((generated + sum(len(p) for p in prompts)) / seconds, 1),
        "steps": engine.stats.steps - steps_before, "preemptions": engine.scheduler.num_preemptions,
        "kv_blocks": engine.block_manager.total_pages, "budget": 512, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform random token ids",
    }


def run_case(args) -> dict:
    """A small, fixed workload around one kernel, a few launches long: what the ncu captures
    under profiles/ are taken on.  Inputs are larger than L2 where the kernel streams."""
    import torch

    from shrike_b200.ops.cuda_ops import CudaOps

    torch.cuda.set_device(0)
    dev = "cuda"
    ops = CudaOps(torch.bfloat16, dev)
    raw = MODEL_7B
    h, inter = raw["hidden_size"], raw["intermediate_size"]
    heads, kv, d = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    tokens = args.batch
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    filler = []

    def keep_busy():
        """The device is kept busy (about 0.2 ms) while the host prepares the timed launch (plan, tensor
        maps: about 25 us), so that the events bracket the kernel and not the host's work before it."""
        if hasattr(torch.cuda, "_sleep"):
            torch.cuda._sleep(400_000)
        else:
            if not filler:
                filler.append(torch.empty(1 << 30, dtype=torch.uint8, device=dev))
            filler[0].zero_()
    if args.case.startswith("gemm_"):
        shapes = {"gemm_gate_up": (2 * inter, h), "gemm_down": (h, inter), "gemm_qkv": ((heads + 2 * kv) * d, h)}
        n, k = shapes[args.case]
        weights = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) for _ in range(3)]   # rotated: every call reads HBM
        x = torch.randn(tokens, k, device=dev, dtype=torch.bfloat16)
        out = torch.empty(tokens, n, device=dev, dtype=torch.bfloat16 if args.case == "gemm_gate_up" else torch.float32)
        for i in range(6):
            keep_busy()
            start.record()
            ops.linear(x, weights[i % 3], out, allow_partials=args.case != "gemm_gate_up")
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3)
        work = {"bytes": n * k * 2}
    elif args.case in ("attention_single", "attention_portions"):
        single = args.case == "attention_single"
        seqs = tokens if single else 1
        ctx_len = CONTEXT if single else args.prefill_tokens
        q_len = 1 if single else args.prefill_tokens
        blocks = -(-ctx_len // BLOCK_SIZE)
        pages = seqs * blocks + 8
        keys = torch.randn(pages, BLOCK_SIZE, kv, d, device=dev, dtype=torch.bfloat16)
        values = torch.randn_like(keys)
        q = torch.randn(seqs * q_len, heads * d, device=dev, dtype=torch.bfloat16)
        width = max(8, 1 << (blocks - 1).bit_length())
        table = torch.full((seqs, width), -1, dtype=torch.int32, device=dev)
        table[:, :blocks] = torch.arange(seqs * blocks, dtype=torch.int32, device=dev).view(seqs, blocks)
        q_start = torch.arange(seqs + 1, dtype=torch.int32, device=dev) * q_len
        ctx = torch.full((seqs,), ctx_len, dtype=torch.int32, device=dev)
        seq_of = torch.arange(seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len)
        out = torch.empty_like(q)
        for _ in range(6):
            keep_busy()
            start.record()
            ops.paged_attention(q, keys, values, table, q_start, ctx, seq_of, heads, kv, d, d ** -0.5, None, out,
                                max_q_len=q_len, min_q_len=q_len, q_lens=[q_len] * seqs)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3)
        work = {"bytes": seqs * ctx_len * 2 * kv * d * 2} if single else {"flops": 4.0 * heads * d * q_len * (q_len + 1) / 2}
    else:
        raise SystemExit(f"unknown case {args.case!r}")
    ops.check_status()
    best = min(times[2:])
    result = {"case": args.case, "tokens_or_sequences": tokens, "us": round(best, 2), "launch_times_us": [round(t, 1) for t in times]}
    if "bytes" in work:
        result["GBps"] = round(work["bytes"] / best / 1e3, 1)
    else:
        result["TFLOPs"] = round(work["flops"] / best / 1e6, 1)
    return result


def run_timeline(args) -> dict:
    """Where a captured decode step spends its time, kernel by kernel: start and end of every
    kernel of one step from CUPTI activity records (torch.profiler), on a model of the
    benchmark's widths with few layers.  Kernels overlap (each starts while the one before it
    runs), so the figure per kernel is `end - end of the kernel before it`: what the step
    would save if that kernel vanished from the chain.  Medians over the layers."""
    import numpy as np
    import torch
    from torch.profiler import ProfilerActivity, profile

    import shrike_b200.models  # noqa: F401
    from shrike_b200.config import parse_config
    from shrike_b200.engine.batch import StepEntry
    from shrike_b200.engine.llm_engine import LLMEngine
    from shrike_b200.weights.random_init import random_tensors

    torch.cuda.set_device(0)
    raw = dict(SHAPES[args.shape][1])
    context = args.context
    raw["num_hidden_layers"] = layers = args.layers or 6
    config = parse_config(raw)
    tensors = random_tensors(config, seed=0, device=torch.device("cuda:0"), dtype=torch.bfloat16)
    pages = args.batch * (-(-(context + 64) // BLOCK_SIZE)) + 64
    engine = LLMEngine(None, block_size=BLOCK_SIZE, num_blocks=pages, max_tokens_per_step=4096, max_running=64,
                       dtype="bfloat16", config=config, tensors=tensors)
    del tensors
    runner = engine.runner
    rng = np.random.default_rng(0)
    caches = []
    for _ in range(args.batch):
        cache = runner.cache.open()
        ids = rng.integers(0, raw["vocab_size"], context - 1).tolist()
        runner.cache.append(cache, 0, len(ids))
        runner.step([StepEntry(cache, ids, 0, [])])
        caches.append(cache)
    fed = [context - 1]

    def one_step():
        entries = []
        for cache in caches:
            runner.cache.append(cache, fed[0], 1)
            entries.append(StepEntry(cache, [5], fed[0], [0], (0.0, 1.0, 0)))
        _logits, drawn = runner.step(entries, sample=True)
        fed[0] += 1
        return drawn.tolist()

    for _ in range(6):
        one_step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            one_step()
        torch.cuda.synchronize()
    kernels = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in e.name),
                     key=lambda e: e.time_range.start)
    per_step = len(kernels) // 3
    step = kernels[-per_step:]
    rows, previous_end = [], step[0].time_range.start
    for event in step:
        rows.append((event.name.split("(")[0].split("<")[0].split("::")[-1], event.time_range.end - previous_end))
        previous_end = event.time_range.end
    norms = [i for i, (name, _) in enumerate(rows) if "add_rmsnorm" in name]
    first, per_layer = norms[0], norms[2] - norms[0]   # two norms a layer
    products = iter(["qkv product", "o product", "gate_up product", "down product"])
    seen_norms = 0
    labels = []
    for name, _ in rows[first + per_layer: first + 2 * per_layer]:
        if "add_rmsnorm" in name:
            labels.append("norm (feed-forward)" if seen_norms else "norm (mixer)")
            seen_norms += 1
        elif "gemm" in name or "nvjet" in name or "cutlass" in name:
            labels.append(next(products, "product"))
        elif "rope" in name:
            labels.append("rotary + cache store")
        elif "single_token" in name or "portions" in name or "attention" in name:
            labels.append("attention")
        elif "silu" in name:
            labels.append("SiLU product")
        else:
            labels.append(name)
    if "SiLU product" not in labels:
        labels = [label + " with SiLU" if label == "gate_up product" else label for label in labels]
    table = []
    for position in range(per_layer):
        samples = [rows[first + layer * per_layer + position] for layer in range(1, layers)]   # the first layer follows the embedding
        table.append({"kernel": labels[position], "name": samples[0][0], "in_situ_us": round(float(np.median([t for _, t in samples])), 2)})
    layer_us = round(sum(row["in_situ_us"] for row in table), 2)
    rest = rows[:first] + rows[first + layers * per_layer:]
    return {"case": "timeline", "shape": args.shape, "context": context, "batch": args.batch, "layers": layers, "layer_us": layer_us, "per_layer": table,
            "outside_layers": [{"name": name, "in_situ_us": round(t, 2)} for name, t in rest],
            "step_us": round(step[-1].time_range.end - step[0].time_range.start, 1)}


def run_reference(args) -> dict:
    reference = ROOT / "baseline" / "_ref"
    if not (reference / "shrike").is_dir():
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}
    from baseline.reference_arm import run, run_mixed  # the unmodified reference through its own LLMEngine

    if args.workload == "mixed":
        return run_mixed(args, MODEL_1_5B)
    return run(args, SHAPES[args.shape][1], args.context)


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    parser.add_argument("--shape", default="7b", choices=list(SHAPES), help="layer sizes of the decode workload")
    parser.add_argument("--context", type=int, default=1024, help="tokens each sequence holds when decoding is timed")
    parser.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                        help="decode: the headline line; mixed: 64 requests through the scheduler at 1.5B shape")
    parser.add_argument("--num-blocks", type=int, default=0, help="cache pages for --workload mixed (few pages force preemption)")
    parser.add_argument("--skip-mixed", action="store_true", help="leave the mixed workload out of the default line")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="prompt length of --case attention_portions")
    parser.add_argument("--case", default=None,
                        help="run a small single-kernel workload instead (for profiling): gemm_gate_up, gemm_down, "
                             "gemm_qkv, attention_single, attention_portions; --batch gives tokens / sequences.  timeline: per-kernel "
                             "times inside one captured decode step (--layers, default 6)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine runs on a single B200 (asked for {args.gpus})")
        sys.exit(2)
    args.warmup = max(3, args.warmup)
    if args.case == "timeline":
        print(json.dumps(run_timeline(args)))
        return
    if args.case:
        print(json.dumps(run_case(args)))
        return
    if args.workload == "mixed" and args.impl != "reference":
        print(json.dumps(run_mixed(args)))
        return
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    if args.impl != "reference" and args.shape == "7b" and not args.layers and not args.skip_mixed:
        # the scheduler end to end, beside the headline: 64 requests of mixed lengths at 1.5B widths
        import gc

        import torch

        gc.collect()
        torch.cuda.empty_cache()
        mixed_args = argparse.Namespace(**vars(args))
        mixed_args.layers, mixed_args.num_blocks = 0, 0
        mixed = run_mixed(mixed_args)
        result["mixed"] = {key: mixed[key] for key in ("value", "unit", "seconds", "steps", "requests", "model", "budget", "preemptions")}
    print(json.dumps(result))


if __name__ == "__main__":
    main()
