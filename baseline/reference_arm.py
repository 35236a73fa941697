"""The reference arm of bench.py: Azimml/shrike, unmodified, from baseline/_ref.

It drives the reference through its own public API (`LLMEngine(model_dir)`,
`add_request(token ids, SamplingParams)`, `step()`), with the constructor's stock
defaults, on the same metric and shape as bench.py's own arm: decode tokens per second
at batch 8 with 1,024 tokens of context, Qwen2.5-7B sizes, random weights.  None of this
package's models, kernels or engine is on that path; this package is used only to write
the random-weights model folder (config.json, sharded safetensors) the reference loads,
and a minimal tokenizer file, because the reference's engine opens a tokenizer on start.
"""

from __future__ import annotations

import json
import shutil
import statistics
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def write_model_folder(folder: Path, raw: dict) -> None:
    """config.json, one safetensors shard per layer (made on the GPU, seeded), tokenizer files."""
    import torch

    sys.path.insert(0, str(ROOT))
    from shrike_b200.config import parse_config
    from shrike_b200.weights.expected import expected_tensors
    from shrike_b200.weights.random_init import random_tensor
    from shrike_b200.weights.safetensors_io import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw))
    config = parse_config(raw)
    shards: dict[str, dict] = {}
    for name, spec in expected_tensors(config).items():
        parts = name.split(".")
        shard = f"layer{int(parts[2]):03d}" if parts[1] == "layers" else name.replace(".", "_")
        shards.setdefault(shard, {})[name] = spec
    for shard, specs in shards.items():
        tensors = {name: random_tensor(name, spec, 0, "cuda", torch.bfloat16).cpu() for name, spec in specs.items()}
        write_safetensors(folder / f"{shard}.safetensors", tensors)
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    tokenizer = Tokenizer(WordLevel({"<unk>": 0, "a": 1, "b": 2}, unk_token="<unk>"))
    tokenizer.pre_tokenizer = Whitespace()
    tokenizer.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "model_max_length": 32768}))


def run(args, raw_model: dict, context: int) -> dict:
    import numpy as np
    import torch

    sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    try:
        from shrike.engine.engine import LLMEngine
        from shrike.engine.request import SamplingParams
    except Exception as error:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"baseline/_ref does not import: {type(error).__name__}: {error}"[:300]}

    raw = dict(raw_model)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    work = Path(tempfile.mkdtemp(prefix="shrike_reference_"))
    try:
        write_model_folder(work, raw)
        torch.cuda.empty_cache()
        engine = LLMEngine(str(work))
        rng = np.random.default_rng(0)
        vocab = raw["vocab_size"]
        batch, steps, warmup = args.batch, args.steps, max(3, args.warmup)
        params = SamplingParams(max_new_tokens=steps + warmup + 4, temperature=0.0, ignore_eos=True)
        for _ in range(batch):
            engine.add_request(rng.integers(0, vocab, context - 1).tolist(), params, chat=False)
        while any(not request.prefill_done for request in engine.requests.values()) or engine.scheduler.waiting:
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        produced = 0
        for _ in range(steps):
            produced += len(engine.step())
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        value = produced / steps * 1000.0 / ms
        for request in list(engine.requests.values()):
            engine.scheduler.finish(request, "aborted")
        engine.requests.clear()

        times = []
        for _ in range(3):
            prompt = rng.integers(0, vocab, 2048).tolist()   # a new prompt each time: no prefix-cache hit
            torch.cuda.synchronize()
            began = time.perf_counter()
            engine.add_request(prompt, SamplingParams(max_new_tokens=1, ignore_eos=True), chat=False)
            while engine.has_work:
                engine.step()
            torch.cuda.synchronize()
            times.append((time.perf_counter() - began) * 1000.0)
        prefill_ms = statistics.median(times)
        # the same `config` keys and values as the other arm prints for the same options
        sys.path.insert(0, str(ROOT))
        import bench

        weight_gb = bench.model_numbers(raw, raw["num_hidden_layers"])["weight_bytes_per_step"] / 1e9
        peaks_source = bench.load_peaks()["source"]
        return {
            "metric": f"decode_tokens_per_second_qwen2.5-{getattr(args, 'shape', '7b')}_b{batch}_ctx{context}",
            "impl": "reference",
            "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
            "config": {"model": f"Qwen2.5-{getattr(args, 'shape', '7b').upper()} shape", "layers": raw["num_hidden_layers"],
                       "layers_full": raw_model["num_hidden_layers"], "hidden": raw["hidden_size"],
                       "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                       "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
                       "global_batch": batch, "seq_len": context, "block_size": 16, "prefill_tokens": 2048,
                       "parallelism": "single_gpu",
                       "l2": f"inputs larger than L2 (weights read per step: {weight_gb:.1f} GB)", "peaks": peaks_source},
            "e2e": {"value": round(value, 1), "unit": "tok/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
            "prefill": {"value": round(2048 * 1000.0 / prefill_ms, 1), "tokens": 2048, "ms": round(prefill_ms, 3),
                        "note": "through step() with the stock 512-token budget (four portions)"},
            "gpu_launches": None,
        }
    finally:
        shutil.rmtree(work, ignore_errors=True)


def run_mixed(args, raw_model: dict) -> dict:
    """The reference's own offline benchmark shape (bench/bench_engine.py: 64 requests through
    `LLMEngine.generate`, lengths drawn as bench/workload.py:15-22 draws them) on the prompts and
    output lengths of bench.py's `--workload mixed`, with the stock constructor (budget 512)."""
    import random

    import torch

    sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    try:
        from shrike.engine.engine import LLMEngine
        from shrike.engine.request import SamplingParams
    except Exception as error:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"baseline/_ref does not import: {type(error).__name__}: {error}"[:300]}

    raw = dict(raw_model)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    work = Path(tempfile.mkdtemp(prefix="shrike_reference_"))
    try:
        write_model_folder(work, raw)
        torch.cuda.empty_cache()
        engine = LLMEngine(str(work))
        rng = random.Random(20260718)
        outputs = [rng.randint(32, 256) for _ in range(64)]
        prompts = [[rng.randrange(raw["vocab_size"]) for _ in range(rng.randint(32, 2048))] for _ in range(64)]
        params = [SamplingParams(max_new_tokens=n, temperature=0.0, ignore_eos=True) for n in outputs]
        engine.generate(prompts[:4], params[:4], chat=False)   # warm-up, as in the other arm
        torch.cuda.synchronize()
        steps_before = engine.stats.steps
        began = time.perf_counter()
        results = engine.generate(prompts, params, chat=False)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - began
        generated = sum(len(r) for r in results)
        return {
            "impl": "reference", "workload": "mixed", "model": "Qwen2.5-1.5B shape", "layers": raw["num_hidden_layers"],
            "requests": 64, "prompt_tokens": sum(len(p) for p in prompts), "generated_tokens": generated,
            "seconds": round(seconds, 3), "value": round(generated / seconds, 1), "unit": "generated tok/s",
            "steps": engine.stats.steps - steps_before, "budget": 512, "dtype": "bf16",
            "engine_defaults": "stock LLMEngine(model_dir): prefix caching on, einsum attention",
            "data": "synthetic: seeded random weights and uniform random token ids",
        }
    finally:
        shutil.rmtree(work, ignore_errors=True)
