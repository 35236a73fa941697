"""LLMEngine: scheduler + step function + sampler in one loop.

The public surface is Azimml/shrike's (shrike/engine/engine.py:41-203): the
constructor's `block_size`, `gpu_mem_util`, `max_tokens_per_step`, `max_running`;
`add_request(prompt, sampling, chat=True) -> req_id`, `has_work`,
`step() -> [StepOutput(req_id, token_id, finished, finish_reason)]`,
`generate(prompts, sampling) -> [[token ids]]`, `metrics()`, and the attributes
`requests`, `scheduler`, `block_manager`, `tokenizer`, `stats`.  Added: `num_blocks`
(an explicit pool size), `dtype` ("bfloat16" or "float32"), `seed`.  Left out:
prefix caching and speculation.  step() = schedule -> one batched forward -> sample
-> append / finish (engine.py:109-164); the sampled token of a request whose step
reached the end of its known tokens comes from that entry's last row
(shrike/engine/model_runner.py:222-228).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch

from .. import models as _models  # noqa: F401  (registers the architectures)
from ..config.registry import load_config
from ..sampling.rng import step_seed
from ..weights.loader import load_weights
from .batch import StepEntry
from .request import Request, SamplingParams
from .runner import TORCH_DTYPES, ModelRunner
from .scheduler import Scheduler


@dataclass
class StepOutput:
    req_id: int
    token_id: int
    finished: bool
    finish_reason: str | None


@dataclass
class EngineStats:
    steps: int = 0
    tokens_generated: int = 0
    started_at: float = field(default_factory=time.perf_counter)


def make_ops(dtype: str, device):
    from ..ops.cuda_ops import CudaOps

    return CudaOps(TORCH_DTYPES[dtype], device)


def _load_tokenizer(model_dir):
    folder = Path(model_dir)
    if not any((folder / name).is_file() for name in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        return None
    from transformers import AutoTokenizer  # tokenizer only; no model code

    return AutoTokenizer.from_pretrained(str(folder))


class LLMEngine:
    def __init__(
        self,
        model_dir: str | None,
        block_size: int = 16,
        gpu_mem_util: float = 0.85,
        max_tokens_per_step: int = 512,
        max_running: int = 256,
        num_blocks: int | None = None,
        dtype: str | None = None,
        seed: int = 0,
        device: str = "cuda",
        config=None,
        tensors=None,
        ops=None,
    ) -> None:
        """`model_dir` holds config.json and *.safetensors; or pass `config` and
        `tensors` (name -> tensor on `device`) to serve weights made in memory."""
        if config is None:
            config = load_config(model_dir)
        self.config = config
        self.dtype = dtype or config.dtype
        if self.dtype not in TORCH_DTYPES:
            raise ValueError(f"dtype {self.dtype!r}: choose bfloat16 or float32")
        self.device = torch.device(device)
        self.ops = ops if ops is not None else make_ops(self.dtype, self.device)
        if tensors is None:
            tensors = load_weights(model_dir, config, TORCH_DTYPES[self.dtype], self.device)
        self.tokenizer = _load_tokenizer(model_dir) if model_dir is not None else None
        self.runner = ModelRunner(
            config, tensors, self.ops, self.device, self.dtype, page_size=block_size,
            num_pages=num_blocks, gpu_mem_util=gpu_mem_util, max_slots=max_running,
            max_portion=max_tokens_per_step,
        )
        self.block_manager = self.runner.cache
        self.scheduler = Scheduler(self.block_manager, max_tokens_per_step, max_running)
        self.eos_ids = set(config.eos_token_ids)
        self.requests: dict[int, Request] = {}
        self.stats = EngineStats()
        self.seed = seed
        self._arrivals = 0
        self._request_seed: dict[int, int] = {}
        self.launch_ahead = True   # launch the next decode step before this one's tokens are read back
        self._flight = None        # (batch, sampled requests, fetch handle) of a step launched that way

    @classmethod
    def from_random(cls, shape: str, seed: int = 0, dtype: str | None = None, device: str = "cuda", **options):
        """An engine without a checkpoint: `shape` names one of the package's shape files or is the
        path of a config.json (`shrike_b200.shapes.shape_config`); the weights are drawn on the
        device from `seed`, as `weights.random_init` draws them."""
        from ..config.registry import parse_config
        from ..shapes import shape_config
        from ..weights.random_init import random_tensors

        config = parse_config(shape_config(shape))
        dtype = dtype or config.dtype
        tensors = random_tensors(config, seed, device, TORCH_DTYPES[dtype])
        return cls(None, dtype=dtype, seed=seed, device=device, config=config, tensors=tensors, **options)

    def reset_stats(self) -> None:
        """Zeroes what `metrics()` counts (the `/reset` of shrike/cli.py:246-252)."""
        self.stats = EngineStats()
        self.scheduler.num_preemptions = 0

    def warm_up(self, token_counts=(1, 16, 64, 128, 256, 512)) -> float:
        """Runs one throw-away step per token count (one request fed that many tokens at once), so that
        what happens once per kernel and per product shape (loading a kernel's code, the matrix library's
        choice of a product kernel for a token count above 64: 15 to 70 ms a shape) does not fall into
        the first real requests.  Counts above the step's token budget or the pool's size are left out.
        Only with no request in the engine; the pools and the counters are as before afterwards.
        Returns the seconds it took.  Not in the reference; nothing calls it unless asked to."""
        if self.requests or self._flight is not None:
            raise RuntimeError("warm_up() wants an engine without requests")
        began = time.perf_counter()
        cache_manager = self.runner.cache
        limit = min(self.scheduler.max_tokens_per_step, self.config.max_position_embeddings)
        if self.block_manager.portion_limit() is not None:
            limit = min(limit, self.block_manager.portion_limit())
        for count in sorted({int(c) for c in token_counts if 0 < int(c) <= limit}):
            if any(w > have for w, have in zip(self.block_manager.worst_case_pages(count, count), self.block_manager.num_pages)):
                continue
            cache = cache_manager.open()
            try:
                cache_manager.append(cache, 0, count)
                self.runner.step([StepEntry(cache, [0] * count, 0, [count - 1], (0.0, 1.0, 0))], sample=True)
            finally:
                cache_manager.free(cache)
        torch.cuda.synchronize(self.device)
        self.ops.check_status()
        return time.perf_counter() - began

    # ---- requests -------------------------------------------------------------
    def _tokenize(self, prompt: str, chat: bool) -> list[int]:
        if self.tokenizer is None:
            raise ValueError(
                "the model folder has no tokenizer files: pass token ids (a list of int) instead of text"
            )
        if chat:
            encoded = self.tokenizer.apply_chat_template(
                [{"role": "user", "content": prompt}], add_generation_prompt=True
            )
            return list(encoded["input_ids"] if isinstance(encoded, dict) else encoded)
        return list(self.tokenizer(prompt).input_ids)

    def add_request(self, prompt, sampling: SamplingParams, chat: bool = True) -> int:
        token_ids = self._tokenize(prompt, chat) if isinstance(prompt, str) else [int(t) for t in prompt]
        if not token_ids:
            raise ValueError("empty prompt: a request must have at least one token")
        vocab = self.config.vocab_size
        if min(token_ids) < 0 or max(token_ids) >= vocab:
            raise ValueError(f"token ids must lie in [0, {vocab}); got {min(token_ids)}..{max(token_ids)}")
        total = len(token_ids) + sampling.max_new_tokens
        if total > self.config.max_position_embeddings:
            raise ValueError(
                f"{len(token_ids)} prompt + {sampling.max_new_tokens} generated tokens exceed "
                f"max_position_embeddings={self.config.max_position_embeddings}"
            )
        worst = self.block_manager.worst_case_pages(total, self.scheduler.max_tokens_per_step)
        if any(w > have for w, have in zip(worst, self.block_manager.num_pages)):
            raise ValueError(
                f"request needs up to {max(worst)} KV blocks ({len(token_ids)} prompt + "
                f"{sampling.max_new_tokens} generated tokens, block_size={self.block_manager.page_size}) "
                f"but the pool has only {self.block_manager.total_pages}; it could never be scheduled: "
                "shorten the prompt, lower max_new_tokens, or raise gpu_mem_util / num_blocks"
            )
        request = Request(token_ids=token_ids, sampling=sampling)
        self.requests[request.req_id] = request
        base = sampling.seed if sampling.seed is not None else step_seed(self.seed, self._arrivals)
        self._request_seed[request.req_id] = base
        self._arrivals += 1
        self.scheduler.add(request)
        return request.req_id

    def abort(self, req_id: int) -> None:
        request = self.requests.pop(req_id, None)
        if request is not None:
            self.scheduler.abort(request)
            self._request_seed.pop(req_id, None)

    @property
    def has_work(self) -> bool:
        return self.scheduler.has_work

    # ---- the loop ---------------------------------------------------------------
    def _entries(self, batch):
        entries, sampled = [], []
        for request, num_new in batch:
            start = request.num_computed_tokens
            reaches_end = start + num_new >= request.num_tokens
            sampling = None
            if reaches_end:
                params = request.sampling
                sampling = (params.temperature, params.top_p,
                            step_seed(self._request_seed[request.req_id], request.num_tokens))
                sampled.append(request)
            entries.append(StepEntry(request.cache, request.token_ids[start: start + num_new], start,
                                     [num_new - 1] if reaches_end else [], sampling))
        return entries, sampled

    def _launch_ahead(self, batch, sampled):
        """While the device runs a step: schedules, stages and launches the step after it.  A
        request whose token is being drawn by the step in flight goes into the next one with the
        id -1 - row, which the embedding kernel replaces on the device by what that row drew, so
        neither the device nor the host waits for the other.  Done only when it changes nothing
        but the timing: nobody reaches its length limit with the token in flight (its end frees
        pages and a slot that scheduling early would not see), and the pages for whatever the
        next step takes are free, so that scheduling early preempts nobody whom a stop token, seen
        a moment later, would have spared.  Returns the step in flight, or None.

        A request that ends on a stop token while the next step is already in flight has one
        token computed in vain; its row of that step's output is dropped.  Its pages go back at
        once: whatever is given them later is launched later, and the device runs in order."""
        if not self.launch_ahead:
            return None
        if any(r.num_generated + 1 >= r.sampling.max_new_tokens for r in sampled):
            return None
        scheduler, manager = self.scheduler, self.block_manager
        steady = (len(sampled) == len(batch) and not scheduler.waiting and len(batch) == len(scheduler.running)
                  and all(n == 1 for _, n in batch))
        if steady:   # every running request decodes: what the next step takes is known exactly
            need = [0] * len(manager.num_free)
            for request in sampled:
                for group, pages in enumerate(manager.pages_needed(request.cache, request.num_computed_tokens, 1)):
                    need[group] += pages
        else:        # portions, arrivals: at most the token budget in new pages, and one more per request that may run
            candidates = min(len(scheduler.running) + len(scheduler.waiting), scheduler.max_running)
            need = [manager.blocks_for(scheduler.max_tokens_per_step) + candidates + 1] * len(manager.num_free)
        if any(n > free for n, free in zip(need, manager.num_free)):
            return None
        preemptions = scheduler.num_preemptions
        ahead = scheduler.schedule()
        if not ahead or scheduler.num_preemptions != preemptions:
            return None   # scheduling again at the next step does no harm: reserved pages are kept
        row_of = {request.req_id: row for row, request in enumerate(sampled)}
        entries, sampled_ahead = [], []
        for request, num_new in ahead:
            start, known = request.num_computed_tokens, request.num_tokens
            params = request.sampling
            if request.req_id in row_of:
                # its newest token is still on the device: it will sit at position `known`
                if start != known or num_new != 1:
                    raise AssertionError("a request whose token is in flight was scheduled for anything but that token")
                sampling = (params.temperature, params.top_p, step_seed(self._request_seed[request.req_id], known + 1))
                entries.append(StepEntry(request.cache, [-1 - row_of[request.req_id]], start, [0], sampling))
                sampled_ahead.append(request)
                continue
            reaches_end = start + num_new >= known
            sampling = None
            if reaches_end:
                sampling = (params.temperature, params.top_p, step_seed(self._request_seed[request.req_id], known))
                sampled_ahead.append(request)
            entries.append(StepEntry(request.cache, request.token_ids[start: start + num_new], start,
                                     [num_new - 1] if reaches_end else [], sampling))
        return self._launch(ahead, entries, sampled_ahead)

    def _launch(self, batch, entries, sampled):
        result = self.runner.step(entries, sample=bool(sampled))
        self.scheduler.postprocess(batch)
        return batch, sampled, self.runner.fetch(result[1]) if sampled else None

    @torch.inference_mode()
    def step(self) -> list[StepOutput]:
        """One step's outputs.  In the steady state of decoding the step after it is launched
        before this step's tokens are read back, so the device does not wait for the host."""
        flight, self._flight = self._flight, None
        if flight is None:
            batch = self.scheduler.schedule()
            if not batch:
                return []
            entries, sampled = self._entries(batch)
            flight = self._launch(batch, entries, sampled)
        batch, sampled, fetched = flight
        self._flight = self._launch_ahead(batch, sampled)
        try:
            tokens = self.runner.wait(fetched) if sampled else []
        except Exception:
            # a kernel of this step gave up: nothing of it is appended, and the step launched ahead
            # (computed from the same state) is dropped with it
            self._flight = None
            raise

        outputs: list[StepOutput] = []
        for request, token in zip(sampled, tokens):
            if self.requests.get(request.req_id) is not request:
                continue   # ended (stop token, abort) while this step was in flight
            request.token_ids.append(token)
            self.stats.tokens_generated += 1
            finished, reason = False, None
            if token in self.eos_ids and not request.sampling.ignore_eos:
                finished, reason = True, "stop"
            elif request.num_generated >= request.sampling.max_new_tokens:
                finished, reason = True, "length"
            outputs.append(StepOutput(request.req_id, token, finished, reason))
            if finished:
                self.scheduler.finish(request, reason)
                del self.requests[request.req_id]
                self._request_seed.pop(request.req_id, None)
        self.stats.steps += 1
        return outputs

    def _check_kernels(self) -> None:
        """Raises if a kernel left a code in its status word.  Steps that sample see the word with
        their tokens (`ModelRunner.wait`); this reads it once more at the end of `generate`."""
        check = getattr(self.ops, "check_status", None)
        if check is not None:
            check()

    def generate(self, prompts, sampling, chat: bool = True) -> list[list[int]]:
        """Offline batch API (engine.py:166-183): generated token ids per prompt."""
        if isinstance(sampling, SamplingParams):
            sampling = [sampling] * len(prompts)
        id_map = {self.add_request(p, s, chat): i for i, (p, s) in enumerate(zip(prompts, sampling, strict=True))}
        results: list[list[int]] = [[] for _ in prompts]
        while self.has_work:
            for out in self.step():
                results[id_map[out.req_id]].append(out.token_id)
        self._check_kernels()
        return results

    def metrics(self) -> dict:
        elapsed = time.perf_counter() - self.stats.started_at
        return {
            "steps": self.stats.steps,
            "tokens_generated": self.stats.tokens_generated,
            "avg_tokens_per_sec": round(self.stats.tokens_generated / max(elapsed, 1e-9), 1),
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
            "kv_blocks_total": self.block_manager.total_pages,
            "kv_blocks_free": self.block_manager.free_pages,
            "preemptions": self.scheduler.num_preemptions,
        }
