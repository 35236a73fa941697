"""The step function: a batch of (request, its next tokens) in, logits out.

`ModelRunner.step(entries)` runs exactly the tokens it is given, as one batch, on
the cache that earlier steps left, and returns float32 logits at the wanted places
(in the order of the entries and of each entry's `want`).  It is the one path to
the model: generation, trace replay and the benchmark all call it.  Counterpart:
ModelRunner.run in shrike/engine/model_runner.py:182-250, which returns only each
finished entry's last row; pool sizing follows :165-174.
"""

from __future__ import annotations

import torch

from ..cache.manager import CacheManager, group_caches, pages_in_flight, pages_per_group
from ..cache.storage import CacheStorage, page_bytes, state_bytes
from ..config.model_config import ModelConfig
from .batch import BatchBuilder, StepEntry
from .model import DecoderModel, Runtime

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class Prepared:
    """A step whose metadata is staged on the host: what `ModelRunner.launch` needs."""

    __slots__ = ("staged", "sample", "graphable", "key", "decode", "rows")

    def __init__(self, staged, sample: bool, graphable: bool, key=None, decode: bool = False):
        self.staged = staged
        self.sample = sample
        self.graphable = graphable
        self.key = key
        self.decode = decode
        self.rows = staged.rows   # wanted rows without padding: what the caller gets back


class ModelRunner:
    def __init__(
        self,
        config: ModelConfig,
        tensors: dict,
        ops,
        device,
        dtype: str,
        page_size: int = 16,
        num_pages: int | None = None,
        gpu_mem_util: float = 0.85,
        max_slots: int = 256,
        max_portion: int | None = None,
    ):
        """`num_pages`: pages of every group (an int) or of each group (a list); None sizes the pools
        from free device memory: `gpu_mem_util` of it, less the per-request state of `max_slots`
        requests, shared out by `pages_per_group` (groups that keep every key get equal counts, a
        group with a window what `max_slots` requests fed `max_portion` tokens a step can hold)."""
        self.config = config
        self.device = torch.device(device)
        self.dtype = TORCH_DTYPES[dtype]
        self.ops = ops
        self.runtime = Runtime(self.device, self.dtype)
        self.model = DecoderModel(config, tensors, ops, self.runtime)
        kv_needs, state_needs = self.model.cache_needs()
        self.groups = group_caches(kv_needs)
        self.page_size = page_size
        element = torch.empty((), dtype=self.dtype).element_size()
        per_group = [page_bytes(g, page_size, element) for g in self.groups]
        self.bytes_per_page = sum(per_group)
        self.state_bytes = state_bytes(state_needs, max_slots)
        if num_pages is None:
            free, _total = torch.cuda.mem_get_info(self.device)
            budget = int(free * gpu_mem_util) - self.state_bytes
            num_pages = pages_per_group(self.groups, page_size, budget, per_group, max_slots,
                                        max_portion or config.max_position_embeddings)
        elif isinstance(num_pages, int):
            # an explicit count: that many pages for a group that keeps every key, and no more than its
            # requests can ever hold for a group with a window
            portion = max_portion or config.max_position_embeddings
            num_pages = [num_pages if g.window is None else
                         min(num_pages, max_slots * pages_in_flight(1 << 40, g.window, portion, page_size))
                         for g in self.groups]
        if any(count < 1 for count in num_pages):
            raise ValueError("no room for a single cache page; lower the model size or raise gpu_mem_util")
        self.num_pages = list(num_pages)
        self.cache = CacheManager(self.groups, page_size, num_pages, max_slots)
        self.storage = CacheStorage(
            self.groups, page_size, num_pages, state_needs, max_slots, self.dtype, self.device
        )
        self.builder = BatchBuilder(page_size, len(self.groups), self.device, self.storage)
        self.use_graphs = True
        # steps are recorded as CUDA graphs (decode batches at once, batches with portions once their
        # shape repeats) only if every part says that its forward() depends on the batch's shape alone
        # (`capture_safe`; a model with a part that does not say so, such as one that branches on a
        # request's position on the host, runs every step kernel by kernel)
        self.capture_safe = bool(getattr(self.model, "capture_safe", False))
        self.capture_portions = self.capture_safe
        # batches of single tokens are padded up to a few sizes (multiples of eight), so that a
        # workload whose batch shrinks and grows request by request replays a handful of captured
        # sequences instead of capturing one per size; on the same condition, because a padding
        # row carries slot -1 and state slot -1, which a part with state of its own must skip
        self.pad_decode = self.capture_portions
        self._graphs: dict = {}
        self._seen: dict = {}
        self.portion_sightings = 5   # a shape with portions is captured when it comes for the sixth time
        # the kernels' status word and the sampled tokens of a step lie side by side, so that one
        # copy brings both to the host: a step whose kernels gave up is seen before its tokens are used
        self._status_block = torch.zeros(4 + 4096, dtype=torch.int32, device=self.device)
        self._drawn = self._status_block[4:]
        if hasattr(ops, "adopt_status"):
            ops.adopt_status(self._status_block[:4])
        self._drawn_generation = 0
        self._fetch_host = [None, None]
        self._fetch_turn = 0
        self._capture_stream = None

    # ---- the step ---------------------------------------------------------------
    def _run(self, ctx, sample: bool):
        if ctx.num_rows > self._drawn.numel():   # rare: more sampled rows than any step before
            self._drawn = torch.zeros(2 * ctx.num_rows, dtype=torch.int32, device=self.device)
            self._drawn_generation += 1
        # the tokens drawn by the step before are still in `_drawn` while the embedding runs;
        # this step's sampling, at its very end, overwrites them
        ctx.previous_tokens = self._drawn
        hold = getattr(self.ops, "hold_stream", None)
        if hold is not None:
            hold(True)
        try:
            logits = self.model.forward(ctx)
            tokens = None
            if sample:
                tokens = self._drawn[: ctx.num_rows]
                self.ops.sample(logits, ctx.sample_temperature, ctx.sample_top_p, ctx.sample_seed, tokens)
        finally:
            if hold is not None:
                hold(False)
        return logits, tokens

    def _capture(self, ctx, sample: bool):
        """Records the step's launch sequence on a side stream.  What `torch.cuda.graph` does around a
        capture besides (a garbage collection, handing every cached block back to the driver) is left
        out: it costs milliseconds, tens of them when much is cached, in the middle of serving, and a
        step allocates nothing while it is recorded (the run just before it has sized every buffer)."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
        graph = torch.cuda.CUDAGraph()
        side = self._capture_stream
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            graph.capture_begin()
            try:
                outputs = self._run(ctx, sample)
            finally:
                graph.capture_end()
        torch.cuda.current_stream(self.device).wait_stream(side)
        return graph, outputs

    def _generation(self):
        return (self.runtime.generation, self.builder.generation, getattr(self.ops, "generation", 0),
                self._drawn_generation)

    def step(self, entries: list[StepEntry], sample: bool = False):
        """Runs the entries' tokens as one batch: `launch(prepare(entries, sample))`."""
        return self.launch(self.prepare(entries, sample))

    def prepare(self, entries: list[StepEntry], sample: bool = False) -> "Prepared":
        """The host half of a step: the batch's metadata packed into pinned memory, nothing sent
        yet.  It may run while the device still works on the step before."""
        pad_to = 0
        if self.pad_decode and self.use_graphs and self.device.type == "cuda" and len(entries) > 8:
            pad_to = -(-len(entries) // 8) * 8
        staged = self.builder.stage(entries, defer=True, pad_to=pad_to)
        if sample and not staged.sampled:
            raise ValueError("sample=True needs `sampling` on every entry that wants logits")
        decode = max(staged.q_lens) == 1 and staged.r == staged.s and all(e.want == [0] for e in entries)
        if not decode and staged.rows != staged.r:
            raise AssertionError("only batches of single tokens that all want their logits are padded")
        # a launch sequence is recorded and replayed only if every part promises that its forward pass
        # depends on the batch's shape alone (`capture_safe`): a part that reads positions or slots on
        # the host would replay the values of the step it was recorded in
        graphable = (self.use_graphs and self.device.type == "cuda" and self.capture_safe
                     and (decode or self.capture_portions))
        # what a captured launch sequence has baked in: the number of entries, every entry's
        # length (grids and shapes follow from them), the number of wanted rows, the table widths
        key = (staged.s if decode else tuple(staged.q_lens), staged.r, tuple(staged.max_blocks), sample)
        return Prepared(staged, sample, graphable, key, decode)

    def fetch(self, tokens: torch.Tensor):
        """Starts the copy of a step's drawn tokens to pinned host memory and returns a handle for
        `wait`.  The copy is ordered before whatever is launched next, so a later step may
        overwrite the device buffer."""
        count = tokens.numel()
        if self.device.type != "cuda":
            return tokens.tolist(), count, None
        self._fetch_turn ^= 1
        if self._fetch_host[self._fetch_turn] is None or self._fetch_host[self._fetch_turn].numel() < 4 + count:
            self._fetch_host[self._fetch_turn] = torch.zeros(max(256, 4 + 2 * count), dtype=torch.int32, pin_memory=True)
        host = self._fetch_host[self._fetch_turn]
        if count and tokens.data_ptr() == self._drawn.data_ptr() and self._drawn.data_ptr() == self._status_block[4:].data_ptr():
            host[: 4 + count].copy_(self._status_block[: 4 + count], non_blocking=True)   # status word and tokens at once
        else:
            host[:4].copy_(self._status_block[:4], non_blocking=True)
            host[4: 4 + count].copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return host, count, event

    def wait(self, handle) -> list[int]:
        """The tokens of a fetched step.  Raises before handing them out when a kernel of that step
        (or of one before it) left a code in the status word."""
        host, count, event = handle
        if event is None:
            return host
        event.synchronize()
        code = int(host[0])
        if code:
            self.ops.raise_status(code)
        return host[4: 4 + count].tolist()

    @torch.inference_mode()
    def launch(self, prepared: "Prepared"):
        """The device half of a step.  Returns float32 logits [wanted, vocab];
        with `sample=True` (every entry with wanted rows carries `sampling`) returns
        (logits, int32 tokens [wanted]) instead, the tokens drawn by the sampling kernel.

        A batch of single tokens that all want their logits is the steady state of
        decoding; its launch sequence is captured once per (batch size, table width) as a
        CUDA graph and replayed afterwards, because at small batch the step is bound by
        launch latency otherwise (the remedy shrike's README names for its own per-layer
        dispatch cost).  Other batches are captured when their exact shape (every entry's
        length, the wanted rows, the table widths) has been seen a few times.  A captured sequence
        bakes in what the parts computed on the host from the shape; parts must not branch on
        other host-side values of the step (positions, slots) if they are to be captured."""
        staged, sample, graphable, rows = prepared.staged, prepared.sample, prepared.graphable, prepared.rows
        self.storage.zero_slots(self.cache.take_opened())   # requests opened since the last step start from zero state
        self.builder.commit(staged)
        key = prepared.key
        if graphable and not prepared.decode and key not in self._graphs:
            # a batch with portions: captured only when the same shape has come several times (a long
            # prompt cut into equal portions, a benchmark's repeats).  Capturing costs a few steps'
            # time, and most shapes of a mixed workload come once or twice.
            if len(self._seen) >= 1024:
                self._seen.clear()
            self._seen[key] = self._seen.get(key, 0) + 1
            graphable = self._seen[key] > self.portion_sightings
        if not graphable:
            logits, tokens = self._run(self.builder.context(staged), sample)
            return (logits[:rows], tokens[:rows]) if sample else logits[:rows]
        held = self._graphs.get(key)
        if held is not None and held[0] == self._generation():
            held[1].replay()   # the metadata is already on its way; no views are needed
            self.ops.launches += held[4]
            self.ops.library_calls += held[5]
            return (held[2][:rows], held[3][:rows]) if sample else held[2][:rows]
        ctx = self.builder.context(staged)
        # first time (or buffers moved): run eagerly for this step's result, then capture
        logits, tokens = self._run(ctx, sample)
        generation = self._generation()
        before = (self.ops.launches, self.ops.library_calls)
        graph, (g_logits, g_tokens) = self._capture(ctx, sample)
        counted = (self.ops.launches - before[0], self.ops.library_calls - before[1])
        self.ops.launches, self.ops.library_calls = before
        if generation == self._generation():
            if len(self._graphs) >= 64:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = (generation, graph, g_logits, g_tokens, counted[0], counted[1])
        return (logits[:rows], tokens[:rows]) if sample else logits[:rows]
