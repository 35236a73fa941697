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

from ..cache.manager import CacheManager, group_caches
from ..cache.storage import CacheStorage, page_bytes
from ..config.model_config import ModelConfig
from .batch import BatchBuilder, StepEntry
from .model import DecoderModel, Runtime

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


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
    ):
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
        self.bytes_per_page = sum(page_bytes(g, page_size, element) for g in self.groups)
        if num_pages is None:
            free, _total = torch.cuda.mem_get_info(self.device)
            num_pages = int(free * gpu_mem_util) // max(1, self.bytes_per_page)
        if num_pages < 1:
            raise ValueError("no room for a single cache page; lower the model size or raise gpu_mem_util")
        self.num_pages = num_pages
        self.cache = CacheManager(self.groups, page_size, num_pages, max_slots)
        self.storage = CacheStorage(
            self.groups, page_size, num_pages, state_needs, max_slots, self.dtype, self.device
        )
        self.builder = BatchBuilder(page_size, len(self.groups), self.device, self.storage)

    @torch.inference_mode()
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        ctx = self.builder.build(entries)
        return self.model.forward(ctx)
