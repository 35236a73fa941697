"""The model as data: parts built from the configuration, run in the listed order.

Embedding, the layer runs, the final norm on the wanted rows only and the head
(shrike/models/qwen.py:160-164,181-192).  Which class serves a part (the embedding and
the head included) comes from the spec's `kind` through the part registries; which parts
a layer has from its spec's roles; which layer runs when, and on which cache, from
`config.order`.
"""

from __future__ import annotations

import torch

from ..config.model_config import ModelConfig
from ..parts.base import part_class
from ..weights.expected import tensor_names


class Runtime:
    """What parts share on the device: dtype, device and named scratch buffers.

    A named buffer keeps its address while its capacity suffices, so captured
    launch sequences stay valid; the same name is reused by every layer."""

    def __init__(self, device, act_dtype: torch.dtype):
        self.device = torch.device(device)
        self.act_dtype = act_dtype
        self._buffers: dict[str, torch.Tensor] = {}
        self._views: dict = {}   # (name, shape, dtype) -> view, while the buffer has not moved
        self.generation = 0  # grows when a buffer moves

    def buffer(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        count = 1
        for extent in shape:
            count *= extent
        held = self._buffers.get(name)
        if held is None or held.dtype != dtype or held.numel() < count:
            capacity = count if held is None or held.dtype != dtype else max(count, 2 * held.numel())
            held = torch.empty(max(capacity, 1), dtype=dtype, device=self.device)
            self._buffers[name] = held
            self.generation += 1
            self._views = {k: v for k, v in self._views.items() if k[0] != name}
        if len(self._views) > 4096:
            self._views.clear()
        view = held[:count].view(shape)
        self._views[key] = view
        return view

    def reserve(self, name: str, count: int, dtype: torch.dtype) -> None:
        self.buffer(name, (count,), dtype)

    def scratch_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buffers.values())


def _take(tensors: dict, prefix: str, names) -> dict:
    return {local: tensors[prefix + local] for local in names}


class DecoderModel:
    def __init__(self, config: ModelConfig, tensors: dict[str, torch.Tensor], ops, runtime: Runtime):
        self.config = config
        self.ops = ops
        self.runtime = runtime
        names = tensor_names(config)
        spec = config.embedding
        cls = part_class("embedding", spec.kind)
        self.embedding = cls(spec, {local: tensors[names.embedding_name(local)] for local in cls.parameters(spec)},
                             ops, runtime)
        parts = [self.embedding]
        self.blocks = []
        for index, layer in enumerate(config.layers):
            built = {}
            for role, category, spec in layer.roles():
                cls = part_class(category, spec.kind)
                built[role] = cls(spec, _take(tensors, names.layer_part(index, role), cls.parameters(spec)), ops, runtime)
            self.blocks.append(part_class("block", layer.block)(**built))
            if hasattr(self.blocks[-1], "prepare"):
                self.blocks[-1].prepare()
            parts += [*built.values(), self.blocks[-1]]
        norm = config.final_norm
        cls = part_class("norm", norm.kind)
        self.final_norm = cls(norm, _take(tensors, names.final_norm_prefix, cls.parameters(norm)), ops, runtime)
        spec = config.head
        cls = part_class("head", spec.kind)
        local_tensors = {}
        for local in cls.parameters(spec):
            name = names.head_name(local)
            if name in tensors:
                local_tensors[local] = tensors[name]
            elif local == "weight" and getattr(spec, "tied", False) and getattr(self.embedding, "table", None) is not None:
                local_tensors[local] = self.embedding.table
            else:
                raise KeyError(f"{name} is absent and the configuration does not tie it to the embedding")
        self.head = cls(spec, local_tensors, ops, runtime)
        parts += [self.final_norm, self.head]
        self.capture_safe = all(getattr(part, "capture_safe", False) for part in parts)

    def cache_needs(self):
        """cache id -> KVNeed, and cache id -> StateNeed, over the run order."""
        from ..parts.base import KVNeed, StateNeed

        kv, state = {}, {}
        for run in self.config.order:
            spec = self.config.layers[run.layer].mixer
            for need in part_class("mixer", spec.kind).cache_needs(spec):
                table = kv if isinstance(need, KVNeed) else state
                if run.cache in table and table[run.cache] != need:
                    raise ValueError(f"cache {run.cache} is used by runs with different needs")
                if isinstance(need, (KVNeed, StateNeed)):
                    table[run.cache] = need
        return kv, state

    def weight_bytes(self) -> int:
        """Bytes of every distinct tensor the parts hold (a tied table counts once)."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for value in vars(obj).values():
                if isinstance(value, torch.Tensor):
                    if value.data_ptr() not in seen:
                        seen.add(value.data_ptr())
                        total += value.numel() * value.element_size()
                elif hasattr(value, "__dict__") and not isinstance(value, (Runtime, type)) and value is not self.ops:
                    if id(value) not in seen:
                        seen.add(id(value))
                        visit(value)

        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            visit(part)
        return total

    def forward(self, ctx) -> torch.Tensor:
        """float32 logits [R, vocab] at `ctx.out_rows`."""
        resid = self.embedding.forward(ctx)
        delta = None
        for run in self.config.order:
            resid, delta = self.blocks[run.layer].forward(resid, delta, ctx, run)
        if not ctx.num_rows:
            return self.runtime.buffer("logits", (0, self.config.vocab_size), torch.float32)
        return self.head.forward(self.final_norm.gather_norm(resid, delta, ctx.out_rows))
