"""Device memory behind the cache manager's ids.

Each group of key/value caches is one tensor
`[caches in group, 2, pages, page_size, kv heads, head size]` in the engine dtype:
the layout Azimml/shrike uses for its single pool
(shrike/engine/model_runner.py:52-60, per layer viewed as pages at :74-75), once
per group.  Per-request state of fixed size is one tensor `[slots, *shape]` per
cache id that asked for it; `zero_slots` clears the slots of requests that were just opened,
which the step function calls before their first token runs (a part never has to).
"""

from __future__ import annotations

import torch

from .manager import KVGroupSpec


def page_bytes(group: KVGroupSpec, page_size: int, element_size: int) -> int:
    return len(group.cache_ids) * 2 * page_size * group.num_kv_heads * group.head_dim * element_size


def state_bytes(state_needs: dict, max_slots: int) -> int:
    """Bytes of all per-request state: every stateful cache holds `max_slots` slots of its shape."""
    total = 0
    for need in state_needs.values():
        count = 1
        for extent in need.shape:
            count *= extent
        total += max_slots * count * torch.empty((), dtype=getattr(torch, need.dtype)).element_size()
    return total


class CacheStorage:
    def __init__(self, groups, page_size, num_pages, state_needs, max_slots, dtype, device):
        self.groups = list(groups)
        self.page_size = page_size
        self.group_of_cache: dict[int, tuple[int, int]] = {}
        self.kv: list[torch.Tensor] = []
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        for index, (group, count) in enumerate(zip(self.groups, counts)):
            self.kv.append(
                torch.zeros(
                    len(group.cache_ids), 2, count, page_size, group.num_kv_heads, group.head_dim,
                    dtype=dtype, device=device,
                )
            )
            for position, cache_id in enumerate(group.cache_ids):
                self.group_of_cache[cache_id] = (index, position)
        self.state: dict[int, torch.Tensor] = {
            cache_id: torch.zeros((max_slots, *need.shape), dtype=getattr(torch, need.dtype), device=device)
            for cache_id, need in state_needs.items()
        }

    def zero_slots(self, slots: list[int]) -> None:
        """Zeroes the state of `slots` in every stateful cache (one indexed fill each)."""
        if not slots or not self.state:
            return
        first = next(iter(self.state.values()))
        index = torch.tensor(slots, dtype=torch.long, device=first.device)
        for tensor in self.state.values():
            tensor.index_fill_(0, index, 0)

    def keys_values(self, cache_id: int):
        """(group index, keys, values), each `[pages, page_size, kv heads, head size]`."""
        group, position = self.group_of_cache[cache_id]
        slab = self.kv[group][position]
        return group, slab[0], slab[1]

    def bytes(self) -> int:
        total = sum(t.numel() * t.element_size() for t in self.kv)
        return total + sum(t.numel() * t.element_size() for t in self.state.values())
