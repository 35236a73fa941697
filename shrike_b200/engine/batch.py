"""A step's batch: entries in, one packed block of int32 metadata out.

An entry is (a request's cache, its next tokens, the position of the first, the
places whose logits are wanted).  Portions of prompts and single tokens lie side
by side in one flat token batch, as in Azimml/shrike's ModelRunner.run
(shrike/engine/model_runner.py:195-229): token ids, positions start..start+n-1,
slot = page * page_size + position % page_size (:211-214), context length
start + n (:215).  Unlike the reference, which treats rows with one token and
longer rows through different metadata (:217-221), every row here is described the
same way (query start, context length, block-table row, state slot), and all of
it travels to the device as ONE copy from pinned memory.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


FIRST_GROUP = 11   # index of the first per-group part of the packed block (see BatchBuilder.stage)


@dataclass
class StepEntry:
    cache: object  # cache.RequestCache
    tokens: list[int]
    start: int
    want: list[int] = field(default_factory=list)
    sampling: tuple | None = None  # (temperature, top_p, seed) for this entry's wanted rows


@dataclass
class GroupView:
    slot_mapping: torch.Tensor  # int32 [N]: where each new token's key/value goes
    block_table: torch.Tensor  # int32 [S, max_blocks], -1 where no page is held
    max_blocks: int


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    num_rows: int
    token_ids: torch.Tensor  # int32 [N]
    positions: torch.Tensor  # int32 [N]
    seq_of_token: torch.Tensor  # int32 [N]
    q_start: torch.Tensor  # int32 [S + 1]
    ctx_len: torch.Tensor  # int32 [S], new tokens included
    state_slot: torch.Tensor  # int32 [S]
    seq_start: torch.Tensor  # int32 [S]: position of each entry's first token (0: the request begins)
    out_rows: torch.Tensor  # int32 [R]
    groups: list[GroupView]
    storage: object  # cache.storage.CacheStorage
    max_q_len: int
    min_q_len: int
    max_ctx_len: int
    q_lens: list[int]
    starts: list[int]
    slots: list[int]  # host copy of state_slot
    all_single: bool = False  # every entry brings exactly one token
    sample_temperature: torch.Tensor | None = None  # float32 [R], when every wanted row is sampled
    sample_top_p: torch.Tensor | None = None  # float32 [R]
    sample_seed: torch.Tensor | None = None  # int64 [R]
    previous_tokens: torch.Tensor | None = None  # int32: what the step before drew; an id of -1 - r means its row r


@dataclass
class Staged:
    """What `BatchBuilder.stage` copied: counts, the layout of the block, host-side lists."""

    n: int
    s: int
    r: int
    max_blocks: list
    sizes: list
    offsets: list
    total: int
    sampled: bool
    q_lens: list
    starts: list
    ctx_lens: list
    slots: list
    rows: int = 0              # wanted rows that belong to entries (the rest of `r` is padding)
    host: object = None        # the pinned buffer that holds the block until `commit` copies it
    turn: int = 0
    committed: bool = False


class BatchBuilder:
    """Packs entries into pinned host memory and copies them in one transfer."""

    def __init__(self, page_size: int, num_groups: int, device, storage):
        self.page_size = page_size
        self.num_groups = num_groups
        self.device = torch.device(device)
        self.storage = storage
        self._host: list[torch.Tensor] = []
        self._events: list = []
        self._turn = 0
        self._dev = None
        self._range = None
        self.generation = 0  # grows when the device buffer moves: captured launch sequences are stale then
        self.copied_bytes = 0  # host-to-device bytes of all steps so far

    def _staging(self, count: int):
        pinned = self.device.type == "cuda"
        if not self._host or self._host[0].numel() < count:
            capacity = max(4096, 2 * count)
            self._host = [torch.empty(capacity, dtype=torch.int32, pin_memory=pinned) for _ in range(2)]
            self._events = [None, None]
            self._dev = torch.empty(capacity, dtype=torch.int32, device=self.device)
            self.generation += 1
        self._turn ^= 1
        event = self._events[self._turn]
        if event is not None:
            event.synchronize()
        return self._host[self._turn]

    def build(self, entries: list[StepEntry]) -> StepContext:
        """Stages the entries and returns the device views of the step's metadata."""
        return self.context(self.stage(entries))

    def stage(self, entries: list[StepEntry], defer: bool = False, pad_to: int = 0) -> "Staged":
        """Fills the pinned buffer and starts its copy to the device.  The returned record holds
        only host-side facts; `context` turns it into device views when a forward pass needs them
        (a replayed launch sequence does not).

        `defer=True` fills the buffer only; `commit` starts the copy later.  A deferred block
        must be committed (or dropped) before two more blocks are staged: there are two pinned
        buffers.  A token id of -1 - r stands for the token that the step before drew in its row
        r (the embedding kernel fetches it on the device), which is how a step is staged and
        launched before the host has seen those tokens.

        `pad_to` > len(entries), for a batch of single tokens that all want their logits: the block
        describes `pad_to` rows, so that one captured launch sequence serves every batch size up to
        it.  A padding row is a one-token sequence at position 0 that stores nothing (slot -1, state
        slot -1), reads page 0 of every group (whatever it holds) and is sampled greedily; its
        logits and token come last and are dropped by the step function."""
        page = self.page_size
        q_lens = [len(e.tokens) for e in entries]
        if not entries or min(q_lens) < 1:
            raise ValueError("a step needs entries, each with at least one token")
        n, s = sum(q_lens), len(entries)
        r = sum(len(e.want) for e in entries)
        starts = [e.start for e in entries]
        ctx_lens = [st + q for st, q in zip(starts, q_lens)]
        real = s
        pad = pad_to - s if max(q_lens) == 1 and all(e.want == [0] for e in entries) else 0
        if pad > 0:
            n = s = r = pad_to
        else:
            pad = 0
        need_max = -(-max(ctx_lens) // page)
        max_blocks = [1] * self.num_groups
        for g in range(self.num_groups):
            short = min(e.cache.tables[g].length + (need_max - -(-c // page)) for e, c in zip(entries, ctx_lens))
            if short < need_max:   # some entry holds fewer pages than its context needs: say which
                for e, ctx in zip(entries, ctx_lens):
                    if e.cache.tables[g].length < -(-ctx // page):
                        raise ValueError(f"entry holds {e.cache.tables[g].length} pages in group {g} "
                                         f"but its context of {ctx} needs {-(-ctx // page)}")
            max_blocks[g] = need_max
        # table widths grow in powers of two, so that the layout of a decode batch (and a
        # launch sequence captured for it) stays the same while contexts grow
        max_blocks = [max(8, 1 << (mb - 1).bit_length()) for mb in max_blocks]
        sampled = r > 0 and all(e.sampling is not None for e in entries if e.want)

        sizes = [2 * r, r, r, n, n, n, s + 1, s, s, r, s]
        for g in range(self.num_groups):
            sizes += [n, s * max_blocks[g]]   # parts[FIRST_GROUP + 2 g], parts[FIRST_GROUP + 2 g + 1]
        offsets = [0]
        for size in sizes:
            offsets.append(offsets[-1] + size)
        total = offsets[-1]
        host = self._staging(total)
        flat = host.numpy()
        parts = [flat[offsets[i]: offsets[i + 1]] for i in range(len(sizes))]
        seeds, temps, top_ps = parts[0].view(np.int64), parts[1].view(np.float32), parts[2].view(np.float32)
        ids, pos, seq_of, q_start, ctx_arr, slot_arr, out_rows, start_arr = parts[3:11]
        slots_host = [e.cache.slot for e in entries]
        start_arr[:real] = starts
        if pad > 0:
            start_arr[real:] = 0

        if max(q_lens) == 1:
            # the steady state of decoding: one token per entry, filled without per-token work
            ids[:real] = [e.tokens[0] for e in entries]
            pos[:real] = starts
            seq_of[:] = self._arange(s)
            q_start[:] = self._arange(s + 1)
            ctx_arr[:real] = ctx_lens
            slot_arr[:real] = slots_host
            if pad:
                ids[real:], pos[real:], ctx_arr[real:], slot_arr[real:] = 0, 0, 1, -1
            if r == s and all(e.want == [0] for e in entries):
                out_rows[:] = self._arange(s)
                if sampled:
                    temps[:real] = [e.sampling[0] for e in entries]
                    top_ps[:real] = [e.sampling[1] for e in entries]
                    seeds[:real] = [e.sampling[2] for e in entries]
                    if pad:
                        temps[real:], top_ps[real:], seeds[real:] = 0.0, 1.0, 0
            else:
                row = 0
                for index, e in enumerate(entries):
                    for w in e.want:
                        if w != 0:
                            raise ValueError(f"wanted place {w} is outside the entry's 1 tokens")
                        out_rows[row] = index
                        if sampled:
                            temps[row], top_ps[row], seeds[row] = e.sampling
                        row += 1
            for g in range(self.num_groups):
                slots = parts[FIRST_GROUP + 2 * g]
                table2d = parts[FIRST_GROUP + 1 + 2 * g].reshape(s, max_blocks[g])
                table2d[:] = -1
                width = max_blocks[g]
                for index, e in enumerate(entries):
                    table = e.cache.tables[g]
                    pages = table.pages
                    held = table.length if table.length < width else width
                    table2d[index, :held] = pages[:held]
                    p = starts[index]
                    page_of = int(pages[p // page])
                    if page_of < 0:
                        raise ValueError(f"entry {index} writes into a page of group {g} it no longer holds")
                    slots[index] = page_of * page + p % page
                if pad:
                    slots[real:] = -1
                    table2d[real:, 0] = 0
        else:
            self._fill_general(entries, q_lens, parts, max_blocks, sampled, page, s)

        if pad:
            q_lens, starts = q_lens + [1] * pad, starts + [0] * pad
            ctx_lens, slots_host = ctx_lens + [1] * pad, slots_host + [-1] * pad
        staged = Staged(n, s, r, max_blocks, sizes, offsets, total, sampled, q_lens, starts, ctx_lens, slots_host,
                        rows=r - pad, host=host, turn=self._turn)
        if not defer:
            self.commit(staged)
        return staged

    def commit(self, staged: "Staged") -> None:
        """Starts the copy of a staged block to the device."""
        if staged.committed:
            return
        if staged.host is not self._host[staged.turn]:
            raise ValueError("the staging buffers were replaced since this block was staged")
        self._dev[: staged.total].copy_(staged.host[: staged.total], non_blocking=True)
        self.copied_bytes += 4 * staged.total
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
            self._events[staged.turn] = event
        staged.committed = True

    def _arange(self, count: int) -> np.ndarray:
        if self._range is None or len(self._range) < count:
            self._range = np.arange(max(count, 1024), dtype=np.int32)
        return self._range[:count]

    def context(self, staged: "Staged") -> StepContext:
        """Device views of what `stage` copied."""
        n, s, r, max_blocks, sizes, offsets = staged.n, staged.s, staged.r, staged.max_blocks, staged.sizes, staged.offsets
        dev = self._dev[: staged.total]
        views = [dev[offsets[i]: offsets[i + 1]] for i in range(len(sizes))]
        groups = [
            GroupView(views[FIRST_GROUP + 2 * g], views[FIRST_GROUP + 1 + 2 * g].view(s, max_blocks[g]), max_blocks[g])
            for g in range(self.num_groups)
        ]
        sampled = staged.sampled
        return StepContext(
            num_tokens=n, num_seqs=s, num_rows=r,
            token_ids=views[3], positions=views[4], seq_of_token=views[5], q_start=views[6],
            ctx_len=views[7], state_slot=views[8], seq_start=views[10], out_rows=views[9], groups=groups,
            storage=self.storage, max_q_len=max(staged.q_lens), min_q_len=min(staged.q_lens),
            max_ctx_len=max(staged.ctx_lens), q_lens=staged.q_lens, starts=staged.starts, slots=staged.slots,
            all_single=max(staged.q_lens) == 1,
            sample_temperature=views[1].view(torch.float32) if sampled else None,
            sample_top_p=views[2].view(torch.float32) if sampled else None,
            sample_seed=views[0].view(torch.int64) if sampled else None,
        )

    def _fill_general(self, entries, q_lens, parts, max_blocks, sampled, page, s):
        """Entries of any length: portions beside single tokens."""
        seeds, temps, top_ps = parts[0].view(np.int64), parts[1].view(np.float32), parts[2].view(np.float32)
        ids, pos, seq_of, q_start, ctx_arr, slot_arr, out_rows = parts[3:10]
        ctx_lens = [e.start + q for e, q in zip(entries, q_lens)]
        cursor = 0
        row = 0
        q_start[0] = 0
        for index, e in enumerate(entries):
            q = q_lens[index]
            ids[cursor: cursor + q] = e.tokens
            pos[cursor: cursor + q] = np.arange(e.start, e.start + q, dtype=np.int32)
            seq_of[cursor: cursor + q] = index
            q_start[index + 1] = cursor + q
            ctx_arr[index] = ctx_lens[index]
            slot_arr[index] = e.cache.slot
            for w in e.want:
                if not 0 <= w < q:
                    raise ValueError(f"wanted place {w} is outside the entry's {q} tokens")
                out_rows[row] = cursor + w
                if sampled:
                    temps[row], top_ps[row], seeds[row] = e.sampling
                row += 1
            cursor += q

        for g in range(self.num_groups):
            slots = parts[FIRST_GROUP + 2 * g]
            table_flat = parts[FIRST_GROUP + 1 + 2 * g]
            table_flat[:] = -1
            table2d = table_flat.reshape(s, max_blocks[g])
            cursor = 0
            for index, e in enumerate(entries):
                q = q_lens[index]
                pages = e.cache.tables[g].view()
                held = min(len(pages), max_blocks[g])
                table2d[index, :held] = pages[:held]
                p = pos[cursor: cursor + q]
                page_of = pages[p // page]
                if (page_of < 0).any():
                    raise ValueError(f"entry {index} writes into a page of group {g} it no longer holds")
                slots[cursor: cursor + q] = page_of * page + p % page
                cursor += q

