"""Requests and their sampling parameters.

Names, defaults and bounds follow Azimml/shrike (shrike/engine/request.py:10-79):
`SamplingParams(max_new_tokens=128, temperature=0.0, top_p=1.0, ignore_eos=False)`
validated at construction; a `Request` keeps prompt and generated tokens in one
list, counts the tokens whose keys and values are in the cache, and has a status.
Added here: `seed`, so that a request's sampled tokens do not depend on what else
is in the batch, and the request's `cache` (block tables and state slot) in place
of a bare `block_table`.
"""

from __future__ import annotations

import enum
import itertools
from dataclasses import dataclass, field


class Status(enum.Enum):
    WAITING = enum.auto()
    RUNNING = enum.auto()
    FINISHED = enum.auto()


@dataclass
class SamplingParams:
    """Per-request decoding controls.

    max_new_tokens: most tokens to generate (>= 1); reaching it ends the request
        with reason "length".
    temperature: 0 selects the largest logit (lowest index on ties); otherwise the
        softmax of logits / temperature is sampled.  Must be >= 0.
    top_p: in (0, 1]; keeps the most probable tokens while the mass before a token
        is below top_p (the most probable is always kept).  Ignored when greedy.
    ignore_eos: keep generating past an end-of-sequence token.
    seed: None draws one from the engine's seed and the request id.
    """

    max_new_tokens: int = 128
    temperature: float = 0.0
    top_p: float = 1.0
    ignore_eos: bool = False
    seed: int | None = None

    def __post_init__(self) -> None:
        problems = []
        if not self.max_new_tokens >= 1:
            problems.append(f"max_new_tokens={self.max_new_tokens!r}: a request generates at least one token")
        if not self.temperature >= 0.0:
            problems.append(f"temperature={self.temperature!r}: zero (greedy) or a positive number")
        if not 0.0 < self.top_p <= 1.0:
            problems.append(f"top_p={self.top_p!r}: a probability mass above 0 and at most 1")
        if problems:
            raise ValueError("SamplingParams: " + "; ".join(problems))


_request_ids = itertools.count()


@dataclass(eq=False)
class Request:
    token_ids: list[int]
    sampling: SamplingParams
    req_id: int = field(default_factory=lambda: next(_request_ids))
    status: Status = Status.WAITING
    num_prompt_tokens: int = 0
    num_computed_tokens: int = 0
    cache: object | None = None  # cache.RequestCache while pages or a slot are held
    finish_reason: str | None = None

    def __post_init__(self):
        self.num_prompt_tokens = len(self.token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def prefill_done(self) -> bool:
        return self.num_computed_tokens >= self.num_prompt_tokens

    @property
    def num_generated(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def block_table(self) -> list[int]:
        """Pages of the first cache group, as Azimml/shrike's `Request.block_table`."""
        if self.cache is None or not self.cache.tables:
            return []
        return self.cache.tables[0].tolist()
