"""The scheduler: which requests run in the next step, and with how many tokens.

The policy is Azimml/shrike's (shrike/engine/scheduler.py:69-148), restated:

1. Running requests first, in admission order, while budget remains.  A request
   whose prompt is in the cache takes one token (this includes a resumed request
   replaying its generated history); one still in its prompt takes
   min(rest of prompt, budget) tokens, cut anywhere.
2. When the pages for that do not fit, the NEWEST running request is preempted:
   its pages and slot are given back, its computed count drops to 0 and it goes to
   the FRONT of the waiting queue.  If the request itself is the newest, it is the
   victim and sits this step out.  Nothing preempted was scheduled in this step:
   victims are always later in the list.
3. Waiting requests are admitted first-come first-served while budget, the
   running cap and pages allow; the head of the queue blocks those behind it.
4. Single tokens are listed before portions.

What happens when pages run out is therefore: preempt newest, recompute later.  A
request that could never fit is refused at admission by the engine.
"""

from __future__ import annotations

from collections import deque

from ..cache.manager import CacheManager
from .request import Request, Status


class Scheduler:
    def __init__(self, cache: CacheManager, max_tokens_per_step: int = 512, max_running: int = 256):
        self.cache = cache
        self.max_tokens_per_step = max_tokens_per_step
        self.max_running = max_running
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.num_preemptions = 0

    def add(self, request: Request) -> None:
        self.waiting.append(request)

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _release(self, request: Request) -> None:
        if request.cache is not None:
            self.cache.free(request.cache)
            request.cache = None

    def _preempt_newest(self, for_request: Request) -> bool:
        """Returns False when `for_request` itself was the victim."""
        victim = self.running.pop()
        self.num_preemptions += 1
        self._release(victim)
        victim.num_computed_tokens = 0
        victim.status = Status.WAITING
        self.waiting.appendleft(victim)
        return victim is not for_request

    def preempt_newest(self) -> Request | None:
        """Preempts the newest running request as a shortage of pages would (an operator's lever,
        and what tests of recomputation use); returns it, or None when nothing runs."""
        if not self.running:
            return None
        victim = self.running[-1]
        self._preempt_newest(victim)
        return victim

    def schedule(self) -> list[tuple[Request, int]]:
        singles: list[tuple[Request, int]] = []
        portions: list[tuple[Request, int]] = []
        budget = self.max_tokens_per_step
        longest = self.cache.portion_limit() or budget   # what a windowed group's pool can hold of one request

        for request in list(self.running):
            if budget == 0:
                break
            if request.status is not Status.RUNNING:
                continue
            if request.prefill_done:
                num_new = 1
            else:
                num_new = min(request.num_prompt_tokens - request.num_computed_tokens, budget, longest)
            if not self.cache.has_room(request.cache, request.num_computed_tokens + num_new):
                while not self.cache.can_append(request.cache, request.num_computed_tokens, num_new):
                    if not self._preempt_newest(request):
                        num_new = 0
                        break
                if num_new == 0:
                    continue
                self.cache.append(request.cache, request.num_computed_tokens, num_new)
            (singles if num_new == 1 else portions).append((request, num_new))
            budget -= num_new

        while self.waiting and budget > 0 and len(self.running) < self.max_running:
            request = self.waiting[0]
            num_new = min(request.num_prompt_tokens - request.num_computed_tokens, budget, longest)
            if not self.cache.can_append(None, request.num_computed_tokens, num_new):
                break
            self.waiting.popleft()
            request.cache = self.cache.open()
            self.cache.append(request.cache, request.num_computed_tokens, num_new)
            request.status = Status.RUNNING
            self.running.append(request)
            (singles if num_new == 1 else portions).append((request, num_new))
            budget -= num_new

        return singles + portions

    def postprocess(self, batch: list[tuple[Request, int]]) -> None:
        """After the step ran: the tokens are in the cache; windows move on."""
        for request, num_new in batch:
            request.num_computed_tokens += num_new
            if request.cache is not None:
                self.cache.advance(request.cache, request.num_computed_tokens)

    def finish(self, request: Request, reason: str) -> None:
        """Ends a request and gives back what it holds.  It is usually running; it may be waiting
        when it was preempted while the step that produced its last token was still in flight."""
        request.status = Status.FINISHED
        request.finish_reason = reason
        if request in self.running:
            self.running.remove(request)
        elif request in self.waiting:
            self.waiting.remove(request)
        self._release(request)

    def abort(self, request: Request) -> None:
        """Ends a request wherever it is (shrike/cli.py:131-141)."""
        self.finish(request, "aborted")
