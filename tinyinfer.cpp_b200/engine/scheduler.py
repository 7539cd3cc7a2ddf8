"""The scheduler: which tokens of which requests the next step runs.

The reference has no scheduler: all prompts (at most 16) are prefilled in one forward and
then every live sequence decodes one token per step (src/main.cpp:178,211-219,266-297).
Here requests wait in a queue and are admitted while request slots and pages last; a step
first takes one token of every request that is decoding, then gives the rest of its token
budget to prompt portions, oldest first, each at most ``chunk`` tokens.

When pages run out
------------------
A decoding request that needs a new page while none is free makes the scheduler *preempt*
the most recently admitted running request (possibly the needy one itself): its pages go
back, and it returns to the head of the waiting queue to be recomputed later from its
prompt and the tokens it has generated.  A prompt portion that does not fit is shortened
to the room there is, or waits.  A request that could never fit in the whole pool is
finished at once with reason ``"too_long"``.  If nothing at all can run, the newest running
request is preempted so that the oldest makes progress.  All of this is host-side and
deterministic.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    req_id: Hashable
    prompt: list[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    number: int = 0                 # arrival number, keys the request's random draws
    output: list[int] = field(default_factory=list)
    computed: int = 0               # tokens whose keys and values are in the cache
    state: str = WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def span(self, start: int, count: int) -> list[int]:
        """Tokens start .. start + count of prompt followed by output, without joining the two."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - n]

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed


@dataclass(frozen=True)
class Scheduled:
    """Run ``count`` tokens of ``request`` starting at its position ``start``; ``samples`` says
    that the portion ends at the request's last known token, so its next token is chosen."""
    request: Request
    start: int
    count: int
    samples: bool


class Scheduler:
    def __init__(self, cache, *, max_num_seqs: int, max_batched_tokens: int,
                 chunk: Optional[int] = None, max_position: int,
                 eos_token_ids: Sequence[int] = ()):
        if max_num_seqs < 1 or max_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_batched_tokens must be positive")
        if chunk is not None and chunk < 1:
            raise ValueError("chunk must be positive")
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_batched_tokens = max_batched_tokens
        self.chunk = chunk
        self.max_position = max_position
        self.eos = frozenset(eos_token_ids)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []          # in order of admission
        self.num_preemptions = 0
        self._arrivals = 0

    # ---- arrivals ------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        request.number = self._arrivals
        self._arrivals += 1
        if not request.prompt:
            raise ValueError(f"request {request.req_id!r} has an empty prompt")
        if len(request.prompt) > self.max_position:
            self._finish(request, "too_long")
            return
        # The longest the request can get must fit in an empty pool: all of it in a group that
        # keeps every key; in a group with a window, the window and a token more, with the pages
        # at both ends cut (portions are shortened to the room there is).  State of fixed size
        # needs no such check: every request slot has its state allocated from the start.
        most = min(self.max_position, len(request.prompt) + request.params.max_tokens)
        ps = self.cache.page_size
        for g in self.cache.groups:
            need = -(-most // ps)
            if g.spec.window is not None:
                need = min(need, -(-(g.spec.window + 1) // ps) + 1)
            if need > g.pool.count:
                self._finish(request, "too_long")
                return
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step ------------------------------------------------------------------------
    def schedule(self) -> list[Scheduled]:
        while True:
            plan = self._plan()
            if plan or not self.running:
                return plan
            self._preempt(self.running[-1])       # nothing fits: free the newest, retry

    def _plan(self) -> list[Scheduled]:
        budget = self.max_batched_tokens
        planned: list[Scheduled] = []
        taken = [0] * len(self.cache.groups)

        def room(req: Request, n: int) -> bool:
            need = self.cache.pages_needed(req.req_id, n)
            free = self.cache.free_pages()
            return all(k <= f - t for k, f, t in zip(need, free, taken))

        def take(req: Request, n: int) -> None:
            for g, k in enumerate(self.cache.pages_needed(req.req_id, n)):
                taken[g] += k
            planned.append(Scheduled(req, req.computed, n, req.computed + n == req.num_tokens))

        # 1. one token for every decoding request
        for req in list(self.running):
            if req.state != RUNNING or req.remaining != 1 or budget < 1:
                continue
            while req.state == RUNNING and not room(req, 1):
                victim = self.running[-1]
                if any(s.request is victim for s in planned):
                    break                         # only older, already planned ones are left
                self._preempt(victim)
            if req.state == RUNNING and room(req, 1):
                take(req, 1)
                budget -= 1
        # 2. prompt portions of running requests, oldest first
        for req in self.running:
            if req.remaining <= 1 or budget < 1 or any(s.request is req for s in planned):
                continue
            n = self._fit(req, min(req.remaining, budget, self.chunk or req.remaining), room)
            if n:
                take(req, n)
                budget -= n
        # 3. admissions
        while self.waiting and len(self.running) < self.max_num_seqs and budget > 0:
            req = self.waiting[0]
            n = min(req.remaining, budget, self.chunk or req.remaining)
            if self.cache.state_slots.num_free - sum(
                    1 for s in planned if not self.cache.has_request(s.request.req_id)) < 1:
                break
            if not room(req, n):
                break
            self.waiting.popleft()
            req.state = RUNNING
            self.running.append(req)
            take(req, n)
            budget -= n
        return planned

    def _fit(self, req: Request, n: int, room) -> int:
        """The largest count <= n whose pages are free (whole pages at a time)."""
        while n > 0 and not room(req, n):
            ps = self.cache.page_size
            length = self.cache.length(req.req_id) if self.cache.has_request(req.req_id) else 0
            end = ((length + n - 1) // ps) * ps          # drop the last, partial page
            n = max(0, end - length)
        return n

    def lookahead(self, plan: Sequence[Scheduled]) -> Optional[list[Scheduled]]:
        """The plan of the step after ``plan``, told while ``plan`` is still running and its tokens
        are unknown (its pages are reserved, ``step_done`` has not been called for it): one token
        for each of its requests, in the same order.  None unless that is certain but for a stop
        token: every request of ``plan`` is choosing a token now and none ends by its length,
        nothing waits for admission, and the pages are there.  A request that does stop on the
        unknown token runs one token too many in the step told here; ``step_done`` drops it."""
        if self.waiting or len(plan) != len(self.running):
            return None
        taken = [0] * len(self.cache.groups)
        free = self.cache.free_pages()
        told = []
        for s in plan:
            req = s.request
            if req.state != RUNNING or not s.samples:
                return None
            if (len(req.output) + 1 >= req.params.max_tokens
                    or req.num_tokens + 1 >= self.max_position):
                return None
            for g, k in enumerate(self.cache.pages_needed(req.req_id, 1)):
                taken[g] += k
                if taken[g] > free[g]:
                    return None
            told.append(Scheduled(req, s.start + s.count, 1, True))
        return told

    # ---- results -------------------------------------------------------------------------
    def step_done(self, plan: Sequence[Scheduled], sampled: Sequence[int]) -> list[Request]:
        """Account for a finished step; ``sampled`` holds one token per entry that samples, in
        plan order.  Returns the requests that finished.  An entry whose request stopped while
        the step was already running (``lookahead``) is dropped with its token."""
        finished = []
        it = iter(sampled)
        for s in plan:
            req = s.request
            tok = int(next(it)) if s.samples else None
            if req.state != RUNNING:
                continue
            req.computed += s.count
            if not s.samples:
                continue
            req.output.append(tok)
            reason = None
            if tok in self.eos or tok in req.params.stop_token_ids:
                reason = "stop"
            elif len(req.output) >= req.params.max_tokens:
                reason = "length"
            elif req.num_tokens >= self.max_position:
                reason = "context"
            if reason:
                self.running.remove(req)
                if self.cache.has_request(req.req_id):
                    self.cache.free_request(req.req_id)
                self._finish(req, reason)
                finished.append(req)
        return finished

    def _finish(self, req: Request, reason: str) -> None:
        req.state = FINISHED
        req.finish_reason = reason

    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        if self.cache.has_request(req.req_id):
            self.cache.free_request(req.req_id)
        req.computed = 0
        req.state = WAITING
        req.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)
