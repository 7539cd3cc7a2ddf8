"""The Python entry point: token ids in, generated token ids out.

``LLM`` owns an engine, a scheduler and a sampler and runs the loop the reference runs in
``main`` (prefill, then one token per live sequence per step, src/main.cpp:210-297), but over
the one step function: prompt portions and decoding tokens share batches, and requests
come and go while others are running.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence

import torch

from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .engine import Engine
from .scheduler import RUNNING, Request, Scheduler


@dataclass
class _InFlight:
    """A step on the device whose chosen ids the host has not read yet."""
    plan: list
    samplers: list
    ids: Any                # int32 on the device, one per sampling entry
    host: Any               # pinned; the copy of ``ids`` lands here
    read: Any               # event after that copy


@dataclass
class Generation:
    prompt: list[int]
    tokens: list[int]
    finish_reason: Optional[str]
    preemptions: int = 0


@dataclass
class RunStats:
    steps: int = 0
    prompt_tokens: int = 0        # tokens run as parts of prompts (recomputed ones included)
    decode_tokens: int = 0        # tokens run one at a time after a request's prompt
    generated: int = 0
    preemptions: int = 0
    seconds: float = 0.0
    step_log: list = field(default_factory=list)


class LLM:
    """model_dir or (config, seed); ``max_seq`` caps a request's context (the reference's
    ``--max-seq``, default 2048, src/main.cpp:131,150); the cache holds ``kv_tokens`` tokens
    (default ``max_num_seqs * max_seq``, what the reference allocates, src/inference.cu:146-148)."""

    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[Mapping[str, Any]] = None,
                 seed: Optional[int] = None, dtype="bfloat16", device="cuda:0",
                 max_seq: int = 2048, max_num_seqs: int = 16, max_batched_tokens: int = 2048,
                 chunk: Optional[int] = None, page_size: int = 64,
                 kv_tokens: Optional[int] = None, cuda_graph: bool = False, lookahead: bool = True,
                 ops=None):
        if kv_tokens is None:
            kv_tokens = max_num_seqs * max_seq
        self.engine = Engine(model_dir, config=config, seed=seed, dtype=dtype, device=device,
                             page_size=page_size, num_pages=-(-kv_tokens // page_size),
                             max_requests=max_num_seqs, ops=ops, step_graphs=cuda_graph)
        self.max_seq = min(max_seq, self.engine.plan.max_position)
        self.max_num_seqs = max_num_seqs
        self.max_batched_tokens = max_batched_tokens
        self.chunk = chunk
        self.cuda_graph = cuda_graph
        self.lookahead = lookahead        # with cuda_graph: launch a step before the last one's ids are read
        self.sampler = Sampler(self.engine.ops, self.engine.device)
        eos = getattr(self.engine.config, "eos_token_ids", ())
        self.eos_token_ids = tuple(eos)
        self.stats = RunStats()

    def start(self, prompts: Sequence[Sequence[int]],
              params: SamplingParams | Sequence[SamplingParams] = SamplingParams(),
              log_steps: bool = False) -> "Session":
        """Queue the prompts and return the running generation; ``Session.step()`` advances it by
        one engine step (for callers that stream tokens or measure steps)."""
        return Session(self, prompts, params, log_steps)

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: SamplingParams | Sequence[SamplingParams] = SamplingParams(),
                 log_steps: bool = False) -> list[Generation]:
        session = self.start(prompts, params, log_steps)
        while not session.done:
            session.step()
        return session.finish()


class Session:
    """One call of ``LLM.generate`` in progress."""

    def __init__(self, llm: LLM, prompts, params, log_steps: bool = False):
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        self.llm = llm
        self.log_steps = log_steps
        self.sched = Scheduler(llm.engine.cache, max_num_seqs=llm.max_num_seqs,
                               max_batched_tokens=llm.max_batched_tokens, chunk=llm.chunk,
                               max_position=llm.max_seq, eos_token_ids=llm.eos_token_ids)
        self.requests = [Request(req_id=("gen", i), prompt=[int(t) for t in p], params=sp)
                         for i, (p, sp) in enumerate(zip(prompts, params))]
        for r in self.requests:
            self.sched.add(r)
        self.stats = llm.stats = RunStats()
        self._t0 = time.perf_counter()
        self._pending: Optional[_InFlight] = None
        self._on_gpu = llm.engine.device.type == "cuda"
        self._host = [self._host_buffer(len(self.requests)) for _ in range(2)]
        self._turn = 0

    def _host_buffer(self, n: int):
        return torch.empty(max(n, 1), dtype=torch.int32, pin_memory=self._on_gpu)

    @property
    def done(self) -> bool:
        return self._pending is None and not self.sched.has_work()

    def _launch(self, plan, fed=None) -> "_InFlight":
        """Put one step and its sampling on the device.  ``fed``: the step before, still running,
        whose chosen ids (on the device) are this step's tokens."""
        llm, engine = self.llm, self.llm.engine
        samplers = [s for s in plan if s.samples]
        ahead = 0 if fed is None else 1           # tokens the host has not appended yet
        if fed is not None:
            entries = [StepEntry(s.request.req_id, [0], [0]) for s in plan]
            logits = engine.decode_step(entries, fed.ids)
        else:
            entries = []
            decoding = llm.cuda_graph
            for s in plan:
                toks = s.request.span(s.start, s.count)
                entries.append(StepEntry(s.request.req_id, toks, [s.count - 1] if s.samples else []))
                decoding = decoding and s.count == 1 and s.samples
            logits = engine.decode_step(entries) if decoding else engine.step(entries)
        ids = llm.sampler(logits, [s.request.params for s in samplers],
                          [s.request.number for s in samplers],
                          [len(s.request.output) + ahead for s in samplers])
        host = self._host[self._turn]
        self._turn = (self._turn + 1) % len(self._host)
        host[:len(samplers)].copy_(ids, non_blocking=True)
        read = None
        if self._on_gpu:
            read = torch.cuda.Event()
            read.record()
        return _InFlight(plan, samplers, ids, host, read)

    def step(self) -> list[tuple[int, int]]:
        """Advance by one engine step; returns (prompt index, token) for every token it generated.

        With CUDA graphs the step after this one is put on the device before this one's tokens are
        read, whenever the scheduler can tell it without them (``Scheduler.lookahead``); it takes
        its tokens from the device, and the host's work overlaps it."""
        llm, sched, stats = self.llm, self.sched, self.stats
        if self._pending is None:
            plan = sched.schedule()
            if not plan:
                raise RuntimeError("the scheduler found nothing to run although requests wait; "
                                   "the cache pool is too small for the oldest request")
            self._pending = self._launch(plan)
        cur = self._pending
        told = sched.lookahead(cur.plan) if llm.cuda_graph and llm.lookahead else None
        self._pending = self._launch(told, cur) if told else None
        if cur.read is not None:
            cur.read.synchronize()
        sampled = cur.host[:len(cur.samplers)].tolist()
        kept = [s.request.state == RUNNING for s in cur.samplers]
        stats.steps += 1
        for s in cur.plan:
            if s.request.state != RUNNING:
                continue                          # stopped while this step was already running
            if s.count == 1 and s.start >= len(s.request.prompt):
                stats.decode_tokens += 1
            else:
                stats.prompt_tokens += s.count
        stats.generated += sum(kept)
        if self.log_steps:
            stats.step_log.append([(s.request.req_id, s.start, s.count) for s in cur.plan])
        sched.step_done(cur.plan, sampled)
        return [(s.request.req_id[1], t) for s, t, k in zip(cur.samplers, sampled, kept) if k]

    def finish(self) -> list[Generation]:
        while self._pending is not None:          # a step told ahead of a request that stopped
            self.step()
        self.llm.engine.ops.check_status()
        self.stats.preemptions = self.sched.num_preemptions
        self.stats.seconds = time.perf_counter() - self._t0
        return [Generation(r.prompt, r.output, r.finish_reason, r.preemptions) for r in self.requests]
