"""CUDA-graph replay of decode steps.

A step in which every request brings exactly one token and wants its logits has a fixed
shape once the batch is padded to a bucket (1, 2, 4, ... requests).  For each bucket the
whole forward is captured once over static device buffers (token ids, positions, block
tables, lengths); a later step copies its integers into those buffers with one transfer
and replays the graph.  Padding rows use the cache's null page, so they touch no request.
Kernels take everything that varies between steps from device memory, and a row's result
does not depend on the batch around it, so replay gives the same logits as the eager step.
The reference captures one graph per decode batch size (src/inference.cu:267-295) and
checks replay against eager the same way (src/inference.cu:297-341).
"""
from __future__ import annotations

import gc
import weakref
from typing import Sequence

import numpy as np
import torch

from .batch import StepBatch, StepEntry, build_lists, build_step_batch


def capture(graph: "torch.cuda.CUDAGraph", run):
    """Capture ``run()`` into ``graph`` and return what it returns.  Python's cycle collector
    stays off meanwhile and runs once before: an old engine it finds (engines and their graphs
    refer to each other) would destroy CUDA graphs and free device memory in the middle of the
    capture, which CUDA refuses and which makes the capture invalid."""
    gc.collect()
    was_on = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            return run()
    finally:
        if was_on:
            gc.enable()


def bucket_of(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class _Bucket:
    def __init__(self, engine, size: int):
        cache = engine.cache
        dev = engine.device
        self.size = size
        self.width = -(-engine.plan.max_position // cache.page_size)
        groups = len(cache.groups)
        b = size
        # the lists that kernels and parts want of a step: those that depend on the token counts
        # only are built once, those that also depend on the positions travel with every step
        ones, zeros = [1] * b, [0] * b
        fixed = build_lists([sl for sl in engine.step_lists if not sl.uses_starts], ones, zeros)
        self.moving = [sl for sl in engine.step_lists if sl.uses_starts]
        moving = build_lists(self.moving, ones, zeros)
        self.moving = [sl for sl in self.moving if moving[sl.name].size]
        # layout of the packed integers: tok, pos, ctx, slots, the moving lists (all of which
        # change with every step), then one block table per group (of which a step changes little)
        self.moving_at = {}
        at = 4 * b
        for sl in self.moving:
            self.moving_at[sl.name] = (at, moving[sl.name].shape)
            at += moving[sl.name].size
        self.head = at
        self.total = self.head + groups * b * self.width
        # a ring of pinned staging buffers: one is rewritten only after the copy that read it
        # has run on the device (the host runs ahead of the device by several steps)
        self.hosts = [torch.empty(self.total, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self.copied = [None] * len(self.hosts)
        self.turn = 0
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=dev)
        d = self.dev
        ar = torch.arange(b, dtype=torch.int32, device=dev)
        tables = [d[self.head + g * b * self.width: self.head + (g + 1) * b * self.width].view(b, self.width)
                  for g in range(groups)]
        self.batch = StepBatch(
            num_tokens=b, num_requests=b, num_logit_rows=b, act_dtype=engine.dtype,
            q_lens=[1] * b, q_starts=[0] * b, ctx_lens=[engine.plan.max_position] * b,
            max_q_len=1, max_ctx_len=engine.plan.max_position, portion_reach=0,
            token_ids=d[0:b], positions=d[b:2 * b], req_of_tok=ar,
            cu_q=torch.arange(b + 1, dtype=torch.int32, device=dev),
            q_start_dev=d[b:2 * b], ctx_len_dev=d[2 * b:3 * b], logit_rows=ar,
            state_slots=d[3 * b:4 * b],
            max_position=engine.plan.max_position, block_tables=tables)
        for name, arr in fixed.items():
            self.batch.lists[name] = torch.from_numpy(arr.astype(np.int32)).to(dev)
        for name, arr in moving.items():
            if name in self.moving_at:
                lo, shape = self.moving_at[name]
                self.batch.lists[name] = d[lo:lo + arr.size].view(shape)
            else:                                           # empty for steps of single tokens
                self.batch.lists[name] = torch.from_numpy(arr.astype(np.int32)).to(dev)
        self.graph = None
        self.logits = None
        self.launches = 0
        # host mirror of the packed integers and what each row holds
        self.mirror = np.zeros(self.total, dtype=np.int32)
        self.row_req: list = [None] * b
        self.row_version = [0] * b
        self.row_blocks = [[0] * groups for _ in range(b)]
        # per group the span of its table that the device has not seen yet: [first, past the last]
        self.stale = [[self.total, 0] for _ in range(groups)]
        self.last_copy_ints = 0
        self.copied_ints = 0               # all integers sent to the device so far
        for i in range(b):
            self._reset_row(i, cache)
            self.row_req[i] = _PADDING

    def fill(self, engine, entries: Sequence[StepEntry], starts: Sequence[int],
             device_tokens=None) -> None:
        """Stage the step's integers and start their copy to the device.  A host mirror keeps what
        the rows held last time: a request that sits in the same row as before only gets the
        block-table entries it has gained since (decoding adds a page every ``page_size`` steps).
        ``device_tokens`` (int32, one per entry, on the device) replaces the entries' tokens: the
        ids the previous step chose, which the host has not read yet."""
        cache = engine.cache
        b, w = self.size, self.width
        n = len(entries)
        m = self.mirror
        for i, e in enumerate(entries):
            req = e.req_id
            if self.row_req[i] != req or cache.table_version(req) != self.row_version[i]:
                self._reset_row(i, cache)
                self.row_req[i] = req
                self.row_version[i] = cache.table_version(req)
                m[3 * b + i] = cache.state_slot(req)
            have = self.row_blocks[i]
            for g in range(len(cache.groups)):
                tb = cache.block_table(g, req)
                if len(tb) > have[g]:
                    base = self.head + g * b * w + i * w
                    m[base + have[g]: base + len(tb)] = tb[have[g]:]
                    self._touched(g, base + have[g], base + len(tb))
                    have[g] = len(tb)
        for i in range(n, b):                                   # padding rows
            if self.row_req[i] is not _PADDING:
                self._reset_row(i, cache)
                self.row_req[i] = _PADDING
        m[0:n] = [int(e.tokens[0]) for e in entries]
        m[b:b + n] = starts
        m[2 * b:2 * b + n] = m[b:b + n] + 1
        if self.moving:
            now = build_lists(self.moving, [1] * b, list(starts) + [0] * (b - n))
            for name, arr in now.items():
                lo, shape = self.moving_at[name]
                if arr.shape != shape:
                    raise ValueError(f"step list {name!r} changed its shape with the positions")
                m[lo:lo + arr.size] = arr.reshape(-1)
        turn = self.turn
        self.turn = (turn + 1) % len(self.hosts)
        if self.copied[turn] is not None:
            self.copied[turn].synchronize()
        host = self.hosts[turn]
        staged = host.numpy()
        # only what changed travels: the head, and of each table the span that was written
        spans = [(0, self.head)] + [(lo, hi) for lo, hi in self.stale if lo < hi]
        self.last_copy_ints = 0
        for lo, hi in spans:
            staged[lo:hi] = m[lo:hi]
            self.dev[lo:hi].copy_(host[lo:hi], non_blocking=True)
            self.last_copy_ints += hi - lo
        self.copied_ints += self.last_copy_ints
        for span in self.stale:
            span[0], span[1] = self.total, 0
        if device_tokens is not None:
            self.dev[0:n].copy_(device_tokens)
        done = torch.cuda.Event()
        done.record()
        self.copied[turn] = done

    def _reset_row(self, i: int, cache) -> None:
        """Row ``i`` as a padding row: token 0 at position 0 of a request of one token that owns
        the spare state slot and only null pages."""
        b, w, m = self.size, self.width, self.mirror
        m[i] = 0
        m[b + i] = 0
        m[2 * b + i] = 1
        m[3 * b + i] = cache.max_requests
        for g in range(len(cache.groups)):
            base = self.head + g * b * w + i * w
            # a row that held fewer blocks than its width has null pages behind them already
            used = w if self.row_req[i] is None else max(self.row_blocks[i][g], 0)
            m[base:base + used] = cache.null_page
            self._touched(g, base, base + used)
        self.row_blocks[i] = [0] * len(cache.groups)

    def _touched(self, group: int, lo: int, hi: int) -> None:
        if lo < hi:
            span = self.stale[group]
            span[0], span[1] = min(span[0], lo), max(span[1], hi)


_PADDING = object()


class _OfEngine:
    """Keeps its engine by a weak reference: the engine owns this object, and a cycle between the
    two would leave the engine's graphs and device memory to the cycle collector."""

    def __init__(self, engine):
        self._engine = weakref.ref(engine)

    @property
    def engine(self):
        return self._engine()


class DecodeGraphs(_OfEngine):
    def __init__(self, engine):
        super().__init__(engine)
        self.buckets: dict[int, _Bucket] = {}

    def run(self, entries: Sequence[StepEntry], starts: Sequence[int],
            device_tokens=None) -> torch.Tensor:
        eng = self.engine
        size = bucket_of(len(entries))
        bk = self.buckets.get(size)
        if bk is None:
            bk = self.buckets[size] = _Bucket(eng, size)
        bk.fill(eng, entries, starts, device_tokens)
        if bk.graph is None:
            # run this step once outside capture (loads kernels, sizes the allocator), then capture
            side = torch.cuda.Stream(device=eng.device)
            side.wait_stream(torch.cuda.current_stream(eng.device))
            with torch.cuda.stream(side):
                first = eng.forward(bk.batch)
            torch.cuda.current_stream(eng.device).wait_stream(side)
            torch.cuda.synchronize(eng.device)
            graph = torch.cuda.CUDAGraph()
            before = getattr(eng.ops, "launches", 0)
            bk.logits = capture(graph, lambda: eng.forward(bk.batch))
            bk.graph = graph
            bk.launches = getattr(eng.ops, "launches", 0) - before
            # This step has run, eagerly, just now.  Replaying it as well would run it twice: the
            # cache pages would be written with the same values again, but a mixer with state of
            # its own would advance that state a second time.
            bk.logits.copy_(first)
            return bk.logits[:len(entries)]
        bk.graph.replay()
        if hasattr(eng.ops, "launches"):
            eng.ops.launches += bk.launches
        return bk.logits[:len(entries)]


class StepGraphs(_OfEngine):
    """CUDA-graph replay of whole steps of any shape (prompt portions, mixed batches).

    A step's launches depend only on its entries' token counts and wanted places: positions,
    block tables and everything else are data in one packed device buffer.  A shape that has
    been seen before is captured (after running eagerly once more); later steps of that shape
    copy their integers into the graph's buffer and replay it, which removes the host's work of
    launching some hundreds of kernels.  The least recently used graphs are dropped beyond
    ``capacity``.  The logits tensor of a shape is reused by its next replay.
    """

    def __init__(self, engine, capacity: int = 8):
        from collections import Counter, OrderedDict
        super().__init__(engine)
        self.capacity = capacity
        self.graphs: "OrderedDict[tuple, dict]" = OrderedDict()
        self.seen: Counter = Counter()
        self.width = -(-engine.plan.max_position // engine.cache.page_size)

    def run(self, entries, starts, tables, slots):
        """Logits of the step, or None if the step should run eagerly (a shape seen for the first time)."""
        eng = self.engine
        from .batch import portion_reach
        lens = [len(e.tokens) for e in entries]
        key = (tuple(lens), tuple(tuple(e.want) for e in entries),
               portion_reach(lens, [s + n for s, n in zip(starts, lens)]))
        ent = self.graphs.get(key)
        build = dict(act_dtype=eng.dtype, device=eng.device, min_blocks=self.width,
                     max_position=eng.plan.max_position, lists=eng.step_lists)
        if ent is not None:
            self.graphs.move_to_end(key)
            build_step_batch(entries, starts, tables, slots, dev_buffer=ent["buffer"], **build)
            ent["graph"].replay()
            if hasattr(eng.ops, "launches"):
                eng.ops.launches += ent["launches"]
            return ent["logits"]
        self.seen[key] += 1
        if self.seen[key] < 2:
            return None
        probe = build_step_batch(entries, starts, tables, slots, **build)
        buffer = torch.zeros(probe.packed_size, dtype=torch.int32, device=eng.device)
        batch = build_step_batch(entries, starts, tables, slots, dev_buffer=buffer, **build)
        logits = eng.forward(batch)                    # this step, eagerly
        torch.cuda.synchronize(eng.device)
        graph = torch.cuda.CUDAGraph()
        before = getattr(eng.ops, "launches", 0)
        static_logits = capture(graph, lambda: eng.forward(batch))
        self.graphs[key] = {"graph": graph, "buffer": buffer, "logits": static_logits,
                            "launches": getattr(eng.ops, "launches", 0) - before}
        while len(self.graphs) > self.capacity:
            self.graphs.popitem(last=False)
        return logits
