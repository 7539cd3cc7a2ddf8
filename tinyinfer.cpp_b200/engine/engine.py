"""The engine: a model, its kernels, its cache, and the one step function.

``Engine.step(entries)`` runs only the tokens it is given, as one batch, from
the cache that earlier steps left, and returns float32 logits at the wanted
places.  Everything above it (scheduler, generation, trace replay) goes through
this call.  The reference's counterpart is ``Inference::forward``
(src/inference.cu:178-265), which is tied to a contiguous per-sequence cache.
"""
from __future__ import annotations

import os
from typing import Any, Hashable, Mapping, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..config.registry import architecture_of, load_config
from ..parts.model import CausalLM
from ..weights.loader import load_gguf, load_model_weights, load_model_weights_gguf
from ..weights.random_init import random_tensor
from .batch import StepBatch, StepEntry, build_step_batch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"engine dtype must be bfloat16 or float32, got {dtype!r}") from None


class Engine:
    """A loaded model with its cache.

    model_dir    folder with ``config.json`` and ``model.safetensors``, or a ``.gguf`` file; or
    config+seed  a ``config.json`` dictionary and a seed: random weights made on the device.
    dtype        ``bfloat16``: the kernels and precisions of serving (bfloat16 activations and
                 cache, float32 residual stream, norms, softmax); ``float32``: everything in
                 true 32-bit arithmetic.
    max_tokens   how many tokens the cache holds over all live requests (each request's
                 count rounded up to whole pages); or ``num_pages`` directly.
    ops          the kernel set; by default the CUDA kernels, which must be available.
    step_graphs  replay steps of a shape seen before from CUDA graphs (``step`` then returns a
                 logits tensor that the next step of the same shape reuses).
    """

    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[Mapping[str, Any]] = None,
                 seed: Optional[int] = None, dtype="bfloat16", device="cuda:0",
                 page_size: int = 64, max_tokens: Optional[int] = None,
                 num_pages: Optional[int] = None, max_requests: int = 64, ops=None,
                 step_graphs: bool = False):
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        if ops is None:
            # a kernel set of its own: its switches and what it holds back belong to this engine
            from ..kernels import CudaOps
            ops = CudaOps(self.device)
        self.ops = ops
        gguf_file = None
        if model_dir is not None and os.path.isfile(model_dir):
            # a file instead of a folder: a GGUF model (the reference's own format)
            gguf_file, arch, gguf_cfg = load_gguf(model_dir)
            typed = arch.from_dict(gguf_cfg)
        elif model_dir is not None:
            arch, typed = load_config(model_dir)
        elif config is not None:
            arch = architecture_of(config)
            typed = arch.from_dict(config)
        else:
            raise ValueError("Engine needs a model folder, or a configuration and a seed")
        self.config = typed
        self.plan = arch.build_plan(typed)
        self.model = CausalLM(self.plan)
        if gguf_file is not None:
            try:
                load_model_weights_gguf(self.model, gguf_file, arch, self.device, ops)
            finally:
                gguf_file.close()
        elif model_dir is not None:
            load_model_weights(self.model, model_dir, self.device, ops)
        else:
            if seed is None:
                raise ValueError("random weights need a seed")
            expected = self.model.expected_tensors()
            self.model.load_weights(
                lambda name: random_tensor(seed, name, expected[name], device=self.device), ops)
        if num_pages is None:
            if max_tokens is None:
                max_tokens = self.plan.max_position
            # every live request may waste up to one page less a token
            num_pages = -(-max_tokens // page_size) + max_requests
        self.page_size = page_size
        self.cache = CacheManager(self.model.cache_specs(), page_size=page_size,
                                  num_pages=num_pages, max_requests=max_requests,
                                  kv_dtype=self.dtype, device=self.device)
        # what the kernel set and the parts want built on the host for every step
        wanted: dict = {}
        for sl in list(ops.step_lists(self.dtype) if hasattr(ops, "step_lists") else []) + \
                self.model.step_lists():
            wanted.setdefault(sl.name, sl)
        self.step_lists = list(wanted.values())
        self.last_batch: Optional[StepBatch] = None
        self._graphs = None
        self._step_graphs = None
        if step_graphs:
            from .graphs import StepGraphs
            self._step_graphs = StepGraphs(self)

    # ---- requests ------------------------------------------------------------------------
    def add_request(self, req_id: Hashable) -> None:
        self.cache.add_request(req_id)

    def finish(self, req_id: Hashable) -> None:
        """Give back everything the request holds."""
        self.cache.free_request(req_id)

    def length(self, req_id: Hashable) -> int:
        return self.cache.length(req_id)

    # ---- the step ------------------------------------------------------------------------
    def reserve(self, entries: Sequence[StepEntry]) -> list[int]:
        """Make room in the cache for the step's tokens, for all entries or for none."""
        return self.cache.reserve_step([(e.req_id, len(e.tokens)) for e in entries],
                                       self.plan.max_position)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; returns logits ``[wanted, vocab]`` in the order of entries and ``want``."""
        entries = list(entries)
        if not entries:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        vocab = self.plan.vocab_size
        for e in entries:
            ids = np.asarray(e.tokens, dtype=np.int64)
            if ids.size and (ids.min() < 0 or ids.max() >= vocab):
                bad = int(ids[(ids < 0) | (ids >= vocab)][0])
                raise ValueError(f"request {e.req_id!r}: token id {bad} is outside [0, {vocab})")
            for place in e.want:
                if not 0 <= int(place) < len(e.tokens):
                    raise IndexError(f"request {e.req_id!r}: wanted place {place} is outside its "
                                     f"{len(e.tokens)} tokens")
        starts = self.reserve(entries)
        tables = [[self.cache.block_table(g, e.req_id) for e in entries]
                  for g in range(len(self.cache.groups))]
        slots = [self.cache.state_slot(e.req_id) for e in entries]
        logits = None
        if self._step_graphs is not None:
            logits = self._step_graphs.run(entries, starts, tables, slots)
        if logits is None:
            batch = build_step_batch(entries, starts, tables, slots, self.dtype, self.device,
                                     max_position=self.plan.max_position, lists=self.step_lists)
            logits = self.forward(batch)
            self.last_batch = batch
        for e in entries:
            self.cache.release_passed(e.req_id)
        return logits

    def decode_step(self, entries: Sequence[StepEntry], device_tokens=None) -> torch.Tensor:
        """A step in which every request brings one token and wants its logits, replayed from a
        CUDA graph.  Returns ``[requests, vocab]``; the tensor is reused by the next call.
        With ``device_tokens`` (int32 on the device, one per entry, each a valid id) the entries'
        own tokens are placeholders and the step runs the given ones: the ids that the step
        before chose, fed back without a round trip through the host."""
        entries = list(entries)
        vocab = self.plan.vocab_size
        for e in entries:
            if len(e.tokens) != 1 or list(e.want) != [0]:
                raise ValueError("decode_step takes one token per request and wants its logits")
            if not 0 <= int(e.tokens[0]) < vocab:
                raise ValueError(f"request {e.req_id!r}: token id {e.tokens[0]} is outside [0, {vocab})")
        if not entries:
            return torch.empty((0, vocab), dtype=torch.float32, device=self.device)
        if device_tokens is not None and (device_tokens.dtype != torch.int32
                                          or tuple(device_tokens.shape) != (len(entries),)
                                          or device_tokens.device != self.device):
            raise ValueError("device_tokens must be int32 on the engine's device, one per entry")
        if self._graphs is None:
            from .graphs import DecodeGraphs
            self._graphs = DecodeGraphs(self)
        starts = self.reserve(entries)
        logits = self._graphs.run(entries, starts, device_tokens)
        for e in entries:
            self.cache.release_passed(e.req_id)
        return logits

    def forward(self, batch: StepBatch) -> torch.Tensor:
        views = {}
        for entry in self.plan.schedule:
            key = (entry.cache_slot, entry.writes_cache)
            if key not in views:
                views[key] = self.cache.view(entry.cache_slot, entry.writes_cache,
                                             batch.block_tables, batch.state_slots)
        return self.model.forward(self.ops, batch, views)
