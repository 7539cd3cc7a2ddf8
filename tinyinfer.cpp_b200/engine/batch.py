"""The ragged batch of one step, as the parts and kernels see it.

A step runs the next tokens of some requests as one flat batch of ``T`` tokens:
portions of prompts beside single decoded tokens, cut anywhere.  All integer
metadata is packed into one pinned host buffer and copied to the device once.
The reference passes flat ``tokens/positions/seq_ids`` the same way
(src/inference.cu:190-198) but only ever sends whole prompts or one token per
sequence (src/main.cpp:211-219,269-274).

What a kernel needs beyond that description (which flat tokens are single-token rows, how
portions fall into its tiles) is not known here: the kernel set and the parts register
``StepList`` builders, and the step packs what they return into the same upload.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Hashable, Optional, Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class StepEntry:
    """The next ``tokens`` of request ``req_id``; ``want`` lists the places among these
    tokens (0-based) whose logits are asked for."""
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass(frozen=True)
class StepList:
    """A list of integers that a kernel set or a part derives on the host from a step's shape:
    which flat tokens are single-token rows, how portions are cut into a kernel's tiles, and
    the like.  ``build(q_lens, starts)`` gets every entry's token count and first position and
    returns an integer array of one or two dimensions.  Its shape may depend on the token
    counts only, never on the positions: a step of the same shape is replayed from a CUDA graph
    over the same addresses, with only the contents renewed.  ``uses_starts`` says whether the
    contents depend on the positions at all (a list that does not is built once per graph).
    The step hands each list out as ``step.lists[name]`` (int32 on the device)."""
    name: str
    build: Callable[[Sequence[int], Sequence[int]], np.ndarray]
    uses_starts: bool = False


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    num_logit_rows: int
    act_dtype: torch.dtype
    # host copies (launch geometry, kernel choice)
    q_lens: list[int]
    q_starts: list[int]
    ctx_lens: list[int]
    max_q_len: int
    max_ctx_len: int
    # how far back the requests that bring several tokens reach (0: at most SHORT_CONTEXT keys,
    # 1: at most LONG_CONTEXT, 2: further): kernels may choose by it (a step's graph is kept per
    # class, since the choice is captured with it)
    portion_reach: int
    # device tensors, int32
    token_ids: torch.Tensor          # [T]
    positions: torch.Tensor          # [T] absolute position of each token in its request
    req_of_tok: torch.Tensor         # [T] row of the token's request in the tables below
    cu_q: torch.Tensor               # [R+1] first token of each request in the flat batch
    q_start_dev: torch.Tensor        # [R] position of each request's first new token
    ctx_len_dev: torch.Tensor        # [R] length of each request after this step
    logit_rows: torch.Tensor         # [K] flat token indices whose logits are wanted
    state_slots: torch.Tensor        # [R] state slot of each request
    max_position: int = 0            # the model's longest context (bounds that do not vary by step)
    packed_size: int = 0             # int32 values in the packed device buffer
    block_tables: list[torch.Tensor] = field(default_factory=list)   # per group [R, blocks]
    lists: dict = field(default_factory=dict)     # name -> int32 device tensor of a registered StepList
    scratch: dict = field(default_factory=dict)   # what kernels derive from the step, kept for one forward pass


def build_lists(lists: Sequence[StepList], q_lens: Sequence[int], starts: Sequence[int]) -> dict:
    """Every list's array for a step of these token counts and first positions."""
    out = {}
    for sl in lists:
        arr = np.asarray(sl.build(q_lens, starts))
        if arr.size and arr.dtype.kind not in "iu":
            raise TypeError(f"step list {sl.name!r} must hold integers, got {arr.dtype}")
        if arr.ndim not in (1, 2):
            raise ValueError(f"step list {sl.name!r} must have one or two dimensions")
        if sl.name in out:
            raise ValueError(f"two step lists are named {sl.name!r}")
        out[sl.name] = arr.astype(np.int64, copy=False)
    return out


SHORT_CONTEXT = 1536    # keys: up to here a prompt portion's attention walks few tiles of keys
LONG_CONTEXT = 6144     # keys: from here on it is a long walk


def portion_reach(q_lens, ctx_lens) -> int:
    """The class of a step by the longest context of a request that brings several tokens:
    0 up to SHORT_CONTEXT keys (or no such request), 1 up to LONG_CONTEXT, 2 beyond."""
    far = max((c for n, c in zip(q_lens, ctx_lens) if n > 1), default=0)
    return 0 if far <= SHORT_CONTEXT else 1 if far <= LONG_CONTEXT else 2


def build_step_batch(entries: Sequence[StepEntry], starts: Sequence[int],
                     tables: Sequence[Sequence[Sequence[int]]], slots: Sequence[int],
                     act_dtype: torch.dtype, device, min_blocks: int = 1,
                     max_position: int = 0, dev_buffer: Optional[torch.Tensor] = None,
                     lists: Sequence[StepList] = ()) -> StepBatch:
    """Pack one step.  ``starts[r]`` is the position of entry r's first token,
    ``tables[g][r]`` its block table in group g (already covering the new tokens);
    ``lists`` are the integer lists that the kernel set and the parts have asked for.

    The packed layout depends only on the entries' token counts and wanted places once
    ``min_blocks`` fixes the block tables' width.  ``dev_buffer`` (int32, at least
    ``packed_size`` long) receives the integers instead of a fresh device tensor, so that a
    captured graph finds a later step of the same shape at the same addresses."""
    q_lens = [len(e.tokens) for e in entries]
    r = len(entries)
    t = sum(q_lens)
    ctx = [s + n for s, n in zip(starts, q_lens)]
    cu = np.zeros(r + 1, dtype=np.int64)
    np.cumsum(q_lens, out=cu[1:])
    rows: list[int] = []
    for i, e in enumerate(entries):
        for w in e.want:
            if not 0 <= w < q_lens[i]:
                raise IndexError(
                    f"request {e.req_id!r}: wanted place {w} is outside its {q_lens[i]} tokens")
            rows.append(int(cu[i]) + int(w))
    k = len(rows)
    extra = build_lists(lists, q_lens, list(starts))
    widths = [max(min_blocks, max((len(tb) for tb in grp), default=0)) for grp in tables]
    total = (3 * t + (r + 1) + 3 * r + k + sum(a.size for a in extra.values())
             + sum(r * w for w in widths))
    host = torch.empty(max(total, 1), dtype=torch.int32,
                       pin_memory=(torch.device(device).type == "cuda"))
    buf = host.numpy()
    o = 0

    def put(values, n):
        nonlocal o
        buf[o:o + n] = values
        span = (o, o + n)
        o += n
        return span

    tok = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]) if t else np.zeros(0, dtype=np.int64)
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, q_lens)]) if t else tok
    roft = np.repeat(np.arange(r), q_lens)
    spans = {
        "tok": put(tok, t), "pos": put(pos, t), "roft": put(roft, t), "cu": put(cu, r + 1),
        "qs": put(np.asarray(starts, dtype=np.int64), r), "ctx": put(np.asarray(ctx), r),
        "slots": put(np.asarray(slots, dtype=np.int64), r), "rows": put(np.asarray(rows), k),
    }
    list_spans = {name: (put(a.reshape(-1), a.size), a.shape) for name, a in extra.items()}
    bt_spans = []
    for grp, w in zip(tables, widths):
        arr = np.full((r, w), -1, dtype=np.int64)
        for i, tb in enumerate(grp):
            arr[i, :len(tb)] = tb
        bt_spans.append((put(arr.reshape(-1), r * w), w))
    if dev_buffer is None:
        dev = host.to(device, non_blocking=True)
    else:
        dev = dev_buffer[:host.shape[0]]
        dev.copy_(host, non_blocking=True)

    def view(name):
        a, b = spans[name]
        return dev[a:b]

    return StepBatch(
        num_tokens=t, num_requests=r, num_logit_rows=k, act_dtype=act_dtype,
        q_lens=q_lens, q_starts=list(starts), ctx_lens=ctx,
        max_q_len=max(q_lens, default=0), max_ctx_len=max(ctx, default=0),
        portion_reach=portion_reach(q_lens, ctx),
        token_ids=view("tok"), positions=view("pos"), req_of_tok=view("roft"), cu_q=view("cu"),
        q_start_dev=view("qs"), ctx_len_dev=view("ctx"), logit_rows=view("rows"),
        state_slots=view("slots"),
        max_position=max_position, packed_size=host.shape[0],
        block_tables=[dev[a:b].view(r, w) for (a, b), w in bt_spans],
        lists={name: dev[a:b].view(shape) for name, ((a, b), shape) in list_spans.items()})
