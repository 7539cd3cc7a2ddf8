"""The ragged batch of one step, as the parts and kernels see it.

A step runs the next tokens of some requests as one flat batch of ``T`` tokens:
portions of prompts beside single decoded tokens, cut anywhere.  All integer
metadata is packed into one pinned host buffer and copied to the device once.
The reference passes flat ``tokens/positions/seq_ids`` the same way
(src/inference.cu:190-198) but only ever sends whole prompts or one token per
sequence (src/main.cpp:211-219,269-274).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import numpy as np
import torch


PREFILL_TILE_ROWS = 64     # query rows per block of the prompt-portion attention kernel (mma.sync)
PREFILL_TILE_ROWS_BIG = 128    # the same for the tcgen05 kernel


@dataclass(frozen=True)
class StepEntry:
    """The next ``tokens`` of request ``req_id``; ``want`` lists the places among these
    tokens (0-based) whose logits are asked for."""
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


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
    # device tensors, int32
    token_ids: torch.Tensor          # [T]
    positions: torch.Tensor          # [T] absolute position of each token in its request
    req_of_tok: torch.Tensor         # [T] row of the token's request in the tables below
    cu_q: torch.Tensor               # [R+1] first token of each request in the flat batch
    q_start_dev: torch.Tensor        # [R] position of each request's first new token
    ctx_len_dev: torch.Tensor        # [R] length of each request after this step
    logit_rows: torch.Tensor         # [K] flat token indices whose logits are wanted
    state_slots: torch.Tensor        # [R] state slot of each request
    decode_rows: torch.Tensor        # flat indices of tokens that are their request's only token
    chunk_rows: torch.Tensor         # flat indices of the tokens of requests that bring several
    chunk_tiles: torch.Tensor        # [n, 3] {request row, first flat token, rows} in tiles of 64
    chunk_tiles_big: torch.Tensor    # the same in tiles of 128
    max_position: int = 0            # the model's longest context (bounds that do not vary by step)
    packed_size: int = 0             # int32 values in the packed device buffer
    block_tables: list[torch.Tensor] = field(default_factory=list)   # per group [R, blocks]
    scratch: dict = field(default_factory=dict)   # what kernels derive from the step, kept for one forward pass


def build_step_batch(entries: Sequence[StepEntry], starts: Sequence[int],
                     tables: Sequence[Sequence[Sequence[int]]], slots: Sequence[int],
                     act_dtype: torch.dtype, device, min_blocks: int = 1,
                     max_position: int = 0, dev_buffer: Optional[torch.Tensor] = None) -> StepBatch:
    """Pack one step.  ``starts[r]`` is the position of entry r's first token,
    ``tables[g][r]`` its block table in group g (already covering the new tokens).

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
    dec = [int(cu[i]) for i in range(r) if q_lens[i] == 1]
    chk_parts = [np.arange(cu[i], cu[i + 1]) for i in range(r) if q_lens[i] > 1]
    chk = np.concatenate(chk_parts) if chk_parts else np.zeros(0, dtype=np.int64)
    def tile_list(rows_per_tile):
        found = []
        for i in range(r):
            if q_lens[i] > 1:
                for lo in range(0, q_lens[i], rows_per_tile):
                    found.append((starts[i] + lo, i, int(cu[i]) + lo, min(rows_per_tile, q_lens[i] - lo)))
        found.sort(key=lambda x: -x[0])               # longest contexts first
        return [x[1:] for x in found]

    tiles = tile_list(PREFILL_TILE_ROWS)
    tiles_big = tile_list(PREFILL_TILE_ROWS_BIG)
    widths = [max(min_blocks, max((len(tb) for tb in grp), default=0)) for grp in tables]
    total = 4 * t + (r + 1) + 3 * r + k + 3 * len(tiles) + 3 * len(tiles_big) + sum(r * w for w in widths)
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
        "dec": put(np.asarray(dec, dtype=np.int64), len(dec)),
        "chk": put(chk, len(chk)),
        "tiles": put(np.asarray(tiles, dtype=np.int64).reshape(-1), 3 * len(tiles)),
        "tiles_big": put(np.asarray(tiles_big, dtype=np.int64).reshape(-1), 3 * len(tiles_big)),
    }
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
        token_ids=view("tok"), positions=view("pos"), req_of_tok=view("roft"), cu_q=view("cu"),
        q_start_dev=view("qs"), ctx_len_dev=view("ctx"), logit_rows=view("rows"),
        state_slots=view("slots"), decode_rows=view("dec"), chunk_rows=view("chk"),
        chunk_tiles=view("tiles").view(-1, 3), chunk_tiles_big=view("tiles_big").view(-1, 3),
        max_position=max_position, packed_size=host.shape[0],
        block_tables=[dev[a:b].view(r, w) for (a, b), w in bt_spans])
