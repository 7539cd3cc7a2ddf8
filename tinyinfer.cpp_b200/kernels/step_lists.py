"""The integer lists that this kernel set's attention kernels want from every step.

A step's single-token rows go to the flash-decoding kernel and its prompt portions to the
prompt-attention kernels, which work on tiles of query rows whose height is the kernel's own
(asked from the compiled library, so the two cannot disagree).  The step builder knows none of
this: it packs whatever the builders below return (``engine.batch.StepList``).
"""
from __future__ import annotations

from functools import partial
from typing import Sequence

import numpy as np


def single_rows(q_lens: Sequence[int], starts: Sequence[int]) -> np.ndarray:
    """Flat indices of the tokens that are their request's only token in this step."""
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    return np.asarray([cu[i] for i, n in enumerate(q_lens) if n == 1], dtype=np.int64)


def portion_rows(q_lens: Sequence[int], starts: Sequence[int]) -> np.ndarray:
    """Flat indices of the tokens of requests that bring several tokens."""
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    parts = [np.arange(cu[i], cu[i + 1]) for i, n in enumerate(q_lens) if n > 1]
    return np.concatenate(parts) if parts else np.zeros(0, dtype=np.int64)


def portion_tiles(q_lens: Sequence[int], starts: Sequence[int], rows: int) -> np.ndarray:
    """``[n, 3]`` {request row, first flat token, rows} of the portions cut into tiles of ``rows``
    query rows, the tiles with the longest contexts first (they take longest)."""
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    found = []
    for i, n in enumerate(q_lens):
        if n > 1:
            for lo in range(0, n, rows):
                found.append((starts[i] + lo, i, int(cu[i]) + lo, min(rows, n - lo)))
    found.sort(key=lambda x: -x[0])
    return np.asarray([x[1:] for x in found], dtype=np.int64).reshape(-1, 3)


def attention_lists(tile_heights: Sequence[int]):
    from ..engine.batch import StepList
    out = [StepList("single_rows", single_rows), StepList("portion_rows", portion_rows)]
    for rows in sorted(set(tile_heights)):
        out.append(StepList(f"portion_tiles_{rows}", partial(portion_tiles, rows=rows), uses_starts=True))
    return out
