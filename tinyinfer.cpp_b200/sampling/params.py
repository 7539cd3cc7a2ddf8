"""Sampling options of one request, with the reference's names and meanings where it has them.

temperature  ``-t``: 0 (the default) is greedy, the first maximum winning ties
             (src/main.cpp:24,31-38; GPU: src/cuda/sample.cu:5-11).  Above 0 the logits are
             divided by it before the softmax.  (The reference subtracts the unscaled maximum
             after scaling, src/main.cpp:57-60, which overflows for small temperatures; here
             the maximum is taken after scaling.)
top_k        ``--top-k``: keep the k largest logits; 0 keeps the whole vocabulary.  (The
             reference's 0 silently means 512, src/main.cpp:47-55.)
top_p        ``--top-p``: keep the shortest run of most likely tokens whose probability
             reaches p, the crossing one included (src/main.cpp:63-73); 1.0 keeps all.
seed         ``--seed``: default 42 (src/main.cpp:27).  A request's draws depend on the seed,
             on the request's number and on how many tokens it has drawn, never on what else
             is in the batch.  (The reference shares one generator among all sequences,
             src/main.cpp:75-83, so its draws depend on the batch order.)
max_tokens   ``-n``: new tokens per request, default 128 (src/main.cpp:129,138).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 42
    max_tokens: int = 128
    stop_token_ids: tuple[int, ...] = ()

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0.0
