"""Interfaces of the parts a decoder is put together from, and their registry.

Categories: ``norm``, ``position``, ``mixer``, ``ffn``, ``block``, ``embedding``,
``head``.  A part is built from a ``PartSpec`` (kind + parameters); it declares
the tensors it needs under names local to itself (``weight_specs``), receives
them once (``load_weights``), and then runs on device tensors through the
kernel set ``ops`` that the step hands it.  A part never sees the model's
configuration, its layer index or its checkpoint names.

Interfaces
----------
norm      ``forward(ops, x, out_dtype) -> h``; ``forward_rows(ops, x, rows, out_dtype)``.
position  ``rotation(device) -> Rotation``: the pairing rule, rotated width and table that the
          mixer hands on to the kernel that norms, rotates and stores its heads.
mixer     ``cache_spec()``: what it keeps per request (``PagedKVSpec``, ``FixedStateSpec`` or
          None); ``forward(ops, h, residual, step, cache)``: adds its output to ``residual``.
ffn       ``forward(ops, h, residual, step)``: adds its output to ``residual``.
block     arrangement of the four parts of a layer: ``forward(ops, x, step, cache)``.
embedding ``forward(ops, token_ids, out)``;  head ``forward(ops, h) -> logits``.

``h`` is the normed activation in the engine's activation dtype (bfloat16 or
float32); ``residual``/``x`` is the float32 residual stream ``[T, hidden]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional

import torch

from ..config.plan import PartSpec

MATRIX = "matrix"        # random mode: N(0, 0.02), stored in bfloat16
NORM_WEIGHT = "norm"     # random mode: 1 + N(0, 0.02), stored in float32


@dataclass(frozen=True)
class WeightSpec:
    shape: tuple[int, ...]
    init: str = MATRIX


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every past token (or of the last ``window`` tokens) in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: all keys are kept


@dataclass(frozen=True)
class FixedStateSpec:
    """Per-request state of fixed size, zero when a request starts."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    category = ""

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {}

    def load_weights(self, tensors: Mapping[str, torch.Tensor], ops: Any) -> None:
        """Take the tensors named in ``weight_specs`` (already on the device, dtype as stored)."""

    def step_lists(self) -> list:
        """Integer lists (``engine.batch.StepList``) that this part wants built on the host for
        every step and handed to it as ``step.lists[name]``."""
        return []

    def shared_weights(self) -> dict[str, torch.Tensor]:
        """Tensors another part may alias (for instance the embedding table for a tied head)."""
        return {}


_REGISTRY: dict[tuple[str, str], Callable[..., Part]] = {}
CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")


def register_part(category: str, kind: str, factory: Callable[..., Part]) -> None:
    """Make ``factory(**params)`` the builder of parts of ``kind`` in ``category``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; known: {', '.join(CATEGORIES)}")
    _REGISTRY[(category, kind)] = factory


def build_part(category: str, spec: PartSpec, **extra: Any) -> Part:
    try:
        factory = _REGISTRY[(category, spec.kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise ValueError(
            f"no {category} of kind {spec.kind!r} is registered; known: {', '.join(known)}") from None
    return factory(**dict(spec.params), **extra)


def as_float32(t: torch.Tensor) -> torch.Tensor:
    """Norm weights and tables are used in float32; widening bfloat16 is exact."""
    return t if t.dtype == torch.float32 else t.to(torch.float32)
