"""Random weights from a configuration and a seed.

Matrices and embedding tables are N(0, 0.02); every norm weight is 1 + N(0, 0.02).
Each tensor has a generator of its own, seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or in which order they
are drawn.  ``write_random_model`` writes a model folder (``config.json`` and
``model.safetensors``; matrices in bfloat16, norm weights in float32 unless
another storage dtype is asked for); ``random_tensor`` serves engines that fill
their weights directly on the device.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Mapping

import torch

from ..config.registry import architecture_of
from ..parts.base import MATRIX, NORM_WEIGHT, WeightSpec
from ..parts.model import CausalLM
from .safetensors_io import write_safetensors

INIT_STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(seed: int, name: str, spec: WeightSpec, device="cpu",
                  dtype: torch.dtype | None = None) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    t.normal_(0.0, INIT_STD, generator=gen)
    if spec.init == NORM_WEIGHT:
        t += 1.0
        default = torch.float32
    elif spec.init == MATRIX:
        default = torch.bfloat16
    else:
        raise ValueError(f"tensor {name!r}: unknown initialisation class {spec.init!r}")
    return t.to(dtype or default)


def write_random_model(model_dir: str, config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype | None = None) -> None:
    """Write ``config.json`` and ``model.safetensors`` for the architecture ``config`` names."""
    arch = architecture_of(config)
    typed = arch.from_dict(config)
    model = CausalLM(arch.build_plan(typed))
    os.makedirs(model_dir, exist_ok=True)
    tensors = {name: random_tensor(seed, name, spec, dtype=dtype)
               for name, spec in model.expected_tensors().items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    cfg = typed.to_dict() if hasattr(typed, "to_dict") else dict(config)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=2)
        fh.write("\n")
