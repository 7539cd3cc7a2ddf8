"""Random weights from a configuration and a seed.

Matrices and embedding tables are N(0, 0.02); every norm weight is 1 + N(0, 0.02).
The generator is counter-based: element ``i`` of a tensor is a function of (seed, tensor name, i)
alone, made of integer arithmetic and two float32 operations, so a tensor's values do not depend
on which other tensors exist, in which order they are drawn or in how many pieces, and the CPU
and the GPU produce the same bits (an engine fills the 32B shape directly on the device, a test
writes the same model to a folder on the host).  A standard normal value is the sum of twelve
16-bit uniform integers taken from three rounds of a 64-bit mixing function (splitmix64's
finaliser) of the element's index, centred and scaled: exact in float32, mean 0, variance 1,
within 6 standard deviations.  ``write_random_model`` writes a model folder (``config.json`` and
``model.safetensors``; matrices in bfloat16, norm weights in float32 unless another storage dtype
is asked for); ``random_tensor`` serves engines that fill their weights directly on the device.
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
_PIECE = 1 << 24                   # elements drawn at once (bounds the integer temporaries)


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _signed(x: int) -> int:
    """A 64-bit pattern as the int64 that holds it."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


def _shift_right(z: torch.Tensor, k: int) -> torch.Tensor:
    """Logical shift of int64 patterns (torch's ``>>`` keeps the sign)."""
    return (z >> k) & ((1 << (64 - k)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    """splitmix64's finaliser on int64 patterns (multiplication wraps around)."""
    z = (z ^ _shift_right(z, 30)) * _signed(0xBF58476D1CE4E5B9)
    z = (z ^ _shift_right(z, 27)) * _signed(0x94D049BB133111EB)
    return z ^ _shift_right(z, 31)


def standard_normal(key: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """Elements ``start .. start + count`` of the stream that ``key`` names, float32."""
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    total = torch.zeros(count, dtype=torch.int64, device=device)
    for r in range(3):
        z = _mix((idx * 3 + r) * _signed(0x9E3779B97F4A7C15) + _signed(key))
        for shift in (0, 16, 32, 48):
            total += _shift_right(z, shift) & 0xFFFF if shift else z & 0xFFFF
    # twelve uniform integers of 0 .. 65535: mean 12 * 32767.5, variance 65536^2 (nearly)
    return (total - 393210).to(torch.float32) * (1.0 / 65536.0)


def random_tensor(seed: int, name: str, spec: WeightSpec, device="cpu",
                  dtype: torch.dtype | None = None) -> torch.Tensor:
    if spec.init == NORM_WEIGHT:
        default = torch.float32
    elif spec.init == MATRIX:
        default = torch.bfloat16
    else:
        raise ValueError(f"tensor {name!r}: unknown initialisation class {spec.init!r}")
    key = _tensor_seed(seed, name)
    numel = 1
    for d in spec.shape:
        numel *= int(d)
    out = torch.empty(numel, dtype=dtype or default, device=device)
    for start in range(0, numel, _PIECE):
        count = min(_PIECE, numel - start)
        t = standard_normal(key, start, count, device) * INIT_STD
        if spec.init == NORM_WEIGHT:
            t += 1.0
        out[start:start + count] = t.to(out.dtype)
    return out.view(tuple(spec.shape))


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
