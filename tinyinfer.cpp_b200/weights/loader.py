"""Load a model's tensors from a folder by tensor name, and say clearly what does not fit.

Storage precision is never narrowed: bfloat16 stays bfloat16, float32 stays
float32, float16 and float64 become float32, integer tables become int32.  The
reference loads tensor by tensor and stops at the first problem
(src/model.cpp:63-117); here the whole folder is checked first and one error
lists every missing tensor, every unexpected tensor and every wrong shape.
"""
from __future__ import annotations

import warnings
from typing import Mapping

import torch

from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsError, open_model_files, tensor_index


class WeightsError(ValueError):
    """The folder's tensors do not match what the model needs."""

    def __init__(self, where: str, missing, unexpected, wrong_shape):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)          # (name, expected, found)
        lines = [f"{where}: tensors do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        super().__init__("\n".join(lines))


def check_tensors(where: str, expected: Mapping[str, WeightSpec],
                  found: Mapping[str, tuple[int, ...]],
                  duplicates: Mapping[str, str] = {}) -> None:
    """``duplicates``: names that may be present although the model does not need them, each
    with the expected tensor it repeats; such a tensor is not "unexpected", but it must have the
    shape of the one it repeats."""
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected and n not in duplicates]
    wrong = [(n, expected[n].shape, found[n]) for n in expected
             if n in found and tuple(found[n]) != tuple(expected[n].shape)]
    wrong += [(n, expected[of].shape, found[n]) for n, of in duplicates.items()
              if n in found and n not in expected and of in expected
              and tuple(found[n]) != tuple(expected[of].shape)]
    if missing or unexpected or wrong:
        raise WeightsError(where, missing, unexpected, wrong)


def _same_values(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and a.dtype == b.dtype and torch.equal(a, b)


def storage_dtype(dtype: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor is kept in."""
    if dtype in (torch.bfloat16, torch.float32):
        return dtype
    if dtype.is_floating_point:
        return torch.float32
    return torch.int32


def load_model_weights(model, model_dir: str, device, ops) -> None:
    """Check the folder against ``model.expected_tensors()`` and hand each part its tensors."""
    files = open_model_files(model_dir)
    try:
        index = tensor_index(files)
        expected = model.expected_tensors()
        duplicates = model.duplicate_tensors() if hasattr(model, "duplicate_tensors") else {}
        check_tensors(model_dir, expected, {n: f.shape(n) for n, f in index.items()}, duplicates)
        for name, of in duplicates.items():
            if name in index and of in index and not _same_values(index[name].get(name),
                                                                  index[of].get(of)):
                warnings.warn(f"{model_dir}: {name} is stored beside {of} although the two are "
                              f"tied, and its values differ; {of} is used", stacklevel=2)

        def fetch(name: str) -> torch.Tensor:
            t = index[name].get(name)
            return t.to(device=device, dtype=storage_dtype(t.dtype), copy=True)

        model.load_weights(fetch, ops)
    finally:
        for f in files:
            f.close()


def load_gguf(path: str):
    """Open a GGUF file; returns ``(file, architecture, config.json dictionary)``."""
    from ..config.registry import ConfigError, get_architecture
    from .gguf import GgufFile
    f = GgufFile(path)
    name = f.metadata.get("general.architecture")
    if not isinstance(name, str):
        raise ConfigError(f"{path}: GGUF metadata lacks 'general.architecture'")
    arch = get_architecture(name)
    if arch.config_from_gguf is None:
        raise ConfigError(f"architecture {name!r} has no GGUF support")
    cfg = arch.config_from_gguf(f.metadata, {n: f.shape(n) for n in f.names()})
    return f, arch, cfg


def load_model_weights_gguf(model, gguf_file, arch, device, ops) -> None:
    """As ``load_model_weights``, from an open GGUF file; names in errors are the file's own."""
    expected = model.expected_tensors()
    to_gguf = {name: arch.gguf_tensor_name(name) for name in expected}
    check_tensors(gguf_file.path, {to_gguf[n]: spec for n, spec in expected.items()},
                  {n: gguf_file.shape(n) for n in gguf_file.names()})

    def fetch(name: str) -> torch.Tensor:
        t = gguf_file.get(to_gguf[name])
        return t.to(device=device, dtype=storage_dtype(t.dtype), copy=True)

    model.load_weights(fetch, ops)


__all__ = ["SafetensorsError", "load_gguf", "load_model_weights_gguf", "WeightsError", "check_tensors", "load_model_weights",
           "storage_dtype"]
