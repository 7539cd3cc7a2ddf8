"""Reader and writer for the safetensors container, by tensor name.

Layout of a file: an unsigned 64-bit little-endian header length ``n``, ``n``
bytes of JSON mapping each tensor name to ``{"dtype", "shape",
"data_offsets": [begin, end]}`` (offsets relative to the end of the header),
then the raw little-endian tensor bytes.  The reader maps the file and hands
out tensors that alias the mapping; nothing is converted here.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterable, Mapping

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A mapped safetensors file; ``names()``, ``shape(name)``, ``dtype(name)``, ``get(name)``."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as exc:
            raise SafetensorsError(f"{path}: cannot open ({exc.strerror})") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a header")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON ({exc})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        self._entries: dict[str, dict] = {}
        for name, ent in header.items():
            dt = ent.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            shape = tuple(int(s) for s in ent["shape"])
            begin, end = (int(v) for v in ent["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if end - begin != want or begin < 0 or self._base + end > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} {dt} needs {want} bytes, "
                    f"its offsets [{begin}, {end}) give {end - begin} (file has {size - self._base})")
            self._entries[name] = {"dtype": _DTYPES[dt], "shape": shape, "begin": begin, "end": end}
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self._entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self._entries[name]["shape"]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name]["dtype"]

    def get(self, name: str) -> torch.Tensor:
        """The tensor as stored (a read-only view of the mapping; clone or copy before writing)."""
        ent = self._entries[name]
        nbytes = ent["end"] - ent["begin"]
        if nbytes == 0:
            return torch.empty(ent["shape"], dtype=ent["dtype"])
        buf = memoryview(self._map)[self._base + ent["begin"]: self._base + ent["end"]]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # torch warns that the buffer is read-only
            flat = torch.frombuffer(buf, dtype=ent["dtype"])
        return flat.reshape(ent["shape"])

    def close(self) -> None:
        # Tensors handed out alias the mapping; it is released when they are gone.
        self._fh.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> None:
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = list(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {t.dtype}, which the format lacks")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> list[SafetensorsFile]:
    """Every ``*.safetensors`` file of a model folder (``model.safetensors`` or shards)."""
    names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"{model_dir}: holds no .safetensors file")
    return [SafetensorsFile(os.path.join(model_dir, n)) for n in names]


def tensor_index(files: Iterable[SafetensorsFile]) -> dict[str, SafetensorsFile]:
    index: dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.names():
            if name in index:
                raise SafetensorsError(f"tensor {name!r} is stored in {index[name].path} and {f.path}")
            index[name] = f
    return index
