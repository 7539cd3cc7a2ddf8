"""Reader and writer for GGUF (versions 2 and 3), the second loader.

Layout, as the reference reads it (src/gguf_reader.cpp:31-82): magic ``GGUF``, version
(uint32), tensor count and metadata count (uint64), the metadata pairs (key string, value type,
value; strings are a uint64 length and bytes; arrays are an element type, a uint64 count and the
elements), the tensor infos (name, number of dimensions, dimensions with the contiguous one
first, ggml type, offset), then the tensor data from the next boundary of ``general.alignment``
(32 by default) bytes, each tensor at its offset from there.  Tensor types read here: F32 (0),
F16 (1) and BF16 (30); the reference accepts BF16 matrices and F32 norms only
(src/model.cpp:7-8,70,100).
"""
from __future__ import annotations

import mmap
import os
import struct
from typing import Any, Mapping

import torch

UINT8, INT8, UINT16, INT16, UINT32, INT32, FLOAT32, BOOL, STRING, ARRAY, UINT64, INT64, FLOAT64 = range(13)
_SCALARS = {UINT8: "<B", INT8: "<b", UINT16: "<H", INT16: "<h", UINT32: "<I", INT32: "<i",
            FLOAT32: "<f", BOOL: "<?", UINT64: "<Q", INT64: "<q", FLOAT64: "<d"}
GGML_F32, GGML_F16, GGML_BF16 = 0, 1, 30
_TENSOR_DTYPES = {GGML_F32: torch.float32, GGML_F16: torch.float16, GGML_BF16: torch.bfloat16}
_GGML_OF = {v: k for k, v in _TENSOR_DTYPES.items()}


class GgufError(ValueError):
    pass


class _Cursor:
    def __init__(self, buf, path):
        self.buf, self.pos, self.path = buf, 0, path

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError(f"{self.path}: file ends inside its header")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError(f"{self.path}: a string of {n} bytes runs past the end of the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def value(self, vtype):
        if vtype in _SCALARS:
            return self.take(_SCALARS[vtype])
        if vtype == STRING:
            return self.string()
        if vtype == ARRAY:
            etype, count = self.take("<I"), self.take("<Q")
            return [self.value(etype) for _ in range(count)]
        raise GgufError(f"{self.path}: unsupported metadata value type {vtype}")


class GgufFile:
    """A mapped GGUF file: ``metadata`` (key -> value), ``names()``, ``shape``, ``dtype``, ``get``."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as exc:
            raise GgufError(f"{path}: cannot open ({exc.strerror})") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 24:
            raise GgufError(f"{path}: too short to be a GGUF file")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        cur = _Cursor(memoryview(self._map), path)
        if bytes(cur.buf[:4]) != b"GGUF":
            raise GgufError(f"{path}: not a GGUF file (bad magic)")
        cur.pos = 4
        self.version = cur.take("<I")
        if self.version not in (2, 3):
            raise GgufError(f"{path}: unsupported GGUF version {self.version}")
        n_tensors, n_kv = cur.take("<Q"), cur.take("<Q")
        self.metadata: dict[str, Any] = {}
        for _ in range(n_kv):
            key = cur.string()
            self.metadata[key] = cur.value(cur.take("<I"))
        self._tensors: dict[str, dict] = {}
        for _ in range(n_tensors):
            name = cur.string()
            ne = [cur.take("<Q") for _ in range(cur.take("<I"))]
            ttype, offset = cur.take("<I"), cur.take("<Q")
            if ttype not in _TENSOR_DTYPES:
                raise GgufError(f"{path}: tensor {name!r} has ggml type {ttype}; only F32, F16 and "
                                "BF16 are read (no quantised formats)")
            self._tensors[name] = {"shape": tuple(reversed(ne)), "dtype": _TENSOR_DTYPES[ttype],
                                   "offset": offset}
        align = int(self.metadata.get("general.alignment", 32))
        self._data = -(-cur.pos // align) * align
        for name, t in self._tensors.items():
            numel = 1
            for s in t["shape"]:
                numel *= s
            t["nbytes"] = numel * torch.empty((), dtype=t["dtype"]).element_size()
            if self._data + t["offset"] + t["nbytes"] > size:
                raise GgufError(f"{path}: tensor {name!r} runs past the end of the file")

    def names(self) -> list[str]:
        return list(self._tensors)

    def shape(self, name: str) -> tuple[int, ...]:
        return self._tensors[name]["shape"]

    def dtype(self, name: str) -> torch.dtype:
        return self._tensors[name]["dtype"]

    def get(self, name: str) -> torch.Tensor:
        t = self._tensors[name]
        if t["nbytes"] == 0:
            return torch.empty(t["shape"], dtype=t["dtype"])
        start = self._data + t["offset"]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            flat = torch.frombuffer(memoryview(self._map)[start:start + t["nbytes"]], dtype=t["dtype"])
        return flat.reshape(t["shape"])

    def close(self) -> None:
        self._fh.close()


def _put_string(out: bytearray, s: str) -> None:
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _put_value(out: bytearray, value: Any) -> None:
    """Writes the value's type and the value; Python types choose the GGUF type."""
    if isinstance(value, bool):
        out += struct.pack("<I?", BOOL, value)
    elif isinstance(value, int):
        out += struct.pack("<II", UINT32, value) if 0 <= value < 2 ** 32 else struct.pack("<Iq", INT64, value)
    elif isinstance(value, float):
        out += struct.pack("<If", FLOAT32, value)
    elif isinstance(value, str):
        out += struct.pack("<I", STRING)
        _put_string(out, value)
    elif isinstance(value, (list, tuple)):
        etype = STRING if value and isinstance(value[0], str) else FLOAT32 if value and isinstance(
            value[0], float) else UINT32
        out += struct.pack("<IIQ", ARRAY, etype, len(value))
        for v in value:
            if etype == STRING:
                _put_string(out, v)
            else:
                out += struct.pack(_SCALARS[etype], v)
    else:
        raise GgufError(f"cannot write metadata value {value!r}")


def write_gguf(path: str, metadata: Mapping[str, Any], tensors: Mapping[str, torch.Tensor],
               version: int = 3, alignment: int = 32) -> None:
    head = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(metadata)))
    for key, value in metadata.items():
        _put_string(head, key)
        _put_value(head, value)
    offset = 0
    blobs = []
    for name, t in tensors.items():
        if t.dtype not in _GGML_OF:
            raise GgufError(f"tensor {name!r} has dtype {t.dtype}; GGUF tensors here are F32, F16 or BF16")
        _put_string(head, name)
        head += struct.pack("<I", t.dim())
        for s in reversed(t.shape):
            head += struct.pack("<Q", s)
        head += struct.pack("<IQ", _GGML_OF[t.dtype], offset)
        blob = t.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes()
        blob += b"\0" * (-len(blob) % alignment)
        blobs.append(blob)
        offset += len(blob)
    head += b"\0" * (-len(head) % alignment)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(head)
        for blob in blobs:
            fh.write(blob)
    os.replace(tmp, path)
