"""Bindings of the hand-written CUDA kernels (sm_100a)."""
from .build import BuildError, build_all, build_library, load_library, register_library
from .cuda_ops import CudaOps, KernelError

_OPS: dict[str, CudaOps] = {}


def cuda_ops(device) -> CudaOps:
    """A kernel set for ``device`` that callers share (tests of single kernels, tools); an engine
    makes its own ``CudaOps``, so that its switches are its own.  Raises if CUDA or the compiled
    library is missing."""
    key = str(device)
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]


__all__ = ["BuildError", "CudaOps", "KernelError", "build_all", "build_library", "cuda_ops",
           "load_library", "register_library"]
