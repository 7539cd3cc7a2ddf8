"""Compile the CUDA sources of ``csrc/`` for sm_100a with nvcc and load them with ctypes.

Libraries are built on first use, in-tree under ``_build/`` (or under the temporary
folder when the tree is read-only), one ``.so`` per library below, and rebuilt when a
source, a header or a flag changes.  Only the library that is asked for is compiled,
so a float32 engine does not wait for the bfloat16 tensor-core kernels.  While nvcc
runs, a line is printed to stderr every few seconds.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

# library name -> sources (each library is self-contained and links common.cu)
LIBRARIES = {
    "core": ["common.cu", "rowwise.cu", "gemm_simple.cu", "attention_simple.cu", "sampling.cu"],
    "bf16": ["common.cu", "gemm_skinny.cu", "gemm_tcgen05.cu", "gemm_tcgen05_2sm.cu",
             "gemm_tcgen05_few.cu", "ffn_decode.cu", "attn_decode.cu", "attn_prefill.cu", "attn_prefill_tc.cu",
             "attn_prefill_tc2.cu"],
}

# libraries that parts bring themselves: name -> (absolute source paths, include folders)
_EXTRA: dict[str, tuple[list[str], list[str]]] = {}


def register_library(name: str, sources: list[str], include_dirs: list[str] = ()) -> None:
    """Make ``load_library(name)`` build and load CUDA sources that live outside ``csrc/``: a part
    with kernels of its own registers them from its module and binds the entry points itself.
    The sources may include the headers of ``csrc/`` (``common.cuh`` and the rest); they are
    compiled with the same flags, for sm_100a, into the same build folder."""
    if name in LIBRARIES:
        raise ValueError(f"library name {name!r} is taken by the engine's own kernels")
    paths = [os.path.abspath(p) for p in sources]
    for p in paths:
        if not os.path.isfile(p):
            raise BuildError(f"library {name!r}: source {p} does not exist")
    _EXTRA[name] = (paths, [os.path.abspath(d) for d in include_dirs])
    _LOADED.pop(name, None)


def _sources_of(name: str) -> tuple[list[str], list[str]]:
    """Absolute source paths and extra include folders of a library."""
    if name in LIBRARIES:
        return [os.path.join(CSRC, s) for s in LIBRARIES[name]], []
    if name in _EXTRA:
        return _EXTRA[name]
    known = ", ".join(sorted(list(LIBRARIES) + list(_EXTRA)))
    raise BuildError(f"no kernel library is named {name!r}; known: {known}")


NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("TINYINFER_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $TINYINFER_NVCC, $CUDA_HOME/bin, "
                     "/usr/local/cuda/bin and PATH); the CUDA kernels cannot be built")


def build_dir() -> str:
    """In-tree ``_build`` when it can be written, else a per-user folder under the temp dir."""
    override = os.environ.get("TINYINFER_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(os.path.dirname(CSRC), "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"tinyinfer_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for the compiled kernels: tried " + ", ".join(cands))


def _digest(sources: list[str], include_dirs: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    headers = []
    for d in [CSRC, *include_dirs]:
        headers += sorted(os.path.join(d, n) for n in os.listdir(d) if n.endswith((".cuh", ".h")))
    for path in list(sources) + headers:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _say(msg: str) -> None:
    print(f"[tinyinfer_b200] {msg}", file=sys.stderr, flush=True)


def _run_all(cmds: dict[str, list[str]], what: str) -> None:
    """Run the commands at once; report now and then; raise with the output of a failure."""
    start = time.time()
    procs = {n: subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for n, c in cmds.items()}
    outputs: dict[str, str] = {}
    last = start
    while procs:
        for n in list(procs):
            if procs[n].poll() is not None:
                outputs[n] = procs[n].communicate()[0]
                if procs[n].returncode != 0:
                    for other in procs.values():
                        if other.poll() is None:
                            other.kill()
                    raise BuildError(f"{what}: {n} failed\n$ {' '.join(cmds[n])}\n{outputs[n]}")
                del procs[n]
        if procs:
            time.sleep(0.2)
            if time.time() - last >= 5.0:
                last = time.time()
                _say(f"{what}: still compiling {', '.join(sorted(procs))} "
                     f"({int(last - start)} s)")


def build_library(name: str, verbose: bool = True) -> str:
    """Make sure ``lib<name>`` is built and current; returns the path of the ``.so``."""
    sources, include_dirs = _sources_of(name)
    out_dir = build_dir()
    so_path = os.path.join(out_dir, f"libtinyinfer_b200_{name}.so")
    stamp = so_path + ".sha256"
    digest = _digest(sources, include_dirs)
    with open(os.path.join(out_dir, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(so_path) and os.path.isfile(stamp):
                with open(stamp) as fh:
                    if fh.read().strip() == digest:
                        return so_path
            nvcc = find_nvcc()
            if verbose:
                _say(f"compiling the '{name}' kernels for sm_100a ({len(sources)} files) "
                     f"into {out_dir}")
            t0 = time.time()
            objs = {}
            cmds = {}
            includes = [x for d in [CSRC, *include_dirs] for x in ("-I", d)]
            if name not in LIBRARIES:                  # ti_fail and friends live in common.cu
                sources = [os.path.join(CSRC, "common.cu"), *sources]
            for path in sources:
                src = os.path.basename(path)
                obj = os.path.join(out_dir, f"{name}_{os.path.splitext(src)[0]}.o")
                objs[src] = obj
                cmds[src] = [nvcc, *NVCC_FLAGS, *includes, "-c", path, "-o", obj]
            _run_all(cmds, f"'{name}' kernels")
            tmp = so_path + f".tmp{os.getpid()}"
            _run_all({"link": [nvcc, "-shared", "-o", tmp, *objs.values()]},
                     f"'{name}' kernels")
            os.replace(tmp, so_path)
            with open(stamp, "w") as fh:
                fh.write(digest)
            if verbose:
                _say(f"'{name}' kernels ready ({time.time() - t0:.0f} s)")
            return so_path
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_LOADED: dict[str, ctypes.CDLL] = {}


def load_library(name: str) -> ctypes.CDLL:
    if name not in _LOADED:
        _LOADED[name] = ctypes.CDLL(build_library(name))
    return _LOADED[name]


def build_all(verbose: bool = True) -> list[str]:
    return [build_library(n, verbose) for n in LIBRARIES]
