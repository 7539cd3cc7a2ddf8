#!/usr/bin/env python3
"""Run the reference's own model code on the CPU and keep its logits as golden outputs.

    python tests/golden/make_golden.py [--reference /path/to/tinyinfer.cpp] [--check] [--asan]

beyondHJM/tinyinfer.cpp has no CPU model path: its arithmetic is CUDA kernels and its loader
calls cudaMalloc.  Here its untouched sources (src/gguf_reader.cpp, src/model.cpp,
src/inference.cu, src/cuda/*.cu) are copied to a temporary folder, the launches
``kernel<<<grid, block, smem, stream>>>(args)`` are rewritten to ``CPU_LAUNCH(kernel, grid,
block, args)``, the body of its one inline-PTX function (mma.sync m16n8k16, src/cuda/gemm.cu:142-150)
is replaced by a call of the stand-in's fragment arithmetic, and everything is compiled with g++
against ``cuda_on_cpu/`` (blocks and threads on host threads, warp shuffles, __syncthreads,
cudaMalloc on host memory).  Nothing else of the sources changes.

For each case below a tiny random model (head size 128, which the reference's attention
requires, src/cuda/attention.cu:321) is written as a GGUF file by this repository's writer, read
by the reference's own loader, and run by the reference's own ``Inference::forward``: a prompt in
one pass, then tokens one by one, a longer prompt, and two sequences in one batch.  The logits go to ``<case>.f32`` with
``<case>.json`` beside them (the configuration, the seed, the passes, a checksum of the
weights).  ``tests/test_golden.py`` rebuilds the same model from the seed and compares the plain
implementation with these files.  ``--check`` compares fresh outputs with the stored ones
instead of writing; ``--asan`` builds with the address sanitizer.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import re
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

SOURCES = ["src/gguf_reader.cpp", "src/model.cpp", "src/inference.cu", "src/cuda/attention.cu",
           "src/cuda/ffn.cu", "src/cuda/gemm.cu", "src/cuda/lm_head.cu", "src/cuda/rms_norm.cu",
           "src/cuda/sample.cu"]

ARCH = ["Qwen3ForCausalLM"]
# Every pass brings at most 32 tokens and every product has N a multiple of 32 and K a multiple
# of 256, so that the reference takes its small-M product (gemv2_bf16_kernel,
# src/cuda/gemm.cu:37-85,272-283) within what that kernel assumes: its threads take K / 8
# elements each, four 16-byte pieces at a time (src/cuda/gemm.cu:46,55-58), so a K that is no
# multiple of 256 makes them read into their neighbours' slices, and the sizes check at
# src/cuda/gemm.cu:276 asks for a multiple of 64 only (a model with 3 heads of 128 gave logits
# half the largest logit away from the plain implementation; with 4 heads it agrees).  Its tiled mma.sync product (src/cuda/gemm.cu:152-251), which
# larger passes and other sizes fall to, is left out on purpose: in the sources as they stand a
# warp's columns start at warp_col * WARP_COLS with WARP_COLS = TN / 2 = 32 for four column warps
# (src/cuda/gemm.cu:156,201), so the warps reach columns 64..111 of a 64-column tile: they read
# past the shared tile `Bs` and leave columns 16..31 and 48..63 of every tile unwritten.  Run
# here under the address sanitizer (--asan with a pass of more than 32 tokens) it is reported as
# an overflow of `Bs`; on a B200 the same pass ended with "an illegal memory access".
CASES = {
    "gqa": dict(config=dict(architectures=ARCH, num_hidden_layers=2, hidden_size=256, num_attention_heads=2,
                            num_key_value_heads=1, head_dim=128, intermediate_size=512, vocab_size=320,
                            rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                            max_position_embeddings=64),
                seed=21, prompt=20, decode=5, long_prompt=32, pair=(7, 11)),
    # other sizes and constants, no grouping of heads
    "mha": dict(config=dict(architectures=ARCH, num_hidden_layers=3, hidden_size=512, num_attention_heads=4,
                            num_key_value_heads=4, head_dim=128, intermediate_size=768, vocab_size=224,
                            rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
                            max_position_embeddings=64),
                seed=22, prompt=9, decode=4, long_prompt=31, pair=(3, 13)),
}


def split_top_level(text: str) -> list[str]:
    parts, depth, cur = [], 0, ""
    for ch in text:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur.strip())
            cur = ""
        else:
            cur += ch
    parts.append(cur.strip())
    return parts


def rewrite(text: str) -> str:
    """Launch syntax and the one inline-PTX statement; nothing else."""
    def launch(m):
        cfg = split_top_level(m.group(2))
        args = m.group(3).strip()
        return f"CPU_LAUNCH({m.group(1)}, {cfg[0]}, {cfg[1]}{', ' + args if args else ''});"
    text = re.sub(r"(\w+)\s*<<<(.*?)>>>\s*\((.*?)\);", launch, text, flags=re.S)
    text = re.sub(r"asm volatile\(\s*\"mma\.sync\.aligned\.m16n8k16.*?\);",
                  "cpu_mma_m16n8k16_bf16(a0, a1, a2, a3, b0, b1, c0, c1, c2, c3);", text, flags=re.S)
    return text


def build(reference: str, work: str, asan: bool) -> str:
    src = os.path.join(work, "src")
    shutil.copytree(os.path.join(reference, "src"), src)
    objs = []
    flags = ["-std=c++20", "-O1", "-pthread", "-D__CUDACC__", "-I", os.path.join(HERE, "cuda_on_cpu"),
             "-I", src, "-I", os.path.join(src, "cuda"), "-w"]
    if asan:
        flags += ["-fsanitize=address", "-g", "-fno-omit-frame-pointer"]
    units = [os.path.join(work, rel) for rel in SOURCES]
    for path in units:
        with open(path, "r", encoding="utf-8") as fh:
            text = rewrite(fh.read())
        if "<<<" in text or "asm volatile" in text:
            raise SystemExit(f"{path}: a launch or inline assembly was left unrewritten")
        out = os.path.splitext(path)[0] + "_cpu.cpp"
        with open(out, "w", encoding="utf-8") as fh:
            fh.write(text)
        objs.append(out)
    exe = os.path.join(work, "run_reference")
    cmd = ["g++", *flags, os.path.join(HERE, "run_reference.cpp"), os.path.join(HERE, "cuda_on_cpu", "simt.cpp"),
           *objs, "-o", exe]
    subprocess.run(cmd, check=True)
    return exe


def model_files(case: dict, work: str, name: str):
    """The case's random model as a folder (for the plain implementation) and as the GGUF file
    the reference reads; returns (folder, gguf path, config, weights, checksum of the weights)."""
    from plain_qwen3 import load_folder
    from tinyinfer_b200 import write_random_model
    from tinyinfer_b200.config import Qwen3Config
    from tinyinfer_b200.config.qwen3 import gguf_metadata, gguf_tensor_name
    from tinyinfer_b200.weights import write_gguf
    folder = os.path.join(work, f"model_{name}")
    write_random_model(folder, case["config"], seed=case["seed"])
    cfg, w = load_folder(folder)
    digest = hashlib.sha256()
    for key in sorted(w):
        digest.update(key.encode())
        digest.update(w[key].contiguous().view(-1).view(dtype=__import__("torch").uint8).numpy().tobytes())
    gguf = os.path.join(work, f"{name}.gguf")
    write_gguf(gguf, gguf_metadata(Qwen3Config.from_dict(cfg)), {gguf_tensor_name(n): t for n, t in w.items()})
    return folder, gguf, cfg, w, digest.hexdigest()


def passes_of(case: dict) -> list[dict]:
    """The forward passes of a case: what goes in, and which (sequence, position) logits come out."""
    from util import random_tokens
    vocab = case["config"]["vocab_size"]
    n, d = case["prompt"], case["decode"]
    a = random_tokens(vocab, n + d, seed=case["seed"] * 10 + 1)
    long_seq = random_tokens(vocab, case["long_prompt"], seed=case["seed"] * 10 + 2)
    pa, pb = case["pair"]
    b0 = random_tokens(vocab, pa, seed=case["seed"] * 10 + 3)
    b1 = random_tokens(vocab, pb, seed=case["seed"] * 10 + 4)
    passes = [dict(name="prompt", reset=True, seqs={0: (0, a[:n])})]
    for i in range(d):
        passes.append(dict(name=f"decode{i}", reset=False, seqs={0: (n + i, [a[n + i]])}))
    passes.append(dict(name="long_prompt", reset=True, seqs={0: (0, long_seq)}))
    passes.append(dict(name="pair", reset=True, seqs={0: (0, b0), 1: (0, b1)}))
    passes.append(dict(name="pair_decode", reset=False, seqs={0: (pa, [5]), 1: (pb, [9])}))
    return passes, {"a": a, "long": long_seq, "b0": b0 + [5], "b1": b1 + [9]}


def plan_text(passes: list[dict], max_seq: int) -> str:
    lines = [f"{max_seq} 2"]
    for p in passes:
        items = []
        # the reference takes the tokens of all sequences of a pass flat, sequence after sequence
        for s, (start, toks) in sorted(p["seqs"].items()):
            items += [f"{s}:{start + i}:{t}" for i, t in enumerate(toks)]
        lines.append(f"{len(p['seqs'])} " + " ".join(items))
    return "\n".join(lines) + "\n"


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--reference", default=os.environ.get("TINYINFER_REFERENCE", os.path.join(ROOT, "baseline", "_ref", "src")),
                    help="the reference's tree (default: $TINYINFER_REFERENCE, else baseline/_ref/src)")
    ap.add_argument("--check", action="store_true", help="compare with the stored files instead of writing")
    ap.add_argument("--asan", action="store_true", help="build with the address sanitizer")
    ap.add_argument("--keep", action="store_true", help="keep the temporary folder and print its path")
    ap.add_argument("--only", default=None, help="one case only")
    ap.add_argument("--long-pass", type=int, default=0, metavar="TOKENS",
                    help="instead of the cases: run one pass of this many tokens of case 'gqa' and write nothing "
                         "(more than 32 tokens reach the reference's tiled product; with --asan it reports the overflow)")
    args = ap.parse_args()
    import numpy as np
    work = tempfile.mkdtemp(prefix="golden_")
    try:
        exe = build(args.reference, work, args.asan)
        worst = 0.0
        if args.long_pass:
            from util import random_tokens
            case = CASES["gqa"]
            _, gguf, cfg, _, _ = model_files(case, work, "gqa")
            toks = random_tokens(cfg["vocab_size"], args.long_pass, seed=1)
            plan = os.path.join(work, "long.plan")
            with open(plan, "w") as fh:
                fh.write(plan_text([dict(seqs={0: (0, toks)})], max(64, args.long_pass)))
            return subprocess.run([exe, gguf, plan, os.path.join(work, "long.f32")]).returncode
        for name, case in CASES.items():
            if args.only and name != args.only:
                continue
            _, gguf, cfg, _, checksum = model_files(case, work, name)
            passes, _ = passes_of(case)
            plan = os.path.join(work, f"{name}.plan")
            with open(plan, "w") as fh:
                fh.write(plan_text(passes, cfg["max_position_embeddings"]))
            out = os.path.join(work, f"{name}.f32")
            subprocess.run([exe, gguf, plan, out], check=True, stdout=subprocess.DEVNULL)
            data = np.fromfile(out, dtype="<f4")
            rows = sum(len(p["seqs"]) for p in passes)
            assert data.size == rows * cfg["vocab_size"], (data.size, rows)
            meta = dict(case=name, config=case["config"], seed=case["seed"], weights_sha256=checksum,
                        rows=[[p["name"], s] for p in passes for s in sorted(p["seqs"])],
                        made_by="tests/golden/make_golden.py: the reference's src/model.cpp, src/inference.cu and "
                                "src/cuda/*.cu compiled with g++ against tests/golden/cuda_on_cpu")
            if args.check:
                old = np.fromfile(os.path.join(HERE, f"{name}.f32"), dtype="<f4")
                diff = float(np.abs(old - data).max())
                worst = max(worst, diff)
                print(f"{name}: max difference from the stored logits {diff:.3e}")
            else:
                shutil.copy(out, os.path.join(HERE, f"{name}.f32"))
                with open(os.path.join(HERE, f"{name}.json"), "w") as fh:
                    json.dump(meta, fh, indent=1)
                    fh.write("\n")
                print(f"{name}: wrote {rows} rows of {cfg['vocab_size']} logits")
        return 1 if worst > 1e-5 else 0
    finally:
        if args.keep:
            print("kept", work)
        else:
            shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
