#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096]
    python bench.py --impl reference        # the reference arm (see below)

Default run: the Qwen3-0.6B layer sizes (28 layers, hidden 1024, 16 heads over 8 kv heads of
128, intermediate 3072, vocabulary 151936, tied head) with seeded random weights, 8 requests
decoding at a context of 4,096 tokens, pages of 64 tokens.  A step is one decode step of the
whole batch.  Prints one JSON line:

value      decoded tokens a second, timed on the device with CUDA events over K graph-replayed
           steps with the argmax on the device (nothing is read back inside the timed region);
e2e        the same through the Python entry point (LLM.start and Session.step, after the prompts
           have run): every step schedules, copies its host token ids and block tables to the
           device from pinned memory, decodes, samples and reads the chosen tokens back;
prefill    one request's 2,048-token prompt in one step: tokens a second and the step's
           flops / time / bf16 peak;
roofline   the bytes a decode step has to read (every weight once, and the keys and values of
           the live requests) / its time, against the copy bandwidth;
points     decode tokens a second at batch 1 and 64, the same steps without a CUDA graph, a mixed
           step (63 requests decoding beside a 512-token portion of a prompt that ends between
           3,072 and 4,096 tokens); then, as `page16_*`, `8b_*` and
           `32b_*`, the page size of 16 tokens and the Qwen3-8B and Qwen3-32B shapes (decode at
           batch 1, 8, 64, the 2,048-token prefill, the 8B mixed step);
points_frac  for each point its fraction of its roofline (decode: bytes / time / copy bandwidth;
           prefill: flops / time / the bf16 peak, the sustained one for steps over 5 ms).

Peaks come from MEASURED_PEAKS.json beside this file when present, else from an earlier
measurement on this pool (6.65 TB/s, 1.59 PFLOP/s), and the fractions say which.  The working
set (1.2 GB of weights and gigabytes of cache) is far larger than the 126 MB L2, so no flush is
needed between steps.  Keys and values of the decoding requests are filled with random numbers
instead of being computed from prompts: a decode step's work does not depend on their values.

The reference arm (``--impl reference``): beyondHJM/tinyinfer.cpp is a CMake project of C++/CUDA
executables, not a Python package, so the offline `pip install` fails ("Neither 'setup.py' nor
'pyproject.toml' found").  Its command-line program is instead built from an untouched copy of
its tree under ``baseline/_ref/src`` with its own CMakeLists (sm_100) into
``baseline/_ref/build/tinyinfer`` and run through its own command line on a GGUF file of the same
shape with seeded random weights: ``--batch`` prompts of three tokens each, decoded greedily to
the context length with ``--cuda-graph``.  Its prompts stay this short because a pass of more than
32 tokens takes its tiled mma.sync product, which reads past its shared tile as the sources
stand (src/cuda/gemm.cu:156,201: found by reading and by running that code on the CPU under the
address sanitizer, tests/golden/make_golden.py --asan --long-pass 40; on a B200 such a pass ended
with an illegal memory access) and is therefore never run here.  The number it reports is its own
("main: decode: ... tok/s", src/main.cpp:306-308): tokens a second over the whole decode, from a
context of 3 to the full one, where this engine's `value` is taken at the full context.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_0_6B = dict(
    architectures=["Qwen3ForCausalLM"], num_hidden_layers=28, hidden_size=1024,
    num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
    max_position_embeddings=4096)
# the two larger shapes of the same architecture (untied heads)
QWEN3_8B = dict(QWEN3_0_6B, num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, intermediate_size=12288, tie_word_embeddings=False)
QWEN3_32B = dict(QWEN3_0_6B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 num_key_value_heads=8, intermediate_size=25600, tie_word_embeddings=False)
SHAPES = {"0.6b": ("Qwen3-0.6B shape", QWEN3_0_6B), "8b": ("Qwen3-8B shape", QWEN3_8B),
          "32b": ("Qwen3-32B shape", QWEN3_32B)}
PAGE = 64
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
MAX_POSITION = 40960           # the longest context of the published models of this architecture


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS), "fallback"


def flops_peak(pk, ms):
    """The bf16 peak a step of `ms` milliseconds is held against: the burst figure for a short
    step, the figure sustained under the power cap for one of more than a few milliseconds."""
    if ms > 5.0:
        return pk["bf16_tflops_sustained"], "sustained"
    return pk["bf16_tflops"], "burst"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def model_numbers(cfg):
    h, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nq = cfg["num_attention_heads"] * cfg["head_dim"]
    nk = cfg["num_key_value_heads"] * cfg["head_dim"]
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]
    layer_params = (nq + 2 * nk) * h + h * nq + 3 * inter * h
    head_params = vocab * h
    weight_bytes = 2 * (L * layer_params + head_params) + 4 * (L * (2 * h + 2 * cfg["head_dim"]) + h)
    if not cfg["tie_word_embeddings"]:
        pass                                     # the embedding table is gathered, not streamed
    kv_bytes_per_token = L * 2 * nk * 2
    return dict(layer_params=layer_params, head_params=head_params, weight_bytes=weight_bytes,
                kv_bytes_per_token=kv_bytes_per_token, nq=nq)


def prefill_flops(cfg, t):
    n = model_numbers(cfg)
    gemm = 2.0 * t * cfg["num_hidden_layers"] * n["layer_params"] + 2.0 * n["head_params"]
    attn = cfg["num_hidden_layers"] * 4.0 * n["nq"] * t * (t + 1) / 2.0
    return gemm + attn


def fill_requests(engine, batch, context, torch):
    """``batch`` live requests holding ``context`` tokens each, keys and values random."""
    ids = [("bench", i) for i in range(batch)]
    engine.cache.reserve_step([(r, context) for r in ids], engine.plan.max_position)
    for g in engine.cache.groups:
        g.storage.normal_(0.0, 1.0)
    return ids


def decode_device_timed(engine, ids, steps, warmup, torch):
    """K graph-replayed decode steps with the argmax on the device; nothing is read back
    inside the timed region, so host work overlaps the device's."""
    from tinyinfer_b200 import StepEntry
    b = len(ids)
    out = torch.empty(b, dtype=torch.int32, device=engine.device)

    def one():
        logits = engine.decode_step([StepEntry(r, [1], [0]) for r in ids])
        engine.ops.argmax(logits, out)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    before = engine.ops.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clocks:
        start.record()
        for _ in range(steps):
            one()
        stop.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    return ms / steps, clocks.summary(), engine.ops.launches - before


def decode_eager_timed(engine, batch, context, steps, warmup, torch):
    """The same decode steps launched kernel by kernel (no CUDA graph): what the graphs save."""
    from tinyinfer_b200 import StepEntry
    ids = fill_requests(engine, batch, context - (steps + warmup) - 2, torch)
    out = torch.empty(batch, dtype=torch.int32, device=engine.device)
    graphs, engine._step_graphs = engine._step_graphs, None
    try:
        def one():
            engine.ops.argmax(engine.step([StepEntry(r, [1], [0]) for r in ids]), out)
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps
    finally:
        engine._step_graphs = graphs
        for r in ids:
            engine.finish(r)


def decode_e2e(llm, batch, context, steps, warmup, torch):
    """The same steps through the Python entry point (``LLM.start`` / ``Session.step``): prompts
    are run first; then every timed step packs the host's token ids, copies them to the device
    from pinned memory, decodes, samples and reads the chosen tokens back."""
    from tinyinfer_b200 import SamplingParams
    g = torch.Generator().manual_seed(1)
    # requests that finish their prompt early decode while the others' prompts still run: room
    # for those tokens, so that nobody reaches its limit inside the timed steps
    slack = -(-batch * context // llm.max_batched_tokens) + batch + 4
    prompt_len = context - (steps + warmup) - slack - 2
    prompts = [torch.randint(0, llm.engine.plan.vocab_size, (prompt_len,), generator=g).tolist()
               for _ in range(batch)]
    session = llm.start(prompts, SamplingParams(max_tokens=steps + warmup + slack + 1))
    while not all(r.output for r in session.requests):      # the prompts, in portions
        session.step()
    for _ in range(warmup):
        session.step()
    torch.cuda.synchronize()
    buckets = llm.engine._graphs.buckets
    copied = sum(bk.copied_ints for bk in buckets.values())
    t0 = time.perf_counter()
    for _ in range(steps):
        made = session.step()
        assert len(made) == batch
    torch.cuda.synchronize()
    sec = time.perf_counter() - t0
    copied = sum(bk.copied_ints for bk in buckets.values()) - copied
    while not session.done:
        session.step()
    session.finish()
    # what a step copies: its tokens, positions, lengths and slots, and the block-table entries
    # its requests gained (a mean over the timed steps), not the whole table
    return sec / steps * 1e3, round(copied * 4 / steps), batch * 4


def measure_decode(engine, batch, context, steps, warmup, torch):
    ids = fill_requests(engine, batch, context - (steps + warmup) - 2, torch)
    try:
        return decode_device_timed(engine, ids, steps, warmup, torch)
    finally:
        for r in ids:
            engine.finish(r)


def measure_prefill(engine, tokens, reps, torch):
    from tinyinfer_b200 import StepEntry
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, engine.plan.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(reps + 3):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(("prefill", i), prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.finish(("prefill", i))
        if i >= 3:                       # the first steps run eagerly and capture the step's graph
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def measure_mixed(engine, decoders, chunk, context, torch):
    """One step with ``decoders`` requests decoding near ``context`` and a portion of ``chunk``
    tokens of another request's prompt beside them (the step shape of chunked prefill under
    load).  The prompt's first tokens run alone; then five portions follow beside the decoders, the
    last one ending at ``context``: the first two steps run eagerly and capture the shape's
    graph, the other three are timed.  Returns ms per step (median)."""
    from tinyinfer_b200 import StepEntry
    g = torch.Generator().manual_seed(2)
    steps, timed = 5, 3
    lead = max(chunk, context - steps * chunk)
    ids = fill_requests(engine, decoders, context - steps - 2, torch)
    prompt = torch.randint(0, engine.plan.vocab_size, (lead + steps * chunk,), generator=g).tolist()
    times = []
    try:
        engine.step([StepEntry(("bench", "prompt"), prompt[:lead], [])])
        for i in range(steps):
            entries = [StepEntry(r, [1], [0]) for r in ids]
            entries.append(StepEntry(("bench", "prompt"), prompt[lead + i * chunk:lead + (i + 1) * chunk], []))
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            engine.step(entries)
            stop.record()
            torch.cuda.synchronize()
            if i >= steps - timed:
                times.append(start.elapsed_time(stop))
    finally:
        for r in ids + [("bench", "prompt")]:
            engine.finish(r)
    return statistics.median(times)


def measure_chains(engine, batch, torch):
    """Each decode product alone: a CUDA graph of 56 dependent launches with distinct weights,
    timed with CUDA events; microseconds per launch."""
    ops, dev, bf = engine.ops, engine.device, torch.bfloat16
    cfg = engine.config
    h, inter = cfg.hidden_size, cfg.intermediate_size
    nq = cfg.num_attention_heads * cfg.head_dim
    nqkv = nq + 2 * cfg.num_key_value_heads * cfg.head_dim

    def rnd(*shape):
        return torch.randn(*shape, device=dev).to(bf)

    x, xb, o, y = torch.randn(batch, h, device=dev), rnd(batch, h), rnd(batch, nq), rnd(batch, inter)
    qkv = torch.empty(batch, nqkv, device=dev)
    yo = torch.empty(batch, inter, device=dev, dtype=bf)
    xn = torch.empty(batch, h, device=dev, dtype=bf)
    norm_w = torch.ones(h, device=dev)
    n = 56
    wq, wo = [rnd(nqkv, h) for _ in range(n)], [rnd(h, nq) for _ in range(n)]
    wg = [ops.pack_gate_up(rnd(inter, h), rnd(inter, h)) for _ in range(n)]
    wd = [rnd(h, inter) for _ in range(n)]
    cases = {
        "qkv": lambda: [ops.linear(xb, w, qkv) for w in wq],
        "o_accumulate": lambda: [ops.linear(o, w, x, accumulate=True) for w in wo],
        "gate_up_swiglu": lambda: [ops.gate_up_swiglu(xb, w, yo) for w in wg],
        "down_accumulate": lambda: [ops.linear(y, w, x, accumulate=True) for w in wd],
        "rmsnorm": lambda: [ops.rmsnorm(x, norm_w, 1e-6, xn) for _ in range(n)],
    }
    out = {}
    for name, fn in cases.items():
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(3):
            graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(20):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        out[name] = round(start.elapsed_time(stop) / 20 / n * 1e3, 2)
    return out


def shape_points(shape_key, page_size, context, steps, warmup, batches, prefill, mixed, pk, torch, prefix):
    """Decode at the given batches, the 2,048-token prefill and the mixed step for another shape
    or page size, each with its fraction of its roofline.  Returns (points, fractions)."""
    import gc
    from tinyinfer_b200 import LLM
    shape_name, shape_cfg = SHAPES[shape_key]
    cfg = dict(shape_cfg, max_position_embeddings=MAX_POSITION)
    nums = model_numbers(cfg)
    max_batch = max(list(batches) + ([64] if mixed else []) + [1])
    llm = LLM(config=cfg, seed=0, dtype="bfloat16", page_size=page_size, max_seq=context,
              max_num_seqs=max_batch + 1, kv_tokens=max_batch * context, cuda_graph=True)
    engine = llm.engine
    points, fracs = {}, {}
    try:
        for b in batches:
            n = min(steps, 32)
            ms, _, _ = measure_decode(engine, b, context, n, warmup, torch)
            points[f"{prefix}decode_b{b}"] = round(b / (ms * 1e-3), 1)
            step_bytes = nums["weight_bytes"] + b * (context - n // 2) * nums["kv_bytes_per_token"]
            fracs[f"{prefix}decode_b{b}"] = round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        if prefill:
            ms = measure_prefill(engine, 2048, 3, torch)
            peak, which = flops_peak(pk, ms)
            points[f"{prefix}prefill_2048"] = round(2048 / (ms * 1e-3), 1)
            fracs[f"{prefix}prefill_2048"] = round(prefill_flops(cfg, 2048) / (ms * 1e-3) / (peak * 1e12), 4)
            fracs[f"{prefix}prefill_2048_peak"] = which
        if mixed:
            ms = measure_mixed(engine, 63, 512, context, torch)
            points[f"{prefix}mixed_63_decoding_512_portion"] = round((63 + 512) / (ms * 1e-3), 1)
    finally:
        del engine, llm
        gc.collect()
        torch.cuda.empty_cache()
    return points, fracs


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def reference_binary():
    """The reference's command-line program, built with its own CMakeLists if it is not there yet.
    Returns (path, None) or (None, why not)."""
    exe = os.path.join(REF_DIR, "build", "tinyinfer")
    if os.path.isfile(exe) and os.access(exe, os.X_OK):
        return exe, None
    src = os.path.join(REF_DIR, "src")
    if not os.path.isfile(os.path.join(src, "CMakeLists.txt")):
        return None, ("beyondHJM/tinyinfer.cpp is a CMake C++/CUDA project (pip: \"Neither 'setup.py' nor "
                      "'pyproject.toml' found\") and no copy of its tree lies under baseline/_ref/src to build")
    try:
        log = os.path.join(REF_DIR, "build.log")
        with open(log, "w") as fh:
            subprocess.run(["cmake", "-S", src, "-B", os.path.join(REF_DIR, "build"),
                            "-DCMAKE_CUDA_ARCHITECTURES=100", "-DCMAKE_BUILD_TYPE=Release"],
                           stdout=fh, stderr=subprocess.STDOUT, check=True, timeout=600)
            subprocess.run(["cmake", "--build", os.path.join(REF_DIR, "build"), "--target", "tinyinfer", "-j", "8"],
                           stdout=fh, stderr=subprocess.STDOUT, check=True, timeout=1200)
    except (OSError, subprocess.SubprocessError) as exc:
        return None, f"building the reference with its own CMakeLists failed ({type(exc).__name__}; baseline/_ref/build.log)"
    return (exe, None) if os.path.isfile(exe) else (None, "the reference's build left no program")


def reference_gguf(cfg, seed, path):
    """A GGUF file of the configuration with seeded random weights and a tokenizer of single
    letters (so that a prompt of three letters is three tokens); end-of-text is an id no token has."""
    import torch
    from tinyinfer_b200.config import Qwen3Config
    from tinyinfer_b200.config.qwen3 import gguf_metadata, gguf_tensor_name
    from tinyinfer_b200.config.registry import architecture_of
    from tinyinfer_b200.parts.model import CausalLM
    from tinyinfer_b200.weights import write_gguf
    from tinyinfer_b200.weights.random_init import random_tensor
    arch = architecture_of(cfg)
    typed = arch.from_dict(cfg)
    model = CausalLM(arch.build_plan(typed))
    # drawn on the GPU when there is one (the generator gives the same bits there, much sooner)
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    tensors = {gguf_tensor_name(n): random_tensor(seed, n, spec, device=dev).cpu()
               for n, spec in model.expected_tensors().items()}
    meta = gguf_metadata(Qwen3Config.from_dict(cfg))
    letters = [chr(ord("a") + i) for i in range(26)]
    meta["tokenizer.ggml.tokens"] = letters
    meta["tokenizer.ggml.token_type"] = [1] * len(letters)
    meta["tokenizer.ggml.eos_token_id"] = 2 ** 32 - 1
    write_gguf(path, meta, tensors)


def reference_decode(exe, gguf, batch, context, cuda_graph=True):
    """Runs the reference's program: `batch` prompts of three tokens, decoded to `context`.
    Returns (tokens a second as it reports them, generated tokens, decode ms, the tail of its log)."""
    import re
    # its loop ends when all sequences together have made batch + n tokens (src/main.cpp:276)
    n_predict = batch * (context - 4)
    cmd = [exe, "-m", gguf, "-n", str(n_predict), "--max-seq", str(context)]
    for i in range(batch):
        cmd += ["-p", "abc"]
    if cuda_graph:
        cmd.append("--cuda-graph")
    proc = subprocess.run(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True, timeout=900)
    tail = proc.stderr[-600:]
    m = re.search(r"main: decode: ([0-9.]+) ms, (\d+) tokens, ([0-9.]+) tok/s", proc.stderr)
    if proc.returncode != 0 or not m:
        raise RuntimeError(f"the reference's program ended with {proc.returncode}: {tail.strip()[-300:]}")
    return float(m.group(3)), int(m.group(2)), float(m.group(1)), tail


def reference_arm(args) -> int:
    shape_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    cfg["max_position_embeddings"] = max(args.context, 2048)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    if not cfg["tie_word_embeddings"]:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference always ties the head to the embedding (src/inference.cu:70-71); "
                          f"the {shape_name} has a head of its own"}))
        return 0
    if args.batch > 16:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs at most 16 sequences (src/main.cpp:178)"}))
        return 0
    exe, why = reference_binary()
    if exe is None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    import tempfile
    gguf = os.path.join(tempfile.gettempdir(), f"tinyinfer_ref_{args.shape}_{cfg['num_hidden_layers']}l_{os.getuid()}.gguf")
    try:
        if not os.path.isfile(gguf):
            reference_gguf(cfg, 0, gguf)
        with ClockSampler() as clocks:
            tps, generated, decode_ms, tail = reference_decode(exe, gguf, args.batch, args.context)
        points = {}
        if not args.no_points and args.batch != 1:
            points["decode_b1"] = reference_decode(exe, gguf, 1, args.context)[0]
    except Exception as exc:           # the line must still come out
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}))
        return 0
    steps = generated // args.batch
    nums = model_numbers(cfg)
    pk, pk_kind = peaks()
    ctx_mean = args.context // 2
    step_bytes = nums["weight_bytes"] + args.batch * ctx_mean * nums["kv_bytes_per_token"]
    ms_per_step = decode_ms / max(steps, 1)
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    line = {
        "impl": "reference",
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} ({shape_name})",
        "value": tps, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 0,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights in a GGUF file, prompts of three tokens, greedy decoding",
        "config": {
            "model": shape_name, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied": True, "global_batch": args.batch, "seq_len": args.context,
            "measured_over": "the whole decode, context 3 to seq_len (its own report)",
            "cuda_graph": True, "program": "baseline/_ref/build/tinyinfer (its own CMakeLists, sm_100)",
            "parallelism": "single GPU", "peaks": pk_kind,
        },
        "clocks": clocks.summary(),
        "e2e": {"value": tps, "unit": "tokens/s", "note": "the same run: its command line is its public API"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "at": "mean context seq_len / 2"},
        "prefill": None,
        "points": points,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers (named in config)")
    ap.add_argument("--shape", choices=list(SHAPES), default="0.6b", help="layer sizes of the model")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64 and the other shapes")
    ap.add_argument("--no-shapes", action="store_true", help="skip the 8B and 32B shapes and the page-16 run")
    ap.add_argument("--page-size", type=int, default=PAGE, help="tokens per cache page")
    ap.add_argument("--prefill-tokens", type=int, default=2048,
                    help="with --only prefill: the length of the prompt (the default run's is 2,048)")
    ap.add_argument("--mixed-decoders", type=int, default=63,
                    help="with --only mixed: the number of decoding requests beside the 512-token portion")
    ap.add_argument("--attention-in-turn", action="store_true",
                    help="with --only mixed: flash-decoding behind the prompt attention kernel, not beside it")
    ap.add_argument("--only", choices=["decode", "prefill", "chains", "mixed"], default=None,
                    help="run one part only and print a short line (for profiling small cases)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; this engine does no work on several (asked for {args.gpus})")
        return 2
    warmup = max(args.warmup, 3)

    import torch
    from tinyinfer_b200 import LLM

    shape_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    cfg["max_position_embeddings"] = max(args.context, MAX_POSITION)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk, pk_kind = peaks()
    nums = model_numbers(cfg)
    max_batch = max(args.batch, 1 if (args.no_points or args.only not in (None, "mixed")) else 64)
    longest = max(args.context, args.prefill_tokens + args.page_size if args.only == "prefill" else 0)
    llm = LLM(config=cfg, seed=0, dtype="bfloat16", page_size=args.page_size, max_seq=longest,
              max_num_seqs=max_batch + 1, kv_tokens=max(max_batch * args.context, longest), cuda_graph=True)
    engine = llm.engine

    if args.only == "decode":
        ms, _, launches = measure_decode(engine, args.batch, args.context, args.steps, warmup, torch)
        print(json.dumps({"only": "decode", "batch": args.batch, "context": args.context,
                          "ms_per_step": round(ms, 4), "gpu_launches": launches}))
        return 0
    if args.only == "chains":
        print(json.dumps({"only": "chains", "batch": args.batch, "us_per_launch":
                          measure_chains(engine, args.batch, torch)}))
        return 0
    if args.only == "mixed":
        engine.ops.attention_side_by_side = not args.attention_in_turn
        mx_ms = measure_mixed(engine, args.mixed_decoders, 512, args.context, torch)
        print(json.dumps({"only": "mixed", "decoding": args.mixed_decoders, "portion": 512, "ms": round(mx_ms, 3),
                          "attention": "in turn" if args.attention_in_turn else "side by side"}))
        return 0
    if args.only == "prefill":
        pf_ms = measure_prefill(engine, args.prefill_tokens, max(1, min(args.steps, 8)), torch)
        print(json.dumps({"only": "prefill", "tokens": args.prefill_tokens, "ms": round(pf_ms, 3)}))
        return 0
    ms, clocks, launches = measure_decode(engine, args.batch, args.context, args.steps, warmup, torch)
    e2e_ms, h2d, d2h = decode_e2e(llm, args.batch, args.context, args.steps, warmup, torch)
    ctx_mid = args.context - args.steps // 2
    step_bytes = nums["weight_bytes"] + args.batch * ctx_mid * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9

    points, fracs = {}, {}
    if not args.no_points:
        for b in (1, 64):
            n = min(args.steps, 32)
            pms, _, _ = measure_decode(engine, b, args.context, n, warmup, torch)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            b_bytes = nums["weight_bytes"] + b * (args.context - n // 2) * nums["kv_bytes_per_token"]
            fracs[f"decode_b{b}"] = round(b_bytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        eager_ms = decode_eager_timed(engine, args.batch, args.context, min(args.steps, 32), warmup, torch)
        points[f"decode_b{args.batch}_no_graph"] = round(args.batch / (eager_ms * 1e-3), 1)
        # chunked prefill under load: 63 requests decode beside a 512-token portion of a prompt
        mx_ms = measure_mixed(engine, 63, 512, args.context, torch)
        points["mixed_63_decoding_512_portion"] = round((63 + 512) / (mx_ms * 1e-3), 1)

    pf_tokens = 2048
    pf_ms = measure_prefill(engine, pf_tokens, 3, torch)
    pf_peak, pf_which = flops_peak(pk, pf_ms)
    pf_frac = prefill_flops(cfg, pf_tokens) / (pf_ms * 1e-3) / (pf_peak * 1e12)

    if not args.no_points and not args.no_shapes and args.shape == "0.6b" and not args.layers:
        # the page size and the two larger shapes that the baseline names, as points of their own
        import gc
        del engine, llm
        gc.collect()
        torch.cuda.empty_cache()
        for key, page, batches, pre, mix, prefix in (
                ("0.6b", 16, (8,), True, False, "page16_"),
                ("8b", args.page_size, (1, 8, 64), True, True, "8b_"),
                ("32b", args.page_size, (1, 8, 64), True, False, "32b_")):
            try:
                p2, f2 = shape_points(key, page, args.context, args.steps, warmup, batches, pre, mix, pk, torch, prefix)
            except Exception as exc:                    # a point that fails must not lose the line
                p2, f2 = {f"{prefix}error": f"{type(exc).__name__}: {str(exc)[:120]}"}, {}
            points.update(p2)
            fracs.update(f2)

    value = args.batch / (ms * 1e-3)
    line = {
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} ({shape_name})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, random token ids, random keys and values",
        "config": {
            "model": shape_name, "layers": cfg["num_hidden_layers"],
            "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "tied": cfg["tie_word_embeddings"], "global_batch": args.batch,
            "seq_len": args.context, "page_size": args.page_size, "max_position": cfg["max_position_embeddings"],
            "parallelism": "single GPU", "cuda_graph": True, "l2": "working set > L2, no flush", "peaks": pk_kind,
        },
        "clocks": clocks,
        "e2e": {"value": round(args.batch / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(pf_tokens / (pf_ms * 1e-3), 1), "tokens": pf_tokens,
                    "ms": round(pf_ms, 3), "frac": round(pf_frac, 4), "peak": pf_which},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "points_frac": fracs,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
