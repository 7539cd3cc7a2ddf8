"""Replay of the same requests cut in different ways, against the plain implementation.

Each request alone and whole; most of it in one step and the last 32 tokens one by one;
portions of changing size down to two tokens; and mixed, up to four live requests with so
few pages that they are used again.  In float32 and in bfloat16, for three tiny
configurations that differ in every size and option.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import traces
from plain_qwen3 import load_folder, plain_forward
from util import BF16_RTOL, FP32_RTOL, TINY, assert_close_logits, make_model, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 120, 33, 90, 64, 17, 2], "B": [100, 9, 33, 64, 250, 77, 1, 130],
           "C": [150, 40, 300, 64, 97, 210, 31], "D": [200, 33, 520, 64, 130, 95, 17, 2],
           "E": [300, 70, 150, 33, 260, 129]}
PAGE = {"E": 64}              # the other configurations run with pages of 16 tokens
TOL = {"float32": FP32_RTOL, "bfloat16": BF16_RTOL}
FAMILIES = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions,
            "mixed": traces.mixed}


def _requests(name):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}


_PLAIN = {}


def _plain(model_dir, name, dtype):
    key = (name, dtype)
    if key not in _PLAIN:
        cfg, w = load_folder(model_dir)
        _PLAIN[key] = {r: plain_forward(cfg, w, t, emulate_bf16=(dtype == "bfloat16"))
                       for r, t in _requests(name).items()}
    return _PLAIN[key]


def _run_engine(model_dir, dtype, steps, max_tokens, page_size=16):
    from tinyinfer_b200 import Engine, StepEntry
    eng = Engine(model_dir, dtype=dtype, page_size=page_size, num_pages=-(-max_tokens // page_size),
                 max_requests=8)
    outputs = {}
    for s in steps:
        lg = eng.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        outputs[s["step"]] = lg.cpu()
        for r in s["end"]:
            eng.finish(r)
    eng.ops.check_status()
    eng.cache.check()
    assert eng.cache.live_requests() == []
    return outputs


def _compare(steps, outputs, plain, rtol, what):
    rows = traces.collect(steps, outputs)
    worst = 0.0
    for r, items in rows.items():
        pos = torch.tensor([p for p, _ in items])
        got = torch.stack([row for _, row in items])
        worst = max(worst, assert_close_logits(got, plain[r][pos], rtol, f"{what} request {r}"))
    return worst


_ROWS = {}          # (name, family, dtype) -> request id -> [(position, logits row)]


def _rows_of(tmp_path_factory, name, family, dtype):
    key = (name, family, dtype)
    if key not in _ROWS:
        model_dir = make_model(tmp_path_factory.getbasetemp(), name)
        steps = FAMILIES[family](_requests(name))
        max_tokens = traces.max_live_tokens(steps)
        outputs = _run_engine(model_dir, dtype, steps, max_tokens, PAGE.get(name, 16))
        _ROWS[key] = (steps, outputs, traces.collect(steps, outputs))
    return _ROWS[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_cuttings_match_plain(tmp_path_factory, name, family, dtype):
    model_dir = make_model(tmp_path_factory.getbasetemp(), name)
    steps, outputs, _ = _rows_of(tmp_path_factory, name, family, dtype)
    err = _compare(steps, outputs, _plain(model_dir, name, dtype), TOL[dtype],
                   f"tiny-{name} {family} {dtype}")
    print(f"tiny-{name} {family} {dtype}: max error {err:.2e} of the largest logit")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_float32_cuttings_give_the_same_bits(tmp_path_factory, name):
    """In 32-bit the logits at a (request, position) are the same bits however the tokens were
    cut into steps, whatever else was in the batch and whichever pages held them: every kernel
    of that path adds in an order that depends on the token's own place only."""
    base = _rows_of(tmp_path_factory, name, "whole", "float32")[2]
    for family in ("tail", "portions", "mixed"):
        rows = _rows_of(tmp_path_factory, name, family, "float32")[2]
        assert rows.keys() == base.keys()
        for r in base:
            assert [p for p, _ in rows[r]] == [p for p, _ in base[r]]
            got = torch.stack([row for _, row in rows[r]])
            want = torch.stack([row for _, row in base[r]])
            if not torch.equal(got, want):
                first = int((got != want).any(dim=-1).nonzero()[0])
                raise AssertionError(
                    f"tiny-{name} float32: '{family}' and 'whole' differ in bits for request {r}, "
                    f"first at position {base[r][first][0]} "
                    f"(max difference {(got - want).abs().max().item():.3e})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path_factory, tmp_path, dtype):
    """The replay program itself, as a user starts it."""
    name = "B"
    model_dir = make_model(tmp_path_factory.getbasetemp(), name)
    steps = traces.mixed(_requests(name), seed=3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dir,
         "--dtype", dtype, "--out", out, "--max-tokens", str(traces.max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    vocab = TINY[name]["vocab_size"]
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            data = np.fromfile(os.path.join(out, f"{s['step']}.f32"), dtype="<f4")
            outputs[s["step"]] = torch.from_numpy(data.reshape(wanted, vocab).copy())
    _compare(steps, outputs, _plain(model_dir, name, dtype), TOL[dtype], f"trace_run {dtype}")
