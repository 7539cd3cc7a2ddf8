"""The plain implementation against logits that the reference's own code produced.

``tests/golden/make_golden.py`` compiles beyondHJM/tinyinfer.cpp's untouched loader, forward pass
and kernels (src/model.cpp, src/inference.cu, src/cuda/*.cu) for the CPU against a stand-in for
CUDA and runs them on tiny random models; the logits it got are stored beside it.  Here the same
models are made again from their seeds and ``plain_forward`` (with the reference's rounding
points) must agree with the stored logits: this pins the plain implementation, which every other
test compares the engine with, to the reference itself and not only to a reading of it.
"""
import glob
import hashlib
import json
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import make_golden  # noqa: E402
from plain_qwen3 import load_folder, plain_forward  # noqa: E402
from tinyinfer_b200 import write_random_model  # noqa: E402

CASES = sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(HERE, "golden", "*.json")))
GOLDEN_RTOL = 5e-3      # of the largest logit: float32 sums against float64 ones, both rounded to bfloat16 at the same places


def _checksum(w):
    digest = hashlib.sha256()
    for key in sorted(w):
        digest.update(key.encode())
        digest.update(w[key].contiguous().view(-1).view(dtype=torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def test_golden_files_exist():
    assert CASES, "tests/golden holds no outputs of the reference (run tests/golden/make_golden.py)"


@pytest.mark.parametrize("name", CASES)
def test_plain_implementation_matches_the_reference_run_on_the_cpu(tmp_path, name):
    with open(os.path.join(HERE, "golden", f"{name}.json")) as fh:
        meta = json.load(fh)
    case = make_golden.CASES[name]
    assert meta["config"] == case["config"] and meta["seed"] == case["seed"], "stale golden files"
    folder = str(tmp_path / name)
    write_random_model(folder, meta["config"], seed=meta["seed"])
    cfg, w = load_folder(folder)
    # the generator of the random weights is integer arithmetic of its own, so the weights are
    # the same wherever the test runs
    assert _checksum(w) == meta["weights_sha256"], \
        "the random weights are not those the golden files were made with: run tests/golden/make_golden.py"
    vocab = cfg["vocab_size"]
    golden = torch.from_numpy(np.fromfile(os.path.join(HERE, "golden", f"{name}.f32"), dtype="<f4")
                              .reshape(-1, vocab).copy()).double()
    passes, _ = make_golden.passes_of(case)
    assert [[p["name"], s] for p in passes for s in sorted(p["seqs"])] == meta["rows"]
    row, hist = 0, {}
    errs, errs_unrounded = [], []
    for p in passes:
        if p["reset"]:
            hist = {}
        for s, (start, toks) in sorted(p["seqs"].items()):
            assert start == len(hist.get(s, []))
            hist[s] = hist.get(s, []) + list(toks)
        for s in sorted(p["seqs"]):
            want = golden[row]
            got = plain_forward(cfg, w, hist[s], emulate_bf16=True)[-1]
            scale = want.abs().max().item()
            err = (got - want).abs().max().item() / scale
            assert err <= GOLDEN_RTOL, f"{name} {p['name']} sequence {s}: {err:.2e} of the largest logit"
            top = want.topk(2).values
            if (top[0] - top[1]).item() > 2 * GOLDEN_RTOL * scale:
                assert int(got.argmax()) == int(want.argmax())
            errs.append(err)
            unrounded = plain_forward(cfg, w, hist[s], emulate_bf16=False)[-1]
            errs_unrounded.append((unrounded - want).abs().max().item() / scale)
            row += 1
    assert row == golden.shape[0]
    # rounding where the reference rounds brings the plain implementation closer to it
    assert sum(errs) < sum(errs_unrounded)
