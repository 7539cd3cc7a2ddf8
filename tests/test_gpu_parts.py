"""Each part alone against the plain functions, and toy architectures defined here.

The first toy architecture has a mixer with state of its own (a running mean over the
request's tokens, kept in a fixed-size state slot) whose update is a CUDA kernel that the test
itself brings as a library of its own, layers of different kinds, a layer that runs twice and
an entry that reads the cache another entry wrote.  It is registered, built, loaded and stepped
through the engine, eagerly, from the decode graphs and through the generation loop with steps
launched ahead, without a change to the framework's files.  A second toy architecture has a
feed-forward with a router and experts in some of its layers and a position encoding of a kind
the kernel set has no kernel for, which brings its own handler.  Neither is a model of anyone's.
"""
import math
from dataclasses import dataclass

import pytest
import torch

from plain_qwen3 import (load_folder, plain_attention, plain_embedding, plain_rmsnorm,
                         plain_rope_angles, plain_rope_neox, plain_swiglu)
from util import FP32_RTOL, assert_close_logits, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from tinyinfer_b200.kernels import cuda_ops
    return cuda_ops(DEV)


def _w(shape, seed, scale=0.05, one=False):
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(shape, generator=g) * scale
    return (t + 1.0) if one else t


def _close(got, want, rtol, what):
    err = (got.double().cpu() - want.double()).abs().max().item()
    scale = want.abs().max().item()
    assert err <= rtol * scale, f"{what}: error {err:.3e} against {scale:.3e}"


def test_norm_part(ops):
    from tinyinfer_b200.config import PartSpec
    from tinyinfer_b200.parts import build_part
    norm = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 1e-4}))
    assert list(norm.weight_specs()) == ["weight"] and norm.weight_specs()["weight"].shape == (72,)
    w = _w((72,), 1, one=True)
    norm.load_weights({"weight": w.to(torch.bfloat16).to(DEV)}, ops)     # stored in bfloat16: widened
    x = _w((9, 72), 2, scale=2.0)
    want = plain_rmsnorm(x, w.to(torch.bfloat16), 1e-4)
    _close(norm.forward(ops, x.to(DEV), torch.float32), want, 1e-6, "norm")
    rows = torch.tensor([8, 0], dtype=torch.int32, device=DEV)
    _close(norm.forward_rows(ops, x.to(DEV), rows, torch.bfloat16), want[[8, 0]], 8e-3, "norm rows")


def test_position_part():
    from tinyinfer_b200.config import PartSpec
    from tinyinfer_b200.parts import build_part
    rope = build_part("position", PartSpec("rope_neox", {"head_dim": 48, "theta": 5e4}))
    rot = rope.rotation(DEV)
    want = plain_rope_angles(torch.tensor([1]), 48, 5e4)[0]
    assert rot.kind == "neox" and rot.rotary_dim == 48
    assert rot.inv_freq.dtype == torch.float32 and torch.equal(rot.inv_freq.cpu(), want)
    part = build_part("position", PartSpec("rope_neox", {"head_dim": 48, "theta": 5e4, "rotary_dim": 20}))
    assert part.rotation(DEV).rotary_dim == 20 and part.rotation(DEV).inv_freq.shape == (10,)
    assert torch.equal(part.rotation(DEV).inv_freq.cpu(), plain_rope_angles(torch.tensor([1]), 20, 5e4)[0])
    none = build_part("position", PartSpec("none", {"head_dim": 48})).rotation(DEV)
    assert none.kind == "none" and none.rotary_dim == 0
    with pytest.raises(ValueError, match="even"):
        build_part("position", PartSpec("rope_neox", {"head_dim": 7, "theta": 1e4}))
    with pytest.raises(ValueError, match="even"):
        build_part("position", PartSpec("rope_neox", {"head_dim": 8, "theta": 1e4, "rotary_dim": 10}))


def _cache_for(mixer, num_tokens, dtype, page_size=16):
    from tinyinfer_b200.cache import CacheManager
    return CacheManager([mixer.cache_spec()], page_size=page_size, num_pages=-(-num_tokens // page_size) + 1,
                        max_requests=2, kv_dtype=dtype, device=DEV)


def _step(cache, req, tokens_count, dtype):
    from tinyinfer_b200.engine import StepEntry, build_step_batch
    from tinyinfer_b200.kernels import cuda_ops
    start = cache.reserve_step([(req, tokens_count)])[0]
    batch = build_step_batch([StepEntry(req, [0] * tokens_count, [])], [start],
                             [[cache.block_table(g, req)] for g in range(len(cache.groups))],
                             [cache.state_slot(req)], dtype, DEV, max_position=512,
                             lists=cuda_ops(DEV).step_lists(dtype))
    return batch


def _rope_leading(x, positions, rotary_dim, theta):
    """The NeoX rotation over the first ``rotary_dim`` elements of each head, the rest untouched."""
    if rotary_dim == 0:
        return x
    ang = plain_rope_angles(positions, rotary_dim, theta)
    return torch.cat([plain_rope_neox(x[..., :rotary_dim], ang), x[..., rotary_dim:]], dim=-1)


@pytest.mark.parametrize("dtype,rtol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("window,rotary", [(None, 32), (9, 32), (None, 12), (9, 0)])
def test_attention_part_alone(ops, dtype, rtol, window, rotary):
    """Also with a position part that rotates only the first 12 elements of a head, and with
    the one that rotates nothing: other position parts, the same mixer."""
    from tinyinfer_b200.config import PartSpec
    from tinyinfer_b200.parts import build_part
    hidden, heads, kv, hd, eps, theta = 72, 6, 3, 32, 2e-5, 3e4
    position = (PartSpec("none", {"head_dim": hd}) if rotary == 0 else
                PartSpec("rope_neox", {"head_dim": hd, "theta": theta, "rotary_dim": rotary}))
    att = build_part("mixer", PartSpec("attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv, "head_dim": hd,
        "qk_norm_eps": eps, "window": window, "position": position}))
    names = att.weight_specs()
    assert names["q_proj.weight"].shape == (192, 72) and names["k_norm.weight"].shape == (32,)
    wdt = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    w = {n: _w(s.shape, i, scale=0.2, one=("norm" in n)).to(wdt if "proj" in n else torch.float32)
         for i, (n, s) in enumerate(names.items())}
    att.load_weights({n: t.to(DEV) for n, t in w.items()}, ops)
    s_len = 50
    h = _w((s_len, hidden), 20, scale=1.0).to(dtype)
    # plain: whole sequence
    rd = (lambda t: t.to(torch.bfloat16).to(F64)) if dtype == torch.bfloat16 else (lambda t: t.to(F64))
    hh = h.to(F64)
    q = (hh @ w["q_proj.weight"].to(F64).T).view(s_len, heads, hd)
    k = (hh @ w["k_proj.weight"].to(F64).T).view(s_len, kv, hd)
    v = (hh @ w["v_proj.weight"].to(F64).T).view(s_len, kv, hd)
    pos = torch.arange(s_len)
    q = _rope_leading(plain_rmsnorm(q, w["q_norm.weight"], eps), pos, rotary, theta)
    k = rd(_rope_leading(plain_rmsnorm(k, w["k_norm.weight"], eps), pos, rotary, theta))
    o = rd(plain_attention(q, k, rd(v), 1 / math.sqrt(hd), window).reshape(s_len, heads * hd))
    want = o @ w["o_proj.weight"].to(F64).T
    # the part: two portions and a single token, through a paged cache
    cache = _cache_for(att, s_len, dtype)
    got = torch.zeros((s_len, hidden), dtype=torch.float32, device=DEV)
    lo = 0
    for n in (33, 1, 16):
        batch = _step(cache, "r", n, dtype)
        view = cache.view(0, True, batch.block_tables, batch.state_slots)
        att.forward(ops, h[lo:lo + n].to(DEV), got[lo:lo + n], batch, view)
        cache.release_passed("r")
        lo += n
    ops.check_status()
    _close(got, want, rtol, f"attention part window={window} rotary={rotary}")


@pytest.mark.parametrize("dtype,rtol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_feed_forward_part_alone(ops, dtype, rtol):
    from tinyinfer_b200.config import PartSpec
    from tinyinfer_b200.parts import build_part
    ffn = build_part("ffn", PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200}))
    wdt = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    w = {n: _w(s.shape, i, scale=0.2).to(wdt) for i, (n, s) in enumerate(ffn.weight_specs().items())}
    ffn.load_weights({n: t.to(DEV) for n, t in w.items()}, ops)
    h = _w((11, 72), 9, scale=1.0).to(dtype)
    y = plain_swiglu(h.to(F64) @ w["gate_proj.weight"].to(F64).T, h.to(F64) @ w["up_proj.weight"].to(F64).T)
    if dtype == torch.bfloat16:
        y = y.to(torch.bfloat16).to(F64)
    base = _w((11, 72), 10, scale=1.0)
    res = base.clone().to(DEV)
    ffn.forward(ops, h.to(DEV), res, None)
    ops.flush()                            # (the part lets its last product wait for what follows)
    _close(res, base.to(F64) + y @ w["down_proj.weight"].to(F64).T, rtol, "swiglu part")


def test_embedding_and_head_parts(ops):
    from tinyinfer_b200.config import PartSpec
    from tinyinfer_b200.parts import build_part
    emb = build_part("embedding", PartSpec("embedding", {"vocab_size": 300, "hidden_size": 40}))
    table = _w((300, 40), 3).to(torch.bfloat16)
    emb.load_weights({"weight": table.to(DEV)}, ops)
    tok = torch.tensor([5, 299, 0], dtype=torch.int32, device=DEV)
    x = torch.empty((3, 40), device=DEV)
    emb.forward(ops, tok, x)
    assert torch.equal(x.cpu().double(), plain_embedding(table, tok.cpu()))
    tied = build_part("head", PartSpec("lm_head", {"vocab_size": 300, "hidden_size": 40, "tied": True}))
    assert tied.weight_specs() == {}
    tied.tie(emb)
    own = build_part("head", PartSpec("lm_head", {"vocab_size": 300, "hidden_size": 40, "tied": False}))
    head_w = _w((300, 40), 4)
    own.load_weights({"weight": head_w.to(DEV)}, ops)                  # stored in float32: stays so
    h = _w((3, 40), 5, scale=1.0).to(DEV)
    _close(tied.forward(ops, h), h.cpu().double() @ table.double().T, 1e-5, "tied head")
    _close(own.forward(ops, h), h.cpu().double() @ head_w.double().T, 1e-5, "own head")


# ---- a toy architecture, defined in the test ------------------------------------------------

_RUNNING_MEAN_CU = r"""
// The toy mixer's state update: per request the sum of its activations so far lives in the
// request's state slot; a block walks the request's tokens of this step in order.
#include "common.cuh"

__global__ void running_mean_kernel(const float* __restrict__ h, const int* __restrict__ cu_q,
                                    const int* __restrict__ q_start, const int* __restrict__ slots,
                                    float* __restrict__ state, int writes, int hidden,
                                    float* __restrict__ mean) {
    const int r = blockIdx.x;
    const int lo = cu_q[r], hi = cu_q[r + 1], first = q_start[r];
    float* mine = state + (size_t)slots[r] * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float sum = mine[c];
        for (int t = lo; t < hi; ++t) {
            sum += h[(size_t)t * hidden + c];
            mean[(size_t)t * hidden + c] = sum / (float)(first + (t - lo) + 1);
        }
        if (writes) mine[c] = sum;
    }
}

extern "C" int toy_running_mean(const float* h, const int* cu_q, const int* q_start, const int* slots,
                                float* state, int writes, int requests, int hidden, float* mean,
                                void* stream) {
    if (requests == 0) return 0;
    running_mean_kernel<<<requests, 128, 0, (cudaStream_t)stream>>>(h, cu_q, q_start, slots, state,
                                                                  writes, hidden, mean);
    return ti_check_launch("toy_running_mean");
}
"""
_TOY_LIB = {}


def _toy_library(tmp_dir):
    """The toy mixer's kernel as a library that the test registers itself."""
    import ctypes
    import os
    from tinyinfer_b200.kernels import load_library, register_library
    if "lib" not in _TOY_LIB:
        src = os.path.join(str(tmp_dir), "toy_running_mean.cu")
        with open(src, "w") as fh:
            fh.write(_RUNNING_MEAN_CU)
        register_library("toy_running_mean", [src])
        lib = load_library("toy_running_mean")
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.toy_running_mean.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, vp, vp]
        lib.ti_last_error.restype = ctypes.c_char_p
        _TOY_LIB["lib"] = lib
    return _TOY_LIB["lib"]


def _register_toy(tmp_dir):
    from tinyinfer_b200.config import Architecture, PartSpec, register_architecture
    from tinyinfer_b200.config.plan import LayerPlan, ModelPlan, ScheduleEntry
    from tinyinfer_b200.parts import FixedStateSpec, MATRIX, Part, WeightSpec, build_part, register_part
    lib = _toy_library(tmp_dir)

    class RunningMean(Part):
        """out[t] = W mean(h[0..t]) per request; the sum so far is the request's state.  Its kernel
        takes everything that changes from step to step from device memory, so a step with this
        mixer can be captured in a CUDA graph."""
        category = "mixer"

        def __init__(self, hidden_size):
            self.hidden = hidden_size
            self.w = None

        def weight_specs(self):
            return {"mix.weight": WeightSpec((self.hidden, self.hidden), MATRIX)}

        def load_weights(self, tensors, ops):
            self.w = ops.pack_linear(tensors["mix.weight"].float())

        def cache_spec(self):
            return FixedStateSpec((self.hidden,), torch.float32)

        def forward(self, ops, h, residual, step, cache):
            h32 = h if h.dtype == torch.float32 else h.float()
            mean = torch.empty_like(h32)
            rc = lib.toy_running_mean(h32.data_ptr(), step.cu_q.data_ptr(), step.q_start_dev.data_ptr(),
                                      cache.slots.data_ptr(), cache.state.data_ptr(), int(cache.writes),
                                      step.num_requests, self.hidden, mean.data_ptr(), ops.stream())
            ops.launched(rc, lib.ti_last_error().decode())
            ops.linear(mean, self.w, residual, accumulate=True)

    class SlowRope(Part):
        """The rotation of rope_neox with every frequency divided by ``factor``: a position part of
        its own that answers with a kind the kernel set knows."""
        category = "position"

        def __init__(self, head_dim, theta, factor):
            self.inner = build_part("position", PartSpec("rope_neox", {"head_dim": head_dim, "theta": theta}))
            self.factor = float(factor)
            self._rotation = None

        def rotation(self, device):
            from tinyinfer_b200.parts import Rotation
            if self._rotation is None:
                self._rotation = Rotation("neox", self.inner.rotary_dim,
                                          (self.inner.inv_freq() / self.factor).to(device))
            return self._rotation

    register_part("position", "slow_rope", SlowRope)
    register_part("mixer", "running_mean", RunningMean)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        intermediate_size: int
        max_position_embeddings: int

        def to_dict(self):
            return {**self.__dict__, "architectures": ["ToyMixForCausalLM"]}

    def from_dict(cfg):
        return ToyConfig(cfg["hidden_size"], cfg["vocab_size"], cfg["intermediate_size"],
                         cfg["max_position_embeddings"])

    def build_plan(c):
        norm = PartSpec("rmsnorm", {"size": c.hidden_size, "eps": 1e-5})
        ffn = PartSpec("swiglu", {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size})
        mean = PartSpec("running_mean", {"hidden_size": c.hidden_size})
        att = PartSpec("attention", {
            "hidden_size": c.hidden_size, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
            "qk_norm_eps": 1e-5, "window": None,
            "position": PartSpec("slow_rope", {"head_dim": 16, "theta": 1e4, "factor": 4.0})})
        layers = []
        for i, mixer in enumerate([mean, att, mean]):
            p = f"toy.{i}."
            layers.append(LayerPlan(PartSpec("prenorm"), mixer, ffn, norm, norm,
                                    {"mixer": p + "mixer.", "ffn": p + "ffn.",
                                     "mixer_norm": p + "norm1.", "ffn_norm": p + "norm2."}))
        # layer 0 runs twice with a state of its own each time; layer 1 runs twice and reads,
        # the second time, the keys and values that its first run wrote
        schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2),
                    ScheduleEntry(1, 1, writes_cache=False), ScheduleEntry(0, 3)]
        return ModelPlan("ToyMixForCausalLM", c.hidden_size, c.vocab_size, c.max_position_embeddings,
                         layers, schedule,
                         PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}),
                         norm, PartSpec("lm_head", {"vocab_size": c.vocab_size,
                                                    "hidden_size": c.hidden_size, "tied": True}),
                         {"embedding": "toy.embed.", "final_norm": "toy.norm.", "head": "toy.head."})

    register_architecture(Architecture("ToyMixForCausalLM", from_dict, build_plan))


def _toy_plain(w, tokens):
    """The toy model on a whole sequence, from the plain functions."""
    s_len = len(tokens)
    x = plain_embedding(w["toy.embed.weight"], torch.tensor(tokens))
    pos = torch.arange(s_len)
    count = (pos.double() + 1)[:, None]
    kv = {}

    def mean_mixer(i, h):
        return (torch.cumsum(h, 0) / count) @ w[f"toy.{i}.mixer.mix.weight"].to(F64).T

    def attention(i, h, write):
        p = f"toy.{i}.mixer."
        q = plain_rmsnorm((h @ w[p + "q_proj.weight"].to(F64).T).view(s_len, 4, 16), w[p + "q_norm.weight"], 1e-5)
        ang = plain_rope_angles(pos, 16, 1e4) / 4.0
        q = plain_rope_neox(q, ang)
        if write:
            k = plain_rmsnorm((h @ w[p + "k_proj.weight"].to(F64).T).view(s_len, 2, 16), w[p + "k_norm.weight"], 1e-5)
            kv[i] = (plain_rope_neox(k, ang), (h @ w[p + "v_proj.weight"].to(F64).T).view(s_len, 2, 16))
        o = plain_attention(q, kv[i][0], kv[i][1], 0.25).reshape(s_len, 64)
        return o @ w[p + "o_proj.weight"].to(F64).T

    def ffn(i, h):
        p = f"toy.{i}.ffn."
        return plain_swiglu(h @ w[p + "gate_proj.weight"].to(F64).T,
                            h @ w[p + "up_proj.weight"].to(F64).T) @ w[p + "down_proj.weight"].to(F64).T

    for i, write in [(0, True), (1, True), (2, True), (1, False), (0, True)]:
        h = plain_rmsnorm(x, w[f"toy.{i}.norm1.weight"], 1e-5)
        x = x + (attention(i, h, write) if i == 1 else mean_mixer(i, h))
        x = x + ffn(i, plain_rmsnorm(x, w[f"toy.{i}.norm2.weight"], 1e-5))
    return plain_rmsnorm(x, w["toy.norm.weight"], 1e-5) @ w["toy.embed.weight"].to(F64).T


TOY_CFG = {"architectures": ["ToyMixForCausalLM"], "hidden_size": 64, "vocab_size": 200,
           "intermediate_size": 96, "max_position_embeddings": 256}


def test_toy_architecture_with_a_stateful_mixer(tmp_path):
    from tinyinfer_b200 import Engine, StepEntry, write_random_model
    _register_toy(tmp_path)
    d = str(tmp_path / "toy")
    write_random_model(d, TOY_CFG, seed=3, dtype=torch.float32)
    _, w = load_folder(d)
    reqs = {r: random_tokens(200, n, seed=n) for r, n in (("a", 70), ("b", 41), ("c", 9))}
    plain = {r: _toy_plain(w, t) for r, t in reqs.items()}
    eng = Engine(d, dtype="float32", page_size=16, max_tokens=256, max_requests=2)
    specs = eng.model.cache_specs()
    assert [type(s).__name__ for s in specs] == ["FixedStateSpec", "PagedKVSpec", "FixedStateSpec", "FixedStateSpec"]
    # portions of a beside portions and single tokens of b; c arrives when a has left, so its
    # state slot and pages are used again
    got = {r: [] for r in reqs}
    cut = {"a": [0, 33, 34, 60, 70], "b": [0, 2, 20, 21, 41], "c": [0, 4, 5, 9]}
    for i in range(4):
        entries = [StepEntry(r, reqs[r][cut[r][i]:cut[r][i + 1]], list(range(cut[r][i + 1] - cut[r][i])))
                   for r in ("a", "b")]
        out = eng.step(entries).cpu()
        k = 0
        for e in entries:
            got[e.req_id].append(out[k:k + len(e.tokens)])
            k += len(e.tokens)
    eng.finish("a")
    for i in range(3):
        got["c"].append(eng.step([StepEntry("c", reqs["c"][cut["c"][i]:cut["c"][i + 1]],
                                            list(range(cut["c"][i + 1] - cut["c"][i])))]).cpu())
    for r in reqs:
        assert_close_logits(torch.cat(got[r]), plain[r], FP32_RTOL, f"toy request {r}")
    eng.finish("b")
    eng.finish("c")
    eng.cache.check()


def test_stateful_toy_mixer_from_cuda_graphs_and_with_steps_launched_ahead(tmp_path):
    """The mixer with state of its own under CUDA graphs: decode steps replayed from the decode
    buckets (a bucket's first step must not advance the state twice; padding rows use the spare
    state slot), whole steps replayed by shape, and generation with the next step launched
    before the last one's tokens are read, against the plain functions."""
    from tinyinfer_b200 import LLM, Engine, SamplingParams, StepEntry, write_random_model
    _register_toy(tmp_path)
    d = str(tmp_path / "toy")
    write_random_model(d, TOY_CFG, seed=3, dtype=torch.float32)
    _, w = load_folder(d)
    reqs = {r: random_tokens(200, n, seed=50 + n) for r, n in (("a", 40), ("b", 25), ("c", 33))}
    plain = {r: _toy_plain(w, t) for r, t in reqs.items()}
    eng = Engine(d, dtype="float32", page_size=16, max_tokens=256, max_requests=4, step_graphs=True)
    # prompts: a and b together, c alone; the last 12 tokens of each come from the decode graphs,
    # first a and b (bucket of 2), then all three (bucket of 4 with a padding row), then c alone
    eng.step([StepEntry("a", reqs["a"][:28], []), StepEntry("b", reqs["b"][:13], [])])
    got = {r: [] for r in reqs}
    for s in range(4):
        out = eng.decode_step([StepEntry(r, [reqs[r][n + s]], [0]) for r, n in (("a", 28), ("b", 13))])
        got["a"].append(out[0].cpu())
        got["b"].append(out[1].cpu())
    eng.step([StepEntry("c", reqs["c"][:21], [])])
    for s in range(4, 12):
        out = eng.decode_step([StepEntry(r, [reqs[r][n + s]], [0])
                               for r, n in (("a", 28), ("b", 13), ("c", 21 - 4))])
        for i, r in enumerate("abc"):
            got[r].append(out[i].cpu())
    eng.finish("a")
    eng.finish("b")
    for s in range(8, 12):
        got["c"].append(eng.decode_step([StepEntry("c", [reqs["c"][21 + s]], [0])])[0].cpu())
    assert_close_logits(torch.stack(got["a"]), plain["a"][28:], FP32_RTOL, "toy a from graphs")
    assert_close_logits(torch.stack(got["b"]), plain["b"][13:], FP32_RTOL, "toy b from graphs")
    assert_close_logits(torch.stack(got["c"]), plain["c"][21:], FP32_RTOL, "toy c from graphs")
    eng.finish("c")
    # steps of one shape, replayed from the step graphs for other requests at other places
    for i, r in enumerate(["p", "q", "r", "s"]):
        toks = random_tokens(200, 30, seed=80 + i)
        out = torch.cat([eng.step([StepEntry(r, toks[:17], list(range(17)))]).cpu(),
                         eng.step([StepEntry(r, toks[17:], list(range(13)))]).cpu()])
        assert_close_logits(out, _toy_plain(w, toks), FP32_RTOL, f"toy {r} from step graphs")
        eng.finish(r)
    assert len(eng._step_graphs.graphs) == 2
    eng.cache.check()

    def greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(torch.argmax(_toy_plain(w, seq)[-1])))
        return seq[len(prompt):]

    prompts = [random_tokens(200, n, seed=n) for n in (5, 12, 3)]
    want = [greedy(p, 8) for p in prompts]
    for ahead in (False, True):
        llm = LLM(d, dtype="float32", max_seq=64, max_num_seqs=4, page_size=16, cuda_graph=True,
                  lookahead=ahead)
        outs = llm.generate(prompts, SamplingParams(max_tokens=8))
        assert [o.tokens for o in outs] == want, f"lookahead={ahead}"
        llm.engine.cache.check()


# ---- a second toy architecture: a feed-forward with routing, another position encoding -----------

def _register_routed_toy():
    from tinyinfer_b200.config import Architecture, PartSpec, register_architecture
    from tinyinfer_b200.config.plan import LayerPlan, ModelPlan, default_schedule
    from tinyinfer_b200.parts import MATRIX, Part, WeightSpec, build_part, register_part

    class NeighbourPairs(Part):
        """A rotation that pairs each element with its neighbour, (x[2k], x[2k+1]), instead of with
        the element half a head away.  The kernel set has no kernel for this kind, so the part
        brings a handler of its own (device-side tensor expressions: a toy, not a fast path) and
        registers it with the kernel set the first time it is asked."""
        category = "position"
        KIND = "neighbour_pairs"

        def __init__(self, head_dim, theta):
            self.inner = build_part("position", PartSpec("rope_neox", {"head_dim": head_dim, "theta": theta}))
            self._rotation = None

        def rotation(self, device):
            from tinyinfer_b200.kernels import cuda_ops
            from tinyinfer_b200.parts import Rotation
            if self._rotation is None:
                cuda_ops(device).register_rotation(self.KIND, NeighbourPairs.norm_rotate_store)
                self._rotation = Rotation(self.KIND, self.inner.rotary_dim, self.inner.inv_freq().to(device))
            return self._rotation

        @staticmethod
        def norm_rotate_store(ops, qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                              num_heads, num_kv_heads, head_dim):
            t = qkv.shape[0]
            nq, nk = num_heads * head_dim, num_kv_heads * head_dim
            q = qkv[:, :nq].view(t, num_heads, head_dim)
            k = qkv[:, nq:nq + nk].view(t, num_kv_heads, head_dim)
            v = qkv[:, nq + nk:].view(t, num_kv_heads, head_dim)
            ang = step.positions.float()[:, None] * rotation.inv_freq[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

            def norm_rotate(x, w):
                x = x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w
                x0, x1 = x[..., 0::2], x[..., 1::2]
                return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).flatten(-2)

            q_out.copy_(norm_rotate(q, q_weight).reshape(t, nq))
            if cache.writes:
                pos = step.positions.long()
                page = cache.block_table[step.req_of_tok.long(), pos // cache.page_size].long()
                cache.pages[page, 0, :, pos % cache.page_size, :] = norm_rotate(k, k_weight).to(cache.pages.dtype)
                cache.pages[page, 1, :, pos % cache.page_size, :] = v.to(cache.pages.dtype)

    class TopOneExperts(Part):
        """Each token goes to the expert with the largest router logit (float32): a SwiGLU of its
        own.  The experts are the framework's swiglu parts; routing is done here."""
        category = "ffn"

        def __init__(self, hidden_size, intermediate_size, num_experts):
            self.hidden, self.n = hidden_size, num_experts
            spec = PartSpec("swiglu", {"hidden_size": hidden_size, "intermediate_size": intermediate_size})
            self.experts = [build_part("ffn", spec) for _ in range(num_experts)]
            self.router = None

        def weight_specs(self):
            specs = {"router.weight": WeightSpec((self.n, self.hidden), MATRIX)}
            for e, part in enumerate(self.experts):
                specs.update({f"experts.{e}.{k}": v for k, v in part.weight_specs().items()})
            return specs

        def load_weights(self, tensors, ops):
            self.router = tensors["router.weight"].float().contiguous()
            for e, part in enumerate(self.experts):
                pre = f"experts.{e}."
                part.load_weights({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}, ops)

        def forward(self, ops, h, residual, step):
            logits = torch.empty((h.shape[0], self.n), dtype=torch.float32, device=h.device)
            ops.linear(h, self.router, logits)
            choice = logits.argmax(dim=-1)
            for e, part in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    out = torch.zeros((rows.numel(), self.hidden), dtype=torch.float32, device=h.device)
                    part.forward(ops, h[rows].contiguous(), out, step)
                    residual.index_add_(0, rows, out)

    register_part("position", "neighbour_pairs", NeighbourPairs)
    register_part("ffn", "top_one_experts", TopOneExperts)

    @dataclass(frozen=True)
    class RoutedConfig:
        hidden_size: int
        vocab_size: int
        intermediate_size: int
        max_position_embeddings: int
        num_experts: int

        def to_dict(self):
            return {**self.__dict__, "architectures": ["ToyRoutedForCausalLM"]}

    def from_dict(cfg):
        return RoutedConfig(*(cfg[k] for k in ("hidden_size", "vocab_size", "intermediate_size",
                                               "max_position_embeddings", "num_experts")))

    def build_plan(c):
        norm = PartSpec("rmsnorm", {"size": c.hidden_size, "eps": 1e-5})
        dense = PartSpec("swiglu", {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size})
        routed = PartSpec("top_one_experts", {"hidden_size": c.hidden_size, "num_experts": c.num_experts,
                                              "intermediate_size": c.intermediate_size})
        att = PartSpec("attention", {
            "hidden_size": c.hidden_size, "num_heads": 3, "num_kv_heads": 1, "head_dim": 32,
            "qk_norm_eps": 1e-5, "window": None,
            "position": PartSpec("neighbour_pairs", {"head_dim": 32, "theta": 1e4})})
        layers = []
        for i, ffn in enumerate([routed, dense, routed]):          # feed-forwards differ by layer
            p = f"toy.{i}."
            layers.append(LayerPlan(PartSpec("prenorm"), att, ffn, norm, norm,
                                    {"mixer": p + "mixer.", "ffn": p + "ffn.",
                                     "mixer_norm": p + "norm1.", "ffn_norm": p + "norm2."}))
        return ModelPlan("ToyRoutedForCausalLM", c.hidden_size, c.vocab_size, c.max_position_embeddings,
                         layers, default_schedule(len(layers)),
                         PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size}),
                         norm, PartSpec("lm_head", {"vocab_size": c.vocab_size,
                                                    "hidden_size": c.hidden_size, "tied": False}),
                         {"embedding": "toy.embed.", "final_norm": "toy.norm.", "head": "toy.head."})

    register_architecture(Architecture("ToyRoutedForCausalLM", from_dict, build_plan))


def _routed_plain(w, tokens, num_experts):
    """The routed toy model on a whole sequence; also the smallest gap between a token's two best
    router logits, relative to the largest logit."""
    s_len = len(tokens)
    x = plain_embedding(w["toy.embed.weight"], torch.tensor(tokens))
    ang = plain_rope_angles(torch.arange(s_len), 32, 1e4).to(F64)
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    gap = math.inf

    def rope_pairs(x):                       # pairs (x[2k], x[2k + 1]) rotated by pos * inv_freq[k]
        x0, x1 = x[..., 0::2], x[..., 1::2]
        return torch.stack([x0 * cs - x1 * sn, x0 * sn + x1 * cs], dim=-1).flatten(-2)

    def swiglu(p, h):
        return plain_swiglu(h @ w[p + "gate_proj.weight"].to(F64).T,
                            h @ w[p + "up_proj.weight"].to(F64).T) @ w[p + "down_proj.weight"].to(F64).T

    for i in range(3):
        p = f"toy.{i}.mixer."
        h = plain_rmsnorm(x, w[f"toy.{i}.norm1.weight"], 1e-5)
        q = rope_pairs(plain_rmsnorm((h @ w[p + "q_proj.weight"].to(F64).T).view(s_len, 3, 32),
                                     w[p + "q_norm.weight"], 1e-5))
        k = rope_pairs(plain_rmsnorm((h @ w[p + "k_proj.weight"].to(F64).T).view(s_len, 1, 32),
                                     w[p + "k_norm.weight"], 1e-5))
        v = (h @ w[p + "v_proj.weight"].to(F64).T).view(s_len, 1, 32)
        x = x + plain_attention(q, k, v, 1.0 / math.sqrt(32)).reshape(s_len, 96) @ w[p + "o_proj.weight"].to(F64).T
        h = plain_rmsnorm(x, w[f"toy.{i}.norm2.weight"], 1e-5)
        p = f"toy.{i}.ffn."
        if i == 1:
            x = x + swiglu(p, h)
            continue
        logits = h @ w[p + "router.weight"].to(F64).T
        top = logits.topk(2, dim=-1).values
        gap = min(gap, ((top[:, 0] - top[:, 1]) / logits.abs().max()).min().item())
        choice = logits.argmax(dim=-1)
        y = torch.zeros_like(x)
        for e in range(num_experts):
            rows = (choice == e).nonzero().flatten()
            y[rows] = swiglu(f"{p}experts.{e}.", h[rows])
        x = x + y
    return plain_rmsnorm(x, w["toy.norm.weight"], 1e-5) @ w["toy.head.weight"].to(F64).T, gap


def test_toy_architecture_with_routing_and_another_position_encoding(tmp_path):
    """A feed-forward with a router and experts (in some layers only) and a position encoding of a
    kind the kernel set has no kernel for (it brings its own handler), both defined here,
    registered and run through the engine in portions and token by token, against the plain
    functions."""
    from tinyinfer_b200 import Engine, StepEntry, write_random_model
    _register_routed_toy()
    cfg = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "vocab_size": 150,
           "intermediate_size": 80, "max_position_embeddings": 128, "num_experts": 3}
    tokens = random_tokens(150, 60, seed=2)
    for seed in range(20):           # a model whose routing does not hang on the last bits
        d = str(tmp_path / f"routed{seed}")
        write_random_model(d, cfg, seed=seed, dtype=torch.float32)
        _, w = load_folder(d)
        plain, gap = _routed_plain(w, tokens, 3)
        if gap > 1e-3:
            break
    else:
        pytest.fail("no seed gave a clear routing")
    eng = Engine(d, dtype="float32", page_size=16, max_tokens=128, max_requests=2)
    got = [eng.step([StepEntry("a", tokens[:23], list(range(23)))]).cpu(),
           eng.step([StepEntry("a", tokens[23:41], list(range(18)))]).cpu()]
    got += [eng.step([StepEntry("a", [t], [0])]).cpu() for t in tokens[41:]]
    assert_close_logits(torch.cat(got), plain, FP32_RTOL, "routed toy")
    eng.finish("a")
    eng.cache.check()
