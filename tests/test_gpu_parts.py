"""Each part alone against the plain functions, and a toy architecture defined here.

The toy architecture has a mixer with state of its own (a running mean over the request's
tokens, kept in a fixed-size state slot), layers of different kinds, a layer that runs twice
and an entry that reads the cache another entry wrote.  It is registered, built, loaded and
stepped through the engine without a change to the framework's files.  A second toy architecture
has a feed-forward with a router and experts in some of its layers and a position encoding of
its own.  Neither is a model of anyone's.
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
    table = rope.table(DEV)
    want = plain_rope_angles(torch.tensor([1]), 48, 5e4)[0]
    assert table.dtype == torch.float32 and torch.equal(table.cpu(), want)
    with pytest.raises(ValueError, match="even"):
        build_part("position", PartSpec("rope_neox", {"head_dim": 7, "theta": 1e4}))


def _cache_for(mixer, num_tokens, dtype, page_size=16):
    from tinyinfer_b200.cache import CacheManager
    return CacheManager([mixer.cache_spec()], page_size=page_size, num_pages=-(-num_tokens // page_size) + 1,
                        max_requests=2, kv_dtype=dtype, device=DEV)


def _step(cache, req, tokens_count, dtype):
    from tinyinfer_b200.engine import StepEntry, build_step_batch
    start = cache.reserve_step([(req, tokens_count)])[0]
    batch = build_step_batch([StepEntry(req, [0] * tokens_count, [])], [start],
                             [[cache.block_table(g, req)] for g in range(len(cache.groups))],
                             [cache.state_slot(req)], dtype, DEV, max_position=512)
    return batch


@pytest.mark.parametrize("dtype,rtol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_alone(ops, dtype, rtol, window):
    from tinyinfer_b200.config import PartSpec
    from tinyinfer_b200.parts import build_part
    hidden, heads, kv, hd, eps, theta = 72, 6, 3, 32, 2e-5, 3e4
    att = build_part("mixer", PartSpec("attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv, "head_dim": hd,
        "qk_norm_eps": eps, "window": window,
        "position": PartSpec("rope_neox", {"head_dim": hd, "theta": theta})}))
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
    ang = plain_rope_angles(torch.arange(s_len), hd, theta)
    q = plain_rope_neox(plain_rmsnorm(q, w["q_norm.weight"], eps), ang)
    k = rd(plain_rope_neox(plain_rmsnorm(k, w["k_norm.weight"], eps), ang))
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
    _close(got, want, rtol, f"attention part window={window}")


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

def _register_toy():
    from tinyinfer_b200.config import Architecture, PartSpec, register_architecture
    from tinyinfer_b200.config.plan import LayerPlan, ModelPlan, ScheduleEntry
    from tinyinfer_b200.parts import FixedStateSpec, MATRIX, Part, WeightSpec, register_part

    class RunningMean(Part):
        """out[t] = W mean(h[0..t]) per request; the sum so far is the request's state."""
        category = "mixer"

        def __init__(self, hidden_size):
            self.hidden = hidden_size
            self.w = None

        def weight_specs(self):
            return {"mix.weight": WeightSpec((self.hidden, self.hidden), MATRIX)}

        def load_weights(self, tensors, ops):
            self.w = tensors["mix.weight"].float()

        def cache_spec(self):
            return FixedStateSpec((self.hidden,), torch.float32)

        def forward(self, ops, h, residual, step, cache):
            slots = step.state_slots.tolist()
            lo = 0
            for r, n in enumerate(step.q_lens):
                run = torch.cumsum(h[lo:lo + n].float(), dim=0) + cache.state[slots[r]]
                if cache.writes:
                    cache.state[slots[r]] = run[-1]
                count = (step.positions[lo:lo + n].float() + 1.0)[:, None]
                residual[lo:lo + n] += (run / count) @ self.w.T
                lo += n

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
            "position": PartSpec("rope_neox", {"head_dim": 16, "theta": 1e4})})
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
        ang = plain_rope_angles(pos, 16, 1e4)
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


def test_toy_architecture_with_a_stateful_mixer(tmp_path):
    from tinyinfer_b200 import Engine, StepEntry, write_random_model
    _register_toy()
    cfg = {"architectures": ["ToyMixForCausalLM"], "hidden_size": 64, "vocab_size": 200,
           "intermediate_size": 96, "max_position_embeddings": 256}
    d = str(tmp_path / "toy")
    write_random_model(d, cfg, seed=3, dtype=torch.float32)
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


# ---- a second toy architecture: a feed-forward with routing, another position encoding -----------

def _register_routed_toy():
    from tinyinfer_b200.config import Architecture, PartSpec, register_architecture
    from tinyinfer_b200.config.plan import LayerPlan, ModelPlan, default_schedule
    from tinyinfer_b200.parts import MATRIX, Part, WeightSpec, build_part, register_part

    class SlowRope(Part):
        """The rotation of rope_neox with every frequency divided by ``factor``."""
        category = "position"

        def __init__(self, head_dim, theta, factor):
            self.inner = build_part("position", PartSpec("rope_neox", {"head_dim": head_dim, "theta": theta}))
            self.factor = float(factor)
            self._table = None

        def table(self, device):
            if self._table is None:
                self._table = (self.inner.inv_freq() / self.factor).to(device)
            return self._table

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

    register_part("position", "slow_rope", SlowRope)
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
            "position": PartSpec("slow_rope", {"head_dim": 32, "theta": 1e4, "factor": 4.0})})
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
    ang = plain_rope_angles(torch.arange(s_len), 32, 1e4) / 4.0
    gap = math.inf

    def swiglu(p, h):
        return plain_swiglu(h @ w[p + "gate_proj.weight"].to(F64).T,
                            h @ w[p + "up_proj.weight"].to(F64).T) @ w[p + "down_proj.weight"].to(F64).T

    for i in range(3):
        p = f"toy.{i}.mixer."
        h = plain_rmsnorm(x, w[f"toy.{i}.norm1.weight"], 1e-5)
        q = plain_rope_neox(plain_rmsnorm((h @ w[p + "q_proj.weight"].to(F64).T).view(s_len, 3, 32),
                                          w[p + "q_norm.weight"], 1e-5), ang)
        k = plain_rope_neox(plain_rmsnorm((h @ w[p + "k_proj.weight"].to(F64).T).view(s_len, 1, 32),
                                          w[p + "k_norm.weight"], 1e-5), ang)
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
    """A feed-forward with a router and experts (in some layers only) and a position encoding of
    its own, both defined here, registered and run through the engine in portions and token by
    token, against the plain functions."""
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
