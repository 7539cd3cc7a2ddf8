"""The engine on the GPU beyond replay: long decoding, the first tokens of a sequence, graph
replay against eager, generation through the entry points, sharp attention, the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

import traces
from plain_qwen3 import load_folder, plain_forward, plain_greedy
from tinyinfer_b200.weights import write_safetensors
from util import BF16_RTOL, FP32_RTOL, TINY, assert_close_logits, make_model, random_tokens

pytestmark = pytest.mark.gpu
TOL = {"float32": FP32_RTOL, "bfloat16": BF16_RTOL}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _engine(model_dir, dtype, max_tokens=1024, **kw):
    from tinyinfer_b200 import Engine
    return Engine(model_dir, dtype=dtype, page_size=16, max_tokens=max_tokens, max_requests=8, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_long_decoding(tmp_path_factory, name, dtype):
    """Hundreds of tokens one by one (eagerly and from the graph) against the whole sequence."""
    from tinyinfer_b200 import StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), name)
    cfg, w = load_folder(d)
    n = min(460, cfg["max_position_embeddings"])
    toks = random_tokens(cfg["vocab_size"], n, seed=9)
    ref = plain_forward(cfg, w, toks, emulate_bf16=(dtype == "bfloat16"))
    eng = _engine(d, dtype)
    rows = [eng.step([StepEntry("e", toks[:7], list(range(7)))]).cpu()]
    rows += [eng.step([StepEntry("e", [t], [0])]).cpu() for t in toks[7:]]
    assert_close_logits(torch.cat(rows), ref, TOL[dtype], f"{name} eager decoding")
    rows = [eng.step([StepEntry("g", toks[:7], list(range(7)))]).cpu()]
    rows += [eng.decode_step([StepEntry("g", [t], [0])]).cpu() for t in toks[7:]]
    assert_close_logits(torch.cat(rows), ref, TOL[dtype], f"{name} graph decoding")
    eng.ops.check_status()


@pytest.mark.parametrize("name", ["A", "D"])
def test_decoding_with_every_few_rows_product_on_the_split_k_kernel(tmp_path_factory, name):
    """The engine's small weights never reach the split-K tcgen05 product by themselves; forced
    onto it, prompts in portions, decoding and a mixed batch still match the plain implementation."""
    from tinyinfer_b200 import StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), name)
    cfg, w = load_folder(d)
    toks = random_tokens(cfg["vocab_size"], 90, seed=4)
    other = random_tokens(cfg["vocab_size"], 40, seed=5)
    ref = plain_forward(cfg, w, toks, emulate_bf16=True)
    ref_other = plain_forward(cfg, w, other, emulate_bf16=True)
    eng = _engine(d, "bfloat16")
    keep = eng.ops.few_tc_min_bytes                  # (the engine has a kernel set of its own)
    eng.ops.few_tc_min_bytes = 0
    before = eng.ops.launches
    try:
        rows = [eng.step([StepEntry("a", toks[:30], list(range(30)))]).cpu()]
        both = eng.step([StepEntry("a", toks[30:50], list(range(20))), StepEntry("b", other, list(range(40)))]).cpu()
        rows.append(both[:20])
        rows += [eng.step([StepEntry("a", [t], [0])]).cpu() for t in toks[50:]]
    finally:
        eng.ops.few_tc_min_bytes = keep
    assert_close_logits(torch.cat(rows), ref, BF16_RTOL, f"{name} on the split-K product")
    assert_close_logits(both[20:], ref_other, BF16_RTOL, f"{name} second request on the split-K product")
    assert eng.ops.launches > before
    eng.ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tmp_path_factory, dtype):
    from tinyinfer_b200 import StepEntry
    for name in ("A", "B", "D"):
        d = make_model(tmp_path_factory.getbasetemp(), name)
        cfg, w = load_folder(d)
        toks = random_tokens(cfg["vocab_size"], 4, seed=3)
        ref = plain_forward(cfg, w, toks, emulate_bf16=(dtype == "bfloat16"))
        eng = _engine(d, dtype)
        alone = eng.step([StepEntry("one", toks[:1], [0])])                 # a prompt of one token
        assert_close_logits(alone, ref[:1], TOL[dtype], f"{name} one-token prompt")
        nxt = eng.step([StepEntry("one", toks[1:2], [0])])                  # its first decoded token
        assert_close_logits(nxt, ref[1:2], TOL[dtype], f"{name} position 1")
        pair = eng.step([StepEntry("two", toks[:2], [0, 1])])
        assert_close_logits(pair, ref[:2], TOL[dtype], f"{name} two-token prompt")
        rest = eng.step([StepEntry("two", toks[2:], [0, 1]), StepEntry("one", toks[2:3], [0])])
        assert_close_logits(rest, torch.cat([ref[2:4], ref[2:3]]), TOL[dtype], f"{name} positions 2, 3")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_eager_bit_for_bit(tmp_path_factory, dtype):
    """The same decode steps, eagerly and replayed from CUDA graphs, for batches of 1 to 5
    requests of different lengths (so that padding rows and several buckets are used)."""
    from tinyinfer_b200 import StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), "D")
    vocab = TINY["D"]["vocab_size"]
    prompts = [random_tokens(vocab, n, seed=n) for n in (70, 3, 129, 31, 64)]
    feed = [random_tokens(vocab, 12, seed=100 + i) for i in range(5)]
    results = []
    for graph in (False, True):
        eng = _engine(d, dtype, max_tokens=2048)
        out = []
        for live in (1, 3, 5, 2):
            ids = [f"{live}-{i}" for i in range(live)]
            eng.step([StepEntry(r, prompts[i], []) for i, r in enumerate(ids)])
            for s in range(12):
                entries = [StepEntry(r, [feed[i][s]], [0]) for i, r in enumerate(ids)]
                lg = eng.decode_step(entries) if graph else eng.step(entries)
                out.append(lg.clone())
            for r in ids:
                eng.finish(r)
        results.append(torch.cat(out))
        eng.ops.check_status()
    assert torch.equal(results[0], results[1]), "graph replay and eager steps differ"


@pytest.mark.parametrize("name", ["C", "D"])
def test_graph_replay_with_requests_coming_going_and_changing_rows(tmp_path_factory, name):
    """Replayed decode steps keep a host mirror of each row's block table and send only what a
    request gained.  Here requests finish, new ones take their rows, the order of the batch
    changes, an id is used again and (configuration C) windows give pages back: every step must
    equal the eager engine bit for bit."""
    from tinyinfer_b200 import StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), name)
    vocab = TINY[name]["vocab_size"]
    limit = TINY[name]["max_position_embeddings"]
    rng = torch.Generator().manual_seed(5)
    engines = [_engine(d, "bfloat16", max_tokens=4096), _engine(d, "bfloat16", max_tokens=4096)]
    live, fresh, out = [], 0, [[], []]
    lengths = {}
    for step in range(70):
        if step % 9 == 0 and len(live) < 4:                       # a new request joins
            rid = f"r{fresh % 5}"                                 # ids come round again
            fresh += 1
            if rid not in live:
                prompt = random_tokens(vocab, 5 + 13 * (fresh % 4), seed=fresh)
                for eng in engines:
                    eng.step([StepEntry(rid, prompt, [])])
                live.append(rid)
                lengths[rid] = len(prompt)
        if step % 13 == 12 and live:                              # the oldest one finishes
            gone = live.pop(0)
            for eng in engines:
                eng.finish(gone)
        if step % 7 == 6:                                         # the batch changes its order
            live = live[1:] + live[:1]
        live = [r for r in live if lengths[r] < limit - 1]
        if not live:
            continue
        toks = torch.randint(0, vocab, (len(live),), generator=rng).tolist()
        entries = [StepEntry(r, [t], [0]) for r, t in zip(live, toks)]
        out[0].append(engines[0].step(entries).clone())
        out[1].append(engines[1].decode_step(entries).clone())
        for r in live:
            lengths[r] += 1
    assert len(out[0]) > 50
    for a, b in zip(out[0], out[1]):
        assert torch.equal(a, b), "graph replay and eager steps differ"
    for eng in engines:
        eng.ops.check_status()
        eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_step_graphs_equal_eager_bit_for_bit(tmp_path_factory, dtype):
    """Steps of a shape seen before are replayed from CUDA graphs: prompt portions of the same
    sizes for different requests at different positions, and mixed steps, give the same bits."""
    from tinyinfer_b200 import StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), "D")
    vocab = TINY["D"]["vocab_size"]
    toks = {r: random_tokens(vocab, 400, seed=i) for i, r in enumerate("abcd")}
    results = []
    for graphs in (False, True):
        eng = _engine(d, dtype, max_tokens=2048, step_graphs=graphs)
        out = []
        done = {r: 0 for r in toks}
        def portion(r, n, want):
            e = StepEntry(r, toks[r][done[r]:done[r] + n], want)
            done[r] += n
            return e
        for rnd in range(4):
            for r in "abcd":                                   # the same shape 16 times
                out.append(eng.step([portion(r, 70, [0, 69])]).clone())
            out.append(eng.step([portion("a", 1, [0]), portion("b", 20, [19]), portion("c", 2, [1])]).clone())
        if graphs:
            assert len(eng._step_graphs.graphs) == 2 and eng.ops.launches > 0
        results.append(torch.cat(out))
        eng.ops.check_status()
    assert torch.equal(results[0], results[1]), "replayed steps differ from eager steps"


@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, graph):
    from tinyinfer_b200 import LLM, SamplingParams
    d = make_model(tmp_path_factory.getbasetemp(), "B")
    cfg, w = load_folder(d)
    prompts = [random_tokens(512, n, seed=n) for n in (1, 9, 33, 64)]
    want = [plain_greedy(cfg, w, p, 12) for p in prompts]
    llm = LLM(d, dtype="float32", max_seq=128, max_num_seqs=4, max_batched_tokens=48, chunk=16,
              kv_tokens=160, page_size=16, cuda_graph=graph)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12))
    assert [o.tokens for o in outs] == want
    assert llm.stats.preemptions >= 1                    # 160 tokens of cache for four requests
    llm.engine.cache.check()
    # bfloat16: the same tokens unless two logits are within rounding of each other
    outs16 = LLM(d, dtype="bfloat16", max_seq=128, max_num_seqs=4, cuda_graph=graph).generate(
        prompts, SamplingParams(max_tokens=12))
    agree = sum(a == b for o, ww in zip(outs16, want) for a, b in zip(o.tokens, ww))
    assert agree >= 40, f"bfloat16 greedy tokens agree in only {agree} of 48 places"


def test_steps_launched_ahead_give_the_same_tokens(tmp_path_factory):
    """With graphs a decode step is launched before the ids of the step before it are read, its
    tokens fed on the device.  The same tokens as without that, also when a request stops on a
    stop token in the middle (its extra step is dropped), when the pool is so small that
    requests are preempted, and with sampling."""
    from tinyinfer_b200 import LLM, SamplingParams
    d = make_model(tmp_path_factory.getbasetemp(), "B")
    prompts = [random_tokens(512, n, seed=n) for n in (5, 9, 33, 64)]
    kw = dict(dtype="bfloat16", max_seq=128, max_num_seqs=4, page_size=16, cuda_graph=True)
    base = LLM(d, lookahead=False, **kw)
    plain = base.generate(prompts, SamplingParams(max_tokens=20))
    # every request gets a stop token that it meets at a different place
    stops = [SamplingParams(max_tokens=20, stop_token_ids=(o.tokens[3 + 4 * i],)) for i, o in enumerate(plain)]
    temp = [SamplingParams(temperature=0.7, seed=3 + i, max_tokens=15) for i in range(4)]
    for params, more in ((SamplingParams(max_tokens=20), {}), (stops, {}), (temp, {}),
                         (SamplingParams(max_tokens=20), {"kv_tokens": 192})):
        want = LLM(d, lookahead=False, **kw, **more).generate(prompts, params)
        llm = LLM(d, **kw, **more)
        got = llm.generate(prompts, params)
        assert [o.tokens for o in got] == [o.tokens for o in want]
        assert [o.finish_reason for o in got] == [o.finish_reason for o in want]
        llm.engine.cache.check()
        assert llm.engine.cache.live_requests() == []
    assert any(o.finish_reason == "stop" and len(o.tokens) < 20
               for o in LLM(d, **kw).generate(prompts, stops))


def test_temperature_sampling_is_reproducible_across_cuttings(tmp_path_factory):
    """tiny-B, temperature 0.8 with a fixed seed: the same tokens whether prompts run whole or
    in portions of 16 beside decoding, eager or from graphs."""
    from tinyinfer_b200 import LLM, SamplingParams
    d = make_model(tmp_path_factory.getbasetemp(), "B")
    prompts = [random_tokens(512, n, seed=n) for n in (1, 9, 33, 64)]
    sp = SamplingParams(temperature=0.8, seed=1234, max_tokens=12)
    a = LLM(d, dtype="float32", max_seq=128, max_num_seqs=4, max_batched_tokens=256).generate(prompts, sp)
    b = LLM(d, dtype="float32", max_seq=128, max_num_seqs=4, max_batched_tokens=32, chunk=16,
            cuda_graph=True).generate(prompts, sp)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    assert len({tuple(o.tokens) for o in a}) > 1


def _sharpen(model_dir, out_dir, factor):
    """A copy of the model whose per-head q/k norm weights are scaled, so that attention is
    sharper: a key that is missed or wrongly included moves the logits more."""
    cfg, w = load_folder(model_dir)
    w = {k: (v * factor if ("q_norm" in k or "k_norm" in k) else v) for k, v in w.items()}
    os.makedirs(out_dir, exist_ok=True)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), w)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return out_dir


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_sharp_attention_at_window_and_page_edges(tmp_path_factory, tmp_path, name, dtype):
    """Scores scaled by 1.5^2 (further sharpening would amplify float32 rounding itself beyond
    the tolerance).  A window that is one key too wide moves the logits by tens of times the
    tolerance, so an edge that is off by one cannot pass."""
    from tinyinfer_b200 import StepEntry
    d = _sharpen(make_model(tmp_path_factory.getbasetemp(), name), str(tmp_path / "sharp"), 1.5)
    cfg, w = load_folder(d)
    emulate = dtype == "bfloat16"
    reqs = {f"r{i}": random_tokens(cfg["vocab_size"], n, seed=70 + i)
            for i, n in enumerate([130, 47, 260, 64, 33, 200])}
    plain = {r: plain_forward(cfg, w, t, emulate_bf16=emulate) for r, t in reqs.items()}
    wider = plain_forward({**cfg, "sliding_window": cfg["sliding_window"] + 1}, w, reqs["r0"],
                          emulate_bf16=emulate)
    moved = (wider - plain["r0"]).abs().max().item() / plain["r0"].abs().max().item()
    assert moved > 10 * TOL[dtype], f"a window one key too wide moves the logits by only {moved:.2e}"
    for family in (traces.portions, traces.mixed):
        steps = family(reqs)
        eng = _engine(d, dtype, max_tokens=traces.max_live_tokens(steps))
        outputs = {}
        for s in steps:
            outputs[s["step"]] = eng.step(
                [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).cpu()
            for r in s["end"]:
                eng.finish(r)
        for r, items in traces.collect(steps, outputs).items():
            got = torch.stack([row for _, row in items])
            assert_close_logits(got, plain[r][[p for p, _ in items]], TOL[dtype],
                                f"sharp {name} {family.__name__} {r}")
        eng.ops.check_status()


def test_command_line(tmp_path_factory):
    d = make_model(tmp_path_factory.getbasetemp(), "B")
    cfg, w = load_folder(d)
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "tinyinfer"), "-m", d, "-n", "5", "-p", "7 8 9",
         "-p", "100,200", "--dtype", "float32", "--max-seq", "64", "--cuda-graph"],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    outs = [l.split("] ", 1)[1] for l in proc.stdout.splitlines() if l.startswith("[output]")]
    assert outs == [" ".join(map(str, plain_greedy(cfg, w, p, 5))) for p in ([7, 8, 9], [100, 200])]
    assert "tok/s [cuda-graph: on]" in proc.stderr
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "tinyinfer"), "-m", d],
                         capture_output=True, text=True, timeout=120)
    assert bad.returncode == 1 and "usage" in bad.stderr


def test_engine_from_configuration_and_seed_equals_the_written_model(tmp_path):
    """Random weights are a function of (seed, tensor name, element): drawn on the GPU they have
    the bits of the folder written on the host, so the two engines give the same logits."""
    from tinyinfer_b200 import Engine, StepEntry, write_random_model
    from tinyinfer_b200.parts.base import MATRIX, WeightSpec
    from tinyinfer_b200.weights.random_init import random_tensor
    from util import TINY, random_tokens
    spec = WeightSpec((300, 70), MATRIX)
    host = random_tensor(11, "some.weight", spec, dtype=torch.float32)
    assert torch.equal(host, random_tensor(11, "some.weight", spec, device="cuda:0", dtype=torch.float32).cpu())
    cfg = TINY["D"]
    folder = str(tmp_path / "written")
    write_random_model(folder, cfg, seed=21)
    toks = random_tokens(cfg["vocab_size"], 40, seed=2)
    for dtype in ("float32", "bfloat16"):
        a = Engine(folder, dtype=dtype, max_tokens=256, max_requests=2)
        b = Engine(config=cfg, seed=21, dtype=dtype, max_tokens=256, max_requests=2)
        la = a.step([StepEntry("r", toks, list(range(40)))])
        lb = b.step([StepEntry("r", toks, list(range(40)))])
        assert torch.equal(la, lb), f"{dtype}: weights drawn on the device differ from the written ones"
        a.ops.check_status()
