"""The engine at the layer sizes and in the step shapes that ``bench.py`` times.

The tiny configurations never reach the paths a benchmark of the Qwen3-0.6B shape runs: the
products on pairs of SMs, the split-K few-rows product on a 311 MB head, the tcgen05 attention
over sixteen tiles, flash-decoding cut into many splits, batches of 64.  Here the layer sizes
are the benchmark's (hidden 1024, 16 heads over 8 kv heads of 128, intermediate 3072,
vocabulary 151,936, tied head; two layers instead of 28), the weights are the seeded random
weights that ``Engine(config=, seed=)`` makes on the device, and the bfloat16 engine is held
against the true 32-bit engine with the same weights (the reference checks its bfloat16 logits
against a second implementation the same way, docs/report.md:21-33).

Random weights give nearly flat attention, which would hide a lost tile of keys; so the q and
k head norms are scaled up in both engines until a query's weight sits on a few keys that lie
anywhere in its context.
"""
import pytest
import torch

from plain_qwen3 import load_folder, plain_forward
from util import BF16_RTOL, TINY, assert_close_logits, make_model, random_tokens

pytestmark = pytest.mark.gpu

BENCH_SHAPE = dict(
    architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=1024,
    num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
    max_position_embeddings=4096)
SHARPEN = 1.4          # factor on q_norm and k_norm: scores spread twice as wide (beyond that the
                       # rounding of bfloat16 queries and keys itself moves the logits past the tolerance)
SEED = 5


def _engines(max_tokens, max_requests, page_size=64, config=None, **kw):
    """A bfloat16 and a float32 engine with the same random weights (the device generator is
    seeded per tensor name), attention sharpened in both."""
    from tinyinfer_b200 import Engine
    pair = []
    for dtype in ("bfloat16", "float32"):
        eng = Engine(config=config or BENCH_SHAPE, seed=SEED, dtype=dtype, page_size=page_size,
                     max_tokens=max_tokens, max_requests=max_requests,
                     **(kw if dtype == "bfloat16" else {}))
        for blk in eng.model.blocks:
            blk.mixer.q_norm.mul_(SHARPEN)
            blk.mixer.k_norm.mul_(SHARPEN)
        pair.append(eng)
    a, b = pair
    wa, wb = a.model.blocks[1].ffn.w_down, b.model.blocks[1].ffn.w_down
    assert wa.dtype == wb.dtype == torch.bfloat16 and torch.equal(wa, wb)
    assert torch.equal(a.model.blocks[0].mixer.q_norm, b.model.blocks[0].mixer.q_norm)
    return a, b


def _check(got, want, what):
    """bfloat16 logits against the 32-bit ones: within the tolerance everywhere, and the same
    first choice wherever the 32-bit margin between first and second is wider than twice that."""
    assert_close_logits(got, want, BF16_RTOL, what)
    want = want.float()
    top2 = want.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 * BF16_RTOL * want.abs().max()
    same = got.argmax(dim=-1) == want.argmax(dim=-1)
    assert bool((same | ~clear).all()), f"{what}: another first choice although the margin is clear"
    return int(clear.sum())


def _tokens(n, seed):
    return random_tokens(BENCH_SHAPE["vocab_size"], n, seed)


def test_random_weights_on_the_device_are_reproducible_and_of_the_right_kind():
    """``Engine(config=, seed=)``: the same seed gives the same bits, another seed does not;
    matrices are bfloat16 N(0, 0.02), norm weights float32 around 1."""
    from tinyinfer_b200 import Engine
    small = dict(BENCH_SHAPE, vocab_size=2048, num_hidden_layers=1)
    a = Engine(config=small, seed=3, dtype="bfloat16", max_tokens=64, max_requests=1)
    b = Engine(config=small, seed=3, dtype="float32", max_tokens=64, max_requests=1)
    c = Engine(config=small, seed=4, dtype="bfloat16", max_tokens=64, max_requests=1)
    wa, wb, wc = (e.model.blocks[0].mixer.w_qkv for e in (a, b, c))
    assert wa.dtype == torch.bfloat16 and torch.equal(wa, wb) and not torch.equal(wa, wc)
    assert abs(wa.float().std().item() - 0.02) < 1e-3 and abs(wa.float().mean().item()) < 1e-3
    n = a.model.final_norm.weight
    assert n.dtype == torch.float32 and abs(n.mean().item() - 1.0) < 5e-3
    assert a.model.head.table is a.model.embedding.table
    assert torch.equal(a.model.embedding.table, b.model.embedding.table)


@pytest.mark.parametrize("page_size", [16, 64])
def test_prompt_of_2048_tokens_in_one_step(page_size):
    """What ``prefill`` times: one request's 2,048 tokens in one step, eagerly and replayed from
    the step's CUDA graph (the third step of a shape is the first replay)."""
    from tinyinfer_b200 import StepEntry
    bf, fp = _engines(3 * 2048, 4, page_size=page_size, step_graphs=True)
    want_at = [0, 1, 63, 64, 127, 128, 1000, 1023, 1024, 2046, 2047]
    clear = 0
    for i in range(3):
        toks = _tokens(2048, seed=40 + i)
        want = fp.step([StepEntry("p", toks, want_at)])
        got = bf.step([StepEntry("p", toks, want_at)]).clone()
        clear += _check(got, want, f"2,048-token prompt, page {page_size}, pass {i}")
        fp.finish("p")
        bf.finish("p")
    assert len(bf._step_graphs.graphs) == 1
    assert clear > 0
    bf.ops.check_status()


def test_long_prompt_with_two_heads_per_attention_block():
    """Prompts with several (head, tile) pairs per SM take the attention kernel that walks the keys
    once for two heads of a kv group; here a 2,048-token prompt is sent through it (forced) in two
    portions, the second one seeing the first through the cache, eagerly and from the graph."""
    from tinyinfer_b200 import StepEntry
    bf, fp = _engines(2 * 2048, 2, step_graphs=True)
    bf.ops.tc_attention_pairs_from = 0
    want_at = [0, 5, 127, 128, 700, 1023]
    before = bf.ops.launches
    for i in range(3):
        toks = _tokens(2048, seed=60 + i)
        for part in (toks[:1024], toks[1024:]):
            want = fp.step([StepEntry("p", part, want_at)])
            got = bf.step([StepEntry("p", part, want_at)]).clone()
            _check(got, want, f"2,048-token prompt in two portions, two heads per block, pass {i}")
        fp.finish("p")
        bf.finish("p")
    assert bf.ops.launches > before
    bf.ops.check_status()


def test_portions_that_reach_far_back():
    """Portions of a prompt past 6,144 keys (the step's `portion_reach` 2) take the two-heads
    attention kernel, with the keys of their tiles cut into runs when there are fewer blocks than
    SMs; shorter ones the one-head kernel, cut as well.  Against the 32-bit engine, eagerly and
    from the steps' graphs (a shape's graph is kept per class)."""
    from tinyinfer_b200 import StepEntry
    bf, fp = _engines(8192, 1, config=dict(BENCH_SHAPE, max_position_embeddings=8192), step_graphs=True)
    toks = _tokens(5120 + 5 * 512, seed=91)
    head = [StepEntry("p", toks[:5120], [])]
    bf.step(head)
    fp.step(head)
    classes = set()
    for i in range(5):                     # contexts 5,632 and 6,144: not long; 6,656 to 7,680: long
        lo = 5120 + i * 512
        entries = [StepEntry("p", toks[lo:lo + 512], [0, 130, 511])]
        want = fp.step(entries)
        got = bf.step(entries).clone()
        _check(got, want, f"512-token portion ending at {lo + 512}")
        classes.add(lo + 512 > 6144)
    assert classes == {False, True} and len(bf._step_graphs.graphs) == 2
    bf.ops.check_status()


@pytest.mark.parametrize("batch", [8, 64])
def test_batches_decoding_after_computed_prompts(batch):
    """Batch 8 and 64: prompts of 600 to 900 tokens run through the engine (several requests
    per step, as a scheduler would pack them), then 16 decode steps from the decode graphs."""
    from tinyinfer_b200 import StepEntry
    bf, fp = _engines(batch * 1024, batch)
    lengths = [600 + (37 * i) % 301 for i in range(batch)]
    ids = [f"d{i}" for i in range(batch)]
    prompts = [_tokens(n, seed=200 + i) for i, n in enumerate(lengths)]
    for lo in range(0, batch, 4):                      # about 3,000 tokens a step
        entries = [StepEntry(ids[i], prompts[i], []) for i in range(lo, min(batch, lo + 4))]
        bf.step(entries)
        fp.step(entries)
    feed = [_tokens(16, seed=900 + i) for i in range(batch)]
    clear = 0
    for s in range(16):
        entries = [StepEntry(ids[i], [feed[i][s]], [0]) for i in range(batch)]
        want = fp.step(entries)
        got = bf.decode_step(entries)
        clear += _check(got, want, f"batch {batch}, decode step {s}")
    assert clear > 0
    bf.ops.check_status()
    bf.cache.check()


def test_mixed_step_of_decoding_rows_beside_a_long_portion():
    """The benchmark's mixed step: 63 requests decode beside a 512-token portion of another
    request's prompt that has 1,024 earlier tokens in the cache; then the same shape again."""
    from tinyinfer_b200 import StepEntry
    bf, fp = _engines(64 * 1024 + 4096, 64, step_graphs=True)
    ids = [f"m{i}" for i in range(63)]
    lengths = [300 + (53 * i) % 600 for i in range(63)]
    for lo in range(0, 63, 4):
        entries = [StepEntry(ids[i], _tokens(lengths[i], seed=300 + i), [])
                   for i in range(lo, min(63, lo + 4))]
        bf.step(entries)
        fp.step(entries)
    long_prompt = _tokens(1024 + 3 * 512, seed=77)
    head = [StepEntry("long", long_prompt[:1024], [])]
    bf.step(head)
    fp.step(head)
    for i in range(3):                                  # the third is replayed from the graph
        lo = 1024 + i * 512
        entries = [StepEntry(r, [(7 * i + 11 * k) % 1000], [0]) for k, r in enumerate(ids)]
        entries.append(StepEntry("long", long_prompt[lo:lo + 512], [0, 255, 511]))
        want = fp.step(entries)
        got = bf.step(entries).clone()
        _check(got, want, f"mixed step {i}")
    assert len(bf._step_graphs.graphs) == 1
    bf.ops.check_status()


@pytest.mark.parametrize("decoders,before", [(3, 384), (8, 384), (40, 384), (5, 6400)])
def test_decoding_rows_run_beside_a_portion_with_the_same_bits(decoders, before):
    """In a step of single-token rows and a prompt portion, flash-decoding is released by the
    prompt-attention kernel after that kernel's own wait and runs beside it, with one block
    waiting for it at the end.  The logits are those of the two kernels one after the other,
    eagerly and replayed from the step's graph; with 6,400 earlier tokens the portion takes the
    two-heads kernel."""
    from tinyinfer_b200 import Engine, StepEntry
    eng = Engine(config=dict(BENCH_SHAPE, max_position_embeddings=8192), seed=SEED, dtype="bfloat16",
                 max_tokens=decoders * 512 + before + 1664, max_requests=decoders + 1, step_graphs=True)
    for blk in eng.model.blocks:
        blk.mixer.q_norm.mul_(SHARPEN)
        blk.mixer.k_norm.mul_(SHARPEN)
    ids = [f"s{i}" for i in range(decoders)]
    prompts = [_tokens(200 + 37 * (i % 7), seed=500 + i) for i in range(decoders)]
    long_prompt = _tokens(before + 3 * 300, seed=78)
    assert eng.ops.attention_side_by_side
    logits = {}
    try:
        eng.ops.split_prompt_keys = False       # (whether a tile's keys are cut depends on the order)
        for beside in (False, True):
            eng.ops.attention_side_by_side = beside
            for lo in range(0, decoders, 4):
                eng.step([StepEntry(ids[i], prompts[i], []) for i in range(lo, min(decoders, lo + 4))])
            eng.step([StepEntry("long", long_prompt[:before], [])])
            outs = []
            for i in range(3):                          # the third is replayed from the graph
                lo = before + i * 300
                entries = [StepEntry(r, [(5 * i + 13 * k) % 1000], [0]) for k, r in enumerate(ids)]
                entries.append(StepEntry("long", long_prompt[lo:lo + 300], [0, 150, 299]))
                outs.append(eng.step(entries).clone())
            logits[beside] = torch.stack(outs)
            for r in ids + ["long"]:
                eng.finish(r)
            eng._step_graphs = type(eng._step_graphs)(eng)      # captured with this order of launches
    finally:
        eng.ops.attention_side_by_side = eng.ops.split_prompt_keys = True
    eng.ops.check_status()
    eng.cache.check()
    assert torch.isfinite(logits[True]).all()
    assert torch.equal(logits[True], logits[False])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_at_later_starts_beside_decoding_rows(tmp_path_factory, dtype):
    """Tiny-E (head size 128) against the plain implementation: portions of 130 to 300 tokens
    that start in the middle of a request, beside single tokens of other requests."""
    from tinyinfer_b200 import Engine, StepEntry
    from util import FP32_RTOL
    d = make_model(tmp_path_factory.getbasetemp(), "E")
    cfg, w = load_folder(d)
    vocab = TINY["E"]["vocab_size"]
    reqs = {"a": random_tokens(vocab, 600, 1), "b": random_tokens(vocab, 420, 2),
            "c": random_tokens(vocab, 202, 3), "d": random_tokens(vocab, 66, 4)}
    plain = {r: plain_forward(cfg, w, t, emulate_bf16=(dtype == "bfloat16")) for r, t in reqs.items()}
    cuts = [  # step -> request -> (from, to)
        {"a": (0, 100), "c": (0, 199)},
        {"a": (100, 400), "c": (199, 200), "b": (0, 128)},
        {"a": (400, 401), "b": (128, 420), "c": (200, 201), "d": (0, 64)},
        {"a": (401, 600), "c": (201, 202), "d": (64, 65)},
        {"d": (65, 66)},
    ]
    eng = Engine(d, dtype=dtype, page_size=64, max_tokens=1600, max_requests=4)
    tol = FP32_RTOL if dtype == "float32" else BF16_RTOL
    for i, step in enumerate(cuts):
        entries = [StepEntry(r, reqs[r][lo:hi], list(range(hi - lo))) for r, (lo, hi) in step.items()]
        got = eng.step(entries).cpu()
        want = torch.cat([plain[r][lo:hi] for r, (lo, hi) in step.items()])
        assert_close_logits(got, want, tol, f"tiny-E {dtype} step {i}")
    eng.ops.check_status()
