"""The engine's host logic (step function, block tables, windows, generation loop) run through
the plain PyTorch statement of the kernels, so that it is tested without a GPU.  The product
itself has no CPU path; the kernel set used here lives under tests/."""
import pytest
import torch

import traces
from plain_qwen3 import load_folder, plain_forward, plain_greedy
from ref_ops import RefOps
from tinyinfer_b200 import Engine, LLM, SamplingParams, StepEntry
from tinyinfer_b200.cache import OutOfPages
from tinyinfer_b200.kernels import KernelError
from util import TINY, assert_close_logits, make_model, random_tokens


def _requests(name, lengths):
    return {f"r{i}": random_tokens(TINY[name]["vocab_size"], n, seed=50 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name,lengths", [("A", [40, 9, 70, 33, 2]), ("C", [90, 30, 120, 45])])
@pytest.mark.parametrize("family", ["tail", "portions", "mixed"])
def test_cuttings_on_the_host_path(tmp_path, name, lengths, family):
    d = make_model(tmp_path, name)
    cfg, w = load_folder(d)
    reqs = _requests(name, lengths)
    steps = {"tail": traces.tail_decoded, "portions": traces.portions, "mixed": traces.mixed}[family](reqs)
    eng = Engine(d, dtype="float32", device="cpu", ops=RefOps(), page_size=16,
                 num_pages=traces.max_live_tokens(steps) // 16, max_requests=4)
    outputs = {}
    for s in steps:
        outputs[s["step"]] = eng.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        for r in s["end"]:
            eng.finish(r)
        eng.cache.check()
    for r, items in traces.collect(steps, outputs).items():
        ref = plain_forward(cfg, w, reqs[r])
        got = torch.stack([row for _, row in items])
        assert_close_logits(got, ref[[p for p, _ in items]], 2e-5, f"{name} {family} {r}")
    assert eng.cache.live_requests() == [] and eng.cache.free_pages() == [eng.cache.num_pages] * len(eng.cache.groups)


def test_step_refuses_what_it_cannot_run(tmp_path):
    d = make_model(tmp_path, "A")
    eng = Engine(d, dtype="float32", device="cpu", ops=RefOps(), page_size=16, num_pages=2, max_requests=2)
    with pytest.raises(ValueError, match="token id 256"):
        eng.step([StepEntry("a", [1, 256], [0])])
    with pytest.raises(IndexError, match="wanted place 3"):
        eng.step([StepEntry("a", [1, 2, 3], [3])])
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", list(range(40)), [])])
    assert eng.cache.live_requests() == []            # nothing was kept of the refused step
    with pytest.raises(ValueError, match="allows 128"):
        Engine(d, dtype="float32", device="cpu", ops=RefOps(), num_pages=20).step(
            [StepEntry("b", [1] * 129, [])])
    assert eng.step([]).shape == (0, 256)
    with pytest.raises(ValueError, match="dtype"):
        Engine(d, dtype="float16", device="cpu", ops=RefOps())


def test_engine_needs_cuda_kernels_without_injected_ops(tmp_path):
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(KernelError, match="CUDA device only"):
        Engine(make_model(tmp_path, "A"), dtype="float32")


def test_generation_loop_with_preemption_matches_plain_greedy(tmp_path):
    d = make_model(tmp_path, "B")
    cfg, w = load_folder(d)
    prompts = [random_tokens(512, n, seed=n) for n in (1, 9, 33, 64)]
    # so few pages that running requests are preempted and recomputed
    llm = LLM(d, dtype="float32", device="cpu", ops=RefOps(), max_seq=128, max_num_seqs=4,
              max_batched_tokens=48, chunk=16, kv_tokens=128)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12), log_steps=True)
    for p, o in zip(prompts, outs):
        assert o.tokens == plain_greedy(cfg, w, p, 12) and o.finish_reason == "length"
    assert llm.stats.preemptions >= 1 and sum(o.preemptions for o in outs) == llm.stats.preemptions
    assert any(len(step) > 1 and any(c > 1 for _, _, c in step) and any(c == 1 for _, _, c in step)
               for step in llm.stats.step_log), "no step mixed a prompt portion with decoding"
    llm.engine.cache.check()
    assert llm.engine.cache.live_requests() == []


def test_sampling_does_not_depend_on_the_batch(tmp_path):
    d = make_model(tmp_path, "B")
    prompts = [random_tokens(512, n, seed=n) for n in (5, 9, 17)]
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=7, max_tokens=6)
    together = LLM(d, dtype="float32", device="cpu", ops=RefOps(), max_seq=64, max_num_seqs=4,
                   max_batched_tokens=64).generate(prompts, sp)
    chunked = LLM(d, dtype="float32", device="cpu", ops=RefOps(), max_seq=64, max_num_seqs=2,
                  max_batched_tokens=8, chunk=4).generate(prompts, sp)
    assert [o.tokens for o in together] == [o.tokens for o in chunked]
    other_seed = LLM(d, dtype="float32", device="cpu", ops=RefOps(), max_seq=64).generate(
        prompts, SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=8, max_tokens=6))
    assert [o.tokens for o in other_seed] != [o.tokens for o in together]


def test_a_generation_can_be_stepped_and_streams_its_tokens(tmp_path):
    """``LLM.start`` + ``Session.step``: the tokens each step reports, put together, are what
    ``generate`` returns."""
    d = make_model(tmp_path, "A")
    prompts = [random_tokens(TINY["A"]["vocab_size"], n, seed=n) for n in (3, 20, 41)]
    sp = SamplingParams(max_tokens=9)
    kw = dict(dtype="float32", device="cpu", ops=RefOps(), max_seq=64, max_num_seqs=3, max_batched_tokens=24)
    want = LLM(d, **kw).generate(prompts, sp)
    session = LLM(d, **kw).start(prompts, sp)
    streamed = {i: [] for i in range(len(prompts))}
    while not session.done:
        for index, token in session.step():
            streamed[index].append(token)
    got = session.finish()
    assert [o.tokens for o in got] == [o.tokens for o in want]
    assert [streamed[i] for i in range(len(prompts))] == [o.tokens for o in want]


def test_request_span_reads_across_prompt_and_output():
    from tinyinfer_b200.engine.scheduler import Request
    r = Request(req_id="r", prompt=[1, 2, 3, 4], output=[5, 6, 7])
    for start in range(7):
        for count in range(0, 8 - start):
            assert r.span(start, count) == r.tokens[start:start + count]
    assert r.num_tokens == 7


def test_step_lists_are_packed_with_the_step():
    """Lists that a kernel set or a part derives from a step's shape travel in the step's one
    upload; the kernel set's own builders cut portions into tiles of a given height."""
    import numpy as np
    from tinyinfer_b200.engine.batch import StepList, build_lists, build_step_batch
    from tinyinfer_b200.kernels.step_lists import attention_lists
    entries = [StepEntry("a", [1] * 150, [149]), StepEntry("b", [2], [0]), StepEntry("c", [3] * 70, []),
               StepEntry("d", [4], [0])]
    starts = [10, 99, 300, 5]
    lists = attention_lists([64, 128]) + [StepList("twice", lambda q, s: np.asarray(q) * 2)]
    batch = build_step_batch(entries, starts, [[[0, 1, 2], [3, 4], [5, 6, 7, 8, 9, 10], [11]]], [0, 1, 2, 3],
                             torch.float32, "cpu", lists=lists)
    assert batch.lists["single_rows"].tolist() == [150, 221]
    assert batch.lists["portion_rows"].tolist() == list(range(150)) + list(range(151, 221))
    # tiles {request row, first flat token, rows}, the longest contexts first
    assert batch.lists["portion_tiles_64"].tolist() == [[2, 215, 6], [2, 151, 64], [0, 128, 22], [0, 64, 64], [0, 0, 64]]
    assert batch.lists["portion_tiles_128"].tolist() == [[2, 151, 70], [0, 128, 22], [0, 0, 128]]
    assert batch.lists["twice"].tolist() == [300, 2, 140, 2]
    assert batch.block_tables[0].shape == (4, 6) and batch.block_tables[0][1].tolist() == [3, 4, -1, -1, -1, -1]
    assert batch.positions[150].item() == 99 and batch.logit_rows.tolist() == [149, 150, 221]
    # the layout depends on the token counts only: other positions, the same addresses
    again = build_step_batch(entries, [0, 0, 0, 0], [[[0, 1, 2], [3, 4], [5, 6, 7, 8, 9, 10], [11]]],
                             [0, 1, 2, 3], torch.float32, "cpu", lists=lists)
    assert again.packed_size == batch.packed_size
    assert {k: tuple(v.shape) for k, v in again.lists.items()} == {k: tuple(v.shape) for k, v in batch.lists.items()}
    with pytest.raises(ValueError, match="two step lists"):
        build_lists([lists[0], lists[0]], [1], [0])
    with pytest.raises(TypeError, match="integers"):
        build_lists([StepList("bad", lambda q, s: np.asarray([0.5]))], [1], [0])


def test_a_step_is_classed_by_how_far_its_portions_reach_back():
    """Single tokens never count, however long their context; a portion counts by where it ends."""
    from tinyinfer_b200.engine.batch import LONG_CONTEXT, SHORT_CONTEXT, build_step_batch, portion_reach
    assert portion_reach([1, 1], [30000, 9000]) == 0
    assert portion_reach([512, 1], [SHORT_CONTEXT, 30000]) == 0
    assert portion_reach([512, 1], [SHORT_CONTEXT + 1, 5]) == 1
    assert portion_reach([2, 300], [LONG_CONTEXT, 400]) == 1
    assert portion_reach([2, 300], [LONG_CONTEXT + 1, 400]) == 2
    assert portion_reach([], []) == 0
    entries = [StepEntry("a", [1] * 40, []), StepEntry("b", [2], [0])]
    for start, want in ((0, 0), (SHORT_CONTEXT, 1), (LONG_CONTEXT, 2)):
        blocks = -(-(start + 40) // 16)
        batch = build_step_batch(entries, [start, 9000], [[list(range(blocks)), list(range(600))]], [0, 1],
                                 torch.float32, "cpu")
        assert batch.portion_reach == want


def test_which_prompt_attention_kernel_takes_a_step():
    """The choice between the one-head and the two-heads tcgen05 prompt kernels and the number of
    runs a tile's keys are cut into follow from the step's shape (B200: 148 SMs)."""
    from tinyinfer_b200.kernels.cuda_ops import choose_prompt_attention as choose
    sms = 148
    # a whole 2,048-token prompt of 16 heads: 256 pairs, one head per block, uncut
    assert choose(16, 16, sms, reach=1) == (False, 1)
    # 16,384 tokens: 128 tiles, many pairs per SM: two heads per block
    assert choose(128, 16, sms, reach=2) == (True, 1)
    # a fresh 512-token prompt: few key tiles per row, nothing to cut
    assert choose(4, 16, sms, reach=0) == (False, 1)
    # a 512-token portion at a context of 4,096: 64 pairs, two runs of one head; four of two heads pay
    assert choose(4, 16, sms, reach=1) == (True, 4)
    assert choose(4, 16, sms, reach=1, two_heads_ok=False) == (False, 2)
    # 1,024 tokens at a middling context: 128 pairs, left alone; far back: two heads, two runs
    assert choose(8, 16, sms, reach=1) == (False, 1)
    assert choose(8, 16, sms, reach=2) == (True, 2)
    # 2,048 tokens far back: two heads, uncut (128 blocks); with a window the walk is short
    assert choose(16, 16, sms, reach=2) == (True, 1)
    assert choose(16, 16, sms, reach=2, window=512) == (False, 1)
    # one tile: at most eight runs
    assert choose(1, 16, sms, reach=1) == (False, 8)
    # beside flash-decoding: uncut when its blocks fit on the SMs the uncut kernel leaves free
    assert choose(4, 16, sms, reach=1, decode_blocks=320) == (False, 1)
    assert choose(4, 16, sms, reach=1, decode_blocks=504) == (True, 4)
    # switched off
    assert choose(4, 16, sms, reach=1, cut_keys=False) == (False, 1)
    assert choose(128, 16, sms, reach=2, pairs_from=None) == (False, 1)
