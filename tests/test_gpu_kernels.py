"""Each CUDA kernel alone against its plain PyTorch statement, at sizes other than the engine's."""
import math
from types import SimpleNamespace

import pytest
import torch

from ref_ops import RefOps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from tinyinfer_b200.kernels import cuda_ops
    return cuda_ops(DEV)


def _rand(shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=DEV) * scale).to(dtype)


def _sum_rtol(k):
    """Bound on the rounding of a float32 sum of k products, as a fraction of the largest
    output: the error of a running sum grows like sqrt(k) roundings of 2^-24 each."""
    return 2e-7 * max(4.0, math.sqrt(k))


def _close(got, want, rtol, what):
    got, want = got.double(), want.double()
    err = (got - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= rtol * max(scale, 1e-30), f"{what}: error {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(ops, dtype):
    table = _rand((331, 80), dtype)
    tok = torch.tensor([0, 330, 7, 7, 100], dtype=torch.int32, device=DEV)
    out, ref = torch.empty((5, 80), device=DEV), torch.empty((5, 80), device=DEV)
    ops.embed(table, tok, out)
    RefOps().embed(table, tok, ref)
    assert torch.equal(out, ref)


@pytest.mark.parametrize("n", [1, 48, 80, 1000, 5120])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(ops, n, out_dtype):
    x = _rand((7, n), scale=3.0)
    w = 1 + _rand((n,), seed=1, scale=0.1)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    for r in (None, rows):
        k = 7 if r is None else 3
        out = torch.empty((k, n), dtype=out_dtype, device=DEV)
        ref = torch.empty((k, n), dtype=out_dtype, device=DEV)
        ops.rmsnorm(x, w, 1e-5, out, rows=r)
        RefOps().rmsnorm(x, w, 1e-5, ref, rows=r)
        _close(out, ref, 1e-6 if out_dtype == torch.float32 else 8e-3, f"rmsnorm n={n}")


@pytest.mark.parametrize("a_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 5, 3), (5, 261, 1024), (70, 130, 50), (129, 64, 17), (3, 331, 80)])
def test_linear_every_dtype_and_size(ops, a_dtype, w_dtype, shape):
    m, n, k = shape
    a, w = _rand((m, k), a_dtype), _rand((n, k), w_dtype, seed=1)
    base = _rand((m, n), seed=2)
    for acc in (False, True):
        out, ref = base.clone(), base.clone()
        ops.linear(a, w, out, accumulate=acc)
        RefOps().linear(a, w, ref, accumulate=acc)
        _close(out, a.double() @ w.double().T + (base.double() if acc else 0), _sum_rtol(k),
               f"linear {shape} acc={acc}")


@pytest.mark.parametrize("m", [1, 5, 8, 13, 33, 64])
@pytest.mark.parametrize("nk", [(48, 64), (100, 96), (4096, 1024), (1024, 3072), (331, 128)])
def test_linear_few_rows_bf16(ops, m, nk):
    """The decode product (tensor cores, operands straight from global memory)."""
    n, k = nk
    a, w = _rand((m, k), torch.bfloat16), _rand((n, k), torch.bfloat16, seed=1)
    base = _rand((m, n), seed=2)
    for acc in (False, True):
        out = base.clone()
        ops.linear(a, w, out, accumulate=acc)
        want = a.double() @ w.double().T + (base.double() if acc else 0)
        _close(out, want, _sum_rtol(k), f"few rows m={m} n={n} k={k} acc={acc}")
    # a row's result does not depend on how many rows there are
    alone = torch.empty((1, n), device=DEV)
    ops.linear(a[m - 1:m], w, alone)
    full = torch.empty((m, n), device=DEV)
    ops.linear(a, w, full)
    assert torch.equal(alone[0], full[m - 1])


@pytest.mark.parametrize("m", [1, 5, 16, 17, 33, 64])
@pytest.mark.parametrize("nk", [(48, 64), (100, 96), (1000, 520), (4096, 1024), (1024, 3072), (331, 128),
                                (6144, 2048), (20000, 256)])
def test_linear_few_rows_on_tcgen05(ops, m, nk):
    """The few-rows product for large weights (W as the MMA's 128-row side, K split over blocks,
    the last block of a tile adds the partial sums), forced here at every size."""
    n, k = nk
    a, w = _rand((m, k), torch.bfloat16), _rand((n, k), torch.bfloat16, seed=1)
    base = _rand((m, n), seed=2)
    keep = ops.few_tc_min_bytes
    ops.few_tc_min_bytes = 0
    try:
        before = ops.launches
        for acc in (False, True):
            out = base.clone()
            assert ops._few_tc(a, w, out, None, 1 if acc else 0)
            ops.check_status()
            want = a.double() @ w.double().T + (base.double() if acc else 0)
            _close(out, want, _sum_rtol(k), f"few rows on tcgen05 m={m} n={n} k={k} acc={acc}")
        assert ops.launches == before + 2
        # a row's result does not depend on how many rows there are, nor on the rows beside it
        alone = torch.empty((1, n), device=DEV)
        ops.linear(a[m - 1:m], w, alone)
        full = torch.empty((m, n), device=DEV)
        ops.linear(a, w, full)
        assert torch.equal(alone[0], full[m - 1])
        if n % 16 == 0:
            gate, up = w[:n // 2] * 0.2, w[n // 2:] * 0.2
            y = torch.zeros((m, n // 2), dtype=torch.bfloat16, device=DEV)
            ref = torch.empty_like(y)
            ops.gate_up_swiglu(a, ops.pack_gate_up(gate.contiguous(), up.contiguous()), y)
            r = RefOps()
            r.gate_up_swiglu(a, r.pack_gate_up(gate, up), ref)
            _close(y, ref, 8e-3, f"few rows on tcgen05, swiglu m={m} {nk}")
        ops.check_status()
    finally:
        ops.few_tc_min_bytes = keep


def test_large_weights_go_to_the_split_k_kernel(ops):
    """The dispatch: more than 32 MiB of weights and at most 64 rows."""
    w = _rand((6144, 4096), torch.bfloat16, seed=1, scale=0.05)
    a = _rand((8, 4096), torch.bfloat16)
    out = torch.empty((8, 6144), device=DEV)
    ops.linear(a, w, out)
    _close(out, a.double() @ w.double().T, _sum_rtol(4096), "6144 x 4096 at 8 rows")
    keep = ops.few_tc_min_bytes
    try:
        ops.few_tc_min_bytes = None
        other = torch.empty_like(out)
        ops.linear(a, w, other)
        assert not torch.equal(out, other), "both runs took the same kernel"
        _close(other, out, _sum_rtol(4096), "the two few-rows kernels")
    finally:
        ops.few_tc_min_bytes = keep
    # exactly 32 MiB stays with the other kernel: both settings give the same bits
    w = w[:4096]
    out = torch.empty((8, 4096), device=DEV)
    ops.linear(a, w, out)
    try:
        ops.few_tc_min_bytes = None
        other = torch.empty_like(out)
        ops.linear(a, w, other)
        assert torch.equal(out, other), "32 MiB of weights took the split-K kernel"
    finally:
        ops.few_tc_min_bytes = keep
    ops.check_status()


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("sizes", [(1024, 3072), (256, 640), (512, 1536), (2048, 2048)])
def test_decode_feed_forward_in_one_launch(ops, m, sizes):
    """gate/up, SwiGLU and down projection of a decode step as one launch (weights copied to
    shared memory ahead of the dependency wait): the same bits as the two launches, also when
    launched many times in a row (the arrival counters return to zero), and the plain formula."""
    from ref_ops import RefOps
    hidden, inter = sizes
    gate = _rand((inter, hidden), torch.bfloat16, seed=1, scale=0.05)
    up = _rand((inter, hidden), torch.bfloat16, seed=2, scale=0.05)
    down = _rand((hidden, inter), torch.bfloat16, seed=3, scale=0.05)
    x = _rand((m, hidden), torch.bfloat16, seed=4)
    res = _rand((m, hidden), torch.float32, seed=5)
    w_gu = ops.pack_gate_up(gate, up)
    assert ops.bf16.ti_ffn_decode_supported(m, hidden, inter, hidden, hidden, inter, inter, hidden)
    keep = ops.fuse_decode_ffn
    try:
        ops.fuse_decode_ffn = False
        want = res.clone()
        ops.swiglu_ffn(x, w_gu, down, want)
        ops.fuse_decode_ffn = True
        for _ in range(5):
            got = res.clone()
            ops.swiglu_ffn(x, w_gu, down, got)
            assert torch.equal(got, want), "the fused feed-forward differs from the two launches"
    finally:
        ops.fuse_decode_ffn = keep
    assert int(ops._ffn_counters[:2].view(torch.int64).item()) % ops.num_sms == 0, "a block did not arrive"
    r = RefOps()
    ref = res.clone()
    r.swiglu_ffn(x, r.pack_gate_up(gate, up), down, ref)
    _close(got, ref, 1e-2, f"fused feed-forward m={m} {sizes}")
    ops.check_status()


def _tail_inputs(m, hidden, inter, nq):
    return dict(
        attn=_rand((m, nq), torch.bfloat16, seed=6),
        w_o=_rand((hidden, nq), torch.bfloat16, seed=7, scale=0.05),
        norm_w=1.0 + 0.1 * _rand((hidden,), torch.float32, seed=8),
        gate=_rand((inter, hidden), torch.bfloat16, seed=1, scale=0.05),
        up=_rand((inter, hidden), torch.bfloat16, seed=2, scale=0.05),
        down=_rand((hidden, inter), torch.bfloat16, seed=3, scale=0.05),
        res=_rand((m, hidden), torch.float32, seed=5))


def _run_tail(o, t, w_gu, eps):
    """A mixer's last product, the norm and the feed-forward, as a block asks for them."""
    res = t["res"].clone()
    o.linear(t["attn"], t["w_o"], res, accumulate=True, may_defer=True)
    h = torch.empty(res.shape, dtype=torch.bfloat16, device=res.device)
    o.rmsnorm(res, t["norm_w"], eps, h)
    o.swiglu_ffn(h, w_gu, t["down"], res)
    o.flush()
    return res


@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("sizes", [(1024, 3072, 2048), (256, 640, 384), (512, 1536, 512), (1024, 2048, 1024)])
def test_decode_tail_in_one_launch(ops, m, sizes):
    """Output projection into the residual, norm of the residual and feed-forward as one launch:
    the same bits as the four launches (the norm adds its squares in the order of the
    block-per-row kernel), repeatedly, and the plain formula."""
    from ref_ops import RefOps
    hidden, inter, nq = sizes
    t = _tail_inputs(m, hidden, inter, nq)
    eps = 1e-5
    w_gu = ops.pack_gate_up(t["gate"], t["up"])
    assert ops.bf16.ti_attn_out_ffn_decode_supported(m, hidden, inter, nq, nq, nq, hidden, inter, inter, hidden)
    keep = ops.fuse_decode_tail, ops.fuse_decode_ffn
    try:
        ops.fuse_decode_tail = ops.fuse_decode_ffn = False
        want = _run_tail(ops, t, w_gu, eps)
        ops.fuse_decode_ffn = True
        assert torch.equal(_run_tail(ops, t, w_gu, eps), want), "the fused feed-forward differs"
        ops.fuse_decode_tail = True
        before = ops.launches
        for _ in range(4):
            got = _run_tail(ops, t, w_gu, eps)
            assert torch.equal(got, want), "the fused tail differs from the separate launches"
        assert ops.launches - before == 4, "the tail did not run as one launch"
    finally:
        ops.fuse_decode_tail, ops.fuse_decode_ffn = keep
    r = RefOps()
    ref = _run_tail(r, t, r.pack_gate_up(t["gate"], t["up"]), eps)
    _close(got, ref, 1e-2, f"fused tail m={m} {sizes}")
    ops.check_status()


def test_a_held_back_product_is_launched_by_whatever_comes_next(ops):
    """``linear(..., may_defer=True)`` may be held back; any other operation, ``flush()`` and
    ``stream()`` launch it, with the norm that was held back behind it."""
    m, hidden, inter, nq = 4, 256, 640, 384
    t = _tail_inputs(m, hidden, inter, nq)
    want = t["res"] + t["attn"].float() @ t["w_o"].float().T
    for how in ("flush", "stream", "linear", "norm of something else", "norm then linear"):
        res = t["res"].clone()
        ops.linear(t["attn"], t["w_o"], res, accumulate=True, may_defer=True)
        h = torch.empty((m, hidden), dtype=torch.bfloat16, device=DEV)
        if how == "flush":
            ops.flush()
        elif how == "stream":
            ops.stream()
        elif how == "linear":
            other = torch.zeros((m, hidden), device=DEV)
            ops.linear(t["attn"], t["w_o"], other)
        elif how == "norm of something else":
            ops.rmsnorm(t["res"], t["norm_w"], 1e-5, h)
        else:
            ops.rmsnorm(res, t["norm_w"], 1e-5, h)                    # held back too
            other = torch.zeros((m, hidden), device=DEV)
            ops.linear(t["attn"], t["w_o"], other)                    # launches both, in order
            x = res.double()
            normed = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * t["norm_w"].double()
            _close(h, normed, 1e-2, "the held-back norm")
        assert ops._pending is None
        _close(res, want, _sum_rtol(nq) * 4, f"held-back product launched by {how}")
    ops.check_status()


def test_decode_feed_forward_falls_back(ops):
    """More than 16 rows, or weights that do not fit into shared memory, take the two launches."""
    assert not ops.bf16.ti_ffn_decode_supported(17, 1024, 3072, 1024, 1024, 3072, 3072, 1024)
    assert not ops.bf16.ti_ffn_decode_supported(8, 4096, 12288, 4096, 4096, 12288, 12288, 4096)
    assert not ops.bf16.ti_ffn_decode_supported(8, 1000, 3072, 1000, 1000, 3072, 3072, 1000)
    from ref_ops import RefOps
    hidden, inter, m = 256, 640, 20
    gate = _rand((inter, hidden), torch.bfloat16, seed=1, scale=0.05)
    up = _rand((inter, hidden), torch.bfloat16, seed=2, scale=0.05)
    down = _rand((hidden, inter), torch.bfloat16, seed=3, scale=0.05)
    x = _rand((m, hidden), torch.bfloat16, seed=4)
    res = _rand((m, hidden), torch.float32, seed=5)
    got = res.clone()
    ops.swiglu_ffn(x, ops.pack_gate_up(gate, up), down, got)
    r = RefOps()
    ref = res.clone()
    r.swiglu_ffn(x, r.pack_gate_up(gate, up), down, ref)
    _close(got, ref, 1e-2, "feed-forward of 20 rows")
    ops.check_status()


@pytest.mark.parametrize("m", [65, 128, 129, 300, 1000])
@pytest.mark.parametrize("nk", [(128, 64), (136, 72), (4096, 1024), (1024, 3072), (1000, 520), (331, 128)])
def test_linear_many_rows_bf16(ops, m, nk):
    """The prefill product (tcgen05, TMA, tensor memory); (331, 128) falls to the plain kernel."""
    n, k = nk
    a, w = _rand((m, k), torch.bfloat16), _rand((n, k), torch.bfloat16, seed=1)
    base = _rand((m, n), seed=2)
    for acc in (False, True):
        out = base.clone()
        ops.linear(a, w, out, accumulate=acc)
        ops.check_status()
        want = a.double() @ w.double().T + (base.double() if acc else 0)
        _close(out, want, _sum_rtol(k), f"many rows m={m} n={n} k={k} acc={acc}")
    # a row's result does not depend on how many rows there are (above the few-rows kernel), as
    # long as K is cut the same way (an output of few tiles has its K cut into runs)
    if m >= 70:
        part = torch.empty((70, n), device=DEV)
        ops.linear(a[m - 70:], w, part)
        full = torch.empty((m, n), device=DEV)
        ops.linear(a, w, full)
        if ops.bf16.ti_gemm_tcgen05_splits(70, n, k, 0) == ops.bf16.ti_gemm_tcgen05_splits(m, n, k, 0):
            assert torch.equal(part, full[m - 70:])
        else:
            _close(part, full[m - 70:], _sum_rtol(k), "rows alone against rows among others")
        keep = ops.split_k_portions
        try:
            ops.split_k_portions = False
            ops.linear(a[m - 70:], w, part)
            ops.linear(a, w, full)
            assert torch.equal(part, full[m - 70:])
        finally:
            ops.split_k_portions = keep


@pytest.mark.parametrize("shape", [(512, 1024, 2048), (512, 1024, 3072), (128, 1024, 2048), (300, 1000, 1096),
                                   (575, 1024, 3072), (100, 2048, 520), (1024, 1024, 2048)])
def test_linear_with_k_cut_into_runs(ops, shape):
    """An output of few tiles (a short prompt portion into a narrow output) has its K cut into
    runs whose sums a second launch adds in ascending order of K: right against float64, store and
    accumulate, and the same from call to call; outputs of many tiles are not cut."""
    m, n, k = shape
    a, w = _rand((m, k), torch.bfloat16), _rand((n, k), torch.bfloat16, seed=1)
    base = _rand((m, n), seed=2)
    runs = ops.bf16.ti_gemm_tcgen05_splits(m, n, k, 0)
    assert 1 <= runs <= 8 and (runs == 1 or runs * 4 <= -(-k // 64))
    if ops.num_sms == 148:                   # what the rule's estimate picks on a B200
        assert runs == {(512, 1024, 2048): 4, (512, 1024, 3072): 4, (128, 1024, 2048): 8, (1024, 1024, 2048): 1,
                        (575, 1024, 3072): 3}.get(shape, runs)
    assert ops.bf16.ti_gemm_tcgen05_splits(m, n, k, 2) == 1        # never with the SwiGLU epilogue
    assert ops.bf16.ti_gemm_tcgen05_splits(2048, 1024, 2048, 1) == 1 # an output that fills the SMs is not cut
    for acc in (False, True):
        out = base.clone()
        ops.linear(a, w, out, accumulate=acc)
        again = base.clone()
        ops.linear(a, w, again, accumulate=acc)
        ops.check_status()
        assert torch.equal(out, again)
        want = a.double() @ w.double().T + (base.double() if acc else 0)
        _close(out, want, _sum_rtol(k), f"K in {runs} runs m={m} n={n} k={k} acc={acc}")


@pytest.mark.parametrize("shape", [(512, 1024, 2048), (128, 1024, 3072), (300, 1000, 2056), (100, 4096, 4096)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_norm_that_adds_the_runs_of_a_cut_product(ops, shape, accumulate):
    """A product whose K is cut, asked for with ``may_defer``, leaves its runs to the norm of its
    output that follows: output and normed rows have the bits of product, adding launch and
    norm in turn, with one launch less; anything else that follows adds the runs first."""
    m, n, k = shape
    a, w = _rand((m, k), torch.bfloat16), _rand((n, k), torch.bfloat16, seed=1, scale=0.05)
    base = _rand((m, n), seed=2)
    norm_w = 1.0 + 0.1 * _rand((n,), torch.float32, seed=3)
    assert ops.bf16.ti_gemm_tcgen05_splits(m, n, k, int(accumulate)) > 1
    keep = ops.norm_adds_runs
    res, normed, launches = {}, {}, {}
    try:
        for fused in (False, True):
            ops.norm_adds_runs = fused
            res[fused] = base.clone()
            normed[fused] = torch.zeros((m, n), dtype=torch.bfloat16, device=DEV)
            before = ops.launches
            ops.linear(a, w, res[fused], accumulate=accumulate, may_defer=True)
            ops.rmsnorm(res[fused], norm_w, 1e-6, normed[fused])
            ops.flush()
            launches[fused] = ops.launches - before
        # something else than the norm of that output comes next: the runs are added first
        other = base.clone()
        ops.linear(a, w, other, accumulate=accumulate, may_defer=True)
        h = torch.zeros((m, n), dtype=torch.bfloat16, device=DEV)
        ops.rmsnorm(base.clone(), norm_w, 1e-6, h)
        assert ops._pending_runs is None and torch.equal(other, res[False])
        ops.linear(a, w, other, accumulate=False, may_defer=True)
        ops.flush()
        assert ops._pending_runs is None
    finally:
        ops.norm_adds_runs = keep
    ops.check_status()
    assert torch.equal(res[True], res[False]) and torch.equal(normed[True], normed[False])
    assert launches[False] - launches[True] == 1
    want = a.double() @ w.double().T + (base.double() if accumulate else 0)
    _close(res[True], want, _sum_rtol(k), f"cut product m={m} n={n} k={k}")


@pytest.mark.parametrize("shape", [(2048, 4096, 1024), (1100, 5000, 520), (2048, 6144, 136), (4096, 2560, 64)])
def test_linear_on_pairs_of_sms(ops, shape):
    """Outputs with many 256 x 256 tiles run on pairs of SMs (tcgen05 cta_group::2): same bits as
    the one-SM kernel, right against float64."""
    m, n, k = shape
    a, w = _rand((m, k), torch.bfloat16), _rand((n, k), torch.bfloat16, seed=1)
    base = _rand((m, n), seed=2)
    assert ops._tc_gemm(m, n) is ops.bf16.ti_gemm_tcgen05_2sm
    for acc in (False, True):
        out = base.clone()
        ops.linear(a, w, out, accumulate=acc)
        ops.check_status()
        ops.use_2sm_gemm = False
        try:
            one = base.clone()
            ops.linear(a, w, one, accumulate=acc)
        finally:
            ops.use_2sm_gemm = True
        assert torch.equal(out, one), "pair kernel and one-SM kernel differ"
        _close(out, a.double() @ w.double().T + (base.double() if acc else 0), _sum_rtol(k),
               f"pairs {shape} acc={acc}")
    gate, up = _rand((n // 2, k), torch.bfloat16, seed=3, scale=0.2), _rand((n // 2, k), torch.bfloat16, seed=4, scale=0.2)
    y = torch.empty((m, n // 2), dtype=torch.bfloat16, device=DEV)
    ref = torch.empty_like(y)
    ops.gate_up_swiglu(a, ops.pack_gate_up(gate, up), y)
    r = RefOps()
    r.gate_up_swiglu(a, r.pack_gate_up(gate, up), ref)
    _close(y, ref, 8e-3, f"pairs swiglu {shape}")
    ops.check_status()


@pytest.mark.parametrize("m", [1, 8, 40, 64, 100])
@pytest.mark.parametrize("hk", [(128, 320), (1024, 3072), (80, 176), (64, 24)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_up_swiglu(ops, m, hk, dtype):
    hidden, inter = hk
    wdt = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    gate, up = _rand((inter, hidden), wdt, seed=1, scale=0.2), _rand((inter, hidden), wdt, seed=2, scale=0.2)
    h = _rand((m, hidden), dtype)
    out = torch.empty((m, inter), dtype=dtype, device=DEV)
    ref = torch.empty((m, inter), dtype=dtype, device=DEV)
    ops.gate_up_swiglu(h, ops.pack_gate_up(gate, up), out)
    r = RefOps()
    r.gate_up_swiglu(h, r.pack_gate_up(gate, up), ref)
    _close(out, ref, 2e-5 if dtype == torch.float32 else 8e-3, f"swiglu m={m} {hk}")


def _paged_case(num_heads, num_kv, hd, page_size, ctx_lens, q_lens, dtype, seed=0):
    """Requests with ``ctx_lens[r]`` tokens of which the last ``q_lens[r]`` are new; pages are
    handed out in a scrambled order so that neighbours in a request are far apart in memory."""
    r = len(ctx_lens)
    blocks = [-(-c // page_size) for c in ctx_lens]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(blocks)
    bt = torch.full((r, width), -1, dtype=torch.int32)
    it = iter(perm)
    for i, b in enumerate(blocks):
        bt[i, :b] = torch.tensor([next(it) for _ in range(b)], dtype=torch.int32)
    pages = _rand((num_pages, 2, num_kv, page_size, hd), dtype, seed=seed + 1)
    positions, req_of_tok = [], []
    for i, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        for j in range(ql):
            positions.append(c - ql + j)
            req_of_tok.append(i)
    ti = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    # the lists the kernel set asks of a step (single-token rows, portions cut into its tiles)
    from tinyinfer_b200.engine.batch import build_lists
    from tinyinfer_b200.kernels import cuda_ops
    lists = build_lists(cuda_ops(DEV).step_lists(torch.bfloat16), list(q_lens),
                        [c - ql for c, ql in zip(ctx_lens, q_lens)])
    step = SimpleNamespace(positions=ti(positions), req_of_tok=ti(req_of_tok),
                           lists={name: torch.from_numpy(a).to(torch.int32).to(DEV) for name, a in lists.items()},
                           max_position=max(ctx_lens), max_ctx_len=max(ctx_lens), scratch={})
    cache = SimpleNamespace(pages=pages, block_table=bt.to(DEV), page_size=page_size, writes=True)
    q = _rand((len(positions), num_heads * hd), dtype, seed=seed + 2)
    return step, cache, q


@pytest.mark.parametrize("case", [(4096, 512), (700, 128), (5000, 300), (1300, 1024), (129, 2)])
@pytest.mark.parametrize("window", [None, 600])
def test_prompt_attention_with_the_keys_of_a_tile_cut_into_runs(ops, case, window):
    """A step with fewer (tile, head) pairs than SMs cuts every tile's keys into runs of key tiles,
    a block each, and adds them in a second launch: against the plain statement, and close to
    the uncut kernel (they differ by the rounding of the partial sums only)."""
    from ref_ops import RefOps
    ctx, ql = case
    heads, kv, hd, ps = 8, 4, 128, 64
    step, cache, q = _paged_case(heads, kv, hd, ps, [ctx], [ql], torch.bfloat16, seed=4)
    # one key far back gets a large score for one query row: a lost run of keys would show
    far = 3 if window is None else max(0, ctx - ql - window + 5)
    page = int(cache.block_table[0, far // ps])
    cache.pages[page, 0, 1, far % ps] *= 6.0
    q[ql - 1, 2 * hd:3 * hd] = cache.pages[page, 0, 1, far % ps].to(q.dtype)
    scale = 1.0 / math.sqrt(hd)
    n_tiles = step.lists["portion_tiles_128"].shape[0]
    runs = ops.bf16.ti_attn_prefill_tc_splits(n_tiles, heads)
    assert runs == min(8, max(1, ops.num_sms // (n_tiles * heads)))
    out = {}
    keep = ops.split_prompt_keys
    try:
        for split in (False, True):
            ops.split_prompt_keys = split
            out[split] = torch.zeros_like(q)
            ops.paged_attention(q, step, cache, out[split], heads, kv, hd, window, scale)
    finally:
        ops.split_prompt_keys = keep
    ops.check_status()
    ref = torch.zeros_like(q)
    RefOps().paged_attention(q, step, cache, ref, heads, kv, hd, window, scale)
    _close(out[True], ref, 1.5e-2, f"cut into {runs} runs, context {ctx}, portion {ql}, window {window}")
    _close(out[True], out[False], 1e-2, "cut against uncut")
    if runs > 1:
        assert not torch.equal(out[True], out[False]) or ql <= 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("geom", [(4, 2, 16, 16), (3, 1, 48, 16), (16, 8, 128, 16), (8, 1, 64, 32),
                                  (6, 3, 80, 16), (32, 2, 32, 16), (5, 5, 144, 16), (2, 1, 256, 64)])
@pytest.mark.parametrize("window", [None, 1, 37])
def test_paged_attention(ops, dtype, geom, window):
    """Decoding rows and prompt portions side by side, lengths around the edges of pages and
    tiles, against the plain statement."""
    heads, kv, hd, ps = geom
    ctx = [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 200, 517, 40, 129, 300, 64, 700]
    qls = [1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 23, 2, 300, 64, 131]
    step, cache, q = _paged_case(heads, kv, hd, ps, ctx, qls, dtype)
    out, ref = torch.zeros_like(q), torch.zeros_like(q)
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(q, step, cache, out, heads, kv, hd, window, scale)
    RefOps().paged_attention(q, step, cache, ref, heads, kv, hd, window, scale)
    ops.check_status()
    _close(out, ref, 2e-5 if dtype == torch.float32 else 1.5e-2, f"attention {geom} window={window}")


@pytest.mark.parametrize("geom", [(16, 8, 128, 16), (4, 1, 128, 32), (6, 6, 128, 16), (4, 2, 128, 64),
                                  (2, 1, 128, 128), (3, 1, 128, 48), (2, 2, 128, 256)])
@pytest.mark.parametrize("window", [None, 1, 200])
def test_prompt_attention_on_tcgen05_matches_the_mma_kernel_and_the_plain_statement(ops, geom, window):
    """Head size 128 takes the tcgen05 kernel: long and short portions, earlier context, ragged ends."""
    heads, kv, hd, ps = geom
    ctx = [700, 128, 129, 1, 300, 1000, 257, 64]
    qls = [131, 128, 129, 1, 2, 1000, 129, 33]
    step, cache, q = _paged_case(heads, kv, hd, ps, ctx, qls, torch.bfloat16, seed=3)
    scale = 1.0 / math.sqrt(hd)
    got, ref, mma = torch.zeros_like(q), torch.zeros_like(q), torch.zeros_like(q)
    assert ops.use_tc_attention
    ops.paged_attention(q, step, cache, got, heads, kv, hd, window, scale)
    ops.check_status()
    ops.use_tc_attention = False
    try:
        ops.paged_attention(q, step, cache, mma, heads, kv, hd, window, scale)
    finally:
        ops.use_tc_attention = True
    RefOps().paged_attention(q, step, cache, ref, heads, kv, hd, window, scale)
    _close(mma, ref, 1.5e-2, f"mma attention {geom} window={window}")
    _close(got, ref, 1.5e-2, f"tcgen05 attention {geom} window={window}")
    # the kernel with two heads of a kv group per block (for long prompts), forced on this case
    if ops.bf16.ti_attn_prefill_tc2_supported(hd, ps, heads, kv):
        keep = ops.tc_attention_pairs_from
        ops.tc_attention_pairs_from = 0
        try:
            pairs = torch.zeros_like(q)
            before = ops.launches
            ops.paged_attention(q, step, cache, pairs, heads, kv, hd, window, scale)
            ops.check_status()
        finally:
            ops.tc_attention_pairs_from = keep
        _close(pairs, ref, 1.5e-2, f"tcgen05 attention, two heads per block {geom} window={window}")


def test_decode_attention_finds_a_far_key(ops):
    """One key among thousands carries the whole weight: its value must come back."""
    heads, kv, hd, ps = 8, 2, 64, 16
    ctx = [3000, 2049]
    step, cache, q = _paged_case(heads, kv, hd, ps, ctx, [1, 1], torch.bfloat16, seed=5)
    cache.pages.mul_(0.05)
    targets = [(0, 1234), (1, 2048 - 33)]
    for r, p in targets:
        page = int(cache.block_table[r, p // ps])
        for h in range(kv):
            cache.pages[page, 0, h, p % ps, :] = 4.0
            cache.pages[page, 1, h, p % ps, :] = torch.arange(hd, device=DEV).to(torch.bfloat16)
    q.fill_(4.0)
    out = torch.zeros_like(q)
    ops.paged_attention(q, step, cache, out, heads, kv, hd, None, 1.0 / math.sqrt(hd))
    want = torch.arange(hd, device=DEV).to(torch.bfloat16).float().repeat(heads)
    for row in range(2):
        assert (out[row].float() - want).abs().max() < 0.51, "the far key's value was not returned"


def _rotation(hd, rotary_dim=None, theta=1e6):
    from tinyinfer_b200.parts import Rotation
    rot = hd if rotary_dim is None else rotary_dim
    if rot == 0:
        return Rotation("none", 0, None)
    inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64),
                         -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).float().to(DEV)
    return Rotation("neox", rot, inv_freq)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("geom", [(4, 2, 16, 16, None), (3, 1, 48, 16, None), (16, 8, 128, 32, None),
                                  (5, 5, 144, 16, None), (3, 1, 48, 16, 20), (4, 2, 128, 16, 64),
                                  (2, 2, 80, 16, 0), (6, 2, 33, 16, 0)])
def test_qk_norm_rope_store(ops, dtype, geom):
    """Also with a rotation over a part of the head only, and with none at all."""
    heads, kv, hd, ps, rotary = geom
    ctx, qls = [5, 33, 64, 100], [5, 1, 17, 2]
    step, cache, _ = _paged_case(heads, kv, hd, ps, ctx, qls, dtype)
    t = step.positions.shape[0]
    qkv = _rand((t, (heads + 2 * kv) * hd), seed=3, scale=2.0)
    qw, kw = 1 + _rand((hd,), seed=4, scale=0.1), 1 + _rand((hd,), seed=5, scale=0.1)
    rotation = _rotation(hd, rotary)
    ref_cache = SimpleNamespace(**vars(cache))
    ref_cache.pages = cache.pages.clone()
    q_out = torch.empty((t, heads * hd), dtype=dtype, device=DEV)
    q_ref = torch.empty_like(q_out)
    ops.qk_norm_rope_store(qkv, qw, kw, 1e-6, rotation, step, cache, q_out, heads, kv, hd)
    RefOps().qk_norm_rope_store(qkv, qw, kw, 1e-6, rotation, step, ref_cache, q_ref, heads, kv, hd)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    _close(q_out, q_ref, tol, "rotated queries")
    _close(cache.pages, ref_cache.pages, tol, "pages after the store")
    ops.check_status()


def test_rotation_kinds_without_a_kernel_are_refused_and_can_be_registered(ops):
    from tinyinfer_b200.kernels import KernelError
    from tinyinfer_b200.parts import Rotation
    step, cache, _ = _paged_case(2, 1, 16, 16, [5], [5], torch.float32)
    qkv = _rand((5, 4 * 16), seed=3)
    qw = kw = torch.ones(16, device=DEV)
    q_out = torch.zeros((5, 32), device=DEV)
    odd = Rotation("pairs_of_neighbours", 16, None)
    with pytest.raises(KernelError, match="pairs_of_neighbours"):
        ops.qk_norm_rope_store(qkv, qw, kw, 1e-6, odd, step, cache, q_out, 2, 1, 16)
    with pytest.raises(KernelError, match="pairs_of_neighbours"):
        ops.qkv_rope_store(qkv[:, :8].contiguous(), _rand((64, 8), seed=1), qw, kw, 1e-6, odd, step,
                           cache, q_out, 2, 1, 16)
    assert not q_out.any()
    seen = []
    ops.register_rotation("pairs_of_neighbours", lambda *a: seen.append(a[5].kind))
    try:
        ops.qk_norm_rope_store(qkv, qw, kw, 1e-6, odd, step, cache, q_out, 2, 1, 16)
    finally:
        del ops._rotations["pairs_of_neighbours"]
    assert seen == ["pairs_of_neighbours"]


@pytest.mark.parametrize("geom", [(16, 8, 1024, [2048], [2048]), (5, 1, 136, [300, 77, 500], [150, 70, 333]),
                                  (3, 3, 64, [90], [65]), (16, 8, 1024, [700, 64, 100], [700, 1, 100])])
@pytest.mark.parametrize("writes", [True, False])
def test_qkv_product_with_norm_rotation_and_store_in_its_epilogue(ops, geom, writes):
    """Prompt portions with head size 128: the tcgen05 QKV product whose epilogue norms, rotates
    and stores each head (on one SM or on pairs, by size) against the separate kernels."""
    heads, kv, k, ctx, qls = geom
    hd, ps = 128, 16
    step, cache, _ = _paged_case(heads, kv, hd, ps, ctx, qls, torch.bfloat16)
    cache.writes = writes
    t = step.positions.shape[0]
    h = _rand((t, k), torch.bfloat16, seed=7)
    w = _rand(((heads + 2 * kv) * hd, k), torch.bfloat16, seed=8, scale=2.0 / math.sqrt(k))
    qw, kw = 1 + _rand((hd,), seed=4, scale=0.1), 1 + _rand((hd,), seed=5, scale=0.1)
    rotation = _rotation(hd)
    ref_cache = SimpleNamespace(**vars(cache))
    ref_cache.pages = cache.pages.clone()
    untouched = cache.pages.clone()
    q_out = torch.zeros((t, heads * hd), dtype=torch.bfloat16, device=DEV)
    q_ref = torch.empty_like(q_out)
    before = ops.launches
    ops.qkv_rope_store(h, w, qw, kw, 1e-6, rotation, step, cache, q_out, heads, kv, hd)
    assert ops.launches - before == 2                    # the rotation table of the step, the product
    ops.qkv_rope_store(h, w, qw, kw, 1e-6, rotation, step, cache, q_out, heads, kv, hd)
    assert ops.launches - before == 3                    # the next layer finds the table
    ops.check_status()
    RefOps().qkv_rope_store(h, w, qw, kw, 1e-6, rotation, step, ref_cache, q_ref, heads, kv, hd)
    _close(q_out, q_ref, 8e-3, "rotated queries")
    _close(cache.pages, ref_cache.pages, 8e-3, "pages after the store")
    if not writes:
        assert torch.equal(cache.pages, untouched)
    # unfused on this device: the same numbers up to the order of the norm's sum
    keep = ops.fuse_qkv_epilogue
    ops.fuse_qkv_epilogue = False
    try:
        q_two = torch.empty_like(q_out)
        two = SimpleNamespace(**vars(cache))
        two.pages = untouched.clone()
        ops.qkv_rope_store(h, w, qw, kw, 1e-6, rotation, step, two, q_two, heads, kv, hd)
    finally:
        ops.fuse_qkv_epilogue = keep
    _close(q_out, q_two, 8e-3, "fused against separate kernels")
    assert (q_out != q_two).float().mean().item() < 0.02


@pytest.mark.parametrize("geom", [(16, 8, 128, 16), (8, 1, 128, 64), (4, 4, 64, 16), (6, 2, 64, 32), (32, 8, 128, 16)])
@pytest.mark.parametrize("window", [None, 40])
@pytest.mark.parametrize("writes", [True, False])
def test_decoding_rows_from_the_raw_qkv_product(ops, geom, window, writes):
    """A step of single-token rows: flash-decoding takes the float32 QKV product, norms, rotates
    and stores by itself.  Against the plain statement and against the separate kernels; contexts
    that end at the edges of tiles, pages and splits."""
    heads, kv, hd, ps = geom
    k = 96
    ctx = [1, 2, 31, 32, 33, 64, 65, 129, 500, 1024, 1025, 3000, 17]
    step, cache, _ = _paged_case(heads, kv, hd, ps, ctx, [1] * len(ctx), torch.bfloat16)
    cache.writes = writes
    t = len(ctx)
    h = _rand((t, k), torch.bfloat16, seed=7)
    w = _rand(((heads + 2 * kv) * hd, k), torch.bfloat16, seed=8, scale=2.0 / math.sqrt(k))
    qw, kw = 1 + _rand((hd,), seed=4, scale=0.1), 1 + _rand((hd,), seed=5, scale=0.1)
    rotation = _rotation(hd)
    scale = 1.0 / math.sqrt(hd)
    results = {}
    for name in ("fused", "separate", "plain"):
        c = SimpleNamespace(**vars(cache))
        c.pages = cache.pages.clone()
        out = torch.zeros((t, heads * hd), dtype=torch.bfloat16, device=DEV)
        keep = ops.fuse_decode_rope
        ops.fuse_decode_rope = name == "fused"
        before = ops.launches
        try:
            (RefOps() if name == "plain" else ops).qkv_attention(
                h, w, qw, kw, 1e-6, rotation, step, c, out, heads, kv, hd, window, scale)
        finally:
            ops.fuse_decode_rope = keep
        results[name] = (out, c.pages, ops.launches - before)
    ops.check_status()
    assert results["fused"][2] == 2 and results["separate"][2] == 3          # one launch less
    _close(results["fused"][0], results["plain"][0], 1.5e-2, f"fused decoding {geom} window={window}")
    _close(results["fused"][1], results["plain"][1], 8e-3, "pages after the fused store")
    # the same arithmetic in the same order as the separate kernels: the same bits
    assert torch.equal(results["fused"][1], results["separate"][1]), "stored keys and values differ"
    assert torch.equal(results["fused"][0], results["separate"][0]), "attention output differs"
    if not writes:
        assert torch.equal(results["fused"][1], cache.pages)


@pytest.mark.parametrize("vocab", [151936, 1009, 16384])
def test_argmax_first_maximum_wins(ops, vocab):
    logits = _rand((5, vocab))
    logits[1, 77] = logits[1, vocab - 9] = 50.0
    logits[2, :] = 0.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    ref = torch.empty(5, dtype=torch.int32, device=DEV)
    RefOps().argmax(logits, ref)
    assert out.tolist() == ref.tolist() and out[1] == 77 and out[2] == 0


def test_sample_matches_sorted_statement(ops):
    vocab = 1537
    logits = _rand((64, vocab), scale=3.0)
    temp = torch.full((64,), 0.8, device=DEV)
    temp[:4] = 0.0
    top_k = torch.tensor([0, 5, 50, 1] * 16, dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 0.9, 0.5, 0.95] * 16, device=DEV)
    u = torch.rand(64, generator=torch.Generator().manual_seed(1)).to(DEV)
    out = torch.empty(64, dtype=torch.int32, device=DEV)
    ref = torch.empty(64, dtype=torch.int32, device=DEV)
    ops.sample(logits, temp, top_k, top_p, u, out)
    RefOps().sample(logits, temp, top_k, top_p, u, ref)
    agree = (out == ref).float().mean().item()
    assert agree >= 0.95, f"only {agree:.2f} of the rows agree with the sorted statement"
    # a disagreement can only come from a rounding difference at a boundary: the tokens
    # must then be neighbours among the kept ones
    assert all(int(k) != 1 or int(o) == int(logits[i].argmax())
               for i, (k, o) in enumerate(zip(top_k.tolist(), out.tolist())) if temp[i] > 0)


@pytest.mark.parametrize("vocab", [151936, 5000, 700])
def test_sample_ways_agree_with_the_sorted_statement(ops, vocab):
    """Every way through the sampling kernel against the sorted statement: few survivors (listed
    in shared memory), top-p alone on a peaked and on a flat row, more survivors than the list
    holds (a large k, ties at the k-th place), and no filter at all."""
    g = torch.Generator(device=DEV).manual_seed(vocab)
    cases = []                                   # (logits row, k, p)
    peaked = torch.randn(vocab, generator=g, device=DEV) * 4.0
    flat = torch.randn(vocab, generator=g, device=DEV) * 0.01
    tied = peaked.clone()
    tied[torch.randperm(vocab, generator=torch.Generator().manual_seed(1))[:min(vocab, 3000)].to(DEV)] = 7.5
    for k, p in ((40, 0.9), (1, 1.0), (5, 0.5), (1000, 0.95), (0, 0.9), (0, 0.5), (0, 1.0), (3000, 0.9),
                 (vocab - 1, 0.99)):
        cases.append((peaked, k, p))
    cases += [(flat, 0, 0.9), (flat, 50, 0.3), (tied, 10, 0.9), (tied, 10, 1.0), (tied, 0, 0.999)]
    rows = len(cases) * 3
    logits = torch.stack([c[0] for c in cases] * 3)
    top_k = torch.tensor([c[1] for c in cases] * 3, dtype=torch.int32, device=DEV)
    top_p = torch.tensor([c[2] for c in cases] * 3, device=DEV)
    temp = torch.tensor([0.8] * len(cases) + [1.0] * len(cases) + [0.3] * len(cases), device=DEV)
    u = torch.rand(rows, generator=torch.Generator().manual_seed(3)).to(DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ref = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, temp, top_k, top_p, u, out)
    again = torch.empty_like(out)
    ops.sample(logits, temp, top_k, top_p, u, again)
    assert torch.equal(out, again), "two runs of the sampler differ"
    RefOps().sample(logits, temp, top_k, top_p, u, ref)
    wrong = [(i, int(o), int(r)) for i, (o, r) in enumerate(zip(out.tolist(), ref.tolist())) if o != r]
    # float32 sums against float64 ones: a row may differ where u * total meets a boundary, not often
    assert len(wrong) <= max(1, rows // 20), f"rows that differ from the sorted statement: {wrong}"
    for i, o, r in wrong:                        # ... and then the two tokens are neighbours among the kept ones
        x = logits[i].double()
        kept = torch.exp((x - x.max()) / float(temp[i]))
        lo, hi = min(o, r), max(o, r)
        between = kept[lo + 1:hi]
        assert float(between.sum()) <= 1e-4 * float(kept.sum()), f"row {i}: {o} against {r}"


def test_sample_follows_the_distribution(ops):
    vocab, n = 50, 4000
    base = _rand((1, vocab), scale=1.5)
    logits = base.expand(n, vocab).contiguous()
    u = torch.rand(n, generator=torch.Generator().manual_seed(2)).to(DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, torch.ones(n, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
               torch.ones(n, device=DEV), u, out)
    freq = torch.bincount(out.long(), minlength=vocab).float() / n
    prob = torch.softmax(base[0], dim=-1)
    assert (freq - prob).abs().max().item() < 0.03
