"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some users of the library cannot give a kernel scratch memory: their program has handed the
whole device to a pool of its own and forbids cudaMalloc, or it is plain C code without a
tensor library's allocator, or it sits in a loop where an allocation's possible device
synchronisation is not acceptable.  ``ti_attn_decode_noalloc`` keeps the scratch in an 8 MiB
array inside the library instead.  Here it is called twice in a row on different inputs (the
array keeps what the first call left) and compared with the plain PyTorch statement of paged
attention, within the tolerance the kernel tests use, and with ``ti_attn_decode``, which takes
its scratch from the caller and must give the same bits (the same kernel, the same cut into
splits); a request beyond the array's size must be refused.

The file sorts last so that, in a run that stops at the first failure, every other test has
already run.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _library():
    from tinyinfer_b200.kernels import load_library
    lib = load_library("bf16")
    lib.ti_last_error.restype = ctypes.c_char_p
    lib.ti_attn_decode.argtypes = [vp, vp, ci, vp, vp, vp, ci, vp, ci, ci, ci, ci, ci, ci, cf, ci,
                                   vp, vp, vp, vp, vp]
    lib.ti_attn_decode_noalloc.argtypes = [vp, vp, ci, vp, vp, vp, ci, vp, ci, ci, ci, ci, ci, ci,
                                           cf, ci, vp, vp, vp]
    return lib


def _case(seed, heads, kv_heads, hd, page, contexts):
    g = torch.Generator(device=DEV).manual_seed(seed)
    rows = len(contexts)
    blocks = [-(-c // page) for c in contexts]
    num_pages = sum(blocks) + 2
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((rows, max(blocks)), -1, dtype=torch.int32)
    it = iter(order)
    for r, b in enumerate(blocks):
        table[r, :b] = torch.tensor([next(it) for _ in range(b)], dtype=torch.int32)
    pages = torch.randn((num_pages, 2, kv_heads, page, hd), generator=g, device=DEV).to(torch.bfloat16)
    q = torch.randn((rows, heads * hd), generator=g, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV)
    req = torch.arange(rows, dtype=torch.int32, device=DEV)
    return q, positions, req, table.to(DEV), pages


def _run_both(lib, seed, heads, kv_heads, hd, page, contexts, splits, window):
    q, positions, req, table, pages = _case(seed, heads, kv_heads, hd, page, contexts)
    rows = q.shape[0]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(hd)
    common = (q.data_ptr(), None, rows, positions.data_ptr(), req.data_ptr(), table.data_ptr(),
              table.stride(0), pages.data_ptr(), pages.shape[0], page, heads, kv_heads, hd, window,
              scale, splits)
    want = torch.zeros_like(q)
    part_o = torch.empty((rows, heads, splits, hd), dtype=torch.float32, device=DEV)
    part_ml = torch.empty((rows, heads, splits, 2), dtype=torch.float32, device=DEV)
    rc = lib.ti_attn_decode(*common, part_o.data_ptr(), part_ml.data_ptr(), want.data_ptr(),
                            status.data_ptr(), stream)
    assert rc == 0, lib.ti_last_error().decode()
    got = torch.zeros_like(q)
    rc = lib.ti_attn_decode_noalloc(*common, got.data_ptr(), status.data_ptr(), stream)
    assert rc == 0, lib.ti_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # the same kernel over another scratch: a slip in the array's layout would show as other bits
    assert torch.equal(got, want), "the no-alloc entry point and ti_attn_decode differ"
    # and both against the plain statement, so that a fault the two share does not pass
    from types import SimpleNamespace
    from ref_ops import RefOps
    plain = torch.zeros_like(q)
    RefOps().paged_attention(
        q, SimpleNamespace(positions=positions, req_of_tok=req),
        SimpleNamespace(pages=pages, block_table=table, page_size=page), plain, heads, kv_heads, hd,
        window or None, scale)
    err = (got.float() - plain.float()).abs().max().item()
    scale_ref = plain.float().abs().max().item()
    assert err <= 1.5e-2 * scale_ref, f"no-alloc result differs: {err:.3e} against {scale_ref:.3e}"
    return got


def test_no_alloc_entry_point_matches_twice_and_refuses_too_much():
    lib = _library()
    first = _run_both(lib, 1, heads=16, kv_heads=8, hd=128, page=16,
                      contexts=[1, 33, 500, 2049, 64, 777, 31, 1000], splits=9, window=0)
    # a second call of another shape reuses the array and what the first call left in it
    second = _run_both(lib, 2, heads=8, kv_heads=2, hd=64, page=32,
                       contexts=[300, 17, 65], splits=4, window=40)
    # one split: the block writes the result itself (no partial result goes through memory)
    # where ti_attn_decode, without counters, still writes one and merges it in a second launch
    third = _run_both(lib, 4, heads=16, kv_heads=8, hd=128, page=64,
                      contexts=[1, 33, 500, 1025, 64], splits=1, window=0)
    assert torch.isfinite(first.float()).all() and torch.isfinite(second.float()).all()
    assert torch.isfinite(third.float()).all()
    # 64 rows x 64 heads x 64 splits x (128 + 2) floats is far more than 8 MiB
    q, positions, req, table, pages = _case(3, 64, 8, 128, 16, [40] * 64)
    out = torch.zeros_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib.ti_attn_decode_noalloc(
        q.data_ptr(), None, 64, positions.data_ptr(), req.data_ptr(), table.data_ptr(),
        table.stride(0), pages.data_ptr(), pages.shape[0], 16, 64, 8, 128, 0, 0.1, 64,
        out.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"scratch" in lib.ti_last_error()
    torch.cuda.synchronize()
    assert not out.any(), "a refused call must launch nothing"
