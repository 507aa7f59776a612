"""The allocation-free decode attention entry point (csrc/noalloc.h), called through its exported C
symbol the way an embedding host would, against the regular entry point that takes scratch buffers
from its caller.  Collected last on purpose: if it fails, a run that stops at the first failure has
already run everything else.  It needs nothing from other tests and passes alone in a fresh
process as well as after them (GPU)."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

_c_int, _c_f, _ptr = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def _library():
    from pytriton_llama_b200.ops import build
    lib = ctypes.CDLL(str(build.library_path()))
    lib.ptl_decode_attention_bf16_noalloc.argtypes = [_ptr] * 7 + [_c_int] * 8 + [_c_f] + [_c_int] * 3 + [_ptr]
    lib.ptl_decode_attention_bf16_noalloc.restype = _c_int
    lib.ptl_decode_attention_bf16.argtypes = [_ptr] * 9 + [_c_int] * 8 + [_c_f] + [_c_int] * 3 + [_ptr, _ptr]
    lib.ptl_decode_attention_bf16.restype = _c_int
    lib.ptl_noalloc_scratch_bytes.restype = ctypes.c_ulonglong
    lib.ptl_last_error.restype = ctypes.c_char_p
    return lib


def _case(seed, n_items, nq, nkv, d, page, ctx_lens):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-c // page) for c in ctx_lens) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    width = max(-(-c // page) for c in ctx_lens)
    bt = torch.full((n_items, width), -1, dtype=torch.int32)
    for r, c in enumerate(ctx_lens):
        for b in range(-(-c // page)):
            bt[r, b] = perm.pop()
    cache = torch.randn((pages, 2, nkv, page, d), generator=g).to(torch.bfloat16)
    q = (2.0 * torch.randn((n_items, nq * d), generator=g)).to(torch.bfloat16)
    return dict(q=q.cuda(), cache=cache.cuda(), bt=bt.cuda(), tok_req=torch.arange(n_items, dtype=torch.int32).cuda(),
                positions=torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32).cuda(), pages=pages)


def _run(lib, case, nq, nkv, d, page, splits, noalloc):
    n = case["q"].shape[0]
    out = torch.full((n, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    common = (case["q"].data_ptr(), case["cache"].data_ptr(), case["bt"].data_ptr(), None, case["tok_req"].data_ptr(),
              case["positions"].data_ptr(), n, nq * d, nq * d, case["bt"].shape[1], nq, nkv, d, page, 1 / math.sqrt(d), 0,
              splits, case["pages"], stream)
    if noalloc:
        rc = lib.ptl_decode_attention_bf16_noalloc(out.data_ptr(), *common)
    else:
        acc = torch.empty((n, nq, splits, d), dtype=torch.float32, device="cuda")
        ml = torch.empty((n, nq, splits, 2), dtype=torch.float32, device="cuda")
        rc = lib.ptl_decode_attention_bf16(out.data_ptr(), acc.data_ptr(), ml.data_ptr(), *common[:-1], None, common[-1])
    assert rc == 0, lib.ptl_last_error().decode()
    torch.cuda.synchronize()
    return out.float().cpu()


def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row():
    lib = _library()
    assert lib.ptl_noalloc_scratch_bytes() == 8 << 20
    # first call: 5 tokens, 8 query heads in groups of 4, head size 64, 6 splits
    a = _case(1, 5, 8, 2, 64, 16, [700, 64, 1, 333, 1500])
    want_a = _run(lib, a, 8, 2, 64, 16, 6, noalloc=False)
    got_a = _run(lib, a, 8, 2, 64, 16, 6, noalloc=True)
    assert torch.isfinite(got_a).all()
    assert (got_a - want_a).abs().max() <= 2 ** -7 * 4.0           # the bfloat16 kernels' tolerance in these tests
    # second call right after it: other sizes, fewer splits, so stale partial results of the first
    # call lie in the shared array beside and beyond the ones this call writes
    b = _case(2, 3, 6, 2, 128, 32, [90, 2000, 513])
    want_b = _run(lib, b, 6, 2, 128, 32, 3, noalloc=False)
    got_b = _run(lib, b, 6, 2, 128, 32, 3, noalloc=True)
    assert torch.isfinite(got_b).all()
    assert (got_b - want_b).abs().max() <= 2 ** -7 * 4.0
    # and the first case once more: the array is reused, results do not drift
    again = _run(lib, a, 8, 2, 64, 16, 6, noalloc=True)
    assert torch.equal(again, got_a)
    # one split needs no scratch at all
    one = _run(lib, a, 8, 2, 64, 16, 1, noalloc=True)
    assert (one - want_a).abs().max() <= 2 ** -7 * 4.0


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _library()
    c = _case(3, 4, 8, 2, 64, 16, [100, 100, 100, 100])
    out = torch.zeros((4, 8 * 64), dtype=torch.bfloat16, device="cuda")
    # 40000 tokens x 32 heads x 32 splits x 66 floats is far beyond 8 MiB: refused before any launch
    rc = lib.ptl_decode_attention_bf16_noalloc(out.data_ptr(), c["q"].data_ptr(), c["cache"].data_ptr(), c["bt"].data_ptr(), None,
                                               c["tok_req"].data_ptr(), c["positions"].data_ptr(), 40000, 512, 512,
                                               c["bt"].shape[1], 32, 8, 64, 16, 0.125, 0, 32, c["pages"], None)
    assert rc == -1
    msg = lib.ptl_last_error().decode()
    assert "exceed the built-in scratch" in msg and "8388608" in msg
    torch.cuda.synchronize()
    assert out.abs().sum() == 0
