"""The allocation-free decode attention entry point (csrc/noalloc.h), called through its exported C
symbol the way an embedding host would, against the regular entry point that takes scratch buffers
from its caller and against the plain float64 statement of attention.  Collected last on purpose:
if it fails, a run that stops at the first failure has already run everything else.  It needs
nothing from other tests and passes alone in a fresh process as well as after them (GPU).

Which path a call takes inside the kernel decides whether the built-in array is touched at all:
2 to 8 splits with few blocks are merged through shared memory of a thread-block cluster and use
no global scratch; more than 8 splits, or more than 296 blocks, write their partial results to the
array and a second kernel merges them.  Most cases below are of the second kind, and the array is
filled with NaNs between calls: a wrong address of the array, a wrong offset of its second half or
a word that a call reads without having written it shows as a NaN or a wrong number."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

_c_int, _c_f, _ptr = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
TOL = 2 ** -7 * 4.0          # the bfloat16 kernels' tolerance in these tests: outputs of size up to ~4


def _library():
    from pytriton_llama_b200.ops import build
    lib = ctypes.CDLL(str(build.library_path()))
    lib.ptl_decode_attention_bf16_noalloc.argtypes = [_ptr] * 7 + [_c_int] * 8 + [_c_f] + [_c_int] * 3 + [_ptr]
    lib.ptl_decode_attention_bf16_noalloc.restype = _c_int
    lib.ptl_decode_attention_bf16.argtypes = [_ptr] * 9 + [_c_int] * 8 + [_c_f] + [_c_int] * 3 + [_ptr, _ptr]
    lib.ptl_decode_attention_bf16.restype = _c_int
    lib.ptl_noalloc_scratch_bytes.restype = ctypes.c_ulonglong
    lib.ptl_noalloc_scratch_address.argtypes = [ctypes.POINTER(_ptr)]
    lib.ptl_noalloc_scratch_address.restype = _c_int
    lib.ptl_last_error.restype = ctypes.c_char_p
    return lib


class _DeviceArray:
    """Lets torch address device memory that it did not allocate (the library's built-in array)."""

    def __init__(self, address, floats):
        self.__cuda_array_interface__ = {"shape": (floats,), "typestr": "<f4", "data": (address, False), "version": 2}


def _scratch(lib):
    """The built-in array as a float32 tensor, through the library's own look-up of its address."""
    address = _ptr()
    assert lib.ptl_noalloc_scratch_address(ctypes.byref(address)) == 0, lib.ptl_last_error().decode()
    assert address.value and address.value % 256 == 0
    holder = _DeviceArray(address.value, lib.ptl_noalloc_scratch_bytes() // 4)
    t = torch.as_tensor(holder, device="cuda")
    assert t.data_ptr() == address.value
    return t


def _case(seed, nq, nkv, d, page, ctx_lens):
    n_items = len(ctx_lens)
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
    host = dict(q=q, cache=cache, bt=bt, tok_req=torch.arange(n_items, dtype=torch.int32),
                positions=torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32))
    case = {k: v.cuda() for k, v in host.items()}
    case.update(pages=pages, host=host, sizes=(nq, nkv, d, page))
    return case


def _plain(case):
    """softmax(q k^T / sqrt(d)) v over each token's keys in float64, from the same bfloat16 inputs."""
    from torch_ops import TorchOps
    nq, nkv, d, page = case["sizes"]
    h = case["host"]
    return TorchOps().paged_attention(h["q"].double(), h["cache"].double(), h["bt"], h["tok_req"], h["positions"], nq, nkv, d,
                                      page, 1 / math.sqrt(d)).float()


def _run(lib, case, splits, noalloc):
    nq, nkv, d, page = case["sizes"]
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


def _check(lib, case, splits, scratch, expect_scratch_used):
    """One call of each entry point on the same inputs, the built-in array full of NaNs before."""
    plain = _plain(case)
    want = _run(lib, case, splits, noalloc=False)
    assert (want - plain).abs().max() <= TOL
    scratch.fill_(float("nan"))
    torch.cuda.synchronize()
    got = _run(lib, case, splits, noalloc=True)
    assert torch.isfinite(got).all(), "the call read a word of the built-in array that it had not written"
    assert (got - want).abs().max() <= TOL
    assert (got - plain).abs().max() <= TOL
    written = int((~torch.isnan(scratch)).sum())          # (an empty split's maximum is -inf, which is a written word too)
    nq, nkv, d, page = case["sizes"]
    if expect_scratch_used:
        # every partial accumulator and (max, sum) pair of the call lies in the array, nothing else was touched
        assert written == case["q"].shape[0] * nq * splits * (d + 2)
    else:
        assert written == 0
    return got


def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row():
    lib = _library()
    assert lib.ptl_noalloc_scratch_bytes() == 8 << 20
    scratch = _scratch(lib)
    # first call: 5 tokens, 8 query heads in groups of 4, head size 64, 12 splits: more than a
    # cluster merges, so the partial results go through the built-in array and the merge kernel
    a = _case(1, 8, 2, 64, 16, [700, 64, 1, 333, 1500])
    got_a = _check(lib, a, 12, scratch, expect_scratch_used=True)
    # second call right after it: other sizes and fewer splits, but 40 tokens x 2 kv heads x 4
    # splits = 320 blocks, which is more than clusters are used for; what the first call left (here:
    # NaNs again) lies beside and beyond the words this call writes
    b = _case(2, 6, 2, 128, 32, [90, 2000, 513, 77] * 10)
    _check(lib, b, 4, scratch, expect_scratch_used=True)
    # the first case once more, this time on top of the second call's leftovers: same bits
    again = _run(lib, a, 12, noalloc=True)
    assert torch.equal(again, got_a)
    # a call that the kernel merges inside a cluster leaves the array alone
    _check(lib, a, 6, scratch, expect_scratch_used=False)
    # one split needs no scratch at all
    one = _run(lib, a, 1, noalloc=True)
    assert (one - _plain(a)).abs().max() <= TOL


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _library()
    c = _case(3, 8, 2, 64, 16, [100, 100, 100, 100])
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
