"""Each CUDA kernel alone against its plain PyTorch statement (tests/torch_ops.py), at sizes other
than the engine's tests use: widths that are no power of two, rows that are not 16-byte
multiples, head sizes from 16 to 256, odd head counts and groups (GPU)."""
import math

import pytest
import torch

import plain_llama
from torch_ops import TorchOps

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def _ops():
    from pytriton_llama_b200.ops.cuda import CudaOps
    return CudaOps(torch.device("cuda:0"))


@pytest.fixture
def ops(_ops):
    """The kernels; after every test, no wait inside a kernel may have given up (a kernel whose
    waits run out still ends and may even leave a right result behind)."""
    yield _ops
    _ops.check_status()


REF = TorchOps("cpu")


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(shape, generator=g)).to(dtype)


def close(got, ref, dtype, what="", scale=None):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    s = scale if scale is not None else max(1.0, float(ref.abs().max()))
    tol = 2e-5 * s if dtype == "float32" else 2 ** -7 * s      # bfloat16: one rounding of the result, twice over
    d = (got - ref).abs().max()
    assert d <= tol, f"{what}: max |diff| {d:.3e} > {tol:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vocab, hidden", [(1000, 200), (257, 100), (50, 2048), (33, 7)])
def test_embed(ops, dtype, vocab, hidden):
    table = rnd((vocab, hidden), DT[dtype], 1)
    ids = torch.tensor([0, vocab - 1, 5, 5, vocab // 2], dtype=torch.int32)
    out = ops.embed(ids.cuda(), table.cuda())
    assert torch.equal(out.cpu(), table[ids.long()])
    assert not ops.bad_token_seen()
    ops.embed(torch.tensor([vocab], dtype=torch.int32).cuda(), table.cuda())
    assert ops.bad_token_seen() and not ops.bad_token_seen()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, hidden, eps", [(5, 200, 1e-5), (3, 2048, 1e-6), (2, 5000, 3e-4), (4, 100, 1e-2), (1, 30000, 1e-5),
                                               (300, 2048, 1e-5), (257, 512, 1e-6), (1000, 4096, 1e-5), (260, 3072, 1e-5),
                                               (300, 1536, 1e-6), (256, 3584, 1e-5), (270, 2560, 1e-5)])   # many rows: a warp per row
def test_add_rmsnorm(ops, dtype, rows, hidden, eps):
    x = rnd((rows, hidden), DT[dtype], 2, 3.0)
    res = rnd((rows, hidden), torch.float32, 3, 5.0)
    w = 1 + rnd((hidden,), torch.float32, 4, 0.1)
    y_ref, r_ref = REF.add_rmsnorm(x.clone(), res.clone(), w, eps, dtype=DT[dtype])
    rc = res.clone().cuda()
    y, r = ops.add_rmsnorm(x.cuda(), rc, w.cuda(), eps)
    assert r.data_ptr() == rc.data_ptr()                      # the residual is updated in place
    close(r, r_ref, "float32", "residual")
    close(y, y_ref, dtype, "normed")
    # first layer: no residual yet, the input becomes it
    y0_ref, r0_ref = REF.add_rmsnorm(x.clone(), None, w, eps, dtype=DT[dtype])
    y0, r0 = ops.add_rmsnorm(x.cuda(), None, w.cuda(), eps)
    assert torch.equal(r0.cpu(), x.float())
    close(y0, y0_ref, dtype, "first layer")
    # wanted rows only (the final norm): gathers, writes no residual
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32)
    yg_ref, _ = REF.add_rmsnorm(x.clone(), res.clone(), w, eps, rows=idx, dtype=DT[dtype])
    rc2 = res.clone().cuda()
    yg, none = ops.add_rmsnorm(x.cuda(), rc2, w.cuda(), eps, rows=idx.cuda())
    assert none is None and torch.equal(rc2.cpu(), res)
    close(yg, yg_ref, dtype, "gathered rows")


@pytest.mark.parametrize("M, N, K", [(1, 300, 77), (7, 64, 200), (130, 257, 96), (33, 1000, 513), (300, 48, 2048)])
def test_linear_float32_is_true_32_bit(ops, M, N, K):
    x, w = rnd((M, K), torch.float32, 5), rnd((N, K), torch.float32, 6)
    ref = x.double() @ w.double().T
    out = ops.linear(x.cuda(), w.cuda())
    # a product of K terms in float32: error ~ sqrt(K) * 2^-24 * |x||w|; a 10-bit-mantissa tensor-core mode would be 1e-3
    assert (out.double().cpu() - ref).abs().max() < 3e-6 * math.sqrt(K) * 4


@pytest.mark.parametrize("M, N, K", [(1, 304, 80), (7, 64, 200), (130, 264, 96), (64, 1000, 512)])
def test_linear_bfloat16(ops, M, N, K):
    x, w = rnd((M, K), torch.bfloat16, 5), rnd((N, K), torch.bfloat16, 6)
    ref = x.double() @ w.double().T
    close(ops.linear(x.cuda(), w.cuda()), ref, "bfloat16", "bf16 out")
    out32 = ops.linear(x.cuda(), w.cuda(), out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    assert (out32.double().cpu() - ref).abs().max() < 1e-4 * math.sqrt(K)
    close(ops.linear_simt(x.cuda(), w.cuda()), ref, "bfloat16", "CUDA-core product")
    assert (ops.linear_simt(x.cuda(), w.cuda(), out_dtype=torch.float32).double().cpu() - ref).abs().max() < 1e-4 * math.sqrt(K)


@pytest.mark.parametrize("M, N, K", [
    (128, 128, 64), (130, 264, 96), (200, 1000, 512), (300, 128, 4096), (1100, 768, 200),      # many tokens: 128-token tiles
    (300, 3072, 128), (260, 2304, 64),                                                          # ... of 192 features
    (130, 2048, 8192), (520, 2048, 2048), (1000, 1024, 1024),                                   # ... too few tiles: the add cuts the K range
    (1024, 8192, 128), (600, 4096, 192), (2048, 3072, 256),                                     # ... wide tiles: pairs of blocks (MMAs of 256 rows)
    (1, 304, 80), (8, 3072, 2048), (16, 2048, 2048), (17, 1000, 72), (33, 2048, 8192), (64, 1000, 512),
    (64, 9600, 512), (40, 16384, 2048), (8, 16384, 2048), (24, 12000, 1024),    # few: swapped, K split 2, 4 or 8 ways
    (50, 1002, 1024), (64, 2050, 2048), (36, 4098, 512)])                       # ... feature counts that end inside a group of four
def test_tensor_core_product_and_its_epilogues(ops, M, N, K):
    """The tcgen05/TMEM product against a float64 product: plain bfloat16 and float32 outputs, the
    in-place add into a float32 residual, and SiLU(gate)*up on alternating weight rows."""
    x, w = rnd((M, K), torch.bfloat16, 5), rnd((N, K), torch.bfloat16, 6, 0.5)
    ref = x.double() @ w.double().T
    scale = float(ref.abs().max())
    out = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_BF16)
    assert out is not None and out.dtype == torch.bfloat16
    assert (out.double().cpu() - ref).abs().max() <= 2 ** -8 * scale
    out32 = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_F32)
    assert out32.dtype == torch.float32
    assert (out32.double().cpu() - ref).abs().max() <= 2e-6 * math.sqrt(K) * scale / 10 + 1e-5
    res = rnd((M, N), torch.float32, 7, 3.0)
    acc = res.clone().cuda()
    assert ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_ADD_F32, out=acc) is acc
    assert (acc.double().cpu() - (ref + res.double())).abs().max() <= 2e-6 * math.sqrt(K) * scale / 10 + 1e-5
    act = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_SILU_MUL)
    g, u = ref[:, 0::2], ref[:, 1::2]
    want = g * torch.sigmoid(g) * u
    assert act.shape == (M, N // 2)
    assert (act.double().cpu() - want).abs().max() <= 2 ** -8 * float(want.abs().max())
    assert ops.gemm_tc_status() == 0
    # the same product twice gives the same bits (split partial sums are added in a fixed order)
    assert torch.equal(ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_F32), out32)


@pytest.mark.parametrize("M, N, K, parts", [(130, 264, 200, 3), (300, 512, 1024, 4), (65, 128, 4096, 16)])
def test_tensor_core_product_in_parts_of_the_K_range(ops, M, N, K, parts):
    """With more than 64 tokens the product can be asked for as float32 partial sums over parts of the
    K range (K = 200 in three parts of two 64-blocks leaves the last part empty: it must hold zeros)."""
    x, w = rnd((M, K), torch.bfloat16, 15), rnd((N, K), torch.bfloat16, 16, 0.5)
    ref = x.double() @ w.double().T
    out = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_F32, splits=parts)
    assert out.shape == (parts, M, N)
    per = -(-(-(-K // 64)) // parts) * 64                         # K values per part: whole 64-blocks
    for i in range(parts):
        lo, hi = min(K, i * per), min(K, (i + 1) * per)
        want = x[:, lo:hi].double() @ w[:, lo:hi].double().T
        assert (out[i].double().cpu() - want).abs().max() <= 2e-6 * math.sqrt(K) * float(ref.abs().max()) / 10 + 1e-5, i
    assert 1 <= ops.lib.ptl_gemm_tc_k_parts(300, 2048, 8192) <= 8 and ops.lib.ptl_gemm_tc_k_parts(4096, 8192, 2048) == 1


@pytest.mark.parametrize("M, K, nq, nkv, d, page", [(300, 512, 8, 2, 64, 16), (1100, 256, 6, 2, 128, 16), (130, 192, 5, 1, 64, 8),
                                                    (2048, 128, 32, 8, 64, 16), (700, 320, 24, 8, 128, 32)])
def test_projection_with_rotary_encoding_and_cache_write_in_its_epilogue(ops, M, K, nq, nkv, d, page):
    """The q|k|v projection of many tokens that rotates q and k and writes k and v to the cache
    itself, against the projection followed by ``rope_kv_write``: the same bits in the q columns
    and in every page of the cache (some tokens have no slot and must leave no trace)."""
    N = (nq + 2 * nkv) * d
    x, w = rnd((M, K), torch.bfloat16, 41), rnd((N, K), torch.bfloat16, 42, 0.3)
    g = torch.Generator().manual_seed(43)
    pages = -(-M // page) + 3
    slots = torch.randperm(pages * page, generator=g)[:M].int()
    slots[::7] = -1
    positions = torch.randint(0, 100000, (M,), generator=g).int()
    inv_freq = (10000.0 ** (-torch.arange(0, d, 2).float() / d))
    blank = rnd((pages, 2, nkv, page, d), torch.bfloat16, 44)
    # apart
    qkv = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_BF16)
    cache_a = blank.clone().cuda()
    ops.rope_kv_write(qkv, positions.cuda(), inv_freq.cuda(), d, slots.cuda(), cache_a, nq, nkv, d, page)
    # as one
    cache_b = blank.clone().cuda()
    ops.begin_forward()
    table = ops._rope_table(positions.cuda(), inv_freq.cuda(), d // 2)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    xc, wc, sc = x.cuda(), w.cuda(), slots.cuda()
    rc = ops.lib.ptl_gemm_tc_bf16_qkv_rope(out.data_ptr(), xc.data_ptr(), wc.data_ptr(), M, N, K,
                                           ops._tc_status_word().data_ptr(), table.data_ptr(), sc.data_ptr(),
                                           cache_b.data_ptr(), nq, nkv, d, page, pages * page, ops._stream())
    assert rc == 0, ops.lib.ptl_last_error()
    torch.cuda.synchronize()
    assert torch.equal(out[:, :nq * d], qkv[:, :nq * d])
    assert torch.equal(cache_b, cache_a)
    assert bool((out[:, nq * d:] == 7.0).all())          # the k and v columns of the output are left alone


@pytest.mark.parametrize("M, N, K", [(129, 50, 512), (520, 50, 4096), (128, 130, 1000), (300, 2048, 2048)])
def test_library_product_keeps_float32_sums(ops, M, N, K):
    """Products that go to the library (more than 64 tokens and few tiles) are exact to the rounding
    of the result, element by element, also for widths that are no multiple of 8, where the
    library's default would add the parts of a split K range in bfloat16."""
    x, w = rnd((M, K), torch.bfloat16, 41), rnd((N, K), torch.bfloat16, 42, 0.5)
    ref = x.double() @ w.double().T
    assert ops.library_product(M, N, K, ops.EPI_BF16)
    out = ops.linear(x.cuda(), w.cuda()).double().cpu()
    err = (out - ref).abs()
    assert (err <= 2 ** -8 * ref.abs() + 1e-5 * float(ref.abs().max())).all(), float((err / (ref.abs() + 1e-9)).max())
    assert torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction in (True, False)     # (left as it was found)


def test_tensor_core_product_leaves_other_sizes_to_the_library(ops):
    x, w = rnd((4, 100), torch.bfloat16, 1), rnd((32, 100), torch.bfloat16, 2)    # K no multiple of 8
    assert ops.gemm_tc(x.cuda(), w.cuda()) is None
    assert ops.gemm_tc(x[:, :32].contiguous().cuda(), w[:, :32].contiguous().cuda()) is None   # K below one tile
    close(ops.linear(x.cuda(), w.cuda()), x.double() @ w.double().T, "bfloat16")               # linear() still answers


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, nq, nkv, d, page", [(70, 6, 2, 64, 16), (131, 8, 2, 128, 32), (64, 5, 5, 48, 8), (257, 32, 8, 64, 16)])
def test_rope_kv_write_of_many_tokens(ops, dtype, T, nq, nkv, d, page):
    """From 64 tokens on, whole heads rotated and rows of whole 16-byte packets go through the
    kernel that takes four tokens per block and moves 16-byte packets only (head size 48 in
    bfloat16 has no whole packets per half head and keeps the other kernel): token counts that
    are no multiple of four, a token without a slot, a slot beyond the pool."""
    pages = -(-T // page) + 3
    g = torch.Generator().manual_seed(T)
    qkv = rnd((T, (nq + 2 * nkv) * d), DT[dtype], 18)
    positions = torch.randint(0, 100000, (T,), generator=g).int()
    inv_freq = plain_llama.rope_inv_freq({"head_dim": d, "hidden_size": 1, "num_attention_heads": 1, "rope_theta": 500000.0})
    slots = torch.randperm(pages * page, generator=g)[:T].int()
    slots[3] = -1
    cache_ref = torch.zeros((pages, 2, nkv, page, d), dtype=DT[dtype])
    q_ref = qkv.clone()
    REF.rope_kv_write(q_ref, positions, inv_freq, d, slots, cache_ref, nq, nkv, d, page)
    beyond = slots.clone()
    beyond[5] = pages * page + 2                                         # refused by the kernel: nothing is written for it
    keep = cache_ref.clone()
    s5 = int(slots[5])
    keep[s5 // page, :, :, s5 % page] = 0
    cache = torch.zeros_like(cache_ref).cuda()
    q = qkv.clone().cuda()
    ops.rope_kv_write(q, positions.cuda(), inv_freq.cuda(), d, beyond.cuda(), cache, nq, nkv, d, page)
    close(q[:, : nq * d], q_ref[:, : nq * d], dtype, "rotated q", scale=4.0)
    close(cache, keep, dtype, "cache", scale=4.0)
    assert torch.equal(cache.cpu()[:, 1], keep[:, 1])                      # values are copied, not rotated
    assert torch.equal(q[:, (nq + nkv) * d:].cpu(), qkv[:, (nq + nkv) * d:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, inter", [(3, 264), (2, 8192), (5, 101), (1, 24)])
def test_silu_mul(ops, dtype, rows, inter):
    gu = rnd((rows, 2 * inter), DT[dtype], 7, 3.0)
    close(ops.silu_mul(gu.cuda()), REF.silu_mul(gu), dtype)


def _random_paging(num_reqs, lens, page_size, num_pages, seed):
    """Block tables that scatter each request over random pages of the pool."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    width = max(-(-n // page_size) for n in lens)
    bt = torch.full((num_reqs, width), -1, dtype=torch.int32)
    for r, n in enumerate(lens):
        for b in range(-(-n // page_size)):
            bt[r, b] = perm.pop()
    return bt


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, d, rot, page", [(5, 5, 48, 48, 16), (6, 2, 32, 32, 8), (4, 1, 16, 16, 4), (3, 1, 64, 32, 16),
                                                   (8, 2, 128, 128, 32), (2, 2, 256, 256, 16)])
def test_rope_kv_write(ops, dtype, nq, nkv, d, rot, page):
    T, pages = 9, 12
    qkv = rnd((T, (nq + 2 * nkv) * d), DT[dtype], 8)
    positions = torch.tensor([0, 1, 2, 63, 64, 65, 1000, 4095, 70000], dtype=torch.int32)
    inv_freq = plain_llama.rope_inv_freq({"head_dim": rot, "hidden_size": 1, "num_attention_heads": 1, "rope_theta": 500000.0,
                                          "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                           "high_freq_factor": 4.0, "original_max_position_embeddings": 64}})
    slots = torch.tensor([5, 0, page * 3 + 1, -1, page * pages - 1, 17, 18, page * 2, 7], dtype=torch.int32)
    cache_ref = torch.zeros((pages, 2, nkv, page, d), dtype=DT[dtype])
    q_ref = qkv.clone()
    REF.rope_kv_write(q_ref, positions, inv_freq, rot, slots, cache_ref, nq, nkv, d, page)
    cache = torch.zeros_like(cache_ref).cuda()
    q = qkv.clone().cuda()
    ops.rope_kv_write(q, positions.cuda(), inv_freq.cuda(), rot, slots.cuda(), cache, nq, nkv, d, page)
    close(q[:, : nq * d], q_ref[:, : nq * d], dtype, "rotated q", scale=4.0)
    close(cache, cache_ref, dtype, "cache", scale=4.0)
    assert torch.equal(cache.cpu()[:, 1], cache_ref[:, 1])                 # values are copied, not rotated
    # the rotation angle is float32(position) * inv_freq: exact against a float64 sin/cos of that product
    if dtype == "float32":
        t = 7   # position 4095
        ang = (torch.tensor(4095.0) * inv_freq).double()
        x = qkv[t, :d].double()
        want = x[: rot // 2] * ang.cos() - x[rot // 2: rot] * ang.sin()
        assert (q[t, : rot // 2].double().cpu() - want).abs().max() < 2e-6
    # without a table nothing is rotated, everything is stored
    cache2 = torch.zeros_like(cache)
    q2 = qkv.clone().cuda()
    ops.rope_kv_write(q2, positions.cuda(), None, 0, slots.cuda(), cache2, nq, nkv, d, page)
    assert torch.equal(q2.cpu(), qkv)
    page0, off0 = divmod(5, page)
    assert torch.equal(cache2[page0, 0, :, off0].cpu().reshape(-1), qkv[0, nq * d:(nq + nkv) * d])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, d, page, window, splits", [
    (5, 5, 48, 16, 0, 1), (6, 2, 32, 8, 0, 3), (4, 1, 16, 4, 0, 1), (8, 2, 128, 32, 0, 4), (2, 1, 256, 16, 0, 1),
    (6, 3, 64, 16, 37, 1), (3, 1, 80, 8, 9, 2), (32, 8, 64, 16, 0, 8)])
def test_paged_attention_mixed_batch(ops, dtype, nq, nkv, d, page, window, splits):
    """Three requests in one call: a 70-token prompt portion after 50 cached tokens, a single decoded
    token after 333, and a whole 19-token prompt; pages scattered at random."""
    q_lens, ctx = [70, 1, 19], [120, 334, 19]
    pages = sum(-(-c // page) for c in ctx) + 3
    bt = _random_paging(3, ctx, page, pages, seed=d + nq)
    cache = rnd((pages, 2, nkv, page, d), DT[dtype], 9)
    T = sum(q_lens)
    q = rnd((T, (nq + 2 * nkv) * d), DT[dtype], 10, 2.0)      # a qkv buffer: only its q part is read
    tok_req = torch.repeat_interleave(torch.arange(3), torch.tensor(q_lens)).int()
    positions = torch.cat([torch.arange(c - n, c) for n, c in zip(q_lens, ctx)]).int()
    scale = 1 / math.sqrt(d)
    ref = REF.paged_attention(q, cache, bt, tok_req, positions, nq, nkv, d, page, scale, window=window)
    out = ops.paged_attention(q.cuda(), cache.cuda(), bt.cuda(), tok_req.cuda(), positions.cuda(), nq, nkv, d, page,
                              scale, window=window, splits=splits)
    close(out, ref, dtype, "attention", scale=1.0 if dtype == "float32" else 4.0)


def _hints(q_lens, ctx):
    """The work lists the engine hands to the tensor-core attention kernels, as the operator set plans them."""
    from pytriton_llama_b200.ops.cuda import CudaOps
    return CudaOps(torch.device("cuda:0")).hints_for(q_lens, ctx)


def _work(tensor, items, in_order=False):
    from pytriton_llama_b200.ops.worklists import StepWork
    return StepWork(tensor, items, in_order)


@pytest.mark.parametrize("nq, nkv, d, page, window", [
    (32, 8, 64, 16, 0), (8, 2, 128, 16, 0), (6, 2, 64, 8, 0), (16, 1, 64, 32, 0), (3, 3, 128, 4, 0),
    (32, 8, 64, 16, 200), (4, 2, 128, 16, 33), (5, 1, 64, 1, 0)])
def test_tensor_core_attention_mixed_batch(ops, nq, nkv, d, page, window):
    """The bfloat16 tensor-core kernels (split-key decode, tiled prompt) on one mixed call: portions
    of 150 (after 50 cached), 2 and 64 tokens, a whole 19-token prompt, and single tokens after 0,
    63, 333 and 1500 cached tokens; against the plain statement and against the CUDA-core kernel."""
    q_lens = [150, 1, 2, 1, 64, 1, 19, 1]
    ctx = [200, 334, 66, 1, 128, 64, 19, 1501]
    pages = sum(-(-c // page) for c in ctx) + 3
    bt = _random_paging(len(ctx), ctx, page, pages, seed=d + nq + page)
    cache = rnd((pages, 2, nkv, page, d), torch.bfloat16, 9)
    T = sum(q_lens)
    q = rnd((T, (nq + 2 * nkv) * d), torch.bfloat16, 10, 2.0)
    tok_req = torch.repeat_interleave(torch.arange(len(ctx)), torch.tensor(q_lens)).int()
    positions = torch.cat([torch.arange(c - n, c) for n, c in zip(q_lens, ctx)]).int()
    scale = 1 / math.sqrt(d)
    ref = REF.paged_attention(q, cache, bt, tok_req, positions, nq, nkv, d, page, scale, window=window)
    args = (q.cuda(), cache.cuda(), bt.cuda(), tok_req.cuda(), positions.cuda(), nq, nkv, d, page, scale)
    launches = ops.launches
    out = ops.paged_attention(*args, window=window, hints=_hints(q_lens, ctx))
    assert ops.launches - launches in (2, 3)                    # decode (+ merge) and prompt kernel, not the CUDA-core one
    close(out, ref, "bfloat16", "tensor cores", scale=4.0)
    simt = ops.paged_attention(*args, window=window, splits=2)
    close(out, simt, "bfloat16", "against the CUDA-core kernel", scale=4.0)


@pytest.mark.parametrize("d, nq, nkv", [(64, 8, 2), (128, 6, 2)])
@pytest.mark.parametrize("merge", ["cluster", "ticket", "second_kernel", "many_blocks_ticket", "many_blocks_second_kernel"])
def test_decode_attention_merges_its_splits_in_every_way(ops, d, nq, nkv, merge):
    """The split-key decode kernel combines the splits of a (token, kv head) in one of three ways:
    through the shared memory of a thread-block cluster (2-8 splits, few blocks), by the block that
    takes the last ticket of a counter, or by a second kernel when it is given no counters.  Each
    is pinned here by the split count, the number of blocks and the presence of counters, on
    tokens after 1 to 3,000 cached tokens, and compared with the plain statement."""
    page = 16
    base_ctx = [1, 64, 65, 700, 3000, 129, 1500, 333]
    if merge.startswith("many_blocks"):          # more than 296 blocks: 64-key tiles, no clusters
        ctx, splits = base_ctx * 6, 4
    else:
        ctx, splits = base_ctx[:5], (6 if merge == "cluster" else 12)
    n = len(ctx)
    pages = sum(-(-c // page) for c in ctx) + 3
    bt = _random_paging(n, ctx, page, pages, seed=d + n)
    cache = rnd((pages, 2, nkv, page, d), torch.bfloat16, 41)
    q = rnd((n, nq * d), torch.bfloat16, 42, 2.0)
    tok_req = torch.arange(n).int()
    positions = torch.tensor([c - 1 for c in ctx]).int()
    scale = 1 / math.sqrt(d)
    ref = REF.paged_attention(q, cache, bt, tok_req, positions, nq, nkv, d, page, scale)
    hints = _hints([1] * n, ctx)
    hints.decode_splits = splits
    hints.decode_counters = "second_kernel" not in merge
    launches = ops.launches
    out = ops.paged_attention(q.cuda(), cache.cuda(), bt.cuda(), tok_req.cuda(), positions.cuda(), nq, nkv, d, page, scale,
                              hints=hints)
    assert ops.launches - launches == (2 if "second_kernel" in merge else 1)
    close(out, ref, "bfloat16", merge, scale=4.0)
    if "ticket" in merge:
        assert int(ops._decode_counters.abs().sum()) == 0         # left ready for the next call


def test_decode_attention_padding_rows_named_several_times_leave_the_counters_clean(ops):
    """A captured step of a padded shape names one padding row (request -1) in every item it has too
    many.  Such rows must not take tickets of the split merge: more blocks than splits on one counter
    would leave it non-zero, and a later step with a real token in that row would merge too early or
    never.  20 real tokens and 12 items that all name row 20, 8 kv heads, 2 splits (the counter
    path), called twice; then a call in which row 20 is a real token."""
    nq, nkv, d, page = 32, 8, 64, 16
    real = 20
    ctx = [200 + 37 * i for i in range(real + 1)]
    n_rows = real + 1
    pages = sum(-(-c // page) for c in ctx) + 3
    bt = _random_paging(n_rows, ctx, page, pages, seed=5)
    cache = rnd((pages, 2, nkv, page, d), torch.bfloat16, 51)
    q = rnd((n_rows, nq * d), torch.bfloat16, 52, 2.0)
    positions = torch.tensor([c - 1 for c in ctx]).int()
    scale = 1 / math.sqrt(d)
    full_req = torch.arange(n_rows).int()
    ref = REF.paged_attention(q, cache, bt, full_req, positions, nq, nkv, d, page, scale)
    padded_req = full_req.clone()
    padded_req[real] = -1
    hints = _hints([1] * n_rows, ctx)
    hints.work["decode_items"] = _work(torch.tensor(list(range(real)) + [real] * 12, dtype=torch.int32).cuda(), real + 12)
    hints.decode_splits = 2
    dev = (q.cuda(), cache.cuda(), bt.cuda())
    for _ in range(2):
        out = ops.paged_attention(*dev, padded_req.cuda(), positions.cuda(), nq, nkv, d, page, scale, hints=hints)
        close(out[:real], ref[:real], "bfloat16", "real rows beside padding", scale=4.0)
        assert float(out[real].float().abs().sum()) == 0.0
        assert int(ops._decode_counters.abs().sum()) == 0
    hints = _hints([1] * n_rows, ctx)
    hints.decode_splits = 14                                     # 21 x 8 x 14 blocks: tickets again, row 20 real this time
    out = ops.paged_attention(*dev, full_req.cuda(), positions.cuda(), nq, nkv, d, page, scale, hints=hints)
    close(out, ref, "bfloat16", "row 20 as a real token", scale=4.0)


@pytest.mark.parametrize("d, page, window", [(64, 16, 0), (128, 16, 0), (128, 32, 600), (64, 64, 600), (128, 8, 0)])
def test_tensor_core_attention_over_a_long_prompt(ops, d, page, window):
    """A 1,300-token portion after 700 cached tokens: dozens of key tiles per query tile, so that the
    roles inside the kernel run ahead of one another as far as their barriers let them."""
    nq, nkv = 4, 2
    q_lens, ctx = [1300], [2000]
    pages = -(-ctx[0] // page) + 5
    bt = _random_paging(1, ctx, page, pages, seed=d + page)
    cache = rnd((pages, 2, nkv, page, d), torch.bfloat16, 21)
    q = rnd((q_lens[0], (nq + 2 * nkv) * d), torch.bfloat16, 22, 2.0)
    tok_req = torch.zeros(q_lens[0], dtype=torch.int32)
    positions = torch.arange(ctx[0] - q_lens[0], ctx[0]).int()
    scale = 1 / math.sqrt(d)
    ref = REF.paged_attention(q, cache, bt, tok_req, positions, nq, nkv, d, page, scale, window=window)
    launches = ops.launches
    out = ops.paged_attention(q.cuda(), cache.cuda(), bt.cuda(), tok_req.cuda(), positions.cuda(), nq, nkv, d, page, scale,
                              window=window, hints=_hints(q_lens, ctx))
    assert ops.launches - launches == 1                          # the prompt kernel alone
    close(out, ref, "bfloat16", "long prompt", scale=4.0)


@pytest.mark.parametrize("d, window", [(64, 0), (128, 0), (64, 5000)])
def test_tensor_core_attention_over_more_pages_than_the_kernels_stage(ops, d, window):
    """The attention kernels keep a request's block-table entries in shared memory up to a limit
    (264 entries for a prompt tile pair, 512 for a decode split) and read the table from global
    memory beyond it: 9,000 cached tokens in pages of 16 are 563 entries.  A 130-token portion at the
    end of such a context, a single token after 9,000 and one after 600, scattered pages."""
    nq, nkv, page = 4, 2, 16
    q_lens, ctx = [130, 1, 1], [9000, 9000, 600]
    pages = sum(-(-c // page) for c in ctx) + 7
    bt = _random_paging(3, ctx, page, pages, seed=d)
    cache = rnd((pages, 2, nkv, page, d), torch.bfloat16, 31)
    q = rnd((sum(q_lens), (nq + 2 * nkv) * d), torch.bfloat16, 32, 2.0)
    tok_req = torch.repeat_interleave(torch.arange(3), torch.tensor(q_lens)).int()
    positions = torch.cat([torch.arange(c - n, c) for n, c in zip(q_lens, ctx)]).int()
    scale = 1 / math.sqrt(d)
    ref = REF.paged_attention(q, cache, bt, tok_req, positions, nq, nkv, d, page, scale, window=window)
    out = ops.paged_attention(q.cuda(), cache.cuda(), bt.cuda(), tok_req.cuda(), positions.cuda(), nq, nkv, d, page, scale,
                              window=window, hints=_hints(q_lens, ctx))
    close(out, ref, "bfloat16", "long context", scale=4.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_finds_one_far_key(ops, dtype, window):
    """Random scores would hide a key that is skipped or read from the wrong slot.  Here every query
    has ONE key whose score stands out (the key equals the query direction, scaled up), at places
    where paging can go wrong: the first and last slot of a page, key 0, the query's own position,
    the far edge of the window.  The output must be that key's value."""
    nq, nkv, d, page = 4, 2, 64, 16
    ctx = 700
    pages = -(-ctx // page) + 2
    bt = _random_paging(1, [ctx], page, pages, seed=3)
    g = torch.Generator().manual_seed(4)
    k = 0.05 * torch.randn(ctx, nkv, d, generator=g)
    v = torch.randn(ctx, nkv, d, generator=g)
    positions = torch.tensor([ctx - 1, ctx - 2, 640, 639, 512, 300], dtype=torch.int32)
    lo = [(int(p) - window + 1 if window else 0) for p in positions]
    targets = [lo[0], int(positions[1]), 639 if window else 15, 624 if window else 16, lo[4] + 1, lo[5]]
    T = len(targets)
    q = torch.zeros(T, nq, d)
    for t, key in enumerate(targets):
        for h in range(nq):
            direction = torch.randn(d, generator=g)
            direction /= direction.norm()
            q[t, h] = direction * 40.0
            k[key, h // 2] = k[key, h // 2] + direction * 8.0
    cache = torch.zeros(pages, 2, nkv, page, d)
    for n in range(ctx):
        p, o = int(bt[0, n // page]), n % page
        cache[p, 0, :, o] = k[n]
        cache[p, 1, :, o] = v[n]
    cache = cache.to(DT[dtype])
    out = ops.paged_attention(q.reshape(T, nq * d).to(DT[dtype]).cuda(), cache.cuda(), bt.cuda(),
                              torch.zeros(T, dtype=torch.int32).cuda(), positions.cuda(), nq, nkv, d, page,
                              1 / math.sqrt(d), window=window, splits=1 if window else 4).float().cpu().view(T, nq, d)
    outs = [out]
    if dtype == "bfloat16":
        # the same queries as single decode tokens of six requests that share the pages, through the
        # split-key tensor-core kernel, and as one-row "portions" through the prompt kernel
        from types import SimpleNamespace
        qd = q.reshape(T, nq * d).to(DT[dtype]).cuda()
        bt6 = bt.repeat(T, 1).cuda()
        req6 = torch.arange(T, dtype=torch.int32).cuda()
        dec = SimpleNamespace(work={"decode_items": _work(req6, T), "prefill_tiles": _work(req6[:0], 0)}, max_ctx_len=ctx)
        outs.append(ops.paged_attention(qd, cache.cuda(), bt6, req6, positions.cuda(), nq, nkv, d, page, 1 / math.sqrt(d),
                                        window=window, hints=dec).float().cpu().view(T, nq, d))
        tiles = torch.tensor([[t, t, 1, int(positions[t]), t, t + 128, 0, int(positions[t]) + 128] for t in range(T)],
                             dtype=torch.int32).reshape(-1).cuda()          # pairs whose second tile is empty
        pf = SimpleNamespace(work={"decode_items": _work(req6[:0], 0), "prefill_tiles": _work(tiles, 2 * T)}, max_ctx_len=ctx)
        outs.append(ops.paged_attention(qd, cache.cuda(), bt6, req6, positions.cuda(), nq, nkv, d, page, 1 / math.sqrt(d),
                                        window=window, hints=pf).float().cpu().view(T, nq, d))
    for res in outs:
        for t, key in enumerate(targets):
            for h in range(nq):
                want = cache[int(bt[0, key // page]), 1, h // 2, key % page].float()
                assert (res[t, h] - want).abs().max() < 0.05, (t, h, key)


@pytest.mark.parametrize("vocab", [1000, 128256, 37])
def test_sampling(ops, vocab):
    g = torch.Generator().manual_seed(vocab)
    rows = 12
    logits = 3.0 * torch.randn(rows, vocab, generator=g)
    logits[0, vocab - 1] = logits[0, 5] = logits[0].max() + 1            # equal maxima: the lowest index wins
    temperature = torch.tensor([0.0, 0.0, 0.8, 0.8, 0.8, 1.5, 0.3, 1.0, 1.0, 0.6, 0.6, 2.0])
    top_p = torch.tensor([0.9, 0.9, 0.9, 0.5, 1.0, 0.95, 0.9, 0.01, 0.7, 0.9, 0.9, 0.999])
    u = torch.tensor([0.5, 0.5, 0.0, 0.999999, 0.37, 0.81, 0.5, 0.9, 0.123, 0.25, 0.75, 0.6])
    out = ops.sample(logits.cuda(), temperature.cuda(), top_p.cuda(), u.cuda()).cpu()
    assert out[0] == 5 and out[1] == int(torch.argmax(logits[1]))
    assert out[7] == int(torch.argmax(logits[7]))                        # a tiny top_p keeps the most likely token only
    for i in range(2, rows):
        want = plain_llama.sample_token(logits[i], float(temperature[i]), float(top_p[i]), float(u[i]))
        if out[i] != want:
            # float32 sums may tip a token that sits within rounding of a boundary; anything else is a fault
            p = torch.softmax(logits[i].double() / float(temperature[i]), -1)
            keep = plain_llama.top_p_keep_mask(p, float(top_p[i]))
            assert keep[out[i]], f"row {i}: token {int(out[i])} is outside the nucleus"
            kept = torch.where(keep, p, torch.zeros_like(p))
            cdf = torch.cumsum(kept, 0) / kept.sum()
            lo = float(cdf[out[i]] - kept[out[i]] / kept.sum())
            assert lo - 1e-5 <= float(u[i]) <= float(cdf[out[i]]) + 1e-5, f"row {i}: token {int(out[i])} vs {want}"
    greedy = ops.sample(logits.cuda(), None, None, None).cpu()
    assert torch.equal(greedy[1:].long(), torch.argmax(logits[1:], -1))


@pytest.mark.parametrize("vocab", [1000, 128256, 37])
def test_token_logprobs(ops, vocab):
    g = torch.Generator().manual_seed(vocab + 1)
    logits = 4.0 * torch.randn(6, vocab, generator=g)
    tokens = torch.tensor([0, vocab - 1, 5, 7, vocab // 2, 3], dtype=torch.int32)
    want = torch.log_softmax(logits.double(), -1).gather(1, tokens.long().view(-1, 1)).view(-1)
    got = ops.token_logprobs(logits.cuda(), tokens.cuda()).double().cpu()
    assert (got - want).abs().max() < 1e-4


def test_sampling_is_the_same_every_time_and_leaves_its_histograms_clean(ops):
    """The histograms behind the nucleus filter are built with atomics on integer masses: the same
    call gives the same tokens every time, also after calls with other row counts in between (every
    call hands the shared work buffer back zeroed), and a peaked row keeps a single token."""
    vocab = 128256
    g = torch.Generator().manual_seed(9)
    logits = (2.5 * torch.randn(16, vocab, generator=g)).cuda()
    logits[3, 777] = 60.0                                                # nearly all mass on one token
    temperature = torch.full((16,), 0.7).cuda()
    top_p = torch.linspace(0.05, 1.0, 16).cuda()
    u = torch.rand(16, generator=g).cuda()
    first = ops.sample(logits, temperature, top_p, u).cpu()
    assert first[3] == 777
    ops.sample(logits[:5], temperature[:5], top_p[:5], u[:5])
    ops.sample(logits.repeat(5, 1), temperature.repeat(5), top_p.repeat(5), u.repeat(5))     # more rows than the buffer held
    for _ in range(3):
        assert torch.equal(ops.sample(logits, temperature, top_p, u).cpu(), first)
    words = ops.lib.ptl_sample_work_words()
    assert int(ops._sample_work_buf.view(-1, words)[:, :3 * 1024].abs().sum()) == 0       # the three histograms of every row
    for i in range(16):
        want = plain_llama.sample_token(logits[i].cpu(), 0.7, float(top_p[i]), float(u[i]))
        if first[i] != want:                                             # (a boundary within rounding: still inside the nucleus)
            p = torch.softmax(logits[i].double().cpu() / 0.7, -1)
            assert plain_llama.top_p_keep_mask(p, float(top_p[i]))[first[i]]


def test_sampling_follows_the_distribution(ops):
    """Many draws with different uniform numbers reproduce the filtered probabilities."""
    vocab, n = 50, 4000
    g = torch.Generator().manual_seed(0)
    row = 2.0 * torch.randn(vocab, generator=g)
    logits = row.repeat(n, 1)
    u = (torch.arange(n) + 0.5) / n
    out = ops.sample(logits.cuda(), torch.full((n,), 0.9).cuda(), torch.full((n,), 0.8).cuda(), u.cuda()).cpu().long()
    p = torch.softmax(row.double() / 0.9, -1)
    keep = plain_llama.top_p_keep_mask(p, 0.8)
    want = torch.where(keep, p, torch.zeros_like(p))
    want /= want.sum()
    freq = torch.bincount(out, minlength=vocab).double() / n
    assert (freq[~keep] == 0).all()
    assert (freq - want).abs().max() < 2.0 / n + 1e-9


def test_kernels_refuse_sizes_they_cannot_take(ops):
    from pytriton_llama_b200.ops.cuda import KernelError
    q = torch.zeros(1, 3 * 24, device="cuda")
    cache = torch.zeros(2, 2, 1, 16, 24, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(KernelError, match="multiple of 16"):
        ops.paged_attention(q, cache, z.view(1, 1), z, z, 1, 1, 24, 16, 1.0)
    with pytest.raises(KernelError, match="no multiple"):
        ops.paged_attention(torch.zeros(1, 5 * 32, device="cuda"), torch.zeros(2, 2, 2, 16, 32, device="cuda"), z.view(1, 1), z, z, 3, 2, 32, 16, 1.0)
    with pytest.raises(KernelError):
        ops.embed(torch.zeros(2, dtype=torch.int32), torch.zeros(4, 4))       # CPU tensors: there is no CPU path
    with pytest.raises(KernelError, match="row buffer"):
        ops.add_rmsnorm(torch.zeros(1, 60000, device="cuda"), None, torch.ones(60000, device="cuda"), 1e-5)


@pytest.mark.parametrize("nq, nkv, d, page, window, rotate", [(32, 8, 64, 16, 0, True), (8, 2, 128, 32, 0, True),
                                                              (6, 3, 64, 8, 40, True), (4, 4, 64, 16, 0, False)])
def test_decode_attention_with_rope_and_cache_write_folded_in(ops, nq, nkv, d, page, window, rotate):
    """Single-token steps: the decode kernel that rotates q and k itself and writes k and v to the
    cache gives the same output and the same cache as rope_kv_write followed by paged_attention,
    for contexts that end at the start, in the middle and at the end of a page and of a key tile."""
    from types import SimpleNamespace
    lens = [1, 2, page, page + 1, 127, 128, 129, 300, 1025]
    B = len(lens)
    g = torch.Generator().manual_seed(d + nq)
    pages_per = max(-(-n // page) for n in lens)
    num_pages = B * pages_per + 3
    bt = _random_paging(B, lens, page, num_pages, 5).cuda()
    cache0 = (torch.randn(num_pages, 2, nkv, page, d, generator=g) * 0.5).bfloat16()
    qkv0 = (torch.randn(B, (nq + 2 * nkv) * d, generator=g) * 0.7).bfloat16()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    slots = torch.tensor([int(bt[i, (n - 1) // page]) * page + (n - 1) % page for i, n in enumerate(lens)], dtype=torch.int32).cuda()
    tok_req = torch.arange(B, dtype=torch.int32).cuda()
    inv = (1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))).cuda() if rotate else None
    hints = SimpleNamespace(work={"decode_items": _work(tok_req, B, in_order=True), "prefill_tiles": _work(tok_req[:0], 0)},
                            max_ctx_len=max(lens))
    # the two kernels
    qkv_a, cache_a = qkv0.clone().cuda(), cache0.clone().cuda()
    ops.rope_kv_write(qkv_a, pos, inv, d if rotate else 0, slots, cache_a, nq, nkv, d, page)
    want = ops.paged_attention(qkv_a, cache_a, bt, tok_req, pos, nq, nkv, d, page, d ** -0.5, window=window, hints=hints)
    # one kernel
    qkv_b, cache_b = qkv0.clone().cuda(), cache0.clone().cuda()
    got = ops.rope_attention(qkv_b, pos, inv, d if rotate else 0, slots, cache_b, bt, tok_req, nq, nkv, d, page,
                             d ** -0.5, window=window, hints=hints)
    torch.cuda.synchronize()
    assert torch.equal(cache_a, cache_b), "the cache differs"
    assert torch.equal(qkv_b, qkv0.cuda()), "the fused form leaves the projection as it was"
    assert (got.float() - want.float()).abs().max() <= 2 ** -7 * float(want.float().abs().max())
    # a layer that only reads the cache (write=False) rotates q but writes nothing
    cache_c = cache_a.clone()
    got2 = ops.rope_attention(qkv0.clone().cuda(), pos, inv, d if rotate else 0, slots, cache_c, bt, tok_req, nq, nkv, d,
                              page, d ** -0.5, window=window, hints=hints, write=False)
    assert torch.equal(cache_c, cache_a)
    assert (got2.float() - want.float()).abs().max() <= 2 ** -7 * float(want.float().abs().max())


@pytest.mark.parametrize("M, H, K, N2", [(8, 2048, 2048, 3072), (1, 64, 128, 96), (16, 192, 320, 640), (40, 2048, 8192, 256),
                                         (64, 9600, 512, 128), (200, 256, 512, 1000), (1100, 2048, 256, 512),
                                         (130, 192, 64, 384)])
def test_product_prepares_the_next_norm_and_the_next_product_finishes_it(ops, M, H, K, N2):
    """residual += a @ w1^T with the norm that follows prepared in the epilogue (unnormalised
    bfloat16 input and partial sums of squares), then products that take that input and apply the
    row scale: against residual -> RMS norm -> product in float64."""
    a, w1 = rnd((M, K), torch.bfloat16, 1), rnd((H, K), torch.bfloat16, 2, 0.3)
    res0 = rnd((M, H), torch.float32, 3, 2.0)
    nw = (1.0 + 0.2 * torch.randn(H, generator=torch.Generator().manual_seed(4))).float()
    eps = 1e-5
    res = res0.clone().cuda()
    normed = ops.gemm_tc(a.cuda(), w1.cuda(), ops.EPI_ADD_F32, out=res, emit_norm=(nw.cuda(), eps))
    assert normed is not None and normed.slots > 0
    want_res = res0.double() + a.double() @ w1.double().T
    assert (res.double().cpu() - want_res).abs().max() <= 1e-5 * math.sqrt(K) * float(want_res.abs().max())
    got_sq = normed.sumsq[:, :normed.slots].double().sum(1).cpu()
    assert ((got_sq - (want_res ** 2).sum(1)).abs() / (want_res ** 2).sum(1)).max() < 1e-5
    slack = 1e-5 * math.sqrt(K) * float(want_res.abs().max())          # what float32 accumulation may move the residual by
    assert ((normed.xs.double().cpu() - want_res * nw.double()).abs() <= 2 ** -8 * (want_res * nw.double()).abs() + 2 * slack).all()
    y = want_res * torch.rsqrt((want_res ** 2).mean(1, keepdim=True) + eps) * nw.double()
    assert (normed.materialise().double().cpu() - y).abs().max() <= 2 ** -7 * float(y.abs().max())
    # consumers
    w2 = rnd((N2, H), torch.bfloat16, 5, 0.3)
    ref = y @ w2.double().T
    out = ops.gemm_tc(normed, w2.cuda(), ops.EPI_BF16)
    assert (out.double().cpu() - ref).abs().max() <= 2 ** -6 * float(ref.abs().max())
    out32 = ops.gemm_tc(normed, w2.cuda(), ops.EPI_F32)
    plain = ops.gemm_tc(normed.materialise(), w2.cuda(), ops.EPI_F32)
    assert (out32.double().cpu() - ref).abs().max() <= 2 ** -7 * float(ref.abs().max())
    assert (out32 - plain).abs().max() <= 2 ** -7 * float(ref.abs().max())      # the two ways agree to the activation's rounding
    act = ops.gemm_tc(normed, w2.cuda(), ops.EPI_SILU_MUL)
    g, u = ref[:, 0::2], ref[:, 1::2]
    want = g * torch.sigmoid(g) * u
    assert (act.double().cpu() - want).abs().max() <= 2 ** -5 * float(want.abs().max())
    assert (ops.linear(normed, w2.cuda()).double().cpu() - ref).abs().max() <= 2 ** -6 * float(ref.abs().max())
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M, N, K", [(100, 128, 256), (8, 128, 128), (40, 96, 192)])
def test_a_wait_that_runs_out_sets_the_status_and_the_kernel_returns(_ops, M, N, K):
    """Every wait inside the tcgen05 product is bounded.  The library's self-test entry point launches
    the product as one block whose first stage is never filled and whose waits give up after 300
    polls: the kernel must come back by itself, the status word must say which wait gave up (2: for
    a full stage), the operator set must turn it into an error, and the very next product on the same
    device must be right -- tensor memory was freed, nothing is left in flight."""
    import ctypes
    from pytriton_llama_b200.ops.cuda import KernelError
    ops = _ops
    assert ops.gemm_tc_status() == 0
    lib = ops.lib
    lib.ptl_gemm_tc_wait_selftest.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p]
    lib.ptl_gemm_tc_wait_selftest.restype = ctypes.c_int
    x, w = rnd((M, K), torch.bfloat16, 61).cuda(), rnd((N, K), torch.bfloat16, 62).cuda()
    out = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    status = ops._tc_status_word()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    rc = lib.ptl_gemm_tc_wait_selftest(out.data_ptr(), x.data_ptr(), w.data_ptr(), M, N, K, status.data_ptr(), 300,
                                       torch.cuda.current_stream().cuda_stream)
    end.record()
    assert rc == 0, lib.ptl_last_error().decode()
    torch.cuda.synchronize()                                          # returns: the kernel ended by itself
    assert start.elapsed_time(end) < 500.0                            # ... within its bounded waits (milliseconds)
    assert int(status.item()) == 2
    with pytest.raises(KernelError, match="gave up"):
        ops.check_status()
    assert ops.gemm_tc_status() == 0                                  # reading the word cleared it
    # sizes that would make more than one block are refused: nothing else may be left waiting
    assert lib.ptl_gemm_tc_wait_selftest(out.data_ptr(), x.data_ptr(), w.data_ptr(), 300, N, K, status.data_ptr(), 300, None) == -1
    for _ in range(2):
        got = ops.gemm_tc(x, w, ops.EPI_F32)
        close(got, x.float() @ w.float().T, "float32", "the product after the self-test", scale=float(K) ** 0.5 * 50)
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M, N, K", [(1, 2048, 2048), (8, 3072, 2048), (5, 100, 200), (3, 96, 2176), (4, 101, 64), (8, 40, 1000)])
def test_product_for_a_few_tokens_and_small_weights(_ops, M, N, K):
    """Up to 8 tokens and a weight of a few megabytes go to a product of their own (a block owns 8
    output features for the whole K range; mma.sync, no tensor memory, no cluster): every epilogue
    against float64, and against the tcgen05 product that takes the same call when this one is
    switched off.  Around a norm: its sums of squares come one per 8 features."""
    ops = _ops
    x, w = rnd((M, K), torch.bfloat16, 71), rnd((N, K), torch.bfloat16, 72, 0.5)
    ref = x.double() @ w.double().T
    scale = float(ref.abs().max())
    res0 = rnd((M, N), torch.float32, 73, 3.0)
    nw = (1.0 + 0.2 * torch.randn(N, generator=torch.Generator().manual_seed(74))).float()
    eps = 1e-5
    results = {}
    for small in (True, False):
        ops.small_products = small
        try:
            out = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_BF16)
            out32 = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_F32)
            acc = res0.clone().cuda()
            assert ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_ADD_F32, out=acc) is acc
            acc2 = res0.clone().cuda()
            normed = ops.gemm_tc(x.cuda(), w.cuda(), ops.EPI_ADD_F32, out=acc2, emit_norm=(nw.cuda(), eps))
        finally:
            ops.small_products = True
        assert (out.double().cpu() - ref).abs().max() <= 2 ** -8 * scale
        assert (out32.double().cpu() - ref).abs().max() <= 2e-6 * math.sqrt(K) * scale / 10 + 1e-5
        want_res = ref + res0.double()
        assert (acc.double().cpu() - want_res).abs().max() <= 2e-6 * math.sqrt(K) * scale / 10 + 1e-5
        if normed is not None:                        # (the tcgen05 product prepares a norm only for widths that are multiples of 32)
            assert torch.equal(acc2, acc)
            assert normed.slots == (-(-N // 8) if small else -(-N // 16))
            got_sq = normed.sumsq[:, :normed.slots].double().sum(1).cpu()
            assert ((got_sq - (want_res ** 2).sum(1)).abs() / (want_res ** 2).sum(1)).max() < 1e-5
            y = want_res * torch.rsqrt((want_res ** 2).mean(1, keepdim=True) + eps) * nw.double()
            assert (normed.materialise().double().cpu() - y).abs().max() <= 2 ** -7 * float(y.abs().max())
            if N % 8 == 0 and N >= 64:
                # a product that reads the prepared input finishes the norm: both kinds of product
                w2 = rnd((48, N), torch.bfloat16, 75, 0.3)
                want2 = y @ w2.double().T
                for consumer_small in (True, False):
                    ops.small_products = consumer_small
                    try:
                        got2 = ops.gemm_tc(normed, w2.cuda(), ops.EPI_F32)
                    finally:
                        ops.small_products = True
                    assert (got2.double().cpu() - want2).abs().max() <= 2 ** -7 * float(want2.abs().max())
        elif small:
            raise AssertionError("the product for few tokens prepares the next norm for every width")
        results[small] = (out32.cpu(), acc.cpu())
    # the two products agree to float32 accumulation, and the one for few tokens does not depend on how many there are
    assert (results[True][0] - results[False][0]).abs().max() <= 2e-6 * math.sqrt(K) * scale / 10 + 1e-5
    alone = ops.gemm_tc(x[:1].contiguous().cuda(), w.cuda(), ops.EPI_F32)
    assert torch.equal(alone.cpu()[0], results[True][0][0])
    assert ops.gemm_tc_status() == 0
