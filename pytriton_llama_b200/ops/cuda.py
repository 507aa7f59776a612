"""Tensor-level wrappers of the hand-written sm_100a kernels.

``CudaOps`` is the only implementation of the operator set that the engine's parts call.  It
loads the library built from ``csrc/`` through ctypes and launches on torch's current CUDA stream;
torch itself is used for allocation and, in bfloat16, for the plain library matrix products
(cuBLAS) where lite_llama uses nn.Linear / F.linear too (lite_llama/models/llama.py:22-24,37-40).
There is no CPU path: a tensor that is not on a CUDA device, or a library that cannot be built
or loaded, raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import build
from .worklists import PAD_TOKEN_ROW, StepWork, WorkList

_c_int = ctypes.c_int
_c_ll = ctypes.c_longlong
_c_f = ctypes.c_float
_ptr = ctypes.c_void_p

_SIGNATURES = {
    "ptl_embed_gather": [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr],
    "ptl_add_rmsnorm": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_f, _ptr],
    "ptl_silu_mul": [_ptr, _ptr, _c_int, _c_int, _ptr],
    "ptl_rope_kv_write": [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _ptr],
    "ptl_paged_attention_simt": [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _ptr],
}
_GEMM_SIG = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr]


class NormedActivation:
    """The input of an RMS norm whose normalisation is still to be done by the product that reads it:
    ``xs`` = bfloat16(residual * weight) [tokens, width] and, per token, ``slots`` partial sums of
    residual^2 in ``sumsq``.  The row scale rsqrt(sum / width + eps) is applied by the consumer."""
    __slots__ = ("xs", "sumsq", "slots", "eps", "weight", "ops")

    def __init__(self, xs, sumsq, slots, eps, weight, ops=None):
        self.xs, self.sumsq, self.slots, self.eps, self.weight, self.ops = xs, sumsq, slots, eps, weight, ops

    @property
    def shape(self):
        return self.xs.shape

    @property
    def dtype(self):
        return self.xs.dtype

    def materialise(self) -> torch.Tensor:
        """The normed activation as a plain tensor (for consumers that cannot apply the scale)."""
        return self.ops.finish_norm(self)


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


_LIB = None


def load_library() -> ctypes.CDLL:
    """The kernel library, built on first use.  Raises if it cannot be built or loaded."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = build.library_path()
    lib = ctypes.CDLL(str(path))
    for base, sig in _SIGNATURES.items():
        for suffix in ("_f32", "_bf16"):
            fn = getattr(lib, base + suffix)
            fn.argtypes = sig
            fn.restype = _c_int
    for name in ("ptl_gemm_simt_f32", "ptl_gemm_simt_bf16", "ptl_gemm_simt_bf16_f32out"):
        fn = getattr(lib, name)
        fn.argtypes = _GEMM_SIG
        fn.restype = _c_int
    lib.ptl_decode_attention_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int,
                                              _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _ptr, _ptr]
    lib.ptl_decode_attention_bf16.restype = _c_int
    lib.ptl_decode_attention_rope_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int,
                                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _ptr,
                                                   _ptr, _ptr, _ptr]
    lib.ptl_decode_attention_rope_bf16.restype = _c_int
    lib.ptl_prefill_attention_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                               _c_int, _c_int, _c_f, _c_int, _c_int, _ptr]
    lib.ptl_prefill_attention_bf16.restype = _c_int
    lib.ptl_gemm_tc_bf16.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr]
    lib.ptl_gemm_tc_bf16.restype = _c_int
    lib.ptl_gemm_tc_bf16_norm.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int,
                                          _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _c_int, _c_int, _c_f, _ptr]
    lib.ptl_gemm_tc_bf16_norm.restype = _c_int
    lib.ptl_gemm_small_bf16.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _ptr,
                                        _ptr, _c_int, _c_int, _c_f, _ptr]
    lib.ptl_gemm_small_bf16.restype = _c_int
    lib.ptl_finish_norm_bf16.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_f, _ptr]
    lib.ptl_finish_norm_bf16.restype = _c_int
    lib.ptl_gemm_tc_bf16_qkv_rope.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int,
                                              _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_gemm_tc_bf16_qkv_rope.restype = _c_int
    lib.ptl_rope_table.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _ptr]
    lib.ptl_rope_table.restype = _c_int
    lib.ptl_gemm_tc_k_parts.argtypes = [_c_int, _c_int, _c_int]
    lib.ptl_gemm_tc_k_parts.restype = _c_int
    lib.ptl_add_partials.argtypes = [_ptr, _ptr, _c_int, _c_ll, _c_ll, _ptr]
    lib.ptl_add_partials.restype = _c_int
    lib.ptl_prefill_attention_tc_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                  _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _ptr, _ptr]
    lib.ptl_prefill_attention_tc_bf16.restype = _c_int
    lib.ptl_argmax.argtypes = [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_argmax.restype = _c_int
    lib.ptl_take_tokens.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_int, _ptr]
    lib.ptl_take_tokens.restype = _c_int
    lib.ptl_token_logprob.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_token_logprob.restype = _c_int
    lib.ptl_sample.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _ptr]
    lib.ptl_sample.restype = _c_int
    lib.ptl_sample_work_words.argtypes = []
    lib.ptl_sample_work_words.restype = _c_int
    lib.ptl_last_error.restype = ctypes.c_char_p
    lib.ptl_set_dependent_launch.argtypes = [_c_int]
    lib.ptl_get_dependent_launch.restype = _c_int
    if os.environ.get("PTL_DEPENDENT_LAUNCH", "1") == "0":
        lib.ptl_set_dependent_launch(0)
    _LIB = lib
    return lib


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "_f32"
    if dtype == torch.bfloat16:
        return "_bf16"
    raise KernelError(f"unsupported element type {dtype}")


class CudaOps:
    """The operator set of the engine on one CUDA device."""

    name = "cuda"

    def __init__(self, device: torch.device):
        device = torch.device(device)
        if device.type != "cuda":
            raise KernelError(f"the kernels run on CUDA devices only, got {device}")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; this engine has no CPU path")
        self.device = device
        self.lib = load_library()
        major, minor = torch.cuda.get_device_capability(device)
        if major != 10:
            raise KernelError(f"the kernels are compiled for sm_100a only; device reports sm_{major}{minor}")
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        self._device_index = device.index if device.index is not None else torch.cuda.current_device()
        self._sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        self.launches = 0      # kernels of this library launched so far (library matrix products not counted)

    # ------------------------------------------------------------------ work lists of a step
    QUERY_TILE = 128   # query rows per tile of the prompt attention kernels; a block takes a pair of consecutive tiles
    WORK_LISTS = {
        # token rows that are the only new token of their request: the split-key decode attention's items
        "decode_items": WorkList(width=1, group=1, pad=PAD_TOKEN_ROW),
        # tiles of longer portions: (request row, first token row, rows, first position); in pairs, the
        # second tile continues the first or has no rows; a padding tile has no rows
        "prefill_tiles": WorkList(width=4, group=2, pad=0),
    }

    def plan_step(self, q_lens, starts):
        """The attention kernels' work lists of a step whose request r brings ``q_lens[r]`` tokens
        after ``starts[r]`` cached ones (host integers; the engine packs them and hands them back on
        the device in ``StepContext.work``)."""
        tile = self.QUERY_TILE
        dec, tiles, t0 = [], [], 0
        for r, (n, s) in enumerate(zip(q_lens, starts)):
            if n == 1:
                dec.append(t0)
            else:
                for a in range(0, n, 2 * tile):       # the kernel fetches every key once for both tiles of a pair
                    b = a + tile
                    tiles += [r, t0 + a, min(tile, n - a), s + a,
                              r, t0 + b, max(0, min(tile, n - b)), s + b]
            t0 += n
        return {"decode_items": dec, "prefill_tiles": tiles}

    def hints_for(self, q_lens, ctx_lens):
        """What the attention operators read of a step context, for callers that launch them
        without an engine (kernel tests, micro-benchmarks): the work lists of a step whose request r
        brings ``q_lens[r]`` tokens and holds ``ctx_lens[r]`` afterwards, on the device."""
        from types import SimpleNamespace
        lists = self.plan_step(list(q_lens), [c - n for n, c in zip(q_lens, ctx_lens)])
        T = sum(q_lens)
        work = {}
        for name, values in lists.items():
            info = self.WORK_LISTS[name]
            t = torch.tensor(values if values else [0], dtype=torch.int32, device=self.device)[:len(values)]
            work[name] = StepWork(t, len(values) // info.width, info.width == 1 and values == list(range(T)))
        return SimpleNamespace(work=work, max_ctx_len=max(ctx_lens))

    @staticmethod
    def _work(hints, name):
        work = getattr(hints, "work", None)
        return work.get(name) if work else None

    # ------------------------------------------------------------------ timing by class of kernels (diagnostic)
    KERNEL_CLASSES = {
        "embed": "elementwise", "take_tokens": "elementwise", "silu_mul": "elementwise", "add_rmsnorm": "norm",
        "linear": "product", "linear_add": "product", "gate_up_silu": "product", "gemm_tc": "product",
        "_qkv_rope_product": "product", "rope_kv_write": "rope", "_rope_table": "rope",
        "paged_attention": "attention", "_attention_tensor_cores": "attention",
        "sample": "sampling", "token_logprobs": "sampling",
    }

    def enable_timing(self) -> None:
        """From now on every operator call is bracketed by two CUDA events on the launching stream
        and ``take_timings`` reports the device time by class of kernels.  Operators that only chain
        others (projection, rotation and attention of a mixer) are not timed themselves, their links
        are; of nested timed operators the outermost counts.  Not for captured steps: events recorded
        inside a capture measure nothing."""
        if getattr(self, "_timed", None) is not None:
            return
        self._timed, self._timing_depth = [], 0
        for name, cls in self.KERNEL_CLASSES.items():
            setattr(self, name, self._timed_operator(getattr(self, name), cls))

    def _timed_operator(self, fn, cls):
        def call(*args, **kwargs):
            if self._timing_depth:
                return fn(*args, **kwargs)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._timing_depth += 1
            try:
                start.record()
                out = fn(*args, **kwargs)
                end.record()
            finally:
                self._timing_depth -= 1
            self._timed.append((cls, start, end))
            return out
        return call

    def take_timings(self) -> dict:
        """Milliseconds by class of kernels since the last call (waits for the device); {} when timing is off."""
        if getattr(self, "_timed", None) is None:
            return {}
        torch.cuda.synchronize(self.device)
        out = {}
        for cls, start, end in self._timed:
            out[cls] = out.get(cls, 0.0) + start.elapsed_time(end)
        self._timed = []
        return out

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        """The current stream's handle.  Asked for before every launch (a graph capture changes it), so
        through torch's raw accessor where it has one: building a Stream object each time took 7 us."""
        raw = self._raw_stream
        if raw is not None:
            return raw(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, rc: int, kernels: int = 1) -> None:
        if rc != 0:
            raise KernelError(self.lib.ptl_last_error().decode())
        self.launches += kernels

    def _want(self, t: torch.Tensor, name: str, dtype=None) -> None:
        if t.device != self.device:
            raise KernelError(f"{name} lives on {t.device}, expected {self.device}")
        if not t.is_contiguous():
            raise KernelError(f"{name} must be contiguous")
        if dtype is not None and t.dtype != dtype:
            raise KernelError(f"{name} has element type {t.dtype}, expected {dtype}")

    def empty(self, shape, dtype) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ operators
    def embed(self, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        self._want(ids, "ids", torch.int32)
        self._want(table, "table")
        out = self.empty((ids.shape[0], table.shape[1]), table.dtype)
        fn = getattr(self.lib, "ptl_embed_gather" + _suffix(table.dtype))
        self._check(fn(_p(out), _p(table), _p(ids), ids.shape[0], table.shape[1], table.shape[0],
                       _p(self._status), self._stream()))
        return out

    def take_tokens(self, tokens: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor) -> None:
        """tokens[i] = sampled[src[i]] where src[i] >= 0, in place."""
        for name, t in (("tokens", tokens), ("src", src), ("sampled", sampled)):
            self._want(t, name, torch.int32)
        self._check(self.lib.ptl_take_tokens(_p(tokens), _p(src), _p(sampled), tokens.shape[0], sampled.shape[0],
                                             self._stream()))

    def bad_token_seen(self) -> bool:
        """True if an embedding lookup met an id outside the vocabulary since the last call (syncs)."""
        bad = bool(self._status.item())
        if bad:
            self._status.zero_()
        return bad

    def add_rmsnorm(self, x: Optional[torch.Tensor], residual: Optional[torch.Tensor], weight: torch.Tensor,
                    eps: float, rows: Optional[torch.Tensor] = None,
                    dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """y = rmsnorm(residual + x) * weight, the sum kept as the new float32 residual.

        Without ``rows`` the residual tensor is updated in place (created from ``x`` when None).
        With ``rows`` (int32 indices) only those rows are normed and no residual is written."""
        src = x if x is not None else residual
        hidden = src.shape[-1]
        dtype = dtype or (x.dtype if x is not None else None)
        if dtype is None:
            raise KernelError("add_rmsnorm: give dtype when there is no x")
        self._want(weight, "norm weight", torch.float32)
        if x is not None:
            self._want(x, "x", dtype)
        if residual is not None:
            self._want(residual, "residual", torch.float32)
        if rows is not None:
            self._want(rows, "rows", torch.int32)
            n_out = rows.shape[0]
            res_out = None
        else:
            n_out = src.shape[0]
            res_out = residual if residual is not None else self.empty((n_out, hidden), torch.float32)
        y = self.empty((n_out, hidden), dtype)
        fn = getattr(self.lib, "ptl_add_rmsnorm" + _suffix(dtype))
        self._check(fn(_p(y), _p(res_out), _p(residual), _p(x), _p(weight), _p(rows), n_out, hidden,
                       float(eps), self._stream()))
        return y, res_out

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x[T, K] @ w[N, K]^T.  float32: the library's own FFMA kernel (true 32-bit);
        bfloat16: the tensor-core product of this library (a cuBLAS product for sizes it leaves out).
        ``x`` may be a ``NormedActivation``."""
        if isinstance(x, NormedActivation):
            out = self.gemm_tc(x, w, self.EPI_F32 if out_dtype == torch.float32 else self.EPI_BF16)
            if out is not None:
                return out
            x = x.materialise()
        self._want(x, "x")
        self._want(w, "w", x.dtype)
        out_dtype = out_dtype or x.dtype
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: x is [{M},{K}] but w is {list(w.shape)}")
        if x.dtype == torch.float32:
            out = self.empty((M, N), torch.float32)
            self._check(self.lib.ptl_gemm_simt_f32(_p(out), _p(x), _p(w), M, N, K, K, K, N, 0, self._stream()))
            return out
        if not (out_dtype == torch.bfloat16 and self.library_product(M, N, K, self.EPI_BF16)):
            out = self.gemm_tc(x, w, self.EPI_F32 if out_dtype == torch.float32 else self.EPI_BF16)
            if out is not None:
                return out
        # sizes the tensor-core kernel does not take (K no multiple of 8, or below 64) or leaves to the library
        return self._library_mm(x, w, out_dtype)

    @staticmethod
    def _library_mm(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """x @ w^T by the library with float32 sums throughout.  torch lets cuBLAS add the parts of a
        split K range in bfloat16 by default; it does so for widths that are no multiple of 8, and
        an element that is small beside the partial sums it is made of then comes out wrong by as
        much as its own size (a [129, 512] x [50, 512]^T product: 0.4 % of the largest element
        everywhere, 43 % of a small one).  The engine's own shapes are not touched by the setting
        (same kernels, same time); it is put back after the call."""
        matmul = torch.backends.cuda.matmul
        before = matmul.allow_bf16_reduced_precision_reduction
        matmul.allow_bf16_reduced_precision_reduction = False
        try:
            if out_dtype == torch.float32:
                return torch.mm(x, w.t(), out_dtype=torch.float32)
            return torch.mm(x, w.t())
        finally:
            matmul.allow_bf16_reduced_precision_reduction = before

    library_products = os.environ.get("PTL_LIBRARY_PRODUCTS", "1") != "0"

    def library_product(self, M: int, N: int, K: int, epi: int) -> bool:
        """True where the plain library product (cuBLAS through torch.mm, which is what lite_llama's
        nn.Linear layers are: lite_llama/models/llama.py:22-24,37-40) is the one to take.  Measured
        on a B200 with cold caches (``python -m pytriton_llama_b200.ops.microbench product_shapes``):
        a product of more than 64 tokens whose 128 x 256 tiles do not fill the SMs twice is faster
        there, by 2 to 10 us, than this library's tcgen05 kernel even after the library's result has
        been rotated by ``rope_kv_write`` or read once more by the norm that adds it to the residual
        (q|k|v, output and down projection at 128 to 2,048 tokens: few tiles, each walking a long K
        range alone).  The products with the SiLU*up epilogue, of few tokens, with float32 results
        and of many tiles stay with the tcgen05 kernel.  ``PTL_LIBRARY_PRODUCTS=0`` keeps everything there."""
        if not self.library_products or M <= 64 or epi not in (self.EPI_BF16, self.EPI_ADD_F32):
            return False
        return -(-M // 128) * -(-N // 256) <= 2 * self._sm_count

    fuses_next_norm = os.environ.get("PTL_FUSED_NORM", "1") != "0"
    small_products = os.environ.get("PTL_SMALL_PRODUCTS", "1") != "0"      # steps of up to 8 tokens: gemm_small for weights of a few MB
    # Steps of up to this many tokens fold the norms into the products around them.  With more
    # tokens a step is no longer bound by the number of kernels, and the add epilogue of the
    # products with a short K range has no time to spare for the extra stores.
    FUSED_NORM_MAX_TOKENS = int(os.environ.get("PTL_FUSED_NORM_MAX", "64"))

    def linear_add(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, next_norm=None):
        """residual += x @ w^T in the product's epilogue (float32 residual, in place) and None; where
        that is not possible the plain product, for the caller to add.  With ``next_norm`` = (weight,
        eps) of the RMS norm that reads the residual next, the epilogue prepares that norm's input
        as well and a ``NormedActivation`` is returned instead of None (where the sizes allow it)."""
        if x.dtype == torch.bfloat16 and residual is not None and not self.library_product(x.shape[0], w.shape[0], x.shape[1], self.EPI_ADD_F32):
            if next_norm is not None and self.fuses_next_norm and x.shape[0] <= self.FUSED_NORM_MAX_TOKENS:
                normed = self.gemm_tc(x, w, self.EPI_ADD_F32, out=residual, emit_norm=next_norm)
                if normed is not None:
                    return normed
            if self.gemm_tc(x, w, self.EPI_ADD_F32, out=residual) is not None:
                return None
        return self.linear(x, w)

    def fused_ffn_layout(self, dtype: torch.dtype, hidden: int, inter: int) -> bool:
        """True if gate and up rows should alternate (gate_0, up_0, gate_1, ...) so that the
        gate/up product can apply SiLU(gate)*up in its epilogue."""
        return dtype == torch.bfloat16 and hidden % 8 == 0 and hidden >= 64

    def gate_up_silu(self, x, w_alternating: torch.Tensor) -> torch.Tensor:
        out = self.gemm_tc(x, w_alternating, self.EPI_SILU_MUL)
        if out is None and isinstance(x, NormedActivation):
            out = self.gemm_tc(x.materialise(), w_alternating, self.EPI_SILU_MUL)
        if out is None:
            raise KernelError("gate_up_silu: sizes not taken; load the weights in the plain layout instead")
        return out

    # epilogues of the tensor-core product
    EPI_BF16, EPI_F32, EPI_ADD_F32, EPI_SILU_MUL = 0, 1, 2, 3

    def _tc_status_word(self):
        if getattr(self, "_tc_status", None) is None:
            self._tc_status = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._tc_status

    def gemm_tc(self, x, w: torch.Tensor, epi: int = 0, out: Optional[torch.Tensor] = None,
                splits: int = 0, emit_norm=None):
        """x[M,K] @ w[N,K]^T in bfloat16 on the tcgen05 tensor cores with a fused epilogue.
        ``epi``: EPI_BF16 -> [M,N] bfloat16; EPI_F32 -> [M,N] float32; EPI_ADD_F32 adds into ``out``
        (float32 [M,N], in place); EPI_SILU_MUL -> [M,N/2] bfloat16 for weights whose rows alternate
        gate_j, up_j.  ``x`` may be a ``NormedActivation``: its row scale is applied before the
        epilogue.  ``emit_norm`` = (weight, eps) with EPI_ADD_F32 returns the ``NormedActivation`` of the
        norm that follows.  Returns None when the kernel does not take the sizes."""
        scale = None
        if isinstance(x, NormedActivation):
            scale, x = x, x.xs
        self._want(x, "x", torch.bfloat16)
        self._want(w, "w", torch.bfloat16)
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"gemm_tc: x is [{M},{K}] but w is {list(w.shape)}")
        if K % 8 or K < 64:
            return None
        if epi == self.EPI_ADD_F32:
            if out is None:
                raise KernelError("gemm_tc: the add epilogue needs the float32 tensor to add into")
            self._want(out, "out", torch.float32)
            ld = N
        elif epi == self.EPI_SILU_MUL:
            out = self.empty((M, N // 2), torch.bfloat16)
            ld = N // 2
        elif epi == self.EPI_F32 and M > 64 and splits > 1:
            out = self.empty((splits, M, N), torch.float32)      # partial sums of the parts of the K range
            ld = N
        else:
            out = self.empty((M, N), torch.float32 if epi == self.EPI_F32 else torch.bfloat16)
            ld = N
        if epi == self.EPI_ADD_F32 and scale is None and emit_norm is None and M > 64 and N % 4 == 0 and splits == 0:
            # a few hundred tokens, or a narrow product: too few tiles for the SMs, so the K range is
            # cut into parts as well; their float32 partial sums are added into ``out`` in a fixed order
            parts = self.lib.ptl_gemm_tc_k_parts(M, N, K)
            if parts > 1:
                partial = self.empty((parts, M, N), torch.float32)
                self._check(self.lib.ptl_gemm_tc_bf16(_p(partial), _p(x), _p(w), M, N, K, N, self.EPI_F32,
                                                      _p(self._tc_status_word()), parts, self._stream()))
                self._check(self.lib.ptl_add_partials(_p(out), _p(partial), parts, M * N, M * N, self._stream()))
                return out
        normed = slots = None
        if emit_norm is not None:
            weight, eps = emit_norm
            self._want(weight, "norm weight", torch.float32)
            width = (N + 7) // 8           # a slot per 8 features at most (the product for a few tokens), per 16 otherwise
            normed = NormedActivation(self.empty((M, N), torch.bfloat16), self.empty((M, width), torch.float32), 0,
                                      float(eps), weight, ops=self)
            slots = ctypes.c_int(0)
        if M <= 8 and epi != self.EPI_SILU_MUL and splits == 0 and self.small_products:
            # a few tokens and a weight of a few megabytes (q|k|v and output projection of a decode step): the
            # product without tensor memory and clusters, whose latency is a third; -2 where it does not fit
            rc = self.lib.ptl_gemm_small_bf16(
                _p(out), _p(x), _p(w), M, N, K, ld, epi,
                _p(normed.xs) if normed else None, _p(normed.weight) if normed else None,
                _p(normed.sumsq) if normed else None, normed.sumsq.shape[1] if normed else 0,
                ctypes.byref(slots) if normed else None,
                _p(scale.sumsq) if scale else None, scale.slots if scale else 0, scale.sumsq.shape[1] if scale else 0,
                scale.eps if scale else 0.0, self._stream())
            if rc != -2:
                self._check(rc)
                if normed is not None:
                    normed.slots = slots.value
                    return normed
                return out
        if scale is None and emit_norm is None:
            rc = self.lib.ptl_gemm_tc_bf16(_p(out), _p(x), _p(w), M, N, K, ld, epi, _p(self._tc_status_word()), splits,
                                           self._stream())
            if rc == -2:
                return None
            self._check(rc)
            return out
        rc = self.lib.ptl_gemm_tc_bf16_norm(
            _p(out), _p(x), _p(w), M, N, K, ld, epi, _p(self._tc_status_word()), splits,
            _p(normed.xs) if normed else None, _p(normed.weight) if normed else None,
            _p(normed.sumsq) if normed else None, normed.sumsq.shape[1] if normed else 0,
            ctypes.byref(slots) if normed else None,
            _p(scale.sumsq) if scale else None, scale.slots if scale else 0, scale.sumsq.shape[1] if scale else 0,
            scale.eps if scale else 0.0, self._stream())
        if rc == -2:
            return None
        self._check(rc)
        if normed is not None:
            normed.slots = slots.value
            return normed
        return out

    def check_status(self) -> None:
        """Raises if a kernel flagged a problem since the last call: a token outside the vocabulary
        reached the embedding, or a wait inside a tensor-core kernel gave up (synchronises)."""
        if self.bad_token_seen():
            raise KernelError("a token id outside the vocabulary reached the embedding kernel")
        code = self.gemm_tc_status()
        if code:
            raise KernelError(f"a wait inside a tcgen05 kernel gave up (code {code}); results since the last check are invalid")

    def gemm_tc_status(self) -> int:
        """0, or the code of the wait that gave up inside a tensor-core product since the last call (syncs)."""
        if getattr(self, "_tc_status", None) is None:
            return 0
        code = int(self._tc_status.item())
        if code:
            self._tc_status.zero_()
        return code

    def linear_simt(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The CUDA-core product for any element type (checks of the tensor-core kernels)."""
        self._want(x, "x")
        self._want(w, "w", x.dtype)
        out_dtype = out_dtype or x.dtype
        M, K = x.shape
        N = w.shape[0]
        out = self.empty((M, N), out_dtype)
        if x.dtype == torch.float32:
            fn = self.lib.ptl_gemm_simt_f32
        elif out_dtype == torch.float32:
            fn = self.lib.ptl_gemm_simt_bf16_f32out
        else:
            fn = self.lib.ptl_gemm_simt_bf16
        self._check(fn(_p(out), _p(x), _p(w), M, N, K, K, K, N, 0, self._stream()))
        return out

    def finish_norm(self, normed: NormedActivation) -> torch.Tensor:
        """The RMS norm that a product's epilogue prepared, finished as a plain bfloat16 tensor."""
        tokens, width = normed.xs.shape
        out = self.empty((tokens, width), torch.bfloat16)
        self._check(self.lib.ptl_finish_norm_bf16(_p(out), _p(normed.xs), _p(normed.sumsq), tokens, normed.slots, normed.sumsq.shape[1],
                                                  width, float(normed.eps), self._stream()))
        return out

    def silu_mul(self, gu: torch.Tensor) -> torch.Tensor:
        self._want(gu, "gate_up")
        tokens, two_i = gu.shape
        out = self.empty((tokens, two_i // 2), gu.dtype)
        fn = getattr(self.lib, "ptl_silu_mul" + _suffix(gu.dtype))
        self._check(fn(_p(out), _p(gu), tokens, two_i // 2, self._stream()))
        return out

    def rope_kv_write(self, qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                      rot: int, slots: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                      nq: int, nkv: int, d: int, page_size: int) -> None:
        self._want(qkv, "qkv")
        self._want(positions, "positions", torch.int32)
        if inv_freq is not None:
            self._want(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() < rot // 2:
                raise KernelError("inv_freq shorter than half the rotary width")
        if cache is not None:
            self._want(cache, "cache", qkv.dtype)
            self._want(slots, "slots", torch.int32)
            num_slots = cache.shape[0] * page_size
        else:
            num_slots = 0
        if qkv.shape[1] != (nq + 2 * nkv) * d:
            raise KernelError(f"qkv rows have {qkv.shape[1]} elements, expected {(nq + 2 * nkv) * d}")
        fn = getattr(self.lib, "ptl_rope_kv_write" + _suffix(qkv.dtype))
        self._check(fn(_p(qkv), _p(positions), _p(inv_freq), _p(slots), _p(cache), qkv.shape[0], nq, nkv, d,
                       rot, page_size, num_slots, self._stream()))

    def paged_attention(self, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                        tok_req: torch.Tensor, positions: torch.Tensor, nq: int, nkv: int, d: int,
                        page_size: int, scale: float, window: int = 0, splits: int = 1,
                        hints=None) -> torch.Tensor:
        """q is [T, >= nq*d] (the q part of a qkv buffer is fine); returns [T, nq*d]."""
        self._want(q, "q")
        self._want(cache, "cache", q.dtype)
        self._want(block_table, "block_table", torch.int32)
        self._want(tok_req, "tok_req", torch.int32)
        self._want(positions, "positions", torch.int32)
        tokens = q.shape[0]
        out = self.empty((tokens, nq * d), q.dtype)
        if (q.dtype == torch.bfloat16 and d in (64, 128) and nq // nkv <= 16 and self._work(hints, "decode_items") is not None
                and self._work(hints, "prefill_tiles") is not None):
            self._attention_tensor_cores(out, q, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                         window, hints)
            return out
        part_acc = part_ml = None
        if splits > 1:
            part_acc = self.empty((tokens, nq, splits, d), torch.float32)
            part_ml = self.empty((tokens, nq, splits, 2), torch.float32)
        fn = getattr(self.lib, "ptl_paged_attention_simt" + _suffix(q.dtype))
        self._check(fn(_p(out), _p(q), _p(cache), _p(block_table), _p(tok_req), _p(positions), _p(part_acc),
                       _p(part_ml), tokens, q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size,
                       float(scale), int(window), int(splits), cache.shape[0], self._stream()),
                    kernels=2 if splits > 1 else 1)
        return out

    def rope_attention(self, qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int,
                       slots: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                       tok_req: torch.Tensor, nq: int, nkv: int, d: int, page_size: int, scale: float,
                       window: int = 0, splits: int = 1, hints=None, write: bool = True) -> torch.Tensor:
        """``rope_kv_write`` followed by ``paged_attention``.  A bfloat16 step of single tokens only
        runs both in the decode attention kernel (rotation over the whole head, head sizes 64 and
        128); everything else takes the two kernels."""
        dec, tiles = self._work(hints, "decode_items"), self._work(hints, "prefill_tiles")
        fused = (os.environ.get("PTL_FUSED_ROPE", "1") != "0" and qkv.dtype == torch.bfloat16 and d in (64, 128)
                 and nq // nkv <= 16 and dec is not None and tiles is not None
                 and dec.items == qkv.shape[0] and not tiles.items
                 and (inv_freq is None or rot == d) and qkv.shape[1] >= (nq + 2 * nkv) * d)
        if not fused:
            self.rope_kv_write(qkv, positions, inv_freq, rot, slots if write else None, cache if write else None,
                               nq, nkv, d, page_size)
            return self.paged_attention(qkv, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                        window=window, splits=splits, hints=hints)
        for name, t in (("qkv", qkv), ("cache", cache)):
            self._want(t, name, torch.bfloat16)
        for name, t in (("block_table", block_table), ("tok_req", tok_req), ("positions", positions)):
            self._want(t, name, torch.int32)
        if inv_freq is not None:
            self._want(inv_freq, "inv_freq", torch.float32)
        if write:
            self._want(slots, "slots", torch.int32)
        out = self.empty((qkv.shape[0], nq * d), qkv.dtype)
        self._attention_tensor_cores(out, qkv, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                     window, hints, rope=(inv_freq, slots if write else None))
        return out

    def begin_forward(self) -> None:
        """Called by the model at the start of every forward pass: what was worked out for the last
        step's positions (the table of rotary angles) is forgotten."""
        self._rope_memo = None

    def _rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor, half: int) -> torch.Tensor:
        """(cos, sin) [tokens, half] of this step's angles, worked out once per forward pass and used by every layer."""
        key = (positions.data_ptr(), positions._version, inv_freq.data_ptr(), positions.shape[0], half)
        memo = getattr(self, "_rope_memo", None)
        if memo is not None and memo[0] == key:
            return memo[1]
        table = self.empty((positions.shape[0], half, 2), torch.float32)
        self._check(self.lib.ptl_rope_table(_p(table), _p(positions), _p(inv_freq), positions.shape[0], half, self._stream()))
        self._rope_memo = (key, table)
        return table

    def projected_rope_attention(self, x, w_qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                                 rot: int, slots: Optional[torch.Tensor], cache: torch.Tensor, block_table: torch.Tensor,
                                 tok_req: torch.Tensor, nq: int, nkv: int, d: int, page_size: int, scale: float,
                                 window: int = 0, splits: int = 1, hints=None, write: bool = True) -> torch.Tensor:
        """The q|k|v projection, ``rope_kv_write`` and ``paged_attention`` of a mixer.  A bfloat16
        step of more than 64 tokens rotates q and k and writes k and v to the cache in the
        projection's epilogue (head sizes 64 and 128, the whole head rotated); everything else
        projects first and goes on with ``rope_attention``."""
        fused = (os.environ.get("PTL_FUSED_QKV_ROPE", "1") != "0" and isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16
                 and x.shape[0] > 64 and write and slots is not None and inv_freq is not None and rot == d and d in (64, 128)
                 and w_qkv.shape[0] == (nq + 2 * nkv) * d and cache.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                 and x.shape[1] >= 64 and not self.library_product(x.shape[0], w_qkv.shape[0], x.shape[1], self.EPI_BF16))
        if fused:
            self._want(x, "x", torch.bfloat16)
            self._want(w_qkv, "w_qkv", torch.bfloat16)
            self._want(cache, "cache", torch.bfloat16)
            self._want(slots, "slots", torch.int32)
            self._want(positions, "positions", torch.int32)
            self._want(inv_freq, "inv_freq", torch.float32)
            M, K = x.shape
            N = w_qkv.shape[0]
            table = self._rope_table(positions, inv_freq, d // 2)
            qkv = self.empty((M, N), torch.bfloat16)          # only the q columns are written (and read)
            if self._qkv_rope_product(qkv, x, w_qkv, table, slots, cache, nq, nkv, d, page_size):
                return self.paged_attention(qkv, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                            window=window, splits=splits, hints=hints)
        qkv = self.linear(x, w_qkv)
        return self.rope_attention(qkv, positions, inv_freq, rot, slots, cache, block_table, tok_req, nq, nkv, d, page_size,
                                   scale, window=window, splits=splits, hints=hints, write=write)

    def _qkv_rope_product(self, qkv, x, w_qkv, table, slots, cache, nq, nkv, d, page_size) -> bool:
        """The q|k|v projection with rotary encoding and the cache write in its epilogue; False where the kernel does not take the sizes."""
        M, K = x.shape
        rc = self.lib.ptl_gemm_tc_bf16_qkv_rope(_p(qkv), _p(x), _p(w_qkv), M, w_qkv.shape[0], K, _p(self._tc_status_word()), _p(table),
                                                _p(slots), _p(cache), nq, nkv, d, page_size,
                                                cache.shape[0] * page_size, self._stream())
        if rc == -2:
            return False
        self._check(rc)
        return True

    DECODE_BLOCKS = int(os.environ.get("PTL_DECODE_BLOCKS", "592"))    # blocks the decode attention aims for: the four per SM that fit at once
    DECODE_KEYS_PER_WIDE_BLOCK = int(os.environ.get("PTL_DECODE_KEYS_PER_WIDE_BLOCK", "1024"))   # keys a block of the two-per-SM form walks at most

    _DECODE_COUNTERS = 1 << 16

    def _attention_tensor_cores(self, out, q, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                                window, hints, rope=None) -> None:
        """bfloat16 attention on the tensor cores: single tokens through the split-key decode kernel,
        longer portions through the tiled prompt kernel; both write their rows of ``out``."""
        stream = self._stream()
        num_pages = cache.shape[0]
        dec, tiles = hints.work["decode_items"], hints.work["prefill_tiles"]
        n_decode, n_tiles = dec.items, tiles.items
        if n_decode:
            longest = min(hints.max_ctx_len, window) if window else hints.max_ctx_len
            pairs = n_decode * nkv
            # small batches: 128-key tiles at two blocks per SM (296 in flight); large ones: 64-key tiles, four per SM
            target = 296 if pairs <= 148 else self.DECODE_BLOCKS
            splits = max(1, min(target // pairs, -(-longest // 128)))
            if target == 296 and splits > 8:
                splits = 8      # what a cluster merges through shared memory; more splits would go through global memory (slower)
            if target == 296 and longest > self.DECODE_KEYS_PER_WIDE_BLOCK * splits:
                # Long contexts at small batches: a block of the cluster form has two 128-key tiles in
                # flight, and with more than eight to walk that no longer covers the memory's latency
                # (one request of 131,072 tokens: 196 us against 55 us).  Four blocks per SM with three
                # 64-key tiles each in flight do, merged by the last block of a token's splits.
                splits = max(splits, min(self.DECODE_BLOCKS // pairs, -(-longest // 128)))
            # The split count of this kernel is decided here, from the number of blocks the machine
            # holds (``attn_splits`` of the step context is the CUDA-core kernel's).  A caller may fix
            # it (``decode_splits``) and leave the counters out (``decode_counters`` False) to pin one
            # of the three ways of merging.
            splits = int(getattr(hints, "decode_splits", 0) or splits)
            part_acc = part_ml = counters = None
            if splits > 1:
                splits = min(splits, 512)
                part_acc = self.empty((q.shape[0], nq, splits, d), torch.float32)
                part_ml = self.empty((q.shape[0], nq, splits, 2), torch.float32)
                if q.shape[0] * nkv <= self._DECODE_COUNTERS and getattr(hints, "decode_counters", True):
                    if getattr(self, "_decode_counters", None) is None:
                        self._decode_counters = torch.zeros(self._DECODE_COUNTERS, dtype=torch.int32, device=self.device)
                    counters = self._decode_counters        # the last block of a token's splits merges them in the kernel
            items = None if dec.in_order else _p(dec.tensor)
            if rope is not None:
                rc = self.lib.ptl_decode_attention_rope_bf16(
                    _p(out), _p(part_acc), _p(part_ml), _p(q), _p(cache), _p(block_table), items, _p(tok_req),
                    _p(positions), n_decode, q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size,
                    float(scale), int(window), splits, num_pages, _p(counters), _p(rope[0]), _p(rope[1]), stream)
            else:
                rc = self.lib.ptl_decode_attention_bf16(
                    _p(out), _p(part_acc), _p(part_ml), _p(q), _p(cache), _p(block_table), items, _p(tok_req),
                    _p(positions), n_decode, q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size,
                    float(scale), int(window), splits, num_pages, _p(counters), stream)
            group = nq // nkv
            in_cluster = (n_decode * nkv * splits <= 296 and 2 <= splits <= 8
                          and splits * 4 * -(-group // splits) * (d + 2) * 4 <= 16 * 1024)     # as launch_decode decides
            self._check(rc, kernels=2 if splits > 1 and counters is None and not in_cluster else 1)
        if n_tiles:
            if os.environ.get("PTL_PREFILL_TC", "1") != "0":
                rc = self.lib.ptl_prefill_attention_tc_bf16(
                    _p(out), _p(q), _p(cache), _p(block_table), _p(tiles.tensor), n_tiles, q.shape[0],
                    q.shape[1], nq * d, block_table.shape[1], nq, nkv, d, page_size, float(scale), int(window), num_pages,
                    _p(self._tc_status_word()), stream)
                if rc != -2:          # -2: sizes the tcgen05 kernel leaves to the warp-level one
                    self._check(rc)
                    return
            self._check(self.lib.ptl_prefill_attention_bf16(
                _p(out), _p(q), _p(cache), _p(block_table), _p(tiles.tensor), n_tiles, q.shape[1],
                nq * d, block_table.shape[1], nq, nkv, d, page_size, float(scale), int(window), num_pages, stream))

    def token_logprobs(self, logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        """log softmax(logits[row])[tokens[row]] as float32 [rows]."""
        self._want(logits, "logits", torch.float32)
        self._want(tokens, "tokens", torch.int32)
        rows, vocab = logits.shape
        out = self.empty((rows,), torch.float32)
        scratch = self.empty((2, rows, 32), torch.float32)   # per row the maxima of 32 slices and their sums of exponentials
        self._check(self.lib.ptl_token_logprob(_p(out), _p(logits), _p(tokens), _p(scratch[0]), _p(scratch[1]), rows, vocab, vocab,
                                               self._stream()), kernels=2)
        return out

    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
               u: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 token per row (written to ``out`` if given); rows with temperature <= 0 (or
        temperature None) take the argmax."""
        self._want(logits, "logits", torch.float32)
        rows, vocab = logits.shape
        if out is None:
            out = self.empty((rows,), torch.int32)
        else:
            self._want(out, "out", torch.int32)
            if out.shape[0] != rows:
                raise KernelError(f"sample: out has {out.shape[0]} rows, the logits {rows}")
        if temperature is None and rows <= 65535:
            scratch = self.empty((2, rows, 32), torch.float32)   # per row 32 best values, and (as int32) their indices
            self._check(self.lib.ptl_argmax(_p(out), _p(logits), _p(scratch[0]), _p(scratch[1]), rows, vocab, vocab,
                                            self._stream()), kernels=2)
            return out
        probs = work = None
        kernels = 2
        if temperature is not None:
            for name, t in (("temperature", temperature), ("top_p", top_p), ("u", u)):
                self._want(t, name, torch.float32)
            probs = self.empty((rows, vocab), torch.float32)
            work = self._sample_work(rows)
            kernels = 6
        scratch = self.empty((2, rows, 32), torch.float32)   # per row the maxima of 32 slices, and (as int32) their indices
        self._check(self.lib.ptl_sample(_p(out), _p(logits), _p(probs), _p(temperature), _p(top_p), _p(u), _p(scratch[0]),
                                        _p(scratch[1]), _p(work), rows, vocab, vocab, self._stream()), kernels=kernels)
        return out

    def _sample_work(self, rows: int) -> torch.Tensor:
        """The histograms of the sampling kernels: zero before the first call, and every call leaves
        them zero, so one buffer serves all calls on this device's stream."""
        have = getattr(self, "_sample_work_buf", None)
        words = self.lib.ptl_sample_work_words()
        if have is None or have.numel() < rows * words:
            cap = max(64, 1 << (rows - 1).bit_length())
            self._sample_work_buf = have = torch.zeros(cap * words, dtype=torch.int64, device=self.device)
        return have
