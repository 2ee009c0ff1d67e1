"""Bindings of the CUDA kernels: torch tensors in, raw pointers to the libraries.

Every function here launches hand-written sm_100a code from ``csrc/`` on the
current CUDA stream.  There is no CPU path and no library attention or model
code behind any of them: if the libraries cannot be built or loaded, the
first call raises.  Tensors are checked (device, dtype, contiguity) before a
pointer leaves Python.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Dict, Optional, Tuple

import torch

from .csrc import build as _build

GEMM_STORE, GEMM_STORE_F32, GEMM_ADD_F32, GEMM_SWIGLU = 0, 1, 2, 3
STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a page id outside the pool",
               4: "a row index outside the batch", 8: "a bounded device-side wait gave up"}

_c_int, _c_ll, _c_float, _c_ptr = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or a launch failed."""


class DeviceStatusError(RuntimeError):
    """A kernel recorded a fault in the status word (bad token, bad page, ...)."""


# ----------------------------------------------------------------------------
# libraries
# ----------------------------------------------------------------------------
_core_lib: Optional[ctypes.CDLL] = None
_attn_libs: Dict[int, ctypes.CDLL] = {}

# Set to False to send bfloat16 products through the CUDA-core kernel (for A/B checks).
USE_TCGEN05 = os.environ.get("TGE_NO_TCGEN05", "") == ""
# Set to False to send bfloat16 attention through the CUDA-core kernel.
USE_MMA_ATTENTION = os.environ.get("TGE_NO_MMA_ATTENTION", "") == ""


def _declare(lib: ctypes.CDLL, name: str, argtypes) -> None:
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = _c_int


def core() -> ctypes.CDLL:
    global _core_lib
    if _core_lib is None:
        path = _build.build_core()
        lib = ctypes.CDLL(path)
        lib.tge_last_error.restype = ctypes.c_char_p
        _declare(lib, "tge_embedding", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_rmsnorm", [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float,
                                      _c_ptr, _c_ptr])
        _declare(lib, "tge_add_to_stream", [_c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr])
        _declare(lib, "tge_rope_kv_store", [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                            _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_gemm_simt", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int, _c_int,
                                        _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                                           _c_int, _c_int, _c_ptr, _c_ll, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                                           _c_int, _c_float, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_add_defer", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int,
                                                     _c_int, _c_int, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll,
                                                     _c_ptr, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_defer_slices", [_c_int])
        _declare(lib, "tge_scale_rows", [_c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_float, _c_ptr, _c_ll, _c_int,
                                         _c_int, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_add_norm", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                                                    _c_int, _c_ptr, _c_float, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr,
                                                    _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_qkv_rope", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                                                    _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                                    _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                    _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr])
        lib.tge_gemm_tcgen05_pair_mode.argtypes = [_c_int]
        lib.tge_gemm_tcgen05_pair_mode.restype = None
        lib.tge_gemm_tcgen05_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.tge_gemm_tcgen05_scratch_floats.restype = _c_ll
        _declare(lib, "tge_attention_simt", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr,
                                             _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                             _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_sample", [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_apply_penalty", [_c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_sample_cuts", [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                          _c_int, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_random_fill", [_c_ptr, _c_int, _c_ll, _c_ll, ctypes.c_ulonglong, _c_int, _c_float, _c_int,
                                          ctypes.c_uint, _c_ptr])
        _declare(lib, "tge_wait_gives_up", [_c_ptr, _c_ll, _c_ptr, _c_ptr])
        lib.tge_device_sm_count.argtypes = []
        lib.tge_device_sm_count.restype = _c_int
        lib.tge_sample_cuts_padded.argtypes = [_c_int]
        lib.tge_sample_cuts_padded.restype = _c_ll
        _core_lib = lib
    return _core_lib


def attention_lib(head_dim: int) -> ctypes.CDLL:
    if head_dim not in _attn_libs:
        path = _build.build_attention(head_dim)
        lib = ctypes.CDLL(path)
        lib.tge_last_error.restype = ctypes.c_char_p
        _declare(lib, "tge_attention_mma", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr,
                                            _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_int,
                                            _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr])
        lib.tge_attention_mma_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.tge_attention_mma_scratch_floats.restype = _c_ll
        if lib.tge_attention_mma_head_dim() != head_dim:
            raise KernelError(f"{path} was built for another head size")
        _attn_libs[head_dim] = lib
    return _attn_libs[head_dim]


def mma_attention_supports(head_dim: int, heads: int, kv_heads: int, page_size: int) -> bool:
    return (head_dim % 16 == 0 and 16 <= head_dim <= 256 and heads % kv_heads == 0
            and heads // kv_heads <= 64 and 64 % page_size == 0)


def loaded_libraries() -> Tuple[str, ...]:
    names = []
    if _core_lib is not None:
        names.append(_core_lib._name)
    names.extend(lib._name for lib in _attn_libs.values())
    return tuple(names)


UNSUPPORTED = -100
launches = 0          # kernels launched through this module since import (or since the caller reset it)


def _check(rc: int, lib: ctypes.CDLL) -> int:
    """Raises on an error code; otherwise counts and returns the number of kernels launched."""
    global launches
    if rc == UNSUPPORTED:
        return rc
    if rc < 0:
        raise KernelError(lib.tge_last_error().decode("utf-8", "replace"))
    launches += rc
    return rc


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (asked on every launch: a graph capture switches streams)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _want(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _rows_2d(t: torch.Tensor, name: str) -> int:
    """Row stride (elements) of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with dense rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


_FLOAT = (torch.float32, torch.bfloat16)

# ----------------------------------------------------------------------------
# status word and scratch
# ----------------------------------------------------------------------------
_status: Dict[int, torch.Tensor] = {}
_scratch: Dict[int, torch.Tensor] = {}
_outgrown: Dict[int, list] = {}       # earlier scratch buffers, kept alive for the graphs that hold their address


def status_word(device: Optional[torch.device] = None) -> torch.Tensor:
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _status:
        _status[index] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{index}")
    return _status[index]


def check_status() -> None:
    """Reads the status word (synchronises) and raises if a kernel recorded a fault."""
    word = status_word()
    value = int(word.item())
    if value:
        word.zero_()
        what = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise DeviceStatusError("a kernel met " + " and ".join(what or [f"status {value}"]))


def wait_gives_up(limit_ns: int = 1_000_000) -> Tuple[bool, int]:
    """Launches one thread that waits, with the product kernels' bounded wait and a limit of ``limit_ns``
    (at most 10 ms), on a barrier nothing arrives at.  Returns (whether the wait claimed success, nanoseconds
    it took); the status word then carries the time-out bit until :func:`check_status` reads it."""
    lib = core()
    outcome = torch.zeros(2, dtype=torch.int64, device=f"cuda:{torch.cuda.current_device()}")
    _check(lib.tge_wait_gives_up(status_word().data_ptr(), int(limit_ns), outcome.data_ptr(), _stream()), lib)
    arrived, took = outcome.tolist()
    return bool(arrived), int(took)


def scratch_floats(count: int) -> torch.Tensor:
    """A float32 scratch buffer of at least ``count`` elements, reused between calls.

    The buffer grows when a call needs more (never while a CUDA graph is being captured).  A buffer that
    was outgrown is kept, not freed: a graph captured earlier has its address in its kernels and goes on
    writing partial sums there whenever it is replayed.  Buffers at least double, so what is kept is less
    than what is in use.
    """
    index = torch.cuda.current_device()
    have = _scratch.get(index)
    if have is None or have.numel() < count:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("scratch memory must be sized before a CUDA graph is captured "
                              f"(need {count} floats, have {0 if have is None else have.numel()})")
        size = max(count, 1 << 22, 0 if have is None else 2 * have.numel())
        if have is not None:
            _outgrown.setdefault(index, []).append(have)
        _scratch[index] = torch.empty(size, dtype=torch.float32, device=f"cuda:{index}")
    return _scratch[index]


# ----------------------------------------------------------------------------
# kernels
# ----------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, :] = float32(table[ids[t], :])"""
    _want(table, "embedding table", _FLOAT)
    _want(ids, "token ids", torch.int32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    _want(out, "embedding output", torch.float32)
    lib = core()
    _check(lib.tge_embedding(table.data_ptr(), int(table.dtype == torch.bfloat16), ids.data_ptr(), out.data_ptr(),
                             tokens, hidden, vocab, status_word().data_ptr(), _stream()), lib)
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows (optionally gathered by ``rows``) into ``out_dtype``."""
    _want(x, "norm input", torch.float32)
    _want(weight, "norm weight", torch.float32)
    src_rows, hidden = x.shape
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {hidden}")
    out_rows = src_rows if rows is None else rows.numel()
    if rows is not None:
        _want(rows, "norm row index", torch.int32)
    if out is None:
        out = torch.empty((out_rows, hidden), dtype=out_dtype, device=x.device)
    _want(out, "norm output", _FLOAT)
    lib = core()
    _check(lib.tge_rmsnorm(x.data_ptr(), weight.data_ptr(), _ptr(rows), out.data_ptr(),
                           int(out.dtype == torch.bfloat16), out_rows, src_rows, hidden, float(eps),
                           status_word().data_ptr(), _stream()), lib)
    return out


def add_to_stream(x: torch.Tensor, y: torch.Tensor) -> None:
    """x (float32) += y (run dtype), same shape."""
    _want(x, "stream", torch.float32)
    _want(y, "addend", _FLOAT)
    if x.shape != y.shape:
        raise KernelError(f"add_to_stream: shapes differ, {tuple(x.shape)} and {tuple(y.shape)}")
    lib = core()
    _check(lib.tge_add_to_stream(x.data_ptr(), y.data_ptr(), int(y.dtype == torch.bfloat16), x.numel(), _stream()), lib)


def rope_kv_store(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary: int,
                  positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                  k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], heads: int, kv_heads: int,
                  head_dim: int) -> None:
    """Rotates q (in place) and k, and stores k and v into their pages.

    qkv: [T, >= (heads + 2*kv_heads) * head_dim].  cos/sin: float32 [positions, rotary/2]
    (None with rotary == 0: no rotation).  Pages: [num_pages, kv_heads, page_size, head_dim];
    None: nothing is stored (a layer that reads another layer's cache).
    """
    _want(qkv, "qkv", _FLOAT, contiguous=False)
    stride = _rows_2d(qkv, "qkv")
    tokens = qkv.shape[0]
    store = k_pages is not None
    if rotary > 0:
        _want(cos, "cos table", torch.float32)
        _want(sin, "sin table", torch.float32)
        if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != rotary // 2:
            raise KernelError(f"rotary tables must be [positions, {rotary // 2}], got {tuple(cos.shape)}")
    _want(positions, "positions", torch.int32)
    _want(seq_of_token, "seq_of_token", torch.int32)
    num_pages = page_size = max_pages = 0
    if store:
        _want(k_pages, "k pages", qkv.dtype)
        _want(v_pages, "v pages", qkv.dtype)
        _want(block_table, "block table", torch.int32)
        if k_pages.shape != v_pages.shape or k_pages.dim() != 4 or k_pages.shape[1] != kv_heads or k_pages.shape[3] != head_dim:
            raise KernelError(f"pages must be [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pages.shape)}")
        num_pages, _, page_size, _ = k_pages.shape
        max_pages = block_table.shape[1]
    lib = core()
    _check(lib.tge_rope_kv_store(qkv.data_ptr(), int(qkv.dtype == torch.bfloat16), stride, _ptr(cos), _ptr(sin),
                                 0 if cos is None else cos.shape[0], positions.data_ptr(), seq_of_token.data_ptr(),
                                 _ptr(block_table), max_pages, _ptr(k_pages), _ptr(v_pages), num_pages, page_size,
                                 tokens, heads, kv_heads if store else 0, head_dim, rotary, int(store),
                                 status_word().data_ptr(), _stream()), lib)


DEFER_MAX_TOKENS = 128      # rows that may travel without their norm factor (the small-batch products)


class DeferredRows:
    """Rows ``stream * norm_weight`` in bfloat16 that still lack their RMSNorm factor.

    ``sums`` (float32 [slices, M]) holds each row's sum of squares in slices; the factor of row m is
    ``1 / sqrt(sum over slices / width + eps)``.  The product that takes these rows multiplies its result
    by it (``linear`` and ``linear_qkv_rope_store`` do); ``complete()`` gives the normalised rows.
    """

    def __init__(self, rows: torch.Tensor, sums: torch.Tensor, width: int, eps: float):
        self.rows, self.sums, self.width, self.eps = rows, sums, int(width), float(eps)

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    @property
    def device(self):
        return self.rows.device

    def factor_args(self):
        return self.sums.data_ptr(), self.sums.shape[0], self.width, self.eps

    def complete(self) -> torch.Tensor:
        lib = core()
        M, N = self.rows.shape
        out = torch.empty_like(self.rows)
        _check(lib.tge_scale_rows(self.rows.data_ptr(), _rows_2d(self.rows, "rows"), self.sums.data_ptr(),
                                  self.sums.shape[0], self.width, self.eps, out.data_ptr(), N, M, N, _stream()), lib)
        return out


_NO_FACTOR = (None, 0, 0, 0.0)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int,
           out: Optional[torch.Tensor] = None, force_simt: bool = False, force_bn: int = 0,
           force_splits: int = 0) -> torch.Tensor:
    """out = x . w^T with an epilogue.

    x [M, K] and w [N, K] in the run dtype; bias float32 [N] or None.
    GEMM_STORE: out [M, N] run dtype.  GEMM_STORE_F32: out [M, N] float32.
    GEMM_ADD_F32: ``out`` (float32 [M, N], required) += product.
    GEMM_SWIGLU: w rows interleaved (gate_i, up_i); out [M, N/2] run dtype.
    bfloat16 goes to the tcgen05 kernel when the shape allows TMA, else (and all of
    float32) to the CUDA-core kernel.
    """
    deferred = x if isinstance(x, DeferredRows) else None
    if deferred is not None:
        x = deferred.rows
    _want(x, "linear input", _FLOAT, contiguous=False)
    _want(w, "linear weight", x.dtype, contiguous=False)
    ldx, ldw = _rows_2d(x, "linear input"), _rows_2d(w, "linear weight")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: input has {K} columns, weight has {w.shape[1]}")
    if bias is not None:
        _want(bias, "linear bias", torch.float32)
        if bias.numel() != N:
            raise KernelError(f"linear: bias has {bias.numel()} elements for {N} rows")
    if epilogue == GEMM_ADD_F32:
        if out is None:
            raise KernelError("linear: the residual epilogue needs the stream as `out`")
        want_shape, want_dtype = (M, N), torch.float32
    elif epilogue == GEMM_STORE_F32:
        want_shape, want_dtype = (M, N), torch.float32
    elif epilogue == GEMM_SWIGLU:
        want_shape, want_dtype = (M, N // 2), x.dtype
    elif epilogue == GEMM_STORE:
        want_shape, want_dtype = (M, N), x.dtype
    else:
        raise KernelError(f"linear: unknown epilogue {epilogue}")
    if out is None:
        out = torch.empty(want_shape, dtype=want_dtype, device=x.device)
    _want(out, "linear output", want_dtype, contiguous=False)
    if tuple(out.shape) != want_shape:
        raise KernelError(f"linear: output must be {want_shape}, got {tuple(out.shape)}")
    ldo = _rows_2d(out, "linear output")
    lib = core()
    if x.dtype == torch.bfloat16 and USE_TCGEN05 and not force_simt and (deferred is None or M <= DEFER_MAX_TOKENS):
        need = lib.tge_gemm_tcgen05_scratch_floats(M, N, K) if force_splits == 0 else force_splits * M * N
        scratch = scratch_floats(need) if need > 0 else None
        factor = _NO_FACTOR if deferred is None else deferred.factor_args()
        rc = lib.tge_gemm_tcgen05(x.data_ptr(), ldx, w.data_ptr(), ldw, _ptr(bias), out.data_ptr(), ldo, M, N, K,
                                  epilogue, _ptr(scratch), 0 if scratch is None else scratch.numel(), force_bn,
                                  force_splits, status_word().data_ptr(), *factor, _stream())
        if _check(rc, lib) != UNSUPPORTED:
            return out
    if deferred is not None:
        x = deferred.complete()
        ldx = _rows_2d(x, "linear input")
    _check(lib.tge_gemm_simt(x.data_ptr(), ldx, w.data_ptr(), ldw, _ptr(bias), out.data_ptr(), ldo, M, N, K,
                             int(x.dtype == torch.bfloat16), epilogue, _stream()), lib)
    return out


def set_pair_gemm(mode: int) -> None:
    """Whether the bfloat16 product may pair two SMs on one tile: 0 never, 1 where it is expected to be
    faster (the default), 2 wherever the kernel can run (tests)."""
    core().tge_gemm_tcgen05_pair_mode(int(mode))


# Small batches: the product leaves partial sums and one kernel per token row adds them, normalises or rotates and
# stores; larger ones use the product's own epilogue and separate kernels.  Prompts of 144 / 160 / 256 tokens at the
# 7B shape took 4.40 / 4.66 / 5.32 ms the first way and 4.54 / 4.56 / 5.04 ms the second (14B: 8.4 / 9.1 / 11.0 and
# 8.6 / 9.0 / 10.9), so the change is made between 144 and 160.  (The kernels themselves take up to 256 rows.)
FUSED_MAX_TOKENS = 144


def linear_add_norm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], stream: torch.Tensor,
                    norm_weight: torch.Tensor, eps: float, out_dtype: torch.dtype, defer: bool = False):
    """stream (float32 [M, N]) += x . w^T (+ bias); returns RMSNorm(stream) * norm_weight in ``out_dtype``.

    For a small bfloat16 batch the partial sums of the product are added into the stream and the new
    rows normalised by one kernel; otherwise the product and the norm run as separate kernels.
    With ``defer`` (the caller knows that ``linear`` or ``linear_qkv_rope_store`` takes the result) up to 128
    rows may come back as :class:`DeferredRows`: without the norm's factor, which their taker applies.
    """
    M, K = x.shape
    N = w.shape[0]
    if x.dtype == torch.bfloat16 and USE_TCGEN05 and M <= FUSED_MAX_TOKENS and out_dtype == torch.bfloat16:
        _want(x, "linear input", torch.bfloat16, contiguous=False)
        _want(w, "linear weight", torch.bfloat16, contiguous=False)
        _want(stream, "stream", torch.float32, contiguous=False)
        _want(norm_weight, "norm weight", torch.float32)
        if bias is not None:
            _want(bias, "linear bias", torch.float32)
        if tuple(stream.shape) != (M, N) or w.shape[1] != K or norm_weight.numel() != N:
            raise KernelError("linear_add_norm: shapes do not fit")
        lib = core()
        need = max(lib.tge_gemm_tcgen05_scratch_floats(M, N, K), M * N)
        scratch = scratch_floats(need)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        if defer and M <= DEFER_MAX_TOKENS and N % 8 == 0:
            # the taker of these rows applies the norm's factor: no block waits for a whole row here
            sums = torch.empty((lib.tge_gemm_tcgen05_defer_slices(N), M), dtype=torch.float32, device=x.device)
            rc = lib.tge_gemm_tcgen05_add_defer(x.data_ptr(), _rows_2d(x, "linear input"), w.data_ptr(),
                                                _rows_2d(w, "linear weight"), _ptr(bias), stream.data_ptr(),
                                                _rows_2d(stream, "stream"), M, N, K, norm_weight.data_ptr(),
                                                out.data_ptr(), N, sums.data_ptr(), scratch.data_ptr(),
                                                scratch.numel(), status_word().data_ptr(), _stream())
            if _check(rc, lib) != UNSUPPORTED:
                return DeferredRows(out, sums, N, eps)
        rc = lib.tge_gemm_tcgen05_add_norm(x.data_ptr(), _rows_2d(x, "linear input"), w.data_ptr(),
                                           _rows_2d(w, "linear weight"), _ptr(bias), stream.data_ptr(),
                                           _rows_2d(stream, "stream"), M, N, K, norm_weight.data_ptr(), float(eps),
                                           out.data_ptr(), N, scratch.data_ptr(), scratch.numel(),
                                           status_word().data_ptr(), _stream())
        if _check(rc, lib) != UNSUPPORTED:
            return out
    linear(x, w, bias, GEMM_ADD_F32, out=stream)
    return rmsnorm(stream, norm_weight, eps, out_dtype)


def linear_qkv_rope_store(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                          sin: Optional[torch.Tensor], rotary: int, positions: torch.Tensor,
                          seq_of_token: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                          v_pages: torch.Tensor, heads: int, kv_heads: int, head_dim: int) -> torch.Tensor:
    """The fused q/k/v product of an attention layer followed by rotation and the cache store.

    Returns the qkv buffer [T, (heads + 2 kv_heads) * head_dim] whose first heads*head_dim columns hold the
    rotated queries.  For a small bfloat16 batch one kernel per token row adds the product's partial sums,
    rotates and stores; otherwise the product and the rotate-and-store kernel run one after the other
    (then the k and v columns of the buffer are filled as well).
    """
    deferred = x if isinstance(x, DeferredRows) else None
    if deferred is not None:
        x = deferred.rows
    M, K = x.shape
    N = w.shape[0]
    if (x.dtype == torch.bfloat16 and USE_TCGEN05 and M <= FUSED_MAX_TOKENS):
        _want(x, "linear input", torch.bfloat16, contiguous=False)
        _want(w, "linear weight", torch.bfloat16, contiguous=False)
        for name, t in (("positions", positions), ("seq_of_token", seq_of_token), ("block table", block_table)):
            _want(t, name, torch.int32)
        _want(k_pages, "k pages", torch.bfloat16)
        _want(v_pages, "v pages", torch.bfloat16)
        if rotary > 0:
            _want(cos, "cos table", torch.float32)
            _want(sin, "sin table", torch.float32)
        if bias is not None:
            _want(bias, "linear bias", torch.float32)
        num_pages, page_kv, page_size, page_hd = k_pages.shape
        if page_kv != kv_heads or page_hd != head_dim or v_pages.shape != k_pages.shape or w.shape[1] != K:
            raise KernelError("linear_qkv_rope_store: shapes do not fit")
        lib = core()
        need = max(lib.tge_gemm_tcgen05_scratch_floats(M, N, K), M * N)
        scratch = scratch_floats(need)
        qkv = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        rc = lib.tge_gemm_tcgen05_qkv_rope(x.data_ptr(), _rows_2d(x, "linear input"), w.data_ptr(),
                                           _rows_2d(w, "linear weight"), _ptr(bias), qkv.data_ptr(), N, M, N, K,
                                           _ptr(cos), _ptr(sin), 0 if cos is None else cos.shape[0], rotary,
                                           positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                           block_table.shape[1], k_pages.data_ptr(), v_pages.data_ptr(), num_pages,
                                           page_size, heads, kv_heads, head_dim, scratch.data_ptr(), scratch.numel(),
                                           status_word().data_ptr(),
                                           *(_NO_FACTOR if deferred is None else deferred.factor_args()), _stream())
        if _check(rc, lib) != UNSUPPORTED:
            return qkv
    qkv = linear(x if deferred is None else deferred, w, bias, GEMM_STORE)
    rope_kv_store(qkv, cos, sin, rotary, positions, seq_of_token, block_table, k_pages, v_pages, heads, kv_heads,
                  head_dim)
    return qkv


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
              q_start: torch.Tensor, start_pos: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
              num_seqs: int, max_q_len: int, max_ctx_len: int, heads: int, kv_heads: int, head_dim: int,
              scale: float, window: int = 0, split_tokens: int = 0, out: Optional[torch.Tensor] = None,
              force_simt: bool = False, typical_ctx_len: int = 0, decode_prefix: int = 0) -> torch.Tensor:
    """Paged causal attention of a flat batch of portions.

    q: [T, >= heads*head_dim] (dense rows, any row stride) holding rotated queries;
    pages [num_pages, kv_heads, page_size, head_dim] already hold the keys and values of
    every position up to each portion's last token.  Returns [T, heads*head_dim].
    ``split_tokens`` > 0 cuts the keys into runs of that many positions (a multiple of 64)
    that are attended in parallel and merged; 0 picks a value from the batch shape.
    ``decode_prefix``: how many sequences at the head of the batch are known to bring one token each
    while others bring more (0: unknown); the tensor-core path then serves them with its decode kernel.
    """
    _want(q, "queries", _FLOAT, contiguous=False)
    q_stride = _rows_2d(q, "queries")
    tokens = q.shape[0]
    _want(k_pages, "k pages", q.dtype)
    _want(v_pages, "v pages", q.dtype)
    for name, t in (("block table", block_table), ("q_start", q_start), ("start_pos", start_pos),
                    ("positions", positions), ("seq_of_token", seq_of_token)):
        _want(t, name, torch.int32)
    num_pages, page_kv, page_size, page_hd = k_pages.shape
    if page_kv != kv_heads or page_hd != head_dim or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages must be [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pages.shape)}")
    max_pages = block_table.shape[1]
    if out is None:
        out = torch.empty((tokens, heads * head_dim), dtype=q.dtype, device=q.device)
    _want(out, "attention output", q.dtype, contiguous=False)
    out_stride = _rows_2d(out, "attention output")
    use_mma = (q.dtype == torch.bfloat16 and USE_MMA_ATTENTION and not force_simt
               and mma_attention_supports(head_dim, heads, kv_heads, page_size))
    if use_mma:
        lib = attention_lib(head_dim)
        prefix = decode_prefix if decode_prefix >= MIN_DECODE_PREFIX and max_q_len > 1 else 0
        prefix_split = split_tokens
        if split_tokens == 0:
            split_tokens = choose_attention_split(tokens, num_seqs, max_q_len, typical_ctx_len or max_ctx_len,
                                                  heads, kv_heads, bound=max_ctx_len)
            # the single tokens at the head of a mixed step are a decode batch of their own: a few of them deep in
            # long contexts want their keys cut although the portions beside them do not
            prefix_split = choose_attention_split(prefix, prefix, 1, max_ctx_len, heads, kv_heads,
                                                  bound=max_ctx_len) if prefix else 0
        count = lambda split: 1 if split == 0 or max_ctx_len <= split else -(-max_ctx_len // split)
        splits = max(count(split_tokens), count(prefix_split) if prefix else 1)
        need = lib.tge_attention_mma_scratch_floats(tokens, heads, splits)
        scratch = scratch_floats(need) if need > 0 else None
        _check(lib.tge_attention_mma(q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(),
                                     block_table.data_ptr(), max_pages, num_pages, page_size, q_start.data_ptr(),
                                     start_pos.data_ptr(), positions.data_ptr(), num_seqs, tokens, max_q_len,
                                     max_ctx_len, out.data_ptr(), out_stride, heads, kv_heads, float(scale), window,
                                     split_tokens, _ptr(scratch), status_word().data_ptr(), prefix, prefix_split,
                                     _stream()), lib)
        return out
    lib = core()
    _check(lib.tge_attention_simt(q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(),
                                  block_table.data_ptr(), max_pages, num_pages, page_size, positions.data_ptr(),
                                  seq_of_token.data_ptr(), out.data_ptr(), out_stride, tokens, heads, kv_heads,
                                  head_dim, float(scale), window, int(q.dtype == torch.bfloat16),
                                  status_word().data_ptr(), _stream()), lib)
    return out


# Fewer leading single-token sequences than this ride along in the prefill kernel: each fills one query tile,
# which costs less than another launch.
MIN_DECODE_PREFIX = 8


def choose_attention_split(tokens: int, num_seqs: int, max_q_len: int, max_ctx_len: int, heads: int,
                           kv_heads: int, bound: int = 0) -> int:
    """Keys per split for the tensor-core attention: enough blocks to fill the GPU, no more.

    The choice depends on the step's shape only through launch geometry; a row's value
    differs between choices by rounding alone.
    """
    if max_ctx_len <= 256:
        return 0
    group = heads // kv_heads
    if max_q_len <= 1 and group <= 16:
        blocks = num_seqs * kv_heads                      # the decode kernel: one block per (request, kv head)
    elif max_q_len > 1:
        # Portions of prompts.  Cutting their keys pays only where a block's keys are many and the rows to merge
        # few: a short portion deep in a long context.  A block takes 64 rows or more; a prompt of 320 tokens cut
        # in two took 18 us per layer for the attention and 34 us for merging its 8,960 rows of partial states.
        if max_ctx_len < 2048 or tokens * 4 > max_ctx_len:
            return 0
        blocks = -(-tokens // max(64 // group, 1)) * kv_heads
    else:
        blocks = num_seqs * kv_heads
    sms = core().tge_device_sm_count()
    most = -(-max_ctx_len // 128)                             # no split below 128 keys

    def keys_per_split(splits: int) -> int:
        return max(128, -(-(-(-max_ctx_len // splits)) // 64) * 64)

    if max_q_len > 1:
        # Two blocks fit on each SM (148 on a B200) and all blocks should run at once: a few more than that and
        # the last ones run alone.
        want_splits = min(2 * sms // blocks, most)
        return keys_per_split(want_splits) if want_splits > 1 else 0
    # Single tokens.  About one block per SM is best: every split more is a state more to write and to merge, and
    # the merging kernel holds sixteen states in registers (A/B in one process, ms per step of the 7B shape, 296
    # blocks against 148: batch 16 at context 2,048 3.33 / 3.22; batch 8 at 4,096 3.30 / 3.13; batch 4 at 4,096
    # 3.23 / 3.04; batch 4 at 30,000 4.05 / 3.89; batch 1 at 32,000 3.71 / 3.38).  Two exceptions, both measured:
    # splits of no more than 256 keys, sixteen at most over the whole bound, are better taken twice as many
    # (batch 8 at 2,048: 3.03 / 3.07); and requests that alone make half the SMs' worth of blocks or more are
    # still cut in two once their keys are many (batch 32 at 4,096: 4.29 / 4.57).
    want_splits = min(sms // blocks, most)
    twice = min(2 * sms // blocks, most)
    if twice > want_splits and keys_per_split(twice) <= 256 and -(-max(bound, max_ctx_len) // keys_per_split(twice)) <= 16:
        want_splits = twice
    if want_splits <= 1 and 2 * blocks <= 2 * sms and max_ctx_len >= 4096:
        want_splits = 2
    return keys_per_split(want_splits) if want_splits > 1 else 0


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits: arg-max where temperature <= 0, else a draw."""
    _want(logits, "logits", torch.float32, contiguous=False)
    stride = _rows_2d(logits, "logits")
    rows, vocab = logits.shape
    _want(temperature, "temperature", torch.float32)
    _want(uniform, "uniform draws", torch.float32)
    if temperature.numel() != rows or uniform.numel() != rows:
        raise KernelError("sample: one temperature and one uniform draw per row")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _want(out, "sampled ids", torch.int32)
    lib = core()
    _check(lib.tge_sample(logits.data_ptr(), stride, temperature.data_ptr(), uniform.data_ptr(), out.data_ptr(), rows,
                          vocab, _stream()), lib)
    return out


def apply_penalty(logits: torch.Tensor, history: torch.Tensor, history_start: torch.Tensor,
                  penalty: torch.Tensor) -> torch.Tensor:
    """A copy of ``logits`` (float32 [R, V]) with the repetition penalty applied.

    ``history`` (int32) is every row's window of recent tokens, one after another;
    ``history_start`` (int32 [R + 1]) its offsets; ``penalty`` float32 [R], 1.0 = off.
    """
    _want(logits, "logits", torch.float32, contiguous=False)
    stride = _rows_2d(logits, "logits")
    rows, vocab = logits.shape
    for name, t, dtype in (("history", history, torch.int32), ("history offsets", history_start, torch.int32),
                           ("penalty", penalty, torch.float32)):
        _want(t, name, dtype)
    out = logits.clone()
    lib = core()
    _check(lib.tge_apply_penalty(logits.data_ptr(), out.data_ptr(), stride, history.data_ptr(),
                                 history_start.data_ptr(), penalty.data_ptr(), rows, vocab, _stream()), lib)
    return out


def sample_cuts(scores: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                min_p: torch.Tensor, uniform: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row with the top-k / min-p / top-p cuts (0 / 0.0 / 1.0 switch a cut off).  Given ``out``
    (int32 [rows], already holding ids), rows with every cut switched off are left as they are."""
    _want(scores, "scores", torch.float32, contiguous=False)
    stride = _rows_2d(scores, "scores")
    rows, vocab = scores.shape
    for name, t, dtype in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                           ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                           ("uniform draws", uniform, torch.float32)):
        _want(t, name, dtype)
        if t.numel() != rows:
            raise KernelError(f"sample_cuts: one {name} per row")
    lib = core()
    padded = lib.tge_sample_cuts_padded(vocab)
    sort_prob = torch.empty((rows, padded), dtype=torch.float32, device=scores.device)
    sort_index = torch.empty((rows, padded), dtype=torch.int32, device=scores.device)
    skip_uncut = out is not None
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=scores.device)
    _want(out, "sampled ids", torch.int32)
    if out.numel() != rows:
        raise KernelError("sample_cuts: one id per row")
    _check(lib.tge_sample_cuts(scores.data_ptr(), stride, temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                               min_p.data_ptr(), uniform.data_ptr(), sort_prob.data_ptr(), sort_index.data_ptr(),
                               out.data_ptr(), rows, vocab, int(skip_uncut), _stream()), lib)
    return out
