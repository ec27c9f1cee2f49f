"""ctypes binding of libhsa_b200.so (the C ABI declared in include/hsa_b200.h).

There is no fallback: if the library is missing or a call fails, the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import Structure, c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("HSA_B200_LIBRARY", os.path.join(HERE, "libhsa_b200.so"))   # override: a build to compare

HSA_F32, HSA_BF16, HSA_F16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: HSA_F32, torch.bfloat16: HSA_BF16, torch.float16: HSA_F16}

ALGO_AUTO, ALGO_PORTABLE, ALGO_TENSOR_CORE = 0, 1, 2


class HsaView(Structure):
    _fields_ = [("ptr", c_void_p), ("batch_stride", c_int64), ("row_stride", c_int64)]


class HsaError(RuntimeError):
    pass


class GemmEpilogue(Structure):
    """hsa_gemm_epilogue of include/hsa_b200.h."""
    _fields_ = [("relu", c_int), ("rng_state", c_void_p), ("drop_site0", ctypes.c_uint), ("drop_site1", ctypes.c_uint),
                ("drop_threshold", ctypes.c_uint), ("drop_scale", c_float), ("drop_col_begin", c_int),
                ("drop_col_end", c_int), ("drop_rows_total", ctypes.c_longlong), ("drop_row_offset", ctypes.c_longlong),
                ("gate", c_void_p), ("gate_bs", ctypes.c_longlong), ("gate_rs", ctypes.c_longlong), ("gate_scale", c_float),
                ("residual", c_void_p), ("res_bs", ctypes.c_longlong), ("res_rs", ctypes.c_longlong),
                ("copy_bf16", c_void_p), ("copy_bs", ctypes.c_longlong), ("copy_rs", ctypes.c_longlong),
                ("ce_partial", c_void_p), ("ce_targets", c_void_p), ("ce_classes", c_int), ("ce_skip_store", c_int)]


# name -> (restype, argtypes); one entry per declaration in include/hsa_b200.h
V = HsaView
SIGNATURES = {
    "hsa_version": (c_int, []),
    "hsa_last_error": (c_char_p, []),
    "hsa_compiled_arch": (c_int, []),
    "hsa_topology_build": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "hsa_span_input_y_rows": (c_int64, [c_int64]),
    "hsa_span_input_y_fwd": (c_int, [V, V, c_int, c_int, c_int, c_int, c_void_p]),
    "hsa_span_input_y_bwd": (c_int, [V, V, c_int, c_int, c_int, c_int, c_void_p]),
    "hsa_parent_nodes_fwd": (c_int, [V, V, V, V, V, V, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "hsa_parent_nodes_bwd": (c_int, [V] * 11 + [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "hsa_parent_tree_state_bytes": (c_size_t, []),
    "hsa_parent_tree_status": (c_int, [c_void_p, c_void_p]),
    "hsa_parent_tree_fwd": (c_int, [V, V, V, V, V, c_void_p] + [c_int] * 5 + [c_void_p, ctypes.c_uint, ctypes.c_uint, c_float,
                                    c_void_p, c_void_p]),
    "hsa_parent_tree_bwd": (c_int, [V] * 10 + [c_void_p] + [c_int] * 5 + [c_void_p, ctypes.c_uint, ctypes.c_uint, c_float,
                                    c_void_p, c_void_p]),
    "hsa_span_attn_fwd": (c_int, [V, V, V, V, c_void_p] + [c_int] * 8 + [c_void_p]),
    "hsa_span_attn_fwd_wait_expired": (c_int, [c_void_p]),
    "hsa_debug_wait_test": (c_int, [ctypes.c_longlong, ctypes.c_uint]),
    "hsa_span_attn_bwd_workspace_bytes": (c_size_t, [c_int] * 8),
    "hsa_span_attn_bwd": (c_int, [V, V, V, V, c_void_p, V, V, V, V, c_void_p, c_size_t] + [c_int] * 8 + [c_void_p]),
    "hsa_cross_entropy_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_int64,
                                      c_int, c_void_p]),
    "hsa_cross_entropy_bwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                      c_int, c_float, c_int64, c_int, c_void_p]),
    "hsa_layer_norm_supported": (c_int, [c_int]),
    "hsa_layer_norm_bwd_ctas": (c_int, [c_int64]),
    "hsa_layer_norm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float,
                                   c_int, c_void_p]),
    "hsa_layer_norm_bwd": (c_int, [c_void_p] * 9 + [c_int64, c_int, c_int, c_void_p]),
    "hsa_span_attn_logits": (c_int, [V, V, c_void_p] + [c_int] * 8 + [c_void_p]),
    "hsa_sibling_logits": (c_int, [V, V, c_void_p, c_void_p] + [c_int] * 6 + [c_void_p]),
    "hsa_span_attn_decode": (c_int, [V, V, V, V] + [c_int] * 7 + [c_void_p]),
    "hsa_gemm_workspace_bytes": (c_size_t, [c_int] * 7),
    "hsa_gemm_choose_splits": (c_int, [c_int] * 4),
    "hsa_gemm": (c_int, [V, V, V, c_void_p] + [c_int] * 9 + [c_void_p, c_size_t, c_void_p]),
    "hsa_gemm_ex": (c_int, [V, V, V, c_void_p] + [c_int] * 9 + [c_void_p, c_size_t, c_void_p, c_void_p]),
    "hsa_gemm_aborts": (c_int, [c_void_p]),
    "hsa_linear_ce_partial_bytes": (c_size_t, [ctypes.c_longlong, c_int]),
    "hsa_linear_ce_combine": (c_int, [c_void_p, ctypes.c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                      ctypes.c_longlong, c_void_p]),
    "hsa_layer_norm_fwd_mixed": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_float, c_void_p]),
    "hsa_layer_norm_bwd_mixed": (c_int, [c_void_p] * 10 + [c_int64, c_int, c_void_p]),
    "hsa_column_sums_partial_bytes": (c_size_t, [ctypes.c_longlong, c_int]),
    "hsa_column_sums": (c_int, [c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_int, c_void_p, c_void_p, c_void_p]),
    "hsa_dropout_cast_colsum": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_int, c_void_p,
                                        ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, c_float, c_void_p, c_void_p, c_void_p]),
    "hsa_cross_entropy_bwd_inplace": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int,
                                              c_float, ctypes.c_longlong, c_void_p, c_void_p, c_void_p]),
    "hsa_dropout_apply": (c_int, [V, c_int, V, c_int, c_int, c_int, c_int, ctypes.c_longlong, ctypes.c_longlong,
                                  ctypes.c_longlong, ctypes.c_longlong, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, c_float, c_void_p]),
    "hsa_copy_rows_async": (c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_size_t, c_size_t, c_int, c_void_p]),
    "hsa_span_attn_bwd_static": (c_int, [V, V, V, V, c_void_p, V, V, V, V] + [c_int] * 7 + [c_void_p]),
}
STATIC_SCRATCH_MAX_ELEMS = 1 << 20

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the shared library (once).  Raises HsaError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise HsaError(
                f"{LIB_PATH} not found. Build it with `python -m sparseattention_b200.build` "
                "(needs nvcc); this package has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().hsa_last_error().decode(errors="replace")
        raise HsaError(f"{what} failed (code {rc}): {msg}")


DEBUG = os.environ.get("HSA_B200_DEBUG", "0") not in ("", "0")
_expired_seen = {}


def wait_expired_count() -> int:
    """CTAs on the current device whose bounded wait for their bulk copies ran out (synchronises)."""
    count = ctypes.c_uint(0)
    check(load().hsa_span_attn_fwd_wait_expired(ctypes.byref(count)), "hsa_span_attn_fwd_wait_expired")
    return int(count.value)


def debug_check_waits(what: str) -> None:
    """With HSA_B200_DEBUG=1: synchronise after a span-attention call and raise if a CTA of it gave up waiting
    for its copies (its tile then holds NaN).  Without the variable this does nothing: the library itself never
    synchronises."""
    if not DEBUG:
        return
    dev = torch.cuda.current_device()
    now = wait_expired_count()
    if now != _expired_seen.get(dev, 0):
        before = _expired_seen.get(dev, 0)
        _expired_seen[dev] = now
        raise HsaError(f"{what}: {now - before} thread block(s) gave up waiting for their bulk copies; "
                       "their output rows hold NaN")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise HsaError(f"unsupported dtype {t.dtype}; use float32, bfloat16 or float16") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise HsaError("hsa_b200 ops take CUDA tensors only (there is no CPU path)")
        if t.device != dev:
            raise HsaError("all tensors of one call must live on the same device")
    return dev


def rows_view(t: torch.Tensor) -> HsaView:
    """View of a [B, rows, ...] tensor whose trailing dims form one contiguous row."""
    return HsaView(t.data_ptr(), t.stride(0), t.stride(1))


def inner_contiguous(t: torch.Tensor) -> bool:
    """True when dims 2.. of t are packed (so a row is one contiguous block)."""
    expect = 1
    for size, stride in zip(reversed(t.shape[2:]), reversed(t.stride()[2:])):
        if size != 1 and stride != expect:
            return False
        expect *= size
    return True


def as_rows(t: torch.Tensor) -> torch.Tensor:
    """Returns t itself when its rows are packed, else a contiguous copy."""
    return t if inner_contiguous(t) else t.contiguous()


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def on_device(dev: torch.device):
    """Context that makes `dev` the current CUDA device for the calls inside it; free when it already is (the device
    switch of torch.cuda.device costs several microseconds per call, more than a small kernel runs)."""
    idx = dev.index
    if idx is None or torch.cuda.current_device() == idx:
        return _NO_SWITCH
    return torch.cuda.device(idx)


def stream_ptr(dev: torch.device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(dev).cuda_stream)
