"""ctypes binding of libmoa_b200.so, the C-ABI library built from ``moa_b200/csrc``.

There is no fallback: if the library is missing, importing this module raises, and every
wrapper raises ``MoaError`` on a non-zero status.  Build with ``python moa_b200/build.py``.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
#: the library next to this file (built in-tree by ``moa_b200/build.py``)
LIB_PATH = os.path.join(HERE, "libmoa_b200.so")
ABI_VERSION = 2

F16, BF16 = 0, 1

#: every symbol include/moa_b200.h declares
SYMBOLS = (
    "moa_abi_version", "moa_strerror", "moa_last_error_detail",
    "moa_decode_workspace_bytes", "moa_decode_workspace_init", "moa_decode_fwd",
    "moa_cache_append", "moa_cache_scan_mask", "moa_cache_fill", "moa_prefill_fwd",
    "moa_decode_fwd_static", "moa_decode_rope_fwd", "moa_decode_gather_fwd", "moa_selftest_bounded_wait",
    "moa_rope_qk", "moa_peer_alloc", "moa_peer_free", "moa_peer_export", "moa_peer_open", "moa_peer_close",
    "moa_peer_barrier",
)


class MoaError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, text: str, detail: str):
        super().__init__(f"{fn} failed: status {status} ({text}){': ' + detail if detail else ''}")
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: the CUDA library is not built. Run `python moa_b200/build.py` "
            "(needs nvcc; no GPU needed to build). moa_b200 has no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    P, I64, I = c_void_p, c_int64, c_int
    lib.moa_abi_version.restype = c_int
    lib.moa_strerror.restype = c_char_p
    lib.moa_strerror.argtypes = [c_int]
    lib.moa_last_error_detail.restype = c_char_p
    lib.moa_decode_workspace_bytes.restype = c_int64
    lib.moa_decode_workspace_bytes.argtypes = [I, I, I, I64, I]
    lib.moa_decode_workspace_init.argtypes = [P, I64, P]
    # the argument list the decode entry points share: pointers, six strides, index tensors, sizes, out_f32
    decode_args = [P] * 6 + [I64] * 6 + [P] * 5 + [I64, I, I, I, I64, c_float, I, I]
    lib.moa_decode_fwd.argtypes = decode_args + [P, I64, I, P]
    lib.moa_decode_rope_fwd.argtypes = decode_args + [P, P, P, I64, I, P]
    lib.moa_decode_gather_fwd.argtypes = decode_args + [P, P, P, I, P, I, I, P, I64, P, P, I64, I, P]
    lib.moa_decode_fwd_static.argtypes = decode_args + [I, P]
    lib.moa_rope_qk.argtypes = [P, P, I64, I64, I64, P, P, I64, I64, I, I, I64, I, I, P]
    lib.moa_selftest_bounded_wait.argtypes = [P, I64, P]
    lib.moa_peer_alloc.argtypes = [ctypes.POINTER(c_void_p), I64]
    lib.moa_peer_free.argtypes = [P]
    lib.moa_peer_export.argtypes = [P, P]
    lib.moa_peer_open.argtypes = [P, ctypes.POINTER(c_void_p)]
    lib.moa_peer_close.argtypes = [P]
    lib.moa_peer_barrier.argtypes = [P, I, I, ctypes.c_uint32, P, I64, P, P]
    lib.moa_cache_append.argtypes = [P, P, P, P, I64, I64, P, P, P, P, P, I64, I, I, I, I64, I, P]
    lib.moa_cache_scan_mask.argtypes = [P, I64, P, P, I, I64, P]
    lib.moa_cache_fill.argtypes = [P, P, I64, I64, I64, P, P, P, P, P, P, P, P, P, I64, I, I, I64, I, I64, I64, I, P]
    lib.moa_prefill_fwd.argtypes = [P, P, P, P] + [I64] * 12 + [P, P, I, I, I64, I, c_float, I, I, P, P]
    for name in ("moa_decode_workspace_init", "moa_decode_fwd", "moa_decode_rope_fwd", "moa_decode_gather_fwd",
                 "moa_decode_fwd_static", "moa_rope_qk", "moa_selftest_bounded_wait", "moa_cache_append",
                 "moa_cache_scan_mask", "moa_cache_fill", "moa_prefill_fwd", "moa_peer_alloc", "moa_peer_free",
                 "moa_peer_export", "moa_peer_open", "moa_peer_close", "moa_peer_barrier"):
        getattr(lib, name).restype = c_int
    if lib.moa_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH}: ABI version {lib.moa_abi_version()} != {ABI_VERSION}; rebuild it "
                          "(python moa_b200/build.py --force)")
    return lib


lib = _load()


def check(fn: str, status: int) -> None:
    if status != 0:
        raise MoaError(fn, status, lib.moa_strerror(status).decode(), lib.moa_last_error_detail().decode())


def dtype_code(dtype) -> int:
    import torch

    if dtype == torch.float16:
        return F16
    if dtype == torch.bfloat16:
        return BF16
    raise AssertionError(f"MoA attention supports float16 and bfloat16 only, got {dtype}")


def ptr(t) -> int:
    """data_ptr of a tensor or 0 for None."""
    return 0 if t is None else t.data_ptr()


def rows_ok(t) -> bool:
    """True when the kernels can read ``t`` (..., D) through its strides: last dim contiguous, every
    row 16-byte aligned."""
    return t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:-1])


def decode_arguments(q, k_cache, v_cache, k_new, v_new, out, head_start, valid_len, update_index, mask_cache,
                     static_size, kv_len: int, sm_scale: float):
    """The argument list the decode entry points share (include/moa_b200.h), from tensors.
    ``q``, ``k_new``, ``v_new``: ``(B, H, D)`` views (any strides ``rows_ok`` accepts; ``k_new`` and
    ``v_new`` must share theirs); ``out``: ``(B, H, D)`` view, float32 selects the fp32 store;
    ``k_new``/``v_new``/``update_index``/``mask_cache``/``static_size`` may be None."""
    import torch

    B, H, D = q.shape
    S = k_cache.shape[1]
    assert rows_ok(q) and out.stride(-1) == 1
    if k_new is not None:
        assert rows_ok(k_new) and rows_ok(v_new) and k_new.stride() == v_new.stride()
    out_f32 = out.dtype == torch.float32
    assert out_f32 or out.dtype == q.dtype
    return (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), ptr(k_new), ptr(v_new), out.data_ptr(),
            q.stride(0), q.stride(1), 0 if k_new is None else k_new.stride(0), 0 if k_new is None else k_new.stride(1),
            out.stride(0), out.stride(1), head_start.data_ptr(), valid_len.data_ptr(), ptr(update_index),
            ptr(mask_cache), ptr(static_size), int(kv_len), B, H, D, S, float(sm_scale), dtype_code(q.dtype),
            int(out_f32))


def current_stream(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream


_NVTX = os.environ.get("MOA_B200_NVTX") == "1"


def nvtx_range(name: str):
    """NVTX range around a launch when ``MOA_B200_NVTX=1`` (the reference's efficiency script marks its
    prefill and decode steps the same way, scripts/evaluate/effieicency_test.py:81-83); a no-op otherwise."""
    if _NVTX:
        import torch

        return torch.cuda.nvtx.range(name)
    return contextlib.nullcontext()
