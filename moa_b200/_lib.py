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
#: the library next to this file; MOA_B200_LIB points at another build of it (kernel development)
LIB_PATH = os.environ.get("MOA_B200_LIB") or os.path.join(HERE, "libmoa_b200.so")

F16, BF16 = 0, 1

#: every symbol include/moa_b200.h declares
SYMBOLS = (
    "moa_abi_version", "moa_strerror", "moa_last_error_detail",
    "moa_decode_workspace_bytes", "moa_decode_workspace_init", "moa_decode_fwd",
    "moa_cache_append", "moa_cache_scan_mask", "moa_cache_fill", "moa_prefill_fwd",
    "moa_decode_fwd_static", "moa_decode_rope_fwd", "moa_selftest_bounded_wait", "moa_rope_qk",
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
    lib.moa_decode_fwd.argtypes = [P, P, P, P, P, P, I64, I64, P, P, P, P, P, I64, I, I, I, I64, c_float, I, P, I64, I, P]
    lib.moa_decode_rope_fwd.argtypes = [P, P, P, P, P, P, P, P, I64, I64, P, P, P, P, P, I64, I, I, I, I64, c_float, I, P, I64, I, P]
    lib.moa_decode_rope_fwd.restype = c_int
    lib.moa_rope_qk.argtypes = [P, P, I64, I64, I64, P, P, I64, I64, I, I, I64, I, I, P]
    lib.moa_rope_qk.restype = c_int
    lib.moa_selftest_bounded_wait.argtypes = [P, I64, P]
    lib.moa_selftest_bounded_wait.restype = c_int
    lib.moa_decode_fwd_static.argtypes = [P, P, P, P, P, P, I64, I64, P, P, P, P, P, I64, I, I, I, I64, c_float, I, I, P]
    lib.moa_decode_fwd_static.restype = c_int
    lib.moa_cache_append.argtypes = [P, P, P, P, I64, I64, P, P, P, P, P, I64, I, I, I, I64, I, P]
    lib.moa_cache_scan_mask.argtypes = [P, I64, P, P, I, I64, P]
    lib.moa_cache_fill.argtypes = [P, P, I64, I64, I64, P, P, P, P, P, P, P, P, P, I64, I, I, I64, I, I64, I64, I, P]
    lib.moa_prefill_fwd.argtypes = [P, P, P, P] + [I64] * 12 + [P, P, I, I, I64, I, c_float, I, I, P, P]
    for name in ("moa_decode_workspace_init", "moa_decode_fwd", "moa_cache_append", "moa_cache_scan_mask",
                 "moa_cache_fill", "moa_prefill_fwd"):
        getattr(lib, name).restype = c_int
    if lib.moa_abi_version() != 1:
        raise ImportError(f"{LIB_PATH}: ABI version {lib.moa_abi_version()} != 1; rebuild it")
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
