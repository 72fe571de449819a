"""``mixture_of_sparse_attention``: the kernel-level entry of the MoA attention path.

Same signature, argument meaning, return layout and assertion behaviour as
MoA/kernels/mixture_of_attention.py:358-487; the work is done by the sm_100a kernels behind
``libmoa_b200.so``.  Only ``implementation="moa"`` exists: the reference's ``"sdpa"`` and
``"flash_attention2"`` values select its debug paths through other libraries, which this package
does not carry, and there is no CPU path.
"""
from __future__ import annotations

import os
import warnings
from typing import Dict, Optional

import torch
from torch import LongTensor, Tensor

from . import _lib
from ._lib import lib

BLOCK_M = 64
BLOCK_N = 64

_workspaces: Dict = {}
_status: Dict = {}


# what the waiting thread was waiting for (the codes the prefill kernel writes to its status words)
_WAIT_NAMES = {1: "Q tiles", 2: "a K tile", 3: "a free K stage", 4: "S from the tensor core", 5: "P from the softmax warps",
               6: "the last but one P.V", 7: "the final O", 8: "a V tile", 9: "a free V stage",
               11: "its turn on the tensor core", 12: "the next unit of work", 13: "a free slot for the next unit",
               14: "the Q tiles to be free"}


def _status_words(device) -> Tensor:
    """The int32[8] status buffer of the prefill kernel (wait report + its scheduler words), one per device and
    stream: launches on different streams may overlap and must not share one."""
    key = (torch.device(device), torch.cuda.current_stream(device).cuda_stream)
    if key not in _status:
        _status[key] = torch.zeros(8, dtype=torch.int32, device=key[0])
    return _status[key]


def check_device_status(device=None) -> None:
    """Synchronise and raise if a kernel on ``device`` reported that one of its bounded waits ran
    out (its output is then invalid).  Cheap enough for tests and once-per-request checks; the
    hot path never synchronises."""
    want = torch.device(device) if device is not None else None
    if want is not None and want.index is None and want.type == "cuda":
        want = torch.device("cuda", torch.cuda.current_device())
    for (dev, _stream), buf in list(_status.items()):
        if want is not None and dev != want:
            continue
        torch.cuda.synchronize(dev)
        words = buf.tolist()
        if words[0] != 0:
            buf.zero_()
            what = _WAIT_NAMES.get(words[0], "?")
            raise _lib.MoaError("moa_prefill_fwd", 5, lib.moa_strerror(5).decode(),
                                f"wait code {words[0]} ({what}) in block {words[1]} thread {words[3]}")


def _decode_workspace(device, B: int, H: int, D: int, S: int) -> Tensor:
    need = lib.moa_decode_workspace_bytes(B, H, D, S, 0)
    key = torch.device(device)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=key)
        _workspaces[key] = ws
    return ws


def sparse_prefill(query: Tensor, key: Tensor, value: Tensor, sm_scale: float, sink_blocks: Tensor,
                   local_blocks: Tensor, out: Optional[Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """Block-sparse causal prefill.  ``query, key, value``: ``(B, H, N, D)`` (any strides with a
    contiguous last dim); ``sink_blocks, local_blocks``: int32 ``(H,)`` device tensors counting
    64-token blocks.  Returns ``(B, N, H, D)``.  ``out_dtype=torch.float32`` stores the fp32
    accumulator (used to check bf16 runs against the oracle at fp16-level tolerance)."""
    B, H, N, D = query.shape
    device = query.device
    code = _lib.dtype_code(query.dtype)
    tensors = []
    for t in (query, key, value):
        if t.stride(-1) != 1 or any(s % 8 for s in t.stride()[:-1]) or t.data_ptr() % 16:
            t = t.contiguous()
        tensors.append(t)
    q, k, v = tensors
    f32 = out_dtype == torch.float32
    if out is None:
        out = torch.empty(B, N, H, D, dtype=torch.float32 if f32 else query.dtype, device=device)
    assert out.shape == (B, N, H, D) and out.stride(-1) == 1
    assert sink_blocks.dtype == torch.int32 and local_blocks.dtype == torch.int32
    assert sink_blocks.numel() == H and local_blocks.numel() == H
    with torch.cuda.device(device), _lib.nvtx_range("moa_b200.prefill"):
        _lib.check("moa_prefill_fwd", lib.moa_prefill_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
            sink_blocks.data_ptr(), local_blocks.data_ptr(), B, H, N, D, float(sm_scale), code, int(f32),
            _status_words(device).data_ptr(), _lib.current_stream(device)))
    if os.environ.get("MOA_B200_CHECK") == "1":
        check_device_status(device)
    return out


def sparse_decode(query: Tensor, key: Tensor, value: Tensor, head_start_index: Tensor, head_valid_length: Tensor,
                  sm_scale: float, out: Optional[Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """Flash-decoding over the flattened per-head caches (no append).  ``query``: ``(B, H, 1, D)``;
    ``key, value``: ``(B, S, D)`` contiguous; ``head_start_index, head_valid_length``: int64
    ``(B, H)``.  Returns ``(B, 1, H, D)``.  ``out_dtype=torch.float32`` stores the fp32 result unrounded
    (used to check bf16 runs against the oracle at fp16-level tolerance)."""
    B, H, _, D = query.shape
    device = query.device
    assert key.dim() == 3 and value.dim() == 3 and key.shape == value.shape
    assert key.is_contiguous() and value.is_contiguous(), "the flattened caches must be contiguous"
    assert head_start_index.shape == (B, H) and head_valid_length.shape == (B, H)
    assert head_start_index.dtype == torch.int64 and head_valid_length.dtype == torch.int64
    S = key.shape[1]
    q = query[:, :, 0, :]
    if not _lib.rows_ok(q):
        q = q.contiguous()
    hs, hv = head_start_index.contiguous(), head_valid_length.contiguous()
    if out is None:
        out = torch.empty(B, 1, H, D, dtype=out_dtype or query.dtype, device=device)
    assert out.shape == (B, 1, H, D)
    ws = _decode_workspace(device, B, H, D, S)
    with torch.cuda.device(device), _lib.nvtx_range("moa_b200.decode"):
        _lib.check("moa_decode_fwd", lib.moa_decode_fwd(
            *_lib.decode_arguments(q, key, value, None, None, out[:, 0], hs, hv, None, None, None, 0, sm_scale),
            ws.data_ptr(), ws.numel(), 0, _lib.current_stream(device)))
    return out


def mixture_of_sparse_attention(
    query: Tensor,
    key: Tensor,
    value: Tensor,
    sm_scale: float,
    attention_mask: LongTensor = None,
    attention_dropout: float = 0.0,
    head_start_index: LongTensor = None,
    head_valid_length: LongTensor = None,
    sink_size: LongTensor = None,
    local_size: LongTensor = None,
    implementation: str = "moa",
):
    """Causal MoA attention, prefill or decode (mixture_of_attention.py:358-487).

    Prefill (``key.shape[-2] == query.shape[-2]``): ``query, key, value`` are ``(B, H, N, D)``;
    ``sink_size`` and ``local_size`` are ``LongTensor[H]`` in **tokens** (block counts are
    ``// 64``, :441-442); without them the mask is dense causal.  Decode: ``query`` is
    ``(B, H, 1, D)``, ``key, value`` are the flattened caches ``(B, sum_h cap_h, D)`` and
    ``head_start_index, head_valid_length`` are ``(B, H)`` int64.  Returns
    ``(B, q_len, H, D)``.  dtype must be float16 or bfloat16 and the head dims must agree
    (``AssertionError`` otherwise, as in the reference)."""
    dtype = query.dtype
    assert (dtype == torch.float16) or (dtype == torch.bfloat16)
    assert query.shape[-1] == key.shape[-1] and key.shape[-1] == value.shape[-1]
    assert key.dtype == dtype and value.dtype == dtype
    if implementation != "moa":
        raise NotImplementedError(
            f"implementation={implementation!r}: moa_b200 only provides the 'moa' kernels "
            "(the reference's 'sdpa'/'flash_attention2' values are debug paths through other libraries)")
    if query.device.type != "cuda":
        raise RuntimeError("moa_b200 runs on CUDA tensors only (there is no CPU path)")
    if attention_dropout:
        raise NotImplementedError("attention dropout is not supported (inference only)")

    is_prefill = not (key.shape[-2] > query.shape[-2])
    if is_prefill:
        assert key.dim() == 4 and value.dim() == 4 and key.shape == query.shape == value.shape
        B, H, N, D = query.shape
        nb = -(-N // BLOCK_N)
        if sink_size is None or local_size is None:
            if N > BLOCK_N:
                warnings.warn("sink_size/local_size not given: running dense causal prefill")
            sink_blocks = torch.zeros(H, dtype=torch.int32, device=query.device)
            local_blocks = torch.full((H,), nb, dtype=torch.int32, device=query.device)
        else:
            sink_blocks = (sink_size // BLOCK_N).to(device=query.device, dtype=torch.int32)
            local_blocks = (local_size // BLOCK_N).to(device=query.device, dtype=torch.int32)
        return sparse_prefill(query, key, value, sm_scale, sink_blocks, local_blocks)

    assert head_start_index is not None and head_valid_length is not None, \
        "decode needs head_start_index and head_valid_length"
    assert query.shape[-2] == 1, "decode takes one query token per sequence"
    return sparse_decode(query, key, value, head_start_index, head_valid_length, sm_scale)
