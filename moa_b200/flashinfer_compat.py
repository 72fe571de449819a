"""The two functions the reference imports from its external CUDA package.

``MoA/kernels/mixture_of_attention.py:22-30`` does ``from flashinfer import moa_prefill, moa_decode`` and
sets ``CUDA_KERNEL_AVAILABLE`` when that import works; the call sites are ``:436-444`` (prefill) and
``:466-473`` (decode).  This module provides the same two names with the same arguments on top of the
C-ABI library, so that putting it on the import path under the name ``flashinfer`` (or changing that one
import) makes the reference's ``implementation="moa"`` branch run on these kernels unchanged.

    import sys, moa_b200.flashinfer_compat as compat
    sys.modules.setdefault("flashinfer", compat)        # before MoA.kernels.mixture_of_attention is imported
"""
from __future__ import annotations

import torch
from torch import Tensor

from .attention import sparse_decode, sparse_prefill

__all__ = ["moa_prefill", "moa_decode"]


def moa_prefill(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, num_global_blocks: Tensor = None,
                num_band_blocks: Tensor = None, kv_layout: str = "HND") -> Tensor:
    """Block-sparse causal prefill as the reference calls it (``mixture_of_attention.py:436-444``).

    ``q``: ``(B, N, H, D)`` (the caller transposes its ``(B, H, N, D)`` query, which gives a strided view;
    no copy is made here); ``k, v``: ``(B, H, N, D)`` (``kv_layout="HND"``); ``num_global_blocks`` and
    ``num_band_blocks``: ``LongTensor[H]``, sink and window sizes in 64-token blocks.  The scale is
    ``D ** -0.5`` (the call has no scale argument).  Returns ``(B, N, H, D)``."""
    if not causal:
        raise NotImplementedError("moa_prefill: only the causal mask exists in the reference's use of this call")
    if kv_layout != "HND":
        raise NotImplementedError("moa_prefill: kv_layout must be 'HND' (k, v as (B, H, N, D))")
    if num_global_blocks is None or num_band_blocks is None:
        raise ValueError("moa_prefill: num_global_blocks and num_band_blocks are required")
    B, N, H, D = q.shape
    if k.shape != (B, H, N, D) or v.shape != (B, H, N, D):
        raise ValueError(f"moa_prefill: k, v must be (B, H, N, D) = {(B, H, N, D)}, got {tuple(k.shape)}, {tuple(v.shape)}")
    sink = num_global_blocks.to(device=q.device, dtype=torch.int32).contiguous()
    band = num_band_blocks.to(device=q.device, dtype=torch.int32).contiguous()
    return sparse_prefill(q.transpose(1, 2), k, v, D ** -0.5, sink, band)


def moa_decode(q: Tensor, k: Tensor, v: Tensor, head_start_index: Tensor, head_valid_length: Tensor,
               sm_scale: float) -> Tensor:
    """Decode attention over the flattened per-head caches as the reference calls it
    (``mixture_of_attention.py:466-473``): ``q`` ``(B, 1, H, D)``; ``k, v`` ``(B, sum of capacities, D)``;
    ``head_start_index, head_valid_length`` ``LongTensor[B, H]``.  Returns ``(B, 1, H, D)``."""
    if q.dim() != 4 or q.shape[1] != 1:
        raise ValueError(f"moa_decode: q must be (B, 1, H, D), got {tuple(q.shape)}")
    return sparse_decode(q.transpose(1, 2), k, v, head_start_index, head_valid_length, float(sm_scale))
