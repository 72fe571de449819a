"""The allocation-free decode entry point (moa_decode_fwd_static) against moa_decode_fwd.

Collected last on purpose: if it fails, a run that stops at the first failure has already run
every other test.  It is for callers that cannot allocate on the decode path (a server whose
KV-cache pool owns all free HBM, a plugin that must not trigger cudaMalloc's device-wide
synchronisation, an FFI binding without an allocator): its scratch is a fixed array inside the
library, shared by all calls, so the test runs two calls in a row with different shapes and checks
each against the entry point that takes a caller-provided workspace and against the CPU oracle
(fp32 attention over the same cache after the same append).
"""
import ctypes

import numpy as np
import pytest
import torch

from moa_b200 import _lib
from oracle import moa_oracle as orc

pytestmark = pytest.mark.gpu
lib = _lib.lib
STATIC_BYTES = 8 * 1024 * 1024


def _inputs(B, caps, Dh, seed, fused):
    gen = torch.Generator().manual_seed(seed)
    H, S = len(caps), sum(caps)
    starts = np.concatenate([[0], np.cumsum(caps)[:-1]])
    t = {
        "q": torch.randn(B, H, Dh, generator=gen).half(),
        "k": torch.randn(B, S, Dh, generator=gen).half(),
        "v": torch.randn(B, S, Dh, generator=gen).half(),
        "hs": torch.tensor(np.tile(starts, (B, 1)), dtype=torch.int64),
        "valid": torch.tensor(np.tile(caps, (B, 1)), dtype=torch.int64),
    }
    if fused:
        t["k_new"] = torch.randn(B, H, Dh, generator=gen).half()
        t["v_new"] = torch.randn(B, H, Dh, generator=gen).half()
        t["upd"] = t["hs"] + 64 + torch.tensor([[(7 * h + b) % (c - 64) for h, c in enumerate(caps)] for b in range(B)])
        t["mask"] = torch.ones(B, S, dtype=torch.int64)
        t["static"] = torch.full((H,), 64, dtype=torch.int64)
    return {k: x.cuda() for k, x in t.items()}


def _call(entry, t, B, caps, Dh, fused, workspace=None):
    H, S = len(caps), sum(caps)
    t = {k: x.clone() for k, x in t.items()}
    out = torch.empty(B, 1, H, Dh, dtype=torch.float16, device="cuda")
    p = lambda name: t[name].data_ptr() if name in t else 0
    args = [p("q"), p("k"), p("v"), p("k_new"), p("v_new"), out.data_ptr(), H * Dh, Dh, H * Dh, Dh,
            out.stride(0), out.stride(2), p("hs"), p("valid"), p("upd"), p("mask"), p("static"), 1000,
            B, H, Dh, S, Dh ** -0.5, 0, 0]
    stream = torch.cuda.current_stream().cuda_stream
    if entry == "static":
        rc = lib.moa_decode_fwd_static(*args, 0, stream)
    else:
        rc = lib.moa_decode_fwd(*args, workspace.data_ptr(), workspace.numel(), 0, stream)
    assert rc == 0, (rc, lib.moa_last_error_detail())
    torch.cuda.synchronize()
    return out, t


def _same(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    assert (a - b).abs().max().item() <= 2e-3
    assert ((a - b).abs().mean() / b.abs().mean()).item() <= 1e-3


def _oracle(t, B, caps, Dh, fused):
    """fp32 attention of the CPU oracle over the cache as it is after the append (rings are full in these
    cases, so the valid lengths do not change and the new row replaces the one at the write index)."""
    k, v = t["k"].cpu().clone(), t["v"].cpu().clone()
    if fused:
        upd = t["upd"].cpu()
        for b in range(B):
            k[b, upd[b]] = t["k_new"][b].cpu()
            v[b, upd[b]] = t["v_new"][b].cpu()
    return orc.decode_attention_fp32(t["q"].cpu()[:, :, None, :], k, v, t["hs"].cpu(), t["valid"].cpu(), Dh ** -0.5)


def test_static_scratch_entry_matches_workspace_entry_on_two_calls_in_a_row():
    cases = [
        (3, [320, 576, 1088, 2112, 128], 128, 11, False),   # attention only
        (2, [4160, 320, 192], 128, 12, True),               # fused append, different shape: the shared
    ]                                                       # array still holds the first call's partials
    for B, caps, Dh, seed, fused in cases:
        t = _inputs(B, caps, Dh, seed, fused)
        need = lib.moa_decode_workspace_bytes(B, len(caps), Dh, sum(caps), 0)
        assert 0 < need <= STATIC_BYTES
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        ref, t_ref = _call("workspace", t, B, caps, Dh, fused, ws)
        got, t_got = _call("static", t, B, caps, Dh, fused)
        _same(got, ref)
        oracle = _oracle(t, B, caps, Dh, fused)
        _same(got, oracle)
        _same(ref, oracle)
        if fused:   # the append and the bookkeeping happened the same way
            for name in ("k", "v", "valid", "upd", "mask"):
                assert torch.equal(t_got[name], t_ref[name]), name
            assert not torch.equal(t_got["k"], t["k"])


def test_static_scratch_entry_refuses_shapes_beyond_its_array():
    B, H, Dh, S = 64, 64, 128, 64 * 16448
    assert lib.moa_decode_workspace_bytes(B, H, Dh, S, 0) > STATIC_BYTES
    one = torch.zeros(8, dtype=torch.int64, device="cuda")
    rc = lib.moa_decode_fwd_static(one.data_ptr(), one.data_ptr(), one.data_ptr(), 0, 0, one.data_ptr(),
                                   H * Dh, Dh, 0, 0, H * Dh, Dh, one.data_ptr(), one.data_ptr(), 0, 0, 0, 0,
                                   B, H, Dh, S, 0.1, 0, 0, 0, 0)
    assert rc == 6
    assert b"use moa_decode_fwd" in lib.moa_last_error_detail()
