"""Block-sparse prefill kernel (tcgen05/TMEM/TMA) vs the fp32 oracle and the reference fixtures."""
import os

import numpy as np
import pytest
import torch

import moa_b200
from oracle import moa_oracle as orc
import parity

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


# The fp32-store mode of the bf16 kernel: P goes to the tensor core as bf16 (the MMA takes A and B in one
# format only), and its 8-bit mantissa bounds the accuracy whatever the store does: a relative rounding error
# of up to 2^-9 per weight gives about 1.2e-3 - 1.7e-3 mean-rel on N(0,1) data.  Worst measured over these
# tests: max-abs 3.8e-3, mean-rel 1.70e-3 (config 3 at full length: 3.1e-3 / 1.70e-3); the bound is 1.5 x that.
# The bf16 store is checked to be exactly the rounding of the fp32-store result.
BF16_F32_STORE = (5.7e-3, 2.6e-3)


def _close(out, ref, what="", max_abs=parity.MAX_ABS, mean_rel=parity.MEAN_REL):
    parity.check(out, ref, max_abs, mean_rel, f"{what} [{str(out.dtype)[6:]} out]")


def _run(q, k, v, sm, sink_b, local_b, **kw):
    out = moa_b200.sparse_prefill(q.cuda(), k.cuda(), v.cuda(), sm,
                                  torch.as_tensor(sink_b, dtype=torch.int32).cuda(),
                                  torch.as_tensor(local_b, dtype=torch.int32).cuda(), **kw)
    moa_b200.check_device_status()
    return out


def test_reference_triton_fixture_sparse():
    g = np.load(os.path.join(GOLDEN, "prefill_sparse.npz"))
    q, k, v = (torch.from_numpy(g[x]) for x in "qkv")
    out = _run(q, k, v, float(g["sm_scale"]), g["sink_blocks"], g["local_blocks"])
    assert out.shape == (1, 320, 3, 128) and out.is_contiguous()
    _close(out, torch.from_numpy(g["masked_fp32"]), "vs fp32 under the reference-built mask")
    _close(out, torch.from_numpy(g["triton_fp16"]), "vs the reference Triton kernel", 3e-3, 1.5e-3)


def test_reference_triton_fixture_ragged():
    g = np.load(os.path.join(GOLDEN, "prefill_ragged.npz"))
    q, k, v = (torch.from_numpy(g[x]) for x in "qkv")
    out = _run(q, k, v, float(g["sm_scale"]), g["sink_blocks"], g["local_blocks"])
    ref = orc.prefill_attention_fp32(q, k, v, float(g["sm_scale"]), g["sink_blocks"], g["local_blocks"])
    _close(out, ref, "ragged N=200 vs fp32")
    _close(out, torch.from_numpy(g["triton_fp16"]), "ragged vs Triton", 3e-3, 1.5e-3)


def test_reference_own_prefill_test_through_public_entry():
    """tests/attention_kernel_test.py:35-76 of the reference: B2 H4 N128 D128, torch.rand data,
    sm_scale 0.1, sink = local = 64 tokens, compared at rtol = atol = 1e-3."""
    g = np.load(os.path.join(GOLDEN, "prefill_reftest.npz"))
    q, k, v = (torch.from_numpy(g[x]).cuda() for x in "qkv")
    out = moa_b200.mixture_of_sparse_attention(q, k, v, 0.1, attention_dropout=0.0, implementation="moa",
                                               local_size=torch.from_numpy(g["local_size"]).cuda(),
                                               sink_size=torch.from_numpy(g["sink_size"]).cuda())
    moa_b200.check_device_status()
    assert out.shape == (2, 128, 4, 128)
    torch.testing.assert_close(out.cpu(), torch.from_numpy(g["sdpa"]), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(out.cpu(), torch.from_numpy(g["moa"]), rtol=1e-3, atol=1e-3)


CASES = [
    # B, H, N, sink_blocks, local_blocks
    (1, 1, 64, [1], [1]),
    (1, 2, 65, [1, 0], [1, 2]),
    (2, 2, 128, [1, 1], [1, 2]),
    (1, 3, 129, [1, 2, 0], [1, 1, 3]),
    (1, 4, 256, [1, 1, 0, 3], [1, 2, 1, 4]),
    (2, 3, 1000, [1, 1, 2], [2, 5, 40]),
    (1, 4, 2048, [1, 1, 1, 0], [1, 3, 8, 31]),
    (1, 2, 1, [1, 1], [1, 1]),
    (1, 2, 37, [1, 1], [1, 1]),
    # wide sinks: the two tiles of a block take part in different sink blocks near the diagonal
    (1, 3, 1500, [5, 20, 3], [1, 3, 2]),
    (2, 2, 777, [12, 2], [2, 1]),
    # window wider than the sequence: dense causal
    (1, 2, 900, [1, 0], [64, 100]),
    # many heads, short sequence
    (1, 40, 200, [1] * 40, [1 + (i % 4) for i in range(40)]),
]


@pytest.mark.parametrize("case", CASES, ids=[f"B{c[0]}H{c[1]}N{c[2]}" for c in CASES])
def test_fp16_random_against_oracle(case):
    B, H, N, sink_b, local_b = case
    gen = torch.Generator().manual_seed(N * 7 + H)
    q, k, v = (torch.randn(B, H, N, 128, generator=gen).half() for _ in range(3))
    sm = 128 ** -0.5
    out = _run(q, k, v, sm, sink_b, local_b)
    ref = orc.prefill_attention_fp32(q, k, v, sm, sink_b, local_b)
    assert out.shape == (B, N, H, 128)
    _close(out, ref, str(case))


def test_large_scores_force_rescaling():
    """Keys whose scores grow along the sequence make the running max move in every tile."""
    gen = torch.Generator().manual_seed(3)
    B, H, N = 1, 2, 512
    q = torch.randn(B, H, N, 128, generator=gen).half()
    k = (torch.randn(B, H, N, 128, generator=gen) * torch.linspace(0.2, 6.0, N)[None, None, :, None]).half()
    v = torch.randn(B, H, N, 128, generator=gen).half()
    sm = 128 ** -0.5
    out = _run(q, k, v, sm, [1, 1], [8, 2])
    ref = orc.prefill_attention_fp32(q, k, v, sm, [1, 1], [8, 2])
    _close(out, ref, "rescale", 3e-3, 1.5e-3)


def test_strided_inputs_as_the_projection_produces_them():
    gen = torch.Generator().manual_seed(8)
    B, H, N = 2, 3, 300
    # (B, N, H, D) storage viewed as (B, H, N, D): modeling_llama.py:238-240 of the reference
    q, k, v = (torch.randn(B, N, H, 128, generator=gen).half().cuda().transpose(1, 2) for _ in range(3))
    assert not q.is_contiguous()
    sm = 128 ** -0.5
    out = moa_b200.sparse_prefill(q, k, v, sm, torch.tensor([1, 1, 1], dtype=torch.int32).cuda(),
                                  torch.tensor([1, 2, 3], dtype=torch.int32).cuda())
    moa_b200.check_device_status()
    ref = orc.prefill_attention_fp32(q.cpu(), k.cpu(), v.cpu(), sm, [1, 1, 1], [1, 2, 3])
    _close(out, ref, "strided")


def test_bf16_fp32_store_meets_the_tolerance_and_bf16_store_is_its_rounding():
    gen = torch.Generator().manual_seed(12)
    B, H, N = 1, 3, 700
    q, k, v = (torch.randn(B, H, N, 128, generator=gen).bfloat16() for _ in range(3))
    sm = 128 ** -0.5
    sink_b, local_b = [1, 1, 1], [2, 4, 11]
    ref = orc.prefill_attention_fp32(q, k, v, sm, sink_b, local_b)
    out32 = _run(q, k, v, sm, sink_b, local_b, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    # identical math with the accumulator stored unrounded; the bf16 output is exactly the rounding of this
    # result and therefore within half a bf16 ulp of it
    _close(out32, ref, "bf16 inputs, fp32 store", *BF16_F32_STORE)
    out16 = _run(q, k, v, sm, sink_b, local_b)
    assert out16.dtype == torch.bfloat16
    assert torch.equal(out16.cpu(), out32.cpu().bfloat16())
    _close(out16, ref, "bf16 inputs, bf16 store", 1e-2, 3.1e-3)      # measured 6.4e-3 / 2.1e-3


def test_config0_full_size():
    """Config 0 of BASELINE.json: B1 H32 N2048 D128 fp16, 64 sinks, span alpha+beta*N per head."""
    rng = np.random.RandomState(0)
    H, N = 32, 2048
    plan = {"alphas": [[float(rng.choice([128, 256, 512, 1024])) for _ in range(H)]],
            "betas": [[float(rng.uniform(0, 0.5)) for _ in range(H)]]}
    cfg = moa_b200.moa_config_to_cache_config(plan, N, 0, verbose=False)
    caps, static = cfg["cache_size"][0], cfg["static_size"][0]
    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, H, N, 128, generator=gen).half().cuda() for _ in range(3))
    sink = torch.tensor(static, dtype=torch.int64).cuda()
    local = torch.tensor([c - s for c, s in zip(caps, static)], dtype=torch.int64).cuda()
    out = moa_b200.mixture_of_sparse_attention(q, k, v, 128 ** -0.5, sink_size=sink, local_size=local)
    moa_b200.check_device_status()
    ref = orc.prefill_attention_fp32(q.cpu(), k.cpu(), v.cpu(), 128 ** -0.5, [s // 64 for s in static],
                                     [(c - s) // 64 for c, s in zip(caps, static)])
    _close(out, ref, "config 0")


def test_long_sequence_spot_rows():
    """N = 16384: rows from the start, the middle and the end are checked against the oracle."""
    gen = torch.Generator().manual_seed(21)
    B, H, N = 1, 4, 16384
    q, k, v = (torch.randn(B, H, N, 128, generator=gen).half() for _ in range(3))
    sm = 128 ** -0.5
    sink_b, local_b = [1, 1, 1, 1], [8, 33, 64, 250]
    out = _run(q, k, v, sm, sink_b, local_b)
    for a, b in [(0, 256), (8000, 8256), (N - 256, N)]:
        ref = orc.prefill_attention_fp32(q, k, v, sm, sink_b, local_b, row_range=(a, b))
        _close(out[:, a:b], ref, f"rows {a}:{b}")


def test_many_heads_all_sms_busy_with_spot_rows():
    """32 heads x 8192 tokens, bf16, plans as in config 3: every SM runs several blocks back to back and K/V
    come from L2 and HBM at once, so the TMA rings run dry now and then and the issuers fall behind the
    softmax warps — the situation in which hand-off barriers that count phases wrongly would stall.
    Rows from three places are checked against the oracle."""
    rng = np.random.RandomState(3000)
    B, H, N, D = 1, 32, 8192, 128
    plan = {"alphas": [[float(rng.choice([512, 1024, 2048, 4096])) for _ in range(H)]],
            "betas": [[float(rng.uniform(0, 0.3)) for _ in range(H)]]}
    cfg = moa_b200.moa_config_to_cache_config(plan, N, 0, verbose=False)
    sink_b = [s // 64 for s in cfg["static_size"][0]]
    local_b = [(c - s) // 64 for c, s in zip(cfg["cache_size"][0], cfg["static_size"][0])]
    gen = torch.Generator(device="cuda").manual_seed(5)
    q, k, v = (torch.randn(B, H, N, D, generator=gen, device="cuda").bfloat16() for _ in range(3))
    sb, lb = (torch.tensor(x, dtype=torch.int32).cuda() for x in (sink_b, local_b))
    sm = D ** -0.5
    for _ in range(3):      # repeated launches: the rings see different timing each time
        out = moa_b200.sparse_prefill(q, k, v, sm, sb, lb, out_dtype=torch.float32)
        moa_b200.check_device_status()
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    for a, b in [(0, 128), (4000, 4128), (N - 128, N)]:
        ref = orc.prefill_attention_fp32(qc, kc, vc, sm, sink_b, local_b, row_range=(a, b))
        _close(out[:, a:b], ref, f"32 heads x 8192 bf16, fp32 store, rows {a}:{b}", *BF16_F32_STORE)


def test_constant_value_property_full_length():
    """V constant per dim => output equals it for every row, whatever the mask keeps (N = 65536)."""
    gen = torch.Generator(device="cuda").manual_seed(2)
    B, H, N = 1, 2, 65536
    q = torch.randn(B, H, N, 128, generator=gen, device="cuda").bfloat16()
    k = torch.randn(B, H, N, 128, generator=gen, device="cuda").bfloat16()
    const = torch.linspace(-1, 1, 128, device="cuda").bfloat16()
    v = const[None, None, None, :].expand(B, H, N, 128).contiguous()
    out = moa_b200.sparse_prefill(q, k, v, 128 ** -0.5, torch.tensor([1, 1], dtype=torch.int32).cuda(),
                                  torch.tensor([16, 64], dtype=torch.int32).cuda(), out_dtype=torch.float32)
    moa_b200.check_device_status()
    assert (out - const.float()[None, None, None]).abs().max() < 5e-3


def test_config3_full_length_spot_rows():
    """Config 3 of BASELINE.json at full length (N = 65536, bf16, head_dim 128) with four heads of the plan the
    benchmark draws (the narrowest and the widest window among them): 3 x 128 query rows from the start, the
    middle and the end of the sequence against the fp32 oracle in the fp32-store mode, and the bf16 output as
    exactly the rounding of that result."""
    rng = np.random.RandomState(3000)
    Hp, N, D = 32, 65536, 128
    plan = {"alphas": [[float(rng.choice([512, 1024, 2048, 4096])) for _ in range(Hp)]],
            "betas": [[float(rng.uniform(0, 0.3)) for _ in range(Hp)]]}
    cfg = moa_b200.moa_config_to_cache_config(plan, N, 0, verbose=False)
    local_all = [(c - s) // 64 for c, s in zip(cfg["cache_size"][0], cfg["static_size"][0])]
    order = sorted(range(Hp), key=lambda h: local_all[h])
    heads = [order[0], order[Hp // 3], order[2 * Hp // 3], order[-1]]
    sink_b, local_b = [1] * 4, [local_all[h] for h in heads]
    gen = torch.Generator(device="cuda").manual_seed(3001)
    q, k, v = (torch.randn(1, 4, N, D, generator=gen, device="cuda").bfloat16() for _ in range(3))
    sb, lb = (torch.tensor(x, dtype=torch.int32).cuda() for x in (sink_b, local_b))
    sm = D ** -0.5
    out32 = moa_b200.sparse_prefill(q, k, v, sm, sb, lb, out_dtype=torch.float32)
    out16 = moa_b200.sparse_prefill(q, k, v, sm, sb, lb)
    moa_b200.check_device_status()
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    for a, b in [(0, 128), (32768 - 64, 32768 + 64), (N - 128, N)]:
        ref = orc.prefill_attention_fp32(qc, kc, vc, sm, sink_b, local_b, row_range=(a, b))
        _close(out32[:, a:b], ref, f"config 3 full length, local blocks {local_b}, rows {a}:{b}", *BF16_F32_STORE)
        assert torch.equal(out16[:, a:b].cpu(), out32[:, a:b].cpu().bfloat16())


def test_heads_that_see_nothing_give_zero_rows():
    """No sink block and no window block (a local size below one block): nothing is visible, rows are zero."""
    gen = torch.Generator().manual_seed(8)
    q, k, v = (torch.randn(1, 2, 300, 128, generator=gen).half() for _ in range(3))
    out = torch.full((1, 300, 2, 128), float("nan"), dtype=torch.float16, device="cuda")
    moa_b200.sparse_prefill(q.cuda(), k.cuda(), v.cuda(), 0.1, torch.tensor([0, 1], dtype=torch.int32).cuda(),
                            torch.tensor([0, 2], dtype=torch.int32).cuda(), out=out)
    moa_b200.check_device_status()
    assert torch.isfinite(out).all() and out[:, :, 0].abs().sum() == 0
    _close(out, orc.prefill_attention_fp32(q, k, v, 0.1, [0, 1], [0, 2]), "head 0 sees nothing")


@pytest.mark.parametrize("B,H,N", [(2, 3, 513), (1, 3, 17), (1, 41, 2061)])
def test_super_tiles_that_visit_no_block_load_nothing(B, H, N):
    """At most 64 rows in the last super-tile, under a head without sink and window: that super-tile visits no KV
    block at all, so nobody waits for its Q.  The kernel must not load it (a copy in flight when the block ends,
    or, in the persistent form, the Q barrier armed twice in one phase).  2061 tokens of 41 heads are 369 units:
    the persistent form.  Launched repeatedly; rows of the blind heads are zero, the rest matches the oracle."""
    gen = torch.Generator().manual_seed(N)
    q, k, v = (torch.randn(B, H, N, 128, generator=gen).half() for _ in range(3))
    sink_b = [(0, 1, 0)[h % 3] for h in range(H)]
    local_b = [(0, 3, 0)[h % 3] if h % 6 else 7 for h in range(H)]
    sm = 128 ** -0.5
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    sb, lb = (torch.tensor(x, dtype=torch.int32).cuda() for x in (sink_b, local_b))
    outs = [moa_b200.sparse_prefill(qd, kd, vd, sm, sb, lb) for _ in range(25)]
    moa_b200.check_device_status()
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    blind = [h for h in range(H) if sink_b[h] == 0 and local_b[h] == 0]
    assert blind and outs[0][:, :, blind].abs().sum() == 0
    _close(outs[0], orc.prefill_attention_fp32(q, k, v, sm, sink_b, local_b), f"blind heads at a ragged end, N={N}")


def test_short_prompt_without_sizes_is_dense_causal():
    gen = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 2, 40, 128, generator=gen).half() for _ in range(3))
    out = moa_b200.mixture_of_sparse_attention(q.cuda(), k.cuda(), v.cuda(), 0.1)
    moa_b200.check_device_status()
    ref = orc.prefill_attention_fp32(q, k, v, 0.1, [0, 0], [1, 1])
    _close(out, ref, "dense causal N=40")


def test_a_wait_that_runs_out_is_reported_and_leaves_the_context_usable():
    """Failure detection without a fault: a bounded wait on a barrier nobody signals gives up after its
    limit, the status words carry the code, check_device_status raises, and the next launch works."""
    from moa_b200 import _lib
    from moa_b200.attention import _status_words
    st = _status_words("cuda:0")
    st.zero_()
    rc = _lib.lib.moa_selftest_bounded_wait(st.data_ptr(), 20_000_000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    with pytest.raises(moa_b200.MoaError, match="wait"):
        moa_b200.check_device_status("cuda:0")
    assert st.tolist() == [0] * 8                 # cleared by the check
    gen = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 1, 128, 128, generator=gen).half() for _ in range(3))
    out = _run(q, k, v, 0.1, [1], [1])            # the context is alive and the kernel still right
    _close(out, orc.prefill_attention_fp32(q, k, v, 0.1, [1], [1]), "after the timed-out wait")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_64(dtype):
    """Llama-3.2-1B has 64-wide heads (one of the reference's example plans)."""
    gen = torch.Generator().manual_seed(64)
    B, H, N = 2, 3, 700
    q, k, v = (torch.randn(B, H, N, 64, generator=gen).to(dtype) for _ in range(3))
    sm = 64 ** -0.5
    sink_b, local_b = [1, 1, 2], [1, 4, 9]
    ref = orc.prefill_attention_fp32(q, k, v, sm, sink_b, local_b)
    if dtype == torch.float16:
        out = _run(q, k, v, sm, sink_b, local_b)
        assert out.shape == (B, N, H, 64)
        _close(out, ref, "D=64 fp16")
    else:
        out32 = _run(q, k, v, sm, sink_b, local_b, out_dtype=torch.float32)
        _close(out32, ref, "D=64 bf16, fp32 store", *BF16_F32_STORE)
        out16 = _run(q, k, v, sm, sink_b, local_b)
        assert torch.equal(out16.cpu(), out32.cpu().bfloat16())


@pytest.mark.parametrize("N", [200, 321, 1000])
def test_poisoned_rows_past_the_sequence_and_guard_rows(N):
    """q, k, v are the first N rows of longer buffers whose remaining rows hold NaN (a kernel that reads past
    the sequence end poisons its output: the TMA boxes of the last tile reach beyond N), and the output is a
    window of a larger buffer whose rows before and after must keep their marker."""
    gen = torch.Generator().manual_seed(N)
    B, H, D, pad = 1, 3, 128, 130
    sink_b, local_b = [1, 1, 2], [2, 5, 3]
    big = [torch.randn(B, H, N + pad, D, generator=gen).half() for _ in range(3)]
    for t in big:
        t[:, :, N:] = float("nan")
    q, k, v = (t[:, :, :N] for t in big)
    ref = orc.prefill_attention_fp32(q, k, v, D ** -0.5, sink_b, local_b)
    marker = 321.0
    outbuf = torch.full((B, N + 2 * 64, H, D), marker, dtype=torch.float16, device="cuda")
    out = outbuf[:, 64:64 + N]
    qc, kc, vc = (t.cuda()[:, :, :N] for t in big)
    assert not qc.is_contiguous()
    moa_b200.sparse_prefill(qc, kc, vc, D ** -0.5, torch.tensor(sink_b, dtype=torch.int32).cuda(),
                            torch.tensor(local_b, dtype=torch.int32).cuda(), out=out)
    moa_b200.check_device_status()
    assert torch.isfinite(out.float()).all(), "rows past the sequence end were read"
    _close(out, ref, f"poisoned tail, N={N}")
    assert (outbuf[:, :64] == marker).all() and (outbuf[:, 64 + N:] == marker).all(), "rows outside the output were written"


def test_persistent_form_ragged_many_units_against_oracle():
    """480 units on 148 SMs: the launcher picks the persistent form (blocks take unit after unit from the counter).
    Ragged length (the last super-tile has one tile of 88 rows), two batch rows, 80 heads whose plans cycle through
    wide, narrow, sink-less and all-invisible spans: every role sees units with nothing to do next to full ones.
    Whole output against the fp32 oracle; a second launch on the same buffers must give the same bits (the
    scheduler words were put back to zero)."""
    gen = torch.Generator().manual_seed(77)
    B, H, N = 2, 80, 600
    sink_b = [(1, 1, 0, 2, 0)[h % 5] for h in range(H)]
    local_b = [(10, 1, 3, 2, 0)[h % 5] for h in range(H)]
    q, k, v = (torch.randn(B, H, N, 128, generator=gen).half() for _ in range(3))
    sm = 128 ** -0.5
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    sb, lb = (torch.tensor(x, dtype=torch.int32).cuda() for x in (sink_b, local_b))
    out = moa_b200.sparse_prefill(qd, kd, vd, sm, sb, lb)
    again = moa_b200.sparse_prefill(qd, kd, vd, sm, sb, lb)
    moa_b200.check_device_status()
    assert torch.equal(out, again)
    _close(out, orc.prefill_attention_fp32(q, k, v, sm, sink_b, local_b), "persistent form, ragged, 480 units")
    from moa_b200.attention import _status_words
    assert _status_words("cuda:0").tolist() == [0] * 8


def test_prefill_launches_on_two_streams_do_not_share_scheduler_state():
    """Two persistent-form launches that overlap in time (two streams) each own a status buffer; results equal the
    launches run one after the other."""
    gen = torch.Generator(device="cuda").manual_seed(78)
    shapes = [(1, 48, 2048), (1, 40, 2304)]
    data = []
    for B, H, N in shapes:
        q, k, v = (torch.randn(B, H, N, 128, generator=gen, device="cuda").half() for _ in range(3))
        sb = torch.ones(H, dtype=torch.int32, device="cuda")
        lb = torch.tensor([1 + (3 * h) % 20 for h in range(H)], dtype=torch.int32, device="cuda")
        data.append((q, k, v, sb, lb))
    want = [moa_b200.sparse_prefill(q, k, v, 0.09, sb, lb) for q, k, v, sb, lb in data]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for rnd in range(3):
        got = []
        for s, (q, k, v, sb, lb) in zip(streams, data):
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                got.append(moa_b200.sparse_prefill(q, k, v, 0.09, sb, lb))
        for s in streams:
            torch.cuda.current_stream().wait_stream(s)
        moa_b200.check_device_status()
        for g, w in zip(got, want):
            assert torch.equal(g, w)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_64_persistent_form(dtype):
    """64-wide heads with enough units (384 on 148 SMs) for the launcher to pick the persistent form."""
    gen = torch.Generator().manual_seed(640)
    B, H, N = 2, 64, 700
    q, k, v = (torch.randn(B, H, N, 64, generator=gen).to(dtype) for _ in range(3))
    sm = 64 ** -0.5
    sink_b = [(1, 0, 2)[h % 3] for h in range(H)]
    local_b = [1 + (5 * h) % 11 for h in range(H)]
    ref = orc.prefill_attention_fp32(q, k, v, sm, sink_b, local_b)
    if dtype == torch.float16:
        _close(_run(q, k, v, sm, sink_b, local_b), ref, "D=64 fp16, persistent form")
    else:
        out32 = _run(q, k, v, sm, sink_b, local_b, out_dtype=torch.float32)
        _close(out32, ref, "D=64 bf16, fp32 store, persistent form", *BF16_F32_STORE)
        assert torch.equal(_run(q, k, v, sm, sink_b, local_b).cpu(), out32.cpu().bfloat16())
