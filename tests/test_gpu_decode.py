"""Flash-decoding kernel vs the fp32 oracle, through the public API and the raw C ABI."""
import os

import numpy as np
import pytest
import torch

import moa_b200
from moa_b200 import _lib
from oracle import moa_oracle as orc
import parity

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")

# fp16 results and the fp32-store mode of the bf16 kernel are held to the tolerance the project states
# (max-abs 2e-3, mean-rel 1e-3 against fp32); measured: fp16 about 1.2e-4 / 1.8e-4, bf16 with fp32 store
# about 5e-7 / 5e-7.  A bf16 *store* alone costs up to half a bf16 ulp (3.9e-3 at |x| in [1, 2), about
# 1.4e-3 mean-rel), so bf16 outputs are checked two ways: they must be exactly the rounding of the fp32-store
# result, and against the oracle they get 1.5 x the worst error measured over these tests (5.8e-3 / 1.5e-3).
TOL = {torch.float16: (parity.MAX_ABS, parity.MEAN_REL), torch.bfloat16: (9e-3, 2.3e-3)}


def _close(out, ref, dtype, what=""):
    a, r = TOL[dtype] if out.dtype != torch.float32 else (parity.MAX_ABS, parity.MEAN_REL)
    parity.check(out, ref, a, r, f"{what} [{str(dtype)[6:]} in, {str(out.dtype)[6:]} out]")


def _random_cache(B, caps, Dh, dtype, gen, full=False):
    S = sum(caps)
    k = torch.randn(B, S, Dh, generator=gen).to(dtype)
    v = torch.randn(B, S, Dh, generator=gen).to(dtype)
    starts = np.concatenate([[0], np.cumsum(caps)[:-1]])
    hs = torch.tensor(np.tile(starts, (B, 1)), dtype=torch.int64)
    if full:
        valid = torch.tensor(np.tile(caps, (B, 1)), dtype=torch.int64)
    else:
        valid = torch.stack([torch.tensor([int(torch.randint(0, c + 1, (1,), generator=gen)) for c in caps])
                             for _ in range(B)]).to(torch.int64)
        valid[0, 0] = caps[0]
        if B > 1:
            valid[1, -1] = 0
    return k, v, hs, valid


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Dh", [128, 64])
@pytest.mark.parametrize("caps", [[128, 128, 256, 320], [5, 10, 333, 100, 7], [4160, 320, 2112], [64] * 9])
def test_sparse_decode_matches_oracle(dtype, Dh, caps):
    gen = torch.Generator().manual_seed(hash((Dh, len(caps))) % 1000)
    B = 3
    k, v, hs, valid = _random_cache(B, caps, Dh, dtype, gen)
    q = torch.randn(B, len(caps), 1, Dh, generator=gen).to(dtype)
    sm = Dh ** -0.5
    ref = orc.decode_attention_fp32(q, k, v, hs, valid, sm)
    out = moa_b200.mixture_of_sparse_attention(q.cuda(), k.cuda(), v.cuda(), sm, head_start_index=hs.cuda(),
                                               head_valid_length=valid.cuda())
    assert out.shape == (B, 1, len(caps), Dh) and out.dtype == dtype
    _close(out, ref, dtype, f"caps={caps}")
    # heads with nothing valid give zeros, not NaN
    assert torch.isfinite(out.float()).all()
    # fp32-store mode: same math, unrounded result, held to the stated tolerance for both dtypes;
    # the 16-bit output is exactly its rounding
    out32 = moa_b200.sparse_decode(q.cuda(), k.cuda(), v.cuda(), hs.cuda(), valid.cuda(), sm, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    _close(out32, ref, dtype, f"caps={caps}")
    assert torch.equal(out32.to(dtype), out)


@pytest.mark.parametrize("chunk", [64, 96, 128, 256, 1000, 100000])
def test_every_chunk_size_gives_the_same_answer(chunk):
    """The split size only changes how partial sums are grouped; results agree to fp32 rounding."""
    gen = torch.Generator().manual_seed(9)
    caps, B, Dh, dtype = [320, 576, 1088, 128, 2112], 2, 128, torch.float16
    k, v, hs, valid = _random_cache(B, caps, Dh, dtype, gen)
    q = torch.randn(B, len(caps), 1, Dh, generator=gen).to(dtype)
    ref = orc.decode_attention_fp32(q, k, v, hs, valid, 0.09)
    qd, kd, vd, hsd, vald = q.cuda(), k.cuda(), v.cuda(), hs.cuda(), valid.cuda()
    H, S = len(caps), sum(caps)
    need = _lib.lib.moa_decode_workspace_bytes(B, H, Dh, S, chunk)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    out = torch.empty(B, 1, H, Dh, dtype=dtype, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):  # second call reuses the workspace (tickets reset themselves)
        rc = _lib.lib.moa_decode_fwd(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), 0, 0, out.data_ptr(), H * Dh, Dh, 0, 0,
                                     out.stride(0), out.stride(2), hsd.data_ptr(), vald.data_ptr(), 0, 0, 0, 0,
                                     B, H, Dh, S, 0.09, 0, 0, ws.data_ptr(), need, chunk, stream)
        assert rc == 0, _lib.lib.moa_last_error_detail()
        _close(out, ref, dtype, f"chunk={chunk}")
    # too small a workspace is refused, not overrun
    rc = _lib.lib.moa_decode_fwd(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), 0, 0, out.data_ptr(), H * Dh, Dh, 0, 0,
                                 out.stride(0), out.stride(2), hsd.data_ptr(), vald.data_ptr(), 0, 0, 0, 0,
                                 B, H, Dh, S, 0.09, 0, 0, ws.data_ptr(), need - 1, chunk, stream)
    assert rc == 4


def test_reference_sdpa_decode_fixture():
    """Prefill 400 tokens, three decode steps; outputs recorded from the reference's "sdpa" path."""
    g = np.load(os.path.join(GOLDEN, "decode_sdpa.npz"))
    caps = g["caps"].tolist()
    B, H, Dh = 2, len(caps), 128
    cache = moa_b200.StaticCircularCache([caps], B, Dh, [[64] * H], "cuda", torch.float16)
    cache.update(torch.from_numpy(g["k_prefill"]).cuda(), torch.from_numpy(g["v_prefill"]).cuda(), 0)
    sm = float(g["sm_scale"])
    for s in range(g["q"].shape[0]):
        q = torch.from_numpy(g["q"][s]).cuda()
        kc, vc = cache.update(torch.from_numpy(g["k_new"][s]).cuda(), torch.from_numpy(g["v_new"][s]).cuda(), 0)
        out = moa_b200.mixture_of_sparse_attention(q, kc, vc, sm, head_start_index=cache.cache_head_start_index[0],
                                                   head_valid_length=cache.cache_valid_length[0])
        _close(out, torch.from_numpy(g["out"][s]), torch.float16, f"step {s}")
    assert np.array_equal(cache.key_cache[0].cpu().numpy(), g["key_cache_final"])
    assert np.array_equal(cache.cache_update_index[0].cpu().numpy(), g["update_index_final"])


def test_out_may_be_a_slice_of_a_gather_buffer():
    gen = torch.Generator().manual_seed(2)
    caps, B, Dh = [128, 256], 2, 128
    cache = moa_b200.StaticCircularCache([caps], B, Dh, [[64, 64]], "cuda", torch.float16)
    kp = torch.randn(B, 2, 300, Dh, generator=gen).half().cuda()
    cache.update(kp, kp, 0)
    q, k1, v1 = (torch.randn(B, 2, 1, Dh, generator=gen).half().cuda() for _ in range(3))
    gather = torch.zeros(B, 1, 6, Dh, dtype=torch.float16, device="cuda")
    state = (cache.cache_update_index[0].clone(), cache.cache_valid_length[0].clone(), cache.key_cache[0].clone(),
             cache.value_cache[0].clone(), cache.mask_cache[0].clone(), cache._kv_len[0])
    ref = cache.decode_attention(q, k1, v1, 0, 0.1)
    cache.cache_update_index[0].copy_(state[0]); cache.cache_valid_length[0].copy_(state[1])
    cache.key_cache[0].copy_(state[2]); cache.value_cache[0].copy_(state[3]); cache.mask_cache[0].copy_(state[4])
    cache._kv_len[0] = state[5]
    cache.decode_attention(q, k1, v1, 0, 0.1, out=gather[:, :, 2:4])
    assert torch.equal(gather[:, :, 2:4], ref)
    assert gather[:, :, :2].abs().sum() == 0 and gather[:, :, 4:].abs().sum() == 0


def test_config1_rings_wrap_and_match_oracle():
    """Config 1 of BASELINE.json at reduced batch: 32 heads, windows from {256..4096} + 64 sinks, caches
    filled from a 16k-token stream, 256 fused decode steps; every ring crosses its end at step 64."""
    gen = torch.Generator().manual_seed(1001)
    B, H, Dh, N, steps = 2, 32, 128, 16384, 256
    W = sorted(int(w) for w in np.random.RandomState(1).choice([256, 512, 1024, 2048, 4096], H))
    caps = [64 + w for w in W]
    o = orc.RingCacheOracle([caps], [[64] * H], B, Dh, dtype=np.float16)
    c = moa_b200.StaticCircularCache([caps], B, Dh, [[64] * H], "cuda", torch.float16)
    k = torch.randn(B, H, N, Dh, generator=gen).half()
    v = torch.randn(B, H, N, Dh, generator=gen).half()
    o.update(k.numpy(), v.numpy(), 0)
    c.update(k.cuda(), v.cuda(), 0)
    assert np.array_equal(c.key_cache[0].cpu().numpy(), o.key_cache[0])
    starts = o.head_index[0][:-1]
    assert np.array_equal(o.cache_update_index[0][0] - starts - 64, np.asarray(W) - 64)
    sm = Dh ** -0.5
    crossings = np.zeros(H, dtype=np.int64)
    check_at = {0, 1, 63, 64, 65, 128, 255}
    for step in range(steps):
        q, k1, v1 = (torch.randn(B, H, 1, Dh, generator=gen).half() for _ in range(3))
        before = o.cache_update_index[0][0].copy()
        kc, vc = o.update(k1.numpy(), v1.numpy(), 0)
        crossings += (o.cache_update_index[0][0] < before)
        out = c.decode_attention(q.cuda(), k1.cuda(), v1.cuda(), 0, sm)
        if step in check_at:
            ref = orc.decode_attention_fp32(q, torch.from_numpy(kc), torch.from_numpy(vc),
                                            torch.from_numpy(o.cache_head_start_index[0]),
                                            torch.from_numpy(o.cache_valid_length[0]), sm)
            _close(out, ref, torch.float16, f"step {step}")
            assert np.array_equal(c.cache_update_index[0].cpu().numpy(), o.cache_update_index[0])
    assert (crossings == 1).all()
    assert np.array_equal(c.key_cache[0].cpu().numpy(), o.key_cache[0])
    assert np.array_equal(c.value_cache[0].cpu().numpy(), o.value_cache[0])
    assert np.array_equal(c.cache_valid_length[0].cpu().numpy(), o.cache_valid_length[0])


def test_full_size_config1_properties():
    """Batch 16 x 32 heads at full capacities (445 MB of K/V): size-independent checks.
    (1) V == per-dim constant  =>  output == that constant (weights sum to one);
    (2) every head with a one-hot q.k winner returns that slot's V row."""
    B, H, Dh = 16, 32, 128
    W = sorted(int(w) for w in np.random.RandomState(1).choice([256, 512, 1024, 2048, 4096], H))
    caps = [64 + w for w in W]
    S = sum(caps)
    gen = torch.Generator(device="cuda").manual_seed(4)
    k = torch.randn(B, S, Dh, generator=gen, device="cuda").half()
    const = torch.linspace(-2, 2, Dh, device="cuda").half()
    v = const[None, None, :].expand(B, S, Dh).contiguous()
    starts = torch.tensor(np.concatenate([[0], np.cumsum(caps)[:-1]]), device="cuda")
    hs = starts[None].expand(B, H).contiguous()
    valid = torch.tensor(caps, device="cuda")[None].expand(B, H).contiguous()
    q = torch.randn(B, H, 1, Dh, generator=gen, device="cuda").half()
    out = moa_b200.mixture_of_sparse_attention(q, k, v, Dh ** -0.5, head_start_index=hs, head_valid_length=valid)
    assert (out.float() - const.float()[None, None, None]).abs().max() < 2e-3
    # one-hot winner: slot w of each head has key == 30*q/|q|^2-ish, the others ~0
    k2 = torch.zeros(B, S, Dh, device="cuda", dtype=torch.float16)
    v2 = torch.randn(B, S, Dh, generator=gen, device="cuda").half()
    win = (starts + torch.tensor([c // 3 for c in caps], device="cuda"))
    qn = q[:, :, 0] / (q[:, :, 0].float().pow(2).sum(-1, keepdim=True)).half()
    bidx = torch.arange(B, device="cuda")[:, None].expand(B, H)
    k2[bidx, win[None].expand(B, H)] = (qn.float() * 400).half()
    out2 = moa_b200.mixture_of_sparse_attention(q, k2, v2, 1.0, head_start_index=hs, head_valid_length=valid)
    want = v2[bidx, win[None].expand(B, H)]
    assert (out2[:, 0].float() - want.float()).abs().max() < 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Dh", [128, 64])
def test_rotary_embedding_inside_the_kernel_matches_rotating_first(dtype, Dh):
    """decode_attention(..., rope=(cos, sin)) on raw q/k equals rotating q and k (fp32, one rounding)
    and then calling the plain fused step; the rotated K row is what lands in the cache."""
    from moa_b200.module import rotary_cos_sin
    gen = torch.Generator().manual_seed(17)
    B, caps = 3, [128, 320, 192]
    H = len(caps)
    mk = lambda: moa_b200.StaticCircularCache([caps], B, Dh, [[64] * H], "cuda", dtype)
    a, b = mk(), mk()
    kp = torch.randn(B, H, 250, Dh, generator=gen).to(dtype).cuda()
    vp = torch.randn(B, H, 250, Dh, generator=gen).to(dtype).cuda()
    a.update(kp, vp, 0)
    b.update(kp, vp, 0)
    for step in range(4):
        q, k1, v1 = (torch.randn(B, H, 1, Dh, generator=gen).to(dtype).cuda() for _ in range(3))
        pos = torch.tensor([[250 + step], [7 + step], [100000 + step]], device="cuda")
        cos, sin = rotary_cos_sin(pos, Dh, 10000.0, dtype)
        out_a = a.decode_attention(q, k1, v1, 0, Dh ** -0.5, rope=(cos, sin))
        q_rot = orc.apply_rope(q.float().cpu(), cos.float().cpu(), sin.float().cpu()).to(dtype).cuda()
        k_rot = orc.apply_rope(k1.float().cpu(), cos.float().cpu(), sin.float().cpu()).to(dtype).cuda()
        out_b = b.decode_attention(q_rot, k_rot, v1, 0, Dh ** -0.5)
        assert torch.equal(out_a, out_b), step
    assert torch.equal(a.key_cache[0], b.key_cache[0]) and torch.equal(a.value_cache[0], b.value_cache[0])
    assert torch.equal(a.cache_update_index[0], b.cache_update_index[0])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_poisoned_unused_slots_and_guard_rows(dtype):
    """Out-of-range reads and writes, made visible: every cache slot past a head's valid length holds NaN (a
    kernel that reads one poisons its output), and the output sits between two guard rows that must come
    back untouched."""
    gen = torch.Generator().manual_seed(77)
    B, Dh = 3, 128
    caps = [128, 192, 320, 64, 1088]
    H = len(caps)
    k, v, hs, valid = _random_cache(B, caps, Dh, dtype, gen)
    q = torch.randn(B, H, 1, Dh, generator=gen).to(dtype)
    sm = Dh ** -0.5
    ref = orc.decode_attention_fp32(q, k, v, hs, valid, sm)
    kp, vp = k.clone(), v.clone()
    for b in range(B):
        for h in range(H):
            lo, hi = int(hs[b, h]) + int(valid[b, h]), int(hs[b, h]) + caps[h]
            kp[b, lo:hi] = float("nan")
            vp[b, lo:hi] = float("nan")
    guard = 1234.5
    buf = torch.full((B + 2, 1, H, Dh), guard, dtype=dtype, device="cuda")
    out = moa_b200.sparse_decode(q.cuda(), kp.cuda(), vp.cuda(), hs.cuda(), valid.cuda(), sm, out=buf[1:B + 1])
    assert torch.isfinite(out.float()).all(), "a slot past the valid length was read"
    _close(out, ref, dtype, "poisoned cache")
    assert (buf[0] == guard).all() and (buf[B + 1] == guard).all(), "the output's guard rows were written"


def test_fused_decode_leaves_other_slots_alone():
    """The fused append writes exactly one row per (batch, head): every other slot of caches pre-filled with a
    marker value, and the guard rows around the flattened caches, keep it."""
    B, Dh, dtype = 2, 64, torch.float16
    caps = [128, 192, 320]
    H = len(caps)
    cache = moa_b200.StaticCircularCache([caps], B, Dh, [[64] * H], "cuda", dtype)
    gen = torch.Generator(device="cuda").manual_seed(5)
    k0 = torch.randn(B, H, 50, Dh, generator=gen, device="cuda").to(dtype)
    cache.update(k0, k0, 0)
    marker = 7.0
    S = sum(caps)
    pad = 64
    # the cache payload lives in the middle of a larger allocation whose first and last rows are guards
    big_k = torch.full((B * S + 2 * pad, Dh), marker, dtype=dtype, device="cuda")
    big_v = torch.full((B * S + 2 * pad, Dh), marker, dtype=dtype, device="cuda")
    written_before = cache.cache_update_index[0].clone()
    cache.key_cache[0] = big_k[pad:pad + B * S].view(B, S, Dh)
    cache.value_cache[0] = big_v[pad:pad + B * S].view(B, S, Dh)
    q, k1, v1 = (torch.randn(B, H, 1, Dh, generator=gen, device="cuda").to(dtype) for _ in range(3))
    cache.decode_attention(q, k1, v1, 0, Dh ** -0.5)
    kc = cache.key_cache[0]
    touched = torch.zeros(B, S, dtype=torch.bool, device="cuda")
    touched.scatter_(1, written_before, True)
    assert (kc[~touched] == marker).all() and (cache.value_cache[0][~touched] == marker).all()
    for b in range(B):
        for h in range(H):
            slot = int(written_before[b, h])
            assert torch.equal(kc[b, slot], k1[b, h, 0]) and torch.equal(cache.value_cache[0][b, slot], v1[b, h, 0])
    for big in (big_k, big_v):                                         # nothing outside the cache's own rows
        assert (big[:pad] == marker).all() and (big[pad + B * S:] == marker).all()


def test_config4_shape_multi_chunk_merge_bf16():
    """The decode shape of config 4 of BASELINE.json at reduced batch and head count: bf16, head_dim 128,
    8 heads with windows drawn from U[1k, 16k] (rounded up to 64) plus 64 sinks, batch 4, rings filled from a
    prompt longer than the largest ring, three fused decode steps, with the 2048-row chunk the library picks
    at config 4's full batch: every head is split over several blocks and the last-arriver merge combines up
    to eight partial records per head.  Checked per step: the fp32-store
    output against the fp32 oracle at the stated tolerance, the bf16 output as exactly its rounding, and the
    ring state bit-exactly."""
    rng = np.random.RandomState(4000)
    B, H, Dh = 4, 8, 128
    caps = [64 + int(-(-int(w) // 64) * 64) for w in rng.uniform(1024, 16384, H)]
    N = max(caps) + 100
    gen = torch.Generator().manual_seed(4001)
    dtype = torch.bfloat16
    # the oracle keeps bf16 values exactly in float32 (numpy has no bf16)
    o = orc.RingCacheOracle([caps], [[64] * H], B, Dh, dtype=np.float32)
    c = moa_b200.StaticCircularCache([caps], B, Dh, [[64] * H], "cuda", dtype)
    c.decode_chunk = 2048      # what the library chooses at config 4's full batch of 64
    k = torch.randn(B, H, N, Dh, generator=gen).to(dtype)
    v = torch.randn(B, H, N, Dh, generator=gen).to(dtype)
    o.update(k.float().numpy(), v.float().numpy(), 0)
    c.update(k.cuda(), v.cuda(), 0)
    del k, v
    assert np.array_equal(c.key_cache[0].float().cpu().numpy(), o.key_cache[0])
    sm = Dh ** -0.5
    for step in range(3):
        q, k1, v1 = (torch.randn(B, H, 1, Dh, generator=gen).to(dtype) for _ in range(3))
        kc, vc = o.update(k1.float().numpy(), v1.float().numpy(), 0)
        ref = orc.decode_attention_fp32(q, torch.from_numpy(kc), torch.from_numpy(vc),
                                        torch.from_numpy(o.cache_head_start_index[0]),
                                        torch.from_numpy(o.cache_valid_length[0]), sm)
        # same step twice from the same state: fp32 store, then (state restored) bf16 store
        state = (c.cache_update_index[0].clone(), c.cache_valid_length[0].clone(), c.mask_cache[0].clone(), c._kv_len[0],
                 c.cache_position)
        out32 = c.decode_attention(q.cuda(), k1.cuda(), v1.cuda(), 0, sm, out_dtype=torch.float32)
        c.cache_update_index[0].copy_(state[0]); c.cache_valid_length[0].copy_(state[1]); c.mask_cache[0].copy_(state[2])
        c._kv_len[0], c.cache_position = state[3], state[4]
        out16 = c.decode_attention(q.cuda(), k1.cuda(), v1.cuda(), 0, sm)
        _close(out32, ref, dtype, f"config-4 shape, step {step}")
        _close(out16, ref, dtype, f"config-4 shape, step {step}")
        assert torch.equal(out32.to(dtype), out16)
        assert np.array_equal(c.cache_update_index[0].cpu().numpy(), o.cache_update_index[0])
        assert np.array_equal(c.cache_valid_length[0].cpu().numpy(), o.cache_valid_length[0])
    assert np.array_equal(c.key_cache[0].float().cpu().numpy(), o.key_cache[0])
    assert np.array_equal(c.value_cache[0].float().cpu().numpy(), o.value_cache[0])


def test_heads_without_rows_get_zero_output():
    """Two heads share a start index, so the first of them owns no rows: its output row is defined (zeros)."""
    gen = torch.Generator().manual_seed(5)
    B, Dh = 2, 128
    caps = [128, 0, 192]
    S = sum(caps)
    k = torch.randn(B, S, Dh, generator=gen).half()
    v = torch.randn(B, S, Dh, generator=gen).half()
    hs = torch.tensor([[0, 128, 128]] * B, dtype=torch.int64)
    valid = torch.tensor([[128, 0, 192]] * B, dtype=torch.int64)
    q = torch.randn(B, 3, 1, Dh, generator=gen).half()
    out = torch.full((B, 1, 3, Dh), float("nan"), dtype=torch.float16, device="cuda")
    moa_b200.sparse_decode(q.cuda(), k.cuda(), v.cuda(), hs.cuda(), valid.cuda(), 0.1, out=out)
    assert torch.isfinite(out).all() and out[:, :, 1].abs().sum() == 0
    _close(out, orc.decode_attention_fp32(q, k, v, hs, valid, 0.1), torch.float16, "zero-capacity head")


def test_gather_launch_with_its_barrier_on_one_gpu():
    """The decode launch that also delivers its rows and ends with the cross-rank barrier, on one GPU:
    (1) a one-rank group: same result as the plain fused step, call after call, the device-side call counter
    advances; (2) a pretended two-rank group whose other rank never arrives: the bounded wait inside the kernel
    runs out, the status words say who was missing, the output is still right and the next launch works."""
    import ctypes
    gen = torch.Generator().manual_seed(41)
    B, Dh = 3, 128
    caps = [320, 576, 128, 1088]
    H = len(caps)
    kp = torch.randn(B, H, 700, Dh, generator=gen).half().cuda()
    vp = torch.randn(B, H, 700, Dh, generator=gen).half().cuda()
    c_ref = moa_b200.StaticCircularCache([caps], B, Dh, [[64] * H], "cuda", torch.float16)
    c_one = moa_b200.StaticCircularCache([caps], B, Dh, [[64] * H], "cuda", torch.float16)
    c_ref.update(kp, vp, 0)
    c_one.update(kp, vp, 0)
    sh = moa_b200.HeadSharding(caps, 1, 0)
    pg = moa_b200.PeerGather(sh, B, Dh, torch.float16, "cuda")
    for step in range(3):
        q, k1, v1 = (torch.randn(B, H, 1, Dh, generator=gen).half().cuda() for _ in range(3))
        want = c_ref.decode_attention(q, k1, v1, 0, 0.09)
        got = pg.decode_and_gather(c_one, q, k1, v1, 0, 0.09)
        assert torch.equal(got, want)
    pg.check()
    assert pg._calls.item() == 3
    pg.close()

    flags0 = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags1 = torch.zeros(8, dtype=torch.int32, device="cuda")       # the absent rank's (nobody reads them)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    calls = torch.zeros(1, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(flags0.data_ptr(), flags1.data_ptr())
    q, k1, v1 = (torch.randn(B, H, 1, Dh, generator=gen).half().cuda() for _ in range(3))
    want = c_ref.decode_attention(q, k1, v1, 0, 0.09)
    got = c_one.decode_attention(q, k1, v1, 0, 0.09,
                                 barrier=(ptrs, 0, 2, calls.data_ptr(), 20_000_000, status.data_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert status.tolist() == [21, 1, 1, 0] and calls.item() == 1
    assert flags0.tolist()[:2] == [1, 0] and flags1.tolist()[0] == 1
    want = c_ref.decode_attention(q, k1, v1, 0, 0.09)                # the rows-written counter was put back to zero
    got = c_one.decode_attention(q, k1, v1, 0, 0.09)
    assert torch.equal(got, want)
