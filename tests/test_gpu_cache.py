"""Ring-cache kernels vs traces recorded from the reference's StaticCircularCache (bit-exact)."""
import glob
import os

import numpy as np
import pytest
import torch

import moa_b200
from oracle import moa_oracle as orc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
D = 64


def _coded(B, H, n, base, dtype, device, split=False):
    """K rows carry (token, head, batch) in dims 0..2 — all exactly representable in fp16.  With ``split`` the
    token id is stored as (id % 128, id // 128) in dims 0 and 3, which bf16 (8 significant bits) holds exactly."""
    x = torch.zeros(B, H, n, D, dtype=torch.float32)
    tok = torch.arange(n, dtype=torch.float32)[None, None, :] + base
    if split:
        x[..., 0] = tok % 128
        x[..., 3] = torch.floor(tok / 128)
    else:
        x[..., 0] = tok
    x[..., 1] = torch.arange(H, dtype=torch.float32)[None, :, None]
    x[..., 2] = torch.arange(B, dtype=torch.float32)[:, None, None]
    return x.to(dtype).to(device)


def _decode_golden(g):
    """golden value t + 1e4*h + 1e6*b (+0.5 for V) -> (t, h, b)"""
    g = np.floor(g)
    return g % 10000, (g // 10000) % 100, g // 1000000


def _check_state(cache, g, step, tag, split=False):
    assert np.array_equal(cache.cache_update_index[0].cpu().numpy(), g["update_index"][step]), (tag, step)
    assert np.array_equal(cache.cache_valid_length[0].cpu().numpy(), g["valid_length"][step]), (tag, step)
    assert np.array_equal(cache.mask_cache[0].cpu().numpy(), g["mask_cache"][step]), (tag, step)
    assert cache._kv_len[0] == int(g["kv_len"][step])
    k = cache.key_cache[0].float().cpu().numpy()
    v = cache.value_cache[0].float().cpu().numpy()
    t, h, b = _decode_golden(g["key0"][step])
    tv, _, _ = _decode_golden(g["val0"][step])
    frac = g["val0"][step] - np.floor(g["val0"][step])
    if split:   # token id in two dims, the V marker (0.5) in dim 4
        assert np.array_equal(k[..., 0] + 128 * k[..., 3], t), (tag, step)
        assert np.array_equal(v[..., 0] + 128 * v[..., 3], tv) and np.array_equal(v[..., 4], frac), (tag, step)
    else:
        assert np.array_equal(k[..., 0], t), (tag, step)
        assert np.array_equal(v[..., 0], tv + frac), (tag, step)
    assert np.array_equal(k[..., 1], h) and np.array_equal(k[..., 2], b), (tag, step)


def _mask_of(g, B, n):
    if not int(g["use_mask"]):
        return None
    mask = torch.zeros(B, n, dtype=torch.int64)
    for i, L in enumerate(g["prefill_lens"]):
        mask[i, n - int(L):] = 1
    return mask.cuda()


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "cache_trace_*.npz"))))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_update_replays_reference_trace(path, dtype):
    g = np.load(path)
    B, n = int(g["B"]), int(g["n_prefill"])
    split = dtype == torch.bfloat16
    H = len(g["cache_size"][0])
    cache = moa_b200.StaticCircularCache(g["cache_size"].tolist(), B, D, g["static_size"].tolist(), "cuda", dtype)
    base = 0
    for step in range(int(g["decode_steps"]) + 1):
        q = n if step == 0 else 1
        k = _coded(B, H, q, base, dtype, "cuda", split)
        v = k.clone()
        v[..., 4 if split else 0] += 0.5
        ret = cache.update(k, v, 0, _mask_of(g, B, n) if step == 0 else None)
        base += q
        if step == 0:
            assert ret[0] is k and ret[1] is v          # prefill returns the states it was given
        else:
            assert ret[0] is cache.key_cache[0]         # decode returns the flattened caches
        _check_state(cache, g, step, os.path.basename(path), split)


@pytest.mark.parametrize("name", ["wrap", "short", "leftpad", "exact", "nostatic", "one", "smoke"])
def test_fused_decode_advances_like_reference(name):
    """decode_attention (append fused into the attention launch) leaves the same cache state as
    update(), and returns the same attention output as update() + mixture_of_sparse_attention."""
    g = np.load(os.path.join(GOLDEN, f"cache_trace_{name}.npz"))
    B, n = int(g["B"]), int(g["n_prefill"])
    H = len(g["cache_size"][0])
    dtype = torch.float16
    mk = lambda: moa_b200.StaticCircularCache(g["cache_size"].tolist(), B, D, g["static_size"].tolist(), "cuda", dtype)
    fused, plain = mk(), mk()
    k = _coded(B, H, n, 0, dtype, "cuda")
    v = k.clone()
    v[..., 0] += 0.5
    fused.update(k, v, 0, _mask_of(g, B, n))
    plain.update(k, v, 0, _mask_of(g, B, n))
    base = n
    gen = torch.Generator(device="cuda").manual_seed(3)
    for step in range(1, int(g["decode_steps"]) + 1):
        k = _coded(B, H, 1, base, dtype, "cuda")
        v = k.clone()
        v[..., 0] += 0.5
        q = torch.randn(B, H, 1, D, generator=gen, device="cuda").to(dtype)
        out_f = fused.decode_attention(q, k, v, 0, 0.2)
        kc, vc = plain.update(k, v, 0)
        out_p = moa_b200.mixture_of_sparse_attention(q, kc, vc, 0.2, head_start_index=plain.cache_head_start_index[0],
                                                     head_valid_length=plain.cache_valid_length[0])
        base += 1
        _check_state(fused, g, step, name)
        assert out_f.shape == (B, 1, H, D)
        assert torch.equal(out_f, out_p), (name, step)


def test_update_cache_content_false_only_moves_indices():
    g = np.load(os.path.join(GOLDEN, "cache_trace_wrap.npz"))
    B, H = int(g["B"]), len(g["cache_size"][0])
    cache = moa_b200.StaticCircularCache(g["cache_size"].tolist(), B, D, g["static_size"].tolist(), "cuda",
                                         torch.float16, update_cache_content=True)
    k = _coded(B, H, int(g["n_prefill"]), 0, torch.float16, "cuda")
    cache.update(k, k, 0)
    cache.update_cache_content = False
    before = cache.key_cache[0].clone()
    for step in range(1, 20):
        cache.update(None, None, 0)
        assert np.array_equal(cache.cache_update_index[0].cpu().numpy(), g["update_index"][step])
        assert np.array_equal(cache.cache_valid_length[0].cpu().numpy(), g["valid_length"][step])
    assert torch.equal(before, cache.key_cache[0])


def test_random_prefill_then_decode_matches_oracle_bit_exact():
    rng = np.random.RandomState(5)
    for trial in range(6):
        H, B = int(rng.randint(1, 6)), int(rng.randint(1, 4))
        caps = [int(rng.choice([128, 192, 256, 448, 1024])) for _ in range(H)]
        static = [64] * H
        n = int(rng.randint(2, 1500))
        lens = [int(rng.randint(1, n + 1)) for _ in range(B)]
        lens[0] = n
        mask = np.zeros((B, n), dtype=np.int64)
        for i, L in enumerate(lens):
            mask[i, n - L:] = 1
        use_mask = trial % 2 == 0
        o = orc.RingCacheOracle([caps], [static], B, D, dtype=np.float16)
        c = moa_b200.StaticCircularCache([caps], B, D, [static], "cuda", torch.float16)
        k = torch.randn(B, H, n, D).half()
        v = torch.randn(B, H, n, D).half()
        o.update(k.numpy(), v.numpy(), 0, mask if use_mask else None)
        # strided input: (B, n, H, D) storage viewed as (B, H, n, D), as the projection produces it
        kd = k.transpose(1, 2).contiguous().cuda().transpose(1, 2)
        vd = v.transpose(1, 2).contiguous().cuda().transpose(1, 2)
        c.update(kd, vd, 0, torch.from_numpy(mask).cuda() if use_mask else None)
        for step in range(40):
            k1, v1 = torch.randn(B, H, 1, D).half(), torch.randn(B, H, 1, D).half()
            o.update(k1.numpy(), v1.numpy(), 0)
            c.update(k1.cuda(), v1.cuda(), 0)
        assert np.array_equal(c.cache_update_index[0].cpu().numpy(), o.cache_update_index[0])
        assert np.array_equal(c.cache_valid_length[0].cpu().numpy(), o.cache_valid_length[0])
        assert np.array_equal(c.mask_cache[0].cpu().numpy(), o.mask_cache[0])
        assert np.array_equal(c.key_cache[0].cpu().numpy(), o.key_cache[0])
        assert np.array_equal(c.value_cache[0].cpu().numpy(), o.value_cache[0])


def test_state_dict_round_trip_continues_bit_exactly():
    """Checkpoint / resume of the cache: decoding from a restored state gives the same outputs and the same
    cache as decoding on without interruption."""
    B, H, Dh, dtype = 2, 3, 64, torch.float16
    caps, static = [[128, 192, 320]], [[64, 64, 64]]
    gen = torch.Generator(device="cuda").manual_seed(9)
    mk = lambda: moa_b200.StaticCircularCache(caps, B, Dh, static, "cuda", dtype)
    a = mk()
    k0, v0 = (torch.randn(B, H, 150, Dh, generator=gen, device="cuda").to(dtype) for _ in range(2))
    a.update(k0, v0, 0)
    steps = [[torch.randn(B, H, 1, Dh, generator=gen, device="cuda").to(dtype) for _ in range(3)] for _ in range(8)]
    for q, k, v in steps[:3]:
        a.decode_attention(q, k, v, 0, 0.125)
    saved = a.state_dict()
    outs_a = [a.decode_attention(q, k, v, 0, 0.125).clone() for q, k, v in steps[3:]]
    b = mk()
    b.load_state_dict(saved)
    outs_b = [b.decode_attention(q, k, v, 0, 0.125).clone() for q, k, v in steps[3:]]
    for x, y in zip(outs_a, outs_b):
        assert torch.equal(x, y)
    assert torch.equal(a.key_cache[0], b.key_cache[0]) and torch.equal(a.value_cache[0], b.value_cache[0])
    assert torch.equal(a.cache_update_index[0], b.cache_update_index[0])
    assert torch.equal(a.cache_valid_length[0], b.cache_valid_length[0]) and torch.equal(a.mask_cache[0], b.mask_cache[0])
    assert a._kv_len == b._kv_len
    with pytest.raises(ValueError):
        moa_b200.StaticCircularCache([[128, 192, 256]], B, Dh, static, "cuda", dtype).load_state_dict(saved)
