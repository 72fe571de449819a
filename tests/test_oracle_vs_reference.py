"""Randomised comparison of the CPU oracle (and of the host-side mirror) with the reference itself.

Runs only where a thu-nics/MoA checkout is available (``MOA_REF``, or a directory named ``reference`` next
to this repository); elsewhere the whole module is skipped and the committed fixtures under
``tests/golden/`` are what pins the oracle.  Everything here is CPU work: the reference's plan arithmetic,
head permutation, ``StaticCircularCache`` and block-sparse mask builders, driven with seeded random cases.
"""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import moa_oracle as orc

_HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("MOA_REF") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
if not os.path.isdir(os.path.join(REF, "MoA")):
    pytest.skip("no reference checkout on this machine", allow_module_level=True)

sys.dont_write_bytecode = True
sys.path.insert(0, REF)
try:
    import transformers.cache_utils as tcu

    tcu.Cache.__init__ = lambda self, *a, **k: None     # the reference targets an older transformers
    from MoA.attention.cache_utils import StaticCircularCache as RefCache, moa_config_to_cache_config as ref_cache_config
    from MoA.attention.convert import layout_to_mask
    from MoA.attention.pattern import gen_bigbird_pattern, gen_causal_pattern
    from MoA.attention.permutation_utils import moa_config_to_permutation as ref_permutation
except Exception as exc:  # pragma: no cover - depends on the machine
    pytest.skip(f"the reference does not import here: {exc!r}", allow_module_level=True)
finally:
    sys.path.remove(REF)


def _random_plan(rng, layers, heads):
    alphas = [[float(rng.choice([-1024, -100.5, 0, 63, 64, 65, 128, 500.25, 1000.7, 4096, 8192])) for _ in range(heads)]
              for _ in range(layers)]
    betas = [[float(rng.choice([0, 0.01, 0.125, 0.3333, 0.5, 0.875, 1.0, 1.5])) for _ in range(heads)]
             for _ in range(layers)]
    return {"alphas": alphas, "betas": betas}


def test_cache_config_random_plans():
    import moa_b200
    rng = np.random.RandomState(101)
    for case in range(150):
        plan = _random_plan(rng, int(rng.randint(1, 4)), int(rng.randint(1, 9)))
        seq_len, max_new = int(rng.randint(1, 70000)), int(rng.choice([0, 1, 64, 1024]))
        kw = {}
        if case % 3 == 0:
            kw = {"sink_size": int(rng.choice([64, 128, 4])), "minimum_cache_size": int(rng.choice([128, 64, 256])),
                  "split_size": int(rng.choice([64, 32, 128]))}
        want = ref_cache_config(plan, seq_len=seq_len, max_new_token=max_new, verbose=False, **kw)
        assert orc.cache_config(plan, seq_len, max_new, **kw) == want, (case, plan, seq_len, max_new, kw)
        assert moa_b200.moa_config_to_cache_config(plan, seq_len, max_new, verbose=False, **kw) == want, case


def test_permutation_random_plans():
    import moa_b200
    rng = np.random.RandomState(202)
    for case in range(60):
        plan = _random_plan(rng, int(rng.randint(1, 4)), int(rng.randint(1, 17)))
        perms, clusters = ref_permutation(plan)
        o_perms, o_clusters = orc.permutation(plan)
        assert o_perms == [p.tolist() for p in perms], case
        assert [{int(k): tuple(v) for k, v in c.items()} for c in o_clusters] == \
               [{int(k): tuple(v) for k, v in c.items()} for c in clusters], case
        m_perms, m_clusters = moa_b200.moa_config_to_permutation(plan)
        assert [torch.as_tensor(p).tolist() for p in m_perms] == [p.tolist() for p in perms], case
        assert [{int(k): tuple(v) for k, v in c.items()} for c in m_clusters] == \
               [{int(k): tuple(v) for k, v in c.items()} for c in clusters], case


def _coded(B, H, n, D, base):
    t = np.arange(n, dtype=np.float32)[None, None, :, None] + base
    h = np.arange(H, dtype=np.float32)[None, :, None, None] * 10000.0
    b = np.arange(B, dtype=np.float32)[:, None, None, None] * 1000000.0
    return np.broadcast_to(t + h + b, (B, H, n, D)).copy()


def test_ring_cache_random_traces_bit_exact():
    """Prefill (with and without left padding) then decode steps, every piece of cache state after every
    update, against the reference's StaticCircularCache."""
    rng = np.random.RandomState(303)
    D = 8
    for case in range(40):
        H, B = int(rng.randint(1, 4)), int(rng.randint(1, 4))
        caps = [int(rng.choice([128, 192, 320, 448])) for _ in range(H)]      # what the plan arithmetic can produce
        static = [int(rng.choice([0, 64])) for _ in caps] if case % 4 == 0 else [64 for _ in caps]
        n = int(rng.randint(1, 500))
        steps = int(rng.randint(0, 90))
        use_mask = bool(case % 2)
        lens = [int(rng.randint(1, n + 1)) for _ in range(B)]
        ref = RefCache(cache_size=[caps], static_size=[static], batch_size=B, head_dim=D, device="cpu", dtype=torch.float32)
        mine = orc.RingCacheOracle([caps], [static], B, D)
        mask = None
        if use_mask:
            mask = np.zeros((B, n), dtype=np.int64)
            for i, L in enumerate(lens):
                mask[i, n - L:] = 1
        base = 0
        for step in range(steps + 1):
            q = n if step == 0 else 1
            k = _coded(B, H, q, D, base)
            m = mask if step == 0 else None
            ref.update(torch.from_numpy(k), torch.from_numpy(k + 0.5), 0, None if m is None else torch.from_numpy(m))
            mine.update(k, k + 0.5, 0, m)
            base += q
            tag = (case, step, caps, static, n, lens if use_mask else None)
            assert np.array_equal(mine.cache_update_index[0], ref.cache_update_index[0].numpy()), tag
            assert np.array_equal(mine.cache_valid_length[0], ref.cache_valid_length[0].numpy()), tag
            assert np.array_equal(mine.mask_cache[0], ref.mask_cache[0].numpy()), tag
            assert np.array_equal(mine.key_cache[0], ref.key_cache[0].numpy()), tag
            assert np.array_equal(mine.value_cache[0], ref.value_cache[0].numpy()), tag
            assert mine._kv_len[0] == ref._kv_len[0], tag


def test_prefill_mask_random_shapes():
    """The block layout and the element mask the oracle's prefill uses, against the reference's own builders
    (gen_bigbird_pattern & gen_causal_pattern -> layout_to_mask, block 64, causal)."""
    rng = np.random.RandomState(404)
    for case in range(30):
        nb = int(rng.randint(1, 24))
        sink_b, local_b = int(rng.randint(1, min(nb, 3) + 1)), int(rng.randint(1, 30))   # the builder needs sink_b <= nb
        lay = gen_bigbird_pattern(nb, nb, 2 * local_b - 1, sink_b, 0).squeeze(0) & gen_causal_pattern(nb, nb).squeeze(0)
        lay = lay.reshape(nb, nb)
        assert np.array_equal(orc.block_layout(nb, sink_b, local_b).astype(bool), lay.numpy().astype(bool)), \
            (case, nb, sink_b, local_b)
        if nb <= 8:
            want = layout_to_mask(lay[None], 64, True)[0].numpy().astype(bool)
            got = orc.prefill_mask(nb * 64, sink_b, local_b).astype(bool)
            assert np.array_equal(got, want), (case, nb, sink_b, local_b)


def test_decode_against_reference_sdpa_path_random_full_rings():
    """Ring update + decode attention, end to end on CPU, against the reference's own CPU-runnable decode
    (``implementation="sdpa"``: regroup the flattened cache, SDPA per group).  That path derives its head
    boundaries from the capacities, so it is exact only once every ring is full; the prompts here are longer
    than the largest capacity."""
    from MoA.kernels.mixture_of_attention import mixture_of_sparse_attention as ref_attention
    rng = np.random.RandomState(505)
    for case in range(6):
        H, B, D = int(rng.randint(2, 6)), int(rng.randint(1, 3)), 64
        caps = sorted(int(rng.choice([128, 192, 256, 320])) for _ in range(H))     # equal capacities adjacent
        n = max(caps) + int(rng.randint(1, 100))
        g = torch.Generator().manual_seed(case)
        ref = RefCache(cache_size=[caps], static_size=[[64] * H], batch_size=B, head_dim=D, device="cpu", dtype=torch.float16)
        mine = orc.RingCacheOracle([caps], [[64] * H], B, D)
        k, v = (torch.randn(B, H, n, D, generator=g).half() for _ in range(2))     # the reference path is 16-bit only
        ref.update(k, v, 0)
        mine.update(k.float().numpy(), v.float().numpy(), 0)
        sm = D ** -0.5
        for _ in range(4):
            q1, k1, v1 = (torch.randn(B, H, 1, D, generator=g).half() for _ in range(3))
            kc, vc = ref.update(k1, v1, 0)
            want = ref_attention(q1, kc, vc, sm, head_start_index=ref.cache_head_start_index[0],
                                 head_valid_length=ref.cache_valid_length[0], implementation="sdpa")
            mine.update(k1.float().numpy(), v1.float().numpy(), 0)
            got = orc.decode_attention_fp32(q1, torch.from_numpy(mine.key_cache[0]), torch.from_numpy(mine.value_cache[0]),
                                            torch.from_numpy(mine.cache_head_start_index[0]),
                                            torch.from_numpy(mine.cache_valid_length[0]), sm)
            # both are (B, 1, H, D); the reference's is fp16 out of an fp16 SDPA, the oracle's fp32
            assert want.shape == got.shape == (B, 1, H, D)
            assert float((want.float() - got).abs().max()) <= 1e-3, case
