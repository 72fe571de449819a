"""Pins the CPU oracle (oracle/moa_oracle.py) to fixtures produced by running the reference."""
import glob
import json
import os

import numpy as np
import pytest
import torch

from oracle import moa_oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_cache_config_matches_reference():
    cases = json.load(open(os.path.join(GOLDEN, "cache_config.json")))
    assert len(cases) >= 30
    for c in cases:
        got = orc.cache_config(c["plan"], c["seq_len"], c["max_new_token"], **c["kwargs"])
        assert got == c["result"], c["model"]


def test_permutation_matches_reference():
    for c in json.load(open(os.path.join(GOLDEN, "permutation.json"))):
        perms, clusters = orc.permutation(c["plan"])
        assert perms == c["perms"]
        assert [{str(k): list(v) for k, v in cl.items()} for cl in clusters] == c["clusters"]


def _coded(B, H, n, D, base):
    t = np.arange(n, dtype=np.float32)[None, None, :, None] + base
    h = np.arange(H, dtype=np.float32)[None, :, None, None] * 10000.0
    b = np.arange(B, dtype=np.float32)[:, None, None, None] * 1000000.0
    return np.broadcast_to(t + h + b, (B, H, n, D)).copy()


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "cache_trace_*.npz"))))
def test_ring_cache_trace_bit_exact(path):
    g = np.load(path)
    B, D = int(g["B"]), int(g["D"])
    cache = orc.RingCacheOracle(g["cache_size"].tolist(), g["static_size"].tolist(), B, D)
    H = len(g["cache_size"][0])
    n = int(g["n_prefill"])
    mask = None
    if int(g["use_mask"]):
        mask = np.zeros((B, n), dtype=np.int64)
        for i, L in enumerate(g["prefill_lens"]):
            mask[i, n - int(L):] = 1
    assert np.array_equal(cache.head_index[0], g["head_index"])
    assert np.array_equal(cache.cache_head_start_index[0], g["head_start"])
    base = 0
    for step in range(int(g["decode_steps"]) + 1):
        q = n if step == 0 else 1
        k = _coded(B, H, q, D, base)
        cache.update(k, k + 0.5, 0, mask if step == 0 else None)
        base += q
        assert np.array_equal(cache.cache_update_index[0], g["update_index"][step]), step
        assert np.array_equal(cache.cache_valid_length[0], g["valid_length"][step]), step
        assert np.array_equal(cache.mask_cache[0], g["mask_cache"][step]), step
        assert np.array_equal(cache.key_cache[0][..., 0], g["key0"][step]), step
        assert np.array_equal(cache.value_cache[0][..., 0], g["val0"][step]), step
        assert cache._kv_len[0] == int(g["kv_len"][step])


def test_slot_rule_against_trace():
    g = np.load(os.path.join(GOLDEN, "cache_trace_wrap.npz"))
    caps, hs = g["cache_size"][0], g["head_index"]
    n_total = int(g["n_prefill"]) + int(g["decode_steps"])
    key = g["key0"][-1]
    for h, cap in enumerate(caps):
        for t in range(n_total):
            slot = orc.slot_of_token(t, int(cap), 64)
            newest = max(tt for tt in range(n_total) if orc.slot_of_token(tt, int(cap), 64) == slot)
            if newest == t:
                assert key[0, hs[h] + slot] == t + 10000.0 * h


def test_block_layout_matches_reference_patterns():
    g = np.load(os.path.join(GOLDEN, "layouts.npz"))
    n = 0
    for name in g.files:
        if name.startswith("layout_"):
            nb, s, L = map(int, name.split("_")[1:])
            assert np.array_equal(orc.block_layout(nb, s, L), g[name]), name
            n += 1
    assert n >= 8
    assert np.array_equal(orc.prefill_mask(256, 1, 2), g["mask_4_1_2"])


def test_prefill_fp32_matches_reference_mask_and_triton():
    g = np.load(os.path.join(GOLDEN, "prefill_sparse.npz"))
    q, k, v = (torch.from_numpy(g[x]) for x in "qkv")
    out = orc.prefill_attention_fp32(q, k, v, float(g["sm_scale"]), g["sink_blocks"], g["local_blocks"])
    ref = torch.from_numpy(g["masked_fp32"])
    assert (out - ref).abs().max() < 2e-5
    tri = torch.from_numpy(g["triton_fp16"]).float()
    assert (out - tri).abs().max() < 2e-3
    assert (out - tri).abs().mean() / ref.abs().mean() < 1e-3
    # chunked evaluation is the same function
    out2 = orc.prefill_attention_fp32(q, k, v, float(g["sm_scale"]), g["sink_blocks"], g["local_blocks"], row_chunk=100)
    assert (out - out2).abs().max() < 2e-5


def test_prefill_fp32_ragged_matches_triton():
    g = np.load(os.path.join(GOLDEN, "prefill_ragged.npz"))
    q, k, v = (torch.from_numpy(g[x]) for x in "qkv")
    out = orc.prefill_attention_fp32(q, k, v, float(g["sm_scale"]), g["sink_blocks"], g["local_blocks"])
    tri = torch.from_numpy(g["triton_fp16"]).float()
    assert (out - tri).abs().max() < 2e-3


def test_prefill_reference_own_test_case():
    g = np.load(os.path.join(GOLDEN, "prefill_reftest.npz"))
    q, k, v = (torch.from_numpy(g[x]) for x in "qkv")
    out = orc.prefill_attention_fp32(q, k, v, float(g["sm_scale"]), g["sink_size"] // 64, g["local_size"] // 64)
    torch.testing.assert_close(out, torch.from_numpy(g["sdpa"]).float(), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(out, torch.from_numpy(g["moa"]).float(), rtol=1e-3, atol=1e-3)


def test_decode_matches_reference_sdpa_path():
    g = np.load(os.path.join(GOLDEN, "decode_sdpa.npz"))
    caps = g["caps"].tolist()
    B, H, D = 2, len(caps), 128
    cache = orc.RingCacheOracle([caps], [[64] * H], B, D, dtype=np.float16)
    cache.update(g["k_prefill"], g["v_prefill"], 0)
    for s in range(g["q"].shape[0]):
        kc, vc = cache.update(g["k_new"][s], g["v_new"][s], 0)
        out = orc.decode_attention_fp32(torch.from_numpy(g["q"][s]), torch.from_numpy(kc), torch.from_numpy(vc),
                                        torch.from_numpy(cache.cache_head_start_index[0]),
                                        torch.from_numpy(cache.cache_valid_length[0]), float(g["sm_scale"]))
        ref = torch.from_numpy(g["out"][s]).float()
        assert (out - ref).abs().max() < 2e-3
        grp = orc.decode_attention_grouped_sdpa(torch.from_numpy(g["q"][s]), torch.from_numpy(kc), torch.from_numpy(vc),
                                                torch.from_numpy(cache.head_index[0]), float(g["sm_scale"]))
        assert (grp.float() - ref).abs().max() < 1e-3
    assert np.array_equal(cache.key_cache[0], g["key_cache_final"])
    assert np.array_equal(cache.cache_update_index[0], g["update_index_final"])


def test_masked_sdpa_route_equals_the_fp32_oracle():
    """The timed CPU baseline of the prefill (one scaled_dot_product_attention call with the boolean mask that
    ``prefill_mask`` builds, which the layout fixtures above pin) gives the oracle's result."""
    import torch
    gen = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(2, 4, 300, 64, generator=gen) for _ in range(3))
    sink_b, local_b = [1, 1, 0, 2], [1, 2, 3, 8]
    a = orc.prefill_attention_masked_sdpa(q, k, v, 0.11, sink_b, local_b)
    b = orc.prefill_attention_fp32(q, k, v, 0.11, sink_b, local_b)
    assert a.shape == b.shape == (2, 300, 4, 64)
    assert (a - b).abs().max().item() < 2e-5
