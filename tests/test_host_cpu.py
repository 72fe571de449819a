"""Host-side logic and the C-ABI boundary, without a GPU."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

import moa_b200
from moa_b200 import _lib, plan
from oracle import moa_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "moa_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(moa_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    raw = ctypes.CDLL(moa_b200.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} declared in include/moa_b200.h but not exported"
    assert declared == set(_lib.SYMBOLS)
    assert _lib.lib.moa_abi_version() == _lib.ABI_VERSION == 2


def test_status_strings_and_argument_checks_without_gpu():
    lib = _lib.lib
    assert lib.moa_strerror(0) == b"ok"
    assert b"workspace" in lib.moa_strerror(4)
    rc = lib.moa_decode_fwd(*([0] * 6), *([0] * 6), *([0] * 5), 0, 1, 1, 128, 1, 1.0, 0, 0, 0, 0, 0, 0)
    assert rc == 1 and b"null pointer" in lib.moa_last_error_detail()
    rc = lib.moa_prefill_fwd(*([0] * 4), *([0] * 12), 0, 0, 1, 1, 64, 128, 1.0, 0, 0, 0, 0)
    assert rc == 1
    rc = lib.moa_cache_fill(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 128, 1, 1, 0, 0)
    assert rc == 1
    assert lib.moa_decode_workspace_bytes(16, 32, 128, 54272, 0) > 16 * 32 * 4
    assert lib.moa_decode_workspace_bytes(0, 32, 128, 54272, 0) == 0


def test_cpu_tensors_are_rejected_not_silently_computed():
    q = torch.zeros(1, 2, 128, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        moa_b200.mixture_of_sparse_attention(q, q, q, 0.1)
    cache = moa_b200.StaticCircularCache([[128, 128]], 1, 128, [[64, 64]])
    with pytest.raises(RuntimeError, match="CUDA"):
        cache.update(q[:, :, :1], q[:, :, :1], 0)


def test_invalid_input_raises_assertion_like_the_reference():
    # tests/attention_kernel_test.py:140-149 of the reference
    q = torch.rand(2, 4, 10, 64).half()
    k = torch.rand(2, 4, 10, 65).half()
    with pytest.raises(AssertionError):
        moa_b200.mixture_of_sparse_attention(q, k, q, 0.1)
    with pytest.raises(AssertionError):
        moa_b200.mixture_of_sparse_attention(q.float(), q.float(), q.float(), 0.1)


def test_cache_config_matches_reference_fixtures():
    for c in json.load(open(os.path.join(GOLDEN, "cache_config.json"))):
        got = plan.moa_config_to_cache_config(c["plan"], c["seq_len"], c["max_new_token"], verbose=False, **c["kwargs"])
        assert got == c["result"]


def test_permutation_matches_reference_fixtures():
    for c in json.load(open(os.path.join(GOLDEN, "permutation.json"))):
        perms, clusters = plan.moa_config_to_permutation(c["plan"])
        assert [p.tolist() for p in perms] == c["perms"]
        assert [{str(k): list(v) for k, v in cl.items()} for cl in clusters] == c["clusters"]


def test_projection_permutation_round_trip():
    torch.manual_seed(0)
    H, D, hid = 4, 8, 16
    perm = torch.tensor([2, 0, 3, 1])
    q_proj, o_proj = torch.nn.Linear(hid, H * D, bias=True), torch.nn.Linear(H * D, hid, bias=False)
    x = torch.randn(3, hid)
    heads = q_proj(x).view(3, H, D)
    y = o_proj(heads.reshape(3, -1))
    plan.permute_attention_projection(q_proj, perm, H)
    plan.permute_output_projection(o_proj, perm, H)
    heads_p = q_proj(x).view(3, H, D)
    assert torch.allclose(heads_p, heads[:, perm], atol=1e-6)
    assert torch.allclose(o_proj(heads_p.reshape(3, -1)), y, atol=1e-5)


def test_cache_constructor_attributes_match_reference_trace():
    g = np.load(os.path.join(GOLDEN, "cache_trace_wrap.npz"))
    cache = moa_b200.StaticCircularCache(g["cache_size"].tolist(), int(g["B"]), int(g["D"]), g["static_size"].tolist())
    assert np.array_equal(cache.head_index[0].numpy(), g["head_index"])
    assert np.array_equal(cache.cache_head_start_index[0].numpy(), g["head_start"])
    assert cache.cache_update_index[0].dtype == torch.int64
    assert cache.key_cache[0].device.type == "meta"
    assert cache.circular_cache_size[0].tolist() == [64, 128, 256]
    assert cache.mask_cache[0].shape == (2, 640)
    groups = moa_b200.StaticCircularCache.to_group_contigious(torch.arange(2 * 640 * 2).view(2, 640, 2).float(),
                                                             cache.head_index[0])
    assert [tuple(x.shape) for x in groups] == [(2, 1, 128, 2), (2, 1, 192, 2), (2, 1, 320, 2)]


def test_work_counters_agree_with_oracle():
    rng = np.random.RandomState(0)
    for _ in range(50):
        n, H = int(rng.randint(1, 4000)), int(rng.randint(1, 6))
        s, l = rng.randint(0, 3, H), rng.randint(1, 50, H)
        assert plan.prefill_block_visits(n, s, l) == orc.prefill_block_visits(n, s, l)
        assert plan.prefill_flops(2, n, 128, s, l) == orc.prefill_flops(2, n, 128, s, l)
    assert plan.decode_bytes(16, [320, 576], 128, 2) == orc.decode_bytes(16, [320, 576], 128, 2)


def test_shard_heads_balances_and_partitions():
    rng = np.random.RandomState(1)
    caps = [int(64 + rng.choice([256, 512, 1024, 2048, 4096])) for _ in range(32)]
    for world in (1, 2, 4, 8):
        shards = plan.shard_heads(caps, world)
        assert sorted(h for s in shards for h in s) == list(range(32))
        assert all(len(s) == 32 // world for s in shards)
        loads = [sum(caps[h] for h in s) for s in shards]
        assert max(loads) - min(loads) <= max(caps)
        for s in shards:
            assert [caps[h] for h in s] == sorted(caps[h] for h in s)


def test_flashinfer_compat_exports_the_names_the_reference_imports():
    """MoA/kernels/mixture_of_attention.py:23 imports moa_prefill and moa_decode from its CUDA package."""
    import inspect
    from moa_b200 import flashinfer_compat as fi
    assert list(inspect.signature(fi.moa_prefill).parameters) == [
        "q", "k", "v", "causal", "num_global_blocks", "num_band_blocks", "kv_layout"]
    assert list(inspect.signature(fi.moa_decode).parameters) == [
        "q", "k", "v", "head_start_index", "head_valid_length", "sm_scale"]


def _tiny_hf_llama(tie=False):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=2, vocab_size=128, max_position_embeddings=512, rope_theta=10000.0,
                      rms_norm_eps=1e-5, tie_word_embeddings=tie)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).half().eval()


def test_llama_checkpoint_state_dict_loads_as_it_is():
    """Parameter names are those of a HuggingFace Llama checkpoint (`model.layers.N.mlp.*`, `lm_head`), so the
    plan the offline pipeline produces can be run on real weights."""
    hf = _tiny_hf_llama()
    m = moa_b200.MoALlamaForCausalLM.from_config(hf.config.to_dict())
    attn = m.model.layers[0].self_attn
    fused = attn.fused_qkv_weight()                         # the three projections now alias one tensor
    result = m.load_state_dict(hf.state_dict(), strict=True)
    assert not result.missing_keys and not result.unexpected_keys
    assert attn.fused_qkv_weight() is fused                 # loading copied in place, the aliasing survived
    hf_attn = hf.model.layers[0].self_attn
    assert torch.equal(fused, torch.cat([hf_attn.q_proj.weight, hf_attn.k_proj.weight, hf_attn.v_proj.weight]))
    assert m.model.norm.eps == 1e-5 and m.model.rope_theta == 10000.0
    assert torch.equal(m.lm_head.weight, hf.lm_head.weight)


def test_update_model_function_adopts_a_loaded_model_without_copying():
    hf = _tiny_hf_llama()
    m = moa_b200.update_model_function(hf, "meta-llama/Llama-2-7b-hf")
    assert isinstance(m, moa_b200.MoALlamaForCausalLM) and hasattr(m.model, "set_mixture_of_attention")
    assert m.model.layers[1].mlp.down_proj.weight.data_ptr() == hf.model.layers[1].mlp.down_proj.weight.data_ptr()
    assert moa_b200.update_model_function(m, "llama") is m
    tied = moa_b200.update_model_function(_tiny_hf_llama(tie=True), "vicuna")
    assert tied.lm_head.weight.data_ptr() == tied.model.embed_tokens.weight.data_ptr()
    with pytest.raises(NotImplementedError):
        moa_b200.update_model_function(hf, "mistral-7b")
    # a head permutation replaces the projection weights; the fused weight follows
    m.set_mixture_of_attention({"alphas": [[1024.0, 128.0]] * 2, "betas": [[0.0, 0.0]] * 2}, permute_head=True)
    attn, hf_attn = m.model.layers[0].self_attn, hf.model.layers[0].self_attn
    D = 128
    assert torch.equal(attn.fused_qkv_weight()[:D], hf_attn.q_proj.weight[D:])           # head 1 first now
    assert torch.equal(attn.o_proj.weight[:, :D], hf_attn.o_proj.weight[:, D:])


def test_model_head_sharding_slices_weights_and_plan():
    plan_ = {"alphas": [[128.0, 1024.0, 512.0, 256.0]] * 2, "betas": [[0.0, 0.2, 0.0, 0.1]] * 2}
    torch.manual_seed(3)
    ref = moa_b200.MoALlamaModel(2, 64, 4, 128, vocab_size=50, dtype=torch.float32)
    full_q = ref.layers[0].self_attn.q_proj.weight.data.clone()
    full_o = ref.layers[0].self_attn.o_proj.weight.data.clone()
    seen = []
    for rank in range(2):
        torch.manual_seed(3)
        m = moa_b200.MoALlamaModel(2, 64, 4, 128, vocab_size=50, dtype=torch.float32)
        m.set_mixture_of_attention(plan_, moa_max_new_token=0)
        m.shard_heads(2, rank, seq_len=4096)
        sh = m.head_shardings[0]
        attn = m.layers[0].self_attn
        assert attn.num_local_heads == 2 and attn.q_proj.weight.shape == (32, 64)
        assert attn.fused_qkv_weight().shape == (96, 64)
        for i, h in enumerate(sh.local_heads):                        # rows of the local heads, in shard order
            assert torch.equal(attn.q_proj.weight[16 * i:16 * (i + 1)], full_q[16 * h:16 * (h + 1)])
        for i, h in enumerate(sh.order):                              # o_proj columns follow the gathered order
            assert torch.equal(attn.o_proj.weight[:, 16 * i:16 * (i + 1)], full_o[:, 16 * h:16 * (h + 1)])
        assert m.local_moa_config["alphas"][0] == [plan_["alphas"][0][h] for h in sh.local_heads]
        seen += sh.local_heads
        with pytest.raises(AssertionError):
            m.shard_heads(2, rank, seq_len=4096)
    assert sorted(seen) == [0, 1, 2, 3]
