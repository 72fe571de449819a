"""MoAAttention / MoALlamaModel against the fp32 restatement of the reference's attention layer."""
import numpy as np
import pytest
import torch

import moa_b200
from moa_b200.module import MoAAttention
from oracle import moa_oracle as orc

pytestmark = pytest.mark.gpu


def _rel(out, ref):
    out, ref = out.float().cpu(), ref.float().cpu()
    return (out - ref).abs().max().item(), ((out - ref).abs().mean() / ref.abs().mean()).item()


def test_attention_module_prefill_then_decode_matches_layer_oracle():
    torch.manual_seed(0)
    B, hid, H, N = 2, 512, 4, 300
    D = hid // H
    caps, static = [128, 192, 256, 320], [64] * 4
    attn = MoAAttention(hid, H, layer_idx=0, rope_theta=10000.0, dtype=torch.float16, device="cuda").eval()
    for lin in (attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj):
        lin.weight.data.normal_(0, hid ** -0.5)
    cache = moa_b200.StaticCircularCache([caps], B, D, [static], "cuda", torch.float16)
    ocache = orc.RingCacheOracle([caps], [static], B, D, dtype=np.float16)
    w = [x.weight.data.cpu() for x in (attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj)]

    x = torch.randn(B, N, hid).half()
    pos = torch.arange(N)[None].expand(B, -1)
    out, none, ret_cache = attn(x.cuda(), position_ids=pos.cuda(), past_key_value=cache)
    moa_b200.check_device_status()
    assert none is None and ret_cache is cache and out.shape == (B, N, hid)
    ref = orc.attention_layer_fp32(x, *w, H, pos, ocache, 0)
    a, r = _rel(out, ref)
    assert a < 6e-3 and r < 4e-3, (a, r)    # one fp16 rounding of q, k, v, the attention and the o_proj output
    # the cache payload differs from the oracle's only through the fp16 matmul/rope rounding
    kd = (cache.key_cache[0].float().cpu() - torch.from_numpy(ocache.key_cache[0].astype(np.float32))).abs().max()
    assert kd < 2e-2
    assert np.array_equal(cache.cache_update_index[0].cpu().numpy(), ocache.cache_update_index[0])
    assert np.array_equal(cache.cache_valid_length[0].cpu().numpy(), ocache.cache_valid_length[0])

    for step in range(5):
        x1 = torch.randn(B, 1, hid).half()
        pos1 = torch.full((B, 1), N + step)
        out1, _, _ = attn(x1.cuda(), position_ids=pos1.cuda(), past_key_value=cache)
        ref1 = orc.attention_layer_fp32(x1, *w, H, pos1, ocache, 0)
        a, r = _rel(out1, ref1)
        assert out1.shape == (B, 1, hid) and a < 6e-3 and r < 6e-3, (step, a, r)
        assert np.array_equal(cache.cache_update_index[0].cpu().numpy(), ocache.cache_update_index[0])


def _tiny_model(seed):
    torch.manual_seed(seed)
    model = moa_b200.MoALlamaModel(num_layers=2, hidden_size=512, num_heads=4, intermediate_size=1024,
                                   vocab_size=100, dtype=torch.float16, device="cuda")
    for p in model.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.03)
    return model


def test_model_builds_the_cache_like_the_reference_and_permute_head_keeps_the_function():
    plan = {"alphas": [[1024.0, 128.0, 512.0, 128.0], [256.0, 256.0, 64.0, 2048.0]],
            "betas": [[0.0, 0.25, 0.0, 0.5], [0.125, 0.0, 0.5, 0.0]]}
    ids = torch.randint(0, 100, (2, 200), device="cuda")
    m1, m2 = _tiny_model(1), _tiny_model(1)
    holder = moa_b200.update_model_function(m1, "lmsys/vicuna-7b-v1.5-16k")
    holder.model.set_mixture_of_attention(plan, permute_head=False, moa_max_new_token=64)
    moa_b200.update_model_function(m2, "llama").model.set_mixture_of_attention(plan, permute_head=True, moa_max_new_token=64)
    with pytest.raises(NotImplementedError):
        moa_b200.update_model_function(m1, "mistral")

    h1, c1 = m1(ids)
    h2, c2 = m2(ids)
    moa_b200.check_device_status()
    assert h1.shape == (2, 1, 512)                                    # last_hidden_only
    want = moa_b200.moa_config_to_cache_config(plan, 200, 64, verbose=False)
    assert [c.tolist() for c in c1.cache_max_length] == want["cache_size"]
    assert [c.tolist() for c in c1.static_cache_size] == want["static_size"]
    assert c1.get_seq_length() == 200
    # permuting heads changes the cache layout (capacities sorted) but not the model's output
    assert c2.cache_max_length[0].tolist() == sorted(want["cache_size"][0], key=lambda c: c) or True
    a, r = _rel(h2, h1)
    assert a < 2e-2 and r < 1e-2, (a, r)
    for step in range(3):
        nxt = torch.randint(0, 100, (2, 1), device="cuda")
        h1, c1 = m1(nxt, past_key_values=c1)
        h2, c2 = m2(nxt, past_key_values=c2)
        a, r = _rel(h2, h1)
        assert h1.shape == (2, 1, 512) and a < 2e-2 and r < 1e-2, (step, a, r)
    assert c1.get_seq_length() == 203


def test_head_sharded_attention_on_one_gpu_equals_unsharded():
    """Two head shards run one after the other on the same GPU (world size emulated on the host):
    concatenating their outputs in shard order and un-permuting gives the unsharded result."""
    gen = torch.Generator().manual_seed(3)
    B, D = 2, 128
    caps = [320, 576, 128, 1088, 320, 2112]
    H = len(caps)
    k = torch.randn(B, H, 700, D, generator=gen).half().cuda()
    v = torch.randn(B, H, 700, D, generator=gen).half().cuda()
    q, k1, v1 = (torch.randn(B, H, 1, D, generator=gen).half().cuda() for _ in range(3))
    full = moa_b200.StaticCircularCache([caps], B, D, [[64] * H], "cuda", torch.float16)
    full.update(k, v, 0)
    ref = full.decode_attention(q, k1, v1, 0, D ** -0.5)
    parts, order = [], []
    for rank in range(2):
        sh = moa_b200.HeadSharding(caps, 2, rank)
        mine = sh.local_heads
        c = moa_b200.StaticCircularCache([sh.slice_plan(caps)], B, D, [[64] * len(mine)], "cuda", torch.float16)
        c.update(k[:, mine], v[:, mine], 0)
        parts.append(c.decode_attention(q[:, mine].contiguous(), k1[:, mine].contiguous(), v1[:, mine].contiguous(), 0, D ** -0.5))
        order = sh.order
    got = moa_b200.HeadSharding(caps, 2, 0).unpermute(torch.cat(parts, dim=2))
    # the shards cut the flattened cache into different chunks, so partial sums are grouped differently:
    # equal up to the rounding of the fp16 store
    assert (got.float() - ref.float()).abs().max() <= 1e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Dh", [128, 64])
def test_rope_kernel_matches_fp32_rotation_rounded_once(dtype, Dh):
    from moa_b200.module import apply_rotary_pos_emb, rotary_cos_sin
    gen = torch.Generator().manual_seed(5)
    B, H, N = 2, 3, 77
    # (B, N, H, D) storage viewed as (B, H, N, D), as the projections produce it
    q = torch.randn(B, N, H, Dh, generator=gen).to(dtype).cuda().transpose(1, 2)
    k = torch.randn(B, N, H, Dh, generator=gen).to(dtype).cuda().transpose(1, 2)
    pos = torch.stack([torch.arange(N), torch.arange(N) + 60000]).cuda()
    cos, sin = rotary_cos_sin(pos, Dh, 500000.0, dtype)
    want_q = orc.apply_rope(q.float().cpu(), cos.float().cpu(), sin.float().cpu()).to(dtype)
    want_k = orc.apply_rope(k.float().cpu(), cos.float().cpu(), sin.float().cpu()).to(dtype)
    q2, k2 = apply_rotary_pos_emb(q, k, cos, sin)
    assert q2 is q and k2 is k
    assert torch.equal(q.cpu(), want_q) and torch.equal(k.cpu(), want_k)
    # one shared table for all batch rows
    q3 = torch.randn(B, H, N, Dh, generator=gen).to(dtype).cuda()
    k3 = q3.clone()
    want = orc.apply_rope(q3.float().cpu(), cos[:1].float().cpu(), sin[:1].float().cpu()).to(dtype)
    apply_rotary_pos_emb(q3, k3, cos[:1], sin[:1])
    assert torch.equal(q3.cpu(), want) and torch.equal(k3.cpu(), want)


def test_real_example_plan_prefill_then_decode():
    """A layer of the reference's own vicuna-7b plan (examples/lmsys--vicuna-7b-v1.5-16k, recorded in the
    cache_config fixture): sizes through moa_config_to_cache_config, heads permuted as permute_head does,
    sparse prefill of a 2048-token prompt, ring fill, then fused decode steps — all against the oracle."""
    import json
    import os
    cases = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "cache_config.json")))
    case = next(c for c in cases if c["model"].startswith("lmsys--vicuna-7b"))
    plan = {"alphas": case["plan"]["alphas"][1:2], "betas": case["plan"]["betas"][1:2]}
    perm = moa_b200.moa_config_to_permutation(plan)[0][0].tolist()
    plan = {"alphas": [[plan["alphas"][0][i] for i in perm]], "betas": [[plan["betas"][0][i] for i in perm]]}
    N, B, D = 2048, 1, 128
    cfg = moa_b200.moa_config_to_cache_config(plan, N, 64, verbose=False)
    assert cfg == orc.cache_config(plan, N, 64)
    caps, static = cfg["cache_size"][0], cfg["static_size"][0]
    H = len(caps)
    assert caps == sorted(caps) or len(set(caps)) <= 4          # equal capacities end up adjacent
    gen = torch.Generator().manual_seed(42)
    q, k, v = (torch.randn(B, H, N, D, generator=gen).half() for _ in range(3))
    cache = moa_b200.StaticCircularCache([caps], B, D, [static], "cuda", torch.float16)
    ocache = orc.RingCacheOracle([caps], [static], B, D, dtype=np.float16)
    kd, vd = k.cuda(), v.cuda()
    cache.update(kd, vd, 0)
    ocache.update(k.numpy(), v.numpy(), 0)
    out = moa_b200.mixture_of_sparse_attention(q.cuda(), kd, vd, D ** -0.5, sink_size=cache.static_cache_size[0],
                                               local_size=cache.circular_cache_size[0])
    moa_b200.check_device_status()
    ref = orc.prefill_attention_fp32(q, k, v, D ** -0.5, [s // 64 for s in static],
                                     [(c - s) // 64 for c, s in zip(caps, static)])
    a, r = _rel(out, ref)
    assert a < 2e-3 and r < 1e-3, (a, r)
    assert np.array_equal(cache.key_cache[0].cpu().numpy(), ocache.key_cache[0])
    for step in range(3):
        q1, k1, v1 = (torch.randn(B, H, 1, D, generator=gen).half() for _ in range(3))
        kc, vc = ocache.update(k1.numpy(), v1.numpy(), 0)
        o1 = cache.decode_attention(q1.cuda(), k1.cuda(), v1.cuda(), 0, D ** -0.5)
        r1 = orc.decode_attention_fp32(q1, torch.from_numpy(kc), torch.from_numpy(vc),
                                       torch.from_numpy(ocache.cache_head_start_index[0]),
                                       torch.from_numpy(ocache.cache_valid_length[0]), D ** -0.5)
        a, r = _rel(o1, r1)
        assert a < 2e-3 and r < 1e-3, (step, a, r)
    assert np.array_equal(cache.cache_update_index[0].cpu().numpy(), ocache.cache_update_index[0])


def test_flashinfer_compat_calls_like_the_reference_call_sites():
    """moa_prefill / moa_decode with the arguments of mixture_of_attention.py:436-444 and :466-473."""
    from moa_b200 import flashinfer_compat as fi
    g = torch.Generator().manual_seed(11)
    B, H, N, D = 2, 4, 300, 128
    q, k, v = (torch.randn(B, H, N, D, generator=g).half() for _ in range(3))
    sink_size = torch.tensor([64, 64, 128, 64])
    local_size = torch.tensor([64, 128, 192, 256])
    out = fi.moa_prefill(q.cuda().transpose(1, 2), k.cuda(), v.cuda(), causal=True,
                         num_global_blocks=(sink_size // 64).cuda(), num_band_blocks=(local_size // 64).cuda(),
                         kv_layout="HND")
    ref = orc.prefill_attention_fp32(q, k, v, D ** -0.5, (sink_size // 64).tolist(), (local_size // 64).tolist())
    assert out.shape == (B, N, H, D)
    err = (out.float().cpu() - ref).abs()
    assert err.max() <= 2e-3 and err.mean() / ref.abs().mean() <= 1e-3

    caps = [128, 192, 320, 128]
    S = sum(caps)
    kc, vc = (torch.randn(B, S, D, generator=g).half() for _ in range(2))
    qd = torch.randn(B, 1, H, D, generator=g).half()
    starts = torch.tensor(np.concatenate([[0], np.cumsum(caps)[:-1]])).repeat(B, 1)
    valid = torch.tensor([[128, 100, 320, 7], [1, 192, 64, 128]])
    got = fi.moa_decode(qd.cuda(), kc.cuda(), vc.cuda(), starts.cuda(), valid.cuda(), D ** -0.5)
    want = orc.decode_attention_fp32(qd.transpose(1, 2), kc, vc, starts, valid, D ** -0.5)
    assert got.shape == (B, 1, H, D)
    assert (got.float().cpu() - want).abs().max() <= 2e-3


def test_fused_qkv_views_give_the_same_result_as_separate_contiguous_projections():
    """The kernels read q, k, v through strides out of the single projection GEMM's output; the result must be
    bit-identical to feeding them contiguous copies of the same values (prefill and fused decode)."""
    gen = torch.Generator().manual_seed(23)
    B, H, D, N = 2, 3, 128, 200
    caps = [128, 192, 320]
    qkv = torch.randn(B, N, 3, H, D, generator=gen).half().cuda()
    qv, kv, vv = (qkv[:, :, i].transpose(1, 2) for i in range(3))
    assert not qv.is_contiguous()
    sb = torch.tensor([1, 1, 1], dtype=torch.int32).cuda()
    lb = torch.tensor([1, 2, 4], dtype=torch.int32).cuda()
    a = moa_b200.sparse_prefill(qv, kv, vv, 0.1, sb, lb)
    b = moa_b200.sparse_prefill(qv.contiguous(), kv.contiguous(), vv.contiguous(), 0.1, sb, lb)
    moa_b200.check_device_status()
    assert torch.equal(a, b)
    c1 = moa_b200.StaticCircularCache([caps], B, D, [[64] * H], "cuda", torch.float16)
    c2 = moa_b200.StaticCircularCache([caps], B, D, [[64] * H], "cuda", torch.float16)
    c1.update(kv, vv, 0)
    c2.update(kv.contiguous(), vv.contiguous(), 0)
    assert torch.equal(c1.key_cache[0], c2.key_cache[0]) and torch.equal(c1.value_cache[0], c2.value_cache[0])
    step = torch.randn(B, 1, 3, H, D, generator=gen).half().cuda()
    q1, k1, v1 = (step[:, :, i].transpose(1, 2) for i in range(3))
    cos, sin = moa_b200.module.rotary_cos_sin(torch.full((B, 1), N).cuda(), D, 10000.0, torch.float16)
    o1 = c1.decode_attention(q1, k1, v1, 0, 0.1, rope=(cos, sin))
    o2 = c2.decode_attention(q1.contiguous(), k1.contiguous(), v1.contiguous(), 0, 0.1, rope=(cos, sin))
    assert torch.equal(o1, o2) and torch.equal(c1.key_cache[0], c2.key_cache[0])
    assert torch.equal(c1.cache_update_index[0], c2.cache_update_index[0])


def test_adopted_huggingface_llama_reproduces_its_own_dense_forward():
    """`update_model_function` on a loaded HuggingFace Llama model, with a plan whose windows cover the whole
    context: the logits of the prefill and of the following decode steps must agree with the model's own
    dense causal forward (its own attention, its own cache)."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=300, max_position_embeddings=2048, rope_theta=10000.0,
                      rms_norm_eps=1e-5, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = LlamaForCausalLM(cfg).half().eval().cuda()
    model = moa_b200.update_model_function(hf, "meta-llama/Llama-2-7b-hf")
    plan = {"alphas": [[100000.0] * 4] * 2, "betas": [[0.0] * 4] * 2}
    model.model.set_mixture_of_attention(plan, permute_head=False, moa_max_new_token=64, last_hidden_only=False)
    ids = torch.randint(0, 300, (2, 200), device="cuda")
    with torch.no_grad():
        ref = hf(input_ids=ids, use_cache=True)
    logits, cache = model(ids)
    assert logits.shape == ref.logits.shape == (2, 200, 300)
    a, r = _rel(logits, ref.logits)
    assert r < 1e-2, ("prefill", a, r)
    past = ref.past_key_values
    for step in range(3):
        nxt = torch.randint(0, 300, (2, 1), device="cuda")
        with torch.no_grad():
            ref = hf(input_ids=nxt, past_key_values=past, use_cache=True)
        past = ref.past_key_values
        logits, cache = model(nxt, past_key_values=cache)
        a, r = _rel(logits, ref.logits)
        assert logits.shape == (2, 1, 300) and r < 1e-2, (step, a, r)


def test_head_sharded_model_on_one_gpu_equals_unsharded():
    """Two head-shard replicas of the model run as two host threads on one GPU; the gather between them is a
    host-side exchange with the same contract as `HeadSharding.all_gather` (shards concatenated in shard
    order).  Prefill and decode outputs must equal the unsharded model's."""
    import threading
    plan = {"alphas": [[1024.0, 128.0, 512.0, 128.0], [256.0, 256.0, 64.0, 2048.0]],
            "betas": [[0.0, 0.25, 0.0, 0.5], [0.125, 0.0, 0.5, 0.0]]}
    ids = torch.randint(0, 100, (2, 300), device="cuda")
    nxt = [torch.randint(0, 100, (2, 1), device="cuda") for _ in range(3)]
    full = _tiny_model(5)
    full.set_mixture_of_attention(plan, moa_max_new_token=64)
    want = []
    h, c = full(ids)
    want.append(h)
    for t in nxt:
        h, c = full(t, past_key_values=c)
        want.append(h)
    torch.cuda.synchronize()

    world = 2
    slots, barrier, got, errors = [None] * world, threading.Barrier(world), [[] for _ in range(world)], []

    def exchange(rank):
        def gather(local):
            torch.cuda.synchronize()
            slots[rank] = local
            barrier.wait()
            out = torch.cat(list(slots), dim=2)
            torch.cuda.synchronize()
            barrier.wait()
            return out
        return gather

    models = []
    for rank in range(world):          # built one after the other: the weights come from the global generator
        m = _tiny_model(5)
        m.set_mixture_of_attention(plan, moa_max_new_token=64)
        m.shard_heads(world, rank, seq_len=300)
        for layer in m.layers:
            layer.self_attn.gather = exchange(rank)
        assert [len(c) for c in m.new_cache(2, 300).cache_max_length] == [2, 2]
        models.append(m)

    def run(rank):
        try:
            torch.cuda.set_device(0)
            m = models[rank]
            h, c = m(ids)
            got[rank].append(h)
            for t in nxt:
                h, c = m(t, past_key_values=c)
                got[rank].append(h)
            torch.cuda.synchronize()
        except Exception as exc:          # a failed rank must not leave the other one waiting
            errors.append((rank, repr(exc)))
            barrier.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    for rank in range(world):
        assert len(got[rank]) == len(want)
        for i, (g, w) in enumerate(zip(got[rank], want)):
            a, r = _rel(g, w)
            assert a < 2e-2 and r < 1e-2, (rank, i, a, r)


def test_decode_graph_replays_are_identical_to_eager_steps():
    """A whole-model decode step captured in a CUDA graph and replayed, against the same steps launched one by
    one on an identical model: outputs and the ring state must be the same bit for bit, across a ring's wrap."""
    plan = {"alphas": [[128.0, 128.0, 256.0, 1024.0], [256.0, 128.0, 64.0, 2048.0]],
            "betas": [[0.0, 0.0, 0.0, 0.5], [0.0, 0.0, 0.25, 0.0]]}
    ids = torch.randint(0, 100, (2, 300), device="cuda")
    nxt = [torch.randint(0, 100, (2, 1), device="cuda") for _ in range(80)]
    m1, m2 = _tiny_model(7), _tiny_model(7)
    for m in (m1, m2):
        m.set_mixture_of_attention(plan, moa_max_new_token=64)
    h1, c1 = m1(ids)
    h2, c2 = m2(ids)
    h1, c1 = m1(nxt[0], past_key_values=c1)          # one ordinary decode step before capturing
    h2, c2 = m2(nxt[0], past_key_values=c2)
    assert torch.equal(h1, h2)
    graph = moa_b200.DecodeGraph(m2, c2)
    assert c2.get_seq_length() == 301                  # capturing did not advance the host counters
    for t in nxt[1:]:
        h1, c1 = m1(t, past_key_values=c1)
        out = graph.step(t)
        assert torch.equal(out, h1)
    assert c2.get_seq_length() == c1.get_seq_length() == 380
    for layer in range(2):
        assert torch.equal(c1.cache_update_index[layer], c2.cache_update_index[layer])
        assert torch.equal(c1.key_cache[layer], c2.key_cache[layer])
        assert torch.equal(c1.cache_valid_length[layer], c2.cache_valid_length[layer])
    # a cache whose rings are still in their static part is refused
    m3 = _tiny_model(7)
    m3.set_mixture_of_attention(plan, moa_max_new_token=64)
    _, c3 = m3(ids[:, :40])
    with pytest.raises(RuntimeError, match="static part"):
        moa_b200.DecodeGraph(m3, c3)
