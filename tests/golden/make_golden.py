"""Generate the golden fixtures in this folder by running thu-nics/MoA's own code on CPU.

Run once, in a container that has the MoA checkout (read-only is fine):

    TRITON_INTERPRET=1 PYTHONDONTWRITEBYTECODE=1 MOA_REF=/path/to/MoA \
        python tests/golden/make_golden.py

What runs is the reference, unmodified: ``moa_config_to_cache_config``,
``StaticCircularCache`` (MoA/attention/cache_utils.py), ``moa_config_to_permutation``
(MoA/attention/permutation_utils.py), ``gen_bigbird_pattern``/``gen_causal_pattern``/
``layout_to_mask`` (MoA/attention/pattern.py, convert.py), the Triton prefill kernel
``_sparse_attention_moa_prefill`` (MoA/kernels/block_sparse_attention_prefill.py:631-696) under
the Triton interpreter, and ``mixture_of_sparse_attention(..., implementation="sdpa")``
(MoA/kernels/mixture_of_attention.py:358-427).  One harness-side shim is needed because the
reference targets transformers 4.44: ``transformers.cache_utils.Cache.__init__`` is stubbed.

The fixtures are small (< 3 MB in total) and are what the tests on the GPU machine read; the
MoA checkout is not needed there.
"""

import glob
import json
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
# the reference checkout: MOA_REF, or a directory named "reference" next to this repository
REF = os.environ.get("MOA_REF") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(
    os.path.abspath(__file__))))), "reference")
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

import numpy as np
import torch

import transformers.cache_utils as tcu

tcu.Cache.__init__ = lambda self, *a, **k: None

from MoA.attention.cache_utils import StaticCircularCache, moa_config_to_cache_config  # noqa: E402
from MoA.attention.convert import layout_to_mask  # noqa: E402
from MoA.attention.pattern import gen_bigbird_pattern, gen_causal_pattern  # noqa: E402
from MoA.attention.permutation_utils import moa_config_to_permutation  # noqa: E402
from MoA.kernels.block_sparse_attention_prefill import _sparse_attention_moa_prefill  # noqa: E402
from MoA.kernels.mixture_of_attention import mixture_of_sparse_attention  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def gen_cache_config():
    cases = []
    rng = np.random.RandomState(7)
    for path in sorted(glob.glob(os.path.join(REF, "examples", "*", "moa_alpha_beta.json"))):
        plan = json.load(open(path))
        layers = [0, len(plan["alphas"]) // 2, len(plan["alphas"]) - 1]
        sub = {"alphas": [plan["alphas"][i] for i in layers], "betas": [plan["betas"][i] for i in layers]}
        for seq_len, max_new in [(2048, 0), (16384, 1024), (100, 1024), (65536, 1024)]:
            r = moa_config_to_cache_config(sub, seq_len=seq_len, max_new_token=max_new, verbose=False)
            cases.append({"model": os.path.basename(os.path.dirname(path)), "plan": sub, "seq_len": seq_len,
                          "max_new_token": max_new, "kwargs": {}, "result": r})
    for _ in range(12):
        H = int(rng.randint(1, 9))
        plan = {"alphas": [[float(rng.choice([-1024, -100.5, 0, 63, 64, 65, 128, 1000.7, 4096])) for _ in range(H)]],
                "betas": [[float(rng.choice([0, 0.01, 0.125, 0.3333, 0.5, 1.0, 1.5])) for _ in range(H)]]}
        seq_len, max_new = int(rng.randint(1, 5000)), int(rng.choice([0, 1, 1024]))
        kw = {"sink_size": int(rng.choice([64, 128, 4])), "minimum_cache_size": int(rng.choice([128, 64, 256])),
              "split_size": int(rng.choice([64, 32, 128]))}
        r = moa_config_to_cache_config(plan, seq_len=seq_len, max_new_token=max_new, verbose=False, **kw)
        cases.append({"model": "random", "plan": plan, "seq_len": seq_len, "max_new_token": max_new,
                      "kwargs": kw, "result": r})
    json.dump(cases, open(os.path.join(OUT, "cache_config.json"), "w"))
    print("cache_config cases", len(cases))


def gen_permutation():
    cases = []
    for path in sorted(glob.glob(os.path.join(REF, "examples", "*", "moa_alpha_beta.json")))[:3]:
        plan = json.load(open(path))
        sub = {"alphas": plan["alphas"][:3], "betas": plan["betas"][:3]}
        perms, clusters = moa_config_to_permutation(sub)
        cases.append({"plan": sub, "perms": [p.tolist() for p in perms],
                      "clusters": [{str(k): list(v) for k, v in c.items()} for c in clusters]})
    json.dump(cases, open(os.path.join(OUT, "permutation.json"), "w"))


def coded(B, H, n, D, base):
    """K/V whose value identifies (b, h, token): every slot's occupant can be read back."""
    t = torch.arange(n, dtype=torch.float32)[None, None, :, None] + base
    h = torch.arange(H, dtype=torch.float32)[None, :, None, None] * 10000.0
    b = torch.arange(B, dtype=torch.float32)[:, None, None, None] * 1000000.0
    return (t + h + b).expand(B, H, n, D).contiguous()


def run_trace(name, cache_size, static_size, B, D, prefill_lens, n_prefill, decode_steps, use_mask):
    """Drive the reference cache: one prefill of n_prefill tokens (left padded per row when
    use_mask) followed by decode steps; record the metadata after every update."""
    cache = StaticCircularCache(cache_size=cache_size, static_size=static_size, batch_size=B, head_dim=D,
                                device="cpu", dtype=torch.float32)
    H = len(cache_size[0])
    mask = None
    if use_mask:
        mask = torch.zeros(B, n_prefill, dtype=torch.int64)
        for i, L in enumerate(prefill_lens):
            mask[i, n_prefill - L:] = 1
    rec = {k: [] for k in ("update_index", "valid_length", "mask_cache", "key0", "val0", "kv_len")}

    def snap():
        rec["update_index"].append(cache.cache_update_index[0].clone().numpy())
        rec["valid_length"].append(cache.cache_valid_length[0].clone().numpy())
        rec["mask_cache"].append(cache.mask_cache[0].clone().numpy())
        rec["key0"].append(cache.key_cache[0][..., 0].clone().numpy())
        rec["val0"].append(cache.value_cache[0][..., 0].clone().numpy())
        rec["kv_len"].append(cache._kv_len[0])

    base = 0
    k = coded(B, H, n_prefill, D, base)
    cache.update(k, k + 0.5, 0, mask)
    base += n_prefill
    snap()
    for _ in range(decode_steps):
        k = coded(B, H, 1, D, base)
        cache.update(k, k + 0.5, 0, None)
        base += 1
        snap()
    np.savez_compressed(
        os.path.join(OUT, f"cache_trace_{name}.npz"),
        cache_size=np.asarray(cache_size), static_size=np.asarray(static_size), B=B, D=D,
        n_prefill=n_prefill, decode_steps=decode_steps, use_mask=int(use_mask),
        prefill_lens=np.asarray(prefill_lens),
        head_index=cache.head_index[0].numpy(),
        head_start=cache.cache_head_start_index[0].numpy(),
        **{k: np.stack(v) for k, v in rec.items()})
    print("trace", name, "steps", decode_steps)


def gen_traces():
    # the scenario of the reference's own print-only smoke (cache_utils.py:1301-1371)
    run_trace("smoke", [[5, 10]], [[2, 3]], 3, 4, [14, 9, 5], 14, 9, True)
    run_trace("wrap", [[128, 192, 320]], [[64, 64, 64]], 2, 4, [300, 300], 300, 200, False)
    run_trace("short", [[128, 256]], [[64, 64]], 2, 4, [50, 50], 50, 260, False)
    run_trace("leftpad", [[128, 256]], [[64, 64]], 3, 4, [400, 250, 30], 400, 150, True)
    run_trace("exact", [[128, 128]], [[64, 64]], 1, 4, [128], 128, 70, False)
    run_trace("nostatic", [[64, 96]], [[0, 0]], 2, 4, [100, 100], 100, 100, False)
    run_trace("one", [[128]], [[64]], 1, 4, [2], 2, 140, False)


def gen_layouts():
    out = {}
    for nb, sink_b, L in [(4, 1, 1), (8, 1, 2), (8, 1, 3), (16, 1, 7), (16, 1, 16), (16, 1, 40), (32, 1, 5), (5, 1, 2)]:
        lay = gen_bigbird_pattern(nb, nb, 2 * L - 1, sink_b, 0).squeeze() & gen_causal_pattern(nb, nb).squeeze()
        out[f"layout_{nb}_{sink_b}_{L}"] = lay.numpy()
    lay = gen_bigbird_pattern(4, 4, 3, 1, 0).squeeze() & gen_causal_pattern(4, 4).squeeze()
    out["mask_4_1_2"] = layout_to_mask(lay[None], 64, True)[0].numpy()
    np.savez_compressed(os.path.join(OUT, "layouts.npz"), **out)
    print("layouts", len(out))


def masked_fp32(q, k, v, sm_scale, mask):
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * sm_scale
    s = s.masked_fill(~mask, float("-inf"))
    return torch.matmul(torch.softmax(s, -1), v.float())


def gen_prefill():
    g = torch.Generator().manual_seed(11)
    # (a) block-sparse, N multiple of 64: Triton kernel + fp32 attention under the reference-built mask
    B, H, N, D = 1, 3, 320, 128
    q, k, v = (torch.randn(B, H, N, D, generator=g).to(torch.float16) for _ in range(3))
    sm = D ** -0.5
    sink_b = torch.tensor([1, 1, 1])
    local_b = torch.tensor([1, 2, 4])
    tri = _sparse_attention_moa_prefill.apply(q, k, v, sm, sink_b, local_b, 64, 64)
    nb = N // 64
    ref32 = torch.empty(B, H, N, D)
    for h in range(H):
        lay = gen_bigbird_pattern(nb, nb, 2 * int(local_b[h]) - 1, int(sink_b[h]), 0).squeeze() & \
            gen_causal_pattern(nb, nb).squeeze()
        m = layout_to_mask(lay[None], 64, True)[0]
        ref32[:, h] = masked_fp32(q[:, h], k[:, h], v[:, h], sm, m)
    np.savez_compressed(os.path.join(OUT, "prefill_sparse.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(), sm_scale=sm,
                        sink_blocks=sink_b.numpy(), local_blocks=local_b.numpy(),
                        triton_fp16=tri.transpose(1, 2).contiguous().numpy(),
                        masked_fp32=ref32.transpose(1, 2).contiguous().numpy())
    # (b) ragged N: Triton kernel only (the reference utilities need N % 64 == 0)
    B, H, N, D = 2, 2, 200, 128
    q, k, v = (torch.randn(B, H, N, D, generator=g).to(torch.float16) for _ in range(3))
    sink_b, local_b = torch.tensor([1, 1]), torch.tensor([1, 2])
    tri = _sparse_attention_moa_prefill.apply(q, k, v, sm, sink_b, local_b, 64, 64)
    np.savez_compressed(os.path.join(OUT, "prefill_ragged.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(), sm_scale=sm,
                        sink_blocks=sink_b.numpy(), local_blocks=local_b.numpy(),
                        triton_fp16=tri.transpose(1, 2).contiguous().numpy())
    # (c) the reference's own prefill test: B2 H4 N128 D128, torch.rand, sm_scale 0.1,
    #     sink = local = 64 tokens => dense causal; "sdpa" vs "moa" at rtol=atol=1e-3
    #     (tests/attention_kernel_test.py:35-76)
    B, H, N, D = 2, 4, 128, 128
    q, k, v = (torch.rand(B, H, N, D, generator=g).to(torch.float16) for _ in range(3))
    sink = torch.full((H,), 64, dtype=torch.int64)
    local = torch.full((H,), 64, dtype=torch.int64)
    sdpa = mixture_of_sparse_attention(q, k, v, 0.1, implementation="sdpa", sink_size=sink, local_size=local)
    moa = mixture_of_sparse_attention(q, k, v, 0.1, implementation="moa", sink_size=sink, local_size=local)
    np.savez_compressed(os.path.join(OUT, "prefill_reftest.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(), sm_scale=0.1,
                        sink_size=sink.numpy(), local_size=local.numpy(), sdpa=sdpa.numpy(), moa=moa.numpy())
    print("prefill fixtures done")


def gen_decode():
    g = torch.Generator().manual_seed(5)
    B, D = 2, 128
    caps = [128, 128, 256, 320]
    H = len(caps)
    cache = StaticCircularCache(cache_size=[caps], static_size=[[64] * H], batch_size=B, head_dim=D,
                                device="cpu", dtype=torch.float16)
    N = 400
    k = torch.randn(B, H, N, D, generator=g).to(torch.float16)
    v = torch.randn(B, H, N, D, generator=g).to(torch.float16)
    cache.update(k, v, 0)
    outs, qs, ks, vs = [], [], [], []
    sm = D ** -0.5
    for _ in range(3):
        q1 = torch.randn(B, H, 1, D, generator=g).to(torch.float16)
        k1 = torch.randn(B, H, 1, D, generator=g).to(torch.float16)
        v1 = torch.randn(B, H, 1, D, generator=g).to(torch.float16)
        kc, vc = cache.update(k1, v1, 0)
        o = mixture_of_sparse_attention(q1, kc, vc, sm, head_start_index=cache.cache_head_start_index[0],
                                        head_valid_length=cache.cache_valid_length[0], implementation="sdpa")
        outs.append(o.numpy()); qs.append(q1.numpy()); ks.append(k1.numpy()); vs.append(v1.numpy())
    np.savez_compressed(os.path.join(OUT, "decode_sdpa.npz"), caps=np.asarray(caps), k_prefill=k.numpy(),
                        v_prefill=v.numpy(), q=np.stack(qs), k_new=np.stack(ks), v_new=np.stack(vs),
                        out=np.stack(outs), sm_scale=sm, key_cache_final=cache.key_cache[0].numpy(),
                        update_index_final=cache.cache_update_index[0].numpy())
    print("decode fixture done")


if __name__ == "__main__":
    gen_cache_config()
    gen_permutation()
    gen_traces()
    gen_layouts()
    gen_prefill()
    gen_decode()
