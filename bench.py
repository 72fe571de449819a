#!/usr/bin/env python
"""Benchmark of the MoA attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (config 1 of BASELINE.json): one layer of MoA decode with circular KV caches —
batch 16, 32 heads, head_dim 128, fp16, per-head capacity 64 sinks + window W_h drawn from
{256, 512, 1024, 2048, 4096} (heads sorted by W, as the reference's permute_head arranges),
caches filled from a 16k-token random sequence, then decode steps with one new token per
sequence.  A "step" is one fused decode launch (ring append + flash-decoding + bookkeeping)
over one batch.  `value` is decode tokens/s with the step inputs resident in HBM; `e2e` is the
same loop through the public API with the step's q/k/v coming from pinned host memory and
the step's output copied back (copies double-buffered on their own streams, so they overlap the
neighbouring steps' kernels).  The K/V working set (about 0.55 GB at the default seed) is larger
than L2 (126 MB), so no L2 flush is needed between steps.

With N > 1 (torchrun) every rank owns the ring caches of one 32-head shard (heads, or equally
layers' caches, sharded; no collective on the data path), so per-GPU work is fixed ("weak").

A second, informational leg times the block-sparse prefill kernel on one layer of BASELINE.json
config 3 (B1 H32 N65536 D128 bf16) and reports dense-equivalent TFLOP/s on the band.

`--impl reference` times the CPU restatement of the reference's own path (ring update +
grouped SDPA, oracle/moa_oracle.py) on the host cores, on the same config.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, H, D = 16, 32, 128
PREFILL_TOKENS = 16384
WINDOWS = (256, 512, 1024, 2048, 4096)
SINK = 64
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# DRAM bytes per byte of algorithmic traffic for the decode kernel (dram__bytes_read.sum +
# dram__bytes_write.sum over moa_b200.decode_bytes) from the ncu capture summarised in
# profiles/decode_config1_ncu.md (taken at batch 4; traffic grows in proportion to the rows streamed).
DECODE_DRAM_TRAFFIC_RATIO = 1.027
# DRAM bytes per prefill launch relative to "Q, K, V read once, O written once" (profiles/prefill_config3_ncu.md)
PREFILL_DRAM_TRAFFIC_RATIO = 0.967


def config1_caps(seed: int):
    rng = np.random.RandomState(seed)
    w = sorted(int(x) for x in rng.choice(WINDOWS, H))
    return [SINK + x for x in w]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", ident, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, windows):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7 or not any(a - 0.06 <= ts <= b + 0.06 for a, b in windows):
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's own path restated (oracle), on the host cores
# ----------------------------------------------------------------------------------------------
def cpu_decode_tok_per_s(caps, steps: int, seed: int):
    from oracle import moa_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    S = sum(caps)
    caps_t = torch.tensor(caps)
    head_index = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(caps_t, 0)])
    state = {
        "key_cache": torch.randn(B, S, D, generator=g).half(), "value_cache": torch.randn(B, S, D, generator=g).half(),
        "valid_length": caps_t[None].repeat(B, 1), "max_length": caps_t, "static": torch.full((H,), SINK),
        "circ": caps_t - SINK, "circ_start": head_index[:-1] + SINK, "kv_len": PREFILL_TOKENS,
    }
    # write pointer where a 16k-token fill leaves it: ring offset (16384 - 64) mod W
    state["update_index"] = (state["circ_start"] + (PREFILL_TOKENS - SINK) % state["circ"])[None].repeat(B, 1)
    sm = D ** -0.5
    qs = [tuple(torch.randn(B, H, 1, D, generator=g).half() for _ in range(3)) for _ in range(min(steps, 8))]

    def one(i):
        q, k, v = qs[i % len(qs)]
        orc.ring_cache_step_torch(state, k, v)
        return orc.decode_attention_grouped_sdpa(q, state["key_cache"], state["value_cache"], head_index, sm)

    one(0)
    t0 = time.perf_counter()
    for i in range(steps):
        one(i)
    dt = time.perf_counter() - t0
    return B * steps / dt, dt / steps, torch.get_num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    caps = config1_caps(1000)
    warm = max(1, min(args.warmup, 3))
    cpu_decode_tok_per_s(caps, warm, 1000)
    steps = max(1, min(args.steps, 200))
    val, per_step, cores = cpu_decode_tok_per_s(caps, steps, 1000)
    line = {
        "impl": "reference", "metric": "moa_decode_tokens_per_s", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "config1: one-layer MoA decode, B16 H32 D128 fp16, caps 64+W_h, W_h in {256..4096}",
                   "batch": B, "heads": H, "head_dim": D, "kv_slots_per_row": sum(caps)},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} decode steps at full config-1 size (rings pre-filled with random data, "
                                   "write pointers where a 16k-token fill leaves them); ring update + grouped SDPA "
                                   "as in the reference's implementation='sdpa' path"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def build_cache(caps, device, seed, fill_tokens):
    import moa_b200

    gen = torch.Generator(device=device).manual_seed(seed)
    cache = moa_b200.StaticCircularCache([caps], B, D, [[SINK] * H], device, torch.float16)
    k = torch.randn(B, H, fill_tokens, D, generator=gen, device=device, dtype=torch.float16)
    v = torch.randn(B, H, fill_tokens, D, generator=gen, device=device, dtype=torch.float16)
    cache.update(k, v, 0)
    torch.cuda.synchronize(device)
    del k, v
    return cache, gen


def time_region(fn, steps, device, dist, drain=None):
    """barrier + sync, CUDA events on the launching stream around exactly `steps` calls, max over ranks.
    `drain` makes the launching stream wait for work the steps put on other streams before the end event."""
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    for i in range(steps):
        fn(i)
    if drain is not None:
        drain()
    e1.record()
    torch.cuda.synchronize(device)
    w1 = time.time()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms, (w0, w1)


def prefill_leg(device, peaks_tf, which, N=65536):
    """One layer of config 3: B1 H32 N65536 D128 bf16, alpha in {512..4096}, beta in [0, 0.3).
    (A smaller N is only for profiler captures.)"""
    import moa_b200

    try:
        rng = np.random.RandomState(3000)
        Hp = 32
        plan = {"alphas": [[float(rng.choice([512, 1024, 2048, 4096])) for _ in range(Hp)]],
                "betas": [[float(rng.uniform(0, 0.3)) for _ in range(Hp)]]}
        cfg = moa_b200.moa_config_to_cache_config(plan, N, 0, verbose=False)
        caps, static = cfg["cache_size"][0], cfg["static_size"][0]
        sink_b = [s // 64 for s in static]
        local_b = [(c - s) // 64 for c, s in zip(caps, static)]
        gen = torch.Generator(device=device).manual_seed(3000)
        q, k, v = (torch.randn(1, Hp, N, D, generator=gen, device=device, dtype=torch.bfloat16) for _ in range(3))
        sb = torch.tensor(sink_b, dtype=torch.int32, device=device)
        lb = torch.tensor(local_b, dtype=torch.int32, device=device)
        out = torch.empty(1, N, Hp, D, dtype=torch.bfloat16, device=device)
        sm = D ** -0.5
        for _ in range(3):
            moa_b200.sparse_prefill(q, k, v, sm, sb, lb, out=out)
        moa_b200.check_device_status(device)
        iters = 5 if N <= 65536 else 3
        # Timed the way the tensor peak it is compared with was measured (single launches, best of N, CUDA
        # events on the launching stream); the mean of the same launches back to back is reported beside it.
        times = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            moa_b200.sparse_prefill(q, k, v, sm, sb, lb, out=out)
            e1.record()
            torch.cuda.synchronize(device)
            times.append(e0.elapsed_time(e1))
        moa_b200.check_device_status(device)
        ms_best, ms_mean = min(times), sum(times) / len(times)
        flops = moa_b200.prefill_flops(1, N, D, sink_b, local_b)
        tf = flops / (ms_best * 1e-3) / 1e12
        return {"workload": f"config3 one layer: block-sparse prefill B1 H32 N{N} D128 bf16",
                "tflops_band_dense_equiv": tf, "ms_per_layer": ms_best, "flop_per_layer": flops,
                "timing": f"best of {iters} single launches (as the peak was measured)",
                "tflops_mean_of_launches": flops / (ms_mean * 1e-3) / 1e12,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks_tf, "unit": "TFLOP/s",
                             "frac": tf / peaks_tf, "peak_source": which,
                             "traffic": PREFILL_DRAM_TRAFFIC_RATIO * 4 * Hp * N * D * 2}}
    except Exception as exc:  # the decode headline must still be reported
        return {"error": f"{type(exc).__name__}: {exc}"}


def model_leg(device, steps: int = 8, warmup: int = 3, batch: int = 32, context: int = 16384, layers: int = 32):
    """Informational: config 2 of BASELINE.json — Vicuna-7B-16k architecture (32 layers, hidden 4096, 32 heads x 128,
    FFN 11008, RoPE, fp16) with random-init weights, decode with batch 32 at 16k context on one GPU.
    The per-layer plan is drawn as in config 0 with N = 16384; the ring caches are filled layer by layer
    from random K/V (a 16k-token model prefill at batch 32 is not part of this leg).  One step = one new
    token for every sequence through all layers (GEMMs are library kernels, attention is the fused
    decode launch of this package)."""
    import moa_b200

    rng = np.random.RandomState(2000)
    hidden, heads, ffn = 4096, 32, 11008
    plan = {"alphas": [[float(rng.choice([128, 256, 512, 1024])) for _ in range(heads)] for _ in range(layers)],
            "betas": [[float(rng.uniform(0, 0.5)) for _ in range(heads)] for _ in range(layers)]}
    model = moa_b200.MoALlamaModel(layers, hidden, heads, ffn, vocab_size=32000, rope_theta=10000.0,
                                   dtype=torch.float16, device=device)
    gen = torch.Generator(device=device).manual_seed(2000)
    for prm in model.parameters():
        if prm.dim() > 1:
            prm.data.normal_(0, 0.02, generator=gen)
    model.set_mixture_of_attention(plan, permute_head=True, moa_max_new_token=1024)
    cache = model.new_cache(batch, context)
    kv_bytes = 0
    for layer in range(layers):
        k = torch.randn(batch, heads, context, 128, generator=gen, device=device, dtype=torch.float16)
        cache.update(k, k, layer)          # same tensor for K and V: only sizes and traffic matter here
        kv_bytes += 2 * batch * cache.layer_cache_size[layer] * 128 * 2
        del k
    torch.cuda.synchronize(device)
    ids = torch.randint(0, 32000, (batch, 1), device=device, generator=gen)

    def step(i):
        model(ids, past_key_values=cache)

    for i in range(warmup):
        step(i)
    ms, _ = time_region(step, steps, device, None)
    weights = sum(prm.numel() for prm in model.parameters() if prm.dim() > 1 and prm is not model.embed_tokens.weight) * 2
    per_step = ms / steps
    return {"workload": f"config2: Vicuna-7B-16k architecture, random weights, decode B{batch} at {context} context, "
                        f"{layers} layers, 1 GPU", "tokens_per_s": batch / (per_step * 1e-3), "ms_per_step": per_step,
            "kv_bytes_per_step": kv_bytes, "weight_bytes_per_step": weights,
            "hbm_gbs": (kv_bytes + weights) / (per_step * 1e-3) / 1e9}


def layer_leg(device, dist, world: int, rank: int, steps: int = 64, warmup: int = 5):
    """Informational: the attention part of one decode step of one layer of config 4 of BASELINE.json (Llama-3-70B as
    MHA: 64 heads x 128, bf16, batch 64, per-head window drawn from U[1k, 16k] rounded to 64, plus 64 sinks,
    rings full).  The 64 heads are placed on the ranks by cost (longest-processing-time packing); every rank
    runs the fused decode launch on its shard and the outputs are all-gathered over NCCL into (B, 1, 64, D).
    Strong scaling: the layer is fixed, the work per GPU shrinks with the number of GPUs."""
    import moa_b200

    Bl, Hl, Dl = 64, 64, 128
    rng = np.random.RandomState(4000)
    caps = [SINK + int(-(-int(w) // 64) * 64) for w in rng.uniform(1024, 16384, Hl)]
    sh = moa_b200.HeadSharding(caps, world, rank, group=None)
    mine = sh.slice_plan(caps)
    gen = torch.Generator(device=device).manual_seed(4000 + rank)
    cache = moa_b200.StaticCircularCache([mine], Bl, Dl, [[SINK] * len(mine)], device, torch.bfloat16)
    fill = max(mine)
    k = torch.randn(Bl, len(mine), fill, Dl, generator=gen, device=device, dtype=torch.bfloat16)
    cache.update(k, k, 0)            # same tensor for K and V: only sizes and traffic matter here
    del k
    trio = [torch.randn(Bl, len(mine), 1, Dl, generator=gen, device=device, dtype=torch.bfloat16) for _ in range(3)]
    out = torch.empty(Bl, 1, len(mine), Dl, dtype=torch.bfloat16, device=device)
    sm = Dl ** -0.5

    def step(i):
        cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)
        sh.all_gather(out)

    for i in range(warmup):
        step(i)
    ms, _ = time_region(step, steps, device, dist)

    # The step after attention: o_proj (hidden 8192) in its gathered and its row-parallel form, and the
    # gathered form with the batch split in two so that one half's all-gather runs under the other half's
    # attention.
    hidden = Hl * Dl
    w_full = torch.randn(hidden, Hl * Dl, generator=gen, device=device, dtype=torch.bfloat16) * 0.02
    w_loc = sh.local_output_columns(w_full, Dl).contiguous()

    def step_gather(i):
        cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)
        sh.output_projection(out, w_full, mode="gather")

    def step_row(i):
        cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)
        sh.output_projection(out, w_loc, mode="row_parallel")

    res = {}
    for name, fn in (("gather", step_gather), ("row_parallel", step_row)):
        for i in range(warmup):
            fn(i)
        t, _ = time_region(fn, steps, device, dist)
        res[name + "_us"] = t / steps * 1e3

    half = Bl // 2
    halves = []
    for part in range(2):
        c = moa_b200.StaticCircularCache([mine], half, Dl, [[SINK] * len(mine)], device, torch.bfloat16)
        kk = torch.randn(half, len(mine), fill, Dl, generator=gen, device=device, dtype=torch.bfloat16)
        c.update(kk, kk, 0)
        del kk
        halves.append((c, [t[part * half:(part + 1) * half].contiguous() for t in trio],
                       torch.empty(half, 1, len(mine), Dl, dtype=torch.bfloat16, device=device)))

    def step_overlap(i):
        handles = []
        for part, (c, tr, o) in enumerate(halves):
            c.decode_attention(tr[0], tr[1], tr[2], 0, sm, out=o)
            handles.append(sh.all_gather_start(o, slot=part))
        for h in handles:
            full = sh.all_gather_finish(h)
            torch.nn.functional.linear(full.reshape(half, 1, Hl * Dl), w_full)

    for i in range(warmup):
        step_overlap(i)
    t, _ = time_region(step_overlap, steps, device, dist)
    res["gather_two_microbatches_us"] = t / steps * 1e3

    kv_bytes_all = moa_b200.decode_bytes(Bl, caps, Dl, 2)
    loads = [sum(caps[h] for h in s) for s in sh.shards]
    return {"workload": "config4 one layer, attention + all-gather: B64 H64 D128 bf16, windows U[1k,16k] + 64 sinks, "
                        f"heads sharded over {world} GPU(s)", "us_per_step": ms / steps * 1e3,
            "tokens_per_s": Bl / (ms / steps * 1e-3), "aggregate_hbm_gbs": kv_bytes_all / (ms / steps * 1e-3) / 1e9,
            "allgather_bytes_per_step": Bl * Hl * Dl * 2 if world > 1 else 0,
            "shard_imbalance": max(loads) / (sum(loads) / len(loads)),
            "with_o_proj": dict(res, note="attention + o_proj (8192 x 8192 bf16): gathered form, row-parallel form "
                                          "(all-reduce of partial products), gathered form in two micro-batches "
                                          "with the all-gather started asynchronously")}


def run_gpu(args):
    import moa_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the kernels have no CPU path); use --impl reference for the CPU arm")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("nccl", device_id=device)
        dist = dist_mod

    if args.leg == "prefill":
        hbm_peak, tf_peak, which = measured_peaks()
        print(json.dumps({"prefill": prefill_leg(device, tf_peak, which, args.prefill_n)}), flush=True)
        return
    if args.leg == "model":
        print(json.dumps({"model": model_leg(device, steps=max(1, min(args.steps, 16)))}), flush=True)
        return
    seed = 1000 + rank
    caps = config1_caps(1000)       # same capacities on every rank; data differs by rank
    cache, gen = build_cache(caps, device, seed, args.fill_tokens)
    sm = D ** -0.5
    n_pool = 8
    pool = [tuple(torch.randn(B, H, 1, D, generator=gen, device=device, dtype=torch.float16) for _ in range(3))
            for _ in range(n_pool)]
    out = torch.empty(B, 1, H, D, dtype=torch.float16, device=device)

    def step_resident(i):
        q, k, v = pool[i % n_pool]
        cache.decode_attention(q, k, v, 0, sm, out=out)

    # end-to-end: q/k/v of the step come from pinned host memory, the output goes back to it
    # (the host keeps q, k, v of a step packed in one pinned buffer, so a step costs one copy each way;
    # the copies run on their own streams, double-buffered, so that the upload of step i+1 and the
    # download of step i-1 overlap the kernel of step i — every step still uploads its inputs and downloads
    # its output inside the timed region)
    host_in = [torch.stack([t.cpu() for t in trio]).pin_memory() for trio in pool]
    dev_in = [torch.empty(3, B, H, 1, D, dtype=torch.float16, device=device) for _ in range(2)]
    dev_out = [torch.empty(B, 1, H, D, dtype=torch.float16, device=device) for _ in range(2)]
    host_out = [torch.empty(B, 1, H, D, dtype=torch.float16).pin_memory() for _ in range(2)]
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]
    main = torch.cuda.current_stream(device)
    for ev in in_free + out_free:
        ev.record(main)

    def step_e2e(i):
        s = i & 1
        with torch.cuda.stream(up):
            up.wait_event(in_free[s])
            dev_in[s].copy_(host_in[i % n_pool], non_blocking=True)
            in_ready[s].record(up)
        main.wait_event(in_ready[s])
        main.wait_event(out_free[s])
        cache.decode_attention(dev_in[s][0], dev_in[s][1], dev_in[s][2], 0, sm, out=dev_out[s])
        in_free[s].record(main)
        out_ready[s].record(main)
        with torch.cuda.stream(down):
            down.wait_event(out_ready[s])
            host_out[s].copy_(dev_out[s], non_blocking=True)
            out_free[s].record(down)

    def e2e_drain():
        main.wait_stream(up)
        main.wait_stream(down)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    warm = max(args.warmup, 3)
    for i in range(warm):
        step_resident(i)
    ms, win1 = time_region(step_resident, args.steps, device, dist)
    for i in range(warm):
        step_e2e(i)
    e2e_drain()
    ms_e2e, win2 = time_region(step_e2e, args.steps, device, dist, drain=e2e_drain)

    # informational: the same K steps captured once in a CUDA graph and replayed (one graph launch per K steps)
    graph_info = None
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            step_resident(0)
        main.wait_stream(side)
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(args.steps):
                step_resident(i)
        g.replay()
        torch.cuda.synchronize(device)
        ms_graph, _ = time_region(lambda i: g.replay() if i == 0 else None, args.steps, device, dist)
        graph_info = {"us_per_step": ms_graph / args.steps * 1e3,
                      "note": f"{args.steps} decode steps captured in one CUDA graph, one replay timed"}
    except Exception as exc:   # capture is an extra, never a reason to lose the bench line
        graph_info = {"unavailable": repr(exc)[:200]}

    hbm_peak, tf_peak, which = measured_peaks()
    prefill = prefill_leg(device, tf_peak, which, args.prefill_n) if (world == 1 and not args.no_prefill) else None
    layer = layer_leg(device, dist, world, rank) if (world > 1 or args.leg == "layer") else None
    if dist is not None:
        dist.barrier()
    clocks = sampler.stop([win1, win2]) if sampler else None

    if rank == 0:
        tokens = B * args.steps * world
        value = tokens / (ms * 1e-3)
        bytes_per_launch = moa_b200.decode_bytes(B, caps, D, 2)
        achieved = bytes_per_launch / (ms / args.steps * 1e-3) / 1e9
        line = {
            "metric": "moa_decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "config1: one-layer MoA decode, B16 H32 D128 fp16, caps 64+W_h, W_h in {256..4096}, "
                                   "caches filled from a 16k-token random sequence; fused append + flash-decoding",
                       "batch": B, "fill_tokens": args.fill_tokens, "heads_per_gpu": H, "head_dim": D, "kv_slots_per_row": sum(caps),
                       "parallelism": f"head/cache shards x{world}, one 32-head shard per GPU, no collective",
                       "l2": f"K/V working set {moa_b200.decode_bytes(B, caps, D, 2) / 1e6:.0f} MB per step exceeds the "
                             "126 MB L2; no flush between steps",
                       "seed": 1000},
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": 3 * B * H * D * 2, "d2h_bytes_per_step": B * H * D * 2},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_source": which,
                         "algorithmic_bytes_per_launch": bytes_per_launch,
                         "traffic": DECODE_DRAM_TRAFFIC_RATIO * bytes_per_launch},
            "clocks": clocks,
        }
        if graph_info is not None:
            line["cuda_graph"] = graph_info
        if prefill is not None:
            line["prefill"] = prefill
        if layer is not None:
            line["layer_allgather"] = layer
        if world == 1 and not args.no_cpu_baseline:
            val, per_step, cores = cpu_decode_tok_per_s(caps, 30, 1000)
            line["cpu_baseline"] = {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": "30 decode steps at full config-1 size on the host cores (ring update + "
                                              "grouped SDPA, the reference's implementation='sdpa' path restated)"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="moa_b200", choices=["moa_b200", "reference"])
    ap.add_argument("--batch", type=int, default=16, help="batch size (16 = config 1; smaller only for profiler captures)")
    ap.add_argument("--fill-tokens", type=int, default=PREFILL_TOKENS, help="tokens the caches are filled from")
    ap.add_argument("--leg", default="all", choices=["all", "prefill", "model", "layer"],
                    help="'prefill': only the prefill leg; 'model': whole-model decode of config 2; "
                         "'layer': also time the config-4 attention layer with its all-gather (always on with N > 1)")
    ap.add_argument("--prefill-n", type=int, default=65536, help="sequence length of the prefill leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the informational prefill leg")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    global B
    B = args.batch
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
