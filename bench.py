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
the step's output copied back.  The K/V working set (about 0.55 GB at the default seed) is larger
than L2 (126 MB), so no L2 flush is needed between steps.

Timing: after W warm-up steps the K steps are timed as a block between two CUDA events on the launching
stream, and the block is repeated R times back to back (R >= 25 and long enough for a quarter of a second
of GPU time, so that short K still gives a steady-state figure and the clock sampler sees the load);
`ms_per_step` is the median block divided by K, with min and max beside it.  With N > 1 (torchrun) every
block time is the maximum over the ranks.

With N > 1 every rank owns the ring caches of one 32-head shard (heads, or equally layers' caches,
sharded; no collective on the data path), so per-GPU work is fixed ("weak").

Further legs on the same line (each with its own roofline): `prefill` — the block-sparse prefill kernel
on one layer of config 3 (B1 H32 N65536 D128 bf16), its 32 heads sharded over the N GPUs, and on config 0
(B1 H32 N2048 fp16) on one GPU; `layer_allgather` — one decode layer of config 4 (64 heads, batch 64,
bf16) with its heads sharded over the N GPUs and the outputs gathered before o_proj (strong scaling);
`model_config2` (alone: `--leg model`) — whole-model decode of config 2 with its heads sharded over the N GPUs.

`--impl reference` times the CPU restatement of the reference's own path (ring update + grouped SDPA,
the oracle under oracle/) on the host cores, on the same config.
"""
from __future__ import annotations

import argparse
import json
import math
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
MIN_BLOCKS = 25            # repeats of the K-step block
MIN_REGION_S = 0.25        # GPU time the repeated blocks should add up to
# DRAM traffic per launch is not measured by this program: it is scaled from one ncu capture of the same
# kernel on a smaller case (decode: batch 4; prefill: N = 32768, the smallest size that runs in the same kernel
# form as config 3), where dram__bytes_read.sum + dram__bytes_write.sum came to these multiples of the
# algorithmic bytes; traffic grows in proportion to the rows streamed (decode) and to the tensor sizes
# (prefill: Q, K, V read once, O written once).
DECODE_DRAM_TRAFFIC_RATIO = 1.027
PREFILL_DRAM_TRAFFIC_RATIO = 0.985


def config1_caps(seed: int):
    rng = np.random.RandomState(seed)
    w = sorted(int(x) for x in rng.choice(WINDOWS, H))
    return [SINK + x for x in w]


def config1_dict(caps, fill_tokens: int, world: int):
    """The `config` object of the bench line — the same for the GPU arm and the reference arm."""
    return {"workload": "config1: one-layer MoA decode, B16 H32 D128 fp16, caps 64+W_h, W_h in {256..4096}, "
                        "caches filled from a 16k-token random sequence; ring append + decode attention per step",
            "batch": B, "fill_tokens": fill_tokens, "heads_per_gpu": H, "head_dim": D, "kv_slots_per_row": sum(caps),
            "parallelism": f"head/cache shards x{world}, one 32-head shard per GPU, no collective",
            "l2": f"K/V working set {decode_bytes_of(caps) / 1e6:.0f} MB per step exceeds the 126 MB L2; "
                  "no flush between steps",
            "seed": 1000}


def decode_bytes_of(caps, batch=None, itemsize=2):
    b = B if batch is None else batch
    return b * int(sum(caps)) * D * 2 * itemsize + 4 * b * len(caps) * D * itemsize


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (read-only query) while the timed regions run."""

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
                ["nvidia-smi", "-i", ident, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
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
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7 or not any(a <= ts <= b + 0.03 for a, b in windows):
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


def cpu_prefill_tflops(q, k, v, sm, sink_b, local_b, flops):
    """The PyTorch CPU route (one SDPA call with the boolean mask) on host tensors; timed in fp32 and in the
    tensors' own dtype, the faster of the two is reported."""
    from oracle import moa_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)
    best, which = None, None
    for name, cast in (("fp32", torch.float32), (str(q.dtype)[6:], q.dtype)):
        qq, kk, vv = q.to(cast), k.to(cast), v.to(cast)
        t0 = time.perf_counter()
        orc.prefill_attention_masked_sdpa(qq, kk, vv, sm, sink_b, local_b)
        dt = time.perf_counter() - t0
        if best is None or dt < best:
            best, which = dt, name
    return flops / best / 1e12, best, which, torch.get_num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
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
        "config": config1_dict(caps, args.fill_tokens, max(world, args.gpus)),
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


def time_blocks(fn, steps, device, dist, drain=None, min_blocks=MIN_BLOCKS, min_region_s=MIN_REGION_S, est_ms=None):
    """Times `steps` calls of fn as one block between two CUDA events on the launching stream, repeated R times
    back to back (barrier + synchronize before the first and after the last block).  Returns the per-block
    times in ms (element-wise maximum over the ranks), and the wall-clock window of the whole region.
    `drain` makes the launching stream wait for work the steps put on other streams before a block's end event."""
    if est_ms is None:       # one untimed block to size R
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        for i in range(steps):
            fn(i)
        if drain is not None:
            drain()
        torch.cuda.synchronize(device)
        est_ms = (time.perf_counter() - t0) * 1e3
    reps = int(max(min_blocks, min(5000, math.ceil(min_region_s * 1e3 / max(est_ms, 1e-3)))))
    if dist is not None:     # every rank must run the same number of blocks
        t = torch.tensor([reps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        reps = int(t.item())
        dist.barrier()
    torch.cuda.synchronize(device)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    w0 = time.time()
    events[0].record()
    for r in range(reps):
        for i in range(steps):
            fn(r * steps + i)
        if drain is not None:
            drain()
        events[r + 1].record()
    torch.cuda.synchronize(device)
    w1 = time.time()
    ms = torch.tensor([events[r].elapsed_time(events[r + 1]) for r in range(reps)], device=device)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
    return ms.tolist(), (w0, w1)


def block_stats(ms_list, steps):
    med = statistics.median(ms_list)
    return {"blocks": len(ms_list), "steps_per_block": steps, "ms_per_step_median": med / steps,
            "ms_per_step_min": min(ms_list) / steps, "ms_per_step_max": max(ms_list) / steps,
            "timed_region_ms": sum(ms_list)}


def time_single_launches(fn, iters, device, dist, behind=None):
    """Single launches, each between its own pair of CUDA events with a synchronize on both sides (the way the
    burst tensor peak was measured); with several ranks a barrier precedes every launch and the time of a
    launch is the maximum over the ranks.  `behind`, if given, is enqueued right before the first event and is
    still running while the host enqueues the launch, so that the launch's host-side cost (tensor maps, the call
    itself: 15-20 us) is not inside the event pair; it is used to flush L2 for inputs that would fit in it."""
    times = []
    for _ in range(iters):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)
        if behind is not None:
            behind()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(device)
        times.append(e0.elapsed_time(e1))
    t = torch.tensor(times, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def draw_plan(seed, heads, alphas, beta_max, N):
    import moa_b200

    rng = np.random.RandomState(seed)
    plan = {"alphas": [[float(rng.choice(alphas)) for _ in range(heads)]],
            "betas": [[float(rng.uniform(0, beta_max)) for _ in range(heads)]]}
    cfg = moa_b200.moa_config_to_cache_config(plan, N, 0, verbose=False)
    caps, static = cfg["cache_size"][0], cfg["static_size"][0]
    return [s // 64 for s in static], [(c - s) // 64 for c, s in zip(caps, static)]


def prefill_config3_leg(device, dist, world, rank, peaks_tf, which, N=65536, e2e=True, cpu=True):
    """One layer of config 3: B1 H32 N65536 D128 bf16, alpha in {512..4096}, beta in [0, 0.3), 64 sinks.  The 32
    heads are placed on the ranks by their visited-block counts (longest-processing-time packing); every rank
    runs the kernel on its heads (no exchange: heads are independent), then — as the whole-layer variant —
    the outputs are all-gathered into (G, 1, N, H/G, D) with NCCL.  (A smaller N is only for profiler captures.)"""
    import moa_b200

    try:
        Hp = 32
        sink_b, local_b = draw_plan(3000, Hp, [512, 1024, 2048, 4096], 0.3, N)
        costs = [moa_b200.prefill_block_visits(N, [s], [l]) for s, l in zip(sink_b, local_b)]
        sh = moa_b200.HeadSharding(costs, world, rank, group=None)
        mine = sh.local_heads
        Hl = len(mine)
        my_sink, my_local = [sink_b[h] for h in mine], [local_b[h] for h in mine]
        gen = torch.Generator(device=device).manual_seed(3000 + rank)
        q, k, v = (torch.randn(1, Hl, N, D, generator=gen, device=device, dtype=torch.bfloat16) for _ in range(3))
        sb = torch.tensor(my_sink, dtype=torch.int32, device=device)
        lb = torch.tensor(my_local, dtype=torch.int32, device=device)
        out = torch.empty(1, N, Hl, D, dtype=torch.bfloat16, device=device)
        sm = D ** -0.5

        def launch():
            moa_b200.sparse_prefill(q, k, v, sm, sb, lb, out=out)

        for _ in range(3):
            launch()
        moa_b200.check_device_status(device)
        iters = 5 if N <= 65536 else 3
        flush = None
        if 4 * Hl * N * D * 2 <= (1 << 30):     # Q, K, V, O within reach of L2: flush it, and hide the host side
            scratch = torch.empty(256 << 20, dtype=torch.uint8, device=device)
            flush = lambda: scratch.fill_(1)
            iters = 9
        times = time_single_launches(launch, iters, device, dist, behind=flush)
        moa_b200.check_device_status(device)
        ms_best, ms_mean = min(times), sum(times) / len(times)
        flops = moa_b200.prefill_flops(1, N, D, sink_b, local_b)          # the whole layer, all ranks
        my_flops = moa_b200.prefill_flops(1, N, D, my_sink, my_local)
        tf = flops / (ms_best * 1e-3) / 1e12
        loads = [sum(costs[h] for h in s) for s in sh.shards]
        res = {"workload": f"config3 one layer: block-sparse prefill B1 H32 N{N} D128 bf16, heads sharded over "
                           f"{world} GPU(s) by visited blocks, no collective",
               "tflops_band_dense_equiv": tf, "tflops_aggregate": tf, "tflops_per_gpu": tf / world,
               "ms_per_layer": ms_best, "flop_per_layer": flops,
               "timing": f"best of {iters} single launches (as the peak was measured), max over ranks per launch"
                         + (", each enqueued behind a 256 MB fill that flushes L2" if flush is not None else ""),
               "tflops_mean_of_launches": flops / (ms_mean * 1e-3) / 1e12,
               "shard_imbalance": max(loads) / (sum(loads) / len(loads)),
               "roofline": {"bound": "tensor", "achieved": tf / world, "peak": peaks_tf, "unit": "TFLOP/s",
                            "frac": tf / world / peaks_tf, "peak_source": which, "per": "GPU"}}
        if 2 * Hl * N * D * 2 > (384 << 20):       # the kernel form that was captured (one block per unit)
            res["roofline"].update(traffic=PREFILL_DRAM_TRAFFIC_RATIO * 4 * Hl * N * D * 2,
                                   traffic_source="ncu at N = 32768 (same kernel form), scaled by the tensor sizes")
        else:
            res["roofline"].update(traffic=None, traffic_source="no capture of the persistent form at this shape (at 32 "
                                   "heads x 16384 tokens it read 2.5 x the tensors' bytes: chunked unit order)")
        if world > 1:
            # whole-layer variant: gather the ranks' outputs (bandwidth-bound: 512/G MiB per rank)
            full = torch.empty(world, 1, N, Hl, D, dtype=torch.bfloat16, device=device)

            def gather():
                dist.all_gather_into_tensor(full, out)

            for _ in range(2):
                gather()
            gt = time_single_launches(gather, 5, device, dist)
            g_ms = min(gt)
            recv = (world - 1) * out.numel() * 2
            res["allgather"] = {"ms": g_ms, "bytes_received_per_gpu": recv, "gbs_per_gpu_in": recv / (g_ms * 1e-3) / 1e9,
                                "note": "NCCL all_gather_into_tensor of the (1, N, H/G, D) outputs into local HBM, "
                                        "timed alone; 770 GB/s per direction was measured for a peer copy on this pool"}
            res["ms_per_layer_with_allgather"] = ms_best + g_ms
        if rank == 0 and world == 1 and e2e:
            # end to end: q, k, v from pinned host memory, output back to it, one stream
            hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
            ho = torch.empty(out.shape, dtype=out.dtype).pin_memory()

            def e2e_once():
                q.copy_(hq, non_blocking=True)
                k.copy_(hk, non_blocking=True)
                v.copy_(hv, non_blocking=True)
                launch()
                ho.copy_(out, non_blocking=True)

            e2e_once()
            t = min(time_single_launches(e2e_once, 3, device, None))
            res["e2e"] = {"value": flops / (t * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": t,
                          "h2d_bytes_per_step": 3 * q.numel() * 2, "d2h_bytes_per_step": out.numel() * 2,
                          "note": "host q/k/v -> device, kernel, output -> host, serialised on one stream"}
            del hq, hk, hv, ho
        if rank == 0 and world == 1 and cpu:
            # bounded CPU sample: the first two heads over the first 4096 tokens of the same plan
            n_s, heads_s = 4096, [0, 1]
            sb_s, lb_s = [sink_b[mine[h]] for h in heads_s], [local_b[mine[h]] for h in heads_s]
            fl = moa_b200.prefill_flops(1, n_s, D, sb_s, lb_s)
            qs, ks, vs = (t[:, heads_s, :n_s].cpu() for t in (q, k, v))
            tfc, sec, dt_name, cores = cpu_prefill_tflops(qs, ks, vs, sm, sb_s, lb_s, fl)
            res["cpu_baseline"] = {"value": tfc, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                   "sample": f"2 heads x the first {n_s} tokens of the same plan, one SDPA call with "
                                             f"the boolean mask ({dt_name}, {sec:.2f} s), flop counted the same way"}
        return res
    except Exception as exc:  # the decode headline must still be reported
        return {"error": f"{type(exc).__name__}: {exc}"}


def prefill_config0_leg(device, peaks_tf, which, cpu=True):
    """Config 0 (the CPU-runnable one): B1 H32 N2048 D128 fp16, alpha in {128..1024}, beta in [0, 0.5), 64 sinks.
    All of Q, K, V and O (64 MB) fit in L2, so a buffer larger than L2 is written between the timed launches."""
    import moa_b200

    try:
        Hp, N = 32, 2048
        sink_b, local_b = draw_plan(0, Hp, [128, 256, 512, 1024], 0.5, N)
        gen = torch.Generator(device=device).manual_seed(0)
        q, k, v = (torch.randn(1, Hp, N, D, generator=gen, device=device, dtype=torch.float16) for _ in range(3))
        sb = torch.tensor(sink_b, dtype=torch.int32, device=device)
        lb = torch.tensor(local_b, dtype=torch.int32, device=device)
        out = torch.empty(1, N, Hp, D, dtype=torch.float16, device=device)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        sm = D ** -0.5

        def launch():
            moa_b200.sparse_prefill(q, k, v, sm, sb, lb, out=out)

        for _ in range(5):
            launch()
        moa_b200.check_device_status(device)
        cold = time_single_launches(launch, 20, device, None, behind=lambda: flush.fill_(1))
        ms_blocks, _ = time_blocks(lambda i: launch(), 20, device, None, min_blocks=25, min_region_s=0.05)
        warm_ms = statistics.median(ms_blocks) / 20
        moa_b200.check_device_status(device)
        flops = moa_b200.prefill_flops(1, N, D, sink_b, local_b)
        ms = statistics.median(cold)
        tf = flops / (ms * 1e-3) / 1e12
        res = {"workload": "config0: block-sparse prefill B1 H32 N2048 D128 fp16",
               "tflops_band_dense_equiv": tf, "ms": ms, "flop": flops,
               "timing": "median of 20 single launches, each enqueued behind a 256 MB fill that flushes L2",
               "ms_back_to_back_l2_warm": warm_ms, "tflops_back_to_back_l2_warm": flops / (warm_ms * 1e-3) / 1e12,
               "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks_tf, "unit": "TFLOP/s",
                            "frac": tf / peaks_tf, "peak_source": which, "traffic": None,
                            "traffic_source": "not captured at this size (Q, K, V and O, 64 MB, fit in L2)"}}
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        ho = torch.empty(out.shape, dtype=out.dtype).pin_memory()

        def e2e_once():
            q.copy_(hq, non_blocking=True)
            k.copy_(hk, non_blocking=True)
            v.copy_(hv, non_blocking=True)
            launch()
            ho.copy_(out, non_blocking=True)

        e2e_once()
        t = statistics.median(time_single_launches(e2e_once, 10, device, None))
        res["e2e"] = {"value": flops / (t * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": t,
                      "h2d_bytes_per_step": 3 * q.numel() * 2, "d2h_bytes_per_step": out.numel() * 2,
                      "note": "host q/k/v -> device, kernel, output -> host, serialised on one stream"}
        if cpu:
            tfc, sec, dt_name, cores = cpu_prefill_tflops(hq, hk, hv, sm, sink_b, local_b, flops)
            res["cpu_baseline"] = {"value": tfc, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                   "sample": f"the whole of config 0, one SDPA call with the boolean mask "
                                             f"({dt_name}, {sec:.2f} s), flop counted the same way"}
        return res
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"}


def fill_rings_directly(cache, layer, device, head_ids, kv_len, seed_base):
    """Rings of a long context, pre-filled: every slot of head h holds random data drawn from a generator seeded
    by the head's global id (so any rank can regenerate any head), lengths = capacities, write pointers where a
    kv_len-token context leaves them."""
    cache._materialize(layer, device)
    starts = cache.head_index[layer].tolist()
    for i, h in enumerate(head_ids):
        g = torch.Generator(device=device).manual_seed(seed_base + h)
        rows = starts[i + 1] - starts[i]
        for t in (cache.key_cache[layer], cache.value_cache[layer]):
            t[:, starts[i]:starts[i + 1]] = torch.randn(cache.batch_size, rows, cache.head_dim, generator=g,
                                                        device=device, dtype=cache.dtype)
    cache.cache_valid_length[layer].copy_(cache.cache_max_length[layer][None].expand(cache.batch_size, -1))
    cache.mask_cache[layer].fill_(1)
    circ = cache.circular_cache_size[layer]
    upd = cache.circular_cache_head_index[layer] + (kv_len - cache.static_cache_size[layer]) % circ
    cache.cache_update_index[layer].copy_(upd[None].expand(cache.batch_size, -1))
    cache._kv_len[layer] = kv_len


def layer_leg(device, dist, world: int, rank: int, steps: int = 64, warmup: int = 5):
    """The attention part of one decode step of one layer of config 4 of BASELINE.json (Llama-3-70B as MHA: 64
    heads x 128, bf16, batch 64, per-head window drawn from U[1k, 16k] rounded to 64, plus 64 sinks, rings
    full at a 131072-token context).  The 64 heads are placed on the ranks by capacity (longest-processing-time
    packing); every rank runs the fused decode launch on its shard and the outputs are gathered into
    (B, 1, 64, D) on every rank.  Strong scaling: the layer is fixed, the work per GPU shrinks with N."""
    import moa_b200
    from oracle import moa_oracle as orc

    Bl, Hl, Dl = 64, 64, 128
    rng = np.random.RandomState(4000)
    caps = [SINK + int(-(-int(w) // 64) * 64) for w in rng.uniform(1024, 16384, Hl)]
    sh = moa_b200.HeadSharding(caps, world, rank, group=None)
    mine_ids = sh.local_heads
    mine = sh.slice_plan(caps)
    cache = moa_b200.StaticCircularCache([mine], Bl, Dl, [[SINK] * len(mine)], device, torch.bfloat16)
    fill_rings_directly(cache, 0, device, mine_ids, 131072, 4000)

    def head_rows(h, what):      # the step's q / k / v row of head h (global id): same on every rank
        g = torch.Generator(device=device).manual_seed(500000 + 3 * h + what)
        return torch.randn(Bl, 1, Dl, generator=g, device=device, dtype=torch.bfloat16)

    trio = [torch.stack([head_rows(h, w) for h in mine_ids], dim=1) for w in range(3)]      # (B, H/G, 1, D)
    out = torch.empty(Bl, 1, len(mine), Dl, dtype=torch.bfloat16, device=device)
    sm = Dl ** -0.5

    # correctness probe, outside the timed regions: one step from the known state, gathered (with N > 1 once
    # through the NCCL all-gather and once, from the same state, through the fused peer-store gather); rank 0
    # recomputes one head of its own and one of the last rank's with the fp32 oracle on its CPU (2 batch rows)
    cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)
    gathered = sh.all_gather(out).clone()
    pg = None
    fused_equal = None
    peer_error = None
    if world > 1:
        try:        # set-up fails on all ranks alike or on none (PeerGather agrees on the outcome first)
            pg = moa_b200.PeerGather(sh, Bl, Dl, torch.bfloat16, device)
        except Exception as exc:
            peer_error = f"{type(exc).__name__}: {exc}"[:300]
    if pg is not None:
        try:        # a barrier that gave up on any rank sends every rank down the NCCL path together
            fill_rings_directly(cache, 0, device, mine_ids, 131072, 4000)
            fused = pg.decode_and_gather(cache, trio[0], trio[1], trio[2], 0, sm)
            pg.check(collective=True)
            fused_equal = bool(torch.equal(fused, gathered))
        except moa_b200.MoaError as exc:
            peer_error = f"{type(exc).__name__}: {exc}"[:300]
            pg.close()
            pg = None
    probe = None
    if rank == 0:
        worst = 0.0
        for h in (sh.shards[0][0], sh.shards[-1][0]):
            g = torch.Generator(device=device).manual_seed(4000 + h)
            kh = torch.randn(Bl, caps[h], Dl, generator=g, device=device, dtype=torch.bfloat16)[:2].cpu()
            vh = torch.randn(Bl, caps[h], Dl, generator=g, device=device, dtype=torch.bfloat16)[:2].cpu()
            slot = SINK + (131072 - SINK) % (caps[h] - SINK)
            kh[:, slot], vh[:, slot] = head_rows(h, 1)[:2, 0].cpu(), head_rows(h, 2)[:2, 0].cpu()
            ref = orc.decode_attention_fp32(head_rows(h, 0)[:2, None].cpu(), kh, vh, torch.zeros(2, 1, dtype=torch.int64),
                                            torch.full((2, 1), caps[h]), sm)
            got = gathered[:2, :, sh.order.index(h)].float().cpu()
            worst = max(worst, float((got - ref[:, :, 0]).abs().max()))
        probe = worst

    def step_attention(i):
        cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)

    def step(i):
        cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)
        sh.all_gather(out)

    def step_fused(i):
        pg.decode_and_gather(cache, trio[0], trio[1], trio[2], 0, sm)

    variants = [("attention_only", step_attention), ("attention_allgather", step)]
    if pg is not None:
        variants.append(("attention_peer_gather", step_fused))
    res = {}
    for name, fn in variants:
        for i in range(warmup):
            fn(i)
        ms, _ = time_blocks(fn, steps, device, dist, min_blocks=5, min_region_s=0.1)
        res[name + "_us"] = statistics.median(ms) / steps * 1e3
    us_nccl = res["attention_allgather_us"]
    us = res.get("attention_peer_gather_us", us_nccl)

    # The step after attention: o_proj (hidden 8192) in its gathered and its row-parallel form.
    hidden = Hl * Dl
    gen = torch.Generator(device=device).manual_seed(4000)
    w_full = torch.randn(hidden, Hl * Dl, generator=gen, device=device, dtype=torch.bfloat16) * 0.02
    w_loc = sh.local_output_columns(w_full, Dl).contiguous()

    def step_gather(i):
        cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)
        sh.output_projection(out, w_full, mode="gather")

    def step_row(i):
        cache.decode_attention(trio[0], trio[1], trio[2], 0, sm, out=out)
        sh.output_projection(out, w_loc, mode="row_parallel")

    def step_fused_proj(i):
        full = pg.decode_and_gather(cache, trio[0], trio[1], trio[2], 0, sm)
        torch.nn.functional.linear(full.view(Bl, 1, Hl * Dl), w_full)

    proj = {}
    for name, fn in (("gather", step_gather), ("row_parallel", step_row)) + \
            ((("peer_gather", step_fused_proj),) if pg is not None else ()):
        for i in range(warmup):
            fn(i)
        ms, _ = time_blocks(fn, steps, device, dist, min_blocks=5, min_region_s=0.1)
        proj[name + "_us"] = statistics.median(ms) / steps * 1e3
    if pg is not None:
        pg.check(collective=True)
        pg.close()

    kv_bytes_all = moa_b200.decode_bytes(Bl, caps, Dl, 2)
    loads = [sum(caps[h] for h in s) for s in sh.shards]
    return {"workload": "config4 one layer, attention + gather of the head shards: B64 H64 D128 bf16, windows "
                        f"U[1k,16k] + 64 sinks, heads sharded over {world} GPU(s)", "us_per_step": us,
            "tokens_per_s": Bl / (us * 1e-6), "aggregate_hbm_gbs": kv_bytes_all / (us * 1e-6) / 1e9,
            "gather": "one launch: the decode kernel stores its rows into every rank's buffer over NVLink and its last block "
                      "runs the cross-rank barrier" if pg is not None
                      else ("none (one GPU)" if world == 1 else f"NCCL all-gather + copy (peer buffers unavailable: {peer_error})"),
            "extrapolated_80_layers_ms": us * 80 / 1e3,
            "breakdown_us": {"attention_kernel": res["attention_only_us"],
                             "peer_stores_and_barrier_in_the_launch": us - res["attention_only_us"],
                             "nccl_allgather_and_copy": us_nccl - res["attention_only_us"]},
            "us_per_step_nccl_allgather": us_nccl,
            "fused_gather_equals_nccl_gather": fused_equal,
            "allgather_bytes_per_step": Bl * Hl * Dl * 2 if world > 1 else 0,
            "shard_imbalance": max(loads) / (sum(loads) / len(loads)),
            "gather_max_abs": probe,
            "gather_check": "rank 0 recomputed one head of its own and one of the last rank's (2 batch rows) from the "
                            "gathered (B, 1, 64, D) with the fp32 CPU oracle; bf16 outputs",
            "with_o_proj": dict(proj, note="attention + o_proj (8192 x 8192 bf16): NCCL-gathered form, row-parallel form "
                                           "(all-reduce of partial products), peer-store gather form")}


def model_leg(device, dist, world: int, rank: int, steps: int = 8, warmup: int = 3, batch: int = 32,
              context: int = 16384, layers: int = 32):
    """Config 2 of BASELINE.json — Vicuna-7B-16k architecture (32 layers, hidden 4096, 32 heads x 128, FFN 11008,
    RoPE, fp16) with random-init weights, decode with batch 32 at 16k context, heads sharded over the N GPUs
    (per-layer placement by capacity; q/k/v projections and ring caches sharded, the attention outputs
    all-gathered before the replicated o_proj and MLP).  The per-layer plan is drawn as in config 0 with
    N = 16384; the rings are pre-filled directly (a 16k-token model prefill at batch 32 is not part of this leg).
    One step = one new token for every sequence through all layers: per layer one fused-QKV GEMM, one fused
    decode launch, the gather, o_proj and the MLP (GEMMs and norms are library kernels)."""
    import moa_b200

    rng = np.random.RandomState(2000)
    hidden, heads, ffn = 4096, 32, 11008
    plan = {"alphas": [[float(rng.choice([128, 256, 512, 1024])) for _ in range(heads)] for _ in range(layers)],
            "betas": [[float(rng.uniform(0, 0.5)) for _ in range(heads)] for _ in range(layers)]}
    model = moa_b200.MoALlamaForCausalLM(layers, hidden, heads, ffn, vocab_size=32000, rope_theta=10000.0,
                                         dtype=torch.float16, device=device)
    gen = torch.Generator(device=device).manual_seed(2000)       # same weights on every rank
    for prm in model.parameters():
        if prm.dim() > 1:
            prm.data.normal_(0, 0.02, generator=gen)
    model.set_mixture_of_attention(plan, permute_head=True, moa_max_new_token=1024)
    if world > 1:
        model.model.shard_heads(world, rank, seq_len=context)
    cache = model.model.new_cache(batch, context)
    kv_bytes = 0
    for layer in range(layers):
        ids_ = model.model.head_shardings[layer].local_heads if world > 1 else list(range(heads))
        fill_rings_directly(cache, layer, device, ids_, context, 2000 + 1000 * layer)
        kv_bytes += 2 * batch * cache.layer_cache_size[layer] * 128 * 2
    torch.cuda.synchronize(device)
    ids = torch.randint(0, 32000, (batch, 1), device=device, generator=gen)

    def step(i):
        model(ids, past_key_values=cache)

    for i in range(warmup):
        step(i)
    ms, _ = time_blocks(step, steps, device, dist, min_blocks=3, min_region_s=0.2)
    per_step_eager = per_step_nccl = statistics.median(ms) / steps
    pg = None
    if world > 1:        # the same steps with the gather done by the decode kernel (peer stores + barrier kernel)
        try:             # set-up fails on all ranks alike or on none
            pg = model.model.enable_peer_gather(batch)
        except Exception:
            pg = None
    if pg is not None:
        for i in range(warmup):
            step(i)
        ms, _ = time_blocks(step, steps, device, dist, min_blocks=3, min_region_s=0.2)
        per_step_eager = statistics.median(ms) / steps
    # the whole step captured once in a CUDA graph and replayed
    graph = moa_b200.DecodeGraph(model, cache)

    def step_graph(i):
        graph.step(ids)

    for i in range(warmup):
        step_graph(i)
    ms, _ = time_blocks(step_graph, steps, device, dist, min_blocks=3, min_region_s=0.2)
    per_step = statistics.median(ms) / steps
    del graph
    peer_error = None
    if pg is not None:
        try:        # a barrier that gave up on any rank: every rank reports the NCCL figure instead
            pg.check(collective=True)
        except moa_b200.MoaError as exc:
            peer_error = f"{type(exc).__name__}: {exc}"[:300]
            per_step = per_step_eager = per_step_nccl
        pg.close()
        if peer_error is not None:
            pg = None
    weights = sum(prm.numel() for name, prm in model.named_parameters()
                  if prm.dim() > 1 and "embed_tokens" not in name) * 2
    return {"workload": f"config2: Vicuna-7B-16k architecture, random weights, decode B{batch} at {context} context, "
                        f"{layers} layers, heads sharded over {world} GPU(s)",
            "tokens_per_s": batch / (per_step * 1e-3), "ms_per_step": per_step,
            "how": "one CUDA graph per decode step (all layers)" + (", gather and barrier inside the decode launch"
                   if pg is not None else (", NCCL all-gather" if world > 1 else "")) +
                   (f" (eager launches; the peer gather was abandoned: {peer_error})" if peer_error else ""),
            "ms_per_step_eager_launches": per_step_eager,
            "ms_per_step_eager_nccl_allgather": per_step_nccl if world > 1 else None,
            "kv_bytes_per_step_per_gpu": kv_bytes, "weight_bytes_per_step_per_gpu": weights,
            "hbm_gbs_per_gpu": (kv_bytes + weights) / (per_step * 1e-3) / 1e9}


def model_prefill_leg(device, n_tokens: int = 65536, layers: int = 32):
    """Config 3 of BASELINE.json as a whole model: Llama-3-8B architecture converted to MHA (32 layers, 32 heads x
    128, hidden 4096, FFN 14336, rope_theta 5e5, bf16), random-init weights, one 65536-token random-token
    sequence, per-head plan alpha in {512..4096}, beta in [0, 0.3), 64 sinks.  One forward = per layer the fused
    QKV GEMM, the rotary embedding of q and k in place, the ring-cache fill, the block-sparse prefill kernel (all
    reading the GEMM's output through strides), o_proj and the MLP; GEMMs and norms are library kernels."""
    import moa_b200

    hidden, heads, ffn = 4096, 32, 14336
    rng = np.random.RandomState(3000)
    plan = {"alphas": [[float(rng.choice([512, 1024, 2048, 4096])) for _ in range(heads)] for _ in range(layers)],
            "betas": [[float(rng.uniform(0, 0.3)) for _ in range(heads)] for _ in range(layers)]}
    model = moa_b200.MoALlamaForCausalLM(layers, hidden, heads, ffn, vocab_size=32000, rope_theta=500000.0,
                                         dtype=torch.bfloat16, device=device, rms_norm_eps=1e-5)
    gen = torch.Generator(device=device).manual_seed(3000)
    for prm in model.parameters():
        if prm.dim() > 1:
            prm.data.normal_(0, 0.02, generator=gen)
    model.set_mixture_of_attention(plan, permute_head=True, moa_max_new_token=0)
    ids = torch.randint(0, 32000, (1, n_tokens), device=device, generator=gen)
    cfg = moa_b200.moa_config_to_cache_config(model.model.moa_config, n_tokens, 0, verbose=False)
    attn_flops = sum(moa_b200.prefill_flops(1, n_tokens, 128, [s // 64 for s in st], [(c - s) // 64 for c, s in zip(cs, st)])
                     for cs, st in zip(cfg["cache_size"], cfg["static_size"]))
    gemm_flops = layers * 2 * n_tokens * (hidden * 3 * hidden + hidden * hidden + 3 * hidden * ffn)
    times = []
    for i in range(3):
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits, cache = model(ids)
        e1.record()
        torch.cuda.synchronize(device)
        times.append(e0.elapsed_time(e1))
        del cache
    ms = min(times[1:])
    return {"workload": f"config3 whole model: Llama-3-8B-as-MHA architecture, random weights, prefill of {n_tokens} tokens, "
                        f"{layers} layers, bf16, 1 GPU", "ms": ms, "tokens_per_s": n_tokens / (ms * 1e-3),
            "attention_tflop": attn_flops / 1e12, "gemm_tflop": gemm_flops / 1e12,
            "tflops_total": (attn_flops + gemm_flops) / (ms * 1e-3) / 1e12,
            "timing": "best of 2 forwards after one warm-up, CUDA events, ring caches built and filled inside",
            "logits_finite": bool(torch.isfinite(logits.float()).all())}


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
    hbm_peak, tf_peak, which = measured_peaks()

    def finish(obj):
        if rank == 0:
            print(json.dumps(obj), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()

    if args.leg == "prefill":
        res = {"prefill": prefill_config3_leg(device, dist, world, rank, tf_peak, which, args.prefill_n,
                                              e2e=not args.no_e2e, cpu=not args.no_cpu_baseline)}
        if world == 1 and args.prefill_n == 65536:
            res["prefill_config0"] = prefill_config0_leg(device, tf_peak, which, cpu=not args.no_cpu_baseline)
        return finish(res)
    if args.leg == "model":
        return finish({"model": model_leg(device, dist, world, rank, steps=max(1, min(args.steps, 16)),
                                          layers=args.model_layers)})
    if args.leg == "model-prefill":
        return finish({"model_prefill": model_prefill_leg(device, args.prefill_n, args.model_layers)} if rank == 0 else None)
    if args.leg == "layer":
        return finish({"layer_allgather": layer_leg(device, dist, world, rank)})

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

    # End to end: q/k/v of the step come from pinned host memory (packed in one buffer, so a step costs one copy
    # each way), the output goes back to pinned host memory.  Two forms:
    #  - pipelined: the copies run on their own streams, double-buffered, so that the upload of step i+1 and the
    #    download of step i-1 overlap the kernel of step i (a server that batches independent requests);
    #  - serialised: upload, kernel and download of a step follow one another on one stream (autoregressive
    #    decoding of one batch, where the next query depends on this step's output).
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

    def step_e2e_serial(i):
        dev_in[0].copy_(host_in[i % n_pool], non_blocking=True)
        cache.decode_attention(dev_in[0][0], dev_in[0][1], dev_in[0][2], 0, sm, out=dev_out[0])
        host_out[0].copy_(dev_out[0], non_blocking=True)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    warm = max(args.warmup, 3)
    steps = args.steps
    for i in range(warm):
        step_resident(i)
    ms_blocks, win1 = time_blocks(step_resident, steps, device, dist)
    for i in range(warm):
        step_e2e(i)
    e2e_drain()
    ms_e2e_blocks, win2 = time_blocks(step_e2e, steps, device, dist, drain=e2e_drain)
    for i in range(warm):
        step_e2e_serial(i)
    ms_ser_blocks, win3 = time_blocks(step_e2e_serial, steps, device, dist)
    clocks = sampler.stop([win1, win2, win3]) if sampler else None

    # the same K steps captured once in a CUDA graph and replayed (one graph launch per K steps)
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
            for i in range(steps):
                step_resident(i)
        g.replay()
        torch.cuda.synchronize(device)
        ms_graph, _ = time_blocks(lambda i: g.replay() if i % steps == 0 else None, steps, device, dist)
        graph_info = {"us_per_step": statistics.median(ms_graph) / steps * 1e3,
                      "note": f"{steps} decode steps captured in one CUDA graph; median of {len(ms_graph)} replays"}
    except Exception as exc:   # capture is an extra, never a reason to lose the bench line
        graph_info = {"unavailable": repr(exc)[:200]}

    prefill = prefill0 = None
    if not args.no_prefill:
        prefill = prefill_config3_leg(device, dist, world, rank, tf_peak, which, args.prefill_n,
                                      e2e=not args.no_e2e, cpu=not args.no_cpu_baseline)
        if world == 1:
            prefill0 = prefill_config0_leg(device, tf_peak, which, cpu=not args.no_cpu_baseline)
    del cache, pool
    torch.cuda.empty_cache()
    layer = None
    if not args.no_layer:
        try:
            layer = layer_leg(device, dist, world, rank)
        except Exception as exc:      # the decode headline must still be reported
            layer = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    model = None
    if not args.no_model:
        torch.cuda.empty_cache()
        try:
            model = model_leg(device, dist, world, rank, steps=8, layers=args.model_layers)
        except Exception as exc:      # the decode headline must still be reported
            model = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    line = None
    if rank == 0:
        st = block_stats(ms_blocks, steps)
        per_step_ms = st["ms_per_step_median"]
        value = B * world / (per_step_ms * 1e-3)
        bytes_per_launch = moa_b200.decode_bytes(B, caps, D, 2)
        achieved = bytes_per_launch / (per_step_ms * 1e-3) / 1e9
        e2e_ms = statistics.median(ms_e2e_blocks) / steps
        ser_ms = statistics.median(ms_ser_blocks) / steps
        h2d, d2h = 3 * B * H * D * 2, B * H * D * 2
        line = {
            "metric": "moa_decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": steps, "warmup": args.warmup, "ms_per_step": per_step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config1_dict(caps, args.fill_tokens, world),
            "timing": dict(st, note="the K-step block between two CUDA events, repeated back to back; ms_per_step = "
                                    "median block / K; max over ranks per block"),
            "e2e": {"value": B * world / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "mode": "pipelined",
                    "note": "through StaticCircularCache.decode_attention; q/k/v from pinned host memory and the output "
                            "back to it every step, copies double-buffered on their own streams beside the kernel"},
            "e2e_serialised": {"value": B * world / (ser_ms * 1e-3), "unit": "tok/s", "ms_per_step": ser_ms,
                               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "mode": "serialised",
                               "note": "the same calls with upload, kernel and download of a step one after the other "
                                       "on one stream (the next query depends on this output)"},
            "gpu_launches": steps * len(ms_blocks),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "frac_of_nominal_8tbs": achieved / 8000.0, "peak_source": which,
                         "algorithmic_bytes_per_launch": bytes_per_launch,
                         "traffic": DECODE_DRAM_TRAFFIC_RATIO * bytes_per_launch,
                         "traffic_source": "ncu at batch 4, scaled by the rows streamed"},
            "clocks": clocks,
        }
        if graph_info is not None:
            line["cuda_graph"] = graph_info
        if prefill is not None:
            line["prefill"] = prefill
        if prefill0 is not None:
            line["prefill_config0"] = prefill0
        if layer is not None:
            line["layer_allgather"] = layer
        if model is not None:
            line["model_config2"] = model
        if world == 1 and not args.no_cpu_baseline:
            val, per_step, cores = cpu_decode_tok_per_s(caps, 30, 1000)
            line["cpu_baseline"] = {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": "30 decode steps at full config-1 size on the host cores (ring update + "
                                              "grouped SDPA, the reference's implementation='sdpa' path restated)"}
    finish(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="moa_b200", choices=["moa_b200", "reference"])
    ap.add_argument("--batch", type=int, default=16, help="batch size (16 = config 1; smaller only for profiler captures)")
    ap.add_argument("--fill-tokens", type=int, default=PREFILL_TOKENS, help="tokens the caches are filled from")
    ap.add_argument("--leg", default="all", choices=["all", "prefill", "model", "model-prefill", "layer"],
                    help="'prefill': only the prefill legs; 'model': whole-model decode of config 2 (heads sharded over "
                         "the GPUs); 'model-prefill': whole-model prefill of config 3 (one GPU); 'layer': only the "
                         "config-4 attention layer with its gather")
    ap.add_argument("--prefill-n", type=int, default=65536, help="sequence length of the config-3 prefill leg")
    ap.add_argument("--model-layers", type=int, default=32, help="layers of the config-2 model leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill legs")
    ap.add_argument("--no-layer", action="store_true", help="skip the config-4 layer leg")
    ap.add_argument("--no-model", action="store_true", help="skip the config-2 whole-model decode leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-to-host timing of the prefill leg")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline legs")
    args = ap.parse_args()
    global B
    B = args.batch
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
