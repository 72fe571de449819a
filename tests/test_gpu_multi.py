"""Head-sharded decode over NCCL on two GPUs (skipped on a single-GPU machine)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import moa_b200
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        gen = torch.Generator().manual_seed(3)               # same data on every rank
        B, D = 2, 128
        caps = [320, 576, 128, 1088, 320, 2112, 576, 128]
        H = len(caps)
        k = torch.randn(B, H, 700, D, generator=gen).half().to(dev)
        v = torch.randn(B, H, 700, D, generator=gen).half().to(dev)
        full = moa_b200.StaticCircularCache([caps], B, D, [[64] * H], dev, torch.float16)
        full.update(k, v, 0)
        sh = moa_b200.HeadSharding(caps, world, rank)
        sh.verify_consistent()                                # every rank built the same shard table
        mine = sh.local_heads
        local = moa_b200.StaticCircularCache([sh.slice_plan(caps)], B, D, [[64] * len(mine)], dev, torch.float16)
        local.update(k[:, mine], v[:, mine], 0)
        worst = 0.0
        for _ in range(4):
            q, k1, v1 = (torch.randn(B, H, 1, D, generator=gen).half().to(dev) for _ in range(3))
            ref = full.decode_attention(q, k1, v1, 0, D ** -0.5)
            out = local.decode_attention(q[:, mine].contiguous(), k1[:, mine].contiguous(), v1[:, mine].contiguous(),
                                         0, D ** -0.5)
            gathered = sh.all_gather(out)
            got = sh.unpermute(gathered)
            worst = max(worst, float((got.float() - ref.float()).abs().max()))
            # o_proj: gathered and row-parallel forms against the projection of the single-GPU output
            w = (torch.randn(256, H * D, generator=gen) * 0.05).half().to(dev)       # columns in head order
            w_perm = w.view(256, H, D)[:, sh.order].reshape(256, H * D).contiguous()
            y_ref = torch.nn.functional.linear(ref.reshape(B, 1, H * D).float(), w.float())
            y_g = sh.output_projection(out, w_perm, mode="gather")
            y_r = sh.output_projection(out, sh.local_output_columns(w_perm, D).contiguous(), mode="row_parallel")
            scale = float(y_ref.abs().max())
            worst = max(worst, float((y_g.float() - y_ref).abs().max()) / scale * 0.25,
                        float((y_r.float() - y_ref).abs().max()) / scale * 0.25)   # fp16 GEMM: 4e-3 relative
        # the fused form: the decode kernel stores its rows into every rank's gather buffer, a barrier kernel
        # orders them; same result as the collective, bit for bit, call after call (two buffers alternate)
        local2 = moa_b200.StaticCircularCache([sh.slice_plan(caps)], B, D, [[64] * len(mine)], dev, torch.float16)
        local2.update(k[:, mine], v[:, mine], 0)
        local3 = moa_b200.StaticCircularCache([sh.slice_plan(caps)], B, D, [[64] * len(mine)], dev, torch.float16)
        local3.update(k[:, mine], v[:, mine], 0)
        pg = moa_b200.PeerGather(sh, B, D, torch.float16, dev)
        for _ in range(5):
            q, k1, v1 = (torch.randn(B, H, 1, D, generator=gen).half().to(dev) for _ in range(3))
            args = (q[:, mine].contiguous(), k1[:, mine].contiguous(), v1[:, mine].contiguous(), 0, D ** -0.5)
            want = sh.all_gather(local2.decode_attention(*args)).clone()
            got = pg.decode_and_gather(local3, *args)
            assert torch.equal(got, want)
        pg.check()
        pg.check(collective=True)
        # A failure reported on one rank only (set by the host here, no kernel involved): the collective form of
        # the check raises on every rank, so that the ranks of a job abandon the fused gather together.
        if rank == 0:
            pg.status[0] = 21
        try:
            pg.check(collective=True)
            raised = False
        except moa_b200.MoaError as exc:
            raised = True
            assert ("gave up waiting" in str(exc)) == (rank == 0)
        assert raised
        pg.check(collective=True)         # the words were cleared: the next check passes on every rank
        pg.close()

        # model level: head-sharded model (collective gather, then the fused gather) against the unsharded model
        plan = {"alphas": [[1024.0, 128.0, 512.0, 128.0], [256.0, 256.0, 64.0, 2048.0]],
                "betas": [[0.0, 0.25, 0.0, 0.5], [0.125, 0.0, 0.5, 0.0]]}

        def tiny():
            torch.manual_seed(5)
            m = moa_b200.MoALlamaForCausalLM(2, 512, 4, 1024, vocab_size=100, dtype=torch.float16, device=dev)
            for p in m.parameters():
                if p.dim() > 1:
                    p.data.normal_(0, 0.03)
            m.set_mixture_of_attention(plan, moa_max_new_token=64)
            return m

        gen2 = torch.Generator().manual_seed(9)
        ids = torch.randint(0, 100, (2, 300), generator=gen2).to(dev)
        nxt = [torch.randint(0, 100, (2, 1), generator=gen2).to(dev) for _ in range(4)]
        ref_m, sh_m = tiny(), tiny()
        sh_m.model.shard_heads(world, rank, seq_len=300)
        for h in sh_m.model.head_shardings:
            h.verify_consistent()
        a, ca = ref_m(ids)
        b, cb = sh_m(ids)
        rel = lambda x, y: float((x.float() - y.float()).abs().mean() / y.float().abs().mean())
        worst_model = rel(b, a)
        pg = None
        for i, t in enumerate(nxt):
            if i == 2:                      # from here on the decode kernel does the gather itself
                pg = sh_m.model.enable_peer_gather(2)
            a, ca = ref_m(t, past_key_values=ca)
            b, cb = sh_m(t, past_key_values=cb)
            worst_model = max(worst_model, rel(b, a))
        # the same steps from a CUDA graph (fused gather inside; the barrier kernel counts its calls on the device)
        graph = moa_b200.DecodeGraph(sh_m, cb)
        for t in [torch.randint(0, 100, (2, 1), generator=gen2).to(dev) for _ in range(6)]:
            a, ca = ref_m(t, past_key_values=ca)
            b = graph.step(t)
            worst_model = max(worst_model, rel(b, a))
        pg.check()
        del graph
        pg.close()
        assert worst_model < 1e-2, worst_model
        ret[rank] = worst
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_head_sharded_decode_equals_single_gpu():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        # shards chunk the flattened cache differently: equal up to the rounding of the fp16 store
        assert len(ret) == world and all(v <= 1e-3 for v in ret.values()), dict(ret)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_driving_two_gpus():
    """The reference's own multi-GPU mode is one process with layers on several devices (device_map="auto";
    its cache materialises each layer on that layer's device).  Per-device launch state (the prefill kernel's
    shared-memory opt-in, the decode kernel's grid sizing) must therefore be kept per device."""
    import moa_b200
    from oracle import moa_oracle as orc
    gen = torch.Generator().manual_seed(31)
    q, k, v = (torch.randn(1, 2, 300, 128, generator=gen).half() for _ in range(3))
    ref = orc.prefill_attention_fp32(q, k, v, 0.1, [1, 1], [1, 3])
    caps = [128, 320]
    S = sum(caps)
    kc, vc = (torch.randn(2, S, 128, generator=gen).half() for _ in range(2))
    qd = torch.randn(2, 2, 1, 128, generator=gen).half()
    starts = torch.tensor([[0, 128]] * 2)
    valid = torch.tensor([[128, 320], [100, 7]])
    dref = orc.decode_attention_fp32(qd, kc, vc, starts, valid, 0.1)
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        sb = torch.tensor([1, 1], dtype=torch.int32, device=dev)
        lb = torch.tensor([1, 3], dtype=torch.int32, device=dev)
        out = moa_b200.sparse_prefill(q.to(dev), k.to(dev), v.to(dev), 0.1, sb, lb)
        moa_b200.check_device_status(dev)
        assert out.device == torch.device(dev)
        assert (out.float().cpu() - ref).abs().max() <= 2e-3, dev
        got = moa_b200.sparse_decode(qd.to(dev), kc.to(dev), vc.to(dev), starts.to(dev), valid.to(dev), 0.1)
        assert (got.float().cpu() - dref).abs().max() <= 2e-3, dev


def test_peer_barrier_gives_up_when_a_rank_never_arrives():
    """Failure detection without a fault: rank 0 of a pretended two-rank group runs the barrier, the flag word
    the absent rank would set stays zero, the bounded wait runs out, the status words say who was missing, and
    the context stays usable (one GPU, no peer)."""
    import ctypes
    from moa_b200 import _lib
    lib = _lib.lib
    flags0 = torch.zeros(8, dtype=torch.int32, device="cuda")      # rank 0's flag words
    flags1 = torch.zeros(8, dtype=torch.int32, device="cuda")      # stands for the absent rank's (nobody reads them)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(flags0.data_ptr(), flags1.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.moa_peer_barrier(ptrs, 0, 2, 1, 0, 20_000_000, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert status.tolist() == [21, 1, 1, 0]
    assert flags0.tolist()[:2] == [1, 0] and flags1.tolist()[0] == 1      # rank 0 published its arrival to both
    # a barrier whose partner has arrived (the word is already there) passes and leaves the status alone
    status.zero_()
    flags0[1] = 2
    assert lib.moa_peer_barrier(ptrs, 0, 2, 2, 0, 20_000_000, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    # the call number counted on the device: the third call waits for 3, which the partner has not published
    calls = torch.full((1,), 2, dtype=torch.int32, device="cuda")
    assert lib.moa_peer_barrier(ptrs, 0, 2, 0, calls.data_ptr(), 20_000_000, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert calls.item() == 3 and status.tolist() == [21, 1, 3, 0] and flags1.tolist()[0] == 3
    assert lib.moa_peer_barrier(ptrs, 0, 9, 3, 0, 1000, status.data_ptr(), stream) == 1    # more than 8 ranks: refused
