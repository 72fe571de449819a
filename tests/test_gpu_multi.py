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
            # the asynchronous gather returns the same tensor
            assert torch.equal(sh.all_gather_finish(sh.all_gather_start(out)), gathered)
            # o_proj: gathered and row-parallel forms against the projection of the single-GPU output
            w = (torch.randn(256, H * D, generator=gen) * 0.05).half().to(dev)       # columns in head order
            w_perm = w.view(256, H, D)[:, sh.order].reshape(256, H * D).contiguous()
            y_ref = torch.nn.functional.linear(ref.reshape(B, 1, H * D).float(), w.float())
            y_g = sh.output_projection(out, w_perm, mode="gather")
            y_r = sh.output_projection(out, sh.local_output_columns(w_perm, D).contiguous(), mode="row_parallel")
            scale = float(y_ref.abs().max())
            worst = max(worst, float((y_g.float() - y_ref).abs().max()) / scale * 0.25,
                        float((y_r.float() - y_ref).abs().max()) / scale * 0.25)   # fp16 GEMM: 4e-3 relative
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
