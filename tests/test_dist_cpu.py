"""Head sharding + all-gather over two gloo ranks on CPU (no GPU needed).

The attention of each shard is computed by the CPU oracle; what is under test is the host logic of the
multi-GPU path: LPT head placement, shard-order bookkeeping and the gather back to full head order."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moa_b200 import HeadSharding
from oracle import moa_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, caps, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(0)           # same data on every rank
        B, D, H = 2, 64, len(caps)
        S = sum(caps)
        k = torch.randn(B, S, D, generator=gen)
        v = torch.randn(B, S, D, generator=gen)
        q = torch.randn(B, H, 1, D, generator=gen)
        starts = np.concatenate([[0], np.cumsum(caps)[:-1]])
        hs = torch.tensor(np.tile(starts, (B, 1)))
        valid = torch.tensor(np.tile(caps, (B, 1)))
        full = orc.decode_attention_fp32(q, k, v, hs, valid, 0.125)          # (B, 1, H, D)

        sh = HeadSharding(caps, world, rank)
        assert sorted(sh.order) == list(range(H)) and sh.heads_per_rank == H // world
        loads = [sum(caps[h] for h in s) for s in sh.shards]
        assert max(loads) - min(loads) <= max(caps)
        mine = sh.local_heads
        # this rank only holds its heads' caches, concatenated in shard order
        k_loc = torch.cat([k[:, starts[h]:starts[h] + caps[h]] for h in mine], dim=1)
        v_loc = torch.cat([v[:, starts[h]:starts[h] + caps[h]] for h in mine], dim=1)
        caps_loc = sh.slice_plan(caps)
        st_loc = np.concatenate([[0], np.cumsum(caps_loc)[:-1]])
        out_loc = orc.decode_attention_fp32(q[:, mine], k_loc, v_loc, torch.tensor(np.tile(st_loc, (B, 1))),
                                            torch.tensor(np.tile(caps_loc, (B, 1))), 0.125)
        gathered = sh.all_gather(out_loc)
        assert gathered.shape == (B, 1, H, D)
        assert torch.equal(gathered[:, :, rank * len(mine):(rank + 1) * len(mine)], out_loc)
        restored = sh.unpermute(gathered)
        err = float((restored - full).abs().max())
        # o_proj after attention: gathered form and row-parallel form against the unsharded product.
        # The weight's columns follow the head order, so they are permuted into shard order first.
        from moa_b200 import permute_output_projection
        hidden = 48
        lin = torch.nn.Linear(H * D, hidden, bias=False)
        lin.weight.data = torch.randn(hidden, H * D, generator=gen)
        ref = lin(full.reshape(B, 1, H * D)).detach()
        permute_output_projection(lin, torch.tensor(sh.order), H)
        w_perm = lin.weight.data
        y_gather = sh.output_projection(out_loc, w_perm, mode="gather")
        y_row = sh.output_projection(out_loc, sh.local_output_columns(w_perm, D), mode="row_parallel")
        err = max(err, float((y_gather - ref).abs().max() / ref.abs().max()),
                  float((y_row - ref).abs().max() / ref.abs().max()))
        ret[rank] = err
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharding_matches_unsharded():
    caps = [320, 576, 1088, 320, 2112, 576, 128, 4160]
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), caps, ret), nprocs=world, join=True)
        assert len(ret) == world
        assert all(v < 1e-5 for v in ret.values()), dict(ret)


def test_single_rank_sharding_is_identity():
    sh = HeadSharding([3.0, 1.0, 2.0], 1, 0)
    x = torch.arange(2 * 1 * 3 * 4, dtype=torch.float32).view(2, 1, 3, 4)
    assert sh.all_gather(x) is x
    assert sh.order == [1, 2, 0]                       # sorted by cost inside the shard
    assert torch.equal(sh.unpermute(x[:, :, sh.order]), x)


# ---------------------------------------------------------------------------------------------------
# failures, made on the host: ranks that disagree on the shard table; a rank that never joins a gather
# ---------------------------------------------------------------------------------------------------
def _mismatch_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        caps = [320, 576, 1088, 320] if rank == 0 else [1088, 576, 320, 320]     # rank 1 read another plan
        sh = HeadSharding(caps, world, rank)
        try:
            sh.verify_consistent()
            ret[rank] = "no error"
        except RuntimeError as exc:
            ret[rank] = str(exc)
        same = HeadSharding([320, 576, 1088, 320], world, rank)
        same.verify_consistent()                                                 # agreeing ranks pass
    finally:
        dist.destroy_process_group()


def test_ranks_with_different_shard_tables_are_detected():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_mismatch_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert len(ret) == world
        assert all("shard tables differ" in v for v in ret.values()), dict(ret)


def _absent_worker(rank, world, port, ret):
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        sh = HeadSharding([128, 128, 256, 256], world, rank)
        x = torch.zeros(1, 1, sh.heads_per_rank, 8)
        sh.all_gather(x)                               # one gather everybody takes part in
        if rank == 1:
            ret[rank] = "left between steps"           # leaves with nothing of its own in flight
            return
        t0 = time.time()
        try:
            sh.all_gather(x)                           # rank 1 never joins this one
            ret[rank] = "no error"
        except Exception as exc:                       # the process group's timeout ends the collective
            ret[rank] = f"error after {time.time() - t0:.1f}s: {type(exc).__name__}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_never_joins_ends_the_gather_with_an_error():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_absent_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert ret[1] == "left between steps"
        assert ret[0].startswith("error after"), dict(ret)
        assert float(ret[0].split()[2][:-2]) < 30.0, dict(ret)
