"""Head sharding across the GPUs of one node.

Heads are independent in attention and each owns its ring cache, so the path shards by heads with no
exchange inside attention.  Where a whole layer runs, the per-rank outputs ``(B, q, H/G, D)`` are
all-gathered into ``(B, q, H, D)`` before ``o_proj`` (NCCL over NVLink; ``gloo`` on CPU in the tests).
One process per GPU (``torchrun``).  ``HeadSharding.all_gather`` is the plain collective; ``PeerGather`` is
the decode path's fused form: the decode kernel stores its output rows straight into every rank's
``(B, 1, H, D)`` buffer over NVLink and ends with a cross-rank barrier that orders the stores before the reads,
so the step has no collective launch and no copy after it.

The step after attention, ``o_proj`` (``MoA/models/llama/modeling_llama.py:329-330`` in the reference),
comes in two forms here: the gathered one (all-gather the head shards, then the full projection on every
rank, as the reference's single-GPU code computes it) and a row-parallel one (every rank multiplies its
heads by its column block of the weight and the partial results are summed with an all-reduce), which
moves ``1/G`` of the weight per rank instead of all of it.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from . import _lib
from .plan import shard_heads


def init_process_group(backend: Optional[str] = None) -> None:
    """``torchrun``-style initialisation (RANK / WORLD_SIZE / MASTER_* from the environment)."""
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group(backend)


class HeadSharding:
    """Which heads of one layer live on which rank, balanced by per-head cost (cache capacity for
    decode bytes, visited blocks for prefill flops) with longest-processing-time packing.

    ``order`` is the head order after sharding (rank 0's heads, then rank 1's, ...): permuting the
    q/k/v row blocks and o_proj column blocks by it (``permute_attention_projection`` /
    ``permute_output_projection``) makes every rank's shard a contiguous slice, the same mechanism the
    reference uses for ``permute_head``."""

    def __init__(self, costs: Sequence[float], world_size: int, rank: int, group=None):
        self.world_size, self.rank, self.group = world_size, rank, group
        self.shards: List[List[int]] = shard_heads(costs, world_size)
        self.order: List[int] = [h for s in self.shards for h in s]
        self.local_heads: List[int] = self.shards[rank]
        self.heads_per_rank = len(self.local_heads)
        self._gather_buffers: Dict = {}

    def verify_consistent(self) -> None:
        """Raises on every rank unless all ranks hold the same shard table (built from the same per-head
        costs): ranks that disagree would gather heads into the wrong places without any other symptom.
        One small all-gather of the table itself; call it once after construction."""
        if self.world_size == 1:
            return
        mine = torch.tensor(self.order, dtype=torch.int64)
        if dist.get_backend(self.group) == "nccl":
            mine = mine.cuda()
        everyone = [torch.empty_like(mine) for _ in range(self.world_size)]
        dist.all_gather(everyone, mine, group=self.group)
        bad = [r for r, t in enumerate(everyone) if not torch.equal(t, everyone[0])]
        if bad:
            raise RuntimeError(f"head shard tables differ between ranks (ranks {bad} disagree with rank 0): "
                               "every rank must build HeadSharding from the same per-head costs")

    def slice_plan(self, values: Sequence) -> List:
        """Per-head values (capacities, alphas, ...) of this rank's heads, in shard order."""
        return [values[h] for h in self.local_heads]

    def all_gather(self, local: Tensor) -> Tensor:
        """``(B, q, H/G, D)`` of every rank -> ``(B, q, H, D)`` in ``order``.  The collective writes
        into a cached ``(G*B, q, H/G, D)`` buffer; one small permuting copy puts the ranks' heads
        next to each other."""
        if self.world_size == 1:
            return local
        B, q, Hl, D = local.shape
        key = (local.device, local.dtype, B, q, Hl, D)
        buf = self._gather_buffers.get(key)
        if buf is None:
            buf = torch.empty(self.world_size * B, q, Hl, D, dtype=local.dtype, device=local.device)
            self._gather_buffers[key] = buf
        with _lib.nvtx_range("moa_b200.all_gather"):
            dist.all_gather_into_tensor(buf, local.contiguous(), group=self.group)   # rank r fills rows [r*B, (r+1)*B)
        return buf.view(self.world_size, B, q, Hl, D).permute(1, 2, 0, 3, 4).reshape(B, q, self.world_size * Hl, D)

    def local_output_columns(self, w_o: Tensor, head_dim: int) -> Tensor:
        """The column block of an ``o_proj`` weight ``(hidden, H*D)`` (columns already in ``order``, see
        ``permute_output_projection``) that multiplies this rank's heads."""
        n = self.heads_per_rank * head_dim
        return w_o[:, self.rank * n:(self.rank + 1) * n]

    def output_projection(self, local: Tensor, w_o: Tensor, mode: str = "gather") -> Tensor:
        """``o_proj`` of the sharded attention output ``(B, q, H/G, D)`` -> ``(B, q, hidden)`` on every rank.

        ``mode="gather"``: all-gather the shards and apply the full weight ``w_o (hidden, H*D)`` (columns in
        ``order``) on every rank.  ``mode="row_parallel"``: ``w_o`` is this rank's column block
        ``(hidden, H/G*D)`` (``local_output_columns``); partial products are summed over the ranks with an
        all-reduce, in the tensor's dtype, so the result differs from the gathered form by the rounding of
        ``G`` partial sums."""
        B, q, Hl, D = local.shape
        if mode == "gather":
            full = self.all_gather(local).reshape(B, q, self.world_size * Hl * D)
            return torch.nn.functional.linear(full, w_o)
        if mode != "row_parallel":
            raise ValueError(f"unknown output projection mode {mode!r}")
        if w_o.shape[1] != Hl * D:
            raise ValueError(f"row_parallel expects this rank's column block (hidden, {Hl * D}), got {tuple(w_o.shape)}")
        part = torch.nn.functional.linear(local.reshape(B, q, Hl * D), w_o)
        if self.world_size > 1:
            dist.all_reduce(part, group=self.group)
        return part

    def unpermute(self, gathered: Tensor) -> Tensor:
        """``(B, q, H, D)`` in shard order -> original head order (for checks against an unsharded run)."""
        inv = torch.empty(len(self.order), dtype=torch.long, device=gathered.device)
        inv[torch.tensor(self.order, device=gathered.device)] = torch.arange(len(self.order), device=gathered.device)
        return gathered[:, :, inv]


class _RawDeviceMemory:
    """A device pointer presented through ``__cuda_array_interface__`` so that torch can view it (no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerGather:
    """The gather of the head shards' decode outputs done by the decode kernel itself.

    Every rank owns two ``(B, 1, H, D)`` buffers (used alternately) and a row of flag words in one piece of
    device memory that the other ranks of the node map into their address space (CUDA IPC).
    ``decode_and_gather`` runs the fused decode step with ``out`` = this rank's head slice of its own buffer
    and ``out_peers`` = the same slice of every other rank's buffer (``moa_decode_gather_fwd``: plain stores over
    NVLink, nothing is loaded from a peer); the block that writes the launch's last row then publishes the call
    number to every rank and waits for theirs, so that when the kernel has finished the buffer holds all heads in
    shard order on every rank.  (``targets()`` + ``barrier()`` are the same thing as two launches, for callers
    that bring their own kernel.)  Two buffers are enough: a rank that is writing buffer
    ``k`` of call ``c + 2`` has passed the barrier of call ``c + 1``, which every other rank enters only after
    its ``o_proj`` of call ``c`` has read buffer ``k``.  Calls must be made by all ranks in the same order.

    The barrier kernel numbers the calls itself (a counter in device memory), so a CUDA graph that contains an
    even number of ``decode_and_gather`` calls (the buffer in turn is chosen on the host when the call is
    captured) can be replayed, by every rank alike.

    The barrier's wait is bounded (``wait_seconds``); if a rank never arrives the others carry on with an
    incomplete buffer and ``check()`` raises.  ``close()`` unmaps and frees; call it on every rank before the
    process group is destroyed."""

    def __init__(self, sharding: HeadSharding, batch_size: int, head_dim: int, dtype: torch.dtype, device,
                 wait_seconds: float = 2.0):
        self.sh = sharding
        self.B, self.D, self.dtype = batch_size, head_dim, dtype
        self.device = torch.device(device)
        G, Hl = sharding.world_size, sharding.heads_per_rank
        assert 1 <= G <= 8, "PeerGather serves the GPUs of one node (at most 8 ranks)"
        self.H = G * Hl
        item = torch.empty((), dtype=dtype).element_size()
        self.row_bytes = Hl * head_dim * item
        payload = batch_size * self.H * head_dim * item
        self.slot_bytes = (payload + 255) // 256 * 256
        total = 2 * self.slot_bytes + 256
        lib = _lib.lib
        self._own = None
        self.bases: List[int] = []
        failure: Optional[Exception] = None
        with torch.cuda.device(self.device):
            # Set-up is collective: every step is attempted on every rank and the outcome is agreed on before
            # anybody raises, so that a rank whose mapping failed cannot leave the others waiting in a collective.
            base = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            try:
                _lib.check("moa_peer_alloc", lib.moa_peer_alloc(ctypes.byref(base), total))
                self._own = base.value
                _lib.check("moa_peer_export", lib.moa_peer_export(base, handle))
            except Exception as exc:
                failure = exc
            handles: List[Optional[bytes]] = [None] * G
            if G > 1:
                dist.all_gather_object(handles, handle.raw if failure is None else None, group=sharding.group)
            if failure is None and any(h is None for g, h in enumerate(handles) if g != sharding.rank):
                failure = RuntimeError("PeerGather: another rank could not allocate or export its buffer")
            if failure is None:
                try:
                    for g in range(G):
                        if g == sharding.rank:
                            self.bases.append(base.value)
                        else:
                            p = ctypes.c_void_p()
                            _lib.check("moa_peer_open", lib.moa_peer_open(handles[g], ctypes.byref(p)))
                            self.bases.append(p.value)
                except Exception as exc:
                    failure = exc
            if G > 1:
                outcomes: List[Optional[bool]] = [None] * G
                dist.all_gather_object(outcomes, failure is None, group=sharding.group)
                if failure is None and not all(outcomes):
                    failure = RuntimeError("PeerGather: another rank could not map the buffers (CUDA IPC between "
                                           f"the ranks' GPUs is needed); ranks that failed: "
                                           f"{[g for g, ok in enumerate(outcomes) if not ok]}")
            if failure is not None:
                for g, b in enumerate(self.bases):
                    if g != sharding.rank:
                        lib.moa_peer_close(b)
                if self._own is not None:
                    lib.moa_peer_free(self._own)
                    self._own = None
                raise failure
        raw = torch.as_tensor(_RawDeviceMemory(base.value, total), device=self.device)
        self.buffers = [raw[k * self.slot_bytes:k * self.slot_bytes + payload].view(dtype).view(batch_size, 1, self.H, head_dim)
                        for k in range(2)]
        self._flag_ptrs = (ctypes.c_void_p * G)(*[b + 2 * self.slot_bytes for b in self.bases])
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._calls = torch.zeros(1, dtype=torch.int32, device=self.device)    # the barrier kernel counts its calls here
        self.epoch = 0
        self.limit_cycles = int(min(2e10, max(1.0, wait_seconds) * 2.0e9))
        if G > 1:
            dist.barrier(group=sharding.group)       # every rank has mapped every buffer before the first store

    def targets(self) -> Tuple[Tensor, List[int]]:
        """This call's destination: the local head slice ``(B, 1, H/G, D)`` of the buffer in turn, and the
        addresses of the same slice in the other ranks' buffers."""
        k = self.epoch & 1
        r, Hl = self.sh.rank, self.sh.heads_per_rank
        off = k * self.slot_bytes + r * self.row_bytes
        peers = [b + off for g, b in enumerate(self.bases) if g != r]
        return self.buffers[k][:, :, r * Hl:(r + 1) * Hl], peers

    def barrier(self) -> Tensor:
        """Orders every rank's stores of this call before the reads that follow on this stream; returns the
        full ``(B, 1, H, D)`` buffer of the call and moves on to the other buffer."""
        full = self.buffers[self.epoch & 1]
        self.epoch += 1
        with torch.cuda.device(self.device):
            _lib.check("moa_peer_barrier", _lib.lib.moa_peer_barrier(
                self._flag_ptrs, self.sh.rank, self.sh.world_size, 0, self._calls.data_ptr(), self.limit_cycles,
                self.status.data_ptr(), _lib.current_stream(self.device)))
        return full

    def decode_and_gather(self, cache, query_states: Tensor, key_states: Tensor, value_states: Tensor,
                          layer_idx: int, sm_scale: float, rope=None) -> Tensor:
        """``StaticCircularCache.decode_attention`` on this rank's heads with the gather folded in — one launch:
        the kernel stores its rows into every rank's buffer and its last block runs the cross-rank barrier.
        Returns ``(B, 1, H, D)`` with all ranks' heads in shard order."""
        out, peers = self.targets()
        full = self.buffers[self.epoch & 1]
        self.epoch += 1
        cache.decode_attention(query_states, key_states, value_states, layer_idx, sm_scale, out=out, rope=rope,
                               out_peers=peers,
                               barrier=(self._flag_ptrs, self.sh.rank, self.sh.world_size, self._calls.data_ptr(),
                                        self.limit_cycles, self.status.data_ptr()))
        return full

    def check(self, collective: bool = False) -> None:
        """Synchronises and raises if a barrier gave up waiting for a rank.  ``collective=True`` (every rank of the
        group calls it): all ranks raise when any rank's barrier gave up, so that the ranks of a job take the same
        path afterwards."""
        torch.cuda.synchronize(self.device)
        words = self.status.tolist()
        failed = words[0] != 0
        elsewhere = False
        if collective and self.sh.world_size > 1:
            flag = torch.tensor([int(failed)], dtype=torch.int32, device=self.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.sh.group)
            elsewhere = bool(flag.item()) and not failed
        if failed:
            self.status.zero_()
            raise _lib.MoaError("moa_peer_barrier", 5, _lib.lib.moa_strerror(5).decode(),
                                f"rank {words[3]} gave up waiting for rank {words[1]} at call {words[2]}")
        if elsewhere:
            raise _lib.MoaError("moa_peer_barrier", 5, _lib.lib.moa_strerror(5).decode(),
                                "the barrier gave up on another rank of the group")

    def close(self) -> None:
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        if self.sh.world_size > 1:
            dist.barrier(group=self.sh.group)        # nobody is still storing into a buffer that goes away
        with torch.cuda.device(self.device):
            for g, b in enumerate(self.bases):
                if g != self.sh.rank:
                    _lib.lib.moa_peer_close(b)
            self.buffers = []
            _lib.lib.moa_peer_free(self._own)
        self._own = None
