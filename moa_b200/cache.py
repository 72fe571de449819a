"""Per-head static + circular KV cache, bookkeeping done by CUDA kernels.

``StaticCircularCache`` keeps the constructor, attribute names, tensor shapes/dtypes and
``update`` semantics of MoA/attention/cache_utils.py:644-1180 so that code written against the
reference (``LlamaMixtureAttention.forward``, MoA/models/llama/modeling_llama.py:262, 302-306)
runs unchanged.  What differs is where the work happens: ``update`` launches one kernel for a
decode step and two or three for a prefill instead of ~15 eager index operations and 100 MB-class
int64 temporaries, and ``decode_attention`` fuses the append with flash-decoding in one launch.
"""
from __future__ import annotations

import ctypes
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from . import _lib
from ._lib import lib


class StaticCircularCache:
    """A cache that does not grow: head ``h`` of layer ``l`` owns ``cache_size[l][h]`` rows of a
    flattened ``(batch, sum_h cache_size, head_dim)`` tensor; the first ``static_size[l][h]`` rows
    keep the first tokens (attention sink), the rest is a ring over the most recent tokens.

    Constructor arguments as in cache_utils.py:653-662.  ``update_cache_content=False`` keeps the
    reference's meaning: ``update`` advances indices, lengths and mask but leaves the payload
    to the attention kernel.
    """

    def __init__(
        self,
        cache_size: List[List[int]],
        batch_size: int = 1,
        head_dim: int = 128,
        static_size: Optional[List[List[int]]] = None,
        device: torch.device = "cpu",
        dtype: torch.dtype = None,
        update_cache_content: bool = True,
    ) -> None:
        self.dtype = dtype if dtype is not None else torch.float16
        self.device = device
        self.update_cache_content = update_cache_content
        self.batch_size = batch_size
        self.head_dim = head_dim
        self.num_layers = len(cache_size)
        self.num_head_for_each_layer = [len(c) for c in cache_size]
        if static_size is None:
            static_size = [[0] * len(c) for c in cache_size]
        assert len(static_size) == self.num_layers
        for c, s in zip(cache_size, static_size):
            assert len(c) == len(s)

        i64 = dict(device=device, dtype=torch.int64)
        self.cache_max_length = [torch.tensor(c, **i64) for c in cache_size]
        self.static_cache_size = [torch.tensor(s, **i64) for s in static_size]
        self.circular_cache_size = [c - s for c, s in zip(self.cache_max_length, self.static_cache_size)]
        self.layer_cache_size = [sum(c) for c in cache_size]
        starts = []
        for c in cache_size:
            acc, row = 0, []
            for x in c:
                row.append(acc)
                acc += x
            row.append(acc)
            starts.append(row)
        self.cache_head_start_index = [torch.tensor(r[:-1], **i64)[None, :].expand(batch_size, -1).contiguous()
                                       for r in starts]
        self.head_index = [torch.tensor(r, **i64) for r in starts]
        self.circular_cache_head_index = [torch.tensor([r[h] + s[h] for h in range(len(s))], **i64)
                                          for r, s in zip(starts, static_size)]
        self.cache_update_index = [torch.tensor(r[:-1], **i64)[None, :].expand(batch_size, -1).contiguous()
                                   for r in starts]
        self.cache_position = 0
        self._kv_len = [0] * self.num_layers
        # payload is created on first use, on the device of the incoming states (cache_utils.py:784-804, 989-993)
        self.key_cache: List[Tensor] = [torch.zeros(batch_size, n, head_dim, dtype=self.dtype, device="meta")
                                        for n in self.layer_cache_size]
        self.value_cache: List[Tensor] = [torch.zeros(batch_size, n, head_dim, dtype=self.dtype, device="meta")
                                          for n in self.layer_cache_size]
        self.mask_cache = [torch.zeros(batch_size, n, **i64) for n in self.layer_cache_size]
        self.cache_valid_length = [torch.zeros(batch_size, h, **i64) for h in self.num_head_for_each_layer]

        # host-side copies used to size grids and to reject layouts the reference cannot run either
        self._max_cap = [max(c) for c in cache_size]
        self._static_host = [list(s) for s in static_size]
        self._cap_host = [list(c) for c in cache_size]
        #: rows of the flattened cache per thread block of the decode kernel (0 = library default)
        self.decode_chunk = int(os.environ.get("MOA_B200_DECODE_CHUNK", "0"))
        self._workspace: Dict[Any, Tensor] = {}
        self._scan_buffers: Dict[Any, Tuple[Tensor, Tensor]] = {}

    # ------------------------------------------------------------------ helpers of the reference
    @staticmethod
    def head_start_index_valid_length_to_head_index(head_start_index: Tensor, head_valid_length: Tensor) -> Tensor:
        """cache_utils.py:820-840 (asserts identical batch rows; last head's length closes the index)."""
        assert (head_start_index == head_start_index[0]).all().item()
        assert (head_valid_length == head_valid_length[0]).all().item()
        return torch.cat((head_start_index[0],
                          (head_start_index[0][-1] + head_valid_length[0][-1]).reshape(-1))).contiguous()

    @staticmethod
    def to_uncontigious(tensor: Tensor, head_index: Tensor) -> List[Tensor]:
        """cache_utils.py:867-887: one view per head."""
        return [tensor[:, head_index[h]:head_index[h + 1]] for h in range(len(head_index) - 1)]

    @staticmethod
    def to_group_contigious(tensor: Tensor, head_index: Tensor) -> List[Tensor]:
        """cache_utils.py:889-951: one ``(B, heads_in_group, cap[, D])`` tensor per run of equal capacities."""
        sizes = (head_index[1:] - head_index[:-1]).tolist()
        starts = head_index.tolist()
        groups, h = [], 0
        while h < len(sizes):
            g = h
            while g < len(sizes) and sizes[g] == sizes[h]:
                g += 1
            part = tensor[:, starts[h]:starts[g]]
            shape = (tensor.shape[0], g - h, sizes[h]) + tuple(tensor.shape[2:])
            groups.append(part.reshape(shape).contiguous())
            h = g
        return groups

    # ------------------------------------------------------------------ internals
    def _materialize(self, layer_idx: int, device) -> None:
        if self.key_cache[layer_idx].device == torch.device("meta"):
            self.key_cache[layer_idx] = torch.zeros_like(self.key_cache[layer_idx], device=device)
        if self.value_cache[layer_idx].device == torch.device("meta"):
            self.value_cache[layer_idx] = torch.zeros_like(self.value_cache[layer_idx], device=device)
        for name in ("mask_cache", "cache_update_index", "cache_head_start_index", "circular_cache_head_index",
                     "cache_valid_length", "cache_max_length", "circular_cache_size", "static_cache_size"):
            lst = getattr(self, name)
            if lst[layer_idx].device != device:
                lst[layer_idx] = lst[layer_idx].to(device=device)

    def _check_layout(self, layer_idx: int) -> None:
        for cap, st in zip(self._cap_host[layer_idx], self._static_host[layer_idx]):
            if cap - st <= 0:
                raise ValueError("every head needs a circular part: cache_size must exceed static_size "
                                 "(the reference divides by the circular size)")

    def decode_workspace(self, layer_idx: int, device) -> Tensor:
        """Scratch of the decode kernel (tickets + split partials), one per device, sized for the
        largest layer and zeroed once."""
        key = torch.device(device)
        ws = self._workspace.get(key)
        if ws is None:
            need = max(lib.moa_decode_workspace_bytes(self.batch_size, h, self.head_dim, s, self.decode_chunk)
                       for h, s in zip(self.num_head_for_each_layer, self.layer_cache_size))
            ws = torch.zeros(need, dtype=torch.uint8, device=key)
            self._workspace[key] = ws
        return ws

    # ------------------------------------------------------------------ update
    def update(
        self,
        key_states: Tensor,
        value_states: Tensor,
        layer_idx: int,
        attention_mask: Optional[Tensor] = None,
        cache_kwargs: Optional[Dict[str, Any]] = None,
    ) -> Tuple[Tensor, Tensor]:
        """Append ``(B, H, q_len, D)`` states.  q_len == 1: decode branch (cache_utils.py:1020-1058),
        returns the whole flattened caches ``(B, sum cap, D)``.  q_len > 1: prefill branch
        (:1060-1164) with an optional ``(B, kv_len)`` 0/1 int64 ``attention_mask`` for left
        padding, returns the states it was given."""
        assert layer_idx < self.num_layers
        H = self.num_head_for_each_layer[layer_idx]
        if key_states is not None:
            assert key_states.shape[1] == H
            device = key_states.device
            assert value_states.device == device, "key_states and value_states should be on the same device"
        else:
            assert not self.update_cache_content, "key_states may be None only with update_cache_content=False"
            device = self.cache_update_index[layer_idx].device
        if device.type != "cuda":
            raise RuntimeError("moa_b200.StaticCircularCache runs on CUDA tensors only (there is no CPU path)")
        if attention_mask is not None:
            assert attention_mask.device == device, "attention_mask should be on the same device as key_states"
        self._materialize(layer_idx, device)
        self._check_layout(layer_idx)

        seq_len = key_states.shape[-2] if key_states is not None else 1
        B = key_states.shape[0] if key_states is not None else self.batch_size
        assert B == self.batch_size
        D, S = self.head_dim, self.layer_cache_size[layer_idx]
        if layer_idx == 0:
            self.cache_position += seq_len
        stream = _lib.current_stream(device)
        code = _lib.dtype_code(self.dtype)
        kc, vc = self.key_cache[layer_idx], self.value_cache[layer_idx]

        if seq_len == 1:
            k_new = v_new = None
            nbs = nhs = 0
            if self.update_cache_content:
                assert key_states.dtype == self.dtype and value_states.dtype == self.dtype
                k_new = key_states[:, :, -1, :]
                v_new = value_states[:, :, -1, :]
                if k_new.stride(-1) != 1 or k_new.stride(0) % 8 or k_new.stride(1) % 8 or \
                        k_new.stride() != v_new.stride():
                    k_new, v_new = k_new.contiguous(), v_new.contiguous()
                nbs, nhs = k_new.stride(0), k_new.stride(1)
            with torch.cuda.device(device), _lib.nvtx_range("moa_b200.cache_append"):
                _lib.check("moa_cache_append", lib.moa_cache_append(
                    kc.data_ptr(), vc.data_ptr(), _lib.ptr(k_new), _lib.ptr(v_new), nbs, nhs,
                    self.cache_head_start_index[layer_idx].data_ptr(), self.cache_valid_length[layer_idx].data_ptr(),
                    self.cache_update_index[layer_idx].data_ptr(), self.mask_cache[layer_idx].data_ptr(),
                    self.static_cache_size[layer_idx].data_ptr(), self._kv_len[layer_idx], B, H, D, S, code, stream))
            self._kv_len[layer_idx] += 1
            return kc, vc

        assert self.update_cache_content, "prefill needs update_cache_content=True"
        assert key_states.dtype == self.dtype and value_states.dtype == self.dtype
        k, v = key_states, value_states
        if k.stride(-1) != 1 or any(s % 8 for s in k.stride()[:-1]) or k.stride() != v.stride():
            k, v = k.contiguous(), v.contiguous()
        pos = count = None
        with torch.cuda.device(device), _lib.nvtx_range("moa_b200.cache_fill"):
            if attention_mask is not None:
                assert attention_mask.dim() == 2, \
                    "The shape of the attention mask should be [batch_size, kv_len] and the dtype should be torch.int64."
                am = attention_mask[:, -seq_len:]
                if am.dtype != torch.int64 or am.stride(-1) != 1:
                    am = am.to(torch.int64).contiguous()
                key = (torch.device(device), seq_len)
                if key not in self._scan_buffers:
                    self._scan_buffers = {key: (torch.empty(B, seq_len, dtype=torch.int32, device=device),
                                                torch.empty(B, dtype=torch.int32, device=device))}
                pos, count = self._scan_buffers[key]
                _lib.check("moa_cache_scan_mask", lib.moa_cache_scan_mask(
                    am.data_ptr(), am.stride(0), pos.data_ptr(), count.data_ptr(), B, seq_len, stream))
            _lib.check("moa_cache_fill", lib.moa_cache_fill(
                k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.stride(2), kc.data_ptr(), vc.data_ptr(),
                _lib.ptr(pos), _lib.ptr(count), self.cache_head_start_index[layer_idx].data_ptr(),
                self.cache_valid_length[layer_idx].data_ptr(), self.cache_update_index[layer_idx].data_ptr(),
                self.mask_cache[layer_idx].data_ptr(), self.static_cache_size[layer_idx].data_ptr(),
                self._kv_len[layer_idx], B, H, seq_len, D, S, self._max_cap[layer_idx], code, stream))
        self._kv_len[layer_idx] += seq_len
        return key_states, value_states

    # ------------------------------------------------------------------ fused decode step
    def decode_attention(self, query_states: Tensor, key_states: Tensor, value_states: Tensor, layer_idx: int,
                         sm_scale: float, out: Optional[Tensor] = None,
                         rope: Optional[Tuple[Tensor, Tensor]] = None, out_dtype: Optional[torch.dtype] = None,
                         out_peers: Optional[Sequence[int]] = None, barrier: Optional[Tuple] = None) -> Tensor:
        """One decode step of one layer in one launch: append the new ``(B, H, 1, D)`` K/V rows at
        the ring's write index, attend over the cache including the new token, advance the
        bookkeeping.  Same result as ``update(...)`` followed by
        ``mixture_of_sparse_attention(...)``.  Returns ``(B, 1, H, D)``; ``out`` may be a
        pre-allocated tensor (or a ``(B, 1, H', D)`` slice of a wider gather buffer).

        ``query_states, key_states, value_states`` are read through their strides (no copy) as long as
        their rows are contiguous and 16-byte aligned — e.g. the three slices of one fused QKV
        projection output.  ``rope=(cos, sin)``, tables of shape ``(B, 1, D)`` or ``(B, D)`` in the cache
        dtype, makes the kernel apply the rotary embedding (Llama ``rotate_half`` convention) to
        ``query_states`` and ``key_states`` itself; they are then the raw projection outputs.
        ``out_dtype=torch.float32`` stores the fp32 result unrounded (parity checks of the bf16 path).
        ``out_peers``: device addresses of the same slice in other GPUs' gather buffers (mapped into
        this process); every output row is also stored there.  ``barrier``: the arguments of the cross-rank
        barrier that then ends the launch, ``(flag pointer array, rank, world, call-counter address, limit in
        cycles, status address)``; both are what ``PeerGather.decode_and_gather`` passes.

        The ring's write rule depends on the layer's token count, which is passed to the kernel by
        value from the host counter ``_kv_len``: a CUDA graph captured over this call replays the
        captured count.  That is exact once every ring has left its static part
        (``_kv_len > max(static_size)``, i.e. after any prompt longer than the sink); the host
        counters (``_kv_len``, ``cache_position``) are not advanced by a replay — the caller adds the
        replayed steps itself."""
        H = self.num_head_for_each_layer[layer_idx]
        B, D, S = self.batch_size, self.head_dim, self.layer_cache_size[layer_idx]
        device = query_states.device
        if device.type != "cuda":
            raise RuntimeError("moa_b200 runs on CUDA tensors only (there is no CPU path)")
        assert query_states.shape == (B, H, 1, D) and key_states.shape == (B, H, 1, D)
        assert value_states.shape == (B, H, 1, D)
        assert query_states.dtype == self.dtype and key_states.dtype == self.dtype and value_states.dtype == self.dtype
        self._materialize(layer_idx, device)
        self._check_layout(layer_idx)
        q = query_states[:, :, 0, :]
        if not _lib.rows_ok(q):
            q = q.contiguous()
        k_new, v_new = key_states[:, :, 0, :], value_states[:, :, 0, :]
        if not (_lib.rows_ok(k_new) and _lib.rows_ok(v_new) and k_new.stride() == v_new.stride()):
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
        if out is None:
            out = torch.empty(B, 1, H, D, dtype=out_dtype or self.dtype, device=device)
        assert out.shape == (B, 1, H, D) and out.stride(-1) == 1 and out.dtype in (self.dtype, torch.float32)
        ws = self.decode_workspace(layer_idx, device)
        if layer_idx == 0:
            self.cache_position += 1
        args = _lib.decode_arguments(
            q, self.key_cache[layer_idx], self.value_cache[layer_idx], k_new, v_new, out[:, 0],
            self.cache_head_start_index[layer_idx], self.cache_valid_length[layer_idx],
            self.cache_update_index[layer_idx], self.mask_cache[layer_idx], self.static_cache_size[layer_idx],
            self._kv_len[layer_idx], sm_scale)
        tail = (ws.data_ptr(), ws.numel(), self.decode_chunk, _lib.current_stream(device))
        cos = sin = None
        if rope is not None:
            cos, sin = rope
            cos, sin = cos.reshape(B, D).contiguous(), sin.reshape(B, D).contiguous()
            assert cos.dtype == self.dtype and sin.dtype == self.dtype and cos.device == device
        with torch.cuda.device(device):
            if out_peers or barrier is not None:
                n_peers = len(out_peers) if out_peers else 0
                peers = (ctypes.c_void_p * max(n_peers, 1))(*[int(a) for a in (out_peers or [])])
                bar = barrier if barrier is not None else (None, 0, 0, None, 0, None)
                with _lib.nvtx_range("moa_b200.decode_gather"):
                    _lib.check("moa_decode_gather_fwd", lib.moa_decode_gather_fwd(
                        *args, _lib.ptr(cos), _lib.ptr(sin), peers, n_peers, *bar, *tail))
            elif rope is not None:
                with _lib.nvtx_range("moa_b200.decode_rope_fused"):
                    _lib.check("moa_decode_rope_fwd", lib.moa_decode_rope_fwd(
                        *args, cos.data_ptr(), sin.data_ptr(), *tail))
            else:
                with _lib.nvtx_range("moa_b200.decode_fused"):
                    _lib.check("moa_decode_fwd", lib.moa_decode_fwd(*args, *tail))
        self._kv_len[layer_idx] += 1
        return out

    # ------------------------------------------------------------------ misc API of the reference
    def __len__(self):
        return len(self.key_cache)

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return self._kv_len[layer_idx]

    def get_max_length(self) -> Optional[int]:
        return None

    def reorder_cache(self, beam_idx: torch.LongTensor):
        raise NotImplementedError("Reordering the cache is not implemented currently!")

    # ------------------------------------------------------------------ checkpoint / resume (not in the reference)
    def state_dict(self) -> Dict[str, Any]:
        """Everything needed to continue decoding later: the sizes the cache was built with and, per layer,
        the payload, mask, valid lengths, next write indices and token count.  Tensors are clones."""
        materialised = [k.device.type != "meta" for k in self.key_cache]
        return {
            "cache_size": [list(c) for c in self._cap_host],
            "static_size": [list(c) for c in self._static_host],
            "batch_size": self.batch_size,
            "head_dim": self.head_dim,
            "dtype": str(self.dtype),
            "kv_len": list(self._kv_len),
            "cache_position": self.cache_position,
            "key_cache": [k.clone() if m else None for k, m in zip(self.key_cache, materialised)],
            "value_cache": [v.clone() if m else None for v, m in zip(self.value_cache, materialised)],
            "mask_cache": [t.clone() for t in self.mask_cache],
            "cache_valid_length": [t.clone() for t in self.cache_valid_length],
            "cache_update_index": [t.clone() for t in self.cache_update_index],
        }

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        """Restores a ``state_dict()`` into a cache built with the same sizes, batch, head_dim and dtype."""
        if (state["cache_size"] != [list(c) for c in self._cap_host] or
                state["static_size"] != [list(c) for c in self._static_host] or
                state["batch_size"] != self.batch_size or state["head_dim"] != self.head_dim or
                state["dtype"] != str(self.dtype)):
            raise ValueError("load_state_dict: the state was taken from a cache of a different shape or dtype")
        for layer in range(self.num_layers):
            k, v = state["key_cache"][layer], state["value_cache"][layer]
            if k is not None:     # tensors stay on the device they were saved from; update() moves what it needs
                self.key_cache[layer] = k.clone()
                self.value_cache[layer] = v.clone()
            self.mask_cache[layer] = state["mask_cache"][layer].clone()
            self.cache_valid_length[layer] = state["cache_valid_length"][layer].clone()
            self.cache_update_index[layer] = state["cache_update_index"][layer].clone()
        self._kv_len = list(state["kv_len"])
        self.cache_position = state["cache_position"]
