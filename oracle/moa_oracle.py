"""CPU restatement of the MoA attention hot path.  TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA kernels in ``moa_b200/csrc``: the tests, the smoke
entry and the CPU-baseline leg of the benchmark are its only callers.  Nothing in the
``moa_b200`` package imports it, and the package has no CPU fallback.

Every function restates one piece of thu-nics/MoA and cites the file:line it follows
(paths are relative to the MoA repository root).  Integer results (cache sizes, slot
indices, valid lengths, masks, block layouts) are meant to be bit-exact with the reference;
floating-point results are fp32 evaluations of the same mask, which is what the fp16/bf16
kernels are compared with (max-abs 2e-3, mean-rel 1e-3).

Parity pin: the golden fixtures under ``tests/golden`` were produced by running the
reference's own code (``StaticCircularCache``, ``moa_config_to_cache_config``,
``gen_bigbird_pattern``/``layout_to_mask``, the Triton prefill kernel under the Triton
interpreter and the ``"sdpa"`` decode path) on CPU; ``tests/test_oracle_golden.py`` checks this
restatement against them.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

BLOCK = 64  # MoA/kernels/mixture_of_attention.py:32-33 (BLOCK_M = BLOCK_N = 64)


# --------------------------------------------------------------------------------------
# plan -> cache sizes                                   MoA/attention/cache_utils.py:1183-1298
# --------------------------------------------------------------------------------------
def cache_config(
    moa_config: Dict,
    seq_len: int,
    max_new_token: int = 1024,
    sink_size: int = 64,
    minimum_cache_size: int = 128,
    split_size: int = 64,
) -> Dict[str, List[List[int]]]:
    """Per-head cache capacity and static (sink) size.

    Follows cache_utils.py:1224-1237: ``int()`` truncation toward zero, clamp to
    ``seq_len + max_new_token`` *before* rounding up to ``split_size``.
    """
    cache_size, static_size = [], []
    total = seq_len + max_new_token
    for alphas, betas in zip(moa_config["alphas"], moa_config["betas"]):
        cs, ss = [], []
        for a, b in zip(alphas, betas):
            c = int(a + total * b)
            c = min(c, total)
            c = math.ceil(max(c, minimum_cache_size) / split_size) * split_size
            cs.append(c)
            ss.append(min(c, sink_size))
        cache_size.append(cs)
        static_size.append(ss)
    return {"cache_size": cache_size, "static_size": static_size}


def permutation(moa_config: Dict) -> Tuple[List[List[int]], List[Dict[int, Tuple[int, int]]]]:
    """Head order that clusters equal (alpha, beta).  MoA/attention/permutation_utils.py:219-269."""
    perms, clusters = [], []
    for alphas, betas in zip(moa_config["alphas"], moa_config["betas"]):
        combined = sorted(zip(alphas, betas, range(len(alphas))), key=lambda x: (x[0], x[1]))
        perms.append([c[2] for c in combined])
        cl, start = {}, 0
        for i in range(1, len(combined)):
            if combined[i - 1][:2] != combined[i][:2]:
                cl[len(cl)] = (start, i - 1)
                start = i
        cl[len(cl)] = (start, len(combined) - 1)
        clusters.append(cl)
    return perms, clusters


# --------------------------------------------------------------------------------------
# prefill mask                    MoA/kernels/block_sparse_attention_prefill.py:555-580
# --------------------------------------------------------------------------------------
def block_layout(nb: int, sink_blocks: int, local_blocks: int) -> np.ndarray:
    """Boolean [nb, nb] block layout visited by the reference prefill kernel.

    q-block ``bi`` visits kv-block ``j`` iff ``j <= bi`` and (``j <= sink_blocks-1`` or
    ``j >= bi+1-local_blocks``)  (block_sparse_attention_prefill.py:558-567).
    """
    bi = np.arange(nb)[:, None]
    j = np.arange(nb)[None, :]
    return (j <= bi) & ((j <= sink_blocks - 1) | (j >= bi + 1 - local_blocks))


def prefill_mask(n: int, sink_blocks: int, local_blocks: int) -> np.ndarray:
    """Boolean [n, n] element mask: block layout expanded to tokens, and-ed with causal
    (block_sparse_attention_prefill.py:579-580)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    bi, bj = i // BLOCK, j // BLOCK
    return (j <= i) & ((bj <= sink_blocks - 1) | (bj >= bi + 1 - local_blocks))


def prefill_block_visits(n: int, sink_blocks: Sequence[int], local_blocks: Sequence[int]) -> int:
    """Number of 64x64 blocks the reference kernel computes for one batch row."""
    nb = -(-n // BLOCK)
    return int(sum(block_layout(nb, int(s), int(l)).sum() for s, l in zip(sink_blocks, local_blocks)))


def prefill_attention_fp32(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: float,
    sink_blocks: Sequence[int],
    local_blocks: Sequence[int],
    row_chunk: int = 2048,
    row_range: Optional[Tuple[int, int]] = None,
) -> torch.Tensor:
    """fp32 softmax(mask(q k^T * sm_scale)) v with the MoA mask.

    q, k, v: (B, H, N, D) any float dtype.  Returns (B, N, H, D) fp32, the layout
    ``mixture_of_sparse_attention`` returns (mixture_of_attention.py:399, 459).
    Rows are processed in chunks so N = 64k stays within host memory.  ``row_range=(a, b)``
    evaluates only query rows [a, b) and returns (B, b-a, H, D): long sequences are spot-checked
    this way.
    """
    B, H, N, D = q.shape
    ra, rb = row_range if row_range is not None else (0, N)
    out = torch.empty(B, rb - ra, H, D, dtype=torch.float32)
    for h in range(H):
        s_b, l_b = int(sink_blocks[h]), int(local_blocks[h])
        for r0 in range(ra, rb, row_chunk):
            r1 = min(rb, r0 + row_chunk)
            kf = k[:, h, :r1].float()
            vf = v[:, h, :r1].float()
            # columns that can be visible to rows [r0, r1): sink blocks + band
            i = torch.arange(r0, r1)[:, None]
            j = torch.arange(0, r1)[None, :]
            vis = (j <= i) & (((j // BLOCK) <= s_b - 1) | ((j // BLOCK) >= (i // BLOCK) + 1 - l_b))
            keep = vis.any(dim=0)                      # drop columns no row of the chunk sees
            cols = torch.nonzero(keep).flatten()
            s = torch.matmul(q[:, h, r0:r1].float(), kf[:, cols].transpose(-1, -2)) * sm_scale
            s = s.masked_fill(~vis[None][:, :, cols], float("-inf"))
            p = torch.softmax(s, dim=-1)
            out[:, r0 - ra:r1 - ra, h] = torch.matmul(p, vf[:, cols])
    return out


def prefill_attention_masked_sdpa(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: float,
    sink_blocks: Sequence[int],
    local_blocks: Sequence[int],
) -> torch.Tensor:
    """The PyTorch route to the same result, as a timed CPU baseline: one scaled_dot_product_attention call
    over all heads with the boolean element mask (the mask MoA/attention/convert.py:159-192 ``layout_to_mask``
    expands from the block layout of MoA/attention/pattern.py:149-183, and-ed with causal), in the tensors'
    dtype.  q, k, v: (B, H, N, D); returns (B, N, H, D)."""
    n = q.shape[2]
    mask = torch.from_numpy(np.stack([prefill_mask(n, int(s), int(l)) for s, l in zip(sink_blocks, local_blocks)]))
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask[None], scale=sm_scale)
    return out.transpose(1, 2)


# --------------------------------------------------------------------------------------
# ring cache bookkeeping                       MoA/attention/cache_utils.py:644-1180
# --------------------------------------------------------------------------------------
def _pymod(x: np.ndarray, m: np.ndarray) -> np.ndarray:
    """Python/torch ``%`` on integers: result has the sign of the divisor."""
    return np.mod(x, m)


class RingCacheOracle:
    """numpy restatement of ``StaticCircularCache`` for one layer list.

    State per layer (names follow cache_utils.py:698-818): ``cache_max_length`` [H],
    ``static_cache_size`` [H], ``circular_cache_size`` [H], ``head_index`` [H+1],
    ``cache_head_start_index`` [B,H], ``circular_cache_head_index`` [H],
    ``cache_update_index`` [B,H], ``cache_valid_length`` [B,H], ``mask_cache`` [B,S],
    ``key_cache``/``value_cache`` [B,S,D], ``_kv_len`` int.
    """

    def __init__(self, cache_size, static_size=None, batch_size=1, head_dim=128, dtype=np.float32):
        self.num_layers = len(cache_size)
        if static_size is None:
            static_size = [[0] * len(c) for c in cache_size]
        self.batch_size, self.head_dim = batch_size, head_dim
        self.cache_max_length = [np.asarray(c, dtype=np.int64) for c in cache_size]
        self.static_cache_size = [np.asarray(s, dtype=np.int64) for s in static_size]
        self.circular_cache_size = [c - s for c, s in zip(self.cache_max_length, self.static_cache_size)]
        self.head_index = [np.concatenate([[0], np.cumsum(c)]).astype(np.int64) for c in self.cache_max_length]
        self.layer_cache_size = [int(h[-1]) for h in self.head_index]
        self.cache_head_start_index = [np.tile(h[:-1][None], (batch_size, 1)) for h in self.head_index]
        self.circular_cache_head_index = [h[:-1] + s for h, s in zip(self.head_index, self.static_cache_size)]
        self.cache_update_index = [np.tile(h[:-1][None], (batch_size, 1)) for h in self.head_index]
        self.cache_valid_length = [np.zeros((batch_size, len(c)), dtype=np.int64) for c in cache_size]
        self.mask_cache = [np.zeros((batch_size, s), dtype=np.int64) for s in self.layer_cache_size]
        self.key_cache = [np.zeros((batch_size, s, head_dim), dtype=dtype) for s in self.layer_cache_size]
        self.value_cache = [np.zeros((batch_size, s, head_dim), dtype=dtype) for s in self.layer_cache_size]
        self._kv_len = [0] * self.num_layers
        self.cache_position = 0

    def update(self, key: np.ndarray, value: np.ndarray, layer: int, attention_mask: Optional[np.ndarray] = None):
        """key/value: (B, H, q_len, D).  Decode branch cache_utils.py:1020-1058, prefill
        branch :1060-1164.  Returns what the reference returns."""
        B, H, n, _ = key.shape
        if layer == 0:
            self.cache_position += n
        upd = self.cache_update_index[layer]
        cs = self.circular_cache_head_index[layer][None, :]
        circ = self.circular_cache_size[layer][None, :]
        static = self.static_cache_size[layer][None, :]
        kv = self._kv_len[layer]
        bidx = np.arange(B)[:, None]
        if n == 1:
            self.mask_cache[layer][bidx, upd] = 1
            self.value_cache[layer][bidx, upd] = value[:, :, -1, :]
            self.key_cache[layer][bidx, upd] = key[:, :, -1, :]
            self.cache_valid_length[layer] += self.cache_valid_length[layer] < self.cache_max_length[layer][None, :]
            is_circ = (kv + 1) > static
            nxt_c = _pymod(upd + 1 - cs, circ) + cs
            self.cache_update_index[layer] = np.where(is_circ, nxt_c, upd + 1)
            self._kv_len[layer] += 1
            return self.key_cache[layer], self.value_cache[layer]

        if attention_mask is None:
            am = np.ones((B, n), dtype=np.int64)
        else:
            am = np.asarray(attention_mask)[:, -n:].astype(np.int64)
        adv = np.cumsum(am, axis=-1) - 1
        adv = np.concatenate([adv, adv[:, -1:] + 1], axis=-1)            # (B, n+1)
        rev = np.flip(np.cumsum(np.flip(am, -1), axis=-1), -1)           # (B, n)
        a3 = adv[:, :, None]
        idx_c = _pymod(upd[:, None, :] + a3 - cs[None], circ[None]) + cs[None]
        idx_s = upd[:, None, :] + a3
        idx = np.where(kv + a3 > static[None], idx_c, idx_s)             # (B, n+1, H)
        self.cache_update_index[layer] = idx[:, -1, :].copy()
        idx = idx[:, :-1, :].transpose(0, 2, 1)                          # (B, H, n)
        keep = ((rev[:, None, :] <= circ[:, :, None]) | (idx < cs[:, :, None])) & (am[:, None, :] == 1)
        self.cache_valid_length[layer] += keep.sum(-1)
        self._kv_len[layer] += n
        b_ix, h_ix, t_ix = np.nonzero(keep)
        slots = idx[b_ix, h_ix, t_ix]
        self.mask_cache[layer][b_ix, slots] = 1
        self.key_cache[layer][b_ix, slots] = key[b_ix, h_ix, t_ix]
        self.value_cache[layer][b_ix, slots] = value[b_ix, h_ix, t_ix]
        return key, value


def slot_of_token(t: int, cap: int, sink: int) -> int:
    """Local slot of the t-th unmasked token of a row: ``t`` inside the sink, else the ring
    (consequence of cache_utils.py:1041-1054 / :1088-1107 when the cache starts empty)."""
    return t if t < sink else sink + (t - sink) % (cap - sink)


# --------------------------------------------------------------------------------------
# decode attention            MoA/kernels/mixture_of_attention.py:226-310, 465-473
# --------------------------------------------------------------------------------------
def decode_attention_fp32(
    q: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    head_start_index: torch.Tensor,
    head_valid_length: torch.Tensor,
    sm_scale: float,
) -> torch.Tensor:
    """fp32 softmax(q K[start:start+valid]^T * sm_scale) V per (batch, head).

    q: (B, H, 1, D); caches (B, S, D); start/valid (B, H).  Returns (B, 1, H, D) fp32 — the
    contract of the ``moa_decode`` call at mixture_of_attention.py:466-473.
    """
    B, H, _, D = q.shape
    out = torch.zeros(B, 1, H, D, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            s0 = int(head_start_index[b, h])
            n = int(head_valid_length[b, h])
            if n == 0:
                continue
            kk = key_cache[b, s0 : s0 + n].float()
            vv = value_cache[b, s0 : s0 + n].float()
            s = (kk @ q[b, h, 0].float()) * sm_scale
            p = torch.softmax(s, dim=0)
            out[b, 0, h] = p @ vv
    return out


def decode_attention_grouped_sdpa(
    q: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    head_index: torch.Tensor,
    sm_scale: float,
) -> torch.Tensor:
    """The reference's own CPU-runnable decode path (``implementation="sdpa"``): regroup runs of
    equal-capacity heads into (B, Hg, cap, D) and call SDPA per group
    (cache_utils.py:889-951, mixture_of_attention.py:226-310).  Computes in the cache dtype,
    exact only for full rings.  Used as the timed CPU baseline."""
    B, H, _, D = q.shape
    caps = (head_index[1:] - head_index[:-1]).tolist()
    outs, h = [], 0
    while h < H:
        g = h
        while g < H and caps[g] == caps[h]:
            g += 1
        s0, s1 = int(head_index[h]), int(head_index[g])
        kk = key_cache[:, s0:s1].view(B, g - h, caps[h], D)
        vv = value_cache[:, s0:s1].view(B, g - h, caps[h], D)
        outs.append(torch.nn.functional.scaled_dot_product_attention(q[:, h:g], kk, vv, scale=sm_scale))
        h = g
    return torch.cat(outs, dim=1).transpose(1, 2)


def ring_cache_step_torch(state: Dict, key: torch.Tensor, value: torch.Tensor) -> None:
    """Decode-branch cache update on torch CPU tensors, for the timed CPU baseline
    (cache_utils.py:1020-1058).  ``state`` holds key_cache, value_cache, update_index,
    valid_length, max_length, static, circ, circ_start, kv_len."""
    B = key.shape[0]
    bidx = torch.arange(B)[:, None]
    upd = state["update_index"]
    state["value_cache"][bidx, upd] = value[:, :, -1, :]
    state["key_cache"][bidx, upd] = key[:, :, -1, :]
    state["valid_length"] += state["valid_length"] < state["max_length"][None]
    is_c = (state["kv_len"] + 1 > state["static"])[None]
    cs, circ = state["circ_start"][None], state["circ"][None]
    state["update_index"] = torch.where(is_c, (upd + 1 - cs) % circ + cs, upd + 1)
    state["kv_len"] += 1


# --------------------------------------------------------------------------------------
# algorithmic work
# --------------------------------------------------------------------------------------
def prefill_flops(batch: int, n: int, d: int, sink_blocks, local_blocks) -> int:
    """4*64*64*D flop for every visited 64x64 block (two GEMMs, 2 flop per MAC)."""
    return batch * prefill_block_visits(n, sink_blocks, local_blocks) * 4 * BLOCK * BLOCK * d


def decode_bytes(batch: int, valid_lengths: Sequence[int], d: int, itemsize: int) -> int:
    """K and V rows read for every valid slot, plus q read, o write and the new K/V rows."""
    h = len(valid_lengths)
    return batch * int(sum(valid_lengths)) * d * 2 * itemsize + 4 * batch * h * d * itemsize


# --------------------------------------------------------------------------------------
# one attention layer      MoA/models/llama/modeling_llama.py:206-332 (LlamaMixtureAttention.forward)
# --------------------------------------------------------------------------------------
def rope_cos_sin(position_ids: torch.Tensor, head_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables of shape (B, q, D) in fp32, as the Llama rotary embedding builds them:
    inv_freq = theta^(-2i/D), angles duplicated over the two halves of the head dim."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = position_ids[:, :, None].float() * inv_freq[None, None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (B, H, q, D): x*cos + rotate_half(x)*sin with rotate_half(x) = cat(-x[D/2:], x[:D/2])."""
    d = x.shape[-1]
    rot = torch.cat([-x[..., d // 2:], x[..., : d // 2]], dim=-1)
    return x * cos[:, None] + rot * sin[:, None]


def attention_layer_fp32(
    hidden: torch.Tensor,
    wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor,
    num_heads: int,
    position_ids: torch.Tensor,
    cache: "RingCacheOracle",
    layer: int,
    rope_theta: float = 10000.0,
    cache_dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """fp32 restatement of one MoA attention layer: q/k/v projection -> view (B,H,q,D) -> RoPE ->
    cache.update -> sparse prefill (q_len > 1) or decode over the ring (q_len == 1) -> o_proj.
    Q/K/V are rounded to ``cache_dtype`` where the reference holds them in the model dtype, so the
    cache payload can be compared bit-for-bit.  Returns (B, q, hidden) fp32."""
    B, q_len, hid = hidden.shape
    D = wq.shape[0] // num_heads
    x = hidden.float()
    q = (x @ wq.float().T).view(B, q_len, num_heads, D).transpose(1, 2)
    k = (x @ wk.float().T).view(B, q_len, num_heads, D).transpose(1, 2)
    v = (x @ wv.float().T).view(B, q_len, num_heads, D).transpose(1, 2)
    cos, sin = rope_cos_sin(position_ids, D, rope_theta)
    q = apply_rope(q, cos, sin).to(cache_dtype)
    k = apply_rope(k, cos, sin).to(cache_dtype)
    v = v.to(cache_dtype)
    sm = D ** -0.5
    np_dtype = np.float16 if cache_dtype == torch.float16 else np.float32
    to_np = (lambda t: t.contiguous().numpy()) if cache_dtype == torch.float16 else (lambda t: t.float().contiguous().numpy())
    if q_len > 1:
        cache.update(to_np(k), to_np(v), layer)
        sink_b = (cache.static_cache_size[layer] // BLOCK).tolist()
        local_b = (cache.circular_cache_size[layer] // BLOCK).tolist()
        attn = prefill_attention_fp32(q, k, v, sm, sink_b, local_b)            # (B, q, H, D)
    else:
        kc, vc = cache.update(to_np(k), to_np(v), layer)
        attn = decode_attention_fp32(q, torch.from_numpy(kc.astype(np.float32)), torch.from_numpy(vc.astype(np.float32)),
                                     torch.from_numpy(cache.cache_head_start_index[layer]),
                                     torch.from_numpy(cache.cache_valid_length[layer]), sm)
    return attn.reshape(B, q_len, num_heads * D) @ wo.float().T
