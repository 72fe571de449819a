"""Plan JSON handling: cache sizes, head permutation, algorithmic work, head sharding.

Mirrors, by name and argument meaning, MoA/attention/cache_utils.py:1183-1298
(``moa_config_to_cache_config``) and MoA/attention/permutation_utils.py:5-96, 219-269.
A plan is ``{"alphas": [[float]*H]*L, "betas": [[float]*H]*L}``
(MoA/universal/elastic_block_sparse.py:231-252).
"""
from __future__ import annotations

import json
import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

BLOCK = 64  # block size of the prefill mask and of the cache split


def load_plan(path: str) -> Dict:
    with open(path) as f:
        plan = json.load(f)
    assert "alphas" in plan and "betas" in plan, "a MoA plan needs 'alphas' and 'betas'"
    assert len(plan["alphas"]) == len(plan["betas"])
    return plan


def moa_config_to_cache_config(
    moa_config: Dict,
    seq_len: int,
    max_new_token: int = 1024,
    sink_size: int = 64,
    minimum_cache_size: int = 128,
    split_size: int = 64,
    verbose: bool = True,
) -> Dict[str, List[List[int]]]:
    """Per-head cache capacity ``int(alpha + (seq_len+max_new_token)*beta)``, clamped to
    ``seq_len+max_new_token``, raised to ``minimum_cache_size`` and rounded up to
    ``split_size``; static part ``min(capacity, sink_size)``  (cache_utils.py:1224-1237)."""
    total = seq_len + max_new_token
    cache_size, static_size = [], []
    for alphas, betas in zip(moa_config["alphas"], moa_config["betas"]):
        c_layer, s_layer = [], []
        for alpha, beta in zip(alphas, betas):
            c = int(alpha + total * beta)
            c = min(c, total)
            c = math.ceil(max(c, minimum_cache_size) / split_size) * split_size
            c_layer.append(c)
            s_layer.append(min(c, sink_size))
        cache_size.append(c_layer)
        static_size.append(s_layer)
    if verbose:
        print("Cache configuration")
        for i, (c, s) in enumerate(zip(cache_size, static_size)):
            ratio = [x / total for x in c]
            print(f"  layer {i}: cache mean {sum(c) / len(c):.2f} min {min(c)} max {max(c)}; "
                  f"static mean {sum(s) / len(s):.2f}; ratio mean {sum(ratio) / len(ratio):.2f}")
    return {"cache_size": cache_size, "static_size": static_size}


def moa_config_to_permutation(moa_config: Dict) -> Tuple[List[torch.Tensor], List[Dict[int, Tuple[int, int]]]]:
    """Per layer, the head order sorted by (alpha, beta) (stable) and the clusters
    ``{i: (start, end_inclusive)}`` of equal pairs  (permutation_utils.py:219-269)."""
    permutations, clusters = [], []
    for alphas, betas in zip(moa_config["alphas"], moa_config["betas"]):
        order = sorted(zip(alphas, betas, range(len(alphas))), key=lambda x: (x[0], x[1]))
        permutations.append(torch.tensor([o[2] for o in order]))
        cluster, start = {}, 0
        for i in range(1, len(order)):
            if order[i - 1][:2] != order[i][:2]:
                cluster[len(cluster)] = (start, i - 1)
                start = i
        cluster[len(cluster)] = (start, len(order) - 1)
        clusters.append(cluster)
    return permutations, clusters


def permute_attention_projection(layer: torch.nn.Linear, permutation: Optional[torch.Tensor] = None,
                                 num_heads: Optional[int] = None, num_key_value_groups: Optional[int] = None) -> None:
    """Reorder the head row-blocks of a q/k/v projection  (permutation_utils.py:5-53)."""
    if permutation is None:
        return
    assert permutation.dim() == 1 and permutation.shape[0] == num_heads
    if num_key_value_groups is not None and num_key_value_groups != 1:
        g = num_key_value_groups
        permutation = torch.tensor([i * g + r for i in permutation.tolist() for r in range(g)],
                                   device=permutation.device, dtype=permutation.dtype)
        num_heads = num_heads * g
    w = layer.weight.data
    head_dim = layer.out_features // num_heads
    layer.weight.data = w.reshape(num_heads, head_dim, layer.in_features)[permutation].reshape_as(w).contiguous()
    if layer.bias is not None:
        bias = layer.bias.data
        layer.bias.data = bias.reshape(num_heads, head_dim)[permutation].reshape_as(bias).contiguous()


def permute_output_projection(layer: torch.nn.Linear, permutation: Optional[torch.Tensor] = None,
                              num_heads: Optional[int] = None, num_key_value_groups: Optional[int] = None) -> None:
    """Reorder the head column-blocks of o_proj so it accepts permuted heads  (permutation_utils.py:55-96)."""
    if permutation is None:
        return
    assert permutation.dim() == 1 and permutation.shape[0] == num_heads
    if num_key_value_groups is not None and num_key_value_groups != 1:
        g = num_key_value_groups
        permutation = torch.tensor([i * g + r for i in permutation.tolist() for r in range(g)],
                                   device=permutation.device, dtype=permutation.dtype)
        num_heads = num_heads * g
    w = layer.weight.data
    head_dim = layer.in_features // num_heads
    layer.weight.data = (w.reshape(layer.out_features, num_heads, head_dim)[:, permutation]
                         .reshape_as(w).contiguous())


# ---------------------------------------------------------------------------------------------
# algorithmic work (what the roofline fractions are computed from)
# ---------------------------------------------------------------------------------------------
def prefill_block_visits(n: int, sink_blocks: Sequence[int], local_blocks: Sequence[int]) -> int:
    """64x64 blocks inside sink U band, per batch row: q-block i visits
    ``min(i+1, sink) + band blocks not already counted``."""
    nb = -(-n // BLOCK)
    total = 0
    for s, l in zip(sink_blocks, local_blocks):
        s, l = int(s), int(l)
        for i in range(nb):
            n_sink = min(s, i + 1)
            band_lo = max(n_sink, i + 1 - l)
            total += n_sink + max(0, i + 1 - band_lo)
    return total


def prefill_flops(batch: int, n: int, head_dim: int, sink_blocks, local_blocks) -> int:
    """Dense-equivalent flop on the band: 4*64*64*D per visited block."""
    return batch * prefill_block_visits(n, sink_blocks, local_blocks) * 4 * BLOCK * BLOCK * head_dim


def decode_bytes(batch: int, valid_lengths: Sequence[int], head_dim: int, itemsize: int) -> int:
    """Bytes one decode step of one layer must move: K and V of every valid slot, plus q, o and
    the new K/V row of every head."""
    h = len(valid_lengths)
    return batch * int(sum(valid_lengths)) * head_dim * 2 * itemsize + 4 * batch * h * head_dim * itemsize


# ---------------------------------------------------------------------------------------------
# head sharding across GPUs
# ---------------------------------------------------------------------------------------------
def shard_heads(costs: Sequence[float], world_size: int) -> List[List[int]]:
    """Longest-processing-time bin packing of heads onto ``world_size`` ranks with an equal number
    of heads per rank (H must divide).  Returns the head ids of every rank, each list sorted by
    cost (so equal-capacity heads stay adjacent, as ``permute_head`` arranges in the reference)."""
    h = len(costs)
    assert h % world_size == 0, "the number of heads must be a multiple of the number of ranks"
    per = h // world_size
    loads = [0.0] * world_size
    shards: List[List[int]] = [[] for _ in range(world_size)]
    for head in sorted(range(h), key=lambda i: (-costs[i], i)):
        r = min((r for r in range(world_size) if len(shards[r]) < per), key=lambda r: (loads[r], r))
        shards[r].append(head)
        loads[r] += costs[head]
    return [sorted(s, key=lambda i: (costs[i], i)) for s in shards]
