"""Property tests (hypothesis) of the host-side plan arithmetic, head placement and the oracle's ring rules."""
import numpy as np
from hypothesis import given, settings, strategies as st

import moa_b200
from moa_b200 import plan as mplan
from oracle import moa_oracle as orc

heads = st.integers(min_value=1, max_value=12)


@settings(max_examples=200, deadline=None)
@given(st.data())
def test_cache_config_properties(data):
    H = data.draw(heads)
    alphas = data.draw(st.lists(st.floats(min_value=-4096, max_value=16384, allow_nan=False), min_size=H, max_size=H))
    betas = data.draw(st.lists(st.floats(min_value=0, max_value=2, allow_nan=False), min_size=H, max_size=H))
    n = data.draw(st.integers(min_value=1, max_value=200000))
    max_new = data.draw(st.sampled_from([0, 1, 64, 1024]))
    cfg = {"alphas": [alphas], "betas": [betas]}
    got = moa_b200.moa_config_to_cache_config(cfg, n, max_new, verbose=False)
    assert got == orc.cache_config(cfg, n, max_new)
    for cap, static in zip(got["cache_size"][0], got["static_size"][0]):
        assert cap % 64 == 0 and cap >= 128                       # rounded up to blocks, never below the minimum
        assert cap < n + max_new + 64 or cap == 128                # capped by the sequence (before rounding)
        assert static == min(cap, 64)


@settings(max_examples=200, deadline=None)
@given(st.data())
def test_shard_heads_is_a_balanced_partition(data):
    world = data.draw(st.sampled_from([1, 2, 4, 8]))
    per = data.draw(st.integers(min_value=1, max_value=8))
    costs = data.draw(st.lists(st.integers(min_value=64, max_value=20000), min_size=world * per, max_size=world * per))
    shards = mplan.shard_heads(costs, world)
    assert sorted(h for s in shards for h in s) == list(range(len(costs)))   # a partition of the heads
    assert all(len(s) == per for s in shards)                                # equal head counts
    assert all(s == sorted(s, key=lambda i: (costs[i], i)) for s in shards)  # sorted by cost inside a shard
    loads = [sum(costs[h] for h in s) for s in shards]
    assert max(loads) - min(loads) <= max(costs)                             # LPT bound for equal-count bins


@settings(max_examples=200, deadline=None)
@given(st.integers(min_value=0, max_value=100000), st.sampled_from([128, 192, 320, 1088, 4160]),
       st.sampled_from([0, 64]))
def test_slot_rule(t, cap, sink):
    """Token t of a row lives at slot t while it is a sink token, then cycles through the ring."""
    slot = orc.slot_of_token(t, cap, sink)
    assert 0 <= slot < cap
    if t < sink:
        assert slot == t
    else:
        assert sink <= slot and (slot - sink) == (t - sink) % (cap - sink)


@settings(max_examples=100, deadline=None)
@given(st.integers(min_value=1, max_value=40), st.integers(min_value=0, max_value=4), st.integers(min_value=1, max_value=50))
def test_block_layout_counts_match_the_flop_formula(nb, sink_b, local_b):
    lay = orc.block_layout(nb, sink_b, local_b)
    assert int(lay.sum()) == orc.prefill_block_visits(nb * 64, [sink_b], [local_b]) == \
        mplan.prefill_block_visits(nb * 64, [sink_b], [local_b])
    assert not np.triu(lay, 1).any()                                         # causal at block level
    assert lay.diagonal().all() or local_b == 0                              # a block always sees itself
