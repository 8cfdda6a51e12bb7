"""Host-side logic that needs no GPU: the split-count model of the attention wrapper and the prepared-call table's
keys (the calls themselves are covered by the GPU tests)."""
import torch

from omnistack_rs_b200.kernels import fused_attention as fa


def test_split_counts_of_the_benchmark_configurations():
    # the box-serving shard and the 64-user call are not split: plenty of work items, or too few keys
    assert fa._auto_splits(16384, 32, 32, 1, 2048, False) == 1
    assert fa._auto_splits(64, 8, 8, 1, 50, False) == 1
    # grouped-query decode over ragged long contexts: split, and coarser where the library orders the users by length
    assert fa._auto_splits(256, 32, 8, 1, 8192, True) == 4
    assert fa._auto_splits(256, 8, 8, 1, 8192, True) == 8            # one query column per kv head: index order
    assert fa._auto_splits(20000, 32, 8, 1, 8192, True) <= 8         # more users than the ordering handles
    # a single user with a long cache is split many ways, never below 64 keys per split
    s = fa._auto_splits(1, 32, 8, 1, 6000, False)
    assert s > 8 and 6000 // s >= 64
    # split counts never exceed what the C entry points accept
    for shape in [(1, 1, 1, 1, 1 << 20, False), (3, 8, 2, 16, 100000, True), (4096, 32, 8, 1, 128, False)]:
        assert 1 <= fa._auto_splits(*shape) <= 1024


def test_prepared_call_keys_tell_calls_apart():
    q = torch.zeros(2, 4, 1, 128, dtype=torch.bfloat16)
    a, b = torch.zeros(1), torch.zeros(1)
    flags = (True, False, False, False)
    k1 = fa._plan_key(q, [a, b], 0, 0.1, flags, None, None)
    assert k1 == fa._plan_key(q, [a, b], 0, 0.1, flags, None, None)
    assert k1 != fa._plan_key(q, [b, a], 0, 0.1, flags, None, None)                    # other tensors
    assert k1 != fa._plan_key(q.float(), [a, b], 0, 0.1, flags, None, None)            # other query dtype
    assert k1 != fa._plan_key(q[:1], [a, b], 0, 0.1, flags, None, None)                # other query shape
    assert k1 != fa._plan_key(q, [a, b], 1, 0.1, flags, None, None)                    # other user id
    assert k1 != fa._plan_key(q, [a, b], 0, 0.2, flags, None, None)                    # other scale
    assert k1 != fa._plan_key(q, [a, b], 0, 0.1, (True, True, False, False), None, None)
    assert k1 != fa._plan_key(q, [a, b], 0, 0.1, flags, 2, None)                       # explicit split count
    assert k1 != fa._plan_key(q, [a, b], 0, 0.1, flags, None, (None, None, None, None, 0.5))
    fa.clear_prepared_calls()
    assert len(fa._PLANS) == 0
