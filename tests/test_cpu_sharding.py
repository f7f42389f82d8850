"""Sequence-to-GPU assignment of the batched decode (greedy bin-packing on algorithmic bytes)."""
import numpy as np

from bonsai_mojo_1bit_optimization_t4_cuda_b200 import sharding


def test_every_sequence_is_assigned_once_and_loads_are_even():
    rng = np.random.default_rng(3)
    ctx = rng.integers(4096, 32769, size=256)
    win = rng.integers(128, 257, size=256)
    c_len = 128 * ((ctx - win) // 128)
    cost = sharding.algorithmic_bytes(c_len, ctx - c_len)
    for n in (1, 2, 4, 8):
        parts = sharding.partition_sequences(cost, n)
        assert len(parts) == n
        allidx = np.concatenate(parts)
        assert sorted(allidx.tolist()) == list(range(256))
        assert sharding.imbalance(cost, parts) < 1.01  # 256 uniform-random contexts pack to within 1 %
        # better than, or as good as, dealing them round-robin
        rr = [np.arange(r, 256, n) for r in range(n)]
        assert sharding.imbalance(cost, parts) <= sharding.imbalance(cost, rr) + 1e-12


def test_degenerate_inputs():
    assert [p.tolist() for p in sharding.partition_sequences([5], 3)] == [[0], [], []]
    assert [p.tolist() for p in sharding.partition_sequences([], 2)] == [[], []]
    parts = sharding.partition_sequences([7, 7, 7, 7], 2)
    assert sorted(len(p) for p in parts) == [2, 2]
    # deterministic: same costs, same answer
    again = sharding.partition_sequences([7, 7, 7, 7], 2)
    assert all((a == b).all() for a, b in zip(parts, again))
