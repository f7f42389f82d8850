"""Which GPU serves which sequence.

Batched decode shards by sequence with no collective: every GPU holds all layers of its own
sequences.  A step lasts as long as the most loaded GPU, and a sequence's cost is its algorithmic
bytes ``B_alg = 4 * (220 * c_len + 1024 * win_len)`` per layer, so the sequences are dealt by
greedy bin-packing on that figure (longest first, each to the least loaded GPU so far).  The
reference serves one sequence on one GPU and has nothing to compare with.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np


def algorithmic_bytes(c_len, win_len) -> np.ndarray:
    """Per-sequence bytes one attention layer-step has to read."""
    return 4 * (220 * np.asarray(c_len, np.int64) + 1024 * np.asarray(win_len, np.int64))


def partition_sequences(cost: Sequence[int], n_ranks: int) -> List[np.ndarray]:
    """Greedy longest-first bin-packing.  Returns, per rank, the sorted indices of its sequences;
    every index appears exactly once.  Ties go to the lower rank, so every process computes the
    same assignment from the same costs."""
    cost = np.asarray(cost, np.int64)
    if n_ranks <= 0:
        raise ValueError("n_ranks must be positive")
    load = np.zeros(n_ranks, np.int64)
    count = np.zeros(n_ranks, np.int64)
    bins: List[List[int]] = [[] for _ in range(n_ranks)]
    for i in np.argsort(-cost, kind="stable"):
        # least loaded; among equals the one holding fewer sequences, then the lower rank
        r = int(np.lexsort((np.arange(n_ranks), count, load))[0])
        bins[r].append(int(i))
        load[r] += cost[i]
        count[r] += 1
    return [np.array(sorted(b), np.int64) for b in bins]


def imbalance(cost: Sequence[int], parts: Sequence[np.ndarray]) -> float:
    """max rank load / mean rank load (1.0 = perfectly even)."""
    cost = np.asarray(cost, np.int64)
    loads = np.array([cost[p].sum() if len(p) else 0 for p in parts], np.float64)
    return float(loads.max() / max(loads.mean(), 1.0))
