"""Grouping of node blocks by fan-in so that padded edge tables waste little work.

Restates PyJuice's ``partition_nodes_by_n_edges`` (layer/backend/node_partition.py:179-226,
algorithm "dp_with_coalesce") in plain Python/NumPy.  The result decides the shapes of every
compiled index table, so the arithmetic follows the original step by step, including the way
its back-trace walks one fixed column of the DP table (node_partition.py:43-47).
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np

_INT31_MAX = 2 ** 31 - 1


def next_power_of_2(x: np.ndarray) -> np.ndarray:
    """Smallest power of two >= x, elementwise, for positive integers (layer/compilation.py:95-100)."""
    x = np.asarray(x, dtype=np.int64)
    return np.array([1 << (int(v) - 1).bit_length() if v > 1 else 1 for v in x.reshape(-1)], dtype=np.int64).reshape(x.shape)


def _coalesce(vals: np.ndarray):
    """Merge runs of distinct values lying within floor((max-min)/1000) of the run's first value;
    a run is represented by its last (largest) value and its total multiplicity
    (node_partition.py:72-114)."""
    uniq, counts = np.unique(vals, return_counts=True)
    tol = int(math.floor((int(uniq.max()) - int(uniq.min())) / 1000))
    keep_vals, keep_counts = [], []
    run_first, run_count = None, 0
    for i in range(uniq.shape[0]):
        if run_first is None:
            run_first, run_count = int(uniq[i]), int(counts[i])
        elif int(uniq[i]) - run_first <= tol:
            run_count += int(counts[i])
        else:
            keep_vals.append(int(uniq[i - 1]))
            keep_counts.append(run_count)
            run_first, run_count = int(uniq[i]), int(counts[i])
    if run_first is not None:
        keep_vals.append(int(uniq[-1]))
        keep_counts.append(run_count)
    return np.asarray(keep_vals, dtype=np.int64), np.asarray(keep_counts, dtype=np.int64)


def _weighted_dp(vals: np.ndarray, counts: np.ndarray, max_num_partitions: int, target_overhead: int):
    """dp[i][p] = least padded work covering values[0..i] with p groups, each group padded to its
    largest value (node_partition.py:117-176)."""
    n = vals.shape[0]
    cum = np.cumsum(counts)
    dp = np.zeros((n, max_num_partitions + 1), dtype=np.int64)
    back = np.zeros((n, max_num_partitions + 1), dtype=np.int64)
    dp[:, 1] = vals * cum
    if dp[n - 1, 1] <= target_overhead:
        return 1, back
    chosen = max_num_partitions
    for p in range(2, max_num_partitions + 1):
        dp[0, p] = vals[0] * cum[0]
        back[0, p] = 0
        for i in range(1, n):
            # candidates j = 0..i-1, first minimum wins
            cand = dp[:i, p - 1] + vals[i] * (cum[i] - cum[:i])
            j = int(np.argmin(cand))
            if cand[j] < _INT31_MAX:
                dp[i, p], back[i, p] = cand[j], j
            else:
                dp[i, p], back[i, p] = _INT31_MAX, -1
        if dp[n - 1, p] <= target_overhead:
            chosen = p
            break
    return chosen, back


def partition_nodes_by_n_edges(node_n_edges, max_num_partitions: Optional[int] = None,
                               sparsity_tolerance: Optional[float] = None) -> np.ndarray:
    """Sorted group maxima (int64) for the given per-block fan-ins."""
    node_n_edges = np.asarray(node_n_edges, dtype=np.int64).reshape(-1)
    if sparsity_tolerance is not None and sparsity_tolerance < 1e-6:
        sparsity_tolerance = None
        max_num_partitions = 1
    if sparsity_tolerance is not None:
        assert 1e-6 < sparsity_tolerance <= 1.0
        if max_num_partitions is None:
            max_num_partitions = max(min(np.unique(node_n_edges).shape[0], 16), 1)
    elif max_num_partitions is None:
        max_num_partitions = 1
    else:
        assert max_num_partitions >= 1, "Should provide at least 1 partition."

    target = 0 if sparsity_tolerance is None else int(math.ceil(int(node_n_edges.sum()) * (1.0 + sparsity_tolerance)))
    if max_num_partitions == 1:
        return np.array([node_n_edges.max()], dtype=np.int64)

    vals = np.sort(node_n_edges)
    vals = vals[vals != 0]
    uvals, ucounts = _coalesce(vals)
    chosen, back = _weighted_dp(uvals, ucounts, max_num_partitions, target)

    picks = np.zeros(chosen, dtype=np.int64)
    i = uvals.shape[0] - 1
    for p in range(chosen, 0, -1):
        picks[p - 1] = i
        i = int(back[i, chosen])
    return np.unique(uvals[picks])


def partition_maxima(node_n_edges, max_num_partitions, sparsity_tolerance) -> np.ndarray:
    """Group maxima rounded up to powers of two and de-duplicated — the padded table widths
    (sum_layer.py:169-175, prod_layer.py:66-72)."""
    return np.unique(next_power_of_2(partition_nodes_by_n_edges(node_n_edges, max_num_partitions, sparsity_tolerance)))


def assign_partitions(counts: np.ndarray, maxima: np.ndarray, first_min: int):
    """Partition id and in-partition rank (order of appearance) of every block
    (sum_layer.py:186-195: ranges [first_min, m0], [m0+1, m1], ...)."""
    counts = np.asarray(counts, dtype=np.int64)
    part = np.zeros(counts.shape[0], dtype=np.int64)
    rank = np.zeros(counts.shape[0], dtype=np.int64)
    sizes = np.zeros(maxima.shape[0], dtype=np.int64)
    lo = first_min
    for p, hi in enumerate(maxima):
        sel = (counts >= lo) & (counts <= hi)
        k = int(sel.sum())
        part[sel] = p
        rank[sel] = np.arange(k)
        sizes[p] = k
        lo = int(hi) + 1
    return part, rank, sizes
