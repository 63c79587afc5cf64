"""Restatement of the reference's batch former (test infrastructure).

Follows ``CustomFIFOQueue.pop_optimal_batches`` (infinity_emb/inference/queue.py:35-76):
take the first ``size * max_n_batches`` queued items; sort them ascending by priority
(stable) only if MORE than ``size`` items were taken; cut into chunks of ``size``.
Checked against orders produced by the reference itself (tests/golden/batching_golden.json).
"""
from __future__ import annotations

from typing import List, Sequence


def pop_all_batches(priorities: Sequence[int], size: int, max_n_batches: int) -> List[List[int]]:
    """Item indices of every batch, draining the queue pop by pop."""
    queue = list(range(len(priorities)))
    batches: List[List[int]] = []
    while queue:
        taken, queue = queue[: size * max_n_batches], queue[size * max_n_batches:]
        if len(taken) > size:
            taken = sorted(taken, key=lambda i: priorities[i])  # list.sort is stable
        for s in range(0, len(taken), size):
            batches.append(taken[s: s + size])
    return batches
