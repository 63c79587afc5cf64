"""Token-balanced data parallelism over replicated weights.

Sequences are independent, so a batch splits by whole sequences with no exchange step:
every shard runs the full layer stack on its own GPU and the rows are put back in batch
order on the host. The reference instead hands whole batches to one replica per device
through a shared queue (infinity_emb/inference/batch_handler.py:111, 130-141;
infinity_emb/inference/select_model.py:80-83).

The assignment is the C library's partitioner (longest processing time first on the cost
``a*L + b*L^2``), so one process driving several GPUs and several processes driving one
GPU each (torchrun) cut a batch identically.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np

from .configs import ModelSpec
from .engine import partition


def cost_coefficients(spec: ModelSpec) -> Tuple[float, float]:
    """Per-layer flops per token (GEMMs) and per token pair (attention)."""
    H, F = spec.hidden, spec.ffn
    qkv = (spec.n_heads + 2 * spec.n_kv_heads) * spec.head_dim
    return 2.0 * H * qkv + 2.0 * H * H + 4.0 * H * F, 4.0 * H


def shard_indices(lengths: Sequence[int], n_shards: int, spec: ModelSpec) -> List[np.ndarray]:
    """Indices (ascending, i.e. batch order kept inside a shard) of the sequences of each shard."""
    if n_shards == 1:
        return [np.arange(len(lengths))]
    a, b = cost_coefficients(spec)
    owner = partition(lengths, n_shards, a, b)
    return [np.nonzero(owner == s)[0] for s in range(n_shards)]


def scatter_rows(out: np.ndarray, shard_rows: np.ndarray, indices: np.ndarray) -> None:
    """Puts a shard's result rows back at their batch positions."""
    out[indices] = shard_rows
