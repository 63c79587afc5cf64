"""Token-balanced data parallelism over replicated weights.

Sequences are independent, so a batch splits by whole sequences with no exchange step:
every shard runs the full layer stack on its own GPU and the rows are put back in batch
order on the host. The reference instead hands whole batches to one replica per device
through a shared queue (infinity_emb/inference/batch_handler.py:111, 130-141;
infinity_emb/inference/select_model.py:80-83).

The assignment is the C library's partitioner (longest processing time first on the cost
``a*L + b*L^2``) with the coefficients the library itself derives from the model description
(``b200emb_cost_model``), so one process driving several GPUs through one handle and several
processes driving one GPU each (torchrun) cut a batch identically for every architecture.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np

import ctypes as C

from . import _lib
from .configs import ModelSpec
from .engine import make_desc, partition


def cost_coefficients(spec: ModelSpec) -> Tuple[float, float]:
    """The library's cost model for this architecture: (cost per token, cost per token pair)."""
    desc = make_desc(spec)
    a, b = C.c_double(), C.c_double()
    _lib.check(_lib.load().b200emb_cost_model(C.byref(desc), C.byref(a), C.byref(b)))
    return a.value, b.value


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
