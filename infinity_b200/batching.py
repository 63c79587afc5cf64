"""Batch cuts for the caller of ``encode_core``: by token budget instead of by sequence count.

The reference's queue pops up to ``size * max_n_batches`` waiting items, sorts them by length and cuts
the sorted list every ``size`` items (infinity_emb/inference/queue.py:57-76); a batch of ``size`` long
texts then costs many times a batch of ``size`` short ones, and device memory has to be provisioned for
``size * max_len`` tokens. With the ragged layout the cost of a forward is a function of the tokens in
it, so the cut can be made where a token budget is reached: batches take about the same device time
and the workspace bound is the budget itself.

Both cuts are here: :func:`count_batches` restates the reference's, :func:`token_budget_batches` is the
replacement. They return lists of indices into the caller's item list, so the caller keeps its own
item objects, futures and ordering.
"""
from __future__ import annotations

from typing import List, Optional, Sequence


def _sorted_indices(lengths: Sequence[int]) -> List[int]:
    # ascending by length, ties in arrival order (the reference sorts PrioritizedQueueItem objects,
    # whose order is the length alone; Python's sort is stable)
    return sorted(range(len(lengths)), key=lambda i: lengths[i])


def count_batches(lengths: Sequence[int], size: int, sort: Optional[bool] = None) -> List[List[int]]:
    """The reference's cut (queue.py:57-76): sorted by length when more than one batch is waiting,
    then every ``size`` items."""
    if size <= 0:
        raise ValueError("size must be positive")
    n = len(lengths)
    if sort is None:
        sort = n > size
    order = _sorted_indices(lengths) if sort else list(range(n))
    return [order[i: i + size] for i in range(0, n, size)]


def token_budget_batches(lengths: Sequence[int], max_tokens: int, max_seqs: Optional[int] = None,
                         quadratic_weight: float = 0.0) -> List[List[int]]:
    """Cuts the length-sorted items where the running cost would pass ``max_tokens``.

    The cost of a sequence of ``L`` tokens is ``L + quadratic_weight * L * L`` (the second term stands
    for attention; 0 counts tokens only). A batch holds at most ``max_seqs`` sequences when given. A
    single sequence whose cost exceeds the budget forms a batch of its own, so every index appears in
    exactly one batch whatever the lengths are.
    """
    if max_tokens <= 0:
        raise ValueError("max_tokens must be positive")
    if max_seqs is not None and max_seqs <= 0:
        raise ValueError("max_seqs must be positive")
    batches: List[List[int]] = []
    current: List[int] = []
    cost = 0.0
    for i in _sorted_indices(lengths):
        length = int(lengths[i])
        if length < 0:
            raise ValueError(f"item {i} has negative length {length}")
        c = length + quadratic_weight * length * length
        full = current and (cost + c > max_tokens or (max_seqs is not None and len(current) >= max_seqs))
        if full:
            batches.append(current)
            current, cost = [], 0.0
        current.append(i)
        cost += c
    if current:
        batches.append(current)
    return batches


class TokenBudgetQueue:
    """Drop-in for the reference's ``CustomFIFOQueue`` (infinity_emb/inference/queue.py:15-76: ``extend``,
    ``pop_optimal_batches``, ``__len__``) that cuts batches by token budget.

    A pop takes the first ``size * max_n_batches`` waiting items exactly as the reference does, sorts them
    by priority when more than ``size`` were taken, drops items whose future is already done, and then cuts
    the list where the running cost ``sum(L + quadratic_weight * L^2)`` would pass ``max_tokens`` (and at
    ``size`` items at the latest). The priority of an item is its length: token count with
    ``lengths_via_tokenize=True``, else characters (batch_handler.py:356-374), so give ``max_tokens`` in the
    same unit. With ``max_tokens=None`` every pop yields the reference's batches, item for item.

    Items are duck-typed like ``PrioritizedQueueItem`` (primitives.py): ``.priority`` and ``.item`` with
    ``.item.future.done()``; this module does not import infinity_emb. To use it, assign an instance to
    ``BatchHandler._queue_prio`` before ``spawn()`` (batch_handler.py:110 creates the queue, :327 fills it,
    :401 pops it).
    """

    def __init__(self, max_tokens: Optional[int] = None, quadratic_weight: float = 0.0) -> None:
        import threading
        if max_tokens is not None and max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        self.max_tokens = max_tokens
        self.quadratic_weight = float(quadratic_weight)
        self._lock = threading.Lock()
        self._queue: list = []
        self._sync_event = threading.Event()

    def __len__(self) -> int:
        return len(self._queue)

    def extend(self, items: list) -> None:
        with self._lock:
            self._queue.extend(items)
        self._sync_event.set()

    def pop_optimal_batches(self, size: int, max_n_batches: int = 4, timeout: float = 0.2, **kwargs):
        """Generator of batches (lists of ``.item`` objects), none longer than ``size`` or, unless it is a
        single item, dearer than ``max_tokens``. Yields nothing when the queue stays empty for ``timeout``."""
        if not self._queue:
            if not self._sync_event.wait(timeout):
                return
        take = size * max_n_batches
        with self._lock:
            taken, self._queue = self._queue[:take], self._queue[take:]
            if not self._queue:
                self._sync_event.clear()
        if len(taken) > size:
            taken.sort(key=lambda entry: entry.priority)  # stable, as the reference's sort on the items is
        live = [entry for entry in taken if not entry.item.future.done()]
        if self.max_tokens is None:
            for i in range(0, len(live), size):
                yield [entry.item for entry in live[i: i + size]]
            return
        current: list = []
        cost = 0.0
        for entry in live:
            length = int(entry.priority)
            c = length + self.quadratic_weight * length * length
            if current and (cost + c > self.max_tokens or len(current) >= size):
                yield current
                current, cost = [], 0.0
            current.append(entry.item)
            cost += c
        if current:
            yield current
