"""The three threads the reference runs around one backend, without the reference.

``ModelWorker`` of the reference (infinity_emb/inference/batch_handler.py:470-624) drives one
replica from three threads joined by bounded queues: tokenise (``encode_pre``) -> queue of 3
-> inference (``encode_core``) -> queue of 5 -> post-processing (``encode_post``), which hands
``results[i]`` to item i (batch_handler.py:445-447). :class:`ThreeStageWorker` is that
structure with the same queue depths and the same calls from the same three roles, for
callers (and tests) that want the overlap of the stages without importing infinity_emb:
the backend sees exactly the call pattern the reference produces, including the delay
between ``encode_core`` writing a result and the caller reading its rows.
"""
from __future__ import annotations

import threading
from queue import Queue
from typing import Any, Callable, Iterable, List, Optional, Sequence

_STOP = object()


class ThreeStageWorker:
    """Feeds batches (lists of sentences or of pairs) through ``backend`` on three threads.

    ``deliver(batch_index, batch, results)`` is called on the post-processing thread with
    what ``encode_post`` returned; row i of ``results`` belongs to ``batch[i]``. An exception
    in a stage ends that stage and is re-raised by :meth:`run` (the reference logs it and
    raises ``ValueError``, batch_handler.py:556-558, 586-588, 622-624)."""

    FEATURE_QUEUE_DEPTH = 3      # batch_handler.py:499
    POSTPROCESS_QUEUE_DEPTH = 5  # batch_handler.py:500

    def __init__(self, backend: Any, deliver: Callable[[int, Sequence, Any], None]):
        self.backend = backend
        self.deliver = deliver
        self._features: Queue = Queue(self.FEATURE_QUEUE_DEPTH)
        self._post: Queue = Queue(self.POSTPROCESS_QUEUE_DEPTH)
        self._error: Optional[BaseException] = None
        self._failed = threading.Event()

    def _fail(self, exc: BaseException) -> None:
        if self._error is None:
            self._error = exc
        self._failed.set()

    def _put(self, q: Queue, item) -> bool:
        while not self._failed.is_set():
            try:
                q.put(item, timeout=0.1)
                return True
            except Exception:
                continue
        return False

    def _get(self, q: Queue):
        while not self._failed.is_set():
            try:
                return q.get(timeout=0.1)
            except Exception:
                continue
        return _STOP

    def _pre(self, batches: Iterable[Sequence]) -> None:
        try:
            for index, batch in enumerate(batches):
                feat = self.backend.encode_pre(list(batch))
                if not self._put(self._features, (index, batch, feat)):
                    return
        except BaseException as exc:  # noqa: BLE001 - handed to run()
            self._fail(exc)
        finally:
            self._put(self._features, _STOP)

    def _core(self) -> None:
        try:
            while True:
                item = self._get(self._features)
                if item is _STOP:
                    return
                index, batch, feat = item
                out = self.backend.encode_core(feat)
                if not self._put(self._post, (index, batch, out)):
                    return
        except BaseException as exc:  # noqa: BLE001
            self._fail(exc)
        finally:
            self._put(self._post, _STOP)

    def _postprocess(self) -> None:
        try:
            while True:
                item = self._get(self._post)
                if item is _STOP:
                    return
                index, batch, out = item
                results = self.backend.encode_post(out)
                if len(results) != len(batch):
                    raise ValueError(f"batch {index}: {len(results)} results for {len(batch)} items")
                self.deliver(index, batch, results)
        except BaseException as exc:  # noqa: BLE001
            self._fail(exc)

    def run(self, batches: Iterable[Sequence]) -> None:
        """Processes every batch, returns when the last one has been delivered."""
        threads: List[threading.Thread] = [
            threading.Thread(target=self._pre, args=(batches,), name="b200-pre"),
            threading.Thread(target=self._core, name="b200-core"),
            threading.Thread(target=self._postprocess, name="b200-post"),
        ]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if self._error is not None:
            raise ValueError(f"a worker stage failed: {self._error!r}") from self._error
