"""numpy restatement of the output-embedding quantisation (test infrastructure only).

The reference applies it in ``quant_embedding_decorator`` around ``encode_post``
(infinity_emb/transformer/quantization/interface.py:124-154) by calling
``sentence_transformers.quantization.quantize_embeddings`` (sentence-transformers 3.3.1, a
dependency that is not vendored in the reference tree: libs/infinity_emb/poetry.lock:3806-3807).
Its published algorithm, restated:

* ``int8`` / ``uint8``: ``starts = ranges[0]``, ``steps = (ranges[1] - ranges[0]) / 255``;
  ``uint8 = ((x - starts) / steps).astype(uint8)``, ``int8 = ((x - starts) / steps - 128).astype(int8)``
  (float64 arithmetic because ``ranges`` is float64; ``astype`` truncates toward zero);
  ``ranges`` are the calibration ranges, ``np.percentile(calibration_embeddings, [0, 100], axis=0)`` in the
  reference (interface.py:97-121), or the batch's own min / max when none are given;
* ``ubinary``: ``np.packbits(x > 0)`` per row; ``binary``: the same bytes ``- 128`` as int8.

The matryoshka slice (infinity_emb/inference/batch_handler.py:65-74) is a plain ``[:dim]`` on whatever
rows come back and stays with the reference's caller.
"""
from __future__ import annotations

from typing import Optional

import numpy as np


def calibration_ranges(calibration_embeddings: np.ndarray, percentile: float = 100) -> np.ndarray:
    """interface.py:121: float64 [2, dim]."""
    return np.percentile(calibration_embeddings, [100 - percentile, percentile], axis=0)


def quantize_embeddings(embeddings: np.ndarray, precision: str, ranges: Optional[np.ndarray] = None) -> np.ndarray:
    x = np.asarray(embeddings)
    if precision == "float32":
        return x.astype(np.float32)
    if precision in ("int8", "uint8"):
        if ranges is None:
            ranges = np.vstack((np.min(x, axis=0), np.max(x, axis=0)))
        starts = ranges[0, :]
        steps = (ranges[1, :] - ranges[0, :]) / 255
        if precision == "uint8":
            return ((x - starts) / steps).astype(np.uint8)
        return ((x - starts) / steps - 128).astype(np.int8)
    if precision == "binary":
        return (np.packbits(x > 0).reshape(x.shape[0], -1).astype(np.int16) - 128).astype(np.int8)
    if precision == "ubinary":
        return np.packbits(x > 0).reshape(x.shape[0], -1)
    raise ValueError(f"unknown precision {precision}")
