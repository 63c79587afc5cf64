"""Drop-in backends for the infinity_emb engine: the five-method interface of
``BaseTransformer`` (infinity_emb/transformer/abstract.py:44-69) over the CUDA library.

  B200Embedder      capabilities {"embed"}     replaces SentenceTransformerPatched
                    (infinity_emb/transformer/embedder/sentence_transformer.py:54-169)
  B200CrossEncoder  capabilities {"rerank"}    replaces CrossEncoderPatched
                    (infinity_emb/transformer/crossencoder/torch.py:41-123)
  B200Classifier    capabilities {"classify"}  replaces SentenceClassifier
                    (infinity_emb/transformer/classifier/torch.py:21-91)

The classes are duck-typed (this package does not import infinity_emb), so an instance can
be handed to the reference's ``BatchHandler(model_replicas=[backend], ...)`` as it is.
Same method names, argument meaning and return conventions as the reference:
``encode_pre`` is called from the batcher's tokenisation thread, ``encode_core`` from its
inference thread (never re-entered for one object), ``encode_post`` from its
post-processing thread, ``tokenize_lengths`` from a thread pool. An exception in any of
them propagates, as in the reference (batch_handler.py:556-558, 586-588, 622-624).
"""
from __future__ import annotations

import dataclasses
import threading
from time import perf_counter
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .configs import ModelSpec
from .engine import B200Model
from .packing import HFTokenizer, IdStringTokenizer, PackedFeatures


class _B200Backend:
    capabilities: set = set()

    def __init__(self, *, engine_args: Any = None, spec: ModelSpec, weight_path: Optional[str] = None,
                 device_ids: Sequence[int] = (0,), tokenizer: Any = None, model: Any = None,
                 ring_size: int = 10):
        """``model``: an object with ``forward_arrays(ids, cu, types, out=)`` (tests inject a
        stand-in); by default a :class:`B200Model` on ``device_ids`` is created, which fails
        loudly when the CUDA library or a GPU is missing."""
        self.engine_args = engine_args
        self.spec = spec
        if tokenizer is None:
            limit = spec.max_len if spec.arch == "decoder" else min(spec.max_len, spec.max_pos - spec.pos_offset)
            tokenizer = IdStringTokenizer(limit)
        self.tokenizer = tokenizer
        self.model = model if model is not None else B200Model(spec, weight_path, device_ids)
        # The device-to-host copy of a result lands in page-locked memory, which is slow to
        # allocate, so encode_core writes into a ring of ring_size reusable pinned arrays.
        # A slot must outlive its trip through the bounded queue between the inference and
        # the post-processing thread (depth 5, batch_handler.py:500); encode_post copies the
        # rows out of the ring, so what the caller receives is never overwritten.
        self._ring: List[Optional[np.ndarray]] = [None] * ring_size
        self._ring_pos = 0
        self._lock = threading.Lock()

    # -- shared pieces ----------------------------------------------------------------
    def _result_buffer(self, n_seqs: int) -> np.ndarray:
        with self._lock:
            slot = self._ring_pos
            self._ring_pos = (self._ring_pos + 1) % len(self._ring)
        buf = self._ring[slot]
        if buf is None or buf.shape[0] < n_seqs:
            buf = _pinned_empty(max(n_seqs, 64), self.spec.out_dim)
            self._ring[slot] = buf
        return buf[:n_seqs]

    def encode_core(self, features: PackedFeatures):
        """runs the forward on the GPU(s); returns ``[n_seqs, out_dim]`` float32. In ColBERT mode
        (``spec.pooling == "tokens"``) returns the token rows together with the sequence offsets,
        as the reference hands token_embeddings + attention_mask on (sentence_transformer.py:125-131)."""
        dtype = getattr(self, "embedding_dtype", "float32")
        if dtype != "float32":
            if self.spec.pooling == "tokens":
                raise ValueError("output quantisation is for sentence embeddings")
            if dtype in ("int8", "uint8") and self.calibration_ranges is None:
                raise ValueError("int8 / uint8 embeddings need calibration ranges: call calibrate() first")
            return self.model.forward_quantized(features.input_ids, features.cu_seqlens, dtype,
                                                features.token_type_ids, self.calibration_ranges)
        if self.spec.pooling == "tokens":
            out = self._result_buffer(features.n_tokens)
            self.model.forward_arrays(features.input_ids, features.cu_seqlens, features.token_type_ids, out=out)
            return {"token_embeddings": out, "cu_seqlens": np.array(features.cu_seqlens, dtype=np.int64)}
        out = self._result_buffer(features.n_seqs)
        self.model.forward_arrays(features.input_ids, features.cu_seqlens, features.token_type_ids, out=out)
        return out

    def tokenize_lengths(self, sentences: List[str]) -> List[int]:
        return self.tokenizer.lengths(sentences)

    def _warmup_inputs(self, batch_size: int, n_tokens: int) -> list:
        raise NotImplementedError

    def warmup(self, *, batch_size: int = 64, n_tokens: int = 1) -> Tuple[float, float, str]:
        """Same contract as ``run_warmup`` (abstract.py:228-250): returns embeddings per
        second, inference seconds and a log string."""
        inputs = self._warmup_inputs(batch_size, n_tokens)
        start = perf_counter()
        feat = self.encode_pre(inputs)
        t_tok = perf_counter()
        out = self.encode_core(feat)
        t_inf = perf_counter()
        self.encode_post(out)
        t_post = perf_counter()
        log = (f"Getting timings for batch_size={batch_size} and avg tokens per sentence={feat.n_tokens / max(batch_size, 1):.1f}\n"
               f"\t{(t_tok - start) * 1000:.2f} \t ms tokenization\n"
               f"\t{(t_inf - t_tok) * 1000:.2f} \t ms inference\n"
               f"\t{(t_post - t_inf) * 1000:.2f} \t ms post-processing\n"
               f"\t{(t_post - start) * 1000:.2f} \t ms total\n"
               f"embeddings/sec: {batch_size / (t_post - start):.2f}")
        return batch_size / (t_post - start), t_inf - t_tok, log


def _pinned_empty(rows: int, cols: int) -> np.ndarray:
    """float32 host array in page-locked memory when torch + CUDA are present (the D2H copy
    of the result is then asynchronous on the library's stream); plain numpy otherwise."""
    try:
        import torch
        if torch.cuda.is_available():
            t = torch.empty(rows, cols, dtype=torch.float32).pin_memory()
            return t.numpy()  # the array keeps the pinned tensor alive
    except Exception:
        pass
    return np.empty((rows, cols), dtype=np.float32)


class B200Embedder(_B200Backend):
    capabilities = {"embed"}

    def __init__(self, *, embedding_dtype: str = "float32", calibration_ranges: Optional[np.ndarray] = None, **kw):
        """``embedding_dtype``: float32 | int8 | uint8 | binary | ubinary (EmbeddingDtype,
        primitives.py:145-158). The reference quantises in a decorator around ``encode_post``
        (quantization/interface.py:124-154) with ranges from a downloaded calibration text
        (interface.py:73-121); here the rows are quantised on the device inside ``encode_core``,
        and the ranges for int8 / uint8 come from ``calibration_ranges`` (float64 ``[2, dim]``) or
        from :meth:`calibrate` on sentences the caller supplies."""
        super().__init__(**kw)
        self.embedding_dtype = getattr(embedding_dtype, "value", embedding_dtype)
        self.calibration_ranges = calibration_ranges

    def calibrate(self, sentences: List[str], batch_size: int = 8, percentile: float = 100) -> np.ndarray:
        """Ranges as the reference computes them (interface.py:97-121): float32 embeddings of the
        calibration sentences in batches of 8, then the [100 - p, p] percentiles per dimension."""
        rows = []
        for i in range(0, len(sentences), batch_size):
            f = self.tokenizer.encode(sentences[i: i + batch_size])
            rows.append(np.array(self.model.forward_arrays(f.input_ids, f.cu_seqlens, f.token_type_ids)))
        self.calibration_ranges = np.percentile(np.concatenate(rows), [100 - percentile, percentile], axis=0)
        return self.calibration_ranges

    def _warmup_inputs(self, batch_size, n_tokens):
        if isinstance(self.tokenizer, IdStringTokenizer):
            return [" ".join(["1"] * max(n_tokens, 1))] * batch_size
        return ["warm " * n_tokens] * batch_size

    def encode_pre(self, sentences: List[str]) -> PackedFeatures:
        """tokenises and packs the batch (no padding)"""
        return self.tokenizer.encode(sentences)

    def encode_post(self, embedding, skip_quanitzation: bool = True):
        """float32 rows, already pooled and L2-normalised on the device (the reference does
        this step on the CPU: sentence_transformer.py:142-145). ColBERT mode: one ``[L_i, D]``
        array per sequence (sentence_transformer.py:146-155; there are no padded rows to drop).
        The result is a fresh array the caller owns, as the reference's ``.numpy()`` of a new
        tensor is (sentence_transformer.py:156-157): the batcher hands row views of it to the
        request futures (batch_handler.py:445-447), which may keep them for any time, while
        ``encode_core`` reuses its pinned buffer a few batches later."""
        if isinstance(embedding, dict):
            rows, cu = embedding["token_embeddings"], embedding["cu_seqlens"]
            return [np.array(rows[cu[i]: cu[i + 1]], dtype=np.float32) for i in range(len(cu) - 1)]
        return np.array(embedding)


class B200CrossEncoder(_B200Backend):
    capabilities = {"rerank"}

    def _warmup_inputs(self, batch_size, n_tokens):
        s = " ".join(["1"] * max(n_tokens, 1)) if isinstance(self.tokenizer, IdStringTokenizer) else "warm " * n_tokens
        return [(s, s)] * batch_size

    def encode_pre(self, queries_docs: List[Tuple[str, str]]) -> PackedFeatures:
        """strips, pair-tokenises with longest-first truncation (crossencoder/torch.py:91-98) and packs"""
        return self.tokenizer.encode_pairs(queries_docs)

    def encode_post(self, out_features: np.ndarray) -> np.ndarray:
        """flat float32 raw logits (crossencoder/torch.py:110-111) in a fresh array the caller
        owns (not a view of the recycled pinned buffer); the batcher applies the sigmoid"""
        return np.array(out_features, dtype=np.float32).reshape(-1)


class B200Classifier(_B200Backend):
    capabilities = {"classify"}

    def __init__(self, *, labels: Optional[Sequence[str]] = None, device_scores: bool = False, **kw):
        """``device_scores``: the softmax / sigmoid over the labels runs on the GPU behind the head
        (``ModelSpec.label_scores``) and ``encode_post`` only sorts and names the rows."""
        if device_scores:
            kw["spec"] = dataclasses.replace(kw["spec"], label_scores=True)
        super().__init__(**kw)
        n = self.spec.n_labels
        self.labels = list(labels) if labels is not None else [f"LABEL_{i}" for i in range(n)]
        if len(self.labels) != n:
            raise ValueError(f"{len(self.labels)} labels for a head with {n} outputs")

    def _warmup_inputs(self, batch_size, n_tokens):
        if isinstance(self.tokenizer, IdStringTokenizer):
            return [" ".join(["1"] * max(n_tokens, 1))] * batch_size
        return ["warm " * n_tokens] * batch_size

    def encode_pre(self, sentences: List[str]) -> PackedFeatures:
        return self.tokenizer.encode(sentences)

    def encode_post(self, logits: np.ndarray) -> List[List[Dict[str, Any]]]:
        """What the HF text-classification pipeline returns with ``top_k=None``
        (classifier/torch.py:38-46, 74-80): per input, one dict per label sorted by score
        descending; softmax over the labels, or a sigmoid for a single-label head."""
        x = np.asarray(logits, dtype=np.float64)
        if self.spec.label_scores:
            scores = x
        elif x.shape[1] == 1:
            scores = 1.0 / (1.0 + np.exp(-x))
        else:
            z = x - x.max(axis=1, keepdims=True)
            e = np.exp(z)
            scores = e / e.sum(axis=1, keepdims=True)
        out = []
        for row in scores:
            order = np.argsort(-row, kind="stable")
            out.append([{"label": self.labels[j], "score": float(row[j])} for j in order])
        return out
