"""numpy restatement of the reference's pooling and normalisation (test infrastructure).

Follows infinity_emb/transformer/utils_optimum.py:29-35 (mean_pooling), :38-39
(cls_token_pooling), :42-47 (normalize) and the fp32 + ``F.normalize(p=2, dim=1)`` step of
infinity_emb/transformer/embedder/sentence_transformer.py:142-145. Last-token pooling has no
statement in the reference tree; it is the last position whose mask is 1 under right padding.
"""
from __future__ import annotations

import numpy as np


def mean_pooling(last_hidden_states: np.ndarray, attention_mask: np.ndarray) -> np.ndarray:
    mask = np.expand_dims(attention_mask, axis=-1).astype(float)
    summed = np.sum(last_hidden_states.astype(float) * mask, axis=1)
    count = np.maximum(np.sum(mask, axis=1), 1e-9)
    return summed / count


def cls_token_pooling(last_hidden_states: np.ndarray, attention_mask: np.ndarray | None = None) -> np.ndarray:
    return last_hidden_states[:, 0]


def last_token_pooling(last_hidden_states: np.ndarray, attention_mask: np.ndarray) -> np.ndarray:
    last = attention_mask.astype(np.int64).sum(axis=1) - 1
    return last_hidden_states[np.arange(last_hidden_states.shape[0]), last]


def normalize(x: np.ndarray, p: int = 2, dim: int = 1, eps: float = 1e-12) -> np.ndarray:
    norm = np.linalg.norm(x, ord=p, axis=dim, keepdims=True)
    return x / np.maximum(norm, eps)


POOLERS = {"mean": mean_pooling, "cls": cls_token_pooling, "last": last_token_pooling}


def pool_ragged(hidden: np.ndarray, cu_seqlens: np.ndarray, pooling: str, do_normalize: bool) -> np.ndarray:
    """The same pooling on the un-padded stream [n_tokens, H]: pads to [B, Lmax, H] with a
    mask exactly as the reference's backends see it, then applies the functions above."""
    lens = np.diff(cu_seqlens)
    B, Lmax = len(lens), int(lens.max())
    padded = np.zeros((B, Lmax, hidden.shape[1]), dtype=hidden.dtype)
    mask = np.zeros((B, Lmax), dtype=np.int64)
    for i in range(B):
        padded[i, : lens[i]] = hidden[cu_seqlens[i]: cu_seqlens[i + 1]]
        mask[i, : lens[i]] = 1
    out = POOLERS[pooling](padded, mask)
    return normalize(out) if do_normalize else out
