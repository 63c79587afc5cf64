"""Host side of the boundary: text -> token ids, and ragged packing without padding.

The reference pads every batch to its longest sequence
(infinity_emb/transformer/crossencoder/torch.py:95-97, sentence-transformers' tokenize at
infinity_emb/transformer/embedder/sentence_transformer.py:113-115). Here a batch becomes one
token stream ``input_ids[n_tokens]`` with ``cu_seqlens[n_seqs + 1]``, in exactly the order
the batcher delivered the items (infinity_emb/inference/queue.py:35-76), so result row i
belongs to batch item i (infinity_emb/inference/batch_handler.py:445-447).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np


@dataclass
class PackedFeatures:
    """What ``encode_pre`` hands to ``encode_core``."""
    input_ids: np.ndarray                 # int32 [n_tokens]
    cu_seqlens: np.ndarray                # int32 [n_seqs + 1]
    token_type_ids: Optional[np.ndarray]  # int32 [n_tokens] or None

    @property
    def n_seqs(self) -> int:
        return len(self.cu_seqlens) - 1

    @property
    def n_tokens(self) -> int:
        return int(self.cu_seqlens[-1])


def pack_sequences(seqs: Sequence[Sequence[int]], types: Optional[Sequence[Sequence[int]]] = None) -> PackedFeatures:
    lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=len(seqs))
    if (lens <= 0).any():
        raise ValueError("every sequence needs at least one token")
    cu = np.zeros(len(seqs) + 1, dtype=np.int32)
    np.cumsum(lens, out=cu[1:])
    ids = np.concatenate([np.asarray(s, dtype=np.int32) for s in seqs]) if len(seqs) else np.zeros(0, np.int32)
    tt = None
    if types is not None:
        tt = np.concatenate([np.asarray(t, dtype=np.int32) for t in types]) if len(seqs) else np.zeros(0, np.int32)
    return PackedFeatures(ids, cu, tt)


def truncate_pair_longest_first(q: List[int], d: List[int], budget: int) -> Tuple[List[int], List[int]]:
    """Removes tokens one at a time from the longer side (ties: the second sequence, as HF
    tokenizers' ``longest_first`` does) until both fit ``budget`` tokens."""
    q, d = list(q), list(d)
    over = len(q) + len(d) - budget
    while over > 0:
        if len(q) > len(d):
            q.pop()
        else:
            d.pop()
        over -= 1
    return q, d


class IdStringTokenizer:
    """Sentences are strings of space-separated decimal token ids ("101 5230 17").

    Stands in for a vocabulary-based tokenizer when none is available offline: the string
    travels through the engine and batcher untouched, ``encode`` parses it, and
    ``lengths`` counts the ids so that length-based batching sees true token counts.
    Pairs are joined as ``[start] q [sep] [sep] d [end]`` (the XLM-RoBERTa convention)."""

    def __init__(self, max_len: int, start_id: int = 0, sep_id: int = 2, end_id: int = 2, add_special: bool = False):
        self.max_len, self.start_id, self.sep_id, self.end_id, self.add_special = max_len, start_id, sep_id, end_id, add_special

    @staticmethod
    def _parse(s: str) -> List[int]:
        return [int(x) for x in s.split()]

    def encode(self, sentences: Sequence[str]) -> PackedFeatures:
        seqs = []
        for s in sentences:
            ids = self._parse(s)
            if self.add_special:
                ids = [self.start_id] + ids[: self.max_len - 2] + [self.end_id]
            seqs.append(ids[: self.max_len] or [self.start_id])
        return pack_sequences(seqs)

    def encode_pairs(self, pairs: Sequence[Tuple[str, str]]) -> PackedFeatures:
        seqs = []
        for q, d in pairs:
            qi, di = truncate_pair_longest_first(self._parse(q.strip()), self._parse(d.strip()), self.max_len - 4)
            seqs.append([self.start_id] + qi + [self.sep_id, self.sep_id] + di + [self.end_id])
        return pack_sequences(seqs)

    def lengths(self, sentences: Sequence[str]) -> List[int]:
        return [len(s.split()) for s in sentences]


class HFTokenizer:
    """A ``tokenizers`` (HF, Rust) tokenizer loaded from a ``tokenizer.json``; its encodings go
    straight into the ragged layout, no padding is ever materialised."""

    def __init__(self, tokenizer_or_path, max_len: int):
        import copy

        import tokenizers
        tok = tokenizer_or_path
        if isinstance(tok, (str, bytes)) or hasattr(tok, "__fspath__"):
            tok = tokenizers.Tokenizer.from_file(str(tok))
        self._tok = tok
        self._tok.no_padding()
        self._tok.enable_truncation(max_length=max_len, strategy="longest_first")
        # a second instance for counting lengths from another thread while encode runs
        # (the reference deep-copies its tokenizer for the same reason, sentence_transformer.py:80-92)
        self._len_tok = copy.deepcopy(tok)
        self.max_len = max_len

    def encode(self, sentences: Sequence[str]) -> PackedFeatures:
        enc = self._tok.encode_batch(list(sentences), add_special_tokens=True)
        return pack_sequences([e.ids for e in enc], [e.type_ids for e in enc])

    def encode_pairs(self, pairs: Sequence[Tuple[str, str]]) -> PackedFeatures:
        enc = self._tok.encode_batch([(q.strip(), d.strip()) for q, d in pairs], add_special_tokens=True)
        return pack_sequences([e.ids for e in enc], [e.type_ids for e in enc])

    def lengths(self, sentences: Sequence[str]) -> List[int]:
        enc = self._len_tok.encode_batch(list(sentences), add_special_tokens=False)
        return [len(e.ids) for e in enc]
