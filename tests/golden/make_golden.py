"""Generates the golden fixtures in this directory by running the REFERENCE's own code.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py <reference checkout>/libs/infinity_emb

It imports (never copies) the reference's pure-Python modules with two import-time shims
(no file of the reference is modified): ``importlib.metadata.version("infinity_emb")``
(the package is not installed) and ``huggingface_hub.HfFolder`` (removed from newer hub
releases, imported by ``infinity_emb/transformer/utils_optimum.py:8``).

Fixtures written:
  pooling_golden.npz  inputs + outputs of mean_pooling / cls_token_pooling / normalize
                      (infinity_emb/transformer/utils_optimum.py:29-47)
  batching_golden.json  batch orders produced by CustomFIFOQueue.pop_optimal_batches
                      (infinity_emb/inference/queue.py:35-76) for seeded priorities, and
                      get_lengths_with_tokenize (infinity_emb/transformer/utils.py:103-113)
"""
import importlib.metadata
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def import_reference(ref_root: str):
    os.environ.setdefault("DO_NOT_TRACK", "1")
    os.environ.setdefault("INFINITY_ANONYMOUS_USAGE_STATS", "0")
    scratch = tempfile.mkdtemp(prefix="infinity_home_")
    os.environ.setdefault("INFINITY_HOME", scratch)
    os.environ.setdefault("HF_HOME", scratch)
    real_version = importlib.metadata.version

    def version(name):
        if name == "infinity_emb":
            return "0.0.0+reference"
        return real_version(name)

    importlib.metadata.version = version
    import huggingface_hub
    if not hasattr(huggingface_hub, "HfFolder"):
        class HfFolder:  # stub: only referenced for token lookup
            @staticmethod
            def get_token():
                return None
        huggingface_hub.HfFolder = HfFolder
    sys.path.insert(0, ref_root)
    import infinity_emb  # noqa: F401
    return infinity_emb


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("INFINITY_EMB_SOURCE", "")
    if not ref_root:
        raise SystemExit("usage: make_golden.py <reference checkout>/libs/infinity_emb")
    import_reference(ref_root)
    from infinity_emb.transformer import utils_optimum as uo

    rng = np.random.default_rng(424242)
    cases = {}
    for name, (B, L, H) in {"a": (5, 17, 32), "b": (3, 64, 384), "c": (8, 9, 128), "d": (1, 1, 16)}.items():
        hidden = rng.standard_normal((B, L, H)).astype(np.float32)
        lens = rng.integers(1, L + 1, size=B)
        lens[0] = L
        mask = (np.arange(L)[None, :] < lens[:, None]).astype(np.int64)
        mean = uo.mean_pooling(hidden, mask)
        cls = uo.cls_token_pooling(hidden, mask)
        cases[f"{name}_hidden"] = hidden
        cases[f"{name}_mask"] = mask
        cases[f"{name}_mean"] = mean
        cases[f"{name}_cls"] = cls
        cases[f"{name}_mean_norm"] = uo.normalize(mean)
        cases[f"{name}_cls_norm"] = uo.normalize(cls)
    zero = np.zeros((2, 8), dtype=np.float32)
    cases["zero_in"] = zero
    cases["zero_norm"] = uo.normalize(zero)
    allmasked_hidden = rng.standard_normal((2, 4, 8)).astype(np.float32)
    cases["allmasked_hidden"] = allmasked_hidden
    cases["allmasked_mask"] = np.zeros((2, 4), dtype=np.int64)
    cases["allmasked_mean"] = uo.mean_pooling(allmasked_hidden, cases["allmasked_mask"])
    np.savez_compressed(HERE / "pooling_golden.npz", **cases)

    # batch formation
    import asyncio
    from infinity_emb.inference.queue import CustomFIFOQueue
    from infinity_emb.primitives import EmbeddingInner, EmbeddingSingle, PrioritizedQueueItem
    from infinity_emb.transformer.utils import get_lengths_with_tokenize

    class DoneNever:
        def done(self):
            return False

    out = {"cases": []}
    for n_items, size, n_batches, seed in [(32, 32, 8, 1), (64, 32, 8, 2), (300, 32, 8, 3), (100, 16, 4, 4),
                                           (7, 32, 8, 5), (33, 32, 8, 6), (257, 32, 8, 7)]:
        r = np.random.default_rng(seed)
        prios = r.integers(1, 400, size=n_items).tolist()
        q = CustomFIFOQueue()
        items = []
        for i, p in enumerate(prios):
            inner = EmbeddingInner(content=EmbeddingSingle(sentence=str(i)), future=DoneNever())
            items.append(PrioritizedQueueItem(priority=p, item=inner))
        q.extend(items)
        batches = []
        while len(q) > 0:
            for b in q.pop_optimal_batches(size, n_batches):
                batches.append([int(x.content.sentence) for x in b])
        out["cases"].append({"priorities": prios, "size": size, "max_n_batches": n_batches, "batches": batches})
    lengths, total = get_lengths_with_tokenize(["hi", "you", "a longer sentence"])
    out["char_lengths"] = {"input": ["hi", "you", "a longer sentence"], "lengths": list(map(int, lengths)),
                           "total": int(total)}
    (HERE / "batching_golden.json").write_text(json.dumps(out))
    print("wrote", HERE / "pooling_golden.npz", HERE / "batching_golden.json")


if __name__ == "__main__":
    main()
