"""Host-side logic that needs no GPU: weight file round trip, packing, pair truncation,
classifier post-processing, and the backends driven by the reference's own BatchHandler
(when the reference tree is present) with a stand-in for the device model."""
import asyncio
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from infinity_b200 import batching as bt
from infinity_b200 import configs as cf
from infinity_b200 import packing as pk
from infinity_b200 import weights as wt
from infinity_b200.backend import B200Classifier, B200CrossEncoder, B200Embedder

# the reference's Python sources, when a checkout is mounted next to this repository (the tests that drive its
# batcher are skipped otherwise)
REF = Path(os.environ.get("INFINITY_EMB_SOURCE", str(Path(__file__).resolve().parents[2] / "reference" / "libs" / "infinity_emb")))


def test_weight_file_round_trip(tmp_path):
    spec = cf.tiny_spec("xlmr")
    tensors = cf.runtime_tensors(cf.init_weights(spec, 3, perturb=True))
    path = tmp_path / "w.b2ew"
    wt.save_weights(path, tensors)
    back = wt.load_weights(path)
    assert list(back) == list(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and back[k].shape == tensors[k].shape
        assert torch.equal(back[k].view(torch.int16) if back[k].dtype == torch.bfloat16 else back[k],
                           tensors[k].view(torch.int16) if tensors[k].dtype == torch.bfloat16 else tensors[k])


def test_packing_is_bit_exact_against_the_padded_layout():
    """cu_seqlens / token stream == what mask.nonzero() selects from the reference's padded batch."""
    from oracle import encoder as enc
    rng = np.random.default_rng(1)
    seqs = [rng.integers(0, 1000, size=L) for L in [5, 1, 64, 33, 512, 2]]
    packed = pk.pack_sequences(seqs)
    ids, mask, _ = enc.pad_batch(seqs)
    assert np.array_equal(packed.input_ids, ids[mask.bool()].numpy().astype(np.int32))
    assert np.array_equal(packed.cu_seqlens, np.concatenate([[0], np.cumsum(mask.sum(1).numpy())]))
    assert packed.n_seqs == 6 and packed.n_tokens == sum(len(s) for s in seqs)
    with pytest.raises(ValueError):
        pk.pack_sequences([[1, 2], []])
    empty = pk.pack_sequences([])
    assert empty.n_seqs == 0 and empty.n_tokens == 0


def test_pair_truncation_longest_first():
    q, d = pk.truncate_pair_longest_first(list(range(10)), list(range(100, 130)), 20)
    assert len(q) + len(d) == 20 and q == list(range(10)) and d == list(range(100, 110))
    q, d = pk.truncate_pair_longest_first(list(range(30)), list(range(5)), 20)
    assert len(q) == 15 and len(d) == 5
    q, d = pk.truncate_pair_longest_first([1, 2], [3], 20)
    assert (q, d) == ([1, 2], [3])
    tok = pk.IdStringTokenizer(max_len=16)
    f = tok.encode_pairs([(" 5 6 7 ", "8 9"), ("1 " * 20, "2 " * 20)])
    assert f.input_ids[: f.cu_seqlens[1]].tolist() == [0, 5, 6, 7, 2, 2, 8, 9, 2]
    assert f.cu_seqlens[2] - f.cu_seqlens[1] == 16
    assert tok.lengths(["1 2 3", "4"]) == [3, 1]


def test_hf_tokenizer_packs_without_padding():
    import tokenizers
    from tokenizers import models, pre_tokenizers, processors
    vocab = {"[PAD]": 0, "[UNK]": 1, "[CLS]": 2, "[SEP]": 3, "hello": 4, "world": 5, "warm": 6, "a": 7}
    tok = tokenizers.Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.post_processor = processors.TemplateProcessing(
        single="[CLS] $A [SEP]", pair="[CLS] $A [SEP] $B:1 [SEP]:1", special_tokens=[("[CLS]", 2), ("[SEP]", 3)])
    t = pk.HFTokenizer(tok, max_len=8)
    f = t.encode(["hello world", "a", "warm " * 20])
    assert f.input_ids[:4].tolist() == [2, 4, 5, 3]
    assert np.diff(f.cu_seqlens).tolist() == [4, 3, 8]
    p = t.encode_pairs([("hello", "world a")])
    assert p.input_ids.tolist() == [2, 4, 3, 5, 7, 3] and p.token_type_ids.tolist() == [0, 0, 0, 1, 1, 1]
    assert t.lengths(["hello world", "a"]) == [2, 1]


class FakeDeviceModel:
    """Stands in for B200Model: row i = [n_tokens_i, sum(ids_i), first id, ...]."""

    def __init__(self, out_dim):
        self.out_dim = out_dim
        self.calls = []

    def forward_arrays(self, ids, cu, types=None, out=None, **kw):
        n = len(cu) - 1
        self.calls.append(n)
        for i in range(n):
            seg = ids[cu[i]: cu[i + 1]]
            out[i, :] = 0.0
            out[i, 0] = len(seg)
            if self.out_dim > 1:
                out[i, 1] = float(seg.sum())
        return out


def test_result_rows_are_caller_owned():
    """encode_core reuses a ring of pinned buffers; what encode_post returns must not alias it
    (the reference returns a fresh array per batch, sentence_transformer.py:135-157, and the
    batcher gives row views of it to the request futures, batch_handler.py:445-447)."""
    spec = cf.tiny_spec("bert")
    emb = B200Embedder(spec=spec, model=FakeDeviceModel(spec.hidden), ring_size=4)
    ce = B200CrossEncoder(spec=cf.tiny_spec("xlmr"), model=FakeDeviceModel(1), ring_size=4)
    kept, kept_ce = [], []
    for r in range(13):
        sentences = [" ".join(["7"] * (r + 1 + j)) for j in range(3)]
        kept.append(emb.encode_post(emb.encode_core(emb.encode_pre(sentences))))
        kept_ce.append(ce.encode_post(ce.encode_core(ce.encode_pre([(s, "1") for s in sentences]))))
    for r in range(13):
        assert kept[r][:, 0].tolist() == [r + 1, r + 2, r + 3]
        assert kept_ce[r].tolist() == [r + 1 + j + 1 + 4 for j in range(3)]
    assert len({k.ctypes.data for k in kept}) == 13


def test_three_stage_worker_keeps_row_order_and_rows():
    """The repository's own pre / core / post threads (queue depths 3 and 5 as in
    batch_handler.py:499-500): every row reaches its item, also when the post-processing side
    holds on to all results until the end."""
    from infinity_b200.worker import ThreeStageWorker
    spec = cf.tiny_spec("bert")
    backend = B200Embedder(spec=spec, model=FakeDeviceModel(spec.hidden), ring_size=10)
    rng = np.random.default_rng(5)
    batches = [[" ".join(map(str, rng.integers(1, 900, size=int(L)))) for L in rng.integers(1, 60, size=int(n))]
               for n in rng.integers(1, 9, size=40)]
    got = {}

    def deliver(index, batch, results):
        for i, s in enumerate(batch):
            got[(index, i)] = results[i]          # row views, kept

    ThreeStageWorker(backend, deliver).run(batches)
    assert len(got) == sum(len(b) for b in batches)
    for (index, i), row in got.items():
        toks = [int(x) for x in batches[index][i].split()]
        assert row[0] == len(toks) and row[1] == float(sum(toks))

    class Boom(FakeDeviceModel):
        def forward_arrays(self, *a, **k):
            raise RuntimeError("device error")

    with pytest.raises(ValueError):
        ThreeStageWorker(B200Embedder(spec=spec, model=Boom(spec.hidden)), deliver).run(batches)


def test_classifier_post_processing():
    spec = cf.tiny_spec("xlmr", n_labels=3)
    clf = B200Classifier(spec=spec, model=FakeDeviceModel(3), labels=["neg", "neu", "pos"])
    out = clf.encode_post(np.array([[0.0, 2.0, 1.0], [5.0, -1.0, 0.0]], dtype=np.float32))
    assert [d["label"] for d in out[0]] == ["neu", "pos", "neg"]
    assert abs(sum(d["score"] for d in out[0]) - 1.0) < 1e-6
    assert out[1][0]["label"] == "neg" and out[1][0]["score"] > 0.99
    single = B200Classifier(spec=cf.tiny_spec("xlmr", n_labels=1), model=FakeDeviceModel(1))
    assert abs(single.encode_post(np.array([[0.0]], dtype=np.float32))[0][0]["score"] - 0.5) < 1e-7
    with pytest.raises(ValueError):
        B200Classifier(spec=spec, model=FakeDeviceModel(3), labels=["a"])


def test_classifier_with_device_scores_only_sorts():
    spec = cf.tiny_spec("xlmr", n_labels=3)
    clf = B200Classifier(spec=spec, model=FakeDeviceModel(3), labels=["neg", "neu", "pos"], device_scores=True)
    assert clf.spec.label_scores and not spec.label_scores
    out = clf.encode_post(np.array([[0.2, 0.7, 0.1]], dtype=np.float32))
    assert [(d["label"], round(d["score"], 6)) for d in out[0]] == [("neu", 0.7), ("neg", 0.2), ("pos", 0.1)]


def test_count_batches_restates_the_reference_cut():
    lengths = [9, 3, 7, 1, 5, 8, 2]
    # more items than one batch: sorted by length, then cut every `size`
    assert bt.count_batches(lengths, 3) == [[3, 6, 1], [4, 2, 5], [0]]
    # a single batch keeps arrival order
    assert bt.count_batches(lengths, 8) == [list(range(7))]
    assert bt.count_batches([], 4) == []


def test_token_budget_batches():
    rng = np.random.default_rng(0)
    lengths = rng.integers(1, 513, size=1000).tolist()
    batches = bt.token_budget_batches(lengths, 8192, max_seqs=64)
    assert sorted(i for b in batches for i in b) == list(range(1000))
    for b in batches:
        assert len(b) <= 64 and sum(lengths[i] for i in b) <= 8192
    flat = [lengths[i] for b in batches for i in b]
    assert flat == sorted(lengths)
    # no batch could have taken the first item of the next one
    for b, nxt in zip(batches, batches[1:]):
        assert len(b) == 64 or sum(lengths[i] for i in b) + lengths[nxt[0]] > 8192
    # a huge budget leaves the count limit alone: the reference's cut
    assert bt.token_budget_batches(lengths, 10 ** 9, max_seqs=32) == bt.count_batches(lengths, 32, sort=True)
    # an item above the budget is a batch of its own
    assert bt.token_budget_batches([5, 100, 6], 20) == [[0, 2], [1]]
    # the quadratic term makes long sequences dearer
    assert len(bt.token_budget_batches([100] * 8, 400)) == 2
    assert len(bt.token_budget_batches([100] * 8, 400, quadratic_weight=0.01)) == 4
    with pytest.raises(ValueError):
        bt.token_budget_batches([1], 0)


class _Future:
    def __init__(self, done=False):
        self._done = done

    def done(self):
        return self._done


class _Inner:
    def __init__(self, index, done=False):
        self.index, self.future = index, _Future(done)


class _Prio:
    def __init__(self, priority, index, done=False):
        self.priority, self.item = priority, _Inner(index, done)


def test_token_budget_queue_matches_the_reference_orders_without_a_budget():
    """TokenBudgetQueue with no budget pops exactly the batches the reference's CustomFIFOQueue popped
    (orders generated by the reference itself: tests/golden/batching_golden.json)."""
    import json
    golden = json.loads((Path(__file__).parent / "golden" / "batching_golden.json").read_text())
    for case in golden["cases"]:
        q = bt.TokenBudgetQueue()
        q.extend([_Prio(p, i) for i, p in enumerate(case["priorities"])])
        assert len(q) == len(case["priorities"])
        got = []
        while len(q):
            got.extend([[it.index for it in b] for b in q.pop_optimal_batches(case["size"], case["max_n_batches"])])
        assert got == case["batches"]
    assert list(bt.TokenBudgetQueue().pop_optimal_batches(4, timeout=0.01)) == []


def test_token_budget_queue_cuts_by_tokens():
    rng = np.random.default_rng(3)
    lengths = rng.integers(1, 513, size=300).tolist()
    q = bt.TokenBudgetQueue(max_tokens=4096)
    q.extend([_Prio(L, i, done=(i % 50 == 7)) for i, L in enumerate(lengths)])
    seen = []
    while len(q):
        for batch in q.pop_optimal_batches(32, max_n_batches=4):
            idx = [it.index for it in batch]
            assert 1 <= len(idx) <= 32 and (len(idx) == 1 or sum(lengths[i] for i in idx) <= 4096)
            assert [lengths[i] for i in idx] == sorted(lengths[i] for i in idx)
            seen.extend(idx)
    assert sorted(seen) == [i for i in range(300) if i % 50 != 7]      # finished futures are dropped
    with pytest.raises(ValueError):
        bt.TokenBudgetQueue(max_tokens=0)


def test_backend_warmup_contract():
    spec = cf.tiny_spec("bert")
    emb = B200Embedder(spec=spec, model=FakeDeviceModel(spec.hidden))
    eps, seconds, log = emb.warmup(batch_size=4, n_tokens=7)
    assert eps > 0 and seconds >= 0 and "embeddings/sec" in log
    ce = B200CrossEncoder(spec=cf.tiny_spec("xlmr"), model=FakeDeviceModel(1))
    assert ce.warmup(batch_size=2, n_tokens=3)[0] > 0
    assert emb.capabilities == {"embed"} and ce.capabilities == {"rerank"}


@pytest.fixture(scope="module")
def reference():
    if not REF.exists():
        pytest.skip("reference tree not mounted on this machine")
    sys.path.insert(0, str(Path(__file__).parent / "golden"))
    import make_golden
    return make_golden.import_reference(str(REF))


def test_embed_through_the_reference_batch_handler(reference):
    """The reference's fake-backend pins (tests/unit_test/test_engine.py:24-35: row i carries
    the length of sentence i; usage == sum of lengths) with our backend behind its BatchHandler."""
    from infinity_emb.inference.batch_handler import BatchHandler
    spec = cf.tiny_spec("bert")
    backend = B200Embedder(spec=spec, model=FakeDeviceModel(spec.hidden))
    rng = np.random.default_rng(0)
    # 400 sentences in batches of 16: 25 batches, more than the backend's ring of result buffers
    sentences = [" ".join(map(str, rng.integers(1, 900, size=int(L)))) for L in rng.integers(1, 120, size=400)]

    async def run():
        bh = BatchHandler(model_replicas=[backend], max_batch_size=16, lengths_via_tokenize=True)
        await bh.spawn()
        try:
            return await bh.embed(sentences)
        finally:
            await bh.shutdown()

    embeddings, usage = asyncio.run(run())
    assert usage == sum(len(s.split()) for s in sentences)
    assert len(embeddings) == len(sentences)
    for s, e in zip(sentences, embeddings):
        toks = [int(x) for x in s.split()]
        assert e.shape == (spec.hidden,) and e[0] == len(toks) and e[1] == float(sum(toks))
    assert max(backend.model.calls) <= 16


def test_token_budget_queue_inside_the_reference_batch_handler(reference):
    """The one-assignment swap: BatchHandler._queue_prio = TokenBudgetQueue(...). Every sentence still gets
    its own row, and no encode_core call sees more tokens than the budget."""
    from infinity_emb.inference.batch_handler import BatchHandler
    spec = cf.tiny_spec("bert")
    model = FakeDeviceModel(spec.hidden)
    tokens_per_call = []
    plain_forward = model.forward_arrays

    def counting_forward(ids, cu, types=None, out=None, **kw):
        tokens_per_call.append(int(cu[-1]))
        return plain_forward(ids, cu, types, out=out, **kw)

    model.forward_arrays = counting_forward
    backend = B200Embedder(spec=spec, model=model)
    rng = np.random.default_rng(4)
    sentences = [" ".join(map(str, rng.integers(1, 900, size=int(L)))) for L in rng.integers(1, 120, size=300)]

    async def run():
        bh = BatchHandler(model_replicas=[backend], max_batch_size=32, lengths_via_tokenize=True)
        bh._queue_prio = bt.TokenBudgetQueue(max_tokens=600)
        await bh.spawn()
        try:
            return await bh.embed(sentences)
        finally:
            await bh.shutdown()

    embeddings, usage = asyncio.run(run())
    assert usage == sum(len(s.split()) for s in sentences)
    for s, e in zip(sentences, embeddings):
        toks = [int(x) for x in s.split()]
        assert e[0] == len(toks) and e[1] == float(sum(toks))
    assert max(tokens_per_call) <= 600 and max(model.calls) <= 32 and len(tokens_per_call) > 300 * 60 // 600 // 2


def test_rerank_through_the_reference_batch_handler(reference):
    """Raw logits go back flat; the batcher applies the sigmoid and sorts (batch_handler.py:208-219)."""
    from infinity_emb.inference.batch_handler import BatchHandler
    spec = cf.tiny_spec("xlmr")
    backend = B200CrossEncoder(spec=spec, model=FakeDeviceModel(1))
    query = "7 8 9"
    docs = ["1 2", "1 2 3 4 5 6", "1"]

    async def run():
        bh = BatchHandler(model_replicas=[backend], max_batch_size=8)
        await bh.spawn()
        try:
            return await bh.rerank(query=query, docs=docs, raw_scores=False)
        finally:
            await bh.shutdown()

    results, usage = asyncio.run(run())
    # logit = token count of [start] q [sep][sep] d [end]
    want = {i: 1 / (1 + np.exp(-(len(query.split()) + len(d.split()) + 4))) for i, d in enumerate(docs)}
    assert [r.index for r in results] == [1, 0, 2]
    for r in results:
        assert abs(r.relevance_score - want[r.index]) < 1e-6


def test_engine_api_with_patched_select_model(reference):
    """The reference's public engine API (AsyncEmbeddingEngine.embed / rerank) with our backend
    returned by a patched ``select_model`` (engine.py:56-58 looks the name up at call time): the
    drop-in route that needs no edit of the reference tree."""
    import infinity_emb.engine as engine_mod
    from infinity_emb.args import EngineArgs

    spec = cf.tiny_spec("bert")
    made = {}

    def fake_select_model(engine_args):
        backend = B200Embedder(engine_args=engine_args, spec=spec, model=FakeDeviceModel(spec.hidden))
        made["backend"] = backend
        return [backend], 0.0, 0.0

    original = engine_mod.select_model
    engine_mod.select_model = fake_select_model
    try:
        args = EngineArgs(model_name_or_path="b200/tiny", engine="debugengine", batch_size=8, model_warmup=False,
                          lengths_via_tokenize=True)
        eng = engine_mod.AsyncEmbeddingEngine.from_args(args)

        async def run():
            async with eng:
                return await eng.embed(sentences=["1 2 3", "4 5 6 7 8", "9"])

        embeddings, usage = asyncio.run(run())
    finally:
        engine_mod.select_model = original
    assert usage == 9
    assert [int(e[0]) for e in embeddings] == [3, 5, 1]
    assert [int(e[1]) for e in embeddings] == [6, 30, 9]
    assert made["backend"].engine_args.model_name_or_path == "b200/tiny" and made["backend"].engine_args.batch_size == 8
