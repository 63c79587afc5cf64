"""The reference-interface backends (encode_pre -> encode_core -> encode_post) on the real CUDA
model, with id-string sentences standing in for tokenised text."""
import numpy as np
import pytest

from helpers import cosines
from infinity_b200 import configs as cf
from infinity_b200 import weights as wt
from infinity_b200.backend import B200Classifier, B200CrossEncoder, B200Embedder
from infinity_b200.packing import IdStringTokenizer
from oracle import encoder as enc

pytestmark = pytest.mark.gpu


def _weights(tmp_path, spec, seed):
    master = cf.init_weights(spec, seed, perturb=True)
    path = tmp_path / f"{spec.name}.b2ew"
    wt.save_weights(path, cf.runtime_tensors(master))
    return str(path), cf.oracle_tensors(spec, master)


def _sentence(rng, n, vocab):
    return " ".join(str(int(x)) for x in rng.integers(3, vocab, size=n))


def test_embedder_backend_pipeline(tmp_path):
    spec = cf.tiny_spec("bert")
    path, W = _weights(tmp_path, spec, 51)
    backend = B200Embedder(spec=spec, weight_path=path, device_ids=(0,))
    rng = np.random.default_rng(0)
    sentences = [_sentence(rng, n, spec.vocab) for n in (5, 90, 17, 160, 1)]
    assert backend.tokenize_lengths(sentences) == [5, 90, 17, 160, 1]
    feats = backend.encode_pre(sentences)
    out = backend.encode_post(backend.encode_core(feats))
    assert out.shape == (5, spec.hidden) and out.dtype == np.float32
    ref = enc.forward_batch(spec, W, cf.pack([np.array(s.split(), dtype=np.int64) for s in sentences]))
    assert cosines(out, ref).min() >= 0.9999
    # encode_post hands out memory of its own: later batches leave earlier results alone
    again = backend.encode_post(backend.encode_core(feats))
    assert again.ctypes.data != out.ctypes.data and np.array_equal(again, out)
    eps, secs, log = backend.warmup(batch_size=8, n_tokens=64)
    assert eps > 0 and "ms inference" in log
    st = backend.model.stats
    assert st["calls"] == 3 and st["sequences"] == 5 + 5 + 8 and st["tokens"] == 2 * 273 + 8 * 64 and st["launches"] > 0
    backend.model.close()


def test_three_thread_pipeline_keeps_every_row(tmp_path):
    """The CUDA model behind the call pattern of the reference's ModelWorker (batch_handler.py:499-514):
    encode_pre, encode_core and encode_post on three threads joined by queues of depth 3 and 5.
    Thirty batches go through, every returned row is kept (as a view, the way the batcher stores
    results[i] in a future, batch_handler.py:445-447) and compared with the oracle at the end:
    rows that aliased a recycled result buffer would have been overwritten by then."""
    from infinity_b200.worker import ThreeStageWorker
    spec = cf.tiny_spec("bert")
    path, W = _weights(tmp_path, spec, 55)
    backend = B200Embedder(spec=spec, weight_path=path, device_ids=(0,))
    rng = np.random.default_rng(7)
    batches = [[_sentence(rng, int(n), spec.vocab) for n in rng.integers(1, 120, size=int(b))]
               for b in rng.integers(1, 12, size=30)]
    kept = {}

    def deliver(index, batch, results):
        for i in range(len(batch)):
            kept[(index, i)] = results[i]

    ThreeStageWorker(backend, deliver).run(batches)
    assert len(kept) == sum(len(b) for b in batches)
    worst = 1.0
    for index, batch in enumerate(batches):
        ref = enc.forward_batch(spec, W, cf.pack([np.array(s.split(), dtype=np.int64) for s in batch]))
        got = np.stack([kept[(index, i)] for i in range(len(batch))])
        worst = min(worst, float(cosines(got, ref).min()))
    assert worst >= 0.9999, worst
    assert backend.model.stats["calls"] == 30
    backend.model.close()

    # the reranker's flat logits are the caller's too
    xspec = cf.tiny_spec("xlmr")
    xpath, XW = _weights(tmp_path, xspec, 56)
    ce = B200CrossEncoder(spec=xspec, weight_path=xpath, device_ids=(0,),
                          tokenizer=IdStringTokenizer(xspec.max_pos - xspec.pos_offset))
    pair_batches = [[(_sentence(rng, int(q), xspec.vocab), _sentence(rng, int(d), xspec.vocab))
                     for q, d in zip(rng.integers(2, 20, size=int(b)), rng.integers(2, 80, size=int(b)))]
                    for b in rng.integers(1, 8, size=14)]
    logits = {}
    ThreeStageWorker(ce, lambda index, batch, res: logits.__setitem__(index, res)).run(pair_batches)
    for index, batch in enumerate(pair_batches):
        f = ce.encode_pre(batch)
        ref = enc.forward_batch(xspec, XW, cf.Batch(f.input_ids, f.cu_seqlens))
        assert logits[index].shape == (len(batch),) and np.abs(logits[index] - ref[:, 0]).max() <= 1e-2
    ce.model.close()


def test_embedder_backend_colbert_mode(tmp_path):
    """ColBERT mode through the backend: encode_post returns one [L_i, hidden] float32 array per
    sentence, not normalised (sentence_transformer.py:87-90, 146-155)."""
    spec = cf.tiny_spec("bert", pooling="tokens", normalize=False)
    path, W = _weights(tmp_path, spec, 53)
    backend = B200Embedder(spec=spec, weight_path=path, device_ids=(0,))
    rng = np.random.default_rng(2)
    lens = (5, 90, 17, 160, 1)
    sentences = [_sentence(rng, n, spec.vocab) for n in lens]
    out = backend.encode_post(backend.encode_core(backend.encode_pre(sentences)))
    assert isinstance(out, list) and [o.shape for o in out] == [(n, spec.hidden) for n in lens]
    batch = cf.pack([np.array(s.split(), dtype=np.int64) for s in sentences])
    ref = enc.forward_tokens(spec, W, batch)
    got = np.concatenate(out, axis=0)
    assert got.dtype == np.float32 and cosines(got, ref).min() >= 0.999
    eps, _, _ = backend.warmup(batch_size=4, n_tokens=16)
    assert eps > 0
    backend.model.close()


def test_embedder_backend_embedding_dtypes(tmp_path):
    """EmbeddingDtype on the backend (primitives.py:145-158): rows equal the numpy quantiser applied
    to the float32 rows, with ranges calibrated on caller-supplied sentences."""
    from oracle import quant_embeddings as QE
    spec = cf.tiny_spec("bert")
    path, _ = _weights(tmp_path, spec, 54)
    rng = np.random.default_rng(3)
    sentences = [_sentence(rng, n, spec.vocab) for n in (5, 90, 17, 160, 1)]
    calib = [_sentence(rng, n, spec.vocab) for n in rng.integers(4, 120, size=20)]
    plain = B200Embedder(spec=spec, weight_path=path, device_ids=(0,))
    rows = np.array(plain.encode_post(plain.encode_core(plain.encode_pre(sentences))))
    for dtype in ("uint8", "binary"):
        be = B200Embedder(spec=spec, weight_path=path, device_ids=(0,), embedding_dtype=dtype)
        if dtype == "uint8":
            with pytest.raises(ValueError):
                be.encode_core(be.encode_pre(sentences))
            ranges = be.calibrate(calib)
            assert ranges.shape == (2, spec.hidden)
        out = be.encode_post(be.encode_core(be.encode_pre(sentences)))
        assert np.array_equal(out, QE.quantize_embeddings(rows, dtype, be.calibration_ranges))
        be.model.close()
    plain.model.close()


def test_cross_encoder_and_classifier_backends(tmp_path):
    spec = cf.tiny_spec("xlmr")
    path, W = _weights(tmp_path, spec, 52)
    ce = B200CrossEncoder(spec=spec, weight_path=path, device_ids=(0,),
                          tokenizer=IdStringTokenizer(spec.max_pos - spec.pos_offset))
    rng = np.random.default_rng(1)
    pairs = [(_sentence(rng, q, spec.vocab), _sentence(rng, d, spec.vocab)) for q, d in ((4, 30), (10, 120), (3, 3), (60, 200))]
    feats = ce.encode_pre(pairs)
    assert feats.n_seqs == 4 and int(np.diff(feats.cu_seqlens).max()) <= spec.max_pos - spec.pos_offset
    logits = ce.encode_post(ce.encode_core(feats))
    assert logits.shape == (4,) and logits.dtype == np.float32
    ref = enc.forward_batch(spec, W, cf.Batch(feats.input_ids, feats.cu_seqlens))
    assert np.abs(logits - ref[:, 0]).max() <= 1e-2
    ce.model.close()

    spec3 = cf.tiny_spec("xlmr", n_labels=3)
    path3, W3 = _weights(tmp_path, spec3, 53)
    clf = B200Classifier(spec=spec3, weight_path=path3, device_ids=(0,), labels=["neg", "neu", "pos"])
    sentences = [_sentence(rng, n, spec3.vocab) for n in (7, 50)]
    res = clf.encode_post(clf.encode_core(clf.encode_pre(sentences)))
    ref3 = enc.forward_batch(spec3, W3, cf.pack([np.array(s.split(), dtype=np.int64) for s in sentences]))
    z = np.exp(ref3 - ref3.max(1, keepdims=True))
    probs = z / z.sum(1, keepdims=True)
    for row, p in zip(res, probs):
        assert [d["label"] for d in row] == [["neg", "neu", "pos"][j] for j in np.argsort(-p)]
        assert abs(row[0]["score"] - p.max()) < 1e-2
    clf.model.close()
    dev = B200Classifier(spec=spec3, weight_path=path3, device_ids=(0,), labels=["neg", "neu", "pos"], device_scores=True)
    res_dev = dev.encode_post(dev.encode_core(dev.encode_pre(sentences)))
    for row, row_dev in zip(res, res_dev):
        assert [d["label"] for d in row] == [d["label"] for d in row_dev]
        assert max(abs(a["score"] - b["score"]) for a, b in zip(row, row_dev)) < 1e-5
    dev.model.close()
