"""End-to-end parity of the CUDA forward (through the C ABI, host buffers in and out)
against the fp32 CPU oracle on the same seeded weights and inputs.

Tolerances (bf16 compute against the fp32 oracle that sees the same stored weights):
cosine >= 0.9999 per embedding; classifier logits within 1e-2 absolute.
"""
import numpy as np
import pytest
import torch

from infinity_b200 import configs as cf
from infinity_b200 import weights as wt
from infinity_b200.engine import B200Model
from oracle import encoder as enc

pytestmark = pytest.mark.gpu

COS_TOL = 0.9999
LOGIT_TOL = 1e-2


from helpers import build_model, cosines  # noqa: E402

COS_TOL_BLOCK = 0.999  # MXFP8 / NVFP4 weights, against the oracle run with the same dequantised weights


@pytest.mark.parametrize("pooling", ["cls", "mean", "last"])
@pytest.mark.parametrize("hidden,heads,hd", [(128, 4, 32), (256, 4, 64), (512, 4, 128)])
def test_tiny_encoder_matches_oracle(tmp_path, pooling, hidden, heads, hd):
    spec = cf.tiny_spec("bert", hidden=hidden, n_heads=heads, n_kv_heads=heads, head_dim=hd, ffn=2 * hidden,
                        pooling=pooling)
    model, W = build_model(tmp_path, spec, 11, perturb=True)
    batch = cf.random_batch(spec, [1, 2, 9, 64, 65, 127, 128, 160, 33, 77], 5, with_types=True)
    got = model.forward(batch)
    ref = enc.forward_batch(spec, W, batch)
    assert got.shape == ref.shape == (batch.n_seqs, hidden)
    cos = cosines(got, ref)
    assert cos.min() >= COS_TOL, cos
    np.testing.assert_allclose(np.linalg.norm(got, axis=1), 1.0, atol=1e-5)
    model.close()


@pytest.mark.parametrize("normalize", [False, True])
def test_token_level_outputs_match_oracle(tmp_path, normalize):
    """ColBERT mode: one float32 row per real token, packed in batch order, normalisation off by
    default as in the reference (sentence_transformer.py:87-90, 125-131, 146-155)."""
    spec = cf.tiny_spec("bert", hidden=256, n_heads=4, n_kv_heads=4, head_dim=64, ffn=512, pooling="tokens",
                        normalize=normalize)
    model, W = build_model(tmp_path, spec, 17, perturb=True)
    batch = cf.random_batch(spec, [1, 2, 9, 64, 65, 127, 128, 160, 33, 77], 5, with_types=True)
    got = model.forward(batch)
    ref = enc.forward_tokens(spec, W, batch)
    assert got.shape == ref.shape == (batch.n_tokens, 256)
    cos = cosines(got, ref)
    assert cos.min() >= 0.999 and np.median(cos) >= COS_TOL, (cos.min(), np.median(cos))
    if normalize:
        np.testing.assert_allclose(np.linalg.norm(got, axis=1), 1.0, atol=1e-5)
    else:
        # magnitudes too: the rows are LayerNorm outputs rounded to bf16
        assert np.abs(got - ref).max() <= 0.05 * np.abs(ref).max()
    # a sequence's token rows do not depend on its neighbours
    cu = batch.cu_seqlens
    alone = model.forward(cf.pack([batch.sequences()[3]], [batch.token_type_ids[cu[3]:cu[4]]]))
    assert np.array_equal(alone, got[cu[3]:cu[4]])
    model.close()


def test_quantised_output_rows(tmp_path):
    """b200emb_forward_quantized = the numpy quantiser applied to b200emb_forward's float32 rows, bit for
    bit, for every EmbeddingDtype; int8 / uint8 with ranges calibrated as the reference does."""
    from oracle import quant_embeddings as QE
    spec = cf.tiny_spec("bert", hidden=256, n_heads=4, n_kv_heads=4, head_dim=64, ffn=512)
    model, _ = build_model(tmp_path, spec, 19, perturb=True)
    batch = cf.random_batch(spec, [3, 50, 128, 9, 77, 160, 1], 4, with_types=True)
    rows = np.array(model.forward(batch))
    calib = np.array(model.forward(cf.random_batch(spec, [20, 40, 60, 80, 100, 120], 6, with_types=True)))
    ranges = QE.calibration_ranges(calib)
    for precision in ("int8", "uint8", "binary", "ubinary"):
        got = model.forward_quantized(batch.input_ids, batch.cu_seqlens, precision, batch.token_type_ids,
                                      ranges if precision in ("int8", "uint8") else None)
        ref = QE.quantize_embeddings(rows, precision, ranges if precision in ("int8", "uint8") else None)
        assert got.dtype == ref.dtype and got.shape == ref.shape
        assert np.array_equal(got, ref), precision
    with pytest.raises(RuntimeError, match="calibration ranges"):
        model.forward_quantized(batch.input_ids, batch.cu_seqlens, "int8", batch.token_type_ids, None)
    model.close()


def test_tiny_reranker_matches_oracle(tmp_path):
    spec = cf.tiny_spec("xlmr")
    model, W = build_model(tmp_path, spec, 12, perturb=True)
    batch = cf.random_batch(spec, [4, 30, 99, 158, 64], 6)
    got = model.forward(batch)
    ref = enc.forward_batch(spec, W, batch)
    assert got.shape == (5, 1)
    assert np.abs(got - ref).max() <= LOGIT_TOL, (got, ref)
    model.close()


@pytest.mark.parametrize("n_labels", [1, 3, 40])
def test_label_scores_on_the_device(tmp_path, n_labels):
    """softmax over the labels (sigmoid for one label) behind the classifier head equals the oracle's
    float64 softmax of its own logits; rows of a multi-label head sum to 1"""
    import dataclasses
    spec = dataclasses.replace(cf.tiny_spec("xlmr", n_labels=n_labels), label_scores=True)
    model, W = build_model(tmp_path, spec, 15 + n_labels, perturb=True)
    batch = cf.random_batch(spec, [4, 30, 99, 158, 64, 1], 7)
    got = model.forward(batch)
    ref = enc.forward_batch(spec, W, batch)
    raw = enc.forward_batch(dataclasses.replace(spec, label_scores=False), W, batch)
    assert got.shape == (6, n_labels) and ref.shape == got.shape
    assert np.allclose(ref, enc.label_scores(raw), atol=1e-7)
    assert np.abs(got - ref).max() <= LOGIT_TOL, (got, ref)
    assert (got >= 0).all() and (got <= 1).all()
    if n_labels > 1:
        assert np.abs(got.sum(1) - 1.0).max() <= 1e-5
    model.close()


def test_repeated_small_forwards_are_bit_identical(tmp_path):
    """Small batches run with programmatic dependent launch (each kernel's set-up overlaps its predecessor's
    tail): a kernel that touched its inputs before the predecessor finished would show as run-to-run noise."""
    spec = cf.tiny_spec("bert", hidden=128, n_heads=2, n_kv_heads=2, head_dim=64, ffn=256, max_pos=256)
    model, W = build_model(tmp_path, spec, 21, perturb=True)
    batch = cf.random_batch(spec, [5, 130, 64, 17, 200, 1, 33], 9)
    first = model.forward(batch).copy()
    assert cosines(first, enc.forward_batch(spec, W, batch)).min() >= COS_TOL
    for _ in range(40):
        assert np.array_equal(model.forward(batch), first)
    model.close()


def test_label_scores_need_a_classifier_head(tmp_path):
    import dataclasses
    from infinity_b200._lib import B200EmbError
    spec = dataclasses.replace(cf.tiny_spec("bert"), label_scores=True)
    with pytest.raises(B200EmbError, match="label_scores"):
        build_model(tmp_path, spec, 16, perturb=False)


def _oracle_forward(spec, W, batch):
    if spec.arch == "decoder":
        from oracle import decoder as dec
        return dec.forward_batch(spec, W, batch)
    return enc.forward_batch(spec, W, batch)


@pytest.mark.parametrize("kw", [dict(), dict(hidden=512, n_heads=4, n_kv_heads=1, head_dim=128, ffn=1024),
                                dict(pooling="mean", n_kv_heads=4)])
def test_tiny_decoder_matches_oracle(tmp_path, kw):
    """Pre-RMSNorm decoder: RoPE, causal grouped-query attention, fused SwiGLU, fp32 residual stream."""
    spec = cf.tiny_spec("decoder", **kw)
    model, W = build_model(tmp_path, spec, 21, perturb=True)
    batch = cf.random_batch(spec, [1, 2, 9, 64, 65, 127, 128, 300, 33, 77], 5)
    got = model.forward(batch)
    ref = _oracle_forward(spec, W, batch)
    cos = cosines(got, ref)
    assert cos.min() >= COS_TOL, cos
    model.close()


@pytest.mark.parametrize("fmt,tol", [("bf16", COS_TOL), ("nvfp4", COS_TOL_BLOCK)])
def test_qwen2_7b_layer_shapes(tmp_path, fmt, tol):
    """Two layers with the exact Qwen2-7B matrix shapes (hidden 3584, 28/4 heads of 128, FFN 18944)
    and a reduced vocabulary: exercises the real GEMM / attention / SwiGLU tile shapes, with bf16
    weights and with the configuration's NVFP4 weights."""
    from dataclasses import replace
    spec = replace(cf.QWEN2_7B, n_layers=2, vocab=4096, name="qwen2-7b-2layer", weight_format=fmt)
    model, W = build_model(tmp_path, spec, cf.SEEDS["c5"][2], perturb=False)
    batch = cf.random_batch(spec, [32, 700, 2048, 129, 1024, 63], 6)
    got = model.forward(batch)
    ref = _oracle_forward(spec, W, batch)
    cos = cosines(got, ref)
    print("qwen2 shape", fmt, "cosine", cos)
    assert cos.min() >= tol
    model.close()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_tiny_decoder_block_quantised_weights(tmp_path, fmt):
    """Layer matrices quantised by the CUDA quantisers and expanded per GEMM; the oracle runs the
    fp32 forward on the numpy-dequantised weights."""
    spec = cf.tiny_spec("decoder", weight_format=fmt)
    model, W = build_model(tmp_path, spec, 22, perturb=True)
    batch = cf.random_batch(spec, [3, 64, 129, 300, 31], 7)
    got = model.forward(batch)
    ref = _oracle_forward(spec, W, batch)
    cos = cosines(got, ref)
    print(fmt, "cosine", cos)
    assert cos.min() >= COS_TOL_BLOCK, cos
    # and the quantisation really happened: different from the bf16 model beyond rounding noise
    model.close()


def test_encoder_block_quantised_weights(tmp_path):
    spec = cf.tiny_spec("bert", weight_format="mxfp8")
    model, W = build_model(tmp_path, spec, 23, perturb=True)
    batch = cf.random_batch(spec, [5, 77, 128, 160], 8, with_types=True)
    cos = cosines(model.forward(batch), enc.forward_batch(spec, W, batch))
    assert cos.min() >= COS_TOL_BLOCK, cos
    model.close()


@pytest.mark.parametrize("fmt,tol", [("bf16", COS_TOL), ("mxfp8", COS_TOL_BLOCK)])
def test_tiny_moe_encoder_matches_oracle(tmp_path, fmt, tol):
    """Mixture-of-experts encoder: router, expert-contiguous scatter, grouped GEMM over all experts,
    gated combine + LayerNorm. With mxfp8 only the expert matrices are quantised."""
    spec = cf.tiny_spec("moe", weight_format=fmt)
    model, W = build_model(tmp_path, spec, 31, perturb=True)
    batch = cf.random_batch(spec, [1, 2, 9, 64, 65, 127, 128, 160, 33, 77], 5)
    got = model.forward(batch)
    ref = enc.forward_batch(spec, W, batch)
    cos = cosines(got, ref)
    print("moe", fmt, cos.min())
    assert cos.min() >= tol, cos
    again = model.forward(batch)  # slots inside an expert segment may move; results must not
    assert np.array_equal(got, again)
    model.close()


def test_moe_encoder_layer_shapes(tmp_path):
    """Two layers with the configuration-4 shapes (hidden 768, 12 heads, 8 experts of width 3072,
    top-2, MXFP8 expert matrices) and a reduced vocabulary."""
    from dataclasses import replace
    spec = replace(cf.MOE_ENCODER, n_layers=2, vocab=4096, name="moe-2layer")
    model, W = build_model(tmp_path, spec, cf.SEEDS["c4"][2], perturb=False)
    batch = cf.random_batch(spec, [16, 512, 300, 129, 64, 77, 511, 200] * 4, 6)
    got = model.forward(batch)
    ref = enc.forward_batch(spec, W, batch)
    cos = cosines(got, ref)
    print("c4 shape cosine min", cos.min())
    assert cos.min() >= COS_TOL_BLOCK
    model.close()


def test_order_and_batch_independence(tmp_path):
    """Row i belongs to sequence i whatever the order, and a sequence's embedding does not
    depend on its neighbours in the batch (bit-exact: same kernels, same per-row math)."""
    spec = cf.tiny_spec("bert")
    model, _ = build_model(tmp_path, spec, 13, perturb=True)
    lens = [5, 150, 31, 64, 100, 7, 129]
    batch = cf.random_batch(spec, lens, 8)
    full = model.forward(batch)
    seqs = batch.sequences()
    perm = [3, 0, 6, 2, 5, 1, 4]
    permuted = model.forward(cf.pack([seqs[i] for i in perm]))
    assert np.array_equal(permuted, full[perm])
    single = model.forward(cf.pack([seqs[1]]))
    assert np.array_equal(single[0], full[1])
    model.close()


def test_multi_device_handle_equals_single_device(tmp_path):
    """One handle over several GPUs: token-balanced split, rows scattered back to batch order; the
    result must be bit-identical to the single-GPU result (same kernels, same per-sequence math)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    spec = cf.tiny_spec("bert", hidden=256, n_heads=4, n_kv_heads=4, head_dim=64, ffn=512)
    single, _ = build_model(tmp_path, spec, 41, perturb=True, device_ids=(0,))
    n_dev = min(torch.cuda.device_count(), 4)
    multi, _ = build_model(tmp_path, spec, 41, perturb=True, device_ids=tuple(range(n_dev)))
    rng = np.random.default_rng(3)
    batch = cf.random_batch(spec, rng.integers(1, 161, size=97), 9, with_types=True)
    a = single.forward(batch)
    b = multi.forward(batch)
    assert multi.last_timing["n_devices"] == n_dev
    assert np.array_equal(a, b)
    cu = batch.cu_seqlens
    one = multi.forward(cf.pack([batch.sequences()[5]], [batch.token_type_ids[cu[5]:cu[6]]]))  # runs on the first device
    assert np.array_equal(one[0], a[5])
    q1 = single.forward_quantized(batch.input_ids, batch.cu_seqlens, "ubinary", batch.token_type_ids)
    q2 = multi.forward_quantized(batch.input_ids, batch.cu_seqlens, "ubinary", batch.token_type_ids)
    assert q1.shape == (97, 32) and np.array_equal(q1, q2)
    single.close()
    multi.close()
    # token-level outputs: rows return to packed batch order
    spec_t = cf.tiny_spec("bert", hidden=256, n_heads=4, n_kv_heads=4, head_dim=64, ffn=512, pooling="tokens",
                          normalize=False)
    single_t, _ = build_model(tmp_path, spec_t, 41, perturb=True, device_ids=(0,))
    multi_t, _ = build_model(tmp_path, spec_t, 41, perturb=True, device_ids=tuple(range(n_dev)))
    at, bt = single_t.forward(batch), multi_t.forward(batch)
    assert at.shape == (batch.n_tokens, 256) and np.array_equal(at, bt)
    single_t.close()
    multi_t.close()


def test_forward_device_range_checks_ids_on_the_device(tmp_path):
    """b200emb_forward_device never sees the ids on the host: the embedding kernel checks them against the table,
    reads row 0 for a bad one (no out-of-bounds access) and the call reports an invalid argument at its end;
    the handle stays usable."""
    from infinity_b200._lib import B200EmbError
    spec = cf.tiny_spec("bert")
    model, _ = build_model(tmp_path, spec, 16, perturb=True)
    batch = cf.random_batch(spec, [40, 3, 77], 5, with_types=True)
    want = model.forward(batch)
    d_cu = torch.from_numpy(batch.cu_seqlens).cuda()
    d_types = torch.from_numpy(batch.token_type_ids).cuda()
    d_out = torch.empty(batch.n_seqs, spec.out_dim, dtype=torch.float32, device="cuda")

    def run(ids, types):
        d_ids = torch.from_numpy(ids).cuda()
        d_ty = torch.from_numpy(types).cuda()
        torch.cuda.synchronize()
        model.forward_device(d_ids.data_ptr(), d_ty.data_ptr(), d_cu.data_ptr(), batch.cu_seqlens, batch.n_tokens, d_out.data_ptr())
        torch.cuda.synchronize()
        return d_out.cpu().numpy()

    assert np.array_equal(run(batch.input_ids, batch.token_type_ids), want)
    bad = batch.input_ids.copy()
    bad[17] = spec.vocab + 5
    with pytest.raises(B200EmbError, match="input id"):
        run(bad, batch.token_type_ids)
    bad = batch.input_ids.copy()
    bad[2] = -1
    with pytest.raises(B200EmbError, match="input id"):
        run(bad, batch.token_type_ids)
    bad_t = batch.token_type_ids.copy()
    bad_t[5] = spec.type_vocab
    with pytest.raises(B200EmbError, match="token type"):
        run(batch.input_ids, bad_t)
    assert np.array_equal(run(batch.input_ids, batch.token_type_ids), want)
    model.close()


def test_failed_workspace_growth_leaves_the_handle_usable(tmp_path):
    """A workspace allocation that fails part-way (the failure is injected on the host; the
    allocator is not called and no device fault is involved) must give a clean status, and the
    next, smaller batch must run on freshly allocated buffers, not on freed ones."""
    from infinity_b200 import _lib
    from infinity_b200._lib import B200EmbError
    spec = cf.tiny_spec("bert")
    model, _ = build_model(tmp_path, spec, 15, perturb=True)
    lib = _lib.load()
    small = cf.random_batch(spec, [40, 3, 77], 5)
    want = model.forward(small)
    big = cf.random_batch(spec, [150] * 20, 6)      # 3000 tokens: beyond the initial 1024-token workspaces
    try:
        for after in (0, 3, 7):                     # fail the first, a middle and a late allocation of the group
            lib.b200emb_test_fail_allocs(after, 1)
            with pytest.raises(B200EmbError, match="injected"):
                model.forward(big)
            lib.b200emb_test_fail_allocs(0, 0)
            assert np.array_equal(model.forward(small), want)
    finally:
        lib.b200emb_test_fail_allocs(0, 0)
    got_big = model.forward(big)
    assert np.isfinite(got_big).all() and np.array_equal(model.forward(small), want)
    model.close()


def test_tensor_maps_are_encoded_once_per_buffer_and_shape(tmp_path):
    """The second forward of a batch shape asks the driver for no descriptor: every request is
    served from the table; a new token count encodes the activation-side maps again and still
    finds the weight-side ones."""
    import ctypes as C
    from infinity_b200 import _lib
    lib = _lib.load()

    def stats():
        h, m = C.c_uint64(), C.c_uint64()
        assert lib.b200emb_tensor_map_stats(C.byref(h), C.byref(m)) == 0
        return h.value, m.value

    spec = cf.tiny_spec("bert")
    model, _ = build_model(tmp_path, spec, 21, perturb=True)
    a = cf.random_batch(spec, [40, 3, 77], 5)
    first = model.forward(a)
    h0, m0 = stats()
    again = model.forward(a)
    h1, m1 = stats()
    assert m1 == m0 and h1 > h0
    assert np.array_equal(first, again)
    model.forward(cf.random_batch(spec, [33, 9], 6))      # other token count: new activation maps, same weight maps
    h2, m2 = stats()
    assert m2 > m1 and h2 > h1
    model.close()


def test_invalid_inputs_are_rejected(tmp_path):
    from infinity_b200._lib import B200EmbError
    spec = cf.tiny_spec("bert")
    model, _ = build_model(tmp_path, spec, 14, perturb=False)
    ids = np.array([1, 2, 3, 4], dtype=np.int32)
    with pytest.raises(B200EmbError, match="strictly increasing"):
        model.forward_arrays(ids, np.array([0, 2, 2, 4], dtype=np.int32))
    with pytest.raises(B200EmbError, match="cu_seqlens\\[0\\]"):
        model.forward_arrays(ids, np.array([1, 4], dtype=np.int32))
    with pytest.raises(B200EmbError, match="vocabulary"):
        model.forward_arrays(np.array([1, 2, 3, spec.vocab], dtype=np.int32), np.array([0, 4], dtype=np.int32))
    with pytest.raises(B200EmbError, match="position table"):
        long = np.ones(spec.max_pos + 1, dtype=np.int32)
        model.forward_arrays(long, np.array([0, len(long)], dtype=np.int32))
    # empty batch: no work, no error
    out = model.forward_arrays(np.zeros(0, np.int32), np.zeros(1, np.int32))
    assert out.shape == (0, spec.hidden)
    model.close()


def test_config1_bge_small_shape(tmp_path):
    """Configuration 1 in full: 32 sequences, 7715 tokens, CLS pooling, fp32 master weights."""
    spec = cf.BGE_SMALL
    model, W = build_model(tmp_path, spec, cf.SEEDS["c1"][2], perturb=False)
    batch = cf.synth_batch("c1")
    assert batch.n_tokens == 7715
    got = model.forward(batch)
    ref = enc.forward_batch(spec, W, batch)
    cos = cosines(got, ref)
    print("c1 cosine min/mean", cos.min(), cos.mean())
    assert cos.min() >= COS_TOL
    model.close()


def test_config3_xlmr_large_reranker_subset(tmp_path):
    """Configuration 3 weights (XLM-R-large shape, 250002-row vocabulary, classification head):
    256 of its pairs on the GPU, 24 of them against the oracle; logits within 1e-2 and the
    sigmoid scores the batcher derives from them (batch_handler.py:208-210) within 1e-2 too."""
    spec = cf.XLMR_LARGE_RERANK
    model, W = build_model(tmp_path, spec, cf.SEEDS["c3"][2], perturb=False)
    batch = cf.synth_batch("c3", 256)
    assert batch.lengths.max() <= 512 and batch.lengths.min() >= 8 + 64 + 4
    full = model.forward(batch)
    assert full.shape == (256, 1) and np.isfinite(full).all()
    pick = list(range(0, 256, 11))[:24]
    seqs = batch.sequences()
    sub = cf.pack([seqs[i] for i in pick])
    got = model.forward(sub)
    assert np.array_equal(got, full[pick])
    ref = enc.forward_batch(spec, W, sub)
    print("c3 max |logit diff|", np.abs(got - ref).max())
    assert np.abs(got - ref).max() <= LOGIT_TOL
    sig = lambda z: 1.0 / (1.0 + np.exp(-z))
    assert np.abs(sig(got) - sig(ref)).max() <= LOGIT_TOL
    model.close()


def test_config2_bert_large_shape_subset(tmp_path):
    """Configuration 2 weights, 48 of its sequences (the oracle needs ~1 s per sequence on CPU);
    the GPU runs the full 1024-sequence batch and the rows of the subset must be identical."""
    spec = cf.BERT_LARGE
    model, W = build_model(tmp_path, spec, cf.SEEDS["c2"][2], perturb=False)
    batch = cf.synth_batch("c2")
    full = model.forward(batch)
    assert full.shape == (1024, 1024) and np.isfinite(full).all()
    np.testing.assert_allclose(np.linalg.norm(full, axis=1), 1.0, atol=1e-5)
    pick = list(range(0, 1024, 22))[:48]
    seqs = batch.sequences()
    sub = cf.pack([seqs[i] for i in pick])
    got = model.forward(sub)
    assert np.array_equal(got, full[pick])
    ref = enc.forward_batch(spec, W, sub)
    cos = cosines(got, ref)
    print("c2 cosine min/mean", cos.min(), cos.mean())
    assert cos.min() >= COS_TOL
    model.close()
