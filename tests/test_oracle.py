"""Pins the oracle: pooling / normalisation and batch formation against golden vectors the
reference's own code produced (tests/golden/make_golden.py), and the encoder restatement
against the locally installed ``transformers`` model classes the reference calls."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from infinity_b200 import configs as cf
from oracle import batching as OB
from oracle import encoder as enc
from oracle import pooling as OP

GOLD = Path(__file__).parent / "golden"


def test_pooling_matches_reference_golden():
    g = np.load(GOLD / "pooling_golden.npz")
    for name in "abcd":
        h, m = g[f"{name}_hidden"], g[f"{name}_mask"]
        assert np.array_equal(OP.mean_pooling(h, m), g[f"{name}_mean"])
        assert np.array_equal(OP.cls_token_pooling(h, m), g[f"{name}_cls"])
        assert np.array_equal(OP.normalize(OP.mean_pooling(h, m)), g[f"{name}_mean_norm"])
        assert np.array_equal(OP.normalize(OP.cls_token_pooling(h, m)), g[f"{name}_cls_norm"])
    assert np.array_equal(OP.normalize(g["zero_in"]), g["zero_norm"])
    assert np.array_equal(OP.mean_pooling(g["allmasked_hidden"], g["allmasked_mask"]), g["allmasked_mean"])


def test_ragged_pooling_equals_padded():
    g = np.load(GOLD / "pooling_golden.npz")
    h, m = g["b_hidden"], g["b_mask"]
    lens = m.sum(1)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ragged = np.concatenate([h[i, : lens[i]] for i in range(len(lens))])
    assert np.array_equal(OP.pool_ragged(ragged, cu, "mean", True), g["b_mean_norm"])
    assert np.array_equal(OP.pool_ragged(ragged, cu, "cls", False), g["b_cls"])
    last = OP.pool_ragged(ragged, cu, "last", False)
    assert np.array_equal(last, np.stack([h[i, lens[i] - 1] for i in range(len(lens))]))


def test_batch_former_matches_reference_golden():
    g = json.loads((GOLD / "batching_golden.json").read_text())
    assert len(g["cases"]) >= 7
    for case in g["cases"]:
        got = OB.pop_all_batches(case["priorities"], case["size"], case["max_n_batches"])
        assert got == case["batches"]
    # exactly `size` queued items come out in submission order, unsorted
    first = g["cases"][0]
    assert first["batches"] == [list(range(32))]
    assert g["char_lengths"]["lengths"] == [2, 3, 17] and g["char_lengths"]["total"] == 22


def _bert_state_dict(spec, W):
    sd = {
        "embeddings.word_embeddings.weight": W["emb.word"],
        "embeddings.position_embeddings.weight": W["emb.pos"],
        "embeddings.token_type_embeddings.weight": W["emb.type"],
        "embeddings.LayerNorm.weight": W["emb.ln.g"], "embeddings.LayerNorm.bias": W["emb.ln.b"],
    }
    H = spec.hidden
    for l in range(spec.n_layers):
        p, q = f"layer.{l}.", f"encoder.layer.{l}."
        wq, wk, wv = W[p + "qkv.w"].split(H, 0)
        bq, bk, bv = W[p + "qkv.b"].split(H, 0)
        sd.update({
            q + "attention.self.query.weight": wq, q + "attention.self.query.bias": bq,
            q + "attention.self.key.weight": wk, q + "attention.self.key.bias": bk,
            q + "attention.self.value.weight": wv, q + "attention.self.value.bias": bv,
            q + "attention.output.dense.weight": W[p + "o.w"], q + "attention.output.dense.bias": W[p + "o.b"],
            q + "attention.output.LayerNorm.weight": W[p + "ln1.g"], q + "attention.output.LayerNorm.bias": W[p + "ln1.b"],
            q + "intermediate.dense.weight": W[p + "ffn1.w"], q + "intermediate.dense.bias": W[p + "ffn1.b"],
            q + "output.dense.weight": W[p + "ffn2.w"], q + "output.dense.bias": W[p + "ffn2.b"],
            q + "output.LayerNorm.weight": W[p + "ln2.g"], q + "output.LayerNorm.bias": W[p + "ln2.b"],
        })
    return sd


def test_encoder_matches_transformers_bert():
    """The restatement against ``transformers.BertModel`` (the class behind
    SentenceTransformer.forward at sentence_transformer.py:124) with identical weights."""
    from transformers import BertConfig, BertModel
    spec = cf.tiny_spec("bert", hidden=64, n_heads=4, n_kv_heads=4, head_dim=16, ffn=128, vocab=300, max_pos=64)
    W = cf.oracle_tensors(spec, cf.init_weights(spec, 5, perturb=True))
    cfg = BertConfig(vocab_size=spec.vocab, hidden_size=spec.hidden, num_hidden_layers=spec.n_layers,
                     num_attention_heads=spec.n_heads, intermediate_size=spec.ffn, max_position_embeddings=spec.max_pos,
                     type_vocab_size=2, layer_norm_eps=spec.norm_eps, hidden_act="gelu",
                     hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    model = BertModel(cfg, add_pooling_layer=False).eval()
    missing, unexpected = model.load_state_dict(_bert_state_dict(spec, W), strict=False)
    assert not unexpected and all("position_ids" in m for m in missing), (missing, unexpected)
    batch = cf.random_batch(spec, [3, 17, 64, 40], 9, with_types=True)
    cu = batch.cu_seqlens
    types = [batch.token_type_ids[cu[i]: cu[i + 1]] for i in range(batch.n_seqs)]
    ids, mask, tt = enc.pad_batch(batch.sequences(), types)
    with torch.no_grad():
        ref = model(input_ids=ids, attention_mask=mask, token_type_ids=tt).last_hidden_state
    got = enc.encoder_hidden(spec, W, ids, mask, tt)
    m = mask.bool()
    assert (got[m] - ref[m]).abs().max().item() < 2e-5


def test_reranker_matches_transformers_xlmr():
    """The restatement against ``XLMRobertaForSequenceClassification`` (what
    AutoModelForSequenceClassification resolves to at crossencoder/torch.py:106)."""
    from transformers import XLMRobertaConfig, XLMRobertaForSequenceClassification
    spec = cf.tiny_spec("xlmr", hidden=64, n_heads=4, n_kv_heads=4, head_dim=16, ffn=128, vocab=300, max_pos=66)
    W = cf.oracle_tensors(spec, cf.init_weights(spec, 6, perturb=True))
    cfg = XLMRobertaConfig(vocab_size=spec.vocab, hidden_size=spec.hidden, num_hidden_layers=spec.n_layers,
                           num_attention_heads=spec.n_heads, intermediate_size=spec.ffn,
                           max_position_embeddings=spec.max_pos, type_vocab_size=1, layer_norm_eps=spec.norm_eps,
                           hidden_act="gelu", hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                           num_labels=1, pad_token_id=1, classifier_dropout=0.0)
    model = XLMRobertaForSequenceClassification(cfg).eval()
    sd = {"roberta." + k: v for k, v in _bert_state_dict(spec, W).items()}
    sd.update({"classifier.dense.weight": W["head.dense.w"], "classifier.dense.bias": W["head.dense.b"],
               "classifier.out_proj.weight": W["head.out.w"], "classifier.out_proj.bias": W["head.out.b"]})
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and all("position_ids" in m for m in missing), (missing, unexpected)
    lens = [5, 30, 64, 12]
    rng = np.random.default_rng(3)
    seqs = [rng.integers(2, spec.vocab, size=L) for L in lens]  # id 1 is the pad token
    ids, mask, _ = enc.pad_batch(seqs, None, pad_id=1)
    with torch.no_grad():
        ref = model(input_ids=ids, attention_mask=mask).logits.numpy()
    got = enc.forward_padded(spec, W, ids, mask)
    assert np.abs(got - ref).max() < 2e-5
    # and the ragged driver returns rows in batch order whatever the internal sort
    out = enc.forward_batch(spec, W, cf.pack(seqs), batch_size=2)
    assert np.abs(out - ref).max() < 2e-5


def test_decoder_matches_transformers_qwen2():
    """The decoder restatement against ``transformers.Qwen2Model`` with identical weights."""
    from transformers import Qwen2Config, Qwen2Model
    from oracle import decoder as dec
    spec = cf.tiny_spec("decoder", hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=128, vocab=300, max_pos=64)
    W = cf.oracle_tensors(spec, cf.init_weights(spec, 8, perturb=True))
    cfg = Qwen2Config(vocab_size=spec.vocab, hidden_size=spec.hidden, intermediate_size=spec.ffn,
                      num_hidden_layers=spec.n_layers, num_attention_heads=spec.n_heads,
                      num_key_value_heads=spec.n_kv_heads, max_position_embeddings=spec.max_pos,
                      rms_norm_eps=spec.norm_eps, rope_theta=spec.rope_theta, attention_dropout=0.0,
                      use_sliding_window=False, tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    model = Qwen2Model(cfg).eval()
    nh, nkv, d = spec.n_heads, spec.n_kv_heads, spec.head_dim
    sd = {"embed_tokens.weight": W["emb.word"], "norm.weight": W["norm.g"]}
    for l in range(spec.n_layers):
        p, q = f"layer.{l}.", f"layers.{l}."
        wq, wk, wv = W[p + "qkv.w"].split([nh * d, nkv * d, nkv * d], 0)
        bq, bk, bv = W[p + "qkv.b"].split([nh * d, nkv * d, nkv * d], 0)
        sd.update({q + "self_attn.q_proj.weight": wq, q + "self_attn.q_proj.bias": bq,
                   q + "self_attn.k_proj.weight": wk, q + "self_attn.k_proj.bias": bk,
                   q + "self_attn.v_proj.weight": wv, q + "self_attn.v_proj.bias": bv,
                   q + "self_attn.o_proj.weight": W[p + "o.w"],
                   q + "mlp.gate_proj.weight": W[p + "gate.w"], q + "mlp.up_proj.weight": W[p + "up.w"],
                   q + "mlp.down_proj.weight": W[p + "down.w"],
                   q + "input_layernorm.weight": W[p + "ln1.g"], q + "post_attention_layernorm.weight": W[p + "ln2.g"]})
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and not [m for m in missing if "rotary" not in m], (missing, unexpected)
    rope = getattr(cfg, "rope_parameters", None) or {}
    assert float(rope.get("rope_theta", getattr(cfg, "rope_theta", 0))) == spec.rope_theta
    batch = cf.random_batch(spec, [3, 17, 64, 40], 9)
    ids, mask, _ = enc.pad_batch(batch.sequences())
    with torch.no_grad():
        ref = model(input_ids=ids, attention_mask=mask).last_hidden_state
    got = dec.decoder_hidden(spec, W, ids, mask)
    m = mask.bool()
    assert (got[m] - ref[m]).abs().max().item() < 5e-5


def test_token_level_oracle_is_consistent_with_pooled_oracle():
    """ColBERT-mode rows (sentence_transformer.py:125-131, 146-155) pooled by the in-tree mean /
    cls statements give the sentence embeddings of the pooled path: the two oracle entry points
    restate one forward."""
    import dataclasses
    spec = cf.tiny_spec("bert", hidden=64, n_heads=2, n_kv_heads=2, head_dim=32, ffn=128, pooling="mean")
    W = {k: v.float() for k, v in cf.init_weights(spec, 5, perturb=True).items()}
    batch = cf.random_batch(spec, [3, 17, 40, 1, 9], 2, with_types=True)
    tok_spec = dataclasses.replace(spec, pooling="tokens", normalize=False)
    rows = enc.forward_tokens(tok_spec, W, batch, batch_size=2)
    assert rows.shape == (batch.n_tokens, 64) and rows.dtype == np.float32
    for pooling in ("mean", "cls"):
        pooled = OP.pool_ragged(rows, batch.cu_seqlens, pooling, True)
        ref = enc.forward_batch(dataclasses.replace(spec, pooling=pooling), W, batch)
        np.testing.assert_allclose(pooled, ref, atol=2e-6)
    with pytest.raises(ValueError):
        enc.forward_batch(tok_spec, W, batch)


def test_output_quantisation_known_answers():
    """Hand-computed vectors for the restated sentence-transformers quantize_embeddings
    (called from infinity_emb/transformer/quantization/interface.py:147-151)."""
    from oracle import quant_embeddings as QE
    x = np.array([[0.5, -0.1, 0.0, 2.0, -3.0, 0.2, 0.3, -0.4, 1, 1, 1, 1, 1, 1, 1, 1]], dtype=np.float32)
    # bits (x > 0), most significant first: 1001 0110 = 150, 1111 1111 = 255
    assert QE.quantize_embeddings(x, "ubinary").tolist() == [[150, 255]]
    assert QE.quantize_embeddings(x, "binary").tolist() == [[22, 127]]
    assert QE.quantize_embeddings(x, "binary").dtype == np.int8
    r = np.array([[-1.0] * 16, [1.0] * 16])
    # (x + 1) / (2 / 255), truncated: 0.5 -> 191, -0.1 -> 114, 0 -> 127, in range
    u = QE.quantize_embeddings(x, "uint8", r)
    assert u.dtype == np.uint8 and u[0, :3].tolist() == [191, 114, 127] and u[0, 5:8].tolist() == [153, 165, 76]
    i = QE.quantize_embeddings(x, "int8", r)
    assert i.dtype == np.int8 and i[0, :3].tolist() == [63, -13, 0] and i[0, 5:8].tolist() == [25, 37, -51]
    # without ranges the batch's own min / max are used, in the embeddings' float32: the step 1/255 rounds
    # up in float32, so the maximum lands just below 255 and truncates to 254
    y = np.array([[0.0, 1.0], [1.0, 0.0], [0.25, 0.5]], dtype=np.float32)
    assert QE.quantize_embeddings(y, "uint8").tolist() == [[0, 254], [254, 0], [63, 127]]
    rng = QE.calibration_ranges(y)
    assert rng.shape == (2, 2) and rng.dtype == np.float64 and rng.tolist() == [[0.0, 0.0], [1.0, 1.0]]


def test_label_scores_match_the_text_classification_pipeline():
    """The reference's classifier is a transformers text-classification pipeline with top_k=None
    (classifier/torch.py:38-46): its post-processing functions are the pin for the oracle's scores."""
    tc = pytest.importorskip("transformers.pipelines.text_classification")
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal((7, 5)) * 4).astype(np.float32)
    assert np.allclose(enc.label_scores(logits), tc.softmax(logits), atol=1e-7)
    single = (rng.standard_normal((7, 1)) * 4).astype(np.float32)
    assert np.allclose(enc.label_scores(single), tc.sigmoid(single), atol=1e-7)
    assert np.allclose(enc.label_scores(np.array([[0.0]], dtype=np.float32)), [[0.5]])
    assert np.allclose(enc.label_scores(np.array([[1000.0, 0.0]], dtype=np.float32)), [[1.0, 0.0]])


def test_fast_nvfp4_dequantiser_equals_the_numpy_statement():
    """The table look-up used by the full-depth GPU test to stream a 7 G-parameter NVFP4 file."""
    from helpers import fast_dequantize_nvfp4
    from oracle import quant as Q
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.02, size=(64, 256)).astype(np.float32)
    w[3, :16] = 0.0
    packed, scales, gs = Q.quantize_nvfp4(w)
    want = Q.dequantize_nvfp4(packed, scales, gs)
    got = fast_dequantize_nvfp4(torch.from_numpy(packed), torch.from_numpy(scales), float(gs)).numpy()
    assert np.array_equal(got, want)
