"""Checkpoint directories written by the locally installed ``transformers`` classes (random weights:
no published checkpoint is reachable here) -> the runtime's weight file -> the same numbers as the
transformers forward the reference would run (sentence_transformer.py:124, crossencoder/torch.py:106)."""
import json

import numpy as np
import pytest
import torch

from infinity_b200 import checkpoints as ck
from infinity_b200 import configs as cf
from infinity_b200 import weights as wt
from oracle import encoder as enc
from oracle import pooling as OP


def _save(model, tmp_path, name, st_pooling=None):
    # the runtime stores matrices in bf16: give the transformers model exactly those values
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() == 2:
                p.copy_(p.to(torch.bfloat16).float())
    d = tmp_path / name
    model.save_pretrained(d, safe_serialization=True)
    if st_pooling:
        (d / "modules.json").write_text(json.dumps([
            {"idx": 0, "name": "0", "path": "", "type": "sentence_transformers.models.Transformer"},
            {"idx": 1, "name": "1", "path": "1_Pooling", "type": "sentence_transformers.models.Pooling"},
            {"idx": 2, "name": "2", "path": "2_Normalize", "type": "sentence_transformers.models.Normalize"}]))
        (d / "1_Pooling").mkdir()
        (d / "1_Pooling" / "config.json").write_text(json.dumps({
            "word_embedding_dimension": model.config.hidden_size,
            "pooling_mode_cls_token": st_pooling == "cls", "pooling_mode_mean_tokens": st_pooling == "mean",
            "pooling_mode_lasttoken": st_pooling == "last"}))
    return d


def _bert(tmp_path, st_pooling="mean"):
    from transformers import BertConfig, BertModel
    torch.manual_seed(0)
    cfg = BertConfig(vocab_size=500, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, intermediate_size=256,
                     max_position_embeddings=96, type_vocab_size=2, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    model = BertModel(cfg, add_pooling_layer=False).eval()
    return model, _save(model, tmp_path, "bert-ckpt", st_pooling)


def _xlmr_reranker(tmp_path):
    from transformers import XLMRobertaConfig, XLMRobertaForSequenceClassification
    torch.manual_seed(1)
    cfg = XLMRobertaConfig(vocab_size=500, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                           intermediate_size=256, max_position_embeddings=98, type_vocab_size=1, layer_norm_eps=1e-5,
                           hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, num_labels=1, pad_token_id=1,
                           classifier_dropout=0.0)
    model = XLMRobertaForSequenceClassification(cfg).eval()
    return model, _save(model, tmp_path, "xlmr-ckpt")


def _qwen2(tmp_path):
    from transformers import Qwen2Config, Qwen2Model
    torch.manual_seed(2)
    cfg = Qwen2Config(vocab_size=500, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-6,
                      rope_theta=1e6, attention_dropout=0.0, use_sliding_window=False, tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    model = Qwen2Model(cfg).eval()
    return model, _save(model, tmp_path, "qwen2-ckpt", "last")


def _hf_embeddings(model, spec, batch):
    pad_id = 1 if spec.arch == "xlmr" else 0
    cu = batch.cu_seqlens
    types = None
    if batch.token_type_ids is not None:
        types = [batch.token_type_ids[cu[i]: cu[i + 1]] for i in range(batch.n_seqs)]
    ids, mask, tt = enc.pad_batch(batch.sequences(), types, pad_id)
    kw = dict(input_ids=ids, attention_mask=mask)
    if spec.type_vocab > 1:
        kw["token_type_ids"] = tt
    with torch.no_grad():
        out = model(**kw)
    if spec.head == "classifier":
        return out.logits.float().numpy()
    pooled = OP.POOLERS[spec.pooling](out.last_hidden_state.float().numpy(), mask.numpy()).astype(np.float32)
    return OP.normalize(pooled) if spec.normalize else pooled


def test_plain_checkpoint_without_pooling_files_gets_mean_pooling():
    """A plain transformers directory (no modules.json / 1_Pooling): the reference loads it through
    SentenceTransformer, which adds mean pooling; a classification checkpoint reads the first token."""
    base = dict(model_type="bert", hidden_size=128, num_attention_heads=4, num_hidden_layers=2, intermediate_size=256,
                vocab_size=1000, max_position_embeddings=96)
    assert ck.spec_from_hf_config(dict(base, architectures=["BertModel"])).pooling == "mean"
    clf = ck.spec_from_hf_config(dict(base, architectures=["BertForSequenceClassification"], num_labels=3))
    assert clf.pooling == "cls" and clf.head == "classifier" and clf.n_labels == 3
    assert ck.spec_from_hf_config(dict(base, architectures=["BertModel"]), pooling="cls").pooling == "cls"


def test_spec_and_tensor_names_from_checkpoints(tmp_path):
    model, d = _bert(tmp_path, "mean")
    spec = ck.convert_checkpoint(d, tmp_path / "bert.b2ew")
    assert (spec.arch, spec.n_layers, spec.hidden, spec.n_heads, spec.head_dim, spec.ffn) == ("bert", 2, 128, 4, 32, 256)
    assert spec.pooling == "mean" and spec.normalize and spec.head == "none" and spec.max_len == 96
    W = wt.load_weights(tmp_path / "bert.b2ew")
    assert W["layer.0.qkv.w"].shape == (384, 128) and W["layer.0.qkv.w"].dtype == torch.bfloat16
    assert W["emb.ln.g"].dtype == torch.float32
    # the converted tensors reproduce the transformers forward through the oracle
    batch = cf.random_batch(spec, [3, 17, 64, 40], 9, with_types=True)
    Wf = {k: v.float() for k, v in W.items()}
    assert np.abs(enc.forward_batch(spec, Wf, batch) - _hf_embeddings(model, spec, batch)).max() < 2e-5

    model, d = _xlmr_reranker(tmp_path)
    spec = ck.convert_checkpoint(d, tmp_path / "xlmr.b2ew")
    assert (spec.arch, spec.pos_offset, spec.type_vocab, spec.head, spec.n_labels, spec.normalize, spec.max_len) == \
        ("xlmr", 2, 1, "classifier", 1, False, 96)
    Wf = {k: v.float() for k, v in wt.load_weights(tmp_path / "xlmr.b2ew").items()}
    rng = np.random.default_rng(3)
    batch = cf.pack([rng.integers(2, 500, size=L) for L in (5, 30, 64, 12)])
    assert np.abs(enc.forward_batch(spec, Wf, batch) - _hf_embeddings(model, spec, batch)).max() < 2e-5

    _, d = _qwen2(tmp_path)
    spec = ck.convert_checkpoint(d, tmp_path / "qwen2.b2ew")
    assert (spec.arch, spec.n_kv_heads, spec.head_dim, spec.rope_theta, spec.pooling) == ("decoder", 2, 32, 1e6, "last")
    W = wt.load_weights(tmp_path / "qwen2.b2ew")
    assert W["layer.1.gu.w"].shape == (512, 128) and "layer.1.gate.w" not in W
    with pytest.raises(ValueError):
        ck.spec_from_hf_config({"model_type": "t5"})


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["bert", "xlmr", "qwen2"])
def test_converted_checkpoint_runs_like_transformers(tmp_path, kind):
    """Checkpoint directory -> weight file -> CUDA forward, against the transformers class itself
    (fp32 on the CPU, the reference's CPU path): cosine >= 0.9999, logits within 1e-2."""
    from infinity_b200.engine import B200Model
    model, d = {"bert": _bert, "xlmr": _xlmr_reranker, "qwen2": _qwen2}[kind](tmp_path)
    path = tmp_path / f"{kind}.b2ew"
    spec = ck.convert_checkpoint(d, path)
    gpu = B200Model(spec, str(path))
    rng = np.random.default_rng(5)
    lens = [1, 9, 33, 64, 90, 17]
    if kind == "bert":
        batch = cf.random_batch(spec, lens, 7, with_types=True)
    else:
        batch = cf.pack([rng.integers(2, 500, size=L) for L in lens])
    got = gpu.forward(batch)
    ref = _hf_embeddings(model, spec, batch)
    if spec.head == "classifier":
        assert np.abs(got - ref).max() <= 1e-2
    else:
        cos = (got * ref).sum(1) / (np.linalg.norm(got, axis=1) * np.linalg.norm(ref, axis=1))
        assert cos.min() >= 0.9999, cos
    gpu.close()
