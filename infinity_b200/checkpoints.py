"""Hugging Face checkpoint directory -> :class:`ModelSpec` + weight file for the CUDA runtime.

The reference loads such a directory through sentence-transformers / transformers
(infinity_emb/transformer/embedder/sentence_transformer.py:72-78,
infinity_emb/transformer/crossencoder/torch.py:54-67,
infinity_emb/transformer/classifier/torch.py:38-46). This module reads the same files
(``config.json``, ``model.safetensors`` or its shards, and the sentence-transformers
``modules.json`` / ``1_Pooling/config.json`` when present) and writes the runtime's tensors:

* ``BertModel`` / ``BertForSequenceClassification`` -> arch ``bert``
* ``XLMRobertaModel`` / ``RobertaModel`` / ``...ForSequenceClassification`` -> arch ``xlmr``
  (learned positions offset by ``pad_token_id + 1``, classification head ``dense`` -> tanh -> ``out_proj``)
* ``Qwen2Model`` / ``Qwen2ForCausalLM`` (the language-model head is dropped) -> arch ``decoder``

q / k / v projections are fused into one ``qkv`` matrix, gate / up are interleaved for the fused
SwiGLU epilogue (``configs.runtime_tensors``). Only the file formats are needed: ``safetensors`` and
``json``; ``transformers`` is not imported.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch

from . import weights as wt
from .configs import ModelSpec, runtime_tensors


def _load_state_dict(model_dir: Path) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    index = model_dir / "model.safetensors.index.json"
    if index.exists():
        files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    else:
        files = ["model.safetensors"]
    sd: Dict[str, torch.Tensor] = {}
    for f in files:
        path = model_dir / f
        if not path.exists():
            raise FileNotFoundError(f"{path}: only safetensors checkpoints are read")
        sd.update(load_file(str(path)))
    return sd


def _strip_prefix(sd: Dict[str, torch.Tensor], marker: str) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
    """Splits the state dict into the backbone (keys rebased to start at ``marker``) and the rest
    (heads). Checkpoints prefix the backbone with ``bert.``, ``roberta.``, ``model.`` or nothing."""
    prefix = None
    for k in sd:
        i = k.find(marker)
        if i >= 0:
            prefix = k[:i]
            break
    if prefix is None:
        raise ValueError(f"no tensor named like '{marker}' in the checkpoint")
    body = {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)} if prefix else dict(sd)
    rest = {k: v for k, v in sd.items() if not (prefix and k.startswith(prefix))} if prefix else {}
    return body, rest


def spec_from_hf_config(config: dict, *, name: str = "checkpoint", pooling: Optional[str] = None,
                        normalize: Optional[bool] = None, head: Optional[str] = None) -> ModelSpec:
    """The runtime's model descriptor for a transformers ``config.json``."""
    mt = config.get("model_type", "")
    archs = " ".join(config.get("architectures") or [])
    classifier = head == "classifier" or (head is None and "ForSequenceClassification" in archs)
    if mt == "bert" or mt in ("xlm-roberta", "roberta"):
        xlmr = mt != "bert"
        if config.get("hidden_act", "gelu") != "gelu":
            raise ValueError(f"hidden_act {config.get('hidden_act')} is not supported (exact GELU only)")
        if config.get("position_embedding_type", "absolute") != "absolute":
            raise ValueError("only absolute learned positions are supported")
        H, nh = config["hidden_size"], config["num_attention_heads"]
        pos_offset = config.get("pad_token_id", 1) + 1 if xlmr else 0
        n_labels = len(config.get("id2label") or {}) or config.get("num_labels", 1) if classifier else 0
        return ModelSpec(
            name=name, arch="xlmr" if xlmr else "bert", n_layers=config["num_hidden_layers"], hidden=H, n_heads=nh,
            n_kv_heads=nh, head_dim=H // nh, ffn=config["intermediate_size"], vocab=config["vocab_size"],
            max_pos=config["max_position_embeddings"], type_vocab=config.get("type_vocab_size", 2),
            pos_offset=pos_offset, norm_eps=config.get("layer_norm_eps", 1e-12),
            # no sentence-transformers pooling files: SentenceTransformer builds Transformer + Pooling(mean) for a
            # plain checkpoint directory, which is what the reference loads (sentence_transformer.py:57-78);
            # a classification head reads the first token
            pooling=pooling or ("cls" if classifier else "mean"),
            normalize=(not classifier) if normalize is None else normalize,
            head="classifier" if classifier else "none", n_labels=n_labels,
            max_len=config["max_position_embeddings"] - pos_offset)
    if mt == "qwen2":
        H, nh = config["hidden_size"], config["num_attention_heads"]
        rope = config.get("rope_theta") or (config.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        return ModelSpec(
            name=name, arch="decoder", n_layers=config["num_hidden_layers"], hidden=H, n_heads=nh,
            n_kv_heads=config.get("num_key_value_heads", nh), head_dim=config.get("head_dim") or H // nh,
            ffn=config["intermediate_size"], vocab=config["vocab_size"], max_pos=config["max_position_embeddings"],
            type_vocab=0, norm_eps=config.get("rms_norm_eps", 1e-6), rope_theta=float(rope),
            pooling=pooling or "last", normalize=True if normalize is None else normalize,
            max_len=config["max_position_embeddings"])
    raise ValueError(f"model_type '{mt}' is not supported (bert, roberta, xlm-roberta, qwen2)")


def tensors_from_hf_state_dict(spec: ModelSpec, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """fp32 master tensors under the runtime's names (the inverse of the name mapping the parity
    tests use to load the oracle's weights into the transformers classes)."""
    W: Dict[str, torch.Tensor] = {}
    f = lambda t: t.detach().to(torch.float32).contiguous()
    if spec.arch == "decoder":
        body, _ = _strip_prefix(sd, "embed_tokens.weight")
        W["emb.word"] = f(body["embed_tokens.weight"])
        for l in range(spec.n_layers):
            p, q = f"layer.{l}.", f"layers.{l}."
            W[p + "ln1.g"] = f(body[q + "input_layernorm.weight"])
            W[p + "qkv.w"] = torch.cat([f(body[q + f"self_attn.{n}_proj.weight"]) for n in "qkv"], 0)
            W[p + "qkv.b"] = torch.cat([f(body[q + f"self_attn.{n}_proj.bias"]) for n in "qkv"], 0)
            W[p + "o.w"] = f(body[q + "self_attn.o_proj.weight"])
            W[p + "ln2.g"] = f(body[q + "post_attention_layernorm.weight"])
            W[p + "gate.w"] = f(body[q + "mlp.gate_proj.weight"])
            W[p + "up.w"] = f(body[q + "mlp.up_proj.weight"])
            W[p + "down.w"] = f(body[q + "mlp.down_proj.weight"])
        W["norm.g"] = f(body["norm.weight"])
        return W
    body, rest = _strip_prefix(sd, "embeddings.word_embeddings.weight")
    W["emb.word"] = f(body["embeddings.word_embeddings.weight"])
    W["emb.pos"] = f(body["embeddings.position_embeddings.weight"])
    if spec.type_vocab > 0:
        W["emb.type"] = f(body["embeddings.token_type_embeddings.weight"])
    W["emb.ln.g"], W["emb.ln.b"] = f(body["embeddings.LayerNorm.weight"]), f(body["embeddings.LayerNorm.bias"])
    for l in range(spec.n_layers):
        p, q = f"layer.{l}.", f"encoder.layer.{l}."
        W[p + "qkv.w"] = torch.cat([f(body[q + f"attention.self.{n}.weight"]) for n in ("query", "key", "value")], 0)
        W[p + "qkv.b"] = torch.cat([f(body[q + f"attention.self.{n}.bias"]) for n in ("query", "key", "value")], 0)
        W[p + "o.w"], W[p + "o.b"] = f(body[q + "attention.output.dense.weight"]), f(body[q + "attention.output.dense.bias"])
        W[p + "ln1.g"], W[p + "ln1.b"] = f(body[q + "attention.output.LayerNorm.weight"]), f(body[q + "attention.output.LayerNorm.bias"])
        W[p + "ffn1.w"], W[p + "ffn1.b"] = f(body[q + "intermediate.dense.weight"]), f(body[q + "intermediate.dense.bias"])
        W[p + "ffn2.w"], W[p + "ffn2.b"] = f(body[q + "output.dense.weight"]), f(body[q + "output.dense.bias"])
        W[p + "ln2.g"], W[p + "ln2.b"] = f(body[q + "output.LayerNorm.weight"]), f(body[q + "output.LayerNorm.bias"])
    if spec.head == "classifier":
        both = {**rest, **body}
        if "classifier.dense.weight" in both:  # RoBERTa / XLM-R: dense -> tanh -> out_proj on the first token
            names = ("classifier.dense", "classifier.out_proj")
        elif "pooler.dense.weight" in both and "classifier.weight" in both:  # BERT: pooler (dense -> tanh) -> classifier
            names = ("pooler.dense", "classifier")
        else:
            raise ValueError("classification head: expected classifier.dense / out_proj or pooler.dense / classifier")
        W["head.dense.w"], W["head.dense.b"] = f(both[names[0] + ".weight"]), f(both[names[0] + ".bias"])
        W["head.out.w"], W["head.out.b"] = f(both[names[1] + ".weight"]), f(both[names[1] + ".bias"])
    return W


def _sentence_transformers_options(model_dir: Path) -> Tuple[Optional[str], Optional[bool]]:
    """Pooling mode and whether a Normalize module follows, from the sentence-transformers files."""
    pooling = normalize = None
    modules = model_dir / "modules.json"
    if modules.exists():
        mods = json.loads(modules.read_text())
        normalize = any(m.get("type", "").endswith("Normalize") for m in mods)
        for m in mods:
            if m.get("type", "").endswith("Pooling"):
                cfg = model_dir / m.get("path", "1_Pooling") / "config.json"
                if cfg.exists():
                    c = json.loads(cfg.read_text())
                    if c.get("pooling_mode_cls_token"):
                        pooling = "cls"
                    elif c.get("pooling_mode_mean_tokens"):
                        pooling = "mean"
                    elif c.get("pooling_mode_lasttoken"):
                        pooling = "last"
    return pooling, normalize


def convert_checkpoint(model_dir, out_path, *, pooling: Optional[str] = None, normalize: Optional[bool] = None,
                       head: Optional[str] = None) -> ModelSpec:
    """Reads a checkpoint directory and writes the runtime's weight file; returns its descriptor.
    The reference's engine always L2-normalises embeddings (sentence_transformer.py:85, 142-145), which is
    the default here too unless the model is a classifier / reranker."""
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    st_pooling, _ = _sentence_transformers_options(model_dir)
    spec = spec_from_hf_config(config, name=model_dir.name, pooling=pooling or st_pooling, normalize=normalize, head=head)
    master = tensors_from_hf_state_dict(spec, _load_state_dict(model_dir))
    wt.save_weights(out_path, runtime_tensors(master))
    return spec


if __name__ == "__main__":
    import argparse
    import dataclasses

    ap = argparse.ArgumentParser(description="checkpoint directory -> weight file + model descriptor (JSON on stdout)")
    ap.add_argument("model_dir")
    ap.add_argument("out_path")
    ap.add_argument("--pooling", choices=["cls", "mean", "last", "tokens"])
    a = ap.parse_args()
    print(json.dumps(dataclasses.asdict(convert_checkpoint(a.model_dir, a.out_path, pooling=a.pooling))))
