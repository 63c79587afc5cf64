"""Model shapes, seeded random-init weights and seeded synthetic batches.

The five named configurations are the benchmark / parity cases of this repository:
random-init weights (normal, std 0.02; zero biases; unit norm gains) and token ids drawn
directly from the stated ranges, because neither checkpoints nor tokenizer vocabularies
are reachable offline. Lengths include the special tokens.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


@dataclass(frozen=True)
class ModelSpec:
    name: str
    arch: str = "bert"            # bert | xlmr | moe | decoder
    n_layers: int = 12
    hidden: int = 384
    n_heads: int = 12
    n_kv_heads: int = 12
    head_dim: int = 32
    ffn: int = 1536
    vocab: int = 30522
    max_pos: int = 512            # rows of the position table
    type_vocab: int = 2
    pos_offset: int = 0
    norm_eps: float = 1e-12
    rope_theta: float = 0.0
    n_experts: int = 0
    top_k: int = 0
    moe_every: int = 0
    pooling: str = "cls"          # cls | mean | last | tokens (one output row per token: ColBERT mode)
    normalize: bool = True
    head: str = "none"            # none | classifier
    n_labels: int = 0
    label_scores: bool = False    # classifier head: softmax (sigmoid for one label) applied on the device
    weight_format: str = "bf16"
    weight_dtype: str = "bf16"    # storage precision the oracle sees: "fp32" or "bf16"
    max_len: int = 512            # longest sequence the model accepts (tokens)

    @property
    def out_dim(self) -> int:
        return self.n_labels if self.head == "classifier" else self.hidden


# -- the five named configurations ------------------------------------------------------
BGE_SMALL = ModelSpec(name="bge-small-shape", arch="bert", n_layers=12, hidden=384, n_heads=12, n_kv_heads=12,
                      head_dim=32, ffn=1536, vocab=30522, max_pos=512, type_vocab=2, pooling="cls",
                      weight_dtype="fp32")
BERT_LARGE = ModelSpec(name="bert-large-shape", arch="bert", n_layers=24, hidden=1024, n_heads=16, n_kv_heads=16,
                       head_dim=64, ffn=4096, vocab=30522, max_pos=512, type_vocab=2, pooling="mean")
XLMR_LARGE_RERANK = ModelSpec(name="xlmr-large-reranker-shape", arch="xlmr", n_layers=24, hidden=1024, n_heads=16,
                              n_kv_heads=16, head_dim=64, ffn=4096, vocab=250002, max_pos=514, type_vocab=1,
                              pos_offset=2, norm_eps=1e-5, pooling="cls", normalize=False, head="classifier",
                              n_labels=1)

MOE_ENCODER = ModelSpec(name="moe-encoder-shape", arch="moe", n_layers=12, hidden=768, n_heads=12, n_kv_heads=12,
                        head_dim=64, ffn=3072, vocab=250048, max_pos=512, type_vocab=1, pooling="mean",
                        n_experts=8, top_k=2, moe_every=2, weight_format="mxfp8")
QWEN2_7B = ModelSpec(name="qwen2-7b-shape", arch="decoder", n_layers=28, hidden=3584, n_heads=28, n_kv_heads=4,
                     head_dim=128, ffn=18944, vocab=151646, max_pos=2048, type_vocab=0, norm_eps=1e-6,
                     rope_theta=1e6, pooling="last", max_len=2048, weight_format="nvfp4")

SPECS: Dict[str, ModelSpec] = {"c1": BGE_SMALL, "c2": BERT_LARGE, "c3": XLMR_LARGE_RERANK, "c4": MOE_ENCODER,
                               "c5": QWEN2_7B}
SEEDS = {"c1": (1001, 2001, 3001), "c2": (1002, 2002, 3002), "c3": (1003, 2003, 3003), "c4": (1004, 2004, 3004),
         "c5": (1005, 2005, 3005)}


def is_moe_layer(spec: "ModelSpec", l: int) -> bool:
    return spec.arch == "moe" and spec.moe_every > 0 and l % spec.moe_every == spec.moe_every - 1


def tiny_spec(arch: str = "bert", **kw) -> ModelSpec:
    """A two-layer model for fast parity tests."""
    base = dict(name=f"tiny-{arch}", arch=arch, n_layers=2, hidden=128, n_heads=4, n_kv_heads=4, head_dim=32,
                ffn=256, vocab=1000, max_pos=160, type_vocab=2, pooling="mean")
    if arch == "xlmr":
        base.update(type_vocab=1, pos_offset=2, norm_eps=1e-5, pooling="cls", normalize=False, head="classifier",
                    n_labels=1)
    if arch == "moe":
        base.update(hidden=128, n_heads=2, n_kv_heads=2, head_dim=64, ffn=256, type_vocab=1, n_experts=8, top_k=2,
                    moe_every=2, n_layers=4)
    if arch == "decoder":
        base.update(hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=384, type_vocab=0, norm_eps=1e-6,
                    rope_theta=1e6, pooling="last", max_pos=320, max_len=320)
    base.update(kw)
    return ModelSpec(**base)


# -- weights ------------------------------------------------------------------------------
def init_weights(spec: ModelSpec, seed: int, perturb: bool = False) -> Dict[str, torch.Tensor]:
    """fp32 master weights under the runtime's tensor names.

    ``perturb=False``: matrices and tables N(0, 0.02), biases 0, norm gains 1 (the named
    configurations). ``perturb=True`` also draws biases and norm parameters, so that tests
    exercise every operand.
    """
    g = torch.Generator().manual_seed(seed)
    H, F = spec.hidden, spec.ffn
    QKV = (spec.n_heads + 2 * spec.n_kv_heads) * spec.head_dim

    def mat(*shape):
        return torch.empty(*shape, dtype=torch.float32).normal_(0.0, 0.02, generator=g)

    def bias(n):
        return mat(n) if perturb else torch.zeros(n)

    def gain(n):
        return 1.0 + mat(n) * 5 if perturb else torch.ones(n)

    w: Dict[str, torch.Tensor] = {}
    w["emb.word"] = mat(spec.vocab, H)
    if spec.arch == "decoder":
        # Qwen2 layout: q/k/v carry biases, o / gate / up / down do not; RMSNorm gains only
        for l in range(spec.n_layers):
            p = f"layer.{l}."
            w[p + "ln1.g"] = gain(H)
            w[p + "qkv.w"], w[p + "qkv.b"] = mat(QKV, H), bias(QKV)
            w[p + "o.w"] = mat(H, spec.n_heads * spec.head_dim)
            w[p + "ln2.g"] = gain(H)
            w[p + "gate.w"], w[p + "up.w"] = mat(F, H), mat(F, H)
            w[p + "down.w"] = mat(H, F)
        w["norm.g"] = gain(H)
        return w
    w["emb.pos"] = mat(spec.max_pos, H)
    if spec.type_vocab > 0:
        w["emb.type"] = mat(spec.type_vocab, H)
    w["emb.ln.g"], w["emb.ln.b"] = gain(H), bias(H)
    for l in range(spec.n_layers):
        p = f"layer.{l}."
        w[p + "qkv.w"], w[p + "qkv.b"] = mat(QKV, H), bias(QKV)
        w[p + "o.w"], w[p + "o.b"] = mat(H, spec.n_heads * spec.head_dim), bias(H)
        w[p + "ln1.g"], w[p + "ln1.b"] = gain(H), bias(H)
        if is_moe_layer(spec, l):
            # router in fp32; the experts' matrices stacked along the rows: expert e owns rows [e*F, (e+1)*F)
            E = spec.n_experts
            w[p + "router.w"], w[p + "router.b"] = mat(E, H), bias(E)
            w[p + "experts.ffn1.w"], w[p + "experts.ffn1.b"] = mat(E * F, H), bias(E * F)
            w[p + "experts.ffn2.w"], w[p + "experts.ffn2.b"] = mat(E * H, F), bias(E * H)
        else:
            w[p + "ffn1.w"], w[p + "ffn1.b"] = mat(F, H), bias(F)
            w[p + "ffn2.w"], w[p + "ffn2.b"] = mat(H, F), bias(H)
        w[p + "ln2.g"], w[p + "ln2.b"] = gain(H), bias(H)
    if spec.head == "classifier":
        w["head.dense.w"], w["head.dense.b"] = mat(H, H), bias(H)
        w["head.out.w"], w["head.out.b"] = mat(spec.n_labels, H), bias(spec.n_labels)
    return w


def is_matrix(name: str) -> bool:
    """Stored in bf16 by the runtime (the router stays fp32)."""
    if name.endswith("router.w"):
        return False
    return name.endswith(".w") or name in ("emb.word", "emb.pos", "emb.type")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[F, H] gate and up matrices -> one [2F, H] matrix in blocks of ``block`` gate rows followed by
    the ``block`` up rows of the same output columns (the layout the fused SwiGLU epilogue reads)."""
    F, H = gate.shape
    assert F % block == 0 and up.shape == gate.shape
    g = gate.reshape(F // block, block, H)
    u = up.reshape(F // block, block, H)
    return torch.stack([g, u], dim=1).reshape(2 * F, H).contiguous()


def runtime_tensors(master: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """What the CUDA runtime loads: matrices and tables in bf16, vectors in fp32; the decoder's
    gate and up projections fused block-interleaved into ``gu.w``."""
    out: Dict[str, torch.Tensor] = {}
    for k, v in master.items():
        if k.endswith("gate.w"):
            out[k[:-6] + "gu.w"] = interleave_gate_up(v, master[k[:-6] + "up.w"]).to(torch.bfloat16)
        elif k.endswith("up.w"):
            continue
        else:
            out[k] = v.to(torch.bfloat16) if is_matrix(k) else v.float()
    return out


def oracle_tensors(spec: ModelSpec, master: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """What the fp32 oracle computes with: the storage precision of the configuration
    (bf16-rounded values widened back to fp32, or the fp32 masters)."""
    if spec.weight_dtype == "fp32":
        return {k: v.float() for k, v in master.items()}
    return {k: (v.to(torch.bfloat16).float() if is_matrix(k) else v.float()) for k, v in master.items()}


# -- synthetic batches ----------------------------------------------------------------------
@dataclass
class Batch:
    input_ids: np.ndarray              # int32 [n_tokens]
    cu_seqlens: np.ndarray             # int32 [n_seqs + 1]
    token_type_ids: Optional[np.ndarray] = None

    @property
    def n_seqs(self) -> int:
        return len(self.cu_seqlens) - 1

    @property
    def n_tokens(self) -> int:
        return int(self.cu_seqlens[-1])

    @property
    def lengths(self) -> np.ndarray:
        return np.diff(self.cu_seqlens)

    def sequences(self) -> List[np.ndarray]:
        return [self.input_ids[self.cu_seqlens[i]:self.cu_seqlens[i + 1]] for i in range(self.n_seqs)]


def pack(seqs: List[np.ndarray], types: Optional[List[np.ndarray]] = None) -> Batch:
    """Ragged packing without padding, in the order given (the batcher's order)."""
    lens = np.array([len(s) for s in seqs], dtype=np.int64)
    cu = np.zeros(len(seqs) + 1, dtype=np.int32)
    np.cumsum(lens, out=cu[1:])
    ids = np.concatenate(seqs).astype(np.int32) if seqs else np.zeros(0, np.int32)
    tt = np.concatenate(types).astype(np.int32) if types is not None and seqs else None
    return Batch(ids, cu, tt)


def synth_lengths(cfg: str, n_seqs: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    if cfg == "c1":
        return rng.integers(16, 513, size=n_seqs)
    if cfg == "c2":
        z = rng.standard_normal(n_seqs)
        return np.clip(np.rint(np.exp(np.log(128.0) + 0.8 * z)), 8, 512).astype(np.int64)
    raise KeyError(cfg)


def synth_batch(cfg: str, n_seqs: Optional[int] = None, seed_offset: int = 0) -> Batch:
    """Seeded synthetic batch of a named configuration (``seed_offset`` gives other draws of
    the same distribution, e.g. one per rank)."""
    len_seed, id_seed, _ = SEEDS[cfg]
    len_seed += 7919 * seed_offset
    id_seed += 7919 * seed_offset
    rng = np.random.default_rng(id_seed)
    if cfg in ("c1", "c2"):
        n = n_seqs if n_seqs is not None else (32 if cfg == "c1" else 1024)
        lens = synth_lengths(cfg, n, len_seed)
        seqs = []
        for L in lens:
            s = rng.integers(1000, 30522, size=int(L))
            s[0] = 101  # CLS
            seqs.append(s)
        return pack(seqs)
    if cfg == "c4":
        n = n_seqs if n_seqs is not None else 8192
        lens = np.random.default_rng(len_seed).integers(16, 513, size=n)
        return pack([rng.integers(1000, 250048, size=int(L)) for L in lens])
    if cfg == "c5":
        n = n_seqs if n_seqs is not None else 512
        lens = np.random.default_rng(len_seed).integers(32, 2049, size=n)
        return pack([rng.integers(1000, 151646, size=int(L)) for L in lens])
    if cfg == "c3":
        n = n_seqs if n_seqs is not None else 2048
        lrng = np.random.default_rng(len_seed)
        q = lrng.integers(8, 65, size=n)
        d = lrng.integers(64, 449, size=n)
        seqs = []
        for qi, di in zip(q, d):
            di = min(int(di), 512 - 4 - int(qi))  # truncate the document
            s = np.concatenate([[0], rng.integers(1000, 250002, size=int(qi)), [2, 2],
                                rng.integers(1000, 250002, size=di), [2]])
            seqs.append(s)
        return pack(seqs)
    raise KeyError(cfg)


def random_batch(spec: ModelSpec, lengths, seed: int, with_types: bool = False) -> Batch:
    rng = np.random.default_rng(seed)
    seqs = [rng.integers(0, spec.vocab, size=int(L)) for L in lengths]
    types = None
    if with_types and spec.type_vocab > 1:
        types = [(np.arange(int(L)) >= int(L) // 2).astype(np.int64) for L in lengths]
    return pack(seqs, types)
