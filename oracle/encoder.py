"""Plain-torch fp32 restatement of the post-LayerNorm encoder forward (test infrastructure).

The reference computes this step by calling third-party code:
``SentenceTransformer.forward`` at infinity_emb/transformer/embedder/sentence_transformer.py:124
and ``AutoModelForSequenceClassification`` at infinity_emb/transformer/crossencoder/torch.py:106,
i.e. ``transformers`` ``BertModel`` / ``XLMRobertaForSequenceClassification`` (locked 4.47.0;
not in the reference tree). This file restates that published algorithm -- embeddings
(word + token-type + position, LayerNorm), N x [self-attention, output dense + residual +
LayerNorm, GELU feed-forward + residual + LayerNorm], then either pooling + L2 normalise
(infinity_emb/transformer/utils_optimum.py:29-47, sentence_transformer.py:142-145) or the
classification head ``out_proj(tanh(dense(h[:, 0])))`` -- on PADDED, length-sorted batches,
which is how the reference's CPU path runs it (fp32 on CPU: infinity_emb/inference/loading_strategy.py:87-88;
padding: crossencoder/torch.py:95-97). ``tests/test_oracle.py`` checks it against the local
``transformers`` classes loaded with the same weights.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch
import torch.nn.functional as F

from . import pooling as P


def _ln(x, g, b, eps):
    return F.layer_norm(x, (x.shape[-1],), g, b, eps)


@torch.no_grad()
def encoder_hidden(spec, W: Dict[str, torch.Tensor], ids: torch.Tensor, mask: torch.Tensor,
                   types: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ids, mask, types: [B, L] (right padded). Returns the last hidden state [B, L, H] in fp32."""
    B, L = ids.shape
    H, nh, d = spec.hidden, spec.n_heads, spec.head_dim
    pos = torch.arange(L).unsqueeze(0).expand(B, L) + spec.pos_offset
    if spec.arch == "xlmr":
        # padded positions take the padding index (pos_offset - 1), as create_position_ids_from_input_ids does
        pos = torch.where(mask.bool(), pos, torch.full_like(pos, spec.pos_offset - 1))
    x = W["emb.word"][ids]
    if spec.type_vocab > 0:
        tt = types if types is not None else torch.zeros_like(ids)
        x = x + W["emb.type"][tt]
    x = x + W["emb.pos"][pos]
    x = _ln(x, W["emb.ln.g"], W["emb.ln.b"], spec.norm_eps)
    neg = torch.finfo(torch.float32).min
    add_mask = (1.0 - mask.float())[:, None, None, :] * neg
    for l in range(spec.n_layers):
        p = f"layer.{l}."
        qkv = x @ W[p + "qkv.w"].t() + W[p + "qkv.b"]
        q, k, v = qkv.split(H, dim=-1)
        q = q.view(B, L, nh, d).transpose(1, 2)
        k = k.view(B, L, nh, d).transpose(1, 2)
        v = v.view(B, L, nh, d).transpose(1, 2)
        s = q @ k.transpose(-1, -2) / math.sqrt(d) + add_mask
        a = torch.softmax(s, dim=-1) @ v
        a = a.transpose(1, 2).reshape(B, L, H)
        x = _ln(x + a @ W[p + "o.w"].t() + W[p + "o.b"], W[p + "ln1.g"], W[p + "ln1.b"], spec.norm_eps)
        if spec.arch == "moe" and spec.moe_every > 0 and l % spec.moe_every == spec.moe_every - 1:
            y = moe_ffn(spec, W, p, x)
        else:
            y = F.gelu(x @ W[p + "ffn1.w"].t() + W[p + "ffn1.b"]) @ W[p + "ffn2.w"].t() + W[p + "ffn2.b"]
        x = _ln(x + y, W[p + "ln2.g"], W[p + "ln2.b"], spec.norm_eps)
    return x


def moe_route(x: np.ndarray, wr: np.ndarray, br: np.ndarray, top_k: int):
    """Router of the mixture-of-experts layers: fp32 logits, softmax over all experts, top_k
    experts per token with ties going to the lower index, gate = softmax probability of the
    chosen expert, not renormalised. x [T, H] -> (idx int32 [T, k], gate float32 [T, k], probs)."""
    logits = x.astype(np.float32) @ wr.astype(np.float32).T + br.astype(np.float32)
    z = np.exp(logits - logits.max(axis=1, keepdims=True))
    probs = (z / z.sum(axis=1, keepdims=True)).astype(np.float32)
    work = probs.copy()
    idx = np.zeros((x.shape[0], top_k), dtype=np.int32)
    gate = np.zeros((x.shape[0], top_k), dtype=np.float32)
    rows = np.arange(x.shape[0])
    for k in range(top_k):
        best = np.argmax(work, axis=1)  # first occurrence = lowest index on ties
        idx[:, k] = best
        gate[:, k] = probs[rows, best]
        work[rows, best] = -1.0
    return idx, gate, probs


def moe_ffn(spec, W, p: str, x: torch.Tensor) -> torch.Tensor:
    """sum_k gate_k * FFN_{e_k}(x), FFN_e = ffn2_e(gelu(ffn1_e(x))); x [B, L, H]. This block has no
    third-party or reference implementation to follow: it is written from the benchmark
    configuration's description (8 GELU experts of width F, top-2 softmax routing)."""
    B, L, H = x.shape
    F_, E = spec.ffn, spec.n_experts
    flat = x.reshape(B * L, H)
    idx, gate, _ = moe_route(flat.numpy(), W[p + "router.w"].numpy(), W[p + "router.b"].numpy(), spec.top_k)
    out = torch.zeros_like(flat)
    w1, b1 = W[p + "experts.ffn1.w"], W[p + "experts.ffn1.b"]
    w2, b2 = W[p + "experts.ffn2.w"], W[p + "experts.ffn2.b"]
    for e in range(E):
        for k in range(spec.top_k):
            sel = np.nonzero(idx[:, k] == e)[0]
            if len(sel) == 0:
                continue
            xe = flat[sel]
            he = F.gelu(xe @ w1[e * F_:(e + 1) * F_].t() + b1[e * F_:(e + 1) * F_])
            ye = he @ w2[e * H:(e + 1) * H].t() + b2[e * H:(e + 1) * H]
            out[sel] += torch.from_numpy(gate[sel, k])[:, None] * ye
    return out.reshape(B, L, H)


def pad_batch(seqs, types=None, pad_id: int = 0):
    B, L = len(seqs), max(len(s) for s in seqs)
    ids = torch.full((B, L), pad_id, dtype=torch.long)
    mask = torch.zeros((B, L), dtype=torch.long)
    tt = torch.zeros((B, L), dtype=torch.long)
    for i, s in enumerate(seqs):
        ids[i, : len(s)] = torch.as_tensor(np.asarray(s), dtype=torch.long)
        mask[i, : len(s)] = 1
        if types is not None:
            tt[i, : len(s)] = torch.as_tensor(np.asarray(types[i]), dtype=torch.long)
    return ids, mask, tt


def label_scores(logits: np.ndarray) -> np.ndarray:
    """Raw logits [B, n_labels] -> scores: softmax over the labels, the logistic function for a
    single-output head -- what the text-classification pipeline behind the reference's classifier
    applies (infinity_emb/transformer/classifier/torch.py:38-46, 74-80) and what its batcher applies to
    rerank logits (infinity_emb/inference/batch_handler.py:207-210). float64 arithmetic, float32 result."""
    x = np.asarray(logits, dtype=np.float64)
    if x.shape[1] == 1:
        return (1.0 / (1.0 + np.exp(-x))).astype(np.float32)
    e = np.exp(x - x.max(axis=1, keepdims=True))
    return (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


@torch.no_grad()
def forward_padded(spec, W, ids, mask, types=None) -> np.ndarray:
    """One padded batch -> [B, out_dim] float32 (embeddings, or raw logits for classifier heads)."""
    h = encoder_hidden(spec, W, ids, mask, types)
    if spec.head == "classifier":
        c = torch.tanh(h[:, 0] @ W["head.dense.w"].t() + W["head.dense.b"])
        logits = (c @ W["head.out.w"].t() + W["head.out.b"]).float().numpy()
        return label_scores(logits) if getattr(spec, "label_scores", False) else logits
    if spec.pooling == "tokens":
        raise ValueError("token-level outputs are ragged: use forward_tokens")
    pooled = P.POOLERS[spec.pooling](h.numpy(), mask.numpy())
    pooled = pooled.astype(np.float32)  # sentence_transformer.py:142: embeddings go to fp32 first
    if spec.normalize:
        pooled = P.normalize(pooled)
    return pooled.astype(np.float32)


@torch.no_grad()
def forward_tokens(spec, W, batch, batch_size: int = 32) -> np.ndarray:
    """ColBERT mode (sentence_transformer.py:125-131, 146-155): the final hidden state of every real
    token, float32, padded rows dropped; returned packed as [n_tokens, hidden] in batch order
    (sequence i owns rows cu_seqlens[i] .. cu_seqlens[i+1]-1). L2-normalised per token only if
    ``spec.normalize`` (the reference switches normalisation off in this mode)."""
    seqs = batch.sequences()
    cu = batch.cu_seqlens
    types = None
    if batch.token_type_ids is not None:
        types = [batch.token_type_ids[cu[i]: cu[i + 1]] for i in range(batch.n_seqs)]
    out = np.zeros((int(cu[-1]), spec.hidden), dtype=np.float32)
    pad_id = 1 if spec.arch == "xlmr" else 0
    for s in range(0, batch.n_seqs, batch_size):
        idx = list(range(s, min(s + batch_size, batch.n_seqs)))
        ids, mask, tt = pad_batch([seqs[i] for i in idx], None if types is None else [types[i] for i in idx], pad_id)
        h = encoder_hidden(spec, W, ids, mask, tt if types is not None else None).float().numpy()
        for k, i in enumerate(idx):
            rows = h[k, : len(seqs[i])]
            out[cu[i]: cu[i + 1]] = P.normalize(rows) if spec.normalize else rows
    return out


def forward_batch(spec, W, batch, batch_size: int = 32, sort: bool = True) -> np.ndarray:
    """A ragged batch through the reference's CPU recipe: (optionally) sort by length, cut
    into padded sub-batches of ``batch_size`` (EngineArgs.batch_size default 32), run each,
    and return rows in the original order."""
    seqs = batch.sequences()
    types = None
    if batch.token_type_ids is not None:
        cu = batch.cu_seqlens
        types = [batch.token_type_ids[cu[i]: cu[i + 1]] for i in range(batch.n_seqs)]
    order = np.argsort(batch.lengths, kind="stable") if sort else np.arange(batch.n_seqs)
    out = np.zeros((batch.n_seqs, spec.out_dim), dtype=np.float32)
    pad_id = 1 if spec.arch == "xlmr" else 0
    for s in range(0, batch.n_seqs, batch_size):
        idx = order[s: s + batch_size]
        ids, mask, tt = pad_batch([seqs[i] for i in idx], [types[i] for i in idx] if types else None, pad_id)
        out[idx] = forward_padded(spec, W, ids, mask, tt if types else None)
    return out
