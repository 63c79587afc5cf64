"""Plain-torch fp32 restatement of the decoder-style embedder forward (test infrastructure).

Decoder embedders reach the reference through the same call as the encoders
(``SentenceTransformer.forward`` at infinity_emb/transformer/embedder/sentence_transformer.py:124),
which runs ``transformers`` ``Qwen2Model`` (not in the reference tree). This file restates that
published algorithm: token embedding, N x [RMSNorm, q/k/v projections with bias, rotary
position embedding (rotate-half convention, theta 1e6), causal grouped-query attention, output
projection, residual, RMSNorm, SwiGLU feed-forward, residual], final RMSNorm; then last-token
pooling and L2 normalisation (oracle/pooling.py). Padded batches, fp32, as the reference's CPU
path runs it. ``tests/test_oracle.py`` checks it against the local ``transformers.Qwen2Model``.
"""
from __future__ import annotations

import math
from typing import Dict

import numpy as np
import torch
import torch.nn.functional as F

from . import pooling as P


def _rms(x, g, eps):
    var = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * g


def _rope_tables(spec, L):
    d = spec.head_dim
    inv_freq = 1.0 / (spec.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    freqs = torch.arange(L).float()[:, None] * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([-x2, x1], dim=-1)


@torch.no_grad()
def decoder_hidden(spec, W: Dict[str, torch.Tensor], ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """ids, mask: [B, L] right padded. Returns the final normalised hidden state [B, L, H]."""
    B, L = ids.shape
    H, nh, nkv, d = spec.hidden, spec.n_heads, spec.n_kv_heads, spec.head_dim
    cos, sin = _rope_tables(spec, L)
    neg = torch.finfo(torch.float32).min
    causal = torch.ones(L, L).triu(1)[None, None] * neg
    pad = (1.0 - mask.float())[:, None, None, :] * neg
    add_mask = torch.clamp(causal + pad, min=neg)
    h = W["emb.word"][ids]
    for l in range(spec.n_layers):
        p = f"layer.{l}."
        x = _rms(h, W[p + "ln1.g"], spec.norm_eps)
        qkv = x @ W[p + "qkv.w"].t() + W[p + "qkv.b"]
        q, k, v = qkv.split([nh * d, nkv * d, nkv * d], dim=-1)
        q = q.view(B, L, nh, d).transpose(1, 2)
        k = k.view(B, L, nkv, d).transpose(1, 2)
        v = v.view(B, L, nkv, d).transpose(1, 2)
        q = q * cos + _rotate_half(q) * sin
        k = k * cos + _rotate_half(k) * sin
        k = k.repeat_interleave(nh // nkv, dim=1)
        v = v.repeat_interleave(nh // nkv, dim=1)
        s = q @ k.transpose(-1, -2) / math.sqrt(d) + add_mask
        a = (torch.softmax(s, dim=-1) @ v).transpose(1, 2).reshape(B, L, nh * d)
        h = h + a @ W[p + "o.w"].t()
        x = _rms(h, W[p + "ln2.g"], spec.norm_eps)
        f = F.silu(x @ W[p + "gate.w"].t()) * (x @ W[p + "up.w"].t())
        h = h + f @ W[p + "down.w"].t()
    return _rms(h, W["norm.g"], spec.norm_eps)


@torch.no_grad()
def forward_padded(spec, W, ids, mask) -> np.ndarray:
    h = decoder_hidden(spec, W, ids, mask)
    pooled = P.POOLERS[spec.pooling](h.numpy(), mask.numpy()).astype(np.float32)
    if spec.normalize:
        pooled = P.normalize(pooled)
    return pooled.astype(np.float32)


def forward_batch(spec, W, batch, batch_size: int = 32, sort: bool = True) -> np.ndarray:
    from .encoder import pad_batch
    seqs = batch.sequences()
    order = np.argsort(batch.lengths, kind="stable") if sort else np.arange(batch.n_seqs)
    out = np.zeros((batch.n_seqs, spec.out_dim), dtype=np.float32)
    for s in range(0, batch.n_seqs, batch_size):
        idx = order[s: s + batch_size]
        ids, mask, _ = pad_batch([seqs[i] for i in idx])
        out[idx] = forward_padded(spec, W, ids, mask)
    return out
