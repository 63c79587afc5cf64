"""numpy / torch statement of the NVFP4 and MXFP8 weight quantisers (test infrastructure).

The reference has no block-format quantiser (its hook, ``quant_interface`` at
infinity_emb/transformer/quantization/interface.py:28-70, offers int8 and fp8 only), so these
follow the published formats: NVFP4 = e2m1 elements in 16-element blocks with an e4m3 block
scale and an fp32 tensor scale; MXFP8 = OCP Microscaling, e4m3 elements in 32-element blocks
with an e8m0 (power of two) block scale, shared exponent floor(log2(amax)) - emax(e4m3) = - 8.
All arithmetic is fp32 with round-to-nearest-even and saturation, in exactly the order the CUDA
kernels use (infinity_b200/csrc/quant.cu), so the two agree bit for bit.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np
import torch

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def _e2m1_codes(v: np.ndarray) -> np.ndarray:
    """fp32 -> 4-bit e2m1 code (sign in bit 3), round to nearest even, saturating at 6."""
    a = np.abs(v)
    # midpoints between neighbours; on a tie the code with an even low bit wins (0, 1, 2, 4)
    code = np.zeros(a.shape, dtype=np.uint8)
    code[a > 0.25] = 1
    code[a >= 0.75] = 2
    code[a > 1.25] = 3
    code[a >= 1.75] = 4
    code[a > 2.5] = 5
    code[a >= 3.5] = 6
    code[a > 5.0] = 7
    sign = (np.signbit(v)).astype(np.uint8) << 3
    return code | sign


def _e4m3_round(x: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """fp32 (already clamped to <= 448) -> (e4m3 bits, value as fp32)."""
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.float8_e4m3fn)
    return t.view(torch.uint8).numpy(), t.float().numpy()


def quantize_nvfp4(w: np.ndarray):
    """w fp32 [rows, K] (K % 16 == 0) -> (packed uint8 [rows, K/2], scales uint8 [rows, K/16], gs float32)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, K = w.shape
    amax_t = np.float32(np.abs(w).max())
    gs = np.float32(2688.0) / amax_t if amax_t > 0 else np.float32(1.0)
    blocks = w.reshape(rows, K // 16, 16)
    amax_b = np.abs(blocks).max(axis=2).astype(np.float32)
    s_enc = np.minimum((amax_b / np.float32(6.0)).astype(np.float32) * gs, np.float32(448.0)).astype(np.float32)
    s_bits, s_val = _e4m3_round(s_enc)
    s_dec = (s_val / gs).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = np.where(s_dec[..., None] > 0, blocks / s_dec[..., None], np.float32(0.0)).astype(np.float32)
    codes = _e2m1_codes(v).reshape(rows, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, s_bits.reshape(rows, K // 16), np.float32(gs)


def dequantize_nvfp4(packed: np.ndarray, scales: np.ndarray, gs: float, with_tensor_scale: bool = True) -> np.ndarray:
    rows = packed.shape[0]
    codes = np.empty((rows, packed.shape[1] * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 15
    codes[:, 1::2] = packed >> 4
    vals = E2M1_VALUES[codes & 7] * np.where(codes & 8, np.float32(-1), np.float32(1))
    s = torch.from_numpy(np.ascontiguousarray(scales)).view(torch.float8_e4m3fn).float().numpy()
    out = (vals.reshape(rows, -1, 16) * s[..., None]).astype(np.float32)
    if with_tensor_scale:
        out = (out / np.float32(gs)).astype(np.float32)
    return out.reshape(rows, -1)


def quantize_mxfp8(w: np.ndarray):
    """w fp32 [rows, K] (K % 32 == 0) -> (e4m3 bits uint8 [rows, K], e8m0 scales uint8 [rows, K/32])."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, K = w.shape
    blocks = w.reshape(rows, K // 32, 32)
    amax = np.abs(blocks).max(axis=2).astype(np.float32)
    _, ex = np.frexp(amax)  # amax = m * 2^ex with m in [0.5, 1): floor(log2(amax)) = ex - 1
    e = np.clip(ex.astype(np.int32) - 1 - 8, -127, 127)
    e = np.where(amax > 0, e, -127)
    inv = np.where(e == -127, np.float32(0.0), np.exp2(-e.astype(np.float32))).astype(np.float32)
    v = np.clip((blocks * inv[..., None]).astype(np.float32), -448.0, 448.0)
    bits, _ = _e4m3_round(v)
    return bits.reshape(rows, K), (e + 127).astype(np.uint8)


def dequantize_mxfp8(bits: np.ndarray, scales: np.ndarray) -> np.ndarray:
    rows, K = bits.shape
    vals = torch.from_numpy(np.ascontiguousarray(bits)).view(torch.float8_e4m3fn).float().numpy()
    s = np.exp2(scales.astype(np.float32) - 127.0).astype(np.float32)
    return (vals.reshape(rows, K // 32, 32) * s[..., None]).astype(np.float32).reshape(rows, K)
