"""Test-only helpers shared by the GPU parity tests (they import the oracle)."""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from infinity_b200 import configs as cf
from infinity_b200 import weights as wt
from infinity_b200.engine import B200Model
from oracle import quant as Q


def cosines(a, b):
    return (a * b).sum(1) / (np.linalg.norm(a, axis=1) * np.linalg.norm(b, axis=1))


def deinterleave_gate_up(gu: torch.Tensor, block: int = 128):
    F2, H = gu.shape
    v = gu.reshape(F2 // (2 * block), 2, block, H)
    return v[:, 0].reshape(F2 // 2, H).contiguous(), v[:, 1].reshape(F2 // 2, H).contiguous()


def quantized_oracle_tensors(spec, master: Dict[str, torch.Tensor], fmt: str) -> Dict[str, torch.Tensor]:
    """fp32 weights the oracle computes with when the runtime loads block-quantised layer matrices:
    the same tensors the runtime quantises (fused qkv, block-interleaved gate/up), quantised and
    dequantised by the numpy statement, mapped back to the oracle's names."""
    rt = cf.runtime_tensors(master)
    has_experts = any(".experts." in k for k in rt)
    out: Dict[str, torch.Tensor] = {}
    for k, v in rt.items():
        block = 16 if fmt == "nvfp4" else 32
        sel = (k.startswith("layer.") and k.endswith(".w") and v.dim() == 2 and v.shape[1] % block == 0
               and (not has_experts or ".experts." in k))
        if sel:
            w = v.float().numpy()
            if fmt == "nvfp4":
                d = Q.dequantize_nvfp4(*Q.quantize_nvfp4(w))
            else:
                d = Q.dequantize_mxfp8(*Q.quantize_mxfp8(w))
            t = torch.from_numpy(d)
        else:
            t = v.float()
        if k.endswith("gu.w"):
            g, u = deinterleave_gate_up(t)
            out[k[:-4] + "gate.w"], out[k[:-4] + "up.w"] = g, u
        else:
            out[k] = t
    return out


def build_model(tmp_path, spec, seed, perturb, device_ids=(0,)):
    """Writes the seeded weights, (for block formats) quantises the file with the CUDA quantisers,
    loads it; returns the model and the fp32 tensors the oracle must use."""
    master = cf.init_weights(spec, seed, perturb=perturb)
    path = tmp_path / f"{spec.name}.b2ew"
    wt.save_weights(path, cf.runtime_tensors(master))
    if spec.weight_format != "bf16":
        qpath = tmp_path / f"{spec.name}.{spec.weight_format}.b2ew"
        wt.quantize_weight_file(path, qpath, spec.weight_format)
        return B200Model(spec, str(qpath), device_ids), quantized_oracle_tensors(spec, master, spec.weight_format)
    return B200Model(spec, str(path), device_ids), cf.oracle_tensors(spec, master)


def _e2m1_pair_table() -> np.ndarray:
    """byte -> the two e2m1 values it packs (low nibble = even element), as two fp16 in one uint32."""
    e2m1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float16)
    byte = np.arange(256)
    return np.stack([e2m1[byte & 15], e2m1[byte >> 4]], axis=1).view(np.uint32).reshape(256)


_E2M1_PAIRS = _e2m1_pair_table()


def fast_dequantize_nvfp4(packed: torch.Tensor, scales: torch.Tensor, gs: float) -> torch.Tensor:
    """oracle.quant.dequantize_nvfp4 for matrices of hundreds of millions of elements: one table
    look-up per byte, then the same two fp32 operations in the same order (value * block scale, / tensor
    scale), in place. The tests check it against the numpy statement before relying on it."""
    rows = packed.shape[0]
    halves = np.take(_E2M1_PAIRS, packed.numpy()).view(np.float16).reshape(rows, -1)
    vals = torch.from_numpy(halves).float().reshape(rows, -1, 16)
    vals.mul_(scales.view(torch.float8_e4m3fn).float()[..., None])
    vals.div_(np.float32(gs))
    return vals.reshape(rows, -1)


class StreamedDecoderWeights:
    """The oracle's weight mapping for a block-quantised decoder weight FILE, one tensor at a time:
    ``W[name]`` reads the stored bytes of that tensor, dequantises them (NVFP4) and returns fp32, so
    a 28-layer 7B model never sits in host memory in fp32. The file is what the runtime loads, so
    the oracle and the kernels compute with the same stored weights."""

    def __init__(self, path):
        self.reader = wt.WeightFileReader(path)
        self._gu = (None, None)

    def _matrix(self, name: str) -> torch.Tensor:
        r = self.reader
        if name + ".q" in r:
            gs = float(r.read(name + ".gs").reshape(-1)[0])
            return fast_dequantize_nvfp4(r.read(name + ".q"), r.read(name + ".s"), gs)
        return r.read(name).float()

    def __getitem__(self, name: str) -> torch.Tensor:
        if name.endswith("gate.w") or name.endswith("up.w"):
            base = name[: name.rfind(".", 0, len(name) - 2) + 1]  # "layer.L."
            if self._gu[0] != base:
                self._gu = (base, deinterleave_gate_up(self._matrix(base + "gu.w")))
            return self._gu[1][0 if name.endswith("gate.w") else 1]
        if name.endswith(".w") or name == "emb.word":
            return self._matrix(name)
        return self.reader.read(name).float()
