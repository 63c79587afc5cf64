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
