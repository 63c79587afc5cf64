"""Weight file shared by the CUDA runtime and the oracle.

Layout (little endian): magic ``B2EW0001``, u32 n_tensors, u32 reserved, u64 data_offset,
n_tensors entries ``{char name[64]; u32 dtype; u32 ndim; u64 dims[4]; u64 offset; u64 nbytes}``
and a data region whose tensors start on 256-byte boundaries. dtype: 0 fp32, 1 bf16,
2 u8, 3 i32. Matrices are stored the way ``torch.nn.Linear`` holds them, ``[out, in]``.

Tensor names of the encoder family:
``emb.word [V,H]``, ``emb.pos [P,H]``, ``emb.type [Tv,H]`` (bf16), ``emb.ln.g/b [H]`` (fp32),
per layer ``layer.{l}.qkv.w [3H,H]`` (query rows, then key rows, then value rows), ``qkv.b``,
``o.w``, ``o.b``, ``ln1.g/b``, ``ffn1.w [F,H]``, ``ffn1.b``, ``ffn2.w [H,F]``, ``ffn2.b``, ``ln2.g/b``,
and for classifier heads ``head.dense.w [H,H]``, ``head.dense.b``, ``head.out.w [n_labels,H]``, ``head.out.b``.
"""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Dict

import numpy as np
import torch

MAGIC = b"B2EW0001"
_ENTRY = struct.Struct("<64sII4QQQ")
_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.uint8: 2, torch.int32: 3}
_DTYPES_INV = {v: k for k, v in _DTYPES.items()}


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def save_weights(path: str | Path, tensors: Dict[str, torch.Tensor]) -> None:
    """Writes ``tensors`` (name -> fp32 / bf16 / uint8 / int32 tensor) to ``path``."""
    names = list(tensors.keys())
    header_size = len(MAGIC) + 4 + 4 + 8 + _ENTRY.size * len(names)
    data_offset = (header_size + 255) // 256 * 256
    entries, blobs, off = [], [], 0
    for name in names:
        t = tensors[name]
        if t.dtype not in _DTYPES:
            raise TypeError(f"{name}: dtype {t.dtype} not storable")
        if t.dim() > 4 or len(name.encode()) > 63:
            raise ValueError(f"{name}: at most 4 dims and 63 name bytes")
        raw = _raw_bytes(t)
        dims = list(t.shape) + [1] * (4 - t.dim())
        entries.append(_ENTRY.pack(name.encode(), _DTYPES[t.dtype], t.dim(), *dims, off, len(raw)))
        blobs.append((off, raw))
        off = (off + len(raw) + 255) // 256 * 256
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<IIQ", len(names), 0, data_offset))
        for e in entries:
            f.write(e)
        f.write(b"\0" * (data_offset - header_size))
        pos = 0
        for o, raw in blobs:
            if o > pos:
                f.write(b"\0" * (o - pos))
            f.write(raw)
            pos = o + len(raw)


def load_weights(path: str | Path) -> Dict[str, torch.Tensor]:
    """Reads a weight file back into torch tensors (used by the oracle and by tests)."""
    buf = Path(path).read_bytes()
    if buf[:8] != MAGIC:
        raise ValueError(f"{path}: not a b200emb weight file")
    n, _, data_offset = struct.unpack_from("<IIQ", buf, 8)
    out: Dict[str, torch.Tensor] = {}
    for i in range(n):
        name, dt, ndim, d0, d1, d2, d3, off, nbytes = _ENTRY.unpack_from(buf, 24 + i * _ENTRY.size)
        name = name.split(b"\0", 1)[0].decode()
        shape = [d0, d1, d2, d3][:ndim]
        raw = buf[data_offset + off: data_offset + off + nbytes]
        dtype = _DTYPES_INV[dt]
        if dtype == torch.bfloat16:
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.int16).copy()).view(torch.bfloat16)
        else:
            np_dt = {torch.float32: np.float32, torch.uint8: np.uint8, torch.int32: np.int32}[dtype]
            t = torch.from_numpy(np.frombuffer(raw, dtype=np_dt).copy())
        out[name] = t.reshape(shape)
    return out


class WeightFileReader:
    """Reads single tensors of a weight file on demand (the file is memory-mapped, nothing is read
    until a tensor is asked for): for tools that walk a large file one layer at a time."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        with open(self.path, "rb") as f:
            head = f.read(24)
            if head[:8] != MAGIC:
                raise ValueError(f"{path}: not a b200emb weight file")
            n, _, self._data_offset = struct.unpack_from("<IIQ", head, 8)
            table = f.read(_ENTRY.size * n)
        self.entries: Dict[str, tuple] = {}
        for i in range(n):
            name, dt, ndim, d0, d1, d2, d3, off, nbytes = _ENTRY.unpack_from(table, i * _ENTRY.size)
            self.entries[name.split(b"\0", 1)[0].decode()] = (dt, [d0, d1, d2, d3][:ndim], off, nbytes)
        self._map = np.memmap(self.path, dtype=np.uint8, mode="r")

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def names(self):
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        dt, shape, off, nbytes = self.entries[name]
        raw = np.array(self._map[self._data_offset + off: self._data_offset + off + nbytes])
        dtype = _DTYPES_INV[dt]
        if dtype == torch.bfloat16:
            t = torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16)
        else:
            np_dt = {torch.float32: np.float32, torch.uint8: np.uint8, torch.int32: np.int32}[dtype]
            t = torch.from_numpy(raw.view(np_dt))
        return t.reshape(shape)


def quantize_weight_file(in_path: str | Path, out_path: str | Path, weight_format: str, device_id: int = 0) -> None:
    """Block-quantises the layer matrices of a bf16 weight file on the GPU (``b200emb_quantize_weights``)."""
    from . import _lib
    lib = _lib.load()
    _lib.check(lib.b200emb_quantize_weights(str(in_path).encode(), str(out_path).encode(), _lib.WFMT[weight_format],
                                            device_id))
