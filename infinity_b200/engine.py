"""Python owner of one ``b200emb_handle``: builds the model descriptor, keeps pinned host
buffers for results, and calls ``b200emb_forward`` through ctypes.

torch is used here only to own pinned host memory and (for the device-resident variant)
device buffers whose raw pointers cross the C ABI; no torch operator runs on the path.
"""
from __future__ import annotations

import ctypes as C
import os
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _lib
from .configs import Batch, ModelSpec


def make_desc(spec: ModelSpec, max_tokens: int = 0) -> _lib.ModelDesc:
    d = _lib.ModelDesc()
    d.abi_version = _lib.ABI_VERSION
    d.arch = _lib.ARCH[spec.arch]
    d.n_layers, d.hidden, d.n_heads, d.n_kv_heads = spec.n_layers, spec.hidden, spec.n_heads, spec.n_kv_heads
    d.head_dim, d.ffn, d.vocab, d.max_pos = spec.head_dim, spec.ffn, spec.vocab, spec.max_pos
    d.type_vocab, d.pos_offset = spec.type_vocab, spec.pos_offset
    d.norm_eps, d.rope_theta = spec.norm_eps, spec.rope_theta
    d.n_experts, d.top_k, d.moe_every = spec.n_experts, spec.top_k, spec.moe_every
    d.pooling = _lib.POOL[spec.pooling]
    d.normalize = 1 if spec.normalize else 0
    d.head = _lib.HEAD[spec.head]
    d.n_labels = spec.n_labels
    d.label_scores = 1 if spec.label_scores else 0
    d.weight_format = _lib.WFMT[spec.weight_format]
    d.max_tokens = max_tokens
    return d


def timing_dict(t: _lib.Timing) -> Dict:
    return {
        "n_devices": t.n_devices, "h2d_ms": t.h2d_ms, "kernels_ms": t.kernels_ms, "d2h_ms": t.d2h_ms,
        "total_ms": t.total_ms, "launches": t.launches, "gemm_flops": t.gemm_flops,
        "kclass_ms": {n: t.kclass_ms[i] for i, n in enumerate(_lib.KCLASS_NAMES) if t.kclass_launches[i]},
        "kclass_launches": {n: t.kclass_launches[i] for i, n in enumerate(_lib.KCLASS_NAMES) if t.kclass_launches[i]},
    }


class B200Model:
    """One model replica set (weights replicated on ``device_ids``) behind the C ABI."""

    def __init__(self, spec: ModelSpec, weight_path: str, device_ids: Sequence[int] = (0,), max_tokens: int = 0):
        self.spec = spec
        self._lib = _lib.load()
        self._handle = C.c_void_p()
        desc = make_desc(spec, max_tokens)
        ids = (C.c_int32 * len(device_ids))(*device_ids)
        _lib.check(self._lib.b200emb_create(C.byref(desc), str(weight_path).encode(), ids, len(device_ids),
                                            C.byref(self._handle)))
        self.device_ids = list(device_ids)
        self.last_timing: Optional[Dict] = None
        # per-replica counters (the reference exposes only wall-clock warm-up numbers and queue
        # statistics: abstract.py:228-250, infinity_server.py:189-214); B200EMB_TRACE=1 prints one line per call
        self.stats: Dict[str, float] = {"calls": 0, "sequences": 0, "tokens": 0, "total_ms": 0.0, "kernels_ms": 0.0,
                                        "h2d_ms": 0.0, "d2h_ms": 0.0, "launches": 0}
        self._trace = os.environ.get("B200EMB_TRACE", "0") not in ("", "0")

    def _account(self, n_seqs: int, n_tokens: int) -> None:
        t = self.last_timing
        st = self.stats
        st["calls"] += 1
        st["sequences"] += n_seqs
        st["tokens"] += n_tokens
        for k in ("total_ms", "kernels_ms", "h2d_ms", "d2h_ms", "launches"):
            st[k] += t[k]
        if self._trace:
            print(f"[b200emb] {n_seqs} seqs {n_tokens} tokens: h2d {t['h2d_ms']:.3f} ms, kernels {t['kernels_ms']:.3f} ms "
                  f"({t['launches']} launches), d2h {t['d2h_ms']:.3f} ms, total {t['total_ms']:.3f} ms", file=sys.stderr)

    def close(self) -> None:
        if getattr(self, "_handle", None) is not None and self._handle.value:
            self._lib.b200emb_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward_arrays(self, input_ids: np.ndarray, cu_seqlens: np.ndarray,
                       token_type_ids: Optional[np.ndarray] = None, out: Optional[np.ndarray] = None,
                       per_kernel: bool = False) -> np.ndarray:
        """Host arrays in, ``[n_seqs, out_dim]`` float32 out (row i = sequence i); with
        ``pooling == "tokens"`` the result is ``[n_tokens, out_dim]`` in packed token order."""
        ids = np.ascontiguousarray(input_ids, dtype=np.int32)
        cu = np.ascontiguousarray(cu_seqlens, dtype=np.int32)
        tt = None if token_type_ids is None else np.ascontiguousarray(token_type_ids, dtype=np.int32)
        n_seqs = len(cu) - 1
        n_tokens = int(len(ids))
        n_rows = n_tokens if self.spec.pooling == "tokens" else n_seqs
        if out is None:
            out = np.empty((n_rows, self.spec.out_dim), dtype=np.float32)
        assert out.dtype == np.float32 and out.flags.c_contiguous and out.shape == (n_rows, self.spec.out_dim)
        timing = _lib.Timing()
        timing.per_kernel = 1 if per_kernel else 0
        _lib.check(self._lib.b200emb_forward(
            self._handle, ids.ctypes.data, None if tt is None else tt.ctypes.data, cu.ctypes.data, n_seqs, n_tokens,
            out.ctypes.data, self.spec.out_dim, C.byref(timing)))
        self.last_timing = timing_dict(timing)
        self._account(n_seqs, n_tokens)
        return out

    def forward_quantized(self, input_ids: np.ndarray, cu_seqlens: np.ndarray, precision: str,
                          token_type_ids: Optional[np.ndarray] = None, ranges: Optional[np.ndarray] = None) -> np.ndarray:
        """The same forward with the result rows quantised on the device before the copy back
        (``precision``: int8 | uint8 | binary | ubinary; ``ranges``: float64 ``[2, dim]`` calibration
        ranges for the 8-bit formats). Returns int8 / uint8 rows of ``dim`` or ``dim / 8`` bytes."""
        ids = np.ascontiguousarray(input_ids, dtype=np.int32)
        cu = np.ascontiguousarray(cu_seqlens, dtype=np.int32)
        tt = None if token_type_ids is None else np.ascontiguousarray(token_type_ids, dtype=np.int32)
        n_seqs, n_tokens = len(cu) - 1, int(len(ids))
        n_rows = n_tokens if self.spec.pooling == "tokens" else n_seqs
        dim = self.spec.out_dim
        width = dim // 8 if precision in ("binary", "ubinary") else dim
        out = np.empty((n_rows, width), dtype=_lib.EMB_NUMPY[precision])
        rg = None if ranges is None else np.ascontiguousarray(ranges, dtype=np.float64)
        if rg is not None and rg.shape != (2, dim):
            raise ValueError(f"ranges must have shape (2, {dim})")
        timing = _lib.Timing()
        _lib.check(self._lib.b200emb_forward_quantized(
            self._handle, ids.ctypes.data, None if tt is None else tt.ctypes.data, cu.ctypes.data, n_seqs, n_tokens,
            _lib.EMB[precision], None if rg is None else rg.ctypes.data, out.ctypes.data, out.strides[0],
            C.byref(timing)))
        self.last_timing = timing_dict(timing)
        self._account(n_seqs, n_tokens)
        return out

    def forward(self, batch: Batch, **kw) -> np.ndarray:
        return self.forward_arrays(batch.input_ids, batch.cu_seqlens, batch.token_type_ids, **kw)

    def forward_device(self, d_ids: int, d_types: Optional[int], d_cu: int, h_cu: np.ndarray, n_tokens: int,
                       d_out: int, per_kernel: bool = False) -> Dict:
        """Device-resident variant: raw device pointers in, result stays on the device."""
        cu = np.ascontiguousarray(h_cu, dtype=np.int32)
        timing = _lib.Timing()
        timing.per_kernel = 1 if per_kernel else 0
        _lib.check(self._lib.b200emb_forward_device(self._handle, d_ids, d_types, d_cu, cu.ctypes.data, len(cu) - 1,
                                                    n_tokens, d_out, self.spec.out_dim, C.byref(timing)))
        self.last_timing = timing_dict(timing)
        return self.last_timing


def partition(lengths: Sequence[int], n_shards: int, cost_linear: float = 1.0, cost_quadratic: float = 0.0) -> np.ndarray:
    """Token-balanced assignment of sequences to shards (the library's own partitioner)."""
    lens = np.ascontiguousarray(lengths, dtype=np.int32)
    out = np.zeros(len(lens), dtype=np.int32)
    lib = _lib.load()
    _lib.check(lib.b200emb_partition(lens.ctypes.data, len(lens), n_shards, cost_linear, cost_quadratic,
                                     out.ctypes.data))
    return out
