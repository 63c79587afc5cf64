"""ctypes binding of ``libb200emb.so`` (the C ABI declared in ``include/b200emb.h``).

The library is the only compute path: when it is missing, or when it reports that no
CUDA device is usable, the callers raise. Nothing here falls back to torch or numpy.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

ABI_VERSION = 1
N_KCLASS = 8
KCLASS_NAMES = ["embed", "gemm", "attention", "norm", "pool", "other", "k6", "k7"]

ARCH = {"bert": 0, "xlmr": 1, "moe": 2, "decoder": 3}
POOL = {"cls": 0, "mean": 1, "last": 2, "tokens": 3}
# output embedding precisions (EmbeddingDtype, infinity_emb/primitives.py:145-158)
EMB = {"float32": 0, "int8": 1, "uint8": 2, "binary": 3, "ubinary": 4}
EMB_NUMPY = {"float32": "float32", "int8": "int8", "uint8": "uint8", "binary": "int8", "ubinary": "uint8"}
HEAD = {"none": 0, "classifier": 1}
WFMT = {"bf16": 0, "mxfp8": 1, "nvfp4": 2}
EPI = {"bias": 0, "gelu": 1, "tanh": 2, "swiglu": 3}


class ModelDesc(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("arch", C.c_int32), ("n_layers", C.c_int32), ("hidden", C.c_int32),
        ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32),
        ("vocab", C.c_int32), ("max_pos", C.c_int32), ("type_vocab", C.c_int32), ("pos_offset", C.c_int32),
        ("norm_eps", C.c_float), ("rope_theta", C.c_float), ("n_experts", C.c_int32), ("top_k", C.c_int32),
        ("moe_every", C.c_int32), ("pooling", C.c_int32), ("normalize", C.c_int32), ("head", C.c_int32),
        ("n_labels", C.c_int32), ("weight_format", C.c_int32), ("max_tokens", C.c_int32),
        ("label_scores", C.c_int32), ("reserved", C.c_int32 * 7),
    ]


class Timing(C.Structure):
    _fields_ = [
        ("per_kernel", C.c_int32), ("n_devices", C.c_int32), ("h2d_ms", C.c_float), ("kernels_ms", C.c_float),
        ("d2h_ms", C.c_float), ("total_ms", C.c_float), ("launches", C.c_int32),
        ("kclass_ms", C.c_float * N_KCLASS), ("kclass_launches", C.c_int32 * N_KCLASS),
        ("gemm_flops", C.c_double),
    ]


class B200EmbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"b200emb status {code}: {message}")
        self.code = code


# name -> (restype, argtypes); every symbol include/b200emb.h declares
_P = C.c_void_p
_I32P = C.POINTER(C.c_int32)
SIGNATURES = {
    "b200emb_create": (C.c_int, [C.POINTER(ModelDesc), C.c_char_p, _I32P, C.c_int32, C.POINTER(_P)]),
    "b200emb_destroy": (C.c_int, [_P]),
    "b200emb_quantize_weights": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int32, C.c_int32]),
    "b200emb_forward": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, _P, C.c_int64, C.POINTER(Timing)]),
    "b200emb_forward_device": (C.c_int, [_P, _P, _P, _P, _P, C.c_int32, C.c_int32, _P, C.c_int64, C.POINTER(Timing)]),
    "b200emb_partition": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_double, C.c_double, _P]),
    "b200emb_cost_model": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "b200emb_test_fail_allocs": (C.c_int, [C.c_int32, C.c_int32]),
    "b200emb_checked_build": (C.c_int, []),
    "b200emb_tensor_map_stats": (C.c_int, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "b200emb_last_error": (C.c_char_p, []),
    "b200emb_device_count": (C.c_int, []),
    "b200emb_selftest_bounded_wait": (C.c_int, [C.c_int32]),
    "b200emb_op_gemm_bf16": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P]),
    "b200emb_op_gemm_nvfp4": (C.c_int, [_P, _P, _P, C.c_float, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P]),
    "b200emb_op_gemm_mxfp8": (C.c_int, [_P, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P]),
    "b200emb_op_attention": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P]),
    "b200emb_op_attention_static": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P]),
    "b200emb_op_quantize": (C.c_int, [_P, C.c_int64, C.c_int64, C.c_int32, _P, _P, _P, _P]),
    "b200emb_op_dequantize": (C.c_int, [_P, _P, C.c_int64, C.c_int64, C.c_int32, _P, _P]),
    "b200emb_op_moe_router": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P]),
    "b200emb_op_embed_ln": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_float, _P, _P]),
    "b200emb_op_add_ln": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_float, _P, _P]),
    "b200emb_op_pool": (C.c_int, [_P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, C.c_int64, C.c_int32, _P]),
    "b200emb_forward_quantized": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, _P, _P, C.c_int64, C.POINTER(Timing)]),
    "b200emb_op_quantize_embeddings": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int64, C.c_int32, _P, _P, C.c_int64, _P]),
}

_lib = None


def lib_path() -> Path:
    """The in-tree library, or the file named by B200EMB_LIBRARY (to compare two builds)."""
    override = os.environ.get("B200EMB_LIBRARY")
    return Path(override) if override else _build.LIB_PATH


def load(build_if_missing: bool = True) -> C.CDLL:
    """Loads the shared library (building it first when absent) and types every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        if not build_if_missing:
            raise FileNotFoundError(f"{path} is missing: run `python -m infinity_b200.build`")
        _build.build()
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the header and the library drift apart
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return (load().b200emb_last_error() or b"").decode("utf-8", "replace")


def check(status: int) -> None:
    if status != 0:
        raise B200EmbError(status, last_error())
