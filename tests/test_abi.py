"""The C ABI: the shared library loads, exports every symbol the header declares, and the
ctypes structures have the layout the C compiler gives them. No compute call needs a GPU here."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

from infinity_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200emb.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200emb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header drifted apart"


def test_struct_layouts_match_the_compiler(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b200emb.h"\n'
                   'int main(){printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(b200emb_model_desc), sizeof(b200emb_timing),'
                   ' offsetof(b200emb_model_desc, norm_eps), offsetof(b200emb_model_desc, max_tokens),'
                   ' offsetof(b200emb_timing, kclass_ms), offsetof(b200emb_timing, gemm_flops));return 0;}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = list(map(int, subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()))
    want = [C.sizeof(_lib.ModelDesc), C.sizeof(_lib.Timing), _lib.ModelDesc.norm_eps.offset,
            _lib.ModelDesc.max_tokens.offset, _lib.Timing.kclass_ms.offset, _lib.Timing.gemm_flops.offset]
    assert got == want


def test_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "b200emb.h"\nint main(void){return B200EMB_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)


def test_partition_is_token_balanced_and_deterministic(lib):
    from infinity_b200.engine import partition
    rng = np.random.default_rng(0)
    lens = rng.integers(8, 513, size=1024).astype(np.int32)
    for shards in (1, 2, 4, 8):
        owner = partition(lens, shards, 1.0, 0.0)
        assert owner.min() >= 0 and owner.max() < shards
        loads = np.array([lens[owner == s].sum() for s in range(shards)])
        assert loads.sum() == lens.sum()
        assert loads.max() - loads.min() <= lens.max()  # LPT bound
        assert np.array_equal(owner, partition(lens, shards, 1.0, 0.0))
    # ties go to the lower shard; equal lengths alternate
    assert partition([5, 5, 5, 5], 2).tolist() == [0, 1, 0, 1]
    # quadratic cost moves long sequences apart
    owner = partition([512, 512, 8, 8, 8, 8], 2, 1.0, 1.0)
    assert owner[0] != owner[1]
    assert partition([], 4).tolist() == []


def test_cost_model_follows_the_architecture(lib):
    """sharding.cost_coefficients asks the library, so a process-per-GPU driver and a multi-device
    handle cut a batch identically: 6 H F for the gated decoder FFN, top_k experts in routed layers."""
    from infinity_b200 import configs as cf
    from infinity_b200.sharding import cost_coefficients
    bert = cf.tiny_spec("bert")
    a, b = cost_coefficients(bert)
    H, F = bert.hidden, bert.ffn
    assert a == 2.0 * H * 3 * H + 2.0 * H * H + 4.0 * H * F and b > 0
    dec = cf.tiny_spec("decoder")
    a_d, b_d = cost_coefficients(dec)
    qkv = (dec.n_heads + 2 * dec.n_kv_heads) * dec.head_dim
    assert a_d == 2.0 * dec.hidden * qkv + 2.0 * dec.hidden ** 2 + 6.0 * dec.hidden * dec.ffn
    assert b_d / dec.hidden == 0.5 * b / H            # causal attention: half the pairs
    moe = cf.tiny_spec("moe")
    a_m, _ = cost_coefficients(moe)
    Hm, Fm = moe.hidden, moe.ffn
    routed = sum(1 for l in range(moe.n_layers) if l % moe.moe_every == moe.moe_every - 1)
    ffn = (routed * (moe.top_k * 4.0 * Hm * Fm + 2.0 * Hm * moe.n_experts) + (moe.n_layers - routed) * 4.0 * Hm * Fm) / moe.n_layers
    assert abs(a_m - (2.0 * Hm * 3 * Hm + 2.0 * Hm * Hm + ffn)) < 1e-6 * a_m
    assert lib.b200emb_cost_model(None, None, None) == -1


def test_partition_rejects_bad_arguments(lib):
    assert lib.b200emb_partition(None, 3, 2, 1.0, 0.0, None) == -1
    assert "partition" in _lib.last_error()
    assert lib.b200emb_partition(None, 0, 0, 1.0, 0.0, None) == -1


def test_create_fails_loudly_without_gpu_or_file(lib, tmp_path):
    """No CPU fallback: without a device (or without a weight file) create returns an error."""
    from infinity_b200 import configs as cf
    from infinity_b200.engine import make_desc
    desc = make_desc(cf.tiny_spec())
    h = C.c_void_p()
    ids = (C.c_int32 * 1)(0)
    st = lib.b200emb_create(C.byref(desc), str(tmp_path / "missing.b2ew").encode(), ids, 1, C.byref(h))
    assert st != 0 and not h.value
    msg = _lib.last_error()
    assert ("no CUDA device" in msg) or ("cannot open" in msg)
    desc.abi_version = 99
    assert lib.b200emb_create(C.byref(desc), b"x", ids, 1, C.byref(h)) == -1
    assert "abi_version" in _lib.last_error()
