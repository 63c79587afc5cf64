"""The allocation-free attention entry point against the allocating one.

``b200emb_op_attention_static`` serves callers that must not allocate device memory inside
a library call: processes whose own memory pool already holds almost all of the GPU, and
latency-critical threads for which the device-wide synchronisation of cudaMalloc / cudaFree
is not acceptable. Its scratch (tile list + error word) is a fixed array inside the library
that every call re-uses, so the test runs it twice in a row, the second time on a smaller
and different batch, and each result must equal ``b200emb_op_attention`` bit for bit (both
run the same kernel on the same rows; only the order of the tiles differs).

This file sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""
import numpy as np
import pytest
import torch

from infinity_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(lib, fn, qkv, cu, nh, nkv, d, causal):
    T = int(cu[-1])
    out = torch.full((T, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    d_cu = torch.from_numpy(cu).cuda()
    torch.cuda.synchronize()
    _lib.check(fn(qkv.data_ptr(), out.data_ptr(), d_cu.data_ptr(), cu.ctypes.data, len(cu) - 1, T, nh, nkv, d, causal,
                  torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("d,nh,nkv,causal", [(64, 8, 8, 0), (128, 4, 2, 1), (32, 4, 4, 0)])
def test_static_attention_matches_allocating_entry_point_twice(lib, d, nh, nkv, causal):
    batches = [[300, 1, 128, 129, 64, 500, 17], [40, 256, 3]]  # second call: smaller, stale tiles left behind
    for k, lens in enumerate(batches):
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        g = torch.Generator(device="cuda").manual_seed(100 * d + k)
        qkv = torch.randn(int(cu[-1]), (nh + 2 * nkv) * d, generator=g, device="cuda").to(torch.bfloat16)
        want = _run(lib, lib.b200emb_op_attention, qkv, cu, nh, nkv, d, causal)
        got = _run(lib, lib.b200emb_op_attention_static, qkv, cu, nh, nkv, d, causal)
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got, want), f"call {k}: max abs diff {(got.float() - want.float()).abs().max().item()}"


def test_static_attention_many_short_sequences_and_forced_kernel(lib):
    """More sequences than the tile-building kernel has threads (each thread then scans several),
    and the flag that forces the one-CTA-per-SM kernel for head_dim 64."""
    rng = np.random.default_rng(5)
    lens = rng.integers(1, 40, size=3000).tolist()
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    for d, nh, flags in ((64, 2, 0), (64, 2, 0x200), (64, 2, 0x201)):
        g = torch.Generator(device="cuda").manual_seed(d + flags)
        qkv = torch.randn(int(cu[-1]), 3 * nh * d, generator=g, device="cuda").to(torch.bfloat16)
        want = _run(lib, lib.b200emb_op_attention, qkv, cu, nh, nh, d, flags)
        got = _run(lib, lib.b200emb_op_attention_static, qkv, cu, nh, nh, d, flags)
        assert torch.equal(got, want)


def test_static_attention_allocates_no_device_memory(lib):
    """Free device memory as the driver reports it is the same before and after a warmed call."""
    lens = [300, 1, 128, 129, 64, 500, 17]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    qkv = torch.randn(int(cu[-1]), 3 * 8 * 64, device="cuda").to(torch.bfloat16)
    _run(lib, lib.b200emb_op_attention_static, qkv, cu, 8, 8, 64, 0)  # first call on the device: set-up
    out = torch.empty(int(cu[-1]), 8 * 64, dtype=torch.bfloat16, device="cuda")
    d_cu = torch.from_numpy(cu).cuda()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        _lib.check(lib.b200emb_op_attention_static(qkv.data_ptr(), out.data_ptr(), d_cu.data_ptr(), cu.ctypes.data,
                                                   len(lens), int(cu[-1]), 8, 8, 64, 0, None))
    assert torch.cuda.mem_get_info()[0] == free_before


def test_static_attention_rejects_batches_beyond_its_scratch(lib):
    n = 16385  # one query tile each: one more than B200EMB_STATIC_ATTN_MAX_TILES
    cu = np.arange(n + 1, dtype=np.int32)
    qkv = torch.zeros(n, 3 * 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(n, 64, dtype=torch.bfloat16, device="cuda")
    d_cu = torch.from_numpy(cu).cuda()
    st = lib.b200emb_op_attention_static(qkv.data_ptr(), out.data_ptr(), d_cu.data_ptr(), cu.ctypes.data, n, n, 1, 1, 64,
                                         0, None)
    assert st == -2 and "exceed the fixed scratch" in _lib.last_error()
