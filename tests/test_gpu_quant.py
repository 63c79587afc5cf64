"""Block-format weight quantisers: the CUDA kernels (through the C ABI) must produce exactly
the bytes of the numpy statement in oracle/quant.py, and dequantisation must invert them."""
import numpy as np
import pytest
import torch

from infinity_b200 import _lib
from oracle import quant as Q

pytestmark = pytest.mark.gpu

NVFP4, MXFP8 = _lib.WFMT["nvfp4"], _lib.WFMT["mxfp8"]


def _cases():
    rng = np.random.default_rng(7)
    out = {
        "gauss": rng.standard_normal((96, 512)).astype(np.float32) * 0.02,
        "wide": (rng.standard_normal((33, 256)) * np.exp(rng.standard_normal((33, 256)) * 3)).astype(np.float32),
        "zeros": np.zeros((4, 64), dtype=np.float32),
    }
    zb = rng.standard_normal((8, 128)).astype(np.float32)
    zb[:, 32:64] = 0.0  # a zero block next to non-zero ones
    zb[3] = 0.0
    out["zero_blocks"] = zb
    # values that land exactly on e2m1 midpoints after scaling (ties)
    ties = np.tile(np.array([6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 6],
                            dtype=np.float32), (2, 4))
    out["ties"] = ties
    return {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in out.items()}


@pytest.mark.parametrize("name", ["gauss", "wide", "zeros", "zero_blocks", "ties"])
def test_nvfp4_quantiser_bit_exact(lib, name):
    w = _cases()[name].cuda()
    rows, cols = w.shape
    q = torch.zeros(rows, cols // 2, dtype=torch.uint8, device="cuda")
    s = torch.zeros(rows, cols // 16, dtype=torch.uint8, device="cuda")
    gs = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.b200emb_op_quantize(w.data_ptr(), rows, cols, NVFP4, q.data_ptr(), s.data_ptr(), gs.data_ptr(), None))
    pq, ps, pgs = Q.quantize_nvfp4(w.float().cpu().numpy())
    assert np.float32(gs.item()) == pgs
    assert np.array_equal(s.cpu().numpy(), ps)
    assert np.array_equal(q.cpu().numpy(), pq)
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.b200emb_op_dequantize(q.data_ptr(), s.data_ptr(), rows, cols, NVFP4, out.data_ptr(), None))
    torch.cuda.synchronize()
    want = Q.dequantize_nvfp4(pq, ps, pgs, with_tensor_scale=False)
    assert np.array_equal(out.float().cpu().numpy(), want)  # q * block scale is exact in bf16


@pytest.mark.parametrize("name", ["gauss", "wide", "zeros", "zero_blocks"])
def test_mxfp8_quantiser_bit_exact(lib, name):
    w = _cases()[name].cuda()
    rows, cols = w.shape
    q = torch.zeros(rows, cols, dtype=torch.uint8, device="cuda")
    s = torch.zeros(rows, cols // 32, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.b200emb_op_quantize(w.data_ptr(), rows, cols, MXFP8, q.data_ptr(), s.data_ptr(), None, None))
    pq, ps = Q.quantize_mxfp8(w.float().cpu().numpy())
    assert np.array_equal(s.cpu().numpy(), ps)
    assert np.array_equal(q.cpu().numpy(), pq)
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.b200emb_op_dequantize(q.data_ptr(), s.data_ptr(), rows, cols, MXFP8, out.data_ptr(), None))
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy(), Q.dequantize_mxfp8(pq, ps))


def test_quantiser_round_trip_error_and_idempotence(lib):
    """Size-independent properties at a real layer shape (Qwen2-7B down projection, 3584 x 18944):
    relative error in the expected range, and quantising the dequantised tensor changes nothing."""
    rows, cols = 3584, 18944
    g = torch.Generator(device="cuda").manual_seed(0)
    w = (torch.randn(rows, cols, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    for fmt, div, blk, lo, hi in ((NVFP4, 2, 16, 0.05, 0.13), (MXFP8, 1, 32, 0.01, 0.05)):
        q = torch.zeros(rows, cols // div, dtype=torch.uint8, device="cuda")
        s = torch.zeros(rows, cols // blk, dtype=torch.uint8, device="cuda")
        gs = torch.ones(1, dtype=torch.float32, device="cuda")
        _lib.check(lib.b200emb_op_quantize(w.data_ptr(), rows, cols, fmt, q.data_ptr(), s.data_ptr(), gs.data_ptr(), None))
        d = torch.empty_like(w)
        _lib.check(lib.b200emb_op_dequantize(q.data_ptr(), s.data_ptr(), rows, cols, fmt, d.data_ptr(), None))
        torch.cuda.synchronize()
        deq = d.float() / gs if fmt == NVFP4 else d.float()
        rel = ((deq - w.float()).norm() / w.float().norm()).item()
        assert lo < rel < hi, rel
        if fmt == MXFP8:  # dequantised values are bf16-exact: a second pass must reproduce the same bytes
            q2, s2 = torch.zeros_like(q), torch.zeros_like(s)
            _lib.check(lib.b200emb_op_quantize(d.data_ptr(), rows, cols, fmt, q2.data_ptr(), s2.data_ptr(), None, None))
            assert torch.equal(q2, q) and torch.equal(s2, s)


def test_quantiser_rejects_bad_shapes(lib):
    w = torch.zeros(4, 40, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(4, 40, dtype=torch.uint8, device="cuda")
    assert lib.b200emb_op_quantize(w.data_ptr(), 4, 40, MXFP8, q.data_ptr(), q.data_ptr(), None, None) == -1
    assert "multiple of the block size" in _lib.last_error()
    assert lib.b200emb_op_quantize(w.data_ptr(), 4, 40, 9, q.data_ptr(), q.data_ptr(), None, None) == -1


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 256, 384), (1000, 768, 3072), (4099, 3072, 768)])
@pytest.mark.parametrize("epi", ["bias", "gelu"])
def test_gemm_mxfp8_block_scaled(lib, M, N, K, epi):
    """The block-scaled tensor-core GEMM against fp32 matmul of the dequantised operands: the
    activation is quantised on the fly with the same rule as the numpy statement, so the only
    differences are fp32 summation order and the bf16 rounding of the output."""
    import math
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g, device="cuda") * torch.exp(torch.randn(M, 1, generator=g, device="cuda"))).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g, device="cuda") * 0.3
    wq = torch.zeros(N, K, dtype=torch.uint8, device="cuda")
    ws = torch.zeros(N, K // 32, dtype=torch.uint8, device="cuda")
    _lib.check(lib.b200emb_op_quantize(w.data_ptr(), N, K, MXFP8, wq.data_ptr(), ws.data_ptr(), None, None))
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.b200emb_op_gemm_mxfp8(a.data_ptr(), wq.data_ptr(), ws.data_ptr(), bias.data_ptr(), c.data_ptr(), M, N, K,
                                         _lib.EPI[epi], None))
    a_dq = torch.from_numpy(Q.dequantize_mxfp8(*Q.quantize_mxfp8(a.float().cpu().numpy()))).cuda()
    w_dq = torch.from_numpy(Q.dequantize_mxfp8(wq.cpu().numpy(), ws.cpu().numpy())).cuda()
    ref = a_dq @ w_dq.t() + bias
    if epi == "gelu":
        ref = torch.nn.functional.gelu(ref)
    err = (c.float() - ref).abs().max().item()
    tol = 2.0 ** -8 * max(1.0, ref.abs().max().item()) + 2e-3
    assert err <= tol, (err, tol)
