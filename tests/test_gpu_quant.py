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


def _nvfp4_weights(N, K, seed, amax=None):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).clamp_(-0.04, 0.04)
    if amax is not None:
        w[0, 0] = amax
    w = w.to(torch.bfloat16)
    q = torch.zeros(N, K // 2, dtype=torch.uint8, device="cuda")
    s = torch.zeros(N, K // 16, dtype=torch.uint8, device="cuda")
    gs = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    _lib.check(_lib.load().b200emb_op_quantize(w.data_ptr(), N, K, NVFP4, q.data_ptr(), s.data_ptr(), gs.data_ptr(), None))
    return q, s, float(gs.item())


@pytest.mark.parametrize("M,N,K", [(20000, 512, 256), (19000, 1024, 1024), (40001, 256, 3584), (1, 256, 64), (300, 768, 192)])
def test_nvfp4_gemm_expands_weights_in_the_kernel(lib, M, N, K):
    """b200emb_op_gemm_nvfp4 reads the stored e2m1 bytes and e4m3 scales itself: against the fp32 product with the
    numpy-dequantised weights, and bit for bit against the expansion kernel followed by the bf16 GEMM (the tensor
    scale is a power of two here, so that its factor commutes with the rounding to bf16)."""
    amax = 2688.0 / 65536.0  # exactly representable in bf16: gs = 2688 / amax = 65536
    q, s, gs = _nvfp4_weights(N, K, 11 + N, amax)
    assert gs == 65536.0
    g = torch.Generator(device="cuda").manual_seed(M)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    bias = torch.randn(N, generator=g, device="cuda") * 0.5
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.b200emb_op_gemm_nvfp4(a.data_ptr(), q.data_ptr(), s.data_ptr(), gs, bias.data_ptr(), c.data_ptr(), M, N, K,
                                         _lib.EPI["bias"], None))
    w_dq = torch.from_numpy(Q.dequantize_nvfp4(q.cpu().numpy(), s.cpu().numpy(), np.float32(gs))).cuda()
    rows = slice(0, 2048)
    ref = a[rows].float() @ w_dq.t() + bias
    err = (c[rows].float() - ref).abs().max().item()
    assert err <= 2.0 ** -8 * max(1.0, ref.abs().max().item()) + 1e-3, err
    assert not torch.isnan(c.float()).any()
    # the unfused path: expansion kernel, then the bf16 GEMM on q * block scale with the bias scaled by gs
    w_exp = torch.empty(N, K, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.b200emb_op_dequantize(q.data_ptr(), s.data_ptr(), N, K, NVFP4, w_exp.data_ptr(), None))
    c2 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    bias_scaled = (bias * gs).contiguous()
    torch.cuda.synchronize()
    _lib.check(lib.b200emb_op_gemm_bf16(a.data_ptr(), w_exp.data_ptr(), bias_scaled.data_ptr(), c2.data_ptr(), M, N, K,
                                        _lib.EPI["bias"] | (257 << 8), None))
    assert torch.equal((c2.float() / gs).to(torch.bfloat16), c)


def test_nvfp4_gemm_swiglu_and_limits(lib):
    from infinity_b200.configs import interleave_gate_up
    M, F, K = 20000, 512, 512
    g = torch.Generator(device="cuda").manual_seed(3)
    wg = (torch.randn(F, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    wu = (torch.randn(F, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w = interleave_gate_up(wg, wu).contiguous()
    q = torch.zeros(2 * F, K // 2, dtype=torch.uint8, device="cuda")
    s = torch.zeros(2 * F, K // 16, dtype=torch.uint8, device="cuda")
    gs = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.b200emb_op_quantize(w.data_ptr(), 2 * F, K, NVFP4, q.data_ptr(), s.data_ptr(), gs.data_ptr(), None))
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    c = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    _lib.check(lib.b200emb_op_gemm_nvfp4(a.data_ptr(), q.data_ptr(), s.data_ptr(), float(gs.item()), None, c.data_ptr(), M, 2 * F, K,
                                         _lib.EPI["swiglu"], None))
    w_dq = torch.from_numpy(Q.dequantize_nvfp4(q.cpu().numpy(), s.cpu().numpy(), np.float32(gs.item()))).cuda()
    from helpers import deinterleave_gate_up
    gd, ud = deinterleave_gate_up(w_dq)
    rows = slice(0, 1024)
    ref = torch.nn.functional.silu(a[rows].float() @ gd.t()) * (a[rows].float() @ ud.t())
    err = (c[rows].float() - ref).abs().max().item()
    assert err <= 2.0 ** -8 * max(1.0, ref.abs().max().item()) + 2e-3, err
    # an unsupported epilogue or shape: a clean status, nothing launched
    st = lib.b200emb_op_gemm_nvfp4(a.data_ptr(), q.data_ptr(), s.data_ptr(), 1.0, None, c.data_ptr(), M, 2 * F, K, _lib.EPI["gelu"], None)
    assert st == -2 and "gemm_w4" in _lib.last_error()
    st = lib.b200emb_op_gemm_nvfp4(a.data_ptr(), q.data_ptr(), s.data_ptr(), 1.0, None, c.data_ptr(), M, 2 * F - 128, K, _lib.EPI["bias"], None)
    assert st == -2
