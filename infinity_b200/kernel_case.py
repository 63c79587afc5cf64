"""Runs one kernel a few times on seeded inputs, for profiling a small case under ncu:

    python -m infinity_b200.kernel_case gemm --m 32768 --n 3072 --k 1024 --epi bias --launches 3
    python -m infinity_b200.kernel_case attention --seqs 256 --len 384 --heads 16 --head-dim 64 --launches 3
    python -m infinity_b200.kernel_case add_ln --rows 65536 --hidden 1024 --launches 3
    python -m infinity_b200.kernel_case nvfp4 --m 1024 --n 37888 --k 3584 --epi swiglu --launches 5

The nvfp4 case also times its two ways of multiplying by NVFP4 weights (CUDA events, best of the launches):
expansion inside the GEMM (b200emb_op_gemm_nvfp4) against the expansion kernel followed by the bf16 GEMM.

Every case checks its result against a torch computation before exiting 0.
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch

from . import _lib
from . import configs as cf


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attention", "add_ln", "nvfp4", "mxfp8"])
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--epi", default="bias", choices=list(_lib.EPI))
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--len", type=int, default=384)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--causal", type=int, default=0)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--lengths-of", default=None, choices=sorted(cf.SPECS),
                    help="attention: take the sequence lengths of this configuration's synthetic batch instead of --seqs x --len")
    a = ap.parse_args()
    lib = _lib.load()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    if a.kernel == "gemm":
        A = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
        W = (torch.randn(a.n, a.k, device="cuda") / math.sqrt(a.k)).to(torch.bfloat16)
        bias = torch.randn(a.n, device="cuda")
        Cm = torch.empty(a.m, a.n, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        for _ in range(a.launches):
            _lib.check(lib.b200emb_op_gemm_bf16(A.data_ptr(), W.data_ptr(), bias.data_ptr(), Cm.data_ptr(), a.m, a.n,
                                                a.k, _lib.EPI[a.epi] | (a.bn << 8), stream))
        rows = slice(0, min(a.m, 2048))
        ref = A[rows].float() @ W.float().t() + bias
        if a.epi == "gelu":
            ref = torch.nn.functional.gelu(ref)
        elif a.epi == "tanh":
            ref = torch.tanh(ref)
        err = (Cm[rows].float() - ref).abs().max().item()
        assert err < 0.05, err
        print(f"gemm {a.m}x{a.n}x{a.k} ok, max abs err {err:.4f}")
    elif a.kernel == "mxfp8":
        # the block-scaled fp8 GEMM and the bf16 GEMM on the same shape, one after the other (dense, not grouped)
        MXFP8 = _lib.WFMT["mxfp8"]
        A = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
        W = (torch.randn(a.n, a.k, device="cuda") / math.sqrt(a.k)).to(torch.bfloat16)
        bias = torch.randn(a.n, device="cuda") * 0.1
        wq = torch.zeros(a.n, a.k, dtype=torch.uint8, device="cuda")
        ws = torch.zeros(a.n, a.k // 32, dtype=torch.uint8, device="cuda")
        _lib.check(lib.b200emb_op_quantize(W.data_ptr(), a.n, a.k, MXFP8, wq.data_ptr(), ws.data_ptr(), None, stream))
        c8 = torch.empty(a.m, a.n, dtype=torch.bfloat16, device="cuda")
        c16 = torch.empty(a.m, a.n, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        for _ in range(a.launches):
            _lib.check(lib.b200emb_op_gemm_mxfp8(A.data_ptr(), wq.data_ptr(), ws.data_ptr(), bias.data_ptr(), c8.data_ptr(), a.m, a.n,
                                                 a.k, _lib.EPI[a.epi], stream))
            _lib.check(lib.b200emb_op_gemm_bf16(A.data_ptr(), W.data_ptr(), bias.data_ptr(), c16.data_ptr(), a.m, a.n, a.k,
                                                _lib.EPI[a.epi] | (a.bn << 8), stream))
        torch.cuda.synchronize()
        rows = slice(0, min(a.m, 2048))
        err = (c8[rows].float() - c16[rows].float()).abs().max().item()
        scale = c16[rows].float().abs().max().item()
        assert err < 0.1 * max(1.0, scale), (err, scale)
        print(f"mxfp8 and bf16 gemm {a.m}x{a.n}x{a.k} {a.epi} ok, max abs difference {err:.4f} (largest output {scale:.2f})")
    elif a.kernel == "nvfp4":
        NVFP4 = _lib.WFMT["nvfp4"]
        w = (torch.randn(a.n, a.k, device="cuda") * 0.02).to(torch.bfloat16)
        q = torch.zeros(a.n, a.k // 2, dtype=torch.uint8, device="cuda")
        sc = torch.zeros(a.n, a.k // 16, dtype=torch.uint8, device="cuda")
        gs = torch.zeros(1, dtype=torch.float32, device="cuda")
        _lib.check(lib.b200emb_op_quantize(w.data_ptr(), a.n, a.k, NVFP4, q.data_ptr(), sc.data_ptr(), gs.data_ptr(), stream))
        del w
        A = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
        n_out = a.n // 2 if a.epi == "swiglu" else a.n
        c1 = torch.empty(a.m, n_out, dtype=torch.bfloat16, device="cuda")
        c2 = torch.empty(a.m, n_out, dtype=torch.bfloat16, device="cuda")
        wexp = torch.empty(a.n, a.k, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()

        def timed(fn):
            best = float("inf")
            for _ in range(a.launches):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            return best

        def fused():
            _lib.check(lib.b200emb_op_gemm_nvfp4(A.data_ptr(), q.data_ptr(), sc.data_ptr(), float(gs.item()), None,
                                                 c1.data_ptr(), a.m, a.n, a.k, _lib.EPI[a.epi], stream))

        def expanded():
            _lib.check(lib.b200emb_op_dequantize(q.data_ptr(), sc.data_ptr(), a.n, a.k, NVFP4, wexp.data_ptr(), stream))
            _lib.check(lib.b200emb_op_gemm_bf16(A.data_ptr(), wexp.data_ptr(), None, c2.data_ptr(), a.m, a.n, a.k,
                                                _lib.EPI[a.epi], stream))

        t_fused, t_exp = timed(fused), timed(expanded)
        assert torch.isfinite(c1.float()).all()
        if a.epi == "bias":  # same B tiles; the tensor scale is applied to the accumulator in one and left out in the other
            ratio = (c1.float().abs().mean() / c2.float().abs().mean()).item()
            assert abs(ratio * float(gs.item()) - 1.0) < 2e-2, (ratio, float(gs.item()))
        flops = 2.0 * a.m * a.n * a.k
        print(f"nvfp4 gemm {a.m}x{a.n}x{a.k} {a.epi}: expansion in the kernel {t_fused:.3f} ms ({flops / t_fused / 1e9:.0f} TFLOP/s), "
              f"expansion kernel + bf16 gemm {t_exp:.3f} ms ({flops / t_exp / 1e9:.0f} TFLOP/s)")
    elif a.kernel == "attention":
        nkv = a.kv_heads or a.heads
        if a.lengths_of:
            lengths = cf.synth_batch(a.lengths_of).lengths
            a.seqs, a.len = len(lengths), int(lengths[0])
            cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
        else:
            cu = (np.arange(a.seqs + 1) * a.len).astype(np.int32)
        T = int(cu[-1])
        qkv = torch.randn(T, (a.heads + 2 * nkv) * a.head_dim, device="cuda").to(torch.bfloat16)
        out = torch.empty(T, a.heads * a.head_dim, dtype=torch.bfloat16, device="cuda")
        d_cu = torch.from_numpy(cu).cuda()
        torch.cuda.synchronize()
        for _ in range(a.launches):
            _lib.check(lib.b200emb_op_attention(qkv.data_ptr(), out.data_ptr(), d_cu.data_ptr(), cu.ctypes.data,
                                                a.seqs, T, a.heads, nkv, a.head_dim, a.causal, stream))
        q, k, v = qkv[: a.len].float().split([a.heads * a.head_dim, nkv * a.head_dim, nkv * a.head_dim], dim=1)
        rep = a.heads // nkv
        qh = q.view(a.len, a.heads, a.head_dim).transpose(0, 1)
        kh = k.view(a.len, nkv, a.head_dim).transpose(0, 1).repeat_interleave(rep, 0)
        vh = v.view(a.len, nkv, a.head_dim).transpose(0, 1).repeat_interleave(rep, 0)
        s = qh @ kh.transpose(1, 2) / math.sqrt(a.head_dim)
        if a.causal:
            s = s.masked_fill(torch.ones(a.len, a.len, device="cuda").triu(1).bool(), float("-inf"))
        ref = (torch.softmax(s, -1) @ vh).transpose(0, 1).reshape(a.len, -1)
        err = (out[: a.len].float() - ref).abs().max().item()
        assert err < 2e-2, err
        flop = 4.0 * float((np.diff(cu).astype(np.float64) ** 2).sum()) * a.heads * a.head_dim * (0.5 if a.causal & 1 else 1.0)
        print(f"attention {a.seqs} sequences, {T} tokens ok, max abs err {err:.4f}, {flop / 1e9:.1f} GFLOP algorithmic")
    else:
        x = torch.randn(a.rows, a.hidden, device="cuda").to(torch.bfloat16)
        y = torch.randn(a.rows, a.hidden, device="cuda").to(torch.bfloat16)
        g = torch.ones(a.hidden, device="cuda")
        b = torch.zeros(a.hidden, device="cuda")
        out = torch.empty_like(x)
        torch.cuda.synchronize()
        for _ in range(a.launches):
            _lib.check(lib.b200emb_op_add_ln(x.data_ptr(), y.data_ptr(), g.data_ptr(), b.data_ptr(), a.rows, a.hidden,
                                             1e-12, out.data_ptr(), stream))
        torch.cuda.synchronize()
        ref = torch.nn.functional.layer_norm(x[:1024].float() + y[:1024].float(), (a.hidden,), g, b, 1e-12)
        err = (out[:1024].float() - ref).abs().max().item()
        assert err < 3e-2, err
        print(f"add_ln {a.rows}x{a.hidden} ok, max abs err {err:.4f}")


if __name__ == "__main__":
    main()
