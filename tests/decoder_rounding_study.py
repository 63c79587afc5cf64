"""Where does the full-depth decoder lose its cosine? A CPU study, not a test (pytest does not collect it):

    python tests/decoder_rounding_study.py [n_layers]

fp32 forward of the Qwen2-7B shape (28 layers, hidden 3584, 28 / 4 heads of 128, FFN 18944; seeded N(0, 0.02)
matrices rounded to bf16, the four sequence lengths of test_config5_qwen2_7b_shape_full_depth) in several
variants that differ only in which activations are rounded to bf16 where the CUDA path stores them between
kernels: the RMSNorm outputs ("norm"), q / k / v ("qkv"), q and k after the rotation ("rope"), the attention
probabilities as the P V operand ("p"), the attention output ("ctx"), the sub-layer outputs added to the fp32
residual stream ("y") and the SwiGLU output ("act"). Prints the minimum last-token cosine against the unrounded
forward at a few depths. Result (28 layers, about 2.5 minutes on 8 cores): every rounding the kernels make 0.99908;
the same with fp32 sub-layer outputs 0.99919; without the P rounding 0.99915; only norm + qkv + rope 0.99935; only the
sub-layer outputs 0.99989; only P 0.99997. The operands of the tensor-core products (norm, q, k, v) carry most of the
loss, so it comes with bf16 tensor-core compute itself and not with a storage choice that could be changed cheaply.
"""
import math, sys, time, torch, numpy as np
import torch.nn.functional as F
torch.set_num_threads(32)
H, nh, nkv, d, FF, NL = 3584, 28, 4, 128, 18944, int(sys.argv[1]) if len(sys.argv) > 1 else 28
theta, eps = 1e6, 1e-6
lens = [32, 100, 61, 48]
rb = lambda x: x.bfloat16().float()
VARIANTS = {
  "fp32": set(),
  "kernels": {"norm", "qkv", "rope", "p", "ctx", "y", "act"},
  "y_fp32": {"norm", "qkv", "rope", "p", "ctx", "act"},
  "p_fp32": {"norm", "qkv", "rope", "ctx", "y", "act"},
  "y_p_fp32": {"norm", "qkv", "rope", "ctx", "act"},
  "only_y": {"y"},
  "only_p": {"p"},
  "only_norm_qkv_rope": {"norm", "qkv", "rope"},
}
def rms(x, g): return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g
def rot(x):
    a, b = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([-b, a], -1)
g = torch.Generator().manual_seed(5)
def mat(*s): return rb(torch.empty(*s).normal_(0.0, 0.02, generator=g))
L = max(lens); B = len(lens)
mask = torch.zeros(B, L)
for i, n in enumerate(lens): mask[i, :n] = 1
h0 = mat(B, L, H)
inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
fr = torch.arange(L).float()[:, None] * inv[None]
cos, sin = torch.cat([fr, fr], -1).cos(), torch.cat([fr, fr], -1).sin()
neg = torch.finfo(torch.float32).min
add_mask = torch.clamp(torch.ones(L, L).triu(1)[None, None] * neg + (1 - mask)[:, None, None, :] * neg, min=neg)
hs = {k: h0.clone() for k in VARIANTS}
t0 = time.time()
with torch.no_grad():
  for l in range(NL):
    wqkv, bq, wo, wg, wu, wd = mat((nh + 2 * nkv) * d, H), torch.zeros((nh + 2 * nkv) * d), mat(H, nh * d), mat(FF, H), mat(FF, H), mat(H, FF)
    for name, R in VARIANTS.items():
        r = lambda x, key: rb(x) if key in R else x
        h = hs[name]
        x = r(rms(h, 1.0), "norm")
        qkv = r(x @ wqkv.t() + bq, "qkv")
        q, k, v = qkv.split([nh * d, nkv * d, nkv * d], -1)
        q = q.view(B, L, nh, d).transpose(1, 2); k = k.view(B, L, nkv, d).transpose(1, 2); v = v.view(B, L, nkv, d).transpose(1, 2)
        q = r(q * cos + rot(q) * sin, "rope"); k = r(k * cos + rot(k) * sin, "rope")
        k = k.repeat_interleave(nh // nkv, 1); v = v.repeat_interleave(nh // nkv, 1)
        s = q @ k.transpose(-1, -2) / math.sqrt(d) + add_mask
        m = s.max(-1, keepdim=True).values
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)          # the kernels sum the fp32 exponentials and round only the P operand
        a = (r(e, "p") @ v) / den
        a = r(a.transpose(1, 2).reshape(B, L, nh * d), "ctx")
        h = h + r(a @ wo.t(), "y")
        x = r(rms(h, 1.0), "norm")
        f = r(F.silu(x @ wg.t()) * (x @ wu.t()), "act")
        h = h + r(f @ wd.t(), "y")
        hs[name] = h
    if l in (1, 7, 13, 20, NL - 1):
        ref = rms(hs["fp32"], 1.0)
        line = []
        for name in VARIANTS:
            o = rms(hs[name], 1.0)
            c = []
            for i, n in enumerate(lens):
                a_, b_ = o[i, n - 1], ref[i, n - 1]
                c.append(float((a_ @ b_) / (a_.norm() * b_.norm())))
            line.append(f"{name} {min(c):.6f}")
        print(f"layer {l + 1:2d} ({time.time() - t0:.0f} s): " + " | ".join(line), flush=True)
