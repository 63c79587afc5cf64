// Mixture-of-experts feed-forward around the grouped GEMM (memory-bound kernels):
//   router      fp32 logits x W_r^T + b_r, softmax over the experts, top-k (ties -> lower expert
//               index), gate weights = the softmax probabilities of the chosen experts (not
//               renormalised); also counts tokens per expert
//   offsets     exclusive scan of the counts rounded up to 128 rows per expert (so a GEMM row
//               block never straddles two experts) and the row-block -> expert table
//   scatter     copies every token row to its slot(s) in expert-contiguous order
//   combine+LN  out = LayerNorm(x + sum_k gate_k * y[slot_k])
// The slot a token gets inside its expert's segment depends on atomics and may differ from run
// to run; results do not, because every GEMM row is computed independently of its position.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bounds.cuh"
#include "kernels.h"

namespace b2 {

static constexpr int MOE_MAX_E = 16;
static constexpr int MOE_MAX_K = 4;
static constexpr int MOE_WARPS = 8;

__device__ __forceinline__ void unpack8m(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8m(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ float warp_sum_m(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_router_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wr, const float* __restrict__ br,
                  int n_tokens, int hidden, int n_experts, int top_k, int32_t* __restrict__ topk_idx,
                  float* __restrict__ topk_w, int32_t* __restrict__ counts) {
  extern __shared__ float wr_s[];  // [n_experts, hidden]
  __shared__ int32_t cnt_s[MOE_MAX_E];  // tokens per expert seen by this CTA (one global atomic per expert at the end)
  for (int i = threadIdx.x; i < n_experts * hidden; i += blockDim.x) wr_s[i] = wr[i];
  if (threadIdx.x < MOE_MAX_E) cnt_s[threadIdx.x] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int n_chunks = hidden >> 3;
  const int warps_total = gridDim.x * MOE_WARPS;
  constexpr int TPW = 4;  // tokens per warp step: every router-matrix chunk read from shared memory serves four tokens
  for (int t0 = (blockIdx.x * MOE_WARPS + (threadIdx.x >> 5)) * TPW; t0 < n_tokens; t0 += warps_total * TPW) {
    float acc[TPW][MOE_MAX_E];
#pragma unroll
    for (int j = 0; j < TPW; ++j)
#pragma unroll
      for (int e = 0; e < MOE_MAX_E; ++e) acc[j][e] = 0.f;
    for (int c = lane; c < n_chunks; c += 32) {
      float v[TPW][8];
#pragma unroll
      for (int j = 0; j < TPW; ++j) {
        const int t = min(t0 + j, n_tokens - 1);
        unpack8m(*reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * hidden + c * 8), v[j]);
      }
#pragma unroll
      for (int e = 0; e < MOE_MAX_E; ++e) {
        if (e < n_experts) {
          const float4 w0 = *reinterpret_cast<const float4*>(wr_s + e * hidden + c * 8);
          const float4 w1 = *reinterpret_cast<const float4*>(wr_s + e * hidden + c * 8 + 4);
#pragma unroll
          for (int j = 0; j < TPW; ++j)
            acc[j][e] += v[j][0] * w0.x + v[j][1] * w0.y + v[j][2] * w0.z + v[j][3] * w0.w + v[j][4] * w1.x +
                         v[j][5] * w1.y + v[j][6] * w1.z + v[j][7] * w1.w;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < TPW; ++j)
#pragma unroll
      for (int e = 0; e < MOE_MAX_E; ++e)
        if (e < n_experts) acc[j][e] = warp_sum_m(acc[j][e]);
    // lane j finishes token t0 + j (softmax, top-k)
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
      if (lane == j && t0 + j < n_tokens) {
        const int t = t0 + j;
        float* a = acc[j];
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < MOE_MAX_E; ++e)
          if (e < n_experts) {
            a[e] += br != nullptr ? br[e] : 0.f;
            mx = fmaxf(mx, a[e]);
          }
        float den = 0.f;
#pragma unroll
        for (int e = 0; e < MOE_MAX_E; ++e)
          if (e < n_experts) {
            a[e] = expf(a[e] - mx);
            den += a[e];
          }
        uint32_t taken = 0;
        for (int k = 0; k < top_k; ++k) {
          int best = -1;
          float bv = -1.f;
#pragma unroll
          for (int e = 0; e < MOE_MAX_E; ++e)
            if (e < n_experts && !((taken >> e) & 1u) && a[e] > bv) {  // strict >: a tie keeps the lower index
              bv = a[e];
              best = e;
            }
          taken |= 1u << best;
          topk_idx[static_cast<size_t>(t) * top_k + k] = best;
          topk_w[static_cast<size_t>(t) * top_k + k] = bv / den;
          atomicAdd(&cnt_s[best], 1);
        }
      }
    }
  }
  __syncthreads();
  if (counts != nullptr && threadIdx.x < n_experts && cnt_s[threadIdx.x] > 0) atomicAdd(counts + threadIdx.x, cnt_s[threadIdx.x]);
}

// Router for up to 8 experts, eight tokens per warp step.
//  * the router matrix sits in shared memory as [expert][half][chunk] float4 (chunk = 8 consecutive
//    hidden elements, half = its first / last four), so that a warp's 16-byte reads are consecutive;
//    one pass over it serves eight tokens;
//  * every lane accumulates the 8 x 8 (token, expert) partial dot products over its chunks; a
//    reduce-scatter over the warp (32 + 16 + 8 + 4 + 2 shuffles instead of 64 x 5 for a butterfly per
//    value) leaves lane l with token l / 4, experts 2 (l % 4) and 2 (l % 4) + 1;
//  * the four lanes of a token exchange their pairs and each computes softmax and top-k (same
//    instructions in all lanes, no divergence); the first of them writes.
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_router8_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wr, const float* __restrict__ br,
                   int n_tokens, int hidden, int n_experts, int top_k, int32_t* __restrict__ topk_idx,
                   float* __restrict__ topk_w, int32_t* __restrict__ counts) {
  constexpr int E = 8, TPW = 8;
  extern __shared__ float4 wr4_s[];  // [E][2][n_chunks]
  __shared__ int32_t cnt_s[E];
  const int n_chunks = hidden >> 3;
  for (int i = threadIdx.x; i < E * 2 * n_chunks; i += blockDim.x) {
    const int e = i / (2 * n_chunks), half = (i / n_chunks) & 1, c = i % n_chunks;
    wr4_s[i] = e < n_experts ? *reinterpret_cast<const float4*>(wr + static_cast<size_t>(e) * hidden + c * 8 + half * 4)
                             : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (threadIdx.x < E) cnt_s[threadIdx.x] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * MOE_WARPS;
  for (int t0 = (blockIdx.x * MOE_WARPS + (threadIdx.x >> 5)) * TPW; t0 < n_tokens; t0 += warps_total * TPW) {
    float acc[TPW * E];  // index token * 8 + expert
#pragma unroll
    for (int i = 0; i < TPW * E; ++i) acc[i] = 0.f;
    for (int c = lane; c < n_chunks; c += 32) {
      uint4 raw[TPW];
#pragma unroll
      for (int j = 0; j < TPW; ++j)
        raw[j] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(min(t0 + j, n_tokens - 1)) * hidden + c * 8);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float4 w0 = wr4_s[(e * 2) * n_chunks + c];
        const float4 w1 = wr4_s[(e * 2 + 1) * n_chunks + c];
#pragma unroll
        for (int j = 0; j < TPW; ++j) {
          float v[8];
          unpack8m(raw[j], v);
          acc[j * E + e] += v[0] * w0.x + v[1] * w0.y + v[2] * w0.z + v[3] * w0.w + v[4] * w1.x + v[5] * w1.y +
                            v[6] * w1.z + v[7] * w1.w;
        }
      }
    }
    // reduce-scatter: at each stage a lane keeps the half of its values chosen by one bit of its index
    // and adds the partner's copy of that half
#pragma unroll
    for (int stage = 0; stage < 5; ++stage) {
      const int mask = 16 >> stage, half = (TPW * E / 2) >> stage;
      const bool upper = (lane & mask) != 0;
#pragma unroll
      for (int k = 0; k < half; ++k) {
        const float send = upper ? acc[k] : acc[k + half];
        const float keep = upper ? acc[k + half] : acc[k];
        acc[k] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
      }
    }
    // lane l: token t0 + l / 4, experts 2 (l % 4) and 2 (l % 4) + 1; gather the token's eight logits
    float a[E];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      a[2 * q] = __shfl_sync(0xffffffffu, acc[0], (lane & ~3) + q);
      a[2 * q + 1] = __shfl_sync(0xffffffffu, acc[1], (lane & ~3) + q);
    }
    const int t = t0 + (lane >> 2);
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      a[e] = e < n_experts ? a[e] + (br != nullptr ? br[e] : 0.f) : -INFINITY;
      mx = fmaxf(mx, a[e]);
    }
    float den = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      a[e] = expf(a[e] - mx);  // 0 for the experts that do not exist
      den += a[e];
    }
    uint32_t taken = 0;
    for (int k = 0; k < top_k; ++k) {
      int best = 0;
      float bv = -1.f;
#pragma unroll
      for (int e = 0; e < E; ++e)
        if (e < n_experts && !((taken >> e) & 1u) && a[e] > bv) {  // strict >: a tie keeps the lower index
          bv = a[e];
          best = e;
        }
      taken |= 1u << best;
      if ((lane & 3) == 0 && t < n_tokens) {
        topk_idx[static_cast<size_t>(t) * top_k + k] = best;
        topk_w[static_cast<size_t>(t) * top_k + k] = bv / den;
        atomicAdd(&cnt_s[best], 1);
      }
    }
  }
  __syncthreads();
  if (counts != nullptr && threadIdx.x < n_experts && cnt_s[threadIdx.x] > 0) atomicAdd(counts + threadIdx.x, cnt_s[threadIdx.x]);
}

// Router for up to 8 experts on the warp-level tensor-core instruction (mma.sync m16n8k16, bf16 x bf16 ->
// fp32): 16 tokens x 8 experts per warp step, which makes the kernel memory-bound (x is read once).
//  * The fp32 router matrix is split into two bf16 matrices, W = hi + lo (|W - hi - lo| <= 2^-17 |W|), and
//    both are multiplied: the activations are bf16 already, so the products are exact and the logits keep
//    fp32 accuracy.
//  * The contraction index is permuted so that one 16-byte load per lane and row feeds two MMAs: within a
//    32-column block, the lane with quad index q holds columns 8q .. 8q+7 of its two rows (g and g + 8);
//    pairs (0,1), (2,3) go to the first MMA's k slots (2q, 2q+1), (2q+8, 2q+9), pairs (4,5), (6,7) to the
//    second MMA's. The B fragments are laid out once per CTA in shared memory in the same permuted order
//    ([block][lane] -> 16 bytes hi, 16 bytes lo), so consecutive lanes read consecutive 16-byte words.
//  * The accumulator fragment leaves lane (g, q) with experts 2q, 2q+1 of tokens g and g + 8: the four
//    lanes of a quad exchange them and compute softmax / top-k for both tokens; lane q = 0 writes.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_router_mma_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wr, const float* __restrict__ br,
                      int n_tokens, int hidden, int n_experts, int top_k, int32_t* __restrict__ topk_idx,
                      float* __restrict__ topk_w, int32_t* __restrict__ counts) {
  constexpr int E = 8;
  extern __shared__ uint4 wfrag_s[];  // [hidden / 32][32 lanes][2]: hi fragment words, lo fragment words
  __shared__ int32_t cnt_s[E];
  const int n_blocks = hidden >> 5;
  for (int i = threadIdx.x; i < n_blocks * 32; i += blockDim.x) {
    const int kb = i >> 5, l = i & 31, n = l >> 2, q = l & 3;
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {  // column pairs (0,1), (2,3), (4,5), (6,7) of this lane's eight columns
      float w0 = 0.f, w1 = 0.f;
      if (n < n_experts) {
        w0 = wr[static_cast<size_t>(n) * hidden + kb * 32 + q * 8 + 2 * p];
        w1 = wr[static_cast<size_t>(n) * hidden + kb * 32 + q * 8 + 2 * p + 1];
      }
      const __nv_bfloat16 h0 = __float2bfloat16_rn(w0), h1 = __float2bfloat16_rn(w1);
      const __nv_bfloat162 hh = __halves2bfloat162(h0, h1);
      const __nv_bfloat162 ll = __floats2bfloat162_rn(w0 - __bfloat162float(h0), w1 - __bfloat162float(h1));
      hi[p] = *reinterpret_cast<const uint32_t*>(&hh);
      lo[p] = *reinterpret_cast<const uint32_t*>(&ll);
    }
    wfrag_s[2 * i] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    wfrag_s[2 * i + 1] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
  if (threadIdx.x < E) cnt_s[threadIdx.x] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int warps_total = gridDim.x * MOE_WARPS;
  for (int t0 = (blockIdx.x * MOE_WARPS + (threadIdx.x >> 5)) * 16; t0 < n_tokens; t0 += warps_total * 16) {
    const __nv_bfloat16* r0 = x + static_cast<size_t>(min(t0 + g, n_tokens - 1)) * hidden + q * 8;
    const __nv_bfloat16* r1 = x + static_cast<size_t>(min(t0 + g + 8, n_tokens - 1)) * hidden + q * 8;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int kb = 0; kb < n_blocks; ++kb) {
      const uint4 u0 = *reinterpret_cast<const uint4*>(r0 + kb * 32);
      const uint4 u1 = *reinterpret_cast<const uint4*>(r1 + kb * 32);
      const uint4 wh = wfrag_s[2 * (kb * 32 + lane)];
      const uint4 wl = wfrag_s[2 * (kb * 32 + lane) + 1];
      const uint32_t a_first[4] = {u0.x, u1.x, u0.y, u1.y};   // (row g, row g+8) x (pair 0, pair 1)
      const uint32_t a_second[4] = {u0.z, u1.z, u0.w, u1.w};  // pairs 2 and 3
      mma_bf16_16816(c, a_first, wh.x, wh.y);
      mma_bf16_16816(c, a_first, wl.x, wl.y);
      mma_bf16_16816(c, a_second, wh.z, wh.w);
      mma_bf16_16816(c, a_second, wl.z, wl.w);
    }
    // lane (g, q): c[0], c[1] = experts 2q, 2q+1 of token t0 + g; c[2], c[3] = the same of token t0 + g + 8
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float a[E];
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        a[2 * s] = __shfl_sync(0xffffffffu, c[2 * half], (lane & ~3) + s);
        a[2 * s + 1] = __shfl_sync(0xffffffffu, c[2 * half + 1], (lane & ~3) + s);
      }
      const int t = t0 + g + 8 * half;
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        a[e] = e < n_experts ? a[e] + (br != nullptr ? br[e] : 0.f) : -INFINITY;
        mx = fmaxf(mx, a[e]);
      }
      float den = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        a[e] = expf(a[e] - mx);  // 0 for the experts that do not exist
        den += a[e];
      }
      uint32_t taken = 0;
      for (int k = 0; k < top_k; ++k) {
        int best = 0;
        float bv = -1.f;
#pragma unroll
        for (int e = 0; e < E; ++e)
          if (e < n_experts && !((taken >> e) & 1u) && a[e] > bv) {  // strict >: a tie keeps the lower index
            bv = a[e];
            best = e;
          }
        taken |= 1u << best;
        if (q == 0 && t < n_tokens) {
          topk_idx[static_cast<size_t>(t) * top_k + k] = best;
          topk_w[static_cast<size_t>(t) * top_k + k] = bv / den;
          atomicAdd(&cnt_s[best], 1);
        }
      }
    }
  }
  __syncthreads();
  if (counts != nullptr && threadIdx.x < n_experts && cnt_s[threadIdx.x] > 0) atomicAdd(counts + threadIdx.x, cnt_s[threadIdx.x]);
}

// counts[e] -> seg_off[e] (row offset of expert e's segment, multiples of 128), cursor[e] = seg_off[e],
// tile_expert[row block] = expert or -1.
__global__ void moe_offsets_kernel(const int32_t* __restrict__ counts, int n_experts, int max_blocks,
                                   int32_t* __restrict__ cursor, int32_t* __restrict__ tile_expert) {
  __shared__ int32_t off[MOE_MAX_E + 1];
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < n_experts; ++e) {
      off[e] = o;
      cursor[e] = o;
      o += (counts[e] + 127) / 128 * 128;
    }
    off[n_experts] = o;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) {
    const int row = b * 128;
    int owner = -1;
    for (int e = 0; e < n_experts; ++e)
      if (row >= off[e] && row < off[e] + (counts[e] + 127) / 128 * 128) owner = e;
    tile_expert[b] = owner;
  }
}

__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_idx, int n_slots, int top_k,
                   int hidden, int32_t* __restrict__ cursor, int32_t* __restrict__ row_of,
                   __nv_bfloat16* __restrict__ xperm) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * MOE_WARPS;
  // a warp takes 32 consecutive (token, k) slots: lanes that chose the same expert reserve their rows
  // with ONE atomic (the lowest such lane adds the group size), then the warp copies the 32 rows
  for (int s0 = (blockIdx.x * MOE_WARPS + (threadIdx.x >> 5)) * 32; s0 < n_slots; s0 += warps_total * 32) {
    const int s = s0 + lane;
    const int e = s < n_slots ? static_cast<int>(B2_IDX(topk_idx[s], 0, BOUNDS_MOE_EXPERT)) : -1 - lane;  // distinct dummies for lanes past the end
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    const int leader = __ffs(peers) - 1;
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int base = 0;
    if (lane == leader && e >= 0) base = atomicAdd(cursor + e, __popc(peers));
    base = __shfl_sync(0xffffffffu, base, leader);
    const int my_row = s < n_slots ? static_cast<int>(B2_IDX(base + rank, 1, BOUNDS_MOE_ROW)) : 0;
    if (s < n_slots) row_of[s] = my_row;
    const int n_here = min(32, n_slots - s0);
    for (int j = 0; j < n_here; ++j) {
      const int row = __shfl_sync(0xffffffffu, my_row, j);
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>((s0 + j) / top_k) * hidden);
      uint4* dst = reinterpret_cast<uint4*>(xperm + static_cast<size_t>(row) * hidden);
      for (int c = lane; c < (hidden >> 3); c += 32) dst[c] = src[c];
    }
  }
}

// Scatter that quantises on the way: the expert-contiguous copy is written as MXFP8 (e4m3 bytes +
// e8m0 scales in the 512-byte atoms the block-scaled GEMM reads), so the expert GEMM needs no
// separate activation-quantisation pass. Lane b of the warp owns 32-element block b of the row.
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_scatter_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_idx, int n_slots,
                         int top_k, int hidden, int32_t* __restrict__ cursor, int32_t* __restrict__ row_of,
                         uint8_t* __restrict__ xq, uint8_t* __restrict__ sf_atoms) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * MOE_WARPS;
  const int kblocks = hidden >> 5, kgroups = hidden >> 7;
  for (int s0 = (blockIdx.x * MOE_WARPS + (threadIdx.x >> 5)) * 32; s0 < n_slots; s0 += warps_total * 32) {
    const int s = s0 + lane;
    const int e = s < n_slots ? static_cast<int>(B2_IDX(topk_idx[s], 0, BOUNDS_MOE_EXPERT)) : -1 - lane;
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    const int leader = __ffs(peers) - 1;
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int base = 0;
    if (lane == leader && e >= 0) base = atomicAdd(cursor + e, __popc(peers));
    base = __shfl_sync(0xffffffffu, base, leader);
    const int my_row = s < n_slots ? static_cast<int>(B2_IDX(base + rank, 1, BOUNDS_MOE_ROW)) : 0;
    if (s < n_slots) row_of[s] = my_row;
    const int n_here = min(32, n_slots - s0);
    // The top_k slots of a token are consecutive: its row is loaded and quantised once and written to
    // each of its destinations; the next token's loads are in flight meanwhile.
    for (int b0 = 0; b0 < kblocks; b0 += 32) {
      const int b = b0 + lane;
      const bool active = b < kblocks;
      uint4 nxt[4];
      auto prefetch = [&](int tok) {
        if (active) {
          const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(tok) * hidden + b * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) nxt[i] = src[i];
        }
      };
      int cur_tok = -1;
      uint32_t out[8];
      int ex = -127;
      prefetch(s0 / top_k);
      for (int j = 0; j < n_here; ++j) {
        const size_t row = static_cast<size_t>(__shfl_sync(0xffffffffu, my_row, j));
        const int tok = (s0 + j) / top_k;
        if (tok != cur_tok) {  // warp-uniform
          cur_tok = tok;
          float v[32];
          if (active) {
#pragma unroll
            for (int i = 0; i < 4; ++i) unpack8m(nxt[i], reinterpret_cast<float(&)[8]>(v[i * 8]));
          }
          if ((tok + 1) * top_k < s0 + n_here) prefetch(tok + 1);
          if (active) {
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
            ex = -127;
            if (amax > 0.f) {
              ex = ilogbf(amax) - 8;
              ex = ex < -127 ? -127 : (ex > 127 ? 127 : ex);
            }
            const float inv = ex == -127 ? 0.f : exp2f(static_cast<float>(-ex));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              uint32_t word = 0;
#pragma unroll
              for (int k = 0; k < 4; k += 2) {
                const uint32_t two = __nv_cvt_float2_to_fp8x2(make_float2(v[i * 4 + k] * inv, v[i * 4 + k + 1] * inv),
                                                              __NV_SATFINITE, __NV_E4M3);
                word |= (two & 0xffffu) << (8 * k);
              }
              out[i] = word;
            }
          }
        }
        if (active) {
          uint4* dst = reinterpret_cast<uint4*>(xq + row * hidden + b * 32);
          dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
          dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
          sf_atoms[((row >> 7) * kgroups + (b >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (b & 3)] =
              static_cast<uint8_t>(ex + 127);
        }
      }
    }
  }
}

// out[t] = LayerNorm(x[t] + sum_k gate[t, k] * yperm[row_of[t, k]]). Persistent warps; the row indices and
// gates of the next token are read, and its x row and (up to two) expert rows requested, before the current
// token is reduced and stored, so a warp keeps two tokens of gathers in flight. (Without the look-ahead
// every token paid the index load and the dependent gathers in sequence: 62 % of the HBM rate.)
template <int NCH>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_combine_ln_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ yperm,
                      const int32_t* __restrict__ row_of, const float* __restrict__ topk_w, int top_k,
                      const float* __restrict__ gamma, const float* __restrict__ beta, int n_tokens, int hidden,
                      float eps, __nv_bfloat16* __restrict__ out) {
  extern __shared__ float ln_s[];  // gamma[hidden], beta[hidden]
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    ln_s[i] = gamma[i];
    ln_s[hidden + i] = beta[i];
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int n_chunks = hidden >> 3;
  const int warps_total = gridDim.x * MOE_WARPS;
  int t = blockIdx.x * MOE_WARPS + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  constexpr int PRE = 2;  // expert rows fetched ahead; further ones (top_k > 2) are read in the loop
  uint4 xn[NCH], yn[PRE][NCH];
  float gn[PRE];
  auto load_token = [&](int tok) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(tok) * hidden;
    const __nv_bfloat16* yr[PRE];
#pragma unroll
    for (int k = 0; k < PRE; ++k) {
      yr[k] = nullptr;
      gn[k] = 0.f;
      if (k < top_k) {
        gn[k] = __ldg(topk_w + static_cast<size_t>(tok) * top_k + k);
        yr[k] = yperm + static_cast<size_t>(B2_IDX(__ldg(row_of + static_cast<size_t>(tok) * top_k + k), 1, BOUNDS_MOE_ROW)) * hidden;
      }
    }
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        xn[i] = *reinterpret_cast<const uint4*>(xr + c * 8);
#pragma unroll
        for (int k = 0; k < PRE; ++k)
          if (yr[k] != nullptr) yn[k][i] = *reinterpret_cast<const uint4*>(yr[k] + c * 8);
      }
    }
  };
  load_token(t);
  while (t < n_tokens) {
    float v[NCH][8];
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        unpack8m(xn[i], v[i]);
#pragma unroll
        for (int k = 0; k < PRE; ++k)
          if (k < top_k) {  // experts are added in the order k = 0, 1, ... as before
            float a[8];
            unpack8m(yn[k][i], a);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[i][e] = fmaf(gn[k], a[e], v[i][e]);
          }
      }
    }
    for (int k = PRE; k < top_k; ++k) {
      const float g = topk_w[static_cast<size_t>(t) * top_k + k];
      const __nv_bfloat16* yr = yperm + static_cast<size_t>(B2_IDX(row_of[static_cast<size_t>(t) * top_k + k], 1, BOUNDS_MOE_ROW)) * hidden;
#pragma unroll
      for (int i = 0; i < NCH; ++i) {
        const int c = lane + 32 * i;
        if (c < n_chunks) {
          float a[8];
          unpack8m(*reinterpret_cast<const uint4*>(yr + c * 8), a);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] = fmaf(g, a[e], v[i][e]);
        }
      }
    }
    const int next = t + warps_total;
    if (next < n_tokens) load_token(next);  // in flight while this token is reduced and stored
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i)
      if (lane + 32 * i < n_chunks) {
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += v[i][e];
      }
    const float mean = warp_sum_m(sum) / hidden;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i)
      if (lane + 32 * i < n_chunks) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = v[i][e] - mean;
          sq += d * d;
        }
      }
    const float rstd = rsqrtf(warp_sum_m(sq) / hidden + eps);
    __nv_bfloat16* dst = out + static_cast<size_t>(t) * hidden;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd * ln_s[c * 8 + e] + ln_s[hidden + c * 8 + e];
        *reinterpret_cast<uint4*>(dst + c * 8) = pack8m(o);
      }
    }
    t = next;
  }
}

int moe_init_device() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  B2_CUDA_CHECK(cudaFuncSetAttribute(moe_router8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  B2_CUDA_CHECK(cudaFuncSetAttribute(moe_router_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  return B200EMB_OK;
}

static int persistent_grid(int n_rows) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int full = (n_rows + MOE_WARPS - 1) / MOE_WARPS;
  return full < sms * 4 ? (full > 0 ? full : 1) : sms * 4;
}

int launch_moe_router(const void* x, const float* wr, const float* br, int n_tokens, int hidden, int n_experts,
                      int top_k, int32_t* topk_idx, float* topk_w, int32_t* counts, cudaStream_t stream) {
  if (n_tokens <= 0) return B200EMB_OK;
  if (n_experts < 1 || n_experts > MOE_MAX_E || top_k < 1 || top_k > MOE_MAX_K || top_k > n_experts)
    return set_error(B200EMB_ERR_UNSUPPORTED, "router: need 1 <= top_k <= min(%d, n_experts) and n_experts <= %d", MOE_MAX_K, MOE_MAX_E);
  if (hidden % 8) return set_error(B200EMB_ERR_UNSUPPORTED, "router: hidden %d not a multiple of 8", hidden);
  const size_t smem = static_cast<size_t>(n_experts) * hidden * sizeof(float);
  if (smem > 96 * 1024) return set_error(B200EMB_ERR_UNSUPPORTED, "router: n_experts * hidden too large for shared memory");
  if (counts != nullptr) B2_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int32_t) * n_experts, stream));
  if (n_experts <= 8 && hidden % 32 == 0 && static_cast<size_t>(hidden) * 32 <= 96 * 1024) {
    moe_router_mma_kernel<<<persistent_grid((n_tokens + 15) / 16), MOE_WARPS * 32, static_cast<size_t>(hidden) * 32, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), wr, br, n_tokens, hidden, n_experts, top_k, topk_idx, topk_w, counts);
    cudaError_t em = cudaGetLastError();
    if (em != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "router launch: %s", cudaGetErrorString(em));
    return B200EMB_OK;
  }
  if (n_experts <= 8) {
    const size_t smem8 = static_cast<size_t>(8) * hidden * sizeof(float);
    if (smem8 <= 96 * 1024) {
      moe_router8_kernel<<<persistent_grid((n_tokens + 7) / 8), MOE_WARPS * 32, smem8, stream>>>(
          reinterpret_cast<const __nv_bfloat16*>(x), wr, br, n_tokens, hidden, n_experts, top_k, topk_idx, topk_w, counts);
      cudaError_t e8 = cudaGetLastError();
      if (e8 != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "router launch: %s", cudaGetErrorString(e8));
      return B200EMB_OK;
    }
  }
  moe_router_kernel<<<persistent_grid((n_tokens + 3) / 4), MOE_WARPS * 32, smem, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), wr, br, n_tokens, hidden, n_experts, top_k, topk_idx, topk_w, counts);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "router launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int moe_max_row_blocks(int n_tokens, int top_k, int n_experts) {
  return (n_tokens * top_k + n_experts * 127 + 127) / 128;
}

int launch_moe_scatter(const void* x, const int32_t* topk_idx, const int32_t* counts, int n_tokens, int top_k,
                       int hidden, int n_experts, int32_t* cursor, int32_t* tile_expert, int32_t* row_of, void* xperm,
                       cudaStream_t stream, void* xq, void* sf_atoms) {
  if (n_tokens <= 0) return B200EMB_OK;
  const int max_blocks = moe_max_row_blocks(n_tokens, top_k, n_experts);
  B2_SET_LIMIT(0, n_experts, stream);
  B2_SET_LIMIT(1, static_cast<long long>(max_blocks) * 128, stream);  // also the limit of the combine that follows
  moe_offsets_kernel<<<1, 256, 0, stream>>>(counts, n_experts, max_blocks, cursor, tile_expert);
  if (xq != nullptr) {
    if (hidden % 128) return set_error(B200EMB_ERR_INVALID, "moe scatter (mxfp8): hidden %d not a multiple of 128", hidden);
    moe_scatter_mxfp8_kernel<<<persistent_grid((n_tokens * top_k + 31) / 32), MOE_WARPS * 32, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), topk_idx, n_tokens * top_k, top_k, hidden, cursor, row_of,
        reinterpret_cast<uint8_t*>(xq), reinterpret_cast<uint8_t*>(sf_atoms));
  } else
  moe_scatter_kernel<<<persistent_grid((n_tokens * top_k + 31) / 32), MOE_WARPS * 32, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), topk_idx, n_tokens * top_k, top_k, hidden, cursor, row_of,
      reinterpret_cast<__nv_bfloat16*>(xperm));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "moe scatter launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_moe_combine_ln(const void* x, const void* yperm, const int32_t* row_of, const float* topk_w, int top_k,
                          const float* gamma, const float* beta, int n_tokens, int hidden, float eps, void* out,
                          cudaStream_t stream) {
  if (n_tokens <= 0) return B200EMB_OK;
  if (hidden % 8 || (hidden >> 3) > 32 * 4)
    return set_error(B200EMB_ERR_UNSUPPORTED, "moe combine: hidden %d unsupported (multiple of 8, at most 1024)", hidden);
  const int nch = ((hidden >> 3) + 31) / 32;
  const size_t smem = 2 * static_cast<size_t>(hidden) * sizeof(float);
  const int grid = persistent_grid(n_tokens);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* yp = reinterpret_cast<const __nv_bfloat16*>(yperm);
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(out);
  switch (nch) {
    case 1: moe_combine_ln_kernel<1><<<grid, MOE_WARPS * 32, smem, stream>>>(xp, yp, row_of, topk_w, top_k, gamma, beta, n_tokens, hidden, eps, op); break;
    case 2: moe_combine_ln_kernel<2><<<grid, MOE_WARPS * 32, smem, stream>>>(xp, yp, row_of, topk_w, top_k, gamma, beta, n_tokens, hidden, eps, op); break;
    case 3: moe_combine_ln_kernel<3><<<grid, MOE_WARPS * 32, smem, stream>>>(xp, yp, row_of, topk_w, top_k, gamma, beta, n_tokens, hidden, eps, op); break;
    default: moe_combine_ln_kernel<4><<<grid, MOE_WARPS * 32, smem, stream>>>(xp, yp, row_of, topk_w, top_k, gamma, beta, n_tokens, hidden, eps, op); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "moe combine launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int moe_bounds_status(cudaStream_t stream) {
  (void)stream;
  return B2_TAKE_STATUS(stream);
}

}  // namespace b2

using namespace b2;

extern "C" int b200emb_op_moe_router(const void* x, const float* router_w, const float* router_b, int32_t n_tokens,
                                     int32_t hidden, int32_t n_experts, int32_t top_k, int32_t* topk_idx,
                                     float* topk_weight, int32_t* counts, void* stream) {
  if (x == nullptr || router_w == nullptr || topk_idx == nullptr || topk_weight == nullptr)
    return set_error(B200EMB_ERR_INVALID, "moe_router: null pointer");
  int rc = kernels_init_device();
  if (rc) return rc;
  return launch_moe_router(x, router_w, router_b, n_tokens, hidden, n_experts, top_k, topk_idx, topk_weight, counts,
                           reinterpret_cast<cudaStream_t>(stream));
}
