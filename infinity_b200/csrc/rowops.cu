// Memory-bound row kernels over the ragged token stream [n_tokens, hidden] (bf16):
//   embed_ln   : word + position + token-type gather, then LayerNorm
//   add_ln     : LayerNorm(x + y)   (post-LN residual step of BERT-style blocks)
//   pool       : CLS / mean / last-token pooling per sequence + L2 normalisation
//   small_proj : [n, hidden] x [n_labels, hidden]^T for classifier heads with few labels
// One warp owns one row; a lane holds hidden/256 (rounded up) 16-byte chunks in registers,
// statistics are fp32 with warp-shuffle reductions (two-pass: mean, then centred variance).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bounds.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace b2 {

// Self-test of the bounded-wait mechanism every pipelined kernel relies on: one thread waits on an
// mbarrier that nothing ever signals. The wait must give up after limit_ns, record a code in the
// error word and let the kernel end normally, leaving the context usable.
__global__ void wait_selftest_kernel(unsigned long long limit_ns, int* err_flag) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    if (!mbar_wait(&bar, 0, limit_ns)) atomicExch(err_flag, 9);
  }
}

int launch_wait_selftest(unsigned long long limit_ns, int* err_flag, cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(limit_ns, err_flag);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "wait self-test launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

static constexpr int ROW_WARPS = 8;  // rows per CTA

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// Normalises the row held in v[NCH][8] (chunk c = lane + 32*i valid iff c < n_chunks) and stores bf16. The
// arithmetic runs on packed fp32 pairs (FADD2 / FFMA2: one instruction per two values): inside a forward the SM
// clock sits near 1.4 GHz under the power cap, where the scalar version's instruction stream, not HBM, set the pace.
template <int NCH>
__device__ __forceinline__ void layernorm_store(float (&v)[NCH][8], int lane, int n_chunks, int hidden,
                                                const float* __restrict__ gamma, const float* __restrict__ beta,
                                                float eps, __nv_bfloat16* __restrict__ dst) {
  float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NCH; ++i)
    if (lane + 32 * i < n_chunks) {
#pragma unroll
      for (int e = 0; e < 8; e += 2) s2 = __fadd2_rn(s2, make_float2(v[i][e], v[i][e + 1]));
    }
  const float mean = warp_sum(s2.x + s2.y) / hidden;
  const float2 nmean2 = make_float2(-mean, -mean);
  float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NCH; ++i)
    if (lane + 32 * i < n_chunks) {
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const float2 d = __fadd2_rn(make_float2(v[i][e], v[i][e + 1]), nmean2);
        q2 = __ffma2_rn(d, d, q2);
      }
    }
  const float rstd = rsqrtf(warp_sum(q2.x + q2.y) / hidden + eps);
  const float2 rstd2 = make_float2(rstd, rstd);
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = lane + 32 * i;
    if (c < n_chunks) {
      const float4 g0 = *reinterpret_cast<const float4*>(gamma + c * 8);
      const float4 g1 = *reinterpret_cast<const float4*>(gamma + c * 8 + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(beta + c * 8);
      const float4 b1 = *reinterpret_cast<const float4*>(beta + c * 8 + 4);
      const float2 g[4] = {make_float2(g0.x, g0.y), make_float2(g0.z, g0.w), make_float2(g1.x, g1.y), make_float2(g1.z, g1.w)};
      const float2 b[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
      uint4 u;
      uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 t = __fmul2_rn(__fadd2_rn(make_float2(v[i][2 * e], v[i][2 * e + 1]), nmean2), rstd2);
        const float2 o = __ffma2_rn(t, g[e], b[e]);
        __nv_bfloat162 p = __floats2bfloat162_rn(o.x, o.y);
        w[e] = *reinterpret_cast<uint32_t*>(&p);
      }
      *reinterpret_cast<uint4*>(dst + c * 8) = u;
    }
  }
}

// Index that is safe to use whatever the caller put on the device: an id outside [0, limit) is reported in the
// error word (first writer wins; the host turns the code into an invalid-argument status when the forward ends)
// and replaced by 0, so that no kernel reads outside its table. limit <= 0 switches the check off.
static constexpr int ERR_BAD_TOKEN_ID = 32, ERR_BAD_TOKEN_TYPE = 33;
__device__ __forceinline__ int checked_index(int v, int limit, int* err_flag, int code) {
  if (limit > 0 && (v < 0 || v >= limit)) {
    if (err_flag != nullptr) atomicCAS(err_flag, 0, code);
    return 0;
  }
  return v;
}

// Plain row gather out[t,:] = table[ids[t],:] (decoder embedding lookup): persistent warps, four
// 16-byte loads in flight per lane, nothing kept in registers.
__global__ void __launch_bounds__(ROW_WARPS * 32)
gather_rows_kernel(const int32_t* __restrict__ ids, int n_tokens, const __nv_bfloat16* __restrict__ table, int hidden,
                   __nv_bfloat16* __restrict__ out, int vocab, int* __restrict__ err_flag) {
  const int lane = threadIdx.x & 31;
  const int n_chunks = hidden >> 3;
  const int warps_total = gridDim.x * ROW_WARPS;
  for (int t = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); t < n_tokens; t += warps_total) {
    const int id = checked_index(__ldg(ids + t), vocab, err_flag, ERR_BAD_TOKEN_ID);
    const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden);
    for (int c = lane; c < n_chunks; c += 128) {
      uint4 u[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + 32 * j < n_chunks) u[j] = __ldg(src + c + 32 * j);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + 32 * j < n_chunks) dst[c + 32 * j] = u[j];
    }
  }
}

static constexpr int EMB_TOK = 4;  // tokens per warp of embed_ln_kernel

template <int NCH>
__global__ void __launch_bounds__(ROW_WARPS * 32)
embed_ln_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ types, const int32_t* __restrict__ cu,
                int n_seqs, int n_tokens, const __nv_bfloat16* __restrict__ word,
                const __nv_bfloat16* __restrict__ pos, const __nv_bfloat16* __restrict__ type_table,
                const float* __restrict__ gamma, const float* __restrict__ beta, int hidden, int pos_offset,
                float eps, __nv_bfloat16* __restrict__ out, int vocab, int type_vocab, int* __restrict__ err_flag) {
  // A warp takes EMB_TOK consecutive tokens, one after the other (a CTA of one token per warp lives about two
  // microseconds, too short for the block scheduler to keep the SMs full). Lane k reads the id and the type of token
  // k; the sequence of the first token is found by bisection, the following tokens walk on from it.
  const int t0 = (blockIdx.x * ROW_WARPS + (threadIdx.x >> 5)) * EMB_TOK;
  if (t0 >= n_tokens) return;
  const int lane = threadIdx.x & 31;
  const int n_chunks = hidden >> 3;
  int my_id = 0, my_ty = 0;
  if (lane < EMB_TOK && t0 + lane < n_tokens) {
    my_id = checked_index(__ldg(ids + t0 + lane), vocab, err_flag, ERR_BAD_TOKEN_ID);
    if (type_table != nullptr && types != nullptr)
      my_ty = checked_index(__ldg(types + t0 + lane), type_vocab, err_flag, ERR_BAD_TOKEN_TYPE);
  }
  int seq = 0, seq_end = 0;
  if (pos != nullptr) {
    // sequence of token t0: largest i with cu[i] <= t0 (only needed for the position rows)
    int lo = 0, hi = n_seqs;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(cu + mid) <= t0) lo = mid; else hi = mid;
    }
    seq = lo;
    seq_end = __ldg(cu + seq + 1);
  }
#pragma unroll 1
  for (int k = 0; k < EMB_TOK; ++k) {
    const int t = t0 + k;
    if (t >= n_tokens) break;
    int p = 0;
    if (pos != nullptr) {
      while (t >= seq_end && seq + 1 < n_seqs) {  // sequences are not empty: at most EMB_TOK steps in all
        ++seq;
        seq_end = __ldg(cu + seq + 1);
      }
      p = static_cast<int>(B2_IDX(pos_offset + t - __ldg(cu + seq), 2, BOUNDS_EMBED_POSITION));
    }
    const int id = __shfl_sync(0xffffffffu, my_id, k);
    const __nv_bfloat16* wrow = word + static_cast<size_t>(id) * hidden;
    const __nv_bfloat16* prow = pos != nullptr ? pos + static_cast<size_t>(p) * hidden : nullptr;
    const __nv_bfloat16* trow = nullptr;
    if (type_table != nullptr) trow = type_table + static_cast<size_t>(__shfl_sync(0xffffffffu, my_ty, k)) * hidden;

    float v[NCH][8];
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(wrow + c * 8)), v[i]);
        if (trow != nullptr) {
          float a[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(trow + c * 8)), a);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += a[e];
        }
        if (prow != nullptr) {
          float a[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(prow + c * 8)), a);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += a[e];
        }
      }
    }
    __nv_bfloat16* dst = out + static_cast<size_t>(t) * hidden;
    if (gamma == nullptr) {
#pragma unroll
      for (int i = 0; i < NCH; ++i) {
        const int c = lane + 32 * i;
        if (c < n_chunks) *reinterpret_cast<uint4*>(dst + c * 8) = pack8(v[i]);
      }
      continue;
    }
    layernorm_store<NCH>(v, lane, n_chunks, hidden, gamma, beta, eps, dst);
  }
}

// Persistent: every warp walks rows warp_id, warp_id + n_warps, ...; gamma and beta are staged once
// per CTA in shared memory, and the loads of the next row are issued before the current row is
// reduced, so each warp keeps two rows of loads in flight.
template <int NCH>
__global__ void __launch_bounds__(ROW_WARPS * 32)
add_ln_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
              const float* __restrict__ gamma, const float* __restrict__ beta, int n_rows, int hidden, float eps,
              __nv_bfloat16* __restrict__ out) {
  extern __shared__ float ln_smem[];  // gamma[hidden], beta[hidden]
  float* g_s = ln_smem;
  float* b_s = ln_smem + hidden;
  // gamma and beta are weights, which no kernel writes: they are staged while the previous kernel in the
  // stream may still be running; x and y are its results and are read only after pdl_wait().
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    g_s[i] = gamma[i];
    b_s[i] = beta[i];
  }
  __syncthreads();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int n_chunks = hidden >> 3;
  const int warps_total = gridDim.x * ROW_WARPS;
  int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  uint4 xn[NCH], yn[NCH];
  auto load_row = [&](int r) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(r) * hidden;
    const __nv_bfloat16* yr = y != nullptr ? y + static_cast<size_t>(r) * hidden : nullptr;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        xn[i] = *reinterpret_cast<const uint4*>(xr + c * 8);
        if (yr != nullptr) yn[i] = *reinterpret_cast<const uint4*>(yr + c * 8);
      }
    }
  };
  load_row(row);
  while (row < n_rows) {
    float v[NCH][8];
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        unpack8(xn[i], v[i]);
        if (y != nullptr) {
          float a[8];
          unpack8(yn[i], a);
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const float2 t = __fadd2_rn(make_float2(v[i][e], v[i][e + 1]), make_float2(a[e], a[e + 1]));
            v[i][e] = t.x;
            v[i][e + 1] = t.y;
          }
        }
      }
    }
    const int next = row + warps_total;
    if (next < n_rows) load_row(next);  // in flight while this row is reduced and stored
    else pdl_launch_dependents();       // last row of this warp: the next kernel may start its set-up
    layernorm_store<NCH>(v, lane, n_chunks, hidden, g_s, b_s, eps, out + static_cast<size_t>(row) * hidden);
    row = next;
  }
}

// Pre-norm residual step of decoder blocks: h (fp32 residual stream) += y (bf16 sub-layer output,
// nullable), then out = h / sqrt(mean(h^2) + eps) * gamma in bf16. Persistent warps, gamma in
// shared memory. The residual stream stays fp32 so that 2 x n_layers additions do not
// accumulate bf16 rounding.
template <int NCH>
__global__ void __launch_bounds__(ROW_WARPS * 32)
add_rmsnorm_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ y, const float* __restrict__ gamma,
                   int n_rows, int hidden, float eps, __nv_bfloat16* __restrict__ out) {
  extern __shared__ float ln_smem[];
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) ln_smem[i] = gamma[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int n_chunks = hidden >> 3;
  const int warps_total = gridDim.x * ROW_WARPS;
  for (int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); row < n_rows; row += warps_total) {
    float* hr = h + static_cast<size_t>(row) * hidden;
    const __nv_bfloat16* yr = y != nullptr ? y + static_cast<size_t>(row) * hidden : nullptr;
    float v[NCH][8];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        const float4 a0 = *reinterpret_cast<const float4*>(hr + c * 8);
        const float4 a1 = *reinterpret_cast<const float4*>(hr + c * 8 + 4);
        v[i][0] = a0.x; v[i][1] = a0.y; v[i][2] = a0.z; v[i][3] = a0.w;
        v[i][4] = a1.x; v[i][5] = a1.y; v[i][6] = a1.z; v[i][7] = a1.w;
        if (yr != nullptr) {
          float b[8];
          unpack8(*reinterpret_cast<const uint4*>(yr + c * 8), b);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += b[e];
          *reinterpret_cast<float4*>(hr + c * 8) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          *reinterpret_cast<float4*>(hr + c * 8 + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sq += v[i][e] * v[i][e];
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) / hidden + eps);
    __nv_bfloat16* dst = out + static_cast<size_t>(row) * hidden;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane + 32 * i;
      if (c < n_chunks) {
        const float4 g0 = *reinterpret_cast<const float4*>(ln_smem + c * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(ln_smem + c * 8 + 4);
        float o[8];
        o[0] = v[i][0] * rstd * g0.x; o[1] = v[i][1] * rstd * g0.y; o[2] = v[i][2] * rstd * g0.z; o[3] = v[i][3] * rstd * g0.w;
        o[4] = v[i][4] * rstd * g1.x; o[5] = v[i][5] * rstd * g1.y; o[6] = v[i][6] * rstd * g1.z; o[7] = v[i][7] * rstd * g1.w;
        *reinterpret_cast<uint4*>(dst + c * 8) = pack8(o);
      }
    }
  }
}

// Same step for wide rows (hidden > 2048): one CTA of 256 threads per row, at most two 16-byte
// chunks per thread, so few registers and many rows in flight per SM; the sum of squares meets in
// shared memory.
static constexpr int RMS_BLOCK = 256;
__global__ void __launch_bounds__(RMS_BLOCK)
add_rmsnorm_wide_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ y, const float* __restrict__ gamma,
                        int n_rows, int hidden, float eps, __nv_bfloat16* __restrict__ out) {
  __shared__ float red[RMS_BLOCK / 32];
  const int n_chunks = hidden >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // The loads of the CTA's next row are issued before the current row is reduced (two block barriers and a dependent
  // store pass per row), so each CTA keeps two rows of loads in flight.
  float4 ha[2][2];
  uint4 ya[2];
  auto load_row = [&](int r) {
    const float* hr = h + static_cast<size_t>(r) * hidden;
    const __nv_bfloat16* yr = y != nullptr ? y + static_cast<size_t>(r) * hidden : nullptr;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = threadIdx.x + RMS_BLOCK * i;
      if (c < n_chunks) {
        ha[i][0] = *reinterpret_cast<const float4*>(hr + c * 8);
        ha[i][1] = *reinterpret_cast<const float4*>(hr + c * 8 + 4);
        if (yr != nullptr) ya[i] = *reinterpret_cast<const uint4*>(yr + c * 8);
      }
    }
  };
  if (static_cast<int>(blockIdx.x) < n_rows) load_row(blockIdx.x);
  for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
    float* hr = h + static_cast<size_t>(row) * hidden;
    float v[2][8];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = threadIdx.x + RMS_BLOCK * i;
      if (c < n_chunks) {
        v[i][0] = ha[i][0].x; v[i][1] = ha[i][0].y; v[i][2] = ha[i][0].z; v[i][3] = ha[i][0].w;
        v[i][4] = ha[i][1].x; v[i][5] = ha[i][1].y; v[i][6] = ha[i][1].z; v[i][7] = ha[i][1].w;
        if (y != nullptr) {
          float b[8];
          unpack8(ya[i], b);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += b[e];
          *reinterpret_cast<float4*>(hr + c * 8) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          *reinterpret_cast<float4*>(hr + c * 8 + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sq += v[i][e] * v[i][e];
      }
    }
    if (row + static_cast<int>(gridDim.x) < n_rows) load_row(row + gridDim.x);
    sq = warp_sum(sq);
    __syncthreads();  // the previous row's readers of red[] are done
    if (lane == 0) red[warp] = sq;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < RMS_BLOCK / 32; ++w) tot += red[w];  // same order in every thread: deterministic
    const float rstd = rsqrtf(tot / hidden + eps);
    __nv_bfloat16* dst = out + static_cast<size_t>(row) * hidden;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = threadIdx.x + RMS_BLOCK * i;
      if (c < n_chunks) {
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c * 8));
        const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma + c * 8 + 4));
        float o[8];
        o[0] = v[i][0] * rstd * g0.x; o[1] = v[i][1] * rstd * g0.y; o[2] = v[i][2] * rstd * g0.z; o[3] = v[i][3] * rstd * g0.w;
        o[4] = v[i][4] * rstd * g1.x; o[5] = v[i][5] * rstd * g1.y; o[6] = v[i][6] * rstd * g1.z; o[7] = v[i][7] * rstd * g1.w;
        *reinterpret_cast<uint4*>(dst + c * 8) = pack8(o);
      }
    }
  }
}

// bf16 rows -> fp32 rows (starts the fp32 residual stream from the embedding gather).
__global__ void widen_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, size_t n_chunks) {
  for (size_t c = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; c < n_chunks;
       c += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(x + c * 8), v);
    *reinterpret_cast<float4*>(out + c * 8) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(out + c * 8 + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// Rotary position embedding, in place on the query and key heads of the packed qkv buffer
// (rotate-half convention: element i pairs with i + d/2; angle = position * theta^(-2i/d)).
// Positions restart at every sequence. cs holds (cos, sin) per (position, i), fp32.
__global__ void __launch_bounds__(256)
rope_kernel(__nv_bfloat16* __restrict__ qkv, const int32_t* __restrict__ cu, int n_seqs, int n_tokens, int n_rot_heads,
            int row_width, int head_dim, const float2* __restrict__ cs) {
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  int lo = 0, hi = n_seqs;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(cu + mid) <= t) lo = mid; else hi = mid;
  }
  const int pos = static_cast<int>(B2_IDX(t - __ldg(cu + lo), 1, BOUNDS_ROPE_POSITION));
  const int half = head_dim >> 1;
  const int per_head = half >> 3;  // 16-byte groups of 8 pairs
  const float2* cst = cs + static_cast<size_t>(pos) * half;
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * row_width;
  for (int w = threadIdx.x; w < n_rot_heads * per_head; w += blockDim.x) {
    const int head = w / per_head, g = w % per_head;
    __nv_bfloat16* p1 = row + head * head_dim + g * 8;
    __nv_bfloat16* p2 = p1 + half;
    float a[8], b[8], o1[8], o2[8];
    unpack8(*reinterpret_cast<const uint4*>(p1), a);
    unpack8(*reinterpret_cast<const uint4*>(p2), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float2 c = __ldg(cst + g * 8 + e);
      o1[e] = a[e] * c.x - b[e] * c.y;
      o2[e] = b[e] * c.x + a[e] * c.y;
    }
    *reinterpret_cast<uint4*>(p1) = pack8(o1);
    *reinterpret_cast<uint4*>(p2) = pack8(o2);
  }
}

// One CTA of 512 threads per sequence. Threads tile the hidden dimension in 16-byte chunks; when the block
// has more threads than chunks the spare threads split the rows (mean pooling), every thread keeps eight
// rows of loads in flight, and the partial sums meet in shared memory in a fixed order: the result depends
// on the sequence alone, not on the batch around it. (With 256 threads and four rows in flight a 512-token
// sequence kept its CTA busy for most of the kernel: 23-39 % of the HBM rate on batches of 1024-2048 sequences.)
static constexpr int POOL_THREADS = 512;
static constexpr int POOL_MAXC = 2;  // chunks per thread: hidden <= 512 * 8 * 2 = 8192
static constexpr int POOL_ROWS = 8;  // rows in flight per thread

template <int PC>
__global__ void __launch_bounds__(POOL_THREADS)
pool_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ cu, int hidden, int pooling,
            int normalize, void* __restrict__ out, int64_t out_row_stride, int out_bf16) {
  extern __shared__ float pool_smem[];  // [row_groups][hidden] partial sums + 32 reduction slots
  const int seq = blockIdx.x;
  int start = __ldg(cu + seq), end = __ldg(cu + seq + 1);
  if (!B2_RANGE_OK(start, end, 0, BOUNDS_POOL_RANGE)) start = end = 0;  // checked build: an empty sequence instead
  const int n_chunks = hidden >> 3;
  const int cols = n_chunks < POOL_THREADS ? n_chunks : POOL_THREADS;  // threads across the hidden dim
  const int row_groups = POOL_THREADS / cols;
  const int cg = threadIdx.x % cols;
  const int rg = threadIdx.x / cols;
  int r_begin = start, r_end = end;
  if (pooling == B200EMB_POOL_CLS) r_end = start + 1;
  if (pooling == B200EMB_POOL_LAST) r_begin = end - 1;
  const float inv_count = 1.0f / fmaxf(static_cast<float>(r_end - r_begin), 1e-9f);

  float acc[PC][8];
#pragma unroll
  for (int i = 0; i < PC; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  if (rg < row_groups) {
    // rows are added in ascending order within a row group, so the sum does not depend on the unrolling
    for (int r = r_begin + rg; r < r_end; r += POOL_ROWS * row_groups) {
#pragma unroll
      for (int i = 0; i < PC; ++i) {
        const int c = cg + cols * i;
        if (c < n_chunks) {
          // every load is unconditional (rows past the end re-read the last row and are dropped below), so
          // the eight requests go out back to back
          uint4 u[POOL_ROWS];
#pragma unroll
          for (int j = 0; j < POOL_ROWS; ++j) {
            const int rr = min(r + j * row_groups, r_end - 1);
            u[j] = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(rr) * hidden + c * 8));
          }
#pragma unroll
          for (int j = 0; j < POOL_ROWS; ++j) {
            if (r + j * row_groups < r_end) {
              float a[8];
              unpack8(u[j], a);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[i][e] += a[e];
            }
          }
        }
      }
    }
    // partial sums of this row group; combined below in a fixed order (deterministic)
    float* part = pool_smem + static_cast<size_t>(rg) * hidden;
#pragma unroll
    for (int i = 0; i < PC; ++i) {
      const int c = cg + cols * i;
      if (c < n_chunks) {
#pragma unroll
        for (int e = 0; e < 8; ++e) part[c * 8 + e] = acc[i][e];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < hidden; i += POOL_THREADS) {
    float tot = pool_smem[i];
    for (int g2 = 1; g2 < row_groups; ++g2) tot += pool_smem[static_cast<size_t>(g2) * hidden + i];
    pool_smem[i] = tot;  // only this thread touches column i of group 0 from here on
  }

  float* red = pool_smem + static_cast<size_t>(row_groups) * hidden;
  float sq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += POOL_THREADS) {
    const float m = pool_smem[i] * inv_count;
    pool_smem[i] = m;
    sq += m * m;
  }
  float scale = 1.f;
  if (normalize) {
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < POOL_THREADS / 32; ++w) tot += red[w];
    scale = 1.f / fmaxf(sqrtf(tot), 1e-12f);
  }
  if (out_bf16) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<size_t>(seq) * out_row_stride;
    for (int i = threadIdx.x; i < hidden; i += POOL_THREADS) o[i] = __float2bfloat16(pool_smem[i] * scale);
  } else {
    float* o = reinterpret_cast<float*>(out) + static_cast<size_t>(seq) * out_row_stride;
    for (int i = threadIdx.x; i < hidden; i += POOL_THREADS) o[i] = pool_smem[i] * scale;
  }
}

__global__ void __launch_bounds__(ROW_WARPS * 32)
small_proj_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                  const float* __restrict__ bias, int n_rows, int hidden, int n_labels, float* __restrict__ out,
                  int64_t out_row_stride) {
  const int idx = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (idx >= n_rows * n_labels) return;
  const int row = idx / n_labels, label = idx % n_labels;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * hidden;
  const __nv_bfloat16* wr = W + static_cast<size_t>(label) * hidden;
  float acc = 0.f;
  for (int c = lane; c < (hidden >> 3); c += 32) {
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c * 8), a);
    unpack8(__ldg(reinterpret_cast<const uint4*>(wr + c * 8)), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += a[e] * b[e];
  }
  acc = warp_sum(acc);
  if (lane == 0) out[static_cast<size_t>(row) * out_row_stride + label] = acc + (bias != nullptr ? bias[label] : 0.f);
}

// Scores of a classification head, in place on its fp32 logits: softmax over the labels of a row, or the
// logistic function when the head has one output. One warp per row; labels are strided over the lanes.
__global__ void __launch_bounds__(ROW_WARPS * 32)
label_scores_kernel(float* __restrict__ logits, int n_rows, int n_labels, int64_t row_stride) {
  const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  float* r = logits + static_cast<size_t>(row) * row_stride;
  if (n_labels == 1) {
    if (lane == 0) r[0] = 1.f / (1.f + expf(-r[0]));
    return;
  }
  float mx = -INFINITY;
  for (int j = lane; j < n_labels; j += 32) mx = fmaxf(mx, r[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int j = lane; j < n_labels; j += 32) sum += expf(r[j] - mx);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int j = lane; j < n_labels; j += 32) r[j] = expf(r[j] - mx) * inv;
}

// ---- launchers ------------------------------------------------------------------

static int check_hidden(int hidden, int max_chunks_per_lane) {
  if (hidden <= 0 || (hidden % 8) != 0)
    return set_error(B200EMB_ERR_UNSUPPORTED, "hidden size %d must be a positive multiple of 8", hidden);
  if ((hidden >> 3) > 32 * max_chunks_per_lane)
    return set_error(B200EMB_ERR_UNSUPPORTED, "hidden size %d too large for the row kernels", hidden);
  return B200EMB_OK;
}

#define B2_DISPATCH_NCH(nch, CALL)                    \
  switch (nch) {                                      \
    case 1: { constexpr int NCH = 1; CALL; } break;   \
    case 2: { constexpr int NCH = 2; CALL; } break;   \
    case 3: { constexpr int NCH = 3; CALL; } break;   \
    case 4: { constexpr int NCH = 4; CALL; } break;   \
    case 5: case 6: case 7: case 8: { constexpr int NCH = 8; CALL; } break; \
    default: { constexpr int NCH = 16; CALL; } break; \
  }

int launch_embed_ln(const int32_t* ids, const int32_t* types, const int32_t* d_cu, int n_seqs, int n_tokens,
                    const void* word, const void* pos, const void* type_table, const float* gamma, const float* beta,
                    int hidden, int pos_offset, float eps, void* out, cudaStream_t stream, int vocab, int type_vocab,
                    int* err_flag, int n_positions) {
  if (n_tokens <= 0) return B200EMB_OK;
  B2_SET_LIMIT(2, n_positions, stream);
  int rc = check_hidden(hidden, 16);
  if (rc) return rc;
  if (gamma == nullptr && pos == nullptr && type_table == nullptr) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int full = (n_tokens + ROW_WARPS - 1) / ROW_WARPS;
    gather_rows_kernel<<<full < sms * 8 ? full : sms * 8, ROW_WARPS * 32, 0, stream>>>(
        ids, n_tokens, reinterpret_cast<const __nv_bfloat16*>(word), hidden, reinterpret_cast<__nv_bfloat16*>(out), vocab, err_flag);
    cudaError_t eg = cudaGetLastError();
    if (eg != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "gather launch: %s", cudaGetErrorString(eg));
    return B200EMB_OK;
  }
  const int nch = ((hidden >> 3) + 31) / 32;
  const int grid = (n_tokens + ROW_WARPS * EMB_TOK - 1) / (ROW_WARPS * EMB_TOK);
  B2_DISPATCH_NCH(nch, (embed_ln_kernel<NCH><<<grid, ROW_WARPS * 32, 0, stream>>>(
                           ids, types, d_cu, n_seqs, n_tokens, reinterpret_cast<const __nv_bfloat16*>(word),
                           reinterpret_cast<const __nv_bfloat16*>(pos),
                           reinterpret_cast<const __nv_bfloat16*>(type_table), gamma, beta, hidden, pos_offset, eps,
                           reinterpret_cast<__nv_bfloat16*>(out), vocab, type_vocab, err_flag)));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "embed_ln launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_add_ln(const void* x, const void* y, const float* gamma, const float* beta, int n_rows, int hidden,
                  float eps, void* out, cudaStream_t stream) {
  if (n_rows <= 0) return B200EMB_OK;
  int rc = check_hidden(hidden, 16);
  if (rc) return rc;
  const int nch = ((hidden >> 3) + 31) / 32;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int full = (n_rows + ROW_WARPS - 1) / ROW_WARPS;
  const int grid = full < sms * 4 ? full : sms * 4;  // persistent: a few CTAs per SM walk all rows
  const size_t ln_smem = 2 * static_cast<size_t>(hidden) * sizeof(float);
  cudaError_t e = cudaSuccess;
  B2_DISPATCH_NCH(nch, (e = launch_pdl(add_ln_kernel<NCH>, dim3(grid), dim3(ROW_WARPS * 32), ln_smem, stream,
                                       reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(y),
                                       gamma, beta, n_rows, hidden, eps, reinterpret_cast<__nv_bfloat16*>(out))));
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "add_ln launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_add_rmsnorm(float* h, const void* y, const float* gamma, int n_rows, int hidden, float eps, void* out,
                       cudaStream_t stream) {
  if (n_rows <= 0) return B200EMB_OK;
  int rc = check_hidden(hidden, 16);
  if (rc) return rc;
  const int nch = ((hidden >> 3) + 31) / 32;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (hidden > 2048) {
    const int grid_w = n_rows < sms * 8 ? n_rows : sms * 8;
    add_rmsnorm_wide_kernel<<<grid_w, RMS_BLOCK, 0, stream>>>(h, reinterpret_cast<const __nv_bfloat16*>(y), gamma, n_rows,
                                                             hidden, eps, reinterpret_cast<__nv_bfloat16*>(out));
    cudaError_t ew = cudaGetLastError();
    if (ew != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "add_rmsnorm launch: %s", cudaGetErrorString(ew));
    return B200EMB_OK;
  }
  const int full = (n_rows + ROW_WARPS - 1) / ROW_WARPS;
  const int grid = full < sms * 4 ? full : sms * 4;
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  B2_DISPATCH_NCH(nch, (add_rmsnorm_kernel<NCH><<<grid, ROW_WARPS * 32, smem, stream>>>(
                           h, reinterpret_cast<const __nv_bfloat16*>(y), gamma, n_rows, hidden, eps,
                           reinterpret_cast<__nv_bfloat16*>(out))));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "add_rmsnorm launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_widen(const void* x, float* out, size_t n_elems, cudaStream_t stream) {
  if (n_elems == 0) return B200EMB_OK;
  if (n_elems % 8) return set_error(B200EMB_ERR_INVALID, "widen: element count must be a multiple of 8");
  const size_t chunks = n_elems / 8;
  const int grid = static_cast<int>(chunks / 256 + 1 < 148 * 16 ? chunks / 256 + 1 : 148 * 16);
  widen_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, chunks);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "widen launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_rope(void* qkv, const int32_t* d_cu, int n_seqs, int n_tokens, int n_rot_heads, int row_width,
                int head_dim, const float* cos_sin, cudaStream_t stream, int n_positions) {
  if (n_tokens <= 0) return B200EMB_OK;
  B2_SET_LIMIT(1, n_positions, stream);
  if (head_dim % 16 != 0) return set_error(B200EMB_ERR_UNSUPPORTED, "rope: head_dim %d not a multiple of 16", head_dim);
  rope_kernel<<<n_tokens, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(qkv), d_cu, n_seqs, n_tokens, n_rot_heads,
                                           row_width, head_dim, reinterpret_cast<const float2*>(cos_sin));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "rope launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

// One warp per token row: bf16 hidden state -> fp32 output row, optionally divided by max(||row||, 1e-12).
__global__ void __launch_bounds__(ROW_WARPS * 32)
token_rows_kernel(const __nv_bfloat16* __restrict__ x, int n_tokens, int hidden, int normalize,
                  float* __restrict__ out, int64_t out_row_stride) {
  const int lane = threadIdx.x & 31;
  const int n_chunks = hidden >> 3;
  const int warps_total = gridDim.x * ROW_WARPS;
  for (int t = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5); t < n_tokens; t += warps_total) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * hidden);
    float scale = 1.f;
    if (normalize) {
      float ss = 0.f;
      for (int c = lane; c < n_chunks; c += 32) {
        const uint4 u = __ldg(src + c);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      scale = 1.f / fmaxf(sqrtf(ss), 1e-12f);
    }
    float* dst = out + static_cast<size_t>(t) * out_row_stride;
    for (int c = lane; c < n_chunks; c += 32) {
      const uint4 u = __ldg(src + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        dst[c * 8 + 2 * j] = f.x * scale;
        dst[c * 8 + 2 * j + 1] = f.y * scale;
      }
    }
  }
}

int launch_token_rows(const void* x, int n_tokens, int hidden, int normalize, float* out, int64_t out_row_stride,
                      cudaStream_t stream) {
  if (n_tokens <= 0) return B200EMB_OK;
  if (hidden <= 0 || (hidden % 8) != 0) return set_error(B200EMB_ERR_UNSUPPORTED, "token rows: hidden size %d unsupported", hidden);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int full = (n_tokens + ROW_WARPS - 1) / ROW_WARPS;
  const int grid = full < sms * 8 ? full : sms * 8;
  token_rows_kernel<<<grid, ROW_WARPS * 32, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), n_tokens, hidden,
                                                         normalize, out, out_row_stride);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "token rows launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_pool(const void* x, const int32_t* d_cu, int n_seqs, int hidden, int pooling, int normalize, void* out,
                int64_t out_row_stride, int out_bf16, cudaStream_t stream, int n_tokens) {
  if (n_seqs <= 0) return B200EMB_OK;
  B2_SET_LIMIT(0, n_tokens, stream);
  if (hidden <= 0 || (hidden % 8) != 0 || (hidden >> 3) > POOL_THREADS * POOL_MAXC)
    return set_error(B200EMB_ERR_UNSUPPORTED, "pool: hidden size %d unsupported", hidden);
  if (pooling < B200EMB_POOL_CLS || pooling > B200EMB_POOL_LAST)
    return set_error(B200EMB_ERR_INVALID, "pool: unknown pooling %d", pooling);
  const int n_chunks = hidden >> 3;
  const int cols = n_chunks < POOL_THREADS ? n_chunks : POOL_THREADS;
  const size_t smem = (static_cast<size_t>(POOL_THREADS / cols) * hidden + 32) * sizeof(float);
  if (n_chunks > POOL_THREADS)
    pool_kernel<2><<<n_seqs, POOL_THREADS, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), d_cu, hidden,
                                                           pooling, normalize, out, out_row_stride, out_bf16);
  else
    pool_kernel<1><<<n_seqs, POOL_THREADS, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), d_cu, hidden,
                                                           pooling, normalize, out, out_row_stride, out_bf16);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "pool launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

// Output embedding quantisation. One thread per 8 consecutive elements of a row (one packed byte
// for the binary formats, eight bytes for the 8-bit formats).
__global__ void quantize_embeddings_kernel(const float* __restrict__ x, int n_rows, int dim, int64_t x_row_stride,
                                           int precision, const double* __restrict__ ranges,
                                           uint8_t* __restrict__ out, int64_t out_row_stride_bytes) {
  const int groups = dim >> 3;
  const long long total = static_cast<long long>(n_rows) * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / groups), g = static_cast<int>(i % groups);
    const float* src = x + static_cast<size_t>(row) * x_row_stride + g * 8;
    uint8_t* dst = out + static_cast<size_t>(row) * out_row_stride_bytes;
    if (precision == B200EMB_EMB_BINARY || precision == B200EMB_EMB_UBINARY) {
      unsigned bits = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) bits |= (src[j] > 0.f ? 1u : 0u) << (7 - j);  // most significant bit first
      dst[g] = static_cast<uint8_t>(precision == B200EMB_EMB_BINARY ? bits - 128u : bits);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = g * 8 + j;
        const double lo = ranges[c], hi = ranges[dim + c];
        const double step = (hi - lo) / 255.0;
        double v = (static_cast<double>(src[j]) - lo) / step;
        if (precision == B200EMB_EMB_INT8) v -= 128.0;
        // truncation toward zero, then the low 8 bits (what a C cast through a wide integer keeps)
        const long long t = static_cast<long long>(v);
        dst[c] = static_cast<uint8_t>(t & 0xff);
      }
    }
  }
}

int launch_quantize_embeddings(const float* x, int n_rows, int dim, int64_t x_row_stride, int precision,
                               const double* d_ranges, void* out, int64_t out_row_stride_bytes, cudaStream_t stream) {
  if (n_rows <= 0) return B200EMB_OK;
  if (precision < B200EMB_EMB_INT8 || precision > B200EMB_EMB_UBINARY)
    return set_error(B200EMB_ERR_INVALID, "quantize_embeddings: unknown precision %d", precision);
  if (dim <= 0 || (dim % 8) != 0) return set_error(B200EMB_ERR_UNSUPPORTED, "quantize_embeddings: dim %d is not a multiple of 8", dim);
  const bool eight_bit = precision == B200EMB_EMB_INT8 || precision == B200EMB_EMB_UINT8;
  if (eight_bit && d_ranges == nullptr) return set_error(B200EMB_ERR_INVALID, "quantize_embeddings: int8 / uint8 need calibration ranges");
  if (x == nullptr || out == nullptr || x_row_stride < dim || out_row_stride_bytes < (eight_bit ? dim : dim / 8))
    return set_error(B200EMB_ERR_INVALID, "quantize_embeddings: null pointer or row stride too small");
  const long long total = static_cast<long long>(n_rows) * (dim >> 3);
  const int grid = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  quantize_embeddings_kernel<<<grid, 256, 0, stream>>>(x, n_rows, dim, x_row_stride, precision, d_ranges,
                                                       reinterpret_cast<uint8_t*>(out), out_row_stride_bytes);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "quantize_embeddings launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_small_proj(const void* x, const void* W, const float* bias, int n_rows, int hidden, int n_labels,
                      float* out, int64_t out_row_stride, cudaStream_t stream) {
  if (n_rows <= 0 || n_labels <= 0) return B200EMB_OK;
  if ((hidden % 8) != 0) return set_error(B200EMB_ERR_UNSUPPORTED, "small_proj: hidden %d not a multiple of 8", hidden);
  const long long total = static_cast<long long>(n_rows) * n_labels;
  const int grid = static_cast<int>((total + ROW_WARPS - 1) / ROW_WARPS);
  small_proj_kernel<<<grid, ROW_WARPS * 32, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                         reinterpret_cast<const __nv_bfloat16*>(W), bias, n_rows,
                                                         hidden, n_labels, out, out_row_stride);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "small_proj launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_label_scores(float* logits, int n_rows, int n_labels, int64_t row_stride, cudaStream_t stream) {
  if (n_rows <= 0 || n_labels <= 0) return B200EMB_OK;
  const int grid = (n_rows + ROW_WARPS - 1) / ROW_WARPS;
  label_scores_kernel<<<grid, ROW_WARPS * 32, 0, stream>>>(logits, n_rows, n_labels, row_stride);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "label_scores launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int rowops_bounds_status(cudaStream_t stream) {
  (void)stream;
  return B2_TAKE_STATUS(stream);
}

}  // namespace b2
