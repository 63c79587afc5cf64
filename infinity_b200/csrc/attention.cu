// Variable-length attention over a packed qkv stream: softmax(Q K^T / sqrt(d)) V per sequence,
// bidirectional (encoders) or causal with grouped-query heads (decoder-style embedders).
//
// One CTA = one 64-row query tile of one (sequence, head); tiles never cross a sequence
// boundary (the host builds the tile list from cu_seqlens). 4 warps x 16 query rows.
// K/V tiles of 64 keys stream through a double-buffered shared-memory ring with cp.async;
// S = Q K^T and O += P V run on mma.sync m16n8k16 (bf16 in, fp32 accumulate) with an online
// softmax in registers (exp2 with the scale folded in). Rows are padded by 16 bytes in shared
// memory, which makes every ldmatrix phase conflict-free for d = 32, 64 and 128.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "kernels.h"
#include "ptx.cuh"

namespace b2 {

static constexpr int ATT_BQ = 64;
static constexpr int ATT_BKV = 64;
static constexpr int ATT_THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_ptr)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_ptr)));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Copies rows [row0, row0 + 64) x D of one head into padded shared memory; rows past the
// sequence end are zero-filled (source size 0) with the source address clamped to row 0.
template <int D>
__device__ __forceinline__ void load_rows(__nv_bfloat16* dst, const __nv_bfloat16* base, int row_stride, int row0,
                                          int seq_len) {
  constexpr int LD = D + 8;
  constexpr int CHUNKS = D / 8;
  for (int i = threadIdx.x; i < 64 * CHUNKS; i += ATT_THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const int row = row0 + r;
    const bool valid = row < seq_len;
    const __nv_bfloat16* src = base + static_cast<size_t>(valid ? row : 0) * row_stride + c * 8;
    cp_async16(dst + r * LD + c * 8, src, valid ? 16 : 0);
  }
}

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(ATT_THREADS)
attn_varlen_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out,
                   const AttnTile* __restrict__ tiles, int n_heads, int n_kv_heads, float scale_log2) {
  constexpr int LD = D + 8;
  extern __shared__ __align__(16) uint8_t att_smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(att_smem);
  __nv_bfloat16* Ks = Qs + ATT_BQ * LD;
  __nv_bfloat16* Vs = Ks + 2 * ATT_BKV * LD;

  pdl_wait();  // qkv is the previous kernel's result
  pdl_launch_dependents();
  const AttnTile t = tiles[blockIdx.x];
  const int h = blockIdx.y;
  const int hk = h / (n_heads / n_kv_heads);
  const int row_stride = (n_heads + 2 * n_kv_heads) * D;
  const __nv_bfloat16* qbase = qkv + static_cast<size_t>(t.seq_start) * row_stride + h * D;
  const __nv_bfloat16* kbase = qkv + static_cast<size_t>(t.seq_start) * row_stride + (n_heads + hk) * D;
  const __nv_bfloat16* vbase = kbase + n_kv_heads * D;
  const int L = t.seq_len;
  const int q0 = t.q_start;
  const int kv_end = CAUSAL ? min(L, q0 + ATT_BQ) : L;
  const int n_kv = (kv_end + ATT_BKV - 1) / ATT_BKV;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;

  load_rows<D>(Qs, qbase, row_stride, q0, L);
  load_rows<D>(Ks, kbase, row_stride, 0, L);
  load_rows<D>(Vs, vbase, row_stride, 0, L);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();

  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = kk * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qf[kk], Qs + r * LD + c);
  }

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int qrow0 = q0 + warp * 16 + g;  // this thread's rows: qrow0 and qrow0 + 8

  for (int it = 0; it < n_kv; ++it) {
    const int buf = it & 1;
    const __nv_bfloat16* Kt = Ks + buf * ATT_BKV * LD;
    const __nv_bfloat16* Vt = Vs + buf * ATT_BKV * LD;
    if (it + 1 < n_kv) {
      load_rows<D>(Ks + (buf ^ 1) * ATT_BKV * LD, kbase, row_stride, (it + 1) * ATT_BKV, L);
      load_rows<D>(Vs + (buf ^ 1) * ATT_BKV * LD, vbase, row_stride, (it + 1) * ATT_BKV, L);
      cp_async_commit();
    }

    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        uint32_t b[4];
        const int r = jp * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = kk * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(b, Kt + r * LD + c);
        mma_bf16_16816(s[2 * jp], qf[kk], b[0], b[1]);
        mma_bf16_16816(s[2 * jp + 1], qf[kk], b[2], b[3]);
      }
    }

    // mask (sequence end, causal diagonal) and online softmax
    const int key0 = it * ATT_BKV + 2 * tq;
    float mx[2] = {-INFINITY, -INFINITY};
    // only the last key tile (sequence end) and, for causal attention, the tile on the diagonal need a mask
    const bool needs_mask = (it + 1) * ATT_BKV > L || (CAUSAL && (it + 1) * ATT_BKV > q0 + warp * 16 + 1);
    if (needs_mask) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + 8 * j + (e & 1);
          const int qr = qrow0 + (e >> 1) * 8;
          const bool keep = key < L && (!CAUSAL || key <= qr);
          const float v = keep ? s[j][e] : -INFINITY;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;  // fully masked row (only rows past the sequence end)
      corr[r] = fast_exp2((m_run[r] - m_use[r]) * scale_log2);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= corr[0];
      o[j][1] *= corr[0];
      o[j][2] *= corr[1];
      o[j][3] *= corr[1];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = fast_exp2((s[j][e] - m_use[e >> 1]) * scale_log2);
        s[j][e] = p;
        l_run[e >> 1] += p;
      }
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < ATT_BKV / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b[4];
        const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dp * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(b, Vt + r * LD + c);
        mma_bf16_16816(o[2 * dp], a, b[0], b[1]);
        mma_bf16_16816(o[2 * dp + 1], a, b[2], b[3]);
      }
    }

    if (it + 1 < n_kv) cp_async_wait_all();
    __syncthreads();
  }

  // finalise: divide by the row sums and write bf16
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const int out_stride = n_heads * D;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qr = qrow0 + r * 8;
    if (qr < L) {
      const float inv = 1.f / l_run[r];
      __nv_bfloat16* dst = out + static_cast<size_t>(t.seq_start + qr) * out_stride + h * D + 2 * tq;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        *reinterpret_cast<uint32_t*>(dst + 8 * j) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
      }
    }
  }
}

template <int D>
static constexpr int att_smem_bytes() {
  return (ATT_BQ + 4 * ATT_BKV) * (D + 8) * 2;
}

int attention_tile_rows(int head_dim, int causal) {
  return (head_dim == 64 || head_dim == 128 || (head_dim == 32 && !causal)) ? 128 : ATT_BQ;
}

int attention_build_tiles_q(const int32_t* cu, int n_seqs, int bq, AttnTile* tiles) {
  // Longest sequences first, so the most expensive tiles start early and the tail is short.
  std::vector<int> order(n_seqs);
  for (int i = 0; i < n_seqs; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(),
                   [&](int a, int b) { return (cu[a + 1] - cu[a]) > (cu[b + 1] - cu[b]); });
  int n = 0;
  for (int idx = 0; idx < n_seqs; ++idx) {
    const int i = order[idx];
    const int len = cu[i + 1] - cu[i];
    for (int q = 0; q < len; q += bq) {
      if (tiles != nullptr) tiles[n] = AttnTile{cu[i], len, q, 0};
      ++n;
    }
  }
  return n;
}

int attention_init_device() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_varlen_kernel<32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     att_smem_bytes<32>()));
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_varlen_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     att_smem_bytes<64>()));
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_varlen_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     att_smem_bytes<128>()));
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_varlen_kernel<32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     att_smem_bytes<32>()));
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_varlen_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     att_smem_bytes<64>()));
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_varlen_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     att_smem_bytes<128>()));
  return B200EMB_OK;
}

template <int D>
static int launch_d(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_heads, int n_kv_heads,
                    int causal, cudaStream_t stream) {
  const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  dim3 grid(n_tiles, n_heads);
  const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(qkv);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  cudaError_t e;
  if (causal)
    e = launch_pdl(attn_varlen_kernel<D, true>, grid, dim3(ATT_THREADS), att_smem_bytes<D>(), stream, q, o, d_tiles,
                   n_heads, n_kv_heads, scale_log2);
  else
    e = launch_pdl(attn_varlen_kernel<D, false>, grid, dim3(ATT_THREADS), att_smem_bytes<D>(), stream, q, o, d_tiles,
                   n_heads, n_kv_heads, scale_log2);
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_attention(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_heads, int n_kv_heads,
                     int head_dim, int causal, cudaStream_t stream) {
  if (n_tiles <= 0) return B200EMB_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
    return set_error(B200EMB_ERR_INVALID, "attention: n_heads %d must be a multiple of n_kv_heads %d", n_heads,
                     n_kv_heads);
  if (n_heads > 65535) return set_error(B200EMB_ERR_UNSUPPORTED, "attention: too many heads");
  switch (head_dim) {
    case 32: return launch_d<32>(qkv, out, d_tiles, n_tiles, n_heads, n_kv_heads, causal, stream);
    case 64: return launch_d<64>(qkv, out, d_tiles, n_tiles, n_heads, n_kv_heads, causal, stream);
    case 128: return launch_d<128>(qkv, out, d_tiles, n_tiles, n_heads, n_kv_heads, causal, stream);
  }
  return set_error(B200EMB_ERR_UNSUPPORTED, "attention: head_dim %d not in {32, 64, 128}", head_dim);
}

}  // namespace b2
