// Variable-length bidirectional attention on the 5th-generation tensor cores (head_dim 64).
//
// One CTA = one 128-row query tile of one (sequence, head); tiles never cross a sequence
// boundary. Q, K and V tiles (128 rows x 64, 128-byte swizzle) arrive by TMA straight from the
// packed qkv buffer. Per 128-key tile:
//   S = Q K^T      tcgen05.mma 128 x N x 16 (N = valid keys rounded up to 16), fp32 in TMEM
//   softmax        128 threads, one TMEM lane (= one query row) each: two passes over the row
//                  (max, then exp2 / sum), no cross-thread reduction; P is rounded to bf16 and
//                  written back to tensor memory (two keys per 32-bit column)
//   O_tile = P V   tcgen05.mma with the A operand read from tensor memory and V as an MN-major
//                  shared-memory operand (no transpose of V anywhere)
//   O = O * alpha + O_tile in registers (online softmax; nothing to rescale in TMEM)
// Two CTAs share an SM (256 of the 512 TMEM columns each), so one CTA's softmax overlaps the
// other's MMAs. K/V tiles are double-buffered.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "ptx.cuh"

namespace b2 {

static constexpr int TC_BQ = 128;
static constexpr int TC_BKV = 128;
static constexpr int TC_D = 64;
static constexpr int TC_TILE_BYTES = 128 * TC_D * 2;  // 16 KB
static constexpr int TC_SMEM_BYTES = 5 * TC_TILE_BYTES + 128 + 1024;
static constexpr uint32_t TC_TMEM_COLS = 256;  // S 128 | P 64 | O 64
static constexpr uint32_t TC_S_COL = 0, TC_P_COL = 128, TC_O_COL = 192;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(128, 2)
attn_tc_d64_kernel(const __grid_constant__ CUtensorMap tmap_qkv, __nv_bfloat16* __restrict__ out,
                   const AttnTile* __restrict__ tiles, int n_heads, int n_kv_heads, float scale_log2,
                   int* __restrict__ err_flag) {
  extern __shared__ uint8_t att_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = smem + TC_TILE_BYTES;      // [2]
  uint8_t* v_s = smem + 3 * TC_TILE_BYTES;  // [2]
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + 5 * TC_TILE_BYTES);
  uint64_t* bar_kv = bar_q + 1;  // [2]
  uint64_t* bar_s = bar_q + 3;
  uint64_t* bar_o = bar_q + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 5);

  const AttnTile t = tiles[blockIdx.x];
  const int h = blockIdx.y;
  const int hk = h / (n_heads / n_kv_heads);
  const int L = t.seq_len, q0 = t.q_start;
  const int n_kv = (L + TC_BKV - 1) / TC_BKV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_col = h * TC_D;
  const int k_col = (n_heads + hk) * TC_D;
  const int v_col = (n_heads + n_kv_heads + hk) * TC_D;
  const int row0 = t.seq_start;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_qkv);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  int kv_issued = 0;  // K/V tiles requested so far (thread 0)
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_q, TC_TILE_BYTES);
    tma_load_2d(q_s, &tmap_qkv, bar_q, q_col, row0 + q0);
    for (; kv_issued < 2 && kv_issued < n_kv; ++kv_issued) {
      mbar_arrive_expect_tx(&bar_kv[kv_issued], 2 * TC_TILE_BYTES);
      tma_load_2d(k_s + kv_issued * TC_TILE_BYTES, &tmap_qkv, &bar_kv[kv_issued], k_col, row0 + kv_issued * TC_BKV);
      tma_load_2d(v_s + kv_issued * TC_TILE_BYTES, &tmap_qkv, &bar_kv[kv_issued], v_col, row0 + kv_issued * TC_BKV);
    }
  }

  float o_reg[TC_D];
#pragma unroll
  for (int j = 0; j < TC_D; ++j) o_reg[j] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  bool failed = false;
  const int my_row = q0 + warp * 32 + lane;  // query row of this thread, relative to the sequence

  for (int it = 0; it < n_kv; ++it) {
    const int buf = it & 1;
    const int kv0 = it * TC_BKV;
    const int n_valid = min(TC_BKV, L - kv0);
    const int n_eff = (n_valid + 15) & ~15;
    if (threadIdx.x == 0) {
      bool ok = true;
      if (it == 0) ok = mbar_wait(bar_q, 0);
      ok = ok && mbar_wait(&bar_kv[buf], (it >> 1) & 1);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t idesc = make_idesc_bf16_f32(128, n_eff);
        const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(q_s));
        const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(k_s + buf * TC_TILE_BYTES));
#pragma unroll
        for (int k = 0; k < TC_D / 16; ++k) tc_mma_f16(tmem_base + TC_S_COL, a_desc + 2 * k, b_desc + 2 * k, idesc, k != 0);
        tc_commit(bar_s);
      } else {
        failed = true;
      }
    }
    if (!failed && !mbar_wait(bar_s, it & 1)) failed = true;
    tc_fence_after_sync();

    float alpha = 1.f, l_add = 0.f, m_use = 0.f;
    if (!failed) {
      // pass 1: row maximum over the valid keys
      float mx = -INFINITY;
      for (int c = 0; c < n_eff; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + TC_S_COL + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) mx = fmaxf(mx, (c + j < n_valid) ? __uint_as_float(r[j]) : -INFINITY);
      }
      const float m_new = fmaxf(m_run, mx);
      m_use = (m_new == -INFINITY) ? 0.f : m_new;
      alpha = ex2f((m_run - m_use) * scale_log2);
      m_run = m_new;
      const float m_scaled = m_use * scale_log2;
      // pass 2: p = exp2(s * scale - m * scale), bf16 pairs into the P columns
      for (int c = 0; c < n_eff; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + TC_S_COL + c, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = (c + j < n_valid) ? ex2f(fmaf(__uint_as_float(r[j]), scale_log2, -m_scaled)) : 0.f;
          const float p1 = (c + j + 1 < n_valid) ? ex2f(fmaf(__uint_as_float(r[j + 1]), scale_log2, -m_scaled)) : 0.f;
          l_add += p0 + p1;
          __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
          pk[j >> 1] = *reinterpret_cast<uint32_t*>(&b);
        }
        tmem_st_32x32b_x16(lane_base + TC_P_COL + (c >> 1), pk);
      }
      tmem_st_wait();
    }
    tc_fence_before_sync();
    if (__syncthreads_or(failed ? 1 : 0)) {
      failed = true;
      break;
    }
    if (threadIdx.x == 0) {
      tc_fence_after_sync();
      const uint32_t idesc = make_idesc_bf16_f32_b_mn(128, TC_D);
      const uint32_t v_addr = smem_u32(v_s + buf * TC_TILE_BYTES);
      for (int k = 0; k < n_eff / 16; ++k) {
        // 16 keys = two 8-row groups of the MN-major V tile = 2048 bytes; 16 keys of P = 8 columns
        tc_mma_f16_tmem_a(tmem_base + TC_O_COL, tmem_base + TC_P_COL + k * 8, make_mnmajor_sw128_desc(v_addr + k * 2048, 16),
                          idesc, k != 0);
      }
      tc_commit(bar_o);
    }
    if (!mbar_wait(bar_o, it & 1)) failed = true;
    tc_fence_after_sync();
    if (threadIdx.x == 0 && !failed && kv_issued < n_kv) {
      // both MMAs of this tile have read K/V[buf]: refill it with tile it + 2
      mbar_arrive_expect_tx(&bar_kv[buf], 2 * TC_TILE_BYTES);
      tma_load_2d(k_s + buf * TC_TILE_BYTES, &tmap_qkv, &bar_kv[buf], k_col, row0 + kv_issued * TC_BKV);
      tma_load_2d(v_s + buf * TC_TILE_BYTES, &tmap_qkv, &bar_kv[buf], v_col, row0 + kv_issued * TC_BKV);
      ++kv_issued;
    }
    if (!failed) {
      l_run = l_run * alpha + l_add;
#pragma unroll
      for (int c = 0; c < TC_D; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + TC_O_COL + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) o_reg[c + j] = fmaf(o_reg[c + j], alpha, __uint_as_float(r[j]));
      }
    }
  }

  failed = __syncthreads_or(failed ? 1 : 0) != 0;
  if (failed) {
    if (threadIdx.x == 0) {
      atomicExch(err_flag, 4);
      // let copies that are still in flight land before shared memory is released
      mbar_wait(bar_q, 0);
      for (int i = max(0, kv_issued - 2); i < kv_issued; ++i) mbar_wait(&bar_kv[i & 1], (i >> 1) & 1);
    }
  } else if (my_row < L) {
    const float inv = 1.f / l_run;
    __nv_bfloat16* dst = out + static_cast<size_t>(row0 + my_row) * (n_heads * TC_D) + h * TC_D;
#pragma unroll
    for (int c = 0; c < TC_D; c += 8) {
      uint4 u;
      __nv_bfloat162 p0 = __floats2bfloat162_rn(o_reg[c] * inv, o_reg[c + 1] * inv);
      __nv_bfloat162 p1 = __floats2bfloat162_rn(o_reg[c + 2] * inv, o_reg[c + 3] * inv);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(o_reg[c + 4] * inv, o_reg[c + 5] * inv);
      __nv_bfloat162 p3 = __floats2bfloat162_rn(o_reg[c + 6] * inv, o_reg[c + 7] * inv);
      u.x = *reinterpret_cast<uint32_t*>(&p0);
      u.y = *reinterpret_cast<uint32_t*>(&p1);
      u.z = *reinterpret_cast<uint32_t*>(&p2);
      u.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(dst + c) = u;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}

int attention_tc_init_device() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_tc_d64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
  return B200EMB_OK;
}

int launch_attention_tc(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_tokens, int n_heads,
                        int n_kv_heads, int head_dim, int* err_flag, cudaStream_t stream) {
  if (n_tiles <= 0) return B200EMB_OK;
  if (head_dim != TC_D) return set_error(B200EMB_ERR_UNSUPPORTED, "tensor-memory attention is built for head_dim 64");
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535)
    return set_error(B200EMB_ERR_INVALID, "attention: bad head counts %d / %d", n_heads, n_kv_heads);
  CUtensorMap tm;
  const uint64_t width = static_cast<uint64_t>(n_heads + 2 * n_kv_heads) * TC_D;
  int rc = make_tmap_bf16_2d(&tm, qkv, static_cast<uint64_t>(n_tokens), width, 128);
  if (rc) return rc;
  const float scale_log2 = 1.4426950408889634f / 8.0f;  // log2(e) / sqrt(64)
  dim3 grid(n_tiles, n_heads);
  attn_tc_d64_kernel<<<grid, 128, TC_SMEM_BYTES, stream>>>(tm, reinterpret_cast<__nv_bfloat16*>(out), d_tiles, n_heads,
                                                           n_kv_heads, scale_log2, err_flag);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

}  // namespace b2
