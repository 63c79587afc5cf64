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
// The kernel is persistent, two CTAs per SM (256 of the 512 TMEM columns each), so one CTA's
// softmax overlaps the other's MMAs; a producer warp keeps the next tiles' Q / K / V in flight.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "ptx.cuh"

namespace b2 {

static constexpr int TC_BKV = 128;
static constexpr int TC_D = 64;
static constexpr int TC_TILE_BYTES = 128 * TC_D * 2;  // 16 KB
static constexpr int TC_QSLOTS = 2;
static constexpr int TC_KVSTAGES = 2;
static constexpr int TC_SMEM_BYTES = (TC_QSLOTS + 2 * TC_KVSTAGES) * TC_TILE_BYTES + 128 + 1024;
static constexpr int TC_THREADS = 160;         // 4 softmax warps + 1 TMA producer warp
static constexpr uint32_t TC_TMEM_COLS = 256;  // S 128 | P 64 | O 64
static constexpr uint32_t TC_S_COL = 0, TC_P_COL = 128, TC_O_COL = 192;

#ifdef B2_ATT_PROFILE
// Phase timing of CTA 0 / thread 0 (development aid; not part of normal builds).
__device__ long long g_att_prof[16];
#define B2_PROF_DECL long long prof_t0 = clock64(); const bool prof_on = (blockIdx.x == 0 && threadIdx.x == 0);
#define B2_PROF(slot) do { if (prof_on) { const long long n__ = clock64(); g_att_prof[slot] += n__ - prof_t0; prof_t0 = n__; } } while (0)
#else
#define B2_PROF_DECL
#define B2_PROF(slot) do { } while (0)
#endif

__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Position of the MMA issuer in the CTA's sequence of (item, key tile) steps.
struct StepCursor {
  int item, it, n_kv, seq_len;
  int qslot, kvstage;
  uint32_t qphase, kvphase;
};

// Persistent: CTA b serves work items b, b + gridDim.x, ...; item i = (query tile i / n_heads,
// head i % n_heads). Warp 4 runs ahead with the TMA loads (Q double-buffered, K/V through a
// two-stage ring, slots released by tcgen05.commit), so launch, allocation and load latency
// are paid once per CTA, not once per tile.
__global__ void __launch_bounds__(TC_THREADS, 2)
attn_tc_d64_kernel(const __grid_constant__ CUtensorMap tmap_qkv, __nv_bfloat16* __restrict__ out,
                   const AttnTile* __restrict__ tiles, int n_items, int n_heads, int n_kv_heads, float scale_log2,
                   int* __restrict__ err_flag) {
  extern __shared__ uint8_t att_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                                // [TC_QSLOTS]
  uint8_t* kv_s = smem + TC_QSLOTS * TC_TILE_BYTES;   // [TC_KVSTAGES] x (K tile, V tile)
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + (TC_QSLOTS + 2 * TC_KVSTAGES) * TC_TILE_BYTES);
  uint64_t* q_empty = q_full + TC_QSLOTS;
  uint64_t* kv_full = q_empty + TC_QSLOTS;
  uint64_t* kv_empty = kv_full + TC_KVSTAGES;
  uint64_t* bar_s = kv_empty + TC_KVSTAGES;
  uint64_t* bar_o = bar_s + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < TC_QSLOTS; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < TC_KVSTAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_qkv);
      int qslot = 0, kvstage = 0;
      uint32_t qphase = 0, kvphase = 0;
      uint32_t q_fills = 0, kv_fills = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const AttnTile t = tiles[item / n_heads];
        const int h = item % n_heads;
        const int hk = h / (n_heads / n_kv_heads);
        const int n_kv = (t.seq_len + TC_BKV - 1) / TC_BKV;
        if (!mbar_wait(&q_empty[qslot], qphase ^ 1u)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&q_full[qslot], TC_TILE_BYTES);
        tma_load_2d(q_s + qslot * TC_TILE_BYTES, &tmap_qkv, &q_full[qslot], h * TC_D, t.seq_start + t.q_start);
        ++q_fills;
        if (++qslot == TC_QSLOTS) {
          qslot = 0;
          qphase ^= 1u;
        }
        for (int it = 0; it < n_kv; ++it) {
          if (!mbar_wait(&kv_empty[kvstage], kvphase ^ 1u)) {
            ok = false;
            break;
          }
          uint8_t* kdst = kv_s + kvstage * 2 * TC_TILE_BYTES;
          mbar_arrive_expect_tx(&kv_full[kvstage], 2 * TC_TILE_BYTES);
          tma_load_2d(kdst, &tmap_qkv, &kv_full[kvstage], (n_heads + hk) * TC_D, t.seq_start + it * TC_BKV);
          tma_load_2d(kdst + TC_TILE_BYTES, &tmap_qkv, &kv_full[kvstage], (n_heads + n_kv_heads + hk) * TC_D,
                      t.seq_start + it * TC_BKV);
          ++kv_fills;
          if (++kvstage == TC_KVSTAGES) {
            kvstage = 0;
            kvphase ^= 1u;
          }
        }
      }
      if (!ok) {
        atomicExch(err_flag, 5);
        // let the copies still in flight land before shared memory is released (bounded)
        for (uint32_t i = 0; i < (q_fills < TC_QSLOTS ? q_fills : (uint32_t)TC_QSLOTS); ++i) {
          const uint32_t idx = q_fills - 1 - i;
          mbar_wait(&q_full[idx % TC_QSLOTS], (idx / TC_QSLOTS) & 1u);
        }
        for (uint32_t i = 0; i < (kv_fills < TC_KVSTAGES ? kv_fills : (uint32_t)TC_KVSTAGES); ++i) {
          const uint32_t idx = kv_fills - 1 - i;
          mbar_wait(&kv_full[idx % TC_KVSTAGES], (idx / TC_KVSTAGES) & 1u);
        }
      }
    }
  } else {
    // ---------------- softmax warps (thread 0 also issues the MMAs) ----------------
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    int kvstage = 0;
    uint32_t gi = 0;  // KV tiles processed so far by this CTA: phase of bar_s / bar_o
    bool failed = false;

    // Thread 0 issues S = Q K^T one step AHEAD of the softmax: S of step k+1 is issued together with
    // P V of step k (the S columns are free once every thread has read them in pass 2), so its
    // round trip hides behind the P V wait and the O update.
    StepCursor cur;
    cur.item = blockIdx.x;
    cur.it = 0;
    cur.n_kv = 0;
    cur.seq_len = 0;
    cur.qslot = cur.kvstage = 0;
    cur.qphase = cur.kvphase = 0;
    auto issue_s = [&]() -> bool {  // false when a wait gave up
      if (cur.item >= n_items) return true;
      if (cur.it == 0) {
        const AttnTile tt = tiles[cur.item / n_heads];
        cur.seq_len = tt.seq_len;
        cur.n_kv = (tt.seq_len + TC_BKV - 1) / TC_BKV;
        if (!mbar_wait(&q_full[cur.qslot], cur.qphase)) return false;
      }
      if (!mbar_wait(&kv_full[cur.kvstage], cur.kvphase)) return false;
      tc_fence_after_sync();
      const int nv = min(TC_BKV, cur.seq_len - cur.it * TC_BKV);
      const uint32_t idesc = make_idesc_bf16_f32(128, (nv + 15) & ~15);
      const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(q_s + cur.qslot * TC_TILE_BYTES));
      const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(kv_s + cur.kvstage * 2 * TC_TILE_BYTES));
#pragma unroll
      for (int k = 0; k < TC_D / 16; ++k)
        tc_mma_f16(tmem_base + TC_S_COL, a_desc + 2 * k, b_desc + 2 * k, idesc, k != 0);
      tc_commit(bar_s);
      if (cur.it == cur.n_kv - 1) tc_commit(&q_empty[cur.qslot]);  // last use of this Q tile
      if (++cur.kvstage == TC_KVSTAGES) {
        cur.kvstage = 0;
        cur.kvphase ^= 1u;
      }
      if (++cur.it == cur.n_kv) {
        cur.it = 0;
        cur.item += gridDim.x;
        if (++cur.qslot == TC_QSLOTS) {
          cur.qslot = 0;
          cur.qphase ^= 1u;
        }
      }
      return true;
    };
    if (threadIdx.x == 0 && !issue_s()) failed = true;
    B2_PROF_DECL
    for (int item = blockIdx.x; item < n_items && !failed; item += gridDim.x) {
      const AttnTile t = tiles[item / n_heads];
      const int h = item % n_heads;
      const int L = t.seq_len;
      const int n_kv = (L + TC_BKV - 1) / TC_BKV;
      const int my_row = t.q_start + warp * 32 + lane;  // query row of this thread within the sequence
      float2 o_reg[TC_D / 2];
#pragma unroll
      for (int j = 0; j < TC_D / 2; ++j) o_reg[j] = make_float2(0.f, 0.f);
      float m_run = -INFINITY, l_run = 0.f;

      for (int it = 0; it < n_kv; ++it, ++gi) {
        const int kv0 = it * TC_BKV;
        const int n_valid = min(TC_BKV, L - kv0);
        const int n_eff = (n_valid + 15) & ~15;
        uint8_t* v_t = kv_s + kvstage * 2 * TC_TILE_BYTES + TC_TILE_BYTES;
        if (!failed && !mbar_wait(bar_s, gi & 1u)) failed = true;
        failed = __any_sync(0xffffffffu, failed);  // keep the warp-collective TMEM accesses below convergent
        tc_fence_after_sync();
        B2_PROF(2);  // S MMA issue -> visible

        float alpha = 1.f, l_add = 0.f;
        // a warp whose 32 query rows all lie past the end of the sequence has nothing to compute
        const bool warp_active = t.q_start + warp * 32 < L;
        if (!failed && warp_active) {
          // pass 1: row maximum over the valid keys (only the last, partial chunk needs masking)
          float mx0 = -INFINITY, mx1 = -INFINITY;
          for (int c = 0; c < n_eff; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_base + TC_S_COL + c, r);
            tmem_ld_wait();
            if (c + 32 <= n_valid) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                mx0 = max3f(mx0, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                mx1 = max3f(mx1, __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) mx0 = fmaxf(mx0, (c + j < n_valid) ? __uint_as_float(r[j]) : -INFINITY);
            }
          }
          B2_PROF(3);  // pass 1
          const float m_new = fmaxf(m_run, fmaxf(mx0, mx1));
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          alpha = ex2f((m_run - m_use) * scale_log2);
          m_run = m_new;
          const float m_scaled = m_use * scale_log2;
          // pass 2: p = exp2(s * scale - m * scale), bf16 pairs into the P columns
          float l0 = 0.f, l1 = 0.f;
          float2 lsum = make_float2(0.f, 0.f);
          const float2 scale2 = make_float2(scale_log2, scale_log2);
          const float2 negm2 = make_float2(-m_scaled, -m_scaled);
          for (int c = 0; c < n_eff; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_base + TC_S_COL + c, r);
            tmem_ld_wait();
            uint32_t pk[16];
            if (c + 32 <= n_valid) {
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                // packed fp32 pair: one FFMA2 / FADD2 per two keys
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), scale2, negm2);
                const float2 pp = make_float2(ex2f(x.x), ex2f(x.y));
                lsum = __fadd2_rn(lsum, pp);
                __nv_bfloat162 b = __floats2bfloat162_rn(pp.x, pp.y);
                pk[j >> 1] = *reinterpret_cast<uint32_t*>(&b);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const float p0 = (c + j < n_valid) ? ex2f(fmaf(__uint_as_float(r[j]), scale_log2, -m_scaled)) : 0.f;
                const float p1 =
                    (c + j + 1 < n_valid) ? ex2f(fmaf(__uint_as_float(r[j + 1]), scale_log2, -m_scaled)) : 0.f;
                l0 += p0;
                l1 += p1;
                __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                pk[j >> 1] = *reinterpret_cast<uint32_t*>(&b);
              }
            }
            tmem_st_32x32b_x16(lane_base + TC_P_COL + (c >> 1), pk);
          }
          l_add = (l0 + l1) + (lsum.x + lsum.y);
          tmem_st_wait();
        }
        B2_PROF(4);  // pass 2
        tc_fence_before_sync();
        // every softmax thread has written its P row (and agrees on whether to go on)
        if (!named_barrier_and(1, 128, !failed)) {
          failed = true;
          break;
        }
        B2_PROF(5);  // barrier
        if (threadIdx.x == 0) {
          tc_fence_after_sync();
          const uint32_t idesc = make_idesc_bf16_f32_b_mn(128, TC_D);
          const uint32_t v_addr = smem_u32(v_t);
          for (int k = 0; k < n_eff / 16; ++k) {
            // 16 keys = two 8-row groups of the MN-major V tile = 2048 bytes; 16 keys of P = 8 columns
            tc_mma_f16_tmem_a(tmem_base + TC_O_COL, tmem_base + TC_P_COL + k * 8,
                              make_mnmajor_sw128_desc(v_addr + k * 2048, 16), idesc, k != 0);
          }
          tc_commit(bar_o);
          tc_commit(&kv_empty[kvstage]);  // both MMAs of this tile have read the K/V stage
          if (!issue_s()) failed = true;  // S of the next step queues up behind P V
        }
        if (!mbar_wait(bar_o, gi & 1u)) failed = true;
        failed = __any_sync(0xffffffffu, failed);
        tc_fence_after_sync();
        B2_PROF(6);  // PV MMA issue -> visible
        if (!failed && warp_active) {
          l_run = l_run * alpha + l_add;
#pragma unroll
          for (int c = 0; c < TC_D; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_base + TC_O_COL + c, r);
            tmem_ld_wait();
            const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
            for (int j = 0; j < 32; j += 2)
              o_reg[(c + j) >> 1] =
                  __ffma2_rn(o_reg[(c + j) >> 1], alpha2, make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
          }
        }
        if (++kvstage == TC_KVSTAGES) kvstage = 0;
        B2_PROF(7);  // O update
      }
      if (!failed && my_row < L) {
        const float inv = 1.f / l_run;
        __nv_bfloat16* dst = out + static_cast<size_t>(t.seq_start + my_row) * (n_heads * TC_D) + h * TC_D;
        const float2 inv2 = make_float2(inv, inv);
#pragma unroll
        for (int c = 0; c < TC_D; c += 8) {
          uint4 u;
          const float2 a0 = __fmul2_rn(o_reg[c / 2], inv2), a1 = __fmul2_rn(o_reg[c / 2 + 1], inv2);
          const float2 a2 = __fmul2_rn(o_reg[c / 2 + 2], inv2), a3 = __fmul2_rn(o_reg[c / 2 + 3], inv2);
          __nv_bfloat162 p0 = __floats2bfloat162_rn(a0.x, a0.y);
          __nv_bfloat162 p1 = __floats2bfloat162_rn(a1.x, a1.y);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(a2.x, a2.y);
          __nv_bfloat162 p3 = __floats2bfloat162_rn(a3.x, a3.y);
          u.x = *reinterpret_cast<uint32_t*>(&p0);
          u.y = *reinterpret_cast<uint32_t*>(&p1);
          u.z = *reinterpret_cast<uint32_t*>(&p2);
          u.w = *reinterpret_cast<uint32_t*>(&p3);
          *reinterpret_cast<uint4*>(dst + c) = u;
        }
      }
    }
    B2_PROF(8);  // output
    if (failed && lane == 0) atomicExch(err_flag, 4);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}

#ifdef B2_ATT_PROFILE
extern "C" int b200emb_debug_att_prof(long long* out16, int reset) {
  if (out16) cudaMemcpyFromSymbol(out16, g_att_prof, sizeof(long long) * 16);
  if (reset) {
    long long z[16] = {};
    cudaMemcpyToSymbol(g_att_prof, z, sizeof(z));
  }
  return 0;
}
#endif

int attention_tc_init_device() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_tc_d64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
  return B200EMB_OK;
}

int launch_attention_tc(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_tokens, int n_heads,
                        int n_kv_heads, int head_dim, int sm_count, int* err_flag, cudaStream_t stream) {
  if (n_tiles <= 0) return B200EMB_OK;
  if (head_dim != TC_D) return set_error(B200EMB_ERR_UNSUPPORTED, "tensor-memory attention is built for head_dim 64");
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535)
    return set_error(B200EMB_ERR_INVALID, "attention: bad head counts %d / %d", n_heads, n_kv_heads);
  CUtensorMap tm;
  const uint64_t width = static_cast<uint64_t>(n_heads + 2 * n_kv_heads) * TC_D;
  int rc = make_tmap_bf16_2d(&tm, qkv, static_cast<uint64_t>(n_tokens), width, 128);
  if (rc) return rc;
  const float scale_log2 = 1.4426950408889634f / 8.0f;  // log2(e) / sqrt(64)
  const long long n_items = static_cast<long long>(n_tiles) * n_heads;
  if (n_items > 0x7fffffffLL) return set_error(B200EMB_ERR_UNSUPPORTED, "attention: too many tiles");
  const int grid = static_cast<int>(n_items < 2LL * sm_count ? n_items : 2LL * sm_count);
  attn_tc_d64_kernel<<<grid, TC_THREADS, TC_SMEM_BYTES, stream>>>(tm, reinterpret_cast<__nv_bfloat16*>(out), d_tiles,
                                                                 static_cast<int>(n_items), n_heads, n_kv_heads,
                                                                 scale_log2, err_flag);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

}  // namespace b2
