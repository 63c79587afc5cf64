// GEMM against NVFP4 weights with the expansion inside the kernel:
//   C[M,N] = epilogue(alpha * A[M,K] * dequant(Wq, Ws)[N,K]^T + bias),  A and C bf16.
//
// The weights stay in HBM as stored (e2m1 pairs, one byte per two elements, and one e4m3 scale per 16
// elements): 0.5625 bytes per weight instead of the 2 bytes of an expanded copy, and no expansion pass
// in front of the GEMM. The structure is the CTA-pair bf16 kernel (gemm_bf16.cu: 256 x 256 tiles over two
// CTAs of a cluster, tcgen05 cta_group::2, accumulators in tensor memory, A by TMA) with one more role:
//   warp 0        TMA producer: A tiles only (128 x 64, 128-byte swizzle)
//   warp 1        MMA issuer (the pair's leader issues for both CTAs)
//   warps 2..9    epilogue (bias, alpha = 1 / tensor scale, optional fused SwiGLU, TMA stores)
//   warps 10..17  W converters: two threads per row of the CTA's 128 x 64 half of the W tile, each owning 32
//                 elements. A thread reads its 16 packed bytes and 2 scale bytes with plain loads (two
//                 threads fill one 32-byte sector) FOUR K blocks ahead of the one it expands in registers
//                 (a shared-memory table maps a byte to its two elements as bf16, one copy of the table per
//                 bank so that look-ups never conflict; the block scale is applied by one bf16x2 multiply,
//                 which is exact: the product has at most 6 significant bits), writes four 16-byte
//                 chunks into the stage's B buffer in the 128-byte-swizzled K-major layout a TMA load would
//                 have produced, makes them visible to the tensor cores (fence.proxy.async) and arrives, one
//                 lane per warp, on the pair leader's full barrier. A stage is complete when the A bytes of
//                 both CTAs have landed and all sixteen converter warps of the pair have arrived.
// Expansion costs about 90 instructions per thread and K block, two converter warps per scheduler, against
// the 512 cycles the pair's four 256 x 256 x 16 MMAs take. (Expanding with the conversion instructions -
// e2m1 pair -> half pair, two half -> float, multiply, float pair -> bf16 pair, seven instructions per byte -
// ran the kernel at 450-490 TFLOP/s whatever the number of converter warps and the look-ahead.) The B tile that the tensor cores read is
// bit-identical to the expanded matrix, so the result equals that of the expansion kernel followed by the
// bf16 kernel.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "ptx.cuh"
#include "gemm_tiles.cuh"

namespace b2 {

static constexpr int W4_BN = 256;
static constexpr int W4_CONV_WARPS = 8;
static constexpr int W4_THREADS = GEMM_THREADS + 32 * W4_CONV_WARPS;  // 576
// One stage less than the bf16 pair kernel: the 32 KB it frees hold the expansion table.
struct W4Cfg : GemmCfg<W4_BN, true> {
  static constexpr int STAGES = 5;
  static constexpr int LUT_BYTES = 256 * 32 * 4;  // byte -> two bf16 (its e2m1 pair), one copy per lane = per bank
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * CBUF_BYTES + LUT_BYTES + BIAS_BYTES + BAR_BYTES + 1024;
  static_assert(SMEM_BYTES <= 232448, "shared memory per block");
};

// e2m1 code (sign in bit 3) -> bf16 bits
__device__ __forceinline__ uint32_t e2m1_bf16_bits(uint32_t nib) {
  const uint32_t m = nib & 7u;
  // 0, 0.5, 1, 1.5, 2, 3, 4, 6
  const uint32_t mag = m == 0u ? 0u : (m == 1u ? 0x3F00u : ((m + 252u) << 6));
  return mag | ((nib & 8u) << 12);
}

template <int EPI>
__global__ void __launch_bounds__(W4_THREADS, 1)
gemm_w4_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_c,
                       const uint8_t* __restrict__ wq, const uint8_t* __restrict__ ws, const float* __restrict__ bias,
                       float alpha, int M, int N, int K, int group_m, int* __restrict__ err_flag) {
  using Cfg = W4Cfg;
  constexpr int BN = W4_BN;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int TILE_M = 2 * BM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* cstage = smem + STAGES * Cfg::STAGE_BYTES;
  uint32_t* lut_s = reinterpret_cast<uint32_t*>(cstage + 2 * Cfg::CBUF_BYTES);  // [256][32]
  float* bias_s = reinterpret_cast<float*>(cstage + 2 * Cfg::CBUF_BYTES + Cfg::LUT_BYTES);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(cstage + 2 * Cfg::CBUF_BYTES + Cfg::LUT_BYTES + Cfg::BIAS_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full_bar = empty_bar + STAGES;  // [2]
  uint64_t* acc_empty_bar = acc_full_bar + 2;   // [2]
  uint64_t* drain_bar = acc_empty_bar + 2;      // error path only
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const int m_tiles = (M + TILE_M - 1) / TILE_M;
  const int n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = K / BK;  // the launcher requires K % 64 == 0
  const uint32_t cta_rank = cluster_ctarank();
  const int first_tile = blockIdx.x >> 1;
  const int tile_step = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // leader's full barrier: its producer's arrive.expect_tx + the converter warps of both CTAs
      mbar_init(&full_bar[s], 1 + 2 * W4_CONV_WARPS);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], 2 * N_EPI_WARPS);
    }
    mbar_init(drain_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  // expansion table: entry [byte][lane] = (bf16 of the low nibble) | (bf16 of the high nibble) << 16. Lane l reads
  // word byte * 32 + l, i.e. always bank l: a warp's 32 look-ups never conflict whatever bytes they hold.
  for (int i = threadIdx.x; i < 256 * 32; i += W4_THREADS) {
    const uint32_t byte = static_cast<uint32_t>(i) >> 5;
    lut_s[i] = e2m1_bf16_bits(byte & 15u) | (e2m1_bf16_bits(byte >> 4) << 16);
  }
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer (A only) ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_c);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t issued = 0;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
        const int m0 = mt * TILE_M + static_cast<int>(cta_rank) * BM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
            ok = false;
            break;
          }
          if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::A_BYTES);
          const uint32_t leader_full = mapa_shared(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(smem + stage * Cfg::STAGE_BYTES, &tmap_a, leader_full, kb * BK, m0);
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      pdl_launch_dependents();
      if (!ok) {
        atomicExch(err_flag, 1);
        const uint32_t pending = cta_rank != 0 ? 0u : (issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES);
        for (uint32_t i = 0; i < pending; ++i) {
          const uint32_t idx = issued - 1 - i;
          mbar_wait(&full_bar[idx % STAGES], (idx / STAGES) & 1u);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16_f32(TILE_M, BN);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t smem_base = smem_u32(smem);
      auto wait_all = [](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity)); };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local_tile = 0;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
        const int lt = local_tile++;
        const int acc = lt & 1;
        const uint32_t acc_phase = (lt >> 1) & 1u;
        if (!wait_all(&acc_empty_bar[acc], acc_phase ^ 1u)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_u + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!wait_all(&full_bar[stage], phase)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(b_addr);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (elect_one()) tc_mma_f16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (elect_one()) {
            tc_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 0));
            tc_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 1));
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && elect_one()) {
          tc_commit_pair(mapa_shared(smem_u32(&acc_full_bar[acc]), 0));
          tc_commit_pair(mapa_shared(smem_u32(&acc_full_bar[acc]), 1));
        }
      }
      if (!ok) {
        if (lane == 0) atomicExch(err_flag, 2);
        if (elect_one()) tc_commit_pair(mapa_shared(smem_u32(drain_bar), 0));
        mbar_wait(drain_bar, 0);
      }
    }
  } else if (warp >= 2 + N_EPI_WARPS) {
    // ---------------- W converters ----------------
    const int ct = (warp - 2 - N_EPI_WARPS) * 32 + lane;  // 0..255
    const int row = ct >> 1;                               // row of this CTA's half of the W tile
    const int hx = ct & 1;                                 // which 32 elements of the row's 64
    const size_t q_pitch = static_cast<size_t>(K) >> 1, s_pitch = static_cast<size_t>(K) >> 4;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // packed bytes and scales of the next W4_AHEAD K blocks: a register ring, refilled right after a slot is
    // consumed, so that the loads run W4_AHEAD blocks (about 2000 cycles of MMA work) ahead of the expansion
    constexpr int W4_AHEAD = 4;
    uint4 qr[W4_AHEAD];
    uint32_t sr[W4_AHEAD];
    int f_tile = first_tile, f_kb = 0;  // next block to fetch
    auto fetch = [&](uint4& q, uint32_t& sc) {
      q = make_uint4(0u, 0u, 0u, 0u);
      sc = 0u;
      if (f_tile >= total_tiles) return;
      int mt, nt;
      tile_coords(f_tile, m_tiles, n_tiles, group_m, mt, nt);
      const int wrow = nt * BN + static_cast<int>(cta_rank) * Cfg::B_ROWS + row;
      if (wrow < N) {
        q = __ldg(reinterpret_cast<const uint4*>(wq + static_cast<size_t>(wrow) * q_pitch + f_kb * (BK / 2) + hx * 16));
        sc = __ldg(reinterpret_cast<const uint16_t*>(ws + static_cast<size_t>(wrow) * s_pitch + f_kb * (BK / 16) + hx * 2));
      }
      if (++f_kb == k_blocks) {
        f_kb = 0;
        f_tile += tile_step;
      }
    };
#pragma unroll
    for (int j = 0; j < W4_AHEAD; ++j) fetch(qr[j], sr[j]);
    int my_tiles = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step) ++my_tiles;
    const long long n_blocks = static_cast<long long>(my_tiles) * k_blocks;
    for (long long b0 = 0; b0 < n_blocks && ok; b0 += W4_AHEAD) {
#pragma unroll
      for (int j = 0; j < W4_AHEAD; ++j) {  // static ring index: the slots stay in registers
        if (b0 + j < n_blocks && ok) {
          const uint32_t words[4] = {qr[j].x, qr[j].y, qr[j].z, qr[j].w};
          const uint32_t scales = sr[j];
          fetch(qr[j], sr[j]);  // W4_AHEAD blocks ahead of the one expanded now
          if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1u))) {
            ok = false;
          } else {
            uint8_t* brow = smem + stage * Cfg::STAGE_BYTES + Cfg::A_BYTES + row * 128;
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {  // 16 elements = 8 bytes = two 16-byte chunks of bf16
              const __nv_bfloat16 sb = __float2bfloat16_rn(__half2float(__half(__nv_cvt_fp8_to_halfraw(
                  static_cast<__nv_fp8_storage_t>((scales >> (8 * blk)) & 0xffu), __NV_E4M3))));  // e4m3 is exact in bf16
              const __nv_bfloat162 s2 = __halves2bfloat162(sb, sb);
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                const uint32_t w32 = words[blk * 2 + half];
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const uint32_t pair = lut_s[(((w32 >> (8 * e)) & 0xffu) << 5) | static_cast<uint32_t>(lane)];
                  // element * block scale in bf16 arithmetic: exact (2 x 4 significant bits)
                  const __nv_bfloat162 bb = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pair), s2);
                  o[e] = *reinterpret_cast<const uint32_t*>(&bb);
                }
                const int chunk = hx * 4 + blk * 2 + half;  // 16-byte chunk of the row; 128-byte swizzle: chunk ^ (row & 7)
                *reinterpret_cast<uint4*>(brow + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor cores (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(mapa_shared(smem_u32(&full_bar[stage]), 0));
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
    if (!ok && lane == 0) atomicExch(err_flag, 9);
  } else {
    // ---------------- epilogue ----------------
    const int et = threadIdx.x - 64;  // 0..255
    const int ew = warp - 2;          // 0..7
    const int grp = ew >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    constexpr int SUBS = BN / 64;
    constexpr int SUBS_PER_GROUP = SUBS / 2;
    uint8_t* cbuf = cstage + grp * Cfg::CBUF_BYTES;
    const bool store_thread = lane == 0;
    const int warp_row0 = quarter * 32;
    bool ok = true;
    int local_tile = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step) {
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
      const int lt = local_tile++;
      const int m0 = mt * TILE_M + static_cast<int>(cta_rank) * BM;
      const int n0 = nt * BN;
      const int acc = lt & 1;
      const uint32_t acc_phase = (lt >> 1) & 1u;
      named_barrier_sync(1, 32 * N_EPI_WARPS);
      if (et < BN) bias_s[et] = (bias != nullptr && n0 + et < N) ? __ldg(bias + n0 + et) : 0.f;
      const bool ok_local = mbar_wait(&acc_full_bar[acc], acc_phase);
      ok = named_barrier_and(1, 32 * N_EPI_WARPS, ok_local);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if constexpr (EPI == EPI_BIAS_SWIGLU) {
        // accumulator columns are [gate block | up block] (128 each): output column j = silu(gate_j) * up_j
        const int out_col0 = (n0 >> 1) + grp * 64;
        const bool have = out_col0 < (N >> 1);
        if (have) {
          if (store_thread) tma_store_wait_read();
          __syncwarp();
        }
        uint8_t* rowp = cbuf + row_in_tile * 128;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(t_row + grp * 64 + p * 32, g);
          tmem_ld_32x32b_x32(t_row + BN / 2 + grp * 64 + p * 32, u);
          tmem_ld_wait();
          if (p == 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty_bar[acc]), 0));
          }
          if (have) {
            const float* bg = bias_s + grp * 64 + p * 32;
            const float* bu = bias_s + BN / 2 + grp * 64 + p * 32;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 8; e += 2) {
                const float a0 = silu_f(fmaf(__uint_as_float(g[c * 8 + e]), alpha, bg[c * 8 + e])) *
                                 fmaf(__uint_as_float(u[c * 8 + e]), alpha, bu[c * 8 + e]);
                const float a1 = silu_f(fmaf(__uint_as_float(g[c * 8 + e + 1]), alpha, bg[c * 8 + e + 1])) *
                                 fmaf(__uint_as_float(u[c * 8 + e + 1]), alpha, bu[c * 8 + e + 1]);
                __nv_bfloat162 pr = __floats2bfloat162_rn(a0, a1);
                w[e >> 1] = *reinterpret_cast<uint32_t*>(&pr);
              }
              const int chunk = p * 4 + c;
              *reinterpret_cast<uint4*>(rowp + ((chunk ^ (row_in_tile & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (have) {
          fence_proxy_async_smem();
          __syncwarp();
          if (store_thread && m0 + warp_row0 < M) {
            tma_store_2d(&tmap_c, cbuf + warp_row0 * 128, out_col0, m0 + warp_row0);
            tma_store_commit();
          }
        }
      } else {
#pragma unroll
        for (int st = 0; st < SUBS_PER_GROUP; ++st) {
          const int sub = grp * SUBS_PER_GROUP + st;
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(t_row + sub * 64, r0);
          tmem_ld_32x32b_x32(t_row + sub * 64 + 32, r1);
          tmem_ld_wait();
          if (st == SUBS_PER_GROUP - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty_bar[acc]), 0));
          }
          if (n0 + sub * 64 < N) {
            if (store_thread) tma_store_wait_read();
            __syncwarp();
            const float* bsub = bias_s + sub * 64;
            uint8_t* rowp = cbuf + row_in_tile * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(c < 4 ? r0[c * 8 + e] : r1[(c - 4) * 8 + e]);
              const float4 b0 = *reinterpret_cast<const float4*>(bsub + c * 8);
              const float4 b1 = *reinterpret_cast<const float4*>(bsub + c * 8 + 4);
              v[0] = fmaf(v[0], alpha, b0.x); v[1] = fmaf(v[1], alpha, b0.y);
              v[2] = fmaf(v[2], alpha, b0.z); v[3] = fmaf(v[3], alpha, b0.w);
              v[4] = fmaf(v[4], alpha, b1.x); v[5] = fmaf(v[5], alpha, b1.y);
              v[6] = fmaf(v[6], alpha, b1.z); v[7] = fmaf(v[7], alpha, b1.w);
              uint4 packed;
              packed.x = epilogue_pack2<EPI_BIAS>(v[0], v[1]);
              packed.y = epilogue_pack2<EPI_BIAS>(v[2], v[3]);
              packed.z = epilogue_pack2<EPI_BIAS>(v[4], v[5]);
              packed.w = epilogue_pack2<EPI_BIAS>(v[6], v[7]);
              *reinterpret_cast<uint4*>(rowp + ((c ^ (row_in_tile & 7)) << 4)) = packed;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (store_thread && m0 + warp_row0 < M) {
              tma_store_2d(&tmap_c, cbuf + warp_row0 * 128, n0 + sub * 64, m0 + warp_row0);
              tma_store_commit();
            }
          }
        }
      }
    }
    if (store_thread) tma_store_wait_read();
    if (!ok && lane == 0) atomicExch(err_flag, 3);
  }

  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

int gemm_w4_init_device() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_w4_tcgen05_kernel<EPI_BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Cfg::SMEM_BYTES));
  B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_w4_tcgen05_kernel<EPI_BIAS_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Cfg::SMEM_BYTES));
  return B200EMB_OK;
}

bool gemm_w4_supported(int M, int N, int K, int epi) {
  if (epi != EPI_BIAS && epi != EPI_BIAS_SWIGLU) return false;
  return M > 0 && K % BK == 0 && N % W4_BN == 0;
}

int launch_gemm_w4(const void* A, const void* Wq, const void* Ws, const float* bias, void* C, int M, int N, int K, int epi,
                   float alpha, int sm_count, int* err_flag, cudaStream_t stream) {
  if (M <= 0) return B200EMB_OK;
  if (!gemm_w4_supported(M, N, K, epi))
    return set_error(B200EMB_ERR_UNSUPPORTED, "gemm_w4: needs K %% 64 == 0, N %% 256 == 0 and the bias or SwiGLU epilogue "
                     "(M=%d N=%d K=%d)", M, N, K);
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(Wq) & 15) || (reinterpret_cast<uintptr_t>(Ws) & 3) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (bias && (reinterpret_cast<uintptr_t>(bias) & 15)))
    return set_error(B200EMB_ERR_INVALID, "gemm_w4: pointers must be 16-byte aligned (scales: 4-byte)");
  const int n_out = epi == EPI_BIAS_SWIGLU ? N / 2 : N;
  CUtensorMap ta, tc;
  int rc = make_tmap_bf16_2d(&ta, A, (uint64_t)M, (uint64_t)K, BM);
  if (!rc) rc = make_tmap_bf16_2d(&tc, C, (uint64_t)M, (uint64_t)n_out, 32);
  if (rc) return rc;
  const int tiles = ((M + 255) / 256) * (N / W4_BN);
  int pairs = sm_count / 2;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(W4_THREADS, 1, 1);
  cfg.dynamicSmemBytes = W4Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const uint8_t* q = reinterpret_cast<const uint8_t*>(Wq);
  const uint8_t* s = reinterpret_cast<const uint8_t*>(Ws);
  const int group_m = 16;  // the bf16 kernel's tile order (16 row tiles per group)
  cudaError_t e;
  if (epi == EPI_BIAS_SWIGLU)
    e = cudaLaunchKernelEx(&cfg, gemm_w4_tcgen05_kernel<EPI_BIAS_SWIGLU>, ta, tc, q, s, bias, alpha, M, N, K, group_m, err_flag);
  else
    e = cudaLaunchKernelEx(&cfg, gemm_w4_tcgen05_kernel<EPI_BIAS>, ta, tc, q, s, bias, alpha, M, N, K, group_m, err_flag);
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "gemm_w4 launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

}  // namespace b2
