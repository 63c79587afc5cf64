// MXFP8 x MXFP8 GEMM on the block-scaled tensor-core path:
//   C[M,N] (bf16) = epilogue( (A_q * 2^sa) (W_q * 2^sw)^T + bias ),  A_q, W_q e4m3, one e8m0 scale per
//   32 consecutive K elements of a row, fp32 accumulation in TMEM.
// tcgen05.mma.kind::mxf8f6f4.block_scale applies the scales in hardware: per 128 x 32 (A) / N x 32 (W)
// block it reads one scale byte per row from tensor memory. Scale factors travel as 512-byte "atoms"
// (128 rows x 4 K-blocks; byte offset (r % 32) * 16 + (r / 32) * 4 + kblock), one bulk copy per stage,
// and are moved shared -> tensor memory with tcgen05.cp (32x128b, broadcast to the four lane quarters).
// Same persistent warp-specialised structure as the bf16 kernel (TMA producer, MMA issuer, 8 epilogue
// warps, two accumulator buffers, shared-memory staged TMA stores); tiles are 128 x 128 x 128.
// Grouped mode (tile_expert) serves the mixture-of-experts layers: one launch over all experts.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "bounds.cuh"
#include "kernels.h"
#include "ptx.cuh"

// expert of a row block as read from tile_expert[]: -1 (unused block) or [0, n_experts); the checked build
// turns anything else into -1 and records it
#define B2_EXPERT(x) (static_cast<int>(B2_IDX(static_cast<long long>(x) + 1, 0, BOUNDS_GEMM_EXPERT)) - 1)

namespace b2 {

static constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;
static constexpr int F8_STAGES = 5;
static constexpr int F8_TILE_BYTES = 128 * 128;  // one A or W tile (fp8)
static constexpr int F8_SF_BYTES = 512;          // one scale-factor atom
static constexpr int F8_CBUF_BYTES = 128 * 64 * 2;
static constexpr int F8_EPI_WARPS = 8;
static constexpr int F8_THREADS = 32 * (2 + F8_EPI_WARPS);
static constexpr int F8_SMEM_BYTES =
    F8_STAGES * (2 * F8_TILE_BYTES + 2 * F8_SF_BYTES) + 2 * F8_CBUF_BYTES + 512 + 256 + 1024;
static constexpr uint32_t F8_TMEM_COLS = 512;  // accumulators [0, 256), scale factors from column 256
static constexpr uint32_t F8_SF_COL = 256;

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// shared -> tensor memory, 32 rows x 16 bytes, replicated into all four 32-lane quarters
__device__ __forceinline__ void tc_copy_sf(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
// un-swizzled K-major descriptor of a 32 x 16-byte block: 8-row core matrices of 128 contiguous bytes
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(16 >> 4) << 16;   // leading byte offset (unused: one core matrix along K)
  d |= static_cast<uint64_t>(128 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
__device__ __forceinline__ void tc_mma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// block-scaled instruction descriptor: e4m3 x e4m3 (format 0), K-major operands, e8m0 scales, K = 32
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int m, int n) {
  return (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24);
}

// erf GELU, same formulation as the bf16 kernel: x (1 + tanh(h(x))) / 2 with h(x) = x * cubic(min(x^2, 25)),
// one tanh.approx.f32 per value
__device__ __forceinline__ float f8_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float2 f8_gelu2(float2 x) {
  const float2 xx = __fmul2_rn(x, x);
  const float2 u = make_float2(fminf(xx.x, 25.f), fminf(xx.y, 25.f));
  float2 p = __ffma2_rn(u, make_float2(-8.666443136e-06f, -8.666443136e-06f), make_float2(-2.5449786335e-04f, -2.5449786335e-04f));
  p = __ffma2_rn(p, u, make_float2(3.672922030e-02f, 3.672922030e-02f));
  p = __ffma2_rn(p, u, make_float2(7.976911068e-01f, 7.976911068e-01f));
  const float2 h = __fmul2_rn(p, x);
  const float2 t = make_float2(f8_tanh(h.x), f8_tanh(h.y));
  const float2 phi = __ffma2_rn(t, make_float2(0.5f, 0.5f), make_float2(0.5f, 0.5f));
  return __fmul2_rn(x, phi);
}
__device__ __forceinline__ size_t sf_atom_offset(size_t row, int kblock, int k_groups) {
  // atom (row / 128, kblock / 4) of 512 bytes; inside: (row % 32) * 16 + ((row % 128) / 32) * 4 + kblock % 4
  return ((row >> 7) * k_groups + (kblock >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kblock & 3);
}

template <int EPI>
__device__ __forceinline__ uint32_t f8_pack2(float a, float b) {
  float2 v = make_float2(a, b);
  if (EPI == EPI_BIAS_GELU) v = f8_gelu2(v);
  __nv_bfloat162 p = __floats2bfloat162_rn(v.x, v.y);
  return *reinterpret_cast<uint32_t*>(&p);
}

// OUT_FP8: the result is written as MXFP8 as well (e4m3 bytes through tmap_c, which then describes a
// byte matrix, plus e8m0 scales into out_sf_atoms in atom layout), ready to be the next GEMM's A operand.
template <int EPI, bool OUT_FP8>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_c, const uint8_t* __restrict__ sfa_atoms,
                  const uint8_t* __restrict__ sfw_atoms, const float* __restrict__ bias, int M, int N, int K,
                  const int32_t* __restrict__ tile_expert, uint8_t* __restrict__ out_sf_atoms,
                  int* __restrict__ err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tiles = smem;
  uint8_t* w_tiles = a_tiles + F8_STAGES * F8_TILE_BYTES;
  uint8_t* cstage = w_tiles + F8_STAGES * F8_TILE_BYTES;  // 2 x 16 KB
  uint8_t* sfa_s = cstage + 2 * F8_CBUF_BYTES;            // [F8_STAGES][512]
  uint8_t* sfw_s = sfa_s + F8_STAGES * F8_SF_BYTES;
  float* bias_s = reinterpret_cast<float*>(sfw_s + F8_STAGES * F8_SF_BYTES);  // [128]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(bias_s) + 512);
  uint64_t* empty_bar = full_bar + F8_STAGES;
  uint64_t* acc_full_bar = empty_bar + F8_STAGES;
  uint64_t* acc_empty_bar = acc_full_bar + 2;
  uint64_t* drain_bar = acc_empty_bar + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform in the compiler's view too
  const int lane = threadIdx.x & 31;
  const int m_tiles = (M + F8_BM - 1) / F8_BM;
  const int n_tiles = (N + F8_BN - 1) / F8_BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = K / F8_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], F8_EPI_WARPS);
    }
    mbar_init(drain_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, F8_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_c);
      int stage = 0;
      uint32_t phase = 0, issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mb = tile / n_tiles;
        const int m0 = mb * F8_BM;
        const int n0 = (tile % n_tiles) * F8_BN;
        const int expert = tile_expert != nullptr ? B2_EXPERT(__ldg(tile_expert + mb)) : 0;
        if (expert < 0) continue;
        const int w_row0 = expert * N + n0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_bar[stage], 2 * F8_TILE_BYTES + 2 * F8_SF_BYTES);
          tma_load_2d(a_tiles + stage * F8_TILE_BYTES, &tmap_a, &full_bar[stage], kb * F8_BK, m0);
          tma_load_2d(w_tiles + stage * F8_TILE_BYTES, &tmap_w, &full_bar[stage], kb * F8_BK, w_row0);
          bulk_load_1d(sfa_s + stage * F8_SF_BYTES, sfa_atoms + (static_cast<size_t>(mb) * k_blocks + kb) * F8_SF_BYTES,
                       F8_SF_BYTES, &full_bar[stage]);
          bulk_load_1d(sfw_s + stage * F8_SF_BYTES,
                       sfw_atoms + (static_cast<size_t>(w_row0 / 128) * k_blocks + kb) * F8_SF_BYTES, F8_SF_BYTES,
                       &full_bar[stage]);
          ++issued;
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        atomicExch(err_flag, 1);
        const uint32_t pending = issued < (uint32_t)F8_STAGES ? issued : (uint32_t)F8_STAGES;
        for (uint32_t i = 0; i < pending; ++i) {
          const uint32_t idx = issued - 1 - i;
          mbar_wait(&full_bar[idx % F8_STAGES], (idx / F8_STAGES) & 1u);
        }
      }
    }
  } else if (warp == 1) {
    // MMA issuer: all 32 lanes walk the loops (warp-uniform code keeps descriptors and addresses in uniform
    // registers), one elected lane issues each tcgen05 instruction. A stage is two scale-factor copies and
    // four 128 x 128 x 32 MMAs of 64 cycles each; issued from divergent single-thread code every one of the
    // six instructions costs about 90 cycles of operand moves, which made the issuer the bottleneck.
    {
      constexpr uint32_t idesc = make_idesc_mxf8(F8_BM, F8_BN);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t a_base = smem_u32(a_tiles), w_base = smem_u32(w_tiles);
      const uint32_t sfa_base = smem_u32(sfa_s), sfw_base = smem_u32(sfw_s);
      auto wait_all = [](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity)); };
      int stage = 0, local_tile = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (tile_expert != nullptr && __shfl_sync(0xffffffffu, B2_EXPERT(__ldg(tile_expert + tile / n_tiles)), 0) < 0) continue;
        const int lt = local_tile++;
        const int acc = lt & 1;
        if (!wait_all(&acc_empty_bar[acc], ((lt >> 1) & 1u) ^ 1u)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_u + acc * F8_BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!wait_all(&full_bar[stage], phase)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sfa_t = tmem_u + F8_SF_COL + stage * 8;
          const uint32_t sfw_t = sfa_t + 4;
          const uint64_t sfa_desc = make_sf_desc(sfa_base + stage * F8_SF_BYTES);
          const uint64_t sfw_desc = make_sf_desc(sfw_base + stage * F8_SF_BYTES);
          const uint64_t a_desc = make_kmajor_sw128_desc(a_base + stage * F8_TILE_BYTES);
          const uint64_t b_desc = make_kmajor_sw128_desc(w_base + stage * F8_TILE_BYTES);
          if (elect_one()) {
            tc_copy_sf(sfa_t, sfa_desc);
            tc_copy_sf(sfw_t, sfw_desc);
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // K block k of this stage: 32 bytes further along the swizzled row; scale byte k of each 32-bit word
            const uint32_t id = idesc | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4);
            if (elect_one()) tc_mma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, id, sfa_t, sfw_t, (kb | k) != 0 ? 1u : 0u);
          }
          if (elect_one()) tc_commit(&empty_bar[stage]);
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && elect_one()) tc_commit(&acc_full_bar[acc]);
      }
      if (!ok) {
        if (lane == 0) atomicExch(err_flag, 2);
        if (elect_one()) tc_commit(drain_bar);
        mbar_wait(drain_bar, 0);
      }
    }
  } else {
    const int et = threadIdx.x - 64;
    const int ew = warp - 2;
    const int grp = ew >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    uint8_t* cbuf = cstage + grp * F8_CBUF_BYTES;
    const bool store_thread = (ew & 3) == 0 && lane == 0;
    bool ok = true;
    int local_tile = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int expert = tile_expert != nullptr ? B2_EXPERT(__ldg(tile_expert + tile / n_tiles)) : 0;
      if (expert < 0) continue;
      const int lt = local_tile++;
      const int m0 = (tile / n_tiles) * F8_BM;
      const int n0 = (tile % n_tiles) * F8_BN;
      const int acc = lt & 1;
      named_barrier_sync(1, 32 * F8_EPI_WARPS);
      if (et < F8_BN) bias_s[et] = (bias != nullptr && n0 + et < N) ? __ldg(bias + expert * N + n0 + et) : 0.f;
      const bool ok_local = mbar_wait(&acc_full_bar[acc], (lt >> 1) & 1u);
      ok = named_barrier_and(1, 32 * F8_EPI_WARPS, ok_local);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * F8_BN + grp * 64;
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(t_row, r0);
      tmem_ld_32x32b_x32(t_row + 32, r1);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
      if (n0 + grp * 64 < N) {
        if (store_thread) tma_store_wait_read();
        named_barrier_sync(2 + grp, 128);
        const float* bsub = bias_s + grp * 64;
        if constexpr (OUT_FP8) {
          // this thread's 64 columns = two 32-element blocks of its row: one e8m0 scale each
          uint8_t* rowp = cbuf + row_in_tile * 64;  // un-swizzled 64-byte rows
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            float v[32];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              float2 t = make_float2(__uint_as_float(blk == 0 ? r0[e] : r1[e]) + bsub[blk * 32 + e],
                                     __uint_as_float(blk == 0 ? r0[e + 1] : r1[e + 1]) + bsub[blk * 32 + e + 1]);
              if (EPI == EPI_BIAS_GELU) t = f8_gelu2(t);
              v[e] = t.x;
              v[e + 1] = t.y;
            }
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(v[e]));
            int ex = -127;
            if (amax > 0.f) {
              ex = ilogbf(amax) - 8;
              ex = ex < -127 ? -127 : (ex > 127 ? 127 : ex);
            }
            const float inv = ex == -127 ? 0.f : exp2f(static_cast<float>(-ex));
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[i * 4] * inv, v[i * 4 + 1] * inv), __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[i * 4 + 2] * inv, v[i * 4 + 3] * inv), __NV_SATFINITE, __NV_E4M3);
              w[i] = (lo & 0xffffu) | ((hi & 0xffffu) << 16);
            }
            *reinterpret_cast<uint4*>(rowp + blk * 32) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(rowp + blk * 32 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
            const size_t grow = static_cast<size_t>(m0 + row_in_tile);
            const int kblock = ((n0 + grp * 64) >> 5) + blk;
            out_sf_atoms[sf_atom_offset(grow, kblock, N >> 7)] = static_cast<uint8_t>(ex + 127);
          }
        } else {
        uint8_t* rowp = cbuf + row_in_tile * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(c < 4 ? r0[c * 8 + e] : r1[(c - 4) * 8 + e]) + bsub[c * 8 + e];
          uint4 packed;
          packed.x = f8_pack2<EPI>(v[0], v[1]);
          packed.y = f8_pack2<EPI>(v[2], v[3]);
          packed.z = f8_pack2<EPI>(v[4], v[5]);
          packed.w = f8_pack2<EPI>(v[6], v[7]);
          *reinterpret_cast<uint4*>(rowp + ((c ^ (row_in_tile & 7)) << 4)) = packed;
        }
        }
        fence_proxy_async_smem();
        named_barrier_sync(2 + grp, 128);
        if (store_thread) {
          tma_store_2d(&tmap_c, cbuf, n0 + grp * 64, m0);
          tma_store_commit();
        }
      }
    }
    if (store_thread) tma_store_wait_read();
    if (!ok && lane == 0) atomicExch(err_flag, 3);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, F8_TMEM_COLS);
  }
}

// ---- activation quantiser and scale-factor repacking ---------------------------------------------


// x bf16 [rows, K] -> e4m3 [rows, K] + e8m0 scales in atom layout (same rule as the weight quantiser)
__global__ void __launch_bounds__(256)
quant_act_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, size_t rows, int K, uint8_t* __restrict__ q,
                       uint8_t* __restrict__ sf_atoms) {
  const int kblocks = K / 32;
  const size_t b = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (b >= rows * kblocks) return;
  const size_t row = b / kblocks;
  const int kb = static_cast<int>(b % kblocks);
  float v[32];
  const uint4* src = reinterpret_cast<const uint4*>(x + b * 32);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 u = src[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(p[j]);
      v[i * 8 + 2 * j] = t.x;
      v[i * 8 + 2 * j + 1] = t.y;
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(v[e]));
  int ex = -127;
  if (amax > 0.f) {
    ex = ilogbf(amax) - 8;
    ex = ex < -127 ? -127 : (ex > 127 ? 127 : ex);
  }
  const float inv = ex == -127 ? 0.f : exp2f(static_cast<float>(-ex));
  uint32_t out[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      const uint32_t two =
          __nv_cvt_float2_to_fp8x2(make_float2(v[i * 4 + j] * inv, v[i * 4 + j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      word |= (two & 0xffffu) << (8 * j);
    }
    out[i] = word;
  }
  uint4* dst = reinterpret_cast<uint4*>(q + b * 32);
  dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
  dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
  sf_atoms[sf_atom_offset(row, kb, K / 128)] = static_cast<uint8_t>(ex + 127);
}

// row-major scales [rows, K / 32] -> atom layout
__global__ void sf_to_atoms_kernel(const uint8_t* __restrict__ scales, size_t rows, int kblocks, uint8_t* __restrict__ atoms) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= rows * kblocks) return;
  atoms[sf_atom_offset(i / kblocks, static_cast<int>(i % kblocks), kblocks / 4)] = scales[i];
}

size_t mxfp8_sf_atoms_bytes(int64_t rows, int64_t K) {
  return static_cast<size_t>((rows + 127) / 128) * static_cast<size_t>(K / 128) * 512;
}

int launch_quant_act_mxfp8(const void* x, int64_t rows, int K, void* q, void* sf_atoms, cudaStream_t stream) {
  if (rows <= 0) return B200EMB_OK;
  if (K % 128) return set_error(B200EMB_ERR_INVALID, "mxfp8 activations: K = %d must be a multiple of 128", K);
  const size_t blocks = static_cast<size_t>(rows) * (K / 32);
  quant_act_mxfp8_kernel<<<static_cast<unsigned int>((blocks + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), static_cast<size_t>(rows), K, reinterpret_cast<uint8_t*>(q),
      reinterpret_cast<uint8_t*>(sf_atoms));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "mxfp8 activation quantiser launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int launch_sf_to_atoms(const void* scales, int64_t rows, int K, void* atoms, cudaStream_t stream) {
  if (rows <= 0) return B200EMB_OK;
  if (K % 128) return set_error(B200EMB_ERR_INVALID, "mxfp8 scales: K = %d must be a multiple of 128", K);
  const size_t n = static_cast<size_t>(rows) * (K / 32);
  sf_to_atoms_kernel<<<static_cast<unsigned int>((n + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(scales), static_cast<size_t>(rows), K / 32, reinterpret_cast<uint8_t*>(atoms));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "scale repack launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

// ---- host side ---------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn8)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_tmap_u8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols = 128,
                           bool swizzle = true) {
  const TmapKey key{base, rows, cols, 128u, box_cols, swizzle ? 1u : 2u};
  if (tmap_cache_get(key, out)) return B200EMB_OK;
  static EncodeTiledFn8 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn8>(p);
  }
  if (fn == nullptr) return set_error(B200EMB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {box_cols, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(B200EMB_ERR_CUDA, "cuTensorMapEncodeTiled (u8) failed (%d)", (int)r);
  tmap_cache_put(key, out);
  return B200EMB_OK;
}

int gemm_mxfp8_init_device() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel<EPI_BIAS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES));
  B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel<EPI_BIAS_GELU, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES));
  B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel<EPI_BIAS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES));
  B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel<EPI_BIAS_GELU, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES));
  return B200EMB_OK;
}

int launch_gemm_mxfp8(const void* Aq, const void* sfa_atoms, const void* Wq, const void* sfw_atoms, const float* bias,
                      void* C, int M, int N, int K, int epi, int sm_count, int* err_flag, cudaStream_t stream,
                      const int32_t* tile_expert, int n_experts, void* out_sf_atoms) {
  if (M <= 0) return B200EMB_OK;
  if (N <= 0 || K <= 0 || (K % 128) != 0 || (N % 8) != 0)
    return set_error(B200EMB_ERR_INVALID, "mxfp8 gemm: need K %% 128 == 0 and N %% 8 == 0 (N=%d K=%d)", N, K);
  if (tile_expert != nullptr && (N % F8_BN) != 0)
    return set_error(B200EMB_ERR_INVALID, "grouped mxfp8 gemm: N = %d must be a multiple of %d", N, F8_BN);
  if (tile_expert == nullptr && (N % 128) != 0)
    return set_error(B200EMB_ERR_INVALID, "mxfp8 gemm: N = %d must be a multiple of 128 (scale-factor atoms)", N);
  if (epi != EPI_BIAS && epi != EPI_BIAS_GELU) return set_error(B200EMB_ERR_UNSUPPORTED, "mxfp8 gemm: epilogue %d not built", epi);
  CUtensorMap ta, tw, tc;
  int rc = make_tmap_u8_2d(&ta, Aq, (uint64_t)M, (uint64_t)K);
  if (rc) return rc;
  if (tile_expert != nullptr) B2_SET_LIMIT(0, static_cast<long long>(n_experts) + 1, stream);  // values are expert + 1
  rc = make_tmap_u8_2d(&tw, Wq, (uint64_t)N * (tile_expert != nullptr ? n_experts : 1), (uint64_t)K);
  if (rc) return rc;
  const bool out_fp8 = out_sf_atoms != nullptr;
  if (out_fp8 && (N % 128) != 0) return set_error(B200EMB_ERR_INVALID, "mxfp8 gemm: MXFP8 output needs N %% 128 == 0");
  rc = out_fp8 ? make_tmap_u8_2d(&tc, C, (uint64_t)M, (uint64_t)N, 64, false) : make_tmap_bf16_2d(&tc, C, (uint64_t)M, (uint64_t)N, 128);
  if (rc) return rc;
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int grid = tiles < sm_count ? tiles : sm_count;
  const uint8_t* sa = reinterpret_cast<const uint8_t*>(sfa_atoms);
  const uint8_t* sw = reinterpret_cast<const uint8_t*>(sfw_atoms);
  uint8_t* osf = reinterpret_cast<uint8_t*>(out_sf_atoms);
  if (epi == EPI_BIAS_GELU && out_fp8)
    gemm_mxfp8_kernel<EPI_BIAS_GELU, true><<<grid, F8_THREADS, F8_SMEM_BYTES, stream>>>(ta, tw, tc, sa, sw, bias, M, N, K, tile_expert, osf, err_flag);
  else if (epi == EPI_BIAS_GELU)
    gemm_mxfp8_kernel<EPI_BIAS_GELU, false><<<grid, F8_THREADS, F8_SMEM_BYTES, stream>>>(ta, tw, tc, sa, sw, bias, M, N, K, tile_expert, osf, err_flag);
  else if (out_fp8)
    gemm_mxfp8_kernel<EPI_BIAS, true><<<grid, F8_THREADS, F8_SMEM_BYTES, stream>>>(ta, tw, tc, sa, sw, bias, M, N, K, tile_expert, osf, err_flag);
  else
    gemm_mxfp8_kernel<EPI_BIAS, false><<<grid, F8_THREADS, F8_SMEM_BYTES, stream>>>(ta, tw, tc, sa, sw, bias, M, N, K, tile_expert, osf, err_flag);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "mxfp8 gemm launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int gemm_mxfp8_bounds_status(cudaStream_t stream) {
  (void)stream;
  return B2_TAKE_STATUS(stream);
}

}  // namespace b2
