// bf16 GEMM for sm_100a: C[M,N] = epilogue(A[M,K] * W[N,K]^T + bias).
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0        TMA producer: streams 128x64 A tiles and BNx64 W tiles (128-byte swizzle)
//                 through a STAGES-deep shared-memory ring, one mbarrier pair per slot
//   warp 1        allocates TMEM and issues tcgen05.mma (128 x BN x 16 per instruction,
//                 fp32 accumulators in TMEM); two accumulator buffers so the epilogue of
//                 tile i overlaps the MMAs of tile i+1
//   warps 2..9    epilogue, two groups of four warps: tcgen05.ld the accumulator (one TMEM lane =
//                 one output row per thread, 64 columns at a time), release the accumulator,
//                 add the bias (staged in shared memory), apply GELU / tanh, round to bf16,
//                 write a 128x64 sub-tile into 128-byte-swizzled shared memory and hand it to
//                 a TMA store (one staging buffer per group, re-used once its store has read it)
// CTA-pair variant (PAIR, large problems): two CTAs of a cluster own one 256 x 256 tile
// (tcgen05 cta_group::2). Each CTA loads its 128 rows of A and HALF of the W tile (32 KB per
// stage instead of 48 KB, six stages instead of four); both CTAs' TMA loads complete on the
// leader's full barrier, the leader's MMA warp issues the 256 x 256 x 16 MMAs for the pair and
// commits onto both CTAs' empty / accumulator-full barriers, each CTA runs the epilogue of its own
// 128 accumulator rows and releases the accumulator on the leader's barrier. No multicast load.
// M is ragged (token count): TMA zero-fills rows past M on loads and clips them on stores.
// No cluster launch, no multicast: each CTA issues its own loads; W tiles are re-used
// out of L2.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "bounds.cuh"
#include "kernels.h"
#include "ptx.cuh"

// expert of a row block as read from tile_expert[]: -1 (unused block) or [0, n_experts); the checked build
// turns anything else into -1 and records it
#define B2_EXPERT(x) (static_cast<int>(B2_IDX(static_cast<long long>(x) + 1, 0, BOUNDS_GEMM_EXPERT)) - 1)
#include "gemm_tiles.cuh"

namespace b2 {

template <int BN, int EPI, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ CUtensorMap tmap_c, const float* __restrict__ bias, float alpha, int M, int N,
                         int K, const int32_t* __restrict__ tile_expert, int group_m, int* __restrict__ err_flag) {
  using Cfg = GemmCfg<BN, PAIR>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int TILE_M = PAIR ? 2 * BM : BM;  // rows of one scheduled tile (both CTAs of a pair)
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles must start on a 1024-byte boundary.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* cstage = smem + STAGES * Cfg::STAGE_BYTES;  // 2 x 16 KB, each 1024-byte aligned
  float* bias_s = reinterpret_cast<float*>(cstage + 2 * Cfg::CBUF_BYTES);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(cstage + 2 * Cfg::CBUF_BYTES + Cfg::BIAS_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full_bar = empty_bar + STAGES;  // [2]
  uint64_t* acc_empty_bar = acc_full_bar + 2;   // [2]
  uint64_t* drain_bar = acc_empty_bar + 2;  // error path only: MMAs in flight before TMEM is freed
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform in the compiler's view too
  const int lane = threadIdx.x & 31;
  const int m_tiles = (M + TILE_M - 1) / TILE_M;
  const int n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;       // 0 = leader of the pair
  const int first_tile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;  // tiles are dealt to pairs
  const int tile_step = PAIR ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], PAIR ? 2 * N_EPI_WARPS : N_EPI_WARPS);  // pair: both CTAs' epilogue warps
    }
    mbar_init(drain_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_base_slot, Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if (PAIR) cluster_sync_all();  // the peer's barriers exist before anything is signalled on them
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  // The set-up above touched no global memory: it may overlap the tail of the previous kernel in the stream.
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_c);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t issued = 0;  // slots filled so far (for draining on the error path)
      // pair: both CTAs' loads complete on the leader's full barrier, which expects both stages' bytes
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
        const int m0 = mt * TILE_M + static_cast<int>(cta_rank) * BM;
        const int n0 = nt * BN;
        // grouped mode: row block m0/BM belongs to expert e (its weights are rows [e*N, e*N + N) of W);
        // e < 0 marks an unused row block, skipped by every role alike
        const int expert = tile_expert != nullptr ? B2_EXPERT(__ldg(tile_expert + mt)) : 0;
        if (expert < 0) continue;
        const int w_row0 = expert * N + n0 + static_cast<int>(cta_rank) * Cfg::B_ROWS * (PAIR ? 1 : 0);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          if (PAIR) {
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);
            const uint32_t leader_full = mapa_shared(smem_u32(&full_bar[stage]), 0);
            tma_load_2d_pair(a_dst, &tmap_a, leader_full, kb * BK, m0);
            tma_load_2d_pair(b_dst, &tmap_w, leader_full, kb * BK, w_row0);
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
            tma_load_2d(a_dst, &tmap_a, &full_bar[stage], kb * BK, m0);
            tma_load_2d(b_dst, &tmap_w, &full_bar[stage], kb * BK, w_row0);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Every load of this CTA has been issued: the next kernel in the stream may be scheduled and do its
      // set-up while the last tiles finish (triggering at the top of the kernel instead, which parks the
      // next kernel's CTAs beside this one from the start, measured 1.5 % slower on a small-batch forward).
      pdl_launch_dependents();
      if (!ok) {
        atomicExch(err_flag, 1);
        // Let the copies already in flight land before this CTA's shared memory is released:
        // wait (bounded) on the full barrier of every slot filled in the last lap.
        const uint32_t pending = (PAIR && cta_rank != 0) ? 0u : (issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES);
        for (uint32_t i = 0; i < pending; ++i) {
          const uint32_t idx = issued - 1 - i;  // i-th most recent fill
          mbar_wait(&full_bar[idx % STAGES], (idx / STAGES) & 1u);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // All 32 lanes walk the loops (warp-uniform code: descriptors and addresses stay in uniform registers)
    // and one elected lane issues each tcgen05 instruction. Issued from divergent single-thread code an
    // MMA costs about 90 cycles of operand moves, which leaves no slack against the 128 cycles a
    // 128 x 256 x 16 MMA takes to execute.
    if (cta_rank == 0) {  // pair: the leader issues the MMAs of both CTAs
      constexpr uint32_t idesc = make_idesc_bf16_f32(TILE_M, BN);
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t smem_base = smem_u32(smem);
      auto wait_all = [](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity)); };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local_tile = 0;
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
        if (tile_expert != nullptr) {
          int mt, nt;
          tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
          if (__shfl_sync(0xffffffffu, B2_EXPERT(__ldg(tile_expert + mt)), 0) < 0) continue;
        }
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
            // advancing 16 elements along K inside the 128-byte swizzle span = +32 bytes = +2 encoded
            if (elect_one()) {
              if (PAIR) tc_mma_f16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
              else tc_mma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          // slot is free once these MMAs have read it (pair: in both CTAs)
          if (elect_one()) {
            if (PAIR) {
              tc_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 0));
              tc_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 1));
            } else {
              tc_commit(&empty_bar[stage]);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && elect_one()) {  // accumulator complete
          if (PAIR) {
            tc_commit_pair(mapa_shared(smem_u32(&acc_full_bar[acc]), 0));
            tc_commit_pair(mapa_shared(smem_u32(&acc_full_bar[acc]), 1));
          } else {
            tc_commit(&acc_full_bar[acc]);
          }
        }
      }
      if (!ok) {
        if (lane == 0) atomicExch(err_flag, 2);
        // MMAs already issued must finish before the accumulators are freed
        if (elect_one()) {
          if (PAIR) tc_commit_pair(mapa_shared(smem_u32(drain_bar), 0));
          else tc_commit(drain_bar);
        }
        mbar_wait(drain_bar, 0);
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int et = threadIdx.x - 64;  // 0..255
    const int ew = warp - 2;          // 0..7
    const int grp = ew >> 2;          // two groups of four warps
    const int quarter = warp & 3;     // TMEM lane quarter this warp may read
    const int row_in_tile = quarter * 32 + lane;
    constexpr int SUBS = BN / 64;                               // 64-column sub-tiles per tile
    constexpr int SUBS_PER_GROUP = (SUBS >= 2) ? SUBS / 2 : 1;  // BN = 64: group 1 has none
    uint8_t* cbuf = cstage + grp * Cfg::CBUF_BYTES;
    // each epilogue warp stages and stores its own 32 rows (TMA box of 32 x 64): no barrier between warps
    const bool store_thread = lane == 0;
    const int warp_row0 = quarter * 32;
    bool ok = true;
    int local_tile = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step) {
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
      const int expert = tile_expert != nullptr ? B2_EXPERT(__ldg(tile_expert + mt)) : 0;
      if (expert < 0) continue;
      const int lt = local_tile++;
      const int m0 = mt * TILE_M + static_cast<int>(cta_rank) * BM;
      const int n0 = nt * BN;
      const int acc = lt & 1;
      const uint32_t acc_phase = (lt >> 1) & 1u;
      named_barrier_sync(1, 32 * N_EPI_WARPS);  // everyone is done with the previous tile's bias
      if (et < BN) bias_s[et] = (bias != nullptr && n0 + et < N) ? __ldg(bias + expert * N + n0 + et) : 0.f;
      const bool ok_local = mbar_wait(&acc_full_bar[acc], acc_phase);
      // one decision for all epilogue threads (also publishes the bias): leave together or not at all
      ok = named_barrier_and(1, 32 * N_EPI_WARPS, ok_local);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if constexpr (EPI == EPI_BIAS_SWIGLU) {
        // The tile's accumulator columns are [gate block | up block] (BN/2 each): output column j of
        // this tile = silu(gate_j) * up_j. Group g owns output columns [64 g, 64 g + 64).
        const int out_col0 = (n0 >> 1) + grp * 64;
        const bool have = (grp * 64 < BN / 2) && out_col0 < (N >> 1);  // uniform within the group
        if (have) {
          if (store_thread) tma_store_wait_read();  // this warp's previous store has read its rows
          __syncwarp();
        }
        uint8_t* rowp = cbuf + row_in_tile * 128;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          uint32_t g[32], u[32];
          if (grp * 64 < BN / 2) {
            tmem_ld_32x32b_x32(t_row + grp * 64 + p * 32, g);
            tmem_ld_32x32b_x32(t_row + BN / 2 + grp * 64 + p * 32, u);
            tmem_ld_wait();
          }
          if (p == 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty_bar[acc]), 0));  // the leader's barrier
            else mbar_arrive(&acc_empty_bar[acc]);
          }
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
        if (sub < SUBS) {
          tmem_ld_32x32b_x32(t_row + sub * 64, r0);
          tmem_ld_32x32b_x32(t_row + sub * 64 + 32, r1);
          tmem_ld_wait();
        }
        if (st == SUBS_PER_GROUP - 1) {
          // the accumulator is in registers: hand the TMEM buffer back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty_bar[acc]), 0));  // the leader's barrier
            else mbar_arrive(&acc_empty_bar[acc]);
          }
        }
        if (sub < SUBS && n0 + sub * 64 < N) {  // uniform within the group
          if (store_thread) tma_store_wait_read();  // this warp's previous store has read its rows
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
            packed.x = epilogue_pack2<EPI>(v[0], v[1]);
            packed.y = epilogue_pack2<EPI>(v[2], v[3]);
            packed.z = epilogue_pack2<EPI>(v[4], v[5]);
            packed.w = epilogue_pack2<EPI>(v[6], v[7]);
            // 128-byte swizzle: 16-byte chunk c of row r lives at chunk (c ^ (r & 7))
            *reinterpret_cast<uint4*>(rowp + ((c ^ (row_in_tile & 7)) << 4)) = packed;
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA (async proxy)
          __syncwarp();
          if (store_thread && m0 + warp_row0 < M) {
            tma_store_2d(&tmap_c, cbuf + warp_row0 * 128, n0 + sub * 64, m0 + warp_row0);
            tma_store_commit();
          }
        }
      }
      }
    }
    if (store_thread) tma_store_wait_read();  // shared memory must outlive the last stores' reads
    if (!ok && lane == 0) atomicExch(err_flag, 3);
  }

  tc_fence_before_sync();
  if (PAIR) cluster_sync_all();  // neither CTA leaves while the other may still touch its memory or barriers
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

namespace {
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.cols + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= ((static_cast<uint64_t>(k.box_rows) << 40 | static_cast<uint64_t>(k.box_cols) << 16 | k.kind) + (h << 6) + (h >> 2));
    return static_cast<size_t>(h);
  }
};
struct TmapKeyEq {
  bool operator()(const TmapKey& a, const TmapKey& b) const {
    return a.base == b.base && a.rows == b.rows && a.cols == b.cols && a.box_rows == b.box_rows && a.box_cols == b.box_cols &&
           a.kind == b.kind;
  }
};
std::mutex g_tmap_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash, TmapKeyEq> g_tmaps;
uint64_t g_tmap_hits = 0, g_tmap_misses = 0;
constexpr size_t TMAP_CACHE_LIMIT = 16384;
}  // namespace

bool tmap_cache_get(const TmapKey& key, CUtensorMap_st* out) {
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  auto it = g_tmaps.find(key);
  if (it == g_tmaps.end()) {
    ++g_tmap_misses;
    return false;
  }
  ++g_tmap_hits;
  memcpy(out, &it->second, sizeof(CUtensorMap));
  return true;
}

void tmap_cache_put(const TmapKey& key, const CUtensorMap_st* tm) {
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  if (g_tmaps.size() >= TMAP_CACHE_LIMIT) g_tmaps.clear();
  memcpy(&g_tmaps[key], tm, sizeof(CUtensorMap));
}

void tmap_cache_stats(uint64_t* hits, uint64_t* misses) {
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  *hits = g_tmap_hits;
  *misses = g_tmap_misses;
}

// bf16 row-major [rows, cols] matrix, box = [box_rows, 64 columns], 128-byte swizzle; loads zero-fill
// outside the matrix, stores are clipped.
int make_tmap_bf16_2d(CUtensorMap_st* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  const TmapKey key{base, rows, cols, box_rows, static_cast<uint32_t>(BK), 0u};
  if (tmap_cache_get(key, out)) return B200EMB_OK;
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return set_error(B200EMB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(B200EMB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  tmap_cache_put(key, out);
  return B200EMB_OK;
}

// Row tiles per group of the tile order. Measured on the Qwen2-7B and BERT-large GEMM shapes (group sizes 1 to
// 32, interleaved runs): 16 is best or within 1 % of the best everywhere; the gate/up GEMM (W = 271 MB) runs
// 35.2 ms with row-major order and 28.3 ms with 16, the down projection (K = 18944) 17.0 -> 15.7 ms.
static int pick_group_m(int /*tile_rows*/, int /*K*/) { return 16; }

// Pair kernels are launched as clusters of two CTAs; the number of resident pairs is queried once per device.
template <int BN, int EPI>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& tc, const float* bias, float alpha,
                       int M, int N, int K, int sm_count, int* err_flag, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, true>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, EPI, true>;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int pairs = sm_count / 2;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
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
  const int32_t* no_experts = nullptr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tw, tc, bias, alpha, M, N, K, no_experts, pick_group_m(2 * BM, K), err_flag);
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "gemm pair launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

template <int BN, int EPI>
static int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& tc, const float* bias, float alpha,
                      int M, int N, int K, const int32_t* tile_expert, int sm_count, int* err_flag, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, EPI, false>;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int grid = tiles < sm_count ? tiles : sm_count;
  cudaError_t e = launch_pdl(kern, dim3(grid), dim3(GEMM_THREADS), Cfg::SMEM_BYTES, stream, ta, tw, tc, bias, alpha, M, N, K,
                             tile_expert, pick_group_m(BM, K), err_flag);
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "gemm launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

template <int BN>
static int launch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& tc, const float* bias,
                      float alpha, int M, int N, int K, const int32_t* tile_expert, int sm_count, int* err_flag,
                      cudaStream_t stream, bool pair = false) {
  if constexpr (BN == 256) {
    if (pair) {
      switch (epi) {
        case EPI_BIAS: return launch_pair<BN, EPI_BIAS>(ta, tw, tc, bias, alpha, M, N, K, sm_count, err_flag, stream);
        case EPI_BIAS_GELU: return launch_pair<BN, EPI_BIAS_GELU>(ta, tw, tc, bias, alpha, M, N, K, sm_count, err_flag, stream);
        case EPI_BIAS_TANH: return launch_pair<BN, EPI_BIAS_TANH>(ta, tw, tc, bias, alpha, M, N, K, sm_count, err_flag, stream);
        case EPI_BIAS_SWIGLU: return launch_pair<BN, EPI_BIAS_SWIGLU>(ta, tw, tc, bias, alpha, M, N, K, sm_count, err_flag, stream);
      }
      return set_error(B200EMB_ERR_INVALID, "unknown epilogue %d", epi);
    }
  }
  switch (epi) {
    case EPI_BIAS: return launch_cfg<BN, EPI_BIAS>(ta, tw, tc, bias, alpha, M, N, K, tile_expert, sm_count, err_flag, stream);
    case EPI_BIAS_GELU: return launch_cfg<BN, EPI_BIAS_GELU>(ta, tw, tc, bias, alpha, M, N, K, tile_expert, sm_count, err_flag, stream);
    case EPI_BIAS_TANH: return launch_cfg<BN, EPI_BIAS_TANH>(ta, tw, tc, bias, alpha, M, N, K, tile_expert, sm_count, err_flag, stream);
    case EPI_BIAS_SWIGLU:
      if constexpr (BN == 256) return launch_cfg<BN, EPI_BIAS_SWIGLU>(ta, tw, tc, bias, alpha, M, N, K, tile_expert, sm_count, err_flag, stream);
      break;
  }
  return set_error(B200EMB_ERR_INVALID, "unknown epilogue %d", epi);
}

template <int BN, int EPI>
static int init_one() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     GemmCfg<BN>::SMEM_BYTES));
  if constexpr (BN == 256) {
    B2_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       GemmCfg<BN, true>::SMEM_BYTES));
  }
  return B200EMB_OK;
}
template <int BN>
static int init_bn() {
  int rc = init_one<BN, EPI_BIAS>();
  if (!rc) rc = init_one<BN, EPI_BIAS_GELU>();
  if (!rc) rc = init_one<BN, EPI_BIAS_TANH>();
  if constexpr (BN == 256) {
    if (!rc) rc = init_one<BN, EPI_BIAS_SWIGLU>();
  }
  return rc;
}
int gemm_init_device() {
  int rc = init_bn<256>();
  if (!rc) rc = init_bn<128>();
  if (!rc) rc = init_bn<64>();
  return rc;
}

// Tile width. The rule: the widest tile whose grid still fills the machine at least once; small problems take
// narrower tiles. For short reductions (K <= 512: the hidden-384 / 512 encoders) a 256-wide tile has six to eight K
// blocks, fill and epilogue weigh as much as the MMAs, and the count of rounds of the persistent grid decides: there a
// small cost model chooses, rounds x (fixed part + K / 16 steps), with the fixed part growing with the width
// (300 + 5 cycles per column: the epilogue of the last round is not overlapped) and 128, 76 and 55 cycles per step for
// 256, 128 and 64 columns; the 256-wide tile is counted with CTA pairs when the launcher would use them. Measured on the
// bge-small shapes at 7.7 k tokens (N = 1152 and 1536, K = 384: three rounds of pair tiles against four and five of
// tiles half as wide): 128 takes 7 % off the forward. For K >= 1024 the same model was measured wrong (narrow tiles
// stream twice the operand bytes per flop and lose 3-19 % from 5 k tokens on), so it is not consulted there.
int gemm_pick_bn(int M, int N, int K, int sm_count, bool grouped) {
  // Diagnostic override for tuning runs: B200EMB_GEMM_BN_MAP="N:K:width,N:K:width,..." (width 64, 128 or 256).
  for (const char* e = getenv("B200EMB_GEMM_BN_MAP"); e != nullptr && *e != 0;) {
    int n = 0, k = 0, b = 0;
    if (sscanf(e, "%d:%d:%d", &n, &k, &b) == 3 && n == N && k == K && (b == 64 || b == 128 || b == 256)) return b;
    e = strchr(e, ',');
    if (e != nullptr) ++e;
  }
  const long long m_tiles = (M + BM - 1) / BM;
  if (K > 512 || grouped) {
    if (m_tiles * ((N + 255) / 256) >= sm_count) return 256;
    if (m_tiles * ((N + 127) / 128) >= sm_count) return 128;
    return 64;
  }
  const long long k_steps = (K + 15) / 16;
  auto rounds = [&](long long tiles, long long units) { return (tiles + units - 1) / units; };
  const long long pair_tiles = ((M + 255) / 256) * static_cast<long long>((N + 255) / 256);
  const bool pairs = pair_tiles >= sm_count / 2;
  const long long r256 = pairs ? rounds(pair_tiles, sm_count / 2) : rounds(m_tiles * ((N + 255) / 256), sm_count);
  if (r256 >= 8) return 256;  // many rounds: the waves no longer matter
  const long long c256 = r256 * (300 + 5 * 256 + k_steps * 128);
  const long long c128 = rounds(m_tiles * ((N + 127) / 128), sm_count) * (300 + 5 * 128 + k_steps * 76);
  const long long c64 = rounds(m_tiles * ((N + 63) / 64), sm_count) * (300 + 5 * 64 + k_steps * 55);
  if (c256 <= c128 && c256 <= c64) return 256;
  return c128 <= c64 ? 128 : 64;
}

int launch_gemm_bf16(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int epi,
                     int sm_count, int* err_flag, cudaStream_t stream, int force_bn, float alpha,
                     const int32_t* tile_expert, int n_experts) {
  if (M <= 0) return B200EMB_OK;
  if (N <= 0 || K <= 0 || (K % 8) != 0 || (N % 8) != 0)
    return set_error(B200EMB_ERR_INVALID, "gemm: need N, K > 0 and multiples of 8 (N=%d K=%d)", N, K);
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (bias && (reinterpret_cast<uintptr_t>(bias) & 15)))
    return set_error(B200EMB_ERR_INVALID, "gemm: pointers must be 16-byte aligned");
  // force_bn 257 = CTA-pair kernel (256-wide tiles); otherwise pairs are used whenever the widest tile is
  // chosen, the problem is not grouped, and there is at least one 256 x 256 tile per pair of SMs
  bool pair = force_bn == 257;
  int bn = pair ? 256 : (force_bn > 0 ? force_bn : gemm_pick_bn(M, N, K, sm_count, tile_expert != nullptr));
  int n_out = N;
  if (epi == EPI_BIAS_SWIGLU) {
    // W holds 128-row blocks [gate rows | up rows]; a 256-wide tile yields 128 output columns
    if (N % 256 != 0) return set_error(B200EMB_ERR_INVALID, "gemm: the SwiGLU epilogue needs N %% 256 == 0 (N=%d)", N);
    bn = 256;
    n_out = N / 2;
  }
  if (force_bn == 0 && bn == 256 && tile_expert == nullptr &&
      ((M + 255) / 256) * ((N + 255) / 256) >= sm_count / 2)
    pair = true;
  if (pair && tile_expert != nullptr) return set_error(B200EMB_ERR_INVALID, "gemm: the CTA-pair kernel has no grouped mode");
  if (tile_expert != nullptr) B2_SET_LIMIT(0, static_cast<long long>(n_experts) + 1, stream);  // values are expert + 1
  CUtensorMap ta, tw, tc;
  int rc = make_tmap_bf16_2d(&ta, A, (uint64_t)M, (uint64_t)K, BM);
  if (rc) return rc;
  if (tile_expert != nullptr && (N % bn) != 0)
    return set_error(B200EMB_ERR_INVALID, "grouped gemm: N = %d must be a multiple of the tile width %d", N, bn);
  rc = make_tmap_bf16_2d(&tw, W, (uint64_t)N * (tile_expert != nullptr ? n_experts : 1), (uint64_t)K,
                         (uint32_t)(pair ? bn / 2 : bn));
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tc, C, (uint64_t)M, (uint64_t)n_out, 32);  // one epilogue warp's rows per store
  if (rc) return rc;
  switch (bn) {
    case 256: return launch_epi<256>(epi, ta, tw, tc, bias, alpha, M, N, K, tile_expert, sm_count, err_flag, stream, pair);
    case 128: return launch_epi<128>(epi, ta, tw, tc, bias, alpha, M, N, K, tile_expert, sm_count, err_flag, stream);
    case 64: return launch_epi<64>(epi, ta, tw, tc, bias, alpha, M, N, K, tile_expert, sm_count, err_flag, stream);
  }
  return set_error(B200EMB_ERR_INVALID, "gemm: unsupported tile width %d", bn);
}

int gemm_bf16_bounds_status(cudaStream_t stream) {
  (void)stream;
  return B2_TAKE_STATUS(stream);
}

}  // namespace b2
