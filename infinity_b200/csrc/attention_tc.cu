// Variable-length bidirectional attention on the 5th-generation tensor cores (head_dim 64).
//
// One work item = one 128-row query tile of one (sequence, head); tiles never cross a sequence
// boundary. Q, K and V tiles (128 rows x 64, 128-byte swizzle) arrive by TMA straight from the
// packed qkv buffer. Per 128-key tile:
//   S = Q K^T      tcgen05.mma 128 x N x 16 (N = valid keys rounded up to 16), fp32 in TMEM
//   softmax        128 threads, one TMEM lane (= one query row) each, ONE pass over the row in
//                  32-key chunks whose loads run one chunk ahead of the math: p = exp2(s - m_ref)
//                  against a per-row reference point that is the maximum of the row's first 32 keys
//                  and is moved (with a second pass and a rescale of O) only when a tile's row sum of
//                  these exponentials exceeds 2^16 or overflows, so the pass tracks no maximum; no
//                  cross-thread reduction; P is rounded to bf16
//                  and written back to tensor memory (two keys per 32-bit column)
//   O += P V       tcgen05.mma with the A operand read from tensor memory and V as an MN-major
//                  shared-memory operand (no transpose of V anywhere); O accumulates in tensor
//                  memory across the key tiles and is read once per query tile
// Warp roles: 0-3 softmax, 4 TMA producer (Q, K and V double-buffered), 5 MMA
// issuer. The issuer runs warp-uniform code with only the tcgen05 instructions under elect.sync, so
// descriptors live in uniform registers: an MMA issued from divergent single-thread code costs about
// 90 cycles of operand moves, more than the 32-64 cycles these small MMAs take to execute.
// The kernel is persistent, two CTAs per SM (256 of the 512 TMEM columns each), so one CTA's
// softmax overlaps the other's MMAs.
// head_dim 32 (template D = 32) runs the same pipeline on the same 128-row x 64-column, 128-byte-swizzled tiles: a tile
// holds a PAIR of adjacent heads, and the operand descriptors of the odd head start 64 bytes into the swizzled
// row (the way a K step advances them by 32), so S takes two K = 16 instructions and P V is 128 x 32 per 16 keys.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
// mbarrier waits here are short and on the critical chain softmax -> MMA -> softmax: plain polling
// (no suspend-time hint) measured 3-7 % faster than letting the hardware park the waiting thread
#define B2_MBAR_SUSPEND_NS 0
#include "ptx.cuh"

namespace b2 {

static constexpr int TC_BKV = 128;
static constexpr int TC_TILE_COLS = 64;  // columns of a Q / K / V tile: one head of 64 or two heads of 32
static constexpr int TC_TILE_BYTES = 128 * TC_TILE_COLS * 2;  // 16 KB
static constexpr int TC_QSLOTS = 2;
static constexpr int TC_KSLOTS = 2;
static constexpr int TC_VSLOTS = 2;
static constexpr int TC_N_TILES = TC_QSLOTS + TC_KSLOTS + TC_VSLOTS;
static constexpr int TC_STAGE_BYTES = 4 * 16 * 128;  // output staging: 16 rows of 128 bytes per softmax warp
static constexpr int TC_BAR_BYTES = 160;
static constexpr int TC_SMEM_BYTES = TC_N_TILES * TC_TILE_BYTES + TC_STAGE_BYTES + TC_BAR_BYTES + 1024;
static constexpr int TC_THREADS = 192;         // 4 softmax warps + TMA producer warp + MMA warp
static constexpr uint32_t TC_TMEM_COLS = 256;  // S 128 | P 64 | O 64 (32 used for head_dim 32)
static constexpr uint32_t TC_S_COL = 0, TC_P_COL = 128, TC_O_COL = 192;
static constexpr float TC_LAZY_SUM = 65536.f;  // a tile's row sum of exp2(score - reference) above this moves the reference


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

// Persistent: CTA b serves work items b, b + gridDim.x, ...; item i = (query tile i / n_heads,
// head i % n_heads). Every role walks the same sequence of (item, key tile) steps.
template <int D>
__global__ void __launch_bounds__(TC_THREADS, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_qkv, __nv_bfloat16* __restrict__ out,
                   const AttnTile* __restrict__ tiles, int n_items, int n_heads, int n_kv_heads, float scale_log2,
                   int* __restrict__ err_flag) {
  extern __shared__ uint8_t att_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(att_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + TC_QSLOTS * TC_TILE_BYTES;
  uint8_t* v_s = k_s + TC_KSLOTS * TC_TILE_BYTES;
  uint8_t* stage_s = v_s + TC_VSLOTS * TC_TILE_BYTES;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(stage_s + TC_STAGE_BYTES);
  uint64_t* q_empty = q_full + TC_QSLOTS;
  uint64_t* k_full = q_empty + TC_QSLOTS;
  uint64_t* k_empty = k_full + TC_KSLOTS;
  uint64_t* v_full = k_empty + TC_KSLOTS;
  uint64_t* v_empty = v_full + TC_VSLOTS;
  uint64_t* bar_s = v_empty + TC_VSLOTS;  // S of a step is in tensor memory
  uint64_t* bar_p = bar_s + 1;            // all 128 softmax threads have written P of a step
  uint64_t* bar_pv = bar_p + 1;           // P V of a step has finished: P may be overwritten, O may be read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_pv + 1);
  static_assert((2 * TC_QSLOTS + 2 * TC_KSLOTS + 2 * TC_VSLOTS + 3) * 8 + 4 <= TC_BAR_BYTES, "barrier area");
  // shared memory too small once aligned: report and leave before anything is initialised (uniform per CTA)
  if (smem + TC_N_TILES * TC_TILE_BYTES + TC_STAGE_BYTES + TC_BAR_BYTES > att_raw + TC_SMEM_BYTES) {
    pdl_wait();
    if (threadIdx.x == 0) atomicExch(err_flag, 6);
    return;
  }

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // warp-uniform in the compiler's view too
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < TC_QSLOTS; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < TC_KSLOTS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < TC_VSLOTS; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 4);  // one arrival per softmax warp
    mbar_init(bar_pv, 1);
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
  // The set-up above touched no global memory: it may overlap the tail of the previous kernel in the stream.
  pdl_wait();

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_qkv);
      int qslot = 0, kslot = 0, vslot = 0;
      uint32_t qphase = 0, kphase = 0, vphase = 0;
      uint32_t q_fills = 0, k_fills = 0, v_fills = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const AttnTile t = tiles[item / n_heads];
        const int h = item % n_heads;
        const int hk = h / (n_heads / n_kv_heads);
        const int n_kv = (t.seq_len + TC_BKV - 1) / TC_BKV;
        // first column of the tile that holds head column block c (blocks of D columns): for D = 32 the
        // even-aligned pair of blocks, so that the tile starts on a 128-byte boundary
        auto tile_col = [](int c) { return D == 64 ? c * 64 : (c >> 1) * 64; };
        if (!mbar_wait(&q_empty[qslot], qphase ^ 1u)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&q_full[qslot], TC_TILE_BYTES);
        tma_load_2d(q_s + qslot * TC_TILE_BYTES, &tmap_qkv, &q_full[qslot], tile_col(h), t.seq_start + t.q_start);
        ++q_fills;
        if (++qslot == TC_QSLOTS) {
          qslot = 0;
          qphase ^= 1u;
        }
        for (int it = 0; it < n_kv; ++it) {
          if (!mbar_wait(&k_empty[kslot], kphase ^ 1u)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&k_full[kslot], TC_TILE_BYTES);
          tma_load_2d(k_s + kslot * TC_TILE_BYTES, &tmap_qkv, &k_full[kslot], tile_col(n_heads + hk),
                      t.seq_start + it * TC_BKV);
          ++k_fills;
          if (++kslot == TC_KSLOTS) {
            kslot = 0;
            kphase ^= 1u;
          }
          if (!mbar_wait(&v_empty[vslot], vphase ^ 1u)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&v_full[vslot], TC_TILE_BYTES);
          tma_load_2d(v_s + vslot * TC_TILE_BYTES, &tmap_qkv, &v_full[vslot], tile_col(n_heads + n_kv_heads + hk),
                      t.seq_start + it * TC_BKV);
          ++v_fills;
          if (++vslot == TC_VSLOTS) {
            vslot = 0;
            vphase ^= 1u;
          }
        }
      }
      pdl_launch_dependents();  // every load of this CTA is issued: the next kernel may start its set-up
      if (!ok) {
        atomicExch(err_flag, 5);
        // let the copies still in flight land before shared memory is released (bounded)
        auto drain = [](uint64_t* full, uint32_t fills, uint32_t slots) {
          for (uint32_t i = 0; i < (fills < slots ? fills : slots); ++i) {
            const uint32_t idx = fills - 1 - i;
            mbar_wait(&full[idx % slots], (idx / slots) & 1u);
          }
        };
        drain(q_full, q_fills, TC_QSLOTS);
        drain(k_full, k_fills, TC_KSLOTS);
        drain(v_full, v_fills, TC_VSLOTS);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer: all 32 lanes walk the loops, one elected lane issues ----------------
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t q_addr = smem_u32(q_s), k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
    // S = Q K^T runs one step AHEAD of the softmax: S of step n + 1 is issued as soon as every softmax
    // thread has arrived on bar_p for step n (the S columns are free then), in front of P V of step n.
    int s_item = blockIdx.x, s_it = 0, s_nkv = 0, s_len = 0;
    int qslot = 0, kslot = 0, vslot = 0;
    uint32_t qphase = 0, kphase = 0, vphase = 0;
    bool ok = true;
    // every lane waits; the warp agrees on the outcome so that it never splits around elect.sync
    auto wait_all = [](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity)); };
    // S of a step in two parts: prepare_s waits for its operands and builds the descriptors, fire_s issues the
    // instructions. Between a softmax arrival and the next S only fire_s runs: the waits and the descriptor
    // arithmetic of prepare_s are done before the issuer starts waiting for that arrival.
    uint64_t s_a_desc = 0, s_b_desc = 0;
    uint32_t s_idesc = 0;
    bool s_prepared = false;
    auto prepare_s = [&]() -> bool {  // false when a wait gave up
      if (s_item >= n_items) return true;
      if (s_it == 0) {
        s_len = __shfl_sync(0xffffffffu, tiles[s_item / n_heads].seq_len, 0);
        s_nkv = (s_len + TC_BKV - 1) / TC_BKV;
        if (!wait_all(&q_full[qslot], qphase)) return false;
      }
      if (!wait_all(&k_full[kslot], kphase)) return false;
      const int nv = min(TC_BKV, s_len - s_it * TC_BKV);
      s_idesc = make_idesc_bf16_f32(128, (nv + 15) & ~15);
      // head_dim 32: the odd column block of a tile starts 64 bytes (4 descriptor units) into the swizzled row
      const int s_h = s_item % n_heads;
      const int q_odd = D == 32 ? (s_h & 1) : 0;
      const int k_odd = D == 32 ? ((n_heads + s_h / (n_heads / n_kv_heads)) & 1) : 0;
      s_a_desc = make_kmajor_sw128_desc(q_addr + qslot * TC_TILE_BYTES) + 4 * q_odd;
      s_b_desc = make_kmajor_sw128_desc(k_addr + kslot * TC_TILE_BYTES) + 4 * k_odd;
      s_prepared = true;
      return true;
    };
    auto fire_s = [&]() {
      if (!s_prepared) return;
      s_prepared = false;
      tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < D / 16; ++k)
        if (elect_one()) tc_mma_f16(tmem_u + TC_S_COL, s_a_desc + 2 * k, s_b_desc + 2 * k, s_idesc, k != 0);
      if (elect_one()) {
        tc_commit(bar_s);
        tc_commit(&k_empty[kslot]);
        if (s_it == s_nkv - 1) tc_commit(&q_empty[qslot]);  // last use of this Q tile
      }
      if (++kslot == TC_KSLOTS) {
        kslot = 0;
        kphase ^= 1u;
      }
      if (++s_it == s_nkv) {
        s_it = 0;
        s_item += gridDim.x;
        if (++qslot == TC_QSLOTS) {
          qslot = 0;
          qphase ^= 1u;
        }
      }
    };
    ok = prepare_s();
    if (ok) fire_s();
    uint32_t gi = 0;
    const uint32_t idesc_pv = make_idesc_bf16_f32_b_mn(128, D);
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int L = __shfl_sync(0xffffffffu, tiles[item / n_heads].seq_len, 0);
      const int n_kv = (L + TC_BKV - 1) / TC_BKV;
      const int v_odd = D == 32 ? ((n_heads + n_kv_heads + (item % n_heads) / (n_heads / n_kv_heads)) & 1) : 0;
      for (int it = 0; it < n_kv; ++it, ++gi) {
        const int n_eff = (min(TC_BKV, L - it * TC_BKV) + 15) & ~15;
        // operands and descriptors of the next S first, so that only the instructions themselves follow the arrival
        if (!prepare_s()) {
          ok = false;
          break;
        }
        if (!wait_all(bar_p, gi & 1u)) {
          ok = false;
          break;
        }
        // S of the next step first: it only needs the S columns, which bar_p has just released, and lets
        // the next softmax start while P V of this step executes. The softmax threads hold back their
        // first P store of the next step until bar_pv says that P V has read this step's P.
        fire_s();
        if (!wait_all(&v_full[vslot], vphase)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t v_desc = make_mnmajor_sw128_desc(v_addr + vslot * TC_TILE_BYTES, 16) + 4 * v_odd;
        // 16 keys = two 8-row groups of the MN-major V tile = 2048 bytes (128 in descriptor units); 16 keys
        // of P = 8 columns
#pragma unroll
        for (int k = 0; k < TC_BKV / 16; ++k)
          if (k * 16 < n_eff && elect_one())
            tc_mma_f16_tmem_a(tmem_u + TC_O_COL, tmem_u + TC_P_COL + k * 8, v_desc + k * 128, idesc_pv, (it | k) != 0);
        if (elect_one()) {
          tc_commit(bar_pv);
          tc_commit(&v_empty[vslot]);
        }
        if (++vslot == TC_VSLOTS) {
          vslot = 0;
          vphase ^= 1u;
        }
      }
    }
    if (!ok && lane == 0) atomicExch(err_flag, 7);
  } else {
    // ---------------- softmax warps ----------------
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    uint8_t* stage = stage_s + warp * (16 * 128);  // 16 output rows of this warp at a time
    uint32_t gi = 0;  // key tiles processed so far by this CTA: phase of bar_s, bar_p, bar_pv
    // A warp whose wait gave up leaves its loops; the other roles then run into their own bounded waits.
    bool failed = false;
    // Output of the previous work item, written out during the first step of the next one (its last
    // P V has long finished by then, so nobody idles waiting for it).
    bool out_pending = false;
    float out_inv = 0.f;
    int out_rows = 0;
    __nv_bfloat16* out_dst = nullptr;
    const size_t out_stride = static_cast<size_t>(n_heads) * D;
    // O of the pending item -> bf16 rows in global memory, in two parts. load_pending brings the warp's O rows
    // into registers (scaled and packed to bf16 pairs); it has to come before the warp's arrival on bar_p, because the P V that arrival releases
    // overwrites O. store_pending writes them; it runs after the arrival, in the time the
    // warp would otherwise spend waiting for the next S, so only the tensor-memory read is on the chain
    // softmax -> MMA -> softmax. For head_dim 64 each warp stages 16 rows at a time in shared memory (128 bytes
    // per row, 16-byte chunks XOR-swizzled by row so that neither pass has bank conflicts) and writes them out
    // as whole 128-byte lines, four rows per instruction; for head_dim 32 every lane writes its own 64-byte row.
    auto load_pending = [&](uint32_t (&po)[D / 2]) {
      if (!mbar_wait(bar_pv, (gi - 1) & 1u)) failed = true;  // the item's last P V (normally long done)
      failed = __any_sync(0xffffffffu, failed);
      if (failed) return;
      tc_fence_after_sync();
      if (out_rows > 0) {
        const float inv = out_inv;
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_base + TC_O_COL + c, r);
          tmem_ld_wait_for(r);
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
            po[(c + j) >> 1] = *reinterpret_cast<uint32_t*>(&b);
          }
        }
      }
    };
    auto store_pending = [&](const uint32_t (&po)[D / 2]) {
      out_pending = false;
      if (out_rows <= 0) return;
      if (D == 32) {
        if (lane < out_rows) {
          uint4* dst = reinterpret_cast<uint4*>(out_dst + static_cast<size_t>(lane) * out_stride);
#pragma unroll
          for (int c = 0; c < 4; ++c) dst[c] = make_uint4(po[c * 4], po[c * 4 + 1], po[c * 4 + 2], po[c * 4 + 3]);
        }
        return;
      }
      const int sub = lane >> 3, chunk = lane & 7;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if ((lane >> 4) == half) {
#pragma unroll
          for (int c = 0; c < D / 8; ++c)
            *reinterpret_cast<uint4*>(stage + (lane & 15) * 128 + ((c ^ (lane & 7)) << 4)) =
                make_uint4(po[c * 4], po[c * 4 + 1], po[c * 4 + 2], po[c * 4 + 3]);
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rl = i * 4 + sub;  // row within this half
          const int r = half * 16 + rl;
          if (r < out_rows) {
            const uint4 u = *reinterpret_cast<const uint4*>(stage + rl * 128 + ((chunk ^ (rl & 7)) << 4));
            *reinterpret_cast<uint4*>(out_dst + static_cast<size_t>(r) * out_stride + chunk * 8) = u;
          }
        }
        __syncwarp();
      }
    };
    const float2 scale2 = make_float2(scale_log2, scale_log2);
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const AttnTile t = tiles[item / n_heads];
      const int h = item % n_heads;
      const int L = t.seq_len;
      const int n_kv = (L + TC_BKV - 1) / TC_BKV;
      // a warp whose 32 query rows all lie past the end of the sequence has nothing to compute
      const bool warp_active = t.q_start + warp * 32 < L;
      // Softmax reference point of this row (raw score units) and running denominator. The reference is
      // NOT the running maximum: it is only moved when a tile's sum of exp2(score - reference) exceeds
      // TC_LAZY_SUM (or is not finite), so nearly every step leaves O in tensor memory untouched and the pass
      // tracks no maximum at all; numerator and denominator share whatever scale the reference implies.
      float m_ref = 0.f, l_run = 0.f;

      for (int it = 0; it < n_kv; ++it, ++gi) {
        const int kv0 = it * TC_BKV;
        const int n_valid = min(TC_BKV, L - kv0);
        const int n_eff = (n_valid + 15) & ~15;
        const int n_chunks = (n_eff + 31) >> 5;
        if (!mbar_wait(bar_s, gi & 1u)) failed = true;
        failed = __any_sync(0xffffffffu, failed);  // the warp leaves together
        if (failed) break;
        tc_fence_after_sync();

        if (warp_active) {
          uint32_t ra[32], rb[32];
          uint32_t pa[16], pb[16];
          float l0;
          float2 lsum;
          float2 negm2;
          // One 32-key chunk: p = exp2(s * scale - m_ref * scale) as bf16 pairs and their sum. Only the last,
          // partial chunk needs masking.
          auto chunk = [&](const uint32_t (&r)[32], uint32_t (&pk)[16], int c) {
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
                const bool v0 = c + j < n_valid, v1 = c + j + 1 < n_valid;
                const float s0 = __uint_as_float(r[j]), s1 = __uint_as_float(r[j + 1]);
                const float p0 = v0 ? ex2f(fmaf(s0, scale_log2, negm2.x)) : 0.f;
                const float p1 = v1 ? ex2f(fmaf(s1, scale_log2, negm2.x)) : 0.f;
                l0 += p0 + p1;
                __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                pk[j >> 1] = *reinterpret_cast<uint32_t*>(&b);
              }
            }
          };
          auto store_p = [&](const uint32_t (&pk)[16], int c) { tmem_st_32x32b_x16(lane_base + TC_P_COL + (c >> 1), pk); };
          auto reset_sums = [&]() {
            l0 = 0.f;
            lsum = make_float2(0.f, 0.f);
            negm2 = make_float2(-m_ref * scale_log2, -m_ref * scale_log2);
          };

          tmem_ld_32x32b_x32(lane_base + TC_S_COL, ra);
          tmem_ld_wait_for(ra);
          if (it == 0) {
            // first key tile of the row: the reference point is the maximum of its first 32 keys
            float e0 = -INFINITY, e1 = -INFINITY;
            if (n_valid >= 32) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                e0 = max3f(e0, __uint_as_float(ra[j]), __uint_as_float(ra[j + 1]));
                e1 = max3f(e1, __uint_as_float(ra[j + 2]), __uint_as_float(ra[j + 3]));
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) e0 = fmaxf(e0, (j < n_valid) ? __uint_as_float(ra[j]) : -INFINITY);
            }
            m_ref = fmaxf(e0, e1);
          }
          reset_sums();
          // The load of chunk c + 1 is in flight while chunk c is computed. The first two chunks are held
          // in registers until P V of the previous step (issued behind this step's S) has read the P
          // columns; by then that wait is normally over.
          if (n_chunks > 1) tmem_ld_32x32b_x32(lane_base + TC_S_COL + 32, rb);
          chunk(ra, pa, 0);
          if (n_chunks > 1) {
            tmem_ld_wait_for(rb);
            if (n_chunks > 2) tmem_ld_32x32b_x32(lane_base + TC_S_COL + 64, ra);
            chunk(rb, pb, 32);
          }
          if (gi > 0 && !__all_sync(0xffffffffu, mbar_wait(bar_pv, (gi - 1) & 1u))) failed = true;
          if (!failed) {
            store_p(pa, 0);
            if (n_chunks > 1) store_p(pb, 32);
            if (n_chunks > 2) {
              tmem_ld_wait_for(ra);
              if (n_chunks > 3) tmem_ld_32x32b_x32(lane_base + TC_S_COL + 96, rb);
              chunk(ra, pa, 64);
              store_p(pa, 64);
              if (n_chunks > 3) {
                tmem_ld_wait_for(rb);
                chunk(rb, pb, 96);
                store_p(pb, 96);
              }
            }
            float alpha = 1.f;
            const bool move_ref = !(l0 + (lsum.x + lsum.y) <= TC_LAZY_SUM);  // also true for inf / NaN
            if (__any_sync(0xffffffffu, move_ref)) {
              // Rare: some row of this warp met scores far above its reference point. Move the reference to
              // the row maximum of this tile, redo the tile's P with it and rescale what O and l hold so far.
              float mx = -INFINITY;
              for (int c = 0; c < n_eff; c += 32) {
                tmem_ld_32x32b_x32(lane_base + TC_S_COL + c, ra);
                tmem_ld_wait_for(ra);
#pragma unroll
                for (int j = 0; j < 32; ++j) mx = fmaxf(mx, c + j < n_valid ? __uint_as_float(ra[j]) : -INFINITY);
              }
              if (move_ref) {
                const float m_new = fmaxf(m_ref, mx);  // fmaxf drops a NaN maximum (rows past the sequence end)
                alpha = ex2f((m_ref - m_new) * scale_log2);
                m_ref = m_new;
              }
              reset_sums();
              for (int c = 0; c < n_eff; c += 32) {
                tmem_ld_32x32b_x32(lane_base + TC_S_COL + c, ra);
                tmem_ld_wait_for(ra);
                chunk(ra, pa, c);
                store_p(pa, c);
              }
              if (it > 0) {
                // P V of the previous step has finished (waited for above)
                const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                  tmem_ld_32x32b_x32(lane_base + TC_O_COL + c, ra);
                  tmem_ld_wait_for(ra);
#pragma unroll
                  for (int j = 0; j < 32; j += 2) {
                    const float2 o = __fmul2_rn(make_float2(__uint_as_float(ra[j]), __uint_as_float(ra[j + 1])), alpha2);
                    ra[j] = __float_as_uint(o.x);
                    ra[j + 1] = __float_as_uint(o.y);
                  }
#pragma unroll
                  for (int j = 0; j < 16; ++j) pa[j] = ra[j];
                  tmem_st_32x32b_x16(lane_base + TC_O_COL + c, pa);
#pragma unroll
                  for (int j = 0; j < 16; ++j) pb[j] = ra[16 + j];
                  tmem_st_32x32b_x16(lane_base + TC_O_COL + c + 16, pb);
                }
              }
            }
            l_run = l_run * alpha + (l0 + (lsum.x + lsum.y));
            tmem_st_wait();
          }
        }
        if (failed) break;  // warp-uniform: set from __all_sync
        if (out_pending) {  // first step of an item that follows another
          uint32_t po[D / 2];
          load_pending(po);  // previous item's rows; its O is overwritten only after the arrival below
          if (failed) break;
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_p);
          store_pending(po);
        } else {
          // every lane's P row is in tensor memory and its reads of S are done: the warp meets and arrives once
          // (128 separate arrivals on one mbarrier serialise)
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_p);
        }
      }
      if (failed) break;
      out_pending = true;
      out_inv = 1.f / l_run;
      out_rows = warp_active ? min(32, L - (t.q_start + warp * 32)) : 0;
      out_dst = out + static_cast<size_t>(t.seq_start + t.q_start + warp * 32) * out_stride + h * D;
    }
    if (!failed && out_pending) {
      uint32_t po[D / 2];
      load_pending(po);
      if (!failed) store_pending(po);
    }
    if (failed && lane == 0) atomicExch(err_flag, 4);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}


int attention_tc_init_device() {
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
  B2_CUDA_CHECK(cudaFuncSetAttribute(attn_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
  return B200EMB_OK;
}

int launch_attention_tc(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_tokens, int n_heads,
                        int n_kv_heads, int head_dim, int causal, int variant, int sm_count, int* err_flag,
                        cudaStream_t stream) {
  if ((head_dim != 64 && head_dim != 32) || causal || (variant == 1 && head_dim != 32))
    return launch_attention_tc2(qkv, out, d_tiles, n_tiles, n_tokens, n_heads, n_kv_heads, head_dim, causal, sm_count,
                                err_flag, stream);
  if (n_tiles <= 0) return B200EMB_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535)
    return set_error(B200EMB_ERR_INVALID, "attention: bad head counts %d / %d", n_heads, n_kv_heads);
  CUtensorMap tm;
  const uint64_t width = static_cast<uint64_t>(n_heads + 2 * n_kv_heads) * head_dim;
  int rc = make_tmap_bf16_2d(&tm, qkv, static_cast<uint64_t>(n_tokens), width, 128);
  if (rc) return rc;
  const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(head_dim));  // log2(e) / sqrt(head_dim)
  const long long n_items = static_cast<long long>(n_tiles) * n_heads;
  if (n_items > 0x7fffffffLL) return set_error(B200EMB_ERR_UNSUPPORTED, "attention: too many tiles");
  const int grid = static_cast<int>(n_items < 2LL * sm_count ? n_items : 2LL * sm_count);
  cudaError_t e = head_dim == 64
                      ? launch_pdl(attn_tc_kernel<64>, dim3(grid), dim3(TC_THREADS), TC_SMEM_BYTES, stream, tm,
                                   reinterpret_cast<__nv_bfloat16*>(out), d_tiles, static_cast<int>(n_items), n_heads,
                                   n_kv_heads, scale_log2, err_flag)
                      : launch_pdl(attn_tc_kernel<32>, dim3(grid), dim3(TC_THREADS), TC_SMEM_BYTES, stream, tm,
                                   reinterpret_cast<__nv_bfloat16*>(out), d_tiles, static_cast<int>(n_items), n_heads,
                                   n_kv_heads, scale_log2, err_flag);
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

}  // namespace b2
