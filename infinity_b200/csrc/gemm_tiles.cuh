// Pieces shared by the tcgen05 GEMM kernels (gemm_bf16.cu, gemm_w4.cu): tile constants, the shared-memory
// budget of a configuration, the tile order, and the epilogue functions.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "kernels.h"

namespace b2 {

static constexpr int BM = 128;
static constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle span
static constexpr int UMMA_K = 16;
static constexpr int N_EPI_WARPS = 8;
static constexpr int GEMM_THREADS = 32 * (2 + N_EPI_WARPS);

// PAIR: two CTAs of a cluster share one 256 x BN tile (tcgen05 cta_group::2): each CTA loads its 128
// rows of A and only half of the W tile, so a stage is 32 KB instead of 48 KB (six stages instead of four).
template <int BN, bool PAIR = false>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;  // W rows this CTA loads per stage
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (196608 / STAGE_BYTES) < 8 ? (196608 / STAGE_BYTES) : 8;
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;  // two accumulator buffers
  static constexpr int CBUF_BYTES = BM * 64 * 2;  // one 128x64 bf16 output sub-tile
  static constexpr int BIAS_BYTES = 256 * 4;
  static constexpr int BAR_BYTES = 256;  // up to 2 x 8 stage barriers + 5 others + the TMEM address word
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * CBUF_BYTES + BIAS_BYTES + BAR_BYTES + 1024;  // + alignment slack
  static_assert((2 * STAGES + 5) * 8 + 4 <= BAR_BYTES, "barrier area");
  static_assert(SMEM_BYTES <= 232448, "shared memory per block");
};

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// erf GELU for a pair of values with ONE MUFU operation per value: gelu(x) = x * Phi(x) and
// Phi(x) = (1 + erf(x / sqrt2)) / 2 = (1 + tanh(h(x))) / 2 with h = atanh(erf(x / sqrt2)), an odd function that
// a cubic in x^2 follows closely: h(x) = x (c0 + c1 u + c2 u^2 + c3 u^3), u = min(x^2, 25) (beyond |x| = 5 the
// tanh is 1 to fp32 anyway). Fit error of the result < 1.2e-5 absolute; tanh.approx.f32 adds a relative error
// of 2^-11 on tanh, i.e. < 2.5e-4 |x| on the result: a few per cent of a bf16 ulp of the output. (The earlier
// form, erfc from Abramowitz-Stegun 7.1.26, needed a reciprocal and an exponential per value and twice the
// instructions; the GELU epilogue, not the tensor pipe, bounds the FFN up-projection.)
__device__ __forceinline__ float2 gelu_erf2(float2 x) {
  const float2 xx = __fmul2_rn(x, x);
  const float2 u = make_float2(fminf(xx.x, 25.f), fminf(xx.y, 25.f));
  float2 p = __ffma2_rn(u, make_float2(-8.666443136e-06f, -8.666443136e-06f), make_float2(-2.5449786335e-04f, -2.5449786335e-04f));
  p = __ffma2_rn(p, u, make_float2(3.672922030e-02f, 3.672922030e-02f));
  p = __ffma2_rn(p, u, make_float2(7.976911068e-01f, 7.976911068e-01f));
  const float2 h = __fmul2_rn(p, x);
  const float2 t = make_float2(tanh_approx(h.x), tanh_approx(h.y));
  const float2 phi = __ffma2_rn(t, make_float2(0.5f, 0.5f), make_float2(0.5f, 0.5f));
  return __fmul2_rn(x, phi);
}

// silu(x) = x * sigmoid(x) = x * (1 + tanh(x / 2)) / 2: one MUFU operation
__device__ __forceinline__ float silu_f(float x) { return x * fmaf(tanh_approx(0.5f * x), 0.5f, 0.5f); }

// epilogue function on a pair of accumulators, rounded to two bf16
template <int EPI>
__device__ __forceinline__ uint32_t epilogue_pack2(float a, float b) {
  float2 v = make_float2(a, b);
  if (EPI == EPI_BIAS_GELU) v = gelu_erf2(v);
  if (EPI == EPI_BIAS_TANH) v = make_float2(tanhf(a), tanhf(b));
  __nv_bfloat162 p = __floats2bfloat162_rn(v.x, v.y);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Tile order: groups of group_m row tiles; inside a group the column tiles advance slowest, so the CTAs
// that run at the same time share a few W tiles and the group's A tiles instead of one A tile and every W
// tile, and W is streamed from HBM once per group rather than once per row tile. With W larger than the L2
// (a 37888 x 3584 gate/up matrix is 271 MB) the plain row-major order made the GEMM 20 % slower.
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int& mt, int& nt) {
  const int group_tiles = group_m * n_tiles;
  const int group = tile / group_tiles;
  const int first_m = group * group_m;
  const int rows_here = min(group_m, m_tiles - first_m);
  const int r = tile - group * group_tiles;
  mt = first_m + r % rows_here;
  nt = r / rows_here;
}

}  // namespace b2
