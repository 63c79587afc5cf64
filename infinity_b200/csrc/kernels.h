// Internal launcher declarations shared by the runtime and the single-kernel C entry points.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200emb.h"

struct CUtensorMap_st;  // the driver API's tensor-map descriptor (cuda.h)

namespace b2 {

enum {
  EPI_BIAS = B200EMB_EPI_BIAS,
  EPI_BIAS_GELU = B200EMB_EPI_BIAS_GELU,
  EPI_BIAS_TANH = B200EMB_EPI_BIAS_TANH,
  EPI_BIAS_SWIGLU = B200EMB_EPI_BIAS_SWIGLU
};

// Records a thread-local error message and returns `code`.
int set_error(int code, const char* fmt, ...);
#define B2_CUDA_CHECK(expr)                                                                  \
  do {                                                                                       \
    cudaError_t e__ = (expr);                                                                \
    if (e__ != cudaSuccess)                                                                  \
      return ::b2::set_error(B200EMB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__));    \
  } while (0)

// Programmatic dependent launch: a kernel launched through launch_pdl may be scheduled while its predecessor
// in the stream is still draining, so that its set-up (barrier init, tensor-memory allocation, descriptor
// prefetch) overlaps the predecessor's tail. Such a kernel executes pdl_wait() (ptx.cuh) in every thread before
// its first access to global memory; the wait returns when the predecessor grid has completed and its writes
// are visible. The overlap is worth about 2 us per launch: 14 % of a 7.7 k-token bge-small-shape forward
// (86 launches, 1.44 -> 1.24 ms) and 2.7 % of a 9 k-token BERT-large-shape forward; at 19 k tokens of that
// shape it is neutral, and from 38 k tokens on the forward measured 1-2 % SLOWER with it than without. The
// forward therefore switches it on per call while n_tokens x hidden <= PDL_MAX_WORK (thread-local: one thread
// drives one device); single-kernel entry points keep it on. B200EMB_PDL=0 / 1 in the environment forces it
// off / on (for comparisons).
constexpr long long PDL_MAX_WORK = 12ll << 20;
bool pdl_enabled();
void pdl_for_batch(int n_tokens, int hidden);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Opt-in shared-memory attributes of every kernel, for the current device. Idempotent.
int kernels_init_device();

// ---- GEMM (gemm_bf16.cu) ----
// err_flag: device int the kernel sets non-zero when a bounded wait gave up.
// force_bn: 0 = choose the tile width from the problem size, else 64 / 128 / 256.
// alpha scales the accumulator before the bias (1 / tensor scale of NVFP4 weights; 1 otherwise).
// Grouped mode (tile_expert != null): A is [M, K] with rows grouped by expert in 128-row blocks,
// tile_expert[m / 128] = expert of that row block (< 0: unused block, skipped), W is the stack
// [n_experts * N, K], bias [n_experts * N]; one launch covers every expert.
int launch_gemm_bf16(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int epi,
                     int sm_count, int* err_flag, cudaStream_t stream, int force_bn, float alpha = 1.0f,
                     const int32_t* tile_expert = nullptr, int n_experts = 1);
int gemm_init_device();
// TMA descriptor of a bf16 row-major [rows, cols] matrix: box [box_rows x 64 columns], 128-byte swizzle.
int make_tmap_bf16_2d(::CUtensorMap_st* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
// Descriptors depend on (address, shape, box, element kind) only, never on the memory's contents, and a forward
// asks for the same few hundred of them every time (weights, workspace slices): the builders keep the encoded
// 128 bytes per key and skip the driver call on a repeat. `kind` separates element types / swizzle modes.
// Process-wide, guarded by a mutex, emptied when it reaches 16 384 entries.
struct TmapKey {
  const void* base;
  uint64_t rows, cols;
  uint32_t box_rows, box_cols, kind;
};
bool tmap_cache_get(const TmapKey& key, ::CUtensorMap_st* out);
void tmap_cache_put(const TmapKey& key, const ::CUtensorMap_st* tm);
// {hits, misses} since the library was loaded.
void tmap_cache_stats(uint64_t* hits, uint64_t* misses);

// ---- GEMM against NVFP4 weights expanded inside the kernel (gemm_w4.cu) ----
// Wq: packed e2m1 [N, K / 2], Ws: e4m3 block scales [N, K / 16], alpha = 1 / tensor scale. CTA-pair tiles of
// 256 x 256; gemm_w4_supported says whether a shape qualifies (K % 64 == 0, N % 256 == 0, bias or SwiGLU epilogue).
bool gemm_w4_supported(int M, int N, int K, int epi);
int launch_gemm_w4(const void* A, const void* Wq, const void* Ws, const float* bias, void* C, int M, int N, int K, int epi,
                   float alpha, int sm_count, int* err_flag, cudaStream_t stream);
int gemm_w4_init_device();

// ---- MXFP8 block-scaled GEMM (gemm_mxfp8.cu) ----
// Aq / Wq: e4m3 [M, K] / [N (x n_experts), K]; sf*_atoms: e8m0 scales in 512-byte atoms (128 rows x 4 K-blocks).
int launch_gemm_mxfp8(const void* Aq, const void* sfa_atoms, const void* Wq, const void* sfw_atoms, const float* bias,
                      void* C, int M, int N, int K, int epi, int sm_count, int* err_flag, cudaStream_t stream,
                      const int32_t* tile_expert = nullptr, int n_experts = 1, void* out_sf_atoms = nullptr);
// out_sf_atoms != null: C is written as MXFP8 (e4m3 bytes [M, N] + scales in atom layout) instead of bf16
int gemm_mxfp8_init_device();
size_t mxfp8_sf_atoms_bytes(int64_t rows, int64_t K);
int launch_quant_act_mxfp8(const void* x, int64_t rows, int K, void* q, void* sf_atoms, cudaStream_t stream);
int launch_sf_to_atoms(const void* scales, int64_t rows, int K, void* atoms, cudaStream_t stream);

// ---- attention (attention.cu) ----
struct AttnTile {
  int32_t seq_start;  // first token of the sequence
  int32_t seq_len;
  int32_t q_start;    // first query row of this tile, relative to the sequence
  int32_t pad;
};
// Builds the tile list on the host: one entry per bq-row query tile, longest sequences first.
// Returns the number of tiles; `tiles` may be null to only count.
int attention_build_tiles_q(const int32_t* h_cu_seqlens, int n_seqs, int bq, AttnTile* tiles);
// Query-tile height of the kernel that serves (head_dim, causal): 128 for the tensor-memory
// kernels (head_dim 64 and 128, head_dim 32 bidirectional), 64 for the mma.sync kernel.
int attention_tile_rows(int head_dim, int causal);
int launch_attention(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_heads, int n_kv_heads,
                     int head_dim, int causal, cudaStream_t stream);
int attention_init_device();
// Tensor-memory (tcgen05) kernels, 128-row query tiles. launch_attention_tc picks the kernel:
// head_dim 64 or 32 bidirectional -> two CTAs per SM (attention_tc.cu); head_dim 128, or causal -> one CTA per
// SM with double-buffered S (attention_tc2.cu). variant 1 forces the latter for every supported shape.
int launch_attention_tc(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_tokens, int n_heads,
                        int n_kv_heads, int head_dim, int causal, int variant, int sm_count, int* err_flag,
                        cudaStream_t stream);
int launch_attention_tc2(const void* qkv, void* out, const AttnTile* d_tiles, int n_tiles, int n_tokens, int n_heads,
                         int n_kv_heads, int head_dim, int causal, int sm_count, int* err_flag, cudaStream_t stream);
int attention_tc_init_device();
int attention_tc2_init_device();

// ---- block-format weight quantisers (quant.cu) ----
// w bf16 [rows, cols] -> q (packed elements), scales (one byte per block, row-major [rows, cols / block]);
// NVFP4 also writes the tensor scale gs to d_gs and needs a 4-byte device scratch word.
int launch_quantize(const void* w, int64_t rows, int64_t cols, int fmt, void* q, void* scales, float* d_gs,
                    unsigned int* d_amax_scratch, cudaStream_t stream);
// q, scales -> bf16 [rows, cols]; for NVFP4 the result is q * block_scale (the consumer multiplies by 1 / gs)
int launch_dequantize(const void* q, const void* scales, int64_t rows, int64_t cols, int fmt, void* out,
                      cudaStream_t stream);

// ---- mixture of experts (moe.cu) ----
int moe_init_device();
int launch_moe_router(const void* x, const float* wr, const float* br, int n_tokens, int hidden, int n_experts,
                      int top_k, int32_t* topk_idx, float* topk_w, int32_t* counts, cudaStream_t stream);
// upper bound of 128-row blocks of the expert-contiguous layout (segments padded to 128 rows)
int moe_max_row_blocks(int n_tokens, int top_k, int n_experts);
int launch_moe_scatter(const void* x, const int32_t* topk_idx, const int32_t* counts, int n_tokens, int top_k,
                       int hidden, int n_experts, int32_t* cursor, int32_t* tile_expert, int32_t* row_of, void* xperm,
                       cudaStream_t stream, void* xq = nullptr, void* sf_atoms = nullptr);  // xq != null: write MXFP8 instead of bf16
int launch_moe_combine_ln(const void* x, const void* yperm, const int32_t* row_of, const float* topk_w, int top_k,
                          const float* gamma, const float* beta, int n_tokens, int hidden, float eps, void* out,
                          cudaStream_t stream);

// ---- row kernels (rowops.cu) ----
int launch_wait_selftest(unsigned long long limit_ns, int* err_flag, cudaStream_t stream);
// vocab / type_vocab > 0: ids and types outside the tables are reported through err_flag (codes 32 / 33) and read as 0
int launch_embed_ln(const int32_t* ids, const int32_t* types, const int32_t* d_cu, int n_seqs, int n_tokens,
                    const void* word, const void* pos, const void* type_table, const float* gamma, const float* beta,
                    int hidden, int pos_offset, float eps, void* out, cudaStream_t stream, int vocab = 0,
                    int type_vocab = 0, int* err_flag = nullptr, int n_positions = -1);
int launch_add_ln(const void* x, const void* y, const float* gamma, const float* beta, int n_rows, int hidden,
                  float eps, void* out, cudaStream_t stream);
// h (fp32) += y (bf16, nullable); out = RMSNorm(h) * gamma (bf16)
int launch_add_rmsnorm(float* h, const void* y, const float* gamma, int n_rows, int hidden, float eps, void* out,
                       cudaStream_t stream);
int launch_widen(const void* x, float* out, size_t n_elems, cudaStream_t stream);
// rotates the first n_rot_heads heads (queries then keys) of every qkv row in place; cos_sin = [max_pos, head_dim/2] (cos, sin) pairs
int launch_rope(void* qkv, const int32_t* d_cu, int n_seqs, int n_tokens, int n_rot_heads, int row_width,
                int head_dim, const float* cos_sin, cudaStream_t stream, int n_positions = -1);
// output embedding quantisation (int8 / uint8 with calibration ranges, binary / ubinary bit packing)
int launch_quantize_embeddings(const float* x, int n_rows, int dim, int64_t x_row_stride, int precision,
                               const double* d_ranges, void* out, int64_t out_row_stride_bytes, cudaStream_t stream);
// no pooling: every bf16 hidden row -> one fp32 output row (optionally L2-normalised)
int launch_token_rows(const void* x, int n_tokens, int hidden, int normalize, float* out, int64_t out_row_stride,
                      cudaStream_t stream);
int launch_pool(const void* x, const int32_t* d_cu, int n_seqs, int hidden, int pooling, int normalize, void* out,
                int64_t out_row_stride, int out_bf16, cudaStream_t stream, int n_tokens = -1);
// The trailing n_positions / n_tokens of launch_embed_ln, launch_rope and launch_pool are the limits of the checked
// build (-DB200EMB_BOUNDS=1, see bounds.cuh) for the indices those kernels derive from cu_seqlens on the device;
// negative = not checked, ignored by the normal build. Each unit with checks reports and clears its status word:
int rowops_bounds_status(cudaStream_t stream);
int moe_bounds_status(cudaStream_t stream);
int gemm_bf16_bounds_status(cudaStream_t stream);
int gemm_mxfp8_bounds_status(cudaStream_t stream);
// logits[i, l] = dot(x[i, :], W[l, :]) + b[l]; x bf16 [n, hidden], W bf16 [n_labels, hidden], out fp32.
int launch_small_proj(const void* x, const void* W, const float* bias, int n_rows, int hidden, int n_labels,
                      float* out, int64_t out_row_stride, cudaStream_t stream);
// softmax over each row's n_labels logits (logistic function when n_labels == 1), in place
int launch_label_scores(float* logits, int n_rows, int n_labels, int64_t row_stride, cudaStream_t stream);

}  // namespace b2
