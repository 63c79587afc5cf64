/*
 * b200emb.h -- C ABI of the B200-native model-forward path for embedding,
 * reranking and classification.
 *
 * The library replaces the model-forward step that the infinity_emb engine
 * reaches through its backend interface
 *   infinity_emb/transformer/abstract.py:44-69      (BaseTransformer: encode_pre / encode_core / encode_post)
 * and that the reference implements with third-party torch code in
 *   infinity_emb/transformer/embedder/sentence_transformer.py:117-157   (embed: forward, pooling, fp32 + L2 normalise)
 *   infinity_emb/transformer/crossencoder/torch.py:100-111              (rerank: forward + classification head logits)
 *   infinity_emb/transformer/classifier/torch.py:74-76                  (classify: forward + head)
 * The reference has no FFI of its own (it is pure Python); a maintainer binds
 * this header with ctypes (see INTEGRATION.md for the stub).
 *
 * Conventions
 *   - plain C types only; no exceptions cross the boundary;
 *   - every function returns a status: 0 = ok, < 0 = invalid argument,
 *     > 0 = CUDA / runtime failure (including a device-side bounded wait that
 *     gave up). b200emb_last_error() returns the message of the calling
 *     thread's last failure;
 *   - the caller owns every input / output buffer and keeps it alive until
 *     the call returns; calls are synchronous (internal streams are joined
 *     before returning) unless a function says otherwise;
 *   - a handle is not re-entrant (the reference's batcher calls encode_core
 *     from one thread per replica, infinity_emb/inference/batch_handler.py:562-588);
 *     distinct handles are independent;
 *   - there is no CPU fallback: without a usable CUDA device every compute
 *     entry point fails with B200EMB_ERR_CUDA.
 */
#ifndef B200EMB_H_
#define B200EMB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200EMB_ABI_VERSION 1

/* status codes */
#define B200EMB_OK 0
#define B200EMB_ERR_INVALID (-1)     /* bad argument (null pointer, shape, cu_seqlens not monotone, id out of range ...) */
#define B200EMB_ERR_UNSUPPORTED (-2) /* a shape / option the kernels do not cover */
#define B200EMB_ERR_IO (-3)          /* weight file missing, truncated or lacking a tensor */
#define B200EMB_ERR_CUDA 1           /* a CUDA call failed */
#define B200EMB_ERR_DEVICE_WAIT 2    /* a bounded device-side wait ran out; the context stays usable */

/* b200emb_model_desc.arch */
#define B200EMB_ARCH_BERT 0    /* post-LayerNorm encoder, learned absolute positions, token types (BertModel) */
#define B200EMB_ARCH_XLMR 1    /* same block; positions start at pos_offset (XLM-RoBERTa: padding_idx + 1 = 2) */
#define B200EMB_ARCH_MOE 2     /* post-LN encoder whose odd layers route the FFN over n_experts with top_k softmax gating */
#define B200EMB_ARCH_DECODER 3 /* pre-RMSNorm, RoPE, causal grouped-query attention, SwiGLU (Qwen2Model) */

/* b200emb_model_desc.pooling  (reference: PoolingMethod, infinity_emb/primitives.py:161-168;
 * math: infinity_emb/transformer/utils_optimum.py:29-47) */
#define B200EMB_POOL_CLS 0  /* row cu_seqlens[i] */
#define B200EMB_POOL_MEAN 1 /* mean of rows cu_seqlens[i] .. cu_seqlens[i+1]-1, fp32 accumulation */
#define B200EMB_POOL_LAST 2 /* row cu_seqlens[i+1]-1 */
/* No pooling: one fp32 output row per TOKEN, in packed order (sequence i owns rows cu_seqlens[i] ..
 * cu_seqlens[i+1]-1), the reference's ColBERT mode (sentence_transformer.py:87-90 switches normalisation
 * off, :125-131 returns token_embeddings + attention_mask, :146-155 drops the padded rows: the ragged
 * layout has none). The output buffer of b200emb_forward / b200emb_forward_device then has n_tokens rows.
 * Only with B200EMB_HEAD_NONE. */
#define B200EMB_POOL_TOKENS 3

/* b200emb_model_desc.head */
#define B200EMB_HEAD_NONE 0       /* output = pooled (optionally L2-normalised) hidden state, [n_seqs, hidden] */
#define B200EMB_HEAD_CLASSIFIER 1 /* output = out_proj(tanh(dense(h_cls))), [n_seqs, n_labels] raw logits */

/* b200emb_model_desc.weight_format */
#define B200EMB_WFMT_BF16 0
#define B200EMB_WFMT_MXFP8 1 /* e4m3 elements, 32-element K blocks, e8m0 scales */
#define B200EMB_WFMT_NVFP4 2 /* e2m1 elements, 16-element K blocks, e4m3 scales */

/* epilogues of b200emb_op_gemm_bf16 */
#define B200EMB_EPI_BIAS 0
#define B200EMB_EPI_BIAS_GELU 1 /* the erf GELU (not the tanh variant), evaluated to within 5e-4 x of x Phi(x): far inside the bf16 rounding of the output */
#define B200EMB_EPI_BIAS_TANH 2
/* SwiGLU: W is [2F, K] in blocks of 256 rows = 128 gate rows followed by the 128 up rows of the same
 * output columns; C is [M, F] with C[:, j] = silu(gate_j) * up_j. N passed to the call is 2F. */
#define B200EMB_EPI_BIAS_SWIGLU 3

typedef struct b200emb_model_desc {
  int32_t abi_version; /* B200EMB_ABI_VERSION */
  int32_t arch;
  int32_t n_layers;
  int32_t hidden;
  int32_t n_heads;
  int32_t n_kv_heads; /* == n_heads unless grouped-query attention */
  int32_t head_dim;   /* 32, 64 or 128 */
  int32_t ffn;
  int32_t vocab;
  int32_t max_pos;    /* rows of the position table (or longest sequence for RoPE models) */
  int32_t type_vocab; /* 0 = no token-type table */
  int32_t pos_offset; /* position id of the first token of a sequence */
  float norm_eps;
  float rope_theta;
  int32_t n_experts;
  int32_t top_k;
  int32_t moe_every; /* layer l routes its FFN iff moe_every > 0 and l % moe_every == moe_every - 1 */
  int32_t pooling;
  int32_t normalize; /* 1: x / max(||x||_2, 1e-12) after pooling (sentence_transformer.py:142-145) */
  int32_t head;
  int32_t n_labels;
  int32_t weight_format;
  int32_t max_tokens; /* workspace sizing hint (tokens per device per call); workspaces grow when exceeded */
  /* 1 (classifier head only): the output rows are scores instead of raw logits, computed on the device:
   * softmax over the n_labels logits, the logistic function when n_labels == 1. The reference does this
   * on the host after the copy (text-classification pipeline behind classifier/torch.py:38-46, 74-80;
   * rerank scores: batch_handler.py:207-210). */
  int32_t label_scores;
  int32_t reserved[7]; /* zero */
} b200emb_model_desc;

/* Wall and device times of one b200emb_forward call. Device times come from
 * CUDA events recorded on the stream the kernels are launched on. */
#define B200EMB_KCLASS_EMBED 0
#define B200EMB_KCLASS_GEMM 1
#define B200EMB_KCLASS_ATTN 2
#define B200EMB_KCLASS_NORM 3
#define B200EMB_KCLASS_POOL 4
#define B200EMB_KCLASS_OTHER 5
#define B200EMB_N_KCLASS 8
typedef struct b200emb_timing {
  int32_t per_kernel;  /* in: 1 = bracket every launch with events (slower; fills kclass_*) */
  int32_t n_devices;   /* out */
  float h2d_ms;        /* out: max over devices */
  float kernels_ms;    /* out: first launch to last launch, max over devices */
  float d2h_ms;        /* out */
  float total_ms;      /* out: host clock around the whole call */
  int32_t launches;    /* out: kernels launched by this call, all devices */
  float kclass_ms[B200EMB_N_KCLASS];       /* out (per_kernel): summed duration per kernel class, device 0 */
  int32_t kclass_launches[B200EMB_N_KCLASS]; /* out (per_kernel) */
  double gemm_flops;   /* out: algorithmic GEMM flops issued by device 0 (2*M*N*K per launch) */
} b200emb_timing;

typedef struct b200emb_handle b200emb_handle;

/* ---- model lifetime -------------------------------------------------------
 * Replaces the backend constructors that load one replica per device
 * (infinity_emb/inference/select_model.py:80-83,
 *  infinity_emb/transformer/embedder/sentence_transformer.py:57-111).
 * Weights are read from a b200emb weight file (written by
 * infinity_b200.weights.save_weights) and replicated on every listed device. */
int b200emb_create(const b200emb_model_desc* desc, const char* weight_path, const int32_t* device_ids,
                   int32_t n_devices, b200emb_handle** out);
int b200emb_destroy(b200emb_handle* h);

/* Offline weight quantisation: reads a bf16 weight file, replaces every layer matrix
 * ("layer.<l>.<...>.w"; only the expert matrices when the model has experts) by name.q / name.s
 * (/ name.gs) in the given block format using the quantiser kernels on device_id, and writes
 * out_path. Load the result with weight_format set to the same format. The reference's
 * counterpart is the load-time hook quant_interface (quantization/interface.py:28-70). */
int b200emb_quantize_weights(const char* in_path, const char* out_path, int32_t format, int32_t device_id);

/* ---- the hot path -----------------------------------------------------------
 * Replaces encode_core (+ the pooling / normalise part of encode_post):
 *   sentence_transformer.py:117-133 + :142-145, crossencoder/torch.py:100-108,
 *   classifier/torch.py:74-76.
 * Input is the ragged token stream of one batch in the batcher's order
 * (infinity_emb/inference/queue.py:35-76): input_ids[n_tokens],
 * token_type_ids[n_tokens] (nullable = all zero), cu_seqlens[n_seqs + 1] with
 * cu_seqlens[0] == 0, strictly increasing, cu_seqlens[n_seqs] == n_tokens.
 * All are HOST pointers. Output row i belongs to sequence i:
 * out[i * out_row_stride + j], j < hidden (HEAD_NONE) or j < n_labels, fp32.
 * With several devices the sequences are split token-balanced (longest
 * processing time first on cost a*L + b*L^2) and rows are scattered back to
 * batch order on the host; no collective runs. */
int b200emb_forward(b200emb_handle* h, const int32_t* input_ids, const int32_t* token_type_ids,
                    const int32_t* cu_seqlens, int32_t n_seqs, int32_t n_tokens, float* out,
                    int64_t out_row_stride, b200emb_timing* timing /* nullable */);

/* Same computation with every buffer already resident on device 0 of the
 * handle (device pointers; out is device fp32). Used to measure the kernels
 * without host<->device copies. Single-device handles only. Lengths are validated on the
 * host from h_cu_seqlens; ids and token types, which only the device holds, are range-checked
 * by the embedding kernel: an id outside its table is read as 0 (no out-of-bounds access) and
 * the call returns B200EMB_ERR_INVALID when the forward has finished. */
int b200emb_forward_device(b200emb_handle* h, const int32_t* d_input_ids, const int32_t* d_token_type_ids,
                           const int32_t* d_cu_seqlens, const int32_t* h_cu_seqlens, int32_t n_seqs,
                           int32_t n_tokens, float* d_out, int64_t out_row_stride, b200emb_timing* timing);

/* Output embedding precisions (reference: EmbeddingDtype, infinity_emb/primitives.py:145-158, applied by
 * quant_embedding_decorator around encode_post, infinity_emb/transformer/quantization/interface.py:124-154,
 * which calls sentence-transformers 3.3.1 quantization.quantize_embeddings). Per row x[0..dim):
 *   INT8    (int8)  ((x - lo) / ((hi - lo) / 255) - 128), UINT8 (uint8) ((x - lo) / ((hi - lo) / 255)):
 *           float64 arithmetic, truncation toward zero, then the low 8 bits of the integer;
 *           lo = ranges[0, :], hi = ranges[1, :] (the calibration ranges, float64 [2, dim])
 *   UBINARY bit j of byte k = (x[8k + j'] > 0) packed most significant bit first (numpy packbits);
 *   BINARY  the same byte - 128 as int8. dim must be a multiple of 8. */
#define B200EMB_EMB_FLOAT32 0
#define B200EMB_EMB_INT8 1
#define B200EMB_EMB_UINT8 2
#define B200EMB_EMB_BINARY 3
#define B200EMB_EMB_UBINARY 4

/* b200emb_forward with the result rows quantised on the device before they are copied back (the
 * reference quantises on the host after the copy): `out` receives n_seqs rows (n_tokens rows with
 * B200EMB_POOL_TOKENS) of dim bytes (INT8 / UINT8) or dim / 8 bytes (BINARY / UBINARY), row stride
 * out_row_stride_bytes; FLOAT32 gives b200emb_forward's rows (stride in bytes). h_ranges: host float64
 * [2, dim], needed for INT8 / UINT8 only. The matryoshka slice of the reference (batch_handler.py:65-74)
 * is applied by its caller to whatever rows come back, so it is not part of this call. */
int b200emb_forward_quantized(b200emb_handle* h, const int32_t* input_ids, const int32_t* token_type_ids,
                              const int32_t* cu_seqlens, int32_t n_seqs, int32_t n_tokens, int32_t precision,
                              const double* h_ranges, void* out, int64_t out_row_stride_bytes,
                              b200emb_timing* timing);

/* The quantiser alone, on device buffers: x fp32 [n_rows, dim] (row stride x_row_stride floats),
 * d_ranges device float64 [2, dim] (INT8 / UINT8), out device bytes (row stride out_row_stride_bytes). */
int b200emb_op_quantize_embeddings(const float* x, int32_t n_rows, int32_t dim, int64_t x_row_stride,
                                   int32_t precision, const double* d_ranges, void* out,
                                   int64_t out_row_stride_bytes, void* stream);

/* Token-balanced partition used by b200emb_forward, exposed for tests and for
 * callers that run one process per GPU: assigns sequence i (length lens[i]) to
 * shard_of[i] in [0, n_shards). Deterministic; ties go to the lower index. */
int b200emb_partition(const int32_t* lens, int32_t n_seqs, int32_t n_shards, double cost_linear,
                      double cost_quadratic, int32_t* shard_of);

/* The coefficients b200emb_forward uses for that partition on a model of this description:
 * cost of a sequence of L tokens = *cost_linear * L + *cost_quadratic * L * L (GEMM flops per
 * token, averaged over dense and routed layers, and attention flops per token pair weighted by
 * the attention kernels' measured time per flop relative to the GEMMs'). A process-per-GPU driver
 * that passes them to b200emb_partition cuts a batch exactly as a multi-device handle does. */
int b200emb_cost_model(const b200emb_model_desc* desc, double* cost_linear, double* cost_quadratic);

/* 1 when the library is the checked build (compiled with -DB200EMB_BOUNDS=1,
 * `python -m infinity_b200.build --checked` -> libb200emb_checked.so), else 0. In the checked build
 * every index a kernel reads from device memory (expert choices, rows of the expert-contiguous
 * layout, sequence boundaries and positions derived from the device copy of cu_seqlens, the expert
 * of a GEMM row block) is range-checked by the kernel that uses it: a value outside its range is
 * recorded, replaced by index 0 so that the access stays inside its buffer, and the forward returns
 * B200EMB_ERR_INVALID ("device index check: ..."). Nothing traps. It stands in for a memory checker
 * on machines where none may be run; the normal build contains none of it. No counterpart in the reference. */
int b200emb_checked_build(void);

/* TMA descriptors (tensor maps) of weights and workspace slices are encoded once per (address, shape)
 * and kept for the life of the process; these are the counts of descriptor requests served from that
 * table and of those that called the driver's encoder. No counterpart in the reference. */
int b200emb_tensor_map_stats(uint64_t* hits, uint64_t* misses);

/* Thread-local message of the last failure on the calling thread ("" if none). */
const char* b200emb_last_error(void);

/* Number of CUDA devices visible, or a negative status. */
int b200emb_device_count(void);

/* Failure-detection self-test: launches one thread that waits on a barrier nothing signals, with
 * the same bounded wait the pipelined kernels use but a limit of limit_ms. Expected result:
 * B200EMB_ERR_DEVICE_WAIT after about limit_ms, with the context still usable. No GPU fault,
 * trap or endless loop is involved. */
int b200emb_selftest_bounded_wait(int32_t limit_ms);

/* Host-side failure injection for tests of the allocation paths: the next `after` workspace
 * allocations of any handle go through, then n report failure (status B200EMB_ERR_CUDA) without
 * calling the allocator; n = 0 switches it off. Nothing on the GPU is touched. No counterpart in
 * the reference. */
int b200emb_test_fail_allocs(int32_t after, int32_t n);

/* ---- single kernels on device buffers (used by the parity tests) -------------
 * Pointers are DEVICE pointers on the current device; `stream` is a
 * cudaStream_t (NULL = default stream). The calls are asynchronous on that
 * stream except where noted. None has a counterpart function in the reference:
 * each is one step of the third-party torch forward the reference calls at
 * sentence_transformer.py:124. */

/* C[M,N] (bf16; [M, N/2] for the SwiGLU epilogue) = epilogue(A[M,K] (bf16, row-major) * W[N,K]^T (bf16, row-major) + bias[N] (fp32, nullable)).
 * K % 8 == 0, N % 8 == 0. tcgen05 / TMEM kernel fed by TMA. Synchronises the
 * stream before returning and reports a device-side wait that gave up. */
int b200emb_op_gemm_bf16(const void* A, const void* W, const float* bias, void* C, int32_t M, int32_t N,
                         int32_t K, int32_t epilogue, void* stream);

/* C[M,N] (bf16) = epilogue(mxfp8(A) * W^T + bias) on the block-scaled tensor-core path
 * (tcgen05.mma kind::mxf8f6f4.block_scale): A [M,K] bf16 is quantised to MXFP8 on the fly (same rule
 * as b200emb_op_quantize), W_q [N,K] e4m3 and W_scales [N, K/32] e8m0 come from b200emb_op_quantize.
 * N and K multiples of 128; epilogue B200EMB_EPI_BIAS or B200EMB_EPI_BIAS_GELU. Synchronises the stream. */
int b200emb_op_gemm_mxfp8(const void* A_bf16, const void* W_q, const void* W_scales, const float* bias, void* C,
                          int32_t M, int32_t N, int32_t K, int32_t epilogue, void* stream);

/* C[M,N] (bf16; [M, N/2] for the SwiGLU epilogue) = epilogue((A[M,K] (bf16) * dequant(W)^T) / tensor_scale + bias) with
 * the NVFP4 weights expanded inside the kernel: W_q [N, K/2] packed e2m1, W_scales [N, K/16] e4m3, tensor_scale = gs,
 * all three as b200emb_op_quantize writes them. The stored bytes are read once per tile straight from HBM; the
 * result equals b200emb_op_dequantize followed by b200emb_op_gemm_bf16 (with 1 / gs applied to the accumulator)
 * bit for bit. K % 64 == 0, N % 256 == 0, epilogue B200EMB_EPI_BIAS or B200EMB_EPI_BIAS_SWIGLU; otherwise
 * B200EMB_ERR_UNSUPPORTED. The model forward uses it for batches of up to 512 tokens per device on matrices wide
 * enough to fill the GPU with 256-column tiles, and expands the matrix once per GEMM otherwise (in the kernel a weight
 * tile is re-expanded for every 256 rows of A: measured slower from about 1000 rows on). Synchronises the stream. */
int b200emb_op_gemm_nvfp4(const void* A, const void* W_q, const void* W_scales, float tensor_scale, const float* bias,
                          void* C, int32_t M, int32_t N, int32_t K, int32_t epilogue, void* stream);

/* Variable-length attention over a packed qkv buffer [n_tokens, (n_heads + 2*n_kv_heads) * head_dim]
 * (all query heads, then all key heads, then all value heads), bf16.
 * out [n_tokens, n_heads * head_dim] bf16. h_cu_seqlens is the host copy used
 * to build the tile list. causal: 0 = bidirectional, 1 = causal. head_dim 64 and 128, and
 * bidirectional head_dim 32, run on the tensor-memory (tcgen05) kernels, the rest on the mma.sync kernel; adding 0x100 forces the
 * mma.sync kernel, adding 0x200 forces the one-CTA-per-SM tensor-memory kernel (which otherwise serves
 * head_dim 128 and causal batches) for head_dim 64 bidirectional too.
 * Synchronises the stream before returning. */
int b200emb_op_attention(const void* qkv, void* out, const int32_t* d_cu_seqlens, const int32_t* h_cu_seqlens,
                         int32_t n_seqs, int32_t n_tokens, int32_t n_heads, int32_t n_kv_heads,
                         int32_t head_dim, int32_t causal, void* stream);

/* Weight quantisers (the reference's hook for them is quant_interface,
 * infinity_emb/transformer/quantization/interface.py:28-70; it has int8 / fp8 only).
 * w_bf16 [rows, cols] row-major, blocks along cols (K):
 *   B200EMB_WFMT_NVFP4: q_out = rows*cols/2 bytes (two e2m1 per byte, even element in the low
 *     nibble), scales_out = rows*cols/16 e4m3 bytes, *tensor_scale_out (device fp32) = gs with
 *     gs = 2688 / amax(tensor); block scale = e4m3(amax(block) / 6 * gs); x^ = q * scale / gs.
 *   B200EMB_WFMT_MXFP8: q_out = rows*cols e4m3 bytes, scales_out = rows*cols/32 e8m0 bytes
 *     (biased exponent e + 127, e = floor(log2(amax(block))) - 8); x^ = q * 2^e.
 * Round to nearest even, saturating. Synchronises the stream. */
int b200emb_op_quantize(const void* w_bf16, int64_t rows, int64_t cols, int32_t format, void* q_out,
                        void* scales_out, float* tensor_scale_out, void* stream);
/* Inverse: bf16 [rows, cols]; for NVFP4 the result is q * block scale, WITHOUT the 1 / gs factor
 * (exact in bf16; the GEMM applies 1 / gs to its accumulator). Asynchronous on the stream. */
int b200emb_op_dequantize(const void* q, const void* scales, int64_t rows, int64_t cols, int32_t format,
                          void* out_bf16, void* stream);

/* Mixture-of-experts router: fp32 logits x[t,:] (bf16) . router_w[e,:] (fp32) + router_b[e]
 * (nullable), softmax over the n_experts (<= 16) experts, top_k (<= 4) experts per token with
 * ties going to the lower expert index; topk_weight = softmax probability of the chosen expert
 * (not renormalised). counts (nullable, [n_experts]) receives tokens per expert. Asynchronous. */
int b200emb_op_moe_router(const void* x, const float* router_w, const float* router_b, int32_t n_tokens,
                          int32_t hidden, int32_t n_experts, int32_t top_k, int32_t* topk_idx, float* topk_weight,
                          int32_t* counts, void* stream);

/* The same attention for callers that must not allocate device memory. No counterpart in the
 * reference: it exists for processes whose framework pool already holds nearly all GPU memory
 * (so a cudaMalloc inside a library call may fail) and for latency-critical threads that
 * cannot afford cudaMalloc / cudaFree, which synchronise the whole device.
 * Same arguments and result as b200emb_op_attention (without its 0x100 flag), but the
 * query-tile list and the error word live in a fixed array inside the library
 * (B200EMB_STATIC_ATTN_MAX_TILES tile records, about 256 KB, present on every GPU that loads
 * the library until the process exits) and the list is built by a kernel from d_cu_seqlens.
 * The call makes no cudaMalloc, cudaFree or other allocating call. A batch that needs more
 * query tiles (128 rows each for head_dim 64 and 128 and for bidirectional head_dim 32, 64 rows
 * otherwise; a sequence of L tokens takes ceil(L / rows) tiles) is rejected with B200EMB_ERR_UNSUPPORTED. Like
 * b200emb_op_attention it waits for the stream before it returns (it reads the kernels' error
 * word back). The first call on each device looks up the array's device address; make that
 * first call before any stream capture. All calls on a device share the array: two calls whose
 * kernels overlap on the GPU (different streams or threads) race on it. h_cu_seqlens and
 * d_cu_seqlens must hold the same offsets: the tile count comes from the host copy, the tile
 * records from the device copy. */
#define B200EMB_STATIC_ATTN_MAX_TILES 16384
int b200emb_op_attention_static(const void* qkv, void* out, const int32_t* d_cu_seqlens,
                                const int32_t* h_cu_seqlens, int32_t n_seqs, int32_t n_tokens, int32_t n_heads,
                                int32_t n_kv_heads, int32_t head_dim, int32_t causal, void* stream);

/* x[t,:] = LayerNorm(word[ids[t]] + pos[pos_offset + t - cu_seqlens[seq(t)]] + type[types[t]]) -> bf16.
 * Tables are bf16, gamma/beta fp32. type_table / types nullable. With
 * gamma == NULL the sum is written without normalisation (decoder gather). */
int b200emb_op_embed_ln(const int32_t* ids, const int32_t* types, const int32_t* d_cu_seqlens, int32_t n_seqs,
                        int32_t n_tokens, const void* word, const void* pos, const void* type_table,
                        const float* gamma, const float* beta, int32_t hidden, int32_t pos_offset, float eps,
                        void* out, void* stream);

/* out = LayerNorm(x + y) * gamma + beta, rows of `hidden` bf16, fp32 statistics. y nullable. */
int b200emb_op_add_ln(const void* x, const void* y, const float* gamma, const float* beta, int32_t n_rows,
                      int32_t hidden, float eps, void* out, void* stream);

/* Pooling + optional L2 normalisation over the ragged stream:
 * out[i,:] fp32 (out_bf16 == 0) or bf16 (out_bf16 == 1). */
int b200emb_op_pool(const void* x, const int32_t* d_cu_seqlens, int32_t n_seqs, int32_t hidden, int32_t pooling,
                    int32_t normalize, void* out, int64_t out_row_stride, int32_t out_bf16, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200EMB_H_ */
