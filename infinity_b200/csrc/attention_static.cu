// Allocation-free variant of the attention entry point.
//
// b200emb_op_attention() builds its query-tile list on the host and needs device memory for
// it (plus an error word), which it obtains with cudaMalloc / cudaFree on every call. Some
// callers cannot do that: a serving process whose framework pool already holds almost all
// of the GPU's memory (a fresh cudaMalloc may simply fail there), or a latency-critical
// thread that must not call cudaMalloc / cudaFree because both synchronise the whole device
// and stall work queued on other streams. For them this file keeps the scratch in a
// file-scope __device__ array of fixed size, resident on every GPU that loads the library
// until the process exits, and builds the tile list with a small kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "kernels.h"

namespace b2 {

// Scratch layout: [0, 256) error word (first 4 bytes used), then B200EMB_STATIC_ATTN_MAX_TILES
// tile records of 16 bytes. 256 KB + 256 B per GPU.
static constexpr int STATIC_MAX_TILES = B200EMB_STATIC_ATTN_MAX_TILES;
static __device__ __align__(256) unsigned char g_attn_static_scratch[256 + STATIC_MAX_TILES * sizeof(AttnTile)];

// In host code the array's name is only a handle for the runtime, not a device address: the
// address each device gives it is looked up once per device and cached here.
static std::mutex g_static_mu;
static unsigned char* g_static_ptr[64] = {};

static int static_scratch(unsigned char** out) {
  int dev = 0;
  B2_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(B200EMB_ERR_UNSUPPORTED, "device index %d too large", dev);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return set_error(B200EMB_ERR_CUDA, "cudaGetSymbolAddress(static attention scratch): %s", cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_static_ptr[dev];
  return B200EMB_OK;
}

// One CTA: sequence i contributes ceil(len_i / bq) tiles, written in sequence order at the
// exclusive prefix sum of those counts.
__global__ void __launch_bounds__(1024) build_tiles_static_kernel(const int32_t* __restrict__ cu, int n_seqs, int bq,
                                                                  AttnTile* __restrict__ tiles, int max_tiles) {
  __shared__ int partial[1024];
  const int per = (n_seqs + 1023) / 1024;
  const int begin = min(threadIdx.x * per, n_seqs), end = min(begin + per, n_seqs);
  int count = 0;
  for (int i = begin; i < end; ++i) count += (cu[i + 1] - cu[i] + bq - 1) / bq;
  partial[threadIdx.x] = count;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {  // inclusive scan
    const int v = threadIdx.x >= off ? partial[threadIdx.x - off] : 0;
    __syncthreads();
    partial[threadIdx.x] += v;
    __syncthreads();
  }
  int pos = partial[threadIdx.x] - count;
  for (int i = begin; i < end; ++i) {
    const int start = cu[i], len = cu[i + 1] - cu[i];
    for (int q = 0; q < len; q += bq, ++pos)
      if (pos < max_tiles) tiles[pos] = AttnTile{start, len, q, 0};
  }
}

}  // namespace b2

using namespace b2;

extern "C" int b200emb_op_attention_static(const void* qkv, void* out, const int32_t* d_cu_seqlens,
                                           const int32_t* h_cu_seqlens, int32_t n_seqs, int32_t n_tokens,
                                           int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int32_t causal,
                                           void* stream) {
  if (qkv == nullptr || out == nullptr || d_cu_seqlens == nullptr || h_cu_seqlens == nullptr || n_seqs <= 0)
    return set_error(B200EMB_ERR_INVALID, "attention_static: null pointer or empty batch");
  if (h_cu_seqlens[0] != 0 || h_cu_seqlens[n_seqs] != n_tokens)
    return set_error(B200EMB_ERR_INVALID, "attention_static: cu_seqlens does not span n_tokens");
  const int variant = (causal >> 9) & 1;  // bit 9: one-CTA-per-SM tensor-memory kernel whatever the shape
  causal &= 1;
  const int bq = attention_tile_rows(head_dim, causal);
  long long n_tiles = 0;
  for (int i = 0; i < n_seqs; ++i) {
    const int len = h_cu_seqlens[i + 1] - h_cu_seqlens[i];
    if (len <= 0) return set_error(B200EMB_ERR_INVALID, "attention_static: empty sequence %d", i);
    n_tiles += (len + bq - 1) / bq;
  }
  if (n_tiles > STATIC_MAX_TILES)
    return set_error(B200EMB_ERR_UNSUPPORTED,
                     "attention_static: %lld query tiles of %d rows exceed the fixed scratch of %d tiles; "
                     "split the batch or use b200emb_op_attention",
                     n_tiles, bq, STATIC_MAX_TILES);
  int rc = kernels_init_device();
  if (rc) return rc;
  unsigned char* scratch = nullptr;
  rc = static_scratch(&scratch);  // first call on a device: looks the array's device address up
  if (rc) return rc;
  int* d_err = reinterpret_cast<int*>(scratch);
  AttnTile* d_tiles = reinterpret_cast<AttnTile*>(scratch + 256);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the error word must start at zero, and
  // the tile records of this batch are all rewritten below
  B2_CUDA_CHECK(cudaMemsetAsync(d_err, 0, sizeof(int), s));
  build_tiles_static_kernel<<<1, 1024, 0, s>>>(d_cu_seqlens, n_seqs, bq, d_tiles, STATIC_MAX_TILES);
  B2_CUDA_CHECK(cudaGetLastError());
  if (bq == 128) {
    int dev = 0, sms = 0;
    B2_CUDA_CHECK(cudaGetDevice(&dev));
    B2_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    rc = launch_attention_tc(qkv, out, d_tiles, static_cast<int>(n_tiles), n_tokens, n_heads, n_kv_heads, head_dim, causal,
                             variant, sms, d_err, s);
  } else {
    rc = launch_attention(qkv, out, d_tiles, static_cast<int>(n_tiles), n_heads, n_kv_heads, head_dim, causal, s);
  }
  int herr = 0;
  cudaError_t e = cudaMemcpyAsync(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (rc) return rc;
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "attention_static: %s", cudaGetErrorString(e));
  if (herr != 0)
    return set_error(B200EMB_ERR_DEVICE_WAIT, "attention_static: a device-side wait gave up (role %d)", herr);
  return B200EMB_OK;
}
