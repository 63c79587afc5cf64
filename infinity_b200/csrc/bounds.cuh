// Device-side index range checks for the checked build (-DB200EMB_BOUNDS=1).
//
// Indices that kernels read from device memory (expert choices, rows of the expert-contiguous
// layout, sequence boundaries, positions) are produced by other kernels of the same forward, so the
// host never sees them. In the checked build every such index goes through B2_IDX: a value outside
// [0, limit) records a code in a status word of the translation unit and is replaced by 0, so the
// access that follows stays inside the buffer; nothing traps. The host reads and clears the words
// after a forward (<unit>_bounds_status) and turns a non-zero one into an error status. In the normal
// build B2_IDX is the index itself and none of this exists in the binary.
//
// Limits are not kernel parameters: the launcher writes them into a small __device__ array of its
// translation unit on the launch stream (b2_set_limit) before it launches, so kernel signatures are the
// same in both builds.
#pragma once
#include <cuda_runtime.h>

#ifndef B200EMB_BOUNDS
#define B200EMB_BOUNDS 0
#endif

// codes of the status words (also in the error message)
enum BoundsCode : int {
  BOUNDS_OK = 0,
  BOUNDS_POOL_RANGE = 40,      // a sequence's [start, end) leaves the token stream
  BOUNDS_ROPE_POSITION = 41,   // a position beyond the rotary table
  BOUNDS_EMBED_POSITION = 42,  // a position beyond the position table
  BOUNDS_MOE_EXPERT = 43,      // an expert choice outside [0, n_experts)
  BOUNDS_MOE_ROW = 44,         // a row of the expert-contiguous layout beyond its padded size
  BOUNDS_GEMM_EXPERT = 45,     // tile_expert[] names an expert outside [0, n_experts)
};

#if B200EMB_BOUNDS
static __device__ int b2_bounds_word;
static __device__ long long b2_bounds_limit[4] = {-1, -1, -1, -1};

// a negative limit means "not given": the index passes unchecked
__device__ __forceinline__ long long b2_checked(long long i, int slot, int code) {
  const long long limit = b2_bounds_limit[slot];
  if (limit >= 0 && (i < 0 || i >= limit)) {
    atomicCAS(&b2_bounds_word, 0, code);
    return 0;
  }
  return i;
}
// true when lo <= hi and both lie in [0, limit]; records the code otherwise
__device__ __forceinline__ bool b2_checked_range(long long lo, long long hi, int slot, int code) {
  const long long limit = b2_bounds_limit[slot];
  if (limit >= 0 && (lo < 0 || hi < lo || hi > limit)) {
    atomicCAS(&b2_bounds_word, 0, code);
    return false;
  }
  return true;
}
static inline void b2_set_limit(int slot, long long v, cudaStream_t stream) {
  cudaMemcpyToSymbolAsync(b2_bounds_limit, &v, sizeof(v), slot * sizeof(v), cudaMemcpyHostToDevice, stream);
}
// Reads and clears the unit's status word (waits for the stream).
static inline int b2_take_status(cudaStream_t stream) {
  int v = 0;
  if (cudaMemcpyFromSymbolAsync(&v, b2_bounds_word, sizeof(v), 0, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbolAsync(b2_bounds_word, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, stream);
    cudaStreamSynchronize(stream);
  }
  return v;
}
#define B2_IDX(i, slot, code) b2_checked((i), (slot), (code))
#define B2_RANGE_OK(lo, hi, slot, code) b2_checked_range((lo), (hi), (slot), (code))
#define B2_SET_LIMIT(slot, v, stream) b2_set_limit((slot), (v), (stream))
#define B2_TAKE_STATUS(stream) b2_take_status(stream)
#else
#define B2_IDX(i, slot, code) (i)
#define B2_RANGE_OK(lo, hi, slot, code) (true)
#define B2_SET_LIMIT(slot, v, stream) ((void)0)
#define B2_TAKE_STATUS(stream) (0)
#endif
