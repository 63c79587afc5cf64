// Host runtime behind the C ABI: weight loading, per-device workspaces, the layer
// sequence of one forward pass, token-balanced sharding over several devices, and the
// single-kernel entry points used by the parity tests.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <chrono>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "bounds.cuh"
#include "kernels.h"

namespace b2 {

// ---- errors -----------------------------------------------------------------------
static thread_local char g_err[512] = "";

// B200EMB_PDL: unset = by batch size (pdl_for_batch), 0 = never, 1 = always.
static int pdl_env() {
  static const int mode = [] {
    const char* v = getenv("B200EMB_PDL");
    return v == nullptr ? -1 : (v[0] == '0' ? 0 : 1);
  }();
  return mode;
}
static thread_local bool g_pdl_small_batch = true;

bool pdl_enabled() { return pdl_env() < 0 ? g_pdl_small_batch : pdl_env() == 1; }

void pdl_for_batch(int n_tokens, int hidden) { g_pdl_small_batch = static_cast<long long>(n_tokens) * hidden <= PDL_MAX_WORK; }

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static std::mutex g_init_mu;
static bool g_dev_inited[64] = {};

int kernels_init_device() {
  int dev = 0;
  B2_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_init_mu);
  if (dev >= 0 && dev < 64 && g_dev_inited[dev]) return B200EMB_OK;
  int rc = gemm_init_device();
  if (!rc) rc = attention_init_device();
  if (!rc) rc = attention_tc_init_device();
  if (!rc) rc = attention_tc2_init_device();
  if (!rc) rc = gemm_mxfp8_init_device();
  if (!rc) rc = gemm_w4_init_device();
  if (!rc) rc = moe_init_device();
  if (rc) return rc;
  if (dev >= 0 && dev < 64) g_dev_inited[dev] = true;
  return B200EMB_OK;
}

// ---- weight file --------------------------------------------------------------------
// Layout (little endian): magic "B2EW0001", u32 n_tensors, u32 reserved, u64 data_offset,
// then n_tensors entries {char name[64]; u32 dtype; u32 ndim; u64 dims[4]; u64 offset; u64 nbytes},
// then the data region (offsets relative to data_offset, 256-byte aligned).
struct TensorEntry {
  char name[64];
  uint32_t dtype;  // 0 = fp32, 1 = bf16, 2 = u8, 3 = i32
  uint32_t ndim;
  uint64_t dims[4];
  uint64_t offset;
  uint64_t nbytes;
};
static_assert(sizeof(TensorEntry) == 64 + 8 + 32 + 16, "weight-file entry layout");

struct WeightFile {
  std::vector<TensorEntry> entries;
  std::vector<uint8_t> data;
  std::map<std::string, int> index;
};

static int read_weight_file(const char* path, WeightFile* wf) {
  FILE* f = fopen(path, "rb");
  if (f == nullptr) return set_error(B200EMB_ERR_IO, "cannot open weight file %s", path);
  char magic[8];
  uint32_t n = 0, reserved = 0;
  uint64_t data_offset = 0;
  bool ok = fread(magic, 1, 8, f) == 8 && memcmp(magic, "B2EW0001", 8) == 0 && fread(&n, 4, 1, f) == 1 &&
            fread(&reserved, 4, 1, f) == 1 && fread(&data_offset, 8, 1, f) == 1 && n < (1u << 20);
  if (ok) {
    wf->entries.resize(n);
    ok = n == 0 || fread(wf->entries.data(), sizeof(TensorEntry), n, f) == n;
  }
  if (ok) {
    fseek(f, 0, SEEK_END);
    const long end = ftell(f);
    ok = end >= (long)data_offset;
    if (ok) {
      wf->data.resize(end - data_offset);
      fseek(f, (long)data_offset, SEEK_SET);
      ok = wf->data.empty() || fread(wf->data.data(), 1, wf->data.size(), f) == wf->data.size();
    }
  }
  fclose(f);
  if (!ok) return set_error(B200EMB_ERR_IO, "weight file %s is truncated or not a b200emb weight file", path);
  for (size_t i = 0; i < wf->entries.size(); ++i) {
    TensorEntry& e = wf->entries[i];
    e.name[63] = 0;
    if (e.offset + e.nbytes > wf->data.size() || (e.offset & 255) != 0)
      return set_error(B200EMB_ERR_IO, "weight file %s: tensor %s out of bounds", path, e.name);
    wf->index[e.name] = (int)i;
  }
  return B200EMB_OK;
}

// ---- model --------------------------------------------------------------------------
// One GEMM weight: bf16 as stored, or a block-quantised tensor that is expanded into the
// per-device scratch right before its GEMM (alpha = 1 / tensor scale for NVFP4).
struct Mat {
  const __nv_bfloat16* w = nullptr;
  const uint8_t* q = nullptr;
  const uint8_t* s = nullptr;
  uint8_t* sf_atoms = nullptr;  // MXFP8: the scales repacked into the tensor cores' 512-byte atoms (owned by the context)
  float alpha = 1.0f;
  int64_t rows = 0, cols = 0;
};

struct LayerW {
  Mat qkv_w, o_w, ffn1_w, ffn2_w;  // decoder: ffn1_w = block-interleaved gate/up [2F, H], ffn2_w = down
  // mixture-of-experts layers: router (fp32) and the experts' matrices stacked along the rows
  bool is_moe = false;
  const float *router_w = nullptr, *router_b = nullptr;
  const float *qkv_b, *o_b, *ffn1_b, *ffn2_b;
  const float *ln1_g, *ln1_b, *ln2_g, *ln2_b;
};

struct ModelW {
  const __nv_bfloat16 *word, *pos, *type;
  const float *emb_ln_g, *emb_ln_b;
  std::vector<LayerW> layers;
  const __nv_bfloat16 *head_dense_w, *head_out_w;
  const float *head_dense_b, *head_out_b;
  const float* final_norm_g;  // decoder
};

struct EventPair {
  cudaEvent_t a, b;
  int kclass;
};

struct DeviceCtx {
  int dev = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  uint8_t* blob = nullptr;
  ModelW w;
  // workspaces (grown on demand)
  int cap_tokens = 0, cap_seqs = 0, cap_tiles = 0;
  int32_t *d_ids = nullptr, *d_types = nullptr, *d_cu = nullptr;
  AttnTile* d_tiles = nullptr;
  __nv_bfloat16 *x = nullptr, *x2 = nullptr, *qkv = nullptr, *ctx = nullptr, *y = nullptr, *ffn = nullptr;
  __nv_bfloat16 *pooled = nullptr, *head_h = nullptr;
  // mixture of experts: routing tables and the expert-contiguous copies of the activations
  int32_t *topk_idx = nullptr, *row_of = nullptr, *moe_counts = nullptr, *moe_cursor = nullptr, *tile_expert = nullptr;
  float* topk_w = nullptr;
  __nv_bfloat16 *xperm = nullptr, *hperm = nullptr, *yperm = nullptr;
  __nv_bfloat16* wscratch = nullptr;  // expanded copy of the quantised matrix in use
  size_t wscratch_elems = 0;
  // MXFP8 block-scaled GEMMs: the activation operand quantised on the fly
  uint8_t *act_q = nullptr, *act_sf = nullptr;
  size_t act_q_bytes = 0, act_sf_bytes = 0;
  uint8_t *act2_q = nullptr, *act2_sf = nullptr;  // second operand buffer (expert hidden activations)
  size_t act2_q_bytes = 0, act2_sf_bytes = 0;
  std::vector<uint8_t*> owned_atoms;
  float* hres = nullptr;     // decoder: fp32 residual stream [T, H]
  float* rope_cs = nullptr;  // decoder: (cos, sin) table [max_pos, head_dim / 2]
  float* d_out = nullptr;
  uint8_t* d_qout = nullptr;   // quantised output rows (b200emb_forward_quantized)
  size_t d_qout_bytes = 0;
  double* d_ranges = nullptr;  // calibration ranges [2, out_dim]
  int* d_err = nullptr;
  // pinned host staging
  int32_t *h_ids = nullptr, *h_types = nullptr, *h_cu = nullptr;
  AttnTile* h_tiles = nullptr;
  float* h_out = nullptr;
  int* h_err = nullptr;
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  std::vector<EventPair> kev;  // per-kernel event pairs (profiling mode)
  size_t kev_used = 0;
  // per-call bookkeeping
  int launches = 0;
  double gemm_flops = 0;
  bool per_kernel = false;
};

}  // namespace b2

struct b200emb_handle {
  b200emb_model_desc desc;
  int out_dim = 0;
  std::vector<b2::DeviceCtx*> devs;
  double cost_a = 1.0, cost_b = 0.0;
};

namespace b2 {

// Host-side fault injection for the allocation paths (tests only; no device fault is involved):
// b200emb_test_fail_allocs(after, n) lets `after` workspace allocations through, then makes n report failure.
static std::mutex g_fail_mu;
static int g_fail_after = 0, g_fail_allocs = 0;
static bool alloc_fault_injected() {
  std::lock_guard<std::mutex> lk(g_fail_mu);
  if (g_fail_allocs <= 0) return false;
  if (g_fail_after > 0) {
    --g_fail_after;
    return false;
  }
  --g_fail_allocs;
  return true;
}

template <typename T>
static int dev_alloc(T** p, size_t count) {
  if (*p != nullptr) {
    cudaFree(*p);
    *p = nullptr;
  }
  if (count == 0) count = 1;
  if (alloc_fault_injected()) return set_error(B200EMB_ERR_CUDA, "cudaMalloc: injected failure");
  B2_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)));
  return B200EMB_OK;
}
template <typename T>
static int host_alloc(T** p, size_t count) {
  if (*p != nullptr) {
    cudaFreeHost(*p);
    *p = nullptr;
  }
  if (count == 0) count = 1;
  B2_CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(p), count * sizeof(T)));
  return B200EMB_OK;
}

static int ensure_capacity(b200emb_handle* h, DeviceCtx* c, int n_tokens, int n_seqs, int n_tiles) {
  const b200emb_model_desc& d = h->desc;
  int rc = 0;
  // A capacity is set to 0 before its buffers are freed and to the new size only after every
  // allocation of the group succeeded: after a failed allocation the next call allocates again
  // instead of launching kernels on freed or null buffers.
  if (n_tokens > c->cap_tokens) {
    c->cap_tokens = 0;
    const size_t T = (size_t)std::max(n_tokens, std::max(d.max_tokens, 1024));
    const size_t H = d.hidden, QKV = (size_t)(d.n_heads + 2 * d.n_kv_heads) * d.head_dim;
    if (!rc) rc = dev_alloc(&c->d_ids, T);
    if (!rc) rc = dev_alloc(&c->d_types, T);
    if (!rc) rc = dev_alloc(&c->x, T * H);
    if (!rc && d.arch == B200EMB_ARCH_DECODER) rc = dev_alloc(&c->hres, T * H);
    if (!rc && d.arch != B200EMB_ARCH_DECODER) rc = dev_alloc(&c->x2, T * H);
    if (!rc) rc = dev_alloc(&c->y, T * H);
    if (!rc) rc = dev_alloc(&c->ctx, T * (size_t)d.n_heads * d.head_dim);
    if (!rc) rc = dev_alloc(&c->qkv, T * QKV);
    if (!rc) rc = dev_alloc(&c->ffn, T * (size_t)d.ffn);
    if (!rc && d.arch == B200EMB_ARCH_MOE) {
      const size_t K = d.top_k, E = d.n_experts;
      const size_t Mp = (size_t)moe_max_row_blocks((int)T, d.top_k, d.n_experts) * 128;
      rc = dev_alloc(&c->topk_idx, T * K);
      if (!rc) rc = dev_alloc(&c->row_of, T * K);
      if (!rc) rc = dev_alloc(&c->topk_w, T * K);
      if (!rc) rc = dev_alloc(&c->moe_counts, E);
      if (!rc) rc = dev_alloc(&c->moe_cursor, E);
      if (!rc) rc = dev_alloc(&c->tile_expert, Mp / 128);
      if (!rc) rc = dev_alloc(&c->xperm, Mp * H);
      if (!rc) rc = dev_alloc(&c->hperm, Mp * (size_t)d.ffn);
      if (!rc) rc = dev_alloc(&c->yperm, Mp * H);
    }
    if (!rc) rc = host_alloc(&c->h_ids, T);
    if (!rc) rc = host_alloc(&c->h_types, T);
    if (d.pooling == B200EMB_POOL_TOKENS) {  // one output row per token
      if (!rc) rc = dev_alloc(&c->d_out, T * (size_t)h->out_dim);
      if (!rc) rc = host_alloc(&c->h_out, T * (size_t)h->out_dim);
    }
    if (rc) return rc;
    c->cap_tokens = (int)T;
  }
  if (n_seqs > c->cap_seqs) {
    c->cap_seqs = 0;
    const size_t B = (size_t)std::max(n_seqs, 256);
    if (!rc) rc = dev_alloc(&c->d_cu, B + 1);
    if (!rc && d.pooling != B200EMB_POOL_TOKENS) rc = dev_alloc(&c->d_out, B * (size_t)h->out_dim);
    if (!rc) rc = dev_alloc(&c->pooled, B * (size_t)d.hidden);
    if (!rc) rc = dev_alloc(&c->head_h, B * (size_t)d.hidden);
    if (!rc) rc = host_alloc(&c->h_cu, B + 1);
    if (!rc && d.pooling != B200EMB_POOL_TOKENS) rc = host_alloc(&c->h_out, B * (size_t)h->out_dim);
    if (rc) return rc;
    c->cap_seqs = (int)B;
  }
  if (n_tiles > c->cap_tiles) {
    c->cap_tiles = 0;
    const size_t NT = (size_t)std::max(n_tiles, 1024);
    if (!rc) rc = dev_alloc(&c->d_tiles, NT);
    if (!rc) rc = host_alloc(&c->h_tiles, NT);
    if (rc) return rc;
    c->cap_tiles = (int)NT;
  }
  return B200EMB_OK;
}

template <typename T>
static int lookup(const WeightFile& wf, const uint8_t* blob, const char* name, uint32_t dtype, uint64_t elems,
                  const T** out, bool optional = false) {
  auto it = wf.index.find(name);
  if (it == wf.index.end()) {
    *out = nullptr;
    if (optional) return B200EMB_OK;
    return set_error(B200EMB_ERR_IO, "weight file lacks tensor %s", name);
  }
  const TensorEntry& e = wf.entries[it->second];
  uint64_t n = 1;
  for (uint32_t i = 0; i < e.ndim && i < 4; ++i) n *= e.dims[i];
  if (e.dtype != dtype || n != elems)
    return set_error(B200EMB_ERR_IO, "tensor %s: expected dtype %u with %llu elements, file has dtype %u with %llu",
                     name, dtype, (unsigned long long)elems, e.dtype, (unsigned long long)n);
  *out = reinterpret_cast<const T*>(blob + e.offset);
  return B200EMB_OK;
}

// A GEMM weight by name: the bf16 tensor, or (block formats) name.q / name.s / name.gs.
static int lookup_mat(const b200emb_model_desc& d, const WeightFile& wf, DeviceCtx* c, const char* name, uint64_t rows,
                      uint64_t cols, Mat* m) {
  m->rows = (int64_t)rows;
  m->cols = (int64_t)cols;
  char nm[112];
  snprintf(nm, sizeof(nm), "%s.q", name);
  if (d.weight_format == B200EMB_WFMT_BF16 || wf.index.find(nm) == wf.index.end())
    return lookup(wf, c->blob, name, 1, rows * cols, &m->w);
  const bool fp4 = d.weight_format == B200EMB_WFMT_NVFP4;
  const uint64_t block = fp4 ? 16 : 32;
  if (cols % block) return set_error(B200EMB_ERR_IO, "tensor %s: K = %llu not a multiple of %llu", name, (unsigned long long)cols, (unsigned long long)block);
  int rc = lookup(wf, c->blob, nm, 2, fp4 ? rows * cols / 2 : rows * cols, &m->q);
  snprintf(nm, sizeof(nm), "%s.s", name);
  if (!rc) rc = lookup(wf, c->blob, nm, 2, rows * cols / block, &m->s);
  if (!rc && fp4) {
    snprintf(nm, sizeof(nm), "%s.gs", name);
    auto it = wf.index.find(nm);
    if (it == wf.index.end()) return set_error(B200EMB_ERR_IO, "weight file lacks tensor %s", nm);
    const TensorEntry& e = wf.entries[it->second];
    if (e.dtype != 0 || e.nbytes < 4) return set_error(B200EMB_ERR_IO, "tensor %s must be one fp32", nm);
    float gs = 1.f;
    memcpy(&gs, wf.data.data() + e.offset, 4);
    if (!(gs > 0.f)) return set_error(B200EMB_ERR_IO, "tensor %s: tensor scale must be positive", nm);
    m->alpha = 1.0f / gs;
  }
  if (!rc) c->wscratch_elems = std::max(c->wscratch_elems, (size_t)(rows * cols));
  if (!rc && !fp4 && cols % 128 == 0 && rows % 128 == 0) {
    // scales in the layout tcgen05.mma.block_scale reads (one 512-byte atom per 128 rows x 4 K-blocks)
    uint8_t* atoms = nullptr;
    B2_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&atoms), mxfp8_sf_atoms_bytes((int64_t)rows, (int64_t)cols)));
    c->owned_atoms.push_back(atoms);
    rc = launch_sf_to_atoms(m->s, (int64_t)rows, (int)cols, atoms, nullptr);
    if (!rc) B2_CUDA_CHECK(cudaDeviceSynchronize());
    m->sf_atoms = atoms;
  }
  return rc;
}

static int bind_weights(const b200emb_model_desc& d, const WeightFile& wf, DeviceCtx* c) {
  const uint64_t H = d.hidden, F = d.ffn, QKV = (uint64_t)(d.n_heads + 2 * d.n_kv_heads) * d.head_dim;
  const uint64_t HQ = (uint64_t)d.n_heads * d.head_dim;
  const uint8_t* b = c->blob;
  ModelW& w = c->w;
  int rc = lookup(wf, b, "emb.word", 1, (uint64_t)d.vocab * H, &w.word);
  if (d.arch == B200EMB_ARCH_DECODER) {
    w.pos = nullptr;
    w.type = nullptr;
    w.emb_ln_g = w.emb_ln_b = nullptr;
    w.layers.resize(d.n_layers);
    char nm[96];
    for (int l = 0; l < d.n_layers && !rc; ++l) {
      LayerW& L = w.layers[l];
      L = LayerW();
#define B2_LK(field, suffix, dt, n)                         \
  if (!rc) {                                                \
    snprintf(nm, sizeof(nm), "layer.%d." suffix, l);        \
    rc = lookup(wf, b, nm, dt, n, &L.field);                \
  }
#define B2_LM(field, suffix, r, k)                          \
  if (!rc) {                                                \
    snprintf(nm, sizeof(nm), "layer.%d." suffix, l);        \
    rc = lookup_mat(d, wf, c, nm, r, k, &L.field);          \
  }
      B2_LK(ln1_g, "ln1.g", 0, H)
      B2_LM(qkv_w, "qkv.w", QKV, H)
      B2_LK(qkv_b, "qkv.b", 0, QKV)
      B2_LM(o_w, "o.w", H, HQ)
      B2_LK(ln2_g, "ln2.g", 0, H)
      B2_LM(ffn1_w, "gu.w", 2 * F, H)
      B2_LM(ffn2_w, "down.w", H, F)
#undef B2_LM
#undef B2_LK
    }
    if (!rc) rc = lookup(wf, b, "norm.g", 0, H, &w.final_norm_g);
    return rc;
  }
  if (!rc) rc = lookup(wf, b, "emb.pos", 1, (uint64_t)d.max_pos * H, &w.pos);
  if (!rc && d.type_vocab > 0) rc = lookup(wf, b, "emb.type", 1, (uint64_t)d.type_vocab * H, &w.type);
  if (d.type_vocab <= 0) w.type = nullptr;
  if (!rc) rc = lookup(wf, b, "emb.ln.g", 0, H, &w.emb_ln_g);
  if (!rc) rc = lookup(wf, b, "emb.ln.b", 0, H, &w.emb_ln_b);
  w.layers.resize(d.n_layers);
  char nm[96];
  for (int l = 0; l < d.n_layers && !rc; ++l) {
    LayerW& L = w.layers[l];
#define B2_LK(field, suffix, dt, n)                         \
  if (!rc) {                                                \
    snprintf(nm, sizeof(nm), "layer.%d." suffix, l);        \
    rc = lookup(wf, b, nm, dt, n, &L.field);                \
  }
#define B2_LM(field, suffix, r, k)                          \
  if (!rc) {                                                \
    snprintf(nm, sizeof(nm), "layer.%d." suffix, l);        \
    rc = lookup_mat(d, wf, c, nm, r, k, &L.field);          \
  }
    B2_LM(qkv_w, "qkv.w", QKV, H)
    B2_LK(qkv_b, "qkv.b", 0, QKV)
    B2_LM(o_w, "o.w", H, HQ)
    B2_LK(o_b, "o.b", 0, H)
    B2_LK(ln1_g, "ln1.g", 0, H)
    B2_LK(ln1_b, "ln1.b", 0, H)
    L.is_moe = d.arch == B200EMB_ARCH_MOE && d.moe_every > 0 && (l % d.moe_every) == d.moe_every - 1;
    if (L.is_moe) {
      const uint64_t E = d.n_experts;
      B2_LK(router_w, "router.w", 0, E * H)
      B2_LK(router_b, "router.b", 0, E)
      B2_LM(ffn1_w, "experts.ffn1.w", E * F, H)
      B2_LK(ffn1_b, "experts.ffn1.b", 0, E * F)
      B2_LM(ffn2_w, "experts.ffn2.w", E * H, F)
      B2_LK(ffn2_b, "experts.ffn2.b", 0, E * H)
    } else {
      B2_LM(ffn1_w, "ffn1.w", F, H)
      B2_LK(ffn1_b, "ffn1.b", 0, F)
      B2_LM(ffn2_w, "ffn2.w", H, F)
      B2_LK(ffn2_b, "ffn2.b", 0, H)
    }
#undef B2_LM
    B2_LK(ln2_g, "ln2.g", 0, H)
    B2_LK(ln2_b, "ln2.b", 0, H)
#undef B2_LK
  }
  if (!rc && d.head == B200EMB_HEAD_CLASSIFIER) {
    rc = lookup(wf, b, "head.dense.w", 1, H * H, &w.head_dense_w);
    if (!rc) rc = lookup(wf, b, "head.dense.b", 0, H, &w.head_dense_b);
    if (!rc) rc = lookup(wf, b, "head.out.w", 1, (uint64_t)d.n_labels * H, &w.head_out_w);
    if (!rc) rc = lookup(wf, b, "head.out.b", 0, (uint64_t)d.n_labels, &w.head_out_b);
  }
  return rc;
}

static void destroy_ctx(DeviceCtx* c) {
  if (c == nullptr) return;
  cudaSetDevice(c->dev);
  if (c->stream) cudaStreamSynchronize(c->stream);
  cudaFree(c->blob);
  cudaFree(c->d_ids); cudaFree(c->d_types); cudaFree(c->d_cu); cudaFree(c->d_tiles);
  cudaFree(c->x); cudaFree(c->x2); cudaFree(c->qkv); cudaFree(c->ctx); cudaFree(c->y); cudaFree(c->ffn);
  cudaFree(c->pooled); cudaFree(c->head_h); cudaFree(c->d_out); cudaFree(c->d_err);
  cudaFree(c->d_qout); cudaFree(c->d_ranges);
  cudaFree(c->hres); cudaFree(c->rope_cs); cudaFree(c->wscratch); cudaFree(c->act_q); cudaFree(c->act_sf); cudaFree(c->act2_q); cudaFree(c->act2_sf);
  for (uint8_t* p : c->owned_atoms) cudaFree(p);
  cudaFree(c->topk_idx); cudaFree(c->row_of); cudaFree(c->moe_counts); cudaFree(c->moe_cursor); cudaFree(c->tile_expert);
  cudaFree(c->topk_w); cudaFree(c->xperm); cudaFree(c->hperm); cudaFree(c->yperm);
  cudaFreeHost(c->h_ids); cudaFreeHost(c->h_types); cudaFreeHost(c->h_cu); cudaFreeHost(c->h_tiles);
  cudaFreeHost(c->h_out); cudaFreeHost(c->h_err);
  for (auto& e : c->ev) if (e) cudaEventDestroy(e);
  for (auto& p : c->kev) { cudaEventDestroy(p.a); cudaEventDestroy(p.b); }
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
}

static int validate_desc(const b200emb_model_desc& d) {
  if (d.abi_version != B200EMB_ABI_VERSION) return set_error(B200EMB_ERR_INVALID, "abi_version %d != %d", d.abi_version, B200EMB_ABI_VERSION);
  if (d.arch < B200EMB_ARCH_BERT || d.arch > B200EMB_ARCH_DECODER) return set_error(B200EMB_ERR_INVALID, "unknown arch %d", d.arch);
  if (d.arch == B200EMB_ARCH_MOE) {
    if (d.n_experts < 1 || d.n_experts > 16 || d.top_k < 1 || d.top_k > 4 || d.top_k > d.n_experts || d.moe_every < 1)
      return set_error(B200EMB_ERR_UNSUPPORTED, "mixture of experts: need n_experts <= 16, top_k <= min(4, n_experts), moe_every >= 1");
    if (d.hidden > 1024) return set_error(B200EMB_ERR_UNSUPPORTED, "mixture of experts: hidden > 1024 is not built");
  }
  if (d.weight_format < B200EMB_WFMT_BF16 || d.weight_format > B200EMB_WFMT_NVFP4)
    return set_error(B200EMB_ERR_INVALID, "unknown weight_format %d", d.weight_format);
  if (d.n_layers <= 0 || d.hidden <= 0 || d.n_heads <= 0 || d.ffn <= 0 || d.vocab <= 0 || d.max_pos <= 0)
    return set_error(B200EMB_ERR_INVALID, "model dimensions must be positive");
  if (d.arch == B200EMB_ARCH_DECODER) {
    if (d.n_kv_heads <= 0 || d.n_heads % d.n_kv_heads != 0) return set_error(B200EMB_ERR_INVALID, "n_heads must be a multiple of n_kv_heads");
    if (d.ffn % 128 != 0) return set_error(B200EMB_ERR_UNSUPPORTED, "decoder ffn width must be a multiple of 128");
    if (!(d.rope_theta > 0.f)) return set_error(B200EMB_ERR_INVALID, "decoder needs rope_theta > 0");
    if (d.head != B200EMB_HEAD_NONE) return set_error(B200EMB_ERR_UNSUPPORTED, "decoder with a classifier head is not built");
  } else if (d.n_kv_heads != d.n_heads) {
    return set_error(B200EMB_ERR_UNSUPPORTED, "grouped-query attention needs the decoder arch");
  }
  if (d.head_dim != 32 && d.head_dim != 64 && d.head_dim != 128) return set_error(B200EMB_ERR_UNSUPPORTED, "head_dim %d not in {32, 64, 128}", d.head_dim);
  if (d.n_heads * d.head_dim != d.hidden) return set_error(B200EMB_ERR_INVALID, "n_heads * head_dim must equal hidden");
  if (d.hidden % 8 || d.ffn % 8) return set_error(B200EMB_ERR_UNSUPPORTED, "hidden and ffn must be multiples of 8");
  if (d.pooling < B200EMB_POOL_CLS || d.pooling > B200EMB_POOL_TOKENS) return set_error(B200EMB_ERR_INVALID, "unknown pooling %d", d.pooling);
  if (d.pooling == B200EMB_POOL_TOKENS && d.head != B200EMB_HEAD_NONE)
    return set_error(B200EMB_ERR_INVALID, "per-token outputs need head = none");
  if (d.head == B200EMB_HEAD_CLASSIFIER && d.n_labels <= 0) return set_error(B200EMB_ERR_INVALID, "classifier head needs n_labels > 0");
  if (d.head != B200EMB_HEAD_NONE && d.head != B200EMB_HEAD_CLASSIFIER) return set_error(B200EMB_ERR_INVALID, "unknown head %d", d.head);
  if (d.label_scores != 0 && (d.label_scores != 1 || d.head != B200EMB_HEAD_CLASSIFIER))
    return set_error(B200EMB_ERR_INVALID, "label_scores is 0 or 1 and needs the classifier head");
  if (d.pos_offset < 0 || d.pos_offset >= d.max_pos) return set_error(B200EMB_ERR_INVALID, "pos_offset out of range");
  return B200EMB_OK;
}

// ---- one forward pass on one device -------------------------------------------------------
struct KernelScope {  // brackets one launch with events in profiling mode and counts it
  DeviceCtx* c;
  int idx = -1;
  KernelScope(DeviceCtx* c_, int kclass) : c(c_) {
    c->launches++;
    if (!c->per_kernel) return;
    if (c->kev_used == c->kev.size()) {
      EventPair p;
      p.kclass = kclass;
      if (cudaEventCreate(&p.a) != cudaSuccess || cudaEventCreate(&p.b) != cudaSuccess) return;
      c->kev.push_back(p);
    }
    idx = (int)c->kev_used++;
    c->kev[idx].kclass = kclass;
    cudaEventRecord(c->kev[idx].a, c->stream);
  }
  ~KernelScope() {
    if (idx >= 0) cudaEventRecord(c->kev[idx].b, c->stream);
  }
};

static int gemm(DeviceCtx* c, const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int epi) {
  KernelScope ks(c, B200EMB_KCLASS_GEMM);
  c->gemm_flops += 2.0 * M * N * K;
  return launch_gemm_bf16(A, W, bias, C, M, N, K, epi, c->sm_count, c->d_err, c->stream, 0);
}

// Grows a byte buffer; *have is 0 while the buffer is invalid, so a failed allocation is retried by the next call.
static int grow_bytes(uint8_t** p, size_t* have, size_t want, bool zero) {
  if (want <= *have) return B200EMB_OK;
  *have = 0;
  cudaFree(*p);
  *p = nullptr;
  if (alloc_fault_injected()) return set_error(B200EMB_ERR_CUDA, "cudaMalloc: injected failure ");
  B2_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(p), want));
  if (zero) B2_CUDA_CHECK(cudaMemset(*p, 0, want));
  *have = want;
  return B200EMB_OK;
}

// Quantises the activation operand [rows, K] to MXFP8 into the context's buffers (grown on demand).
static int quantize_activation(DeviceCtx* c, const void* A, int rows_padded, int K) {
  const size_t qb = (size_t)rows_padded * K, sb = mxfp8_sf_atoms_bytes(rows_padded, K);
  int rc = grow_bytes(&c->act_q, &c->act_q_bytes, qb, false);
  if (!rc) rc = grow_bytes(&c->act_sf, &c->act_sf_bytes, sb, true);
  if (rc) return rc;
  KernelScope ks(c, B200EMB_KCLASS_OTHER);
  return launch_quant_act_mxfp8(A, rows_padded, K, c->act_q, c->act_sf, c->stream);
}

static bool use_block_scaled(int wfmt, const Mat& W, int epi) {
  return wfmt == B200EMB_WFMT_MXFP8 && W.sf_atoms != nullptr && (epi == EPI_BIAS || epi == EPI_BIAS_GELU);
}

// One launch over all experts: A rows are expert-contiguous in 128-row blocks (tile_expert), W / bias are stacks.
static int gemm_grouped(DeviceCtx* c, int wfmt, const void* A, const Mat& W, const float* bias, void* C, int m_padded,
                        int m_algorithmic, int N, int K, int epi, int n_experts) {
  if (use_block_scaled(wfmt, W, epi)) {
    // MXFP8 x MXFP8 on the block-scaled tensor-core path: quantise the activations, multiply the stored bytes
    int rc = quantize_activation(c, A, m_padded, K);
    if (rc) return rc;
    KernelScope ks(c, B200EMB_KCLASS_GEMM);
    c->gemm_flops += 2.0 * m_algorithmic * N * K;
    return launch_gemm_mxfp8(c->act_q, c->act_sf, W.q, W.sf_atoms, bias, C, m_padded, N, K, epi, c->sm_count, c->d_err,
                             c->stream, c->tile_expert, n_experts);
  }
  const void* w = W.w;
  if (W.q != nullptr) {
    KernelScope ks(c, B200EMB_KCLASS_OTHER);
    int rc = launch_dequantize(W.q, W.s, W.rows, W.cols, wfmt, c->wscratch, c->stream);
    if (rc) return rc;
    w = c->wscratch;
  }
  KernelScope ks(c, B200EMB_KCLASS_GEMM);
  c->gemm_flops += 2.0 * m_algorithmic * N * K;
  return launch_gemm_bf16(A, w, bias, C, m_padded, N, K, epi, c->sm_count, c->d_err, c->stream, N % 256 == 0 ? 256 : 128,
                          W.alpha, c->tile_expert, n_experts);
}

// Up to this many rows (tokens on the device) an NVFP4 GEMM whose 256-column tiles fill the machine expands its
// weights inside the kernel; otherwise the matrix is expanded once into the scratch and multiplied by the bf16
// kernel. In-kernel expansion re-expands a weight tile for every 256-row tile of A that meets it, so its cost grows
// with the rows, while the separate pass costs a fixed 2.6 bytes of traffic per weight. Measured on the Qwen2-7B
// gate/up shape (37888 x 3584, SwiGLU): 0.125 against 0.156 ms at 32 rows, 0.130 against 0.159 ms at 256, 0.37
// against 0.26 ms at 1024, 5.0 against 2.6 ms at 16384; the narrow matrices (14-18 column tiles) lose at every
// row count because the kernel has no tiles narrower than 256. B200EMB_W4_FUSED_MAX_ROWS overrides the default.
static int w4_fused_max_rows() {
  static const int v = [] {
    const char* e = getenv("B200EMB_W4_FUSED_MAX_ROWS");
    return e != nullptr ? atoi(e) : 512;
  }();
  return v;
}

// GEMM against a model weight; a block-quantised weight is expanded into the scratch first.
static int gemm(DeviceCtx* c, int wfmt, const void* A, const Mat& W, const float* bias, void* C, int M, int N, int K,
                int epi) {
  // Dense layers keep bf16 activations (weights are expanded to bf16): quantising the activations of
  // every projection to fp8 as well costs more accuracy than the 0.999 cosine bar allows (0.9987 measured
  // on a two-layer decoder); the block-scaled fp8 x fp8 path is used for the expert GEMMs only.
  const void* w = W.w;
  if (W.q != nullptr && wfmt == B200EMB_WFMT_NVFP4 && M <= w4_fused_max_rows() && N / 256 >= c->sm_count / 2 &&
      gemm_w4_supported(M, N, K, epi)) {
    // NVFP4 weights, few rows: expanded tile by tile inside the GEMM, straight from the stored bytes
    KernelScope ks(c, B200EMB_KCLASS_GEMM);
    c->gemm_flops += 2.0 * M * N * K;
    return launch_gemm_w4(A, W.q, W.s, bias, C, M, N, K, epi, W.alpha, c->sm_count, c->d_err, c->stream);
  }
  if (W.q != nullptr) {
    KernelScope ks(c, B200EMB_KCLASS_OTHER);
    int rc = launch_dequantize(W.q, W.s, W.rows, W.cols, wfmt, c->wscratch, c->stream);
    if (rc) return rc;
    w = c->wscratch;
  }
  KernelScope ks(c, B200EMB_KCLASS_GEMM);
  c->gemm_flops += 2.0 * M * N * K;
  return launch_gemm_bf16(A, w, bias, C, M, N, K, epi, c->sm_count, c->d_err, c->stream, 0, W.alpha);
}

// Enqueues every kernel of one forward on c->stream. Inputs are on the device.
static int enqueue_forward(b200emb_handle* h, DeviceCtx* c, const int32_t* d_ids, const int32_t* d_types,
                           const int32_t* d_cu, int n_seqs, int n_tokens, int n_tiles, float* d_out,
                           int64_t out_row_stride) {
  const b200emb_model_desc& d = h->desc;
  const ModelW& w = c->w;
  const int H = d.hidden, F = d.ffn, T = n_tokens;
  const int QKV = (d.n_heads + 2 * d.n_kv_heads) * d.head_dim;
  int rc;
  pdl_for_batch(T, H);
  if (d.arch == B200EMB_ARCH_DECODER) {
    // pre-RMSNorm decoder block (Qwen2): h is the fp32 residual stream
    {
      KernelScope ks(c, B200EMB_KCLASS_EMBED);
      rc = launch_embed_ln(d_ids, nullptr, d_cu, n_seqs, T, w.word, nullptr, nullptr, nullptr, nullptr, H, 0, d.norm_eps,
                           c->y, c->stream, d.vocab, 0, c->d_err);
      if (rc) return rc;
    }
    {
      KernelScope ks(c, B200EMB_KCLASS_OTHER);
      rc = launch_widen(c->y, c->hres, (size_t)T * H, c->stream);
      if (rc) return rc;
    }
    for (int l = 0; l < d.n_layers; ++l) {
      const LayerW& L = w.layers[l];
      {
        KernelScope ks(c, B200EMB_KCLASS_NORM);
        rc = launch_add_rmsnorm(c->hres, l == 0 ? nullptr : c->y, L.ln1_g, T, H, d.norm_eps, c->x, c->stream);
        if (rc) return rc;
      }
      rc = gemm(c, d.weight_format, c->x, L.qkv_w, L.qkv_b, c->qkv, T, QKV, H, EPI_BIAS);
      if (rc) return rc;
      {
        KernelScope ks(c, B200EMB_KCLASS_OTHER);
        rc = launch_rope(c->qkv, d_cu, n_seqs, T, d.n_heads + d.n_kv_heads, QKV, d.head_dim, c->rope_cs, c->stream, d.max_pos);
        if (rc) return rc;
      }
      {
        KernelScope ks(c, B200EMB_KCLASS_ATTN);
        if (attention_tile_rows(d.head_dim, 1) == 128)
          rc = launch_attention_tc(c->qkv, c->ctx, c->d_tiles, n_tiles, T, d.n_heads, d.n_kv_heads, d.head_dim, 1, 0,
                                   c->sm_count, c->d_err, c->stream);
        else
          rc = launch_attention(c->qkv, c->ctx, c->d_tiles, n_tiles, d.n_heads, d.n_kv_heads, d.head_dim, 1, c->stream);
        if (rc) return rc;
      }
      rc = gemm(c, d.weight_format, c->ctx, L.o_w, nullptr, c->y, T, H, d.n_heads * d.head_dim, EPI_BIAS);
      if (rc) return rc;
      {
        KernelScope ks(c, B200EMB_KCLASS_NORM);
        rc = launch_add_rmsnorm(c->hres, c->y, L.ln2_g, T, H, d.norm_eps, c->x, c->stream);
        if (rc) return rc;
      }
      rc = gemm(c, d.weight_format, c->x, L.ffn1_w, nullptr, c->ffn, T, 2 * F, H, EPI_BIAS_SWIGLU);  // silu(gate) * up fused
      if (rc) return rc;
      rc = gemm(c, d.weight_format, c->ffn, L.ffn2_w, nullptr, c->y, T, H, F, EPI_BIAS);
      if (rc) return rc;
    }
    {
      KernelScope ks(c, B200EMB_KCLASS_NORM);
      rc = launch_add_rmsnorm(c->hres, c->y, w.final_norm_g, T, H, d.norm_eps, c->x, c->stream);
      if (rc) return rc;
    }
    KernelScope ks(c, B200EMB_KCLASS_POOL);
    if (d.pooling == B200EMB_POOL_TOKENS) return launch_token_rows(c->x, T, H, d.normalize, d_out, out_row_stride, c->stream);
    return launch_pool(c->x, d_cu, n_seqs, H, d.pooling, d.normalize, d_out, out_row_stride, 0, c->stream, T);
  }
  {
    KernelScope ks(c, B200EMB_KCLASS_EMBED);
    rc = launch_embed_ln(d_ids, w.type != nullptr ? d_types : nullptr, d_cu, n_seqs, T, w.word, w.pos, w.type,
                         w.emb_ln_g, w.emb_ln_b, H, d.pos_offset, d.norm_eps, c->x, c->stream, d.vocab, d.type_vocab,
                         c->d_err, d.max_pos);
    if (rc) return rc;
  }
  for (int l = 0; l < d.n_layers; ++l) {
    const LayerW& L = w.layers[l];
    rc = gemm(c, d.weight_format, c->x, L.qkv_w, L.qkv_b, c->qkv, T, QKV, H, EPI_BIAS);
    if (rc) return rc;
    {
      KernelScope ks(c, B200EMB_KCLASS_ATTN);
      if (attention_tile_rows(d.head_dim, 0) == 128)
        rc = launch_attention_tc(c->qkv, c->ctx, c->d_tiles, n_tiles, T, d.n_heads, d.n_kv_heads, d.head_dim, 0, 0,
                                 c->sm_count, c->d_err, c->stream);
      else
        rc = launch_attention(c->qkv, c->ctx, c->d_tiles, n_tiles, d.n_heads, d.n_kv_heads, d.head_dim, 0, c->stream);
      if (rc) return rc;
    }
    // The residual is added by the LayerNorm kernel, not by the GEMM epilogue. An epilogue that read its thread's
    // residual row with 16-byte loads (issued before the wait for the accumulator) and added it behind the bias was
    // measured on the BERT-large batch: the 48 GEMMs of a forward took 7 ms longer, the LayerNorms 1.3 ms less
    // (83.1 + 8.3 ms against 76.1 + 9.6 ms), and the 20 extra registers cost the other GEMMs 4 ms as well.
    rc = gemm(c, d.weight_format, c->ctx, L.o_w, L.o_b, c->y, T, H, d.n_heads * d.head_dim, EPI_BIAS);
    if (rc) return rc;
    {
      KernelScope ks(c, B200EMB_KCLASS_NORM);
      rc = launch_add_ln(c->x, c->y, L.ln1_g, L.ln1_b, T, H, d.norm_eps, c->x2, c->stream);
      if (rc) return rc;
    }
    if (L.is_moe) {
      const int Mp = moe_max_row_blocks(T, d.top_k, d.n_experts) * 128;
      {
        KernelScope ks(c, B200EMB_KCLASS_OTHER);
        rc = launch_moe_router(c->x2, L.router_w, L.router_b, T, H, d.n_experts, d.top_k, c->topk_idx, c->topk_w,
                               c->moe_counts, c->stream);
        if (rc) return rc;
      }
      if (use_block_scaled(d.weight_format, L.ffn1_w, EPI_BIAS_GELU) && use_block_scaled(d.weight_format, L.ffn2_w, EPI_BIAS) &&
          H % 128 == 0 && F % 128 == 0) {
        // MXFP8 experts on the block-scaled tensor-core path, activations in MXFP8 end to end: the scatter
        // writes e4m3 + scales, GEMM 1 (GELU) writes its output as MXFP8 again, GEMM 2 returns bf16.
        rc = grow_bytes(&c->act_q, &c->act_q_bytes, (size_t)Mp * H, false);
        if (!rc) rc = grow_bytes(&c->act_sf, &c->act_sf_bytes, mxfp8_sf_atoms_bytes(Mp, H), true);
        if (!rc) rc = grow_bytes(&c->act2_q, &c->act2_q_bytes, (size_t)Mp * F, false);
        if (!rc) rc = grow_bytes(&c->act2_sf, &c->act2_sf_bytes, mxfp8_sf_atoms_bytes(Mp, F), true);
        if (rc) return rc;
        {
          KernelScope ks(c, B200EMB_KCLASS_OTHER);
          c->launches++;
          rc = launch_moe_scatter(c->x2, c->topk_idx, c->moe_counts, T, d.top_k, H, d.n_experts, c->moe_cursor,
                                  c->tile_expert, c->row_of, nullptr, c->stream, c->act_q, c->act_sf);
          if (rc) return rc;
        }
        {
          KernelScope ks(c, B200EMB_KCLASS_GEMM);
          c->gemm_flops += 2.0 * T * d.top_k * (double)F * H;
          rc = launch_gemm_mxfp8(c->act_q, c->act_sf, L.ffn1_w.q, L.ffn1_w.sf_atoms, L.ffn1_b, c->act2_q, Mp, F, H,
                                 EPI_BIAS_GELU, c->sm_count, c->d_err, c->stream, c->tile_expert, d.n_experts, c->act2_sf);
          if (rc) return rc;
        }
        {
          KernelScope ks(c, B200EMB_KCLASS_GEMM);
          c->gemm_flops += 2.0 * T * d.top_k * (double)F * H;
          rc = launch_gemm_mxfp8(c->act2_q, c->act2_sf, L.ffn2_w.q, L.ffn2_w.sf_atoms, L.ffn2_b, c->yperm, Mp, H, F,
                                 EPI_BIAS, c->sm_count, c->d_err, c->stream, c->tile_expert, d.n_experts);
          if (rc) return rc;
        }
        KernelScope ks(c, B200EMB_KCLASS_NORM);
        rc = launch_moe_combine_ln(c->x2, c->yperm, c->row_of, c->topk_w, d.top_k, L.ln2_g, L.ln2_b, T, H, d.norm_eps,
                                   c->x, c->stream);
        if (rc) return rc;
        continue;
      }
      {
        KernelScope ks(c, B200EMB_KCLASS_OTHER);
        c->launches++;  // offsets + scatter
        rc = launch_moe_scatter(c->x2, c->topk_idx, c->moe_counts, T, d.top_k, H, d.n_experts, c->moe_cursor,
                                c->tile_expert, c->row_of, c->xperm, c->stream);
        if (rc) return rc;
      }
      rc = gemm_grouped(c, d.weight_format, c->xperm, L.ffn1_w, L.ffn1_b, c->hperm, Mp, T * d.top_k, F, H, EPI_BIAS_GELU,
                        d.n_experts);
      if (rc) return rc;
      rc = gemm_grouped(c, d.weight_format, c->hperm, L.ffn2_w, L.ffn2_b, c->yperm, Mp, T * d.top_k, H, F, EPI_BIAS,
                        d.n_experts);
      if (rc) return rc;
      KernelScope ks(c, B200EMB_KCLASS_NORM);
      rc = launch_moe_combine_ln(c->x2, c->yperm, c->row_of, c->topk_w, d.top_k, L.ln2_g, L.ln2_b, T, H, d.norm_eps,
                                 c->x, c->stream);
      if (rc) return rc;
      continue;
    }
    rc = gemm(c, d.weight_format, c->x2, L.ffn1_w, L.ffn1_b, c->ffn, T, F, H, EPI_BIAS_GELU);
    if (rc) return rc;
    rc = gemm(c, d.weight_format, c->ffn, L.ffn2_w, L.ffn2_b, c->y, T, H, F, EPI_BIAS);
    if (rc) return rc;
    {
      KernelScope ks(c, B200EMB_KCLASS_NORM);
      rc = launch_add_ln(c->x2, c->y, L.ln2_g, L.ln2_b, T, H, d.norm_eps, c->x, c->stream);
      if (rc) return rc;
    }
  }
  if (d.head == B200EMB_HEAD_NONE) {
    KernelScope ks(c, B200EMB_KCLASS_POOL);
    if (d.pooling == B200EMB_POOL_TOKENS)
      rc = launch_token_rows(c->x, T, H, d.normalize, d_out, out_row_stride, c->stream);
    else
      rc = launch_pool(c->x, d_cu, n_seqs, H, d.pooling, d.normalize, d_out, out_row_stride, 0, c->stream, T);
    if (rc) return rc;
  } else {
    {
      KernelScope ks(c, B200EMB_KCLASS_POOL);
      rc = launch_pool(c->x, d_cu, n_seqs, H, d.pooling, 0, c->pooled, H, 1, c->stream, T);
      if (rc) return rc;
    }
    rc = gemm(c, c->pooled, w.head_dense_w, w.head_dense_b, c->head_h, n_seqs, H, H, EPI_BIAS_TANH);
    if (rc) return rc;
    {
      KernelScope ks(c, B200EMB_KCLASS_OTHER);
      rc = launch_small_proj(c->head_h, w.head_out_w, w.head_out_b, n_seqs, H, d.n_labels, d_out, out_row_stride,
                             c->stream);
      if (rc) return rc;
      if (d.label_scores) {
        rc = launch_label_scores(d_out, n_seqs, d.n_labels, out_row_stride, c->stream);
        if (rc) return rc;
      }
    }
  }
  return B200EMB_OK;
}

static int validate_batch(const b200emb_model_desc& d, const int32_t* ids, const int32_t* types, const int32_t* cu,
                          int n_seqs, int n_tokens) {
  if (n_seqs < 0 || n_tokens < 0) return set_error(B200EMB_ERR_INVALID, "negative batch size");
  if (n_seqs == 0) {
    if (n_tokens != 0) return set_error(B200EMB_ERR_INVALID, "n_tokens must be 0 for an empty batch");
    return B200EMB_OK;
  }
  if (ids == nullptr || cu == nullptr) return set_error(B200EMB_ERR_INVALID, "null input pointer");
  if (cu[0] != 0) return set_error(B200EMB_ERR_INVALID, "cu_seqlens[0] must be 0");
  for (int i = 0; i < n_seqs; ++i) {
    const int len = cu[i + 1] - cu[i];
    if (len <= 0) return set_error(B200EMB_ERR_INVALID, "cu_seqlens must be strictly increasing (sequence %d has length %d)", i, len);
    if (len + d.pos_offset > d.max_pos)
      return set_error(B200EMB_ERR_INVALID, "sequence %d has %d tokens; the position table holds %d", i, len, d.max_pos - d.pos_offset);
  }
  if (cu[n_seqs] != n_tokens) return set_error(B200EMB_ERR_INVALID, "cu_seqlens[n_seqs] = %d != n_tokens = %d", cu[n_seqs], n_tokens);
  for (int t = 0; t < n_tokens; ++t) {
    if (ids[t] < 0 || ids[t] >= d.vocab) return set_error(B200EMB_ERR_INVALID, "input_ids[%d] = %d outside the vocabulary of %d", t, ids[t], d.vocab);
  }
  if (types != nullptr && d.type_vocab > 0) {
    for (int t = 0; t < n_tokens; ++t)
      if (types[t] < 0 || types[t] >= d.type_vocab) return set_error(B200EMB_ERR_INVALID, "token_type_ids[%d] = %d out of range", t, types[t]);
  }
  return B200EMB_OK;
}

struct ShardResult {
  int rc = 0;
  std::string msg;
  float h2d_ms = 0, kernels_ms = 0, d2h_ms = 0;
};

static void collect_kernel_times(DeviceCtx* c, b200emb_timing* timing) {
  for (size_t i = 0; i < c->kev_used; ++i) {
    float ms = 0;
    if (cudaEventElapsedTime(&ms, c->kev[i].a, c->kev[i].b) == cudaSuccess) {
      timing->kclass_ms[c->kev[i].kclass] += ms;
      timing->kclass_launches[c->kev[i].kclass] += 1;
    }
  }
}

// Bytes of one result row at an output precision.
static size_t out_row_bytes(const b200emb_handle* h, int precision) {
  switch (precision) {
    case B200EMB_EMB_INT8:
    case B200EMB_EMB_UINT8: return (size_t)h->out_dim;
    case B200EMB_EMB_BINARY:
    case B200EMB_EMB_UBINARY: return (size_t)h->out_dim / 8;
  }
  return sizeof(float) * (size_t)h->out_dim;
}

// Checked build (-DB200EMB_BOUNDS=1): reads and clears the status words of the units whose kernels check the
// indices they read from device memory; a recorded code becomes B200EMB_ERR_INVALID. Nothing in the normal build.
static int bounds_after_forward(cudaStream_t s) {
#if B200EMB_BOUNDS
  struct Unit {
    const char* name;
    int (*take)(cudaStream_t);
  };
  const Unit units[] = {{"row kernels", rowops_bounds_status},
                        {"mixture-of-experts kernels", moe_bounds_status},
                        {"bf16 GEMM", gemm_bf16_bounds_status},
                        {"MXFP8 GEMM", gemm_mxfp8_bounds_status}};
  int first = 0;
  const char* where = "";
  for (const Unit& u : units) {
    const int v = u.take(s);  // every unit is read, so all words are clear afterwards
    if (v < 0) return set_error(B200EMB_ERR_CUDA, "device index check: could not read the status of the %s", u.name);
    if (v > 0 && first == 0) {
      first = v;
      where = u.name;
    }
  }
  if (first != 0) {
    const char* what = first == BOUNDS_POOL_RANGE        ? "a sequence's token range leaves the token stream"
                       : first == BOUNDS_ROPE_POSITION   ? "a position beyond the rotary table"
                       : first == BOUNDS_EMBED_POSITION  ? "a position beyond the position table"
                       : first == BOUNDS_MOE_EXPERT      ? "an expert choice outside [0, n_experts)"
                       : first == BOUNDS_MOE_ROW         ? "a row beyond the padded expert-contiguous layout"
                       : first == BOUNDS_GEMM_EXPERT     ? "a row block's expert outside [0, n_experts)"
                                                         : "unknown code";
    return set_error(B200EMB_ERR_INVALID, "device index check: code %d (%s) in the %s; the access read index 0 instead", first,
                     what, where);
  }
#else
  (void)s;
#endif
  return B200EMB_OK;
}

// Runs one shard (host inputs, shard-local cu_seqlens) on device context c and leaves the
// result rows in dst (row stride dst_stride_bytes), quantised on the device when precision is not float32.
static void run_shard(b200emb_handle* h, DeviceCtx* c, const int32_t* ids, const int32_t* types, const int32_t* cu,
                      int n_seqs, int n_tokens, uint8_t* dst, int64_t dst_stride_bytes, int precision,
                      const double* h_ranges, bool per_kernel, ShardResult* res) {
  auto fail = [&](int rc) {
    res->rc = rc;
    res->msg = g_err;
  };
  if (cudaSetDevice(c->dev) != cudaSuccess) return fail(set_error(B200EMB_ERR_CUDA, "cudaSetDevice(%d) failed", c->dev));
  c->launches = 0;
  c->gemm_flops = 0;
  c->per_kernel = per_kernel;
  c->kev_used = 0;
  if (n_seqs == 0) return;
  const int bq = attention_tile_rows(h->desc.head_dim, h->desc.arch == B200EMB_ARCH_DECODER);
  const int n_tiles = attention_build_tiles_q(cu, n_seqs, bq, nullptr);
  int rc = ensure_capacity(h, c, n_tokens, n_seqs, n_tiles);
  if (rc) return fail(rc);
  attention_build_tiles_q(cu, n_seqs, bq, c->h_tiles);
  cudaStream_t s = c->stream;
  const bool use_types = types != nullptr && h->desc.type_vocab > 0;
#define B2_TRY(expr)                                                                              \
  do {                                                                                            \
    cudaError_t e__ = (expr);                                                                     \
    if (e__ != cudaSuccess) return fail(set_error(B200EMB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__))); \
  } while (0)
  B2_TRY(cudaEventRecord(c->ev[0], s));
  B2_TRY(cudaMemcpyAsync(c->d_ids, ids, sizeof(int32_t) * n_tokens, cudaMemcpyHostToDevice, s));
  if (use_types) B2_TRY(cudaMemcpyAsync(c->d_types, types, sizeof(int32_t) * n_tokens, cudaMemcpyHostToDevice, s));
  B2_TRY(cudaMemcpyAsync(c->d_cu, cu, sizeof(int32_t) * (n_seqs + 1), cudaMemcpyHostToDevice, s));
  B2_TRY(cudaMemcpyAsync(c->d_tiles, c->h_tiles, sizeof(AttnTile) * n_tiles, cudaMemcpyHostToDevice, s));
  B2_TRY(cudaEventRecord(c->ev[1], s));
  rc = enqueue_forward(h, c, c->d_ids, use_types ? c->d_types : nullptr, c->d_cu, n_seqs, n_tokens, n_tiles, c->d_out,
                       h->out_dim);
  if (rc) {
    cudaStreamSynchronize(s);
    return fail(rc);
  }
  const size_t n_rows = h->desc.pooling == B200EMB_POOL_TOKENS ? n_tokens : n_seqs;
  const size_t row_bytes = out_row_bytes(h, precision);
  const uint8_t* d_rows = reinterpret_cast<const uint8_t*>(c->d_out);
  if (precision != B200EMB_EMB_FLOAT32) {
    if (c->d_qout_bytes < n_rows * row_bytes) {
      cudaFree(c->d_qout);
      c->d_qout = nullptr;
      c->d_qout_bytes = std::max(n_rows * row_bytes, (size_t)1 << 20);
      B2_TRY(cudaMalloc(reinterpret_cast<void**>(&c->d_qout), c->d_qout_bytes));
    }
    if (h_ranges != nullptr) {
      if (c->d_ranges == nullptr) B2_TRY(cudaMalloc(reinterpret_cast<void**>(&c->d_ranges), sizeof(double) * 2 * h->out_dim));
      B2_TRY(cudaMemcpyAsync(c->d_ranges, h_ranges, sizeof(double) * 2 * h->out_dim, cudaMemcpyHostToDevice, s));
    }
    KernelScope ks(c, B200EMB_KCLASS_POOL);
    rc = launch_quantize_embeddings(c->d_out, (int)n_rows, h->out_dim, h->out_dim, precision,
                                    h_ranges != nullptr ? c->d_ranges : nullptr, c->d_qout, (int64_t)row_bytes, s);
    if (rc) {
      cudaStreamSynchronize(s);
      return fail(rc);
    }
    d_rows = c->d_qout;
  }
  B2_TRY(cudaEventRecord(c->ev[2], s));
  B2_TRY(cudaMemcpy2DAsync(dst, (size_t)dst_stride_bytes, d_rows, row_bytes, row_bytes, n_rows, cudaMemcpyDeviceToHost, s));
  B2_TRY(cudaMemcpyAsync(c->h_err, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, s));
  B2_TRY(cudaEventRecord(c->ev[3], s));
  B2_TRY(cudaStreamSynchronize(s));
#undef B2_TRY
  cudaEventElapsedTime(&res->h2d_ms, c->ev[0], c->ev[1]);
  cudaEventElapsedTime(&res->kernels_ms, c->ev[1], c->ev[2]);
  cudaEventElapsedTime(&res->d2h_ms, c->ev[2], c->ev[3]);
  if (*c->h_err != 0) {
    const int code = *c->h_err;
    cudaMemsetAsync(c->d_err, 0, sizeof(int), s);
    cudaStreamSynchronize(s);
    return fail(set_error(B200EMB_ERR_DEVICE_WAIT, "a device-side wait gave up (role %d) on device %d", code, c->dev));
  }
  if (int brc = bounds_after_forward(s)) return fail(brc);
}

// Cost of a sequence of length L on one device, up to a common factor: a * L + b * L * L.
// a = GEMM flops per token averaged over the layers (a routed layer runs top_k experts plus the
// router); b = attention flops per token pair times ATTN_TIME_PER_FLOP, the measured ratio of the
// attention kernels' time per flop to the GEMMs' (the GEMMs run near the tensor peak, attention does
// not: weighting both by flops alone under-weights long sequences and leaves the shards uneven in time).
static constexpr double ATTN_TIME_PER_FLOP = 4.0;
static void cost_model(const b200emb_model_desc& d, double* a, double* b) {
  const double H = d.hidden, F = d.ffn;
  const double QKV = (double)(d.n_heads + 2 * d.n_kv_heads) * d.head_dim;
  const bool dec = d.arch == B200EMB_ARCH_DECODER;
  double ffn = (dec ? 6.0 : 4.0) * H * F;
  if (d.arch == B200EMB_ARCH_MOE && d.moe_every > 0 && d.n_layers > 0) {
    int routed = 0;
    for (int l = 0; l < d.n_layers; ++l) routed += (l % d.moe_every) == d.moe_every - 1;
    const double moe = d.top_k * 4.0 * H * F + 2.0 * H * d.n_experts;
    ffn = (routed * moe + (d.n_layers - routed) * ffn) / d.n_layers;
  }
  *a = 2.0 * H * QKV + 2.0 * H * H + ffn;
  *b = (dec ? 2.0 : 4.0) * H * ATTN_TIME_PER_FLOP;
}

static void partition_lpt(const int32_t* lens, int n, int n_shards, double a, double b, int32_t* shard_of) {
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  auto cost = [&](int i) { return a * lens[i] + b * (double)lens[i] * lens[i]; };
  std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return cost(x) > cost(y); });
  std::vector<double> load(n_shards, 0.0);
  for (int idx = 0; idx < n; ++idx) {
    const int i = order[idx];
    int best = 0;
    for (int s = 1; s < n_shards; ++s)
      if (load[s] < load[best]) best = s;
    shard_of[i] = best;
    load[best] += cost(i);
  }
}

}  // namespace b2

// =====================================================================================
// C ABI
// =====================================================================================
using namespace b2;

extern "C" {

const char* b200emb_last_error(void) { return g_err; }

int b200emb_device_count(void) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) return -set_error(B200EMB_ERR_CUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
  return n;
}

int b200emb_partition(const int32_t* lens, int32_t n_seqs, int32_t n_shards, double cost_linear,
                      double cost_quadratic, int32_t* shard_of) {
  if (n_seqs < 0 || n_shards <= 0 || (n_seqs > 0 && (lens == nullptr || shard_of == nullptr)))
    return set_error(B200EMB_ERR_INVALID, "partition: bad arguments");
  partition_lpt(lens, n_seqs, n_shards, cost_linear, cost_quadratic, shard_of);
  return B200EMB_OK;
}

int b200emb_cost_model(const b200emb_model_desc* desc, double* cost_linear, double* cost_quadratic) {
  if (desc == nullptr || cost_linear == nullptr || cost_quadratic == nullptr)
    return set_error(B200EMB_ERR_INVALID, "cost_model: null argument");
  cost_model(*desc, cost_linear, cost_quadratic);
  return B200EMB_OK;
}

int b200emb_checked_build(void) { return B200EMB_BOUNDS; }

int b200emb_tensor_map_stats(uint64_t* hits, uint64_t* misses) {
  if (hits == nullptr || misses == nullptr) return set_error(B200EMB_ERR_INVALID, "tensor_map_stats: null argument");
  tmap_cache_stats(hits, misses);
  return B200EMB_OK;
}

int b200emb_test_fail_allocs(int32_t after, int32_t n) {
  std::lock_guard<std::mutex> lk(g_fail_mu);
  g_fail_after = after < 0 ? 0 : after;
  g_fail_allocs = n < 0 ? 0 : n;
  return B200EMB_OK;
}

int b200emb_create(const b200emb_model_desc* desc, const char* weight_path, const int32_t* device_ids,
                   int32_t n_devices, b200emb_handle** out) {
  if (desc == nullptr || weight_path == nullptr || out == nullptr || n_devices <= 0 || device_ids == nullptr)
    return set_error(B200EMB_ERR_INVALID, "create: null argument or no device");
  *out = nullptr;
  int rc = validate_desc(*desc);
  if (rc) return rc;
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess || visible <= 0)
    return set_error(B200EMB_ERR_CUDA, "no CUDA device is usable; this library has no CPU path");
  for (int i = 0; i < n_devices; ++i)
    if (device_ids[i] < 0 || device_ids[i] >= visible)
      return set_error(B200EMB_ERR_INVALID, "device id %d not in [0, %d)", device_ids[i], visible);
  WeightFile wf;
  rc = read_weight_file(weight_path, &wf);
  if (rc) return rc;

  b200emb_handle* h = new b200emb_handle();
  h->desc = *desc;
  h->out_dim = desc->head == B200EMB_HEAD_CLASSIFIER ? desc->n_labels : desc->hidden;
  cost_model(*desc, &h->cost_a, &h->cost_b);
  for (int i = 0; i < n_devices && !rc; ++i) {
    DeviceCtx* c = new DeviceCtx();
    h->devs.push_back(c);
    c->dev = device_ids[i];
    cudaError_t e = cudaSetDevice(c->dev);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, c->dev);
    if (e != cudaSuccess) {
      rc = set_error(B200EMB_ERR_CUDA, "device %d: %s", c->dev, cudaGetErrorString(e));
      break;
    }
    if (prop.major != 10) {
      rc = set_error(B200EMB_ERR_UNSUPPORTED, "device %d is sm_%d%d; the kernels are built for sm_100a only", c->dev,
                     prop.major, prop.minor);
      break;
    }
    c->sm_count = prop.multiProcessorCount;
    rc = kernels_init_device();
    if (rc) break;
#define B2_CR(expr)                                                                                   \
  if (!rc) {                                                                                          \
    cudaError_t e2 = (expr);                                                                          \
    if (e2 != cudaSuccess) rc = set_error(B200EMB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e2)); \
  }
    B2_CR(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    for (int k = 0; k < 4; ++k) B2_CR(cudaEventCreate(&c->ev[k]));
    B2_CR(cudaMalloc(reinterpret_cast<void**>(&c->blob), std::max<size_t>(wf.data.size(), 256)));
    B2_CR(cudaMemcpy(c->blob, wf.data.data(), wf.data.size(), cudaMemcpyHostToDevice));
    B2_CR(cudaMalloc(reinterpret_cast<void**>(&c->d_err), sizeof(int)));
    B2_CR(cudaMemset(c->d_err, 0, sizeof(int)));
    B2_CR(cudaMallocHost(reinterpret_cast<void**>(&c->h_err), sizeof(int)));
    if (!rc) rc = bind_weights(*desc, wf, c);
    if (!rc && c->wscratch_elems > 0) {
      B2_CR(cudaMalloc(reinterpret_cast<void**>(&c->wscratch), c->wscratch_elems * sizeof(__nv_bfloat16)));
    }
    if (!rc && desc->arch == B200EMB_ARCH_DECODER) {
      // (cos, sin) of position * theta^(-2i/d), computed in fp32 the way the torch reference does
      const int half = desc->head_dim / 2;
      std::vector<float> cs((size_t)desc->max_pos * half * 2);
      for (int i = 0; i < half; ++i) {
        const float inv_freq = 1.0f / powf(desc->rope_theta, (float)(2 * i) / (float)desc->head_dim);
        for (int p = 0; p < desc->max_pos; ++p) {
          const float ang = (float)p * inv_freq;
          cs[((size_t)p * half + i) * 2] = cosf(ang);
          cs[((size_t)p * half + i) * 2 + 1] = sinf(ang);
        }
      }
      B2_CR(cudaMalloc(reinterpret_cast<void**>(&c->rope_cs), cs.size() * sizeof(float)));
      B2_CR(cudaMemcpy(c->rope_cs, cs.data(), cs.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
#undef B2_CR
    if (!rc) rc = ensure_capacity(h, c, std::max(desc->max_tokens, 1), 256, 1024);
  }
  if (rc) {
    std::string keep = g_err;
    b200emb_destroy(h);
    snprintf(g_err, sizeof(g_err), "%s", keep.c_str());
    return rc;
  }
  *out = h;
  return B200EMB_OK;
}

// Reads a bf16 weight file, replaces every layer matrix ("layer.*.w", or only the expert
// matrices when the file has any) by its block-quantised form and writes a new file:
// name.q (packed elements), name.s (block scales), name.gs (NVFP4 tensor scale).
int b200emb_quantize_weights(const char* in_path, const char* out_path, int32_t format, int32_t device_id) {
  if (in_path == nullptr || out_path == nullptr) return set_error(B200EMB_ERR_INVALID, "quantize_weights: null path");
  if (format != B200EMB_WFMT_NVFP4 && format != B200EMB_WFMT_MXFP8)
    return set_error(B200EMB_ERR_INVALID, "quantize_weights: format must be MXFP8 or NVFP4");
  WeightFile wf;
  int rc = read_weight_file(in_path, &wf);
  if (rc) return rc;
  B2_CUDA_CHECK(cudaSetDevice(device_id));
  const uint64_t block = format == B200EMB_WFMT_NVFP4 ? 16 : 32;
  bool has_experts = false;
  for (const TensorEntry& e : wf.entries)
    if (strstr(e.name, ".experts.") != nullptr) has_experts = true;
  struct OutTensor {
    TensorEntry e;
    std::vector<uint8_t> data;
  };
  std::vector<OutTensor> outs;
  auto add = [&](const char* name, uint32_t dtype, uint32_t ndim, uint64_t d0, uint64_t d1, std::vector<uint8_t>&& data) {
    OutTensor t;
    memset(&t.e, 0, sizeof(t.e));
    snprintf(t.e.name, sizeof(t.e.name), "%.63s", name);
    t.e.dtype = dtype;
    t.e.ndim = ndim;
    t.e.dims[0] = d0; t.e.dims[1] = d1; t.e.dims[2] = 1; t.e.dims[3] = 1;
    t.e.nbytes = data.size();
    t.data = std::move(data);
    outs.push_back(std::move(t));
  };
  unsigned int* d_amax = nullptr;
  float* d_gs = nullptr;
  B2_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&d_amax), sizeof(unsigned int)));
  B2_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&d_gs), sizeof(float)));
  for (const TensorEntry& e : wf.entries) {
    const size_t len = strlen(e.name);
    const bool is_layer_mat = e.dtype == 1 && e.ndim == 2 && strncmp(e.name, "layer.", 6) == 0 && len > 2 &&
                              strcmp(e.name + len - 2, ".w") == 0 && e.dims[1] % block == 0 && len < 60;
    const bool selected = is_layer_mat && (!has_experts || strstr(e.name, ".experts.") != nullptr);
    if (!selected) {
      std::vector<uint8_t> copy(wf.data.begin() + e.offset, wf.data.begin() + e.offset + e.nbytes);
      OutTensor t;
      t.e = e;
      t.data = std::move(copy);
      outs.push_back(std::move(t));
      continue;
    }
    const uint64_t rows = e.dims[0], cols = e.dims[1];
    const size_t q_bytes = format == B200EMB_WFMT_NVFP4 ? rows * cols / 2 : rows * cols;
    const size_t s_bytes = rows * cols / block;
    void *d_w = nullptr, *d_q = nullptr, *d_s = nullptr;
    cudaError_t ce = cudaMalloc(&d_w, e.nbytes);
    if (ce == cudaSuccess) ce = cudaMalloc(&d_q, q_bytes);
    if (ce == cudaSuccess) ce = cudaMalloc(&d_s, s_bytes);
    if (ce == cudaSuccess) ce = cudaMemcpy(d_w, wf.data.data() + e.offset, e.nbytes, cudaMemcpyHostToDevice);
    if (ce == cudaSuccess) {
      rc = launch_quantize(d_w, (int64_t)rows, (int64_t)cols, format, d_q, d_s, d_gs, d_amax, nullptr);
      if (!rc) ce = cudaDeviceSynchronize();
    }
    std::vector<uint8_t> q(q_bytes), sc(s_bytes), gs(4);
    if (ce == cudaSuccess && !rc) ce = cudaMemcpy(q.data(), d_q, q_bytes, cudaMemcpyDeviceToHost);
    if (ce == cudaSuccess && !rc) ce = cudaMemcpy(sc.data(), d_s, s_bytes, cudaMemcpyDeviceToHost);
    if (ce == cudaSuccess && !rc && format == B200EMB_WFMT_NVFP4) ce = cudaMemcpy(gs.data(), d_gs, 4, cudaMemcpyDeviceToHost);
    cudaFree(d_w); cudaFree(d_q); cudaFree(d_s);
    if (ce != cudaSuccess && !rc) rc = set_error(B200EMB_ERR_CUDA, "quantize_weights(%s): %s", e.name, cudaGetErrorString(ce));
    if (rc) break;
    char nm[64];
    snprintf(nm, sizeof(nm), "%.59s.q", e.name);
    add(nm, 2, 2, rows, q_bytes / rows, std::move(q));
    snprintf(nm, sizeof(nm), "%.59s.s", e.name);
    add(nm, 2, 2, rows, cols / block, std::move(sc));
    if (format == B200EMB_WFMT_NVFP4) {
      snprintf(nm, sizeof(nm), "%.59s.gs", e.name);
      add(nm, 0, 1, 1, 1, std::move(gs));
    }
  }
  cudaFree(d_amax);
  cudaFree(d_gs);
  if (rc) return rc;
  // write
  const uint64_t header = 8 + 4 + 4 + 8 + sizeof(TensorEntry) * outs.size();
  const uint64_t data_offset = (header + 255) / 256 * 256;
  uint64_t off = 0;
  for (OutTensor& t : outs) {
    t.e.offset = off;
    off = (off + t.e.nbytes + 255) / 256 * 256;
  }
  FILE* f = fopen(out_path, "wb");
  if (f == nullptr) return set_error(B200EMB_ERR_IO, "cannot write %s", out_path);
  const uint32_t n = (uint32_t)outs.size(), zero = 0;
  bool ok = fwrite("B2EW0001", 1, 8, f) == 8 && fwrite(&n, 4, 1, f) == 1 && fwrite(&zero, 4, 1, f) == 1 &&
            fwrite(&data_offset, 8, 1, f) == 1;
  for (const OutTensor& t : outs) ok = ok && fwrite(&t.e, sizeof(TensorEntry), 1, f) == 1;
  std::vector<uint8_t> pad(256, 0);
  ok = ok && fwrite(pad.data(), 1, data_offset - header, f) == data_offset - header;
  uint64_t pos = 0;
  for (const OutTensor& t : outs) {
    if (t.e.offset > pos) ok = ok && fwrite(pad.data(), 1, t.e.offset - pos, f) == t.e.offset - pos;
    ok = ok && (t.data.empty() || fwrite(t.data.data(), 1, t.data.size(), f) == t.data.size());
    pos = t.e.offset + t.data.size();
  }
  ok = (fclose(f) == 0) && ok;
  if (!ok) return set_error(B200EMB_ERR_IO, "short write to %s", out_path);
  return B200EMB_OK;
}

int b200emb_destroy(b200emb_handle* h) {
  if (h == nullptr) return B200EMB_OK;
  for (DeviceCtx* c : h->devs) destroy_ctx(c);
  delete h;
  return B200EMB_OK;
}

static int forward_impl(b200emb_handle* h, const int32_t* input_ids, const int32_t* token_type_ids,
                        const int32_t* cu_seqlens, int32_t n_seqs, int32_t n_tokens, int precision,
                        const double* h_ranges, uint8_t* out, int64_t out_stride_bytes, b200emb_timing* timing) {
  if (h == nullptr) return set_error(B200EMB_ERR_INVALID, "null handle");
  const auto t0 = std::chrono::steady_clock::now();
  int rc = validate_batch(h->desc, input_ids, token_type_ids, cu_seqlens, n_seqs, n_tokens);
  if (rc) return rc;
  if (precision < B200EMB_EMB_FLOAT32 || precision > B200EMB_EMB_UBINARY)
    return set_error(B200EMB_ERR_INVALID, "unknown output precision %d", precision);
  if (precision != B200EMB_EMB_FLOAT32 && h->desc.head != B200EMB_HEAD_NONE)
    return set_error(B200EMB_ERR_INVALID, "output quantisation applies to embeddings, not to classifier logits");
  if ((precision == B200EMB_EMB_INT8 || precision == B200EMB_EMB_UINT8) && h_ranges == nullptr)
    return set_error(B200EMB_ERR_INVALID, "int8 / uint8 outputs need calibration ranges");
  if (precision != B200EMB_EMB_FLOAT32 && (h->out_dim % 8) != 0)
    return set_error(B200EMB_ERR_UNSUPPORTED, "output quantisation needs a dimension that is a multiple of 8");
  const size_t row_bytes = out_row_bytes(h, precision);
  if (n_seqs > 0 && (out == nullptr || out_stride_bytes < (int64_t)row_bytes))
    return set_error(B200EMB_ERR_INVALID, "output buffer missing or row stride %lld bytes < %zu", (long long)out_stride_bytes, row_bytes);
  const bool per_kernel = timing != nullptr && timing->per_kernel != 0;
  const int G = (int)h->devs.size();
  std::vector<ShardResult> res(G);

  if (G == 1 || n_seqs < 2) {
    run_shard(h, h->devs[0], input_ids, token_type_ids, cu_seqlens, n_seqs, n_tokens, out, out_stride_bytes, precision,
              h_ranges, per_kernel, &res[0]);
  } else {
    // Token-balanced split: whole sequences go to the least-loaded device, most expensive
    // first; each device gets its own packed ids / cu_seqlens; rows return to batch order.
    std::vector<int32_t> lens(n_seqs), shard_of(n_seqs);
    for (int i = 0; i < n_seqs; ++i) lens[i] = cu_seqlens[i + 1] - cu_seqlens[i];
    partition_lpt(lens.data(), n_seqs, G, h->cost_a, h->cost_b, shard_of.data());
    std::vector<std::vector<int>> members(G);
    for (int i = 0; i < n_seqs; ++i) members[shard_of[i]].push_back(i);
    std::vector<std::thread> threads;
    for (int g = 0; g < G; ++g) {
      threads.emplace_back([&, g]() {
        DeviceCtx* c = h->devs[g];
        const std::vector<int>& mem = members[g];
        int tok = 0;
        for (int i : mem) tok += lens[i];
        ShardResult* r = &res[g];
        if (mem.empty()) return;
        if (cudaSetDevice(c->dev) != cudaSuccess) {
          r->rc = B200EMB_ERR_CUDA;
          r->msg = "cudaSetDevice failed";
          return;
        }
        int rc2 = ensure_capacity(h, c, tok, (int)mem.size(), 0);
        if (rc2) {
          r->rc = rc2;
          r->msg = g_err;
          return;
        }
        int pos = 0;
        c->h_cu[0] = 0;
        for (size_t k = 0; k < mem.size(); ++k) {
          const int i = mem[k];
          memcpy(c->h_ids + pos, input_ids + cu_seqlens[i], sizeof(int32_t) * lens[i]);
          if (token_type_ids != nullptr) memcpy(c->h_types + pos, token_type_ids + cu_seqlens[i], sizeof(int32_t) * lens[i]);
          pos += lens[i];
          c->h_cu[k + 1] = pos;
        }
        // the pinned staging rows are sized for float32, the widest precision
        uint8_t* stage = reinterpret_cast<uint8_t*>(c->h_out);
        run_shard(h, c, c->h_ids, token_type_ids != nullptr ? c->h_types : nullptr, c->h_cu, (int)mem.size(), tok,
                  stage, (int64_t)row_bytes, precision, h_ranges, per_kernel, r);
        if (r->rc == 0) {
          if (h->desc.pooling == B200EMB_POOL_TOKENS) {
            // token rows: sequence mem[k] owns batch rows cu_seqlens[i] .. and shard rows h_cu[k] ..
            for (size_t k = 0; k < mem.size(); ++k)
              for (int t = 0; t < lens[mem[k]]; ++t)
                memcpy(out + (size_t)(cu_seqlens[mem[k]] + t) * out_stride_bytes,
                       stage + (size_t)(c->h_cu[k] + t) * row_bytes, row_bytes);
          } else {
            for (size_t k = 0; k < mem.size(); ++k)
              memcpy(out + (size_t)mem[k] * out_stride_bytes, stage + k * row_bytes, row_bytes);
          }
        }
      });
    }
    for (auto& t : threads) t.join();
  }

  for (int g = 0; g < G; ++g)
    if (res[g].rc != 0) return set_error(res[g].rc, "%s", res[g].msg.c_str());
  if (timing != nullptr) {
    const int pk = timing->per_kernel;
    memset(timing, 0, sizeof(*timing));
    timing->per_kernel = pk;
    timing->n_devices = G;
    for (int g = 0; g < G; ++g) {
      timing->h2d_ms = std::max(timing->h2d_ms, res[g].h2d_ms);
      timing->kernels_ms = std::max(timing->kernels_ms, res[g].kernels_ms);
      timing->d2h_ms = std::max(timing->d2h_ms, res[g].d2h_ms);
      timing->launches += h->devs[g]->launches;
    }
    timing->gemm_flops = h->devs[0]->gemm_flops;
    if (per_kernel) {
      cudaSetDevice(h->devs[0]->dev);
      collect_kernel_times(h->devs[0], timing);
    }
    timing->total_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
  }
  return B200EMB_OK;
}

int b200emb_forward(b200emb_handle* h, const int32_t* input_ids, const int32_t* token_type_ids,
                    const int32_t* cu_seqlens, int32_t n_seqs, int32_t n_tokens, float* out, int64_t out_row_stride,
                    b200emb_timing* timing) {
  return forward_impl(h, input_ids, token_type_ids, cu_seqlens, n_seqs, n_tokens, B200EMB_EMB_FLOAT32, nullptr,
                      reinterpret_cast<uint8_t*>(out), out_row_stride * (int64_t)sizeof(float), timing);
}

int b200emb_forward_quantized(b200emb_handle* h, const int32_t* input_ids, const int32_t* token_type_ids,
                              const int32_t* cu_seqlens, int32_t n_seqs, int32_t n_tokens, int32_t precision,
                              const double* h_ranges, void* out, int64_t out_row_stride_bytes,
                              b200emb_timing* timing) {
  return forward_impl(h, input_ids, token_type_ids, cu_seqlens, n_seqs, n_tokens, precision, h_ranges,
                      reinterpret_cast<uint8_t*>(out), out_row_stride_bytes, timing);
}

int b200emb_forward_device(b200emb_handle* h, const int32_t* d_input_ids, const int32_t* d_token_type_ids,
                           const int32_t* d_cu_seqlens, const int32_t* h_cu_seqlens, int32_t n_seqs, int32_t n_tokens,
                           float* d_out, int64_t out_row_stride, b200emb_timing* timing) {
  if (h == nullptr) return set_error(B200EMB_ERR_INVALID, "null handle");
  if (h->devs.size() != 1) return set_error(B200EMB_ERR_UNSUPPORTED, "forward_device needs a single-device handle");
  if (n_seqs <= 0 || n_tokens <= 0 || d_input_ids == nullptr || d_cu_seqlens == nullptr || h_cu_seqlens == nullptr ||
      d_out == nullptr || out_row_stride < h->out_dim)
    return set_error(B200EMB_ERR_INVALID, "forward_device: bad arguments");
  if (h_cu_seqlens[0] != 0 || h_cu_seqlens[n_seqs] != n_tokens)
    return set_error(B200EMB_ERR_INVALID, "forward_device: cu_seqlens does not span n_tokens");
  for (int i = 0; i < n_seqs; ++i) {
    const int len = h_cu_seqlens[i + 1] - h_cu_seqlens[i];
    if (len <= 0 || len + h->desc.pos_offset > h->desc.max_pos)
      return set_error(B200EMB_ERR_INVALID, "forward_device: sequence %d has invalid length %d", i, len);
  }
  const auto t0 = std::chrono::steady_clock::now();
  DeviceCtx* c = h->devs[0];
  B2_CUDA_CHECK(cudaSetDevice(c->dev));
  c->launches = 0;
  c->gemm_flops = 0;
  c->per_kernel = timing != nullptr && timing->per_kernel != 0;
  c->kev_used = 0;
  const int bq = attention_tile_rows(h->desc.head_dim, h->desc.arch == B200EMB_ARCH_DECODER);
  const int n_tiles = attention_build_tiles_q(h_cu_seqlens, n_seqs, bq, nullptr);
  int rc = ensure_capacity(h, c, n_tokens, n_seqs, n_tiles);
  if (rc) return rc;
  attention_build_tiles_q(h_cu_seqlens, n_seqs, bq, c->h_tiles);
  cudaStream_t s = c->stream;
  B2_CUDA_CHECK(cudaEventRecord(c->ev[0], s));
  B2_CUDA_CHECK(cudaMemcpyAsync(c->d_tiles, c->h_tiles, sizeof(AttnTile) * n_tiles, cudaMemcpyHostToDevice, s));
  B2_CUDA_CHECK(cudaEventRecord(c->ev[1], s));
  rc = enqueue_forward(h, c, d_input_ids, d_token_type_ids, d_cu_seqlens, n_seqs, n_tokens, n_tiles, d_out,
                       out_row_stride);
  if (rc) {
    cudaStreamSynchronize(s);
    return rc;
  }
  B2_CUDA_CHECK(cudaEventRecord(c->ev[2], s));
  B2_CUDA_CHECK(cudaMemcpyAsync(c->h_err, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, s));
  B2_CUDA_CHECK(cudaStreamSynchronize(s));
  if (*c->h_err != 0) {
    const int code = *c->h_err;
    cudaMemsetAsync(c->d_err, 0, sizeof(int), s);
    cudaStreamSynchronize(s);
    if (code == 32 || code == 33)
      return set_error(B200EMB_ERR_INVALID, "forward_device: %s outside its table (found by the embedding kernel, which read row 0 instead)",
                       code == 32 ? "an input id" : "a token type id");
    return set_error(B200EMB_ERR_DEVICE_WAIT, "a device-side wait gave up (role %d)", code);
  }
  if (int brc = bounds_after_forward(s)) return brc;
  if (timing != nullptr) {
    const int pk = timing->per_kernel;
    memset(timing, 0, sizeof(*timing));
    timing->per_kernel = pk;
    timing->n_devices = 1;
    cudaEventElapsedTime(&timing->h2d_ms, c->ev[0], c->ev[1]);
    cudaEventElapsedTime(&timing->kernels_ms, c->ev[1], c->ev[2]);
    timing->launches = c->launches;
    timing->gemm_flops = c->gemm_flops;
    if (pk) collect_kernel_times(c, timing);
    timing->total_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
  }
  return B200EMB_OK;
}

// ---- single kernels ---------------------------------------------------------------------

// One error word per device for the single-kernel entry points, allocated on first use and kept.
static int op_error_word(int** out) {
  static std::mutex mu;
  static int* words[64] = {};
  int dev = 0;
  B2_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(B200EMB_ERR_UNSUPPORTED, "device index %d too large", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (words[dev] == nullptr) {
    B2_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&words[dev]), sizeof(int)));
    B2_CUDA_CHECK(cudaMemset(words[dev], 0, sizeof(int)));
  }
  *out = words[dev];
  return B200EMB_OK;
}

static int current_sm_count(int* out) {
  int dev = 0;
  B2_CUDA_CHECK(cudaGetDevice(&dev));
  B2_CUDA_CHECK(cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, dev));
  return B200EMB_OK;
}

int b200emb_op_gemm_bf16(const void* A, const void* W, const float* bias, void* C, int32_t M, int32_t N, int32_t K,
                         int32_t epilogue, void* stream) {
  if (A == nullptr || W == nullptr || C == nullptr) return set_error(B200EMB_ERR_INVALID, "gemm: null pointer");
  int rc = kernels_init_device();
  if (rc) return rc;
  int sms = 0;
  rc = current_sm_count(&sms);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int* d_err = nullptr;
  rc = op_error_word(&d_err);
  if (rc) return rc;
  // epilogue values >= 0x100 select the tile width in the upper bits (tests only): (bn << 8) | epi
  const int force_bn = epilogue >> 8;
  rc = launch_gemm_bf16(A, W, bias, C, M, N, K, epilogue & 0xff, sms, d_err, s, force_bn);
  int herr = 0;
  cudaError_t e = cudaMemcpyAsync(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (rc) return rc;
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "gemm: %s", cudaGetErrorString(e));
  if (herr != 0) {
    cudaMemset(d_err, 0, sizeof(int));
    return set_error(B200EMB_ERR_DEVICE_WAIT, "gemm: a device-side wait gave up (role %d)", herr);
  }
  return B200EMB_OK;
}

int b200emb_op_gemm_nvfp4(const void* A, const void* W_q, const void* W_scales, float tensor_scale, const float* bias,
                          void* C, int32_t M, int32_t N, int32_t K, int32_t epilogue, void* stream) {
  if (A == nullptr || W_q == nullptr || W_scales == nullptr || C == nullptr)
    return set_error(B200EMB_ERR_INVALID, "gemm_nvfp4: null pointer");
  if (!(tensor_scale > 0.f)) return set_error(B200EMB_ERR_INVALID, "gemm_nvfp4: the tensor scale must be positive");
  int rc = kernels_init_device();
  if (rc) return rc;
  int sms = 0;
  rc = current_sm_count(&sms);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int* d_err = nullptr;
  rc = op_error_word(&d_err);
  if (rc) return rc;
  rc = launch_gemm_w4(A, W_q, W_scales, bias, C, M, N, K, epilogue, 1.0f / tensor_scale, sms, d_err, s);
  int herr = 0;
  cudaError_t e = cudaMemcpyAsync(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (rc) return rc;
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "gemm_nvfp4: %s", cudaGetErrorString(e));
  if (herr != 0) {
    cudaMemset(d_err, 0, sizeof(int));
    return set_error(B200EMB_ERR_DEVICE_WAIT, "gemm_nvfp4: a device-side wait gave up (role %d)", herr);
  }
  return B200EMB_OK;
}

int b200emb_selftest_bounded_wait(int32_t limit_ms) {
  if (limit_ms <= 0 || limit_ms > 5000) return set_error(B200EMB_ERR_INVALID, "selftest: limit must be in (0, 5000] ms");
  int* d_err = nullptr;
  int rc = op_error_word(&d_err);
  if (rc) return rc;
  rc = launch_wait_selftest(static_cast<unsigned long long>(limit_ms) * 1000000ull, d_err, nullptr);
  if (rc) return rc;
  int herr = 0;
  B2_CUDA_CHECK(cudaMemcpy(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost));
  B2_CUDA_CHECK(cudaMemset(d_err, 0, sizeof(int)));
  if (herr != 0) return set_error(B200EMB_ERR_DEVICE_WAIT, "self-test: the device-side wait gave up as intended (code %d)", herr);
  return B200EMB_OK;
}

int b200emb_op_gemm_mxfp8(const void* A_bf16, const void* W_q, const void* W_scales, const float* bias, void* C,
                          int32_t M, int32_t N, int32_t K, int32_t epilogue, void* stream) {
  if (A_bf16 == nullptr || W_q == nullptr || W_scales == nullptr || C == nullptr)
    return set_error(B200EMB_ERR_INVALID, "gemm_mxfp8: null pointer");
  if (M <= 0 || N <= 0 || K <= 0 || K % 128 || N % 128)
    return set_error(B200EMB_ERR_INVALID, "gemm_mxfp8: need M > 0 and N, K multiples of 128");
  int rc = kernels_init_device();
  if (rc) return rc;
  int sms = 0;
  rc = current_sm_count(&sms);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int* d_err = nullptr;
  rc = op_error_word(&d_err);
  if (rc) return rc;
  uint8_t *aq = nullptr, *sfa = nullptr, *sfw = nullptr;
  const size_t sfa_bytes = mxfp8_sf_atoms_bytes(M, K), sfw_bytes = mxfp8_sf_atoms_bytes(N, K);
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&aq), (size_t)M * K);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&sfa), sfa_bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&sfw), sfw_bytes);
  if (e == cudaSuccess) e = cudaMemsetAsync(sfa, 0, sfa_bytes, s);  // rows past M of the last atom: scale 2^-127
  if (e != cudaSuccess) rc = set_error(B200EMB_ERR_CUDA, "gemm_mxfp8: %s", cudaGetErrorString(e));
  if (!rc) rc = launch_quant_act_mxfp8(A_bf16, M, K, aq, sfa, s);
  if (!rc) rc = launch_sf_to_atoms(W_scales, N, K, sfw, s);
  if (!rc) rc = launch_gemm_mxfp8(aq, sfa, W_q, sfw, bias, C, M, N, K, epilogue, sms, d_err, s);
  int herr = 0;
  e = cudaMemcpyAsync(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(aq); cudaFree(sfa); cudaFree(sfw);
  if (rc) return rc;
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "gemm_mxfp8: %s", cudaGetErrorString(e));
  if (herr != 0) {
    cudaMemset(d_err, 0, sizeof(int));
    return set_error(B200EMB_ERR_DEVICE_WAIT, "gemm_mxfp8: a device-side wait gave up (role %d)", herr);
  }
  return B200EMB_OK;
}

int b200emb_op_attention(const void* qkv, void* out, const int32_t* d_cu_seqlens, const int32_t* h_cu_seqlens,
                         int32_t n_seqs, int32_t n_tokens, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                         int32_t causal, void* stream) {
  (void)d_cu_seqlens;
  if (qkv == nullptr || out == nullptr || h_cu_seqlens == nullptr || n_seqs <= 0)
    return set_error(B200EMB_ERR_INVALID, "attention: null pointer or empty batch");
  if (h_cu_seqlens[0] != 0 || h_cu_seqlens[n_seqs] != n_tokens)
    return set_error(B200EMB_ERR_INVALID, "attention: cu_seqlens does not span n_tokens");
  for (int i = 0; i < n_seqs; ++i)
    if (h_cu_seqlens[i + 1] <= h_cu_seqlens[i]) return set_error(B200EMB_ERR_INVALID, "attention: empty sequence %d", i);
  int rc = kernels_init_device();
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int force_legacy = (causal >> 8) & 1;  // bit 8: use the mma.sync kernel whatever the shape (tests)
  const int variant = (causal >> 9) & 1;       // bit 9: one-CTA-per-SM tensor-memory kernel whatever the shape
  causal &= 1;
  const bool use_tc = !force_legacy && attention_tile_rows(head_dim, causal) == 128;
  const int bq = use_tc ? 128 : 64;
  const int n_tiles = attention_build_tiles_q(h_cu_seqlens, n_seqs, bq, nullptr);
  std::vector<AttnTile> tiles(n_tiles);
  attention_build_tiles_q(h_cu_seqlens, n_seqs, bq, tiles.data());
  AttnTile* d_tiles = nullptr;
  int* d_err = nullptr;
  B2_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&d_tiles), sizeof(AttnTile) * n_tiles + sizeof(int)));
  d_err = reinterpret_cast<int*>(d_tiles + n_tiles);
  cudaMemsetAsync(d_err, 0, sizeof(int), s);
  cudaMemcpyAsync(d_tiles, tiles.data(), sizeof(AttnTile) * n_tiles, cudaMemcpyHostToDevice, s);
  if (use_tc)
  {
    int sms = 0;
    rc = current_sm_count(&sms);
    if (!rc)
      rc = launch_attention_tc(qkv, out, d_tiles, n_tiles, n_tokens, n_heads, n_kv_heads, head_dim, causal, variant, sms,
                               d_err, s);
  }
  else
    rc = launch_attention(qkv, out, d_tiles, n_tiles, n_heads, n_kv_heads, head_dim, causal, s);
  int herr = 0;
  cudaError_t e = cudaMemcpyAsync(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(d_tiles);
  if (rc) return rc;
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "attention: %s", cudaGetErrorString(e));
  if (herr != 0) return set_error(B200EMB_ERR_DEVICE_WAIT, "attention: a device-side wait gave up (role %d)", herr);
  return B200EMB_OK;
}

int b200emb_op_embed_ln(const int32_t* ids, const int32_t* types, const int32_t* d_cu_seqlens, int32_t n_seqs,
                        int32_t n_tokens, const void* word, const void* pos, const void* type_table,
                        const float* gamma, const float* beta, int32_t hidden, int32_t pos_offset, float eps,
                        void* out, void* stream) {
  if (ids == nullptr || d_cu_seqlens == nullptr || word == nullptr || out == nullptr)
    return set_error(B200EMB_ERR_INVALID, "embed_ln: null pointer");
  return launch_embed_ln(ids, types, d_cu_seqlens, n_seqs, n_tokens, word, pos, type_table, gamma, beta, hidden,
                         pos_offset, eps, out, reinterpret_cast<cudaStream_t>(stream));
}

int b200emb_op_add_ln(const void* x, const void* y, const float* gamma, const float* beta, int32_t n_rows,
                      int32_t hidden, float eps, void* out, void* stream) {
  if (x == nullptr || gamma == nullptr || beta == nullptr || out == nullptr)
    return set_error(B200EMB_ERR_INVALID, "add_ln: null pointer");
  return launch_add_ln(x, y, gamma, beta, n_rows, hidden, eps, out, reinterpret_cast<cudaStream_t>(stream));
}

int b200emb_op_quantize_embeddings(const float* x, int32_t n_rows, int32_t dim, int64_t x_row_stride,
                                   int32_t precision, const double* d_ranges, void* out,
                                   int64_t out_row_stride_bytes, void* stream) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc = launch_quantize_embeddings(x, n_rows, dim, x_row_stride, precision, d_ranges, out, out_row_stride_bytes, s);
  if (rc) return rc;
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return set_error(B200EMB_ERR_CUDA, "quantize_embeddings: %s", cudaGetErrorString(e));
  return B200EMB_OK;
}

int b200emb_op_pool(const void* x, const int32_t* d_cu_seqlens, int32_t n_seqs, int32_t hidden, int32_t pooling,
                    int32_t normalize, void* out, int64_t out_row_stride, int32_t out_bf16, void* stream) {
  if (x == nullptr || d_cu_seqlens == nullptr || out == nullptr) return set_error(B200EMB_ERR_INVALID, "pool: null pointer");
  return launch_pool(x, d_cu_seqlens, n_seqs, hidden, pooling, normalize, out, out_row_stride, out_bf16,
                     reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
