// C++ host side of the attention path: the functions rllm/tch-cuda/src/lib.rs exposes to rLLM,
// with the same names, argument order and meaning, on top of the C ABI of aici_b200.h.
//
//   lib.rs                                   here
//   flash_attn_varlen      (:69-104)         aici::tch::flash_attn_varlen   (alias varlen_attn,
//                                            as rllm-cuda/src/llm/kernels.rs:4-7 re-exports it)
//   reshape_and_cache      (:192-213)        aici::tch::reshape_and_cache
//   gather_cached_kv       (:215-234)        aici::tch::gather_cached_kv
//   copy_blocks            (:276-331)        aici::tch::copy_blocks
//   swap_blocks            (:236-243, todo!)  aici::tch::swap_blocks
//   paged_attention_v1     (:356-391)        aici::tch::paged_attention_v1
//   paged_attention_v2_C   (:122-137)        aici::tch::paged_attention_v2  (the crate has no pub fn)
//
// The crate works on tch::Tensor; without libtorch the same information (data pointer, sizes,
// strides in elements, kind, device) travels in aici::tch::Tensor, which either views memory
// the caller owns or owns a cudaMalloc'd buffer.  Where the crate panics with "<fn>: <message>"
// (lib.rs:12-27) these functions throw aici::tch::Error carrying the same text.  Work is
// enqueued on the stream given last (default: the per-thread default stream, which is what
// the crate's kernels are compiled for, tch-cuda/build.rs:278).  There is no CPU path.
//
// Header-only; link with libaici_b200.so and the CUDA runtime.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "aici_b200.h"

namespace aici {
namespace tch {

class Error : public std::runtime_error {
 public:
  explicit Error(const std::string &what) : std::runtime_error(what) {}
};

// NULL = ok; otherwise the message is wrapped as "<fn>: <message>" and released with free().
inline void check(const char *fn, char *res) {
  if (res == nullptr) return;
  std::string msg = std::string(fn) + ": " + res;
  std::free(res);
  throw Error(msg);
}

inline void cuda_check(const char *fn, cudaError_t e) {
  if (e != cudaSuccess) throw Error(std::string(fn) + ": " + cudaGetErrorString(e));
}

enum class Kind { BFloat16, Half, Float, Int, Int64 };

inline size_t element_size(Kind k) {
  switch (k) {
    case Kind::BFloat16:
    case Kind::Half: return 2;
    case Kind::Float:
    case Kind::Int: return 4;
    default: return 8;
  }
}

// What the crate reads from a tch::Tensor.  device < 0 means host memory.
struct Tensor {
  void *data = nullptr;
  std::vector<int64_t> sizes, strides;  // strides in elements
  Kind kind = Kind::BFloat16;
  int device = 0;
  std::shared_ptr<void> owner;  // set when the buffer belongs to this tensor

  static std::vector<int64_t> contiguous_strides(const std::vector<int64_t> &sizes) {
    std::vector<int64_t> st(sizes.size(), 1);
    for (int i = (int)sizes.size() - 2; i >= 0; --i) st[i] = st[i + 1] * sizes[i + 1];
    return st;
  }
  // A view of memory the caller owns (contiguous unless strides are given).
  static Tensor view(void *data, std::vector<int64_t> sizes, Kind kind, int device,
                     std::vector<int64_t> strides = {}) {
    Tensor t;
    t.data = data;
    t.strides = strides.empty() ? contiguous_strides(sizes) : std::move(strides);
    t.sizes = std::move(sizes);
    t.kind = kind;
    t.device = device;
    return t;
  }
  // Tensor::empty on a CUDA device.
  static Tensor empty(std::vector<int64_t> sizes, Kind kind, int device) {
    int64_t n = 1;
    for (int64_t s : sizes) n *= s;
    int prev = 0;
    cuda_check("Tensor::empty", cudaGetDevice(&prev));
    cuda_check("Tensor::empty", cudaSetDevice(device));
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)(n > 0 ? n : 1) * element_size(kind));
    cudaSetDevice(prev);
    cuda_check("Tensor::empty", e);
    Tensor t = view(p, std::move(sizes), kind, device);
    t.owner = std::shared_ptr<void>(p, [](void *q) { cudaFree(q); });
    return t;
  }
  int64_t dim() const { return (int64_t)sizes.size(); }
  int64_t size(int i) const { return sizes[i]; }
  int64_t stride(int i) const { return strides[i]; }
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t s : sizes) n *= s;
    return n;
  }
  bool is_cuda() const { return device >= 0; }
  bool is_contiguous() const { return strides == contiguous_strides(sizes); }
};

namespace detail {

inline int dtype_of(const char *fn, const Tensor &t) {
  switch (t.kind) {
    case Kind::BFloat16: return AICI_DTYPE_BF16;
    case Kind::Half: return AICI_DTYPE_F16;
    case Kind::Float: return AICI_DTYPE_F32;
    default: throw Error(std::string(fn) + ": unsupported dtype");
  }
}

inline void require(const char *fn, bool cond, const char *msg) {
  if (!cond) throw Error(std::string(fn) + ": " + msg);
}

inline int require_cuda(const char *fn, std::initializer_list<const Tensor *> ts) {
  int dev = (*ts.begin())->device;
  for (const Tensor *t : ts) {
    require(fn, t->is_cuda(), "tensor must be on a CUDA device (there is no CPU path)");
    require(fn, t->device == dev, "tensors are on different devices");
  }
  return dev;
}

struct CacheDims {
  int64_t num_blocks;
  int num_kv_heads, head_size, block_size;
};

inline CacheDims cache_dims(const char *fn, const Tensor &kc, const Tensor &vc) {
  require(fn, kc.dim() == 5 && vc.dim() == 4, "key_cache must be 5-D and value_cache 4-D");
  require(fn, kc.is_contiguous() && vc.is_contiguous(), "caches must be contiguous");
  const int64_t head = kc.size(2) * kc.size(4);
  require(fn, vc.size(0) == kc.size(0) && vc.size(1) == kc.size(1) && vc.size(2) == head &&
                  vc.size(3) == kc.size(3),
          "value_cache shape does not match key_cache");
  require(fn, kc.size(4) * (int64_t)element_size(kc.kind) == 16,
          "last key_cache dimension must span 16 bytes");
  return {kc.size(0), (int)kc.size(1), (int)head, (int)kc.size(3)};
}

// Keeps the thread on `device` for the duration of a call.
struct DeviceGuard {
  int prev = 0;
  explicit DeviceGuard(int device) {
    cuda_check("cudaGetDevice", cudaGetDevice(&prev));
    if (prev != device) cuda_check("cudaSetDevice", cudaSetDevice(device));
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Scratch for the decode kernel, one buffer per (device, stream), grown on demand and kept.
inline void *decode_workspace(int device, cudaStream_t stream, size_t bytes, size_t *have_out) {
  struct Buf {
    void *p = nullptr;
    size_t n = 0;
  };
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, Buf> bufs;
  std::lock_guard<std::mutex> lock(mu);
  Buf &b = bufs[{device, stream}];
  if (b.n < bytes) {
    if (b.p) {
      cuda_check("decode_workspace", cudaStreamSynchronize(stream));
      cudaFree(b.p);
      b.p = nullptr;
      b.n = 0;
    }
    cuda_check("decode_workspace", cudaMalloc(&b.p, bytes));
    b.n = bytes;
  }
  *have_out = b.n;
  return b.p;
}

}  // namespace detail

// softmax(Q K^T * softmax_scale) V over packed variable-length sequences (lib.rs:49-104).
// q [total_q, num_heads_q, head_size], k/v [total_k, num_heads_kv, head_size], seqlens_* the
// cumulative lengths (int32, batch + 1 entries).  Returns a new tensor shaped like q.
inline Tensor flash_attn_varlen(const Tensor &q, const Tensor &k, const Tensor &v,
                                const Tensor &seqlens_q, const Tensor &seqlens_k,
                                size_t max_seqlen_q, size_t max_seqlen_k, float softmax_scale,
                                bool causal, cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "flash_attn_varlen";
  using detail::require;
  const int dev = detail::require_cuda(fn, {&q, &k, &v, &seqlens_q, &seqlens_k});
  require(fn, q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v must be 3-D");
  require(fn, k.kind == q.kind, "query and key must have the same dtype");
  require(fn, v.kind == q.kind, "query and value must have the same dtype");
  require(fn, seqlens_q.kind == Kind::Int, "cu_seqlens_q must have dtype int32");
  require(fn, seqlens_k.kind == Kind::Int, "cu_seqlens_k must have dtype int32");
  require(fn, q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1,
          "Input tensor must have contiguous last dimension");
  require(fn, seqlens_q.is_contiguous() && seqlens_k.is_contiguous(), "cu_seqlens must be contiguous");
  const int batch = (int)seqlens_q.numel() - 1;
  require(fn, seqlens_k.numel() == batch + 1, "cu_seqlens_q and cu_seqlens_k differ in length");
  require(fn, batch > 0, "batch size must be positive");
  require(fn, v.sizes == k.sizes && k.size(2) == q.size(2),
          "k and v must be [total_k, num_heads_k, head_size]");
  Tensor out = Tensor::empty(q.sizes, q.kind, dev);
  detail::DeviceGuard guard(dev);
  check(fn, aici_mha_varlen_fwd(out.data, q.data, k.data, v.data,
                                static_cast<const int32_t *>(seqlens_q.data),
                                static_cast<const int32_t *>(seqlens_k.data), batch, (int)q.size(0),
                                (int)k.size(0), (int)q.size(1), (int)k.size(1), (int)q.size(2),
                                (int)max_seqlen_q, (int)max_seqlen_k, q.stride(0), q.stride(1),
                                k.stride(0), k.stride(1), v.stride(0), v.stride(1), out.stride(0),
                                out.stride(1), softmax_scale, causal ? 1 : 0,
                                detail::dtype_of(fn, q), stream));
  return out;
}

// rllm-cuda re-exports flash_attn_varlen under this name (rllm-cuda/src/llm/kernels.rs:4-7).
inline Tensor varlen_attn(const Tensor &q, const Tensor &k, const Tensor &v, const Tensor &seqlens_q,
                          const Tensor &seqlens_k, size_t max_seqlen_q, size_t max_seqlen_k,
                          float softmax_scale, bool causal,
                          cudaStream_t stream = cudaStreamPerThread) {
  return flash_attn_varlen(q, k, v, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k,
                           softmax_scale, causal, stream);
}

namespace detail {
inline CacheDims check_kv_rows(const char *fn, const Tensor &key, const Tensor &value,
                               const Tensor &key_cache, const Tensor &value_cache,
                               const Tensor &slot_mapping) {
  const CacheDims c = cache_dims(fn, key_cache, value_cache);
  require(fn, key.dim() == 3 && key.sizes == value.sizes,
          "key and value must be [num_tokens, num_heads, head_size]");
  require(fn, key.size(1) == c.num_kv_heads && key.size(2) == c.head_size,
          "key shape does not match the cache");
  require(fn, key.stride(2) == 1 && key.stride(1) == c.head_size && value.stride(2) == 1 &&
                  value.stride(1) == c.head_size,
          "heads of one token must be contiguous");
  require(fn, slot_mapping.is_contiguous() && slot_mapping.numel() == key.size(0),
          "slot_mapping must be contiguous with one entry per token");
  return c;
}
}  // namespace detail

// key/value [num_tokens, num_heads, head_size] -> paged caches at slot_mapping (lib.rs:192-213).
// slot_mapping may be Int (as rLLM builds it) or Int64 (as the crate casts it).
inline void reshape_and_cache(const Tensor &key, const Tensor &value, Tensor &key_cache,
                              Tensor &value_cache, const Tensor &slot_mapping,
                              cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "reshape_and_cache";
  const int dev = detail::require_cuda(fn, {&key, &value, &key_cache, &value_cache, &slot_mapping});
  const detail::CacheDims c = detail::check_kv_rows(fn, key, value, key_cache, value_cache, slot_mapping);
  detail::require(fn, slot_mapping.kind == Kind::Int || slot_mapping.kind == Kind::Int64,
                  "slot_mapping must be int32 or int64");
  detail::require(fn, key_cache.kind == key.kind && value_cache.kind == key.kind,
                  "cache dtype differs from key dtype");
  detail::DeviceGuard guard(dev);
  check(fn, aici_reshape_and_cache(key.data, value.data, key_cache.data, value_cache.data,
                                   slot_mapping.data, slot_mapping.kind == Kind::Int64 ? 1 : 0,
                                   (int)key.size(0), c.num_kv_heads, c.head_size, c.block_size,
                                   c.num_blocks, key.stride(0), value.stride(0),
                                   detail::dtype_of(fn, key), stream));
}

// Inverse of reshape_and_cache: fills key/value from the caches (lib.rs:215-234).
inline void gather_cached_kv(Tensor &key, Tensor &value, const Tensor &key_cache,
                             const Tensor &value_cache, const Tensor &slot_mapping,
                             cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "gather_cached_kv";
  const int dev = detail::require_cuda(fn, {&key, &value, &key_cache, &value_cache, &slot_mapping});
  const detail::CacheDims c = detail::check_kv_rows(fn, key, value, key_cache, value_cache, slot_mapping);
  detail::require(fn, slot_mapping.kind == Kind::Int, "slot_mapping must be int32");
  detail::DeviceGuard guard(dev);
  check(fn, aici_gather_cached_kv(key.data, value.data, key_cache.data, value_cache.data,
                                  static_cast<const int32_t *>(slot_mapping.data), (int)key.size(0),
                                  c.num_kv_heads, c.head_size, c.block_size, c.num_blocks,
                                  key.stride(0), value.stride(0), detail::dtype_of(fn, key), stream));
}

// For every layer and every src -> dst of block_mapping copy one key block and one value block
// (lib.rs:276-331).  Layer addresses and pairs travel as kernel arguments: no upload, no sync.
inline void copy_blocks(std::vector<Tensor> &key_caches, std::vector<Tensor> &value_caches,
                        const std::unordered_map<size_t, std::vector<size_t>> &block_mapping,
                        cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "copy_blocks";
  using detail::require;
  require(fn, key_caches.size() == value_caches.size(), "key_caches and value_caches differ in length");
  if (key_caches.empty()) return;
  const int dev = key_caches[0].device;
  require(fn, dev >= 0, "caches must be on a CUDA device (there is no CPU path)");
  const int64_t tsize = key_caches[0].numel();
  std::vector<int64_t> kp, vp, pairs;
  for (size_t l = 0; l < key_caches.size(); ++l) {
    for (const Tensor *t : {&key_caches[l], &value_caches[l]}) {
      require(fn, t->device == dev && t->numel() == tsize, "all caches must share device and size");
      require(fn, (t->kind == Kind::BFloat16 || t->kind == Kind::Half) && t->is_contiguous(),
              "caches must be contiguous bf16 or f16");
    }
    kp.push_back((int64_t)(uintptr_t)key_caches[l].data);
    vp.push_back((int64_t)(uintptr_t)value_caches[l].data);
  }
  for (const auto &kv : block_mapping)
    for (size_t dst : kv.second) {
      pairs.push_back((int64_t)kv.first);
      pairs.push_back((int64_t)dst);
    }
  if (pairs.empty()) return;
  const Tensor &v0 = value_caches[0];
  require(fn, v0.dim() == 4, "value caches must be [num_blocks, num_heads, head_size, block_size]");
  detail::DeviceGuard guard(dev);
  check(fn, aici_copy_blocks_host(kp.data(), vp.data(), pairs.data(), (int)kp.size(),
                                  (int)(pairs.size() / 2), v0.size(1) * v0.size(2) * v0.size(3),
                                  v0.size(0), detail::dtype_of(fn, key_caches[0]), stream));
}

// dst[d] = src[s] for every s -> d (the crate's swap_blocks is todo!(), lib.rs:236-243; C side
// kernels/vllm/cache_kernels.cu:12-50).  One of the two may be host memory (device < 0).
inline void swap_blocks(const Tensor &src, Tensor &dst,
                        const std::unordered_map<size_t, size_t> &block_mapping,
                        cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "swap_blocks";
  using detail::require;
  require(fn, src.dim() >= 1 && dst.dim() >= 1 && src.kind == dst.kind &&
                  std::vector<int64_t>(src.sizes.begin() + 1, src.sizes.end()) ==
                      std::vector<int64_t>(dst.sizes.begin() + 1, dst.sizes.end()),
          "src and dst must have the same block shape and dtype");
  require(fn, src.is_contiguous() && dst.is_contiguous(), "caches must be contiguous");
  require(fn, src.is_cuda() || dst.is_cuda(), "Invalid device combination");
  require(fn, !(src.is_cuda() && dst.is_cuda()) || src.device == dst.device,
          "src and dst must be on the same GPU");
  std::vector<int64_t> pairs;
  for (const auto &kv : block_mapping) {
    pairs.push_back((int64_t)kv.first);
    pairs.push_back((int64_t)kv.second);
  }
  if (pairs.empty()) return;
  const int64_t block_bytes = src.numel() / src.size(0) * (int64_t)element_size(src.kind);
  detail::DeviceGuard guard(src.is_cuda() ? src.device : dst.device);
  check(fn, aici_swap_blocks(src.data, dst.data, pairs.data(), (int)(pairs.size() / 2), block_bytes,
                             src.size(0), dst.size(0), stream));
}

namespace detail {
struct DecodeDims {
  CacheDims c;
  int num_seqs, num_heads, max_blocks;
};
inline DecodeDims decode_dims(const char *fn, const Tensor &out, const Tensor &query,
                              const Tensor &key_cache, const Tensor &value_cache, int num_kv_heads,
                              const Tensor &block_tables, const Tensor &context_lens,
                              int block_size) {
  const CacheDims c = cache_dims(fn, key_cache, value_cache);
  require(fn, query.dim() == 3 && out.sizes == query.sizes, "out and query must be [num_seqs, num_heads, head_size]");
  require(fn, out.is_contiguous(), "out must be contiguous");
  require(fn, query.stride(2) == 1 && query.stride(1) == query.size(2), "heads of one query row must be contiguous");
  require(fn, query.size(2) == c.head_size, "head_size of query and cache differ");
  require(fn, num_kv_heads == c.num_kv_heads, "num_kv_heads does not match the cache");
  require(fn, block_size == c.block_size, "block_size does not match the cache");
  require(fn, block_tables.kind == Kind::Int && block_tables.dim() == 2 && block_tables.is_contiguous() &&
                  block_tables.size(0) == query.size(0),
          "block_tables must be contiguous int32 [num_seqs, max_num_blocks_per_seq]");
  require(fn, context_lens.kind == Kind::Int && context_lens.is_contiguous() &&
                  context_lens.numel() == query.size(0),
          "context_lens must be contiguous int32 [num_seqs]");
  require(fn, query.kind == key_cache.kind && out.kind == query.kind, "dtypes differ");
  return {c, (int)query.size(0), (int)query.size(1), (int)block_tables.size(1)};
}
}  // namespace detail

// Decode attention over the paged cache, one query token per sequence (lib.rs:356-391).
inline void paged_attention_v1(Tensor &out, const Tensor &query, const Tensor &key_cache,
                               const Tensor &value_cache, int num_kv_heads, float scale,
                               const Tensor &block_tables, const Tensor &context_lens, int block_size,
                               int max_context_len, const Tensor *alibi_slopes = nullptr,
                               cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "paged_attention_v1";
  const int dev = detail::require_cuda(fn, {&out, &query, &key_cache, &value_cache, &block_tables, &context_lens});
  const detail::DecodeDims d = detail::decode_dims(fn, out, query, key_cache, value_cache, num_kv_heads,
                                                   block_tables, context_lens, block_size);
  detail::DeviceGuard guard(dev);
  const size_t need = aici_paged_attention_workspace_bytes(d.num_seqs, d.num_heads, num_kv_heads, max_context_len);
  size_t have = 0;
  void *ws = detail::decode_workspace(dev, stream, need, &have);
  check(fn, aici_paged_attention_v1(out.data, query.data, key_cache.data, value_cache.data, num_kv_heads,
                                    scale, static_cast<const int32_t *>(block_tables.data),
                                    static_cast<const int32_t *>(context_lens.data), block_size,
                                    max_context_len,
                                    alibi_slopes ? static_cast<const float *>(alibi_slopes->data) : nullptr,
                                    d.num_seqs, d.num_heads, d.c.head_size, d.max_blocks, d.c.num_blocks,
                                    query.stride(0), key_cache.stride(0), key_cache.stride(1), ws, have,
                                    detail::dtype_of(fn, query), stream));
}

// One decode step of one layer: reshape_and_cache of the step's new tokens (token i = newest token
// of sequence i, slot_mapping[i] = the cache slot of position context_lens[i] - 1) and
// paged_attention_v1, the pair of crate calls rLLM makes per layer (llm/mod.rs:132-166, 280-316), as
// one library call (aici_decode_step): the decode kernel writes the tokens to the cache itself.
inline void decode_step(Tensor &out, const Tensor &new_key, const Tensor &new_value, const Tensor &slot_mapping,
                        const Tensor &query, Tensor &key_cache, Tensor &value_cache, int num_kv_heads,
                        float scale, const Tensor &block_tables, const Tensor &context_lens, int block_size,
                        int max_context_len, cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "decode_step";
  const int dev = detail::require_cuda(fn, {&out, &new_key, &new_value, &slot_mapping, &query, &key_cache,
                                            &value_cache, &block_tables, &context_lens});
  const detail::DecodeDims d = detail::decode_dims(fn, out, query, key_cache, value_cache, num_kv_heads,
                                                   block_tables, context_lens, block_size);
  detail::require(fn, new_key.dim() == 3 && new_key.sizes == new_value.sizes && new_key.size(0) == d.num_seqs &&
                          new_key.size(1) == num_kv_heads && new_key.size(2) == d.c.head_size,
                  "new key/value must be [num_seqs, num_kv_heads, head_size]");
  detail::require(fn, new_key.stride(2) == 1 && new_key.stride(1) == new_key.size(2) && new_value.stride(2) == 1 &&
                          new_value.stride(1) == new_value.size(2),
                  "heads of one token must be contiguous");
  detail::require(fn, (slot_mapping.kind == Kind::Int || slot_mapping.kind == Kind::Int64) &&
                          slot_mapping.is_contiguous() && slot_mapping.numel() == d.num_seqs,
                  "slot_mapping must be contiguous int32 or int64 with one entry per sequence");
  detail::DeviceGuard guard(dev);
  const size_t need = aici_paged_attention_workspace_bytes(d.num_seqs, d.num_heads, num_kv_heads, max_context_len);
  size_t have = 0;
  void *ws = detail::decode_workspace(dev, stream, need, &have);
  void *outs[1] = {out.data};
  check(fn, aici_decode_step(outs, nullptr, 1, 0, d.num_heads, 0, new_key.data, new_value.data, slot_mapping.data,
                             slot_mapping.kind == Kind::Int64 ? 1 : 0, new_key.stride(0), new_value.stride(0),
                             query.data, key_cache.data, value_cache.data, num_kv_heads, scale,
                             static_cast<const int32_t *>(block_tables.data),
                             static_cast<const int32_t *>(context_lens.data), block_size, max_context_len,
                             d.num_seqs, d.num_heads, d.c.head_size, d.max_blocks, d.c.num_blocks, query.stride(0),
                             key_cache.stride(0), key_cache.stride(1), ws, have, detail::dtype_of(fn, query), stream));
}

// The extern's argument list (lib.rs:122-137): exp_sums / max_logits f32 [num_seqs, num_heads, P],
// tmp_out [num_seqs, num_heads, P, head_size] in the query's dtype, P = ceil(max_context_len / 512).
inline void paged_attention_v2(Tensor &out, Tensor &exp_sums, Tensor &max_logits, Tensor &tmp_out,
                               const Tensor &query, const Tensor &key_cache, const Tensor &value_cache,
                               int num_kv_heads, float scale, const Tensor &block_tables,
                               const Tensor &context_lens, int block_size, int max_context_len,
                               const Tensor *alibi_slopes = nullptr,
                               cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "paged_attention_v2";
  using detail::require;
  const int dev = detail::require_cuda(fn, {&out, &exp_sums, &max_logits, &tmp_out, &query, &key_cache,
                                            &value_cache, &block_tables, &context_lens});
  const detail::DecodeDims d = detail::decode_dims(fn, out, query, key_cache, value_cache, num_kv_heads,
                                                   block_tables, context_lens, block_size);
  const int64_t parts = max_context_len > 0 ? (max_context_len + 511) / 512 : 1;
  const std::vector<int64_t> want = {d.num_seqs, d.num_heads, parts};
  require(fn, exp_sums.kind == Kind::Float && max_logits.kind == Kind::Float && exp_sums.sizes == want &&
                  max_logits.sizes == want && exp_sums.is_contiguous() && max_logits.is_contiguous(),
          "exp_sums and max_logits must be contiguous f32 [num_seqs, num_heads, partitions]");
  require(fn, tmp_out.kind == query.kind && tmp_out.is_contiguous() && tmp_out.dim() == 4 &&
                  tmp_out.size(0) == d.num_seqs && tmp_out.size(1) == d.num_heads &&
                  tmp_out.size(2) == parts && tmp_out.size(3) == d.c.head_size,
          "tmp_out must be contiguous [num_seqs, num_heads, partitions, head_size]");
  detail::DeviceGuard guard(dev);
  check(fn, aici_paged_attention_v2(out.data, static_cast<float *>(exp_sums.data),
                                    static_cast<float *>(max_logits.data), tmp_out.data, query.data,
                                    key_cache.data, value_cache.data, num_kv_heads, scale,
                                    static_cast<const int32_t *>(block_tables.data),
                                    static_cast<const int32_t *>(context_lens.data), block_size,
                                    max_context_len,
                                    alibi_slopes ? static_cast<const float *>(alibi_slopes->data) : nullptr,
                                    d.num_seqs, d.num_heads, d.c.head_size, d.max_blocks, d.c.num_blocks,
                                    query.stride(0), key_cache.stride(0), key_cache.stride(1),
                                    detail::dtype_of(fn, query), stream));
}

// Additions that have no function of their own in the crate --------------------------------------

// Prefill attention with keys/values read from the paged cache through block tables: what
// compute_varlen_attn (rllm-cuda/src/llm/mod.rs:168-278) gets from gather_cached_kv + repeat_kv +
// flash_attn_varlen, without the gathered copy.  seqlens_q cumulative int32 [batch + 1];
// context_lens int32 [batch]; block_tables int32 [batch, max_blocks].
inline Tensor flash_attn_varlen_paged(const Tensor &q, const Tensor &key_cache, const Tensor &value_cache,
                                      const Tensor &seqlens_q, const Tensor &context_lens,
                                      const Tensor &block_tables, size_t max_seqlen_q,
                                      size_t max_context_len, float softmax_scale, bool causal,
                                      cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "flash_attn_varlen_paged";
  using detail::require;
  const int dev = detail::require_cuda(fn, {&q, &key_cache, &value_cache, &seqlens_q, &context_lens, &block_tables});
  const detail::CacheDims c = detail::cache_dims(fn, key_cache, value_cache);
  require(fn, q.dim() == 3 && q.size(2) == c.head_size && q.stride(2) == 1,
          "q must be [total_q, num_heads, head_size] with contiguous last dimension");
  require(fn, seqlens_q.kind == Kind::Int && context_lens.kind == Kind::Int && block_tables.kind == Kind::Int &&
                  seqlens_q.is_contiguous() && context_lens.is_contiguous() && block_tables.is_contiguous(),
          "seqlens_q, context_lens and block_tables must be contiguous int32");
  const int batch = (int)seqlens_q.numel() - 1;
  require(fn, batch > 0 && context_lens.numel() == batch && block_tables.dim() == 2 && block_tables.size(0) == batch,
          "context_lens must be [batch] and block_tables [batch, max_blocks]");
  Tensor out = Tensor::empty(q.sizes, q.kind, dev);
  detail::DeviceGuard guard(dev);
  check(fn, aici_mha_varlen_paged_fwd(out.data, q.data, key_cache.data, value_cache.data,
                                      static_cast<const int32_t *>(seqlens_q.data),
                                      static_cast<const int32_t *>(context_lens.data),
                                      static_cast<const int32_t *>(block_tables.data), batch, (int)q.size(0),
                                      (int)q.size(1), c.num_kv_heads, c.head_size, c.block_size,
                                      (int)max_seqlen_q, (int)max_context_len, (int)block_tables.size(1),
                                      c.num_blocks, q.stride(0), q.stride(1), out.stride(0), out.stride(1),
                                      key_cache.stride(0), key_cache.stride(1), softmax_scale, causal ? 1 : 0,
                                      detail::dtype_of(fn, q), stream));
  return out;
}

// rotary_embedding (lib.rs:139-146) and reshape_and_cache in one pass, as rLLM issues them back to
// back (rllm-cuda/src/llm/mod.rs:107-114, 158-164): query and key are rotated in place (NeoX,
// rot_dim = head_size), the rotated key and value go to the cache at slot_mapping.
inline void rotary_embedding_reshape_and_cache(const Tensor &positions, Tensor &query, Tensor &key,
                                               const Tensor &value, const Tensor &cos_sin_cache,
                                               Tensor &key_cache, Tensor &value_cache,
                                               const Tensor &slot_mapping, bool is_neox = true,
                                               cudaStream_t stream = cudaStreamPerThread) {
  const char *fn = "rotary_embedding_reshape_and_cache";
  using detail::require;
  const int dev = detail::require_cuda(fn, {&positions, &query, &key, &value, &cos_sin_cache, &key_cache,
                                            &value_cache, &slot_mapping});
  const detail::CacheDims c = detail::check_kv_rows(fn, key, value, key_cache, value_cache, slot_mapping);
  require(fn, positions.kind == Kind::Int64 && positions.is_contiguous() && positions.numel() == key.size(0),
          "positions must be contiguous int64 with one entry per token");
  require(fn, query.dim() == 3 && query.size(0) == key.size(0) && query.size(2) == c.head_size &&
                  query.stride(2) == 1 && query.stride(1) == c.head_size,
          "query must be [num_tokens, num_heads, head_size] with contiguous heads");
  require(fn, cos_sin_cache.dim() == 2 && cos_sin_cache.is_contiguous() && cos_sin_cache.kind == key.kind,
          "cos_sin_cache must be contiguous [max_position, rot_dim] in the key's dtype");
  require(fn, slot_mapping.kind == Kind::Int || slot_mapping.kind == Kind::Int64, "slot_mapping must be int32 or int64");
  detail::DeviceGuard guard(dev);
  check(fn, aici_rotary_reshape_and_cache(static_cast<const int64_t *>(positions.data), query.data, key.data,
                                          value.data, cos_sin_cache.data, key_cache.data, value_cache.data,
                                          slot_mapping.data, slot_mapping.kind == Kind::Int64 ? 1 : 0,
                                          (int)key.size(0), (int)query.size(1), c.num_kv_heads, c.head_size,
                                          (int)cos_sin_cache.size(1), is_neox ? 1 : 0, cos_sin_cache.size(0),
                                          c.block_size, c.num_blocks, query.stride(0), key.stride(0),
                                          value.stride(0), detail::dtype_of(fn, key), stream));
}

// Reads and clears the device's sticky status word (no counterpart in the crate; the reference
// kernels trap or read out of bounds where these record a bit and carry on).
inline int last_status() {
  int st = 0;
  check("last_status", aici_last_status(&st));
  return st;
}

}  // namespace tch
}  // namespace aici
