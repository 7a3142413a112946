// GPU comparator shim -- TEST INFRASTRUCTURE ONLY, never linked into the product library.
//
// Wraps the reference's own unmodified CUDA kernels (compiled from where they lie in the
// reference tree: rllm/tch-cuda/kernels/vllm/cache_kernels.cu and
// rllm/tch-cuda/kernels/vllm/attention/attention_kernels.cu) behind plain-pointer entry points,
// so that the GPU tests can compare this repository's kernels with the reference's outputs on
// the same device buffers.  The functions called here are the ones the reference's own
// vllm_bindings.cpp calls (declared in vllm/cache.h and vllm/ops.h).
#include <torch/all.h>

#include <cstring>
#include <map>
#include <string>

#include "vllm/cache.h"
#include "vllm/ops.h"

namespace {
using BlockMap = std::map<int64_t, int64_t>;  // named here: a comma inside REF_PROTECT would split its argument
torch::Tensor wrap(void *p, std::vector<int64_t> sizes, torch::ScalarType t, int dev) {
  return torch::from_blob(p, sizes, torch::TensorOptions().dtype(t).device(torch::kCUDA, dev));
}
}  // namespace

#define REF_PROTECT(body)                                                                       \
  try {                                                                                         \
    body;                                                                                       \
    return nullptr;                                                                             \
  } catch (const std::exception &e) {                                                           \
    return strdup(e.what());                                                                    \
  }

extern "C" {

char *ref_reshape_and_cache(void *key, void *value, void *kc, void *vc, void *slots_i64, int64_t T,
                            int64_t hkv, int64_t d, int64_t nblk, int64_t bs, int dev) {
  REF_PROTECT({
    auto k = wrap(key, {T, hkv, d}, torch::kBFloat16, dev);
    auto v = wrap(value, {T, hkv, d}, torch::kBFloat16, dev);
    auto kcache = wrap(kc, {nblk, hkv, d / 8, bs, 8}, torch::kBFloat16, dev);
    auto vcache = wrap(vc, {nblk, hkv, d, bs}, torch::kBFloat16, dev);
    auto s = wrap(slots_i64, {T}, torch::kInt64, dev);
    reshape_and_cache(k, v, kcache, vcache, s);
  })
}

char *ref_gather_cached_kv(void *key, void *value, void *kc, void *vc, void *slots_i32, int64_t T,
                           int64_t hkv, int64_t d, int64_t nblk, int64_t bs, int dev) {
  REF_PROTECT({
    auto k = wrap(key, {T, hkv, d}, torch::kBFloat16, dev);
    auto v = wrap(value, {T, hkv, d}, torch::kBFloat16, dev);
    auto kcache = wrap(kc, {nblk, hkv, d / 8, bs, 8}, torch::kBFloat16, dev);
    auto vcache = wrap(vc, {nblk, hkv, d, bs}, torch::kBFloat16, dev);
    auto s = wrap(slots_i32, {T}, torch::kInt32, dev);
    gather_cached_kv(k, v, kcache, vcache, s);
  })
}

char *ref_copy_blocks_2(void *kptrs, void *vptrs, void *mapping, int64_t layers, int64_t pairs,
                        void *key0, int64_t nblk, int64_t hkv, int64_t d, int64_t bs, int dev) {
  REF_PROTECT({
    auto kp = wrap(kptrs, {layers}, torch::kInt64, dev);
    auto vp = wrap(vptrs, {layers}, torch::kInt64, dev);
    auto m = wrap(mapping, {2 * pairs}, torch::kInt64, dev);
    auto k0 = wrap(key0, {nblk, hkv, d / 8, bs, 8}, torch::kBFloat16, dev);
    copy_blocks_2(kp, vp, m, k0);
  })
}

// swap_blocks of the reference (vllm/cache_kernels.cu:12-50).  src_dev / dst_dev: device index of
// the tensor, or -1 for host memory (page-locked or not: the reference treats both as "cpu").
// pairs: 2 * num_pairs int64 on the host, (src, dst, ...); sources are unique, as in the
// reference's std::map.
char *ref_swap_blocks(void *src, int src_dev, void *dst, int dst_dev, const int64_t *pairs, int64_t num_pairs,
                      int64_t src_blocks, int64_t dst_blocks, int64_t elems_per_block) {
  REF_PROTECT({
    auto opts = [](int dev) {
      auto o = torch::TensorOptions().dtype(torch::kBFloat16);
      return dev >= 0 ? o.device(torch::kCUDA, dev) : o.device(torch::kCPU);
    };
    auto s = torch::from_blob(src, {src_blocks, elems_per_block}, opts(src_dev));
    auto d = torch::from_blob(dst, {dst_blocks, elems_per_block}, opts(dst_dev));
    BlockMap m;
    for (int64_t i = 0; i < num_pairs; ++i) m[pairs[2 * i]] = pairs[2 * i + 1];
    swap_blocks(s, d, m);
  })
}

char *ref_rotary_embedding(void *positions_i64, void *query, void *key, int64_t T, int64_t hq, int64_t hkv,
                           int64_t d, void *cos_sin, int64_t max_pos, int64_t rot_dim, int is_neox, int dev) {
  REF_PROTECT({
    auto pos = wrap(positions_i64, {T}, torch::kInt64, dev);
    auto q = wrap(query, {T, hq * d}, torch::kBFloat16, dev);
    auto k = wrap(key, {T, hkv * d}, torch::kBFloat16, dev);
    auto cs = wrap(cos_sin, {max_pos, rot_dim}, torch::kBFloat16, dev);
    rotary_embedding(pos, q, k, (int)d, cs, is_neox != 0);
  })
}

char *ref_paged_attention_v1(void *out, void *query, void *kc, void *vc, int num_kv_heads, float scale,
                             void *block_tables, void *context_lens, int block_size,
                             int max_context_len, int64_t S, int64_t hq, int64_t d, int64_t max_blocks,
                             int64_t nblk, int dev) {
  REF_PROTECT({
    auto o = wrap(out, {S, hq, d}, torch::kBFloat16, dev);
    auto q = wrap(query, {S, hq, d}, torch::kBFloat16, dev);
    auto kcache = wrap(kc, {nblk, (int64_t)num_kv_heads, d / 8, (int64_t)block_size, 8}, torch::kBFloat16, dev);
    auto vcache = wrap(vc, {nblk, (int64_t)num_kv_heads, d, (int64_t)block_size}, torch::kBFloat16, dev);
    auto bt = wrap(block_tables, {S, max_blocks}, torch::kInt32, dev);
    auto cl = wrap(context_lens, {S}, torch::kInt32, dev);
    paged_attention_v1(o, q, kcache, vcache, num_kv_heads, scale, bt, cl, block_size, max_context_len,
                       c10::nullopt);
  })
}

char *ref_paged_attention_v2(void *out, void *exp_sums, void *max_logits, void *tmp_out, void *query,
                             void *kc, void *vc, int num_kv_heads, float scale, void *block_tables,
                             void *context_lens, int block_size, int max_context_len, int64_t S,
                             int64_t hq, int64_t d, int64_t max_blocks, int64_t nblk, int dev) {
  REF_PROTECT({
    const int64_t parts = (max_context_len + 511) / 512;
    auto o = wrap(out, {S, hq, d}, torch::kBFloat16, dev);
    auto es = wrap(exp_sums, {S, hq, parts}, torch::kFloat32, dev);
    auto ml = wrap(max_logits, {S, hq, parts}, torch::kFloat32, dev);
    auto to = wrap(tmp_out, {S, hq, parts, d}, torch::kBFloat16, dev);
    auto q = wrap(query, {S, hq, d}, torch::kBFloat16, dev);
    auto kcache = wrap(kc, {nblk, (int64_t)num_kv_heads, d / 8, (int64_t)block_size, 8}, torch::kBFloat16, dev);
    auto vcache = wrap(vc, {nblk, (int64_t)num_kv_heads, d, (int64_t)block_size}, torch::kBFloat16, dev);
    auto bt = wrap(block_tables, {S, max_blocks}, torch::kInt32, dev);
    auto cl = wrap(context_lens, {S}, torch::kInt32, dev);
    paged_attention_v2(o, es, ml, to, q, kcache, vcache, num_kv_heads, scale, bt, cl, block_size,
                       max_context_len, c10::nullopt);
  })
}
}
