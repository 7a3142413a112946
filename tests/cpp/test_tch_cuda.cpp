// Parity tests of the C++ host side (include/aici_b200_tch.hpp) in the manner of the reference's
// own crate tests (rllm/tch-cuda/tests/flash_attn_tests.rs): build inputs in closed form or from a
// seeded generator, call the public function, compare with expected values -- here the CPU oracle
// (oracle/oracle.c, linked as a checker only).  Cache movers must match bit for bit; attention in
// bf16 must stay within max-abs 2e-2 / mean-abs 2e-3 of the fp32-softmax oracle.
//
//   test_tch_cuda            run every test on GPU 0, exit code = number of failures
//   test_tch_cuda --list     print the test names (touches no GPU)
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "aici_b200_tch.hpp"

extern "C" {
void oracle_reshape_and_cache(const uint16_t *key, const uint16_t *value, uint16_t *key_cache,
                              uint16_t *value_cache, const int64_t *slot_mapping, int num_tokens,
                              int64_t key_stride, int64_t value_stride, int num_heads, int head_size,
                              int block_size, int x);
void oracle_copy_blocks(uint16_t *const *key_caches, uint16_t *const *value_caches,
                        const int64_t *block_mapping, int num_layers, int num_pairs,
                        int64_t numel_per_block);
void oracle_paged_attention_v1(float *out_f32, const uint16_t *q, const uint16_t *k_cache,
                               const uint16_t *v_cache, int num_kv_heads, float scale,
                               const int32_t *block_tables, const int32_t *context_lens, int num_seqs,
                               int num_heads, int head_size, int block_size, int x,
                               int max_num_blocks_per_seq, int64_t q_stride, int64_t kv_block_stride,
                               int64_t kv_head_stride, int ref_rounding);
void oracle_varlen_attn(float *out_f32, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                        const int32_t *cu_q, const int32_t *cu_k, int batch, int num_heads,
                        int num_heads_k, int head_size, int64_t q_tok_stride, int64_t q_head_stride,
                        int64_t k_tok_stride, int64_t k_head_stride, int64_t v_tok_stride,
                        int64_t v_head_stride, float scale, int causal, int p_bf16);
void oracle_rotary_embedding_neox(const int64_t *positions, uint16_t *query, uint16_t *key,
                                  const uint16_t *cos_sin_cache, int num_tokens, int num_heads,
                                  int num_kv_heads, int head_size, int rot_dim, int64_t query_stride,
                                  int64_t key_stride);
}

namespace t = aici::tch;
using t::Kind;
using t::Tensor;

// ---- host-side helpers ---------------------------------------------------------------------------
static uint16_t to_bf16(float f) {  // round to nearest even
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float from_bf16(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

struct Rng {  // 64-bit LCG; normal() = sum of 12 uniforms - 6
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 2862933555777941757ull + 3037000493ull) {}
  uint32_t next() {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    return (uint32_t)(s >> 33);
  }
  float uniform() { return (next() & 0xffffff) / 16777216.f; }
  float normal() {
    float a = 0.f;
    for (int i = 0; i < 12; ++i) a += uniform();
    return a - 6.f;
  }
  int below(int n) { return (int)(next() % (uint32_t)n); }
};

static std::vector<uint16_t> randn_bf16(Rng &r, size_t n) {
  std::vector<uint16_t> v(n);
  for (auto &x : v) x = to_bf16(r.normal());
  return v;
}

template <typename T>
static Tensor to_device(const std::vector<T> &h, std::vector<int64_t> sizes, Kind kind) {
  Tensor d = Tensor::empty(std::move(sizes), kind, 0);
  t::cuda_check("to_device", cudaMemcpy(d.data, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}
template <typename T>
static std::vector<T> to_host(const Tensor &d) {
  std::vector<T> h((size_t)d.numel());
  t::cuda_check("to_host", cudaDeviceSynchronize());
  t::cuda_check("to_host", cudaMemcpy(h.data(), d.data, h.size() * sizeof(T), cudaMemcpyDeviceToHost));
  return h;
}

struct Failure {
  std::string msg;
};
#define EXPECT(cond, ...)                          \
  do {                                             \
    if (!(cond)) {                                 \
      char b__[400];                               \
      std::snprintf(b__, sizeof(b__), __VA_ARGS__); \
      throw Failure{b__};                          \
    }                                              \
  } while (0)

static void expect_close(const std::vector<uint16_t> &got, const std::vector<float> &want, float max_abs,
                         float mean_abs) {
  EXPECT(got.size() == want.size(), "size %zu vs %zu", got.size(), want.size());
  double sum = 0, mx = 0;
  for (size_t i = 0; i < got.size(); ++i) {
    const float g = from_bf16(got[i]);
    EXPECT(std::isfinite(g), "element %zu is not finite", i);
    const double d = std::fabs((double)g - want[i]);
    sum += d;
    if (d > mx) mx = d;
  }
  const double mean = got.empty() ? 0 : sum / got.size();
  EXPECT(mx <= max_abs && mean <= mean_abs, "max-abs %.3g (<= %.3g) mean-abs %.3g (<= %.3g)", mx, max_abs,
         mean, mean_abs);
}

// A paged cache with sequences laid out as rLLM's allocator does (paged/blocks.rs:122-127).
struct Paged {
  int nblk, hkv;
  std::vector<uint16_t> kc, vc;            // [nblk, hkv, 16, 16, 8], [nblk, hkv, 128, 16]
  std::vector<int32_t> tables, ctx;        // [seqs, max_blocks], [seqs]
  int max_blocks = 0, max_ctx = 0;
  std::vector<std::vector<int>> rows;
  Paged(Rng &r, int nblk_, int hkv_, const std::vector<int> &lens) : nblk(nblk_), hkv(hkv_) {
    kc = randn_bf16(r, (size_t)nblk * hkv * 2048);
    vc = randn_bf16(r, (size_t)nblk * hkv * 2048);
    std::vector<int> perm(nblk);
    for (int i = 0; i < nblk; ++i) perm[i] = i;
    for (int i = nblk - 1; i > 0; --i) std::swap(perm[i], perm[r.below(i + 1)]);
    int next = 0;
    for (int c : lens) {
      std::vector<int> row;
      for (int b = 0; b < (c + 15) / 16; ++b) row.push_back(perm[next++]);
      max_blocks = std::max(max_blocks, (int)row.size());
      max_ctx = std::max(max_ctx, c);
      rows.push_back(row);
      ctx.push_back(c);
    }
    if (max_blocks == 0) max_blocks = 1;
    tables.assign(rows.size() * max_blocks, 0);
    for (size_t s = 0; s < rows.size(); ++s)
      for (size_t b = 0; b < rows[s].size(); ++b) tables[s * max_blocks + b] = rows[s][b];
  }
  Tensor key_cache() const { return to_device(kc, {nblk, hkv, 16, 16, 8}, Kind::BFloat16); }
  Tensor value_cache() const { return to_device(vc, {nblk, hkv, 128, 16}, Kind::BFloat16); }
};

// ---- tests -----------------------------------------------------------------------------------------
static void reshape_and_cache_then_gather_round_trip() {
  Rng r(11);
  const int T = 37, hkv = 3, nblk = 9;
  Paged p(r, nblk, hkv, {});
  auto key = randn_bf16(r, (size_t)T * hkv * 128), val = randn_bf16(r, (size_t)T * hkv * 128);
  std::vector<int32_t> slots(T);
  std::vector<int> all(nblk * 16);
  for (int i = 0; i < nblk * 16; ++i) all[i] = i;
  for (int i = nblk * 16 - 1; i > 0; --i) std::swap(all[i], all[r.below(i + 1)]);
  for (int i = 0; i < T; ++i) slots[i] = all[i];
  slots[5] = -1;  // padding token: skipped (cache_kernels.cu:183-186)
  Tensor kc = p.key_cache(), vc = p.value_cache();
  Tensor dk = to_device(key, {T, hkv, 128}, Kind::BFloat16), dv = to_device(val, {T, hkv, 128}, Kind::BFloat16);
  Tensor ds = to_device(slots, {T}, Kind::Int);
  t::reshape_and_cache(dk, dv, kc, vc, ds);
  std::vector<int64_t> s64(slots.begin(), slots.end());
  oracle_reshape_and_cache(key.data(), val.data(), p.kc.data(), p.vc.data(), s64.data(), T, hkv * 128,
                           hkv * 128, hkv, 128, 16, 8);
  EXPECT(to_host<uint16_t>(kc) == p.kc, "key cache differs from the oracle");
  EXPECT(to_host<uint16_t>(vc) == p.vc, "value cache differs from the oracle");
  // gather what was scattered (all but the padding token)
  slots[5] = slots[4];
  Tensor ds2 = to_device(slots, {T}, Kind::Int);
  Tensor gk = Tensor::empty({T, hkv, 128}, Kind::BFloat16, 0), gv = Tensor::empty({T, hkv, 128}, Kind::BFloat16, 0);
  t::gather_cached_kv(gk, gv, kc, vc, ds2);
  auto hk = to_host<uint16_t>(gk), hv = to_host<uint16_t>(gv);
  for (int i = 0; i < T; ++i) {
    const int src = i == 5 ? 4 : i;
    EXPECT(std::memcmp(&hk[(size_t)i * hkv * 128], &key[(size_t)src * hkv * 128], hkv * 256) == 0, "key row %d", i);
    EXPECT(std::memcmp(&hv[(size_t)i * hkv * 128], &val[(size_t)src * hkv * 128], hkv * 256) == 0, "value row %d", i);
  }
  EXPECT(t::last_status() == 0, "status word set");
}

static void paged_attention_matches_oracle(bool v2) {
  Rng r(v2 ? 23 : 21);
  const int hq = 8, hkv = 2;
  const std::vector<int> lens = {1, 15, 16, 17, 300, 513, 0, 1100, 47};
  Paged p(r, 160, hkv, lens);
  const int S = (int)lens.size();
  auto q = randn_bf16(r, (size_t)S * hq * 128);
  std::vector<float> want((size_t)S * hq * 128);
  const float scale = 0.0884f;
  oracle_paged_attention_v1(want.data(), q.data(), p.kc.data(), p.vc.data(), hkv, scale, p.tables.data(),
                            p.ctx.data(), S, hq, 128, 16, 8, p.max_blocks, hq * 128, (int64_t)hkv * 2048, 2048, 0);
  Tensor kc = p.key_cache(), vc = p.value_cache();
  Tensor dq = to_device(q, {S, hq, 128}, Kind::BFloat16);
  Tensor bt = to_device(p.tables, {S, p.max_blocks}, Kind::Int), cl = to_device(p.ctx, {S}, Kind::Int);
  Tensor out = Tensor::empty({S, hq, 128}, Kind::BFloat16, 0);
  if (v2) {
    const int64_t parts = (p.max_ctx + 511) / 512;
    Tensor es = Tensor::empty({S, hq, parts}, Kind::Float, 0), ml = Tensor::empty({S, hq, parts}, Kind::Float, 0);
    Tensor tmp = Tensor::empty({S, hq, parts, 128}, Kind::BFloat16, 0);
    t::paged_attention_v2(out, es, ml, tmp, dq, kc, vc, hkv, scale, bt, cl, 16, p.max_ctx);
  } else {
    t::paged_attention_v1(out, dq, kc, vc, hkv, scale, bt, cl, 16, p.max_ctx);
  }
  expect_close(to_host<uint16_t>(out), want, 2e-2f, 2e-3f);
  EXPECT(t::last_status() == 0, "status word set");
}

// One call for the whole decode step against the two crate calls: same cache, same output, bit for bit.
static void decode_step_equals_cache_write_then_decode() {
  Rng r(27);
  const int hq = 8, hkv = 2;
  const std::vector<int> lens = {1, 16, 17, 300, 513, 1100, 47, 32};
  Paged p(r, 160, hkv, lens);
  const int S = (int)lens.size();
  auto q = randn_bf16(r, (size_t)S * hq * 128);
  auto nk = randn_bf16(r, (size_t)S * hkv * 128), nv = randn_bf16(r, (size_t)S * hkv * 128);
  std::vector<int32_t> slots(S);
  for (int s = 0; s < S; ++s) slots[s] = p.tables[(size_t)s * p.max_blocks + (lens[s] - 1) / 16] * 16 + (lens[s] - 1) % 16;
  const float scale = 0.0884f;
  Tensor dq = to_device(q, {S, hq, 128}, Kind::BFloat16);
  Tensor dk = to_device(nk, {S, hkv, 128}, Kind::BFloat16), dv = to_device(nv, {S, hkv, 128}, Kind::BFloat16);
  Tensor ds = to_device(slots, {S}, Kind::Int);
  Tensor bt = to_device(p.tables, {S, p.max_blocks}, Kind::Int), cl = to_device(p.ctx, {S}, Kind::Int);
  Tensor kc_a = p.key_cache(), vc_a = p.value_cache(), kc_b = p.key_cache(), vc_b = p.value_cache();
  Tensor out_a = Tensor::empty({S, hq, 128}, Kind::BFloat16, 0), out_b = Tensor::empty({S, hq, 128}, Kind::BFloat16, 0);
  t::reshape_and_cache(dk, dv, kc_a, vc_a, ds);
  t::paged_attention_v1(out_a, dq, kc_a, vc_a, hkv, scale, bt, cl, 16, p.max_ctx);
  t::decode_step(out_b, dk, dv, ds, dq, kc_b, vc_b, hkv, scale, bt, cl, 16, p.max_ctx);
  EXPECT(to_host<uint16_t>(kc_a) == to_host<uint16_t>(kc_b), "key caches differ");
  EXPECT(to_host<uint16_t>(vc_a) == to_host<uint16_t>(vc_b), "value caches differ");
  EXPECT(to_host<uint16_t>(out_a) == to_host<uint16_t>(out_b), "outputs differ");
  EXPECT(to_host<uint16_t>(kc_a) != p.kc, "the step wrote nothing");
  EXPECT(t::last_status() == 0, "status word set");
}

static void copy_blocks_matches_oracle() {
  Rng r(31);
  const int layers = 3, nblk = 24, hkv = 2;
  std::vector<Paged> host;
  std::vector<Tensor> kcs, vcs;
  for (int l = 0; l < layers; ++l) {
    host.emplace_back(r, nblk, hkv, std::vector<int>{});
    kcs.push_back(host.back().key_cache());
    vcs.push_back(host.back().value_cache());
  }
  std::unordered_map<size_t, std::vector<size_t>> mapping = {{3, {10, 11}}, {7, {12}}, {0, {23, 13, 14}}};
  t::copy_blocks(kcs, vcs, mapping);
  std::vector<int64_t> pairs;
  for (auto &kv : mapping)
    for (size_t d : kv.second) {
      pairs.push_back((int64_t)kv.first);
      pairs.push_back((int64_t)d);
    }
  std::vector<uint16_t *> kp, vp;
  for (auto &h : host) {
    kp.push_back(h.kc.data());
    vp.push_back(h.vc.data());
  }
  oracle_copy_blocks(kp.data(), vp.data(), pairs.data(), layers, (int)pairs.size() / 2, (int64_t)hkv * 2048);
  for (int l = 0; l < layers; ++l) {
    EXPECT(to_host<uint16_t>(kcs[l]) == host[l].kc, "layer %d key cache differs", l);
    EXPECT(to_host<uint16_t>(vcs[l]) == host[l].vc, "layer %d value cache differs", l);
  }
}

static void swap_blocks_out_and_in() {
  Rng r(41);
  const int nblk = 40, hkv = 4;
  Paged p(r, nblk, hkv, {});
  Tensor gpu = p.key_cache();
  uint16_t *pinned = nullptr;
  const size_t bytes = p.kc.size() * 2;
  t::cuda_check("cudaMallocHost", cudaMallocHost((void **)&pinned, bytes));
  std::memset(pinned, 0, bytes);
  Tensor host = Tensor::view(pinned, {nblk, hkv, 16, 16, 8}, Kind::BFloat16, -1);
  std::unordered_map<size_t, size_t> out_map = {{1, 30}, {2, 5}, {17, 0}, {39, 39}};
  t::swap_blocks(gpu, host, out_map);
  t::cuda_check("sync", cudaDeviceSynchronize());
  const size_t blk = (size_t)hkv * 2048;
  for (auto &kv : out_map)
    EXPECT(std::memcmp(pinned + kv.second * blk, &p.kc[kv.first * blk], blk * 2) == 0, "block %zu -> %zu",
           kv.first, kv.second);
  // wipe the device copy, bring the blocks back
  t::cuda_check("memset", cudaMemset(gpu.data, 0xff, bytes));
  std::unordered_map<size_t, size_t> in_map;
  for (auto &kv : out_map) in_map[kv.second] = kv.first;
  t::swap_blocks(host, gpu, in_map);
  auto back = to_host<uint16_t>(gpu);
  for (auto &kv : out_map)
    EXPECT(std::memcmp(&back[kv.first * blk], &p.kc[kv.first * blk], blk * 2) == 0, "block %zu after swap-in", kv.first);
  cudaFreeHost(pinned);
}

static void flash_attn_varlen_case(const std::vector<int> &lens_q, const std::vector<int> &lens_k, int hq, int hkv,
                                   bool causal, bool arange_inputs) {
  Rng r(51 + hq);
  std::vector<int32_t> cu_q = {0}, cu_k = {0};
  int max_q = 0, max_k = 0;
  for (size_t i = 0; i < lens_q.size(); ++i) {
    cu_q.push_back(cu_q.back() + lens_q[i]);
    cu_k.push_back(cu_k.back() + lens_k[i]);
    max_q = std::max(max_q, lens_q[i]);
    max_k = std::max(max_k, lens_k[i]);
  }
  const int tq = cu_q.back(), tk = cu_k.back();
  std::vector<uint16_t> q, k, v;
  if (arange_inputs) {  // closed-form inputs as in flash_attn_tests.rs:37-48: arange / constant
    auto fill = [](size_t n, float div) {
      std::vector<uint16_t> x(n);
      for (size_t i = 0; i < n; ++i) x[i] = to_bf16((float)(i % 4096) / div);
      return x;
    };
    q = fill((size_t)tq * hq * 128, 3000.f);
    k = fill((size_t)tk * hkv * 128, 4000.f);
    v = fill((size_t)tk * hkv * 128, 5000.f);
  } else {
    q = randn_bf16(r, (size_t)tq * hq * 128);
    k = randn_bf16(r, (size_t)tk * hkv * 128);
    v = randn_bf16(r, (size_t)tk * hkv * 128);
  }
  const float scale = 1.f / std::sqrt(128.f);
  std::vector<float> want((size_t)tq * hq * 128);
  oracle_varlen_attn(want.data(), q.data(), k.data(), v.data(), cu_q.data(), cu_k.data(), (int)lens_q.size(), hq,
                     hkv, 128, hq * 128, 128, hkv * 128, 128, hkv * 128, 128, scale, causal ? 1 : 0, 0);
  Tensor dq = to_device(q, {tq, hq, 128}, Kind::BFloat16), dk = to_device(k, {tk, hkv, 128}, Kind::BFloat16);
  Tensor dv = to_device(v, {tk, hkv, 128}, Kind::BFloat16);
  Tensor sq = to_device(cu_q, {(int64_t)cu_q.size()}, Kind::Int), sk = to_device(cu_k, {(int64_t)cu_k.size()}, Kind::Int);
  Tensor out = t::varlen_attn(dq, dk, dv, sq, sk, max_q, max_k, scale, causal);
  EXPECT(out.sizes == dq.sizes, "output shape");
  expect_close(to_host<uint16_t>(out), want, 2e-2f, 2e-3f);
  EXPECT(t::last_status() == 0, "status word set");
}

static void errors_carry_the_function_name() {
  Tensor q = Tensor::empty({4, 2, 128}, Kind::BFloat16, 0), k = Tensor::empty({4, 2, 128}, Kind::Half, 0);
  Tensor cu = Tensor::empty({2}, Kind::Int, 0);
  auto message_of = [](const std::function<void()> &f) {
    try {
      f();
    } catch (const t::Error &e) {
      return std::string(e.what());
    }
    return std::string();
  };
  std::string m = message_of([&] { t::flash_attn_varlen(q, k, k, cu, cu, 4, 4, 1.f, true); });
  EXPECT(m == "flash_attn_varlen: query and key must have the same dtype", "got '%s'", m.c_str());
  Tensor q64 = Tensor::empty({4, 2, 64}, Kind::BFloat16, 0);
  m = message_of([&] { t::flash_attn_varlen(q64, q64, q64, cu, cu, 4, 4, 1.f, true); });
  EXPECT(m.rfind("flash_attn_varlen: ", 0) == 0 && m.find("head_size must be 128") != std::string::npos, "got '%s'",
         m.c_str());
  Tensor host = Tensor::view(nullptr, {4, 2, 128}, Kind::BFloat16, -1);
  m = message_of([&] { t::flash_attn_varlen(host, q, q, cu, cu, 4, 4, 1.f, true); });
  EXPECT(m.find("there is no CPU path") != std::string::npos, "got '%s'", m.c_str());
  Tensor a = Tensor::empty({2, 1, 16, 16, 8}, Kind::BFloat16, 0);
  Tensor hb = Tensor::view(nullptr, {2, 1, 16, 16, 8}, Kind::BFloat16, -1);
  m = message_of([&] { Tensor h2 = hb; t::swap_blocks(hb, h2, {{0, 1}}); });
  EXPECT(m == "swap_blocks: Invalid device combination", "got '%s'", m.c_str());
  m = message_of([&] { Tensor a2 = a; t::swap_blocks(a, a2, {{5, 1}}); });
  EXPECT(m.rfind("swap_blocks: ", 0) == 0 && m.find("outside the cache") != std::string::npos, "got '%s'", m.c_str());
}

static void batch_info_feeds_the_decode_kernel() {
  // A decode step described as entries (batch_info.rs:93-97), built by the native builder into one
  // staging buffer, uploaded with one copy, and consumed in place by reshape_and_cache + decode.
  Rng r(61);
  const int hq = 8, hkv = 2;
  const std::vector<int> lens = {40, 333, 16, 1, 129};
  Paged p(r, 64, hkv, lens);
  const int S = (int)lens.size();
  std::vector<std::vector<int64_t>> slots(S);
  std::vector<int32_t> token(S, 7);
  std::vector<aici_batch_entry> ent(S);
  for (int s = 0; s < S; ++s) {
    for (int tk = 0; tk < lens[s]; ++tk) slots[s].push_back((int64_t)p.rows[s][tk / 16] * 16 + tk % 16);
    ent[s] = {100 + s, &token[s], nullptr, slots[s].data(), 1, lens[s]};
  }
  aici_batch_layout lay;
  t::check("aici_batch_info_layout", aici_batch_info_layout(ent.data(), S, AICI_BATCH_PAGED_DECODE | AICI_BATCH_NO_GATHER_MAP,
                                                            16, 4096, &lay));
  EXPECT(lay.num_paged == S && lay.num_multitoken == 0 && lay.paged_max_context_len == 333, "layout counts");
  void *staging = nullptr;
  t::cuda_check("cudaMallocHost", cudaMallocHost(&staging, (size_t)lay.total_bytes));
  Tensor dev = Tensor::empty({lay.total_bytes}, Kind::Int64, 0);  // over-sized on purpose (8 B elements)
  std::vector<int32_t> order(S);
  t::check("aici_batch_info_build",
           aici_batch_info_build(ent.data(), S, AICI_BATCH_PAGED_DECODE | AICI_BATCH_NO_GATHER_MAP, 16, 4096, staging,
                                 (size_t)lay.total_bytes, dev.data, (size_t)lay.total_bytes * 8, &lay, order.data(),
                                 cudaStreamPerThread));
  char *base = static_cast<char *>(dev.data);
  Tensor slot_mapping = Tensor::view(base + lay.slot_mapping_off, {S}, Kind::Int, 0);
  Tensor bt = Tensor::view(base + lay.block_tables_off, {S, lay.max_blocks_per_seq}, Kind::Int, 0);
  Tensor cl = Tensor::view(base + lay.context_lens_off, {S}, Kind::Int, 0);
  // new token's k/v into the cache, then decode over the whole context
  auto nk = randn_bf16(r, (size_t)S * hkv * 128), nv = randn_bf16(r, (size_t)S * hkv * 128);
  auto q = randn_bf16(r, (size_t)S * hq * 128);
  Tensor kc = p.key_cache(), vc = p.value_cache();
  t::reshape_and_cache(to_device(nk, {S, hkv, 128}, Kind::BFloat16), to_device(nv, {S, hkv, 128}, Kind::BFloat16), kc, vc,
                       slot_mapping);
  Tensor out = Tensor::empty({S, hq, 128}, Kind::BFloat16, 0);
  t::paged_attention_v1(out, to_device(q, {S, hq, 128}, Kind::BFloat16), kc, vc, hkv, 0.09f, bt, cl, 16,
                        lay.paged_max_context_len);
  std::vector<int64_t> s64;
  for (int s = 0; s < S; ++s) s64.push_back(slots[s].back());
  oracle_reshape_and_cache(nk.data(), nv.data(), p.kc.data(), p.vc.data(), s64.data(), S, hkv * 128, hkv * 128, hkv,
                           128, 16, 8);
  std::vector<float> want((size_t)S * hq * 128);
  oracle_paged_attention_v1(want.data(), q.data(), p.kc.data(), p.vc.data(), hkv, 0.09f, p.tables.data(), p.ctx.data(),
                            S, hq, 128, 16, 8, p.max_blocks, hq * 128, (int64_t)hkv * 2048, 2048, 0);
  expect_close(to_host<uint16_t>(out), want, 2e-2f, 2e-3f);
  for (int s = 0; s < S; ++s) EXPECT(order[s] == s, "entry order");
  cudaFreeHost(staging);
}

static void paged_prefill_reads_the_cache_through_block_tables() {
  // A chunk of new tokens behind a cached prefix: keys/values only exist in the paged cache.
  Rng r(71);
  const int hq = 8, hkv = 2;
  const std::vector<int> lens_k = {200, 70, 33}, lens_q = {72, 70, 1};
  Paged p(r, 40, hkv, lens_k);
  const int B = (int)lens_k.size();
  std::vector<int32_t> cu_q = {0}, cu_k = {0};
  for (int i = 0; i < B; ++i) {
    cu_q.push_back(cu_q.back() + lens_q[i]);
    cu_k.push_back(cu_k.back() + lens_k[i]);
  }
  const int tq = cu_q.back(), tk = cu_k.back();
  auto q = randn_bf16(r, (size_t)tq * hq * 128);
  // the packed K/V the oracle wants, read out of the cache layout on the host
  std::vector<uint16_t> k((size_t)tk * hkv * 128), v((size_t)tk * hkv * 128);
  for (int s = 0; s < B; ++s)
    for (int tok = 0; tok < lens_k[s]; ++tok)
      for (int h = 0; h < hkv; ++h)
        for (int d = 0; d < 128; ++d) {
          const size_t blk = (size_t)p.rows[s][tok / 16], off = tok % 16;
          const size_t dst = ((size_t)(cu_k[s] + tok) * hkv + h) * 128 + d;
          k[dst] = p.kc[(((blk * hkv + h) * 16 + d / 8) * 16 + off) * 8 + d % 8];
          v[dst] = p.vc[((blk * hkv + h) * 128 + d) * 16 + off];
        }
  const float scale = 1.f / std::sqrt(128.f);
  std::vector<float> want((size_t)tq * hq * 128);
  oracle_varlen_attn(want.data(), q.data(), k.data(), v.data(), cu_q.data(), cu_k.data(), B, hq, hkv, 128, hq * 128,
                     128, hkv * 128, 128, hkv * 128, 128, scale, 1, 0);
  Tensor out = t::flash_attn_varlen_paged(to_device(q, {tq, hq, 128}, Kind::BFloat16), p.key_cache(), p.value_cache(),
                                          to_device(cu_q, {B + 1}, Kind::Int), to_device(p.ctx, {B}, Kind::Int),
                                          to_device(p.tables, {B, p.max_blocks}, Kind::Int), 72, 200, scale, true);
  expect_close(to_host<uint16_t>(out), want, 2e-2f, 2e-3f);
  EXPECT(t::last_status() == 0, "status word set");
}

static void rotary_and_cache_write_in_one_pass() {
  Rng r(81);
  const int T = 21, hq = 8, hkv = 2, nblk = 6, max_pos = 64;
  Paged p(r, nblk, hkv, {});
  auto q = randn_bf16(r, (size_t)T * hq * 128), k = randn_bf16(r, (size_t)T * hkv * 128);
  auto v = randn_bf16(r, (size_t)T * hkv * 128);
  std::vector<uint16_t> cs((size_t)max_pos * 128);  // [cos | sin] per position (llm/mod.rs:41-60)
  for (int pos = 0; pos < max_pos; ++pos)
    for (int i = 0; i < 64; ++i) {
      const float a = pos * std::pow(10000.f, -2.f * i / 128.f);
      cs[(size_t)pos * 128 + i] = to_bf16(std::cos(a));
      cs[(size_t)pos * 128 + 64 + i] = to_bf16(std::sin(a));
    }
  std::vector<int64_t> positions(T), slots(T);
  for (int i = 0; i < T; ++i) {
    positions[i] = r.below(max_pos);
    slots[i] = 3 + i;  // a run that starts in the middle of a block
  }
  Tensor dq = to_device(q, {T, hq, 128}, Kind::BFloat16), dk = to_device(k, {T, hkv, 128}, Kind::BFloat16);
  Tensor kc = p.key_cache(), vc = p.value_cache();
  t::rotary_embedding_reshape_and_cache(to_device(positions, {T}, Kind::Int64), dq, dk,
                                        to_device(v, {T, hkv, 128}, Kind::BFloat16),
                                        to_device(cs, {max_pos, 128}, Kind::BFloat16), kc, vc,
                                        to_device(slots, {T}, Kind::Int64));
  oracle_rotary_embedding_neox(positions.data(), q.data(), k.data(), cs.data(), T, hq, hkv, 128, 128, hq * 128, hkv * 128);
  oracle_reshape_and_cache(k.data(), v.data(), p.kc.data(), p.vc.data(), slots.data(), T, hkv * 128, hkv * 128, hkv, 128,
                           16, 8);
  EXPECT(to_host<uint16_t>(dq) == q, "rotated query differs from the oracle");
  EXPECT(to_host<uint16_t>(dk) == k, "rotated key differs from the oracle");
  EXPECT(to_host<uint16_t>(kc) == p.kc, "key cache differs from the oracle");
  EXPECT(to_host<uint16_t>(vc) == p.vc, "value cache differs from the oracle");
}

struct Test {
  const char *name;
  std::function<void()> fn;
};

int main(int argc, char **argv) {
  const std::vector<Test> tests = {
      {"reshape_and_cache_then_gather_round_trip", reshape_and_cache_then_gather_round_trip},
      {"paged_attention_v1_matches_oracle", [] { paged_attention_matches_oracle(false); }},
      {"paged_attention_v2_matches_oracle", [] { paged_attention_matches_oracle(true); }},
      {"decode_step_equals_cache_write_then_decode", decode_step_equals_cache_write_then_decode},
      {"copy_blocks_matches_oracle", copy_blocks_matches_oracle},
      {"swap_blocks_out_and_in", swap_blocks_out_and_in},
      {"flash_attn_varlen_causal_ragged_gqa", [] { flash_attn_varlen_case({64, 130, 1, 257}, {64, 130, 1, 257}, 8, 2, true, false); }},
      {"flash_attn_varlen_cached_prefix_bottom_right_mask", [] { flash_attn_varlen_case({5, 70}, {200, 70}, 4, 4, true, false); }},
      {"flash_attn_varlen_non_causal_closed_form_inputs", [] { flash_attn_varlen_case({2, 33}, {2, 33}, 3, 3, false, true); }},
      {"errors_carry_the_function_name", errors_carry_the_function_name},
      {"batch_info_feeds_the_decode_kernel", batch_info_feeds_the_decode_kernel},
      {"paged_prefill_reads_the_cache_through_block_tables", paged_prefill_reads_the_cache_through_block_tables},
      {"rotary_and_cache_write_in_one_pass", rotary_and_cache_write_in_one_pass},
  };
  if (argc > 1 && std::string(argv[1]) == "--list") {
    for (const Test &tc : tests) std::printf("%s\n", tc.name);
    return 0;
  }
  int device_count = 0;
  if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_count == 0) {
    std::printf("no CUDA device: these tests need a GPU (there is no CPU path)\n");
    return 77;
  }
  t::cuda_check("cudaSetDevice", cudaSetDevice(0));
  int failed = 0;
  for (const Test &tc : tests) {
    try {
      tc.fn();
      std::printf("[  OK  ] %s\n", tc.name);
    } catch (const Failure &f) {
      std::printf("[ FAIL ] %s: %s\n", tc.name, f.msg.c_str());
      ++failed;
    } catch (const std::exception &e) {
      std::printf("[ FAIL ] %s: exception: %s\n", tc.name, e.what());
      ++failed;
    }
    std::fflush(stdout);
  }
  std::printf("%d of %zu tests failed\n", failed, tests.size());
  return failed;
}
