/*
 * CPU oracle for the rLLM attention path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Plain-C restatement of the arithmetic and index math of the reference's GPU kernels
 * (paths below are relative to the reference project root).  Only the test-suite, the
 * smoke check and the benchmark's cpu_baseline leg may load this library; the product
 * path (aici_b200/) never does.
 *
 * Parity status: varlen attention is pinned by the reference's one stored known-answer
 * test (rllm/tch-cuda/tests/flash_attn_tests.rs:35-74).  reshape_and_cache,
 * gather_cached_kv, copy_blocks and paged_attention_v1/v2 have no stored vectors in the
 * reference ("parity unpinned" by golden data); they are restated line by line from the
 * kernels cited at each function and cross-checked against an independent PyTorch-CPU
 * restatement of rllm/rllm-cuda/src/llm/refkernels.rs.
 *
 * All 16-bit tensors are passed as uint16_t bit patterns (bf16).  Accumulation is fp32
 * unless stated.  Build: see oracle/build_oracle.py (gcc -O2 -fopenmp -shared).
 */
#include <math.h>
#include <float.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, NaN kept quiet: what __float2bfloat16_rn does */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

/* ------------------------------------------------------------------------------------
 * reshape_and_cache: rllm/tch-cuda/kernels/vllm/cache_kernels.cu:168-213
 *   key/value  [num_tokens, num_heads, head_size] with a free token stride
 *   key_cache  [num_blocks, num_heads, head_size/x, block_size, x]
 *   value_cache[num_blocks, num_heads, head_size, block_size]
 *   slot < 0 is a padding token and is skipped (:183-186).
 * ---------------------------------------------------------------------------------- */
void oracle_reshape_and_cache(const uint16_t *key, const uint16_t *value,
                              uint16_t *key_cache, uint16_t *value_cache,
                              const int64_t *slot_mapping, int num_tokens,
                              int64_t key_stride, int64_t value_stride,
                              int num_heads, int head_size, int block_size, int x) {
  const int n = num_heads * head_size;
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    const int64_t blk = slot / block_size;
    const int64_t off = slot % block_size;
    for (int i = 0; i < n; ++i) {
      const int h = i / head_size, d = i % head_size;
      const int xi = d / x, xo = d % x;
      const int64_t kdst = blk * num_heads * (head_size / x) * block_size * x +
                           (int64_t)h * (head_size / x) * block_size * x +
                           (int64_t)xi * block_size * x + off * x + xo;
      const int64_t vdst = blk * num_heads * head_size * block_size +
                           (int64_t)h * head_size * block_size +
                           (int64_t)d * block_size + off;
      key_cache[kdst] = key[t * key_stride + i];
      value_cache[vdst] = value[t * value_stride + i];
    }
  }
}

/* gather_cached_kv: cache_kernels.cu:301-373 (int32 slots; exact inverse of the above) */
void oracle_gather_cached_kv(uint16_t *key, uint16_t *value, const uint16_t *key_cache,
                             const uint16_t *value_cache, const int32_t *slot_mapping,
                             int num_tokens, int64_t key_stride, int64_t value_stride,
                             int num_heads, int head_size, int block_size, int x) {
  const int n = num_heads * head_size;
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t slot = slot_mapping[t];
    const int64_t blk = slot / block_size;
    const int64_t off = slot % block_size;
    for (int i = 0; i < n; ++i) {
      const int h = i / head_size, d = i % head_size;
      const int xi = d / x, xo = d % x;
      const int64_t ksrc = blk * num_heads * (head_size / x) * block_size * x +
                           (int64_t)h * (head_size / x) * block_size * x +
                           (int64_t)xi * block_size * x + off * x + xo;
      const int64_t vsrc = blk * num_heads * head_size * block_size +
                           (int64_t)h * head_size * block_size +
                           (int64_t)d * block_size + off;
      key[t * key_stride + i] = key_cache[ksrc];
      value[t * value_stride + i] = value_cache[vsrc];
    }
  }
}

/* copy_blocks: cache_kernels.cu:55-81 (kernel) and :141-163 (copy_blocks_2 host side).
 * Pairs are applied in list order; the reference runs them concurrently, which is only
 * well defined when no dst is also a src or repeated (true for the block allocator,
 * rllm/rllm-cuda/src/llm/paged/blocks.rs:221-233). */
void oracle_copy_blocks(uint16_t *const *key_caches, uint16_t *const *value_caches,
                        const int64_t *block_mapping, int num_layers, int num_pairs,
                        int64_t numel_per_block) {
  for (int l = 0; l < num_layers; ++l)
    for (int p = 0; p < num_pairs; ++p) {
      const int64_t src = block_mapping[2 * p], dst = block_mapping[2 * p + 1];
      memmove(key_caches[l] + dst * numel_per_block, key_caches[l] + src * numel_per_block,
              (size_t)numel_per_block * 2);
      memmove(value_caches[l] + dst * numel_per_block,
              value_caches[l] + src * numel_per_block, (size_t)numel_per_block * 2);
    }
}

/* ------------------------------------------------------------------------------------
 * paged attention, one partition [tok0, tok1) of one (sequence, query head):
 * rllm/tch-cuda/kernels/vllm/attention/attention_kernels.cu:85-392.
 *   logits fp32 = scale * q.k (:213-227), max, exp(l-max), sum, p = e/(sum+1e-6)
 *   (:253-265), out = sum_t p[t] * V[t] (:300-330).
 * ref_rounding != 0 reproduces the reference's 16-bit steps: p is cast to bf16 and each
 * p*v product is rounded to bf16 before the fp32 accumulation
 * (attention_kernels.cu:306-307,327; dtype_bfloat16.cuh:205-212).  ref_rounding == 0 is
 * the fp32-softmax reference the acceptance bound is stated against.
 * ---------------------------------------------------------------------------------- */
static void paged_partition(const uint16_t *q, const uint16_t *k_cache,
                            const uint16_t *v_cache, const int32_t *block_table,
                            int64_t kv_block_stride, int64_t kv_head_stride, int kv_head,
                            int head_size, int block_size, int x, float scale, int tok0,
                            int tok1, int ref_rounding, float *logits, float *out,
                            float *max_logit, float *exp_sum) {
  float qf[256];
  for (int d = 0; d < head_size; ++d) qf[d] = bf16_to_f32(q[d]);
  float m = -FLT_MAX;
  for (int t = tok0; t < tok1; ++t) {
    const int64_t blk = block_table[t / block_size];
    const int off = t % block_size;
    const uint16_t *kp = k_cache + blk * kv_block_stride + (int64_t)kv_head * kv_head_stride;
    float acc = 0.f;
    for (int d = 0; d < head_size; ++d)
      acc += qf[d] * bf16_to_f32(kp[(d / x) * block_size * x + off * x + (d % x)]);
    const float l = scale * acc;
    logits[t - tok0] = l;
    if (l > m) m = l;
  }
  float s = 0.f;
  for (int t = 0; t < tok1 - tok0; ++t) {
    logits[t] = expf(logits[t] - m);
    s += logits[t];
  }
  const float inv = 1.f / (s + 1e-6f);
  for (int d = 0; d < head_size; ++d) out[d] = 0.f;
  for (int t = tok0; t < tok1; ++t) {
    float p = logits[t - tok0] * inv;
    if (ref_rounding) p = round_bf16(p);
    const int64_t blk = block_table[t / block_size];
    const int off = t % block_size;
    const uint16_t *vp = v_cache + blk * kv_block_stride + (int64_t)kv_head * kv_head_stride;
    for (int d = 0; d < head_size; ++d) {
      float pv = p * bf16_to_f32(vp[d * block_size + off]);
      if (ref_rounding) pv = round_bf16(pv);
      out[d] += pv;
    }
  }
  *max_logit = m;
  *exp_sum = s;
}

/* paged_attention_v1: attention_kernels.cu:395-418, launcher :571-646.
 * out_f32 [num_seqs, num_heads, head_size] (fp32, before the final cast to T). */
void oracle_paged_attention_v1(float *out_f32, const uint16_t *q, const uint16_t *k_cache,
                               const uint16_t *v_cache, int num_kv_heads, float scale,
                               const int32_t *block_tables, const int32_t *context_lens,
                               int num_seqs, int num_heads, int head_size, int block_size,
                               int x, int max_num_blocks_per_seq, int64_t q_stride,
                               int64_t kv_block_stride, int64_t kv_head_stride,
                               int ref_rounding) {
  const int qpk = num_heads / num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int s = 0; s < num_seqs; ++s)
    for (int h = 0; h < num_heads; ++h) {
      const int ctx = context_lens[s];
      float *o = out_f32 + ((int64_t)s * num_heads + h) * head_size;
      float *logits = (float *)malloc(sizeof(float) * (size_t)(ctx > 0 ? ctx : 1));
      float m, e;
      paged_partition(q + s * q_stride + (int64_t)h * head_size, k_cache, v_cache,
                      block_tables + (int64_t)s * max_num_blocks_per_seq, kv_block_stride,
                      kv_head_stride, h / qpk, head_size, block_size, x, scale, 0, ctx,
                      ref_rounding, logits, o, &m, &e);
      free(logits);
    }
}

/* paged_attention_v2 + reduce: attention_kernels.cu:421-546, launcher :729-814.
 * Partitions of `partition_size` tokens (512 in the reference, :733).  Each partition's
 * normalised output is rounded to bf16 (tmp_out is T, :381-390) when ref_rounding != 0.
 * Reduce (:450-546): out = sum_j tmp_j * exp_sum_j * e^(max_j-max) / (sum + 1e-6);
 * single-partition rows are copied (:467-477). */
void oracle_paged_attention_v2(float *out_f32, const uint16_t *q, const uint16_t *k_cache,
                               const uint16_t *v_cache, int num_kv_heads, float scale,
                               const int32_t *block_tables, const int32_t *context_lens,
                               int num_seqs, int num_heads, int head_size, int block_size,
                               int x, int max_num_blocks_per_seq, int64_t q_stride,
                               int64_t kv_block_stride, int64_t kv_head_stride,
                               int partition_size, int ref_rounding) {
  const int qpk = num_heads / num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int s = 0; s < num_seqs; ++s)
    for (int h = 0; h < num_heads; ++h) {
      const int ctx = context_lens[s];
      const int parts = (ctx + partition_size - 1) / partition_size;
      float *o = out_f32 + ((int64_t)s * num_heads + h) * head_size;
      for (int d = 0; d < head_size; ++d) o[d] = 0.f;
      if (parts == 0) continue;
      float *logits = (float *)malloc(sizeof(float) * (size_t)partition_size);
      float *tmp = (float *)malloc(sizeof(float) * (size_t)parts * head_size);
      float *mx = (float *)malloc(sizeof(float) * (size_t)parts);
      float *es = (float *)malloc(sizeof(float) * (size_t)parts);
      for (int j = 0; j < parts; ++j) {
        const int t0 = j * partition_size;
        const int t1 = t0 + partition_size < ctx ? t0 + partition_size : ctx;
        paged_partition(q + s * q_stride + (int64_t)h * head_size, k_cache, v_cache,
                        block_tables + (int64_t)s * max_num_blocks_per_seq,
                        kv_block_stride, kv_head_stride, h / qpk, head_size, block_size, x,
                        scale, t0, t1, ref_rounding, logits, tmp + (int64_t)j * head_size,
                        &mx[j], &es[j]);
        if (ref_rounding)
          for (int d = 0; d < head_size; ++d)
            tmp[(int64_t)j * head_size + d] = round_bf16(tmp[(int64_t)j * head_size + d]);
      }
      if (parts == 1) {
        for (int d = 0; d < head_size; ++d) o[d] = tmp[d];
      } else {
        float m = -FLT_MAX;
        for (int j = 0; j < parts; ++j)
          if (mx[j] > m) m = mx[j];
        float g = 0.f;
        for (int j = 0; j < parts; ++j) {
          es[j] = es[j] * expf(mx[j] - m);
          g += es[j];
        }
        const float inv = 1.f / (g + 1e-6f);
        for (int d = 0; d < head_size; ++d) {
          float acc = 0.f;
          for (int j = 0; j < parts; ++j) acc += tmp[(int64_t)j * head_size + d] * es[j] * inv;
          o[d] = acc;
        }
      }
      free(logits);
      free(tmp);
      free(mx);
      free(es);
    }
}

/* ------------------------------------------------------------------------------------
 * Variable-length attention: mha_varlen_fwd,
 * rllm/tch-cuda/kernels/flash_attn/flash_api.cpp:447-618 and flash_fwd_kernel.h:590-1136.
 *   q [total_q, Hq, D], k/v [total_k, Hkv, D] with free token/head strides,
 *   cu_seqlens_{q,k} int32 [b+1]; kv head = h / (Hq/Hkv) (flash_fwd_kernel.h:679).
 *   causal mask is bottom-right aligned: row r sees columns < min(len_k, r+1+len_k-len_q)
 *   (softmax.h:159-168; same in rllm-cuda/src/llm/refkernels.rs:102-108).
 *   Rows with no visible column give 0 (flash_fwd_kernel.h:1056).
 * p_bf16 != 0 rounds the unnormalised probabilities to bf16 before PV, as the kernel does
 * (flash_fwd_kernel.h:985,1039); p_bf16 == 0 is the fp32-softmax reference.
 * out_f32 [total_q, Hq, D] contiguous.
 * ---------------------------------------------------------------------------------- */
void oracle_varlen_attn(float *out_f32, const uint16_t *q, const uint16_t *k,
                        const uint16_t *v, const int32_t *cu_q, const int32_t *cu_k,
                        int batch, int num_heads, int num_heads_k, int head_size,
                        int64_t q_tok_stride, int64_t q_head_stride, int64_t k_tok_stride,
                        int64_t k_head_stride, int64_t v_tok_stride, int64_t v_head_stride,
                        float scale, int causal, int p_bf16) {
  const int qpk = num_heads / num_heads_k;
  for (int b = 0; b < batch; ++b) {
    const int q0 = cu_q[b], lq = cu_q[b + 1] - cu_q[b];
    const int k0 = cu_k[b], lk = cu_k[b + 1] - cu_k[b];
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
    for (int h = 0; h < num_heads; ++h)
      for (int r = 0; r < lq; ++r) {
        const int hk = h / qpk;
        float *o = out_f32 + ((int64_t)(q0 + r) * num_heads + h) * head_size;
        for (int d = 0; d < head_size; ++d) o[d] = 0.f;
        int lim = lk;
        if (causal) {
          const int c = r + 1 + lk - lq;
          lim = c < lk ? c : lk;
        }
        if (lim <= 0) continue;
        float qf[256];
        const uint16_t *qp = q + (int64_t)(q0 + r) * q_tok_stride + (int64_t)h * q_head_stride;
        for (int d = 0; d < head_size; ++d) qf[d] = bf16_to_f32(qp[d]);
        float *sc = (float *)malloc(sizeof(float) * (size_t)lim);
        float m = -INFINITY;
        for (int c = 0; c < lim; ++c) {
          const uint16_t *kp = k + (int64_t)(k0 + c) * k_tok_stride + (int64_t)hk * k_head_stride;
          float acc = 0.f;
          for (int d = 0; d < head_size; ++d) acc += qf[d] * bf16_to_f32(kp[d]);
          sc[c] = acc * scale;
          if (sc[c] > m) m = sc[c];
        }
        float sum = 0.f;
        for (int c = 0; c < lim; ++c) {
          float p = expf(sc[c] - m);
          sum += p;
          if (p_bf16) p = round_bf16(p);
          const uint16_t *vp = v + (int64_t)(k0 + c) * v_tok_stride + (int64_t)hk * v_head_stride;
          for (int d = 0; d < head_size; ++d) o[d] += p * bf16_to_f32(vp[d]);
        }
        const float inv = 1.f / sum;
        for (int d = 0; d < head_size; ++d) o[d] *= inv;
        free(sc);
      }
  }
}

/* Row-sampled variant for sizes where the full problem is too slow on a CPU: computes only
 * the listed (token, head) rows; tok is an index into the packed q, seq its batch entry.
 * out_f32 [n_rows, D]. Same arithmetic as oracle_varlen_attn. */
void oracle_varlen_attn_rows(float *out_f32, const uint16_t *q, const uint16_t *k,
                             const uint16_t *v, const int32_t *cu_q, const int32_t *cu_k,
                             const int32_t *row_seq, const int32_t *row_tok,
                             const int32_t *row_head, int n_rows, int num_heads,
                             int num_heads_k, int head_size, int64_t q_tok_stride,
                             int64_t q_head_stride, int64_t k_tok_stride,
                             int64_t k_head_stride, int64_t v_tok_stride,
                             int64_t v_head_stride, float scale, int causal, int p_bf16) {
  const int qpk = num_heads / num_heads_k;
#pragma omp parallel for schedule(dynamic, 4)
  for (int i = 0; i < n_rows; ++i) {
    const int b = row_seq[i], h = row_head[i], hk = h / qpk;
    const int q0 = cu_q[b], lq = cu_q[b + 1] - cu_q[b];
    const int k0 = cu_k[b], lk = cu_k[b + 1] - cu_k[b];
    const int r = row_tok[i] - q0;
    float *o = out_f32 + (int64_t)i * head_size;
    for (int d = 0; d < head_size; ++d) o[d] = 0.f;
    int lim = lk;
    if (causal) {
      const int c = r + 1 + lk - lq;
      lim = c < lk ? c : lk;
    }
    if (lim <= 0) continue;
    float qf[256];
    const uint16_t *qp = q + (int64_t)(q0 + r) * q_tok_stride + (int64_t)h * q_head_stride;
    for (int d = 0; d < head_size; ++d) qf[d] = bf16_to_f32(qp[d]);
    float *sc = (float *)malloc(sizeof(float) * (size_t)lim);
    float m = -INFINITY;
    for (int c = 0; c < lim; ++c) {
      const uint16_t *kp = k + (int64_t)(k0 + c) * k_tok_stride + (int64_t)hk * k_head_stride;
      float acc = 0.f;
      for (int d = 0; d < head_size; ++d) acc += qf[d] * bf16_to_f32(kp[d]);
      sc[c] = acc * scale;
      if (sc[c] > m) m = sc[c];
    }
    float sum = 0.f;
    for (int c = 0; c < lim; ++c) {
      float p = expf(sc[c] - m);
      sum += p;
      if (p_bf16) p = round_bf16(p);
      const uint16_t *vp = v + (int64_t)(k0 + c) * v_tok_stride + (int64_t)hk * v_head_stride;
      for (int d = 0; d < head_size; ++d) o[d] += p * bf16_to_f32(vp[d]);
    }
    const float inv = 1.f / sum;
    for (int d = 0; d < head_size; ++d) o[d] *= inv;
    free(sc);
  }
}

/* rotary_embedding, NeoX pairing: rllm/tch-cuda/kernels/vllm/pos_encoding_kernels.cu:9-80.
 * query [T, Hq, D] and key [T, Hkv, D] rotated in place; cos_sin_cache [max_position, rot_dim]
 * = [cos 0..rot/2 | sin 0..rot/2].  The kernel computes `x*cos - y*sin` and `y*cos + x*sin` on the
 * 16-bit scalar type: every product and the sum/difference is rounded to bf16. */
void oracle_rotary_embedding_neox(const int64_t *positions, uint16_t *query, uint16_t *key,
                                  const uint16_t *cos_sin_cache, int num_tokens, int num_heads,
                                  int num_kv_heads, int head_size, int rot_dim, int64_t query_stride,
                                  int64_t key_stride) {
  const int embed = rot_dim / 2;
  for (int64_t t = 0; t < num_tokens; ++t) {
    const uint16_t *cs = cos_sin_cache + positions[t] * rot_dim;
    for (int pass = 0; pass < 2; ++pass) {
      uint16_t *base = pass == 0 ? query + t * query_stride : key + t * key_stride;
      const int heads = pass == 0 ? num_heads : num_kv_heads;
      for (int h = 0; h < heads; ++h)
        for (int i = 0; i < embed; ++i) {
          uint16_t *arr = base + (int64_t)h * head_size;
          const float c = bf16_to_f32(cs[i]), s = bf16_to_f32(cs[embed + i]);
          const float x = bf16_to_f32(arr[i]), y = bf16_to_f32(arr[embed + i]);
          arr[i] = f32_to_bf16(round_bf16(x * c) - round_bf16(y * s));
          arr[embed + i] = f32_to_bf16(round_bf16(y * c) + round_bf16(x * s));
        }
    }
  }
}

/* bf16 round-trip helper exposed so Python can round an fp32 buffer exactly as the GPU
 * store does (round-to-nearest-even). */
void oracle_round_to_bf16(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
