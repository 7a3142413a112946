// Step metadata staging: the host-side builder that turns the running sequences of one step into
// the index tensors the attention path consumes, laid out in one buffer and uploaded with one copy.
//
// Follows BatchInfoBuilder::finish (rllm-cuda/src/llm/paged/batch_info.rs:196-315) section by
// section: entry order (:209-221), tokens / positions / slot_mapping / logit_idxs (:227-238),
// gather_mapping and the sequence lengths of multi-token entries (:239-245), block tables and
// context lengths of single-token entries (:246-262), offsets as to_offsets makes them
// (llm/kernels.rs:10-21), block-table rows padded with zeros to the longest (:277-293).
// Host code only: the single launch-side effect is the cudaMemcpyAsync at the end.
#include <vector>

#include "common.cuh"

namespace aici {

constexpr int64_t kSectionAlign = 256;

static int64_t place(int64_t *cursor, int64_t bytes) {
  const int64_t off = *cursor;
  *cursor = (off + bytes + kSectionAlign - 1) / kSectionAlign * kSectionAlign;
  return off;
}

// Validates the entries, decides their order and fills every field of `lay`.
// check_slots: also walk the block-start slots (one cache line each); the builder does that walk
// itself while it fills the tables, so it asks for sizes only.
static char *plan_batch(const char *fn, const aici_batch_entry *entries, int n, int flags,
                        int block_size, int64_t max_model_len, aici_batch_layout *lay,
                        std::vector<int> *order, bool check_slots) {
  AICI_CHECK(lay != nullptr, "%s: layout is NULL", fn);
  AICI_CHECK(n > 0 && entries != nullptr, "%s: a step needs at least one sequence", fn);
  AICI_CHECK(block_size > 0, "%s: block_size must be positive", fn);
  AICI_CHECK((flags & ~7) == 0, "%s: unknown flag bits 0x%x", fn, flags);
  const bool paged = (flags & AICI_BATCH_PAGED_DECODE) != 0;
  const bool all_tables = (flags & AICI_BATCH_TABLES_FOR_ALL) != 0;
  const bool gather = (flags & AICI_BATCH_NO_GATHER_MAP) == 0;

  order->clear();
  order->reserve(n);
  for (int i = 0; i < n; ++i) {
    const aici_batch_entry &e = entries[i];
    AICI_CHECK(e.q_len >= 1 && e.k_len >= e.q_len,
               "%s: entry %d: need 1 <= q_len <= k_len (got %d, %d)", fn, i, e.q_len, e.k_len);
    AICI_CHECK(e.tokens != nullptr && e.kv_slots != nullptr, "%s: entry %d: NULL array", fn, i);
    if (!paged || e.q_len != 1) order->push_back(i);
  }
  const int num_multi = static_cast<int>(order->size());
  if (paged)
    for (int i = 0; i < n; ++i)
      if (entries[i].q_len == 1) order->push_back(i);

  int64_t num_tokens = 0, gather_len = 0, q_multi = 0;
  int max_q = 0, max_k = 0, max_blocks = 0, paged_max_ctx = 0;
  for (int idx = 0; idx < n; ++idx) {
    const aici_batch_entry &e = entries[(*order)[idx]];
    for (int j = 0; j < e.q_len; ++j) {
      const int64_t pos = e.positions ? e.positions[j] : (int64_t)(e.k_len - e.q_len + j);
      AICI_CHECK(pos >= 0 && pos < max_model_len,
                 "%s: sequence %lld: position %lld is not below max_model_len %lld", fn,
                 (long long)e.seq_id, (long long)pos, (long long)max_model_len);
    }
    num_tokens += e.q_len;
    const bool multi = idx < num_multi;
    if (multi) {
      if (gather) gather_len += e.k_len;
      q_multi = num_tokens;
      max_q = e.q_len > max_q ? e.q_len : max_q;
      max_k = e.k_len > max_k ? e.k_len : max_k;
    } else {
      paged_max_ctx = e.k_len > paged_max_ctx ? e.k_len : paged_max_ctx;
    }
    if (!multi || all_tables) {
      const int nb = (e.k_len + block_size - 1) / block_size;
      max_blocks = nb > max_blocks ? nb : max_blocks;
      for (int t = 0; check_slots && t < e.k_len; t += block_size) {
        const int64_t slot = e.kv_slots[t];
        AICI_CHECK(slot >= 0 && slot % block_size == 0 && slot / block_size <= INT32_MAX,
                   "%s: sequence %lld: slot %lld at token %d does not start a block of %d", fn,
                   (long long)e.seq_id, (long long)slot, t, block_size);
      }
    }
  }
  AICI_CHECK(num_tokens <= INT32_MAX && gather_len <= INT32_MAX, "%s: step too large", fn);

  memset(lay, 0, sizeof(*lay));
  lay->num_entries = n;
  lay->num_tokens = static_cast<int32_t>(num_tokens);
  lay->num_multitoken = num_multi;
  lay->q_multi = static_cast<int32_t>(q_multi);
  lay->max_seqlen_q = max_q;
  lay->max_seqlen_k = max_k;
  lay->gather_len = static_cast<int32_t>(gather_len);
  lay->num_paged = n - num_multi;
  lay->table_rows = all_tables ? n : n - num_multi;
  lay->paged_row0 = all_tables ? num_multi : 0;
  lay->max_blocks_per_seq = max_blocks;
  lay->paged_max_context_len = paged_max_ctx;
  int64_t cur = 0;
  lay->tokens_off = place(&cur, num_tokens * 4);
  lay->positions_off = place(&cur, num_tokens * 8);
  lay->slot_mapping_off = place(&cur, num_tokens * 4);
  lay->logit_idxs_off = place(&cur, (int64_t)n * 4);
  lay->seqlens_q_off = place(&cur, (int64_t)(num_multi + 1) * 4);
  lay->seqlens_k_off = place(&cur, (int64_t)(num_multi + 1) * 4);
  lay->gather_mapping_off = place(&cur, gather_len * 4);
  lay->block_tables_off = place(&cur, (int64_t)lay->table_rows * max_blocks * 4);
  lay->context_lens_off = place(&cur, (int64_t)lay->table_rows * 4);
  lay->total_bytes = cur;
  return nullptr;
}

}  // namespace aici

using namespace aici;

extern "C" char *aici_batch_info_layout(const aici_batch_entry *entries, int num_entries, int flags,
                                        int block_size, int64_t max_model_len,
                                        aici_batch_layout *layout) {
  std::vector<int> order;
  return plan_batch("aici_batch_info_layout", entries, num_entries, flags, block_size,
                    max_model_len, layout, &order, true);
}

extern "C" char *aici_batch_info_build(const aici_batch_entry *entries, int num_entries, int flags,
                                       int block_size, int64_t max_model_len, void *staging,
                                       size_t staging_bytes, void *device_dst, size_t device_bytes,
                                       aici_batch_layout *layout, int32_t *entry_order,
                                       aici_stream_t stream) {
  const char *fn = "aici_batch_info_build";
  std::vector<int> order;
  if (char *e = plan_batch(fn, entries, num_entries, flags, block_size, max_model_len, layout, &order,
                           false))
    return e;
  const aici_batch_layout &lay = *layout;
  AICI_CHECK(staging != nullptr && staging_bytes >= (size_t)lay.total_bytes,
             "%s: staging buffer of %zu bytes is smaller than the %lld needed", fn, staging_bytes,
             (long long)lay.total_bytes);
  AICI_CHECK((uintptr_t)staging % 16 == 0, "%s: staging buffer must be 16-byte aligned", fn);
  AICI_CHECK(device_dst == nullptr ||
                 (device_bytes >= (size_t)lay.total_bytes && (uintptr_t)device_dst % 256 == 0),
             "%s: device buffer must be 256-byte aligned and hold %lld bytes (got %zu)", fn,
             (long long)lay.total_bytes, device_bytes);

  char *base = static_cast<char *>(staging);
  int32_t *tokens = reinterpret_cast<int32_t *>(base + lay.tokens_off);
  int64_t *positions = reinterpret_cast<int64_t *>(base + lay.positions_off);
  int32_t *slot_mapping = reinterpret_cast<int32_t *>(base + lay.slot_mapping_off);
  int32_t *logit_idxs = reinterpret_cast<int32_t *>(base + lay.logit_idxs_off);
  int32_t *seqlens_q = reinterpret_cast<int32_t *>(base + lay.seqlens_q_off);
  int32_t *seqlens_k = reinterpret_cast<int32_t *>(base + lay.seqlens_k_off);
  int32_t *gather_mapping = reinterpret_cast<int32_t *>(base + lay.gather_mapping_off);
  int32_t *block_tables = reinterpret_cast<int32_t *>(base + lay.block_tables_off);
  int32_t *context_lens = reinterpret_cast<int32_t *>(base + lay.context_lens_off);
  const bool all_tables = (flags & AICI_BATCH_TABLES_FOR_ALL) != 0;
  const bool gather = (flags & AICI_BATCH_NO_GATHER_MAP) == 0;

  if (lay.table_rows > 0 && lay.max_blocks_per_seq > 0)
    memset(block_tables, 0, (size_t)lay.table_rows * lay.max_blocks_per_seq * 4);

  int64_t tok = 0, g = 0;
  int32_t off_q = 0, off_k = 0;
  for (int idx = 0; idx < num_entries; ++idx) {
    const aici_batch_entry &e = entries[order[idx]];
    if (entry_order) entry_order[idx] = order[idx];
    const int first = e.k_len - e.q_len;  // index of the first query token in kv_slots
    for (int j = 0; j < e.q_len; ++j, ++tok) {
      positions[tok] = e.positions ? e.positions[j] : (int64_t)(first + j);
      tokens[tok] = e.tokens[j];
      slot_mapping[tok] = static_cast<int32_t>(e.kv_slots[first + j]);
    }
    logit_idxs[idx] = static_cast<int32_t>(tok - 1);
    const bool multi = idx < lay.num_multitoken;
    if (multi) {
      if (gather)
        for (int t = 0; t < e.k_len; ++t) gather_mapping[g++] = static_cast<int32_t>(e.kv_slots[t]);
      seqlens_q[idx] = off_q;
      seqlens_k[idx] = off_k;
      off_q += e.q_len;
      off_k += e.k_len;
    }
    if (!multi || all_tables) {
      const int row = multi ? idx : lay.paged_row0 + (idx - lay.num_multitoken);
      context_lens[row] = e.k_len;
      int32_t *table = block_tables + (size_t)row * lay.max_blocks_per_seq;
      for (int t = 0, b = 0; t < e.k_len; t += block_size, ++b) {
        const int64_t slot = e.kv_slots[t];
        AICI_CHECK(slot >= 0 && slot % block_size == 0 && slot / block_size <= INT32_MAX,
                   "%s: sequence %lld: slot %lld at token %d does not start a block of %d", fn,
                   (long long)e.seq_id, (long long)slot, t, block_size);
        table[b] = static_cast<int32_t>(slot / block_size);
      }
    }
  }
  seqlens_q[lay.num_multitoken] = off_q;
  seqlens_k[lay.num_multitoken] = off_k;

  if (device_dst != nullptr && lay.total_bytes > 0)
    AICI_CUDA(cudaMemcpyAsync(device_dst, staging, (size_t)lay.total_bytes, cudaMemcpyHostToDevice,
                              static_cast<cudaStream_t>(stream)));
  return nullptr;
}
