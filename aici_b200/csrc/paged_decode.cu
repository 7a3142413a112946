// Decode attention over the paged KV cache for sm_100a (one query token per sequence).
//
// Semantics follow rllm/tch-cuda/kernels/vllm/attention/attention_kernels.cu
// (paged_attention_kernel :85-392, v2 reduce :450-546): fp32 logits scale*q.k over
// t < context_len, softmax with the reference's +1e-6 in the denominator, fp32 accumulation
// of p*V, kv head = head / (num_heads / num_kv_heads).
//
// The traversal is new.  Every warp is an independent streaming agent that works through a list of
// pieces, a piece being some consecutive 16-token tiles of one (sequence, kv head) row:
//   * lane 0 issues 1-D bulk copies (cp.async.bulk, completion on an mbarrier) that bring
//     the 4 KB key tile and the 4 KB value tile of one 16-token cache block into the warp's
//     private shared-memory ring, kStages deep, running ahead across pieces;
//   * the warp multiplies the whole query-head group of that kv head against the tile with
//     bf16 mma.sync (q heads are the M rows, padded to 16), keeps an online softmax per row
//     in registers (warp shuffles for the row max/sum), and accumulates P*V in fp32;
//   * at the end of a piece it writes either the final row (the row had no other piece) or an
//     fp32 partial (max, sum, normalised output) that a merge kernel combines.
// So K/V are read from HBM exactly once per (sequence, kv head) regardless of the group
// size and every byte moves as a 4 KB contiguous burst.
// Two things a decode step needs besides attention can ride on these kernels: the cache write of the
// step's new tokens (aici_decode_step: the warp that reaches a row's last tile writes the token) and,
// with kv heads sharded over GPUs, the ranks' barrier (every CTA of the merge kernel reports to all
// ranks when its rows are stored, one CTA waits for all reports).
// Two ways of cutting the batch into pieces exist.  "Spans" (the default of the v1 entry): the
// tiles of the whole batch are laid end to end and every warp of the grid takes one run of the
// same length, so the load is even whatever the context lengths are (next_piece).  "Chunks": every
// row is cut into chunks of a fixed number of tokens that are dealt out round-robin (fetch_item);
// kept for the v2 calling convention, whose 512-token partitions are part of its output, for
// batches too large to plan inside the kernel, and behind the tuning hook.
#include "common.cuh"

namespace aici {

constexpr int kD = 128;
constexpr int kB = 16;
constexpr int kTileBytes = kD * kB * 2;     // 4096: one (block, kv head) key or value tile
constexpr int kStageBytes = 2 * kTileBytes; // key tile + value tile
constexpr int kWarps = 4;                   // warps per CTA, each with a private ring
constexpr int kStages = 3;                  // ring depth per warp
constexpr int kMaxChunk = 512;              // tokens; 32 tiles, one block id per lane
constexpr int kMaxInlineSeqs = 2048;        // batch size up to which each CTA plans for itself
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeParams {
  const __nv_bfloat16 *q;
  const __nv_bfloat16 *k_cache;
  const __nv_bfloat16 *v_cache;
  // output rows [num_seqs, out_heads, 128] in `world` buffers (this GPU's and, for the fused
  // gather, every peer's): this rank's heads start at out_head0
  __nv_bfloat16 *out[8];
  int world, out_heads, out_head0;
  const int32_t *block_tables;
  const int32_t *context_lens;
  const int2 *entries;   // compacted (seq, chunk) list, or NULL: every (seq, chunk < max_parts)
  const int *n_entries;  // device count for `entries`
  float *part_max;       // [num_seqs, num_heads, max_parts] natural-log-domain max logit
  float *part_sum;       // [num_seqs, num_heads, max_parts] sum of exp(logit - max)
  void *part_out;        // [num_seqs, num_heads, max_parts, 128] fp32 or bf16, normalised
  int num_seqs, num_heads, num_kv_heads, group;
  int max_blocks_per_seq;
  int max_context_len;
  int64_t num_blocks;
  int chunk_tokens;
  int max_parts;
  int always_write_partials;  // v2 calling convention: partials are an output too
  int inline_plan;            // 1: every CTA builds the chunk prefix sums itself (no plan kernel)
  int decode_warps;           // spans mode: warps of the decode grid (the merge kernel derives the span length from it)
  int *span_cum;              // spans mode, large merge grids: [num_seqs + 2] tile prefix sums, then the span length
  int early_sums;             // spans mode: 1 = the merge CTAs add the context lengths up themselves
  int min_span;               // spans mode: fewest tiles a warp takes
  int64_t q_stride, kv_block_stride, kv_head_stride;
  float scale_log2e;
  unsigned int *status;
  // fused cross-GPU barrier in the merge kernel's tail (sync != 0): rank p's flag array
  unsigned int *peer_flags[8];
  int sync, rank;
  // decode step (aici_decode_step): the step's new tokens, one per sequence, still outside the cache.
  // The warp that works on the last tile of a (sequence, kv head) row -- there is exactly one --
  // puts the token into the tile it has staged in shared memory and writes it to the cache.
  const __nv_bfloat16 *new_k;  // [num_seqs, num_kv_heads, 128], NULL = plain decode
  const __nv_bfloat16 *new_v;
  const void *new_slots;       // [num_seqs] int32 or int64; must name position context_len - 1
  int new_slot_is_int64;
  int64_t new_k_stride, new_v_stride;
};

struct Item {
  int seq, chunk, kvh, ctx, tok0, ntiles;
  int single;     // the (sequence, kv head) row has no other piece: write the final row
  int pstep;      // distance between the partials of consecutive heads of the group
  int64_t pbase;  // index of the partial of the group's first head
};

// Spans mode: position in the global tile order (sequence-major, then kv head, then tile) and the
// end of this warp's span.
struct Cursor {
  int x, end;
};

__device__ __forceinline__ int clamp_ctx(const DecodeParams &p, int ctx) {
  int lim = p.max_context_len;
  const int cap = p.max_blocks_per_seq * kB;
  if (cap < lim) lim = cap;
  if (ctx > lim) {
    set_status(p.status, AICI_STATUS_BAD_BLOCK);
    ctx = lim;
  }
  return ctx < 0 ? 0 : ctx;
}

// Decodes work item `idx`; ntiles == 0 marks an empty one (virtual grid only).
__device__ __forceinline__ void fetch_item(const DecodeParams &p, const int *s_cum, int idx, Item &it) {
  const int e = idx / p.num_kv_heads;
  it.kvh = idx - e * p.num_kv_heads;
  if (p.inline_plan) {
    // s_cum[i] = number of chunks of sequences < i (shared memory): the sequence is the last i
    // with s_cum[i] <= e
    int lo = 0, hi = p.num_seqs;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_cum[mid] <= e) lo = mid; else hi = mid;
    }
    it.seq = lo;
    it.chunk = e - s_cum[lo];
  } else if (p.entries != nullptr) {
    const int2 sc = p.entries[e];
    it.seq = sc.x;
    it.chunk = sc.y;
  } else {
    it.seq = e / p.max_parts;
    it.chunk = e - it.seq * p.max_parts;
  }
  it.ctx = clamp_ctx(p, p.context_lens[it.seq]);
  it.tok0 = it.chunk * p.chunk_tokens;
  int n = it.ctx - it.tok0;
  if (n > p.chunk_tokens) n = p.chunk_tokens;
  it.ntiles = n > 0 ? (n + kB - 1) / kB : 0;
  it.single = it.ctx <= p.chunk_tokens;
  it.pstep = p.max_parts;
  it.pbase = ((int64_t)it.seq * p.num_heads + it.kvh * p.group) * p.max_parts + it.chunk;
}

// Spans mode.  All tiles of the batch form one sequence: row (seq, kvh) starts at global tile
// num_kv_heads * cum[seq] + kvh * tiles(seq), cum = tile prefix sums over the batch (s_cum).
// Every warp owns `span` consecutive global tiles, so all warps carry the same load whatever the
// mix of context lengths; a span is cut into pieces at row ends.  The next piece starts at c.x and
// takes at most `cap` tiles; returns false at the end of the span.  Piece number
// x / span + row index is unique, below warps + rows, and consecutive within a row, which is how
// the merge kernel finds a row's partials without any list.
__device__ __forceinline__ bool next_piece(const DecodeParams &p, const int *s_cum, int span,
                                           Cursor &c, int cap, Item &it) {
  if (c.x >= c.end) return false;
  const int H = p.num_kv_heads;
  const int e = c.x / H;
  int lo = 0, hi = p.num_seqs;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_cum[mid] <= e) lo = mid; else hi = mid;
  }
  const int c0 = s_cum[lo], tiles = s_cum[lo + 1] - c0;
  const int rem = c.x - H * c0;
  const int kvh = rem / tiles, t0 = rem - kvh * tiles;
  int n = tiles - t0;
  if (n > c.end - c.x) n = c.end - c.x;
  if (n > cap) n = cap;
  it.seq = lo;
  it.chunk = 0;
  it.kvh = kvh;
  it.ctx = clamp_ctx(p, p.context_lens[lo]);
  it.tok0 = t0 * kB;
  it.ntiles = n;
  const int g0 = c.x - t0;
  it.single = (g0 + tiles - 1) / span == g0 / span;
  it.pstep = 1;
  it.pbase = (int64_t)(c.x / span + lo * H + kvh) * p.group;
  c.x += n;
  return true;
}

template <typename PartT>
__device__ __forceinline__ void store_pair(PartT *dst, float a, float b);
template <>
__device__ __forceinline__ void store_pair<float>(float *dst, float a, float b) {
  *reinterpret_cast<float2 *>(dst) = make_float2(a, b);
}
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16 *dst, float a, float b) {
  *reinterpret_cast<__nv_bfloat162 *>(dst) = __floats2bfloat162_rn(a, b);
}

template <typename PartT, bool kSpans>
__global__ void __launch_bounds__(kWarps * 32, 2) paged_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  uint8_t *ring = smem + warp * (kStages * kStageBytes);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + kWarps * kStages * kStageBytes) + warp * kStages;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncwarp();

  // Programmatic dependent launch: wait for the grid before this one (its writes -- context
  // lengths, the chunk list of the plan kernel, anything else -- are visible from here on), then let
  // the merge grid get resident.  In this order the merge grid, which reads the context lengths
  // before its own wait, cannot start while a producer of those lengths is still running.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  int *s_cum = reinterpret_cast<int *>(smem + kWarps * kStages * kStageBytes + kWarps * kStages * sizeof(uint64_t));
  if (p.inline_plan) {
    // chunk-count prefix sums over the batch, built by every CTA for itself: all threads fetch
    // the context lengths at once (one global-memory latency for the whole batch), then warp 0
    // scans the counts in shared memory
    for (int seq = threadIdx.x; seq < p.num_seqs; seq += kWarps * 32)
      s_cum[seq + 1] = (clamp_ctx(p, p.context_lens[seq]) + p.chunk_tokens - 1) / p.chunk_tokens;
    __syncthreads();
    if (warp == 0) {
      int carry = 0;
      for (int s0 = 0; s0 < p.num_seqs; s0 += 32) {
        const int seq = s0 + lane;
        const int cnt = seq < p.num_seqs ? s_cum[seq + 1] : 0;
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        __syncwarp();
        if (seq < p.num_seqs) s_cum[seq + 1] = carry + incl;
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) s_cum[0] = 0;
    }
    __syncthreads();
  }
  const int n_entries = p.inline_plan ? s_cum[p.num_seqs]
                                      : (p.entries != nullptr ? *p.n_entries : p.num_seqs * p.max_parts);
  const int n_items = n_entries * p.num_kv_heads;
  const int stride = gridDim.x * kWarps;
  const int gw = blockIdx.x * kWarps + warp;
  // spans mode: n_items is the number of tiles of the whole batch (chunk_tokens == 16)
  int span = 1;
  Cursor p_cur = {0, 0}, c_cur = {0, 0};
  if (kSpans) {
    span = (n_items + stride - 1) / stride;
    if (span < p.min_span) span = p.min_span;
    const int64_t x0 = (int64_t)gw * span;
    p_cur.x = c_cur.x = x0 < n_items ? (int)x0 : n_items;
    p_cur.end = c_cur.end = x0 + span < n_items ? (int)(x0 + span) : n_items;
    if (!p.early_sums && blockIdx.x == 0 && warp == 0) {  // what a large merge grid needs to find the pieces of a row
      for (int i = lane; i <= p.num_seqs; i += 32) p.span_cum[i] = s_cum[i];
      if (lane == 0) p.span_cum[p.num_seqs + 1] = span;
    }
  }

  // ---- producer cursor ---------------------------------------------------------------
  int p_idx = gw - stride;
  Item p_item;
  p_item.ntiles = 0;
  p_item.kvh = 0;
  int p_tile = 0, p_blk = 0;
  unsigned p_count = 0;
  bool p_done = false;

  auto produce_one = [&]() {
    if (p_done) return;
    if (p_tile == p_item.ntiles) {
      if (kSpans) {
        if (!next_piece(p, s_cum, span, p_cur, 32, p_item)) {  // 32 tiles: one block id per lane
          p_done = true;
          return;
        }
      } else {
        do {
          p_idx += stride;
          if (p_idx >= n_items) {
            p_done = true;
            return;
          }
          fetch_item(p, s_cum, p_idx, p_item);
        } while (p_item.ntiles == 0);
      }
      int b = 0;
      if (lane < p_item.ntiles) {
        b = p.block_tables[(int64_t)p_item.seq * p.max_blocks_per_seq + p_item.tok0 / kB + lane];
        if (b < 0 || b >= p.num_blocks) {
          set_status(p.status, AICI_STATUS_BAD_BLOCK);
          b = 0;
        }
      }
      p_blk = b;
      p_tile = 0;
    }
    const int blk = __shfl_sync(0xffffffffu, p_blk, p_tile);
    if (lane == 0) {
      const unsigned stage = p_count % kStages;
      uint8_t *dst = ring + stage * kStageBytes;
      const int64_t off = (int64_t)blk * p.kv_block_stride + (int64_t)p_item.kvh * p.kv_head_stride;
      fence_proxy_async_smem();  // order this warp's earlier reads of the stage before the refill
      mbar_expect_tx(&full[stage], kStageBytes);
      bulk_g2s(dst, p.k_cache + off, kTileBytes, &full[stage]);
      bulk_g2s(dst + kTileBytes, p.v_cache + off, kTileBytes, &full[stage]);
    }
    ++p_tile;
    ++p_count;
  };

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) produce_one();

  // ldmatrix lane offsets: lane -> (matrix mi = lane / 8, row = lane % 8)
  const int mi = lane >> 3, mr = lane & 7;
  // key tile [c = d/8][tok][8]: matrices (c even, tok 0-7), (c odd, tok 0-7), (c even, tok 8-15), (c odd, tok 8-15)
  const uint32_t k_lane_off = (((mi & 1) * kB) + 8 * (mi >> 1) + mr) * 16;
  // value tile [d][tok]: matrices (d 0-7, tok 0-7), (d 0-7, tok 8-15), (d 8-15, tok 0-7), (d 8-15, tok 8-15)
  const uint32_t v_lane_off = (8 * (mi >> 1) + mr) * 32 + (mi & 1) * 16;

  unsigned c_count = 0;
  int c_idx = gw - stride;
  bool failed = false;

  while (!failed) {
    Item it;
    if (kSpans) {
      if (!next_piece(p, s_cum, span, c_cur, 0x7fffffff, it)) break;
    } else {
      do {
        c_idx += stride;
        if (c_idx >= n_items) break;
        fetch_item(p, s_cum, c_idx, it);
      } while (it.ntiles == 0);
      if (c_idx >= n_items) break;
    }

    // query fragments: rows = heads of this kv head's group (rows >= group are zero)
    uint32_t qa[8][2];
    {
      const __nv_bfloat16 *qrow =
          p.q + (int64_t)it.seq * p.q_stride + (int64_t)(it.kvh * p.group + g) * kD + 2 * tig;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        if (g < p.group) {
          qa[ks][0] = *reinterpret_cast<const uint32_t *>(qrow + 16 * ks);
          qa[ks][1] = *reinterpret_cast<const uint32_t *>(qrow + 16 * ks + 8);
        } else {
          qa[ks][0] = 0u;
          qa[ks][1] = 0u;
        }
      }
    }

    float o[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    for (int t = 0; t < it.ntiles; ++t) {
      produce_one();
      const unsigned stage = c_count % kStages;
      if (!__all_sync(0xffffffffu, mbar_wait(&full[stage], (c_count / kStages) & 1u, p.status))) {
        failed = true;
        break;
      }
      const uint32_t kbase = smem_u32(ring + stage * kStageBytes);
      const uint32_t vbase = kbase + kTileBytes;

      if (p.new_k != nullptr && it.tok0 + (t + 1) * kB >= it.ctx) {
        // The tile that ends the row holds position ctx - 1, the token of this step, which is not
        // in the cache yet: take it from the step's inputs, put it into the staged tile, and write it
        // to the cache (what reshape_and_cache would have done before this kernel).  No other warp
        // reads this tile, and this warp's own copy of it has landed, so nothing races.
        const int pos = it.ctx - 1 - (it.tok0 + t * kB);
        const int64_t slot = p.new_slot_is_int64 ? static_cast<const int64_t *>(p.new_slots)[it.seq]
                                                  : (int64_t) static_cast<const int32_t *>(p.new_slots)[it.seq];
        int blk = p.block_tables[(int64_t)it.seq * p.max_blocks_per_seq + (it.ctx - 1) / kB];
        if (blk < 0 || blk >= p.num_blocks) blk = 0;  // recorded by the producer when it fetched the id
        if (slot == (int64_t)blk * kB + pos) {
          uint8_t *ktile = ring + stage * kStageBytes;
          uint8_t *vtile = ktile + kTileBytes;
          const int64_t coff = (int64_t)blk * p.kv_block_stride + (int64_t)it.kvh * p.kv_head_stride;
          // (Measured: writing whole 32-byte sectors or whole lines of the patched tile back instead
          // of these 2-byte pieces is not faster.  What the write costs -- about 13 us at 64 sequences
          // x 32 heads, wherever it is issued from -- is the later write-back of its 98 000 dirty
          // lines, one read/write turn-around of a memory channel each, in the middle of the key/value
          // stream; the reference's value layout [d][token] puts one token into every sector of a tile.)
          if (lane < kD / 8) {  // key: chunk `lane` (8 elements) -> [chunk][pos][0..7]
            const uint4 kv = *reinterpret_cast<const uint4 *>(p.new_k + (int64_t)it.seq * p.new_k_stride +
                                                              it.kvh * kD + lane * 8);
            *reinterpret_cast<uint4 *>(ktile + (lane * kB + pos) * 16) = kv;
            *reinterpret_cast<uint4 *>(const_cast<__nv_bfloat16 *>(p.k_cache) + coff + (lane * kB + pos) * 8) = kv;
          }
          const uint2 raw = *reinterpret_cast<const uint2 *>(p.new_v + (int64_t)it.seq * p.new_v_stride +
                                                             it.kvh * kD + lane * 4);
          const uint16_t e[4] = {(uint16_t)(raw.x & 0xffffu), (uint16_t)(raw.x >> 16), (uint16_t)(raw.y & 0xffffu),
                                 (uint16_t)(raw.y >> 16)};
          uint16_t *vg = reinterpret_cast<uint16_t *>(const_cast<__nv_bfloat16 *>(p.v_cache) + coff);
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // value: element d = 4 lane + j -> [d][pos]
            const int d = lane * 4 + j;
            *reinterpret_cast<uint16_t *>(vtile + d * (kB * 2) + pos * 2) = e[j];
            vg[d * kB + pos] = e[j];
          }
        } else if (slot >= 0 && lane == 0) {
          set_status(p.status, AICI_STATUS_BAD_SLOT);  // not the sequence's last position: not written
        }
        __syncwarp();
      }

      // ---- S = Q K^T (16 x 16) -------------------------------------------------------
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t b00, b01, b10, b11;
        ldmatrix_x4(b00, b01, b10, b11, kbase + ks * (2 * kB * 16) + k_lane_off);
        mma_bf16_16816(s0, qa[ks][0], 0u, qa[ks][1], 0u, b00, b01);
        mma_bf16_16816(s1, qa[ks][0], 0u, qa[ks][1], 0u, b10, b11);
      }

      // ---- online softmax for row g (scores in log2 units) ----------------------------
      const int tok_base = it.tok0 + t * kB;
      const bool last = tok_base + kB > it.ctx;
      float x00 = s0[0] * p.scale_log2e, x01 = s0[1] * p.scale_log2e;
      float x10 = s1[0] * p.scale_log2e, x11 = s1[1] * p.scale_log2e;
      uint32_t vm_lo = 0xffffffffu, vm_hi = 0xffffffffu;
      if (last) {
        const int c0 = tok_base + 2 * tig;
        if (c0 >= it.ctx) { x00 = -INFINITY; vm_lo &= 0xffff0000u; }
        if (c0 + 1 >= it.ctx) { x01 = -INFINITY; vm_lo &= 0x0000ffffu; }
        if (c0 + 8 >= it.ctx) { x10 = -INFINITY; vm_hi &= 0xffff0000u; }
        if (c0 + 9 >= it.ctx) { x11 = -INFINITY; vm_hi &= 0x0000ffffu; }
      }
      float mt = fmaxf(fmaxf(x00, x01), fmaxf(x10, x11));
      mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
      mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
      const float m_new = fmaxf(m_run, mt);
      if (!__all_sync(0xffffffffu, m_new == m_run)) {
        const float alpha = fast_exp2(m_run - m_new);  // 0 on the first tile
        l_run *= alpha;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          o[nt][0] *= alpha;
          o[nt][1] *= alpha;
        }
        m_run = m_new;
      }
      const float p00 = fast_exp2(x00 - m_run), p01 = fast_exp2(x01 - m_run);
      const float p10 = fast_exp2(x10 - m_run), p11 = fast_exp2(x11 - m_run);
      l_run += (p00 + p01) + (p10 + p11);
      const uint32_t pa0 = pack_bf16(p00, p01), pa2 = pack_bf16(p10, p11);

      // ---- O += P V (16 x 128) ---------------------------------------------------------
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t v00, v01, v10, v11;
        ldmatrix_x4(v00, v01, v10, v11, vbase + np * (16 * 32) + v_lane_off);
        if (last) {  // cache slots past the context may hold anything, NaN included
          v00 &= vm_lo; v10 &= vm_lo;
          v01 &= vm_hi; v11 &= vm_hi;
        }
        mma_bf16_16816(o[2 * np], pa0, 0u, pa2, 0u, v00, v01);
        mma_bf16_16816(o[2 * np + 1], pa0, 0u, pa2, 0u, v10, v11);
      }
      __syncwarp();
      ++c_count;
    }
    if (failed) break;

    // ---- chunk epilogue ----------------------------------------------------------------
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < p.group) {
      const int head = it.kvh * p.group + g;
      const float inv = __fdividef(1.f, l_run + 1e-6f);
      if (it.single) {
        const int64_t off = ((int64_t)it.seq * p.out_heads + p.out_head0 + head) * kD + 2 * tig;
        for (int w = 0; w < p.world; ++w) {
          __nv_bfloat16 *dst = p.out[w] + off;
#pragma unroll
          for (int nt = 0; nt < 16; ++nt)
            store_pair<__nv_bfloat16>(dst + 8 * nt, o[nt][0] * inv, o[nt][1] * inv);
        }
      }
      if (!it.single || p.always_write_partials) {
        const int64_t pidx = it.pbase + (int64_t)g * it.pstep;
        if (tig == 0) {
          p.part_max[pidx] = m_run * kLn2;
          p.part_sum[pidx] = l_run;
        }
        PartT *dst = static_cast<PartT *>(p.part_out) + pidx * kD + 2 * tig;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) store_pair<PartT>(dst + 8 * nt, o[nt][0] * inv, o[nt][1] * inv);
      }
    }
  }

  if (failed) {
    // give copies already in flight a bounded chance to land before the ring is released
    for (unsigned c = c_count; c != p_count; ++c)
      mbar_wait(&full[c % kStages], (c / kStages) & 1u, p.status);
  }
}

// Combines the partials of one (sequence, head): v2 reduce of the reference
// (attention_kernels.cu:450-546).  A team of kTeam warps works on one row: every warp finds the
// global maximum, then takes every kTeam-th partial -- one weight per lane, handed round by
// shuffle, so the 512-byte row loads of a warp are independent -- and the team's sums meet in
// shared memory.  Lane l owns d = 4l .. 4l+3.  kTeam = 8 (one row per CTA) suits rows with many
// partials; kTeam = 1 (eight rows per CTA) suits the spans mode with large batches, where a row
// has two or three; 2 and 4 lie between (launch_decode picks).  In spans mode the partials of a row
// are consecutive pieces (see next_piece).
constexpr int kMergeWarps = 8;
template <typename PartT, bool kSpans, int kTeam>
__global__ void __launch_bounds__(kMergeWarps * 32) paged_merge_kernel(const DecodeParams p) {
  // a grid launched as a programmatic dependent of this one (the next step's cache write, the next
  // decode call) may become resident now; it waits for this grid before it touches anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kRows = kMergeWarps / kTeam;
  __shared__ float s_acc[kMergeWarps][kD];
  __shared__ float s_w[kMergeWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int team = warp / kTeam, tw = warp - team * kTeam;
  const int row = blockIdx.x * kRows + team;
  const bool active = row < p.num_seqs * p.num_heads;
  const int seq = active ? row / p.num_heads : 0, head = active ? row - seq * p.num_heads : 0;
  // Spans mode: where the pieces of a row lie follows from the context lengths alone (tiles before
  // its sequence, tiles of its sequence, tiles of the batch).  The lengths are an input of the call,
  // complete before the decode grid let this grid in, so a CTA that is resident beside the decode
  // grid adds them up while that grid still runs (one warp, once per length).  The host asks for
  // this only when the whole merge grid fits beside the decode grid; the CTAs of a larger grid
  // start after it and are better served by three loads of what decode CTA 0 left in the workspace.
  int c0 = 0, tiles = 0, total = 0;
  if (kSpans && p.early_sums) {
    __shared__ int s_pre[2 + kRows];  // tiles of the batch, tiles before the CTA's first sequence, tiles of its sequences
    const int row_first = blockIdx.x * kRows;
    const int seq_first = min(row_first / p.num_heads, p.num_seqs - 1);
    if (warp == 0) {
      int before = 0, all = 0;
      for (int s0 = lane; s0 < p.num_seqs; s0 += 32) {
        const int t = (clamp_ctx(p, p.context_lens[s0]) + kB - 1) / kB;
        all += t;
        if (s0 < seq_first) before += t;
        if (s0 >= seq_first && s0 < seq_first + kRows) s_pre[2 + s0 - seq_first] = t;
      }
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) {
        all += __shfl_xor_sync(0xffffffffu, all, o);
        before += __shfl_xor_sync(0xffffffffu, before, o);
      }
      if (lane == 0) {
        s_pre[0] = all;
        s_pre[1] = before;
      }
    }
    __syncthreads();
    total = s_pre[0];
    c0 = s_pre[1];
    for (int s0 = seq_first; s0 < seq; ++s0) c0 += s_pre[2 + s0 - seq_first];  // at most kRows - 1 terms
    tiles = active ? s_pre[2 + seq - seq_first] : 0;
  }
  int n = 0, pstride = 1;
  int64_t base = 0;
  // spans mode: the partials of the row are `n` consecutive pieces from `base` on, `group` apart
  auto locate = [&](int span) {
    if (tiles <= 0) return;
    const int kvh = head / p.group;
    const int g0 = p.num_kv_heads * c0 + kvh * tiles;
    const int first = g0 / span;
    n = (g0 + tiles - 1) / span - first + 1;
    base = (int64_t)(first + seq * p.num_kv_heads + kvh) * p.group + (head - kvh * p.group);
    pstride = p.group;
  };
  if (kSpans && p.early_sums && active) {  // everything but the partials themselves is known before the wait
    const int64_t n_items = (int64_t)total * p.num_kv_heads;
    int span = (int)((n_items + p.decode_warps - 1) / p.decode_warps);
    if (span < p.min_span) span = p.min_span;
    locate(span);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");  // no-op unless launched as a dependent grid
  if (active) {
    if (kSpans) {
      if (!p.early_sums) {
        c0 = p.span_cum[seq];
        tiles = p.span_cum[seq + 1] - c0;
        locate(p.span_cum[p.num_seqs + 1]);
      }
    } else {
      const int ctx = clamp_ctx(p, p.context_lens[seq]);
      n = (ctx + p.chunk_tokens - 1) / p.chunk_tokens;
      base = (int64_t)row * p.max_parts;
    }
  }
  const int64_t out_off = ((int64_t)seq * p.out_heads + p.out_head0 + head) * kD + 4 * lane;
  if (active && n <= 0 && tw == 0)  // empty context: the decode kernel never saw this row
    for (int w = 0; w < p.world; ++w) *reinterpret_cast<uint2 *>(p.out[w] + out_off) = make_uint2(0u, 0u);
  const bool work = active && n > 1;  // n == 1: the decode kernel wrote the row itself
  float wsum = 0.f, a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (work) {
    const PartT *po = static_cast<const PartT *>(p.part_out) + base * kD + 4 * lane;
    auto load_row = [&](int64_t j) {  // lane's four values of partial j of this row
      if (sizeof(PartT) == 4) return *reinterpret_cast<const float4 *>(po + j * pstride * kD);
      const uint2 raw = *reinterpret_cast<const uint2 *>(po + j * pstride * kD);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
      return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
    };
    // Everything the first batch needs is asked for at once -- the maxima of all partials, the
    // maximum and sum of the partials this lane weighs, and the first rows themselves -- so that a
    // row with a handful of partials costs one trip to memory, not one per step of the formula.
    constexpr int kAhead = kTeam == 1 ? 4 : 2;  // more would cost registers, and with them resident CTAs
    const int cnt0 = tw < n ? min(32, (n - tw + kTeam - 1) / kTeam) : 0;
    float m = -INFINITY;
    for (int j = lane; j < n; j += 32) m = fmaxf(m, p.part_max[base + (int64_t)j * pstride]);
    float pm = 0.f, ps = 0.f;
    if (lane < cnt0) {
      const int64_t j = base + (int64_t)(tw + kTeam * lane) * pstride;
      pm = p.part_max[j];
      ps = p.part_sum[j];
    }
    float4 ahead[kAhead];
#pragma unroll
    for (int l = 0; l < kAhead; ++l)
      ahead[l] = l < cnt0 ? load_row(tw + kTeam * l) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // this warp's partials: tw, tw + kTeam, ...; lane l prepares the weight of partial tw + kTeam l
    for (int j0 = tw; j0 < n; j0 += kTeam * 32) {
      const int cnt = min(32, (n - j0 + kTeam - 1) / kTeam);
      float w_lane = 0.f;
      if (j0 == tw) {
        if (lane < cnt) w_lane = ps * __expf(pm - m);
      } else if (lane < cnt) {
        const int64_t j = base + (int64_t)(j0 + kTeam * lane) * pstride;
        w_lane = p.part_sum[j] * __expf(p.part_max[j] - m);
      }
      int l = 0;
      if (j0 == tw) {
#pragma unroll
        for (; l < kAhead; ++l) {
          if (l < cnt) {
            const float w = __shfl_sync(0xffffffffu, w_lane, l);
            wsum += w;
            a0 += w * ahead[l].x; a1 += w * ahead[l].y; a2 += w * ahead[l].z; a3 += w * ahead[l].w;
          }
        }
      }
#pragma unroll 4
      for (; l < cnt; ++l) {
        const float w = __shfl_sync(0xffffffffu, w_lane, l);
        const float4 v = load_row(j0 + kTeam * l);
        wsum += w;
        a0 += w * v.x; a1 += w * v.y; a2 += w * v.z; a3 += w * v.w;
      }
    }
  }
  if (kTeam > 1) {
    *reinterpret_cast<float4 *>(&s_acc[warp][4 * lane]) = make_float4(a0, a1, a2, a3);
    if (lane == 0) s_w[warp] = wsum;
    __syncthreads();
    if (tw == 0) {
      a0 = a1 = a2 = a3 = wsum = 0.f;
#pragma unroll
      for (int w = 0; w < kTeam; ++w) {
        const float4 v = *reinterpret_cast<const float4 *>(&s_acc[team * kTeam + w][4 * lane]);
        a0 += v.x; a1 += v.y; a2 += v.z; a3 += v.w;
        wsum += s_w[team * kTeam + w];
      }
    }
  }
  if (work && tw == 0) {
    const float inv = __fdividef(1.f, wsum + 1e-6f);
    const uint2 packed = make_uint2(pack_bf16(a0 * inv, a1 * inv), pack_bf16(a2 * inv, a3 * inv));
    for (int w = 0; w < p.world; ++w) *reinterpret_cast<uint2 *>(p.out[w] + out_off) = packed;
  }
  if (p.sync) {
    // Fused head-gather barrier.  Every CTA, once its rows are stored, tells every rank so itself:
    // a system-scope fence (the rows are in the peers' memory) and one relaxed add per rank into
    // slot 16 + rank of that rank's flag array.  The CTAs of a grid add up to exactly 2^20 per call
    // whatever the grid size, so after k such calls a rank has 2^20 k from every peer that has
    // finished (counters wrap; differences are compared).  CTA 0 is the one that waits: lane p of
    // its first warp until slot 16 + p of this rank's own array has reached this call's target,
    // bounded to about a second.  The count of calls lives in slot 10 of the rank's own array, so a
    // launch can be replayed.  No CTA waits for another CTA of its own grid through memory of this
    // GPU first, which is what made the former count-then-signal version a round trip longer.
    __syncthreads();
    if (threadIdx.x < p.world) {
      const unsigned int lo = (unsigned int)(((uint64_t)blockIdx.x << 20) / gridDim.x);
      const unsigned int hi = (unsigned int)(((uint64_t)(blockIdx.x + 1) << 20) / gridDim.x);
      // release: the rows are performed at system scope before the add.  Cumulative: covers the
      // stores of the whole CTA (ordered by the barrier above).  An acquire-release fence is enough
      // for that; the sequentially consistent __threadfence_system() is not needed.
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.peer_flags[threadIdx.x] + 16 + p.rank),
                   "r"(hi - lo)
                   : "memory");
    }
    if (blockIdx.x == 0 && threadIdx.x < 32) {
      unsigned int *mine = p.peer_flags[p.rank];
      const unsigned int calls = mine[10] + 1;
      if (lane < p.world) peer_wait_count(mine + 16 + lane, calls << 20, p.status);
      __syncwarp();
      if (lane == 0) mine[10] = calls;
    }
  }
}

// Builds the compact (seq, chunk) list so that every warp of the decode kernel gets the same
// number of non-empty chunks.  One CTA; order = sequences ascending, chunks ascending.
__global__ void __launch_bounds__(1024) paged_plan_kernel(const DecodeParams p, int2 *entries,
                                                          int *n_entries) {
  __shared__ int s_warp[32];
  __shared__ int s_base;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int s0 = 0; s0 < p.num_seqs; s0 += 1024) {
    const int seq = s0 + tid;
    int cnt = 0;
    if (seq < p.num_seqs) {
      const int ctx = clamp_ctx(p, p.context_lens[seq]);
      cnt = (ctx + p.chunk_tokens - 1) / p.chunk_tokens;
    }
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += v;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    const int base = s_base + (warp > 0 ? s_warp[warp - 1] : 0) + incl - cnt;
    for (int c = 0; c < cnt; ++c) entries[base + c] = make_int2(seq, c);
    __syncthreads();
    if (tid == 0) s_base += s_warp[31];
    __syncthreads();
  }
  if (tid == 0) *n_entries = s_base;
}

// ---- host side -------------------------------------------------------------------------------
// Tokens per work item of the fixed-chunk traversal (used by aici_paged_attention_v1_chunked when it
// is given no chunk size, for batches too large to plan inside the kernel, and -- with 512 -- for
// the v2 calling convention).
// 256 (16 cache blocks, 128 KB of K+V) keeps the partial-result traffic near 1 %; with few
// (sequence, kv head) pairs per GPU coarse items leave some warps with one item more than
// others, so the chunk is halved until the upper bound of the item count reaches 16 per resident
// warp, down to 64 tokens.
static int pick_chunk(int num_seqs, int num_kv_heads, int max_context_len) {
  const int64_t warps = (int64_t)2 * sm_count() * kWarps;
  int chunk = 256;
  while (chunk > 64 &&
         (int64_t)num_seqs * ((max_context_len + chunk - 1) / chunk) * num_kv_heads < 16 * warps)
    chunk >>= 1;
  return chunk;
}

// The default traversal gives every warp one span of consecutive tiles (see next_piece); it needs
// the in-kernel plan, hence the batch limit, and 32-bit tile indices.
constexpr int kMinSpanTiles = 4;
static bool use_spans(int num_seqs, int num_kv_heads, int max_context_len) {
  return num_seqs <= kMaxInlineSeqs &&
         (int64_t)num_seqs * num_kv_heads * ((max_context_len + kB - 1) / kB + 1) < (1ll << 30);
}

constexpr size_t kAlign = 256;
static size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct WorkspaceLayout {
  size_t n_entries_off, entries_off, max_off, sum_off, out_off, total;
  int max_parts;
};

static WorkspaceLayout workspace_layout(int num_seqs, int num_heads, int max_context_len,
                                        int chunk) {
  WorkspaceLayout w;
  w.max_parts = max_context_len > 0 ? (max_context_len + chunk - 1) / chunk : 1;
  const size_t parts = (size_t)num_seqs * w.max_parts;
  w.n_entries_off = 0;
  w.entries_off = kAlign;
  w.max_off = w.entries_off + align_up(parts * sizeof(int2));
  w.sum_off = w.max_off + align_up(parts * num_heads * sizeof(float));
  w.out_off = w.sum_off + align_up(parts * num_heads * sizeof(float));
  w.total = w.out_off + align_up(parts * num_heads * kD * sizeof(float));
  return w;
}

// Spans mode: tile prefix sums for the merge kernel (used by large merge grids), then one partial
// per piece and group head; pieces are fewer than warps + rows whatever the context lengths are.
static WorkspaceLayout spans_layout(int num_seqs, int num_heads, int num_kv_heads) {
  WorkspaceLayout w;
  const size_t pieces = (size_t)2 * sm_count() * kWarps + (size_t)num_seqs * num_kv_heads;
  const size_t parts = pieces * (num_heads / num_kv_heads);
  w.max_parts = 1;
  w.n_entries_off = 0;
  w.entries_off = kAlign;  // the prefix sums live where the chunk list would
  w.max_off = w.entries_off + align_up((size_t)(num_seqs + 2) * sizeof(int));
  w.sum_off = w.max_off + align_up(parts * sizeof(float));
  w.out_off = w.sum_off + align_up(parts * sizeof(float));
  w.total = w.out_off + align_up(parts * kD * sizeof(float));
  return w;
}

static char *check_decode_args(const char *fn, const void *out, const void *query,
                               const void *key_cache, const void *value_cache, int num_kv_heads,
                               const int32_t *block_tables, const int32_t *context_lens,
                               int block_size, int max_context_len, const float *alibi_slopes,
                               int num_seqs, int num_heads, int head_size,
                               int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride,
                               int64_t kv_block_stride, int64_t kv_head_stride, int dtype) {
  AICI_CHECK(dtype == AICI_DTYPE_BF16, "%s: only bf16 is supported (dtype=%d)", fn, dtype);
  AICI_CHECK(head_size == kD, "%s: Unsupported head size: %d", fn, head_size);
  AICI_CHECK(block_size == kB, "%s: Unsupported block size: %d", fn, block_size);
  AICI_CHECK(alibi_slopes == nullptr, "%s: alibi_slopes is not supported", fn);
  AICI_CHECK(num_seqs >= 0 && num_heads > 0 && num_kv_heads > 0, "%s: bad sizes", fn);
  AICI_CHECK(num_heads % num_kv_heads == 0, "%s: num_heads %d not divisible by num_kv_heads %d",
             fn, num_heads, num_kv_heads);
  const int group = num_heads / num_kv_heads;
  AICI_CHECK(group == 1 || group == 2 || group == 4 || group == 8,
             "%s: num_heads / num_kv_heads must be 1, 2, 4 or 8 (got %d)", fn, group);
  if (num_seqs == 0) return nullptr;
  AICI_CHECK(out && query && key_cache && value_cache && block_tables && context_lens,
             "%s: NULL pointer", fn);
  AICI_CHECK(max_context_len >= 0 && max_num_blocks_per_seq >= 0, "%s: negative size", fn);
  AICI_CHECK(num_blocks > 0, "%s: num_blocks must be positive", fn);
  AICI_CHECK(q_stride % 8 == 0 && q_stride >= (int64_t)num_heads * kD,
             "%s: q_stride must be a multiple of 8 and cover one row", fn);
  AICI_CHECK(kv_head_stride == kD * kB && kv_block_stride % 8 == 0 &&
                 kv_block_stride >= (int64_t)num_kv_heads * kD * kB,
             "%s: cache must be [blocks, kv_heads, 128/8, 16, 8] with contiguous head tiles", fn);
  AICI_CHECK(((uintptr_t)out | (uintptr_t)query | (uintptr_t)key_cache |
              (uintptr_t)value_cache) % 16 == 0,
             "%s: tensors must be 16-byte aligned", fn);
  AICI_CHECK((int64_t)num_seqs * ((max_context_len + 127) / 128 + 1) * num_kv_heads < (1ll << 30),
             "%s: problem too large for 32-bit work indices", fn);
  return nullptr;
}

template <typename PartT, bool kSpans>
static char *launch_decode(DecodeParams &p, int2 *entries, int *n_entries, cudaStream_t stream) {
  const int smem = kWarps * kStages * kStageBytes + kWarps * kStages * (int)sizeof(uint64_t) +
                   (kMaxInlineSeqs + 1) * (int)sizeof(int);
  static OncePerDevice once;
  if (char *e = once.run([&]() -> char * {
        AICI_CUDA(cudaFuncSetAttribute(paged_decode_kernel<PartT, kSpans>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        // An SM changes its shared-memory / L1 split only when it is empty.  The merge kernel needs
        // 4 KB of shared memory and would get a small carve-out by default, so its CTAs could not
        // join an SM that still runs decode CTAs (or the other way round at the next call) and the
        // programmatic launch would overlap nothing.  Asking for the largest carve-out keeps every
        // kernel of a decode step on one SM configuration.
        AICI_CUDA(cudaFuncSetAttribute(paged_merge_kernel<PartT, kSpans, 1>,
                                       cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        AICI_CUDA(cudaFuncSetAttribute(paged_merge_kernel<PartT, kSpans, 2>,
                                       cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        AICI_CUDA(cudaFuncSetAttribute(paged_merge_kernel<PartT, kSpans, 4>,
                                       cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        AICI_CUDA(cudaFuncSetAttribute(paged_merge_kernel<PartT, kSpans, kMergeWarps>,
                                       cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        return nullptr;
      }))
    return e;
  int grid = 2 * sm_count();
  if (kSpans) {
    p.inline_plan = 1;
    p.entries = nullptr;
    p.n_entries = nullptr;
    const int64_t ub_tiles = (int64_t)p.num_seqs * p.num_kv_heads * ((p.max_context_len + kB - 1) / kB);
    const int64_t need = (ub_tiles + (int64_t)kWarps * kMinSpanTiles - 1) / (kWarps * kMinSpanTiles);
    if (need < grid) grid = (int)need;
  } else {
    // small and medium batches: every CTA plans for itself; very large ones: a plan kernel writes
    // the compact chunk list into the workspace (v2 convention, no workspace: virtual grid)
    p.inline_plan = (entries != nullptr && p.num_seqs <= kMaxInlineSeqs) ? 1 : 0;
    if (entries != nullptr && !p.inline_plan) {
      paged_plan_kernel<<<1, 1024, 0, stream>>>(p, entries, n_entries);
      AICI_CUDA(cudaGetLastError());
    }
    p.entries = p.inline_plan ? nullptr : entries;
    p.n_entries = n_entries;
    const int64_t ub_items = (int64_t)p.num_seqs * p.max_parts * p.num_kv_heads;
    const int64_t need = (ub_items + kWarps - 1) / kWarps;
    if (need < grid) grid = (int)need;
  }
  if (grid < 1) grid = 1;
  // decode and merge are launched as programmatic dependents: their prologues overlap the tail of
  // the grid before them, and each waits (griddepcontrol.wait) before touching its inputs
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  const int rows = p.num_seqs * p.num_heads;
  // How many warps share a row.  Many (sequence, kv head) rows per warp of the decode grid: a row
  // has few partials and one warp merges it.  Fewer rows have more partials each and 2, 4 or 8 warps
  // share a row -- as many as keep the grid within one CTA per SM where that is possible: one
  // merge CTA fits an SM beside the decode grid's two (registers), and a CTA that is resident while
  // the decode grid runs has everything but the partials ready when that grid ends.
  int team = kMergeWarps;
  if (kSpans && (int64_t)p.num_seqs * p.num_kv_heads * 4 >= (int64_t)grid * kWarps) team = 1;
  else if (kSpans && rows > 2 * sm_count()) team = 2;
  else if (kSpans && rows > sm_count()) team = 4;
  const int merge_grid = (rows * team + kMergeWarps - 1) / kMergeWarps;
  p.decode_warps = grid * kWarps;
  p.early_sums = kSpans && merge_grid <= sm_count() ? 1 : 0;
  AICI_CUDA(cudaLaunchKernelEx(&cfg, paged_decode_kernel<PartT, kSpans>, p));
  cfg.blockDim = dim3(kMergeWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.gridDim = dim3(merge_grid);
  if (team == 1) {
    AICI_CUDA(cudaLaunchKernelEx(&cfg, paged_merge_kernel<PartT, kSpans, 1>, p));
  } else if (team == 2) {
    AICI_CUDA(cudaLaunchKernelEx(&cfg, paged_merge_kernel<PartT, kSpans, 2>, p));
  } else if (team == 4) {
    AICI_CUDA(cudaLaunchKernelEx(&cfg, paged_merge_kernel<PartT, kSpans, 4>, p));
  } else {
    AICI_CUDA(cudaLaunchKernelEx(&cfg, paged_merge_kernel<PartT, kSpans, kMergeWarps>, p));
  }
  return nullptr;
}

}  // namespace aici

using namespace aici;

extern "C" size_t aici_paged_attention_workspace_bytes(int num_seqs, int num_heads, int num_kv_heads,
                                                       int max_context_len) {
  if (num_seqs <= 0 || num_heads <= 0 || num_kv_heads <= 0) return kAlign;
  if (use_spans(num_seqs, num_kv_heads, max_context_len))
    return spans_layout(num_seqs, num_heads, num_kv_heads).total;
  return workspace_layout(num_seqs, num_heads, max_context_len,
                          pick_chunk(num_seqs, num_kv_heads, max_context_len)).total;
}

static bool valid_chunk(int chunk_tokens) {
  return chunk_tokens == 0 || (chunk_tokens > 0 && chunk_tokens % kB == 0 && chunk_tokens <= kMaxChunk);
}

extern "C" size_t aici_paged_attention_chunked_workspace_bytes(int num_seqs, int num_heads,
                                                               int num_kv_heads, int max_context_len,
                                                               int chunk_tokens) {
  if (num_seqs <= 0 || num_heads <= 0 || num_kv_heads <= 0 || !valid_chunk(chunk_tokens)) return kAlign;
  const int chunk = chunk_tokens > 0 ? chunk_tokens : pick_chunk(num_seqs, num_kv_heads, max_context_len);
  return workspace_layout(num_seqs, num_heads, max_context_len, chunk).total;
}

// forced_chunk < 0: the default traversal; 0: the fixed-chunk traversal with its own chunk size;
// > 0: the fixed-chunk traversal with that many tokens per chunk.
// The new tokens of a decode step (aici_decode_step).
struct StepTokens {
  const void *key, *value, *slots;
  int slot_is_int64;
  int64_t key_stride, value_stride;
};

static char *paged_attention_v1_impl(const char *fn, void *const *outs, int world, int out_heads,
                                     int out_head0, const void *query, const void *key_cache,
                                     const void *value_cache, int num_kv_heads, float scale,
                                     const int32_t *block_tables, const int32_t *context_lens,
                                     int block_size, int max_context_len, const float *alibi_slopes,
                                     int num_seqs, int num_heads, int head_size,
                                     int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride,
                                     int64_t kv_block_stride, int64_t kv_head_stride, void *workspace,
                                     size_t workspace_bytes, int dtype, aici_stream_t stream,
                                     int forced_chunk = -1, void *const *peer_flags = nullptr,
                                     int rank = 0, const StepTokens *step = nullptr) {
  void *out = outs[0];
  for (int w = 1; w < world; ++w)
    AICI_CHECK(outs[w] != nullptr && (uintptr_t)outs[w] % 16 == 0,
               "%s: peer output %d must be non-NULL and 16-byte aligned", fn, w);
  if (char *e = check_decode_args(fn, out, query, key_cache, value_cache, num_kv_heads,
                                  block_tables, context_lens, block_size, max_context_len,
                                  alibi_slopes, num_seqs, num_heads, head_size,
                                  max_num_blocks_per_seq, num_blocks, q_stride, kv_block_stride,
                                  kv_head_stride, dtype))
    return e;
  if (char *e = check_on_current_device(fn, "query", query)) return e;
  if (num_seqs == 0) return nullptr;
  const bool spans = forced_chunk < 0 && use_spans(num_seqs, num_kv_heads, max_context_len);
  const int chunk = spans ? kB
                          : (forced_chunk > 0 ? forced_chunk
                                              : pick_chunk(num_seqs, num_kv_heads, max_context_len));
  const WorkspaceLayout w = spans ? spans_layout(num_seqs, num_heads, num_kv_heads)
                                  : workspace_layout(num_seqs, num_heads, max_context_len, chunk);
  AICI_CHECK(workspace != nullptr && workspace_bytes >= w.total,
             "%s: workspace too small (%zu bytes given, %zu needed)", fn, workspace_bytes, w.total);
  AICI_CHECK((uintptr_t)workspace % kAlign == 0, "%s: workspace must be 256-byte aligned", fn);
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);
  char *ws = static_cast<char *>(workspace);
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16 *>(query);
  p.k_cache = static_cast<const __nv_bfloat16 *>(key_cache);
  p.v_cache = static_cast<const __nv_bfloat16 *>(value_cache);
  for (int i = 0; i < 8; ++i) p.out[i] = static_cast<__nv_bfloat16 *>(i < world ? outs[i] : nullptr);
  p.world = world;
  p.out_heads = out_heads;
  p.out_head0 = out_head0;
  p.block_tables = block_tables;
  p.context_lens = context_lens;
  p.part_max = reinterpret_cast<float *>(ws + w.max_off);
  p.part_sum = reinterpret_cast<float *>(ws + w.sum_off);
  p.part_out = ws + w.out_off;
  p.num_seqs = num_seqs;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = num_heads / num_kv_heads;
  p.max_blocks_per_seq = max_num_blocks_per_seq;
  p.max_context_len = max_context_len;
  p.num_blocks = num_blocks;
  p.chunk_tokens = chunk;
  p.max_parts = w.max_parts;
  p.always_write_partials = 0;
  p.decode_warps = 0;  // set by launch_decode, like early_sums
  p.span_cum = reinterpret_cast<int *>(ws + w.entries_off);
  p.early_sums = 0;
  p.min_span = kMinSpanTiles;
  p.q_stride = q_stride;
  p.kv_block_stride = kv_block_stride;
  p.kv_head_stride = kv_head_stride;
  p.scale_log2e = scale * kLog2e;
  p.status = st;
  p.sync = peer_flags != nullptr && world > 1 ? 1 : 0;
  p.rank = rank;
  p.new_k = static_cast<const __nv_bfloat16 *>(step ? step->key : nullptr);
  p.new_v = static_cast<const __nv_bfloat16 *>(step ? step->value : nullptr);
  p.new_slots = step ? step->slots : nullptr;
  p.new_slot_is_int64 = step ? step->slot_is_int64 : 0;
  p.new_k_stride = step ? step->key_stride : 0;
  p.new_v_stride = step ? step->value_stride : 0;
  for (int i = 0; i < 8; ++i)
    p.peer_flags[i] = static_cast<unsigned int *>(p.sync && i < world ? peer_flags[i] : nullptr);
  if (spans) return launch_decode<float, true>(p, nullptr, nullptr, static_cast<cudaStream_t>(stream));
  return launch_decode<float, false>(p, reinterpret_cast<int2 *>(ws + w.entries_off),
                                     reinterpret_cast<int *>(ws + w.n_entries_off),
                                     static_cast<cudaStream_t>(stream));
}

extern "C" char *aici_paged_attention_v1(void *out, const void *query, const void *key_cache,
                                         const void *value_cache, int num_kv_heads, float scale,
                                         const int32_t *block_tables, const int32_t *context_lens,
                                         int block_size, int max_context_len,
                                         const float *alibi_slopes, int num_seqs, int num_heads,
                                         int head_size, int max_num_blocks_per_seq,
                                         int64_t num_blocks, int64_t q_stride,
                                         int64_t kv_block_stride, int64_t kv_head_stride,
                                         void *workspace, size_t workspace_bytes, int dtype,
                                         aici_stream_t stream) {
  void *outs[1] = {out};
  return paged_attention_v1_impl("aici_paged_attention_v1", outs, 1, num_heads, 0, query, key_cache,
                                 value_cache, num_kv_heads, scale, block_tables, context_lens, block_size,
                                 max_context_len, alibi_slopes, num_seqs, num_heads, head_size,
                                 max_num_blocks_per_seq, num_blocks, q_stride, kv_block_stride,
                                 kv_head_stride, workspace, workspace_bytes, dtype, stream);
}

// Decode attention whose epilogue is the head-output gather: every finished output row is stored
// to its final place [seq, head0 + head, :] in the output buffer of EVERY rank (plain stores to
// peer-mapped memory over NVLink), so no collective runs afterwards; the ranks only need a
// barrier before reading.  outs[] lists the world's buffers (this rank's own included), each
// [num_seqs, total_heads, 128].
extern "C" char *aici_paged_attention_v1_peers(void *const *outs, int world, int total_heads, int head0,
                                               const void *query, const void *key_cache,
                                               const void *value_cache, int num_kv_heads, float scale,
                                               const int32_t *block_tables, const int32_t *context_lens,
                                               int block_size, int max_context_len, int num_seqs,
                                               int num_heads, int head_size, int max_num_blocks_per_seq,
                                               int64_t num_blocks, int64_t q_stride,
                                               int64_t kv_block_stride, int64_t kv_head_stride,
                                               void *workspace, size_t workspace_bytes, int dtype,
                                               aici_stream_t stream) {
  const char *fn = "aici_paged_attention_v1_peers";
  AICI_CHECK(outs != nullptr && world >= 1 && world <= 8, "%s: world must be 1..8", fn);
  AICI_CHECK(head0 >= 0 && num_heads > 0 && head0 + num_heads <= total_heads,
             "%s: heads [%d, %d) do not fit %d total heads", fn, head0, head0 + num_heads, total_heads);
  return paged_attention_v1_impl(fn, outs, world, total_heads, head0, query, key_cache, value_cache,
                                 num_kv_heads, scale, block_tables, context_lens, block_size,
                                 max_context_len, nullptr, num_seqs, num_heads, head_size,
                                 max_num_blocks_per_seq, num_blocks, q_stride, kv_block_stride,
                                 kv_head_stride, workspace, workspace_bytes, dtype, stream);
}

// The same call with the ranks' barrier folded into its last kernel: flag_ptrs are the flag arrays
// of aici_peer_barrier (and the two may be mixed on the same arrays).  When this call's kernels have
// finished, every rank's buffer holds all heads: no separate barrier launch follows.
extern "C" char *aici_paged_attention_v1_peers_barrier(
    void *const *outs, void *const *flag_ptrs, int world, int rank, int total_heads, int head0,
    const void *query, const void *key_cache, const void *value_cache, int num_kv_heads, float scale,
    const int32_t *block_tables, const int32_t *context_lens, int block_size, int max_context_len,
    int num_seqs, int num_heads, int head_size, int max_num_blocks_per_seq, int64_t num_blocks,
    int64_t q_stride, int64_t kv_block_stride, int64_t kv_head_stride, void *workspace,
    size_t workspace_bytes, int dtype, aici_stream_t stream) {
  const char *fn = "aici_paged_attention_v1_peers_barrier";
  AICI_CHECK(outs != nullptr && flag_ptrs != nullptr && world >= 1 && world <= 8 && rank >= 0 && rank < world,
             "%s: world must be 1..8 and rank inside it", fn);
  AICI_CHECK(head0 >= 0 && num_heads > 0 && head0 + num_heads <= total_heads,
             "%s: heads [%d, %d) do not fit %d total heads", fn, head0, head0 + num_heads, total_heads);
  for (int i = 0; i < world; ++i)
    AICI_CHECK(flag_ptrs[i] != nullptr && (uintptr_t)flag_ptrs[i] % 4 == 0,
               "%s: flag array %d must be non-NULL and 4-byte aligned", fn, i);
  if (char *e = paged_attention_v1_impl(fn, outs, world, total_heads, head0, query, key_cache, value_cache,
                                        num_kv_heads, scale, block_tables, context_lens, block_size,
                                        max_context_len, nullptr, num_seqs, num_heads, head_size,
                                        max_num_blocks_per_seq, num_blocks, q_stride, kv_block_stride,
                                        kv_head_stride, workspace, workspace_bytes, dtype, stream, -1,
                                        flag_ptrs, rank))
    return e;
  // an empty batch launches nothing; the ranks still have to meet
  if (num_seqs == 0) return aici_peer_barrier(flag_ptrs, world, rank, stream);
  return nullptr;
}

// One decode step of one layer in one call: the cache write of the step's new tokens
// (reshape_and_cache: token i is the newest token of sequence i) and decode attention over the
// cache, which rLLM issues as two kernels back to back (rllm-cuda/src/llm/mod.rs:132-166 then
// :280-316).  Here the cache write has no launch of its own: the warp of the decode kernel that
// works on the last tile of a (sequence, kv head) row takes the new token from the call's inputs,
// places it in the tile it has staged and writes it to the cache.  With world > 1 the call is also
// the head-output gather (outs / flag_ptrs as in aici_paged_attention_v1_peers_barrier); with
// world == 1, outs[0] is the output and flag_ptrs may be NULL.
extern "C" char *aici_decode_step(void *const *outs, void *const *flag_ptrs, int world, int rank,
                                  int total_heads, int head0, const void *new_key, const void *new_value,
                                  const void *slot_mapping, int slot_is_int64, int64_t key_stride,
                                  int64_t value_stride, const void *query, void *key_cache,
                                  void *value_cache, int num_kv_heads, float scale,
                                  const int32_t *block_tables, const int32_t *context_lens, int block_size,
                                  int max_context_len, int num_seqs, int num_heads, int head_size,
                                  int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride,
                                  int64_t kv_block_stride, int64_t kv_head_stride, void *workspace,
                                  size_t workspace_bytes, int dtype, aici_stream_t stream) {
  const char *fn = "aici_decode_step";
  AICI_CHECK(outs != nullptr && world >= 1 && world <= 8 && rank >= 0 && rank < world,
             "%s: world must be 1..8 and rank inside it", fn);
  AICI_CHECK(world == 1 || flag_ptrs != nullptr, "%s: flag arrays are needed with more than one rank", fn);
  AICI_CHECK(head0 >= 0 && num_heads > 0 && head0 + num_heads <= total_heads,
             "%s: heads [%d, %d) do not fit %d total heads", fn, head0, head0 + num_heads, total_heads);
  for (int i = 0; world > 1 && i < world; ++i)
    AICI_CHECK(flag_ptrs[i] != nullptr && (uintptr_t)flag_ptrs[i] % 4 == 0,
               "%s: flag array %d must be non-NULL and 4-byte aligned", fn, i);
  if (num_seqs > 0) {
    AICI_CHECK(new_key && new_value && slot_mapping, "%s: NULL pointer", fn);
    AICI_CHECK(((uintptr_t)new_key | (uintptr_t)new_value) % 16 == 0, "%s: tensors must be 16-byte aligned", fn);
    AICI_CHECK(num_kv_heads > 0 && key_stride % 8 == 0 && value_stride % 8 == 0 &&
                   key_stride >= (int64_t)num_kv_heads * 128 && value_stride >= (int64_t)num_kv_heads * 128,
               "%s: token strides must be multiples of 8 elements and cover one row", fn);
    AICI_CHECK(num_seqs <= kMaxInlineSeqs, "%s: at most %d sequences per call", fn, kMaxInlineSeqs);
  }
  const StepTokens step = {new_key, new_value, slot_mapping, slot_is_int64, key_stride, value_stride};
  if (char *e = paged_attention_v1_impl(fn, outs, world, total_heads, head0, query, key_cache, value_cache,
                                        num_kv_heads, scale, block_tables, context_lens, block_size,
                                        max_context_len, nullptr, num_seqs, num_heads, head_size,
                                        max_num_blocks_per_seq, num_blocks, q_stride, kv_block_stride,
                                        kv_head_stride, workspace, workspace_bytes, dtype, stream, -1,
                                        world > 1 ? flag_ptrs : nullptr, rank, &step))
    return e;
  if (num_seqs == 0 && world > 1) return aici_peer_barrier(flag_ptrs, world, rank, stream);
  return nullptr;
}

// aici_paged_attention_v1 through the fixed-chunk traversal (every sequence cut into chunks of
// chunk_tokens tokens, dealt out round-robin): kept so that tests and benchmarks can compare the two
// traversals.  The chunk size is an argument of the call; nothing process-wide is changed.
extern "C" char *aici_paged_attention_v1_chunked(
    void *out, const void *query, const void *key_cache, const void *value_cache, int num_kv_heads,
    float scale, const int32_t *block_tables, const int32_t *context_lens, int block_size,
    int max_context_len, const float *alibi_slopes, int num_seqs, int num_heads, int head_size,
    int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride, int64_t kv_block_stride,
    int64_t kv_head_stride, void *workspace, size_t workspace_bytes, int chunk_tokens, int dtype,
    aici_stream_t stream) {
  const char *fn = "aici_paged_attention_v1_chunked";
  AICI_CHECK(valid_chunk(chunk_tokens), "%s: chunk_tokens must be 0 or a multiple of 16 up to 512", fn);
  void *outs[1] = {out};
  return paged_attention_v1_impl(fn, outs, 1, num_heads, 0, query, key_cache, value_cache, num_kv_heads,
                                 scale, block_tables, context_lens, block_size, max_context_len,
                                 alibi_slopes, num_seqs, num_heads, head_size, max_num_blocks_per_seq,
                                 num_blocks, q_stride, kv_block_stride, kv_head_stride, workspace,
                                 workspace_bytes, dtype, stream, chunk_tokens);
}

extern "C" char *aici_paged_attention_v2(void *out, float *exp_sums, float *max_logits,
                                         void *tmp_out, const void *query, const void *key_cache,
                                         const void *value_cache, int num_kv_heads, float scale,
                                         const int32_t *block_tables, const int32_t *context_lens,
                                         int block_size, int max_context_len,
                                         const float *alibi_slopes, int num_seqs, int num_heads,
                                         int head_size, int max_num_blocks_per_seq,
                                         int64_t num_blocks, int64_t q_stride,
                                         int64_t kv_block_stride, int64_t kv_head_stride,
                                         int dtype, aici_stream_t stream) {
  const char *fn = "aici_paged_attention_v2";
  if (char *e = check_decode_args(fn, out, query, key_cache, value_cache, num_kv_heads,
                                  block_tables, context_lens, block_size, max_context_len,
                                  alibi_slopes, num_seqs, num_heads, head_size,
                                  max_num_blocks_per_seq, num_blocks, q_stride, kv_block_stride,
                                  kv_head_stride, dtype))
    return e;
  if (num_seqs == 0) return nullptr;
  AICI_CHECK(exp_sums && max_logits && tmp_out, "%s: NULL pointer", fn);
  AICI_CHECK((uintptr_t)tmp_out % 4 == 0, "%s: tmp_out must be 4-byte aligned", fn);
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16 *>(query);
  p.k_cache = static_cast<const __nv_bfloat16 *>(key_cache);
  p.v_cache = static_cast<const __nv_bfloat16 *>(value_cache);
  for (int i = 0; i < 8; ++i) p.out[i] = i == 0 ? static_cast<__nv_bfloat16 *>(out) : nullptr;
  p.world = 1;
  p.out_heads = num_heads;
  p.out_head0 = 0;
  p.block_tables = block_tables;
  p.context_lens = context_lens;
  p.part_max = max_logits;
  p.part_sum = exp_sums;
  p.part_out = tmp_out;
  p.num_seqs = num_seqs;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = num_heads / num_kv_heads;
  p.max_blocks_per_seq = max_num_blocks_per_seq;
  p.max_context_len = max_context_len;
  p.num_blocks = num_blocks;
  p.chunk_tokens = 512;  // PARTITION_SIZE of the reference
  p.max_parts = max_context_len > 0 ? (max_context_len + 511) / 512 : 1;
  p.always_write_partials = 1;
  p.decode_warps = 0;
  p.span_cum = nullptr;
  p.early_sums = 0;
  p.min_span = 1;
  p.q_stride = q_stride;
  p.kv_block_stride = kv_block_stride;
  p.kv_head_stride = kv_head_stride;
  p.scale_log2e = scale * kLog2e;
  p.status = st;
  p.sync = 0;
  p.rank = 0;
  p.new_k = p.new_v = nullptr;
  p.new_slots = nullptr;
  p.new_slot_is_int64 = 0;
  p.new_k_stride = p.new_v_stride = 0;
  for (int i = 0; i < 8; ++i) p.peer_flags[i] = nullptr;
  return launch_decode<__nv_bfloat16, false>(p, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

// ---- decode attention for callers that cannot provide scratch memory ------------------------------
//
// aici_paged_attention_v1 needs a workspace for its chunk list and split-context partials, and
// somebody has to allocate it.  Two kinds of caller cannot: a serving loop whose KV-cache pool was
// sized to take (nearly) all free device memory after start-up profiling, so that a later
// allocation can fail or stall the step; and a binding from a runtime that has no device
// allocator of its own (the Rust crate once libtorch is out of the call path).  For them the
// library carries the workspace itself: a fixed array in device memory that exists on every GPU
// that loads the library, from load to exit.
//
// Rules that follow from sharing one array:
//   * sizes whose workspace would exceed kStaticScratchBytes are refused with an error string;
//   * the array keeps whatever the previous call left; nothing in it has to start at zero (the
//     decode kernel writes the prefix sums or the chunk list, every partial is written before it
//     is read), so no clearing pass runs;
//   * two calls that overlap on the GPU (different streams, or different threads on one device)
//     race on the array -- serialise them on one stream;
//   * the first call on each device looks the array's device address up (the name used in host
//     code is only a handle, not an address a kernel could use) and sets a function attribute;
//     make that first call outside any stream capture.
constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB: 256 sequences x 32/8 heads need 6.4 MiB, 2048 x 32/8 do not fit
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

extern "C" char *aici_paged_attention_v1_static(
    void *out, const void *query, const void *key_cache, const void *value_cache, int num_kv_heads,
    float scale, const int32_t *block_tables, const int32_t *context_lens, int block_size,
    int max_context_len, const float *alibi_slopes, int num_seqs, int num_heads, int head_size,
    int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride, int64_t kv_block_stride,
    int64_t kv_head_stride, int dtype, aici_stream_t stream) {
  const char *fn = "aici_paged_attention_v1_static";
  static void *scratch_addr[64] = {nullptr};
  static OncePerDevice once;
  int dev = 0;
  AICI_CUDA(cudaGetDevice(&dev));
  AICI_CHECK(dev >= 0 && dev < 64, "%s: device index %d out of range", fn, dev);
  if (char *e = once.run([&]() -> char * {
        void *p = nullptr;
        AICI_CUDA(cudaGetSymbolAddress(&p, g_decode_scratch));
        AICI_CHECK(p != nullptr, "%s: the scratch array has no device address", fn);
        scratch_addr[dev] = p;
        return nullptr;
      }))
    return e;
  // argument errors first, so that a bad head count is not reported as a size problem
  if (char *e = check_decode_args(fn, out, query, key_cache, value_cache, num_kv_heads, block_tables,
                                  context_lens, block_size, max_context_len, alibi_slopes, num_seqs,
                                  num_heads, head_size, max_num_blocks_per_seq, num_blocks, q_stride,
                                  kv_block_stride, kv_head_stride, dtype))
    return e;
  if (num_seqs > 0) {
    const size_t need =
        aici_paged_attention_workspace_bytes(num_seqs, num_heads, num_kv_heads, max_context_len);
    AICI_CHECK(need <= kStaticScratchBytes,
               "%s: this batch needs %zu bytes of scratch but the built-in array holds %zu "
               "(about 520 bytes per query head and (warp of the grid + sequence x kv head)); use "
               "aici_paged_attention_v1 with a caller-owned workspace",
               fn, need, kStaticScratchBytes);
  }
  return aici_paged_attention_v1(out, query, key_cache, value_cache, num_kv_heads, scale, block_tables,
                                 context_lens, block_size, max_context_len, alibi_slopes, num_seqs,
                                 num_heads, head_size, max_num_blocks_per_seq, num_blocks, q_stride,
                                 kv_block_stride, kv_head_stride, scratch_addr[dev], kStaticScratchBytes,
                                 dtype, stream);
}
