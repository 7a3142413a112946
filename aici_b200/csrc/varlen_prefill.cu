// Variable-length causal prefill attention for sm_100a: tcgen05 MMA with TMEM accumulators,
// operands staged by TMA, online softmax in registers.
//
// Semantics follow mha_varlen_fwd of rllm/tch-cuda/kernels/flash_attn (flash_api.cpp:447-618,
// flash_fwd_kernel.h:590-1136): O = softmax(scale * Q K^T + causal mask) V per packed sequence
// and head, fp32 scores and accumulation, probabilities rounded to bf16 before P V, kv head =
// head / (num_heads / num_heads_k), causal mask aligned to the bottom-right corner
// (softmax.h:159-168), rows that see no column give 0 (flash_fwd_kernel.h:1056).
//
// The kernel comes in three shapes (PrefillCfg below): one query tile per CTA with two CTAs per SM
// for short sequences, two query tiles per CTA for long ones, and the two-tile shape on pairs of
// CTAs whose MMAs span two SMs.  The roles, in the two-tile shape:
// one CTA per SM owns TWO 128-row query tiles that share their key/value tiles: two query heads
// of one kv-head group when the group size is even (same rows, same causal extent), else two
// consecutive row tiles of one head.  Each key/value tile of 128 tokens is loaded once for both.
//   warp 8    : TMA producer (Q0, Q1 once; then K_0, V_0, K_1, V_1, ... through a 4-stage ring of
//               32 KB stages, 128-byte swizzle, no multicast)
//   warp 9    : TMEM owner (all 512 columns: S0, S1, O0, O1) and MMA issuer.  S_t = Q_t K_j^T in SS
//               form, O_t += P_t V_j in TS form (P read from TMEM where it overwrote S_t, V as an
//               MN-major shared-memory operand).  Issue order S0 S1 | PV0 S0' PV1 S1' | ... so that
//               the tensor pipe works on one tile while the other tile's softmax runs.
//   warps 0-3 : softmax of tile 0, warps 4-7: softmax of tile 1.  One query row per thread (= one
//               TMEM lane): tcgen05.ld the scores, mask, exp2 against a running reference maximum
//               (single pass on packed fp32 pairs; the reference moves lazily, judged by the tile's
//               row sum, and a tile whose scores jump too far is redone exactly), bf16 P written
//               back with tcgen05.st; at the end O / sum -> bf16 -> staging in the tile's Q buffer
//               (same swizzled layout) -> TMA stores, or row-by-row stores for a ragged tile.
// (One-tile shape: warps 0-3 softmax, warp 4 producer, warp 5 issuer.)  The grid is ordered
// (head, sequence, row tile), row tile slowest and longest first.
// Every barrier wait is bounded; a timeout sets AICI_STATUS_WAIT_TIMEOUT and unwinds.
#include "tcgen05.cuh"

namespace aici {

constexpr int kBM = 128;               // query rows per tile
constexpr int kBN = 128;               // keys per tile
constexpr int kHD = 128;               // head size
constexpr int kPanelBytes = 128 * 128; // [128 rows][64 bf16] = one 128B-swizzled panel
constexpr int kTileBytes = 2 * kPanelBytes;
constexpr int kMaxKvStages = 6;        // ring of K/V tiles (K_j and V_j alternate)

// Three shapes of the same kernel.
//   1  one query tile per CTA (short sequences): 256 TMEM columns (S/P [0,128) O [128,256)), a 2-stage
//      K/V ring, 4 softmax warps -- half the shared and tensor memory of shape 2, so TWO CTAs share an
//      SM and one CTA's fill (barriers, TMEM allocation, first loads) and drain (epilogue, stores,
//      exit) run under the other's MMAs.
//   2  two query tiles per CTA that share their K/V tiles (long sequences): all 512 TMEM columns
//      (S0/P0 [0,128) S1/P1 [128,256) O0 [256,384) O1 [384,512)), a 4-stage ring, 8 softmax warps.
//   3  shape 2 on a PAIR of CTAs (a cluster of two on neighbouring SMs) that work on four query heads
//      of one kv head: every MMA is one cta_group::2 instruction over both SMs (M = 256, 128 rows in
//      each CTA's tensor memory) and its B operand is split between them -- each CTA loads and holds
//      only half of every key tile (64 keys) and half of every value tile (64 of the 128 columns).
//      An SS-form S = Q K^T step then reads 6 KB of shared memory per SM instead of 8 KB and a P V
//      step 2 KB instead of 4 KB; shared-memory bandwidth into the tensor core (about 64 B/clk) is
//      what holds shape 2 back.  The leader CTA issues; the other CTA's issuer warp relays "my half
//      has landed" to it; completion comes back to both through multicast commits.
template <int kShape>
struct PrefillCfg {
  static constexpr int kTiles = kShape == 1 ? 1 : 2;
  static constexpr bool kPair = kShape == 3;
  static constexpr int kStages = kShape == 1 ? 2 : (kShape == 2 ? 4 : 6);
  static constexpr int kStageBytes = kPair ? kTileBytes / 2 : kTileBytes;
  static constexpr int kSoftmaxWarps = 4 * kTiles;
  static constexpr int kProducerWarp = 4 * kTiles;
  static constexpr int kMmaWarp = 4 * kTiles + 1;
  static constexpr int kThreads = (4 * kTiles + 2) * 32;
  static constexpr uint32_t kCols = 256u * kTiles;
  static constexpr int kSmemBytes = kTiles * kTileBytes + kStages * kStageBytes + 1024 /*align*/ + 512 /*PrefillSmem*/;
  static constexpr int kCtasPerSm = kTiles == 2 ? 1 : 2;
};
constexpr float kRescaleThreshold = 8.f;  // log2 units: the running reference moves once a score exceeds it by this
constexpr float kRescaleSum = 256.f;      // single-pass tiles: a row sum above this moves the reference (some score is 2^8 above it, or many are above it)
constexpr float kDangerSum = 1e30f;       // single-pass tiles: a row sum at or above this (or NaN) means the tile is redone exactly

struct PrefillParams {
  // output [total_q, heads, 128] (strides below) in `world` buffers -- this GPU's and, for the
  // fused head gather, every peer's; this rank's head h is written at head index out_head0 + h
  __nv_bfloat16 *out[8];
  int world, out_head0;
  const int32_t *cu_q;
  const int32_t *cu_k;
  int64_t o_tok_stride, o_head_stride;
  int group;
  int causal;
  int pair_heads;  // 1: the two tiles are heads 2y and 2y+1; 0: two consecutive row tiles of head y
  int tma_store;   // 1: full output tiles leave shared memory as TMA stores (one output buffer only)
  int total_q;     // rows of the packed query / output tensors
  float scale_log2e;
  unsigned int *status;
  // paged variant: keys/values are read from the KV cache through the block table
  const int32_t *block_tables;  // [batch, max_blocks]
  const int32_t *k_lens;        // [batch] tokens of each sequence present in the cache
  int max_blocks;
  int64_t num_blocks;
};

// One tensor map per output buffer (this GPU's and, for the fused gather, every peer's).
struct OutMaps {
  CUtensorMap m[8];
};

struct PrefillSmem {
  uint64_t q_full[2], kv_full[kMaxKvStages], kv_empty[kMaxKvStages], s_full[2], p_ready[2], o_full[2], staged[2], drain;
  uint64_t q_peer[2], kv_peer[kMaxKvStages];  // CTA pairs: the leader's view of "the other CTA's half has landed"
  uint32_t tmem_base;
  uint32_t aborted;
};

struct TileInfo {
  int h;        // query head
  int m0;       // first query row within the sequence
  int rows;     // valid rows (<= 128); 0 = this tile does not exist
  int n_tiles;  // key/value tiles it visits; 0 = nothing visible
};

__device__ __forceinline__ void zero_rows(const PrefillParams &p, int q0, const TileInfo &T, int tid,
                                          int nthreads) {
  for (int i = tid; i < T.rows * (kHD / 8); i += nthreads) {
    const int r = i / (kHD / 8), c = i % (kHD / 8);
    for (int w = 0; w < p.world; ++w)
      *reinterpret_cast<uint4 *>(p.out[w] + (int64_t)(q0 + T.m0 + r) * p.o_tok_stride +
                                 (int64_t)(p.out_head0 + T.h) * p.o_head_stride + c * 8) = make_uint4(0, 0, 0, 0);
  }
}

// kPaged = false: K and V are packed [total_k, Hkv, 128] tensors (tensor maps as for Q).
// kPaged = true : K and V come from the paged cache.  A key tile is 16 half-blocks of
//   [16 chunks][8 tokens][8 elements] (2 KB each, no swizzle: exactly the 8-row x 16-byte core
//   matrices the MMA wants, leading offset 128 B between the two chunks of a K step, stride offset
//   2 KB between 8-token groups); a value tile is 8 blocks of [128 d][16 tokens] loaded with the
//   32-byte swizzle, one K = 16 MMA per block.  Value columns past the sequence end are zeroed in
//   shared memory before P V (cache slots there may hold anything, NaN included).
template <bool kPaged, int kShape>
__global__ void __launch_bounds__(PrefillCfg<kShape>::kThreads, PrefillCfg<kShape>::kCtasPerSm)
varlen_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q,
                      const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v,
                      const __grid_constant__ OutMaps tmap_o, const PrefillParams p) {
  using Cfg = PrefillCfg<kShape>;
  constexpr int kTiles = Cfg::kTiles;
  constexpr bool kPair = Cfg::kPair;
  static_assert(!(kPair && kPaged), "the CTA-pair shape reads packed K/V only");
  constexpr int kKvStages = Cfg::kStages;
  constexpr int kStageBytes = Cfg::kStageBytes;
  constexpr int kPrefillThreads = Cfg::kThreads;
  constexpr uint32_t kTmemCols = Cfg::kCols;
  constexpr uint32_t kOCol = 128u * kTiles;  // first column of O0
  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // The grid is ordered (head, sequence, row tile) with the row tile as the slowest index: all the
  // longest tiles of the batch start first and the CTAs with one key tile fill the tail.
  const int b = blockIdx.y;
  const int q0 = p.cu_q[b], lq = p.cu_q[b + 1] - q0;
  int k0 = 0, lk = 0;
  if (kPaged) {
    lk = p.k_lens[b];
    if (lk > p.max_blocks * 16) {
      if (tid == 0) set_status(p.status, AICI_STATUS_BAD_BLOCK);
      lk = p.max_blocks * 16;
    }
    if (lk < 0) lk = 0;
  } else {
    k0 = p.cu_k[b];
    lk = p.cu_k[b + 1] - k0;
  }
  const int n_mblocks = (lq + kBM - 1) / kBM;

  // ---- which two tiles does this CTA own? (longest causal tiles are scheduled first) ----------
  TileInfo tiles[2];
  {
    int mb[2], hh[2];
    if (kTiles == 1) {
      mb[0] = n_mblocks - 1 - (int)blockIdx.z;
      mb[1] = -1;  // no second tile
      hh[0] = hh[1] = (int)blockIdx.x;
    } else if (kPair) {
      // clusters of two CTAs along x: CTA x = 2y + r holds heads 4y + 2r and 4y + 2r + 1
      mb[0] = mb[1] = n_mblocks - 1 - (int)blockIdx.z;
      hh[0] = 2 * (int)blockIdx.x;
      hh[1] = hh[0] + 1;
    } else if (p.pair_heads) {
      mb[0] = mb[1] = n_mblocks - 1 - (int)blockIdx.z;
      hh[0] = 2 * (int)blockIdx.x;
      hh[1] = hh[0] + 1;
    } else {
      mb[1] = n_mblocks - 1 - 2 * (int)blockIdx.z;
      mb[0] = mb[1] - 1;
      hh[0] = hh[1] = (int)blockIdx.x;
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      TileInfo &T = tiles[t];
      T.h = hh[t];
      T.m0 = mb[t] * kBM;
      T.rows = mb[t] >= 0 && mb[t] < n_mblocks ? min(kBM, lq - T.m0) : 0;
      int lim = lk;
      if (p.causal) lim = min(lk, T.m0 + T.rows + lk - lq);
      T.n_tiles = (T.rows > 0 && lim > 0) ? (lim + kBN - 1) / kBN : 0;
    }
  }
  if (tiles[0].rows == 0 && tiles[1].rows == 0) return;
  const int hk = tiles[1].rows > 0 ? tiles[1].h / p.group : tiles[0].h / p.group;
  // tiles that see no key at all are zero rows (flash_fwd_kernel.h:1056)
  if (tiles[0].rows > 0 && tiles[0].n_tiles == 0) zero_rows(p, q0, tiles[0], tid, kPrefillThreads);
  if (tiles[1].rows > 0 && tiles[1].n_tiles == 0) zero_rows(p, q0, tiles[1], tid, kPrefillThreads);
  const int nt0 = tiles[0].n_tiles, nt1 = tiles[1].n_tiles;
  const int nmax = max(nt0, nt1);
  if (nmax == 0) return;

  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *sQ = smem;                       // two tiles
  uint8_t *sKV = smem + kTiles * kTileBytes;     // kKvStages stages
  PrefillSmem *sh = reinterpret_cast<PrefillSmem *>(smem + kTiles * kTileBytes + kKvStages * kStageBytes);
  // CTA pairs: rank 0 of the cluster is the leader (issues the MMAs of both CTAs)
  const uint32_t pair_rank = kPair ? cluster_ctarank() : 0u;
  const bool leader = pair_rank == 0u;

  if (tid == 0) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      mbar_init(&sh->q_full[t], 1);
      mbar_init(&sh->s_full[t], 1);
      mbar_init(&sh->p_ready[t], kPair ? 8 : 4);  // pairs: the softmax warps of both CTAs report to the leader
      mbar_init(&sh->q_peer[t], 1);
      mbar_init(&sh->o_full[t], 1);
      mbar_init(&sh->staged[t], 4);
    }
#pragma unroll
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&sh->kv_full[s], 1);
      mbar_init(&sh->kv_empty[s], 1);
      mbar_init(&sh->kv_peer[s], 1);
    }
    mbar_init(&sh->drain, 1);
    sh->aborted = 0;
    fence_mbar_init();
  }
  if (warp == Cfg::kMmaWarp) {
    if (kPair) {
      tmem_alloc_pair(&sh->tmem_base, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&sh->tmem_base, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (kPair) cluster_sync_all();  // the other CTA's barriers exist before anything arrives on them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == Cfg::kProducerWarp) {
    // ---------------------------------------------------------------- TMA producer -----------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (tiles[t].n_tiles > 0) {
          mbar_expect_tx(&sh->q_full[t], kTileBytes);
          tma_load_3d(sQ + t * kTileBytes, &tmap_q, 0, tiles[t].h, q0 + tiles[t].m0, &sh->q_full[t]);
          tma_load_3d(sQ + t * kTileBytes + kPanelBytes, &tmap_q, 64, tiles[t].h, q0 + tiles[t].m0,
                      &sh->q_full[t]);
        }
      }
    }
    if (kPaged) {
      // All lanes take part: lane l < 8 owns cache block l of the tile (its id is read once per
      // tile, one tile ahead), lanes 0-15 each issue one half-block key copy, lanes 0-7 one value
      // copy; lane 0 posts the expected byte count.
      const int32_t *bt_row = p.block_tables + (int64_t)b * p.max_blocks;
      auto load_id = [&](int j) {
        int id = 0;
        const int nb = min(8, (lk - j * kBN + 15) / 16);
        if ((lane & 7) < nb && j < nmax) {
          id = bt_row[j * 8 + (lane & 7)];
          if (id < 0 || id >= p.num_blocks) {
            set_status(p.status, AICI_STATUS_BAD_BLOCK);
            id = 0;
          }
        }
        return id;
      };
      int id_cur = load_id(0), id_next = 0;
      bool ok = true;
      for (int i = 0; ok && i < 2 * nmax; ++i) {  // i even: K_{i/2}, i odd: V_{i/2}
        const int stage = i % kKvStages;
        const int j = i >> 1;
        if (!(i & 1)) id_next = load_id(j + 1);
        ok = __all_sync(0xffffffffu,
                        mbar_wait_abortable(&sh->kv_empty[stage], (((uint32_t)i / kKvStages) & 1u) ^ 1u, p.status));
        if (!ok) break;
        uint8_t *dst = sKV + stage * kTileBytes;
        const int nb = min(8, (lk - j * kBN + 15) / 16);  // cache blocks of this tile that exist
        if (lane == 0) mbar_expect_tx(&sh->kv_full[stage], nb * 4096);
        const int bi = lane & 7;
        if (i & 1) {
          if (lane < 8 && bi < nb) tma_load_4d(dst + bi * 4096, &tmap_v, 0, 0, hk, id_cur, &sh->kv_full[stage]);
          id_cur = id_next;
        } else {
          if (lane < 16 && bi < nb)
            tma_load_5d(dst + bi * 4096 + (lane >> 3) * 2048, &tmap_k, 0, (lane >> 3) * 8, 0, hk, id_cur,
                        &sh->kv_full[stage]);
        }
        __syncwarp();
      }
    } else if (lane == 0) {
      for (int i = 0; i < 2 * nmax; ++i) {  // i even: K_{i/2}, i odd: V_{i/2}
        const int stage = i % kKvStages;
        if (!mbar_wait_abortable(&sh->kv_empty[stage], (((uint32_t)i / kKvStages) & 1u) ^ 1u, p.status)) break;
        uint8_t *dst = sKV + stage * kStageBytes;
        const CUtensorMap *tm = (i & 1) ? &tmap_v : &tmap_k;
        mbar_expect_tx(&sh->kv_full[stage], kStageBytes);
        if (!kPair) {
          tma_load_3d(dst, tm, 0, hk, k0 + (i >> 1) * kBN, &sh->kv_full[stage]);
          tma_load_3d(dst + kPanelBytes, tm, 64, hk, k0 + (i >> 1) * kBN, &sh->kv_full[stage]);
        } else if (i & 1) {
          // this CTA's half of the value tile: 64 of the 128 columns, all 128 tokens (one panel)
          tma_load_3d(dst, tm, 64 * (int)pair_rank, hk, k0 + (i >> 1) * kBN, &sh->kv_full[stage]);
        } else {
          // this CTA's half of the key tile: 64 of the 128 tokens (tmap_k's box is 64 rows high),
          // two panels of 64 columns
          const int row = k0 + (i >> 1) * kBN + 64 * (int)pair_rank;
          tma_load_3d(dst, tm, 0, hk, row, &sh->kv_full[stage]);
          tma_load_3d(dst + kPanelBytes / 2, tm, 64, hk, row, &sh->kv_full[stage]);
        }
      }
    }
  } else if (warp == Cfg::kMmaWarp && kPair && !leader) {
    // ---------------------------------------------------------------- relay (pairs, second CTA) --
    // The leader issues the MMAs that read this CTA's shared memory too; it learns from this warp,
    // in consumption order, that this CTA's Q tiles and K/V halves have landed.
    bool ok = true;
    auto wait = [&](uint64_t *bar, uint32_t parity) {
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait_abortable(bar, parity, p.status));
      return ok;
    };
    for (int t = 0; t < 2 && ok; ++t) {
      if (tiles[t].n_tiles > 0 && wait(&sh->q_full[t], 0)) {
        fence_proxy_async_smem();
        if (lane == 0) mbar_arrive_cluster(&sh->q_peer[t], 0);
      }
    }
    for (int i = 0; ok && i < 2 * nmax; ++i) {
      const int stage = i % kKvStages;
      if (!wait(&sh->kv_full[stage], ((uint32_t)i / kKvStages) & 1u)) break;
      const int j = i >> 1;
      if ((i & 1) && lk - j * kBN < kBN) {
        // value rows behind the end of the sequence are cleared (see the leader's copy of this loop)
        const int valid = lk - j * kBN;
        uint8_t *vt = sKV + stage * kStageBytes;
        for (int idx = valid * 8 + lane; idx < kBN * 8; idx += 32)
          *reinterpret_cast<uint4 *>(vt + (idx >> 3) * 128 + (idx & 7) * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&sh->kv_peer[stage], 0);
    }
  } else if (warp == Cfg::kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer -------------
    constexpr uint32_t idesc_s = idesc_bf16(kPair ? 2 * kBM : kBM, kBN, false);
    constexpr uint32_t idesc_pv = idesc_bf16(kPair ? 2 * kBM : kBM, kHD, !kPaged);  // packed V: MN-major; cache V: K-major
    constexpr int kKPanel = kPair ? kPanelBytes / 2 : kPanelBytes;  // one 64-column panel of a key (half) tile
    bool ok = true;
    auto wait = [&](uint64_t *bar, uint32_t parity) {
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait_abortable(bar, parity, p.status));
      return ok;
    };
    // barriers another CTA arrives on: acquire at cluster scope
    auto wait_cluster = [&](uint64_t *bar, uint32_t parity) {
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait_abortable_cluster(bar, parity, p.status));
      return ok;
    };
    auto wait_q = [&](int t) {
      wait(&sh->q_full[t], 0);
      if (kPair) wait_cluster(&sh->q_peer[t], 0);
      return ok;
    };
    auto wait_kv = [&](int i) {
      wait(&sh->kv_full[i % kKvStages], ((uint32_t)i / kKvStages) & 1u);
      if (kPair) wait_cluster(&sh->kv_peer[i % kKvStages], ((uint32_t)i / kKvStages) & 1u);
      return ok;
    };
    auto wait_p = [&](int t, int j) {
      return kPair ? wait_cluster(&sh->p_ready[t], (uint32_t)j & 1u) : wait(&sh->p_ready[t], (uint32_t)j & 1u);
    };
    auto commit = [&](uint64_t *bar) {
      if (kPair) tc_commit_pair(bar, 3);
      else tc_commit(bar);
    };
    // S_t = Q_t K^T.  Q, K: K-major, rows of 128 B, 8-row groups 1024 B apart, two 64-column panels.
    auto issue_s = [&](int t, int i_k) {
      tc_fence_after();
      if (lane == 0) {
        const uint64_t qdesc = smem_desc_sw128(smem_u32(sQ + t * kTileBytes), 16, 1024);
        const uint32_t kaddr = smem_u32(sKV + (i_k % kKvStages) * kStageBytes);
        const uint64_t kdesc = kPaged ? smem_desc(kaddr, 128, 2048, 0) : smem_desc_sw128(kaddr, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < kHD / 16; ++ks) {
          const uint64_t adv = (uint64_t)(((ks >> 2) * kPanelBytes + (ks & 3) * 32) >> 4);
          const uint64_t kadv = kPaged ? (uint64_t)((ks * 256) >> 4)
                                       : (uint64_t)(((ks >> 2) * kKPanel + (ks & 3) * 32) >> 4);
          if (kPair) umma_ss_pair(tmem_base + t * 128, qdesc + adv, kdesc + kadv, idesc_s, ks > 0 ? 1u : 0u);
          else umma_ss(tmem_base + t * 128, qdesc + adv, kdesc + kadv, idesc_s, ks > 0 ? 1u : 0u);
        }
        commit(&sh->s_full[t]);
      }
      __syncwarp();
    };
    // O_t += P_t V.  V as B operand: N (= d) contiguous, 64 d per swizzle atom, second atom one
    // panel further (leading offset), 8-token groups 1024 B apart (stride offset).  In a CTA pair
    // each CTA holds one atom (its 64 columns).
    auto issue_pv = [&](int t, int i_v, bool first, bool last) {
      tc_fence_after();
      if (lane == 0) {
        const uint32_t vaddr = smem_u32(sKV + (i_v % kKvStages) * kStageBytes);
        // packed: one MN-major tile, a K step = 16 token rows of 128 B; cache: one block per K step,
        // rows (d) of 32 B with the 32-byte swizzle, 8-row groups 256 B apart
        const uint64_t vdesc = kPaged ? smem_desc(vaddr, 16, 256, 6) : smem_desc_sw128(vaddr, kPanelBytes, 1024);
        const uint32_t vstep = kPaged ? 4096u : 2048u;
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          if (kPair)
            umma_ts_pair(tmem_base + kOCol + t * 128, tmem_base + t * 128 + 8 * ks,
                         vdesc + (uint64_t)((ks * vstep) >> 4), idesc_pv, (!first || ks > 0) ? 1u : 0u);
          else
            umma_ts(tmem_base + kOCol + t * 128, tmem_base + t * 128 + 8 * ks, vdesc + (uint64_t)((ks * vstep) >> 4),
                    idesc_pv, (!first || ks > 0) ? 1u : 0u);
        }
        if (last) commit(&sh->o_full[t]);
      }
      __syncwarp();
    };
    auto release = [&](int i) {
      if (lane == 0) commit(&sh->kv_empty[i % kKvStages]);
      __syncwarp();
    };

    if (nt0 > 0) wait_q(0);
    if (nt1 > 0) wait_q(1);
    if (wait_kv(0)) {
      if (nt0 > 0) issue_s(0, 0);
      if (nt1 > 0) issue_s(1, 0);
      release(0);
    }
    for (int j = 0; ok && j < nmax; ++j) {
      const int i_v = 2 * j + 1, i_kn = 2 * j + 2;
      if (!wait_kv(i_v)) break;
      if (kPaged && lk - j * kBN < kBN) {
        // last tile of the sequence: zero the value columns of tokens >= lk (generic-proxy stores,
        // made visible to the tensor core with a proxy fence)
        const int valid = lk - j * kBN;
        uint8_t *vt = sKV + (i_v % kKvStages) * kStageBytes;
        for (int bi = valid / 16; bi < 8; ++bi) {
          uint8_t *vb = vt + bi * 4096;
          const int first = max(0, valid - bi * 16);
          if (first == 0) {
            for (int idx = lane; idx < 256; idx += 32) reinterpret_cast<uint4 *>(vb)[idx] = make_uint4(0, 0, 0, 0);
          } else {
            for (int d = lane; d < kHD; d += 32)
              for (int tok = first; tok < 16; ++tok)
                *reinterpret_cast<uint16_t *>(vb + d * 32 + ((((tok >> 3) ^ ((d >> 2) & 1))) << 4) + (tok & 7) * 2) = 0;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
      if (!kPaged && lk - j * kBN < kBN) {
        // Packed layout, last tile of the sequence: the rows behind it belong to the next sequence
        // (or were zero-filled past the end of the tensor).  Their probabilities are 0, but 0 x NaN
        // is NaN, so the rows are cleared as the reference's predicated loads clear them
        // (flash_fwd_kernel.h, Clear_OOB_MN).  A token row is 128 B in each panel (two panels; one
        // in a CTA pair, where the other CTA clears its own); the swizzle only permutes bytes
        // inside a row.
        const int valid = lk - j * kBN;
        uint8_t *vt = sKV + (i_v % kKvStages) * kStageBytes;
        constexpr int kPieces = kPair ? 8 : 16;  // 16-byte pieces of a token row held by this CTA
        for (int idx = valid * kPieces + lane; idx < kBN * kPieces; idx += 32) {
          const int r = idx / kPieces, c = idx % kPieces;
          *reinterpret_cast<uint4 *>(vt + (c >> 3) * kPanelBytes + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
      if (j < nt0) {
        if (!wait_p(0, j)) break;
        issue_pv(0, i_v, j == 0, j == nt0 - 1);
      }
      if (j + 1 < nt0) {
        if (!wait_kv(i_kn)) break;
        issue_s(0, i_kn);
      }
      if (j < nt1) {
        if (!wait_p(1, j)) break;
        issue_pv(1, i_v, j == 0, j == nt1 - 1);
      }
      release(i_v);
      if (j + 1 < nt1) {
        if (!wait_kv(i_kn)) break;
        issue_s(1, i_kn);
      }
      if (j + 1 < nmax) release(i_kn);
    }
    if (!ok && lane == 0) sh->aborted = 1;
  } else {
    // ---------------------------------------------------------------- softmax / epilogue -----
    const int t = warp >> 2;            // tile of this warpgroup
    const int quad = warp & 3;          // TMEM lane quadrant this warp may access
    const int wtid = tid - t * 128;     // thread index inside the warpgroup
    const TileInfo T = tiles[t];
    uint8_t *sQt = sQ + t * kTileBytes;
    const int row = quad * 32 + lane;
    const int qr = T.m0 + row;
    int lim_row = lk;
    if (p.causal) lim_row = min(lk, qr + 1 + lk - lq);
    const uint32_t t_s = tmem_base + t * 128 + ((uint32_t)(quad * 32) << 16);
    const uint32_t t_o = tmem_base + kOCol + t * 128 + ((uint32_t)(quad * 32) << 16);
    const float sc = p.scale_log2e;
    float m_used = -INFINITY, m_next = -INFINITY, l_sum = 0.f;
    bool ok = true, pending = false;

    for (int j = 0; j < T.n_tiles; ++j) {
      ok = mbar_wait_abortable(&sh->s_full[t], (uint32_t)j & 1u, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int n0 = j * kBN;
      // A rescale that the previous tile found necessary but left for now: the previous P V has
      // completed (s_full of this tile is committed after it), so O can be touched.
      if (__any_sync(0xffffffffu, pending)) {
        float alpha = 1.f;
        if (pending) {
          alpha = fast_exp2(m_used - m_next);
          m_used = m_next;
          l_sum *= alpha;
          pending = false;
        }
        uint32_t o[32];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          tmem_ld32(t_o + 32 * c4, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(t_o + 32 * c4, o);
        }
        tmem_wait_st();
      }

      const bool full_tile = n0 + kBN <= lim_row;
      // rows that have not seen a single column so far have no reference yet: exact path, except on
      // the first tile, which takes its reference from its own first 32 columns (below)
      bool exact_path = (j > 0) && __any_sync(0xffffffffu, m_used == -INFINITY);
      if (!exact_path) {
        // ---- single pass against the running reference m_used --------------------------------
        // P is computed for the whole row in registers while S is still intact; if some score
        // left the reference so far behind that the row sum nears the end of the fp32 range the tile
        // is redone exactly; if the row sum shows a score 2^8 above the reference (see below), the
        // reference moves after this tile's P V (pending).
        uint32_t pk[64];
        uint32_t ra[32], rb[32];
        float l0 = 0.f, l1 = 0.f;
        uint64_t acc2 = pack_f32x2(0.f, 0.f);
        tmem_ld32(t_s, ra);
        if (j == 0) {
          // First tile: the reference is the largest visible score among the first 32 columns (the
          // visible columns of a row are a prefix, so a row that sees nothing here sees nothing in
          // the tile).  If the rest of the tile lies far above it, the row sum says so as usual.
          tmem_wait_ld();
          float mx = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < lim_row) mx = fmaxf(mx, __uint_as_float(ra[i]));
          m_used = mx * sc;  // scale > 0 keeps the order
        }
        const float ref = (m_used == -INFINITY) ? 0.f : m_used;
        const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(-ref, -ref);
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          tmem_wait_ld();
          uint32_t(&cur)[32] = (c4 & 1) ? rb : ra;
          uint32_t(&nxt)[32] = (c4 & 1) ? ra : rb;
          if (c4 < 3) tmem_ld32(t_s + 32 * (c4 + 1), nxt);
          if (full_tile) {
            // packed fp32 pairs: one FMA and one add per two scores
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(cur[i]), __uint_as_float(cur[i + 1])), sc2, nm2);
              float x0, x1;
              unpack_f32x2(x, x0, x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              acc2 = add_f32x2(acc2, pack_f32x2(p0, p1));
              pk[16 * c4 + (i >> 1)] = pack_bf16(p0, p1);
            }
          } else {
            const int cb = n0 + 32 * c4;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(cur[i]), __uint_as_float(cur[i + 1])), sc2, nm2);
              float x0, x1;
              unpack_f32x2(x, x0, x1);
              const float p0 = fast_exp2((cb + i < lim_row) ? x0 : -INFINITY);
              const float p1 = fast_exp2((cb + i + 1 < lim_row) ? x1 : -INFINITY);
              acc2 = add_f32x2(acc2, pack_f32x2(p0, p1));
              pk[16 * c4 + (i >> 1)] = pack_bf16(p0, p1);
            }
          }
        }
        // The tile's row sum tells whether the reference is still good: every score at or below it
        // gives a sum of at most 128, one score 2^8 above it a sum above 256, and a sum that left
        // the fp32 range (or is NaN) means the tile has to be redone against its exact maximum.
        {
          float a0, a1;
          unpack_f32x2(acc2, a0, a1);
          l0 += a0;
          l1 += a1;
        }
        const float l_tile = l0 + l1;
        if (__any_sync(0xffffffffu, !(l_tile < kDangerSum))) {
          exact_path = true;  // S is untouched: redo the tile with an exact maximum
        } else {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4)
            tmem_st16(t_s + 16 * c4, *reinterpret_cast<uint32_t(*)[16]>(&pk[16 * c4]));
          l_sum += l_tile;
          if (l_tile > kRescaleSum) {
            // log2 of the sum bounds the largest score from above (by at most 7): a reference a few
            // powers of two above the maximum costs bf16 and fp32 nothing
            pending = true;
            m_next = m_used + __log2f(l_tile);
          }
        }
      }
      if (exact_path) {
        uint32_t r[32];
        // pass 1: row max of the raw scores over visible columns
        float mx = -INFINITY;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          tmem_ld32(t_s + 32 * c4, r);
          tmem_wait_ld();
          const int cb = n0 + 32 * c4;
          if (cb + 32 <= lim_row) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cb + i < lim_row) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
        mx *= sc;  // scale > 0, so the order is preserved

        // immediate rescale of the running output
        if (j == 0) {
          m_used = mx;
        } else {
          const bool need = mx > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            float alpha = 1.f;
            if (need) {
              alpha = fast_exp2(m_used - mx);  // 0 when nothing was visible so far
              m_used = mx;
              l_sum *= alpha;
            }
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              tmem_ld32(t_o + 32 * c4, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st32(t_o + 32 * c4, r);
            }
            tmem_wait_st();
          }
        }
        const float base = (m_used == -INFINITY) ? 0.f : m_used;

        // pass 2: p = exp2(s * scale - base), row sum, bf16 P over the S columns
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          tmem_ld32(t_s + 32 * c4, r);
          tmem_wait_ld();
          const int cb = n0 + 32 * c4;
          uint32_t pk[16];
          if (cb + 32 <= lim_row) {
            const uint64_t sc2 = pack_f32x2(sc, sc), nb2 = pack_f32x2(-base, -base);
            uint64_t acc2 = pack_f32x2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2, nb2), x0, x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              acc2 = add_f32x2(acc2, pack_f32x2(p0, p1));
              pk[i >> 1] = pack_bf16(p0, p1);
            }
            float a0, a1;
            unpack_f32x2(acc2, a0, a1);
            l_sum += a0 + a1;
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = (cb + i < lim_row) ? fast_exp2(fmaf(__uint_as_float(r[i]), sc, -base)) : 0.f;
              const float p1 = (cb + i + 1 < lim_row) ? fast_exp2(fmaf(__uint_as_float(r[i + 1]), sc, -base)) : 0.f;
              l_sum += p0 + p1;
              pk[i >> 1] = pack_bf16(p0, p1);
            }
          }
          tmem_st16(t_s + 16 * c4, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kPair && !leader) mbar_arrive_cluster(&sh->p_ready[t], 0);  // the leader issues this CTA's P V too
        else mbar_arrive(&sh->p_ready[t]);
      }
    }


    if (T.n_tiles == 0) ok = false;
    if (ok) {
      ok = mbar_wait_abortable(&sh->o_full[t], 0, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l_sum > 0.f ? __fdividef(1.f, l_sum) : 0.f;
      // staging tile over the Q buffer in the layout Q arrived in: two panels of [128 rows][64 bf16]
      // with the 128-byte swizzle (16-byte chunk c of a row sits at chunk c ^ (row & 7)), so that a
      // TMA store can take it as it is
      uint8_t *stage = sQt;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t r[32];
        tmem_ld32(t_o + 32 * c4, r);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[8 * q + 0]) * inv, __uint_as_float(r[8 * q + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(r[8 * q + 2]) * inv, __uint_as_float(r[8 * q + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(r[8 * q + 4]) * inv, __uint_as_float(r[8 * q + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(r[8 * q + 6]) * inv, __uint_as_float(r[8 * q + 7]) * inv);
          const int chunk = 4 * c4 + q;
          *reinterpret_cast<uint4 *>(stage + (chunk >> 3) * kPanelBytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4)) = v;
        }
      }
      // the four warps meet on an mbarrier (bounded wait) rather than a hardware barrier, so a
      // warp that unwound early cannot leave the others waiting forever
      fence_proxy_async_smem();  // a TMA store may read what this thread just wrote
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->staged[t]);
      ok = __all_sync(0xffffffffu, mbar_wait(&sh->staged[t], 0, p.status));
    }
    // A tile whose 128 rows all belong to this sequence, or whose sequence ends exactly where the
    // tensor ends (the copy is clipped there), goes out as two TMA stores; any other tile must not
    // touch rows that are not its own and is written row by row.
    const bool whole = p.tma_store && (T.rows == kBM || q0 + lq == p.total_q);
    if (ok && whole) {
      if (wtid == 0) {
        for (int w = 0; w < p.world; ++w) {  // peers' buffers are plain global addresses to the engine
          tma_store_3d(&tmap_o.m[w], sQt, 0, p.out_head0 + T.h, q0 + T.m0);
          tma_store_3d(&tmap_o.m[w], sQt + kPanelBytes, 64, p.out_head0 + T.h, q0 + T.m0);
        }
        // shared memory must outlive the engine's reads; with peers the writes themselves are
        // awaited too, so that they are done when this grid is and the barrier kernel may signal
        if (p.world > 1) tma_store_commit_and_wait_all(); else tma_store_commit_and_wait_read();
      }
    } else if (ok) {
      const uint8_t *stage = sQt;
      const int64_t obase = (int64_t)(q0 + T.m0) * p.o_tok_stride + (int64_t)(p.out_head0 + T.h) * p.o_head_stride;
#pragma unroll 4
      for (int it = 0; it < 16; ++it) {
        const int rr = it * 8 + (wtid >> 4), chunk = wtid & 15;
        if (rr < T.rows) {
          const uint4 v = *reinterpret_cast<const uint4 *>(stage + (chunk >> 3) * kPanelBytes + rr * 128 + (((chunk & 7) ^ (rr & 7)) << 4));
          const int64_t off = obase + (int64_t)rr * p.o_tok_stride + chunk * 8;
          for (int w = 0; w < p.world; ++w) *reinterpret_cast<uint4 *>(p.out[w] + off) = v;
        }
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------------
  tc_fence_before();
  __syncwarp();
  if (warp == Cfg::kMmaWarp && sh->aborted) {
    // bounded wait for whatever the tensor pipe still owes before the columns are released (only
    // the issuing CTA sets the flag)
    if (lane == 0) tc_commit(&sh->drain);
    __syncwarp();
    mbar_wait(&sh->drain, 0, p.status);
  }
  // pairs: neither CTA may leave (its shared and tensor memory are operands of the other's MMAs)
  // before both are through
  if (kPair) cluster_sync_all();
  else __syncthreads();
  if (warp == Cfg::kMmaWarp) {
    if (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Generic tiled map over bf16 data: dims/box innermost first, strides (bytes) for dims 1..rank-1.
static char *make_tmap_nd(const char *fn, CUtensorMap *map, const void *base, int rank,
                          const cuuint64_t *dims, const cuuint64_t *strides, const cuuint32_t *box,
                          CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = encode_fn();
  AICI_CHECK(enc != nullptr, "%s: cuTensorMapEncodeTiled is not available from the driver", fn);
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void *>(base), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  AICI_CHECK(r == CUDA_SUCCESS, "%s: cuTensorMapEncodeTiled failed with code %d", fn, (int)r);
  return nullptr;
}

// Encoded maps are kept in a small table keyed by everything that went into them (base address,
// extents, strides, kind), guarded by a mutex: a serving loop calls with the same buffers step after
// step, and an encode through the driver costs about as much as the launch itself.  A map depends
// on nothing but its key, so an entry can never be stale; the oldest entry is overwritten when the
// table is full.
struct TmapKey {
  const void *base;
  int64_t a, b, c, d;
  int kind;
  bool operator==(const TmapKey &o) const {
    return base == o.base && a == o.a && b == o.b && c == o.c && d == o.d && kind == o.kind;
  }
};
constexpr int kTmapCacheSize = 64;
struct TmapCache {
  std::mutex mu;
  TmapKey keys[kTmapCacheSize];
  CUtensorMap maps[kTmapCacheSize];
  int used = 0, next = 0;
  bool find(const TmapKey &k, CUtensorMap *out) {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
      if (keys[i] == k) {
        *out = maps[i];
        return true;
      }
    return false;
  }
  void put(const TmapKey &k, const CUtensorMap &m) {
    std::lock_guard<std::mutex> lock(mu);
    const int i = used < kTmapCacheSize ? used++ : (next++ % kTmapCacheSize);
    keys[i] = k;
    maps[i] = m;
  }
};
static TmapCache g_tmap_cache;

// [tokens, heads, 128] bf16 with element strides -> 3-D map, box = 64 (d) x 1 (head) x box_rows (tokens;
// 128, or 64 for the key half-tiles of the CTA-pair shape).
static char *make_tmap(const char *fn, CUtensorMap *map, const void *base, int64_t tokens, int heads,
                       int64_t tok_stride, int64_t head_stride, int box_rows = kBM) {
  const TmapKey key = {base, tokens, heads, tok_stride, head_stride, box_rows == kBM ? 0 : 3};
  if (g_tmap_cache.find(key, map)) return nullptr;
  cuuint64_t dims[3] = {(cuuint64_t)kHD, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)head_stride * 2, (cuuint64_t)tok_stride * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  if (char *e = make_tmap_nd(fn, map, base, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
  g_tmap_cache.put(key, *map);
  return nullptr;
}

// Paged caches: kind 1 = key cache (5-D, one half block per box), kind 2 = value cache (4-D, one
// block per box, 32-byte swizzle).
static char *make_cache_tmap(const char *fn, CUtensorMap *map, const void *base, bool value,
                             int num_kv_heads, int64_t num_blocks, int64_t kv_head_stride,
                             int64_t kv_block_stride) {
  const TmapKey key = {base, num_kv_heads, num_blocks, kv_head_stride, kv_block_stride, value ? 2 : 1};
  if (g_tmap_cache.find(key, map)) return nullptr;
  if (!value) {  // [blk][h][c = 16][tok = 16][e = 8]: box = 8 tokens of all chunks
    cuuint64_t dims[5] = {8, 16, 16, (cuuint64_t)num_kv_heads, (cuuint64_t)num_blocks};
    cuuint64_t str[4] = {16, 256, (cuuint64_t)kv_head_stride * 2, (cuuint64_t)kv_block_stride * 2};
    cuuint32_t box[5] = {8, 8, 16, 1, 1};
    if (char *e = make_tmap_nd(fn, map, base, 5, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return e;
  } else {  // [blk][h][d = 128][tok = 16]: box = one block, rows of 32 bytes
    cuuint64_t dims[4] = {16, 128, (cuuint64_t)num_kv_heads, (cuuint64_t)num_blocks};
    cuuint64_t str[3] = {32, (cuuint64_t)kv_head_stride * 2, (cuuint64_t)kv_block_stride * 2};
    cuuint32_t box[4] = {16, 128, 1, 1};
    if (char *e = make_tmap_nd(fn, map, base, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_32B)) return e;
  }
  g_tmap_cache.put(key, *map);
  return nullptr;
}

// Sequences up to this many keys take the one-tile shape (two CTAs per SM), longer ones the
// two-tile shape: with few key tiles per query tile a CTA's fixed cost (fill and drain, about as long
// as three key tiles) is what two resident CTAs hide; with many, sharing each K/V tile between two
// query tiles (half the shared-memory traffic) is worth more.
#ifndef AICI_PREFILL_ONE_TILE_MAX_K
#define AICI_PREFILL_ONE_TILE_MAX_K 2048
#endif

template <bool kPaged, int kShape>
static char *launch_prefill_shape(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                                  const OutMaps &to, PrefillParams &p, int num_heads, int batch,
                                  int max_seqlen_q, cudaStream_t stream) {
  using Cfg = PrefillCfg<kShape>;
  static OncePerDevice once;
  if (char *e = once.run([]() -> char * {
        AICI_CUDA(cudaFuncSetAttribute(varlen_prefill_kernel<kPaged, kShape>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        return nullptr;
      }))
    return e;
  const int mblocks = (max_seqlen_q + kBM - 1) / kBM;
  dim3 grid;
  if (Cfg::kTiles == 1) {
    grid = dim3(num_heads, batch, mblocks);
  } else {
    // two tiles per CTA: two heads of one kv group when the group is even (always so for CTA pairs,
    // whose two CTAs are neighbours in x: four heads of one kv head), else two row tiles
    p.pair_heads = (Cfg::kPair || p.group % 2 == 0) ? 1 : 0;
    grid = dim3(p.pair_heads ? num_heads / 2 : num_heads, batch, p.pair_heads ? mblocks : (mblocks + 1) / 2);
  }
  AICI_CHECK(grid.y <= 65535 && grid.z <= 65535, "prefill: batch and row tiles must fit a grid dimension");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (Cfg::kPair) {
    // clusters of two CTAs along x: the pair works on four query heads of one kv head
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t le = cudaLaunchKernelEx(&cfg, varlen_prefill_kernel<kPaged, kShape>, tq, tk, tv, to, p);
  if (le != cudaSuccess) {
    cudaGetLastError();
    int clusters = -1, max_size = -1;
    cudaError_t e1 = cudaSuccess, e2 = cudaSuccess;
    if (Cfg::kPair) {
      e1 = cudaOccupancyMaxActiveClusters(&clusters, varlen_prefill_kernel<kPaged, kShape>, &cfg);
      cudaLaunchConfig_t probe = cfg;
      probe.attrs = nullptr;
      probe.numAttrs = 0;
      e2 = cudaOccupancyMaxPotentialClusterSize(&max_size, varlen_prefill_kernel<kPaged, kShape>, &probe);
      cudaGetLastError();
    }
    return err("prefill launch (shape %d, grid %u x %u x %u, %d threads, %d bytes of shared memory) failed: %s "
               "[active clusters %d (%s), largest cluster %d (%s)]",
               kShape, grid.x, grid.y, grid.z, Cfg::kThreads, Cfg::kSmemBytes, cudaGetErrorString(le), clusters,
               cudaGetErrorString(e1), max_size, cudaGetErrorString(e2));
  }
  return nullptr;
}

// Which shape a call takes.  `forced` = 0: by sequence length -- shape 1 up to
// AICI_PREFILL_ONE_TILE_MAX_K keys, shape 2 above; the CTA-pair shape is never chosen by itself (on
// the long-context benchmark it runs at 0.83 of shape 2: what it saves in shared-memory reads it
// loses to the cross-SM hand-over between the softmax warps and the issuing thread).  forced = 1, 2,
// 3: that shape, for tests and comparisons; 3 needs packed K/V and four query heads per kv head in
// one CTA pair (group a multiple of 4).
static char *pick_shape(const char *fn, int forced, bool paged, int num_heads, int group, int max_seqlen_k,
                        int *shape) {
  AICI_CHECK(forced >= 0 && forced <= 3, "%s: shape must be 0 (automatic), 1, 2 or 3", fn);
  AICI_CHECK(forced != 3 || (!paged && group % 4 == 0 && num_heads % 4 == 0),
             "%s: the CTA-pair shape needs packed keys/values and a group size that is a multiple of 4", fn);
  *shape = forced != 0 ? forced : (max_seqlen_k <= AICI_PREFILL_ONE_TILE_MAX_K ? 1 : 2);
  return nullptr;
}

template <bool kPaged>
static char *launch_prefill(int shape, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                            const OutMaps &to, PrefillParams &p, int num_heads, int batch, int max_seqlen_q,
                            cudaStream_t stream) {
  p.pair_heads = 0;
  if (shape == 1)
    return launch_prefill_shape<kPaged, 1>(tq, tk, tv, to, p, num_heads, batch, max_seqlen_q, stream);
  if constexpr (!kPaged) {
    if (shape == 3)
      return launch_prefill_shape<false, 3>(tq, tk, tv, to, p, num_heads, batch, max_seqlen_q, stream);
  }
  return launch_prefill_shape<kPaged, 2>(tq, tk, tv, to, p, num_heads, batch, max_seqlen_q, stream);
}

}  // namespace aici

using namespace aici;

static char *mha_varlen_fwd_impl(const char *fn, void *const *outs, int world, int out_head0, const void *q,
                                 const void *k, const void *v,
                                     const int32_t *cu_seqlens_q, const int32_t *cu_seqlens_k,
                                     int batch, int total_q, int total_k, int num_heads,
                                     int num_heads_k, int head_size, int max_seqlen_q,
                                     int max_seqlen_k, int64_t q_tok_stride, int64_t q_head_stride,
                                     int64_t k_tok_stride, int64_t k_head_stride,
                                     int64_t v_tok_stride, int64_t v_head_stride,
                                     int64_t o_tok_stride, int64_t o_head_stride,
                                     float softmax_scale, int is_causal, int dtype,
                                     aici_stream_t stream, int forced_shape = 0) {
  void *out = outs[0];
  for (int w = 1; w < world; ++w)
    AICI_CHECK(outs[w] != nullptr && (uintptr_t)outs[w] % 16 == 0,
               "%s: peer output %d must be non-NULL and 16-byte aligned", fn, w);
  AICI_CHECK(dtype == AICI_DTYPE_BF16, "%s: FlashAttention only support bf16 data type (dtype=%d)", fn, dtype);
  AICI_CHECK(batch > 0, "%s: batch size must be positive", fn);
  AICI_CHECK(head_size == kHD, "%s: head_size must be 128 (got %d)", fn, head_size);
  AICI_CHECK(num_heads > 0 && num_heads_k > 0 && num_heads % num_heads_k == 0,
             "%s: Number of heads in key/value must divide number of heads in query", fn);
  AICI_CHECK(total_q >= 0 && total_k >= 0 && max_seqlen_q >= 0 && max_seqlen_k >= 0, "%s: negative size", fn);
  AICI_CHECK(softmax_scale > 0.f, "%s: softmax_scale must be positive", fn);
  AICI_CHECK(batch <= 65535 && num_heads <= 65535, "%s: batch and num_heads must fit a grid dimension", fn);
  if (total_q == 0 || max_seqlen_q == 0) return nullptr;
  AICI_CHECK(out && q && cu_seqlens_q && cu_seqlens_k, "%s: NULL pointer", fn);
  AICI_CHECK(total_k == 0 || (k && v), "%s: NULL pointer", fn);
  AICI_CHECK(((uintptr_t)out | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 16 == 0,
             "%s: tensors must be 16-byte aligned", fn);
  const int64_t strides[8] = {q_tok_stride, q_head_stride, k_tok_stride, k_head_stride,
                              v_tok_stride, v_head_stride, o_tok_stride, o_head_stride};
  for (int i = 0; i < 8; ++i)
    AICI_CHECK(strides[i] >= kHD && strides[i] % 8 == 0,
               "%s: token and head strides must be multiples of 8 elements and at least head_size", fn);
  // this rank's heads must fit between two token rows of the output buffers
  AICI_CHECK(o_head_stride > o_tok_stride ||
                 (int64_t)(out_head0 + num_heads - 1) * o_head_stride + kHD <= o_tok_stride,
             "%s: heads [%d, %d) do not fit an output row of %lld elements", fn, out_head0,
             out_head0 + num_heads, (long long)o_tok_stride);
  int shape = 0;
  if (char *e = pick_shape(fn, forced_shape, false, num_heads, num_heads / num_heads_k, max_seqlen_k, &shape)) return e;
  if (char *e = check_on_current_device(fn, "q", q)) return e;
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);

  CUtensorMap tq, tk, tv;
  if (char *e = make_tmap(fn, &tq, q, total_q, num_heads, q_tok_stride, q_head_stride)) return e;
  // an empty key tensor still needs a valid map; no tile of it is ever requested
  const void *kk = total_k > 0 ? k : q;
  const void *vv = total_k > 0 ? v : q;
  const int64_t tk_rows = total_k > 0 ? total_k : 1;
  // the CTA-pair shape loads key tiles in halves of 64 tokens
  if (char *e = make_tmap(fn, &tk, kk, tk_rows, num_heads_k, k_tok_stride, k_head_stride, shape == 3 ? 64 : kBM)) return e;
  if (char *e = make_tmap(fn, &tv, vv, tk_rows, num_heads_k, v_tok_stride, v_head_stride)) return e;

  PrefillParams p;
  for (int i = 0; i < 8; ++i) p.out[i] = static_cast<__nv_bfloat16 *>(i < world ? outs[i] : nullptr);
  p.world = world;
  p.out_head0 = out_head0;
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.o_tok_stride = o_tok_stride;
  p.o_head_stride = o_head_stride;
  p.group = num_heads / num_heads_k;
  p.causal = is_causal ? 1 : 0;
  p.scale_log2e = softmax_scale * 1.4426950408889634f;
  p.status = st;
  p.block_tables = nullptr;
  p.k_lens = nullptr;
  p.max_blocks = 0;
  p.num_blocks = 0;
  // every output buffer gets a tensor map like the query's; this rank's heads start at out_head0
  OutMaps to = {};
  p.total_q = total_q;
  p.tma_store = 1;
  for (int w = 0; w < world; ++w)  // the kernel reads m[w] for w < world only
    if (char *e = make_tmap(fn, &to.m[w], outs[w], total_q, out_head0 + num_heads, o_tok_stride, o_head_stride))
      return e;
  return launch_prefill<false>(shape, tq, tk, tv, to, p, num_heads, batch, max_seqlen_q,
                               static_cast<cudaStream_t>(stream));
}

extern "C" char *aici_mha_varlen_fwd(void *out, const void *q, const void *k, const void *v,
                                     const int32_t *cu_seqlens_q, const int32_t *cu_seqlens_k,
                                     int batch, int total_q, int total_k, int num_heads,
                                     int num_heads_k, int head_size, int max_seqlen_q,
                                     int max_seqlen_k, int64_t q_tok_stride, int64_t q_head_stride,
                                     int64_t k_tok_stride, int64_t k_head_stride,
                                     int64_t v_tok_stride, int64_t v_head_stride,
                                     int64_t o_tok_stride, int64_t o_head_stride,
                                     float softmax_scale, int is_causal, int dtype,
                                     aici_stream_t stream) {
  void *outs[1] = {out};
  return mha_varlen_fwd_impl("aici_mha_varlen_fwd", outs, 1, 0, q, k, v, cu_seqlens_q, cu_seqlens_k, batch,
                             total_q, total_k, num_heads, num_heads_k, head_size, max_seqlen_q,
                             max_seqlen_k, q_tok_stride, q_head_stride, k_tok_stride, k_head_stride,
                             v_tok_stride, v_head_stride, o_tok_stride, o_head_stride, softmax_scale,
                             is_causal, dtype, stream);
}

// aici_mha_varlen_fwd with the kernel shape chosen by the caller instead of by sequence length (test
// and benchmark hook): 0 = automatic, 1 = one query tile per CTA and two CTAs per SM, 2 = two query
// tiles per CTA, 3 = shape 2 on CTA pairs with two-SM MMAs (tcgen05 cta_group::2).
extern "C" char *aici_mha_varlen_fwd_shape(void *out, const void *q, const void *k, const void *v,
                                           const int32_t *cu_seqlens_q, const int32_t *cu_seqlens_k,
                                           int batch, int total_q, int total_k, int num_heads,
                                           int num_heads_k, int head_size, int max_seqlen_q,
                                           int max_seqlen_k, int64_t q_tok_stride, int64_t q_head_stride,
                                           int64_t k_tok_stride, int64_t k_head_stride,
                                           int64_t v_tok_stride, int64_t v_head_stride,
                                           int64_t o_tok_stride, int64_t o_head_stride,
                                           float softmax_scale, int is_causal, int shape, int dtype,
                                           aici_stream_t stream) {
  void *outs[1] = {out};
  return mha_varlen_fwd_impl("aici_mha_varlen_fwd_shape", outs, 1, 0, q, k, v, cu_seqlens_q, cu_seqlens_k,
                             batch, total_q, total_k, num_heads, num_heads_k, head_size, max_seqlen_q,
                             max_seqlen_k, q_tok_stride, q_head_stride, k_tok_stride, k_head_stride,
                             v_tok_stride, v_head_stride, o_tok_stride, o_head_stride, softmax_scale,
                             is_causal, dtype, stream, shape);
}

// Prefill attention whose epilogue is the head-output gather: each finished output tile is stored
// at head index head0 + h of the [total_q, total_heads, 128] buffer of EVERY rank (plain stores to
// peer-mapped memory over NVLink, pushed tile by tile while later tiles are still computing), so
// the gather hides under the attention math; the ranks only need a barrier before reading.
extern "C" char *aici_mha_varlen_fwd_peers(void *const *outs, int world, int head0, const void *q,
                                           const void *k, const void *v, const int32_t *cu_seqlens_q,
                                           const int32_t *cu_seqlens_k, int batch, int total_q,
                                           int total_k, int num_heads, int num_heads_k, int head_size,
                                           int max_seqlen_q, int max_seqlen_k, int64_t q_tok_stride,
                                           int64_t q_head_stride, int64_t k_tok_stride,
                                           int64_t k_head_stride, int64_t v_tok_stride,
                                           int64_t v_head_stride, int64_t o_tok_stride,
                                           int64_t o_head_stride, float softmax_scale, int is_causal,
                                           int dtype, aici_stream_t stream) {
  const char *fn = "aici_mha_varlen_fwd_peers";
  AICI_CHECK(outs != nullptr && world >= 1 && world <= 8, "%s: world must be 1..8", fn);
  AICI_CHECK(head0 >= 0, "%s: negative head offset", fn);
  return mha_varlen_fwd_impl(fn, outs, world, head0, q, k, v, cu_seqlens_q, cu_seqlens_k, batch, total_q,
                             total_k, num_heads, num_heads_k, head_size, max_seqlen_q, max_seqlen_k,
                             q_tok_stride, q_head_stride, k_tok_stride, k_head_stride, v_tok_stride,
                             v_head_stride, o_tok_stride, o_head_stride, softmax_scale, is_causal, dtype,
                             stream);
}

extern "C" char *aici_mha_varlen_paged_fwd(void *out, const void *q, const void *key_cache,
                                           const void *value_cache, const int32_t *cu_seqlens_q,
                                           const int32_t *context_lens, const int32_t *block_tables,
                                           int batch, int total_q, int num_heads, int num_kv_heads,
                                           int head_size, int block_size, int max_seqlen_q,
                                           int max_context_len, int max_num_blocks_per_seq,
                                           int64_t num_blocks, int64_t q_tok_stride,
                                           int64_t q_head_stride, int64_t o_tok_stride,
                                           int64_t o_head_stride, int64_t kv_block_stride,
                                           int64_t kv_head_stride, float softmax_scale, int is_causal,
                                           int dtype, aici_stream_t stream) {
  const char *fn = "aici_mha_varlen_paged_fwd";
  AICI_CHECK(dtype == AICI_DTYPE_BF16, "%s: only bf16 is supported (dtype=%d)", fn, dtype);
  AICI_CHECK(batch > 0, "%s: batch size must be positive", fn);
  AICI_CHECK(head_size == kHD, "%s: head_size must be 128 (got %d)", fn, head_size);
  AICI_CHECK(block_size == 16, "%s: block_size must be 16 (got %d)", fn, block_size);
  AICI_CHECK(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0,
             "%s: Number of heads in key/value must divide number of heads in query", fn);
  AICI_CHECK(total_q >= 0 && max_seqlen_q >= 0 && max_context_len >= 0 && max_num_blocks_per_seq >= 0,
             "%s: negative size", fn);
  AICI_CHECK(softmax_scale > 0.f, "%s: softmax_scale must be positive", fn);
  AICI_CHECK(batch <= 65535 && num_heads <= 65535, "%s: batch and num_heads must fit a grid dimension", fn);
  if (total_q == 0 || max_seqlen_q == 0) return nullptr;
  AICI_CHECK(out && q && key_cache && value_cache && cu_seqlens_q && context_lens && block_tables,
             "%s: NULL pointer", fn);
  AICI_CHECK(num_blocks > 0, "%s: num_blocks must be positive", fn);
  AICI_CHECK(((uintptr_t)out | (uintptr_t)q | (uintptr_t)key_cache | (uintptr_t)value_cache) % 16 == 0,
             "%s: tensors must be 16-byte aligned", fn);
  const int64_t strides[4] = {q_tok_stride, q_head_stride, o_tok_stride, o_head_stride};
  for (int i = 0; i < 4; ++i)
    AICI_CHECK(strides[i] >= kHD && strides[i] % 8 == 0,
               "%s: token and head strides must be multiples of 8 elements and at least head_size", fn);
  AICI_CHECK(kv_head_stride == kHD * 16 && kv_block_stride % 8 == 0 &&
                 kv_block_stride >= (int64_t)num_kv_heads * kHD * 16,
             "%s: cache must be [blocks, kv_heads, 128/8, 16, 8] with contiguous head tiles", fn);
  if (char *e = check_on_current_device(fn, "q", q)) return e;
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);

  CUtensorMap tq, tk, tv;
  if (char *e = make_tmap(fn, &tq, q, total_q, num_heads, q_tok_stride, q_head_stride)) return e;
  if (char *e = make_cache_tmap(fn, &tk, key_cache, false, num_kv_heads, num_blocks, kv_head_stride, kv_block_stride))
    return e;
  if (char *e = make_cache_tmap(fn, &tv, value_cache, true, num_kv_heads, num_blocks, kv_head_stride, kv_block_stride))
    return e;
  PrefillParams p;
  for (int i = 0; i < 8; ++i) p.out[i] = i == 0 ? static_cast<__nv_bfloat16 *>(out) : nullptr;
  p.world = 1;
  p.out_head0 = 0;
  p.cu_q = cu_seqlens_q;
  p.cu_k = nullptr;
  p.o_tok_stride = o_tok_stride;
  p.o_head_stride = o_head_stride;
  p.group = num_heads / num_kv_heads;
  p.causal = is_causal ? 1 : 0;
  p.scale_log2e = softmax_scale * 1.4426950408889634f;
  p.status = st;
  p.block_tables = block_tables;
  p.k_lens = context_lens;
  p.max_blocks = max_num_blocks_per_seq;
  p.num_blocks = num_blocks;
  OutMaps to = {};
  p.total_q = total_q;
  p.tma_store = 1;
  if (char *e = make_tmap(fn, &to.m[0], out, total_q, num_heads, o_tok_stride, o_head_stride)) return e;
  int shape = 0;
  if (char *e = pick_shape(fn, 0, true, num_heads, num_heads / num_kv_heads, max_context_len, &shape)) return e;
  return launch_prefill<true>(shape, tq, tk, tv, to, p, num_heads, batch, max_seqlen_q,
                              static_cast<cudaStream_t>(stream));
}
