// KV-cache operations for sm_100a: reshape_and_cache, gather_cached_kv, copy_blocks.
//
// All three are pure data movement and bit-exact.  Index math follows
// rllm/tch-cuda/kernels/vllm/cache_kernels.cu (:168-213 scatter, :301-373 gather,
// :55-81 block copy); the traversal does not: every global access is a 16-byte vector, the
// value tile is transposed through shared memory so that runs of consecutive slots are
// written along block_size as whole 16-byte pieces, and the block copy moves 16 bytes per
// thread per access with the layer/pair tables optionally passed as kernel arguments.
#include "common.cuh"

namespace aici {

constexpr int kD = 128;      // head_size
constexpr int kB = 16;       // block_size (tokens per cache block)
constexpr int kX = 8;        // 16 bytes of bf16
constexpr int kTok = 16;     // tokens per CTA
constexpr int kThreads = 256;

template <bool kSlot64>
__device__ __forceinline__ int64_t load_slot(const void *slots, int64_t i) {
  if (kSlot64) return static_cast<const int64_t *>(slots)[i];
  return static_cast<int64_t>(static_cast<const int32_t *>(slots)[i]);
}

// Writes the CTA's staged value tile s_v[tok][d] (kT tokens x 128) to the cache.
template <int kT>
__device__ __forceinline__ void store_value_tile(const int64_t *s_slot,
                                                 const __nv_bfloat16 (*s_v)[kD + 8],
                                                 __nv_bfloat16 *__restrict__ value_cache,
                                                 int num_kv_heads, int h, int tid) {
  // aligned: every 8-token group is a run of consecutive slots starting at a multiple of 8 (the
  // prefill case: a sequence's tokens fill whole cache blocks in order)
  bool aligned = true;
#pragma unroll
  for (int tb = 0; tb < kT; tb += 8) {
    const int64_t s0 = s_slot[tb];
    aligned = aligned && s0 >= 0 && (s0 % 8) == 0;
#pragma unroll
    for (int j = 1; j < 8; ++j) aligned = aligned && (s_slot[tb + j] == s0 + j);
  }
  if (aligned) {
    // a warp covers 32 consecutive d of one token group: column reads hit 16 distinct banks
#pragma unroll
    for (int u = 0; u < kT / 16; ++u) {
      const int item = u * kThreads + tid;
      const int d = item & (kD - 1), tb = (item >> 7) * 8;
      const int64_t s0 = s_slot[tb];
      uint4 val;
      __nv_bfloat16 *e = reinterpret_cast<__nv_bfloat16 *>(&val);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = s_v[tb + j][d];
      const int64_t blk = s0 / kB, off = s0 % kB;
      *reinterpret_cast<uint4 *>(value_cache + ((blk * num_kv_heads + h) * kD + d) * kB + off) = val;
    }
  } else {
    // any slots (decode steps, chunks that start in the middle of a block, skipped tokens):
    // consecutive threads take the tokens of one d, so tokens with consecutive slots still land
    // in one 32-byte sector per store instruction
    const int tok = tid & (kT - 1);
    const int64_t slot = s_slot[tok];
    if (slot >= 0) {
      const int64_t blk = slot / kB, off = slot % kB;
      __nv_bfloat16 *dst = value_cache + (blk * num_kv_heads + h) * (int64_t)(kD * kB) + off;
#pragma unroll 4
      for (int d = tid / kT; d < kD; d += kThreads / kT) dst[(int64_t)d * kB] = s_v[tok][d];
    }
  }
}

// One CTA moves kT (16 or 32) consecutive tokens of one kv head.
//   K: chunk c (8 elements) of token t -> key_cache[blk][h][c][off][0..7]   (16 B vector)
//   V: element d of token t            -> value_cache[blk][h][d][off]       (2 B, 32 B apart)
// Every global load of the CTA -- the slots, the key vectors, the value vectors -- is issued before
// anything waits: where a token goes does not change what is read, so the three reads share one
// memory round trip and only the stores depend on the slots.  For V the CTA transposes its
// [kT][128] tile in shared memory; a thread then owns (d, 8-token group) pairs and writes 8 tokens
// as one 16-byte store when their slots are consecutive and 8-aligned inside one block (the prefill
// case), else element by element (decode).
template <bool kSlot64, int kT>
__global__ void __launch_bounds__(kThreads)
reshape_and_cache_kernel(const __nv_bfloat16 *__restrict__ key,
                         const __nv_bfloat16 *__restrict__ value,
                         __nv_bfloat16 *__restrict__ key_cache,
                         __nv_bfloat16 *__restrict__ value_cache,
                         const void *__restrict__ slot_mapping, int num_tokens, int num_kv_heads,
                         int64_t num_slots, int64_t key_stride, int64_t value_stride,
                         unsigned int *status) {
  __shared__ int64_t s_slot[kT];
  __shared__ __align__(16) __nv_bfloat16 s_v[kT][kD + 8];  // [tok][d], rows of 272 B
  constexpr int kPer = kT / 16;  // 16-token groups per CTA = key and value vectors per thread
  const int t0 = blockIdx.x * kT;
  const int h = blockIdx.y;
  const int tid = threadIdx.x;

  // K: thread (c, tok) of group u; 16 consecutive threads cover 16 tokens of one chunk, a warp two
  // neighbouring chunks (whole 32-byte sectors).  V: thread (tok, part); 16 threads read one row.
  uint4 kvec[kPer], vvec[kPer];
  const int kc = tid >> 4, ktok = tid & 15;
  const int vtok = tid >> 4, vpart = tid & 15;
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    kvec[u] = make_uint4(0, 0, 0, 0);
    vvec[u] = make_uint4(0, 0, 0, 0);
    if (t0 + 16 * u + ktok < num_tokens)
      kvec[u] = *reinterpret_cast<const uint4 *>(key + (int64_t)(t0 + 16 * u + ktok) * key_stride + h * kD + kc * kX);
    if (t0 + 16 * u + vtok < num_tokens)
      vvec[u] = *reinterpret_cast<const uint4 *>(value + (int64_t)(t0 + 16 * u + vtok) * value_stride + h * kD +
                                                 vpart * kX);
  }
  if (tid < kT) {
    int64_t slot = -1;
    if (t0 + tid < num_tokens) {
      slot = load_slot<kSlot64>(slot_mapping, t0 + tid);
      if (slot >= num_slots) {
        set_status(status, AICI_STATUS_BAD_SLOT);
        slot = -1;
      }
    }
    s_slot[tid] = slot;
  }
#pragma unroll
  for (int u = 0; u < kPer; ++u) *reinterpret_cast<uint4 *>(&s_v[16 * u + vtok][vpart * kX]) = vvec[u];
  __syncthreads();

#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    const int64_t slot = s_slot[16 * u + ktok];
    if (slot >= 0) {
      const int64_t blk = slot / kB, off = slot % kB;
      __nv_bfloat16 *dst = key_cache + ((blk * num_kv_heads + h) * (kD / kX) + kc) * (kB * kX) + off * kX;
      *reinterpret_cast<uint4 *>(dst) = kvec[u];
    }
  }
  store_value_tile<kT>(s_slot, s_v, value_cache, num_kv_heads, h, tid);
}

// Inverse traversal: cache -> packed key/value rows.
__global__ void __launch_bounds__(kThreads)
gather_cached_kv_kernel(__nv_bfloat16 *__restrict__ key, __nv_bfloat16 *__restrict__ value,
                        const __nv_bfloat16 *__restrict__ key_cache,
                        const __nv_bfloat16 *__restrict__ value_cache,
                        const int32_t *__restrict__ slot_mapping, int num_tokens,
                        int num_kv_heads, int64_t num_slots, int64_t key_stride,
                        int64_t value_stride, unsigned int *status) {
  __shared__ int64_t s_slot[kTok];
  __shared__ __align__(16) __nv_bfloat16 s_v[kTok][kD + 8];  // [tok][d], rows of 272 B
  const int t0 = blockIdx.x * kTok;
  const int h = blockIdx.y;
  const int tid = threadIdx.x;

  if (tid < kTok) {
    int64_t slot = -1;
    if (t0 + tid < num_tokens) {
      slot = slot_mapping[t0 + tid];
      if (slot < 0 || slot >= num_slots) {
        set_status(status, AICI_STATUS_BAD_SLOT);
        slot = -1;
      }
    }
    s_slot[tid] = slot;
  }
  __syncthreads();
  {
    const int c = tid >> 4, tok = tid & 15;
    const int64_t slot = s_slot[tok];
    if (slot >= 0) {
      const int64_t blk = slot / kB, off = slot % kB;
      const __nv_bfloat16 *src =
          key_cache + ((blk * num_kv_heads + h) * (kD / kX) + c) * (kB * kX) + off * kX;
      *reinterpret_cast<uint4 *>(key + (int64_t)(t0 + tok) * key_stride + h * kD + c * kX) =
          *reinterpret_cast<const uint4 *>(src);
    }
  }
  {
    const int d = tid & (kD - 1), half = tid >> 7;
    const int tb = half * 8;
    const int64_t s0 = s_slot[tb];
    bool run = s0 >= 0 && (s0 % 8) == 0;
#pragma unroll
    for (int j = 1; j < 8; ++j) run = run && (s_slot[tb + j] == s0 + j);
    if (run) {
      const int64_t blk = s0 / kB, off = s0 % kB;
      const uint4 val = *reinterpret_cast<const uint4 *>(
          value_cache + ((blk * num_kv_heads + h) * kD + d) * kB + off);
      const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&val);
#pragma unroll
      for (int j = 0; j < 8; ++j) s_v[tb + j][d] = e[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int64_t slot = s_slot[tb + j];
        if (slot >= 0) {
          const int64_t blk = slot / kB, off = slot % kB;
          s_v[tb + j][d] = value_cache[((blk * num_kv_heads + h) * kD + d) * kB + off];
        }
      }
    }
  }
  __syncthreads();
  {
    const int tok = tid >> 4, part = tid & 15;
    if (s_slot[tok] >= 0)
      *reinterpret_cast<uint4 *>(value + (int64_t)(t0 + tok) * value_stride + h * kD + part * kX) =
          *reinterpret_cast<const uint4 *>(&s_v[tok][part * kX]);
  }
}

// ---- copy_blocks ---------------------------------------------------------------------------
constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 8;

__device__ __forceinline__ void copy_block_16B(const uint4 *__restrict__ src,
                                               uint4 *__restrict__ dst, int n_vec) {
  for (int base = 0; base < n_vec; base += kCopyThreads * kCopyUnroll) {
    uint4 v[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const int i = base + u * kCopyThreads + threadIdx.x;
      if (i < n_vec) v[u] = src[i];
    }
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const int i = base + u * kCopyThreads + threadIdx.x;
      if (i < n_vec) dst[i] = v[u];
    }
  }
}

// grid (num_pairs, 2 * num_layers): blockIdx.y < num_layers copies a key block, else a value
// block.  Tables live in device memory (the reference's calling convention).
__global__ void __launch_bounds__(kCopyThreads)
copy_blocks_kernel(const int64_t *__restrict__ key_cache_ptrs,
                   const int64_t *__restrict__ value_cache_ptrs,
                   const int64_t *__restrict__ block_mapping, int num_layers,
                   int64_t bytes_per_block, int64_t num_blocks, unsigned int *status) {
  const int pair = blockIdx.x;
  const int layer = blockIdx.y % num_layers;
  const bool is_value = blockIdx.y >= num_layers;
  const int64_t src = block_mapping[2 * pair], dst = block_mapping[2 * pair + 1];
  if (src < 0 || dst < 0 || (num_blocks > 0 && (src >= num_blocks || dst >= num_blocks))) {
    if (threadIdx.x == 0) set_status(status, AICI_STATUS_BAD_BLOCK);
    return;
  }
  if (src == dst) return;
  char *base = reinterpret_cast<char *>(is_value ? value_cache_ptrs[layer] : key_cache_ptrs[layer]);
  copy_block_16B(reinterpret_cast<const uint4 *>(base + src * bytes_per_block),
                 reinterpret_cast<uint4 *>(base + dst * bytes_per_block),
                 static_cast<int>(bytes_per_block / 16));
}

// Same copy with the tables passed by value in the kernel-argument buffer (sm_70+ accepts
// up to 32764 bytes of arguments; this struct is 26112 bytes).
constexpr int kArgLayers = 96;
constexpr int kArgPairs = 3072;
struct CopyArgs {
  int64_t key_ptrs[kArgLayers];
  int64_t value_ptrs[kArgLayers];
  int32_t src[kArgPairs];
  int32_t dst[kArgPairs];
};
static_assert(sizeof(CopyArgs) + 64 <= 32764, "kernel arguments must stay below the 32764-byte limit");

__global__ void __launch_bounds__(kCopyThreads)
copy_blocks_args_kernel(const __grid_constant__ CopyArgs args, int num_layers,
                        int64_t bytes_per_block) {
  const int pair = blockIdx.x;
  const int layer = blockIdx.y % num_layers;
  const bool is_value = blockIdx.y >= num_layers;
  const int64_t src = args.src[pair], dst = args.dst[pair];
  if (src == dst) return;
  char *base = reinterpret_cast<char *>(is_value ? args.value_ptrs[layer] : args.key_ptrs[layer]);
  copy_block_16B(reinterpret_cast<const uint4 *>(base + src * bytes_per_block),
                 reinterpret_cast<uint4 *>(base + dst * bytes_per_block),
                 static_cast<int>(bytes_per_block / 16));
}

static char *check_cache_shape(const char *fn, int num_kv_heads, int head_size, int block_size,
                               int dtype) {
  AICI_CHECK(dtype == AICI_DTYPE_BF16, "%s: only bf16 is supported (dtype=%d)", fn, dtype);
  AICI_CHECK(head_size == kD, "%s: head_size must be 128 (got %d)", fn, head_size);
  AICI_CHECK(block_size == kB, "%s: block_size must be 16 (got %d)", fn, block_size);
  AICI_CHECK(num_kv_heads > 0 && num_kv_heads <= 65535, "%s: bad num_kv_heads %d", fn,
             num_kv_heads);
  return nullptr;
}

}  // namespace aici

using namespace aici;

extern "C" char *aici_reshape_and_cache(const void *key, const void *value, void *key_cache,
                                        void *value_cache, const void *slot_mapping,
                                        int slot_is_int64, int num_tokens, int num_kv_heads,
                                        int head_size, int block_size, int64_t num_blocks,
                                        int64_t key_stride, int64_t value_stride, int dtype,
                                        aici_stream_t stream) {
  const char *fn = "aici_reshape_and_cache";
  if (char *e = check_cache_shape(fn, num_kv_heads, head_size, block_size, dtype)) return e;
  AICI_CHECK(num_tokens >= 0, "%s: negative num_tokens", fn);
  if (num_tokens == 0) return nullptr;
  AICI_CHECK(key && value && key_cache && value_cache && slot_mapping, "%s: NULL pointer", fn);
  AICI_CHECK(num_blocks > 0, "%s: num_blocks must be positive", fn);
  AICI_CHECK(key_stride % 8 == 0 && value_stride % 8 == 0 &&
                 key_stride >= (int64_t)num_kv_heads * head_size &&
                 value_stride >= (int64_t)num_kv_heads * head_size,
             "%s: token strides must be multiples of 8 elements and cover one row", fn);
  AICI_CHECK(((uintptr_t)key | (uintptr_t)value | (uintptr_t)key_cache |
              (uintptr_t)value_cache) % 16 == 0,
             "%s: tensors must be 16-byte aligned", fn);
  if (char *e = check_on_current_device(fn, "key_cache", key_cache)) return e;
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);
  const int64_t num_slots = num_blocks * kB;
  auto k = static_cast<const __nv_bfloat16 *>(key);
  auto v = static_cast<const __nv_bfloat16 *>(value);
  auto kc = static_cast<__nv_bfloat16 *>(key_cache);
  auto vc = static_cast<__nv_bfloat16 *>(value_cache);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 32 tokens per CTA (twice the bytes in flight per thread) once that still leaves four CTAs per
  // multiprocessor; smaller calls keep 16 tokens per CTA so that more of the GPU takes part
  const bool wide = (int64_t)((num_tokens + 31) / 32) * num_kv_heads >= (int64_t)4 * sm_count();
  const int tok = wide ? 32 : 16;
  dim3 grid((num_tokens + tok - 1) / tok, num_kv_heads);
#define AICI_RAC_LAUNCH(S64, T)                                                                     \
  reshape_and_cache_kernel<S64, T><<<grid, kThreads, 0, s>>>(k, v, kc, vc, slot_mapping, num_tokens, \
                                                             num_kv_heads, num_slots, key_stride,    \
                                                             value_stride, st)
  if (slot_is_int64) {
    if (wide) AICI_RAC_LAUNCH(true, 32); else AICI_RAC_LAUNCH(true, 16);
  } else {
    if (wide) AICI_RAC_LAUNCH(false, 32); else AICI_RAC_LAUNCH(false, 16);
  }
#undef AICI_RAC_LAUNCH
  AICI_CUDA(cudaGetLastError());
  return nullptr;
}

extern "C" char *aici_gather_cached_kv(void *key, void *value, const void *key_cache,
                                       const void *value_cache, const int32_t *slot_mapping,
                                       int num_tokens, int num_kv_heads, int head_size,
                                       int block_size, int64_t num_blocks, int64_t key_stride,
                                       int64_t value_stride, int dtype, aici_stream_t stream) {
  const char *fn = "aici_gather_cached_kv";
  if (char *e = check_cache_shape(fn, num_kv_heads, head_size, block_size, dtype)) return e;
  AICI_CHECK(num_tokens >= 0, "%s: negative num_tokens", fn);
  if (num_tokens == 0) return nullptr;
  AICI_CHECK(key && value && key_cache && value_cache && slot_mapping, "%s: NULL pointer", fn);
  AICI_CHECK(num_blocks > 0, "%s: num_blocks must be positive", fn);
  AICI_CHECK(key_stride % 8 == 0 && value_stride % 8 == 0 &&
                 key_stride >= (int64_t)num_kv_heads * head_size &&
                 value_stride >= (int64_t)num_kv_heads * head_size,
             "%s: token strides must be multiples of 8 elements and cover one row", fn);
  AICI_CHECK(((uintptr_t)key | (uintptr_t)value | (uintptr_t)key_cache |
              (uintptr_t)value_cache) % 16 == 0,
             "%s: tensors must be 16-byte aligned", fn);
  if (char *e = check_on_current_device(fn, "key_cache", key_cache)) return e;
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);
  dim3 grid((num_tokens + kTok - 1) / kTok, num_kv_heads);
  gather_cached_kv_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(key), static_cast<__nv_bfloat16 *>(value),
      static_cast<const __nv_bfloat16 *>(key_cache),
      static_cast<const __nv_bfloat16 *>(value_cache), slot_mapping, num_tokens, num_kv_heads,
      num_blocks * kB, key_stride, value_stride, st);
  AICI_CUDA(cudaGetLastError());
  return nullptr;
}

static char *check_copy(const char *fn, int num_layers, int num_pairs, int64_t numel_per_block,
                        int dtype) {
  AICI_CHECK(dtype == AICI_DTYPE_BF16 || dtype == AICI_DTYPE_F16,
             "%s: cache dtype must be bf16 or f16 (dtype=%d)", fn, dtype);
  AICI_CHECK(num_layers >= 0 && num_pairs >= 0, "%s: negative count", fn);
  AICI_CHECK(numel_per_block > 0 && (numel_per_block * 2) % 16 == 0,
             "%s: a block must be a positive multiple of 16 bytes", fn);
  AICI_CHECK(num_layers <= 32767, "%s: too many layers (%d)", fn, num_layers);
  return nullptr;
}

extern "C" char *aici_copy_blocks(const int64_t *key_cache_ptrs, const int64_t *value_cache_ptrs,
                                  const int64_t *block_mapping, int num_layers, int num_pairs,
                                  int64_t numel_per_block, int64_t num_blocks, int dtype,
                                  aici_stream_t stream) {
  const char *fn = "aici_copy_blocks";
  if (char *e = check_copy(fn, num_layers, num_pairs, numel_per_block, dtype)) return e;
  if (num_layers == 0 || num_pairs == 0) return nullptr;
  AICI_CHECK(key_cache_ptrs && value_cache_ptrs && block_mapping, "%s: NULL pointer", fn);
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);
  dim3 grid(num_pairs, 2 * num_layers);
  copy_blocks_kernel<<<grid, kCopyThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      key_cache_ptrs, value_cache_ptrs, block_mapping, num_layers, numel_per_block * 2, num_blocks,
      st);
  AICI_CUDA(cudaGetLastError());
  return nullptr;
}

extern "C" char *aici_copy_blocks_host(const int64_t *key_cache_ptrs_host,
                                       const int64_t *value_cache_ptrs_host,
                                       const int64_t *block_mapping_host, int num_layers,
                                       int num_pairs, int64_t numel_per_block, int64_t num_blocks,
                                       int dtype, aici_stream_t stream) {
  const char *fn = "aici_copy_blocks_host";
  if (char *e = check_copy(fn, num_layers, num_pairs, numel_per_block, dtype)) return e;
  if (num_layers == 0 || num_pairs == 0) return nullptr;
  AICI_CHECK(key_cache_ptrs_host && value_cache_ptrs_host && block_mapping_host,
             "%s: NULL pointer", fn);
  for (int p = 0; p < num_pairs; ++p) {
    const int64_t src = block_mapping_host[2 * p], dst = block_mapping_host[2 * p + 1];
    AICI_CHECK(src >= 0 && dst >= 0 && src <= INT32_MAX && dst <= INT32_MAX &&
                   (num_blocks <= 0 || (src < num_blocks && dst < num_blocks)),
               "%s: pair %d (%lld -> %lld) is outside the cache of %lld blocks", fn, p,
               (long long)src, (long long)dst, (long long)num_blocks);
  }
  for (int l = 0; l < num_layers; ++l)
    AICI_CHECK(key_cache_ptrs_host[l] % 16 == 0 && value_cache_ptrs_host[l] % 16 == 0 &&
                   key_cache_ptrs_host[l] != 0 && value_cache_ptrs_host[l] != 0,
               "%s: layer %d cache base must be non-NULL and 16-byte aligned", fn, l);
  if (char *e = check_on_current_device(fn, "layer 0 key cache",
                                        reinterpret_cast<const void *>(key_cache_ptrs_host[0])))
    return e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int l0 = 0; l0 < num_layers; l0 += kArgLayers) {
    const int nl = num_layers - l0 < kArgLayers ? num_layers - l0 : kArgLayers;
    for (int p0 = 0; p0 < num_pairs; p0 += kArgPairs) {
      const int np = num_pairs - p0 < kArgPairs ? num_pairs - p0 : kArgPairs;
      static thread_local CopyArgs args;
      for (int l = 0; l < nl; ++l) {
        args.key_ptrs[l] = key_cache_ptrs_host[l0 + l];
        args.value_ptrs[l] = value_cache_ptrs_host[l0 + l];
      }
      for (int p = 0; p < np; ++p) {
        args.src[p] = static_cast<int32_t>(block_mapping_host[2 * (p0 + p)]);
        args.dst[p] = static_cast<int32_t>(block_mapping_host[2 * (p0 + p) + 1]);
      }
      dim3 grid(np, 2 * nl);
      copy_blocks_args_kernel<<<grid, kCopyThreads, 0, s>>>(args, nl, numel_per_block * 2);
      AICI_CUDA(cudaGetLastError());
    }
  }
  return nullptr;
}

// ---- rotary embedding fused with the cache write -----------------------------------------------------
//
// The step right before the attention path in rLLM is rotary_embedding on q and k
// (rllm-cuda/src/llm/mod.rs:62-129 -> kernels/vllm/pos_encoding_kernels.cu:40-128), immediately
// followed by reshape_and_cache of k and v.  This kernel does both in one pass over the tokens:
// q and k are rotated in place (NeoX style, element i pairs with i + rot_dim/2, arithmetic in bf16
// exactly as the reference's `x * cos - y * sin` on __nv_bfloat16) and the rotated k together with
// v goes straight into the paged cache, so k is read once instead of three times.
// One CTA = 16 tokens x one kv head (and the query heads of its group).
namespace aici {

__device__ __forceinline__ void rotate8(uint4 &xv, uint4 &yv, const uint4 &cv, const uint4 &sv) {
  __nv_bfloat16 *x = reinterpret_cast<__nv_bfloat16 *>(&xv);
  __nv_bfloat16 *y = reinterpret_cast<__nv_bfloat16 *>(&yv);
  const __nv_bfloat16 *c = reinterpret_cast<const __nv_bfloat16 *>(&cv);
  const __nv_bfloat16 *s = reinterpret_cast<const __nv_bfloat16 *>(&sv);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const __nv_bfloat16 xx = x[j], yy = y[j];
    // every product and the sum is rounded to bf16 on its own, as the reference's 16-bit scalar
    // type does (pos_encoding_kernels.cu:35-36); the _rn forms keep the compiler from fusing
    // a product and the sum into one fma
    x[j] = __hsub_rn(__hmul_rn(xx, c[j]), __hmul_rn(yy, s[j]));
    y[j] = __hadd_rn(__hmul_rn(yy, c[j]), __hmul_rn(xx, s[j]));
  }
}

template <bool kSlot64>
__global__ void __launch_bounds__(kThreads)
rotary_reshape_and_cache_kernel(const int64_t *__restrict__ positions, __nv_bfloat16 *__restrict__ query,
                                __nv_bfloat16 *__restrict__ key, const __nv_bfloat16 *__restrict__ value,
                                const __nv_bfloat16 *__restrict__ cos_sin_cache,
                                __nv_bfloat16 *__restrict__ key_cache, __nv_bfloat16 *__restrict__ value_cache,
                                const void *__restrict__ slot_mapping, int num_tokens, int num_kv_heads,
                                int group, int64_t max_position, int64_t num_slots, int64_t query_stride,
                                int64_t key_stride, int64_t value_stride, unsigned int *status) {
  __shared__ int64_t s_slot[kTok];
  __shared__ int64_t s_pos[kTok];
  __shared__ __align__(16) __nv_bfloat16 s_v[kTok][kD + 8];
  const int t0 = blockIdx.x * kTok;
  const int h = blockIdx.y;
  const int tid = threadIdx.x;

  if (tid < kTok) {
    int64_t slot = -1, pos = -1;
    if (t0 + tid < num_tokens) {
      slot = load_slot<kSlot64>(slot_mapping, t0 + tid);
      if (slot >= num_slots) {
        set_status(status, AICI_STATUS_BAD_SLOT);
        slot = -1;
      }
      pos = positions[t0 + tid];
      if (pos < 0 || pos >= max_position) {
        set_status(status, AICI_STATUS_BAD_SLOT);
        pos = -1;  // token left untouched
      }
    }
    s_slot[tid] = slot;
    s_pos[tid] = pos;
  }
  __syncthreads();

  if (tid < 128) {
    // thread (c, tok): d = 8c .. 8c+7 pairs with d + 64
    const int c = tid >> 4, tok = tid & 15;
    const int64_t pos = s_pos[tok];
    if (t0 + tok < num_tokens && pos >= 0) {
      const __nv_bfloat16 *cs = cos_sin_cache + pos * kD;  // [cos 0..63 | sin 0..63]
      const uint4 cv = *reinterpret_cast<const uint4 *>(cs + c * kX);
      const uint4 sv = *reinterpret_cast<const uint4 *>(cs + kD / 2 + c * kX);
      // key head h
      __nv_bfloat16 *kp = key + (int64_t)(t0 + tok) * key_stride + h * kD;
      uint4 xv = *reinterpret_cast<const uint4 *>(kp + c * kX);
      uint4 yv = *reinterpret_cast<const uint4 *>(kp + kD / 2 + c * kX);
      rotate8(xv, yv, cv, sv);
      *reinterpret_cast<uint4 *>(kp + c * kX) = xv;
      *reinterpret_cast<uint4 *>(kp + kD / 2 + c * kX) = yv;
      const int64_t slot = s_slot[tok];
      if (slot >= 0) {
        const int64_t blk = slot / kB, off = slot % kB;
        __nv_bfloat16 *dst = key_cache + ((blk * num_kv_heads + h) * (kD / kX)) * (kB * kX) + off * kX;
        *reinterpret_cast<uint4 *>(dst + c * (kB * kX)) = xv;
        *reinterpret_cast<uint4 *>(dst + (c + 8) * (kB * kX)) = yv;
      }
      // the query heads of this kv head's group
      for (int gq = 0; gq < group; ++gq) {
        __nv_bfloat16 *qp = query + (int64_t)(t0 + tok) * query_stride + (h * group + gq) * kD;
        uint4 qx = *reinterpret_cast<const uint4 *>(qp + c * kX);
        uint4 qy = *reinterpret_cast<const uint4 *>(qp + kD / 2 + c * kX);
        rotate8(qx, qy, cv, sv);
        *reinterpret_cast<uint4 *>(qp + c * kX) = qx;
        *reinterpret_cast<uint4 *>(qp + kD / 2 + c * kX) = qy;
      }
    }
  } else {
    // value tile -> shared memory (two 16-byte pieces per thread), transposed out below
    const int i = tid - 128;
    const int tok = i >> 3, part = (i & 7) * 2;
    if (s_slot[tok] >= 0) {
      const __nv_bfloat16 *vp = value + (int64_t)(t0 + tok) * value_stride + h * kD;
      *reinterpret_cast<uint4 *>(&s_v[tok][part * kX]) = *reinterpret_cast<const uint4 *>(vp + part * kX);
      *reinterpret_cast<uint4 *>(&s_v[tok][(part + 1) * kX]) = *reinterpret_cast<const uint4 *>(vp + (part + 1) * kX);
    }
  }
  __syncthreads();
  store_value_tile<kTok>(s_slot, s_v, value_cache, num_kv_heads, h, tid);
}

}  // namespace aici

extern "C" char *aici_rotary_reshape_and_cache(const int64_t *positions, void *query, void *key,
                                               const void *value, const void *cos_sin_cache,
                                               void *key_cache, void *value_cache,
                                               const void *slot_mapping, int slot_is_int64,
                                               int num_tokens, int num_heads, int num_kv_heads,
                                               int head_size, int rot_dim, int is_neox,
                                               int64_t max_position, int block_size, int64_t num_blocks,
                                               int64_t query_stride, int64_t key_stride,
                                               int64_t value_stride, int dtype, aici_stream_t stream) {
  const char *fn = "aici_rotary_reshape_and_cache";
  if (char *e = check_cache_shape(fn, num_kv_heads, head_size, block_size, dtype)) return e;
  AICI_CHECK(is_neox, "%s: only the NeoX pairing is supported (the reference's CPU path has no other)", fn);
  AICI_CHECK(rot_dim == head_size, "%s: rot_dim must equal head_size (got %d)", fn, rot_dim);
  AICI_CHECK(num_heads > 0 && num_heads % num_kv_heads == 0, "%s: num_heads must be a multiple of num_kv_heads", fn);
  AICI_CHECK(num_tokens >= 0 && max_position > 0, "%s: bad sizes", fn);
  if (num_tokens == 0) return nullptr;
  AICI_CHECK(positions && query && key && value && cos_sin_cache && key_cache && value_cache && slot_mapping,
             "%s: NULL pointer", fn);
  AICI_CHECK(num_blocks > 0, "%s: num_blocks must be positive", fn);
  AICI_CHECK(query_stride % 8 == 0 && key_stride % 8 == 0 && value_stride % 8 == 0 &&
                 query_stride >= (int64_t)num_heads * head_size &&
                 key_stride >= (int64_t)num_kv_heads * head_size &&
                 value_stride >= (int64_t)num_kv_heads * head_size,
             "%s: token strides must be multiples of 8 elements and cover one row", fn);
  AICI_CHECK(((uintptr_t)query | (uintptr_t)key | (uintptr_t)value | (uintptr_t)cos_sin_cache |
              (uintptr_t)key_cache | (uintptr_t)value_cache) % 16 == 0,
             "%s: tensors must be 16-byte aligned", fn);
  if (char *e = check_on_current_device(fn, "key_cache", key_cache)) return e;
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);
  dim3 grid((num_tokens + kTok - 1) / kTok, num_kv_heads);
  const int group = num_heads / num_kv_heads;
  auto q = static_cast<__nv_bfloat16 *>(query);
  auto k = static_cast<__nv_bfloat16 *>(key);
  auto v = static_cast<const __nv_bfloat16 *>(value);
  auto cs = static_cast<const __nv_bfloat16 *>(cos_sin_cache);
  auto kc = static_cast<__nv_bfloat16 *>(key_cache);
  auto vc = static_cast<__nv_bfloat16 *>(value_cache);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (slot_is_int64)
    rotary_reshape_and_cache_kernel<true><<<grid, kThreads, 0, s>>>(
        positions, q, k, v, cs, kc, vc, slot_mapping, num_tokens, num_kv_heads, group, max_position,
        num_blocks * kB, query_stride, key_stride, value_stride, st);
  else
    rotary_reshape_and_cache_kernel<false><<<grid, kThreads, 0, s>>>(
        positions, q, k, v, cs, kc, vc, slot_mapping, num_tokens, num_kv_heads, group, max_position,
        num_blocks * kB, query_stride, key_stride, value_stride, st);
  AICI_CUDA(cudaGetLastError());
  return nullptr;
}
