// swap_blocks: whole cache blocks moved between the device cache and a host-side cache (swap out /
// swap in of preempted sequences), or between two places of one device.
//
// The reference walks the mapping on the host and issues one cudaMemcpyAsync per block
// (rllm/tch-cuda/kernels/vllm/cache_kernels.cu:12-50, with the remark that this is slow for many
// blocks); rLLM's CacheEngine::swap calls it per layer for K and for V
// (rllm-cuda/src/llm/paged/cache_engine.rs:139-149; the crate-side wrapper is still todo!()).
//
// Here the mapping travels as a kernel argument and ONE launch moves all blocks of a tensor:
// a page-locked host cache is addressable from the device (unified addressing), so the SMs read or
// write it directly over PCIe with 16-byte accesses, 32 KB per CTA step, enough CTAs in flight to
// cover the bus latency and few enough to leave the rest of the GPU to attention kernels running on
// other streams.  A pageable host cache cannot be touched by a kernel; for that case consecutive
// (src, dst) runs are merged and each run becomes one copy-engine transfer.
#include "common.cuh"

namespace aici {

constexpr int kSwapThreads = 256;
constexpr int kSwapUnroll = 8;                                   // 8 x 16 B in flight per thread
constexpr int kSwapStepVec = kSwapThreads * kSwapUnroll;         // 32 KB per CTA step
constexpr int kSwapPairs = 1536;                                 // mapping entries per launch
constexpr int kSwapCtasHost = 96;                                // CTAs when one side is host memory

struct SwapArgs {
  int32_t src[kSwapPairs];
  int32_t dst[kSwapPairs];
};

// Work item = (pair, 32 KB step inside the block); CTAs stride over the items.
__global__ void __launch_bounds__(kSwapThreads)
swap_blocks_kernel(const __grid_constant__ SwapArgs args, const char *__restrict__ src,
                   char *__restrict__ dst, int num_pairs, int64_t block_bytes) {
  const int vec_per_block = static_cast<int>(block_bytes / 16);
  const int steps = (vec_per_block + kSwapStepVec - 1) / kSwapStepVec;
  const int64_t items = (int64_t)num_pairs * steps;
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int pair = static_cast<int>(item / steps);
    const int base = static_cast<int>(item % steps) * kSwapStepVec;
    const uint4 *s = reinterpret_cast<const uint4 *>(src + (int64_t)args.src[pair] * block_bytes);
    uint4 *d = reinterpret_cast<uint4 *>(dst + (int64_t)args.dst[pair] * block_bytes);
    uint4 v[kSwapUnroll];
#pragma unroll
    for (int u = 0; u < kSwapUnroll; ++u) {
      const int i = base + u * kSwapThreads + threadIdx.x;
      if (i < vec_per_block) v[u] = s[i];
    }
#pragma unroll
    for (int u = 0; u < kSwapUnroll; ++u) {
      const int i = base + u * kSwapThreads + threadIdx.x;
      if (i < vec_per_block) d[i] = v[u];
    }
  }
}

enum Place { kPlaceDevice, kPlacePinned, kPlacePageable };

// Where a pointer lives, and the address a kernel may use for it.
static char *classify(const char *fn, const char *what, const void *p, Place *place, int *device,
                      const void **dev_ptr) {
  cudaPointerAttributes attr;
  AICI_CUDA(cudaPointerGetAttributes(&attr, p));
  *device = attr.device;
  *dev_ptr = p;
  switch (attr.type) {
    case cudaMemoryTypeDevice:
    case cudaMemoryTypeManaged:
      *place = kPlaceDevice;
      break;
    case cudaMemoryTypeHost:
      *place = kPlacePinned;
      AICI_CHECK(attr.devicePointer != nullptr, "%s: %s is page-locked but not mapped", fn, what);
      *dev_ptr = attr.devicePointer;
      break;
    default:
      *place = kPlacePageable;
      break;
  }
  return nullptr;
}

}  // namespace aici

using namespace aici;

extern "C" char *aici_swap_blocks(const void *src, void *dst, const int64_t *block_mapping_host,
                                  int num_pairs, int64_t block_bytes, int64_t src_num_blocks,
                                  int64_t dst_num_blocks, aici_stream_t stream) {
  const char *fn = "aici_swap_blocks";
  AICI_CHECK(num_pairs >= 0, "%s: negative pair count", fn);
  AICI_CHECK(block_bytes > 0 && block_bytes % 16 == 0 && block_bytes / 16 <= INT32_MAX,
             "%s: a block must be a positive multiple of 16 bytes (got %lld)", fn,
             (long long)block_bytes);
  if (num_pairs == 0) return nullptr;
  AICI_CHECK(src && dst && block_mapping_host, "%s: NULL pointer", fn);
  AICI_CHECK(((uintptr_t)src | (uintptr_t)dst) % 16 == 0, "%s: caches must be 16-byte aligned", fn);
  AICI_CHECK(src_num_blocks > 0 && dst_num_blocks > 0, "%s: cache sizes must be positive", fn);
  for (int p = 0; p < num_pairs; ++p) {
    const int64_t s = block_mapping_host[2 * p], d = block_mapping_host[2 * p + 1];
    AICI_CHECK(s >= 0 && s < src_num_blocks && s <= INT32_MAX,
               "%s: pair %d: source block %lld is outside the cache of %lld blocks", fn, p,
               (long long)s, (long long)src_num_blocks);
    AICI_CHECK(d >= 0 && d < dst_num_blocks && d <= INT32_MAX,
               "%s: pair %d: destination block %lld is outside the cache of %lld blocks", fn, p,
               (long long)d, (long long)dst_num_blocks);
  }
  Place sp, dp;
  int sdev = -1, ddev = -1;
  const void *s_dev = nullptr, *d_dev = nullptr;
  if (char *e = classify(fn, "src", src, &sp, &sdev, &s_dev)) return e;
  if (char *e = classify(fn, "dst", dst, &dp, &ddev, &d_dev)) return e;
  // the reference's device rules (cache_kernels.cu:17-30)
  AICI_CHECK(sp == kPlaceDevice || dp == kPlaceDevice, "%s: Invalid device combination", fn);
  AICI_CHECK(!(sp == kPlaceDevice && dp == kPlaceDevice) || sdev == ddev,
             "%s: src and dst must be on the same GPU", fn);
  // The reference's cudaMemcpyAsync works from any current device; the copy kernel below runs on
  // the current one, so the device-side cache has to live there.
  int cur = -1;
  AICI_CUDA(cudaGetDevice(&cur));
  const int owner = sp == kPlaceDevice ? sdev : ddev;
  AICI_CHECK(owner == cur,
             "%s: the device cache lives on GPU %d but the current device is %d (make the cache's GPU "
             "current before the call)", fn, owner, cur);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (sp == kPlacePageable || dp == kPlacePageable) {
    // copy engine, one transfer per run of consecutive blocks
    int p = 0;
    while (p < num_pairs) {
      const int64_t s0 = block_mapping_host[2 * p], d0 = block_mapping_host[2 * p + 1];
      int n = 1;
      while (p + n < num_pairs && block_mapping_host[2 * (p + n)] == s0 + n &&
             block_mapping_host[2 * (p + n) + 1] == d0 + n)
        ++n;
      AICI_CUDA(cudaMemcpyAsync(static_cast<char *>(dst) + d0 * block_bytes,
                                static_cast<const char *>(src) + s0 * block_bytes,
                                (size_t)n * block_bytes, cudaMemcpyDefault, st));
      p += n;
    }
    return nullptr;
  }

  const bool host_side = sp == kPlacePinned || dp == kPlacePinned;
  const int vec = static_cast<int>(block_bytes / 16);
  const int steps = (vec + kSwapStepVec - 1) / kSwapStepVec;
  for (int p0 = 0; p0 < num_pairs; p0 += kSwapPairs) {
    const int np = num_pairs - p0 < kSwapPairs ? num_pairs - p0 : kSwapPairs;
    static thread_local SwapArgs args;
    for (int p = 0; p < np; ++p) {
      args.src[p] = static_cast<int32_t>(block_mapping_host[2 * (p0 + p)]);
      args.dst[p] = static_cast<int32_t>(block_mapping_host[2 * (p0 + p) + 1]);
    }
    const int64_t items = (int64_t)np * steps;
    const int64_t cap = host_side ? kSwapCtasHost : (int64_t)8 * sm_count();
    const int grid = static_cast<int>(items < cap ? items : cap);
    swap_blocks_kernel<<<grid, kSwapThreads, 0, st>>>(args, static_cast<const char *>(s_dev),
                                                      static_cast<char *>(const_cast<void *>(d_dev)),
                                                      np, block_bytes);
    AICI_CUDA(cudaGetLastError());
  }
  return nullptr;
}
