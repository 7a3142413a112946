// Shared host/device helpers for the sm_100a attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "../../include/aici_b200.h"

namespace aici {

// ---- error convention: NULL = ok, else malloc'd message ---------------------------------
inline char *err(const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return strdup(buf);
}

#define AICI_CHECK(cond, ...)                                                              \
  do {                                                                                     \
    if (!(cond)) return ::aici::err(__VA_ARGS__);                                          \
  } while (0)

#define AICI_CUDA(call)                                                                    \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return ::aici::err("%s failed: %s", #call, cudaGetErrorString(e__));                 \
  } while (0)

// Status block, one per device (defined in status.cu): word 0 holds the sticky status bits that
// aici_last_status reads and clears; words 2-3 hold a 64-bit %globaltimer stamp of the most recent
// pipeline time-out (see mbar_wait_abortable).  Host code asks for its device address once per
// device and hands it to every kernel as an argument.
unsigned int *status_ptr();

// NULL when `ptr` is not device memory or lives on the current device; else an error string.
char *check_on_current_device(const char *fn, const char *what, const void *ptr);

// Multiprocessor count of the current device (cached per device; 148 if the query fails).
int sm_count();

// Runs `setup` once per device (the current one) under a lock; returns its error string, or NULL.
// Used for cudaFuncSetAttribute and symbol-address look-ups that must happen before a first launch.
struct OncePerDevice {
  std::mutex mu;
  bool done[64] = {false};
  template <typename F>
  char *run(F setup) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return strdup("no current CUDA device");
    std::lock_guard<std::mutex> lock(mu);
    if (done[dev]) return nullptr;
    if (char *e = setup()) return e;
    done[dev] = true;
    return nullptr;
  }
};

__device__ __forceinline__ void set_status(unsigned int *st, unsigned int bits) {
  atomicOr(st, bits);
}

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after ~2^31 clock ticks of polling (about a second), records
// AICI_STATUS_WAIT_TIMEOUT and returns false so the caller can unwind without hanging.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, unsigned int *st) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > (1ll << 31)) {
      set_status(st, AICI_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Same, for kernels whose CTAs wait on each other's roles: also gives up when some CTA of the
// device has timed out within the last two seconds, so that one stuck pipeline cannot hold a grid
// of many waves for a second per wave.  The mark is a time stamp, not a sticky bit: it expires by
// itself, so a time-out that was reported long ago (or a late peer in aici_peer_barrier, which
// has its own status bit and leaves no stamp) never makes a later launch give up.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t *bar, uint32_t parity,
                                                    unsigned int *st) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned polls = 0;
  unsigned long long *stamp = reinterpret_cast<unsigned long long *>(st + 2);
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 255u) == 0u) {
      const unsigned long long seen = *reinterpret_cast<volatile unsigned long long *>(stamp);
      if (seen != 0ull && global_timer_ns() - seen < 2000000000ull) return false;
      if (clock64() - t0 > (1ll << 31)) {
        set_status(st, AICI_STATUS_WAIT_TIMEOUT);
        atomicExch(stamp, global_timer_ns());
        return false;
      }
    }
  }
  return true;
}

// Waits, bounded to about a second, until the counter at `slot` (added to by a peer at system
// scope; it wraps, so the difference is what is compared) has reached `target`.  A peer that never
// gets there is recorded as AICI_STATUS_PEER_TIMEOUT and the thread returns.
__device__ __forceinline__ void peer_wait_count(const unsigned int *slot, unsigned int target,
                                                unsigned int *status) {
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(slot) : "memory");
    if ((int)(v - target) >= 0) return;
    if (clock64() - t0 > (1ll << 31)) {
      set_status(status, AICI_STATUS_PEER_TIMEOUT);
      return;
    }
  }
}

// Barrier between the GPUs that share peer-mapped flag arrays, executed by the first `world` threads
// of one warp: thread p publishes `epoch` into slot `rank` of rank p's array (release store at
// system scope; the caller has fenced its own earlier stores) and waits, bounded to about a second,
// until slot p of this rank's own array holds it.  A peer that never arrives is recorded as
// AICI_STATUS_PEER_TIMEOUT and the thread returns.
__device__ __forceinline__ void peer_signal_and_wait(unsigned int *const *flags, int rank, int p,
                                                     unsigned int epoch, unsigned int *status) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags[p] + rank), "r"(epoch) : "memory");
  const unsigned int *mine = flags[rank] + p;
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - epoch) >= 0) break;
    if (clock64() - t0 > (1ll << 31)) {  // give up, report, keep the context usable
      set_status(status, AICI_STATUS_PEER_TIMEOUT);
      break;
    }
  }
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier (TMA engine, no tensor
// map).  Both addresses 16-byte aligned, size a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                         uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                            uint32_t &r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// Two fp32 values in one 64-bit register pair and the packed arithmetic sm_100 has for them: one
// instruction does the work of two.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace aici
