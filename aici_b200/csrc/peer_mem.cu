// Peer-mapped device memory for the fused head-output gather, and the gather as a stand-alone call.
//
// The reference has no multi-GPU code; its only hook is the kv-head count per rank
// (rllm/rllm-cuda/src/llm/config.rs:49-51, divisibility check :30-36).  With one process per GPU,
// the attention entry points `*_peers` store each rank's heads straight into every rank's output
// buffer, which needs those buffers (and the barrier's flag arrays) mapped into every process.
// These calls do that with nothing but the CUDA driver and runtime: the owner allocates and exports a
// 128-byte handle, the caller moves the handle to the other processes over whatever channel it has
// (a file, a socket, its collective library), and each peer opens it.  No libtorch, no NCCL.
#include <cuda.h>  // driver types only; entry points are resolved at run time, libcuda is not linked
#include <errno.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <vector>

#include "common.cuh"

namespace aici {

// local [rows, heads, 128] (row stride in elements) -> out[w][rows, total_heads, 128] at head0,
// for every rank's buffer; 16 bytes per thread per access, 4 accesses in flight.
__global__ void __launch_bounds__(256) gather_heads_kernel(const uint4 *__restrict__ local,
                                                           int64_t local_row_vec, int heads,
                                                           int64_t rows, int total_heads, int head0,
                                                           int world, uint4 *o0, uint4 *o1, uint4 *o2,
                                                           uint4 *o3, uint4 *o4, uint4 *o5, uint4 *o6,
                                                           uint4 *o7) {
  uint4 *outs[8] = {o0, o1, o2, o3, o4, o5, o6, o7};
  const int vec_per_row = heads * 16;  // 128 bf16 = 16 vectors per head
  const int64_t n = rows * vec_per_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n; i0 += 4 * stride) {
    uint4 v[4];
    int64_t dst[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < n) {
        const int64_t r = i / vec_per_row;
        const int c = static_cast<int>(i - r * vec_per_row);
        v[u] = local[r * local_row_vec + c];
        dst[u] = (r * total_heads + head0) * 16 + c;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * stride < n)
        for (int w = 0; w < world; ++w) outs[w][dst[u]] = v[u];
  }
}

}  // namespace aici

using namespace aici;

// ---- allocation and mapping -------------------------------------------------------------------------
// Two ways of sharing a buffer, chosen by the owner and recorded in the handle:
//   kind 1  CUDA virtual-memory allocation (cuMemCreate, 2 MB pages) exported as a POSIX file
//           descriptor; a peer process duplicates the descriptor with pidfd_getfd and maps the
//           allocation with cuMemMap.  The large pages matter: the prefill epilogue stores 128-byte
//           rows 16 KB apart, and through the small-page mapping that the legacy handles give a peer
//           those stores ran at about 120 GB/s over NVLink, half of what the 8-GPU step needs.
//   kind 2  cudaMalloc + cudaIpcGetMemHandle, used when the driver entry points or the pidfd
//           system calls are not available to this process.
namespace aici {

struct PeerHandle {  // AICI_PEER_HANDLE_BYTES bytes on the wire
  uint32_t magic, kind;
  int32_t pid, fd;
  uint64_t size;
  unsigned char legacy[64];
  unsigned char pad[AICI_PEER_HANDLE_BYTES - 24 - 64];
};
static_assert(sizeof(PeerHandle) == AICI_PEER_HANDLE_BYTES, "handle size");
constexpr uint32_t kPeerMagic = 0x41494349u;  // "AICI"

struct DriverVmm {
  CUresult (*create)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
  CUresult (*granularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
  CUresult (*reserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
  CUresult (*export_handle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*import_handle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
  CUresult (*unmap)(CUdeviceptr, size_t);
  CUresult (*address_free)(CUdeviceptr, size_t);
  CUresult (*release)(CUmemGenericAllocationHandle);
  bool ok;
};

static const DriverVmm &driver_vmm() {
  static DriverVmm d = [] {
    DriverVmm v = {};
    auto get = [](const char *name) -> void * {
      void *sym = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        return nullptr;
      return sym;
    };
    v.create = reinterpret_cast<decltype(v.create)>(get("cuMemCreate"));
    v.granularity = reinterpret_cast<decltype(v.granularity)>(get("cuMemGetAllocationGranularity"));
    v.reserve = reinterpret_cast<decltype(v.reserve)>(get("cuMemAddressReserve"));
    v.map = reinterpret_cast<decltype(v.map)>(get("cuMemMap"));
    v.set_access = reinterpret_cast<decltype(v.set_access)>(get("cuMemSetAccess"));
    v.export_handle = reinterpret_cast<decltype(v.export_handle)>(get("cuMemExportToShareableHandle"));
    v.import_handle = reinterpret_cast<decltype(v.import_handle)>(get("cuMemImportFromShareableHandle"));
    v.unmap = reinterpret_cast<decltype(v.unmap)>(get("cuMemUnmap"));
    v.address_free = reinterpret_cast<decltype(v.address_free)>(get("cuMemAddressFree"));
    v.release = reinterpret_cast<decltype(v.release)>(get("cuMemRelease"));
    v.ok = v.create && v.granularity && v.reserve && v.map && v.set_access && v.export_handle &&
           v.import_handle && v.unmap && v.address_free && v.release;
    return v;
  }();
  return d;
}

#ifndef SYS_pidfd_open
#define SYS_pidfd_open 434
#endif
#ifndef SYS_pidfd_getfd
#define SYS_pidfd_getfd 438
#endif

// A duplicate, in this process, of descriptor `fd` of process `pid`; -1 when the kernel refuses.
static int dup_fd_of(int pid, int fd) {
  const int pidfd = static_cast<int>(syscall(SYS_pidfd_open, pid, 0));
  if (pidfd < 0) return -1;
  const int got = static_cast<int>(syscall(SYS_pidfd_getfd, pidfd, fd, 0));
  close(pidfd);
  return got;
}

// What this process has mapped, so that close / free know how a pointer came to be.
struct PeerMapping {
  void *ptr;
  size_t size;
  CUmemGenericAllocationHandle handle;
  int fd;       // exported descriptor (owner of a kind-1 block), else -1
  int kind;     // 1 or 2
  bool owner;
};
static std::mutex g_peer_mu;
static std::vector<PeerMapping> g_peer_maps;

static void remember(const PeerMapping &m) {
  std::lock_guard<std::mutex> lock(g_peer_mu);
  g_peer_maps.push_back(m);
}
static bool take(void *ptr, bool owner, PeerMapping *out) {
  std::lock_guard<std::mutex> lock(g_peer_mu);
  for (size_t i = 0; i < g_peer_maps.size(); ++i)
    if (g_peer_maps[i].ptr == ptr && g_peer_maps[i].owner == owner) {
      *out = g_peer_maps[i];
      g_peer_maps.erase(g_peer_maps.begin() + i);
      return true;
    }
  return false;
}

// Reserves an address range for `h`, maps it and gives the current device read/write access.
static bool map_vmm(const DriverVmm &d, CUmemGenericAllocationHandle h, size_t size, size_t gran, int dev,
                    CUdeviceptr *out) {
  CUdeviceptr va = 0;
  if (d.reserve(&va, size, gran, 0, 0) != CUDA_SUCCESS) return false;
  if (d.map(va, size, 0, h, 0) != CUDA_SUCCESS) {
    d.address_free(va, size);
    return false;
  }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.set_access(va, size, &acc, 1) != CUDA_SUCCESS) {
    d.unmap(va, size);
    d.address_free(va, size);
    return false;
  }
  *out = va;
  return true;
}

static size_t vmm_granularity(const DriverVmm &d, int dev, CUmemAllocationProp *prop) {
  memset(prop, 0, sizeof(*prop));
  prop->type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop->location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop->location.id = dev;
  prop->requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  if (d.granularity(&gran, prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return 0;
  return gran;
}

// kind 1; false (nothing left behind) when any step is unavailable here
static bool alloc_vmm(size_t bytes, int dev, void **ptr_out, PeerHandle *h) {
  const DriverVmm &d = driver_vmm();
  if (!d.ok) return false;
  CUmemAllocationProp prop;
  const size_t gran = vmm_granularity(d, dev, &prop);
  if (gran == 0) return false;
  const size_t size = (bytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle mh;
  if (d.create(&mh, size, &prop, 0) != CUDA_SUCCESS) return false;
  int fd = -1;
  CUdeviceptr va = 0;
  bool ok = d.export_handle(&fd, mh, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS && fd >= 0;
  if (ok) {  // can a process of this container duplicate the descriptor at all?
    const int probe = dup_fd_of(getpid(), fd);
    ok = probe >= 0;
    if (probe >= 0) close(probe);
  }
  ok = ok && map_vmm(d, mh, size, gran, dev, &va);
  if (!ok) {
    if (fd >= 0) close(fd);
    d.release(mh);
    return false;
  }
  h->kind = 1;
  h->pid = getpid();
  h->fd = fd;
  h->size = size;
  *ptr_out = reinterpret_cast<void *>(va);
  remember({*ptr_out, size, mh, fd, 1, true});
  return true;
}

}  // namespace aici

extern "C" char *aici_peer_alloc(size_t bytes, void **ptr_out, void *handle_out) {
  const char *fn = "aici_peer_alloc";
  AICI_CHECK(ptr_out != nullptr && handle_out != nullptr, "%s: NULL output pointer", fn);
  AICI_CHECK(bytes > 0, "%s: size must be positive", fn);
  int dev = 0;
  AICI_CUDA(cudaGetDevice(&dev));
  AICI_CUDA(cudaFree(nullptr));  // the driver calls below need this device's context to exist
  PeerHandle h;
  memset(&h, 0, sizeof(h));
  h.magic = kPeerMagic;
  void *p = nullptr;
  if (!alloc_vmm(bytes, dev, &p, &h)) {
    AICI_CUDA(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t legacy;
    cudaError_t e = cudaIpcGetMemHandle(&legacy, p);
    if (e != cudaSuccess) {
      cudaFree(p);
      return err("%s: %s", fn, cudaGetErrorString(e));
    }
    static_assert(sizeof(legacy) == sizeof(h.legacy), "legacy handle size");
    memcpy(h.legacy, &legacy, sizeof(legacy));
    h.kind = 2;
    h.size = bytes;
    remember({p, bytes, 0, -1, 2, true});
  }
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    aici_peer_free(p);
    return err("%s: %s", fn, cudaGetErrorString(e));
  }
  memcpy(handle_out, &h, sizeof(h));
  *ptr_out = p;
  return nullptr;
}

extern "C" char *aici_peer_open(const void *handle, void **ptr_out) {
  const char *fn = "aici_peer_open";
  AICI_CHECK(handle != nullptr && ptr_out != nullptr, "%s: NULL pointer", fn);
  PeerHandle h;
  memcpy(&h, handle, sizeof(h));
  AICI_CHECK(h.magic == kPeerMagic && (h.kind == 1 || h.kind == 2), "%s: not a handle made by aici_peer_alloc", fn);
  int dev = 0;
  AICI_CUDA(cudaGetDevice(&dev));
  AICI_CUDA(cudaFree(nullptr));
  if (h.kind == 1) {
    const DriverVmm &d = driver_vmm();
    AICI_CHECK(d.ok, "%s: the driver's virtual-memory entry points are not available", fn);
    AICI_CHECK(h.pid != getpid(), "%s: the handle comes from this process (use the pointer aici_peer_alloc returned)", fn);
    const int fd = dup_fd_of(h.pid, h.fd);
    AICI_CHECK(fd >= 0, "%s: cannot duplicate descriptor %d of process %d (%s); the owner must be alive and in "
               "the same container", fn, h.fd, h.pid, strerror(errno));
    CUmemGenericAllocationHandle mh;
    CUresult r = d.import_handle(&mh, reinterpret_cast<void *>(static_cast<uintptr_t>(fd)),
                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    AICI_CHECK(r == CUDA_SUCCESS, "%s: cuMemImportFromShareableHandle failed with code %d", fn, (int)r);
    CUmemAllocationProp prop;
    const size_t gran = vmm_granularity(d, dev, &prop);
    CUdeviceptr va = 0;
    if (gran == 0 || !map_vmm(d, mh, h.size, gran, dev, &va)) {
      d.release(mh);
      return err("%s: mapping the peer's allocation failed (can this GPU reach the owner's?)", fn);
    }
    *ptr_out = reinterpret_cast<void *>(va);
    remember({*ptr_out, (size_t)h.size, mh, -1, 1, false});
    return nullptr;
  }
  cudaIpcMemHandle_t legacy;
  memcpy(&legacy, h.legacy, sizeof(legacy));
  void *p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, legacy, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return err("%s: cudaIpcOpenMemHandle failed: %s (the handle must come from aici_peer_alloc in "
               "ANOTHER process of this machine, on a GPU this device can reach)",
               fn, cudaGetErrorString(e));
  }
  *ptr_out = p;
  remember({p, (size_t)h.size, 0, -1, 2, false});
  return nullptr;
}

static char *release_mapping(const char *fn, void *ptr, bool owner) {
  if (ptr == nullptr) return nullptr;
  PeerMapping m;
  AICI_CHECK(take(ptr, owner, &m), "%s: %p is not a block this process %s", fn, ptr,
             owner ? "allocated with aici_peer_alloc" : "opened with aici_peer_open");
  if (m.kind == 1) {
    const DriverVmm &d = driver_vmm();
    AICI_CUDA(cudaDeviceSynchronize());
    d.unmap(reinterpret_cast<CUdeviceptr>(m.ptr), m.size);
    d.address_free(reinterpret_cast<CUdeviceptr>(m.ptr), m.size);
    d.release(m.handle);
    if (m.fd >= 0) close(m.fd);
    return nullptr;
  }
  if (owner) {
    AICI_CUDA(cudaFree(ptr));
  } else {
    AICI_CUDA(cudaIpcCloseMemHandle(ptr));
  }
  return nullptr;
}

extern "C" char *aici_peer_close(void *ptr) { return release_mapping("aici_peer_close", ptr, false); }

extern "C" char *aici_peer_free(void *ptr) { return release_mapping("aici_peer_free", ptr, true); }

extern "C" char *aici_gather_heads(void *const *outs, int world, int total_heads, int head0,
                                   const void *local, int64_t rows, int num_heads, int head_size,
                                   int64_t local_row_stride, int dtype, aici_stream_t stream) {
  const char *fn = "aici_gather_heads";
  AICI_CHECK(dtype == AICI_DTYPE_BF16, "%s: only bf16 is supported (dtype=%d)", fn, dtype);
  AICI_CHECK(head_size == 128, "%s: head_size must be 128 (got %d)", fn, head_size);
  AICI_CHECK(outs != nullptr && world >= 1 && world <= 8, "%s: world must be 1..8", fn);
  AICI_CHECK(rows >= 0 && num_heads > 0 && head0 >= 0 && head0 + num_heads <= total_heads,
             "%s: heads [%d, %d) do not fit %d total heads", fn, head0, head0 + num_heads, total_heads);
  if (rows == 0) return nullptr;
  AICI_CHECK(local != nullptr && (uintptr_t)local % 16 == 0, "%s: local must be non-NULL and 16-byte aligned", fn);
  AICI_CHECK(local_row_stride % 8 == 0 && local_row_stride >= (int64_t)num_heads * head_size,
             "%s: local_row_stride must be a multiple of 8 elements and cover one row", fn);
  uint4 *o[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int w = 0; w < world; ++w) {
    AICI_CHECK(outs[w] != nullptr && (uintptr_t)outs[w] % 16 == 0,
               "%s: output %d must be non-NULL and 16-byte aligned", fn, w);
    o[w] = static_cast<uint4 *>(outs[w]);
  }
  if (char *e = check_on_current_device(fn, "local", local)) return e;
  const int64_t n = rows * num_heads * 16;
  int64_t blocks = (n + 4 * 256 - 1) / (4 * 256);
  const int64_t cap = (int64_t)8 * sm_count();
  if (blocks > cap) blocks = cap;
  gather_heads_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(local), local_row_stride / 8, num_heads, rows, total_heads, head0, world,
      o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
  AICI_CUDA(cudaGetLastError());
  return nullptr;
}
