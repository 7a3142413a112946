// Peer-mapped device memory for the fused head-output gather, and the gather as a stand-alone call.
//
// The reference has no multi-GPU code; its only hook is the kv-head count per rank
// (rllm/rllm-cuda/src/llm/config.rs:49-51, divisibility check :30-36).  With one process per GPU,
// the attention entry points `*_peers` store each rank's heads straight into every rank's output
// buffer, which needs those buffers (and the barrier's flag arrays) mapped into every process.
// These calls do that with CUDA IPC handles and nothing else: the owner allocates and exports a
// 64-byte handle, the caller moves the handle to the other processes over whatever channel it has
// (a file, a socket, its collective library), and each peer opens it.  No libtorch, no NCCL.
#include "common.cuh"

namespace aici {

static_assert(sizeof(cudaIpcMemHandle_t) == AICI_PEER_HANDLE_BYTES, "handle size");

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

extern "C" char *aici_peer_alloc(size_t bytes, void **ptr_out, void *handle_out) {
  const char *fn = "aici_peer_alloc";
  AICI_CHECK(ptr_out != nullptr && handle_out != nullptr, "%s: NULL output pointer", fn);
  AICI_CHECK(bytes > 0, "%s: size must be positive", fn);
  void *p = nullptr;
  AICI_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return err("%s: %s", fn, cudaGetErrorString(e));
  }
  memcpy(handle_out, &h, sizeof(h));
  *ptr_out = p;
  return nullptr;
}

extern "C" char *aici_peer_open(const void *handle, void **ptr_out) {
  const char *fn = "aici_peer_open";
  AICI_CHECK(handle != nullptr && ptr_out != nullptr, "%s: NULL pointer", fn);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void *p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return err("%s: cudaIpcOpenMemHandle failed: %s (the handle must come from aici_peer_alloc in "
               "ANOTHER process of this machine, on a GPU this device can reach)",
               fn, cudaGetErrorString(e));
  }
  *ptr_out = p;
  return nullptr;
}

extern "C" char *aici_peer_close(void *ptr) {
  if (ptr == nullptr) return nullptr;
  AICI_CUDA(cudaIpcCloseMemHandle(ptr));
  return nullptr;
}

extern "C" char *aici_peer_free(void *ptr) {
  if (ptr == nullptr) return nullptr;
  AICI_CUDA(cudaFree(ptr));
  return nullptr;
}

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
