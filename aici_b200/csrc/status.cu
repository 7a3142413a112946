// Device status word and library version.
#include "common.cuh"

namespace aici {

// [0] sticky status bits, [1] unused, [2..3] 64-bit time stamp of the latest pipeline time-out
__device__ __align__(16) unsigned int g_status_words[4] = {0, 0, 0, 0};

static std::mutex g_mu;

unsigned int *status_ptr() {
  static unsigned int *cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (cached[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_words) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<unsigned int *>(p);
  }
  return cached[dev];
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(g_mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Entry points work on the CURRENT device; a pointer that lives on another GPU would be
// dereferenced by this device's SMs (a fault without peer access, a silent NVLink access with it).
char *check_on_current_device(const char *fn, const char *what, const void *ptr) {
  if (ptr == nullptr) return nullptr;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;  // not a CUDA pointer the runtime knows: nothing to compare
  }
  if (attr.type != cudaMemoryTypeDevice) return nullptr;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return err("%s: no current CUDA device", fn);
  if (attr.device != dev)
    return err("%s: %s lives on GPU %d but the current device is %d (make the tensors' GPU current "
               "before the call)", fn, what, attr.device, dev);
  return nullptr;
}

}  // namespace aici

extern "C" const char *aici_version(void) { return "aici_b200 0.1 (sm_100a)"; }

extern "C" char *aici_last_status(int *status_out) {
  AICI_CHECK(status_out != nullptr, "aici_last_status: status_out is NULL");
  unsigned int *p = aici::status_ptr();
  AICI_CHECK(p != nullptr, "aici_last_status: no CUDA device");
  unsigned int v = 0;
  AICI_CUDA(cudaDeviceSynchronize());
  AICI_CUDA(cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost));
  AICI_CUDA(cudaMemset(p, 0, sizeof(v)));
  *status_out = static_cast<int>(v);
  return nullptr;
}
