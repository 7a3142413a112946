// Device status word and library version.
#include "common.cuh"

namespace aici {

__device__ unsigned int g_status_word = 0;

unsigned int *status_ptr() {
  static unsigned int *cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<unsigned int *>(p);
  }
  return cached[dev];
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
