// Cross-GPU barrier for the fused head-output gather: after a rank's attention kernels have
// stored their rows into every peer's output buffer, the ranks only need to know that everybody
// is done.  One warp per rank: lane p publishes this rank's epoch into peer p's flag array (a
// release store at system scope, after the preceding kernels of the stream have completed) and
// then waits -- bounded -- until peer p's epoch shows up in its own array.  Flags live in
// peer-mapped symmetric memory; epochs only grow (a per-rank counter kept beside the flags), so
// nothing is ever reset and a launch can be replayed.
#include "common.cuh"

namespace aici {

struct PeerFlags {
  unsigned int *flags[8];  // flags[p] = rank p's array of 32 slots (slot r < 8 is written by rank r)
};

// Slot 8 of a rank's own array is its private barrier counter: every barrier increments it and
// uses the new value as the epoch, so the same launch can be replayed (CUDA graphs) and all ranks,
// which call the barrier the same number of times, agree on the epoch without host involvement.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerFlags f, int world, int rank,
                                                          unsigned int *status) {
  const int p = threadIdx.x;
  unsigned int epoch = 0;
  if (p == 0) {
    epoch = f.flags[rank][8] + 1;
    f.flags[rank][8] = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (p >= world) return;
  __threadfence_system();
  peer_signal_and_wait(f.flags, rank, p, epoch, status);
}

}  // namespace aici

using namespace aici;

extern "C" char *aici_peer_barrier(void *const *flag_ptrs, int world, int rank, aici_stream_t stream) {
  const char *fn = "aici_peer_barrier";
  AICI_CHECK(flag_ptrs != nullptr && world >= 1 && world <= 8 && rank >= 0 && rank < world,
             "%s: world must be 1..8 and rank inside it", fn);
  if (world == 1) return nullptr;
  unsigned int *st = status_ptr();
  AICI_CHECK(st != nullptr, "%s: no CUDA device", fn);
  PeerFlags f;
  for (int i = 0; i < 8; ++i) {
    f.flags[i] = static_cast<unsigned int *>(i < world ? flag_ptrs[i] : nullptr);
    AICI_CHECK(i >= world || (f.flags[i] != nullptr && (uintptr_t)f.flags[i] % 4 == 0),
               "%s: flag array %d must be non-NULL and 4-byte aligned", fn, i);
  }
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, st);
  AICI_CUDA(cudaGetLastError());
  return nullptr;
}
