// Development check of the give-up path of the bounded device waits (built into libkda_b200_debug.so, not into the
// product library).  One warp initialises an mbarrier that nothing ever arrives at and waits for it with the same
// mbar_wait helper the chunk kernels use; the helper runs out of polls, and the kernel then does what those kernels
// do: it sets a bit in the status word at the start of a chunk workspace and returns.  The GPU stays usable and the
// host reads the bit with kda_chunk_status.  Nothing here faults, traps or spins without a limit.
#include "kda_chunk.cuh"

namespace kda {

__global__ void __launch_bounds__(32, 1) wait_giveup_kernel(unsigned* __restrict__ status, unsigned bit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  bool ok = mbar_wait(&bar, 0);      // phase 0 never completes: no arrival, no transaction bytes
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && threadIdx.x == 0) atomicOr(status, bit);
}

}  // namespace kda

// workspace: a chunk workspace (its first bytes are the status word); bit: the KDA_STATUS_* bit to set on give-up.
extern "C" __attribute__((visibility("default"))) int kda_b200_debug_wait_giveup(void* workspace, unsigned bit, void* stream) {
  if (!workspace) return KDA_E_NULL;
  const kda::ChunkWs w = kda::carve_ws(static_cast<unsigned char*>(workspace), nullptr, 0, 0, 1, false);
  kda::wait_giveup_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(w.status, bit);
  return static_cast<int>(cudaGetLastError());
}
