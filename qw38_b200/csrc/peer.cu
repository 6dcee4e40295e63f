// Cross-GPU completion wait for the row-sharded decode path.
//
// Each rank's projection kernel stores its rows into every rank's output buffer and then adds 1
// to its own slot of every rank's flag array (gemv_tma.cu).  All ranks enqueue the same sequence
// of projections, so a rank knows how many arrivals to expect from a peer: as many as it has
// made itself.  This kernel, enqueued after the projections of a step, spins until every slot
// has caught up with the rank's own.  The spin is bounded; on expiry it records 0x610 in the
// status word and returns, leaving the context usable.
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

__global__ void peer_wait_kernel(const uint32_t* flags, uint32_t ranks, uint32_t rank, long long limit_cycles, int* status) {
  pdl_wait();
  uint32_t const g = threadIdx.x;
  if (g >= ranks || g == rank) return;
  const volatile uint32_t* vf = flags;
  uint32_t const mine = vf[rank];
  long long const t0 = clock64();
  for (;;) {
    uint32_t theirs;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(theirs) : "l"(flags + g) : "memory");
    if (int32_t(theirs - mine) >= 0) return;
    if (clock64() - t0 > limit_cycles) {
      atomicExch(status, 0x610);
      return;
    }
    __nanosleep(100);
  }
}

}  // namespace

cudaError_t launch_peer_wait(const uint32_t* flags, uint32_t ranks, uint32_t rank, long long limit_cycles, int* status,
                             cudaStream_t stream) {
  if (!flags || ranks < 1 || ranks > 8 || rank >= ranks || !status) return cudaErrorInvalidValue;
  return launch_kernel(peer_wait_kernel, 1, 32, 0, stream, launch_overlap(), flags, ranks, rank, limit_cycles, status);
}

}  // namespace q4k
