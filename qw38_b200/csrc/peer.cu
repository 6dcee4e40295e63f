// Cross-GPU completion wait for the row-sharded decode path.
//
// Each rank's projection kernel stores its rows into every rank's output buffer (gemv_tma.cu) and
// counts itself as finished; the next kernel of the stream announces finished projections by adding
// to this rank's slot of every rank's flag array.  All ranks enqueue the same sequence of
// projections, so a rank knows how many arrivals to expect from a peer: as many as it has made
// itself.  This kernel, enqueued after the projections of a step, announces what is still
// unannounced and then spins until every slot of its own flag array has caught up with its own.
// The spin is bounded; on expiry it records 0x610 in the status word and returns, leaving the
// context usable.
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

struct PeerWaitParams {
  uint32_t* flags[8];
  uint32_t* unsignalled;
  uint32_t ranks, rank;
  long long limit_cycles;  // < 0: announce only
  int* status;
};

__global__ void peer_wait_kernel(const PeerWaitParams p) {
  pdl_wait();
  if (threadIdx.x == 0) announce_deliveries(p.unsignalled, p.flags, p.ranks, p.rank);
  __syncwarp();
  uint32_t const g = threadIdx.x;
  if (p.limit_cycles < 0 || g >= p.ranks || g == p.rank) return;
  const uint32_t* const mine_flags = p.flags[p.rank];
  uint32_t const mine = *reinterpret_cast<const volatile uint32_t*>(mine_flags + p.rank);
  long long const t0 = clock64();
  for (;;) {
    uint32_t theirs;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(theirs) : "l"(mine_flags + g) : "memory");
    if (int32_t(theirs - mine) >= 0) return;
    if (clock64() - t0 > p.limit_cycles) {
      atomicExch(p.status, 0x610);
      return;
    }
    __nanosleep(100);
  }
}

}  // namespace

cudaError_t launch_peer_wait(uint32_t* const* flags, uint32_t* unsignalled, uint32_t ranks, uint32_t rank,
                             long long limit_cycles, int* status, cudaStream_t stream) {
  if (!flags || !unsignalled || ranks < 1 || ranks > 8 || rank >= ranks || !status) return cudaErrorInvalidValue;
  PeerWaitParams p{};
  for (uint32_t g = 0; g < ranks; ++g) p.flags[g] = flags[g];
  p.unsignalled = unsignalled; p.ranks = ranks; p.rank = rank; p.limit_cycles = limit_cycles; p.status = status;
  return launch_kernel(peer_wait_kernel, 1, 32, 0, stream, launch_overlap(), p);
}

}  // namespace q4k
