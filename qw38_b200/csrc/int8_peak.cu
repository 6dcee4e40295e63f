// Measures the dense int8 tensor throughput of the device with the instruction the prefill kernel
// uses: tcgen05.mma kind::i8, M128 x N256 x K32, operands resident in shared memory, accumulators
// in TMEM.  One block per SM; one thread issues `mmas` MMAs back to back (alternating between the
// two halves of TMEM), committing every 16 to a small ring of mbarriers so that at most 64 are in
// flight.  The figure is the denominator of the prefill roofline (ops = 2 * 128 * 256 * 32 per MMA).
#include <cuda.h>

#include "../../include/q4k_b200.h"
#include "launch.h"
#include "tma.cuh"
#include "umma.cuh"

namespace q4k {
namespace {

constexpr int kBatch = 16, kRing = 4;
constexpr int kSmemA = 128 * 128, kSmemB = 256 * 128;

__global__ void __launch_bounds__(64, 1) int8_peak_kernel(uint32_t mmas, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bars[kRing];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  for (uint32_t i = threadIdx.x; i < (kSmemA + kSmemB) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kRing; ++i) mbar_init(smem_u32(&bars[i]), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) tmem_alloc_all(smem_u32(&tmem_slot));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmem_base = tmem_slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_i8(256);
    uint32_t const a0 = smem_u32(smem), b0 = smem_u32(smem + kSmemA);
    uint32_t const batches = (mmas + kBatch - 1) / kBatch;
    bool ok = true;
    for (uint32_t bt = 0; ok && bt < batches; ++bt) {
      uint32_t const slot = bt % kRing;
      if (bt >= kRing && !mbar_wait(smem_u32(&bars[slot]), ((bt / kRing) - 1) & 1, &abort_flag, status, 0x710)) { ok = false; break; }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        uint32_t const ks = uint32_t(j & 3) * 32;
        // the first MMA into each half clears it; later ones accumulate (the values wrap, which is harmless)
        umma_i8(tmem_base + uint32_t(j & 1) * 256, umma_desc_sw128(a0 + ks), umma_desc_sw128(b0 + ks), idesc, (bt | uint32_t(j >> 1)) != 0);
      }
      umma_commit(smem_u32(&bars[slot]));
    }
    // every batch has completed once the last kRing commits have arrived
    for (uint32_t bt = batches > kRing ? batches - kRing : 0; ok && bt < batches; ++bt)
      if (!mbar_wait(smem_u32(&bars[bt % kRing]), (bt / kRing) & 1, &abort_flag, status, 0x711)) ok = false;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc_all(tmem_base);
  }
}

}  // namespace
}  // namespace q4k

extern "C" int q4k_measure_int8_peak(uint32_t mmas_per_sm, double* tops, double* milliseconds, void* stream_handle) {
  using namespace q4k;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (!mmas_per_sm || !tops) return set_error(Q4K_ERR_INVALID_ARGUMENT, "int8_peak: mmas_per_sm and tops must be given");
  int* status = kernel_status_word();
  if (!status) return Q4K_ERR_STATUS;
  int const smem = kSmemA + kSmemB + 1024;
  cudaError_t st = cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (st != cudaSuccess) return set_error_cuda(st, "int8_peak.attribute");
  cudaEvent_t e0, e1;
  if ((st = cudaEventCreate(&e0)) != cudaSuccess) return set_error_cuda(st, "int8_peak.event");
  if ((st = cudaEventCreate(&e1)) != cudaSuccess) { cudaEventDestroy(e0); return set_error_cuda(st, "int8_peak.event"); }
  int const grid = sm_count();
  int8_peak_kernel<<<grid, 64, smem, stream>>>(16, status);  // warm-up: module load, clocks
  cudaEventRecord(e0, stream);
  int8_peak_kernel<<<grid, 64, smem, stream>>>(mmas_per_sm, status);
  cudaEventRecord(e1, stream);
  st = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (st == cudaSuccess) st = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (st != cudaSuccess) return set_error_cuda(st, "int8_peak.run");
  uint32_t const issued = (mmas_per_sm + kBatch - 1) / kBatch * kBatch;
  double const ops = 2.0 * 128 * 256 * 32 * double(issued) * grid;
  *tops = ops / (double(ms) * 1e-3) / 1e12;
  if (milliseconds) *milliseconds = ms;
  return Q4K_OK;
}
