// Epilogue kernels of the decode entry points (q4k_decode_mmv, _paired, _ranges): the four
// DecodeEpilogue forms of the reference (cuda/decode_mmv.hpp:45-51) applied to fp32 projection
// rows.  StoreFp32 and ResidualAddFp32 need no kernel of their own: the projection writes the
// destination directly (the residual is its last fp32 add, cuda/q4k_q8.cu:100).
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

// sigmoid / SiLU exactly as the reference's decode epilogue states them
// (cuda/decode_mmv.cu:78-89): the exponential is always taken of a non-positive number.
__device__ __forceinline__ float sigmoid_fp32(float u) {
  if (u >= 0.0f) {
    float const e = expf(-u);
    return 1.0f / (1.0f + e);
  }
  float const e = expf(u);
  return e / (1.0f + e);
}

__global__ void store_bf16_kernel(const float* __restrict__ in, uint16_t* __restrict__ out, uint64_t count) {
  pdl_wait();
  pdl_launch_dependents();  // after the wait: the next launch never runs beside anything older than this one
  uint64_t const i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) out[i] = f32_to_bf16_rne(in[i]);
}

// y = bf16(SiLU(gate) * up)  (SwigluStoreBf16, cuda/decode_mmv.cu:238-242)
__global__ void swiglu_store_bf16_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                         uint16_t* __restrict__ out, uint64_t count) {
  pdl_wait();
  pdl_launch_dependents();  // after the wait: the next launch never runs beside anything older than this one
  uint64_t const i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) {
    float const g = gate[i];
    out[i] = f32_to_bf16_rne(g * sigmoid_fp32(g) * up[i]);
  }
}

}  // namespace

cudaError_t launch_store_bf16(const float* in, uint16_t* out, uint64_t count, cudaStream_t stream) {
  if (count == 0) return cudaSuccess;
  return launch_kernel(store_bf16_kernel, unsigned((count + 255) / 256), 256, 0, stream, launch_overlap(), in, out, count);
}

cudaError_t launch_swiglu_store_bf16(const float* gate, const float* up, uint16_t* out, uint64_t count, cudaStream_t stream) {
  if (count == 0) return cudaSuccess;
  return launch_kernel(swiglu_store_bf16_kernel, unsigned((count + 255) / 256), 256, 0, stream, launch_overlap(), gate, up, out, count);
}

}  // namespace q4k
