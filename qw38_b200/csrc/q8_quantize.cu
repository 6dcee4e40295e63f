// Activation producers: bf16/fp32 rows -> Q8 (int8 codes, fp32 scale, int32 sum per 32),
// the fused RMS-norm and SwiGLU producers, and the 36-byte record export.
//
// Arithmetic contract (reference: q8_pack_warp, cuda/q8_device.cuh:5-25):
//   peak = max |x| over the 32 values (columns >= k count as 0),
//   a    = peak == 0 ? 1 : peak / 127      (IEEE fp32 division),
//   z    = clamp(rint(x / a), -127, 127)   (round to nearest even),
//   sum  = sum z.
// A group with a non-finite value (or a scale that is not positive and finite)
// stores zero codes, a NaN scale, sum 0 and raises the failure flag.
//
// Mapping: four lanes own one K32 group, eight values per lane, so a warp covers
// 256 consecutive columns with 16-byte loads and 8-byte stores.
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

constexpr int kThreads = 256;

// Quantise the eight values of this lane; lanes (4j..4j+3) share a group.
__device__ __forceinline__ void pack8(const float (&x)[8], int8_t* codes, float* scales,
                                      int32_t* sums, uint64_t group, uint32_t sub, int* failure) {
  bool finite = true;
  float peak = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    bool f = isfinite(x[i]);
    finite = finite && f;
    peak = fmaxf(peak, f ? fabsf(x[i]) : 0.f);
  }
  peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 1));
  peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 2));
  int fin = finite ? 1 : 0;
  fin &= __shfl_xor_sync(0xffffffffu, fin, 1);
  fin &= __shfl_xor_sync(0xffffffffu, fin, 2);
  float const a = peak == 0.f ? 1.f : __fdiv_rn(peak, 127.f);
  bool const valid = fin && isfinite(a) && a > 0.f;
  int z[8];
  int sum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    z[i] = valid ? max(-127, min(127, __float2int_rn(__fdiv_rn(x[i], a)))) : 0;
    sum += z[i];
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  uint32_t w0 = (uint32_t(z[0]) & 255u) | ((uint32_t(z[1]) & 255u) << 8) |
                ((uint32_t(z[2]) & 255u) << 16) | ((uint32_t(z[3]) & 255u) << 24);
  uint32_t w1 = (uint32_t(z[4]) & 255u) | ((uint32_t(z[5]) & 255u) << 8) |
                ((uint32_t(z[6]) & 255u) << 16) | ((uint32_t(z[7]) & 255u) << 24);
  uint32_t* dst = reinterpret_cast<uint32_t*>(codes + group * 32 + sub * 8);
  dst[0] = w0;
  dst[1] = w1;
  if (sub == 0) {
    scales[group] = valid ? a : __int_as_float(0x7fc00000);
    sums[group] = sum;
    if (!valid) atomicExch(failure, 1);
  }
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<uint16_t>(uint16_t v) { return bf16_bits_to_f32(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

// Vec: rows start 16-byte aligned and k % 8 == 0, so a lane's eight values are
// one (bf16) or two (fp32) aligned 16-byte loads.
template <typename T, bool Vec>
__global__ void __launch_bounds__(kThreads) pack_kernel(const T* __restrict__ in, int8_t* codes,
                                                         float* scales, int32_t* sums, uint32_t m,
                                                         uint32_t k, uint32_t pk, int* failure) {
  pdl_wait();               // the input may come from the kernel before this one
  pdl_launch_dependents();  // the projection that follows may start prefetching its weights (after the wait: the
                            // next launch never runs beside anything older than this one)
  uint32_t const lane = threadIdx.x & 31, sub = lane & 3, grp = lane >> 2;
  uint64_t const chunks_row = pk / 256;
  uint64_t const tasks = uint64_t(m) * chunks_row;
  uint64_t const warps = uint64_t(gridDim.x) * (kThreads / 32);
  for (uint64_t task = uint64_t(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32; task < tasks;
       task += warps) {
    uint32_t const row = uint32_t(task / chunks_row), chunk = uint32_t(task % chunks_row);
    uint32_t const col0 = chunk * 256 + grp * 32 + sub * 8;
    const T* src = in + uint64_t(row) * k;
    float x[8];
    if (Vec && col0 + 8 <= k) {
      if constexpr (sizeof(T) == 2) {
        uint4 v = *reinterpret_cast<const uint4*>(src + col0);
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          x[2 * i] = __uint_as_float(w[i] << 16);
          x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
      } else {
        float4 lo = *reinterpret_cast<const float4*>(src + col0);
        float4 hi = *reinterpret_cast<const float4*>(src + col0 + 4);
        x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
        x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = col0 + i < k ? to_f32<T>(src[col0 + i]) : 0.f;
    }
    pack8(x, codes, scales, sums, uint64_t(row) * (pk / 32) + chunk * 8 + grp, sub, failure);
  }
}

// v = bf16_rne(silu(g) * u); non-finite g or u poisons the value
// (reference: swiglu_pack_kernel, cuda/q4k_q8.cu:52-61).  ffn % 256 == 0.
__global__ void __launch_bounds__(kThreads) swiglu_pack_kernel(const float* __restrict__ gate,
                                                                const float* __restrict__ up,
                                                                int8_t* codes, float* scales,
                                                                int32_t* sums, uint64_t chunks,
                                                                int* failure) {
  uint32_t const lane = threadIdx.x & 31, sub = lane & 3, grp = lane >> 2;
  uint64_t const warps = uint64_t(gridDim.x) * (kThreads / 32);
  for (uint64_t task = uint64_t(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32; task < chunks;
       task += warps) {
    uint64_t const i0 = task * 256 + grp * 32 + sub * 8;
    float4 g0 = *reinterpret_cast<const float4*>(gate + i0), g1 = *reinterpret_cast<const float4*>(gate + i0 + 4);
    float4 u0 = *reinterpret_cast<const float4*>(up + i0), u1 = *reinterpret_cast<const float4*>(up + i0 + 4);
    float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = (g[i] / (1.f + expf(-g[i]))) * u[i];
      if (!isfinite(g[i]) || !isfinite(u[i])) v = __int_as_float(0x7fc00000);
      x[i] = bf16_bits_to_f32(f32_to_bf16_rne(v));
    }
    pack8(x, codes, scales, sums, task * 8 + grp, sub, failure);
  }
}

__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
  for (int off = 16; off; off >>= 1) {
    float o = __shfl_xor_sync(0xffffffffu, v, off);
    v = is_max ? fmaxf(v, o) : v + o;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = scratch[0];
  for (int i = 1; i < kThreads / 32; ++i) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
  return r;
}

// Max-scaled RMS norm, (1 + gamma) gain, bf16 rounding, then the Q8 pack of the
// rounded row (reference: hidden_rms_kernel<3>, cuda/activation.cu:134-190).
// One block per token; hidden % 256 == 0; dynamic shared memory = hidden * 2 bytes.
__global__ void __launch_bounds__(kThreads) hidden_rms_q8_kernel(const float* __restrict__ residual,
                                                                  const uint16_t* __restrict__ gamma,
                                                                  float eps, uint32_t hidden,
                                                                  int8_t* codes, float* scales,
                                                                  int32_t* sums, int* failure) {
  extern __shared__ __align__(16) uint16_t rounded[];
  __shared__ float scratch[kThreads / 32];
  const float* x = residual + uint64_t(blockIdx.x) * hidden;
  float scale = 0.f;
  for (uint32_t i = threadIdx.x; i < hidden; i += kThreads) scale = fmaxf(scale, fabsf(x[i]));
  scale = block_reduce(scale, scratch, true);
  float const safe = scale == 0.f ? 1.f : scale;
  float sumsq = 0.f;
  for (uint32_t i = threadIdx.x; i < hidden; i += kThreads) {
    float s = x[i] / safe;
    sumsq += s * s;
  }
  sumsq = block_reduce(sumsq, scratch, false);
  float const se = sqrtf(eps) / safe;
  float const inv = 1.0f / sqrtf(sumsq / float(hidden) + se * se);
  for (uint32_t i = threadIdx.x; i < hidden; i += kThreads) {
    float g = bf16_bits_to_f32(gamma[i]);
    float v = (1.0f + g) * ((x[i] / safe) * inv);
    rounded[i] = f32_to_bf16_rne(v);
  }
  __syncthreads();
  uint32_t const lane = threadIdx.x & 31, sub = lane & 3, grp = lane >> 2;
  for (uint32_t chunk = threadIdx.x / 32; chunk < hidden / 256; chunk += kThreads / 32) {
    uint32_t const col0 = chunk * 256 + grp * 32 + sub * 8;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = bf16_bits_to_f32(rounded[col0 + i]);
    pack8(v, codes, scales, sums, uint64_t(blockIdx.x) * (hidden / 32) + chunk * 8 + grp, sub, failure);
  }
}

// One thread per K32 group: {fp16 d = a, fp16 s = a * sum, 32 codes}.
__global__ void export_q8_1_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales,
                                   const int32_t* __restrict__ sums, uint64_t groups,
                                   uint32_t* __restrict__ records) {
  uint64_t g = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  float a = scales[g];
  uint32_t d = __half_as_ushort(__float2half_rn(a));
  uint32_t s = __half_as_ushort(__float2half_rn(a * float(sums[g])));
  uint32_t* dst = records + g * 9;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(codes + g * 32);
  dst[0] = d | (s << 16);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[1 + i] = src[i];
}

int grid_for(uint64_t tasks) {
  uint64_t blocks = (tasks + kThreads / 32 - 1) / (kThreads / 32);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return int(blocks ? blocks : 1);
}

}  // namespace

cudaError_t launch_pack_q8(const void* input, bool fp32, Q8Out out, uint32_t k, int* failure,
                           cudaStream_t stream) {
  uint64_t const tasks = uint64_t(out.m) * (out.padded_k / 256);
  int const grid = grid_for(tasks);
  bool const vec = (k % 8 == 0) && (reinterpret_cast<uintptr_t>(input) % 16 == 0);
  if (fp32) {
    auto* in = static_cast<const float*>(input);
    if (vec) return launch_kernel(pack_kernel<float, true>, grid, kThreads, 0, stream, launch_overlap(), in, out.codes, out.scales, out.sums, out.m, k, out.padded_k, failure);
    else return launch_kernel(pack_kernel<float, false>, grid, kThreads, 0, stream, launch_overlap(), in, out.codes, out.scales, out.sums, out.m, k, out.padded_k, failure);
  } else {
    auto* in = static_cast<const uint16_t*>(input);
    if (vec) return launch_kernel(pack_kernel<uint16_t, true>, grid, kThreads, 0, stream, launch_overlap(), in, out.codes, out.scales, out.sums, out.m, k, out.padded_k, failure);
    else return launch_kernel(pack_kernel<uint16_t, false>, grid, kThreads, 0, stream, launch_overlap(), in, out.codes, out.scales, out.sums, out.m, k, out.padded_k, failure);
  }
  return cudaGetLastError();
}

cudaError_t launch_swiglu_pack_q8(const float* gate, const float* up, Q8Out out, int* failure,
                                  cudaStream_t stream) {
  uint64_t const chunks = uint64_t(out.m) * (out.padded_k / 256);
  swiglu_pack_kernel<<<grid_for(chunks), kThreads, 0, stream>>>(gate, up, out.codes, out.scales, out.sums, chunks, failure);
  return cudaGetLastError();
}

cudaError_t launch_hidden_rms_q8(const float* residual, const uint16_t* gamma, float eps,
                                 uint32_t hidden, Q8Out out, int* failure, cudaStream_t stream) {
  size_t const smem = size_t(hidden) * 2;
  if (smem > 48 * 1024) {
    cudaError_t st = cudaFuncSetAttribute(hidden_rms_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (st != cudaSuccess) return st;
  }
  hidden_rms_q8_kernel<<<out.m, kThreads, smem, stream>>>(residual, gamma, eps, hidden, out.codes, out.scales, out.sums, failure);
  return cudaGetLastError();
}

cudaError_t launch_export_q8_1(const int8_t* codes, const float* scales, const int32_t* sums,
                               uint64_t groups, uint8_t* records, cudaStream_t stream) {
  uint64_t const blocks = (groups + 255) / 256;
  export_q8_1_kernel<<<unsigned(blocks), 256, 0, stream>>>(codes, scales, sums, groups, reinterpret_cast<uint32_t*>(records));
  return cudaGetLastError();
}

}  // namespace q4k
