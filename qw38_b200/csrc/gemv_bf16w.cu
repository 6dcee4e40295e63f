// Decode GEMV of the reference's older activation policy (DecodeActivationPolicy::Bf16,
// cuda/decode_mmv.cu:121-140, 182-250): every weight is reconstructed in fp32 as
//     decoded = fsub_rn(fmul_rn(fmul_rn(d, sc), q), fmul_rn(dmin, mn))
// rounded to bf16, and multiplied with the bf16 activation by an fp32 FMA; a row's products are
// summed in fp32 by a warp tree.  The rounding steps are the reference's (and the CPU
// statement's, src/compiler/quantization/reference.cpp:140-163); only the summation order is free,
// which is what the reference's own tolerance (decode_mmv_tol) covers.
//
// CUDA-core bound by construction (about nine operations per weight), so the layout is plain:
// a block takes one row group (eight rows, one contiguous run of tiles), one warp per row; a lane
// owns the eight columns of one 4-byte code word per super-block, so a warp reads one 128-byte
// line per step; activations are staged once per block as fp32 in shared memory.
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

constexpr int kThreads = 256;

template <int M>
__global__ void __launch_bounds__(kThreads) gemv_bf16w_kernel(WeightView w, const uint16_t* __restrict__ x, uint32_t k,
                                                             uint32_t padded_k, float* __restrict__ out,
                                                             const float* __restrict__ residual) {
  extern __shared__ __align__(16) float xs[];  // [M][padded_k], zero beyond k
  pdl_wait();
  pdl_launch_dependents();  // after the wait: the next launch never runs beside anything older than this one
  for (uint32_t i = threadIdx.x; i < M * padded_k; i += kThreads) {
    uint32_t const t = i / padded_k, c = i % padded_k;
    xs[i] = c < k ? bf16_bits_to_f32(x[size_t(t) * k + c]) : 0.f;
  }
  __syncthreads();
  uint32_t const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t const row = blockIdx.x * 8 + warp;
  if (row >= w.n) return;
  uint32_t const group = lane >> 2;
  float acc[M];
#pragma unroll
  for (int t = 0; t < M; ++t) acc[t] = 0.f;
  for (uint32_t kb = 0; kb < w.tiles_k; ++kb) {
    uint64_t const tr = tile_row(row, kb, w.tiles_k);
    uint32_t const word = *reinterpret_cast<const uint32_t*>(w.codes + tr * 128 + lane * 4);
    const uint8_t* const meta = w.meta + tr * 16;
    uint32_t const dd = *reinterpret_cast<const uint32_t*>(meta);
    const uint8_t* const p = meta + 4;
    uint32_t const sc = group < 4 ? p[group] & 63u : (p[group + 4] & 15u) | ((p[group - 4] >> 6) << 4);
    uint32_t const mn = group < 4 ? p[group + 4] & 63u : (p[group + 4] >> 4) | ((p[group] >> 6) << 4);
    float const D = __fmul_rn(fp16_bits_to_f32(dd & 0xffffu), float(sc));
    float const Mn = __fmul_rn(fp16_bits_to_f32(dd >> 16), float(mn));
    float const* const xk = xs + kb * 256 + lane * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float const decoded = __fsub_rn(__fmul_rn(D, float((word >> (4 * i)) & 15u)), Mn);
      float const wv = bf16_bits_to_f32(f32_to_bf16_rne(decoded));
#pragma unroll
      for (int t = 0; t < M; ++t) acc[t] = fmaf(wv, xk[t * padded_k + i], acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < M; ++t) {
    float v = acc[t];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) {
      size_t const o = size_t(t) * w.n + row;
      out[o] = residual ? residual[o] + v : v;
    }
  }
}

template <int M>
cudaError_t launch_m(const WeightView& w, const uint16_t* x, uint32_t k, uint32_t padded_k, float* out, const float* residual,
                     cudaStream_t stream) {
  size_t const smem = size_t(M) * padded_k * 4;
  auto kernel = gemv_bf16w_kernel<M>;
  if (smem > 48 * 1024) {
    cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (st != cudaSuccess) return st;
  }
  return launch_kernel(kernel, (w.n + 7) / 8, kThreads, smem, stream, launch_overlap(), w, x, k, padded_k, out, residual);
}

}  // namespace

// out[t][row] (+ residual[t][row]) for m bf16 input rows; token rows are processed two at a time.
cudaError_t launch_gemv_bf16w(const WeightView& w, const uint16_t* x, uint32_t m, uint32_t k, uint32_t padded_k, float* out,
                              const float* residual, cudaStream_t stream) {
  for (uint32_t t = 0; t < m;) {
    uint32_t const chunk = m - t >= 2 ? 2 : 1;
    float* const o = out + size_t(t) * w.n;
    const float* const r = residual ? residual + size_t(t) * w.n : nullptr;
    const uint16_t* const xi = x + size_t(t) * k;
    cudaError_t st = chunk == 2 ? launch_m<2>(w, xi, k, padded_k, o, r, stream) : launch_m<1>(w, xi, k, padded_k, o, r, stream);
    if (st != cudaSuccess) return st;
    t += chunk;
  }
  return cudaSuccess;
}

}  // namespace q4k
