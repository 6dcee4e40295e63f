// Decode GEMV for 1..4 tokens: HBM-bound stream over the split-tile Q4_K weights.
//
// Equation per output (reference: mmvq, cuda/q4k_q8.cu:63-101):
//   out[t][row] = sum_g a[t,g] * ((d*sc_g) * float(dot_g) - (dmin*m_g) * float(sum[t,g])) (+ residual)
// with dot_g an exact int32 dot of 32 unsigned 4-bit codes and 32 int8 activations,
// reset for every K32 group.
//
// Data movement: a row group (8 rows) is one contiguous run of tiles_k KiB of codes and
// tiles_k*128 B of metadata.  A block of 8 warps takes `rgc` row groups and splits each
// one's K range over 8/rgc warps.  In a warp, lane (r = lane/4, j = lane%4) owns row r and
// the K32 groups 2j, 2j+1 of the current super-block: two 16-byte loads per super-block, so
// a warp instruction reads 512 contiguous bytes.  Activations are staged once per block in
// shared memory, de-interleaved into even/odd columns to match the nibble order of a raw
// weight word (low nibbles = even columns, high nibbles = odd columns).
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;

__device__ __forceinline__ uint4 load16(const uint8_t* p, bool wide) {
  if (wide) return __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
  return make_uint4(__ldg(q), __ldg(q + 1), __ldg(q + 2), __ldg(q + 3));
}
__device__ __forceinline__ uint4 load16_meta(const uint8_t* p, bool wide) {
  if (wide) return __ldg(reinterpret_cast<const uint4*>(p));
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
  uint32_t h[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) h[i] = __ldg(q + i);
  return make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
}

__device__ __forceinline__ int dot32(const uint4& w, const uint4& z0, const uint4& z1) {
  // z0 = {E0,O0,E1,O1}, z1 = {E2,O2,E3,O3}: even / odd columns of weight words 0..3.
  int d = 0;
  d = __dp4a(int(w.x & 0x0f0f0f0fu), int(z0.x), d);
  d = __dp4a(int((w.x >> 4) & 0x0f0f0f0fu), int(z0.y), d);
  d = __dp4a(int(w.y & 0x0f0f0f0fu), int(z0.z), d);
  d = __dp4a(int((w.y >> 4) & 0x0f0f0f0fu), int(z0.w), d);
  d = __dp4a(int(w.z & 0x0f0f0f0fu), int(z1.x), d);
  d = __dp4a(int((w.z >> 4) & 0x0f0f0f0fu), int(z1.y), d);
  d = __dp4a(int(w.w & 0x0f0f0f0fu), int(z1.z), d);
  d = __dp4a(int((w.w >> 4) & 0x0f0f0f0fu), int(z1.w), d);
  return d;
}

// Shared memory: [M][padded_k] permuted codes | [M][G] scales | [M][G] float(sums) |
// [8 warps][8 rows][M] slice sums.
template <int M, bool Dump>
__global__ void __launch_bounds__(kThreads) gemv_dp4a_kernel(WeightView w, Q8View x, float* __restrict__ out,
                                                             const float* __restrict__ residual,
                                                             int32_t* __restrict__ partials, uint32_t rgc,
                                                             bool wide) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t const pk = x.padded_k, G = pk / 32, tiles_k = w.tiles_k;
  uint8_t* zs = smem;
  float* as = reinterpret_cast<float*>(smem + size_t(M) * pk);
  float* fs = as + size_t(M) * G;
  float* red = fs + size_t(M) * G;

  uint32_t const lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t const r = lane >> 2, j = lane & 3;
  uint32_t const ks = kWarps / rgc;
  uint32_t const rg = blockIdx.x * rgc + warp / ks, slice = warp % ks;
  uint32_t const rgs = w.padded_n / 8;
  bool const active = rg < rgs;
  uint32_t const kb0 = (slice * tiles_k) / ks, kb1 = ((slice + 1) * tiles_k) / ks;

  const uint8_t* cp = w.codes + (uint64_t(active ? rg : 0) * tiles_k) * 1024 + r * 128 + j * 32;
  const uint8_t* mp = w.meta + (uint64_t(active ? rg : 0) * tiles_k) * 128 + r * 16;

  // First weight loads go out before the activation staging so they overlap it.
  uint4 wa = make_uint4(0, 0, 0, 0), wb = wa, wm = wa;
  if (active && kb0 < kb1) {
    wa = load16(cp + uint64_t(kb0) * 1024, wide);
    wb = load16(cp + uint64_t(kb0) * 1024 + 16, wide);
    wm = load16_meta(mp + uint64_t(kb0) * 128, wide);
  }

  // Stage activations: 8 source bytes (columns 8c..8c+7 of group g) -> (even, odd) words.
  {
    uint32_t const pairs_row = pk / 8;
    for (uint32_t i = threadIdx.x; i < M * pairs_row; i += kThreads) {
      uint32_t const t = i / pairs_row, p = i % pairs_row;
      uint32_t const kb = p >> 5, g = (p >> 2) & 7, c = p & 3;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(x.codes + size_t(t) * pk + size_t(p) * 8);
      uint32_t z0 = __ldg(src), z1 = __ldg(src + 1);
      uint32_t const chunk = (((g & 1) * 2 + (c >> 1)) * 4 + (g >> 1));
      uint2* dst = reinterpret_cast<uint2*>(zs + size_t(t) * pk + kb * 256 + chunk * 16 + (c & 1) * 8);
      *dst = make_uint2(even_bytes(z0, z1), odd_bytes(z0, z1));
    }
    for (uint32_t i = threadIdx.x; i < M * G; i += kThreads) {
      as[i] = __ldg(x.scales + i);
      fs[i] = float(__ldg(x.sums + i));
    }
  }
  __syncthreads();

  float acc[M];
#pragma unroll
  for (int t = 0; t < M; ++t) acc[t] = 0.f;

  if (active) {
    uint32_t const row = rg * 8 + r;
    for (uint32_t kb = kb0; kb < kb1; ++kb) {
      uint4 const ca = wa, cb = wb, cm = wm;
      if (kb + 1 < kb1) {
        wa = load16(cp + uint64_t(kb + 1) * 1024, wide);
        wb = load16(cp + uint64_t(kb + 1) * 1024 + 16, wide);
        wm = load16_meta(mp + uint64_t(kb + 1) * 128, wide);
      }
      float const d = fp16_bits_to_f32(cm.x & 0xffffu), dmin = fp16_bits_to_f32(cm.x >> 16);
      ScaleMinWords const sm = decode_scale_min(cm.y, cm.z, cm.w);
      uint32_t const scw = j < 2 ? sm.sc_lo : sm.sc_hi, mnw = j < 2 ? sm.mn_lo : sm.mn_hi;
      uint32_t const b0 = (2 * j) & 3;
      float const D0 = d * float(byte_of(scw, b0)), D1 = d * float(byte_of(scw, b0 + 1));
      float const N0 = dmin * float(byte_of(mnw, b0)), N1 = dmin * float(byte_of(mnw, b0 + 1));
      uint32_t const gi = kb * 8 + 2 * j;
#pragma unroll
      for (int t = 0; t < M; ++t) {
        const uint4* zp = reinterpret_cast<const uint4*>(zs + size_t(t) * pk + kb * 256 + j * 16);
        uint4 const z0 = zp[0], z1 = zp[4], z2 = zp[8], z3 = zp[12];
        int const dot0 = dot32(ca, z0, z1), dot1 = dot32(cb, z2, z3);
        float2 const a2 = *reinterpret_cast<const float2*>(as + size_t(t) * G + gi);
        float2 const s2 = *reinterpret_cast<const float2*>(fs + size_t(t) * G + gi);
        acc[t] += a2.x * (D0 * float(dot0) - N0 * s2.x);
        acc[t] += a2.y * (D1 * float(dot1) - N1 * s2.y);
        if (Dump && row < w.n) {
          int32_t* p = partials + (uint64_t(t) * w.n + row) * G + gi;
          p[0] = dot0;
          p[1] = dot1;
        }
      }
    }
  }
  // Fixed-order reduction: the four lanes of a row, then the K slices in slice order.
#pragma unroll
  for (int t = 0; t < M; ++t) {
    acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 1);
    acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 2);
    if (j == 0) red[(warp * 8 + r) * M + t] = acc[t];
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < rgc * 8 * M; i += kThreads) {
    uint32_t const t = i % M, rr = (i / M) % 8, lrg = i / (8 * M);
    uint32_t const row = (blockIdx.x * rgc + lrg) * 8 + rr;
    if (row >= w.n) continue;
    float v = 0.f;
    for (uint32_t s = 0; s < ks; ++s) v += red[((lrg * ks + s) * 8 + rr) * M + t];
    uint64_t const o = uint64_t(t) * w.n + row;
    out[o] = v + (residual ? residual[o] : 0.f);
  }
}

template <int M>
cudaError_t launch_m(const WeightView& w, const Q8View& x, float* out, const float* residual,
                     int32_t* partials, cudaStream_t stream) {
  uint32_t const rgs = w.padded_n / 8;
  // Row groups per block: enough blocks to fill the machine several times over, while each
  // warp keeps at least a few super-blocks of K.
  uint32_t rgc = 8;
  while (rgc > 1 && (rgs / rgc < 148 * 6 || (w.tiles_k * rgc) / kWarps > 24)) rgc >>= 1;
  while (rgc < 8 && w.tiles_k * rgc < kWarps) rgc <<= 1;  // fewer super-blocks than warps
  uint32_t const grid = (rgs + rgc - 1) / rgc;
  size_t const G = x.padded_k / 32;
  size_t const smem = size_t(M) * x.padded_k + 2 * size_t(M) * G * 4 + kWarps * 8 * M * 4;
  bool const wide = (reinterpret_cast<uintptr_t>(w.codes) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(w.meta) % 16 == 0);
  auto kernel = partials ? gemv_dp4a_kernel<M, true> : gemv_dp4a_kernel<M, false>;
  if (smem > 48 * 1024) {
    cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (st != cudaSuccess) return st;
  }
  kernel<<<grid, kThreads, smem, stream>>>(w, x, out, residual, partials, rgc, wide);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemv_dp4a(const WeightView& w, const Q8View& x, float* out, const float* residual,
                             int32_t* partials, cudaStream_t stream) {
  switch (x.m) {
    case 1: return launch_m<1>(w, x, out, residual, partials, stream);
    case 2: return launch_m<2>(w, x, out, residual, partials, stream);
    case 3: return launch_m<3>(w, x, out, residual, partials, stream);
    case 4: return launch_m<4>(w, x, out, residual, partials, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace q4k
