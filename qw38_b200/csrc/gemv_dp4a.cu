// Decode GEMV for 1..4 tokens: HBM-bound stream over the split-tile Q4_K weights on dp4a.
//
// Equation per output (reference: mmvq, cuda/q4k_q8.cu:63-101):
//   out[t][row] = sum_g a[t,g] * ((d*sc_g) * dot_g - (dmin*m_g) * sum[t,g]) (+ residual)
// with dot_g an exact int32 dot of 32 unsigned 4-bit codes and 32 int8 activations, reset for
// every K32 group.  The kernel is issue-bound before it is bandwidth-bound, so the mapping is
// chosen to spend few instructions per byte:
//   * a warp iteration covers two super-blocks of one row group (2 KiB of codes); lane
//     (h = lane/16, r = (lane/2)%8, j = lane%2) owns row r, super-block h and the four K32
//     groups 4j..4j+3: four 16-byte code loads and one 16-byte metadata load per iteration,
//     both six-bit words of the lane's four groups come out of one byte-parallel decode;
//   * low nibbles (even columns) go through (w & 0x0f0f0f0f), high nibbles (odd columns)
//     through (w & 0xf0f0f0f0) with an unsigned-by-signed dp4a, which yields 16 * dot and is
//     shifted back once per group -- no per-word shift;
//   * per super-block and row, d and dmin are applied once: X = sum a_g * (sc_g * dot_g),
//     Y = sum m_g * (a_g * sum_g), acc += d * X - dmin * Y, the integer products converted
//     to fp32 by the 1.5 * 2^23 bias trick on the integer pipe;
//   * activations are staged once per block in shared memory as (even bytes, odd bytes) words,
//     the two halves of a super-block 144 bytes apart so the two j lanes hit different banks.
// A block of 8 warps takes `rgc` row groups and splits each one's K range over 8/rgc warps;
// slice sums are added in slice order.
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kActKb = 288;  // bytes of staged activations per token and super-block (128 + 16 pad + 128 + 16 pad)
constexpr uint32_t kMagicI = 0x4B400000u;
constexpr float kMagicF = 12582912.0f;

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

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {  // unsigned bytes x signed bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Exact dot of one K32 group: z0 = {E0,O0,E1,O1}, z1 = {E2,O2,E3,O3}.
__device__ __forceinline__ int dot32(const uint4& w, const uint4& z0, const uint4& z1) {
  int lo = 0, hi = 0;
  lo = dp4a_us(w.x & 0x0f0f0f0fu, z0.x, lo);
  hi = dp4a_us(w.x & 0xf0f0f0f0u, z0.y, hi);
  lo = dp4a_us(w.y & 0x0f0f0f0fu, z0.z, lo);
  hi = dp4a_us(w.y & 0xf0f0f0f0u, z0.w, hi);
  lo = dp4a_us(w.z & 0x0f0f0f0fu, z1.x, lo);
  hi = dp4a_us(w.z & 0xf0f0f0f0u, z1.y, hi);
  lo = dp4a_us(w.w & 0x0f0f0f0fu, z1.z, lo);
  hi = dp4a_us(w.w & 0xf0f0f0f0u, z1.w, hi);
  return lo + (hi >> 4);  // hi is an exact multiple of 16
}

// Shared memory: [M][tiles_k][288] permuted codes | [M][G] a | [M][G] a*float(sum) | [8 warps][8 rows][M] slice sums
template <int M, bool Dump>
__global__ void __launch_bounds__(kThreads) gemv_dp4a_kernel(WeightView w, Q8View x, float* __restrict__ out,
                                                             const float* __restrict__ residual,
                                                             int32_t* __restrict__ partials, uint32_t rgc, bool wide) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();  // activations (and the residual) may come from the kernel before this one
  pdl_launch_dependents();  // after the wait: the next launch never runs beside anything older than this one
  uint32_t const pk = x.padded_k, G = pk / 32, tiles_k = w.tiles_k;
  uint8_t* const zs = smem;
  float* const as = reinterpret_cast<float*>(smem + size_t(M) * tiles_k * kActKb);
  float* const ws = as + size_t(M) * G;
  float* const red = ws + size_t(M) * G;

  uint32_t const lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t const h = lane >> 4, r = (lane >> 1) & 7, j = lane & 1;
  uint32_t const ks = kWarps / rgc;
  uint32_t const rg = blockIdx.x * rgc + warp / ks, slice = warp % ks;
  uint32_t const rgs = w.padded_n / 8;
  bool const active = rg < rgs;
  uint32_t const kb0 = (slice * tiles_k) / ks, kb1 = ((slice + 1) * tiles_k) / ks;

  const uint8_t* const cp = w.codes + (uint64_t(active ? rg : 0) * tiles_k) * 1024 + r * 128 + j * 64;
  const uint8_t* const mp = w.meta + (uint64_t(active ? rg : 0) * tiles_k) * 128 + r * 16;

  // First weight loads go out before the activation staging so they overlap it.
  uint4 wq[4], wm;
  uint32_t kb = kb0 + h;
  bool have = active && kb < kb1;
#pragma unroll
  for (int i = 0; i < 4; ++i) wq[i] = make_uint4(0, 0, 0, 0);
  wm = make_uint4(0, 0, 0, 0);
  if (have) {
#pragma unroll
    for (int i = 0; i < 4; ++i) wq[i] = load16(cp + uint64_t(kb) * 1024 + i * 16, wide);
    wm = load16_meta(mp + uint64_t(kb) * 128, wide);
  }

  // Stage activations: a 16-byte source chunk holds half a K32 group (columns 16c..16c+15).
  {
    uint32_t const chunks = pk / 16;
    bool const z16 = (reinterpret_cast<uintptr_t>(x.codes) & 15) == 0;
    for (uint32_t t = 0; t < M; ++t) {
      const uint8_t* const src = reinterpret_cast<const uint8_t*>(x.codes) + size_t(t) * pk;
      uint8_t* const dst = zs + size_t(t) * tiles_k * kActKb;
      for (uint32_t c = threadIdx.x; c < chunks; c += kThreads) {
        uint4 z;
        if (z16) z = __ldg(reinterpret_cast<const uint4*>(src + c * 16));
        else {
          const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src + c * 16);
          z = make_uint4(__ldg(s32), __ldg(s32 + 1), __ldg(s32 + 2), __ldg(s32 + 3));
        }
        uint32_t const kbi = c >> 4, g = (c >> 1) & 7, half = c & 1;
        uint32_t const off = kbi * kActKb + (g >> 2) * 144 + (g & 3) * 32 + half * 16;
        *reinterpret_cast<uint4*>(dst + off) =
            make_uint4(even_bytes(z.x, z.y), odd_bytes(z.x, z.y), even_bytes(z.z, z.w), odd_bytes(z.z, z.w));
      }
    }
    for (uint32_t i = threadIdx.x; i < M * G; i += kThreads) {
      float const a = __ldg(x.scales + i);
      as[i] = a;
      ws[i] = a * float(__ldg(x.sums + i));
    }
  }
  __syncthreads();

  float acc[M];
#pragma unroll
  for (int t = 0; t < M; ++t) acc[t] = 0.f;

  if (active) {
    uint32_t const row = rg * 8 + r;
    for (uint32_t base = kb0; base < kb1; base += 2) {
      uint4 cq[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) cq[i] = wq[i];
      uint4 const cm = wm;
      bool const cur = have;
      uint32_t const ckb = kb;
      kb = base + 2 + h;
      have = kb < kb1;
      if (have) {
#pragma unroll
        for (int i = 0; i < 4; ++i) wq[i] = load16(cp + uint64_t(kb) * 1024 + i * 16, wide);
        wm = load16_meta(mp + uint64_t(kb) * 128, wide);
      }
      if (!cur) continue;  // odd tail: this half-warp has no super-block in the last iteration
      float const d = fp16_bits_to_f32(cm.x & 0xffffu), ndmin = -fp16_bits_to_f32(cm.x >> 16);
      ScaleMinWords const sm = decode_scale_min(cm.y, cm.z, cm.w);
      uint32_t const scw = j ? sm.sc_hi : sm.sc_lo, mnw = j ? sm.mn_hi : sm.mn_lo;
      int sc[4];
      float fm[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sc[i] = int(byte_of(scw, i));
        fm[i] = __uint_as_float(kMagicI | byte_of(mnw, i)) - kMagicF;  // float(m_g) without the conversion pipe
      }
      uint32_t const gi = ckb * 8 + j * 4;
#pragma unroll
      for (int t = 0; t < M; ++t) {
        const uint4* const zp = reinterpret_cast<const uint4*>(zs + (size_t(t) * tiles_k + ckb) * kActKb + j * 144);
        float4 const a4 = *reinterpret_cast<const float4*>(as + size_t(t) * G + gi);
        float4 const w4 = *reinterpret_cast<const float4*>(ws + size_t(t) * G + gi);
        float const av[4] = {a4.x, a4.y, a4.z, a4.w}, wv[4] = {w4.x, w4.y, w4.z, w4.w};
        float X = 0.f, Y = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          int const dot = dot32(cq[i], zp[2 * i], zp[2 * i + 1]);
          // sc * dot is an exact integer below 2^22; adding the bias in the multiply-add converts it
          float const q = __uint_as_float(uint32_t(dot * sc[i]) + kMagicI) - kMagicF;
          X = fmaf(av[i], q, X);
          Y = fmaf(fm[i], wv[i], Y);
          if (Dump && row < w.n) partials[(uint64_t(t) * w.n + row) * G + gi + i] = dot;
        }
        acc[t] = fmaf(d, X, acc[t]);
        acc[t] = fmaf(ndmin, Y, acc[t]);
      }
    }
  }
  // Fixed-order reduction: the four lanes of a row (j, then h), then the K slices in slice order.
#pragma unroll
  for (int t = 0; t < M; ++t) {
    acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 1);
    acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 16);
    if ((lane & 17u) == 0) red[(warp * 8 + r) * M + t] = acc[t];
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
cudaError_t launch_m(const WeightView& w, const Q8View& x, float* out, const float* residual, int32_t* partials,
                     cudaStream_t stream) {
  uint32_t const rgs = w.padded_n / 8;
  // Row groups per block: enough blocks to fill the machine several times over, while each
  // warp keeps at least a few super-blocks of K.
  uint32_t rgc = 8;
  while (rgc > 1 && (rgs / rgc < 148 * 3 || (w.tiles_k * rgc) / kWarps > 24)) rgc >>= 1;
  while (rgc < 8 && w.tiles_k * rgc < 2 * kWarps) rgc <<= 1;  // fewer than two super-blocks per warp
  uint32_t const grid = (rgs + rgc - 1) / rgc;
  size_t const G = x.padded_k / 32;
  size_t const smem = size_t(M) * w.tiles_k * kActKb + 2 * size_t(M) * G * 4 + kWarps * 8 * M * 4;
  bool const wide = (reinterpret_cast<uintptr_t>(w.codes) % 16 == 0) && (reinterpret_cast<uintptr_t>(w.meta) % 16 == 0);
  auto kernel = partials ? gemv_dp4a_kernel<M, true> : gemv_dp4a_kernel<M, false>;
  if (smem > 48 * 1024) {
    cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (st != cudaSuccess) return st;
  }
  return launch_kernel(kernel, grid, kThreads, smem, stream, launch_overlap(), w, x, out, residual, partials, rgc, wide);
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
