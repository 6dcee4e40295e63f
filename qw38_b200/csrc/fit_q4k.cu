// Q4_K fitter on the device: float (or bf16) weights -> Q4_K super-blocks, bit for bit what the
// reference's offline compiler produces (compiler::quantize_q4k_block,
// src/compiler/quantization/q4k.cpp:186-278, itself the published llama.cpp Q4_K fit:
// weighted least-squares search over 21 candidate grid steps per 32-weight group, six-bit
// compression of the eight group scales/minima against fp16 super-block scales, then a
// re-quantisation of every weight against the compressed scales).
//
// The fit is a chain of fp32 roundings whose order is part of the result: all sums run over the
// 32 weights of a group in index order, the candidate steps run in ascending order, and an
// accepted candidate moves the minimum that later candidates quantise against.  One THREAD
// therefore owns one group and runs the search exactly in that order; parallelism comes from
// the number of groups (a 5120 x 17408 matrix has 2.8 million).  Every float operation is an
// explicit round-to-nearest intrinsic so that no multiply-add is contracted (the reference
// builds its host code with -ffp-contract=off, src/CMakeLists.txt:35-37).
//
// A block of 128 threads fits 16 consecutive super-blocks.  Their 4096 weights are loaded with
// coalesced reads into shared memory at a row stride of 33 words, from where each thread takes
// "its" 32 weights into registers without bank conflicts.  Output is either the logical form of the
// reference's compiler (int8 codes [blocks][256] + 16 metadata bytes per block) or directly the
// split-tile device layout (src/format/pack.cpp:175-222), which fuses the pack step.
#include <cuda_fp16.h>

#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

constexpr int kFitThreads = 128;            // groups per block
constexpr int kFitBlocks = kFitThreads / 8;  // super-blocks per block
constexpr int kRow = 33;                     // shared-memory words per group

enum FitStatus : uint8_t { kFitOk = 0, kFitNonfinite = 1, kFitRange = 2, kFitReciprocal = 3, kFitCompress = 4, kFitHalf = 5 };

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float quo(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ bool finite(float v) { return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u; }

// Round to nearest through the 1.5 * 2^23 bias (q4k.cpp:87-92): exact for |v| < 2^22, and the
// same bit pattern arithmetic outside that range.
__device__ __forceinline__ int nearest(float v) {
  return int(__float_as_uint(add(v, 12582912.f)) & 0x007fffffu) - 0x00400000;
}
__device__ __forceinline__ int level(float v) { return min(15, max(0, nearest(v))); }

// The same rounding kept as a float: (v + 1.5 * 2^23) - 1.5 * 2^23 is v rounded to the nearest even integer
// whenever |v| < 2^22, and clamping that to [0, 15] gives float(level(v)) without a conversion
// instruction.  Only used where the caller has bounded |v|.
__device__ __forceinline__ float level_bounded(float v) {
  return fminf(fmaxf(sub(add(v, 12582912.f), 12582912.f), 0.f), 15.f);
}
template <bool Bounded>
__device__ __forceinline__ float level_f(float v) { return Bounded ? level_bounded(v) : float(level(v)); }

struct GroupFit {
  float scale, the_min;  // results of the search: step and (negated) minimum
  float grid, origin;    // the levels the search settled on are level(grid * (x - origin))
};

struct Moments { float l, l2, xl; };

// Weighted moments of the levels a candidate grid assigns (the middle loop of the search).
template <bool Bounded>
__device__ __forceinline__ Moments moments(const float (&x)[32], const float (&w)[32], float grid, float origin) {
  Moments s{0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float const v = x[i];
    float const l = level_f<Bounded>(mul(grid, sub(v, origin)));
    float const wl = mul(w[i], l);
    s.l = add(s.l, wl);
    s.l2 = add(s.l2, mul(wl, l));
    s.xl = add(s.xl, mul(wl, v));
  }
  return s;
}

// Weighted squared error of step * level + base against the weights.
template <bool Bounded>
__device__ __forceinline__ float fit_error(const float (&x)[32], const float (&w)[32], float grid, float origin, float step, float base) {
  float err = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float const v = x[i];
    float const l = level_f<Bounded>(mul(grid, sub(v, origin)));
    float const diff = sub(add(mul(step, l), base), v);
    err = add(err, mul(w[i], mul(diff, diff)));
  }
  return err;
}

// The search over one group (make_qkx2_quants with n=32, nmax=15, rmin=-1, rdelta=0.1, nstep=20,
// squared error; q4k.cpp:94-172).  x: the group's 32 weights, held in registers (every loop over them is
// fully unrolled); the importance of a weight, average + |x|, is computed once.
__device__ GroupFit fit_group(const float (&x)[32], float average) {
  float w[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) w[i] = add(average, fabsf(x[i]));
  float lo = x[0], hi = x[0];
  float sum_w = w[0];
  float sum_x = mul(sum_w, x[0]);
#pragma unroll
  for (int i = 1; i < 32; ++i) {
    float const v = x[i];
    if (v < lo) lo = v;
    if (v > hi) hi = v;
    sum_w = add(sum_w, w[i]);
    sum_x = add(sum_x, mul(w[i], v));
  }
  float const x_min = lo;  // smallest weight, before the minimum is capped at zero
  if (lo > 0.f) lo = 0.f;
  GroupFit fit;
  if (hi == lo) {
    fit.scale = 0.f; fit.the_min = -lo; fit.grid = 0.f; fit.origin = lo;
    return fit;
  }
  float grid = quo(15.f, sub(hi, lo));
  float scale = quo(1.f, grid);
  float best = fit_error<false>(x, w, grid, lo, scale, lo);
  fit.grid = grid; fit.origin = lo;
  float floor_ = lo;  // the minimum candidates quantise against; moves when one is accepted
  for (int step = 0; step <= 20; ++step) {
    // (rmin + rdelta*step + nmax) / (max - min), with the minimum as moved so far.
    float const cand_grid = quo(add(add(-1.f, mul(0.1f, float(step))), 15.f), sub(hi, floor_));
    // Every grid * (x - origin) of this candidate is bounded by |grid| times the larger distance of
    // the extreme weights from the origin (rounding is monotonic); below 2^22 the float rounding applies.
    bool const bounded = mul(fabsf(cand_grid), fmaxf(fabsf(sub(hi, floor_)), fabsf(sub(x_min, floor_)))) < 4194304.f;
    Moments const s = bounded ? moments<true>(x, w, cand_grid, floor_) : moments<false>(x, w, cand_grid, floor_);
    float const det = sub(mul(sum_w, s.l2), mul(s.l, s.l));
    if (!(det > 0.f)) continue;
    float cand_scale = quo(sub(mul(sum_w, s.xl), mul(sum_x, s.l)), det);
    float cand_min = quo(sub(mul(s.l2, sum_x), mul(s.l, s.xl)), det);
    if (cand_min > 0.f) {
      cand_min = 0.f;
      cand_scale = quo(s.xl, s.l2);
    }
    float const err = bounded ? fit_error<true>(x, w, cand_grid, floor_, cand_scale, cand_min)
                              : fit_error<false>(x, w, cand_grid, floor_, cand_scale, cand_min);
    if (err < best) {
      best = err;
      scale = cand_scale;
      fit.grid = cand_grid;
      fit.origin = floor_;
      floor_ = cand_min;
    }
  }
  fit.scale = scale;
  fit.the_min = -floor_;
  return fit;
}

// Input element -> float.
__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(uint16_t v) { return __uint_as_float(uint32_t(v) << 16); }

// In: weights [rows][tiles_k * 256] row-major.  Out, Split = false: codes int8 [blocks][256], metadata
// [blocks][16], block = row * tiles_k + kb.  Out, Split = true: tile rows of the split layout for
// padded_rows = ceil8(rows); rows past `rows` are written as zeros.  status (optional): one byte
// per block with the FitStatus of that block; failure is set to 1 when any block fails, and a
// failed block is written as zeros.
template <typename In, bool Split>
__global__ void __launch_bounds__(kFitThreads) fit_q4k_kernel(const In* __restrict__ weights, uint32_t rows, uint32_t out_rows,
                                                              uint32_t tiles_k, uint8_t* __restrict__ codes,
                                                              uint8_t* __restrict__ meta, uint8_t* __restrict__ status,
                                                              int* __restrict__ failure) {
  __shared__ float xs[kFitThreads * kRow];
  __shared__ float scales[kFitThreads], minima[kFitThreads];
  __shared__ uint8_t flaw[kFitThreads];

  uint64_t const in_blocks = uint64_t(rows) * tiles_k, out_blocks = uint64_t(out_rows) * tiles_k;
  uint64_t const block0 = uint64_t(blockIdx.x) * kFitBlocks;
  uint32_t const tid = threadIdx.x;

  for (uint32_t e = tid; e < kFitBlocks * 256; e += kFitThreads) {
    uint64_t const b = block0 + (e >> 8);
    xs[(e >> 5) * kRow + (e & 31)] = b < in_blocks ? widen(weights[b * 256 + (e & 255)]) : 0.f;
  }
  __syncthreads();

  uint64_t const b = block0 + (tid >> 3);
  uint32_t const g = tid & 7;
  bool const live = b < in_blocks;
  float x[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) x[i] = xs[tid * kRow + i];

  // Admission of the inputs (q4k.cpp:189-200): the first offending weight of the block decides.
  uint8_t bad = kFitOk;
#pragma unroll
  for (int i = 31; i >= 0; --i) {
    float const v = x[i];
    if (!finite(v)) bad = kFitNonfinite;
    else if (fabsf(v) > 1.0e10f) bad = kFitRange;
  }
  flaw[tid] = bad;
  __syncthreads();
  uint8_t block_flaw = kFitOk;
  for (int j = 7; j >= 0; --j)
    if (flaw[(tid & ~7u) + j]) block_flaw = flaw[(tid & ~7u) + j];
  __syncthreads();

  GroupFit fit{0.f, 0.f, 0.f, 0.f};
  bad = kFitOk;
  if (live && !block_flaw) {
    float lo = 0.f, hi = x[0], sum_x2 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float const v = x[i];
      if (v < lo) lo = v;
      if (v > hi) hi = v;
      sum_x2 = add(sum_x2, mul(v, v));
    }
    if (hi != lo && !finite(quo(16.f, sub(hi, lo)))) bad = kFitReciprocal;
    else fit = fit_group(x, __fsqrt_rn(quo(sum_x2, 32.f)));
  }
  scales[tid] = fit.scale;
  minima[tid] = fit.the_min;
  flaw[tid] = bad;
  __syncthreads();

  // Six-bit compression against the block maxima (q4k.cpp:231-258); every thread of the block's
  // eight derives the same numbers.
  uint32_t const base = tid & ~7u;
  float max_scale = 0.f, max_min = 0.f;
  for (int j = 0; j < 8; ++j) {
    if (flaw[base + j]) block_flaw = block_flaw ? block_flaw : uint8_t(kFitReciprocal);
    if (scales[base + j] > max_scale) max_scale = scales[base + j];
    if (minima[base + j] > max_min) max_min = minima[base + j];
  }
  float const inv_scale = max_scale > 0.f ? quo(63.f, max_scale) : 0.f;
  float const inv_min = max_min > 0.f ? quo(63.f, max_min) : 0.f;
  if (!block_flaw && (!finite(inv_scale) || !finite(inv_min))) block_flaw = kFitCompress;
  __half const d16 = __float2half_rn(quo(max_scale, 63.f)), dmin16 = __float2half_rn(quo(max_min, 63.f));
  uint32_t const dbits = __half_as_ushort(d16), mbits = __half_as_ushort(dmin16);
  if (!block_flaw && ((dbits & 0x7c00u) == 0x7c00u || (mbits & 0x7c00u) == 0x7c00u)) block_flaw = kFitHalf;

  auto six = [](float inv, float v) { return min(63u, uint32_t(nearest(mul(inv, v))) & 0xffu); };
  uint32_t const sc6 = six(inv_scale, scales[tid]), mn6 = six(inv_min, minima[tid]);

  // Final levels against the compressed scales (q4k.cpp:263-275); a group whose step rounds to
  // zero keeps the levels of the search.
  uint32_t packed[4] = {0, 0, 0, 0};  // 32 levels, low nibble first
  if (live && !block_flaw) {
    float const step = mul(__half2float(d16), float(sc6));
    float const offset = mul(__half2float(dmin16), float(mn6));
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float const v = x[i];
      int const l = step != 0.f ? level(quo(add(v, offset), step)) : level(mul(fit.grid, sub(v, fit.origin)));
      packed[i >> 3] |= uint32_t(l) << (4 * (i & 7));
    }
  }

  if (b >= out_blocks) return;
  uint32_t const row = uint32_t(b / tiles_k), kb = uint32_t(b % tiles_k);
  uint64_t const slot = Split ? ((uint64_t(row >> 3) * tiles_k + kb) * 8 + (row & 7)) : b;
  if (Split) {
    reinterpret_cast<uint4*>(codes)[slot * 8 + g] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  } else {
    uint32_t bytes[8];
    for (int i = 0; i < 8; ++i) {
      uint32_t const n4 = (packed[i >> 1] >> (16 * (i & 1))) & 0xffffu;
      bytes[i] = (n4 & 15u) | ((n4 & 0xf0u) << 4) | ((n4 & 0xf00u) << 8) | ((n4 & 0xf000u) << 12);
    }
    uint4* dst = reinterpret_cast<uint4*>(codes + b * 256 + g * 32);
    dst[0] = make_uint4(bytes[0], bytes[1], bytes[2], bytes[3]);
    dst[1] = make_uint4(bytes[4], bytes[5], bytes[6], bytes[7]);
  }
  if (g == 0) {
    uint32_t words[4] = {0, 0, 0, 0};
    if (live && !block_flaw) {
      uint8_t p[12];
      for (int j = 0; j < 12; ++j) p[j] = 0;
      for (int j = 0; j < 8; ++j) {
        uint32_t const s = six(inv_scale, scales[base + j]), m = six(inv_min, minima[base + j]);
        if (j < 4) {
          p[j] |= uint8_t(s);
          p[j + 4] |= uint8_t(m);
        } else {
          p[j + 4] = uint8_t((s & 15u) | ((m & 15u) << 4));
          p[j - 4] |= uint8_t((s >> 4) << 6);
          p[j] |= uint8_t((m >> 4) << 6);
        }
      }
      words[0] = dbits | (mbits << 16);
      for (int j = 0; j < 12; ++j) words[1 + (j >> 2)] |= uint32_t(p[j]) << (8 * (j & 3));
    }
    reinterpret_cast<uint4*>(meta)[slot] = make_uint4(words[0], words[1], words[2], words[3]);
    if (live) {
      if (status) status[b] = block_flaw;
      if (block_flaw) *failure = 1;
    }
  }
}

template <typename In>
cudaError_t launch_fit(const In* weights, uint32_t rows, uint32_t tiles_k, bool split, uint8_t* codes, uint8_t* meta,
                       uint8_t* status, int* failure, cudaStream_t stream) {
  uint32_t const out_rows = split ? (rows + 7) / 8 * 8 : rows;
  uint64_t const blocks = (uint64_t(out_rows) * tiles_k + kFitBlocks - 1) / kFitBlocks;
  if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
  if (split)
    fit_q4k_kernel<In, true><<<unsigned(blocks), kFitThreads, 0, stream>>>(weights, rows, out_rows, tiles_k, codes, meta, status, failure);
  else
    fit_q4k_kernel<In, false><<<unsigned(blocks), kFitThreads, 0, stream>>>(weights, rows, out_rows, tiles_k, codes, meta, status, failure);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fit_q4k(const void* weights, bool bf16, uint32_t rows, uint32_t tiles_k, bool split, uint8_t* codes,
                           uint8_t* meta, uint8_t* status, int* failure, cudaStream_t stream) {
  return bf16 ? launch_fit(static_cast<const uint16_t*>(weights), rows, tiles_k, split, codes, meta, status, failure, stream)
              : launch_fit(static_cast<const float*>(weights), rows, tiles_k, split, codes, meta, status, failure, stream);
}

}  // namespace q4k
