// Shared device helpers for the Q4_K x Q8 kernels: tile addressing of the
// split-tile weight layout, 6-bit scale/min decode, fp16/bf16 bit conversions.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace q4k {

// Launch-side view of a weight matrix (the fields kernels need).
struct WeightView {
  const uint8_t* codes;  // [padded_n/8][tiles_k][8][128]
  const uint8_t* meta;   // [padded_n/8][tiles_k][8][16]
  uint32_t n, padded_n, tiles_k;  // tiles_k = padded_k / 256
};

struct Q8View {
  const int8_t* codes;   // [m][padded_k]
  const float* scales;   // [m][padded_k/32]
  const int32_t* sums;   // [m][padded_k/32]
  uint32_t m, padded_k;
};

// Index of the 128-byte code row (and 16-byte metadata row) of (row, kb)
// (reference: tile_row, cuda/q4k_q8.cu:27-29).
__host__ __device__ __forceinline__ uint64_t tile_row(uint32_t row, uint32_t kb, uint32_t tiles_k) {
  return (uint64_t(row >> 3) * tiles_k + kb) * 8 + (row & 7);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t x) { return __uint_as_float(uint32_t(x) << 16); }

__device__ __forceinline__ uint16_t f32_to_bf16_rne(float v) {
  uint32_t b = __float_as_uint(v);
  if ((b & 0x7fffffffu) > 0x7f800000u) return uint16_t((b >> 16) | 0x40u);
  b += 0x7fffu + ((b >> 16) & 1u);
  return uint16_t(b >> 16);
}

__device__ __forceinline__ float fp16_bits_to_f32(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)h));
}

// The 12 packed bytes p[0..11] as words w0=p[0..3], w1=p[4..7], w2=p[8..11] hold
// eight 6-bit scales and eight 6-bit mins (reference decode: cuda/q4k_q8.cu:33-35).
// Byte-parallel form: sc[0..3], mn[0..3], sc[4..7], mn[4..7] as four packed words.
struct ScaleMinWords { uint32_t sc_lo, mn_lo, sc_hi, mn_hi; };
__device__ __forceinline__ ScaleMinWords decode_scale_min(uint32_t w0, uint32_t w1, uint32_t w2) {
  ScaleMinWords r;
  r.sc_lo = w0 & 0x3f3f3f3fu;
  r.mn_lo = w1 & 0x3f3f3f3fu;
  r.sc_hi = (w2 & 0x0f0f0f0fu) | ((w0 >> 2) & 0x30303030u);
  r.mn_hi = ((w2 >> 4) & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u);
  return r;
}
__device__ __forceinline__ uint32_t byte_of(uint32_t w, uint32_t i) { return (w >> (8 * i)) & 0xffu; }

// Even / odd bytes of eight consecutive int8 activations z0 = cols 0..3, z1 = cols 4..7.
// A raw weight word holds cols {0,2,4,6} in its low nibbles and {1,3,5,7} in its
// high nibbles, so (w & 0x0f0f0f0f) pairs with even(), ((w >> 4) & 0x0f0f0f0f) with odd().
__device__ __forceinline__ uint32_t even_bytes(uint32_t z0, uint32_t z1) { return __byte_perm(z0, z1, 0x6420); }
__device__ __forceinline__ uint32_t odd_bytes(uint32_t z0, uint32_t z1) { return __byte_perm(z0, z1, 0x7531); }

// Programmatic dependent launch.  A kernel launched with the stream-serialization attribute may
// start while the kernel before it in the stream is still running; it must call pdl_wait()
// before it reads anything that kernel may have written and before it writes global memory.
// pdl_launch_dependents() tells the scheduler that the next kernel in the stream may start as
// soon as every block of this grid has called it (or exited).  Every kernel of this library calls
// it AFTER its pdl_wait(): a successor then never runs beside anything older than its direct
// predecessor, which is what lets a caller flag a projection's input as settled.  Both are no-ops
// for kernels launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Row-sharded decode: tell every rank how many more projections of this rank are complete.  Called by
// one thread at the start of the kernel that FOLLOWS them in the stream, after pdl_wait(): those grids
// have completed, so their stores into the peers' buffers are visible before the counters move.
__device__ __forceinline__ void announce_deliveries(uint32_t* unsignalled, uint32_t* const* peer_flag, uint32_t ranks,
                                                    uint32_t rank) {
  uint32_t const u = *reinterpret_cast<volatile uint32_t*>(unsignalled);
  if (u == 0) return;
  *reinterpret_cast<volatile uint32_t*>(unsignalled) = 0;
#pragma unroll
  for (int g = 0; g < 8; ++g)
    if (g < int(ranks)) atomicAdd_system(peer_flag[g] + rank, u);
}

}  // namespace q4k
