// One-time weight preparation: 144-byte llama.cpp-native Q4_K super-blocks -> the
// split-tile device layout every kernel of this library consumes.
//
// A 144-byte block is {fp16 d, fp16 dmin, 12 scale bytes, 128 quant bytes}; element
// 64c+l of the block is the low nibble of qs[32c+l], element 64c+32+l its high nibble
// (third_party/llama.cpp-q4k/reference.hpp:244-248,253-275).  A tile row keeps the 16
// metadata bytes as they are and stores element 2j in the low and 2j+1 in the high nibble
// of code byte j (src/format/pack.cpp:201-222).  Rows n..ceil8(n)-1 are written as zeros.
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

__global__ void __launch_bounds__(128) repack_blocks144_kernel(const uint8_t* __restrict__ blocks, uint32_t n,
                                                               uint32_t tiles_k, uint8_t* __restrict__ codes,
                                                               uint8_t* __restrict__ meta) {
  uint64_t const tr = blockIdx.x;  // tile row index
  uint32_t const r = uint32_t(tr & 7);
  uint64_t const t = tr >> 3;
  uint32_t const kb = uint32_t(t % tiles_k), row = uint32_t(t / tiles_k) * 8 + r;
  uint32_t const j = threadIdx.x;
  uint8_t v = 0, mv = 0;
  if (row < n) {
    const uint8_t* blk = blocks + (uint64_t(row) * tiles_k + kb) * 144;
    uint32_t const e0 = 2 * j, cc = e0 >> 6, l = e0 & 31, hi = (e0 >> 5) & 1;
    uint32_t const s0 = blk[16 + 32 * cc + l], s1 = blk[16 + 32 * cc + l + 1];
    v = uint8_t(hi ? ((s0 >> 4) | (s1 & 0xf0u)) : ((s0 & 15u) | ((s1 & 15u) << 4)));
    if (j < 16) mv = blk[j];
  }
  codes[tr * 128 + j] = v;
  if (j < 16) meta[tr * 16 + j] = mv;
}

}  // namespace

cudaError_t launch_repack_blocks144(const uint8_t* blocks, uint32_t n, uint32_t k, uint8_t* codes,
                                    uint8_t* meta, cudaStream_t stream) {
  uint32_t const tiles_k = k / 256;
  uint64_t const tile_rows = uint64_t((n + 7) / 8 * 8) * tiles_k;
  repack_blocks144_kernel<<<unsigned(tile_rows), 128, 0, stream>>>(blocks, n, tiles_k, codes, meta);
  return cudaGetLastError();
}

}  // namespace q4k
