// One-time weight preparation: 144-byte llama.cpp-native Q4_K super-blocks -> the
// split-tile device layout every kernel of this library consumes.
//
// A 144-byte block is {fp16 d, fp16 dmin, 12 scale bytes, 128 quant bytes}; element
// 64c+l of the block is the low nibble of qs[32c+l], element 64c+32+l its high nibble
// (third_party/llama.cpp-q4k/reference.hpp:244-248,253-275).  A tile row keeps the 16
// metadata bytes as they are and stores element 2j in the low and 2j+1 in the high nibble
// of code byte j (src/format/pack.cpp:201-222).  Rows n..ceil8(n)-1 are written as zeros.
#include <cuda_bf16.h>

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

// Admissibility of a resident split-tile weight, the Q4_K rows of format::validate_cuda_v0
// (src/format/unpack.cpp:156-226): a padded row (row >= n) holds zero codes and zero metadata; a live
// row's fp16 d and dmin are non-negative and finite.  The reference walks tile rows in index order,
// codes before metadata, and reports the first offence; here every tile row is checked by one thread
// and the smallest key (tile_row, stage, byte) wins an atomic minimum, which is the same offence.
// stage: 0 padded code byte, 1 padded metadata byte, 2 super-block scale.
__global__ void __launch_bounds__(256) validate_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ meta,
                                                       uint32_t n, uint32_t tiles_k, uint64_t tile_rows,
                                                       unsigned long long* __restrict__ key) {
  uint64_t const tr = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tr >= tile_rows) return;
  uint32_t const row = uint32_t((tr >> 3) / tiles_k) * 8 + uint32_t(tr & 7);
  uint4 const m = reinterpret_cast<const uint4*>(meta)[tr];
  unsigned long long found = ~0ull;
  if (row >= n) {
    uint32_t const mw[4] = {m.x, m.y, m.z, m.w};
    for (int w = 3; w >= 0; --w)
      if (mw[w]) found = (tr << 10) | (1u << 8) | uint32_t(4 * w + (__ffs(mw[w]) - 1) / 8);
    const uint4* c = reinterpret_cast<const uint4*>(codes) + tr * 8;
    for (int q = 7; q >= 0; --q) {
      uint4 const v = c[q];
      uint32_t const cw[4] = {v.x, v.y, v.z, v.w};
      for (int w = 3; w >= 0; --w)
        if (cw[w]) found = (tr << 10) | uint32_t(16 * q + 4 * w + (__ffs(cw[w]) - 1) / 8);
    }
  } else {
    uint32_t const d = m.x & 0xffffu, dmin = m.x >> 16;
    if ((dmin & 0x8000u) || (dmin & 0x7c00u) == 0x7c00u) found = (tr << 10) | (2u << 8) | 2u;
    if ((d & 0x8000u) || (d & 0x7c00u) == 0x7c00u) found = (tr << 10) | (2u << 8) | 0u;
  }
  if (found != ~0ull) atomicMin(key, found);
}

// Split tiles -> bf16 weights [n][k] row-major, the values of compiler::dequantize_to_bf16
// (src/compiler/quantization/reference.cpp:141-166): w = bf16_rne((d * sc) * q - dmin * mn) with three
// separately rounded fp32 operations.  One thread turns one code word (8 weights) into one 16-byte
// store.  A block of eight warps takes one group of eight rows and kDeqTiles consecutive K tiles
// (a contiguous run of the tiled input); warp r owns row r, so that it writes kDeqTiles * 512
// contiguous bytes of that row, with all its loads issued before the first store.
constexpr int kDeqTiles = 4;
__global__ void __launch_bounds__(256) dequantize_bf16_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ meta,
                                                              uint32_t n, uint32_t tiles_k, uint32_t chunks_k,
                                                              uint16_t* __restrict__ out) {
  uint32_t const group = blockIdx.x / chunks_k, kb0 = (blockIdx.x % chunks_k) * kDeqTiles;
  uint32_t const r = threadIdx.x >> 5, c = threadIdx.x & 31, g = c >> 2;
  uint32_t const row = group * 8 + r;
  if (row >= n) return;
  uint4 m[kDeqTiles];
  uint32_t w[kDeqTiles];
#pragma unroll
  for (int t = 0; t < kDeqTiles; ++t) {
    if (kb0 + t < tiles_k) {
      uint64_t const tr = (uint64_t(group) * tiles_k + kb0 + t) * 8 + r;
      m[t] = __ldg(reinterpret_cast<const uint4*>(meta) + tr);
      w[t] = __ldg(reinterpret_cast<const uint32_t*>(codes) + tr * 32 + c);
    }
  }
#pragma unroll
  for (int t = 0; t < kDeqTiles; ++t) {
    if (kb0 + t >= tiles_k) break;
    ScaleMinWords const sm = decode_scale_min(m[t].y, m[t].z, m[t].w);
    uint32_t const sc = byte_of(g < 4 ? sm.sc_lo : sm.sc_hi, g & 3), mn = byte_of(g < 4 ? sm.mn_lo : sm.mn_hi, g & 3);
    float const step = __fmul_rn(fp16_bits_to_f32(m[t].x & 0xffffu), float(sc));
    float const offset = __fmul_rn(fp16_bits_to_f32(m[t].x >> 16), float(mn));
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // level -> float through the 2^23 bias (exact, and on the full-rate pipes); the pair is rounded
      // to bf16 by one conversion instruction (round to nearest even; values are finite)
      float const lo = __fsub_rn(__uint_as_float(0x4b000000u | ((w[t] >> (8 * i)) & 15u)), 8388608.f);
      float const hi = __fsub_rn(__uint_as_float(0x4b000000u | ((w[t] >> (8 * i + 4)) & 15u)), 8388608.f);
      __nv_bfloat162 const pair = __floats2bfloat162_rn(__fsub_rn(__fmul_rn(step, lo), offset), __fsub_rn(__fmul_rn(step, hi), offset));
      packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    uint64_t const at = (uint64_t(row) * tiles_k + kb0 + t) * 256 + 8 * c;
    __stcs(reinterpret_cast<uint4*>(out + at), make_uint4(packed[0], packed[1], packed[2], packed[3]));
  }
}

// Split tiles -> the logical form of format::unpack_cuda_v0 (src/format/unpack.cpp:262-380): int8 levels
// [n][k] and the 16 metadata bytes per super-block [n][k/256][16].  Same block shape as the dequantiser.
__global__ void __launch_bounds__(256) unpack_logical_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ meta,
                                                             uint32_t n, uint32_t tiles_k, uint32_t chunks_k,
                                                             int8_t* __restrict__ out_codes, uint8_t* __restrict__ out_meta) {
  uint32_t const group = blockIdx.x / chunks_k, kb0 = (blockIdx.x % chunks_k) * kDeqTiles;
  uint32_t const r = threadIdx.x >> 5, c = threadIdx.x & 31;
  uint32_t const row = group * 8 + r;
  if (row >= n) return;
  auto spread = [](uint32_t n4) { return (n4 & 15u) | ((n4 & 0xf0u) << 4) | ((n4 & 0xf00u) << 8) | ((n4 & 0xf000u) << 12); };
#pragma unroll
  for (int t = 0; t < kDeqTiles; ++t) {
    if (kb0 + t >= tiles_k) break;
    uint64_t const tr = (uint64_t(group) * tiles_k + kb0 + t) * 8 + r;
    uint32_t const w = __ldg(reinterpret_cast<const uint32_t*>(codes) + tr * 32 + c);
    uint64_t const block = uint64_t(row) * tiles_k + kb0 + t;
    *reinterpret_cast<uint2*>(out_codes + block * 256 + 8 * c) = make_uint2(spread(w & 0xffffu), spread(w >> 16));
    if (c < 4) reinterpret_cast<uint32_t*>(out_meta + block * 16)[c] = __ldg(reinterpret_cast<const uint32_t*>(meta + tr * 16) + c);
  }
}

// verdict[1] holds the winning key on entry; rewrites verdict as {kind, byte offset in its span}.
__global__ void validate_verdict_kernel(unsigned long long* verdict) {
  unsigned long long const key = verdict[1];
  if (key == ~0ull) {
    verdict[0] = 0;
    verdict[1] = 0;
    return;
  }
  unsigned long long const tr = key >> 10, stage = (key >> 8) & 3u, byte = key & 0xffu;
  verdict[0] = stage + 1;
  verdict[1] = stage == 0 ? tr * 128 + byte : tr * 16 + byte;
}

}  // namespace

cudaError_t launch_validate_weight(const uint8_t* codes, const uint8_t* meta, uint32_t n, uint32_t k, uint64_t* verdict,
                                   cudaStream_t stream) {
  uint32_t const tiles_k = k / 256;
  uint64_t const tile_rows = uint64_t((n + 7) / 8 * 8) * tiles_k;
  auto* v = reinterpret_cast<unsigned long long*>(verdict);
  cudaError_t st = cudaMemsetAsync(v, 0xff, 16, stream);
  if (st != cudaSuccess) return st;
  validate_kernel<<<unsigned((tile_rows + 255) / 256), 256, 0, stream>>>(codes, meta, n, tiles_k, tile_rows, v + 1);
  validate_verdict_kernel<<<1, 1, 0, stream>>>(v);
  return cudaGetLastError();
}

cudaError_t launch_dequantize_bf16(const uint8_t* codes, const uint8_t* meta, uint32_t n, uint32_t k, uint16_t* out,
                                   cudaStream_t stream) {
  uint32_t const tiles_k = k / 256, chunks_k = (tiles_k + kDeqTiles - 1) / kDeqTiles;
  uint64_t const blocks = uint64_t((n + 7) / 8) * chunks_k;
  if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
  dequantize_bf16_kernel<<<unsigned(blocks), 256, 0, stream>>>(codes, meta, n, tiles_k, chunks_k, out);
  return cudaGetLastError();
}

cudaError_t launch_unpack_logical(const uint8_t* codes, const uint8_t* meta, uint32_t n, uint32_t k, int8_t* out_codes,
                                  uint8_t* out_meta, cudaStream_t stream) {
  uint32_t const tiles_k = k / 256, chunks_k = (tiles_k + kDeqTiles - 1) / kDeqTiles;
  uint64_t const blocks = uint64_t((n + 7) / 8) * chunks_k;
  if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
  unpack_logical_kernel<<<unsigned(blocks), 256, 0, stream>>>(codes, meta, n, tiles_k, chunks_k, out_codes, out_meta);
  return cudaGetLastError();
}

cudaError_t launch_repack_blocks144(const uint8_t* blocks, uint32_t n, uint32_t k, uint8_t* codes,
                                    uint8_t* meta, cudaStream_t stream) {
  uint32_t const tiles_k = k / 256;
  uint64_t const tile_rows = uint64_t((n + 7) / 8 * 8) * tiles_k;
  repack_blocks144_kernel<<<unsigned(tile_rows), 128, 0, stream>>>(blocks, n, tiles_k, codes, meta);
  return cudaGetLastError();
}

}  // namespace q4k
