// Q4_K x Q8 matmul on warp-level int8 tensor-core MMA, any token count.
//
// Same equation and the same "one exact int32 dot per K32 group, never carried into the
// next group" rule as the reference's mmq / mmq_j128 (cuda/q4k_q8.cu:103-267); the tiling
// is this library's own:
//   * a warp owns one row group (8 weight rows = the n side of m16n8k32) and streams its
//     1 KiB code tiles + 128 B metadata with 16-byte cp.async into a private 4-stage ring;
//     the 16-byte column of a tile row is XOR-swizzled with the row so ldmatrix reads it
//     without bank conflicts and hands lane (r = lane/4, c = lane%4) raw word c of row r;
//   * a raw word holds columns 8c+{0,2,4,6} in its low nibbles and 8c+{1,3,5,7} in its high
//     nibbles; (w & 0x0f0f0f0f) and ((w >> 4) & 0x0f0f0f0f) are the two B registers, and the
//     activations are staged in shared memory as (even bytes, odd bytes) pairs to match;
//   * tokens are the m16 side: one MMA = 16 tokens x 8 rows x K32, accumulator zeroed;
//   * grid = (row tiles of 64, token tiles, K slices).  With more than one K slice every
//     block writes its fp32 partial tile to scratch and the last block to arrive (ticket
//     counter) adds the slices in slice order, so the result does not depend on timing.
#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kStages = 4;
constexpr int kStageBytes = 1024 + 128;
constexpr int kTabBytes = 8 * 8 * 8;  // [group][row] (D, Mn)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  c[0] = c[1] = c[2] = c[3] = 0;
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Copy the (row group, kb) tile into a ring stage.  Wide: 16-byte cp.async (pointers are
// 16-byte aligned).  Otherwise 4-byte / 2-byte loads and plain shared stores.
template <bool Wide>
__device__ __forceinline__ void fill_stage(uint8_t* stage, const uint8_t* codes, const uint8_t* meta,
                                           uint32_t lane) {
  if constexpr (Wide) {
    uint32_t const base = smem_u32(stage);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t const q = lane + 32 * i, r = q >> 3, g = q & 7;
      cp_async16(base + r * 128 + ((g ^ r) << 4), codes + q * 16);
    }
    if (lane < 8) cp_async16(base + 1024 + lane * 16, meta + lane * 16);
  } else {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(codes);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t const wi = lane + 32 * i, q = wi >> 2, r = q >> 3, g = q & 7;
      *reinterpret_cast<uint32_t*>(stage + r * 128 + ((g ^ r) << 4) + (wi & 3) * 4) = __ldg(src + wi);
    }
    const uint16_t* ms = reinterpret_cast<const uint16_t*>(meta);
#pragma unroll
    for (int i = 0; i < 2; ++i)
      *reinterpret_cast<uint16_t*>(stage + 1024 + (lane + 32 * i) * 2) = __ldg(ms + lane + 32 * i);
  }
}

template <int TT, bool Dump, bool Wide>
__global__ void __launch_bounds__(kThreads) mmq_mma_kernel(WeightView w, Q8View x, float* __restrict__ out,
                                                           const float* __restrict__ residual,
                                                           int32_t* __restrict__ partials, uint32_t split_k,
                                                           uint32_t kbs_step, float* scratch,
                                                           uint32_t* tickets) {
  constexpr int kTokens = 16 * TT;
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t const act_stride = kbs_step * 256 + 32;  // bytes per token, 32 mod 128
  uint32_t const af_stride = kbs_step * 64 + 8;     // bytes per token of (a, float(sum)) pairs
  uint8_t* ring_all = smem;
  uint8_t* tab_all = ring_all + kWarps * kStages * kStageBytes;
  uint8_t* act = tab_all + kWarps * kTabBytes;
  uint8_t* af = act + kTokens * act_stride;
  __shared__ int s_last;

  uint32_t const lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t const tq = lane >> 2, c = lane & 3;
  uint32_t const tiles_k = w.tiles_k, pk = x.padded_k, G = pk / 32;
  uint32_t const rgs = w.padded_n / 8;
  uint32_t const rg = blockIdx.x * kWarps + warp;
  bool const active = rg < rgs;
  uint32_t const tok0 = blockIdx.y * kTokens;
  uint32_t const slice = blockIdx.z;
  uint32_t const kb0 = uint32_t((uint64_t(slice) * tiles_k) / split_k);
  uint32_t const kb1 = uint32_t((uint64_t(slice + 1) * tiles_k) / split_k);
  bool const upper = tok0 + 8 < x.m;  // tokens tq+8 of the first MMA tile exist

  uint8_t* ring = ring_all + warp * kStages * kStageBytes;
  float2* tab = reinterpret_cast<float2*>(tab_all + warp * kTabBytes);
  const uint8_t* cbase = w.codes + uint64_t(active ? rg : 0) * tiles_k * 1024;
  const uint8_t* mbase = w.meta + uint64_t(active ? rg : 0) * tiles_k * 128;

  float acc[TT][4];
#pragma unroll
  for (int i = 0; i < TT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  // Weight pipeline prologue.
  uint32_t next_load = kb0;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (active && next_load < kb1)
      fill_stage<Wide>(ring + (next_load - kb0) % kStages * kStageBytes, cbase + uint64_t(next_load) * 1024,
                       mbase + uint64_t(next_load) * 128, lane);
    ++next_load;
    cp_async_commit();
  }

  for (uint32_t step0 = kb0; step0 < kb1; step0 += kbs_step) {
    uint32_t const kbs = min(kbs_step, kb1 - step0);
    __syncthreads();  // previous step's readers are done with act / af
    // Stage activations of this step: (even, odd) byte pairs per 8 columns.
    {
      uint32_t const pairs = kbs * 32;
      for (uint32_t i = threadIdx.x; i < kTokens * pairs; i += kThreads) {
        uint32_t const t = i / pairs, p = i % pairs, token = tok0 + t;
        uint32_t z0 = 0, z1 = 0;
        if (token < x.m) {
          const uint32_t* src = reinterpret_cast<const uint32_t*>(x.codes + uint64_t(token) * pk +
                                                                   uint64_t(step0) * 256 + p * 8);
          z0 = __ldg(src);
          z1 = __ldg(src + 1);
        }
        *reinterpret_cast<uint2*>(act + t * act_stride + p * 8) = make_uint2(even_bytes(z0, z1), odd_bytes(z0, z1));
      }
      uint32_t const groups = kbs * 8;
      for (uint32_t i = threadIdx.x; i < kTokens * groups; i += kThreads) {
        uint32_t const t = i / groups, g = i % groups, token = tok0 + t;
        float2 v = make_float2(0.f, 0.f);
        if (token < x.m) {
          uint64_t const gi = uint64_t(token) * G + step0 * 8 + g;
          v = make_float2(__ldg(x.scales + gi), float(__ldg(x.sums + gi)));
        }
        *reinterpret_cast<float2*>(af + t * af_stride + g * 8) = v;
      }
    }
    __syncthreads();

    if (active) {
      for (uint32_t kbl = 0; kbl < kbs; ++kbl) {
        uint32_t const kb = step0 + kbl;
        cp_async_wait<kStages - 2>();
        __syncwarp();
        uint8_t* stage = ring + (kb - kb0) % kStages * kStageBytes;

        // Metadata: lane (r = tq, c) decodes groups c and c+4 of row r into the table.
        {
          uint4 const cm = *reinterpret_cast<const uint4*>(stage + 1024 + tq * 16);
          float const d = fp16_bits_to_f32(cm.x & 0xffffu), dmin = fp16_bits_to_f32(cm.x >> 16);
          ScaleMinWords const sm = decode_scale_min(cm.y, cm.z, cm.w);
          tab[c * 8 + tq] = make_float2(d * float(byte_of(sm.sc_lo, c)), dmin * float(byte_of(sm.mn_lo, c)));
          tab[(c + 4) * 8 + tq] = make_float2(d * float(byte_of(sm.sc_hi, c)), dmin * float(byte_of(sm.mn_hi, c)));
        }
        uint32_t q[8];
        {
          uint32_t const row = lane & 7, mat = lane >> 3;
          uint32_t const base = smem_u32(stage) + row * 128;
          uint32_t r4[4];
          ldmatrix_x4(r4, base + ((mat ^ row) << 4));
          q[0] = r4[0]; q[1] = r4[1]; q[2] = r4[2]; q[3] = r4[3];
          ldmatrix_x4(r4, base + (((mat + 4) ^ row) << 4));
          q[4] = r4[0]; q[5] = r4[1]; q[6] = r4[2]; q[7] = r4[3];
        }
        __syncwarp();  // table visible to the whole warp

#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint32_t const b0 = q[g] & 0x0f0f0f0fu, b1 = (q[g] >> 4) & 0x0f0f0f0fu;
          float4 const dm = *reinterpret_cast<const float4*>(&tab[g * 8 + 2 * c]);  // D,Mn of rows 2c, 2c+1
#pragma unroll
          for (int tt = 0; tt < TT; ++tt) {
            uint32_t const tl = tt * 16 + tq;
            uint2 const lo = *reinterpret_cast<const uint2*>(act + tl * act_stride + kbl * 256 + g * 32 + c * 8);
            uint2 const hi = *reinterpret_cast<const uint2*>(act + (tl + 8) * act_stride + kbl * 256 + g * 32 + c * 8);
            int d4[4];
            mma_s8(d4, lo.x, hi.x, lo.y, hi.y, b0, b1);
            float2 const f0 = *reinterpret_cast<const float2*>(af + tl * af_stride + (kbl * 8 + g) * 8);
            acc[tt][0] += f0.x * (dm.x * float(d4[0]) - dm.y * f0.y);
            acc[tt][1] += f0.x * (dm.z * float(d4[1]) - dm.w * f0.y);
            if (tt > 0 || upper) {
              float2 const f1 = *reinterpret_cast<const float2*>(af + (tl + 8) * af_stride + (kbl * 8 + g) * 8);
              acc[tt][2] += f1.x * (dm.x * float(d4[2]) - dm.y * f1.y);
              acc[tt][3] += f1.x * (dm.z * float(d4[3]) - dm.w * f1.y);
            }
            if (Dump) {
#pragma unroll
              for (int l = 0; l < 4; ++l) {
                uint32_t const token = tok0 + tl + (l >> 1) * 8, row = rg * 8 + 2 * c + (l & 1);
                if (token < x.m && row < w.n)
                  partials[(uint64_t(token) * w.n + row) * G + kb * 8 + g] = d4[l];
              }
            }
          }
        }
        __syncwarp();  // all lanes are done with this stage and the table
        if (next_load < kb1)
          fill_stage<Wide>(ring + (next_load - kb0) % kStages * kStageBytes, cbase + uint64_t(next_load) * 1024,
                           mbase + uint64_t(next_load) * 128, lane);
        ++next_load;
        cp_async_commit();
      }
    }
  }
  cp_async_wait<0>();

  // Output.  Lane holds tokens (tq, tq+8) x rows (2c, 2c+1) of every token tile.
  if (split_k == 1) {
    if (active) {
#pragma unroll
      for (int tt = 0; tt < TT; ++tt)
#pragma unroll
        for (int l = 0; l < 4; ++l) {
          uint32_t const token = tok0 + tt * 16 + tq + (l >> 1) * 8, row = rg * 8 + 2 * c + (l & 1);
          if (token < x.m && row < w.n) {
            uint64_t const o = uint64_t(token) * w.n + row;
            out[o] = acc[tt][l] + (residual ? residual[o] : 0.f);
          }
        }
    }
    return;
  }
  uint64_t const plane = uint64_t(x.m) * w.n;
  if (active) {
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        uint32_t const token = tok0 + tt * 16 + tq + (l >> 1) * 8, row = rg * 8 + 2 * c + (l & 1);
        if (token < x.m && row < w.n) __stcg(scratch + slice * plane + uint64_t(token) * w.n + row, acc[tt][l]);
      }
  }
  __threadfence();
  __syncthreads();
  uint32_t* ticket = tickets + blockIdx.y * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) {
    uint32_t const old = atomicAdd(ticket, 1u);
    s_last = (old == split_k - 1) ? 1 : 0;
    if (s_last) *ticket = 0;  // leave the counter clean for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (active) {
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        uint32_t const token = tok0 + tt * 16 + tq + (l >> 1) * 8, row = rg * 8 + 2 * c + (l & 1);
        if (token < x.m && row < w.n) {
          uint64_t const o = uint64_t(token) * w.n + row;
          float v = 0.f;
          for (uint32_t s = 0; s < split_k; ++s) v += __ldcg(scratch + s * plane + o);
          out[o] = v + (residual ? residual[o] : 0.f);
        }
      }
  }
}

size_t smem_bytes(uint32_t token_tile, uint32_t kbs_step) {
  return size_t(kWarps) * kStages * kStageBytes + size_t(kWarps) * kTabBytes +
         size_t(token_tile) * (kbs_step * 256 + 32) + size_t(token_tile) * (kbs_step * 64 + 8);
}

template <int TT>
cudaError_t launch_tt(const WeightView& w, const Q8View& x, float* out, const float* residual,
                      int32_t* partials, const MmaPlan& plan, void* partial_tiles_v, uint32_t* tickets,
                      cudaStream_t stream) {
  bool const wide = (reinterpret_cast<uintptr_t>(w.codes) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(w.meta) % 16 == 0);
  void (*kernel)(WeightView, Q8View, float*, const float*, int32_t*, uint32_t, uint32_t, float*, uint32_t*);
  if (partials) kernel = wide ? mmq_mma_kernel<TT, true, true> : mmq_mma_kernel<TT, true, false>;
  else kernel = wide ? mmq_mma_kernel<TT, false, true> : mmq_mma_kernel<TT, false, false>;
  size_t const smem = smem_bytes(16 * TT, plan.kbs_per_step);
  cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (st != cudaSuccess) return st;
  uint32_t const row_tiles = (w.padded_n / 8 + kWarps - 1) / kWarps;
  uint32_t const token_tiles = (x.m + 16 * TT - 1) / (16 * TT);
  dim3 grid(row_tiles, token_tiles, plan.split_k);
  float* partial_tiles = static_cast<float*>(partial_tiles_v);
  kernel<<<grid, kThreads, smem, stream>>>(w, x, out, residual, partials, plan.split_k, plan.kbs_per_step,
                                           partial_tiles, tickets);
  return cudaGetLastError();
}

}  // namespace

MmaPlan plan_mma(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request) {
  MmaPlan p;
  p.token_tile = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
  p.kbs_per_step = p.token_tile == 16 ? 8 : (p.token_tile == 32 ? 4 : 2);
  uint32_t const padded_n = (n + 7) / 8 * 8;
  uint32_t const row_tiles = (padded_n / 8 + kWarps - 1) / kWarps;
  uint32_t const token_tiles = (m + p.token_tile - 1) / p.token_tile;
  uint32_t split = split_k_request;
  if (split == 0) {
    // Enough blocks for ~4 per SM, at least two super-blocks of K per slice.
    uint32_t const blocks = row_tiles * token_tiles;
    split = (148 * 4 + blocks - 1) / blocks;
    uint32_t const max_split = tiles_k / 2 ? tiles_k / 2 : 1;
    if (split > max_split) split = max_split;
    if (split > 32) split = 32;
    if (split < 1) split = 1;
  }
  if (split > tiles_k) split = tiles_k;
  p.split_k = split;
  return p;
}

cudaError_t launch_mmq_mma(const WeightView& w, const Q8View& x, float* out, const float* residual,
                           int32_t* partials, const MmaPlan& plan, void* partial_tiles, uint32_t* tickets,
                           cudaStream_t stream) {
  switch (plan.token_tile) {
    case 16: return launch_tt<1>(w, x, out, residual, partials, plan, partial_tiles, tickets, stream);
    case 32: return launch_tt<2>(w, x, out, residual, partials, plan, partial_tiles, tickets, stream);
    case 64: return launch_tt<4>(w, x, out, residual, partials, plan, partial_tiles, tickets, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace q4k
