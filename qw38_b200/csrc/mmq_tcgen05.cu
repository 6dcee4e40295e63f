// Q4_K x Q8 matmul on the 5th-generation tensor cores: tcgen05.mma kind::i8, operands staged
// by TMA, one TMEM accumulator per K32 group, scaling epilogue on CUDA cores.
//
// The per-K32 rule of the reference (cuda/q4k_q8.cu:70-72: one exact int32 dot per 32 columns,
// never carried into the next group) fixes the structure: every MMA has K = 32, starts from a
// cleared accumulator, and its 128 x NTOK int32 results are drained from TMEM and folded into
// fp32 accumulators in registers as  acc += a * (D * float(P) - Mn * float(sum)).
//
// Tile: 128 weight rows (the M side, one TMEM lane per row) x NTOK tokens (the N side) per
// block, K walked in 256-column super-blocks.  Warp roles:
//   warp 0      one lane issues TMA: raw 4-bit code tiles + metadata (3-D maps over the split
//               tile layout, no swizzle), int8 activation tiles (2-D map, 128-byte swizzle,
//               rows beyond m zero-filled) and their fp32 scales / int32 sums;
//   warp 1      allocates TMEM; one lane issues the eight K32 MMAs of a super-block, each into
//               the next accumulator buffer, each followed by tcgen05.commit;
//   warps 2-5   expand nibbles to int8 in the K-major 128-byte-swizzled operand layout and build
//               the (a, a', sum, sum') table of the token pairs;
//   warps 6..   epilogue: thread = weight row; decode that row's six-bit scales once per
//               super-block, then per K32 group tcgen05.ld its accumulator columns and scale.
// Every wait on an mbarrier is bounded: after ~2 s a thread raises the block's abort flag and
// the kernel's status word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "launch.h"

namespace q4k {
namespace {

constexpr int kRows = 128;
constexpr int kProducerWarp = 0, kMmaWarp = 1, kFirstExpander = 2, kExpanders = 4, kFirstEpilogue = 6;
constexpr uint32_t kMagicI = 0x4B400000u;   // bit pattern of 1.5 * 2^23
constexpr float kMagicF = 12582912.0f;
constexpr long long kWaitCycles = 4000000000LL;

template <int NTOK> struct Cfg {
  static constexpr int kEpilogueWarps = NTOK >= 64 ? 8 : 4;
  static constexpr int kWarps = kFirstEpilogue + kEpilogueWarps;
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kColsPerWarp = NTOK / (kEpilogueWarps / 4);
  static constexpr int kAccBufs = (512 / NTOK) > 16 ? 16 : (512 / NTOK);
  static constexpr int kStages = NTOK <= 32 ? 3 : 2;
  // stage layout (bytes)
  static constexpr int kRawCodes = 16 * 1024;
  static constexpr int kRawMeta = 16 * 128;
  static constexpr int kAExp = 2 * kRows * 128;
  static constexpr int kB = 2 * (NTOK < 8 ? 8 : NTOK) * 128;
  static constexpr int kBPad = (kB + 1023) / 1024 * 1024;
  static constexpr int kRawScale = NTOK * 32;
  static constexpr int kAf = 8 * NTOK * 8;
  static constexpr int oAExp = 0;
  static constexpr int oB = oAExp + kAExp;
  static constexpr int oRawCodes = oB + kBPad;
  static constexpr int oRawMeta = oRawCodes + kRawCodes;
  static constexpr int oRawScales = oRawMeta + kRawMeta;
  static constexpr int oRawSums = oRawScales + kRawScale;
  static constexpr int oAf = oRawSums + kRawScale;
  static constexpr int kStageBytes = (oAf + kAf + 1023) / 1024 * 1024;
  static constexpr int kTxBytes = kRawCodes + kRawMeta + 2 * NTOK * 128 + 2 * kRawScale;
  static constexpr int kBarriers = 3 * kStages + 2 * kAccBufs;
  static constexpr int kSmem = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers etc.*/;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  False = gave up (abort raised).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  long long const t0 = clock64();
  for (uint32_t spin = 0;; ++spin) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((spin & 15u) == 15u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        atomicExch(status, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

// K-major, 128-byte swizzle: 8-row atoms of 1024 bytes; version 1; layout type 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return uint64_t((saddr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}
// kind::i8, s8 x s8 -> s32, both operands K-major, M = 128, N = ntok.
__host__ __device__ constexpr uint32_t umma_idesc(int ntok) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(ntok >> 3) << 17) | (uint32_t(kRows >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0), "r"(0) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

struct TcParams {
  const uint8_t* meta;   // kept for the bit-exact dump only
  const float* residual;
  float* out;
  int32_t* partials;
  float* partial_tiles;  // split-K scratch [slice][m][n]
  uint32_t* tickets;
  int* status;
  uint32_t n, m, tiles_k, split_k, G;
};

template <int NTOK, bool Dump>
__global__ void __launch_bounds__(Cfg<NTOK>::kThreads, 1)
mmq_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_codes, const __grid_constant__ CUtensorMap tm_meta,
                   const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_scales,
                   const __grid_constant__ CUtensorMap tm_sums, TcParams p) {
  using C = Cfg<NTOK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* const ctrl = smem + C::kStages * C::kStageBytes;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(ctrl);         // full[S] expanded[S] free[S] acc_full[B] acc_empty[B]
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(ctrl + C::kBarriers * 8);
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(ctrl + C::kBarriers * 8 + 8);
  __shared__ int s_last;

  uint32_t const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t const row_tile = blockIdx.x, tok_tile = blockIdx.y, slice = blockIdx.z;
  uint32_t const row0 = row_tile * kRows, tok0 = tok_tile * NTOK;
  uint32_t const kb0 = uint32_t((uint64_t(slice) * p.tiles_k) / p.split_k);
  uint32_t const kb1 = uint32_t((uint64_t(slice + 1) * p.tiles_k) / p.split_k);
  uint32_t const iters = kb1 - kb0;

  auto bar_full = [&](uint32_t s) { return smem_u32(bars + s); };
  auto bar_expanded = [&](uint32_t s) { return smem_u32(bars + C::kStages + s); };
  auto bar_free = [&](uint32_t s) { return smem_u32(bars + 2 * C::kStages + s); };
  auto bar_acc_full = [&](uint32_t b) { return smem_u32(bars + 3 * C::kStages + b); };
  auto bar_acc_empty = [&](uint32_t b) { return smem_u32(bars + 3 * C::kStages + C::kAccBufs + b); };

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_expanded(s), kExpanders * 32);
      mbar_init(bar_free(s), 1 + C::kEpilogueWarps);
    }
    for (uint32_t b = 0; b < C::kAccBufs; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), C::kEpilogueWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmem_base = *tmem_slot;

  // fp32 accumulators of the epilogue threads: columns [col0, col0 + kColsPerWarp) of this row.
  float2 acc[C::kColsPerWarp / 2];
#pragma unroll
  for (int i = 0; i < C::kColsPerWarp / 2; ++i) acc[i] = make_float2(0.f, 0.f);
  uint32_t const ep = warp - kFirstEpilogue;                 // valid for epilogue warps
  uint32_t const lane_quarter = warp & 3;                    // TMEM lanes this warp may touch
  uint32_t const col0 = (ep >> 2) * C::kColsPerWarp;
  uint32_t const my_row = lane_quarter * 32 + lane;          // row inside the tile

  if (warp == kProducerWarp) {
    if (lane == 0) {
      uint32_t issued = 0;
      for (uint32_t it = 0; it < iters; ++it) {
        uint32_t const s = it % C::kStages, use = it / C::kStages;
        if (!mbar_wait(bar_free(s), (use & 1) ^ 1, abort_flag, p.status, 1)) break;
        uint8_t* const st = smem + s * C::kStageBytes;
        uint32_t const bar = bar_full(s);
        int const kb = int(kb0 + it);
        mbar_expect_tx(bar, C::kTxBytes);
        tma_3d(smem_u32(st + C::oRawCodes), &tm_codes, 0, kb, int(row0 / 8), bar);
        tma_3d(smem_u32(st + C::oRawMeta), &tm_meta, 0, kb, int(row0 / 8), bar);
        tma_2d(smem_u32(st + C::oB), &tm_act, kb * 256, int(tok0), bar);
        tma_2d(smem_u32(st + C::oB + NTOK * 128), &tm_act, kb * 256 + 128, int(tok0), bar);
        tma_2d(smem_u32(st + C::oRawScales), &tm_scales, kb * 8, int(tok0), bar);
        tma_2d(smem_u32(st + C::oRawSums), &tm_sums, kb * 8, int(tok0), bar);
        issued = it + 1;
      }
      if (*abort_flag) {
        // Leaving early: let the copies this thread started land before the block's shared memory goes away.
        uint32_t const first = issued > C::kStages ? issued - C::kStages : 0;
        for (uint32_t it = first; it < issued; ++it) {
          long long const t0 = clock64();
          uint32_t ok = 0;
          while (!ok && clock64() - t0 < 200000000LL)
            asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                         : "=r"(ok) : "r"(bar_full(it % C::kStages)), "r"((it / C::kStages) & 1) : "memory");
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(NTOK);
      for (uint32_t it = 0; it < iters; ++it) {
        uint32_t const s = it % C::kStages, use = it / C::kStages;
        if (!mbar_wait(bar_full(s), use & 1, abort_flag, p.status, 2)) break;
        if (!mbar_wait(bar_expanded(s), use & 1, abort_flag, p.status, 3)) break;
        tc_fence_after();
        uint8_t* const st = smem + s * C::kStageBytes;
        uint32_t const a_base = smem_u32(st + C::oAExp), b_base = smem_u32(st + C::oB);
        bool ok = true;
#pragma unroll
        for (uint32_t g = 0; g < 8; ++g) {
          uint32_t const i = it * 8 + g, b = i % C::kAccBufs, round = i / C::kAccBufs;
          if (!mbar_wait(bar_acc_empty(b), (round & 1) ^ 1, abort_flag, p.status, 4)) { ok = false; break; }
          tc_fence_after();
          uint64_t const ad = umma_desc(a_base + (g >> 2) * (kRows * 128) + (g & 3) * 32);
          uint64_t const bd = umma_desc(b_base + (g >> 2) * (NTOK * 128) + (g & 3) * 32);
          umma_i8(tmem_base + b * NTOK, ad, bd, idesc);
          umma_commit(bar_acc_full(b));
        }
        if (!ok) break;
        umma_commit(bar_free(s));
      }
    }
  } else if (warp < kFirstEpilogue) {
    uint32_t const et = threadIdx.x - kFirstExpander * 32;  // 0..127
    for (uint32_t it = 0; it < iters; ++it) {
      uint32_t const s = it % C::kStages, use = it / C::kStages;
      if (!mbar_wait(bar_full(s), use & 1, abort_flag, p.status, 5)) break;
      uint8_t* const st = smem + s * C::kStageBytes;
      // 1024 raw 16-byte chunks: chunk q = (row group q/64, row (q/8)%8, K32 group q%8).
#pragma unroll 2
      for (uint32_t q = et; q < 1024; q += kExpanders * 32) {
        uint32_t const R = q >> 3, g = q & 7, r7 = R & 7;
        uint4 const w = *reinterpret_cast<const uint4*>(st + C::oRawCodes + q * 16);
        uint32_t const ww[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t const lo = ww[i] & 0x0f0f0f0fu, hi = (ww[i] >> 4) & 0x0f0f0f0fu;
          o[2 * i] = __byte_perm(lo, hi, 0x5140);      // columns 8i .. 8i+3
          o[2 * i + 1] = __byte_perm(lo, hi, 0x7362);  // columns 8i+4 .. 8i+7
        }
        uint8_t* const dst = st + C::oAExp + (g >> 2) * (kRows * 128) + (R >> 3) * 1024 + r7 * 128;
        uint32_t const c = (g & 3) * 2;
        *reinterpret_cast<uint4*>(dst + ((c ^ r7) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(dst + (((c + 1) ^ r7) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      // (a, a', float(sum), float(sum')) per K32 group and token pair.
      for (uint32_t j = et; j < NTOK * 8; j += kExpanders * 32) {
        uint32_t const t = j >> 3, g = j & 7;
        float const a = *reinterpret_cast<const float*>(st + C::oRawScales + j * 4);
        float const fs = float(*reinterpret_cast<const int*>(st + C::oRawSums + j * 4));
        float* const dst = reinterpret_cast<float*>(st + C::oAf + (g * (NTOK / 2) + (t >> 1)) * 16) + (t & 1);
        dst[0] = a;
        dst[2] = fs;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA's async proxy
      mbar_arrive(bar_expanded(s));
    }
  } else {
    for (uint32_t it = 0; it < iters; ++it) {
      uint32_t const s = it % C::kStages, use = it / C::kStages;
      if (!mbar_wait(bar_full(s), use & 1, abort_flag, p.status, 8)) break;      // TMA-written metadata
      if (!mbar_wait(bar_expanded(s), use & 1, abort_flag, p.status, 6)) break;  // scale table
      uint8_t* const st = smem + s * C::kStageBytes;
      // This row's metadata: d, dmin and eight six-bit (scale, min) pairs.
      uint4 const cm = *reinterpret_cast<const uint4*>(st + C::oRawMeta + my_row * 16);
      float const d = fp16_bits_to_f32(cm.x & 0xffffu), ndmin = -fp16_bits_to_f32(cm.x >> 16);
      ScaleMinWords const sm = decode_scale_min(cm.y, cm.z, cm.w);
      bool ok = true;
#pragma unroll
      for (uint32_t g = 0; g < 8; ++g) {
        uint32_t const scw = g < 4 ? sm.sc_lo : sm.sc_hi, mnw = g < 4 ? sm.mn_lo : sm.mn_hi;
        float const D = d * float(byte_of(scw, g & 3)), nMn = ndmin * float(byte_of(mnw, g & 3));
        float const cD = -kMagicF * D;  // exact: D has at most 17 significant bits
        float2 const D2 = make_float2(D, D), cD2 = make_float2(cD, cD), nMn2 = make_float2(nMn, nMn);
        uint32_t const i = it * 8 + g, b = i % C::kAccBufs, round = i / C::kAccBufs;
        if (!mbar_wait(bar_acc_full(b), round & 1, abort_flag, p.status, 7)) { ok = false; break; }
        tc_fence_after();
        uint32_t const taddr = tmem_base + ((lane_quarter * 32u) << 16) + b * NTOK + col0;
        const float4* const afp = reinterpret_cast<const float4*>(st + C::oAf + (g * (NTOK / 2) + col0 / 2) * 16);
#pragma unroll
        for (int cc = 0; cc < C::kColsPerWarp; cc += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + cc, r);
          tmem_wait_ld();
          if (cc + 16 >= C::kColsPerWarp) {  // last read of this buffer: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty(b));
          }
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            float4 const f = afp[(cc + j) / 2];  // (a, a', sum, sum') of tokens col0+cc+j, +1
            float2 const pf = make_float2(__uint_as_float(r[j] + kMagicI), __uint_as_float(r[j + 1] + kMagicI));
            float2 v = __ffma2_rn(pf, D2, cD2);                     // D * float(P), one rounding
            v = __ffma2_rn(nMn2, make_float2(f.z, f.w), v);         // - Mn * float(sum)
            acc[(cc + j) / 2] = __ffma2_rn(make_float2(f.x, f.y), v, acc[(cc + j) / 2]);
          }
          if (Dump) {
            uint32_t const row = row0 + my_row;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              uint32_t const token = tok0 + col0 + cc + j;
              if (row < p.n && token < p.m)
                p.partials[(uint64_t(token) * p.n + row) * p.G + (kb0 + it) * 8 + g] = int32_t(r[j]);
            }
          }
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_free(s));
    }
  }

  // Teardown: everyone meets, TMEM goes back.
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
  if (*abort_flag) return;

  // Output: epilogue thread = row, its columns = tokens.
  bool const is_ep = warp >= kFirstEpilogue;
  uint32_t const row = row0 + my_row;
  if (p.split_k == 1) {
    if (is_ep && row < p.n) {
#pragma unroll
      for (int j = 0; j < C::kColsPerWarp; ++j) {
        uint32_t const token = tok0 + col0 + j;
        if (token < p.m) {
          uint64_t const o = uint64_t(token) * p.n + row;
          float const v = (j & 1) ? acc[j / 2].y : acc[j / 2].x;
          p.out[o] = v + (p.residual ? p.residual[o] : 0.f);
        }
      }
    }
    return;
  }
  uint64_t const plane = uint64_t(p.m) * p.n;
  if (is_ep && row < p.n) {
#pragma unroll
    for (int j = 0; j < C::kColsPerWarp; ++j) {
      uint32_t const token = tok0 + col0 + j;
      if (token < p.m) __stcg(p.partial_tiles + slice * plane + uint64_t(token) * p.n + row, (j & 1) ? acc[j / 2].y : acc[j / 2].x);
    }
  }
  __threadfence();
  __syncthreads();
  uint32_t* const ticket = p.tickets + blockIdx.y * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) {
    uint32_t const old = atomicAdd(ticket, 1u);
    s_last = (old == p.split_k - 1) ? 1 : 0;
    if (s_last) *ticket = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (is_ep && row < p.n) {
#pragma unroll
    for (int j = 0; j < C::kColsPerWarp; ++j) {
      uint32_t const token = tok0 + col0 + j;
      if (token < p.m) {
        uint64_t const o = uint64_t(token) * p.n + row;
        float v = 0.f;
        for (uint32_t s = 0; s < p.split_k; ++s) v += __ldcg(p.partial_tiles + s * plane + o);
        p.out[o] = v + (p.residual ? p.residual[o] : 0.f);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_fn() {
  static EncodeTiled fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<EncodeTiled>(ptr);
  }();
  return fn;
}

bool make_map(CUtensorMap* map, CUtensorMapDataType type, uint32_t rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiled fn = encode_fn();
  if (!fn) return false;
  cuuint64_t d[3], st[2];
  cuuint32_t b[3], es[3] = {1, 1, 1};
  for (uint32_t i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
  for (uint32_t i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
  return fn(map, type, rank, const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NTOK>
cudaError_t launch_ntok(const WeightView& w, const Q8View& x, float* out, const float* residual, int32_t* partials,
                        uint32_t split_k, float* partial_tiles, uint32_t* tickets, int* status, cudaStream_t stream) {
  using C = Cfg<NTOK>;
  CUtensorMap tm_codes, tm_meta, tm_act, tm_scales, tm_sums;
  uint64_t const rgs = w.padded_n / 8, G = x.padded_k / 32;
  {
    uint64_t dims[3] = {256, w.tiles_k, rgs}, strides[2] = {1024, uint64_t(w.tiles_k) * 1024};
    uint32_t box[3] = {256, 1, 16};
    if (!make_map(&tm_codes, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w.codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return cudaErrorInvalidValue;
  }
  {
    uint64_t dims[3] = {32, w.tiles_k, rgs}, strides[2] = {128, uint64_t(w.tiles_k) * 128};
    uint32_t box[3] = {32, 1, 16};
    if (!make_map(&tm_meta, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w.meta, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return cudaErrorInvalidValue;
  }
  {
    uint64_t dims[2] = {x.padded_k, x.m}, strides[1] = {x.padded_k};
    uint32_t box[2] = {128, NTOK};
    if (!make_map(&tm_act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, x.codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return cudaErrorInvalidValue;
  }
  {
    uint64_t dims[2] = {G, x.m}, strides[1] = {G * 4};
    uint32_t box[2] = {8, NTOK};
    if (!make_map(&tm_scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, x.scales, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return cudaErrorInvalidValue;
    if (!make_map(&tm_sums, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, x.sums, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return cudaErrorInvalidValue;
  }
  auto kernel = partials ? mmq_tcgen05_kernel<NTOK, true> : mmq_tcgen05_kernel<NTOK, false>;
  cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (st != cudaSuccess) return st;
  TcParams p{w.meta, residual, out, partials, partial_tiles, tickets, status, w.n, x.m, w.tiles_k, split_k, uint32_t(G)};
  dim3 grid((w.padded_n + kRows - 1) / kRows, (x.m + NTOK - 1) / NTOK, split_k);
  kernel<<<grid, C::kThreads, C::kSmem, stream>>>(tm_codes, tm_meta, tm_act, tm_scales, tm_sums, p);
  return cudaGetLastError();
}

}  // namespace

bool tcgen05_supported(const WeightView& w, const Q8View& x) {
  // TMA needs 16-byte aligned global bases; the maps also need whole 16-byte row strides.
  return encode_fn() != nullptr && reinterpret_cast<uintptr_t>(w.codes) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(w.meta) % 16 == 0 && reinterpret_cast<uintptr_t>(x.codes) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(x.scales) % 16 == 0 && reinterpret_cast<uintptr_t>(x.sums) % 16 == 0;
}

TcPlan plan_tcgen05(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request) {
  TcPlan p;
  p.ntok = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128));
  uint32_t const blocks = ((n + 7) / 8 * 8 + kRows - 1) / kRows * ((m + p.ntok - 1) / p.ntok);
  uint32_t split = split_k_request;
  if (split == 0) {
    split = (148 * 2 + blocks - 1) / blocks;  // about two blocks per SM over the run
    uint32_t const max_split = tiles_k / 4 ? tiles_k / 4 : 1;
    if (split > max_split) split = max_split;
    if (split > 16) split = 16;
  }
  if (split > tiles_k) split = tiles_k;
  if (split < 1) split = 1;
  p.split_k = split;
  return p;
}

cudaError_t launch_mmq_tcgen05(const WeightView& w, const Q8View& x, float* out, const float* residual,
                               int32_t* partials, const TcPlan& plan, void* partial_tiles, uint32_t* tickets,
                               int* status, cudaStream_t stream) {
  float* pt = static_cast<float*>(partial_tiles);
  switch (plan.ntok) {
    case 16: return launch_ntok<16>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    case 32: return launch_ntok<32>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    case 64: return launch_ntok<64>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    case 128: return launch_ntok<128>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace q4k
