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
//   warp 0      lane 0 issues the raw TMA stream: 4-bit code tiles + metadata (3-D maps over the
//               split tile layout, no swizzle) and the activations' fp32 scales / int32 sums;
//               lane 1 issues the int8 activation tiles (2-D map, 128-byte swizzle, rows beyond
//               m zero-filled) into the operand ring;
//   warp 1      allocates TMEM; one lane issues the eight K32 MMAs of a super-block, each into
//               the next accumulator buffer, each followed by tcgen05.commit;
//   warps 2-5   (2-3 for wide tiles) expand nibbles to int8 in the K-major 128-byte-swizzled operand layout and build
//               the (a, a', sum, sum') table of the token pairs;
//   warps 6..   epilogue: thread = weight row; decode that row's six-bit scales once per
//               super-block, then per K32 group tcgen05.ld its accumulator columns and scale.
//               Tiles of 64/128 tokens use 8 warps (two column halves per TMEM lane quarter);
//               tiles of 16/32 tokens (decode) use 16 warps, four per quarter, each taking every
//               fourth K32 group, and add their sums in warp order at the end of the tile.
// The kernel is persistent (one block per SM walks the tile list), so TMEM allocation, barrier
// set-up and pipeline fill are paid once and the loads of the next tile overlap the epilogue of
// the current one.
// Every wait on an mbarrier is bounded: after ~2 s a thread raises the block's abort flag and
// the kernel's status word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "launch.h"
#include "tma.cuh"

namespace q4k {
namespace {

constexpr int kRows = 128;
constexpr int kProducerWarp = 0, kMmaWarp = 1, kFirstExpander = 2;
constexpr uint32_t kMagicI = 0x4B400000u;   // bit pattern of 1.5 * 2^23
constexpr float kMagicF = 12582912.0f;

// NTOK tokens per tile; NCOL <= NTOK accumulator columns actually drained (8 when m <= 8).
//
// Three shared-memory rings, each freed by the role that is last to read it, so that no role
// waits for a slower one it does not depend on:
//   R (raw)      4-bit code tiles, metadata, fp32 scales and int32 sums as TMA delivers them;
//                freed by the expanders.  Deep for narrow tiles: this is the HBM prefetch.
//   O (operands) int8 weight tile written by the expanders + int8 activation tile written by
//                TMA, both in the UMMA K-major 128-byte-swizzled layout; freed by the MMA warp's
//                tcgen05.commit as soon as the eight MMAs of the super-block have read it.
//   S (scales)   per-row metadata copy and the (a, a', sum, sum') table; freed by the epilogue.
// Epilogue warps: every warp may only touch the TMEM lanes of its quarter (warp % 4).  Wide
// tiles split the columns over two warps per quarter; narrow tiles (decode) interleave the
// eight K32 groups over kGroupSplit warps per quarter, whose partial sums are added in warp
// order at the end of a tile.
template <int NTOK, int NCOL> struct Cfg {
  static constexpr int kColSplit = NTOK >= 64 ? 2 : 1;
  static constexpr bool kChunked = NTOK >= 64;
  static constexpr int kGroupSplit = NTOK >= 64 ? 1 : (NTOK >= 32 ? 2 : 4);
  static constexpr int kEpilogueWarps = 4 * kColSplit * kGroupSplit;
  static constexpr int kExpanders = 4;
  static constexpr int kFirstEpilogue = kFirstExpander + kExpanders;
  static constexpr int kWarps = kFirstEpilogue + kEpilogueWarps;
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kColsPerWarp = NCOL / kColSplit;
  static constexpr int kAccBufs = (512 / NTOK) > 16 ? 16 : (512 / NTOK);
  // Narrow tiles: one tcgen05.commit (and one pair of barriers) per four MMAs -- the single
  // issuing thread is otherwise the bottleneck.
  static constexpr int kMmaPerCommit = NTOK <= 32 ? 4 : 1;
  static constexpr int kAccSets = kAccBufs / kMmaPerCommit;
  // ring depths
  static constexpr int kRaw = NTOK <= 16 ? 5 : (NTOK <= 64 ? 4 : 2);
  static constexpr int kOps = 2;
  static constexpr int kScl = 4;
  // raw stage
  static constexpr int kRawCodes = 16 * 1024, kRawMeta = 16 * 128, kRawScale = NTOK * 32;
  static constexpr int oRawCodes = 0, oRawMeta = kRawCodes, oRawScales = oRawMeta + kRawMeta, oRawSums = oRawScales + kRawScale;
  static constexpr int kRawStage = (oRawSums + kRawScale + 1023) / 1024 * 1024;
  static constexpr int kRawTx = kRawCodes + kRawMeta + 2 * kRawScale;
  // operand stage
  static constexpr int kAExp = 2 * kRows * 128, kB = 2 * NTOK * 128;
  static constexpr int oAExp = 0, oB = kAExp;
  static constexpr int kOpStage = (kAExp + kB + 1023) / 1024 * 1024;
  static constexpr int kBTx = kB;
  // scale stage
  static constexpr int kAf = 8 * NTOK * 8;
  static constexpr int oMeta = 0, oAf = kRawMeta;
  static constexpr int kSclStage = (kRawMeta + kAf + 127) / 128 * 128;
  // whole layout
  static constexpr int oOps = 0;
  static constexpr int oRawRing = oOps + kOps * kOpStage;
  static constexpr int oSclRing = oRawRing + kRaw * kRawStage;
  static constexpr int kRedBytes = kGroupSplit > 1 ? kEpilogueWarps * kColsPerWarp * 32 * 4 : 0;
  static constexpr int oRed = oSclRing + kScl * kSclStage;
  static constexpr int oCtrl = oRed + kRedBytes;
  // barriers: raw_full[R] raw_free[R] b_full[O] op_ready[O] op_free[O] s_full[S] s_free[S] acc_full[B] acc_empty[B] ep
  static constexpr int kBarriers = 2 * kRaw + 3 * kOps + 2 * kScl + 2 * kAccSets + 1;
  static constexpr int kSmem = oCtrl + kBarriers * 8 + 64 + 1024 /*alignment slack*/;
  static_assert(kSmem <= 227 * 1024, "shared memory budget");
};

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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

struct TcParams {
  const float* residual;
  float* out;
  int32_t* partials;
  float* partial_tiles;  // split-K scratch [slice][m][n]
  uint32_t* tickets;
  int* status;
  uint32_t n, m, tiles_k, split_k, G, row_tiles, tok_tiles;
};

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}

// Persistent: block b walks tiles b, b + gridDim.x, ...; a tile is (row tile of 128 rows,
// token tile, K slice).  Ring and accumulator-buffer counters run on across tiles, so loads
// and expansion of the next tile overlap the epilogue of the current one.
template <int NTOK, int NCOL, bool Dump>
__global__ void __launch_bounds__(Cfg<NTOK, NCOL>::kThreads, 1)
mmq_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_codes, const __grid_constant__ CUtensorMap tm_meta,
                   const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_scales,
                   const __grid_constant__ CUtensorMap tm_sums, TcParams p) {
  using C = Cfg<NTOK, NCOL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* const red = reinterpret_cast<float*>(smem + C::oRed);
  uint8_t* const ctrl = smem + C::oCtrl;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(ctrl);
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(ctrl + C::kBarriers * 8);
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(ctrl + C::kBarriers * 8 + 8);
  volatile int* const last_flag = reinterpret_cast<volatile int*>(ctrl + C::kBarriers * 8 + 12);

  uint32_t const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t const num_tiles = p.row_tiles * p.tok_tiles * p.split_k;

  uint32_t const bar0 = smem_u32(bars);
  auto bar_raw_full = [&](uint32_t i) { return bar0 + 8 * i; };
  auto bar_raw_free = [&](uint32_t i) { return bar0 + 8 * (C::kRaw + i); };
  auto bar_b_full = [&](uint32_t i) { return bar0 + 8 * (2 * C::kRaw + i); };
  auto bar_op_ready = [&](uint32_t i) { return bar0 + 8 * (2 * C::kRaw + C::kOps + i); };
  auto bar_op_free = [&](uint32_t i) { return bar0 + 8 * (2 * C::kRaw + 2 * C::kOps + i); };
  auto bar_s_full = [&](uint32_t i) { return bar0 + 8 * (2 * C::kRaw + 3 * C::kOps + i); };
  auto bar_s_free = [&](uint32_t i) { return bar0 + 8 * (2 * C::kRaw + 3 * C::kOps + C::kScl + i); };
  auto bar_acc_full = [&](uint32_t i) { return bar0 + 8 * (2 * C::kRaw + 3 * C::kOps + 2 * C::kScl + i); };
  auto bar_acc_empty = [&](uint32_t i) { return bar0 + 8 * (2 * C::kRaw + 3 * C::kOps + 2 * C::kScl + C::kAccSets + i); };
  uint32_t const bar_ep = bar0 + 8 * (C::kBarriers - 1);

  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < C::kRaw; ++i) { mbar_init(bar_raw_full(i), 1); mbar_init(bar_raw_free(i), C::kExpanders); }
    for (uint32_t i = 0; i < C::kOps; ++i) {
      mbar_init(bar_b_full(i), 1);
      mbar_init(bar_op_ready(i), C::kExpanders);
      mbar_init(bar_op_free(i), 1);
    }
    for (uint32_t i = 0; i < C::kScl; ++i) { mbar_init(bar_s_full(i), C::kExpanders); mbar_init(bar_s_free(i), C::kEpilogueWarps); }
    for (uint32_t i = 0; i < C::kAccSets; ++i) { mbar_init(bar_acc_full(i), 1); mbar_init(bar_acc_empty(i), 4 * C::kColSplit * C::kMmaPerCommit); }
    mbar_init(bar_ep, C::kEpilogueWarps);
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

  auto tile_coords = [&](uint32_t t, uint32_t& row_tile, uint32_t& tok_tile, uint32_t& slice, uint32_t& kb0, uint32_t& kb1) {
    tok_tile = t % p.tok_tiles;  // token tile fastest: blocks running together share weight tiles in L2
    uint32_t const rest = t / p.tok_tiles;
    slice = rest % p.split_k;
    row_tile = rest / p.split_k;
    kb0 = uint32_t((uint64_t(slice) * p.tiles_k) / p.split_k);
    kb1 = uint32_t((uint64_t(slice + 1) * p.tiles_k) / p.split_k);
  };
  // After an early exit: let TMA copies that were started land before shared memory goes away.
  auto drain = [&](uint32_t first, uint32_t issued, uint32_t depth, uint32_t bar_base) {
    for (uint32_t j = first; j < issued; ++j) {
      long long const t0 = clock64();
      uint32_t done = 0;
      while (!done && clock64() - t0 < 200000000LL)
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar_base + 8 * (j % depth)), "r"((j / depth) & 1) : "memory");
    }
  };

  if (warp == kProducerWarp) {
    // Raw stream: code tiles, metadata, activation scales and sums of every super-block.
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        uint32_t row_tile, tok_tile, slice, kb0, kb1;
        tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
        int const rg0 = int(row_tile * (kRows / 8)), tok0 = int(tok_tile * NTOK);
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
          uint32_t const r = it % C::kRaw, use = it / C::kRaw;
          if (!mbar_wait(bar_raw_free(r), (use & 1) ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          uint8_t* const st = smem + C::oRawRing + r * C::kRawStage;
          uint32_t const bar = bar_raw_full(r);
          mbar_expect_tx(bar, C::kRawTx);
          tma_3d(smem_u32(st + C::oRawCodes), &tm_codes, 0, int(kb), rg0, bar);
          tma_3d(smem_u32(st + C::oRawMeta), &tm_meta, 0, int(kb), rg0, bar);
          tma_2d(smem_u32(st + C::oRawScales), &tm_scales, int(kb) * 8, tok0, bar);
          tma_2d(smem_u32(st + C::oRawSums), &tm_sums, int(kb) * 8, tok0, bar);
        }
      }
      if (*abort_flag) drain(it > C::kRaw ? it - C::kRaw : 0, it, C::kRaw, bar_raw_full(0));
    } else if (lane == 1) {
      // Activation stream (second lane of the same warp; the two lanes progress independently):
      // int8 tiles straight into the operand ring.
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        uint32_t row_tile, tok_tile, slice, kb0, kb1;
        tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
        int const tok0 = int(tok_tile * NTOK);
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
          uint32_t const o = it % C::kOps, use = it / C::kOps;
          if (!mbar_wait(bar_op_free(o), (use & 1) ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
          uint8_t* const st = smem + C::oOps + o * C::kOpStage;
          uint32_t const bar = bar_b_full(o);
          mbar_expect_tx(bar, C::kBTx);
          tma_2d(smem_u32(st + C::oB), &tm_act, int(kb) * 256, tok0, bar);
          tma_2d(smem_u32(st + C::oB + NTOK * 128), &tm_act, int(kb) * 256 + 128, tok0, bar);
        }
      }
      if (*abort_flag) drain(it > C::kOps ? it - C::kOps : 0, it, C::kOps, bar_b_full(0));
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(NTOK);
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        uint32_t row_tile, tok_tile, slice, kb0, kb1;
        tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
        for (uint32_t kb = kb0; ok && kb < kb1; ++kb, ++it) {
          uint32_t const o = it % C::kOps, use = it / C::kOps;
          if (!mbar_wait(bar_b_full(o), use & 1, abort_flag, p.status, 3)) { ok = false; break; }
          if (!mbar_wait(bar_op_ready(o), use & 1, abort_flag, p.status, 4)) { ok = false; break; }
          tc_fence_after();
          uint8_t* const st = smem + C::oOps + o * C::kOpStage;
          uint32_t const a_base = smem_u32(st + C::oAExp), b_base = smem_u32(st + C::oB);
#pragma unroll
          for (uint32_t g = 0; g < 8; ++g) {
            uint32_t const i = it * 8 + g, b = i % C::kAccBufs, round = i / C::kAccBufs, set = b / C::kMmaPerCommit;
            if (g % C::kMmaPerCommit == 0) {
              if (!mbar_wait(bar_acc_empty(set), (round & 1) ^ 1, abort_flag, p.status, 5)) { ok = false; break; }
              tc_fence_after();
            }
            uint64_t const ad = umma_desc(a_base + (g >> 2) * (kRows * 128) + (g & 3) * 32);
            uint64_t const bd = umma_desc(b_base + (g >> 2) * (NTOK * 128) + (g & 3) * 32);
            umma_i8(tmem_base + b * NTOK, ad, bd, idesc);
            if (g % C::kMmaPerCommit == C::kMmaPerCommit - 1) umma_commit(bar_acc_full(set));
          }
          if (ok) umma_commit(bar_op_free(o));  // operands are free once these MMAs have read them
        }
      }
    }
  } else if (warp < C::kFirstEpilogue) {
    uint32_t const et = threadIdx.x - kFirstExpander * 32;  // 0 .. 32*kExpanders-1
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
      uint32_t row_tile, tok_tile, slice, kb0, kb1;
      tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
      for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
        uint32_t const r = it % C::kRaw, o = it % C::kOps, sc = it % C::kScl;
        if (!mbar_wait(bar_raw_full(r), (it / C::kRaw) & 1, abort_flag, p.status, 6)) { ok = false; break; }
        if (!mbar_wait(bar_op_free(o), ((it / C::kOps) & 1) ^ 1, abort_flag, p.status, 7)) { ok = false; break; }
        if (!mbar_wait(bar_s_free(sc), ((it / C::kScl) & 1) ^ 1, abort_flag, p.status, 8)) { ok = false; break; }
        const uint8_t* const raw = smem + C::oRawRing + r * C::kRawStage;
        uint8_t* const ops = smem + C::oOps + o * C::kOpStage;
        uint8_t* const scl = smem + C::oSclRing + sc * C::kSclStage;
        // 1024 raw 16-byte chunks: chunk q = (row q/8 of the tile, K32 group q%8).
#pragma unroll 2
        for (uint32_t q = et; q < 1024; q += C::kExpanders * 32) {
          uint32_t const R = q >> 3, g = q & 7, r7 = R & 7;
          uint4 const w = *reinterpret_cast<const uint4*>(raw + C::oRawCodes + q * 16);
          uint32_t const ww[4] = {w.x, w.y, w.z, w.w};
          uint32_t ov[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t const lo = ww[i] & 0x0f0f0f0fu, hi = (ww[i] >> 4) & 0x0f0f0f0fu;
            ov[2 * i] = __byte_perm(lo, hi, 0x5140);      // columns 8i .. 8i+3
            ov[2 * i + 1] = __byte_perm(lo, hi, 0x7362);  // columns 8i+4 .. 8i+7
          }
          uint8_t* const dst = ops + C::oAExp + (g >> 2) * (kRows * 128) + (R >> 3) * 1024 + r7 * 128;
          uint32_t const c = (g & 3) * 2;
          *reinterpret_cast<uint4*>(dst + ((c ^ r7) << 4)) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
          *reinterpret_cast<uint4*>(dst + (((c + 1) ^ r7) << 4)) = make_uint4(ov[4], ov[5], ov[6], ov[7]);
        }
        // Metadata rows (16 bytes each) move to the scale ring; the epilogue reads them there.
        for (uint32_t j = et; j < kRows; j += C::kExpanders * 32)
          *reinterpret_cast<uint4*>(scl + C::oMeta + j * 16) = *reinterpret_cast<const uint4*>(raw + C::oRawMeta + j * 16);
        // (a, a', float(sum), float(sum')) per K32 group and token pair.
        for (uint32_t j = et; j < NTOK * 8; j += C::kExpanders * 32) {
          uint32_t const tk = j >> 3, g = j & 7;
          float const a = *reinterpret_cast<const float*>(raw + C::oRawScales + j * 4);
          float const fs = float(*reinterpret_cast<const int*>(raw + C::oRawSums + j * 4));
          float* const dst = reinterpret_cast<float*>(scl + C::oAf + (g * (NTOK / 2) + (tk >> 1)) * 16) + (tk & 1);
          dst[0] = a;
          dst[2] = fs;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA's async proxy
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar_op_ready(o));
          mbar_arrive(bar_s_full(sc));
          mbar_arrive(bar_raw_free(r));
        }
      }
    }
  } else {
    constexpr int GS = C::kGroupSplit, CW = C::kColsPerWarp, CH = CW >= 16 ? 16 : 8;
    uint32_t const ep = warp - C::kFirstEpilogue, quarter = warp & 3;  // TMEM lanes 32*quarter ..
    uint32_t const u = ep >> 2, cs = u % C::kColSplit, gs = u / C::kColSplit;
    uint32_t const col0 = cs * CW;
    uint32_t const my_row = quarter * 32 + lane;  // row inside the tile
    bool const final_warp = gs == 0;               // holds the tile's sums after the group-split reduction
    uint32_t it = 0, ep_phase = 0;
    bool ok = true;
    auto ep_sync = [&](int code) {  // all epilogue warps meet (bounded like every other wait)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ep);
      if (!mbar_wait(bar_ep, ep_phase, abort_flag, p.status, code)) ok = false;
      ep_phase ^= 1;
    };
    for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
      uint32_t row_tile, tok_tile, slice, kb0, kb1;
      tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
      uint32_t const row0 = row_tile * kRows, tok0 = tok_tile * NTOK;
      float2 acc[CW / 2];
#pragma unroll
      for (int i = 0; i < CW / 2; ++i) acc[i] = make_float2(0.f, 0.f);

      for (uint32_t kb = kb0; ok && kb < kb1; ++kb, ++it) {
        uint32_t const sc = it % C::kScl;
        if (!mbar_wait(bar_s_full(sc), (it / C::kScl) & 1, abort_flag, p.status, 9)) { ok = false; break; }
        const uint8_t* const scl = smem + C::oSclRing + sc * C::kSclStage;
        // This row's metadata: d, dmin and eight six-bit (scale, min) pairs.
        uint4 const cm = *reinterpret_cast<const uint4*>(scl + C::oMeta + my_row * 16);
        float const d = fp16_bits_to_f32(cm.x & 0xffffu), ndmin = -fp16_bits_to_f32(cm.x >> 16);
        ScaleMinWords const sm = decode_scale_min(cm.y, cm.z, cm.w);
#pragma unroll(NTOK >= 64 ? 8 : 2)
        for (int tt = 0; tt < 8 / GS; ++tt) {
          uint32_t const g = gs + GS * tt;
          uint32_t const scw = (g < 4) ? sm.sc_lo : sm.sc_hi, mnw = (g < 4) ? sm.mn_lo : sm.mn_hi;
          uint32_t const sh = (g & 3) * 8;
          // six-bit integers to fp32 through the 1.5 * 2^23 bias: stays off the conversion pipe
          float const D = d * (__uint_as_float(kMagicI | ((scw >> sh) & 0xffu)) - kMagicF);
          float const nMn = ndmin * (__uint_as_float(kMagicI | ((mnw >> sh) & 0xffu)) - kMagicF);
          float const cD = -kMagicF * D;  // exact: D has at most 17 significant bits
          float2 const D2 = make_float2(D, D), cD2 = make_float2(cD, cD), nMn2 = make_float2(nMn, nMn);
          uint32_t const i = it * 8 + g, b = i % C::kAccBufs, round = i / C::kAccBufs, set = b / C::kMmaPerCommit;
          if (!mbar_wait(bar_acc_full(set), round & 1, abort_flag, p.status, 10)) { ok = false; break; }
          tc_fence_after();
          uint32_t const taddr = tmem_base + ((quarter * 32u) << 16) + b * NTOK + col0;
          const float4* const afp = reinterpret_cast<const float4*>(scl + C::oAf + (g * (NTOK / 2) + col0 / 2) * 16);
          uint32_t r[CW];
          if constexpr (C::kChunked) {
            // Wide tiles: read and fold 16 columns at a time; with the group loop unrolled the
            // compiler overlaps one chunk's arithmetic with the next chunk's TMEM read.
#pragma unroll
            for (int cc = 0; cc < CW; cc += 16) {
              tmem_ld16(taddr + cc, r + cc);
              tmem_wait_ld();
              if (cc + 16 >= CW) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty(set));
              }
#pragma unroll
              for (int j = cc; j < cc + 16; j += 2) {
                float4 const f = afp[j / 2];
                float2 const pf = make_float2(__uint_as_float(r[j] + kMagicI), __uint_as_float(r[j + 1] + kMagicI));
                float2 v = __ffma2_rn(pf, D2, cD2);
                v = __ffma2_rn(nMn2, make_float2(f.z, f.w), v);
                acc[j / 2] = __ffma2_rn(make_float2(f.x, f.y), v, acc[j / 2]);
              }
            }
          } else {
            // Narrow tiles: all TMEM reads of the group go out before the single wait, and the
            // buffer returns to the MMA warp before the arithmetic.
#pragma unroll
            for (int cc = 0; cc < CW; cc += CH) {
              if constexpr (CH == 16) tmem_ld16(taddr + cc, r + cc);
              else tmem_ld8(taddr + cc, r + cc);
            }
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty(set));
#pragma unroll
            for (int j = 0; j < CW; j += 2) {
              float4 const f = afp[j / 2];  // (a, a', sum, sum') of tokens col0+j, col0+j+1
              float2 const pf = make_float2(__uint_as_float(r[j] + kMagicI), __uint_as_float(r[j + 1] + kMagicI));
              float2 v = __ffma2_rn(pf, D2, cD2);                     // D * float(P), one rounding
              v = __ffma2_rn(nMn2, make_float2(f.z, f.w), v);         // - Mn * float(sum)
              acc[j / 2] = __ffma2_rn(make_float2(f.x, f.y), v, acc[j / 2]);
            }
          }
          if (Dump) {
            uint32_t const row = row0 + my_row;
#pragma unroll
            for (int j = 0; j < CW; ++j) {
              uint32_t const token = tok0 + col0 + j;
              if (row < p.n && token < p.m)
                p.partials[(uint64_t(token) * p.n + row) * p.G + kb * 8 + g] = int32_t(r[j]);
            }
          }
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_free(sc));
      }
      if (!ok) break;

      // ---- end of tile: combine the group-split warps, then write (or hand to the split-K fix-up)
      if constexpr (GS > 1) {
#pragma unroll
        for (int j = 0; j < CW; ++j) red[(ep * CW + j) * 32 + lane] = (j & 1) ? acc[j / 2].y : acc[j / 2].x;
        ep_sync(11);
        if (!ok) break;
        if (final_warp) {
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            float v = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < GS; ++k2) v += red[((ep + 4 * C::kColSplit * k2) * CW + j) * 32 + lane];  // warp order
            if (j & 1) acc[j / 2].y = v; else acc[j / 2].x = v;
          }
        }
      }
      uint32_t const row = row0 + my_row;
      bool const writer = final_warp && row < p.n;
      if (p.split_k == 1) {
        if (writer) {
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            uint32_t const token = tok0 + col0 + j;
            if (token < p.m) {
              uint64_t const o = uint64_t(token) * p.n + row;
              p.out[o] = ((j & 1) ? acc[j / 2].y : acc[j / 2].x) + (p.residual ? p.residual[o] : 0.f);
            }
          }
        }
      } else {
        uint64_t const plane = uint64_t(p.m) * p.n;
        if (writer) {
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            uint32_t const token = tok0 + col0 + j;
            if (token < p.m)
              __stcg(p.partial_tiles + slice * plane + uint64_t(token) * p.n + row, (j & 1) ? acc[j / 2].y : acc[j / 2].x);
          }
        }
        __threadfence();
        ep_sync(12);
        if (!ok) break;
        if (ep == 0 && lane == 0) {
          uint32_t* const ticket = p.tickets + row_tile * p.tok_tiles + tok_tile;
          uint32_t const old = atomicAdd(ticket, 1u);
          int const last = (old == p.split_k - 1) ? 1 : 0;
          if (last) *ticket = 0;  // leave the counter clean for the next launch
          *last_flag = last;
        }
        ep_sync(13);
        if (!ok) break;
        if (*last_flag) {
          __threadfence();
          if (writer) {
#pragma unroll
            for (int j = 0; j < CW; ++j) {
              uint32_t const token = tok0 + col0 + j;
              if (token < p.m) {
                uint64_t const o = uint64_t(token) * p.n + row;
                float v = 0.f;
                for (uint32_t s2 = 0; s2 < p.split_k; ++s2) v += __ldcg(p.partial_tiles + s2 * plane + o);  // slice order
                p.out[o] = v + (p.residual ? p.residual[o] : 0.f);
              }
            }
          }
        }
      }
      if constexpr (GS > 1) {
        ep_sync(14);  // nobody overwrites the sums (or the last-arrival flag) before everybody has read them
      } else if (p.split_k > 1) {
        ep_sync(14);
      }
    }
  }

  // Teardown: everyone meets, TMEM goes back.
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ------------------------------------------------------------------------------------------
template <int NTOK, int NCOL>
cudaError_t launch_ntok(const WeightView& w, const Q8View& x, float* out, const float* residual, int32_t* partials,
                        uint32_t split_k, float* partial_tiles, uint32_t* tickets, int* status, cudaStream_t stream) {
  using C = Cfg<NTOK, NCOL>;
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
  auto kernel = partials ? mmq_tcgen05_kernel<NTOK, NCOL, true> : mmq_tcgen05_kernel<NTOK, NCOL, false>;
  cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (st != cudaSuccess) return st;
  uint32_t const row_tiles = (w.padded_n + kRows - 1) / kRows, tok_tiles = (x.m + NTOK - 1) / NTOK;
  TcParams p{residual, out, partials, partial_tiles, tickets, status, w.n, x.m, w.tiles_k, split_k, uint32_t(G), row_tiles, tok_tiles};
  uint64_t const tiles = uint64_t(row_tiles) * tok_tiles * split_k;
  // Narrow (decode) tiles: one persistent block per SM walks the tile list.  Wide tiles run one
  // block per tile; measured faster there (the hardware scheduler balances the long tiles).
  uint32_t grid = uint32_t(tiles);
  if (NTOK <= 32 && tiles > uint64_t(sm_count())) grid = uint32_t(sm_count());
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
    // Pick the K split whose tile count fills whole rounds of the machine best, among splits
    // that leave at least four super-blocks per slice.  Every extra slice costs a partial tile
    // of m*n fp32 written and read back, which is negligible for a handful of tokens and
    // prohibitive for a prefill chunk -- the penalty grows with m.
    uint32_t const sms = uint32_t(sm_count());
    uint32_t const max_split = tiles_k / 4 ? (tiles_k / 4 > 16 ? 16 : tiles_k / 4) : 1;
    double const penalty = 0.01 + 0.1 * (m >= 128 ? 1.0 : double(m) / 128.0);
    double best = -1.0;
    split = 1;
    for (uint32_t s = 1; s <= max_split; ++s) {
      uint64_t const tiles = uint64_t(blocks) * s;
      uint64_t const rounds = (tiles + sms - 1) / sms;
      double eff = double(tiles) / double(rounds * sms) - penalty * (s - 1);
      if (eff > best + 1e-9) { best = eff; split = s; }
    }
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
    case 16:
      if (x.m <= 8) return launch_ntok<16, 8>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
      return launch_ntok<16, 16>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    case 32: return launch_ntok<32, 32>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    case 64: return launch_ntok<64, 64>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    case 128: return launch_ntok<128, 128>(w, x, out, residual, partials, plan.split_k, pt, tickets, status, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace q4k
