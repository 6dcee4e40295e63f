// Q4_K x Q8 matmul on the 5th-generation tensor cores: tcgen05.mma kind::i8, operands staged
// by TMA, one TMEM accumulator per K32 group, scaling epilogue on CUDA cores.
//
// The per-K32 rule of the reference (cuda/q4k_q8.cu:70-72: one exact int32 dot per 32 columns,
// never carried into the next group) fixes the structure: every data MMA has K = 32 and its
// 128 x NTOK int32 results are drained from TMEM and folded into fp32 accumulators in registers
// as  acc += D * (a * float(P)) - Mn * (a * float(sum)).
//
// What the design is built around (clock64 units on a B200, one block per SM):
//   * Two packed FMAs per pair of partials and nothing else on the fp32 pipe.  No int -> float
//     conversion: before the data MMA of a group a second MMA of two constant tiles (every byte
//     64) writes 32 * 64 * 64 = 2^17 into every accumulator, and the data MMA accumulates on top.
//     The int32 word 2^17 + P, read as an fp32 bit pattern, is the subnormal (2^17 + P) * 2^-149,
//     an affine function of P, so one FMA with the token's scale a' = a * 2^89 and the exact
//     constant c' = -a' * 2^-132 yields a * P * 2^-60 with a single rounding, and the second FMA
//     acc += S * v with the row's S = d * sc * 2^60 completes the term.  The token side goes
//     first because its operands are natural register pairs (two neighbouring tokens), whereas
//     the row scale has to be duplicated into a pair.  Should a' overflow (scales beyond 2^38)
//     the super-block takes a slower loop that reads the plain scale from global memory.
//   * The min term  -dmin * sum_g m[n,g] * (a * sum)[t,g]  is a rank-8 update per super-block
//     and runs on the warp-level tensor MMAs (mma.sync bf16): six-bit mins are exact in bf16,
//     a * sum is split into three bf16 terms that add up to it exactly.
//   * Shared memory (one 128-byte wavefront per clock) is shared by the MMA's operand fetch, the
//     expanders and the epilogue's scale loads.  The accumulators are therefore read in the
//     16x256b shape (the MMA C-fragment layout): a thread owns 4 rows x 8 tokens of its warp's
//     32 x 32 patch and needs the scales of 8 tokens and 4 rows only (an owner of one row x 32
//     tokens would read 32 token scales per group as broadcasts and saturate the pipe).  Tables
//     are laid out so that expander stores and epilogue loads are free of bank conflicts.
//   * tcgen05.ld in that shape delivers 256 B/clk per SM and has a latency of 65 clk unloaded,
//     130 with sixteen warps reading; tcgen05.wait::ld waits for everything outstanding.  The
//     epilogue therefore works in units of two reads (32 rows x 16 tokens) with the next unit's
//     reads in flight, loads its scale operands under the TMEM wait and issues all first FMAs
//     of a unit before the second ones.  The eight groups of a super-block are unrolled, so that
//     every decision about accumulator sets and successors is static and each read has one site.
//   * Every barrier hand-off costs several hundred clocks of exposed latency: accumulator
//     buffers travel in sets (one commit, one wait, one release per set), waits spin on
//     mbarrier.try_wait without back-off, and one thread polls both TMA streams.
//
// Tile: 128 weight rows (the M side, one TMEM lane per row) x NTOK tokens (the N side) per
// block, K walked in 256-column super-blocks.  Warp roles:
//   warp 0      one lane issues both TMA streams: raw 4-bit code tiles + metadata (3-D maps over
//               the split tile layout, no swizzle) into the raw ring, int8 activation tiles (2-D
//               map, 128-byte swizzle, rows beyond m zero-filled) into the operand ring;
//   warp 1      allocates TMEM; one lane issues, set by set, the constant MMAs and the data MMAs
//               into the set's accumulator buffers, then tcgen05.commit;
//   expanders   (5 or 9 warps) expand nibbles to int8 in the K-major 128-byte-swizzled operand
//               layout, decode the six-bit scales into the row tables (S, -dmin, mins as bf16)
//               and build the token tables (a', a * sum in three bf16 terms) from the
//               activations' scales and sums in global memory;
//   one warp    waits for the launch before this one (griddepcontrol.wait) and then releases the next one;
//   epilogue    tiles of 128 tokens: 16 warps, four column quarters per TMEM lane quarter; 64
//               tokens: 8 warps, two column halves; narrower tiles split the eight K32 groups
//               over two warps per lane quarter and add their sums in warp order at the end of
//               a tile.  On the wide tiles the other warps hand registers to the epilogue warps
//               (setmaxnreg).
// The kernel is persistent (one block per SM walks the tile list), so TMEM allocation, barrier
// set-up and pipeline fill are paid once and the loads of the next tile overlap the epilogue of
// the current one.
// Every wait on an mbarrier is bounded: after ~2 s a thread raises the block's abort flag and
// the kernel's status word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "launch.h"
#include "tma.cuh"
#include "umma.cuh"

namespace q4k {
namespace {

constexpr int kRows = 128;
constexpr int kProducerWarp = 0, kMmaWarp = 1, kFirstExpander = 2;
constexpr uint32_t kPreset = 1u << 17;  // what the constant MMA leaves in every accumulator: 32 * 64 * 64
constexpr uint32_t kConstByte = 0x40404040u;
// The int32 word 2^17 + P of an accumulator, read as fp32 bits, is (2^17 + P) * 2^-149.  The token-side table holds
// a' = a * 2^89 and c' = -a' * 2^-132 (so that fma(word, a', c') = a * P * 2^-60 with one rounding), the row-side
// table S = d * sc * 2^60.  Scales above 2^38 would overflow a': their super-block takes the slower loop.
constexpr float kTokScalePow = 0x1p89f, kRowScalePow = 0x1p60f, kBiasOut = -0x1p-132f, kWideAbove = 0x1p38f;
// The constant operand: every byte equal, so neither the swizzle nor which bytes a row reads matters, and the 8-row
// atoms may overlap: the descriptor gives them a stride of 128 bytes instead of 1024 (16 atoms end at 15 * 128 + 1024).
constexpr int kConstBytes = 4 * 1024, kConstAtomStride = 128;

// NTOK tokens per tile; NCOL <= NTOK accumulator columns actually drained (8 when m <= 8).
//
// Three shared-memory rings, each freed by the role that is last to read it, so that no role
// waits for a slower one it does not depend on:
//   R (raw)      4-bit code tiles, metadata, fp32 scales and int32 sums as TMA delivers them;
//                freed by the expanders.  Deep for narrow tiles: this is the HBM prefetch.
//   O (operands) int8 weight tile written by the expanders + int8 activation tile written by
//                TMA, both in the UMMA K-major 128-byte-swizzled layout; freed by the MMA warp's
//                tcgen05.commit as soon as the MMAs of the super-block have read it.
//   S (scales)   per-row metadata copy and the activation-scale table; freed by the epilogue.
// Epilogue warps: every warp may only touch the TMEM lanes of its quarter (warp % 4).
template <int NTOK, int NCOL> struct Cfg {
  static constexpr int kColSplit = NTOK >= 128 ? 4 : (NTOK >= 32 ? 2 : 1);
  static constexpr int kGroupSplit = NTOK >= 64 ? 1 : 2;
  static constexpr int kEpilogueWarps = 4 * kColSplit * kGroupSplit;
  // Roles are aligned to groups of four warps (the register file is shared by the four warps that sit
  // on one scheduler each): producer + MMA + expanders fill the first groups, the epilogue the rest.
  // Measured: 10 or 14 expander warps on the wide tiles slow the block down, and on the 128-token tile 5 instead of 6
  // cost 11 %.  Tiles up to 64 tokens (the weight-streaming regime, where launches should run into each other) give
  // one warp slot to the dependency warp, which waits for the preceding launch and then releases the next one; on the
  // 128-token tile the expanders always wait for the preceding launch themselves and the first of them releases.
  static constexpr bool kHasDepWarp = NTOK < 128;
  static constexpr int kExpanders = NTOK >= 128 ? 6 : (NTOK >= 64 ? 5 : 9);
  static constexpr int kDepWarp = kHasDepWarp ? kFirstExpander + kExpanders : 1 << 20;
  // Wide tiles: the non-epilogue warps give registers back, the epilogue warps take them (setmaxnreg).
  static constexpr bool kRebalance = NTOK >= 128 || NTOK == 32;
  // The block's own allocation is the pool: 24 warps start at 80 registers (8 * 48 + 16 * 96 = 24 * 80), 28 warps at 72
  // (12 * 48 + 16 * 88 <= 28 * 72).  Asking for more than the pool holds blocks the warps forever.
  static constexpr int kRegsLow = 48;
  static constexpr int kFirstEpilogue = kFirstExpander + kExpanders + (kHasDepWarp ? 1 : 0);
  static constexpr int kWarps = kFirstEpilogue + kEpilogueWarps;
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kRegsLaunch = (65536 / kThreads) / 8 * 8 > 128 ? 128 : (65536 / kThreads) / 8 * 8;
  static constexpr int kRegsHighRaw = (kWarps * kRegsLaunch - kFirstEpilogue * kRegsLow) / kEpilogueWarps / 8 * 8;
  static constexpr int kRegsHigh = kRegsHighRaw > 112 ? 112 : kRegsHighRaw;
  static constexpr int kColsPerWarp = NCOL / kColSplit;
  static constexpr int kAccBufs = (512 / NTOK) > 16 ? 16 : (512 / NTOK);
  // One tcgen05.commit, one wait and one release per set of K32 groups (two on 128-token tiles, which have four
  // buffers; four elsewhere): measured, one buffer per set costs 20-30 % and four per set beat two.
  static constexpr int kMmaPerCommit = NTOK <= 64 ? 4 : 2;
  static constexpr int kAccSets = kAccBufs / kMmaPerCommit;
  // ring depths
  static constexpr int kRaw = NTOK <= 16 ? 5 : (NTOK <= 32 ? 4 : (NTOK <= 64 ? 5 : 3));
  static constexpr int kOps = 2;
  static constexpr int kScl = NTOK >= 64 ? 2 : 3;
  // raw stage
  static constexpr int kRawCodes = 16 * 1024, kRawMeta = 16 * 128;
  static constexpr int oRawCodes = 0, oRawMeta = kRawCodes;
  static constexpr int kRawStage = kRawCodes + kRawMeta;
  static constexpr int kRawTx = kRawCodes + kRawMeta;
  // operand stage
  static constexpr int kAExp = 2 * kRows * 128, kB = 2 * NTOK * 128;
  static constexpr int oAExp = 0, oB = kAExp;
  static constexpr int kOpStage = (kAExp + kB + 1023) / 1024 * 1024;
  static constexpr int kBTx = kB;
  // scale stage: row scales S = d * sc * 2^60 ([group][lane quarter][row & 7][row / 8 & 3]) | -dmin (same row order)
  //              | six-bit mins as bf16 [row][8] | a' = a * 2^89 [group][token, padded] | a * sum as three bf16 terms
  //              [token][term][group] | stamp of the last stage with an overflowing a'
  static constexpr int kRowTab = 8 * kRows * 4;
  static constexpr int kAfStride = NTOK + 4;  // floats between groups of the a' table: the expanders' stores (eight groups x four tokens per warp) then fall into 32 different banks
  static constexpr int oS = 0, oNd = kRowTab, oMt = oNd + kRows * 4, oAf = oMt + kRows * 16, oAsT = oAf + 8 * kAfStride * 4,
                       oWide = oAsT + NTOK * 48;
  static constexpr int kSclStage = (oWide + 16 + 127) / 128 * 128;
  // whole layout
  static constexpr int oOps = 0;
  static constexpr int oRawRing = oOps + kOps * kOpStage;
  static constexpr int oConst = oRawRing + kRaw * kRawStage;
  static constexpr int oSclRing = oConst + kConstBytes;
  static constexpr int kRedBytes = kGroupSplit > 1 ? kEpilogueWarps * kColsPerWarp * 32 * 4 : 0;
  static constexpr int oRed = oSclRing + kScl * kSclStage;
  static constexpr int oCtrl = oRed + kRedBytes;
  // barriers: raw_full[R] raw_free[R] b_full[O] op_ready[O] op_free[O] s_full[S] s_free[S] acc_full[B] acc_empty[B] ep
  static constexpr int kBarriers = 2 * kRaw + 3 * kOps + 2 * kScl + 2 * kAccSets + 1;
  static constexpr int kSmem = oCtrl + kBarriers * 8 + 64 + 1024 /*alignment slack*/;
  static_assert(kSmem <= 227 * 1024, "shared memory budget");
  static_assert(kOpStage % 1024 == 0 && oRawRing % 1024 == 0, "swizzled tiles need 1024-byte alignment");
};

struct TcParams {
  const float* xscales;    // activations' fp32 scales [m][G]
  const int32_t* xsums;    // and int32 sums
  const float* residual;   // same geometry as the destinations
  float* out[8];           // fp32 destinations: one buffer, or every rank's copy of a gathered output
  uint16_t* out_bf16;      // when set, the single destination is bf16 (round to nearest even)
  uint32_t* peer_flag[8];  // gather only: rank g's arrival counters; [rank] counts this rank's deliveries
  uint32_t* done;          // gather only: block counter of this launch, zero on entry and on exit
  uint32_t* unsignalled;   // gather only: finished projections of this rank not yet announced to the peers
  uint32_t ndst, rank;
  uint32_t out_stride, out_row0;  // destination element of (token, row) = token * out_stride + out_row0 + row
  int32_t* partials;
  float* partial_tiles;  // split-K scratch [slice][m][n]
  uint32_t* tickets;
  int* status;
  uint32_t n, m, tiles_k, split_k, G, row_tiles, tok_tiles;
  uint32_t input_settled;  // activations and residual were complete before the preceding launch was enqueued
};

// Accumulator patch of 16 TMEM lanes x (8 * NB) columns in the MMA C-fragment layout: register
// 4j + 2i + e of lane l = (lane 8i + l / 4, column 8j + 2 (l % 4) + e) of the patch.
template <int NB> __device__ __forceinline__ void tmem_ld_frag(uint32_t taddr, uint32_t* r) {
  static_assert(NB == 1 || NB == 2 || NB == 4, "column blocks per load");
  if constexpr (NB == 1) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
  } else if constexpr (NB == 2) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
  } else {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
  }
}

__device__ __forceinline__ float2 as_f2(uint32_t x, uint32_t y) { return make_float2(__uint_as_float(x), __uint_as_float(y)); }

// D += A (16 x 16, bf16) * B (16 x 8, bf16), fp32 accumulate: the warp-level tensor-core MMA, used for the min term.
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same with a zero accumulator input (no registers to clear first).
__device__ __forceinline__ void mma_bf16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ float2 lds64f(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts16(uint32_t a, uint16_t x) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"(x) : "memory"); }

// Accumulator buffer and barrier parity of K32 group g of the block's it-th super-block (buffers are used round
// robin, eight per super-block): compile-time for the four-buffer tiles when g is.
template <int AB> __device__ __forceinline__ void acc_slot(uint32_t it, uint32_t g, uint32_t& b, uint32_t& parity) {
  static_assert(AB == 4 || AB == 8 || AB == 16, "accumulator buffers");
  if constexpr (AB == 4) { b = g & 3; parity = (g >> 2) & 1; }
  else if constexpr (AB == 8) { b = g; parity = it & 1; }
  else { b = ((it & 1) << 3) + g; parity = (it >> 1) & 1; }
}

// Persistent: block b walks tiles b, b + gridDim.x, ...; a tile is (row tile of 128 rows,
// token tile, K slice).  Ring and accumulator-buffer counters run on across tiles, so loads
// and expansion of the next tile overlap the epilogue of the current one.
template <int NTOK, int NCOL, bool Dump>
__global__ void __launch_bounds__(Cfg<NTOK, NCOL>::kThreads, 1)
mmq_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_codes, const __grid_constant__ CUtensorMap tm_meta,
                   const __grid_constant__ CUtensorMap tm_act, const TcParams p) {
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
  uint32_t const smem_s = smem_u32(smem);

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
    for (uint32_t i = 0; i < C::kAccSets; ++i) { mbar_init(bar_acc_full(i), 1); mbar_init(bar_acc_empty(i), C::kEpilogueWarps); }
    mbar_init(bar_ep, C::kEpilogueWarps);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The stamps of the scale stages start at zero (a stage is stamped with its super-block number + 1).
  if (threadIdx.x < C::kScl) *reinterpret_cast<uint32_t*>(smem + C::oSclRing + threadIdx.x * C::kSclStage + C::oWide) = 0u;
  // The constant operand: every byte 64.
  for (uint32_t i = threadIdx.x; i < kConstBytes / 4; i += C::kThreads) reinterpret_cast<uint32_t*>(smem + C::oConst)[i] = kConstByte;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == kMmaWarp) tmem_alloc_all(smem_u32(tmem_slot));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t const tmem_base = *tmem_slot;
  // Launched with programmatic stream serialization the block may be running while the launch before it
  // drains.  Weights never depend on that launch.  Everything else does, unless the caller said otherwise
  // (input_settled: activations and residual are older): each role executes griddepcontrol.wait before its first
  // access to such memory -- activations (producer, expanders), outputs, residual, split-K scratch, tickets and
  // the gather's counters (epilogue, at the end of its first tile).  One lane per block waits for the preceding
  // launch on the block's behalf and only then lets the NEXT launch start (launch_dependents): a successor thus
  // never runs beside anything older than its direct predecessor.

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

  if (warp < C::kFirstEpilogue) {
  if constexpr (C::kRebalance) {
    static_assert(C::kFirstEpilogue % 4 == 0 && C::kFirstEpilogue * C::kRegsLow + C::kEpilogueWarps * C::kRegsHigh <= C::kWarps * ((65536 / C::kThreads) / 8 * 8),
                  "the register split must fit the block's allocation");
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::kRegsLow));
  }
  if (warp == kProducerWarp) {
    // One thread feeds both TMA streams: the raw stream (code tiles + metadata of every super-block into the raw
    // ring) and the activation stream (int8 tiles straight into the operand ring).  It polls the two "slot free"
    // barriers without blocking on either, so that neither stream ever waits behind the other.
    if (lane == 0) {
      bool deps_ok = p.input_settled != 0;
      struct Cursor { uint32_t t, kb, kb1, it, row_tile, tok_tile; bool done; };
      auto open_tile = [&](Cursor& c) {
        if (c.t >= num_tiles) { c.done = true; return; }
        uint32_t slice, kb0;
        tile_coords(c.t, c.row_tile, c.tok_tile, slice, kb0, c.kb1);
        c.kb = kb0;
      };
      auto advance = [&](Cursor& c) {
        ++c.it;
        if (++c.kb >= c.kb1) { c.t += gridDim.x; open_tile(c); }
      };
      Cursor ra{blockIdx.x, 0, 0, 0, 0, 0, false}, ac = ra;
      open_tile(ra);
      open_tile(ac);
      long long t_last = clock64();
      uint32_t idle = 0;
      while (!ra.done || !ac.done) {
        bool progressed = false;
        if (!ra.done) {
          uint32_t const r = ra.it % C::kRaw, use = ra.it / C::kRaw;
          if (mbar_test(bar_raw_free(r), (use & 1) ^ 1)) {
            uint8_t* const st = smem + C::oRawRing + r * C::kRawStage;
            uint32_t const bar = bar_raw_full(r);
            int const rg0 = int(ra.row_tile * (kRows / 8));
            mbar_expect_tx(bar, C::kRawTx);
            tma_3d(smem_u32(st + C::oRawCodes), &tm_codes, 0, int(ra.kb), rg0, bar);
            tma_3d(smem_u32(st + C::oRawMeta), &tm_meta, 0, int(ra.kb), rg0, bar);
            advance(ra);
            progressed = true;
          }
        }
        if (!ac.done && !deps_ok && !progressed) {  // the raw ring is full (or done): now the activations are needed
          pdl_wait();
          deps_ok = true;
        }
        if (!ac.done && deps_ok) {
          uint32_t const o = ac.it % C::kOps, use = ac.it / C::kOps;
          if (mbar_test(bar_op_free(o), (use & 1) ^ 1)) {
            uint8_t* const st = smem + C::oOps + o * C::kOpStage;
            uint32_t const bar = bar_b_full(o);
            int const tok0 = int(ac.tok_tile * NTOK);
            mbar_expect_tx(bar, C::kBTx);
            tma_2d(smem_u32(st + C::oB), &tm_act, int(ac.kb) * 256, tok0, bar);
            tma_2d(smem_u32(st + C::oB + NTOK * 128), &tm_act, int(ac.kb) * 256 + 128, tok0, bar);
            advance(ac);
            progressed = true;
          }
        }
        if (progressed) {
          t_last = clock64();
          idle = 0;
        } else if ((++idle & 63u) == 0) {  // bounded like every other wait
          if (*abort_flag) break;
          if (clock64() - t_last > kWaitCycles) {
            *abort_flag = 1;
            atomicExch(p.status, 1);
            break;
          }
        }
      }
      if (*abort_flag) {
        drain(ra.it > C::kRaw ? ra.it - C::kRaw : 0, ra.it, C::kRaw, bar_raw_full(0));
        drain(ac.it > C::kOps ? ac.it - C::kOps : 0, ac.it, C::kOps, bar_b_full(0));
      }
    }
  } else if (warp == C::kDepWarp) {
    // Waits for the launch before this one on the block's behalf (a warp of its own: the wait may last as long as
    // that launch does), then lets the next launch start.
    pdl_wait();
    pdl_launch_dependents();
    // Row-sharded use: the projections that finished before this launch are announced to the peers now (their
    // grids have completed, so their stores into the peers' buffers are visible).
    if (p.done != nullptr && blockIdx.x == 0 && lane == 0) announce_deliveries(p.unsignalled, p.peer_flag, p.ndst, p.rank);
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(NTOK);
      uint64_t const cdesc = umma_desc_sw128(smem_u32(smem + C::oConst), kConstAtomStride);
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        uint32_t row_tile, tok_tile, slice, kb0, kb1;
        tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
        for (uint32_t kb = kb0; ok && kb < kb1; ++kb, ++it) {
          uint32_t const o = it % C::kOps, use = it / C::kOps;
          if (!mbar_wait_inline(bar_b_full(o), use & 1, abort_flag, p.status, 3)) { ok = false; break; }
          if (!mbar_wait_inline(bar_op_ready(o), use & 1, abort_flag, p.status, 4)) { ok = false; break; }
          tc_fence_after();
          uint8_t* const st = smem + C::oOps + o * C::kOpStage;
          uint32_t const a_base = smem_u32(st + C::oAExp), b_base = smem_u32(st + C::oB);
          // Set by set: the constant MMAs of all its buffers first, then the data MMAs, so that an MMA that accumulates
          // on a preset does not queue directly behind the MMA that writes it.
#pragma unroll
          for (uint32_t g0 = 0; g0 < 8; g0 += C::kMmaPerCommit) {
            uint32_t b0, parity;
            acc_slot<C::kAccBufs>(it, g0, b0, parity);
            uint32_t const set = b0 / C::kMmaPerCommit;
            if (!mbar_wait_inline<256, 64>(bar_acc_empty(set), parity ^ 1, abort_flag, p.status, 5)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (uint32_t k = 0; k < C::kMmaPerCommit; ++k) umma_i8(tmem_base + (b0 + k) * NTOK, cdesc, cdesc, idesc, 0);  // every accumulator = 2^17
#pragma unroll
            for (uint32_t k = 0; k < C::kMmaPerCommit; ++k) {
              uint32_t const g = g0 + k;
              uint64_t const ad = umma_desc_sw128(a_base + (g >> 2) * (kRows * 128) + (g & 3) * 32);
              uint64_t const bd = umma_desc_sw128(b_base + (g >> 2) * (NTOK * 128) + (g & 3) * 32);
              umma_i8(tmem_base + (b0 + k) * NTOK, ad, bd, idesc, 1);  // += the K32 dots
            }
            umma_commit(bar_acc_full(set));
          }
          if (ok) umma_commit(bar_op_free(o));  // operands are free once these MMAs have read them
        }
      }
    }
  } else {
    if (!p.input_settled || !C::kHasDepWarp) pdl_wait();  // the activations' scales and sums are read from global memory
    if (!C::kHasDepWarp && warp == kFirstExpander) {
      pdl_launch_dependents();
      if (p.done != nullptr && blockIdx.x == 0 && lane == 0) announce_deliveries(p.unsignalled, p.peer_flag, p.ndst, p.rank);
    }
    uint32_t const et = threadIdx.x - kFirstExpander * 32;  // 0 .. 32*kExpanders-1
    constexpr uint32_t kET = C::kExpanders * 32;
    constexpr uint32_t kEntries = (NTOK * 8 + kET - 1) / kET;  // activation-table entries per thread
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
      uint32_t row_tile, tok_tile, slice, kb0, kb1;
      tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
      uint32_t const tok0 = tok_tile * NTOK;
      for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
        uint32_t const r = it % C::kRaw, o = it % C::kOps, sc = it % C::kScl;
        // The activations' scales and sums of this super-block come straight from global memory (they sit in
        // L2); the loads are in flight while the nibbles are expanded.
        float av[kEntries];
        int sv[kEntries];
#pragma unroll
        for (uint32_t e = 0; e < kEntries; ++e) {
          uint32_t const j = et + e * kET, tk = j >> 3, g = j & 7;
          bool const live = j < NTOK * 8 && tok0 + tk < p.m;
          size_t const idx = size_t(tok0 + tk) * p.G + kb * 8 + g;
          av[e] = live ? __ldg(p.xscales + idx) : 0.f;
          sv[e] = live ? __ldg(p.xsums + idx) : 0;
        }
        if (!mbar_wait_inline<1024, 128>(bar_raw_full(r), (it / C::kRaw) & 1, abort_flag, p.status, 6)) { ok = false; break; }
        if (!mbar_wait_inline<1024, 128>(bar_op_free(o), ((it / C::kOps) & 1) ^ 1, abort_flag, p.status, 7)) { ok = false; break; }
        if (!mbar_wait_inline<1024, 128>(bar_s_free(sc), ((it / C::kScl) & 1) ^ 1, abort_flag, p.status, 8)) { ok = false; break; }
        uint32_t const raw = smem_s + C::oRawRing + r * C::kRawStage;
        uint32_t const ops = smem_s + C::oOps + o * C::kOpStage;
        uint32_t const scl = smem_s + C::oSclRing + sc * C::kSclStage;
        // 1024 raw 16-byte chunks = (row of the tile, K32 group).  A quarter warp takes the eight rows of one
        // 8-row atom, lane i the row i and the group (g0 + i) mod 8: its eight reads and each of its two sets of
        // eight writes fall into eight different 16-byte bank groups.
        // A lane keeps its row-in-atom and its K32 group for the whole walk (octet L takes the units (atom, g0 = L mod 8)
        // with atom = L / 8, + P / 8, ...; P = the octets rounded down to a multiple of eight, the others sit the
        // expansion out): source and destination then advance by a constant, and the loop is loads, logic and stores.
        {
          constexpr uint32_t kOct = kET / 8, P = kOct / 8 * 8;
          uint32_t const i8 = et & 7, L = et >> 3;
          if (L < P) {
            uint32_t const g = ((L & 7) + i8) & 7, c = (g & 3) * 2;
            uint32_t src = raw + C::oRawCodes + (L >> 3) * 1024 + i8 * 128 + g * 16;
            uint32_t dst = ops + C::oAExp + (g >> 2) * (kRows * 128) + (L >> 3) * 1024 + i8 * 128;
            uint32_t const d0 = (c ^ i8) << 4, d1 = ((c + 1) ^ i8) << 4;
#pragma unroll 2
            for (uint32_t atom = L >> 3; atom < 16; atom += P / 8, src += (P / 8) * 1024, dst += (P / 8) * 1024) {
              uint4 const w = lds128(src);
              uint32_t const ww[4] = {w.x, w.y, w.z, w.w};
              uint32_t ov[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint32_t const lo = ww[i] & 0x0f0f0f0fu, hi = (ww[i] >> 4) & 0x0f0f0f0fu;
                ov[2 * i] = __byte_perm(lo, hi, 0x5140);      // columns 8i .. 8i+3
                ov[2 * i + 1] = __byte_perm(lo, hi, 0x7362);  // columns 8i+4 .. 8i+7
              }
              sts128(dst + d0, ov[0], ov[1], ov[2], ov[3]);
              sts128(dst + d1, ov[4], ov[5], ov[6], ov[7]);
            }
          }
        }
        // Row tables: S = d * sc * 2^100 of every (row, group) and -dmin of every row, laid out so that an epilogue
        // lane finds its four rows (l/4, +8, +16, +24 of its lane quarter) in one 16-byte word; the six-bit mins
        // as bf16, one 16-byte row each (the A operand of the min-term MMA).
        for (uint32_t row = et; row < kRows; row += kET) {
          uint4 const cm = lds128(raw + C::oRawMeta + row * 16);
          float const dS = fp16_bits_to_f32(cm.x & 0xffffu) * kRowScalePow, ndmin = -fp16_bits_to_f32(cm.x >> 16);
          ScaleMinWords const sm = decode_scale_min(cm.y, cm.z, cm.w);
          uint32_t const slot = (row >> 5) * 32 + (row & 7) * 4 + ((row >> 3) & 3);
          uint32_t const st = scl + C::oS + slot * 4;
          uint32_t mb[4];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            uint32_t const scw = g < 4 ? sm.sc_lo : sm.sc_hi, mnw = g < 4 ? sm.mn_lo : sm.mn_hi;
            sts32f(st + g * (kRows * 4), dS * float(byte_of(scw, g & 3)));
            uint32_t const mbits = __float_as_uint(float(byte_of(mnw, g & 3))) >> 16;  // a six-bit integer is exact in bf16
            if (g & 1) mb[g >> 1] |= mbits << 16; else mb[g >> 1] = mbits;
          }
          sts128(scl + C::oMt + row * 16, mb[0], mb[1], mb[2], mb[3]);
          sts32f(scl + C::oNd + slot * 4, ndmin);
        }
        // Activation tables: a' = a * 2^49 per (group, token), and a * sum split into three bf16 terms that add up to
        // it exactly (the B operand of the min-term MMA).  A scale so large that a' is not finite stamps the stage,
        // and the epilogue then works from the plain scales.
#pragma unroll
        for (uint32_t e = 0; e < kEntries; ++e) {
          uint32_t const j = et + e * kET, tk = j >> 3, g = j & 7;
          if (j < NTOK * 8) {
            sts32f(scl + C::oAf + (g * C::kAfStride + tk) * 4, av[e] * kTokScalePow);
            // a * sum as three bf16 terms by truncation: each keeps the top eight mantissa bits of what is left, the
            // differences are exact, and the third term has at most eight bits left, so the three add up to it exactly.
            float const as = av[e] * float(sv[e]);
            uint32_t const b0 = __float_as_uint(as) & 0xffff0000u;
            float const r1 = as - __uint_as_float(b0);
            uint32_t const b1 = __float_as_uint(r1) & 0xffff0000u;
            uint32_t const b2 = __float_as_uint(r1 - __uint_as_float(b1));
            uint16_t const t0 = uint16_t(b0 >> 16), t1 = uint16_t(b1 >> 16), t2 = uint16_t(b2 >> 16);
            uint32_t const dst = scl + C::oAsT + tk * 48 + g * 2;
            sts16(dst, t0);
            sts16(dst + 16, t1);
            sts16(dst + 32, t2);
            if (av[e] > kWideAbove) atomicMax(reinterpret_cast<uint32_t*>(smem + C::oSclRing + sc * C::kSclStage + C::oWide), it + 1);
          }
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
  }
  } else {
    if constexpr (C::kRebalance) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kRegsHigh));
    constexpr int GS = C::kGroupSplit, CW = C::kColsPerWarp, NB = CW / 8;
    uint32_t const ep = warp - C::kFirstEpilogue, quarter = warp & 3;  // TMEM lanes 32*quarter ..
    uint32_t const u = ep >> 2, cs = u % C::kColSplit, gs = u / C::kColSplit;
    uint32_t const col0 = cs * CW;
    uint32_t const q = lane & 3, R0 = lane >> 2;
    // This thread's values: v = ((h * NB + j) * 2 + i) * 2 + e  <->  row 32*quarter + 16h + 8i + R0 of the tile,
    // token col0 + 8j + 2q + e of the tile.
    bool const final_warp = gs == 0;               // holds the tile's sums after the group-split reduction
    uint32_t it = 0, ep_phase = 0;
    bool ok = true;
    bool deps_ok = !p.input_settled || Dump;  // otherwise the wait comes at the end of the first tile
    if (deps_ok) pdl_wait();
    auto ep_sync = [&](int code) {  // all epilogue warps meet (bounded like every other wait)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ep);
      if (!mbar_wait_inline(bar_ep, ep_phase, abort_flag, p.status, code)) ok = false;
      ep_phase ^= 1;
    };
    // The accumulator patches are read one half (16 TMEM lanes) at a time into two register buffers, and the read of
    // the next half -- of the same group, of this warp's next group, or of the next super-block's first -- is always
    // in flight while the current half is folded: tcgen05.ld has a latency of several hundred cycles, and four
    // epilogue warps per scheduler cannot hide it by themselves.
    uint32_t const lane_base = tmem_base + ((quarter * 32u) << 16) + col0;
    // A unit = this warp's 32 rows x (8 * UB) tokens of one K32 group, read as two 16-lane halves.  The reads of the
    // next unit -- of the same group, of the warp's next group, or of the next super-block's first -- are in flight
    // while a unit is folded (two buffers, used alternately): tcgen05.ld has a latency of a hundred cycles and
    // more under load, tcgen05.wait::ld waits for everything outstanding, and a unit's arithmetic is short.
    constexpr int UB = NB >= 2 ? 2 : 1, U = NB / UB;  // column blocks per unit, units per group
    uint32_t bufA[2][4 * UB], bufB[2][4 * UB];
    constexpr int PER = C::kMmaPerCommit / GS;  // groups of this warp per accumulator set
    // Issues the reads of unit u of group g2 of super-block it2; first waits for the group's accumulator set when asked.
    auto fetch_unit = [&](uint32_t (&dst)[2][4 * UB], uint32_t it2, uint32_t g2, int u, bool wait_set) -> bool {
      uint32_t b2, parity2;
      acc_slot<C::kAccBufs>(it2, g2, b2, parity2);
      if (wait_set) {
        if (!mbar_wait_inline<512, 128>(bar_acc_full(b2 / C::kMmaPerCommit), parity2, abort_flag, p.status, 10)) return false;
        tc_fence_after();
      }
      uint32_t const ta = lane_base + b2 * NTOK + 8 * UB * u;
      tmem_ld_frag<UB>(ta, dst[0]);
      tmem_ld_frag<UB>(ta + (16u << 16), dst[1]);
      return true;
    };
    if (blockIdx.x < num_tiles) ok = fetch_unit(bufA, 0, gs, 0, true);
    for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
      uint32_t row_tile, tok_tile, slice, kb0, kb1;
      tile_coords(t, row_tile, tok_tile, slice, kb0, kb1);
      uint32_t const row0 = row_tile * kRows + quarter * 32 + R0, tok0 = tok_tile * NTOK + col0 + 2 * q;
      float2 acc[2][NB][2];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < NB; ++j) acc[h][j][0] = acc[h][j][1] = make_float2(0.f, 0.f);

      for (uint32_t kb = kb0; ok && kb < kb1; ++kb, ++it) {
        uint32_t const sc = it % C::kScl;
        bool const has_next = kb + 1 < kb1 || t + gridDim.x < num_tiles;
        if (!mbar_wait_inline<512, 128>(bar_s_full(sc), (it / C::kScl) & 1, abort_flag, p.status, 9)) { ok = false; break; }
        uint32_t const scl = smem_s + C::oSclRing + sc * C::kSclStage;
        bool const wide = lds32(scl + C::oWide) == it + 1;
        uint32_t const ssp = scl + C::oS + (quarter * 8 + R0) * 16;  // this lane's four row scales of group g: + g * 512
        uint32_t const afp = scl + C::oAf + (col0 + 2 * q) * 4;      // a' of tokens col0 + 8j + 2q, +1 of group g: + g * NTOK * 4 + 32 j
        // ---- min term of the whole super-block on the tensor cores: rows x groups (six-bit mins, bf16) times
        // groups x tokens (a * sum in three bf16 terms; products exact, fp32 accumulation), scaled by -dmin.
        // (Where the groups are split over several warps, the first of them adds it.)
        if (GS == 1 || gs == 0) {
          uint32_t const mrow = scl + C::oMt + (quarter * 32 + R0) * 16 + q * 4;
          uint32_t const am00 = lds32(mrow), am01 = lds32(mrow + 8 * 16), am10 = lds32(mrow + 16 * 16), am11 = lds32(mrow + 24 * 16);
          float4 const nd4 = lds128f(scl + C::oNd + (quarter * 8 + R0) * 16);
          float2 const nd2[4] = {make_float2(nd4.x, nd4.x), make_float2(nd4.y, nd4.y), make_float2(nd4.z, nd4.z), make_float2(nd4.w, nd4.w)};
#pragma unroll
          for (int j = 0; j < NB; ++j) {
            uint32_t const brow = scl + C::oAsT + (col0 + 8 * j + R0) * 48 + q * 4;
            uint32_t const b0 = lds32(brow), b1 = lds32(brow + 16), b2 = lds32(brow + 32);
            float m0[4], m1[4];
            mma_bf16_first(m0, am00, am01, am00, am01, b2, 0u);
            mma_bf16_first(m1, am10, am11, am10, am11, b2, 0u);
            mma_bf16(m0, am00, am01, am00, am01, b0, b1);
            mma_bf16(m1, am10, am11, am10, am11, b0, b1);
#pragma unroll
            for (int i2 = 0; i2 < 2; ++i2) {
              acc[0][j][i2] = __ffma2_rn(nd2[i2], make_float2(m0[2 * i2], m0[2 * i2 + 1]), acc[0][j][i2]);
              acc[1][j][i2] = __ffma2_rn(nd2[2 + i2], make_float2(m1[2 * i2], m1[2 * i2 + 1]), acc[1][j][i2]);
            }
          }
        }
        // ---- one K32 group: tt-th group of this warp in the super-block.  With tt known at compile time (the
        // unrolled fast path) every decision about sets and successors is static and each TMEM read has one site.
        auto group = [&](bool const slow, int const tt) -> bool {
          uint32_t const g = gs + GS * tt;
          bool const last_of_set = (tt % PER) == PER - 1;
          uint32_t b, parity;
          acc_slot<C::kAccBufs>(it, g, b, parity);
          float4 const S4 = lds128f(ssp + g * (kRows * 4));
          float const Sr[4] = {S4.x, S4.y, S4.z, S4.w};
          float const kc = slow ? -0x1p-43f : kBiasOut;
          bool got = true;
          auto unit = [&](uint32_t (&cur)[2][4 * UB], uint32_t (&nxt)[2][4 * UB], int const u) {
            // The token-side operands first: their shared-memory latency passes under the wait for TMEM.
            float2 A[UB], Cc[UB];  // a' and c' of tokens col0 + 8j + 2q, +1 of this unit's column blocks j
#pragma unroll
            for (int jj = 0; jj < UB; ++jj) A[jj] = lds64f(afp + g * (C::kAfStride * 4) + 32 * (u * UB + jj));
            if (slow) {  // plain scales from global memory; the accumulator words are scaled by 2^89 first instead
#pragma unroll
              for (int jj = 0; jj < UB; ++jj) {
                uint32_t const tk = tok0 + 8 * (u * UB + jj);
                A[jj].x = tk < p.m ? p.xscales[size_t(tk) * p.G + kb * 8 + g] : 0.f;
                A[jj].y = tk + 1 < p.m ? p.xscales[size_t(tk + 1) * p.G + kb * 8 + g] : 0.f;
              }
            }
#pragma unroll
            for (int jj = 0; jj < UB; ++jj) Cc[jj] = __fmul2_rn(A[jj], make_float2(kc, kc));
            tmem_wait_ld();  // this unit has arrived
            if (u == U - 1) {
              // with its last unit the warp has read all it wants of this group
              if (last_of_set) {  // the set goes back to the MMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty(b / C::kMmaPerCommit));
              }
              if (tt + 1 < 8 / GS) got = fetch_unit(nxt, it, g + GS, 0, last_of_set);
              else if (has_next) got = fetch_unit(nxt, it + 1, gs, 0, true);
            } else {
              fetch_unit(nxt, it, g, u + 1, false);
            }
            // All first FMAs (a * P * 2^-60), then all second ones (+ (D * 2^60) * that): no FMA waits for its predecessor.
            float2 v[2][2][UB];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int i2 = 0; i2 < 2; ++i2)
#pragma unroll
                for (int jj = 0; jj < UB; ++jj) {
                  float2 w = as_f2(cur[h][4 * jj + 2 * i2], cur[h][4 * jj + 2 * i2 + 1]);
                  if (slow) w = __fmul2_rn(w, make_float2(kTokScalePow, kTokScalePow));
                  v[h][i2][jj] = __ffma2_rn(w, A[jj], Cc[jj]);
                }
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int i2 = 0; i2 < 2; ++i2) {
                float2 const s2 = make_float2(Sr[2 * h + i2], Sr[2 * h + i2]);
#pragma unroll
                for (int jj = 0; jj < UB; ++jj) acc[h][u * UB + jj][i2] = __ffma2_rn(s2, v[h][i2][jj], acc[h][u * UB + jj][i2]);
              }
            if (Dump) {
#pragma unroll
              for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int v = 0; v < 4 * UB; ++v) {
                  uint32_t const row = row0 + 16 * h + 8 * ((v >> 1) & 1), token = tok0 + 8 * (u * UB + (v >> 2)) + (v & 1);
                  if (row < p.n && token < p.m)
                    p.partials[(uint64_t(token) * p.n + row) * p.G + kb * 8 + g] = int32_t(cur[h][v] - kPreset);
                }
            }
          };
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (((tt * U + u) & 1) == 0) unit(bufA, bufB, u); else unit(bufB, bufA, u);
          }
          return got;
        };
        if (!wide) {
#pragma unroll
          for (int tt = 0; tt < 8 / GS; ++tt)
            if (ok && !group(false, tt)) ok = false;
        } else {
#pragma unroll 1
          for (int tt = 0; tt < 8 / GS; ++tt)
            if (ok && !group(true, tt)) ok = false;
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_free(sc));
      }
      if (!ok) break;

      // ---- end of tile: combine the group-split warps, then write (or hand to the split-K fix-up)
      if (!deps_ok) {  // outputs, residual, scratch and tickets may still belong to the launch before this one
        pdl_wait();
        deps_ok = true;
      }
      auto value = [&](int v) -> float& {
        float2& a2 = acc[v / (4 * NB)][(v / 4) % NB][(v >> 1) & 1];
        return (v & 1) ? a2.y : a2.x;
      };
      auto row_of = [&](int v) { return row0 + 16 * (v / (4 * NB)) + 8 * ((v >> 1) & 1); };
      auto token_of = [&](int v) { return tok0 + 8 * ((v / 4) % NB) + (v & 1); };
      if constexpr (GS > 1) {
#pragma unroll
        for (int v = 0; v < CW; ++v) red[(ep * CW + v) * 32 + lane] = value(v);
        ep_sync(11);
        if (!ok) break;
        if (final_warp) {
#pragma unroll
          for (int v = 0; v < CW; ++v) {
            float sum = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < GS; ++k2) sum += red[((ep + 4 * C::kColSplit * k2) * CW + v) * 32 + lane];  // warp order
            value(v) = sum;
          }
        }
      }
      auto store = [&](uint32_t token, uint32_t row, float v) {
        uint64_t const o = uint64_t(token) * p.out_stride + p.out_row0 + row;
        if (p.residual) v += p.residual[o];
        if (p.out_bf16) {
          p.out_bf16[o] = f32_to_bf16_rne(v);
        } else {
          p.out[0][o] = v;
#pragma unroll
          for (int g2 = 1; g2 < 8; ++g2)
            if (g2 < int(p.ndst)) p.out[g2][o] = v;
        }
      };
      if (p.split_k == 1) {
        if (final_warp) {
#pragma unroll
          for (int v = 0; v < CW; ++v)
            if (row_of(v) < p.n && token_of(v) < p.m) store(token_of(v), row_of(v), value(v));
        }
      } else {
        uint64_t const plane = uint64_t(p.m) * p.n;
        if (final_warp) {
#pragma unroll
          for (int v = 0; v < CW; ++v)
            if (row_of(v) < p.n && token_of(v) < p.m)
              __stcg(p.partial_tiles + slice * plane + uint64_t(token_of(v)) * p.n + row_of(v), value(v));
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
          if (final_warp) {
            // Slices are added in slice order; all of a slice's values are requested before any is used, so the
            // reads of a slice are in flight together (one memory latency per slice, not per value).
            float sum[CW];
#pragma unroll
            for (int v = 0; v < CW; ++v) sum[v] = 0.f;
            for (uint32_t s2 = 0; s2 < p.split_k; ++s2) {
              float part[CW];
#pragma unroll
              for (int v = 0; v < CW; ++v)
                part[v] = (row_of(v) < p.n && token_of(v) < p.m) ? __ldcg(p.partial_tiles + s2 * plane + uint64_t(token_of(v)) * p.n + row_of(v)) : 0.f;
#pragma unroll
              for (int v = 0; v < CW; ++v) sum[v] += part[v];
            }
#pragma unroll
            for (int v = 0; v < CW; ++v)
              if (row_of(v) < p.n && token_of(v) < p.m) store(token_of(v), row_of(v), sum[v]);
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

  // Teardown: everyone meets (a read of TMEM still in flight after an early exit lands first), TMEM goes back.
  if (warp >= C::kFirstEpilogue) tmem_wait_ld();
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc_all(tmem_base);
  }
  // Row-sharded use: the last block of the grid records one more finished projection.  It is announced to the
  // peers by the next kernel of the stream, once this grid has completed and its peer stores are visible.
  if (p.done != nullptr && threadIdx.x == 0) {
    __threadfence();
    uint32_t const old = atomicAdd(p.done, 1u);
    if (old == gridDim.x - 1) {
      *p.done = 0;
      if (*reinterpret_cast<volatile int*>(p.status) == 0) atomicAdd(p.unsignalled, 1u);
    }
  }
}

// ------------------------------------------------------------------------------------------
template <int NTOK, int NCOL>
cudaError_t launch_ntok(const WeightView& w, const Q8View& x, const TcOutput& o, int32_t* partials,
                        uint32_t split_k, float* partial_tiles, uint32_t* tickets, int* status, cudaStream_t stream) {
  using C = Cfg<NTOK, NCOL>;
  CUtensorMap tm_codes, tm_meta, tm_act;
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
  auto kernel = partials ? mmq_tcgen05_kernel<NTOK, NCOL, true> : mmq_tcgen05_kernel<NTOK, NCOL, false>;
  cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (st != cudaSuccess) return st;
  uint32_t const row_tiles = (w.padded_n + kRows - 1) / kRows, tok_tiles = (x.m + NTOK - 1) / NTOK;
  TcParams p{};
  p.xscales = x.scales; p.xsums = x.sums;
  p.residual = o.residual;
  for (uint32_t g = 0; g < 8; ++g) p.peer_flag[g] = g < o.ndst ? o.flags[g] : nullptr;
  p.done = o.done; p.unsignalled = o.unsignalled; p.rank = o.rank;
  for (uint32_t g = 0; g < 8; ++g) p.out[g] = g < o.ndst ? o.out[g] : nullptr;
  p.out_bf16 = o.out_bf16; p.ndst = o.ndst; p.out_stride = o.stride ? o.stride : w.n; p.out_row0 = o.row0;
  p.partials = partials; p.partial_tiles = partial_tiles; p.tickets = tickets; p.status = status;
  p.input_settled = o.input_settled;
  p.n = w.n; p.m = x.m; p.tiles_k = w.tiles_k; p.split_k = split_k; p.G = uint32_t(G); p.row_tiles = row_tiles; p.tok_tiles = tok_tiles;
  uint64_t const tiles = uint64_t(row_tiles) * tok_tiles * split_k;
  uint32_t const grid = uint32_t(tiles < uint64_t(sm_count()) ? tiles : uint64_t(sm_count()));
  return launch_kernel(kernel, grid, C::kThreads, C::kSmem, stream, launch_overlap(), tm_codes, tm_meta, tm_act, p);
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
    // Pick the K split with the shortest estimated time, in units of one super-block step of a block: a block
    // pays its pipeline fill once, and per tile the K walk plus the tile end (longer with split-K: partial tiles
    // go through global scratch and the last block of a tile adds them).  Measured on 64-token tiles: fill ~1.7,
    // tile end ~1, split-K tile end ~2.5 steps.  Slices keep at least four super-blocks.  With launch overlap on,
    // SMs a launch leaves idle are taken by the next launch, so splitting K to fill them buys less: the extra
    // tile ends are then charged at 5 steps (measured on the 64-layer stream: 4 to 8 give the same plans, and
    // 7 % more throughput than 2.5; 12 and "never split" lose).
    uint32_t const sms = uint32_t(sm_count());
    double const split_end = launch_overlap() ? 5.0 : 2.5;
    uint32_t const max_split = tiles_k / 4 ? (tiles_k / 4 > 16 ? 16 : tiles_k / 4) : 1;
    double best = 1e30;
    split = 1;
    for (uint32_t s = 1; s <= max_split; ++s) {
      uint64_t const tiles = uint64_t(blocks) * s;
      uint64_t const rounds = (tiles + sms - 1) / sms;
      double const cost = 1.7 + double(rounds) * ((s > 1 ? split_end : 1.0) + double((tiles_k + s - 1) / s));
      if (cost < best - 1e-9) { best = cost; split = s; }
    }
  }
  if (split > tiles_k) split = tiles_k;
  if (split < 1) split = 1;
  p.split_k = split;
  return p;
}

cudaError_t launch_mmq_tcgen05(const WeightView& w, const Q8View& x, const TcOutput& out, int32_t* partials,
                               const TcPlan& plan, void* partial_tiles, uint32_t* tickets, int* status, cudaStream_t stream) {
  float* pt = static_cast<float*>(partial_tiles);
  if (out.ndst < 1 || out.ndst > 8 || (out.out_bf16 ? out.ndst != 1 : out.out[0] == nullptr)) return cudaErrorInvalidValue;
  switch (plan.ntok) {
    case 16:
      if (x.m <= 8) return launch_ntok<16, 8>(w, x, out, partials, plan.split_k, pt, tickets, status, stream);
      return launch_ntok<16, 16>(w, x, out, partials, plan.split_k, pt, tickets, status, stream);
    case 32: return launch_ntok<32, 32>(w, x, out, partials, plan.split_k, pt, tickets, status, stream);
    case 64: return launch_ntok<64, 64>(w, x, out, partials, plan.split_k, pt, tickets, status, stream);
    case 128: return launch_ntok<128, 128>(w, x, out, partials, plan.split_k, pt, tickets, status, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace q4k
