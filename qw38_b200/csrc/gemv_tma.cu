// Decode projection (m <= 16) with the activations held in registers and the weights streamed
// through shared memory by TMA.
//
// The 4-bit weights are read exactly once and are the only large operand, so the kernel is
// built around keeping many weight bytes in flight per SM with no instruction cost: one
// producer lane issues two bulk tensor copies per stage (code tiles with the 128-byte swizzle,
// metadata tiles) into a ring that holds most of shared memory.  The work is laid out
// "K-stationary": consumer warp w owns super-block column sb0 + w of the block's K slice for
// the whole kernel and keeps what depends on (token, K) with it -- the int8 activation fragments
// of its eight K32 groups and a * sum split into three tf32 terms in registers, the activation
// scale pairs in a table of its own in shared memory -- while the block walks down its range of
// 16-row tiles.  Per tile a consumer
//   * decodes the 16 rows' six-bit scales/mins of its super-block into a small float table,
//   * ldmatrix's the swizzled code tile into mma A fragments (nibbles -> u8 by mask/shift),
//   * issues one m16n8k32 u8*s8 MMA per K32 group and token octet whose accumulator input is the
//     bit pattern of 1.5*2^23, so the int32 result *is* the float 1.5*2^23 + dot (exact, |dot| <
//     2^22) and no int->float conversion is issued,
//   * folds  a * (sc * dot)  with two packed fp32 FMAs per pair of partials, and the min term
//     sum_g mn[row,g] * (a*sum)[tok,g] with three m16n8k8 tf32 MMAs (mn is a 6-bit integer and the
//     three tf32 terms add up to the fp32 value exactly, so the products are exact),
//   * scales by d / dmin and hands its 16 x 8 partial tile per token octet to that octet's reducer warp,
//     which adds the consumers' tiles in warp order and writes the rows (or the K slice's scratch tile).
// K slices of different blocks are added in slice order by the last block to finish a row range
// (arrival ticket), as in the other split-K kernels of this library.
//
// One launch may walk up to three weights that share the activations (ranges of one matrix, Q/K/V), each
// with its own destination and epilogue applied by the reducer (fp32 or bf16 store, residual added last); for
// a gate / up pair the tiles of the two weights alternate through the blocks and the reducer writes
// bf16(SiLU(gate) * up), or -- for the MLP chain -- quantises that product on the spot into the Q8 codes,
// scales and sums of the down projection's input (two tile pairs = one group of 32 rows per token).
//
// Launched with programmatic stream serialization (launch.h), the producer streams weights while
// the previous kernel of the stream is still draining; the reducers wait for that kernel first and only
// then release the next launch; the consumers wait for it before they load activations unless the caller
// flagged the input as settled (not the work of the launch directly before).  Row-sharded use (GemvTmaGather): the reducers store each value into every rank's copy
// of the gathered output with plain peer stores, and the last block counts the projection as
// finished; the count is announced to the peers by the next kernel of the stream.
//
// Contract notes (reference: cuda/q4k_q8.cu:63-112, mmvq): the int32 dot of a K32 group is exact
// and never carried into the next group; scales stay fp32.  Every mbarrier wait is bounded.
#include <cuda.h>

#include "common.cuh"
#include "launch.h"
#include "tma.cuh"

namespace q4k {
namespace {

constexpr uint32_t kMagicI = 0x4B400000u;  // bit pattern of 1.5 * 2^23
constexpr float kMagicF = 12582912.0f;
constexpr int kProducer = 0, kFirstReducer = 1;  // then NT reducer warps, then the consumers
// Per consumer warp: 16 rows of 112 bytes -- 64 of scale pairs, 32 of mins, 16 of {d, d, -dmin, -dmin}; the
// stride of 28 words puts the eight rows a load touches in different banks -- then NT * 256 bytes of
// activation scale pairs.
constexpr int kTabRow = 112, kTabMn = 64, kTabDd = 96, kTabBytes = 16 * kTabRow;
constexpr int kMaxStages = 8;

// One weight of a multi-weight launch: its destination (fp32, or bf16 rounded to nearest even), its optional residual
// ([m][n] like the destination), its rows, its 16-row tiles and its first row in the concatenated split-K scratch.
struct GtSegment {
  float* out;
  uint16_t* out_bf16;
  const float* residual;
  uint32_t n, tiles, row_base;
};

struct GtParams {
  const int8_t* xcodes;
  const float* xscales;
  const int32_t* xsums;
  const float* residual;      // same geometry as the destinations
  float* out[8];              // destinations: one buffer, or every rank's copy of the gathered output
  uint32_t* peer_flag[8];     // gather only: rank g's arrival counters (uint32[8]); [rank] counts this rank's deliveries
  uint32_t* done;             // gather only: block counter of this launch, zero on entry and on exit
  uint32_t* unsignalled;      // gather only: finished projections of this rank not yet announced to the peers
  uint32_t ndst, rank;        // number of destinations; this rank
  uint32_t out_stride, out_row0;  // destination element of (token, row) = token * out_stride + out_row0 + row
  int32_t* partials;  // optional int32 K32 dots [m][n][G]
  float* slices;      // split-K scratch [slice][m][n]
  uint32_t* tickets;  // one per row range, zero on entry and on exit
  int* status;
  uint32_t n, m, padded_k, tiles_k, G;
  uint32_t row_tiles;        // 16-row tiles
  uint32_t cw;               // consumer warps = super-blocks per K slice
  uint32_t split_k, tiles_per_range, stages;
  uint32_t red_slots;        // 1 or 2 hand-off buffers between the consumers and the reducer
  // General form (one launch over up to three weights that share x, each with its own epilogue; or a gate / up pair
  // whose 16-row tiles alternate and whose result is bf16(SiLU(gate) * up)).  nseg == 0: the plain form above.
  GtSegment seg[3];
  uint32_t nseg, pair, n_total;  // n_total: rows of all segments = row stride of the split-K scratch
  uint32_t input_settled;        // activations were complete before the preceding launch was enqueued
  // pair == 2: the gate / up pair's result is not stored as bf16 but quantised on the spot: Q8 codes, scales and sums
  // of x = bf16(silu(gate) * up), 32 consecutive rows (two 16-row tiles) per group, as swiglu_pack would produce.
  int8_t* q8_codes;
  float* q8_scales;
  int32_t* q8_sums;
  int* q8_failure;
  uint32_t q8_pk;                // row stride of the codes = padded row count of the pair
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D = A(u8, 16x32) * B(s8, 32x8) + C.  C is a block of four registers that the caller fills once
// and keeps alive, so that no per-MMA moves are needed to build the accumulator input.
__device__ __forceinline__ void mma_u8s8(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const uint32_t (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t to_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 as_f2(uint32_t x, uint32_t y) { return make_float2(__uint_as_float(x), __uint_as_float(y)); }

// sigmoid / SiLU as the reference's decode epilogue states them (cuda/decode_mmv.cu:78-89): the exponential is
// always taken of a non-positive number.
__device__ __forceinline__ float silu_fp32(float u) {
  float const e = expf(u >= 0.0f ? -u : u);
  return u * (u >= 0.0f ? 1.0f / (1.0f + e) : e / (1.0f + e));
}
// Which weight a global tile index of a multi-weight launch belongs to, and the tile's index inside it.
__device__ __forceinline__ void locate_tile(const GtParams& p, uint32_t T, uint32_t& s, uint32_t& local) {
  if (p.pair) { s = T & 1u; local = T >> 1; return; }
  s = 0; local = T;
  if (p.nseg > 1 && local >= p.seg[0].tiles) {
    local -= p.seg[0].tiles; s = 1;
    if (p.nseg > 2 && local >= p.seg[1].tiles) { local -= p.seg[1].tiles; s = 2; }
  }
}

// NT = token octets (1: m <= 8, 2: m <= 16).  MAXW bounds the block size for register allocation.
template <int NT, int MAXW, bool Dump>
__global__ void __launch_bounds__(MAXW * 32, 1)
gemv_tma_kernel(const __grid_constant__ CUtensorMap tm_codes, const __grid_constant__ CUtensorMap tm_meta,
                const __grid_constant__ CUtensorMap tm_codes1, const __grid_constant__ CUtensorMap tm_meta1,
                const __grid_constant__ CUtensorMap tm_codes2, const __grid_constant__ CUtensorMap tm_meta2, const GtParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint32_t const smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint32_t const cw = p.cw, stages = p.stages;
  uint32_t const code_stage = cw * 2048, meta_stage = cw * 256;
  uint32_t const s_codes = smem;
  uint32_t const s_meta = s_codes + stages * code_stage;
  uint32_t const s_tab = s_meta + stages * meta_stage;
  uint32_t const tab_bytes = kTabBytes + NT * 256;
  uint32_t const s_red = s_tab + cw * tab_bytes;
  uint32_t const red_slot = cw * NT * 512;
  // barriers: full[stages] empty[stages] red_full[2] red_empty[2], then the abort and "last block" flags
  uint32_t const b_full = s_red + p.red_slots * red_slot, b_empty = b_full + 8 * stages, b_rfull = b_empty + 8 * stages, b_rempty = b_rfull + 16;
  int* const flags = reinterpret_cast<int*>(smem_raw + (b_rempty + 16 - smem_u32(smem_raw)));
  volatile int* const abort_flag = flags;
  int* const last_flag = flags + 1;

  constexpr uint32_t kFirstConsumer = kFirstReducer + NT;
  uint32_t const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t const slot_mask = p.red_slots - 1, slot_shift = p.red_slots - 1;  // red_slots is 1 or 2
  uint32_t const range = blockIdx.x / p.split_k, slice = blockIdx.x % p.split_k;
  uint32_t const sb0 = slice * cw;
  uint32_t const nact = min(cw, p.tiles_k - sb0);  // consumer warps with a real super-block
  uint32_t const t0 = range * p.tiles_per_range;
  uint32_t const t1 = min(p.row_tiles, t0 + p.tiles_per_range);
  uint32_t const ntiles = t1 > t0 ? t1 - t0 : 0;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < stages; ++s) {
      mbar_init(b_full + 8 * s, 1);
      mbar_init(b_empty + 8 * s, nact * 32);
    }
    for (uint32_t s = 0; s < 2; ++s) {
      mbar_init(b_rfull + 8 * s, nact * 32);
      mbar_init(b_rempty + 8 * s, 32 * NT);
    }
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // The producer streams weights at once: they are constant, whatever kernel runs before this
  // one.  Every other role first waits for the preceding kernel of the stream, because the
  // activations, the residual, the output and the split-K scratch may be its to write.
  if (warp == kProducer) {
    if (lane == 0) {
      uint32_t s = 0, ph = 1;  // the first pass over the ring finds every stage free
      for (uint32_t it = 0; it < ntiles; ++it) {
        if (it >= stages && !mbar_wait(b_empty + 8 * s, ph, abort_flag, p.status, 0x510)) break;
        mbar_expect_tx(b_full + 8 * s, code_stage + meta_stage);
        const CUtensorMap* mc = &tm_codes;
        const CUtensorMap* mm = &tm_meta;
        uint32_t local = t0 + it;
        if (p.nseg > 1) {
          uint32_t sg;
          locate_tile(p, t0 + it, sg, local);
          if (sg == 1) { mc = &tm_codes1; mm = &tm_meta1; }
          if (sg == 2) { mc = &tm_codes2; mm = &tm_meta2; }
        }
        int const rg = int(local * 2);
        tma_3d(s_codes + s * code_stage, mc, 0, int(sb0 * 8), rg, b_full + 8 * s);
        tma_3d(s_meta + s * meta_stage, mm, 0, int(sb0), rg, b_full + 8 * s);
        if (++s == stages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp < kFirstConsumer) {
    // One reducer warp per token octet adds the consumers' 16 x 8 tiles in warp order.  Lane
    // (r = lane/4, q = lane%4) owns rows r, r+8 and tokens 2q, 2q+1 -- the MMA accumulator layout.
    uint32_t const nt = warp - kFirstReducer;
    uint32_t const r = lane >> 2, q = lane & 3;
    pdl_wait();
    pdl_launch_dependents();  // after the wait: the next launch never runs beside anything older than this one
    if (p.done != nullptr && blockIdx.x == 0 && warp == kFirstReducer && lane == 0) announce_deliveries(p.unsignalled, p.peer_flag, p.ndst, p.rank);
    // Destination of this warp's values: the K slice's scratch tile, or the output (one buffer, or every
    // rank's copy of the gathered output).  Offsets are those of (tok0, row 0).
    bool const to_slices = p.split_k > 1;
    float* const dst = to_slices ? p.slices + size_t(slice) * p.m * p.n : p.out[0];
    const float* const res = to_slices ? nullptr : p.residual;
    uint32_t const extra = to_slices ? 0u : p.ndst - 1;   // further destinations (row-sharded gather)
    uint32_t const tok0 = nt * 8 + q * 2;
    bool const live0 = tok0 < p.m, live1 = tok0 + 1 < p.m;
    size_t const o0 = to_slices ? size_t(tok0) * p.n : size_t(tok0) * p.out_stride + p.out_row0;
    size_t const o1 = o0 + (to_slices ? p.n : p.out_stride);
    if (p.nseg != 0) {
      // General form: every tile belongs to one of up to three weights with its own destination and epilogue; in
      // pair mode the even tiles are the gate's, the odd ones the up projection's, and bf16(SiLU(gate) * up) is
      // written once both are known.  Same hand-off and summation order as the plain form below.
      float g00 = 0.f, g01 = 0.f, g10 = 0.f, g11 = 0.f;
      float px[4] = {0.f, 0.f, 0.f, 0.f};  // pair == 2: the values of the group's first tile
      for (uint32_t it = 0; it < ntiles; ++it) {
        uint32_t const s = it & slot_mask, use = it >> slot_shift;
        if (!mbar_wait(b_rfull + 8 * s, use & 1, abort_flag, p.status, 0x520)) break;
        float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
        uint32_t src = s_red + s * red_slot + nt * 512 + lane * 16;
#pragma unroll 4
        for (uint32_t w = 0; w < nact; ++w) {
          float4 const v = lds128f(src);
          lo = __fadd2_rn(lo, make_float2(v.x, v.y));
          hi = __fadd2_rn(hi, make_float2(v.z, v.w));
          src += NT * 512;
        }
        mbar_arrive(b_rempty + 8 * s);
        uint32_t sg, local;
        locate_tile(p, t0 + it, sg, local);
        const GtSegment& S = p.seg[sg];
        uint32_t const row = local * 16 + r;
        bool const in0 = row < S.n, in1 = row + 8 < S.n;
        float v00 = lo.x, v01 = lo.y, v10 = hi.x, v11 = hi.y;
        if (to_slices) {  // K slice: plain partial sums, rows of all weights side by side
          float* const d0 = p.slices + (size_t(slice) * p.m + tok0) * p.n_total + S.row_base + row;
          float* const d1 = d0 + p.n_total;
          if (in0 && live0) d0[0] = v00;
          if (in0 && live1) d1[0] = v01;
          if (in1 && live0) d0[8] = v10;
          if (in1 && live1) d1[8] = v11;
          continue;
        }
        size_t const a0 = size_t(tok0) * S.n + row, a1 = a0 + S.n;
        if (p.pair) {
          if (sg == 0) { g00 = v00; g01 = v01; g10 = v10; g11 = v11; continue; }
          if (p.pair == 2) {
            // The activation of the down projection, quantised here (the arithmetic of swiglu_pack_kernel,
            // cuda/q4k_q8.cu:52-61): x = bf16(g / (1 + exp(-g)) * u), a non-finite input poisons the value.
            auto act = [](float gv, float uv) {
              float v = (gv / (1.f + expf(-gv))) * uv;
              if (!isfinite(gv) || !isfinite(uv)) v = __int_as_float(0x7fc00000);
              return bf16_bits_to_f32(f32_to_bf16_rne(v));
            };
            float const cx[4] = {act(g00, v00), act(g01, v01), act(g10, v10), act(g11, v11)};  // (row r | r+8) x (token 0 | 1)
            if ((local & 1u) == 0) {
#pragma unroll
              for (int i = 0; i < 4; ++i) px[i] = cx[i];
              continue;
            }
            // Second tile of a 32-row group: this lane holds rows r, r+8, 16+r, 24+r of the group for two tokens; the
            // eight lanes with the same q hold the rest.
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float const xv[4] = {px[e], px[2 + e], cx[e], cx[2 + e]};
              bool finite = true;
              float peak = 0.f;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                bool const f = isfinite(xv[i]);
                finite = finite && f;
                peak = fmaxf(peak, f ? fabsf(xv[i]) : 0.f);
              }
              int fin = finite ? 1 : 0;
#pragma unroll
              for (int off = 4; off < 32; off <<= 1) {
                peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, off));
                fin &= __shfl_xor_sync(0xffffffffu, fin, off);
              }
              float const a = peak == 0.f ? 1.f : __fdiv_rn(peak, 127.f);
              bool const valid = fin && isfinite(a) && a > 0.f;
              int z[4], sum = 0;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                z[i] = valid ? max(-127, min(127, __float2int_rn(__fdiv_rn(xv[i], a)))) : 0;
                sum += z[i];
              }
#pragma unroll
              for (int off = 4; off < 32; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
              uint32_t const tok = tok0 + e;
              if (tok < p.m) {
                int8_t* const c = p.q8_codes + size_t(tok) * p.q8_pk + (local - 1) * 16 + r;
                c[0] = int8_t(z[0]); c[8] = int8_t(z[1]); c[16] = int8_t(z[2]); c[24] = int8_t(z[3]);
                if (r == 0) {
                  size_t const gi = size_t(tok) * (p.q8_pk / 32) + (local >> 1);
                  p.q8_scales[gi] = valid ? a : __int_as_float(0x7fc00000);
                  p.q8_sums[gi] = sum;
                  if (!valid) atomicExch(p.q8_failure, 1);
                }
              }
            }
            continue;
          }
          uint16_t* const ob = p.seg[0].out_bf16;
          if (in0 && live0) ob[a0] = f32_to_bf16_rne(silu_fp32(g00) * v00);
          if (in0 && live1) ob[a1] = f32_to_bf16_rne(silu_fp32(g01) * v01);
          if (in1 && live0) ob[a0 + 8] = f32_to_bf16_rne(silu_fp32(g10) * v10);
          if (in1 && live1) ob[a1 + 8] = f32_to_bf16_rne(silu_fp32(g11) * v11);
          continue;
        }
        if (S.residual) {
          if (in0 && live0) v00 += S.residual[a0];
          if (in0 && live1) v01 += S.residual[a1];
          if (in1 && live0) v10 += S.residual[a0 + 8];
          if (in1 && live1) v11 += S.residual[a1 + 8];
        }
        if (S.out_bf16) {
          if (in0 && live0) S.out_bf16[a0] = f32_to_bf16_rne(v00);
          if (in0 && live1) S.out_bf16[a1] = f32_to_bf16_rne(v01);
          if (in1 && live0) S.out_bf16[a0 + 8] = f32_to_bf16_rne(v10);
          if (in1 && live1) S.out_bf16[a1 + 8] = f32_to_bf16_rne(v11);
        } else {
          if (in0 && live0) S.out[a0] = v00;
          if (in0 && live1) S.out[a1] = v01;
          if (in1 && live0) S.out[a0 + 8] = v10;
          if (in1 && live1) S.out[a1 + 8] = v11;
        }
      }
    } else
    for (uint32_t it = 0; it < ntiles; ++it) {
      uint32_t const s = it & slot_mask, use = it >> slot_shift;
      if (!mbar_wait(b_rfull + 8 * s, use & 1, abort_flag, p.status, 0x520)) break;
      float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
      uint32_t src = s_red + s * red_slot + nt * 512 + lane * 16;
#pragma unroll 4
      for (uint32_t w = 0; w < nact; ++w) {
        float4 const v = lds128f(src);
        lo = __fadd2_rn(lo, make_float2(v.x, v.y));
        hi = __fadd2_rn(hi, make_float2(v.z, v.w));
        src += NT * 512;
      }
      mbar_arrive(b_rempty + 8 * s);
      uint32_t const row = (t0 + it) * 16 + r;
      bool const in0 = row < p.n, in1 = row + 8 < p.n;
      size_t const a0 = o0 + row, a1 = o1 + row;
      float v00 = lo.x, v01 = lo.y, v10 = hi.x, v11 = hi.y;
      if (res) {
        if (in0 && live0) v00 += res[a0];
        if (in0 && live1) v01 += res[a1];
        if (in1 && live0) v10 += res[a0 + 8];
        if (in1 && live1) v11 += res[a1 + 8];
      }
      if (in0) {
        if (live0) dst[a0] = v00;
        if (live1) dst[a1] = v01;
      }
      if (in1) {
        if (live0) dst[a0 + 8] = v10;
        if (live1) dst[a1 + 8] = v11;
      }
      if (extra) {  // row-sharded gather: the same values into the other ranks' buffers
#pragma unroll
        for (int g = 1; g < 8; ++g) {
          if (g <= int(extra)) {
            float* const peer = p.out[g];
            if (in0 && live0) peer[a0] = v00;
            if (in0 && live1) peer[a1] = v01;
            if (in1 && live0) peer[a0 + 8] = v10;
            if (in1 && live1) peer[a1 + 8] = v11;
          }
        }
      }
    }
    __threadfence();
  } else if (warp - kFirstConsumer < nact) {
    uint32_t const w = warp - kFirstConsumer, sb = sb0 + w;
    uint32_t const r = lane >> 2, q = lane & 3;
    if (!p.input_settled || p.partials != nullptr) pdl_wait();  // activations; the reducer waits before anything is stored
    // ---- K-stationary operands ----
    uint32_t const tab = s_tab + w * tab_bytes;
    // activation scale pairs {a[2q], a[2q+1]} of (octet nt, group g) at ((nt*4 + g/2)*4 + q)*16 + (g%2)*8
    uint32_t const rd_ap = tab + kTabBytes + q * 16;
    uint32_t bfrag[NT][8][2];  // int8 activations of token nt*8 + r: even / odd columns of 8q..8q+7 in group g
    uint32_t asplit[NT][3][2]; // tf32 terms of a*sum for token nt*8 + r, groups q and q+4
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      uint32_t const tokb = nt * 8 + r, tokc = nt * 8 + 2 * q;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint2 z = make_uint2(0u, 0u);
        if (tokb < p.m) z = *reinterpret_cast<const uint2*>(p.xcodes + size_t(tokb) * p.padded_k + sb * 256 + g * 32 + q * 8);
        bfrag[nt][g][0] = even_bytes(z.x, z.y);
        bfrag[nt][g][1] = odd_bytes(z.x, z.y);
        if (r == 0) {  // lanes 0..3 fill the scale-pair table of this warp
          float const a0 = tokc < p.m ? p.xscales[size_t(tokc) * p.G + sb * 8 + g] : 0.f;
          float const a1 = tokc + 1 < p.m ? p.xscales[size_t(tokc + 1) * p.G + sb * 8 + g] : 0.f;
          asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(rd_ap + (nt * 4 + g / 2) * 64 + (g % 2) * 8), "f"(a0), "f"(a1) : "memory");
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float as = 0.f;
        if (tokb < p.m) {
          size_t const i = size_t(tokb) * p.G + sb * 8 + q + 4 * h;
          as = p.xscales[i] * float(p.xsums[i]);
        }
        uint32_t const hi = to_tf32(as);
        float const r1 = as - __uint_as_float(hi);
        uint32_t const mid = to_tf32(r1);
        float const r2 = r1 - __uint_as_float(mid);
        asplit[nt][0][h] = hi;
        asplit[nt][1][h] = mid;
        asplit[nt][2][h] = to_tf32(r2);
      }
    }
    __syncwarp();
    float2 const nmagic2 = make_float2(-kMagicF, -kMagicF);
    uint32_t cmagic[4];  // accumulator input of every MMA; opaque to the compiler so that it stays in four registers
#pragma unroll
    for (int j = 0; j < 4; ++j) asm volatile("mov.u32 %0, %1;" : "=r"(cmagic[j]) : "n"(0x4B400000));
    // decode role of this lane: row16 = lane & 15, half h = lane >> 4 takes groups 4h..4h+3
    uint32_t const drow = lane & 15, dh = lane >> 4;
    // groups 0..3: byte & 0x3f; groups 4..7: (byte of word 3 & 0x0f) | ((byte >> 2) & 0x30)  (mins: high nibble of word 3)
    uint32_t const dsh = dh ? 2u : 0u, dmask_a = dh ? 0x30303030u : 0x3f3f3f3fu, dmask_b = dh ? 0x0f0f0f0fu : 0u;
    uint32_t const dec_meta = s_meta + (drow >> 3) * cw * 128 + w * 128 + (drow & 7) * 16;
    uint32_t const dec_sc = tab + drow * kTabRow + dh * 32, dec_mn = dec_sc - dh * 16 + kTabMn, dec_dd = tab + drow * kTabRow + kTabDd;
    uint32_t const rd_sc = tab + r * kTabRow, rd_mn = rd_sc + kTabMn + q * 4, rd_dd = rd_sc + kTabDd;
    // ldmatrix lane address: matrix j = lane >> 3 (bit 0: row group, bit 1: second K32 group), row i = lane & 7
    uint32_t const lj = lane >> 3, li = lane & 7;
    uint32_t const ld_base = s_codes + (lj & 1) * cw * 1024 + w * 1024 + li * 128;
    uint32_t const ld_x = ((lj >> 1) << 4) ^ (li << 4);
    uint32_t const red_dst = s_red + (w * NT * 32 + lane) * 16;

    uint32_t s = 0, ph = 0, code_off = 0, meta_off = 0;
    for (uint32_t it = 0; it < ntiles; ++it) {
      if (!mbar_wait(b_full + 8 * s, ph, abort_flag, p.status, 0x530)) break;
      uint32_t const cbase = ld_base + code_off;
      uint4 const mw = lds128(dec_meta + meta_off);
      // ---- decode the metadata of 16 rows ----
      {
        uint32_t const sc4 = ((mw.y >> dsh) & dmask_a) | (mw.w & dmask_b);
        uint32_t const mn4 = ((mw.z >> dsh) & dmask_a) | ((mw.w >> 4) & dmask_b);
        // byte -> float without shifts: splice the byte under the exponent of 2^23 (PRMT), then one
        // packed subtraction per pair of values; scales are stored twice, as the packed FMAs read them
        float2 const m23 = make_float2(-8388608.0f, -8388608.0f);
        uint32_t const e0 = __byte_perm(sc4, 0x4b000000u, 0x7650), e1 = __byte_perm(sc4, 0x4b000000u, 0x7651);
        uint32_t const e2 = __byte_perm(sc4, 0x4b000000u, 0x7652), e3 = __byte_perm(sc4, 0x4b000000u, 0x7653);
        float2 const p0 = __fadd2_rn(as_f2(e0, e0), m23), p1 = __fadd2_rn(as_f2(e1, e1), m23);
        float2 const p2 = __fadd2_rn(as_f2(e2, e2), m23), p3 = __fadd2_rn(as_f2(e3, e3), m23);
        sts128f(dec_sc, p0.x, p0.y, p1.x, p1.y);
        sts128f(dec_sc + 16, p2.x, p2.y, p3.x, p3.y);
        float2 const q0 = __fadd2_rn(as_f2(__byte_perm(mn4, 0x4b000000u, 0x7650), __byte_perm(mn4, 0x4b000000u, 0x7651)), m23);
        float2 const q1 = __fadd2_rn(as_f2(__byte_perm(mn4, 0x4b000000u, 0x7652), __byte_perm(mn4, 0x4b000000u, 0x7653)), m23);
        sts128f(dec_mn, q0.x, q0.y, q1.x, q1.y);
        float const d = fp16_bits_to_f32(mw.x & 0xffffu), ndmin = -fp16_bits_to_f32(mw.x >> 16);
        sts128f(dec_dd, d, d, ndmin, ndmin);  // both halves of a row store the same words
      }
      __syncwarp();
      float2 acc[NT][2];
      float mins[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        acc[nt][0] = acc[nt][1] = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) mins[nt][j] = 0.f;
      }
#pragma unroll
      for (int gp = 0; gp < 4; ++gp) {
        uint32_t raw[4];
        ldmatrix_x4(raw, cbase + ((uint32_t(gp) << 5) ^ ld_x));
        // The stage goes back to the producer as soon as its last word is in registers (the arrival has
        // release semantics, so the loads above are performed before it).
        if (gp == 3) mbar_arrive(b_empty + 8 * s);
        float4 const sc_lo = lds128f(rd_sc + gp * 16);         // row r:   {s_g, s_g, s_g+1, s_g+1}
        float4 const sc_hi = lds128f(rd_sc + 8 * kTabRow + gp * 16);   // row r+8
        float4 ap4[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) ap4[nt] = lds128f(rd_ap + (nt * 4 + gp) * 64);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          int const g = gp * 2 + e;
          uint32_t const w0 = raw[2 * e], w1 = raw[2 * e + 1];
          uint32_t const a0 = w0 & 0x0f0f0f0fu, a1 = w1 & 0x0f0f0f0fu;
          uint32_t const a2 = (w0 >> 4) & 0x0f0f0f0fu, a3 = (w1 >> 4) & 0x0f0f0f0fu;
          float2 const s_lo = e ? make_float2(sc_lo.z, sc_lo.w) : make_float2(sc_lo.x, sc_lo.y);
          float2 const s_hi = e ? make_float2(sc_hi.z, sc_hi.w) : make_float2(sc_hi.x, sc_hi.y);
          float2 const c_lo = mul2(s_lo, nmagic2), c_hi = mul2(s_hi, nmagic2);  // exact: 6-bit integer * 1.5*2^23
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint32_t d[4];
            mma_u8s8(d, a0, a1, a2, a3, bfrag[nt][g][0], bfrag[nt][g][1], cmagic);
            if constexpr (Dump) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t const tok = nt * 8 + q * 2 + (j & 1), row = (t0 + it) * 16 + r + (j >> 1) * 8;
                if (tok < p.m && row < p.n) p.partials[(size_t(tok) * p.n + row) * p.G + sb * 8 + g] = int32_t(d[j] - kMagicI);
              }
            }
            float2 const ap = e ? make_float2(ap4[nt].z, ap4[nt].w) : make_float2(ap4[nt].x, ap4[nt].y);
            float2 const t_lo = fma2(as_f2(d[0], d[1]), s_lo, c_lo);  // sc * dot, exact
            float2 const t_hi = fma2(as_f2(d[2], d[3]), s_hi, c_hi);
            acc[nt][0] = fma2(t_lo, ap, acc[nt][0]);
            acc[nt][1] = fma2(t_hi, ap, acc[nt][1]);
          }
        }
      }
      // ---- min term: rows x groups (6-bit integers) times groups x tokens (three tf32 terms of a*sum) ----
      {
        uint32_t const m0 = lds32(rd_mn), m1 = lds32(rd_mn + 8 * kTabRow), m2 = lds32(rd_mn + 16), m3 = lds32(rd_mn + 8 * kTabRow + 16);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int part = 2; part >= 0; --part) mma_tf32(mins[nt], m0, m1, m2, m3, asplit[nt][part][0], asplit[nt][part][1]);
        }
      }
      float4 const dd_lo = lds128f(rd_dd);        // {d, d, -dmin, -dmin} of row r
      float4 const dd_hi = lds128f(rd_dd + 8 * kTabRow);  // row r+8
      // ---- hand the tile to the reducer ----
      uint32_t const rs = it & slot_mask, ruse = it >> slot_shift;
      if (ruse > 0 && !mbar_wait(b_rempty + 8 * rs, (ruse - 1) & 1, abort_flag, p.status, 0x540)) break;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float2 const o_lo = fma2(acc[nt][0], make_float2(dd_lo.x, dd_lo.y),
                                 mul2(make_float2(mins[nt][0], mins[nt][1]), make_float2(dd_lo.z, dd_lo.w)));
        float2 const o_hi = fma2(acc[nt][1], make_float2(dd_hi.x, dd_hi.y),
                                 mul2(make_float2(mins[nt][2], mins[nt][3]), make_float2(dd_hi.z, dd_hi.w)));
        sts128f(red_dst + rs * red_slot + nt * 512, o_lo.x, o_lo.y, o_hi.x, o_hi.y);
      }
      mbar_arrive(b_rfull + 8 * rs);
      __syncwarp();  // every lane has read the tables before the next tile's decode overwrites them
      code_off += code_stage;
      meta_off += meta_stage;
      if (++s == stages) { s = 0; ph ^= 1; code_off = 0; meta_off = 0; }
    }
  }

  // ---- split-K: the last block of a row range adds the slices in order ----
  if (p.split_k > 1) {
    pdl_wait();
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      uint32_t const old = atomicAdd(p.tickets + range, 1u);
      *last_flag = (old == p.split_k - 1) && !*abort_flag;
      if (old == p.split_k - 1) p.tickets[range] = 0;
    }
    __syncthreads();
    if (*last_flag && p.nseg != 0) {
      __threadfence();
      // One thread per (token, row of a tile); in pair mode per row of a gate tile, which also reads the up tile.
      uint32_t const step = p.pair ? 2u : 1u;
      size_t const plane = size_t(p.m) * p.n_total;
      for (uint32_t i = threadIdx.x; i < (ntiles / step) * 16 * p.m; i += blockDim.x) {
        uint32_t const tile = i / (16 * p.m), rem = i % (16 * p.m), tok = rem / 16, r16 = rem % 16;
        uint32_t sg, local;
        locate_tile(p, t0 + tile * step, sg, local);
        const GtSegment& S = p.seg[sg];
        uint32_t const row = local * 16 + r16;
        if (row >= S.n) continue;
        size_t const o = size_t(tok) * p.n_total + S.row_base + row;
        float v = __ldcg(p.slices + o);
        for (uint32_t sl = 1; sl < p.split_k; ++sl) v += __ldcg(p.slices + sl * plane + o);
        size_t const oo = size_t(tok) * S.n + row;
        if (p.pair) {
          size_t const o2 = size_t(tok) * p.n_total + p.seg[1].row_base + row;
          float u = __ldcg(p.slices + o2);
          for (uint32_t sl = 1; sl < p.split_k; ++sl) u += __ldcg(p.slices + sl * plane + o2);
          p.seg[0].out_bf16[oo] = f32_to_bf16_rne(silu_fp32(v) * u);
          continue;
        }
        if (S.residual) v += S.residual[oo];
        if (S.out_bf16) S.out_bf16[oo] = f32_to_bf16_rne(v);
        else S.out[oo] = v;
      }
    } else
    if (*last_flag) {
      __threadfence();
      uint32_t const row0 = t0 * 16, rows = min(p.n, t1 * 16) > row0 ? min(p.n, t1 * 16) - row0 : 0;
      for (uint32_t i = threadIdx.x; i < rows * p.m; i += blockDim.x) {
        uint32_t const tok = i / rows, row = row0 + i % rows;
        size_t const o = size_t(tok) * p.n + row;
        float v = __ldcg(p.slices + o);
        for (uint32_t sl = 1; sl < p.split_k; ++sl) v += __ldcg(p.slices + size_t(sl) * p.m * p.n + o);
        size_t const oo = size_t(tok) * p.out_stride + p.out_row0 + row;
        if (p.residual) v += p.residual[oo];
        p.out[0][oo] = v;
#pragma unroll
        for (int g = 1; g < 8; ++g)
          if (g < int(p.ndst)) p.out[g][oo] = v;
      }
    }
  }

  // ---- gather: the last block of the grid records one more finished projection.  It is announced to
  // the peers by the next kernel of this stream (announce_deliveries), i.e. after this grid has
  // completed and its peer stores are visible system-wide, so no system-scope fence is needed here.
  if (p.done != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      pdl_wait();  // the counters may still belong to the kernel before this one
      __threadfence();
      uint32_t const old = atomicAdd(p.done, 1u);
      if (old == gridDim.x - 1) {
        *p.done = 0;
        // counted only if no block of any launch so far gave up a wait (the status word is shared by all blocks)
        if (!*abort_flag && *reinterpret_cast<volatile int*>(p.status) == 0) atomicAdd(p.unsignalled, 1u);
      }
    }
  }
}

}  // namespace

namespace {

constexpr uint32_t kSmemBudget = 227 * 1024;

uint32_t smem_bytes(uint32_t cw, uint32_t nt, uint32_t stages, uint32_t red_slots) {
  return 1024 + stages * cw * 2304 + cw * (kTabBytes + nt * 256) + red_slots * cw * nt * 512 + (2 * stages + 4) * 8 + 16;
}

struct Maps {
  CUtensorMap codes[3], meta[3];
};

template <int NT, int MAXW>
cudaError_t launch_cfg(const Maps& t, const GtParams& p, bool dump, uint32_t grid, uint32_t smem, cudaStream_t stream) {
  auto kernel = dump ? gemv_tma_kernel<NT, MAXW, true> : gemv_tma_kernel<NT, MAXW, false>;
  cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (st != cudaSuccess) return st;
  return launch_kernel(kernel, grid, (p.cw + kFirstReducer + NT) * 32, smem, stream, launch_overlap(), t.codes[0], t.meta[0],
                       t.codes[1], t.meta[1], t.codes[2], t.meta[2], p);
}

bool make_weight_maps(const WeightView& w, uint32_t cw, CUtensorMap* codes, CUtensorMap* meta) {
  uint64_t const rgs = w.padded_n / 8;
  uint64_t dims[3] = {128, uint64_t(w.tiles_k) * 8, rgs}, strides[2] = {128, uint64_t(w.tiles_k) * 1024};
  uint32_t box[3] = {128, cw * 8, 2};
  if (!make_map(codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w.codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
  uint64_t mdims[3] = {128, w.tiles_k, rgs}, mstrides[2] = {128, uint64_t(w.tiles_k) * 128};
  uint32_t mbox[3] = {128, cw, 2};
  return make_map(meta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w.meta, mdims, mstrides, mbox, CU_TENSOR_MAP_SWIZZLE_NONE);
}

template <class... A>
cudaError_t launch_by_shape(uint32_t nt, uint32_t cw, A&&... a) {
  if (nt == 1) {
    if (cw <= 12) return launch_cfg<1, 14>(a...);
    return launch_cfg<1, kGemvTmaMaxWarpsNarrow + 2>(a...);
  }
  if (cw <= 12) return launch_cfg<2, 15>(a...);
  return launch_cfg<2, kGemvTmaMaxWarpsWide + 3>(a...);
}

}  // namespace

bool gemv_tma_supported(const WeightView& w, const Q8View& x) {
  return x.m <= kGemvTmaMaxTokens && encode_fn() != nullptr && reinterpret_cast<uintptr_t>(w.codes) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(w.meta) % 16 == 0 && reinterpret_cast<uintptr_t>(x.codes) % 8 == 0;
}

GemvTmaPlan plan_gemv_tma(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request, uint32_t warps_request) {
  return plan_gemv_tma_tiles(m, ((n + 7) / 8 * 8 + 15) / 16, tiles_k, split_k_request, warps_request, false);
}

GemvTmaPlan plan_gemv_tma_tiles(uint32_t m, uint32_t row_tiles, uint32_t tiles_k, uint32_t split_k_request, uint32_t warps_request,
                                bool pair) {
  GemvTmaPlan p;
  uint32_t const nt = m <= 8 ? 1 : 2;
  uint32_t const max_cw = nt == 1 ? kGemvTmaMaxWarpsNarrow : kGemvTmaMaxWarpsWide;
  uint32_t split = split_k_request;
  if (split == 0) {
    // Widest K slice by default.  Sixteen tokens on a matrix with few row tiles per SM measured faster
    // with narrower slices (more, shorter blocks in flight and twice the registers per thread).
    uint32_t cw_target = max_cw;
    if (nt == 2 && row_tiles < 1024) cw_target = 12;
    if (warps_request) cw_target = warps_request < max_cw ? warps_request : max_cw;
    split = (tiles_k + cw_target - 1) / cw_target;
  }
  if (split > tiles_k) split = tiles_k;
  if (split < 1) split = 1;
  uint32_t cw = (tiles_k + split - 1) / split;
  while (cw > max_cw) { ++split; cw = (tiles_k + split - 1) / split; }
  split = (tiles_k + cw - 1) / cw;  // drop empty slices
  p.split_k = split;
  p.warps = cw;
  uint32_t ranges = uint32_t(sm_count()) / split;
  if (ranges < 1) ranges = 1;
  if (ranges > row_tiles) ranges = row_tiles;
  p.tiles_per_range = (row_tiles + ranges - 1) / ranges;
  if (pair && (p.tiles_per_range & 1u)) ++p.tiles_per_range;  // a gate tile and its up tile stay in one block
  p.ranges = (row_tiles + p.tiles_per_range - 1) / p.tiles_per_range;
  // Two hand-off buffers unless giving one up buys a third (or second) ring stage.
  auto fit = [&](uint32_t slots) {
    uint32_t st = 1;
    while (st < uint32_t(kMaxStages) && smem_bytes(cw, nt, st + 1, slots) <= kSmemBudget) ++st;
    return st;
  };
  p.red_slots = 2;
  p.stages = fit(2);
  if (p.stages < 3 && fit(1) > p.stages) { p.red_slots = 1; p.stages = fit(1); }
  return p;
}

cudaError_t launch_gemv_tma(const WeightView& w, const Q8View& x, float* out, const float* residual, int32_t* partials,
                            const GemvTmaPlan& plan, void* slices, uint32_t* tickets, int* status, cudaStream_t stream,
                            const GemvTmaGather* gather) {
  uint32_t const nt = x.m <= 8 ? 1 : 2;
  uint32_t const cw = plan.warps;
  if (x.m == 0 || x.m > kGemvTmaMaxTokens || cw < 1 || cw > (nt == 1 ? kGemvTmaMaxWarpsNarrow : kGemvTmaMaxWarpsWide) ||
      plan.split_k * cw < w.tiles_k || plan.stages < 2 || plan.stages > uint32_t(kMaxStages) ||
      (plan.red_slots != 1 && plan.red_slots != 2) || smem_bytes(cw, nt, plan.stages, plan.red_slots) > kSmemBudget ||
      (plan.split_k > 1 && (!slices || !tickets)) ||
      (gather && (gather->ranks < 1 || gather->ranks > 8 || gather->rank >= gather->ranks || !gather->done || !gather->unsignalled || partials)))
    return cudaErrorInvalidValue;
  Maps t{};
  if (!make_weight_maps(w, cw, &t.codes[0], &t.meta[0])) return cudaErrorInvalidValue;
  t.codes[1] = t.codes[2] = t.codes[0];
  t.meta[1] = t.meta[2] = t.meta[0];
  GtParams p{};
  p.xcodes = x.codes; p.xscales = x.scales; p.xsums = x.sums; p.residual = residual;
  if (gather) {
    for (uint32_t g = 0; g < gather->ranks; ++g) { p.out[g] = gather->outputs[g]; p.peer_flag[g] = gather->flags[g]; }
    p.done = gather->done; p.unsignalled = gather->unsignalled; p.ndst = gather->ranks; p.rank = gather->rank;
    p.out_stride = gather->total_rows; p.out_row0 = gather->row_offset;
  } else {
    p.out[0] = out; p.done = nullptr; p.ndst = 1; p.rank = 0; p.out_stride = w.n; p.out_row0 = 0;
  }
  p.partials = partials; p.slices = static_cast<float*>(slices); p.tickets = tickets; p.status = status;
  p.n = w.n; p.m = x.m; p.padded_k = x.padded_k; p.tiles_k = w.tiles_k; p.G = x.padded_k / 32;
  p.row_tiles = (w.padded_n + 15) / 16; p.cw = cw; p.split_k = plan.split_k;
  p.tiles_per_range = plan.tiles_per_range; p.stages = plan.stages; p.red_slots = plan.red_slots;
  p.input_settled = plan.input_settled;
  uint32_t const grid = plan.ranges * plan.split_k, smem = smem_bytes(cw, nt, plan.stages, plan.red_slots);
  bool const dump = partials != nullptr;
  return launch_by_shape(nt, cw, t, p, dump, grid, smem, stream);
}

cudaError_t launch_gemv_tma_multi(const WeightView* ws, const GemvTmaOutput* outs, uint32_t count, bool swiglu_pair, const Q8View& x,
                                  const GemvTmaPlan& plan, void* slices, uint32_t* tickets, int* status, cudaStream_t stream) {
  uint32_t const nt = x.m <= 8 ? 1 : 2;
  uint32_t const cw = plan.warps;
  if (count < 1 || count > 3 || (swiglu_pair && count != 2) || x.m == 0 || x.m > kGemvTmaMaxTokens || cw < 1 ||
      cw > (nt == 1 ? kGemvTmaMaxWarpsNarrow : kGemvTmaMaxWarpsWide) || plan.stages < 2 || plan.stages > uint32_t(kMaxStages) ||
      (plan.red_slots != 1 && plan.red_slots != 2) || smem_bytes(cw, nt, plan.stages, plan.red_slots) > kSmemBudget ||
      (plan.split_k > 1 && (!slices || !tickets)) || (swiglu_pair && (plan.tiles_per_range & 1u)))
    return cudaErrorInvalidValue;
  Maps t{};
  GtParams p{};
  uint32_t total_tiles = 0, total_rows = 0;
  for (uint32_t i = 0; i < count; ++i) {
    if (ws[i].tiles_k != ws[0].tiles_k || plan.split_k * cw < ws[i].tiles_k) return cudaErrorInvalidValue;
    if (swiglu_pair && (ws[i].n != ws[0].n || !outs[0].out_bf16)) return cudaErrorInvalidValue;
    if (!swiglu_pair && !outs[i].out && !outs[i].out_bf16) return cudaErrorInvalidValue;
    if (!make_weight_maps(ws[i], cw, &t.codes[i], &t.meta[i])) return cudaErrorInvalidValue;
    p.seg[i] = GtSegment{outs[i].out, outs[i].out_bf16, outs[i].residual, ws[i].n, (ws[i].padded_n + 15) / 16, total_rows};
    total_tiles += p.seg[i].tiles;
    total_rows += ws[i].n;
  }
  for (uint32_t i = count; i < 3; ++i) { t.codes[i] = t.codes[0]; t.meta[i] = t.meta[0]; }
  p.xcodes = x.codes; p.xscales = x.scales; p.xsums = x.sums;
  p.ndst = 1; p.slices = static_cast<float*>(slices); p.tickets = tickets; p.status = status;
  p.n = ws[0].n; p.m = x.m; p.padded_k = x.padded_k; p.tiles_k = ws[0].tiles_k; p.G = x.padded_k / 32;
  p.row_tiles = total_tiles; p.cw = cw; p.split_k = plan.split_k;
  p.tiles_per_range = plan.tiles_per_range; p.stages = plan.stages; p.red_slots = plan.red_slots;
  p.input_settled = plan.input_settled;
  p.nseg = count; p.pair = swiglu_pair ? 1u : 0u; p.n_total = total_rows;
  uint32_t const grid = plan.ranges * plan.split_k, smem = smem_bytes(cw, nt, plan.stages, plan.red_slots);
  return launch_by_shape(nt, cw, t, p, false, grid, smem, stream);
}

bool plan_gemv_tma_swiglu_q8(uint32_t m, const WeightView& gate, GemvTmaPlan* plan) {
  if (m == 0 || m > kGemvTmaMaxTokens || gate.n % 32 != 0 || gate.n != gate.padded_n) return false;
  uint32_t const tiles = 2 * (gate.padded_n / 16);
  GemvTmaPlan p = plan_gemv_tma_tiles(m, tiles, gate.tiles_k, 1, 0, true);
  if (p.split_k != 1) return false;  // the quantiser needs complete sums: the whole K in one block
  // a group of 32 rows = gate tile, up tile, gate tile, up tile: four consecutive tiles in one block
  p.tiles_per_range = (p.tiles_per_range + 3) / 4 * 4;
  p.ranges = (tiles + p.tiles_per_range - 1) / p.tiles_per_range;
  *plan = p;
  return true;
}

cudaError_t launch_gemv_tma_swiglu_q8(const WeightView& gate, const WeightView& up, const Q8View& x, Q8Out out, int* failure,
                                      const GemvTmaPlan& plan, int* status, cudaStream_t stream) {
  uint32_t const nt = x.m <= 8 ? 1 : 2;
  uint32_t const cw = plan.warps;
  if (x.m == 0 || x.m > kGemvTmaMaxTokens || plan.split_k != 1 || cw < gate.tiles_k || (plan.tiles_per_range & 3u) ||
      cw > (nt == 1 ? kGemvTmaMaxWarpsNarrow : kGemvTmaMaxWarpsWide) || plan.stages < 2 || plan.stages > uint32_t(kMaxStages) ||
      (plan.red_slots != 1 && plan.red_slots != 2) || smem_bytes(cw, nt, plan.stages, plan.red_slots) > kSmemBudget ||
      gate.n != up.n || gate.tiles_k != up.tiles_k || gate.n % 32 != 0 || gate.n != gate.padded_n || out.m != x.m ||
      out.padded_k != gate.n || !out.codes || !out.scales || !out.sums || !failure)
    return cudaErrorInvalidValue;
  Maps t{};
  GtParams p{};
  const WeightView* ws[2] = {&gate, &up};
  for (uint32_t i = 0; i < 2; ++i) {
    if (!make_weight_maps(*ws[i], cw, &t.codes[i], &t.meta[i])) return cudaErrorInvalidValue;
    p.seg[i] = GtSegment{nullptr, nullptr, nullptr, ws[i]->n, ws[i]->padded_n / 16, i * gate.n};
  }
  t.codes[2] = t.codes[0]; t.meta[2] = t.meta[0];
  p.xcodes = x.codes; p.xscales = x.scales; p.xsums = x.sums;
  p.ndst = 1; p.status = status;
  p.n = gate.n; p.m = x.m; p.padded_k = x.padded_k; p.tiles_k = gate.tiles_k; p.G = x.padded_k / 32;
  p.row_tiles = 2 * (gate.padded_n / 16); p.cw = cw; p.split_k = 1;
  p.tiles_per_range = plan.tiles_per_range; p.stages = plan.stages; p.red_slots = plan.red_slots;
  p.input_settled = 0;
  p.nseg = 2; p.pair = 2; p.n_total = 2 * gate.n;
  p.q8_codes = out.codes; p.q8_scales = out.scales; p.q8_sums = out.sums; p.q8_failure = failure; p.q8_pk = out.padded_k;
  uint32_t const grid = plan.ranges, smem = smem_bytes(cw, nt, plan.stages, plan.red_slots);
  return launch_by_shape(nt, cw, t, p, false, grid, smem, stream);
}

}  // namespace q4k
