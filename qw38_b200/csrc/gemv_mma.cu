// Decode projection for up to 16 tokens on warp-level int8 MMA, built to stay close to the
// HBM stream rate: the kernel is instruction-bound long before it is tensor-bound, so every
// choice below removes issue slots per KiB of weights.
//
//   * One warp owns one row group (8 rows = the n8 side of m16n8k32) and streams its 1 KiB
//     code tiles + 128 B metadata with 16-byte cp.async into a private ring; tile rows are
//     XOR-swizzled so one ldmatrix.x4 hands lane (r = lane/4, c = lane%4) raw word c of row r
//     for four K32 groups.  (w & 0x0f0f0f0f) holds columns 8c+{0,2,4,6}, ((w >> 4) & ...)
//     columns 8c+{1,3,5,7}; activations are staged as matching (even, odd) byte words.
//   * All shared-memory strides are compile-time constants and every operand of the inner
//     loop sits at (lane base + immediate): per K32 group a lane issues one 8-byte activation
//     load, one MMA, one 16-byte table load, one 16-byte scale load, two conversions and three
//     packed f32x2 operations for its two (or, with 9..16 tokens, four) partial dots.
//   * Metadata is decoded once per tile by the whole warp (lane (r, c) decodes groups c and
//     c+4 of row r) into a table of (D, D', -Mn, -Mn') for row pairs.
//   * K is split over the blocks of a thread-block cluster; the slices are added in rank order
//     through distributed shared memory, so no global scratch and no dependence on timing.
//
// Arithmetic per partial dot P (exact int32, reset per K32 group), as the reference
// (cuda/q4k_q8.cu:98): acc += a * (D * float(P) - Mn * float(sum)),  D = d*sc, Mn = dmin*m.
#include <cooperative_groups.h>

#include "common.cuh"
#include "launch.h"

namespace cg = cooperative_groups;

namespace q4k {
namespace {

constexpr int kStages = 3;
constexpr int kStageBytes = 1024 + 128;
constexpr int kStep = 4;            // super-blocks of activations staged at a time
constexpr int kActRow = 256 + 32;   // bytes per token per super-block; 32 mod 128 keeps LDS.64 conflict-free
constexpr uint32_t kMagicI = 0x4B400000u;  // bit pattern of 1.5 * 2^23
constexpr float kMagicF = 12582912.0f;

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
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};\n"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Packed pairs of fp32 (sm_100 f32x2 pipe): one issue slot for two lanes of arithmetic.  The
// intrinsics let the compiler keep both halves in an aligned register pair.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

template <bool Wide>
__device__ __forceinline__ void fill_stage(uint8_t* stage, const uint8_t* codes, const uint8_t* meta, uint32_t lane) {
  if constexpr (Wide) {
    uint32_t const base = smem_u32(stage);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t const q = lane + 32 * i, r = q >> 3, g = q & 7;
      cp_async16(base + r * 128 + ((g ^ r) << 4), codes + q * 16);
    }
    if (lane < 8) cp_async16(base + 1024 + lane * 16, meta + lane * 16);
  } else {  // pointers that are only 4-byte (codes) / 2-byte (metadata) aligned
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

template <int Warps, int Tokens> struct Smem {
  static constexpr int kRing = Warps * kStages * kStageBytes;
  static constexpr int kTab = Warps * 8 * 4 * 16;            // [warp][group][row pair] float4
  static constexpr int kAct1 = kStep * Tokens * kActRow;     // [kbl][token][288]
  static constexpr int kAf1 = kStep * 8 * Tokens * 16;       // [kbl*8+g][token] (a, a, fs, fs)
  static constexpr int kAct = 2 * kAct1;                     // double buffered
  static constexpr int kAf = 2 * kAf1;
  static constexpr int kRed = Warps * 32 * 16;               // [warp][lane] float4 slice sums
  static constexpr int kTotal = kRing + kTab + kAct + kAf + kRed;
};

// Upper: tokens 8..15 exist.  Tokens staged = 16 with Upper, else 8.
template <bool Upper, bool Dump, bool Wide, int Warps>
__global__ void __launch_bounds__(Warps * 32) gemv_mma_kernel(WeightView w, Q8View x, float* __restrict__ out,
                                                              const float* __restrict__ residual,
                                                              int32_t* __restrict__ partials, uint32_t split_k) {
  constexpr int Tokens = Upper ? 16 : 8;
  using S = Smem<Warps, Tokens>;
  constexpr int kThreads = Warps * 32;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* const ring_all = smem;
  uint8_t* const tab_all = ring_all + S::kRing;
  uint8_t* const act = tab_all + S::kTab;
  uint8_t* const af = act + S::kAct;
  float4* const red = reinterpret_cast<float4*>(af + S::kAf);

  uint32_t const lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t const tq = lane >> 2, c = lane & 3;
  uint32_t const tiles_k = w.tiles_k, pk = x.padded_k, G = pk / 32;
  uint32_t const rgs = w.padded_n / 8;
  uint32_t const slice = blockIdx.x % split_k, row_tile = blockIdx.x / split_k;
  uint32_t const rg = row_tile * Warps + warp;
  bool const active = rg < rgs;
  uint32_t const kb0 = uint32_t((uint64_t(slice) * tiles_k) / split_k);
  uint32_t const kb1 = uint32_t((uint64_t(slice + 1) * tiles_k) / split_k);

  uint8_t* const ring = ring_all + warp * kStages * kStageBytes;
  uint8_t* const tab = tab_all + warp * (8 * 4 * 16);
  const uint8_t* const cbase = w.codes + uint64_t(active ? rg : 0) * tiles_k * 1024;
  const uint8_t* const mbase = w.meta + uint64_t(active ? rg : 0) * tiles_k * 128;

  float2 acc_lo = make_float2(0.f, 0.f), acc_hi = make_float2(0.f, 0.f);  // tokens tq / tq+8, rows 2c, 2c+1

  // Weight pipeline.  Everything that does not change from tile to tile is computed once:
  // the lane's two source offsets, its swizzled destination offsets, running pointers and a
  // stage counter (no per-tile multiply or modulo).
  uint32_t const q0 = lane, q1 = lane + 32;
  uint32_t const dst0 = (q0 >> 3) * 128 + (((q0 & 7) ^ (q0 >> 3)) << 4), dst1 = (q1 >> 3) * 128 + (((q1 & 7) ^ (q1 >> 3)) << 4);
  uint32_t const ring_s = smem_u32(ring);
  const uint8_t* cptr = cbase + uint64_t(kb0) * 1024;
  const uint8_t* mptr = mbase + uint64_t(kb0) * 128;
  uint32_t next_load = kb0, load_stage = 0;
  auto issue = [&]() {
    if (active && next_load < kb1) {
      if constexpr (Wide) {
        uint32_t const sb = ring_s + load_stage * kStageBytes;
        cp_async16(sb + dst0, cptr + q0 * 16);
        cp_async16(sb + dst1, cptr + q1 * 16);
        if (lane < 8) cp_async16(sb + 1024 + lane * 16, mptr + lane * 16);
      } else {
        fill_stage<false>(ring + load_stage * kStageBytes, cptr, mptr, lane);
      }
    }
    cptr += 1024;
    mptr += 128;
    ++next_load;
    if (++load_stage == kStages) load_stage = 0;
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue();

  bool const act16 = (reinterpret_cast<uintptr_t>(x.codes) & 15) == 0;
  // lane-constant shared addresses
  uint32_t const ldm_row = lane & 7, ldm_mat = lane >> 3;
  uint32_t const ldm_off0 = ldm_row * 128 + ((ldm_mat ^ ldm_row) << 4), ldm_off1 = ldm_row * 128 + (((ldm_mat + 4) ^ ldm_row) << 4);
  const uint8_t* const tab_lane = tab + c * 16;
  float* const tab_wa = reinterpret_cast<float*>(tab + c * 64 + (tq >> 1) * 16) + (tq & 1);
  float* const tab_wb = reinterpret_cast<float*>(tab + (c + 4) * 64 + (tq >> 1) * 16) + (tq & 1);
  float2 const nmagic2 = make_float2(-kMagicF, -kMagicF);

  // Activation staging: the global loads of the next step are issued into registers before the
  // current step is computed and stored (de-interleaved) into the other buffer afterwards.
  constexpr int kTpt = (Tokens * 16 + kThreads - 1) / kThreads;  // tokens per thread
  uint32_t const l16 = threadIdx.x & 15;
  uint4 sz[kTpt][kStep];
  float sa[kTpt][2];
  int ss[kTpt][2];
  auto stage_load = [&](uint32_t s0, uint32_t kbs) {
#pragma unroll
    for (int tt = 0; tt < kTpt; ++tt) {
      uint32_t const t = (threadIdx.x >> 4) + tt * (kThreads / 16);
      bool const live = t < Tokens && t < x.m;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(x.codes) + uint64_t(live ? t : 0) * pk + uint64_t(s0) * 256 + l16 * 16;
#pragma unroll
      for (int kbl = 0; kbl < kStep; ++kbl) {
        uint4 z = make_uint4(0, 0, 0, 0);
        if (live && uint32_t(kbl) < kbs) {
          if (act16) z = __ldg(reinterpret_cast<const uint4*>(src + kbl * 256));
          else {
            const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src + kbl * 256);
            z = make_uint4(__ldg(s32), __ldg(s32 + 1), __ldg(s32 + 2), __ldg(s32 + 3));
          }
        }
        sz[tt][kbl] = z;
      }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        uint32_t const j = l16 + 16 * jj;
        bool const ok = live && j < kbs * 8;
        uint64_t const gi = uint64_t(live ? t : 0) * G + s0 * 8 + (ok ? j : 0);
        sa[tt][jj] = ok ? __ldg(x.scales + gi) : 0.f;
        ss[tt][jj] = ok ? __ldg(x.sums + gi) : 0;
      }
    }
  };
  auto stage_store = [&](uint32_t buf) {
    uint8_t* const ab = act + buf * S::kAct1;
    uint8_t* const fb = af + buf * S::kAf1;
#pragma unroll
    for (int tt = 0; tt < kTpt; ++tt) {
      uint32_t const t = (threadIdx.x >> 4) + tt * (kThreads / 16);
      if (t >= Tokens) continue;
#pragma unroll
      for (int kbl = 0; kbl < kStep; ++kbl) {
        uint4 const z = sz[tt][kbl];
        *reinterpret_cast<uint4*>(ab + (kbl * Tokens + t) * kActRow + l16 * 16) =
            make_uint4(even_bytes(z.x, z.y), odd_bytes(z.x, z.y), even_bytes(z.z, z.w), odd_bytes(z.z, z.w));
      }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        float const a = sa[tt][jj], fs = float(ss[tt][jj]);
        *reinterpret_cast<float4*>(fb + ((l16 + 16 * jj) * Tokens + t) * 16) = make_float4(a, a, fs, fs);
      }
    }
  };

  uint32_t cur = 0, use_stage = 0;
  stage_load(kb0, min(uint32_t(kStep), kb1 - kb0));
  stage_store(0);
  __syncthreads();
  for (uint32_t step0 = kb0; step0 < kb1; step0 += kStep) {
    uint32_t const kbs = min(uint32_t(kStep), kb1 - step0);
    uint32_t const next0 = step0 + kStep;
    bool const has_next = next0 < kb1;
    if (has_next) stage_load(next0, min(uint32_t(kStep), kb1 - next0));

    if (active) {
      const uint8_t* const act_lane = act + cur * S::kAct1 + tq * kActRow + c * 8;
      const uint8_t* const af_lane = af + cur * S::kAf1 + tq * 16;
      for (uint32_t kbl = 0; kbl < kbs; ++kbl) {
        uint32_t const kb = step0 + kbl;
        cp_async_wait<kStages - 2>();
        __syncwarp();
        uint8_t* const stage = ring + use_stage * kStageBytes;
        if (++use_stage == kStages) use_stage = 0;
        {
          // lane (r = tq, c): groups c and c+4 of row r -> table[g][r/2] = (D, D', -Mn, -Mn')
          uint4 const cm = *reinterpret_cast<const uint4*>(stage + 1024 + tq * 16);
          float const d = fp16_bits_to_f32(cm.x & 0xffffu), ndmin = -fp16_bits_to_f32(cm.x >> 16);
          uint32_t const sh = c * 8;
          uint32_t const x0 = cm.y >> sh, x1 = cm.z >> sh, x2 = cm.w >> sh;
          // six-bit integers to fp32 through the 1.5 * 2^23 bias: stays off the conversion pipe
          float const sc_a = __uint_as_float(kMagicI | (x0 & 63u)) - kMagicF, mn_a = __uint_as_float(kMagicI | (x1 & 63u)) - kMagicF;
          float const sc_b = __uint_as_float(kMagicI | (x2 & 15u) | ((x0 >> 2) & 0x30u)) - kMagicF;
          float const mn_b = __uint_as_float(kMagicI | ((x2 >> 4) & 15u) | ((x1 >> 2) & 0x30u)) - kMagicF;
          tab_wa[0] = d * sc_a; tab_wa[2] = ndmin * mn_a;
          tab_wb[0] = d * sc_b; tab_wb[2] = ndmin * mn_b;
        }
        uint32_t q[8];
        {
          uint32_t const base = smem_u32(stage);
          uint32_t r4[4];
          ldmatrix_x4(r4, base + ldm_off0);
          q[0] = r4[0]; q[1] = r4[1]; q[2] = r4[2]; q[3] = r4[3];
          ldmatrix_x4(r4, base + ldm_off1);
          q[4] = r4[0]; q[5] = r4[1]; q[6] = r4[2]; q[7] = r4[3];
        }
        __syncwarp();
        const uint8_t* const a_ptr = act_lane + kbl * (Tokens * kActRow);
        const uint8_t* const f_ptr = af_lane + kbl * (8 * Tokens * 16);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint32_t const b0 = q[g] & 0x0f0f0f0fu, b1 = (q[g] >> 4) & 0x0f0f0f0fu;
          float4 const dm = *reinterpret_cast<const float4*>(tab_lane + g * 64);
          uint2 const lo = *reinterpret_cast<const uint2*>(a_ptr + g * 32);
          uint2 hi = make_uint2(0, 0);
          if (Upper) hi = *reinterpret_cast<const uint2*>(a_ptr + 8 * kActRow + g * 32);
          int d4[4];
          mma_s8(d4, lo.x, hi.x, lo.y, hi.y, b0, b1);
          float4 const f0 = *reinterpret_cast<const float4*>(f_ptr + g * (Tokens * 16));
          float2 const D2 = make_float2(dm.x, dm.y), nMn2 = make_float2(dm.z, dm.w);
          float2 const cD2 = mul2(D2, nmagic2);  // exact: D has at most 17 significant bits
          // D * float(P) in one rounding: (P + 1.5*2^23) * D - 1.5*2^23 * D
          float2 t = fma2(make_float2(__uint_as_float(uint32_t(d4[0]) + kMagicI), __uint_as_float(uint32_t(d4[1]) + kMagicI)), D2, cD2);
          t = fma2(nMn2, make_float2(f0.z, f0.w), t);
          acc_lo = fma2(make_float2(f0.x, f0.y), t, acc_lo);
          if (Upper) {
            float4 const f1 = *reinterpret_cast<const float4*>(f_ptr + g * (Tokens * 16) + 8 * 16);
            float2 u = fma2(make_float2(__uint_as_float(uint32_t(d4[2]) + kMagicI), __uint_as_float(uint32_t(d4[3]) + kMagicI)), D2, cD2);
            u = fma2(nMn2, make_float2(f1.z, f1.w), u);
            acc_hi = fma2(make_float2(f1.x, f1.y), u, acc_hi);
          }
          if (Dump) {
#pragma unroll
            for (int l = 0; l < (Upper ? 4 : 2); ++l) {
              uint32_t const token = tq + (l >> 1) * 8, row = rg * 8 + 2 * c + (l & 1);
              if (token < x.m && row < w.n) partials[(uint64_t(token) * w.n + row) * G + kb * 8 + g] = d4[l];
            }
          }
        }
        __syncwarp();
        issue();
      }
    }
    if (has_next) stage_store(cur ^ 1);
    __syncthreads();
    cur ^= 1;
  }
  cp_async_wait<0>();

  auto store = [&](float2 lo2, float2 hi2) {
    if (!active) return;
    float const v[4] = {lo2.x, lo2.y, hi2.x, hi2.y};
#pragma unroll
    for (int l = 0; l < (Upper ? 4 : 2); ++l) {
      uint32_t const token = tq + (l >> 1) * 8, row = rg * 8 + 2 * c + (l & 1);
      if (token < x.m && row < w.n) {
        uint64_t const o = uint64_t(token) * w.n + row;
        out[o] = v[l] + (residual ? residual[o] : 0.f);
      }
    }
  };
  if (split_k == 1) {
    store(acc_lo, acc_hi);
    return;
  }
  // K slices live in the blocks of one cluster: publish, then rank 0 adds them in rank order.
  cg::cluster_group cluster = cg::this_cluster();
  red[threadIdx.x] = make_float4(acc_lo.x, acc_lo.y, acc_hi.x, acc_hi.y);
  cluster.sync();
  if (cluster.block_rank() == 0) {
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r = 0; r < split_k; ++r) {
      const float4* remote = cluster.map_shared_rank(red, r);
      float4 const v = remote[threadIdx.x];
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    store(make_float2(sum.x, sum.y), make_float2(sum.z, sum.w));
  }
  cluster.sync();  // keep every block's shared memory alive until rank 0 has read it
}

template <bool Upper, int Warps>
cudaError_t launch_cfg(const WeightView& w, const Q8View& x, float* out, const float* residual, int32_t* partials,
                       uint32_t split_k, cudaStream_t stream) {
  bool const wide = (reinterpret_cast<uintptr_t>(w.codes) % 16 == 0) && (reinterpret_cast<uintptr_t>(w.meta) % 16 == 0);
  void (*kernel)(WeightView, Q8View, float*, const float*, int32_t*, uint32_t);
  if (partials) kernel = wide ? gemv_mma_kernel<Upper, true, true, Warps> : gemv_mma_kernel<Upper, true, false, Warps>;
  else kernel = wide ? gemv_mma_kernel<Upper, false, true, Warps> : gemv_mma_kernel<Upper, false, false, Warps>;
  constexpr int smem = Smem<Warps, Upper ? 16 : 8>::kTotal;
  cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (st != cudaSuccess) return st;
  uint32_t const row_tiles = (w.padded_n / 8 + Warps - 1) / Warps;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(row_tiles * split_k);
  cfg.blockDim = dim3(Warps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split_k;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, w, x, out, residual, partials, split_k);
}

}  // namespace

GemvMmaPlan plan_gemv_mma(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request, uint32_t warps_request) {
  (void)m;
  GemvMmaPlan p;
  uint32_t const rgs = (n + 7) / 8;
  // Eight row groups per block share one staged activation slice; measured best on every
  // decode shape except very small matrices, where four keep more blocks in flight.
  p.warps = warps_request ? warps_request : (rgs >= 8 * 64 ? 8 : 4);
  uint32_t const row_tiles = (rgs + p.warps - 1) / p.warps;
  uint32_t split = split_k_request;
  if (split == 0) {
    // About two blocks per SM; a slice keeps at least four super-blocks (measured optimum:
    // 1 for 34816 rows, 2 for 7168, 4 for 5120 rows at K = 5120 / 17408).
    split = uint32_t(296.0 / row_tiles + 0.35);
    uint32_t const max_split = tiles_k / 4 ? tiles_k / 4 : 1;
    if (split > max_split) split = max_split;
  }
  if (split > 8) split = 8;  // portable cluster size
  if (split > tiles_k) split = tiles_k;
  if (split < 1) split = 1;
  p.split_k = split;
  return p;
}

cudaError_t launch_gemv_mma(const WeightView& w, const Q8View& x, float* out, const float* residual,
                            int32_t* partials, const GemvMmaPlan& plan, cudaStream_t stream) {
  if (x.m > 16) return cudaErrorInvalidValue;
  bool const upper = x.m > 8;
  if (plan.warps == 8) {
    return upper ? launch_cfg<true, 8>(w, x, out, residual, partials, plan.split_k, stream)
                 : launch_cfg<false, 8>(w, x, out, residual, partials, plan.split_k, stream);
  }
  return upper ? launch_cfg<true, 4>(w, x, out, residual, partials, plan.split_k, stream)
               : launch_cfg<false, 4>(w, x, out, residual, partials, plan.split_k, stream);
}

}  // namespace q4k
