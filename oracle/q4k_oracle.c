/*
 * CPU oracle for the Q4_K weight x Q8 (32-wide) activation matmul.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker: the tests, the smoke
 * check and the benchmark's CPU-baseline leg call it; the CUDA library never
 * links or falls back to it.
 *
 * It restates, in plain C, the equation the reference engine states in its
 * own tests and device code:
 *   - activation quantiser: cuda/q8_device.cuh:5-25 (rounding authority) and
 *     tests/q4k_q8_test.cpp:83-92 (independent CPU statement);
 *   - Q4_K scale/min decode: third_party/llama.cpp-q4k/reference.hpp:174-181
 *     (get_scale_min_k4), identical in cuda/q4k_q8.cu:30-38;
 *   - affine contraction, accumulated in double:
 *     tests/q8_mlp_integration_test.cpp:21-45 and tests/q4k_q8_test.cpp:121-131;
 *   - split-tile physical layout: src/format/pack.cpp:175-222;
 *   - 144-byte super-block element order:
 *     third_party/llama.cpp-q4k/reference.hpp:244-248,253-275.
 *
 * Parity pins: oracle/ref_bridge.cpp compiles the reference's own host sources
 * (pack/unpack, Q4_K fitter, pinned dequantiser, bf16 GEMV); tests/test_oracle_pins.py
 * checks this file against them and against the literals of tests/q4k_q8_test.cpp.
 *
 * Build with -ffp-contract=off: the float expressions below must round exactly
 * as the reference's host tests do (src/CMakeLists.txt:35-37 sets the same flag).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* fp16 -> fp32, subnormals included (same values as src/format/floatcvt.hpp:18-44). */
float orc_fp16_to_fp32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  if (e == 0) {
    if (m == 0) return bits_f32(sign);
    float v = ldexpf((float)m, -24);
    return sign ? -v : v;
  }
  if (e == 31) return bits_f32(sign | 0x7F800000u | (m << 13));
  return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* fp32 -> fp16 round-to-nearest-even (finite inputs in range; overflow -> inf). */
uint16_t orc_fp32_to_fp16(float f) {
  uint32_t b = f32_bits(f), sign = (b >> 16) & 0x8000u;
  uint32_t a = b & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
  if (a >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* >= 65536 -> inf (65520 rounds up too) */
  float af = bits_f32(a);
  if (af >= 65520.0f) return (uint16_t)(sign | 0x7C00u);
  if (af < 6.103515625e-05f) { /* subnormal half: units of 2^-24 */
    float q = af * 16777216.0f;
    uint32_t r = (uint32_t)lrintf(q); /* RNE under default rounding mode */
    return (uint16_t)(sign | r);
  }
  uint32_t e = (a >> 23) - 112u, man = a & 0x7FFFFFu;
  uint32_t half = (e << 10) | (man >> 13);
  uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
  return (uint16_t)(sign | half);
}

float orc_bf16_to_fp32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* fp32 -> bf16 RNE (NaN kept quiet). */
uint16_t orc_fp32_to_bf16(float f) {
  uint32_t b = f32_bits(f);
  if ((b & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((b >> 16) | 0x40u);
  uint32_t lsb = (b >> 16) & 1u;
  b += 0x7FFFu + lsb;
  return (uint16_t)(b >> 16);
}

/* 6-bit scale / min of sub-block g (0..7) from the 12 packed bytes
 * (third_party/llama.cpp-q4k/reference.hpp:174-181). */
static inline void scale_min(const uint8_t* p, unsigned g, unsigned* sc, unsigned* mn) {
  if (g < 4) { *sc = p[g] & 63u; *mn = p[g + 4] & 63u; }
  else {
    *sc = (p[g + 4] & 15u) | ((unsigned)(p[g - 4] >> 6) << 4);
    *mn = (unsigned)(p[g + 4] >> 4) | ((unsigned)(p[g] >> 6) << 4);
  }
}

void orc_scale_min(const uint8_t* p12, uint8_t* sc8, uint8_t* mn8) {
  for (unsigned g = 0; g < 8; ++g) { unsigned s, m; scale_min(p12, g, &s, &m); sc8[g] = (uint8_t)s; mn8[g] = (uint8_t)m; }
}

/* Inverse of scale_min: pack eight 6-bit scales and mins into 12 bytes. */
void orc_pack_scale_min(const uint8_t* sc8, const uint8_t* mn8, uint8_t* p12) {
  memset(p12, 0, 12);
  for (unsigned g = 0; g < 8; ++g) {
    unsigned s = sc8[g] & 63u, m = mn8[g] & 63u;
    if (g < 4) { p12[g] |= (uint8_t)s; p12[g + 4] |= (uint8_t)m; }
    else {
      p12[g + 4] |= (uint8_t)((s & 15u) | ((m & 15u) << 4));
      p12[g - 4] |= (uint8_t)((s >> 4) << 6);
      p12[g] |= (uint8_t)((m >> 4) << 6);
    }
  }
}

static inline uint64_t tile_row(uint64_t row, uint64_t kb, uint64_t tiles_k) {
  return ((row / 8) * tiles_k + kb) * 8 + row % 8; /* src/format/pack.cpp:181-182 */
}

/* ------------------------------------------------------------------------ */
/* Q8 activation quantiser                                                   */
/* ------------------------------------------------------------------------ */

/* One row of k floats -> padded_k codes, padded_k/32 scales and sums.
 * Columns >= k are zeros and do not raise the peak (cuda/q4k_q8.cu:48).
 * A group holding any non-finite value, or whose scale is not a positive
 * finite number, gets zero codes, a NaN scale, sum 0, and raises *failure
 * (cuda/q8_device.cuh:12-23). */
static void q8_row(const float* x, unsigned k, unsigned padded_k, int8_t* codes,
                   float* scales, int32_t* sums, int* failure) {
  for (unsigned g = 0; g < padded_k / 32; ++g) {
    float v[32]; int finite = 1; float peak = 0.f;
    for (unsigned t = 0; t < 32; ++t) {
      unsigned c = g * 32 + t;
      v[t] = c < k ? x[c] : 0.f;
      if (!isfinite(v[t])) finite = 0; else if (fabsf(v[t]) > peak) peak = fabsf(v[t]);
    }
    float a = peak == 0.f ? 1.f : peak / 127.f;
    int valid = finite && isfinite(a) && a > 0.f;
    int32_t sum = 0;
    for (unsigned t = 0; t < 32; ++t) {
      int z = 0;
      if (valid) {
        float q = nearbyintf(v[t] / a); /* RNE, as __float2int_rn */
        z = q > 127.f ? 127 : q < -127.f ? -127 : (int)q;
      }
      codes[g * 32 + t] = (int8_t)z; sum += z;
    }
    scales[g] = valid ? a : bits_f32(0x7fc00000u);
    sums[g] = sum;
    if (!valid) *failure = 1;
  }
}

void orc_q8_quantize_f32(const float* x, unsigned m, unsigned k, unsigned padded_k,
                         int8_t* codes, float* scales, int32_t* sums, int* failure) {
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (unsigned r = 0; r < m; ++r) {
    int f = 0;
    q8_row(x + (size_t)r * k, k, padded_k, codes + (size_t)r * padded_k,
           scales + (size_t)r * (padded_k / 32), sums + (size_t)r * (padded_k / 32), &f);
    bad |= f;
  }
  if (bad) *failure = 1;
}

void orc_q8_quantize_bf16(const uint16_t* x, unsigned m, unsigned k, unsigned padded_k,
                          int8_t* codes, float* scales, int32_t* sums, int* failure) {
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (unsigned r = 0; r < m; ++r) {
    float* row = (float*)malloc((size_t)k * 4);
    for (unsigned c = 0; c < k; ++c) row[c] = orc_bf16_to_fp32(x[(size_t)r * k + c]);
    int f = 0;
    q8_row(row, k, padded_k, codes + (size_t)r * padded_k,
           scales + (size_t)r * (padded_k / 32), sums + (size_t)r * (padded_k / 32), &f);
    bad |= f; free(row);
  }
  if (bad) *failure = 1;
}

/* "Q8_1" wire form named by the benchmark configs: per 32 values a 36-byte
 * record {fp16 d, fp16 s, int8 q[32]}.  The upstream struct is not part of the
 * reference tree, so this build defines d = fp16_rn(a) and s = fp16_rn(a * sum)
 * from the exact fp32 scale and int32 sum. */
void orc_q8_1_export(const int8_t* codes, const float* scales, const int32_t* sums,
                     uint64_t groups, uint8_t* out36) {
  for (uint64_t g = 0; g < groups; ++g) {
    uint16_t d = orc_fp32_to_fp16(scales[g]);
    uint16_t s = orc_fp32_to_fp16(scales[g] * (float)sums[g]);
    uint8_t* o = out36 + g * 36;
    o[0] = (uint8_t)(d & 255u); o[1] = (uint8_t)(d >> 8); o[2] = (uint8_t)(s & 255u); o[3] = (uint8_t)(s >> 8);
    memcpy(o + 4, codes + g * 32, 32);
  }
}

/* ------------------------------------------------------------------------ */
/* Weight layouts                                                            */
/* ------------------------------------------------------------------------ */

/* Logical (row-major codes 0..15 [n][k], metadata [n][ceil256(k)/256][16]) -> split
 * tiles with zero padding to (ceil8 n, ceil256 k), src/format/pack.cpp:175-222.
 * k need not be a multiple of 256: the reference test builds its logical matrix
 * with k already padded and zero codes in the tail (tests/q4k_q8_test.cpp:38-47),
 * which is the same thing. */
void orc_pack_split(const int8_t* codes, const uint8_t* meta, uint64_t n, uint64_t k,
                                uint8_t* out_codes, uint8_t* out_meta) {
  uint64_t pn = (n + 7) / 8 * 8, pk = (k + 255) / 256 * 256, tiles_k = pk / 256;
  memset(out_codes, 0, pn * pk / 2);
  memset(out_meta, 0, pn * tiles_k * 16);
  for (uint64_t row = 0; row < n; ++row)
    for (uint64_t kb = 0; kb < tiles_k; ++kb) {
      uint64_t tr = tile_row(row, kb, tiles_k);
      memcpy(out_meta + tr * 16, meta + (row * tiles_k + kb) * 16, 16);
      for (unsigned c = 0; c < 256; c += 2) {
        uint64_t col = kb * 256 + c;
        unsigned lo = col < k ? (unsigned)codes[row * k + col] : 0u;
        unsigned hi = col + 1 < k ? (unsigned)codes[row * k + col + 1] : 0u;
        out_codes[tr * 128 + c / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
}

/* 144-byte super-blocks [n][k/256] (k % 256 == 0) -> logical codes + metadata.
 * Element 64c+l is the low nibble of qs[32c+l], element 64c+32+l its high
 * nibble (third_party/llama.cpp-q4k/reference.hpp:253-275). */
void orc_blocks144_to_logical(const uint8_t* blocks, uint64_t n, uint64_t k,
                              int8_t* codes, uint8_t* meta) {
  uint64_t nb = k / 256;
  for (uint64_t b = 0; b < n * nb; ++b) {
    const uint8_t* blk = blocks + b * 144;
    memcpy(meta + b * 16, blk, 16);
    const uint8_t* qs = blk + 16;
    for (unsigned c = 0; c < 4; ++c)
      for (unsigned l = 0; l < 32; ++l) {
        codes[b * 256 + 64 * c + l] = (int8_t)(qs[32 * c + l] & 15u);
        codes[b * 256 + 64 * c + 32 + l] = (int8_t)(qs[32 * c + l] >> 4);
      }
  }
}

void orc_logical_to_blocks144(const int8_t* codes, const uint8_t* meta, uint64_t n, uint64_t k,
                              uint8_t* blocks) {
  uint64_t nb = k / 256;
  for (uint64_t b = 0; b < n * nb; ++b) {
    uint8_t* blk = blocks + b * 144;
    memcpy(blk, meta + b * 16, 16);
    for (unsigned c = 0; c < 4; ++c)
      for (unsigned l = 0; l < 32; ++l)
        blk[16 + 32 * c + l] = (uint8_t)((unsigned)codes[b * 256 + 64 * c + l] |
                                         ((unsigned)codes[b * 256 + 64 * c + 32 + l] << 4));
  }
}

/* 144-byte super-blocks -> split tiles directly (n padded to 8 with zero rows). */
void orc_blocks144_to_split(const uint8_t* blocks, uint64_t n, uint64_t k,
                            uint8_t* out_codes, uint8_t* out_meta) {
  int8_t* codes = (int8_t*)malloc(n * k);
  uint8_t* meta = (uint8_t*)malloc(n * (k / 256) * 16);
  orc_blocks144_to_logical(blocks, n, k, codes, meta);
  orc_pack_split(codes, meta, n, k, out_codes, out_meta);
  free(codes); free(meta);
}

/* Weight code of logical element (row, col) in split tiles. */
static inline int split_code(const uint8_t* wc, uint64_t tiles_k, uint64_t row, uint64_t col) {
  uint64_t tr = tile_row(row, col / 256, tiles_k);
  uint8_t b = wc[tr * 128 + (col % 256) / 2];
  return (col & 1u) ? (b >> 4) : (b & 15u);
}

/* ------------------------------------------------------------------------ */
/* Contraction                                                               */
/* ------------------------------------------------------------------------ */

/* Exact integer partials: dots[(t*n + row)*G + g] = sum_{i<32} q[row][32g+i] * z[t][32g+i],
 * G = padded_k/32.  |dot| <= 60960 (cuda/q4k_q8.hpp:23). */
void orc_q4k_q8_dots(const uint8_t* wcodes, unsigned n, unsigned padded_k,
                     const int8_t* z, unsigned m, int32_t* dots) {
  unsigned G = padded_k / 32, tiles_k = padded_k / 256;
#pragma omp parallel for schedule(static)
  for (unsigned row = 0; row < n; ++row) {
    int8_t* q = (int8_t*)malloc(padded_k);
    for (unsigned c = 0; c < padded_k; ++c) q[c] = (int8_t)split_code(wcodes, tiles_k, row, c);
    for (unsigned t = 0; t < m; ++t) {
      const int8_t* zt = z + (size_t)t * padded_k;
      for (unsigned g = 0; g < G; ++g) {
        int32_t d = 0;
        for (unsigned i = 0; i < 32; ++i) d += (int32_t)q[g * 32 + i] * (int32_t)zt[g * 32 + i];
        dots[((size_t)t * n + row) * G + g] = d;
      }
    }
    free(q);
  }
}

/* out[t*n + row] = float( sum_g double( a[t,g] * ((d*sc)*dot - (dmin*mn)*sum[t,g]) ) ) (+ residual),
 * inner expression in fp32 without contraction, accumulation in double
 * (tests/q8_mlp_integration_test.cpp:30-44).  out64, when non-null, receives the
 * unrounded double accumulator (without residual). */
void orc_q4k_q8_project(const uint8_t* wcodes, const uint8_t* wmeta, unsigned n, unsigned padded_k,
                        const int8_t* z, const float* a, const int32_t* sums, unsigned m,
                        const float* residual, float* out, double* out64) {
  unsigned G = padded_k / 32, tiles_k = padded_k / 256;
#pragma omp parallel for schedule(dynamic, 16)
  for (unsigned row = 0; row < n; ++row) {
    int8_t* q = (int8_t*)malloc(padded_k);
    float* D = (float*)malloc(G * 4); float* Mn = (float*)malloc(G * 4);
    for (unsigned c = 0; c < padded_k; ++c) q[c] = (int8_t)split_code(wcodes, tiles_k, row, c);
    for (unsigned kb = 0; kb < tiles_k; ++kb) {
      const uint8_t* meta = wmeta + tile_row(row, kb, tiles_k) * 16;
      float d = orc_fp16_to_fp32((uint16_t)(meta[0] | (meta[1] << 8)));
      float dm = orc_fp16_to_fp32((uint16_t)(meta[2] | (meta[3] << 8)));
      for (unsigned g = 0; g < 8; ++g) {
        unsigned sc, mn; scale_min(meta + 4, g, &sc, &mn);
        D[kb * 8 + g] = d * (float)sc; Mn[kb * 8 + g] = dm * (float)mn;
      }
    }
    for (unsigned t = 0; t < m; ++t) {
      const int8_t* zt = z + (size_t)t * padded_k;
      double acc = 0;
      for (unsigned g = 0; g < G; ++g) {
        int32_t dot = 0;
        for (unsigned i = 0; i < 32; ++i) dot += (int32_t)q[g * 32 + i] * (int32_t)zt[g * 32 + i];
        float s = a[(size_t)t * G + g];
        float term = s * (D[g] * (float)dot - Mn[g] * (float)sums[(size_t)t * G + g]);
        acc += term;
      }
      size_t o = (size_t)t * n + row;
      if (out64) out64[o] = acc;
      out[o] = (float)acc + (residual ? residual[o] : 0.f);
    }
    free(q); free(D); free(Mn);
  }
}

/* Rows [row0, row0+rows) only; out is [m][rows].  Used for sampled checks at
 * full benchmark sizes and by the timed CPU baseline. */
void orc_q4k_q8_project_rows(const uint8_t* wcodes, const uint8_t* wmeta, unsigned n, unsigned padded_k,
                             const int8_t* z, const float* a, const int32_t* sums, unsigned m,
                             unsigned row0, unsigned rows, float* out) {
  unsigned G = padded_k / 32, tiles_k = padded_k / 256;
  (void)n;
#pragma omp parallel for schedule(dynamic, 16)
  for (unsigned r = 0; r < rows; ++r) {
    unsigned row = row0 + r;
    int8_t* q = (int8_t*)malloc(padded_k);
    float* D = (float*)malloc(G * 4); float* Mn = (float*)malloc(G * 4);
    for (unsigned c = 0; c < padded_k; ++c) q[c] = (int8_t)split_code(wcodes, tiles_k, row, c);
    for (unsigned kb = 0; kb < tiles_k; ++kb) {
      const uint8_t* meta = wmeta + tile_row(row, kb, tiles_k) * 16;
      float d = orc_fp16_to_fp32((uint16_t)(meta[0] | (meta[1] << 8)));
      float dm = orc_fp16_to_fp32((uint16_t)(meta[2] | (meta[3] << 8)));
      for (unsigned g = 0; g < 8; ++g) {
        unsigned sc, mn; scale_min(meta + 4, g, &sc, &mn);
        D[kb * 8 + g] = d * (float)sc; Mn[kb * 8 + g] = dm * (float)mn;
      }
    }
    for (unsigned t = 0; t < m; ++t) {
      const int8_t* zt = z + (size_t)t * padded_k;
      double acc = 0;
      for (unsigned g = 0; g < G; ++g) {
        int32_t dot = 0;
        for (unsigned i = 0; i < 32; ++i) dot += (int32_t)q[g * 32 + i] * (int32_t)zt[g * 32 + i];
        float s = a[(size_t)t * G + g];
        acc += s * (D[g] * (float)dot - Mn[g] * (float)sums[(size_t)t * G + g]);
      }
      out[(size_t)t * rows + r] = (float)acc;
    }
    free(q); free(D); free(Mn);
  }
}

/* ------------------------------------------------------------------------ */
/* Producers around the matmul                                               */
/* ------------------------------------------------------------------------ */

/* v = bf16_rne(silu(g) * u), NaN when g or u is non-finite (cuda/q4k_q8.cu:52-60).
 * expf here is the host libm; the device kernel uses CUDA's expf, so results
 * can differ by one bf16 ulp on rare ties -- compare at bf16 tolerance. */
void orc_swiglu_bf16(const float* gate, const float* up, uint64_t count, uint16_t* out) {
  for (uint64_t i = 0; i < count; ++i) {
    float g = gate[i], u = up[i];
    float v = (g / (1.f + expf(-g))) * u;
    if (!isfinite(g) || !isfinite(u)) v = bits_f32(0x7fc00000u);
    out[i] = orc_fp32_to_bf16(v);
  }
}

/* Max-scaled RMS norm with (1 + gamma), rounded to bf16 (cuda/activation.cu:150-175).
 * The device kernel sums squares in a block tree; this sums sequentially in
 * double and rounds once, so compare at bf16 tolerance. */
void orc_hidden_rms_bf16(const float* x, const uint16_t* gamma, float eps, unsigned m, unsigned h,
                         uint16_t* out) {
  for (unsigned r = 0; r < m; ++r) {
    const float* row = x + (size_t)r * h;
    float scale = 0.f;
    for (unsigned i = 0; i < h; ++i) if (fabsf(row[i]) > scale) scale = fabsf(row[i]);
    float safe = scale == 0.f ? 1.f : scale;
    double ss = 0;
    for (unsigned i = 0; i < h; ++i) { float s = row[i] / safe; ss += (double)(s * s); }
    float sumsq = (float)ss;
    float se = sqrtf(eps) / safe;
    float inv = 1.0f / sqrtf(sumsq / (float)h + se * se);
    for (unsigned i = 0; i < h; ++i) {
      float g = orc_bf16_to_fp32(gamma[i]);
      float v = (1.0f + g) * ((row[i] / safe) * inv);
      out[(size_t)r * h + i] = orc_fp32_to_bf16(v);
    }
  }
}

/* ------------------------------------------------------------------------ */
/* bf16-operand GEMV of the older decode policy                              */
/* ------------------------------------------------------------------------ */

/* w = bf16_rne((d*sc)*q - dmin*mn); y[row] = sum_k w*x in fp32, sequential
 * (src/compiler/quantization/reference.cpp:140-163,230-247). */
void orc_q4k_bf16_gemv(const uint8_t* wcodes, const uint8_t* wmeta, unsigned n, unsigned k,
                       unsigned padded_k, const uint16_t* x_bf16, float* y) {
  unsigned tiles_k = padded_k / 256;
#pragma omp parallel for schedule(static)
  for (unsigned row = 0; row < n; ++row) {
    float acc = 0.f;
    for (unsigned col = 0; col < k; ++col) {
      unsigned kb = col / 256, g = (col % 256) / 32;
      const uint8_t* meta = wmeta + tile_row(row, kb, tiles_k) * 16;
      float d = orc_fp16_to_fp32((uint16_t)(meta[0] | (meta[1] << 8)));
      float dm = orc_fp16_to_fp32((uint16_t)(meta[2] | (meta[3] << 8)));
      unsigned sc, mn; scale_min(meta + 4, g, &sc, &mn);
      float decoded = (d * (float)sc) * (float)split_code(wcodes, tiles_k, row, col) - dm * (float)mn;
      float w = orc_bf16_to_fp32(orc_fp32_to_bf16(decoded));
      acc += w * orc_bf16_to_fp32(x_bf16[col]);
    }
    y[row] = acc;
  }
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the OpenMP team size for the calls that follow (a launcher may export OMP_NUM_THREADS=1 to every
 * rank; the timed CPU baseline wants all host cores whatever the environment says).  Returns the size in
 * effect afterwards. */
int orc_set_threads(int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
  return omp_get_max_threads();
#else
  (void)threads;
  return 1;
#endif
}
