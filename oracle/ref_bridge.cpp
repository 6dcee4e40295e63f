// C-ABI bridge onto the reference engine's OWN host code, used only to pin the
// CPU oracle (oracle/q4k_oracle.c) and to generate golden vectors.
//
// TEST INFRASTRUCTURE ONLY.  Nothing in the CUDA library links this file.
//
// It is compiled, by oracle/Makefile, together with the reference sources where
// they lie in the reference checkout (never copied into this repository):
//   src/format/{error,constants,wire,layout,schema,sha256,pack,unpack}.cpp
//   src/compiler/error.cpp, src/compiler/quantization/{q4k,reference,quantizer}.cpp
//   third_party/llama.cpp-q4k/reference.hpp (header only)
// The output is oracle/_ref/libqw38_ref.so.  The checkout is not present on a
// GPU machine; the tests that use this library skip when it cannot be loaded and
// rely on the golden vectors generated from it (tests/golden/).
#include "compiler/quantization/q4k.hpp"
#include "compiler/quantization/reference.hpp"
#include "format/floatcvt.hpp"
#include "format/logical.hpp"
#include "format/pack.hpp"
#include "format/unpack.hpp"
#include "third_party/llama.cpp-q4k/reference.hpp"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <span>
#include <vector>

namespace {
using namespace qw38;

format::LogicalWeightCodes logical_q4k(std::int8_t const* codes, std::uint8_t const* meta,
                                       std::uint64_t n, std::uint64_t k) {
  format::LogicalWeightCodes l{.quantizer = format::LogicalQuantizerId::Q4KCandidateV2,
                               .n = n, .k = k, .group_size = 256, .qmax = 15};
  l.codes.assign(codes, codes + n * k);
  l.q4k_metadata.assign(meta, meta + n * (k / 256) * 16);
  return l;
}
}  // namespace

extern "C" {

// format::pack_cuda_v0 for the Q4_K split-tile layout (src/format/pack.cpp:80-245).
// k must be a multiple of 256.  Returns 0 on success.
int ref_pack_q4k(std::int8_t const* codes, std::uint8_t const* meta, std::uint64_t n,
                 std::uint64_t k, std::uint8_t* out_codes, std::uint64_t out_codes_bytes,
                 std::uint8_t* out_scales, std::uint64_t out_scales_bytes) {
  auto packed = format::pack_cuda_v0(format::LogicalQuantizerId::Q4KCandidateV2,
                                     format::PhysicalLayoutId::CudaQ4KCandidateV2,
                                     logical_q4k(codes, meta, n, k));
  if (!packed) return 1;
  if (packed->codes.size() != out_codes_bytes || packed->scales.size() != out_scales_bytes) return 2;
  std::memcpy(out_codes, packed->codes.data(), out_codes_bytes);
  std::memcpy(out_scales, packed->scales.data(), out_scales_bytes);
  return 0;
}

// format::validate_cuda_v0 (src/format/unpack.cpp:89-260): 0 when the packed
// domain is admissible, 1 otherwise.
int ref_validate_q4k(std::uint64_t n, std::uint64_t k, std::uint8_t const* codes,
                     std::uint64_t codes_bytes, std::uint8_t const* scales,
                     std::uint64_t scales_bytes) {
  auto st = format::validate_cuda_v0(
      format::LogicalQuantizerId::Q4KCandidateV2, format::PhysicalLayoutId::CudaQ4KCandidateV2, n, k,
      {reinterpret_cast<std::byte const*>(codes), codes_bytes},
      {reinterpret_cast<std::byte const*>(scales), scales_bytes});
  return st ? 0 : 1;
}

// The same with the offence located: 0 admissible; 1 "quantized.codes.padding", 2 "quantized.scales.padding",
// 3 "quantized.scales" (9 anything else); *offset = the error's byte offset inside its span.
int ref_validate_q4k_where(std::uint64_t n, std::uint64_t k, std::uint8_t const* codes,
                           std::uint64_t codes_bytes, std::uint8_t const* scales,
                           std::uint64_t scales_bytes, std::uint64_t* offset) {
  auto st = format::validate_cuda_v0(
      format::LogicalQuantizerId::Q4KCandidateV2, format::PhysicalLayoutId::CudaQ4KCandidateV2, n, k,
      {reinterpret_cast<std::byte const*>(codes), codes_bytes},
      {reinterpret_cast<std::byte const*>(scales), scales_bytes});
  *offset = 0;
  if (st) return 0;
  *offset = st.error().offset;
  if (st.error().field == "quantized.codes.padding") return 1;
  if (st.error().field == "quantized.scales.padding") return 2;
  if (st.error().field == "quantized.scales") return 3;
  return 9;
}

// format::unpack_cuda_v0 (src/format/unpack.cpp:262-380).
int ref_unpack_q4k(std::uint64_t n, std::uint64_t k, std::uint8_t const* codes,
                   std::uint64_t codes_bytes, std::uint8_t const* scales,
                   std::uint64_t scales_bytes, std::int8_t* out_codes, std::uint8_t* out_meta) {
  auto l = format::unpack_cuda_v0(
      format::LogicalQuantizerId::Q4KCandidateV2, format::PhysicalLayoutId::CudaQ4KCandidateV2, n, k,
      {reinterpret_cast<std::byte const*>(codes), codes_bytes},
      {reinterpret_cast<std::byte const*>(scales), scales_bytes});
  if (!l) return 1;
  std::memcpy(out_codes, l->codes.data(), l->codes.size());
  std::memcpy(out_meta, l->q4k_metadata.data(), l->q4k_metadata.size());
  return 0;
}

// compiler::reference_gemv_packed (src/compiler/quantization/reference.cpp:250-279):
// unpack -> dequantise to bf16 -> sequential fp32 GEMV.  x is bf16 bits [k].
int ref_gemv_packed_q4k(std::uint64_t n, std::uint64_t k, std::uint8_t const* codes,
                        std::uint64_t codes_bytes, std::uint8_t const* scales,
                        std::uint64_t scales_bytes, std::uint16_t const* x, float* y) {
  format::PackedMatrix p;
  p.layout = format::PhysicalLayoutId::CudaQ4KCandidateV2;
  p.quantizer = format::LogicalQuantizerId::Q4KCandidateV2;
  p.logical_n = n; p.logical_k = k;
  p.padded_n = format::dense_pad_n(n); p.padded_k = format::dense_pad_k(k);
  p.codes.assign(reinterpret_cast<std::byte const*>(codes),
                 reinterpret_cast<std::byte const*>(codes) + codes_bytes);
  p.scales.assign(reinterpret_cast<std::byte const*>(scales),
                  reinterpret_cast<std::byte const*>(scales) + scales_bytes);
  auto r = compiler::reference_gemv_packed(p, std::span<std::uint16_t const>(x, k));
  if (!r) return 1;
  std::copy(r->begin(), r->end(), y);
  return 0;
}

// compiler::dequantize_to_bf16 (src/compiler/quantization/reference.cpp:124-166).
int ref_dequantize_bf16(std::int8_t const* codes, std::uint8_t const* meta, std::uint64_t n,
                        std::uint64_t k, std::uint16_t* out) {
  auto r = compiler::dequantize_to_bf16(logical_q4k(codes, meta, n, k));
  if (!r) return 1;
  std::copy(r->begin(), r->end(), out);
  return 0;
}

// compiler::quantize_q4k_block (src/compiler/quantization/q4k.cpp:186-278).
int ref_quantize_q4k_block(float const* w256, std::int8_t* codes256, std::uint8_t* meta16) {
  auto st = compiler::quantize_q4k_block(std::span<float const, 256>(w256, 256),
                                         std::span<std::int8_t, 256>(codes256, 256),
                                         std::span<std::uint8_t, 16>(meta16, 16));
  return st ? 0 : 1;
}

// The same over `blocks` consecutive 256-weight blocks, every block attempted.  status[b] = 0 when
// block b was fitted, else the refusal by its message: 1 nonfinite input, 2 fitting range exceeded,
// 3 fitting reciprocal overflow, 4 compression reciprocal overflow, 5 FP16 scale overflow (9 = other).
// Refused blocks are left as zeros.  Returns the number of refused blocks.
std::uint64_t ref_quantize_q4k_blocks(float const* w, std::uint64_t blocks, std::int8_t* codes,
                                      std::uint8_t* meta, std::uint8_t* status) {
  static constexpr char const* kMessages[5] = {
      "Q4_K input is nonfinite", "Q4_K fitting range exceeded", "Q4_K fitting reciprocal overflow",
      "Q4_K compression reciprocal overflow", "Q4_K FP16 scale overflow"};
  std::uint64_t refused = 0;
  for (std::uint64_t b = 0; b < blocks; ++b) {
    std::int8_t c[256] = {};
    std::uint8_t m[16] = {};
    auto st = compiler::quantize_q4k_block(std::span<float const, 256>(w + b * 256, 256),
                                           std::span<std::int8_t, 256>(c, 256),
                                           std::span<std::uint8_t, 16>(m, 16));
    status[b] = 0;
    if (!st) {
      ++refused;
      status[b] = 9;
      for (int i = 0; i < 5; ++i)
        if (st.error().detail == kMessages[i]) status[b] = static_cast<std::uint8_t>(i + 1);
      std::memset(c, 0, sizeof c);
      std::memset(m, 0, sizeof m);
    }
    std::memcpy(codes + b * 256, c, 256);
    std::memcpy(meta + b * 16, m, 16);
  }
  return refused;
}

// Pinned upstream bodies (third_party/llama.cpp-q4k/reference.hpp:183-275):
// 144-byte super-blocks from floats, and floats back.
void ref_llama_quantize_row_q4k(float const* x, std::uint8_t* blocks144, std::int64_t k) {
  std::vector<pinned_llama_q4k::block_q4_K> b(static_cast<std::size_t>(k / 256));
  std::memset(b.data(), 0, b.size() * 144);
  pinned_llama_q4k::quantize_row_q4_K_ref(x, b.data(), k);
  std::memcpy(blocks144, b.data(), b.size() * 144);
}
void ref_llama_dequantize_row_q4k(std::uint8_t const* blocks144, float* y, std::int64_t k) {
  std::vector<pinned_llama_q4k::block_q4_K> b(static_cast<std::size_t>(k / 256));
  std::memcpy(b.data(), blocks144, b.size() * 144);
  pinned_llama_q4k::dequantize_row_q4_K(b.data(), y, k);
}
void ref_llama_scale_min(int j, std::uint8_t const* q12, std::uint8_t* sc, std::uint8_t* mn) {
  pinned_llama_q4k::get_scale_min_k4(j, q12, sc, mn);
}

// src/format/floatcvt.hpp conversions.
float ref_fp16_to_fp32(std::uint16_t h) { return format::fp16_to_fp32(h); }
float ref_bf16_to_fp32(std::uint16_t h) { return format::bf16_to_fp32(h); }
std::uint16_t ref_fp32_to_bf16(float f) { return format::fp32_to_bf16_rne(f); }

}  // extern "C"
