// C++23 host-side shim over the C ABI of q4k_b200.h.
//
// Mirrors the operator interface of the reference engine for this path -- cuda/q4k_q8.hpp:14-49
// (Q8Input, pack_q8, q4k_q8_project, q4k_q8_mlp, q8_mlp_workspace_bytes), cuda/prefill.hpp:33-44
// (PrefillWeight) and cuda/decode_mmv.hpp:45-51,103-121,207-215 (DecodeEpilogue, DecodeMmvDesc,
// launch_decode_mmv / _paired / _ranges) and, for the offline step, compiler::quantize_q4k_block
// (src/compiler/quantization/q4k.hpp) as a batched device call -- with the same names, argument meaning and error
// behaviour: every call returns std::expected<void, Error>, Error carries the reference's
// ErrorCode (cuda/error.hpp:13-26), a rejected call has launched nothing.  The types live in
// namespace q4k_b200::shim so that the header can be compiled next to the reference's own; a
// maintainer who swaps the implementation forwards the reference types field by field instead
// (they are laid out alike).  Header-only; link libq4k_b200.so.
#pragma once

#include <cstddef>
#include <cstdint>
#include <expected>
#include <span>
#include <string>
#include <utility>

#include "q4k_b200.h"

namespace q4k_b200::shim {

enum class ErrorCode : std::uint16_t { Status = 1, InvalidArgument = 2, Overflow = 3 };

struct Error {
  ErrorCode code{ErrorCode::Status};
  int cuda_status{0};
  std::string operation;
  std::string detail;
  friend bool operator==(Error const&, Error const&) = default;
};

// The reference passes its Stream object; here the native handle (cudaStream_t) is enough.
struct Stream {
  void* native{nullptr};
};

struct PrefillWeight {
  void const* codes{};
  void const* scales{};
  std::uint16_t layout{Q4K_LAYOUT_SPLIT_TILES};
  std::uint16_t quantizer{Q4K_QUANTIZER_Q4K};
  std::uint32_t n{}, k{}, padded_n{}, padded_k{};
  std::uint64_t codes_bytes{}, scales_bytes{};
};

struct Q8Input {
  std::span<std::int8_t> codes;
  std::span<float> scales;
  std::span<std::int32_t> sums;
  unsigned m{}, k{}, padded_k{};
};

inline constexpr int kQ4KQ8DotBound = 32 * 15 * 127;
inline constexpr int kQ8SumBound = 32 * 127;

[[nodiscard]] inline std::uint64_t q8_mlp_workspace_bytes(unsigned m, unsigned hidden = 5120, unsigned ffn = 17408) {
  return q4k_q8_mlp_workspace_bytes(m, hidden, ffn);
}

namespace detail {
inline q4k_weight to_abi(PrefillWeight const& w) {
  return {w.codes, w.scales, w.layout, w.quantizer, w.n, w.k, w.padded_n, w.padded_k, w.codes_bytes, w.scales_bytes};
}
inline q4k_q8_input to_abi(Q8Input const& x) {
  return {x.codes.data(), x.scales.data(), x.sums.data(), x.codes.size(), x.scales.size(), x.sums.size(), x.m, x.k, x.padded_k};
}
inline std::expected<void, Error> lift(int status, char const* operation) {
  if (status == Q4K_OK) return {};
  return std::unexpected(Error{static_cast<ErrorCode>(status), q4k_last_cuda_status(), operation, q4k_last_error()});
}
}  // namespace detail

// ---- cuda/q4k_q8.hpp ----------------------------------------------------------------------------

// failure: one int in device memory, set to 1 by any quantiser warp that meets non-finite data.
[[nodiscard]] inline std::expected<void, Error> pack_q8(std::span<std::uint16_t const> input, Q8Input output,
                                                        std::span<int> failure, Stream const& stream) {
  if (failure.size() != 1)
    return std::unexpected(Error{ErrorCode::InvalidArgument, 0, "q8.pack", "invalid geometry"});
  return detail::lift(q4k_pack_q8_bf16(input.data(), input.size(), detail::to_abi(output), failure.data(), stream.native),
                      "q8.pack");
}

[[nodiscard]] inline std::expected<void, Error> q4k_q8_project(PrefillWeight const& weight, Q8Input input,
                                                               std::span<float> output, Stream const& stream,
                                                               std::span<float const> residual = {}) {
  q4k_weight const w = detail::to_abi(weight);
  return detail::lift(::q4k_q8_project(&w, detail::to_abi(input), output.data(), output.size(), residual.data(),
                                       residual.size(), stream.native),
                      "q8.project");
}

// submitted is false for a rejection before any launch, true once device work has been attempted.
[[nodiscard]] inline std::expected<void, Error> q4k_q8_mlp(PrefillWeight const& gate, PrefillWeight const& up,
                                                           PrefillWeight const& down, float const* residual,
                                                           std::uint16_t const* gamma, float eps, float* output, unsigned m,
                                                           std::span<std::byte> workspace, Stream const& stream,
                                                           bool& submitted, int* pending_failure = nullptr) {
  q4k_weight const g = detail::to_abi(gate), u = detail::to_abi(up), d = detail::to_abi(down);
  int sub = 0;
  int const st = ::q4k_q8_mlp(&g, &u, &d, residual, gamma, eps, output, m, workspace.data(), workspace.size(), stream.native,
                              &sub, pending_failure);
  submitted = sub != 0;
  return detail::lift(st, "q8.mlp");
}

// ---- cuda/decode_mmv.hpp ------------------------------------------------------------------------

enum class DecodeActivationPolicy : std::uint8_t { Bf16 = 1, Q8K32 = 2 };  // Q8K32: the value this library adds
enum class DecodeEpilogue : std::uint8_t { StoreBf16 = 1, StoreFp32 = 2, ResidualAddFp32 = 3, SwigluStoreBf16 = 4 };

// One projection of 1..16 bf16 input rows.  The reference's DecodeOperandView metadata collapses to
// pointers here: sizes follow from weight.n / weight.k and `rows`.
struct DecodeMmvDesc {
  PrefillWeight weight{};
  DecodeActivationPolicy activation_policy{DecodeActivationPolicy::Q8K32};
  std::uint16_t const* input{};  // bf16 [rows][k]
  void* output{};                // bf16 or fp32 [rows][n] by epilogue; null = in-place residual update
  float const* residual{};       // fp32 [rows][n], ResidualAddFp32 only
  DecodeEpilogue epilogue{DecodeEpilogue::StoreBf16};
  std::uint32_t rows{1};
};

struct DecodeMmvPairedDesc {
  DecodeMmvDesc a;
  DecodeMmvDesc b;
};

struct DecodeMmvRangeDesc {
  std::span<DecodeMmvDesc const> ranges{};
};

// Caller-owned scratch of a decode call (Q8 pack of the input rows + fp32 rows) and its failure flag.
struct DecodeScratch {
  std::span<std::byte> workspace;
  int* failure{};
};

[[nodiscard]] inline std::uint64_t decode_workspace_bytes(std::uint32_t rows, std::uint64_t n_total, std::uint32_t k) {
  return q4k_decode_workspace_bytes(rows, n_total, k);
}

namespace detail {
inline q4k_decode_desc to_abi(DecodeMmvDesc const& d) {
  std::uint64_t const cells = std::uint64_t(d.rows) * d.weight.n;
  q4k_decode_desc out{};
  out.weight = to_abi(d.weight);
  out.input = d.input;
  out.input_len = std::uint64_t(d.rows) * d.weight.k;
  out.output = d.output;
  out.output_len = d.output ? cells : 0;
  out.residual = d.residual;
  out.residual_len = d.residual ? cells : 0;
  out.m = d.rows;
  out.epilogue = static_cast<std::uint8_t>(d.epilogue);
  out.activation_policy = static_cast<std::uint8_t>(d.activation_policy);
  return out;
}
}  // namespace detail

[[nodiscard]] inline std::expected<void, Error> launch_decode_mmv(DecodeMmvDesc const& desc, DecodeScratch scratch,
                                                                  Stream const& stream) {
  q4k_decode_desc const d = detail::to_abi(desc);
  return detail::lift(q4k_decode_mmv(&d, scratch.workspace.data(), scratch.workspace.size(), scratch.failure, stream.native),
                      "decode_mmv");
}

[[nodiscard]] inline std::expected<void, Error> launch_decode_mmv_paired(DecodeMmvPairedDesc const& desc,
                                                                         DecodeScratch scratch, Stream const& stream) {
  q4k_decode_desc const a = detail::to_abi(desc.a), b = detail::to_abi(desc.b);
  return detail::lift(q4k_decode_mmv_paired(&a, &b, scratch.workspace.data(), scratch.workspace.size(), scratch.failure,
                                            stream.native),
                      "decode_mmv_paired");
}

[[nodiscard]] inline std::expected<void, Error> launch_decode_mmv_ranges(DecodeMmvRangeDesc const& desc,
                                                                         DecodeScratch scratch, Stream const& stream) {
  if (desc.ranges.size() < 2 || desc.ranges.size() > 3)
    return std::unexpected(Error{ErrorCode::InvalidArgument, 0, "decode_mmv_ranges", "two or three ranges"});
  q4k_decode_desc abi[3];
  for (std::size_t i = 0; i < desc.ranges.size(); ++i) abi[i] = detail::to_abi(desc.ranges[i]);
  return detail::lift(q4k_decode_mmv_ranges(abi, static_cast<std::uint32_t>(desc.ranges.size()), scratch.workspace.data(),
                                            scratch.workspace.size(), scratch.failure, stream.native),
                      "decode_mmv_ranges");
}

// ---- compiler/quantization/q4k.hpp ---------------------------------------------------------------

enum class FitStatus : std::uint8_t {
  Ok = Q4K_FIT_OK,
  Nonfinite = Q4K_FIT_NONFINITE,        // CompilerErrorCode::Nonfinite
  RangeExceeded = Q4K_FIT_RANGE,        // the rest: CompilerErrorCode::Unrepresentable
  FitReciprocal = Q4K_FIT_RECIPROCAL,
  CompressReciprocal = Q4K_FIT_COMPRESS,
  HalfOverflow = Q4K_FIT_HALF,
};

// quantize_q4k_block over weights.size() / 256 consecutive blocks; all spans are device memory.
// codes: 256 levels per block, metadata: 16 bytes per block, status: one FitStatus per block (may be
// empty), failure: one int set to 1 when any block is refused.  The host loop of the reference stops
// at the first refused block; here every block is attempted and that block is the lowest index
// with a non-zero status.
[[nodiscard]] inline std::expected<void, Error> quantize_q4k_blocks(std::span<float const> weights,
                                                                    std::span<std::int8_t> codes,
                                                                    std::span<std::uint8_t> metadata,
                                                                    std::span<std::uint8_t> status, std::span<int> failure,
                                                                    Stream const& stream) {
  std::uint64_t const blocks = weights.size() / 256;
  if (weights.size() % 256 != 0 || codes.size() != weights.size() || metadata.size() != blocks * 16 ||
      (!status.empty() && status.size() != blocks) || failure.size() != 1)
    return std::unexpected(Error{ErrorCode::InvalidArgument, 0, "q4k.fit", "invalid geometry"});
  return detail::lift(q4k_fit_blocks(weights.data(), Q4K_FIT_FP32, blocks, codes.data(), metadata.data(),
                                     status.empty() ? nullptr : status.data(), failure.data(), stream.native),
                      "q4k.fit");
}

// The same from row-major [n][k] weights (fp32, or bf16 bits) straight into a split-tile weight:
// the fitter followed by format::pack_cuda_v0.  `weight` describes the destination spans.
[[nodiscard]] inline std::expected<void, Error> quantize_q4k_weight(void const* weights, bool bf16, PrefillWeight const& weight,
                                                                    std::span<std::uint8_t> status, std::span<int> failure,
                                                                    Stream const& stream) {
  if (failure.size() != 1 || (!status.empty() && status.size() != std::uint64_t(weight.n) * (weight.k / 256)))
    return std::unexpected(Error{ErrorCode::InvalidArgument, 0, "q4k.fit", "invalid geometry"});
  return detail::lift(q4k_fit_weight(weights, bf16 ? Q4K_FIT_BF16 : Q4K_FIT_FP32, weight.n, weight.k,
                                     static_cast<std::uint8_t*>(const_cast<void*>(weight.codes)), weight.codes_bytes,
                                     static_cast<std::uint8_t*>(const_cast<void*>(weight.scales)), weight.scales_bytes,
                                     status.empty() ? nullptr : status.data(), failure.data(), stream.native),
                      "q4k.fit");
}

}  // namespace q4k_b200::shim
