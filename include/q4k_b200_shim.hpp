// C++23 host-side shim over the C ABI of q4k_b200.h.
//
// Mirrors the operator interface of the reference engine for this path -- cuda/q4k_q8.hpp:14-49
// (Q8Input, pack_q8, q4k_q8_project, q4k_q8_mlp, q8_mlp_workspace_bytes), cuda/prefill.hpp:33-117
// (PrefillWeight, PrefillProjection, PrefillEngine::create / project / paired_swiglu / mlp) and
// cuda/decode_mmv.hpp:45-121,207-215 (DecodeEpilogue, DecodeOperandView, DecodeMmvDesc,
// launch_decode_mmv / _paired / _ranges with the typed-view validation of cuda/decode_mmv.cu:306-505)
// and, for the offline step, compiler::quantize_q4k_block
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

// Scratch and failure flag of the decode / prefill entries (the reference keeps them in its runtime session and in
// PrefillEngine): device memory owned by this object, created once, borrowed by every call on the stream.
class Session {
 public:
  Session() = default;
  Session(Session&& o) noexcept : handle_(std::exchange(o.handle_, nullptr)) {}
  Session& operator=(Session&& o) noexcept {
    if (this != &o) { q4k_session_destroy(handle_); handle_ = std::exchange(o.handle_, nullptr); }
    return *this;
  }
  Session(Session const&) = delete;
  Session& operator=(Session const&) = delete;
  ~Session() { q4k_session_destroy(handle_); }
  [[nodiscard]] static std::expected<Session, Error> create(std::uint64_t workspace_bytes) {
    Session s;
    if (int st = q4k_session_create(workspace_bytes, &s.handle_); st != Q4K_OK)
      return std::unexpected(Error{static_cast<ErrorCode>(st), q4k_last_cuda_status(), "session.create", q4k_last_error()});
    return s;
  }
  [[nodiscard]] std::span<std::byte> workspace() const noexcept {
    return {static_cast<std::byte*>(q4k_session_workspace(handle_)), static_cast<std::size_t>(q4k_session_workspace_bytes(handle_))};
  }
  [[nodiscard]] int* failure() const noexcept { return q4k_session_failure(handle_); }
  [[nodiscard]] q4k_session* handle() const noexcept { return handle_; }
  [[nodiscard]] bool empty() const noexcept { return handle_ == nullptr; }

 private:
  q4k_session* handle_{nullptr};
};

// The reference passes its Stream object (cuda/stream.hpp), which knows its device and carries the session state;
// here: the native handle (cudaStream_t) and, for the decode entries, the session whose scratch they use.
struct Stream {
  void* native{nullptr};
  Session const* session{nullptr};
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
enum class DecodeMemorySpace : std::uint8_t { Device = 1, Host = 2 };
enum class DecodeDtype : std::uint8_t { Q4 = 1, Q8 = 2, Bf16 = 3, Fp16 = 4, Fp32 = 5, NvFp4 = 6, Fp8 = 7 };
inline constexpr std::uint16_t kDecodeLayoutQ4KV2 = Q4K_LAYOUT_SPLIT_TILES;
inline constexpr std::uint16_t kDecodeQuantizerQ4KV2 = Q4K_QUANTIZER_Q4K;
inline constexpr std::uint16_t kDecodeLayoutBf16VectorV0 = 0x0205;
inline constexpr std::uint16_t kDecodeLayoutFp32VectorV0 = 0x020A;

// Complete borrowed operand metadata at the launch boundary (cuda/decode_mmv.hpp:72-86).  Matrix shapes are
// [N,K]; vectors use logical/padded N with K=1 -- here N = rows * n for the 1..16-row extension.
struct DecodeOperandView {
  void* pointer{};
  DecodeMemorySpace space{DecodeMemorySpace::Device};
  DecodeDtype dtype{};
  std::uint16_t layout{};
  std::uint32_t logical_n{}, logical_k{}, padded_n{}, padded_k{};
  std::uint64_t bytes{};
  std::uint32_t alignment{};
  bool writable{};
  friend bool operator==(DecodeOperandView const&, DecodeOperandView const&) = default;
};

[[nodiscard]] constexpr DecodeOperandView decode_matrix_view(void* pointer, DecodeDtype dtype, std::uint16_t layout,
                                                             std::uint32_t logical_n, std::uint32_t logical_k,
                                                             std::uint32_t padded_n, std::uint32_t padded_k, std::uint64_t bytes,
                                                             std::uint32_t alignment, bool writable = false,
                                                             DecodeMemorySpace space = DecodeMemorySpace::Device) noexcept {
  return {pointer, space, dtype, layout, logical_n, logical_k, padded_n, padded_k, bytes, alignment, writable};
}
[[nodiscard]] constexpr DecodeOperandView decode_vector_view(void* pointer, DecodeDtype dtype, std::uint16_t layout,
                                                             std::uint32_t elements, std::uint64_t bytes, std::uint32_t alignment,
                                                             bool writable,
                                                             DecodeMemorySpace space = DecodeMemorySpace::Device) noexcept {
  return {pointer, space, dtype, layout, elements, 1, elements, 1, bytes, alignment, writable};
}

// One projection (cuda/decode_mmv.hpp:103-121).  `rows` (1..16 input rows, default 1 as in the reference) is this
// library's extension; vector views then hold rows * k (input) and rows * n (output, residual) elements.
struct DecodeMmvDesc {
  std::uint16_t layout{};
  std::uint16_t quantizer{};
  DecodeActivationPolicy activation_policy{DecodeActivationPolicy::Bf16};
  std::uint32_t n{}, k{}, padded_n{}, padded_k{};
  DecodeOperandView codes{};
  DecodeOperandView scales{};  // the fp16-typed span of opaque 16-byte super-block metadata
  DecodeOperandView input{};
  DecodeOperandView output{};
  DecodeOperandView residual{};
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

[[nodiscard]] inline std::uint64_t decode_workspace_bytes(std::uint32_t rows, std::uint64_t n_total, std::uint32_t k) {
  return q4k_decode_workspace_bytes(rows, n_total, k);
}

namespace detail {
inline std::unexpected<Error> invalid(char const* op, std::string detail) {
  return std::unexpected(Error{ErrorCode::InvalidArgument, 0, op, std::move(detail)});
}
// validate_view (cuda/decode_mmv.cu:306-324): space, dtype, layout, shape, byte count, power-of-two alignment that
// the pointer honours, writability -- all must match the contract of the slot the view sits in.
inline std::expected<void, Error> validate_view(DecodeOperandView const& v, DecodeDtype dtype, std::uint16_t layout,
                                                std::uint32_t logical_n, std::uint32_t logical_k, std::uint32_t padded_n,
                                                std::uint32_t padded_k, std::uint64_t bytes, std::uint32_t min_alignment,
                                                bool writable, char const* op, char const* name) {
  if (v.pointer == nullptr || v.space != DecodeMemorySpace::Device || v.dtype != dtype || v.layout != layout ||
      v.logical_n != logical_n || v.logical_k != logical_k || v.padded_n != padded_n || v.padded_k != padded_k ||
      v.bytes != bytes || v.alignment < min_alignment || (v.alignment & (v.alignment - 1u)) != 0u ||
      (reinterpret_cast<std::uintptr_t>(v.pointer) % v.alignment) != 0u || v.writable != writable)
    return invalid(op, std::string(name) + " typed view does not match the required contract");
  return {};
}
inline bool empty_view(DecodeOperandView const& v) noexcept { return v == DecodeOperandView{}; }

// validate_geometry + the epilogue contract (cuda/decode_mmv.cu:375-505) for the one layout this library runs, then
// the plain-pointer form of the C ABI.
inline std::expected<q4k_decode_desc, Error> to_abi(DecodeMmvDesc const& d, char const* op, bool paired_b, bool swiglu_b = false) {
  if (d.layout != kDecodeLayoutQ4KV2 || d.quantizer != kDecodeQuantizerQ4KV2) return invalid(op, "layout/quantizer version mismatch");
  if (d.activation_policy != DecodeActivationPolicy::Bf16 && d.activation_policy != DecodeActivationPolicy::Q8K32)
    return invalid(op, "unsupported decode activation policy");
  if (d.n == 0 || d.k == 0) return invalid(op, "N and K must be nonzero");
  if (d.rows == 0 || d.rows > 16) return invalid(op, "1..16 input rows");
  if (d.padded_n != q4k_pad_n(d.n) || d.padded_k != q4k_pad_k(d.k)) return invalid(op, "padded N/K metadata does not match layout tiles");
  if (d.k % 256 != 0) return invalid(op, "logical K must divide the quantizer group");
  std::uint64_t const want_codes = q4k_code_bytes(d.padded_n, d.padded_k), want_scales = q4k_scale_bytes(d.padded_n, d.padded_k);
  if (auto st = validate_view(d.codes, DecodeDtype::Q4, d.layout, d.n, d.k, d.padded_n, d.padded_k, want_codes, 16, false, op, "codes"); !st)
    return std::unexpected(st.error());
  auto const units = static_cast<std::uint32_t>(want_scales / d.padded_n / 2u);
  if (auto st = validate_view(d.scales, DecodeDtype::Fp16, d.layout, d.padded_n, units, d.padded_n, units, want_scales, 2, false, op, "scales"); !st)
    return std::unexpected(st.error());
  std::uint32_t const in_elems = d.rows * d.k, out_elems = d.rows * d.n;
  if (auto st = validate_view(d.input, DecodeDtype::Bf16, kDecodeLayoutBf16VectorV0, in_elems, 1, in_elems, 1, std::uint64_t(in_elems) * 2u, 2, false, op, "input"); !st)
    return std::unexpected(st.error());
  q4k_decode_desc out{};
  out.weight = q4k_weight{d.codes.pointer, d.scales.pointer, d.layout, d.quantizer, d.n, d.k, d.padded_n, d.padded_k, want_codes, want_scales};
  out.input = static_cast<std::uint16_t const*>(d.input.pointer);
  out.input_len = in_elems;
  out.m = d.rows;
  out.epilogue = static_cast<std::uint8_t>(d.epilogue);
  out.activation_policy = static_cast<std::uint8_t>(d.activation_policy);
  switch (d.epilogue) {
    case DecodeEpilogue::SwigluStoreBf16:
      if (!paired_b) return invalid(op, "SwiGLU epilogue requires paired gate/up launch");
      [[fallthrough]];
    case DecodeEpilogue::StoreBf16:
    case DecodeEpilogue::StoreFp32: {
      if (!empty_view(d.residual)) return invalid(op, "store epilogue must not supply residual");
      if (swiglu_b) {  // the B side of a SwiGLU pair declares no output of its own (cuda/decode_mmv.cu:514-521)
        if (!empty_view(d.output)) return invalid(op, "SwiGLU paired B must not declare a separately materialized output");
        break;
      }
      bool const fp32 = d.epilogue == DecodeEpilogue::StoreFp32;
      if (auto st = validate_view(d.output, fp32 ? DecodeDtype::Fp32 : DecodeDtype::Bf16,
                                  fp32 ? kDecodeLayoutFp32VectorV0 : kDecodeLayoutBf16VectorV0, out_elems, 1, out_elems, 1,
                                  std::uint64_t(out_elems) * (fp32 ? 4u : 2u), fp32 ? 4u : 2u, true, op, "output"); !st)
        return std::unexpected(st.error());
      out.output = d.output.pointer;
      out.output_len = out_elems;
      break;
    }
    case DecodeEpilogue::ResidualAddFp32: {
      bool const separate = !empty_view(d.output);
      if (auto st = validate_view(d.residual, DecodeDtype::Fp32, kDecodeLayoutFp32VectorV0, out_elems, 1, out_elems, 1,
                                  std::uint64_t(out_elems) * 4u, 4, !separate, op, "residual"); !st)
        return std::unexpected(st.error());
      if (separate) {
        if (auto st = validate_view(d.output, DecodeDtype::Fp32, kDecodeLayoutFp32VectorV0, out_elems, 1, out_elems, 1,
                                    std::uint64_t(out_elems) * 4u, 4, true, op, "output"); !st)
          return std::unexpected(st.error());
        out.output = d.output.pointer;
        out.output_len = out_elems;
      }
      out.residual = static_cast<float const*>(d.residual.pointer);
      out.residual_len = out_elems;
      break;
    }
    default:
      return invalid(op, "unknown epilogue");
  }
  return out;
}
inline std::expected<Session const*, Error> session_of(Stream const& stream, char const* op) {
  if (stream.session == nullptr || stream.session->empty()) return invalid(op, "the stream carries no session (scratch and failure flag)");
  return stream.session;
}
}  // namespace detail

// launch_decode_mmv / _paired / _ranges (cuda/decode_mmv.hpp:207-215): same signatures; scratch and failure flag
// come from the session the stream carries.
[[nodiscard]] inline std::expected<void, Error> launch_decode_mmv(DecodeMmvDesc const& desc, Stream const& stream) {
  auto d = detail::to_abi(desc, "decode_mmv", false);
  if (!d) return std::unexpected(d.error());
  auto s = detail::session_of(stream, "decode_mmv");
  if (!s) return std::unexpected(s.error());
  auto const ws = (*s)->workspace();
  return detail::lift(q4k_decode_mmv(&*d, ws.data(), ws.size(), (*s)->failure(), stream.native), "decode_mmv");
}

[[nodiscard]] inline std::expected<void, Error> launch_decode_mmv_paired(DecodeMmvPairedDesc const& desc, Stream const& stream) {
  bool const swiglu = desc.a.epilogue == DecodeEpilogue::SwigluStoreBf16;
  auto a = detail::to_abi(desc.a, "decode_mmv_paired", true);
  if (!a) return std::unexpected(a.error());
  auto b = detail::to_abi(desc.b, "decode_mmv_paired", true, swiglu);
  if (!b) return std::unexpected(b.error());
  auto s = detail::session_of(stream, "decode_mmv_paired");
  if (!s) return std::unexpected(s.error());
  auto const ws = (*s)->workspace();
  return detail::lift(q4k_decode_mmv_paired(&*a, &*b, ws.data(), ws.size(), (*s)->failure(), stream.native), "decode_mmv_paired");
}

[[nodiscard]] inline std::expected<void, Error> launch_decode_mmv_ranges(DecodeMmvRangeDesc const& desc, Stream const& stream) {
  if (desc.ranges.size() < 2 || desc.ranges.size() > 3) return detail::invalid("decode_mmv_ranges", "two or three ranges");
  q4k_decode_desc abi[3];
  for (std::size_t i = 0; i < desc.ranges.size(); ++i) {
    auto d = detail::to_abi(desc.ranges[i], "decode_mmv_ranges", false);
    if (!d) return std::unexpected(d.error());
    abi[i] = *d;
  }
  auto s = detail::session_of(stream, "decode_mmv_ranges");
  if (!s) return std::unexpected(s.error());
  auto const ws = (*s)->workspace();
  return detail::lift(q4k_decode_mmv_ranges(abi, static_cast<std::uint32_t>(desc.ranges.size()), ws.data(), ws.size(), (*s)->failure(),
                                            stream.native),
                      "decode_mmv_ranges");
}

// ---- cuda/prefill.hpp ---------------------------------------------------------------------------

inline constexpr std::uint32_t kPrefillMaxTokens = Q4K_MAX_TOKENS;  // the reference stops at 1024 (cuda/prefill.hpp:21)
inline constexpr std::uint32_t kPrefillDefaultTokens = 1024;

[[nodiscard]] inline std::expected<void, Error> validate_prefill_device_span(void const* pointer, std::uint64_t bytes,
                                                                             std::uint32_t alignment, int device) {
  return detail::lift(q4k_validate_device_span(pointer, bytes, alignment, device), "prefill.span");
}

enum class PrefillEpilogue : std::uint8_t { StoreBf16 = 1, StoreFp32 = 2, ResidualAddFp32 = 3 };
// The reference's two values select its bf16 unpack -> library GEMM routes; Q8Mmq is the value this library adds:
// quantise -> Q4_K x Q8 MMQ -> fused epilogue, the only route it runs.
enum class PrefillDispatch : std::uint8_t { BoundedUnpackBf16Cublas = 1, LocalQ4K = 2, Q8Mmq = 3 };

// All arrays are device resident and token-major; output has physical stride weight.n and only valid_tokens rows
// are written; first_position is carried for the caller, the arithmetic is position free (cuda/prefill.hpp:58-70).
struct PrefillProjection {
  PrefillWeight weight{};
  std::uint16_t const* input{};
  void* output{};
  float const* residual{};
  std::uint32_t valid_tokens{};
  std::uint64_t first_position{};
  PrefillEpilogue epilogue{PrefillEpilogue::StoreBf16};
};

// PrefillEngine (cuda/prefill.hpp:72-117) for Q4_K weights: owns its workspace (sized for token_capacity tokens of
// the widest projection it will see) and its failure flag; project / paired_swiglu / mlp enqueue on the stream given
// at creation.  A non-finite activation is reported by check(), which synchronises.
class PrefillEngine {
 public:
  PrefillEngine() = default;
  PrefillEngine(PrefillEngine&&) noexcept = default;
  PrefillEngine& operator=(PrefillEngine&&) noexcept = default;

  [[nodiscard]] static std::expected<PrefillEngine, Error> create(Stream const& stream, std::uint32_t token_capacity = kPrefillDefaultTokens,
                                                                  std::uint32_t max_n = 34816, std::uint32_t max_k = 17408,
                                                                  PrefillDispatch dispatch = PrefillDispatch::Q8Mmq) {
    if (dispatch != PrefillDispatch::Q8Mmq) return detail::invalid("prefill.create", "only the Q8 MMQ dispatch is implemented");
    if (token_capacity == 0 || token_capacity > kPrefillMaxTokens) return detail::invalid("prefill.create", "token capacity out of range");
    std::uint64_t const projection = q4k_decode_workspace_bytes(token_capacity, max_n, max_k);
    std::uint64_t const mlp = q4k_q8_mlp_workspace_bytes(token_capacity, 5120, max_k);
    auto session = Session::create(projection > mlp ? projection : mlp);
    if (!session) return std::unexpected(session.error());
    PrefillEngine e;
    e.session_ = std::move(*session);
    e.stream_ = stream.native;
    e.token_capacity_ = token_capacity;
    return e;
  }

  [[nodiscard]] std::expected<void, Error> project(PrefillProjection const& p) {
    if (p.valid_tokens == 0 || p.valid_tokens > token_capacity_) return detail::invalid("prefill.project", "valid_tokens exceeds the engine's token capacity");
    std::uint64_t const cells = std::uint64_t(p.valid_tokens) * p.weight.n;
    q4k_decode_desc d{};
    d.weight = detail::to_abi(p.weight);
    d.input = p.input;
    d.input_len = std::uint64_t(p.valid_tokens) * p.weight.k;
    d.output = p.output;
    d.output_len = p.output ? cells : 0;
    d.residual = p.residual;
    d.residual_len = p.residual ? cells : 0;
    d.m = p.valid_tokens;
    d.epilogue = static_cast<std::uint8_t>(p.epilogue);
    d.activation_policy = Q4K_ACTIVATION_Q8_K32;
    auto const ws = session_.workspace();
    return detail::lift(q4k_prefill_project(&d, ws.data(), ws.size(), session_.failure(), stream_), "prefill.project");
  }

  [[nodiscard]] std::expected<void, Error> paired_swiglu(PrefillWeight const& gate, PrefillWeight const& up, std::uint16_t const* normalized,
                                                         std::uint16_t* swiglu, std::uint32_t valid_tokens, std::uint64_t /*first_position*/) {
    if (valid_tokens == 0 || valid_tokens > token_capacity_) return detail::invalid("prefill.paired_swiglu", "valid_tokens exceeds the engine's token capacity");
    q4k_weight const g = detail::to_abi(gate), u = detail::to_abi(up);
    auto const ws = session_.workspace();
    return detail::lift(q4k_prefill_paired_swiglu(&g, &u, normalized, swiglu, valid_tokens, ws.data(), ws.size(), session_.failure(), stream_),
                        "prefill.paired_swiglu");
  }

  [[nodiscard]] std::expected<void, Error> mlp(PrefillWeight const& gate, PrefillWeight const& up, PrefillWeight const& down, float const* h_mid,
                                               std::uint16_t const* gamma, float eps, float* next_h, std::uint32_t valid_tokens,
                                               std::uint64_t /*first_position*/) {
    if (valid_tokens == 0 || valid_tokens > token_capacity_) return detail::invalid("prefill.mlp", "valid_tokens exceeds the engine's token capacity");
    q4k_weight const g = detail::to_abi(gate), u = detail::to_abi(up), d = detail::to_abi(down);
    auto const ws = session_.workspace();
    int submitted = 0;
    return detail::lift(::q4k_q8_mlp(&g, &u, &d, h_mid, gamma, eps, next_h, valid_tokens, ws.data(), ws.size(), stream_, &submitted, session_.failure()),
                        "prefill.mlp");
  }

  // Synchronises the stream and reports (and clears) a non-finite producer seen since the last check.
  [[nodiscard]] std::expected<void, Error> check() { return detail::lift(q4k_session_take_failure(session_.handle(), stream_), "prefill.check"); }
  [[nodiscard]] std::uint64_t workspace_bytes() const noexcept { return session_.workspace().size(); }
  [[nodiscard]] std::uint32_t token_capacity() const noexcept { return token_capacity_; }

 private:
  Session session_{};
  void* stream_{nullptr};
  std::uint32_t token_capacity_{0};
};

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
