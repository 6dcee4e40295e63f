// Compiles the C++23 shim against the C ABI and exercises the rejections that need no GPU.
#include <cstdio>
#include <vector>

#include "q4k_b200_shim.hpp"

using namespace q4k_b200::shim;

int main() {
  int fails = 0;
  auto expect = [&](bool ok, char const* what) {
    if (!ok) { std::printf("FAIL %s\n", what); ++fails; }
  };
  expect(q4k_abi_version() >= 1, "abi version");
  expect(q8_mlp_workspace_bytes(3) == std::uint64_t(3) * (17408 + 17408 / 32 * 8 + 2 * 17408 * 4) + 4, "mlp workspace formula");
  // failure span of the wrong size: rejected in the shim, as the reference does before anything else
  std::vector<int> two(2);
  auto r1 = pack_q8({}, Q8Input{}, two, Stream{});
  expect(!r1 && r1.error().code == ErrorCode::InvalidArgument && r1.error().operation == "q8.pack", "pack_q8 failure span");
  // a null weight descriptor is rejected by the library before any CUDA call
  auto r2 = q4k_q8_project(PrefillWeight{}, Q8Input{}, {}, Stream{});
  expect(!r2 && r2.error().code == ErrorCode::InvalidArgument && !r2.error().detail.empty(), "project rejects empty weight");
  bool submitted = true;
  auto r3 = q4k_q8_mlp(PrefillWeight{}, PrefillWeight{}, PrefillWeight{}, nullptr, nullptr, 1e-6f, nullptr, 1, {}, Stream{}, submitted);
  expect(!r3 && !submitted, "mlp rejection leaves submitted false");
  // typed views (cuda/decode_mmv.cu:306-324): every field of a view is part of the contract
  alignas(16) static unsigned char fake[64];
  std::uint32_t const n = 64, k = 512;
  DecodeMmvDesc d{};
  d.layout = kDecodeLayoutQ4KV2; d.quantizer = kDecodeQuantizerQ4KV2; d.activation_policy = DecodeActivationPolicy::Q8K32;
  d.n = n; d.k = k; d.padded_n = n; d.padded_k = k;
  d.codes = decode_matrix_view(fake, DecodeDtype::Q4, d.layout, n, k, n, k, std::uint64_t(n) * k / 2, 16);
  d.scales = decode_matrix_view(fake, DecodeDtype::Fp16, d.layout, n, 16, n, 16, std::uint64_t(n) * 2 * 16, 2);
  d.input = decode_vector_view(fake, DecodeDtype::Bf16, kDecodeLayoutBf16VectorV0, k, std::uint64_t(k) * 2, 2, false);
  d.output = decode_vector_view(fake, DecodeDtype::Fp32, kDecodeLayoutFp32VectorV0, n, std::uint64_t(n) * 4, 4, true);
  d.epilogue = DecodeEpilogue::StoreFp32;
  auto ok_views = launch_decode_mmv(d, Stream{});  // the views pass; the stream has no session
  expect(!ok_views && ok_views.error().detail.find("session") != std::string::npos, "valid views reach the session check");
  auto broken = [&](auto&& edit, char const* what) {
    DecodeMmvDesc e = d;
    edit(e);
    auto r = launch_decode_mmv(e, Stream{});
    expect(!r && r.error().code == ErrorCode::InvalidArgument && r.error().detail.find("typed view") != std::string::npos, what);
  };
  broken([](DecodeMmvDesc& e) { e.codes.space = DecodeMemorySpace::Host; }, "host-space codes view");
  broken([](DecodeMmvDesc& e) { e.codes.dtype = DecodeDtype::Q8; }, "wrong codes dtype");
  broken([](DecodeMmvDesc& e) { e.codes.bytes -= 1; }, "short codes view");
  broken([](DecodeMmvDesc& e) { e.codes.alignment = 8; }, "codes alignment below 16");
  broken([](DecodeMmvDesc& e) { e.scales.logical_k = 15; }, "scales shape");
  broken([](DecodeMmvDesc& e) { e.input.layout = kDecodeLayoutFp32VectorV0; }, "input layout");
  broken([](DecodeMmvDesc& e) { e.input.alignment = 3; }, "alignment not a power of two");
  broken([](DecodeMmvDesc& e) { e.output.writable = false; }, "read-only output");
  broken([](DecodeMmvDesc& e) { e.output.pointer = fake + 2; e.output.alignment = 4; }, "pointer does not honour its alignment");
  {
    DecodeMmvDesc e = d;
    e.residual = e.output;
    auto r = launch_decode_mmv(e, Stream{});
    expect(!r && r.error().detail == "store epilogue must not supply residual", "store epilogue with residual");
    e = d;
    e.epilogue = DecodeEpilogue::SwigluStoreBf16;
    r = launch_decode_mmv(e, Stream{});
    expect(!r && r.error().detail == "SwiGLU epilogue requires paired gate/up launch", "SwiGLU outside the paired launch");
    e = d;
    e.padded_k = 768;
    r = launch_decode_mmv(e, Stream{});
    expect(!r && r.error().detail == "padded N/K metadata does not match layout tiles", "padding metadata");
  }
  std::vector<DecodeMmvDesc> one(1);
  auto r5 = launch_decode_mmv_ranges(DecodeMmvRangeDesc{one}, Stream{});
  expect(!r5 && r5.error().detail == "two or three ranges", "ranges count");
  auto engine = PrefillEngine::create(Stream{}, 0);
  expect(!engine && engine.error().operation == "prefill.create", "engine rejects a zero token capacity");
  // fitter: span sizes are checked in the shim, geometry in the library, both before any CUDA call
  std::vector<int> flag(1);
  auto r6 = quantize_q4k_blocks(std::span<float const>(static_cast<float const*>(nullptr), 300), {}, {}, {}, flag, Stream{});
  expect(!r6 && r6.error().operation == "q4k.fit" && r6.error().detail == "invalid geometry", "fit span sizes");
  auto r7 = quantize_q4k_weight(nullptr, true, PrefillWeight{}, {}, flag, Stream{});
  expect(!r7 && r7.error().code == ErrorCode::InvalidArgument, "fit rejects empty weight");
  std::printf(fails ? "shim check failed\n" : "shim check ok\n");
  return fails;
}
