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
  DecodeMmvDesc d{};
  auto r4 = launch_decode_mmv(d, DecodeScratch{}, Stream{});
  expect(!r4 && r4.error().code == ErrorCode::InvalidArgument, "decode_mmv rejects empty descriptor");
  std::vector<DecodeMmvDesc> one(1);
  auto r5 = launch_decode_mmv_ranges(DecodeMmvRangeDesc{one}, DecodeScratch{}, Stream{});
  expect(!r5 && r5.error().detail == "two or three ranges", "ranges count");
  // fitter: span sizes are checked in the shim, geometry in the library, both before any CUDA call
  std::vector<int> flag(1);
  auto r6 = quantize_q4k_blocks(std::span<float const>(static_cast<float const*>(nullptr), 300), {}, {}, {}, flag, Stream{});
  expect(!r6 && r6.error().operation == "q4k.fit" && r6.error().detail == "invalid geometry", "fit span sizes");
  auto r7 = quantize_q4k_weight(nullptr, true, PrefillWeight{}, {}, flag, Stream{});
  expect(!r7 && r7.error().code == ErrorCode::InvalidArgument, "fit rejects empty weight");
  std::printf(fails ? "shim check failed\n" : "shim check ok\n");
  return fails;
}
