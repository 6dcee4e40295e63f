// Runs the quantiser, a projection, a decode entry and the fitter through the C++23 shim on the current device.
// Weights are built so that every weight equals 1 (codes 1, six-bit scale 1, min 0, d = 1, dmin = 0) and the
// activations are ones, so every output must equal k.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "q4k_b200_shim.hpp"

using namespace q4k_b200::shim;

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("cuda error %s at %s\n", cudaGetErrorString(e_), #x); return 2; } } while (0)

int main() {
  unsigned const n = 64, k = 512, m = 3, tiles_k = k / 256, G = k / 32;
  std::vector<unsigned char> codes(size_t(n) * k / 2, 0x11), meta(size_t(n) * tiles_k * 16);
  unsigned char const row[16] = {0x00, 0x3C, 0, 0, 1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1};  // d = 1.0 (fp16), dmin = 0, sc = 1, mn = 0
  for (size_t i = 0; i < meta.size(); i += 16) std::memcpy(&meta[i], row, 16);
  std::vector<std::uint16_t> x(size_t(m) * k, 0x3F80);  // bf16 1.0
  void *dc, *dm; std::uint16_t* dx; std::int8_t* qc; float *qs, *out, *out2; std::int32_t* qsum; int* fail; std::byte* ws = nullptr;
  CK(cudaMalloc(&dc, codes.size())); CK(cudaMalloc(&dm, meta.size())); CK(cudaMalloc(&dx, x.size() * 2));
  CK(cudaMalloc(&qc, size_t(m) * k)); CK(cudaMalloc(&qs, size_t(m) * G * 4)); CK(cudaMalloc(&qsum, size_t(m) * G * 4));
  CK(cudaMalloc(&out, size_t(m) * n * 4)); CK(cudaMalloc(&out2, size_t(m) * n * 4)); CK(cudaMalloc(&fail, 4));
  auto session = Session::create(decode_workspace_bytes(m, n, k));
  if (!session) { std::printf("session: %s\n", session.error().detail.c_str()); return 1; }
  (void)ws;
  CK(cudaMemcpy(dc, codes.data(), codes.size(), cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dm, meta.data(), meta.size(), cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dx, x.data(), x.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemset(fail, 0, 4));
  PrefillWeight w{dc, dm, Q4K_LAYOUT_SPLIT_TILES, Q4K_QUANTIZER_Q4K, n, k, n, k, codes.size(), meta.size()};
  Q8Input q{{qc, size_t(m) * k}, {qs, size_t(m) * G}, {qsum, size_t(m) * G}, m, k, k};
  Stream s{nullptr, &*session};
  if (auto r = pack_q8({dx, x.size()}, q, {fail, 1}, s); !r) { std::printf("pack: %s\n", r.error().detail.c_str()); return 1; }
  if (auto r = q4k_q8_project(w, q, {out, size_t(m) * n}, s); !r) { std::printf("project: %s\n", r.error().detail.c_str()); return 1; }
  DecodeMmvDesc d{};
  d.layout = kDecodeLayoutQ4KV2; d.quantizer = kDecodeQuantizerQ4KV2; d.activation_policy = DecodeActivationPolicy::Q8K32;
  d.n = n; d.k = k; d.padded_n = n; d.padded_k = k; d.rows = m; d.epilogue = DecodeEpilogue::StoreFp32;
  d.codes = decode_matrix_view(dc, DecodeDtype::Q4, d.layout, n, k, n, k, codes.size(), 16);
  d.scales = decode_matrix_view(dm, DecodeDtype::Fp16, d.layout, n, tiles_k * 8, n, tiles_k * 8, meta.size(), 2);
  d.input = decode_vector_view(dx, DecodeDtype::Bf16, kDecodeLayoutBf16VectorV0, m * k, std::uint64_t(m) * k * 2, 2, false);
  d.output = decode_vector_view(out2, DecodeDtype::Fp32, kDecodeLayoutFp32VectorV0, m * n, std::uint64_t(m) * n * 4, 4, true);
  if (auto r = launch_decode_mmv(d, s); !r) { std::printf("decode: %s\n", r.error().detail.c_str()); return 1; }
  // PrefillEngine: the same projection with the bf16 -> fp32 store epilogue, from the engine's own workspace
  float* out3;
  CK(cudaMalloc(&out3, size_t(m) * n * 4));
  auto engine = PrefillEngine::create(s, 16, n, k);
  if (!engine) { std::printf("engine: %s\n", engine.error().detail.c_str()); return 1; }
  PrefillProjection proj{w, dx, out3, nullptr, m, 0, PrefillEpilogue::StoreFp32};
  if (auto r = engine->project(proj); !r) { std::printf("engine.project: %s\n", r.error().detail.c_str()); return 1; }
  if (auto r = engine->check(); !r) { std::printf("engine.check: %s\n", r.error().detail.c_str()); return 1; }
  CK(cudaDeviceSynchronize());
  std::vector<float> h(size_t(m) * n), h2(size_t(m) * n);
  int hf = -1;
  CK(cudaMemcpy(h.data(), out, h.size() * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(h2.data(), out2, h2.size() * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(&hf, fail, 4, cudaMemcpyDeviceToHost));
  int bad = hf != 0;
  std::vector<float> h3(size_t(m) * n);
  CK(cudaMemcpy(h3.data(), out3, h3.size() * 4, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < h.size(); ++i) bad += std::fabs(h[i] - float(k)) > 1e-2f || h2[i] != h[i] || h3[i] != h[i];
  // Offline step through the shim: fit a weight whose rows repeat the ramp 0..15 (exactly representable
  // levels), project ones through it: every output is close to the row sum, k / 16 * 120.
  {
    std::vector<float> wf(size_t(n) * k);
    for (size_t i = 0; i < wf.size(); ++i) wf[i] = float(i % 16);
    float* dw; std::uint8_t* st;
    CK(cudaMalloc(&dw, wf.size() * 4)); CK(cudaMalloc(&st, size_t(n) * tiles_k));
    CK(cudaMemcpy(dw, wf.data(), wf.size() * 4, cudaMemcpyHostToDevice));
    if (auto r = quantize_q4k_weight(dw, false, w, {st, size_t(n) * tiles_k}, {fail, 1}, s); !r) { std::printf("fit: %s\n", r.error().detail.c_str()); return 1; }
    if (auto r = q4k_q8_project(w, q, {out, size_t(m) * n}, s); !r) { std::printf("project fitted: %s\n", r.error().detail.c_str()); return 1; }
    CK(cudaDeviceSynchronize());
    std::vector<std::uint8_t> hs(size_t(n) * tiles_k);
    CK(cudaMemcpy(hs.data(), st, hs.size(), cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(h.data(), out, h.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&hf, fail, 4, cudaMemcpyDeviceToHost));
    bad += hf != 0;
    for (auto v : hs) bad += v != static_cast<std::uint8_t>(FitStatus::Ok);
    float const want = float(k) / 16.f * 120.f;
    for (float v : h) bad += std::fabs(v - want) > 0.01f * want;
  }
  std::printf(bad ? "shim gpu check failed (%d)\n" : "shim gpu check ok\n", bad);
  return bad != 0;
}
