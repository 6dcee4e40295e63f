// The reference's own operator test case for this path (tests/q4k_q8_test.cpp:36-142), run through the C++ shim:
// the 137 x 259 fixture matrix, the ten token counts, the quantiser's literal codes, the affine equation evaluated
// independently in double, the tolerance 0.02 + 0.002 |ref|, row-tail guards, reuse and rejection.  Restated here
// from the fixture's definition (codes (7r + 11c) mod 16, six-bit scales (13r + 17g + 3) mod 64 ...); one PASS
// line per token count, exit code 0 only if all ten pass.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "q4k_b200_shim.hpp"

using namespace q4k_b200::shim;

namespace {
int g_failed = 0;
void require(bool ok, char const* why, unsigned m) {
  if (!ok) { std::printf("FAIL (M=%u): %s\n", m, why); ++g_failed; }
}
float fp16_value(std::uint16_t h) {  // normal and subnormal halves only (the fixture has no inf / nan)
  int const e = (h >> 10) & 31, f = h & 1023;
  float const mag = e == 0 ? std::ldexp(float(f), -24) : std::ldexp(float(1024 + f), e - 25);
  return (h & 0x8000) ? -mag : mag;
}
std::uint16_t bf16_rne(float v) {
  std::uint32_t b;
  std::memcpy(&b, &v, 4);
  b += 0x7fffu + ((b >> 16) & 1u);
  return std::uint16_t(b >> 16);
}
float bf16_value(std::uint16_t h) {
  std::uint32_t const b = std::uint32_t(h) << 16;
  float v;
  std::memcpy(&v, &b, 4);
  return v;
}
template <class T> T* device(std::size_t count) {
  void* p = nullptr;
  if (cudaMalloc(&p, std::max<std::size_t>(count, 1) * sizeof(T)) != cudaSuccess) { std::printf("cudaMalloc failed\n"); std::exit(2); }
  return static_cast<T*>(p);
}
template <class T> T* upload(std::vector<T> const& v) {
  T* p = device<T>(v.size());
  cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
  return p;
}
template <class T> std::vector<T> download(T const* p, std::size_t count) {
  std::vector<T> v(count);
  cudaDeviceSynchronize();
  cudaMemcpy(v.data(), p, count * sizeof(T), cudaMemcpyDeviceToHost);
  return v;
}
}  // namespace

int main() {
  constexpr unsigned n = 137, k = 259, pk = 512, pn = 144, groups = pk / 32, tiles_k = pk / 256;
  // ---- the fixture: logical levels and metadata, kept as scalars for the CPU equation, and the split-tile bytes
  std::vector<int> level(n * pk, 0);
  std::vector<float> d(n * 2), dm(n * 2);
  std::vector<unsigned> sc(n * groups), mn(n * groups);
  std::vector<std::uint8_t> codes(std::size_t(pn) * pk / 2, 0), meta(std::size_t(pn) * tiles_k * 16, 0);
  auto tile_row = [&](unsigned row, unsigned kb) { return (std::size_t(row / 8) * tiles_k + kb) * 8 + row % 8; };
  for (unsigned r = 0; r < n; ++r) {
    for (unsigned c = 0; c < k; ++c) {
      int const q = int((r * 7 + c * 11) % 16);
      level[r * pk + c] = q;
      codes[tile_row(r, c / 256) * 128 + (c % 256) / 2] |= std::uint8_t(q << (4 * (c & 1)));
    }
    for (unsigned b = 0; b < 2; ++b) {
      std::uint16_t const dh = r == 0 ? 1 : (r % 3 == 0 ? 0x1400 : (r % 3 == 1 ? 0x1800 : 0x1a00));
      std::uint16_t const mh = r == 0 ? 2 : (b == 0 ? 0x1000 : 0x1400);
      d[r * 2 + b] = fp16_value(dh);
      dm[r * 2 + b] = fp16_value(mh);
      std::uint8_t* m16 = &meta[tile_row(r, b) * 16];
      m16[0] = dh & 255; m16[1] = dh >> 8; m16[2] = mh & 255; m16[3] = mh >> 8;
      std::uint8_t* p = m16 + 4;
      for (unsigned g = 0; g < 8; ++g) {
        unsigned const s = (r * 13 + g * 17 + 3) % 64, m = (r * 11 + g * 7 + 5) % 64;
        sc[r * groups + b * 8 + g] = s;
        mn[r * groups + b * 8 + g] = m;
        if (g < 4) { p[g] |= s; p[g + 4] |= m; }
        else { p[g + 4] |= (s & 15) | ((m & 15) << 4); p[g - 4] |= (s >> 4) << 6; p[g] |= (m >> 4) << 6; }
      }
    }
  }
  auto* wc = upload(codes);
  auto* ws = upload(meta);
  PrefillWeight const w{wc, ws, Q4K_LAYOUT_SPLIT_TILES, Q4K_QUANTIZER_Q4K, n, k, pn, pk, codes.size(), meta.size()};
  Stream const stream{};
  std::vector<float> small_tile;
  for (unsigned m : {1u, 3u, 33u, 127u, 128u, 129u, 256u, 257u, 511u, 512u}) {
    int const before = g_failed;
    std::vector<std::uint16_t> x(std::size_t(m) * k);
    for (unsigned r = 0; r < m; ++r)
      for (unsigned c = 0; c < k; ++c) {
        float v = float(int((r * 23 + c * 19) % 67) - 44) * .125f * float(1 + r % 5);
        if (c >= 32 && c < 64) v = 0;
        float const head[5] = {127.f, .5f, 1.5f, -.5f, -1.5f};
        if (c < 5) v = head[c];
        if (r == 2) v = 0;  // a whole zero token
        x[std::size_t(r) * k + c] = bf16_rne(v);
      }
    auto* dx = upload(x);
    auto* qc = device<std::int8_t>(std::size_t(m) * pk);
    auto* qa = device<float>(std::size_t(m) * groups);
    auto* qs = device<std::int32_t>(std::size_t(m) * groups);
    auto* flag = device<int>(1);
    auto* out = device<float>(std::size_t(m) * n);
    cudaMemset(flag, 0, 4);
    Q8Input q{{qc, std::size_t(m) * pk}, {qa, std::size_t(m) * groups}, {qs, std::size_t(m) * groups}, m, k, pk};
    require(bool(pack_q8({dx, x.size()}, q, {flag, 1}, stream)), "pack_q8 accepted", m);
    auto z = download(qc, std::size_t(m) * pk);
    auto a = download(qa, std::size_t(m) * groups);
    auto sum = download(qs, std::size_t(m) * groups);
    require(download(flag, 1)[0] == 0, "finite pack", m);
    // independent quantiser: peak / 127 (1 for a zero group), round to nearest even, clamp, exact sums, zero padding
    std::vector<int> refz(std::size_t(m) * pk), refs(std::size_t(m) * groups, 0);
    std::vector<float> refa(std::size_t(m) * groups);
    bool codes_ok = true, scales_ok = true, bounds_ok = true;
    for (unsigned r = 0; r < m; ++r)
      for (unsigned g = 0; g < groups; ++g) {
        float peak = 0;
        for (unsigned t = 0; t < 32 && g * 32 + t < k; ++t) peak = std::max(peak, std::fabs(bf16_value(x[std::size_t(r) * k + g * 32 + t])));
        std::size_t const idx = std::size_t(r) * groups + g;
        refa[idx] = peak == 0 ? 1.f : peak / 127.f;
        for (unsigned t = 0; t < 32; ++t) {
          unsigned const c = g * 32 + t;
          float const v = c < k ? bf16_value(x[std::size_t(r) * k + c]) : 0.f;
          int const code = std::clamp(int(std::nearbyint(v / refa[idx])), -127, 127);
          refz[std::size_t(r) * pk + c] = code;
          refs[idx] += code;
          codes_ok = codes_ok && z[std::size_t(r) * pk + c] == code;
        }
        scales_ok = scales_ok && a[idx] == refa[idx] && sum[idx] == refs[idx];
        bounds_ok = bounds_ok && std::abs(sum[idx]) <= kQ8SumBound;
      }
    require(codes_ok, "exact independent codes, ties to even and padding", m);
    require(scales_ok, "exact independent scales and sums", m);
    require(bounds_ok, "sum bound", m);
    require(z[0] == 127 && z[1] == 0 && z[2] == 2 && z[3] == 0 && z[4] == -2, "halfway ties and saturation endpoint", m);
    require(sum[2] < 0, "negative activation sum in the fixture", m);
    require(bool(q4k_q8_project(w, q, {out, std::size_t(m) * n}, stream)), "projection accepted", m);
    auto y = download(out, std::size_t(m) * n);
    if (m == 1) {
      // spans that are only four-byte aligned, a residual, and guard words at both ends of the output
      std::vector<std::uint8_t> shifted(codes.size() + 8, 0);
      std::copy(codes.begin(), codes.end(), shifted.begin() + 4);
      auto* wshift = upload(shifted);
      std::vector<std::int8_t> zshift(pk + 8, 99);
      std::copy(z.begin(), z.end(), zshift.begin() + 4);
      auto* qshift = upload(zshift);
      std::vector<float> guards(n + 2, -12345.f), residual(n);
      for (unsigned r = 0; r < n; ++r) residual[r] = float(int(r % 17) - 8) * .125f;
      auto* guarded = upload(guards);
      auto* res = upload(residual);
      bool same = true, guard = true;
      for (unsigned variant = 0; variant < 4; ++variant) {
        PrefillWeight sw = w;
        Q8Input sq = q;
        if (variant & 1) sw.codes = wshift + 4;
        if (variant & 2) sq.codes = {qshift + 4, pk};
        require(bool(q4k_q8_project(sw, sq, {guarded + 1, n}, stream, {res, n})), "shifted spans accepted", m);
        auto got = download(guarded, n + 2);
        for (unsigned r = 0; r < n; ++r) same = same && got[r + 1] == y[r] + residual[r];
        guard = guard && got.front() == -12345.f && got.back() == -12345.f;
      }
      require(same, "aligned / unaligned loads and residual agree exactly", m);
      require(guard, "row-tail output guards", m);
    }
    if (m == 127) small_tile = y;
    if (m >= 128) require(std::equal(small_tile.begin(), small_tile.end(), y.begin()), "rows do not depend on the token count, bit for bit", m);
    bool dots_ok = true, affine_ok = true;
    for (unsigned t = 0; t < m; ++t)
      for (unsigned r = 0; r < n; ++r) {
        double ref = 0;
        for (unsigned g = 0; g < groups; ++g) {
          int dot = 0;
          for (unsigned j = 0; j < 32 && g * 32 + j < k; ++j) dot += level[r * pk + g * 32 + j] * refz[std::size_t(t) * pk + g * 32 + j];
          dots_ok = dots_ok && std::abs(dot) <= kQ4KQ8DotBound;
          float const s = d[r * 2 + g / 8] * float(sc[r * groups + g]), minimum = dm[r * 2 + g / 8] * float(mn[r * groups + g]);
          ref += double(refa[std::size_t(t) * groups + g]) * (double(s) * dot - double(minimum) * refs[std::size_t(t) * groups + g]);
        }
        float const got = y[std::size_t(t) * n + r];
        affine_ok = affine_ok && std::isfinite(got) && std::fabs(got - ref) <= .02 + .002 * std::fabs(ref);
      }
    require(dots_ok, "raw dot bound", m);
    require(affine_ok, "affine contraction within 0.02 + 0.002 |ref|", m);
    require(bool(q4k_q8_project(w, q, {out, std::size_t(m) * n}, stream)) && download(out, std::size_t(m) * n) == y, "reused pack gives the identical output", m);
    require(download(qc, std::size_t(m) * pk) == z && download(qa, std::size_t(m) * groups) == a && download(qs, std::size_t(m) * groups) == sum,
            "the consumer leaves the pack untouched", m);
    Q8Input bad = q;
    bad.codes = bad.codes.first(1);
    require(!q4k_q8_project(w, bad, {out, std::size_t(m) * n}, stream), "truncated input rejected", m);
    PrefillWeight badw = w;
    --badw.codes_bytes;
    require(!q4k_q8_project(badw, q, {out, std::size_t(m) * n}, stream), "truncated weights rejected", m);
    for (std::uint16_t bits : {std::uint16_t(0x7f80), std::uint16_t(0xff80), std::uint16_t(0x7fc0)}) {
      x[0] = bits;
      cudaMemcpy(dx, x.data(), x.size() * 2, cudaMemcpyHostToDevice);
      cudaMemset(flag, 0, 4);
      require(bool(pack_q8({dx, x.size()}, q, {flag, 1}, stream)), "non-finite pack is enqueued", m);
      require(download(flag, 1)[0] == 1 && std::isnan(download(qa, 1)[0]), "non-finite pack flagged, not a finite zero", m);
    }
    for (void* p : {static_cast<void*>(dx), static_cast<void*>(qc), static_cast<void*>(qa), static_cast<void*>(qs), static_cast<void*>(flag), static_cast<void*>(out)}) cudaFree(p);
    if (g_failed == before) std::printf("Q4_K/Q8 M=%u pack, affine equation, tails, bounds, reuse, rejection PASS\n", m);
  }
  int status = -1;
  q4k_kernel_status(&status);
  require(status == 0, "no bounded wait inside a kernel gave up", 0);
  return g_failed == 0 ? 0 : 1;
}
