// C-ABI layer: argument validation, regime dispatch and scratch ownership.
//
// Validation follows the reference's host checks: geometry (valid_input / valid_weight,
// cuda/q4k_q8.cu:286-298), device-span membership (device_region, cuda/prefill.cu:273-309)
// and pairwise non-overlap of live operands (distinct, cuda/q4k_q8.cu:270-285).  A call
// rejected here has launched nothing and left every device buffer untouched.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <limits>
#include <atomic>
#include <mutex>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "../../include/q4k_b200.h"
#include "launch.h"

namespace {

thread_local char g_error[512] = "";
thread_local int g_cuda_status = 0;

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}
int fail_cuda(cudaError_t st, const char* op) {
  (void)cudaGetLastError();  // consume the sticky status, as the reference's check() does
  g_cuda_status = int(st);
  return fail(Q4K_ERR_STATUS, "%s: %s", op, cudaGetErrorString(st));
}
#define Q4K_CUDA(expr, op)                                  \
  do {                                                      \
    cudaError_t st__ = (expr);                              \
    if (st__ != cudaSuccess) return fail_cuda(st__, op);    \
  } while (0)

// Profiler ranges with the reference's strings (src/runtime/profiling.hpp, cuda/q4k_q8.cu:299-302,326,383), opt-in
// per thread like the reference's, so that traces of the two engines line up.
thread_local bool g_ranges = false;
class ScopedRange {
 public:
  template <class... Args>
  explicit ScopedRange(char const* format, Args... args) noexcept : active_(g_ranges) {
    if (active_) {
      char name[384];
      std::snprintf(name, sizeof name, format, args...);
      nvtxRangePushA(name);
    }
  }
  ~ScopedRange() {
    if (active_) nvtxRangePop();
  }
  ScopedRange(ScopedRange const&) = delete;
  ScopedRange& operator=(ScopedRange const&) = delete;

 private:
  bool active_;
};

using MemGetAddressRange = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
MemGetAddressRange address_range_fn() {
  static MemGetAddressRange fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<MemGetAddressRange>(p);
  }();
  return fn;
}

struct Region {
  const void* p;
  uint64_t bytes;
  uint32_t alignment;
  const char* name;
};

int check_span(const Region& r, int device) {
  auto const begin = reinterpret_cast<uintptr_t>(r.p);
  if (!r.p || r.bytes == 0) return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: empty span", r.name);
  if (r.bytes > std::numeric_limits<uintptr_t>::max() - begin)
    return fail(Q4K_ERR_OVERFLOW, "%s: address overflow", r.name);
  if (r.alignment == 0 || begin % r.alignment != 0)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: misaligned pointer", r.name);
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, r.p) != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: pointer is not device memory", r.name);
  }
  if (attr.type != cudaMemoryTypeDevice || attr.device != device)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: not device memory of the current device", r.name);
  if (auto fn = address_range_fn()) {
    CUdeviceptr base = 0;
    size_t size = 0;
    if (fn(&base, &size, static_cast<CUdeviceptr>(begin)) != CUDA_SUCCESS)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: unknown device allocation", r.name);
    if (begin < base || begin + r.bytes > base + size)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: operand exceeds its allocation", r.name);
  }
  return Q4K_OK;
}

int check_distinct(const Region* regions, int count, bool trusted) {
  int device = 0;
  if (!trusted) Q4K_CUDA(cudaGetDevice(&device), "cudaGetDevice");
  for (int i = 0; i < count; ++i) {
    if (!trusted) {
      if (int st = check_span(regions[i], device)) return st;
    } else if (!regions[i].p) {
      return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: null pointer", regions[i].name);
    }
    auto const b = reinterpret_cast<uintptr_t>(regions[i].p);
    for (int j = 0; j < i; ++j) {
      auto const c = reinterpret_cast<uintptr_t>(regions[j].p);
      if (b < c + regions[j].bytes && c < b + regions[i].bytes)
        return fail(Q4K_ERR_INVALID_ARGUMENT, "live operands overlap: %s and %s", regions[i].name, regions[j].name);
    }
  }
  return Q4K_OK;
}

bool valid_input(const q4k_q8_input& x) {
  return x.m && x.m <= Q4K_MAX_TOKENS && x.k && x.k <= Q4K_MAX_K && x.padded_k == q4k_pad_k(x.k) &&
         x.codes_len == uint64_t(x.m) * x.padded_k && x.scales_len == x.codes_len / 32 &&
         x.sums_len == x.scales_len;
}

int valid_weight(const q4k_weight* w, const char* name) {
  if (!w) return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: null weight", name);
  if (!w->n || w->n > Q4K_MAX_N || !w->k || w->k > Q4K_MAX_K || w->layout != Q4K_LAYOUT_SPLIT_TILES ||
      w->quantizer != Q4K_QUANTIZER_Q4K || w->padded_n != q4k_pad_n(w->n) || w->padded_k != q4k_pad_k(w->k) ||
      w->codes_bytes != q4k_code_bytes(w->padded_n, w->padded_k) ||
      w->scales_bytes != q4k_scale_bytes(w->padded_n, w->padded_k))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "%s: Q4_K split-tile geometry required", name);
  return Q4K_OK;
}

q4k::WeightView view(const q4k_weight& w) {
  return {static_cast<const uint8_t*>(w.codes), static_cast<const uint8_t*>(w.scales), w.n, w.padded_n,
          w.padded_k / 256};
}
q4k::Q8View view(const q4k_q8_input& x) { return {x.codes, x.scales, x.sums, x.m, x.padded_k}; }
q4k::Q8Out out_view(const q4k_q8_input& x) { return {x.codes, x.scales, x.sums, x.m, x.padded_k}; }

// Status word of the kernels that wait on device-side barriers: one per device, in the library's own
// device image, so that it exists without any allocation and whatever scratch a call uses.
__device__ int g_kernel_status_word;
std::mutex g_status_mutex;
int* g_status_address[64];

// Library-owned split-K scratch, one chain per device: [ticket region | fp32 partial tiles].
// Tickets are zeroed at allocation and every kernel leaves them zero.  A block is never freed or
// moved once handed out: launches in flight and captured graphs keep its address, so growing
// allocates a larger block and retires the old one (kept until the process ends).
constexpr uint64_t kTicketRegion = 256 * 1024;
struct Scratch {
  void* p = nullptr;
  uint64_t bytes = 0;
};
std::mutex g_scratch_mutex;
Scratch g_scratch[64];
std::vector<Scratch> g_retired[64];

int own_scratch(uint64_t partial_bytes, void** out, cudaStream_t stream) {
  int device = 0;
  Q4K_CUDA(cudaGetDevice(&device), "cudaGetDevice");
  if (device < 0 || device >= 64) return fail(Q4K_ERR_INVALID_ARGUMENT, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  Scratch& s = g_scratch[device];
  uint64_t const need = kTicketRegion + partial_bytes;
  if (s.bytes < need) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) (void)cudaGetLastError();
    if (cap != cudaStreamCaptureStatusNone)
      return fail(Q4K_ERR_INVALID_ARGUMENT,
                  "split-K scratch of %llu bytes is needed while the stream is capturing: call q4k_reserve_scratch first",
                  static_cast<unsigned long long>(partial_bytes));
    uint64_t const bytes = need < (8ull << 20) ? (8ull << 20) : (need + (1ull << 20) - 1) / (1ull << 20) * (1ull << 20);
    void* p = nullptr;
    Q4K_CUDA(cudaMalloc(&p, bytes), "scratch.alloc");
    cudaError_t st = cudaMemset(p, 0, kTicketRegion);
    if (st != cudaSuccess) { (void)cudaFree(p); return fail_cuda(st, "scratch.clear"); }
    if (s.p) g_retired[device].push_back(s);
    s.p = p;
    s.bytes = bytes;
  }
  *out = s.p;
  return Q4K_OK;
}

// Caller-provided scratch: checked like every other operand, tickets cleared on the stream.
int caller_scratch(const q4k_project_options* opt, uint64_t partial_bytes, uint64_t ticket_bytes, bool trusted,
                   cudaStream_t stream, void** out) {
  if (opt->workspace_bytes < kTicketRegion + partial_bytes || ticket_bytes > kTicketRegion)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: workspace too small");
  if (!trusted) {
    int device = 0;
    Q4K_CUDA(cudaGetDevice(&device), "cudaGetDevice");
    if (int st = check_span(Region{opt->workspace, opt->workspace_bytes, 256, "workspace"}, device)) return st;
  } else if (reinterpret_cast<uintptr_t>(opt->workspace) % 256 != 0) {
    return fail(Q4K_ERR_INVALID_ARGUMENT, "workspace: misaligned pointer");
  }
  if (ticket_bytes) Q4K_CUDA(cudaMemsetAsync(opt->workspace, 0, ticket_bytes, stream), "q4k_q8.clear_tickets");
  *out = opt->workspace;
  return Q4K_OK;
}

constexpr uint32_t kFlagTrustedSpans = 1u, kFlagInputSettled = 2u;

int project_impl(const q4k_weight* weight, const q4k_q8_input& x, float* output, uint64_t output_len,
                 const float* residual, uint64_t residual_len, const q4k_project_options* opt,
                 cudaStream_t stream, bool residual_in_place = false, char const* role = "projection") {
  if (int st = valid_weight(weight, "weight")) return st;
  const q4k_weight& w = *weight;
  if (!valid_input(x) || x.k != w.k || output_len != uint64_t(x.m) * w.n ||
      (residual_len != 0 && residual_len != output_len) || (residual_len != 0 && !residual))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: invalid geometry");
  uint32_t const G = x.padded_k / 32;
  int32_t* partials = opt ? opt->partials : nullptr;
  if (partials && opt->partials_len != uint64_t(x.m) * w.n * G)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: partials length must be m*n*padded_k/32");
  bool const trusted = opt && (opt->flags & kFlagTrustedSpans);
  Region regions[8] = {{w.codes, w.codes_bytes, 4, "weight.codes"},
                       {w.scales, w.scales_bytes, 2, "weight.scales"},
                       {x.codes, x.codes_len, 4, "input.codes"},
                       {x.scales, x.scales_len * 4, 4, "input.scales"},
                       {x.sums, x.sums_len * 4, 4, "input.sums"},
                       {output, output_len * 4, 4, "output"},
                       {nullptr, 0, 4, ""},
                       {nullptr, 0, 4, ""}};
  int count = 6;
  // in place: every kernel reads residual[i] and writes output[i] from the same thread, in that order
  if (residual_len && !(residual_in_place && residual == output)) regions[count++] = {residual, residual_len * 4, 4, "residual"};
  if (partials) regions[count++] = {partials, opt->partials_len * 4, 4, "partials"};
  if (int st = check_distinct(regions, count, trusted)) return st;

  uint32_t kernel = opt ? opt->kernel : Q4K_KERNEL_AUTO;
  if (kernel == Q4K_KERNEL_AUTO) {
    // Up to sixteen tokens: the TMA-streamed kernel when the weights are 16-byte aligned (for a
    // single token only with overlapped launches, where its early weight prefetch pays; serialised,
    // dp4a measured a little faster there), else dp4a / cluster MMA.  Beyond: tcgen05 when TMA
    // alignment allows.
    bool const tma_ok = x.m <= q4k::kGemvTmaMaxTokens && q4k::gemv_tma_supported(view(w), view(x));
    if (tma_ok && (x.m >= 2 || q4k::launch_overlap())) kernel = Q4K_KERNEL_GEMV_TMA;
    else if (x.m <= 2 || (x.m <= q4k::kGemvDp4aMaxTokens && w.padded_n >= 32768)) kernel = Q4K_KERNEL_GEMV_DP4A;
    else if (x.m <= 16) kernel = Q4K_KERNEL_GEMV_MMA;
    else kernel = q4k::tcgen05_supported(view(w), view(x)) ? Q4K_KERNEL_TCGEN05 : Q4K_KERNEL_MMA;
  }
  const float* res = residual_len ? residual : nullptr;
  ScopedRange range("qw38:op name=q4k_project m=%u n=%u k=%u role=%s residual=%u compute=%s", unsigned(x.m), unsigned(w.n),
                    unsigned(w.k), role, unsigned(res != nullptr), kernel == Q4K_KERNEL_GEMV_DP4A ? "integer_dp4a" : "integer_mma");
  if (kernel == Q4K_KERNEL_GEMV_DP4A) {
    if (x.m > q4k::kGemvDp4aMaxTokens) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: dp4a kernel takes m <= 4");
    Q4K_CUDA(q4k::launch_gemv_dp4a(view(w), view(x), output, res, partials, stream), "q4k_q8.gemv_dp4a");
    return Q4K_OK;
  }
  if (kernel == Q4K_KERNEL_GEMV_MMA) {
    if (x.m > 16) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: the cluster mma kernel takes m <= 16");
    uint32_t const rgroups = opt ? opt->row_groups : 0, split = opt ? opt->split_k : 0;
    if ((rgroups != 0 && rgroups != 4 && rgroups != 8) || split > 8)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: row_groups must be 4 or 8 and split_k <= 8");
    q4k::GemvMmaPlan plan = q4k::plan_gemv_mma(x.m, w.n, w.padded_k / 256, split, rgroups);
    Q4K_CUDA(q4k::launch_gemv_mma(view(w), view(x), output, res, partials, plan, stream), "q4k_q8.gemv_mma");
    return Q4K_OK;
  }
  if (kernel == Q4K_KERNEL_GEMV_TMA) {
    if (!q4k::gemv_tma_supported(view(w), view(x)))
      return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: the TMA gemv kernel takes m <= 16 and 16-byte aligned weights");
    q4k::GemvTmaPlan plan = q4k::plan_gemv_tma(x.m, w.n, w.padded_k / 256, opt ? opt->split_k : 0, opt ? opt->row_groups : 0);
    uint64_t const partial_bytes = plan.split_k > 1 ? uint64_t(plan.split_k) * x.m * w.n * 4 : 0;
    void* scratch = nullptr;
    if (opt && opt->workspace) {
      if (int st = caller_scratch(opt, partial_bytes, plan.split_k > 1 ? uint64_t(plan.ranges) * 4 : 0, trusted, stream, &scratch)) return st;
    } else if (int st = own_scratch(partial_bytes, &scratch, stream)) {
      return st;
    }
    int* status = q4k::kernel_status_word();
    if (!status) return Q4K_ERR_STATUS;
    plan.input_settled = (opt && (opt->flags & kFlagInputSettled)) ? 1u : 0u;
    Q4K_CUDA(q4k::launch_gemv_tma(view(w), view(x), output, res, partials, plan,
                                  static_cast<uint8_t*>(scratch) + kTicketRegion, static_cast<uint32_t*>(scratch),
                                  status, stream),
             "q4k_q8.gemv_tma");
    return Q4K_OK;
  }
  if (kernel == Q4K_KERNEL_TCGEN05) {
    if (!q4k::tcgen05_supported(view(w), view(x)))
      return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: the tcgen05 kernel needs 16-byte aligned operands");
    q4k::TcPlan plan = q4k::plan_tcgen05(x.m, w.n, w.padded_k / 256, opt ? opt->split_k : 0);
    uint64_t const tiles = uint64_t((w.padded_n + 127) / 128) * ((x.m + plan.ntok - 1) / plan.ntok);
    if (plan.split_k > 1 && tiles * 4 > kTicketRegion - 64)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: too many tiles for split-K");
    uint64_t const partial_bytes = plan.split_k > 1 ? uint64_t(plan.split_k) * x.m * w.n * 4 : 0;
    void* scratch = nullptr;
    if (opt && opt->workspace) {
      if (int st = caller_scratch(opt, partial_bytes, plan.split_k > 1 ? tiles * 4 : 0, trusted, stream, &scratch)) return st;
    } else if (int st = own_scratch(partial_bytes, &scratch, stream)) {
      return st;
    }
    int* status = q4k::kernel_status_word();
    if (!status) return Q4K_ERR_STATUS;
    q4k::TcOutput tc = q4k::tc_output(output, res);
    tc.input_settled = (opt && (opt->flags & kFlagInputSettled)) ? 1u : 0u;
    Q4K_CUDA(q4k::launch_mmq_tcgen05(view(w), view(x), tc, partials, plan,
                                     static_cast<uint8_t*>(scratch) + kTicketRegion, static_cast<uint32_t*>(scratch),
                                     status, stream),
             "q4k_q8.mmq_tcgen05");
    return Q4K_OK;
  }
  if (kernel == Q4K_KERNEL_MMA) {
    q4k::MmaPlan plan = q4k::plan_mma(x.m, w.n, w.padded_k / 256, opt ? opt->split_k : 0);
    void* scratch = nullptr;
    if (plan.split_k > 1) {
      uint64_t const row_tiles = (w.padded_n / 8 + 7) / 8, token_tiles = (x.m + plan.token_tile - 1) / plan.token_tile;
      if (row_tiles * token_tiles * 4 > kTicketRegion)
        return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: too many tiles for split-K");
      uint64_t const partial_bytes = uint64_t(plan.split_k) * x.m * w.n * 4;
      if (opt && opt->workspace) {
        if (int st = caller_scratch(opt, partial_bytes, row_tiles * token_tiles * 4, trusted, stream, &scratch)) return st;
      } else if (int st = own_scratch(partial_bytes, &scratch, stream)) {
        return st;
      }
    }
    Q4K_CUDA(q4k::launch_mmq_mma(view(w), view(x), output, res, partials, plan,
                                 scratch ? static_cast<uint8_t*>(scratch) + kTicketRegion : nullptr,
                                 static_cast<uint32_t*>(scratch), stream),
             "q4k_q8.mmq_mma");
    return Q4K_OK;
  }
  return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project: unknown kernel selector %u", kernel);
}

int pack_impl(const void* input, bool fp32, uint64_t input_len, const q4k_q8_input& x, int* failure,
              cudaStream_t stream) {
  if (!valid_input(x) || input_len != uint64_t(x.m) * x.k || !failure)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.pack: invalid geometry");
  Region regions[5] = {{input, input_len * (fp32 ? 4u : 2u), fp32 ? 4u : 2u, "input"},
                       {x.codes, x.codes_len, 4, "output.codes"},
                       {x.scales, x.scales_len * 4, 4, "output.scales"},
                       {x.sums, x.sums_len * 4, 4, "output.sums"},
                       {failure, 4, 4, "failure"}};
  if (int st = check_distinct(regions, 5, false)) return st;
  ScopedRange range("qw38:op name=q8_pack m=%u n=%u k=%u", unsigned(x.m), unsigned(x.k), 1u);
  Q4K_CUDA(q4k::launch_pack_q8(input, fp32, out_view(x), x.k, failure, stream), "q8.pack");
  return Q4K_OK;
}

}  // namespace

namespace {
std::atomic<bool> g_launch_overlap{false};
}
namespace q4k {
bool launch_overlap() { return g_launch_overlap.load(std::memory_order_relaxed); }
int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}
int set_error_cuda(cudaError_t status, const char* operation) { return fail_cuda(status, operation); }
int* kernel_status_word() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
    (void)cudaGetLastError();
    fail(Q4K_ERR_STATUS, "kernel status word: no current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_address[device]) {
    void* p = nullptr;
    cudaError_t st = cudaGetSymbolAddress(&p, g_kernel_status_word);
    if (st != cudaSuccess) { fail_cuda(st, "kernel status word"); return nullptr; }
    g_status_address[device] = static_cast<int*>(p);
  }
  return g_status_address[device];
}
int check_operands(const Operand* operands, int count) {
  Region regions[16];
  if (count > 16) return fail(Q4K_ERR_INVALID_ARGUMENT, "too many operands");
  for (int i = 0; i < count; ++i) regions[i] = Region{operands[i].p, operands[i].bytes, operands[i].alignment, operands[i].name};
  return check_distinct(regions, count, false);
}
}  // namespace q4k

extern "C" {

const char* q4k_last_error(void) { return g_error; }
int q4k_last_cuda_status(void) { return g_cuda_status; }
uint32_t q4k_abi_version(void) { return 1; }

void q4k_set_profiling_ranges(int enabled) { g_ranges = enabled != 0; }
int q4k_get_profiling_ranges(void) { return g_ranges ? 1 : 0; }

void q4k_set_launch_overlap(int enabled) { g_launch_overlap.store(enabled != 0, std::memory_order_relaxed); }
int q4k_get_launch_overlap(void) { return g_launch_overlap.load(std::memory_order_relaxed) ? 1 : 0; }

uint64_t q4k_pad_n(uint32_t n) { return n == 0 ? 0 : (uint64_t(n) + 7) / 8 * 8; }
uint32_t q4k_pad_k(uint32_t k) { return k == 0 ? 0 : (k + 255u) / 256u * 256u; }
uint64_t q4k_code_bytes(uint32_t padded_n, uint32_t padded_k) { return uint64_t(padded_n) * padded_k / 2; }
uint64_t q4k_scale_bytes(uint32_t padded_n, uint32_t padded_k) { return uint64_t(padded_n) * (padded_k / 256) * 16; }

int q4k_kernel_status(int* value) {
  if (!value) return fail(Q4K_ERR_INVALID_ARGUMENT, "kernel_status: null output");
  *value = 0;
  int* word = q4k::kernel_status_word();
  if (!word) return Q4K_ERR_STATUS;
  Q4K_CUDA(cudaDeviceSynchronize(), "kernel_status.sync");
  Q4K_CUDA(cudaMemcpy(value, word, 4, cudaMemcpyDeviceToHost), "kernel_status.read");
  if (*value != 0) {
    // A launch that gave up may have left split-K tickets of the library's scratch behind: start clean.
    Q4K_CUDA(cudaMemset(word, 0, 4), "kernel_status.clear");
    int device = 0;
    Q4K_CUDA(cudaGetDevice(&device), "cudaGetDevice");
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (device >= 0 && device < 64) {
      if (g_scratch[device].p) Q4K_CUDA(cudaMemset(g_scratch[device].p, 0, kTicketRegion), "kernel_status.tickets");
      for (auto const& r : g_retired[device]) Q4K_CUDA(cudaMemset(r.p, 0, kTicketRegion), "kernel_status.tickets");
    }
  }
  return Q4K_OK;
}

int q4k_reserve_scratch(uint64_t partial_bytes, void* stream) {
  void* p = nullptr;
  return own_scratch(partial_bytes, &p, static_cast<cudaStream_t>(stream));
}

int q4k_q8_project_gather(const q4k_weight* shard, q4k_q8_input x, const q4k_gather_desc* desc, const float* residual,
                          uint64_t residual_len, void* stream_handle) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (int st = valid_weight(shard, "shard")) return st;
  const q4k_weight& w = *shard;
  if (!desc) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project_gather: null descriptor");
  if (!valid_input(x) || x.k != w.k) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project_gather: invalid geometry");
  if (desc->ranks < 1 || desc->ranks > 8 || desc->rank >= desc->ranks || desc->row_offset % 8 != 0 ||
      uint64_t(desc->row_offset) + w.n > desc->total_rows)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project_gather: ranks 1..8, rank < ranks, row_offset a multiple of 8 and inside total_rows");
  for (uint32_t g = 0; g < desc->ranks; ++g)
    if (!desc->outputs[g] || reinterpret_cast<uintptr_t>(desc->outputs[g]) % 4 != 0 || !desc->flags[g] ||
        reinterpret_cast<uintptr_t>(desc->flags[g]) % 4 != 0)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project_gather: every rank needs a 4-byte aligned output and flag array");
  if ((residual_len != 0 && residual_len != uint64_t(x.m) * desc->total_rows) || (residual_len != 0 && !residual))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project_gather: residual must cover m x total_rows");
  bool const narrow = x.m <= q4k::kGemvTmaMaxTokens;
  if (narrow ? !q4k::gemv_tma_supported(view(w), view(x)) : !q4k::tcgen05_supported(view(w), view(x)))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.project_gather: needs 16-byte aligned weight shards and activations");
  // Peer mappings cannot be checked against this device's allocations; the local operands are.
  Region regions[5] = {{w.codes, w.codes_bytes, 4, "shard.codes"},
                       {w.scales, w.scales_bytes, 2, "shard.scales"},
                       {x.codes, x.codes_len, 4, "input.codes"},
                       {x.scales, x.scales_len * 4, 4, "input.scales"},
                       {x.sums, x.sums_len * 4, 4, "input.sums"}};
  if (int st = check_distinct(regions, 5, false)) return st;
  int* const status = q4k::kernel_status_word();
  if (!status) return Q4K_ERR_STATUS;
  // words 8 and 9 of this rank's own flag array: its unannounced projections and the block counter
  uint32_t* const unsignalled = desc->flags[desc->rank] + 8;
  uint32_t* const done = desc->flags[desc->rank] + 9;
  void* scratch = nullptr;
  if (narrow) {
    q4k::GemvTmaPlan plan = q4k::plan_gemv_tma(x.m, w.n, w.padded_k / 256, 0, 0);
    uint64_t const partial_bytes = plan.split_k > 1 ? uint64_t(plan.split_k) * x.m * w.n * 4 : 0;
    if (int st = own_scratch(partial_bytes, &scratch, stream)) return st;
    uint8_t* const base = static_cast<uint8_t*>(scratch);
    q4k::GemvTmaGather gather{};
    for (uint32_t g = 0; g < desc->ranks; ++g) { gather.outputs[g] = desc->outputs[g]; gather.flags[g] = desc->flags[g]; }
    gather.unsignalled = unsignalled;
    gather.done = done;
    gather.ranks = desc->ranks; gather.rank = desc->rank; gather.row_offset = desc->row_offset; gather.total_rows = desc->total_rows;
    plan.input_settled = (desc->options & kFlagInputSettled) ? 1u : 0u;
    Q4K_CUDA(q4k::launch_gemv_tma(view(w), view(x), nullptr, residual_len ? residual : nullptr, nullptr, plan,
                                  base + kTicketRegion, reinterpret_cast<uint32_t*>(base), status, stream, &gather),
             "q4k_q8.gemv_tma_gather");
    return Q4K_OK;
  }
  // More than sixteen tokens: the tcgen05 kernel, whose writer stores into every rank's buffer the same way.
  q4k::TcPlan plan = q4k::plan_tcgen05(x.m, w.n, w.padded_k / 256, 0);
  uint64_t const tiles = uint64_t((w.padded_n + 127) / 128) * ((x.m + plan.ntok - 1) / plan.ntok);
  if (plan.split_k > 1 && tiles * 4 > kTicketRegion - 64) plan.split_k = 1;
  uint64_t const partial_bytes = plan.split_k > 1 ? uint64_t(plan.split_k) * x.m * w.n * 4 : 0;
  if (int st = own_scratch(partial_bytes, &scratch, stream)) return st;
  uint8_t* const base = static_cast<uint8_t*>(scratch);
  q4k::TcOutput out{};
  for (uint32_t g = 0; g < desc->ranks; ++g) { out.out[g] = desc->outputs[g]; out.flags[g] = desc->flags[g]; }
  out.residual = residual_len ? residual : nullptr;
  out.ndst = desc->ranks; out.stride = desc->total_rows; out.row0 = desc->row_offset;
  out.done = done; out.unsignalled = unsignalled; out.rank = desc->rank;
  out.input_settled = (desc->options & kFlagInputSettled) ? 1u : 0u;
  Q4K_CUDA(q4k::launch_mmq_tcgen05(view(w), view(x), out, nullptr, plan, base + kTicketRegion, reinterpret_cast<uint32_t*>(base),
                                   status, stream),
           "q4k_q8.mmq_tcgen05_gather");
  return Q4K_OK;
}

static int peer_wait_impl(const q4k_gather_desc* desc, long long limit, void* stream_handle) {
  if (!desc || desc->ranks < 1 || desc->ranks > 8 || desc->rank >= desc->ranks)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "peer_wait: descriptor with ranks 1..8 and rank < ranks");
  for (uint32_t g = 0; g < desc->ranks; ++g)
    if (!desc->flags[g] || reinterpret_cast<uintptr_t>(desc->flags[g]) % 4 != 0)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "peer_wait: every rank needs a 4-byte aligned flag array");
  int* const status = q4k::kernel_status_word();
  if (!status) return Q4K_ERR_STATUS;
  Q4K_CUDA(q4k::launch_peer_wait(desc->flags, desc->flags[desc->rank] + 8, desc->ranks, desc->rank, limit, status,
                                 static_cast<cudaStream_t>(stream_handle)),
           "peer_wait");
  return Q4K_OK;
}

int q4k_peer_wait(const q4k_gather_desc* desc, uint64_t limit_cycles, void* stream_handle) {
  long long const limit = limit_cycles == 0 || limit_cycles > 0x7fffffffffffffffull ? 4000000000LL
                                                                                    : static_cast<long long>(limit_cycles);
  return peer_wait_impl(desc, limit, stream_handle);
}

int q4k_peer_announce(const q4k_gather_desc* desc, void* stream_handle) { return peer_wait_impl(desc, -1, stream_handle); }

// ---- decode entry points: quantise bf16 rows, project, apply a DecodeEpilogue -------------------
namespace {
uint64_t align256(uint64_t v) { return (v + 255) / 256 * 256; }

struct DecodeScratch {
  q4k_q8_input q8;
  float* rows;        // 2 * m * n_total floats
  uint64_t rows_len;
};

uint64_t decode_scratch_bytes(uint32_t m, uint64_t n_total, uint32_t k) {
  uint64_t const pk = (uint64_t(k) + 255) / 256 * 256, G = pk / 32;
  return align256(uint64_t(m) * pk) + 2 * align256(uint64_t(m) * G * 4) + align256(2 * uint64_t(m) * n_total * 4);
}

int carve_decode_scratch(void* workspace, uint64_t workspace_bytes, uint32_t m, uint64_t n_total, uint32_t k, DecodeScratch* out) {
  if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || workspace_bytes < decode_scratch_bytes(m, n_total, k))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: workspace must be 256-byte aligned and hold q4k_decode_workspace_bytes");
  uint32_t const pk = uint32_t((uint64_t(k) + 255) / 256 * 256);
  uint64_t const G = pk / 32;
  uint8_t* p = static_cast<uint8_t*>(workspace);
  out->q8.codes = reinterpret_cast<int8_t*>(p); p += align256(uint64_t(m) * pk);
  out->q8.scales = reinterpret_cast<float*>(p); p += align256(uint64_t(m) * G * 4);
  out->q8.sums = reinterpret_cast<int32_t*>(p); p += align256(uint64_t(m) * G * 4);
  out->q8.codes_len = uint64_t(m) * pk; out->q8.scales_len = out->q8.sums_len = uint64_t(m) * G;
  out->q8.m = m; out->q8.k = k; out->q8.padded_k = pk;
  out->rows = reinterpret_cast<float*>(p);
  out->rows_len = 2 * uint64_t(m) * n_total;
  return Q4K_OK;
}

// Geometry and epilogue contract of one descriptor (cuda/decode_mmv.cu:440-505).
int valid_decode_desc(const q4k_decode_desc* d, bool paired_b, const char* what, uint32_t max_m = 16) {
  if (!d) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: null %s descriptor", what);
  if (int st = valid_weight(&d->weight, what)) return st;
  if (d->activation_policy != Q4K_ACTIVATION_Q8_K32 && !(d->activation_policy == Q4K_ACTIVATION_BF16 && max_m <= 16))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: %s activation policy must be Q8-K32 (or Bf16 on the decode entries)", what);
  if (d->activation_policy == Q4K_ACTIVATION_BF16 && reinterpret_cast<uintptr_t>(d->input) % 2 != 0)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: %s input must be 2-byte aligned", what);
  if (d->m < 1 || d->m > max_m || !d->input || d->input_len != uint64_t(d->m) * d->weight.k)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: %s needs 1..%u bf16 input rows of k columns", what, max_m);
  uint64_t const cells = uint64_t(d->m) * d->weight.n;
  switch (d->epilogue) {
    case Q4K_EPILOGUE_SWIGLU_STORE_BF16:
      if (!paired_b) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: SwiGLU epilogue requires paired gate/up launch");
      [[fallthrough]];
    case Q4K_EPILOGUE_STORE_BF16:
    case Q4K_EPILOGUE_STORE_FP32:
      if (d->residual || d->residual_len) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: store epilogue must not supply residual");
      if (!d->output || d->output_len != cells) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: %s output must hold m*n elements", what);
      break;
    case Q4K_EPILOGUE_RESIDUAL_ADD_FP32:
      if (!d->residual || d->residual_len != cells) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: %s residual must hold m*n floats", what);
      if (d->output ? d->output_len != cells : d->output_len != 0)
        return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: %s output must hold m*n floats or be empty (in-place residual update)", what);
      break;
    default:
      return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: unknown epilogue");
  }
  return Q4K_OK;
}

// Projection + epilogue of one descriptor whose input is already quantised.  `rows` is m*n floats of scratch.
// fp32 rows of one descriptor under its activation policy, residual added last.
int decode_rows(const q4k_decode_desc& d, const q4k_q8_input& q8, float* out, const float* residual, cudaStream_t stream) {
  uint64_t const cells = uint64_t(d.m) * d.weight.n;
  if (d.activation_policy == Q4K_ACTIVATION_Q8_K32)
    return project_impl(&d.weight, q8, out, cells, residual, residual ? cells : 0, nullptr, stream, true);
  Region regions[3] = {{d.weight.codes, d.weight.codes_bytes, 4, "weight.codes"},
                       {d.weight.scales, d.weight.scales_bytes, 2, "weight.scales"},
                       {out, cells * 4, 4, "output"}};
  if (int st = check_distinct(regions, 3, false)) return st;
  Q4K_CUDA(q4k::launch_gemv_bf16w(view(d.weight), d.input, d.m, d.weight.k, d.weight.padded_k, out, residual, stream),
           "decode_mmv.gemv_bf16w");
  return Q4K_OK;
}

// Projection + epilogue of one descriptor whose input is already quantised.  `rows` is m*n floats of scratch.
int decode_one(const q4k_decode_desc& d, const q4k_q8_input& q8, float* rows, cudaStream_t stream) {
  uint64_t const cells = uint64_t(d.m) * d.weight.n;
  switch (d.epilogue) {
    case Q4K_EPILOGUE_STORE_FP32:
      return decode_rows(d, q8, static_cast<float*>(d.output), nullptr, stream);
    case Q4K_EPILOGUE_RESIDUAL_ADD_FP32:
      return decode_rows(d, q8, d.output ? static_cast<float*>(d.output) : const_cast<float*>(d.residual), d.residual, stream);
    case Q4K_EPILOGUE_STORE_BF16: {
      if (int st = decode_rows(d, q8, rows, nullptr, stream)) return st;
      Q4K_CUDA(q4k::launch_store_bf16(rows, static_cast<uint16_t*>(d.output), cells, stream), "decode_mmv.store_bf16");
      return Q4K_OK;
    }
    default:
      return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: unknown epilogue");
  }
}

// One launch for up to three descriptors that share the (already quantised) input: every weight's rows, its bf16 /
// fp32 store or residual add, or -- swiglu -- bf16(SiLU(a) * b) of a gate / up pair, all inside the TMA decode kernel
// (the reference applies these epilogues inside its decode kernels too, cuda/decode_mmv.cu:182-250,619-677).
// *fused = false when the operands do not qualify (more than 16 rows, unaligned weights, another activation policy);
// the caller then composes separate launches.
int decode_fused(const q4k_decode_desc* const* descs, uint32_t count, bool swiglu, const q4k_q8_input& q8, cudaStream_t stream,
                 bool* fused) {
  *fused = false;
  q4k::WeightView ws[3];
  q4k::GemvTmaOutput outs[3] = {};
  Region regions[16];
  int nreg = 0;
  regions[nreg++] = {q8.codes, q8.codes_len, 4, "input.codes"};
  regions[nreg++] = {q8.scales, q8.scales_len * 4, 4, "input.scales"};
  regions[nreg++] = {q8.sums, q8.sums_len * 4, 4, "input.sums"};
  uint64_t n_total = 0, tiles = 0;
  for (uint32_t i = 0; i < count; ++i) {
    const q4k_decode_desc& d = *descs[i];
    if (d.activation_policy != Q4K_ACTIVATION_Q8_K32 || d.m > q4k::kGemvTmaMaxTokens || d.weight.k != descs[0]->weight.k) return Q4K_OK;
    ws[i] = view(d.weight);
    if (!q4k::gemv_tma_supported(ws[i], view(q8))) return Q4K_OK;
    uint64_t const cells = uint64_t(d.m) * d.weight.n;
    regions[nreg++] = {d.weight.codes, d.weight.codes_bytes, 4, "weight.codes"};
    regions[nreg++] = {d.weight.scales, d.weight.scales_bytes, 2, "weight.scales"};
    switch (d.epilogue) {
      case Q4K_EPILOGUE_STORE_FP32:
        outs[i].out = static_cast<float*>(d.output);
        regions[nreg++] = {d.output, cells * 4, 4, "output"};
        break;
      case Q4K_EPILOGUE_STORE_BF16:
        outs[i].out_bf16 = static_cast<uint16_t*>(d.output);
        regions[nreg++] = {d.output, cells * 2, 2, "output"};
        break;
      case Q4K_EPILOGUE_RESIDUAL_ADD_FP32:
        outs[i].residual = d.residual;
        outs[i].out = d.output ? static_cast<float*>(d.output) : const_cast<float*>(d.residual);
        regions[nreg++] = {d.residual, cells * 4, 4, "residual"};
        if (d.output && d.output != d.residual) regions[nreg++] = {d.output, cells * 4, 4, "output"};
        break;
      case Q4K_EPILOGUE_SWIGLU_STORE_BF16:
        if (!swiglu) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: SwiGLU epilogue requires paired gate/up launch");
        if (i == 0) {
          outs[0].out_bf16 = static_cast<uint16_t*>(d.output);
          regions[nreg++] = {d.output, cells * 2, 2, "output"};
        }
        break;
      default:
        return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: unknown epilogue");
    }
    n_total += d.weight.n;
    tiles += (d.weight.padded_n + 15) / 16;
  }
  if (int st = check_distinct(regions, nreg, false)) return st;
  q4k::GemvTmaPlan plan = q4k::plan_gemv_tma_tiles(q8.m, uint32_t(tiles), ws[0].tiles_k, 0, 0, swiglu);
  uint64_t const partial_bytes = plan.split_k > 1 ? uint64_t(plan.split_k) * q8.m * n_total * 4 : 0;
  void* scratch = nullptr;
  if (int st = own_scratch(partial_bytes, &scratch, stream)) return st;
  int* const status = q4k::kernel_status_word();
  if (!status) return Q4K_ERR_STATUS;
  uint8_t* const base = static_cast<uint8_t*>(scratch);
  Q4K_CUDA(q4k::launch_gemv_tma_multi(ws, outs, count, swiglu, view(q8), plan, base + kTicketRegion, reinterpret_cast<uint32_t*>(base),
                                      status, stream),
           "decode_mmv.fused");
  *fused = true;
  return Q4K_OK;
}

int decode_pack(const q4k_decode_desc& d, const DecodeScratch& s, int* failure, cudaStream_t stream) {
  if (d.activation_policy == Q4K_ACTIVATION_BF16) return Q4K_OK;  // that policy multiplies the bf16 input as it is
  if (!failure) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv: null failure flag");
  return pack_impl(d.input, false, d.input_len, s.q8, failure, stream);
}
}  // namespace

uint64_t q4k_decode_workspace_bytes(uint32_t m, uint64_t n_total, uint32_t k) { return decode_scratch_bytes(m, n_total, k); }

int q4k_decode_mmv(const q4k_decode_desc* desc, void* workspace, uint64_t workspace_bytes, int* failure, void* stream_handle) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (int st = valid_decode_desc(desc, false, "desc")) return st;
  DecodeScratch s{};
  if (int st = carve_decode_scratch(workspace, workspace_bytes, desc->m, desc->weight.n, desc->weight.k, &s)) return st;
  if (int st = decode_pack(*desc, s, failure, stream)) return st;
  bool fused = false;
  if (int st = decode_fused(&desc, 1, false, s.q8, stream, &fused)) return st;
  if (fused) return Q4K_OK;
  return decode_one(*desc, s.q8, s.rows, stream);
}

int q4k_decode_mmv_paired(const q4k_decode_desc* a, const q4k_decode_desc* b, void* workspace, uint64_t workspace_bytes,
                          int* failure, void* stream_handle) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (int st = valid_decode_desc(a, true, "paired A")) return st;
  if (!b) return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv_paired: null B descriptor");
  bool const swiglu = a->epilogue == Q4K_EPILOGUE_SWIGLU_STORE_BF16;
  q4k_decode_desc bv = *b;
  if (swiglu) {  // B declares no output of its own (cuda/decode_mmv.cu:514-521)
    if (b->output || b->output_len || b->residual || b->residual_len)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv_paired: SwiGLU paired B must not declare a separately materialized output");
    bv.output = a->output;
    bv.output_len = a->output_len;
  }
  if (int st = valid_decode_desc(&bv, true, "paired B")) return st;
  if (b->weight.layout != a->weight.layout || b->weight.quantizer != a->weight.quantizer || b->weight.n != a->weight.n ||
      b->weight.k != a->weight.k || b->epilogue != a->epilogue || b->input != a->input || b->input_len != a->input_len ||
      b->m != a->m || b->activation_policy != a->activation_policy)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv_paired: paired B must match A shape, layout, input, and epilogue contract");
  DecodeScratch s{};
  if (int st = carve_decode_scratch(workspace, workspace_bytes, a->m, a->weight.n, a->weight.k, &s)) return st;
  if (int st = decode_pack(*a, s, failure, stream)) return st;
  uint64_t const cells = uint64_t(a->m) * a->weight.n;
  {
    const q4k_decode_desc* pair[2] = {a, &bv};
    bool fused = false;
    if (int st = decode_fused(pair, 2, swiglu, s.q8, stream, &fused)) return st;
    if (fused) return Q4K_OK;
  }
  if (!swiglu) {
    if (int st = decode_one(*a, s.q8, s.rows, stream)) return st;
    return decode_one(*b, s.q8, s.rows + cells, stream);
  }
  if (int st = decode_rows(*a, s.q8, s.rows, nullptr, stream)) return st;
  if (int st = decode_rows(bv, s.q8, s.rows + cells, nullptr, stream)) return st;
  Q4K_CUDA(q4k::launch_swiglu_store_bf16(s.rows, s.rows + cells, static_cast<uint16_t*>(a->output), cells, stream),
           "decode_mmv.swiglu");
  return Q4K_OK;
}

// PrefillEngine::project / paired_swiglu (cuda/prefill.hpp:88-96) with the quantise -> MMQ dispatch: the same
// composition as the decode entries without the 16-row limit.
int q4k_prefill_project(const q4k_decode_desc* projection, void* workspace, uint64_t workspace_bytes, int* failure,
                        void* stream_handle) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (int st = valid_decode_desc(projection, false, "projection", Q4K_MAX_TOKENS)) return st;
  DecodeScratch s{};
  if (int st = carve_decode_scratch(workspace, workspace_bytes, projection->m, projection->weight.n, projection->weight.k, &s))
    return st;
  if (int st = decode_pack(*projection, s, failure, stream)) return st;
  return decode_one(*projection, s.q8, s.rows, stream);
}

int q4k_prefill_paired_swiglu(const q4k_weight* gate, const q4k_weight* up, const uint16_t* normalized, uint16_t* swiglu,
                              uint32_t valid_tokens, void* workspace, uint64_t workspace_bytes, int* failure,
                              void* stream_handle) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (!gate || !up) return fail(Q4K_ERR_INVALID_ARGUMENT, "paired_swiglu: null weight");
  q4k_decode_desc a{*gate, normalized, uint64_t(valid_tokens) * gate->k, swiglu, uint64_t(valid_tokens) * gate->n, nullptr, 0,
                    valid_tokens, Q4K_EPILOGUE_SWIGLU_STORE_BF16, Q4K_ACTIVATION_Q8_K32};
  q4k_decode_desc b = a;
  b.weight = *up;
  if (int st = valid_decode_desc(&a, true, "gate", Q4K_MAX_TOKENS)) return st;
  if (int st = valid_decode_desc(&b, true, "up", Q4K_MAX_TOKENS)) return st;
  if (up->n != gate->n || up->k != gate->k || up->layout != gate->layout || up->quantizer != gate->quantizer)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "paired_swiglu: gate and up must have the same shape and layout");
  DecodeScratch s{};
  if (int st = carve_decode_scratch(workspace, workspace_bytes, valid_tokens, gate->n, gate->k, &s)) return st;
  if (int st = decode_pack(a, s, failure, stream)) return st;
  uint64_t const cells = uint64_t(valid_tokens) * gate->n;
  if (int st = project_impl(gate, s.q8, s.rows, cells, nullptr, 0, nullptr, stream)) return st;
  if (int st = project_impl(up, s.q8, s.rows + cells, cells, nullptr, 0, nullptr, stream)) return st;
  Q4K_CUDA(q4k::launch_swiglu_store_bf16(s.rows, s.rows + cells, swiglu, cells, stream), "paired_swiglu.epilogue");
  return Q4K_OK;
}

int q4k_decode_mmv_ranges(const q4k_decode_desc* ranges, uint32_t count, void* workspace, uint64_t workspace_bytes,
                          int* failure, void* stream_handle) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (!ranges || count < 2 || count > 3)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv_ranges: two or three ranges");  // cuda/decode_mmv.cu:790
  uint64_t n_total = 0;
  for (uint32_t i = 0; i < count; ++i) {
    if (int st = valid_decode_desc(&ranges[i], false, "range")) return st;
    if (ranges[i].input != ranges[0].input || ranges[i].input_len != ranges[0].input_len || ranges[i].m != ranges[0].m ||
        ranges[i].weight.k != ranges[0].weight.k || ranges[i].weight.layout != ranges[0].weight.layout ||
        ranges[i].activation_policy != ranges[0].activation_policy)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "decode_mmv_ranges: ranges must share K, input and layout");
    n_total += ranges[i].weight.n;
  }
  DecodeScratch s{};
  if (int st = carve_decode_scratch(workspace, workspace_bytes, ranges[0].m, n_total, ranges[0].weight.k, &s)) return st;
  if (int st = decode_pack(ranges[0], s, failure, stream)) return st;
  {
    const q4k_decode_desc* list[3] = {&ranges[0], &ranges[1], count > 2 ? &ranges[2] : nullptr};
    bool fused = false;
    if (int st = decode_fused(list, count, false, s.q8, stream, &fused)) return st;
    if (fused) return Q4K_OK;
  }
  uint64_t off = 0;
  for (uint32_t i = 0; i < count; ++i) {
    if (int st = decode_one(ranges[i], s.q8, s.rows + off, stream)) return st;
    off += uint64_t(ranges[i].m) * ranges[i].weight.n;
  }
  return Q4K_OK;
}

struct q4k_session {
  int device;
  void* workspace;
  uint64_t workspace_bytes;
  int* failure;
};

int q4k_session_create(uint64_t workspace_bytes, q4k_session** out) {
  if (!out || workspace_bytes == 0) return fail(Q4K_ERR_INVALID_ARGUMENT, "session: workspace_bytes and out must be given");
  *out = nullptr;
  int device = 0;
  Q4K_CUDA(cudaGetDevice(&device), "cudaGetDevice");
  uint64_t const bytes = (workspace_bytes + 255) / 256 * 256;
  void* p = nullptr;
  Q4K_CUDA(cudaMalloc(&p, bytes + 256), "session.alloc");
  cudaError_t st = cudaMemset(static_cast<uint8_t*>(p) + bytes, 0, 256);
  if (st != cudaSuccess) { (void)cudaFree(p); return fail_cuda(st, "session.clear"); }
  *out = new q4k_session{device, p, bytes, reinterpret_cast<int*>(static_cast<uint8_t*>(p) + bytes)};
  return Q4K_OK;
}
void q4k_session_destroy(q4k_session* s) {
  if (!s) return;
  (void)cudaFree(s->workspace);
  delete s;
}
void* q4k_session_workspace(const q4k_session* s) { return s ? s->workspace : nullptr; }
uint64_t q4k_session_workspace_bytes(const q4k_session* s) { return s ? s->workspace_bytes : 0; }
int* q4k_session_failure(const q4k_session* s) { return s ? s->failure : nullptr; }
int q4k_session_take_failure(q4k_session* s, void* stream_handle) {
  if (!s) return fail(Q4K_ERR_INVALID_ARGUMENT, "session: null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  int bad = 0;
  Q4K_CUDA(cudaMemcpyAsync(&bad, s->failure, 4, cudaMemcpyDeviceToHost, stream), "session.failure");
  Q4K_CUDA(cudaStreamSynchronize(stream), "session.sync");
  if (bad) {
    Q4K_CUDA(cudaMemsetAsync(s->failure, 0, 4, stream), "session.clear_failure");
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.producer: nonfinite producer or invalid Q8 scale");
  }
  return Q4K_OK;
}

int q4k_validate_device_span(const void* pointer, uint64_t bytes, uint32_t alignment, int device) {
  return check_span(Region{pointer, bytes, alignment, "span"}, device);
}

int q4k_pack_q8_bf16(const uint16_t* input, uint64_t input_len, q4k_q8_input output, int* failure, void* stream) {
  return pack_impl(input, false, input_len, output, failure, static_cast<cudaStream_t>(stream));
}
int q4k_pack_q8_f32(const float* input, uint64_t input_len, q4k_q8_input output, int* failure, void* stream) {
  return pack_impl(input, true, input_len, output, failure, static_cast<cudaStream_t>(stream));
}

int q4k_export_q8_1(q4k_q8_input x, uint8_t* records, uint64_t records_bytes, void* stream) {
  if (!valid_input(x) || records_bytes != x.scales_len * 36)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.export: invalid geometry");
  Region regions[4] = {{x.codes, x.codes_len, 4, "input.codes"},
                       {x.scales, x.scales_len * 4, 4, "input.scales"},
                       {x.sums, x.sums_len * 4, 4, "input.sums"},
                       {records, records_bytes, 4, "records"}};
  if (int st = check_distinct(regions, 4, false)) return st;
  Q4K_CUDA(q4k::launch_export_q8_1(x.codes, x.scales, x.sums, x.scales_len, records, static_cast<cudaStream_t>(stream)),
           "q8.export");
  return Q4K_OK;
}

int q4k_q8_project(const q4k_weight* weight, q4k_q8_input input, float* output, uint64_t output_len,
                   const float* residual, uint64_t residual_len, void* stream) {
  return project_impl(weight, input, output, output_len, residual, residual_len, nullptr,
                      static_cast<cudaStream_t>(stream));
}
int q4k_q8_project_ex(const q4k_weight* weight, q4k_q8_input input, float* output, uint64_t output_len,
                      const float* residual, uint64_t residual_len, const q4k_project_options* options,
                      void* stream) {
  return project_impl(weight, input, output, output_len, residual, residual_len, options,
                      static_cast<cudaStream_t>(stream));
}

uint64_t q4k_project_workspace_bytes(uint32_t m, uint32_t n, uint32_t split_k) {
  return split_k <= 1 ? 0 : kTicketRegion + uint64_t(split_k) * m * n * 4;
}

int q4k_q8_project_ragged(const q4k_weight* weight, q4k_q8_input input, const uint32_t* row_offsets,
                          uint32_t n_requests, float* output, uint64_t output_len,
                          const q4k_project_options* options, void* stream) {
  if (!row_offsets || n_requests == 0) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.ragged: no requests");
  if (row_offsets[0] != 0) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.ragged: row_offsets[0] must be 0");
  for (uint32_t r = 0; r < n_requests; ++r)
    if (row_offsets[r + 1] <= row_offsets[r])
      return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.ragged: request %u is empty or offsets decrease", r);
  if (row_offsets[n_requests] != input.m)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.ragged: offsets cover %u rows, pack holds %u", row_offsets[n_requests], input.m);
  return project_impl(weight, input, output, output_len, nullptr, 0, options, static_cast<cudaStream_t>(stream));
}

int q4k_repack_blocks144(const uint8_t* blocks, uint64_t blocks_bytes, uint32_t n, uint32_t k, uint8_t* out_codes,
                         uint64_t out_codes_bytes, uint8_t* out_scales, uint64_t out_scales_bytes, void* stream) {
  if (!n || n > Q4K_MAX_N || !k || k > Q4K_MAX_K || k % 256 != 0 || blocks_bytes != uint64_t(n) * (k / 256) * 144 ||
      out_codes_bytes != q4k_code_bytes(uint32_t(q4k_pad_n(n)), k) ||
      out_scales_bytes != q4k_scale_bytes(uint32_t(q4k_pad_n(n)), k))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q4k.repack: invalid geometry");
  Region regions[3] = {{blocks, blocks_bytes, 1, "blocks"},
                       {out_codes, out_codes_bytes, 16, "codes"},
                       {out_scales, out_scales_bytes, 16, "scales"}};
  if (int st = check_distinct(regions, 3, false)) return st;
  Q4K_CUDA(q4k::launch_repack_blocks144(blocks, n, k, out_codes, out_scales, static_cast<cudaStream_t>(stream)),
           "q4k.repack");
  return Q4K_OK;
}

int q4k_validate_weight(const q4k_weight* weight, uint64_t* verdict, void* stream) {
  if (int st = valid_weight(weight, "q4k.validate")) return st;
  Region regions[3] = {{weight->codes, weight->codes_bytes, 16, "codes"},
                       {weight->scales, weight->scales_bytes, 16, "scales"},
                       {verdict, 16, 8, "verdict"}};
  if (int st = check_distinct(regions, 3, false)) return st;
  Q4K_CUDA(q4k::launch_validate_weight(static_cast<const uint8_t*>(weight->codes), static_cast<const uint8_t*>(weight->scales),
                                       weight->n, weight->k, verdict, static_cast<cudaStream_t>(stream)),
           "q4k.validate");
  return Q4K_OK;
}

int q4k_dequantize_bf16(const q4k_weight* weight, uint16_t* output, uint64_t output_len, void* stream) {
  if (int st = valid_weight(weight, "q4k.dequantize")) return st;
  if (weight->k % 256 != 0 || output_len != uint64_t(weight->n) * weight->k)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q4k.dequantize: invalid geometry");
  Region regions[3] = {{weight->codes, weight->codes_bytes, 16, "codes"},
                       {weight->scales, weight->scales_bytes, 16, "scales"},
                       {output, output_len * 2, 16, "output"}};
  if (int st = check_distinct(regions, 3, false)) return st;
  Q4K_CUDA(q4k::launch_dequantize_bf16(static_cast<const uint8_t*>(weight->codes), static_cast<const uint8_t*>(weight->scales),
                                       weight->n, weight->k, output, static_cast<cudaStream_t>(stream)),
           "q4k.dequantize");
  return Q4K_OK;
}

int q4k_unpack_logical(const q4k_weight* weight, int8_t* codes, uint64_t codes_len, uint8_t* metadata, uint64_t metadata_len,
                       void* stream) {
  if (int st = valid_weight(weight, "q4k.unpack")) return st;
  if (weight->k % 256 != 0 || codes_len != uint64_t(weight->n) * weight->k ||
      metadata_len != uint64_t(weight->n) * (weight->k / 256) * 16)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q4k.unpack: invalid geometry");
  Region regions[4] = {{weight->codes, weight->codes_bytes, 16, "codes"},
                       {weight->scales, weight->scales_bytes, 16, "scales"},
                       {codes, codes_len, 16, "logical codes"},
                       {metadata, metadata_len, 16, "logical metadata"}};
  if (int st = check_distinct(regions, 4, false)) return st;
  Q4K_CUDA(q4k::launch_unpack_logical(static_cast<const uint8_t*>(weight->codes), static_cast<const uint8_t*>(weight->scales),
                                      weight->n, weight->k, codes, metadata, static_cast<cudaStream_t>(stream)),
           "q4k.unpack");
  return Q4K_OK;
}

int q4k_fit_blocks(const void* weights, uint32_t weights_dtype, uint64_t blocks, int8_t* codes, uint8_t* metadata,
                   uint8_t* block_status, int* failure, void* stream) {
  if (!blocks || blocks > 0xffffffffull || weights_dtype > Q4K_FIT_BF16 || !failure)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q4k.fit: invalid geometry");
  bool const bf16 = weights_dtype == Q4K_FIT_BF16;
  Region regions[5] = {{weights, blocks * 256 * (bf16 ? 2 : 4), 16, "weights"},
                       {codes, blocks * 256, 16, "codes"},
                       {metadata, blocks * 16, 16, "metadata"},
                       {failure, sizeof(int), 4, "failure"},
                       {block_status, blocks, 1, "block_status"}};
  if (int st = check_distinct(regions, block_status ? 5 : 4, false)) return st;
  Q4K_CUDA(q4k::launch_fit_q4k(weights, bf16, uint32_t(blocks), 1, false, reinterpret_cast<uint8_t*>(codes), metadata,
                               block_status, failure, static_cast<cudaStream_t>(stream)),
           "q4k.fit");
  return Q4K_OK;
}

int q4k_fit_weight(const void* weights, uint32_t weights_dtype, uint32_t n, uint32_t k, uint8_t* out_codes,
                   uint64_t out_codes_bytes, uint8_t* out_scales, uint64_t out_scales_bytes, uint8_t* block_status,
                   int* failure, void* stream) {
  if (!n || n > Q4K_MAX_N || !k || k > Q4K_MAX_K || k % 256 != 0 || weights_dtype > Q4K_FIT_BF16 || !failure ||
      out_codes_bytes != q4k_code_bytes(uint32_t(q4k_pad_n(n)), k) ||
      out_scales_bytes != q4k_scale_bytes(uint32_t(q4k_pad_n(n)), k))
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q4k.fit: invalid geometry");
  bool const bf16 = weights_dtype == Q4K_FIT_BF16;
  uint64_t const blocks = uint64_t(n) * (k / 256);
  Region regions[5] = {{weights, blocks * 256 * (bf16 ? 2 : 4), 16, "weights"},
                       {out_codes, out_codes_bytes, 16, "codes"},
                       {out_scales, out_scales_bytes, 16, "scales"},
                       {failure, sizeof(int), 4, "failure"},
                       {block_status, blocks, 1, "block_status"}};
  if (int st = check_distinct(regions, block_status ? 5 : 4, false)) return st;
  Q4K_CUDA(q4k::launch_fit_q4k(weights, bf16, n, k / 256, true, out_codes, out_scales, block_status, failure,
                               static_cast<cudaStream_t>(stream)),
           "q4k.fit");
  return Q4K_OK;
}

uint64_t q4k_q8_mlp_workspace_bytes(uint32_t m, uint32_t hidden, uint32_t ffn) {
  (void)hidden;  // the hidden-width pack reuses the front of the ffn-width pack
  return uint64_t(m) * (uint64_t(ffn) + uint64_t(ffn) / 32 * 8 + 2ull * ffn * 4) + 4;
}

int q4k_hidden_rms_q8(const float* residual, const uint16_t* gamma, float eps, uint32_t m, uint32_t hidden,
                      q4k_q8_input x, int* failure, void* stream) {
  if (!residual || !gamma || !failure || !m || !hidden || hidden % 256 != 0 || hidden > Q4K_MAX_K ||
      !std::isfinite(eps) || eps <= 0 || !valid_input(x) || x.m != m || x.k != hidden)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.rms: invalid operands");
  Region regions[6] = {{residual, uint64_t(m) * hidden * 4, 4, "residual"}, {gamma, uint64_t(hidden) * 2, 2, "gamma"},
                       {x.codes, x.codes_len, 4, "output.codes"},          {x.scales, x.scales_len * 4, 4, "output.scales"},
                       {x.sums, x.sums_len * 4, 4, "output.sums"},         {failure, 4, 4, "failure"}};
  if (int st = check_distinct(regions, 6, false)) return st;
  Q4K_CUDA(q4k::launch_hidden_rms_q8(residual, gamma, eps, hidden, out_view(x), failure, static_cast<cudaStream_t>(stream)),
           "q8.rms_pack");
  return Q4K_OK;
}

int q4k_swiglu_pack_q8(const float* gate, const float* up, uint32_t m, uint32_t ffn, q4k_q8_input x, int* failure,
                       void* stream) {
  if (!gate || !up || !failure || !m || !ffn || ffn % 256 != 0 || !valid_input(x) || x.m != m || x.k != ffn)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.swiglu_pack: invalid operands");
  Region regions[6] = {{gate, uint64_t(m) * ffn * 4, 16, "gate"},  {up, uint64_t(m) * ffn * 4, 16, "up"},
                       {x.codes, x.codes_len, 4, "output.codes"}, {x.scales, x.scales_len * 4, 4, "output.scales"},
                       {x.sums, x.sums_len * 4, 4, "output.sums"}, {failure, 4, 4, "failure"}};
  if (int st = check_distinct(regions, 6, false)) return st;
  Q4K_CUDA(q4k::launch_swiglu_pack_q8(gate, up, out_view(x), failure, static_cast<cudaStream_t>(stream)), "q8.swiglu_pack");
  return Q4K_OK;
}

int q4k_q8_mlp(const q4k_weight* gate, const q4k_weight* up, const q4k_weight* down, const float* residual,
               const uint16_t* gamma, float eps, float* output, uint32_t m, void* workspace, uint64_t workspace_bytes,
               void* stream_v, int* submitted, int* pending_failure) {
  auto stream = static_cast<cudaStream_t>(stream_v);
  if (!submitted) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.mlp: submitted must not be null");
  *submitted = 0;
  if (!pending_failure) {
    // The synchronous form reads the flag back, which a capturing stream cannot do.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    Q4K_CUDA(cudaStreamIsCapturing(stream, &cap), "q8.mlp.capture_status");
    if (cap != cudaStreamCaptureStatusNone)
      return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.mlp: synchronous form needs an uncaptured stream");
  }
  for (auto const* w : {gate, up, down})
    if (int st = valid_weight(w, "mlp weight")) return st;
  uint32_t const hidden = gate->k, ffn = gate->n;
  if (!m || m > Q4K_MAX_TOKENS || !workspace || workspace_bytes < q4k_q8_mlp_workspace_bytes(m, hidden, ffn) ||
      !std::isfinite(eps) || eps <= 0 || hidden % 256 != 0 || ffn % 256 != 0 || up->n != ffn || up->k != hidden ||
      down->n != hidden || down->k != ffn)
    return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.mlp: invalid geometry");
  Region regions[11] = {{gate->codes, gate->codes_bytes, 4, "gate.codes"},   {gate->scales, gate->scales_bytes, 2, "gate.scales"},
                        {up->codes, up->codes_bytes, 4, "up.codes"},         {up->scales, up->scales_bytes, 2, "up.scales"},
                        {down->codes, down->codes_bytes, 4, "down.codes"},   {down->scales, down->scales_bytes, 2, "down.scales"},
                        {residual, uint64_t(m) * hidden * 4, 4, "residual"}, {gamma, uint64_t(hidden) * 2, 2, "gamma"},
                        {output, uint64_t(m) * hidden * 4, 4, "output"},     {workspace, workspace_bytes, 16, "workspace"},
                        {pending_failure, 4, 4, "pending_failure"}};
  if (int st = check_distinct(regions, pending_failure ? 11 : 10, false)) return st;

  // Workspace carve-up, in the reference's order (cuda/q4k_q8.cu:367-372).
  auto* codes = static_cast<int8_t*>(workspace);
  auto* scales = reinterpret_cast<float*>(codes + uint64_t(m) * ffn);
  auto* sums = reinterpret_cast<int32_t*>(scales + uint64_t(m) * (ffn / 32));
  auto* g = reinterpret_cast<float*>(sums + uint64_t(m) * (ffn / 32));
  auto* u = g + uint64_t(m) * ffn;
  int* failure = pending_failure ? pending_failure : reinterpret_cast<int*>(u + uint64_t(m) * ffn);
  *submitted = 1;
  auto bail = [&](int st) {
    if (!pending_failure) (void)cudaStreamSynchronize(stream);
    return st;
  };
  if (!pending_failure) {
    cudaError_t st = cudaMemsetAsync(failure, 0, 4, stream);
    if (st != cudaSuccess) return bail(fail_cuda(st, "q8.clear_failure"));
  }
  // Up to sixteen tokens with TMA-able gate / up weights whose K fits one block: the gate projection, the up
  // projection and the SwiGLU -> Q8 pack run as ONE launch (three launches for the chain instead of five).  That
  // launch reads the hidden activation while it writes the ffn activation, so the hidden activation moves out of
  // the shared region into the (then unused) fp32 gate rows.
  q4k::GemvTmaPlan fused_plan{};
  q4k::Q8View probe{};
  probe.m = m;
  probe.codes = reinterpret_cast<const int8_t*>(g);
  bool const fused = m <= q4k::kGemvTmaMaxTokens && q4k::gemv_tma_supported(view(*gate), probe) &&
                     q4k::gemv_tma_supported(view(*up), probe) && q4k::plan_gemv_tma_swiglu_q8(m, view(*gate), &fused_plan);
  int8_t* const hcodes = fused ? reinterpret_cast<int8_t*>(g) : codes;
  float* const hscales = fused ? reinterpret_cast<float*>(hcodes + uint64_t(m) * hidden) : scales;
  int32_t* const hsums = fused ? reinterpret_cast<int32_t*>(hscales + uint64_t(m) * (hidden / 32)) : sums;
  q4k_q8_input xh{hcodes, hscales, hsums, uint64_t(m) * hidden, uint64_t(m) * (hidden / 32), uint64_t(m) * (hidden / 32), m, hidden, hidden};
  q4k_q8_input xf{codes, scales, sums, uint64_t(m) * ffn, uint64_t(m) * (ffn / 32), uint64_t(m) * (ffn / 32), m, ffn, ffn};
  q4k_project_options opt{};
  opt.flags = kFlagTrustedSpans;  // every span was validated above
  cudaError_t ce;
  {
    ScopedRange range("qw38:op name=hidden_rms_q8_pack m=%u n=%u k=%u", unsigned(m), unsigned(hidden), 1u);
    ce = q4k::launch_hidden_rms_q8(residual, gamma, eps, hidden, out_view(xh), failure, stream);
  }
  if (ce != cudaSuccess) return bail(fail_cuda(ce, "q8.rms_pack"));
  if (fused) {
    int* status = q4k::kernel_status_word();
    if (!status) return bail(Q4K_ERR_STATUS);
    {
      ScopedRange range("qw38:op name=q4k_project m=%u n=%u k=%u role=%s residual=%u compute=%s", unsigned(m), unsigned(2 * ffn),
                        unsigned(hidden), "gate_up_swiglu_q8", 0u, "q8");
      ce = q4k::launch_gemv_tma_swiglu_q8(view(*gate), view(*up), view(xh), out_view(xf), failure, fused_plan, status, stream);
    }
    if (ce != cudaSuccess) return bail(fail_cuda(ce, "q8.gate_up_swiglu_q8"));
  } else {
  if (int st = project_impl(gate, xh, g, uint64_t(m) * ffn, nullptr, 0, &opt, stream, false, "gate")) return bail(st);
  if (int st = project_impl(up, xh, u, uint64_t(m) * ffn, nullptr, 0, &opt, stream, false, "up")) return bail(st);
  {
    ScopedRange range("qw38:op name=swiglu_q8_pack m=%u n=%u k=%u", unsigned(m), unsigned(ffn), 1u);
    ce = q4k::launch_swiglu_pack_q8(g, u, out_view(xf), failure, stream);
  }
  if (ce != cudaSuccess) return bail(fail_cuda(ce, "q8.swiglu_pack"));
  }
  if (int st = project_impl(down, xf, output, uint64_t(m) * hidden, residual, uint64_t(m) * hidden, &opt, stream, false, "down"))
    return bail(st);
  if (pending_failure) return Q4K_OK;
  int bad = 0;
  ce = cudaMemcpyAsync(&bad, failure, 4, cudaMemcpyDeviceToHost, stream);
  if (ce != cudaSuccess) return bail(fail_cuda(ce, "q8.failure"));
  Q4K_CUDA(cudaStreamSynchronize(stream), "q8.mlp.sync");
  if (bad) return fail(Q4K_ERR_INVALID_ARGUMENT, "q8.producer: nonfinite producer or invalid Q8 scale");
  return Q4K_OK;
}

}  // extern "C"
