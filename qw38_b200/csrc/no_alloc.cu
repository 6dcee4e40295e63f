// q4k_q8_project_static: the split-K projection for callers that must not allocate.
//
// Some hosts of this library cannot let a call reach cudaMalloc: a serving loop that has
// handed every byte of device memory to its own arena, a real-time path where an allocation's
// implicit device synchronisation would stall other streams, or an embedding whose allocator
// hooks forbid foreign allocations.  The ordinary entry points keep their split-K scratch in a
// buffer the library allocates on first use; this one keeps it in a fixed array that is part of
// the loaded module, so nothing is allocated or freed, ever -- at the price of a hard size limit
// and of the array occupying device memory on every GPU that loads the library, until exit.
//
// The array's name is a host-side handle, not a device address.  Its address is looked up once
// per device with cudaGetSymbolAddress (with that device current) and only that pointer is
// handed to the kernel.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/q4k_b200.h"
#include "launch.h"

namespace {

constexpr uint64_t kTicketBytes = 16 * 1024;                       // 4096 tiles
constexpr uint64_t kPartialBytes = Q4K_STATIC_SCRATCH_BYTES;       // fp32 partial tiles
static __device__ __align__(256) unsigned char g_static_scratch[kTicketBytes + kPartialBytes];

std::mutex g_mutex;
unsigned char* g_device_ptr[64] = {};

// Set-up, once per device: resolve the array's device address.  No allocation happens here;
// the module's static storage already exists once the library is loaded on the device.
int scratch_for_current_device(unsigned char** out) {
  int device = 0;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return q4k::set_error_cuda(st, "static.cudaGetDevice");
  if (device < 0 || device >= 64) return q4k::set_error(Q4K_ERR_INVALID_ARGUMENT, "static: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_device_ptr[device]) {
    unsigned char* p = nullptr;
    st = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
    if (st != cudaSuccess) return q4k::set_error_cuda(st, "static.cudaGetSymbolAddress");
    if (!p) return q4k::set_error(Q4K_ERR_STATUS, "static: symbol address is null");
    g_device_ptr[device] = p;
  }
  *out = g_device_ptr[device];
  return Q4K_OK;
}

}  // namespace

extern "C" int q4k_q8_project_static(const q4k_weight* w, q4k_q8_input x, float* output, uint64_t output_len,
                                     const float* residual, uint64_t residual_len, uint32_t split_k, void* stream_v) {
  auto stream = static_cast<cudaStream_t>(stream_v);
  if (!w || !w->codes || !w->scales || !x.codes || !x.scales || !x.sums || !output)
    return q4k::set_error(Q4K_ERR_INVALID_ARGUMENT, "static: null operand");
  if (!w->n || w->n > Q4K_MAX_N || !w->k || w->k > Q4K_MAX_K || w->layout != Q4K_LAYOUT_SPLIT_TILES ||
      w->quantizer != Q4K_QUANTIZER_Q4K || w->padded_n != q4k_pad_n(w->n) || w->padded_k != q4k_pad_k(w->k) ||
      w->codes_bytes != q4k_code_bytes(w->padded_n, w->padded_k) ||
      w->scales_bytes != q4k_scale_bytes(w->padded_n, w->padded_k))
    return q4k::set_error(Q4K_ERR_INVALID_ARGUMENT, "static: Q4_K split-tile geometry required");
  if (!x.m || x.m > Q4K_MAX_TOKENS || x.k != w->k || x.padded_k != w->padded_k ||
      x.codes_len != uint64_t(x.m) * x.padded_k || x.scales_len != x.codes_len / 32 || x.sums_len != x.scales_len ||
      output_len != uint64_t(x.m) * w->n || (residual_len != 0 && (residual_len != output_len || !residual)))
    return q4k::set_error(Q4K_ERR_INVALID_ARGUMENT, "static: invalid geometry");
  // The checks of the allocating entry (no allocation is involved in them): every operand aligned, device
  // memory of the current device, inside one allocation, and the live operands pairwise disjoint -- a host
  // pointer is rejected here instead of faulting on the GPU.
  q4k::Operand operands[7] = {{w->codes, w->codes_bytes, 4, "weight.codes"},
                              {w->scales, w->scales_bytes, 2, "weight.scales"},
                              {x.codes, x.codes_len, 4, "input.codes"},
                              {x.scales, x.scales_len * 4, 4, "input.scales"},
                              {x.sums, x.sums_len * 4, 4, "input.sums"},
                              {output, output_len * 4, 4, "output"},
                              {residual, residual_len * 4, 4, "residual"}};
  if (int st = q4k::check_operands(operands, residual_len ? 7 : 6)) return st;

  q4k::WeightView wv{static_cast<const uint8_t*>(w->codes), static_cast<const uint8_t*>(w->scales), w->n, w->padded_n,
                     w->padded_k / 256};
  q4k::Q8View xv{x.codes, x.scales, x.sums, x.m, x.padded_k};
  q4k::MmaPlan plan = q4k::plan_mma(x.m, w->n, w->padded_k / 256, split_k);
  uint64_t const tiles = uint64_t((w->padded_n / 8 + 7) / 8) * ((x.m + plan.token_tile - 1) / plan.token_tile);
  uint64_t const need = plan.split_k > 1 ? uint64_t(plan.split_k) * x.m * w->n * 4 : 0;
  if (need > kPartialBytes)
    return q4k::set_error(Q4K_ERR_INVALID_ARGUMENT,
                          "static: split_k*m*n*4 = %llu bytes exceeds the built-in scratch of %llu bytes; "
                          "lower split_k or use q4k_q8_project_ex with a workspace",
                          static_cast<unsigned long long>(need), static_cast<unsigned long long>(kPartialBytes));
  if (plan.split_k > 1 && tiles * 4 > kTicketBytes)
    return q4k::set_error(Q4K_ERR_INVALID_ARGUMENT, "static: %llu output tiles exceed the built-in limit of %llu",
                          static_cast<unsigned long long>(tiles), static_cast<unsigned long long>(kTicketBytes / 4));
  unsigned char* scratch = nullptr;
  if (int st = scratch_for_current_device(&scratch)) return st;
  if (plan.split_k > 1) {
    // The array keeps whatever the previous call left; the arrival counters must start at zero.
    cudaError_t st = cudaMemsetAsync(scratch, 0, tiles * 4, stream);
    if (st != cudaSuccess) return q4k::set_error_cuda(st, "static.clear_tickets");
  }
  cudaError_t st = q4k::launch_mmq_mma(wv, xv, output, residual_len ? residual : nullptr, nullptr, plan,
                                       scratch + kTicketBytes, reinterpret_cast<uint32_t*>(scratch), stream);
  if (st != cudaSuccess) return q4k::set_error_cuda(st, "static.mmq_mma");
  return Q4K_OK;
}
