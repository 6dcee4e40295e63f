// Internal launch interface between the C-ABI layer (abi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace q4k {

struct Q8Out {
  int8_t* codes;
  float* scales;
  int32_t* sums;
  uint32_t m, padded_k;
};

// q8_quantize.cu
cudaError_t launch_pack_q8(const void* input, bool fp32, Q8Out out, uint32_t k, int* failure,
                           cudaStream_t stream);
cudaError_t launch_swiglu_pack_q8(const float* gate, const float* up, Q8Out out, int* failure,
                                  cudaStream_t stream);
cudaError_t launch_hidden_rms_q8(const float* residual, const uint16_t* gamma, float eps,
                                 uint32_t hidden, Q8Out out, int* failure, cudaStream_t stream);
cudaError_t launch_export_q8_1(const int8_t* codes, const float* scales, const int32_t* sums,
                               uint64_t groups, uint8_t* records, cudaStream_t stream);

// gemv_dp4a.cu : m <= 4.  partials (optional) receives the int32 K32 dots [m][n][G].
cudaError_t launch_gemv_dp4a(const WeightView& w, const Q8View& x, float* out,
                             const float* residual, int32_t* partials, cudaStream_t stream);
constexpr uint32_t kGemvDp4aMaxTokens = 4;

// mmq_mma.cu : any m.  split_k slices of K are reduced in slice order by the last
// block of each tile through `scratch` (fp32 partial tiles followed by tickets).
struct MmaPlan {
  uint32_t token_tile;   // tokens per block: 16, 32 or 64
  uint32_t split_k;      // >= 1
  uint32_t kbs_per_step; // super-blocks staged per shared-memory step
};
MmaPlan plan_mma(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request);
// partial_tiles: split_k * m * n floats; tickets: one zeroed uint32 per (row tile, token tile),
// left zero by the kernel.  Both may be null when plan.split_k == 1.
cudaError_t launch_mmq_mma(const WeightView& w, const Q8View& x, float* out, const float* residual,
                           int32_t* partials, const MmaPlan& plan, void* partial_tiles,
                           uint32_t* tickets, cudaStream_t stream);

// gemv_mma.cu : m <= 16.  K slices are the blocks of a thread-block cluster (<= 8) and are
// added in rank order through distributed shared memory; no global scratch.
struct GemvMmaPlan {
  uint32_t warps;    // row groups per block: 4 or 8
  uint32_t split_k;  // cluster size, 1..8
};
GemvMmaPlan plan_gemv_mma(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request,
                          uint32_t warps_request);
cudaError_t launch_gemv_mma(const WeightView& w, const Q8View& x, float* out, const float* residual,
                            int32_t* partials, const GemvMmaPlan& plan, cudaStream_t stream);

// mmq_tcgen05.cu : tcgen05 kind::i8 with TMEM accumulators, 128 rows x {16,32,64,128} tokens
// per block.  status receives a nonzero site code if a bounded wait inside the kernel gave up.
struct TcPlan {
  uint32_t ntok;
  uint32_t split_k;
};
// Where the rows go: element (token, row) lands at token * stride + row0 + row of every fp32 destination
// (one buffer, or each rank's copy of a gathered output, written with plain peer stores), or of the one
// bf16 destination (round to nearest even).  residual, if set, has the destination's geometry and is
// added last.  stride 0 = the weight's own n.
// Row-sharded use (flags / done / unsignalled as in GemvTmaGather below): done != nullptr makes the launch count
// itself as a finished projection of `rank`.
struct TcOutput {
  float* out[8];
  uint16_t* out_bf16;
  const float* residual;
  uint32_t ndst, stride, row0;
  uint32_t* flags[8];
  uint32_t* done;
  uint32_t* unsignalled;
  uint32_t rank;
  uint32_t input_settled;  // Q4K_FLAG_INPUT_SETTLED: activations and residual do not come from the launch directly before
};
inline TcOutput tc_output(float* out, const float* residual) {
  TcOutput o{};
  o.out[0] = out; o.residual = residual; o.ndst = 1;
  return o;
}
bool tcgen05_supported(const WeightView& w, const Q8View& x);
TcPlan plan_tcgen05(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request);
cudaError_t launch_mmq_tcgen05(const WeightView& w, const Q8View& x, const TcOutput& out, int32_t* partials,
                               const TcPlan& plan, void* partial_tiles, uint32_t* tickets, int* status, cudaStream_t stream);

// gemv_tma.cu : m <= 16.  Weights streamed by TMA into a shared-memory ring, activations held in
// registers by warps that each own one super-block column of the block's K slice; K slices of
// different blocks are added in slice order through `slices` ([split_k][m][n] floats) by the last
// block of a row range (`tickets`: one zeroed uint32 per range, left zero).
constexpr uint32_t kGemvTmaMaxTokens = 16;
constexpr uint32_t kGemvTmaMaxWarpsNarrow = 20;  // m <= 8
constexpr uint32_t kGemvTmaMaxWarpsWide = 20;    // m <= 16
struct GemvTmaPlan {
  uint32_t warps;    // consumer warps = super-blocks per K slice
  uint32_t split_k;  // K slices
  uint32_t ranges, tiles_per_range;  // row ranges (blocks per slice) and 16-row tiles per range
  uint32_t stages;   // depth of the weight ring
  uint32_t red_slots;  // hand-off buffers between consumers and reducer: 1 or 2
  uint32_t input_settled = 0;  // Q4K_FLAG_INPUT_SETTLED: the consumer warps load activations without waiting for the preceding launch
};
bool gemv_tma_supported(const WeightView& w, const Q8View& x);
GemvTmaPlan plan_gemv_tma(uint32_t m, uint32_t n, uint32_t tiles_k, uint32_t split_k_request, uint32_t warps_request);
// Row-sharded use: every value is stored into each rank's copy of the gathered [m][total_rows] output
// (peer pointers mapped into this process) and, when the whole grid has finished, this rank's
// counter is bumped in every rank's flag array.  `done` is a zeroed uint32 the launch returns to zero.
struct GemvTmaGather {
  float* outputs[8];
  uint32_t* flags[8];
  uint32_t* done;         // zeroed uint32 the launch returns to zero
  uint32_t* unsignalled;  // finished-but-unannounced projections of this rank (shared with peer wait)
  uint32_t ranks, rank, row_offset, total_rows;
};
GemvTmaPlan plan_gemv_tma_tiles(uint32_t m, uint32_t row_tiles, uint32_t tiles_k, uint32_t split_k_request, uint32_t warps_request,
                                bool pair);
// One launch over up to three weights that share x (and K), each with its own destination and epilogue: fp32 or bf16
// (round to nearest even) store, optional fp32 residual of the destination's shape added last.  swiglu_pair: exactly
// two weights of equal shape, gate and up; their 16-row tiles alternate through the blocks and the single result
// bf16(SiLU(gate) * up) goes to outs[0].out_bf16.  Plan from plan_gemv_tma_tiles over the tiles of all weights
// (16-row tiles of each padded_n; split-K scratch rows = sum of n).
struct GemvTmaOutput {
  float* out;
  uint16_t* out_bf16;
  const float* residual;
};
cudaError_t launch_gemv_tma_multi(const WeightView* ws, const GemvTmaOutput* outs, uint32_t count, bool swiglu_pair, const Q8View& x,
                                  const GemvTmaPlan& plan, void* slices, uint32_t* tickets, int* status, cudaStream_t stream);
// The gate / up pair of an MLP in one launch whose reducer writes the Q8 activation of the down projection directly
// (codes, scales, sums of bf16(silu(gate) * up), non-finite values raise `failure`): the reference's gate, up and
// swiglu_pack launches in one.  The plan function says whether the shape qualifies (whole K in one block, rows a
// multiple of 32).
bool plan_gemv_tma_swiglu_q8(uint32_t m, const WeightView& gate, GemvTmaPlan* plan);
cudaError_t launch_gemv_tma_swiglu_q8(const WeightView& gate, const WeightView& up, const Q8View& x, Q8Out out, int* failure,
                                      const GemvTmaPlan& plan, int* status, cudaStream_t stream);
cudaError_t launch_gemv_tma(const WeightView& w, const Q8View& x, float* out, const float* residual, int32_t* partials,
                            const GemvTmaPlan& plan, void* slices, uint32_t* tickets, int* status, cudaStream_t stream,
                            const GemvTmaGather* gather = nullptr);

// peer.cu : announces this rank's finished projections to every rank, then waits (bounded) until every
// rank's counter in this rank's own flag array has reached this rank's own; a wait that gives up
// writes 0x610 to *status.  limit_cycles < 0 announces only.
cudaError_t launch_peer_wait(uint32_t* const* flags, uint32_t* unsignalled, uint32_t ranks, uint32_t rank,
                             long long limit_cycles, int* status, cudaStream_t stream);

// decode_entry.cu : bf16 store and SwiGLU epilogues over fp32 projection rows.
cudaError_t launch_store_bf16(const float* in, uint16_t* out, uint64_t count, cudaStream_t stream);
cudaError_t launch_swiglu_store_bf16(const float* gate, const float* up, uint16_t* out, uint64_t count, cudaStream_t stream);

// gemv_bf16w.cu : the reference's Bf16 activation policy (bf16-rounded weights x bf16 activations, fp32 FMA).
cudaError_t launch_gemv_bf16w(const WeightView& w, const uint16_t* x, uint32_t m, uint32_t k, uint32_t padded_k, float* out,
                              const float* residual, cudaStream_t stream);

// abi.cu : process-wide switch set by q4k_set_launch_overlap().  When on, the decode kernels
// (pack, dp4a, TMA gemv) are launched with programmatic stream serialization: they may start,
// and the TMA kernel may prefetch weights, while the preceding kernel of the stream drains.
bool launch_overlap();

// Launch with or without the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          bool overlap, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// abi.cu : records the thread-local error text behind q4k_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...);
int set_error_cuda(cudaError_t status, const char* operation);
// abi.cu : device address of the current device's kernel status word (a __device__ int of the library, resolved once
// per device with cudaGetSymbolAddress; nothing is allocated).  nullptr + thread-local error text on failure.
int* kernel_status_word();
// abi.cu : the host-side operand checks of the projection entries for entry points in other files: every span non-empty,
// aligned, device memory of the current device inside one allocation, and pairwise disjoint.
struct Operand {
  const void* p;
  uint64_t bytes;
  uint32_t alignment;
  const char* name;
};
int check_operands(const Operand* operands, int count);

// fit_q4k.cu: weights [rows][tiles_k*256] (fp32, or bf16 bits) -> Q4_K.  split = false writes int8 codes
// [blocks][256] + metadata [blocks][16]; split = true writes the split-tile layout for ceil8(rows) rows.
cudaError_t launch_fit_q4k(const void* weights, bool bf16, uint32_t rows, uint32_t tiles_k, bool split, uint8_t* codes,
                           uint8_t* meta, uint8_t* status, int* failure, cudaStream_t stream);

// repack.cu
// int8 levels [n][k] and metadata [n][k/256][16] from split tiles (k % 256 == 0).
cudaError_t launch_unpack_logical(const uint8_t* codes, const uint8_t* meta, uint32_t n, uint32_t k, int8_t* out_codes,
                                  uint8_t* out_meta, cudaStream_t stream);
// bf16 weights [n][k] (k % 256 == 0) from split tiles: bf16_rne((d*sc)*q - dmin*mn), each operation rounded.
cudaError_t launch_dequantize_bf16(const uint8_t* codes, const uint8_t* meta, uint32_t n, uint32_t k, uint16_t* out,
                                   cudaStream_t stream);
// verdict (device, two 64-bit words): {0, 0} admissible; else {1 padded code byte | 2 padded metadata byte |
// 3 super-block scale, byte offset of the first offence within the codes (kind 1) or scales span}.
cudaError_t launch_validate_weight(const uint8_t* codes, const uint8_t* meta, uint32_t n, uint32_t k, uint64_t* verdict,
                                   cudaStream_t stream);
cudaError_t launch_repack_blocks144(const uint8_t* blocks, uint32_t n, uint32_t k, uint8_t* codes,
                                    uint8_t* meta, cudaStream_t stream);

}  // namespace q4k
