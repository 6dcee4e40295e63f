/*
 * q4k_b200 -- C ABI of the B200 (sm_100a) Q4_K weight x Q8 activation matmul engine.
 *
 * Every entry point takes plain pointers and sizes, enqueues work on the given
 * CUDA stream (a cudaStream_t passed as void*) and returns a status code.  All
 * device pointers are borrowed and must stay alive until the enqueued work has
 * completed.  Unless stated otherwise nothing is allocated and nothing
 * synchronises, so the calls can be recorded into a CUDA graph.
 *
 * Each declaration names the interface of the reference engine (Enucatl/qw38)
 * that it stands behind, as file:line inside that project.
 */
#ifndef Q4K_B200_H_
#define Q4K_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; 1..3 are the reference's ErrorCode values (cuda/error.hpp:13-17). */
#define Q4K_OK 0
#define Q4K_ERR_STATUS 1           /* a CUDA call failed; see q4k_last_cuda_status() */
#define Q4K_ERR_INVALID_ARGUMENT 2 /* rejected before any device work */
#define Q4K_ERR_OVERFLOW 3         /* address or size arithmetic overflow */

/* Wire ids of the one supported weight format (cuda/decode_mmv.hpp:31,41). */
#define Q4K_LAYOUT_SPLIT_TILES 0x020D
#define Q4K_QUANTIZER_Q4K 0x0105

/* Limits.  The reference stops at m<=512, n,k<=17408 (cuda/q4k_q8.cu:286-298);
 * this library lifts them to the benchmark configurations. */
#define Q4K_MAX_TOKENS 16384u
#define Q4K_MAX_N 262144u
#define Q4K_MAX_K 32768u
#define Q4K_DOT_BOUND (32 * 15 * 127) /* cuda/q4k_q8.hpp:23 */
#define Q4K_SUM_BOUND (32 * 127)      /* cuda/q4k_q8.hpp:24 */

/* Q4_K weight matrix in the reference's split-tile device layout
 * (struct PrefillWeight, cuda/prefill.hpp:33-44; layout src/format/pack.cpp:175-222):
 *   codes : padded_n*padded_k/2 bytes, tile row ((row/8)*(padded_k/256)+kb)*8+row%8
 *           holds 128 bytes, byte j = columns 256kb+2j (low nibble), 256kb+2j+1 (high);
 *   scales: 16 bytes per tile row = fp16 d, fp16 dmin, 12 packed 6-bit scale/min bytes.
 * padded_n = ceil8(n), padded_k = ceil256(k); padding holds zero codes and metadata. */
typedef struct q4k_weight {
  const void* codes;
  const void* scales;
  uint16_t layout;    /* Q4K_LAYOUT_SPLIT_TILES */
  uint16_t quantizer; /* Q4K_QUANTIZER_Q4K */
  uint32_t n, k, padded_n, padded_k;
  uint64_t codes_bytes, scales_bytes;
} q4k_weight;

/* Quantised activations (struct Q8Input, cuda/q4k_q8.hpp:14-21): row-major
 * codes[m][padded_k], fp32 scales[m][padded_k/32], exact int32 sums[m][padded_k/32].
 * The *_len fields are element counts, as the spans' size() in the reference. */
typedef struct q4k_q8_input {
  int8_t* codes;
  float* scales;
  int32_t* sums;
  uint64_t codes_len, scales_len, sums_len;
  uint32_t m, k, padded_k;
} q4k_q8_input;

/* Which kernel family q4k_q8_project_ex runs; 0 lets the library choose by m
 * (the reference's switch m==1 | m>=128 | else is cuda/q4k_q8.cu:303-313). */
#define Q4K_KERNEL_AUTO 0
#define Q4K_KERNEL_GEMV_DP4A 1 /* m <= 4 : dp4a, one lane per K32 group */
#define Q4K_KERNEL_MMA 2       /* any m  : warp-level int8 mma, split-K through global scratch */
#define Q4K_KERNEL_TCGEN05 3   /* m >= 32: tcgen05 kind::i8, TMEM accumulators */
#define Q4K_KERNEL_GEMV_MMA 4  /* m <= 16: warp-level int8 mma, split-K inside a block cluster */
#define Q4K_KERNEL_GEMV_TMA 5  /* m <= 16: weights streamed by TMA, activations held in registers */

typedef struct q4k_project_options {
  uint32_t kernel;       /* Q4K_KERNEL_* */
  uint32_t split_k;      /* 0 = choose; otherwise number of K slices (mma kernels; <= 8 for GEMV_MMA) */
  uint32_t row_groups;   /* 0 = choose; row groups (of 8 rows) per block, 4 or 8 (GEMV_MMA);
                          * super-blocks per K slice, <= 20 (GEMV_TMA) */
  int32_t* partials;     /* optional: int32 dots [m][n][padded_k/32], bit-exact check */
  uint64_t partials_len; /* element count of partials, m*n*padded_k/32 when given */
  void* workspace;       /* optional scratch for split-K; NULL = library-owned scratch */
  uint64_t workspace_bytes;
  uint32_t flags;        /* Q4K_FLAG_* */
} q4k_project_options;

/* Skip the per-call device-span checks (pointer attributes, allocation bounds); geometry
 * and overlap checks still run.  For callers that validated the same buffers once. */
#define Q4K_FLAG_TRUSTED_SPANS 1u
/* With launch overlap on (q4k_set_launch_overlap): the activations (codes, scales, sums) and the residual of this
 * call were NOT written by the launch directly before it on the stream -- they were complete before that launch
 * was enqueued.  The tcgen05 kernel (m > 16) then starts on SMs the preceding launch leaves idle and computes
 * while it drains, waiting for it only before its first store; without the flag it prefetches weights and waits
 * before it reads activations.  Every kernel of this library lets its successor start only once its own
 * predecessor has completed, so "not the launch directly before" is all the caller has to know. */
#define Q4K_FLAG_INPUT_SETTLED 2u

const char* q4k_last_error(void);   /* thread-local text of the last failure */
int q4k_last_cuda_status(void);     /* cudaError_t of the last Q4K_ERR_STATUS */
uint32_t q4k_abi_version(void);

/* Decode projection behind launch_decode_mmv / _paired / _ranges (cuda/decode_mmv.hpp:207-215) with a
 * Q8-K32 activation policy (the reference's enum has only Bf16 = 1, cuda/decode_mmv.hpp:43; this is the
 * value a maintainer adds): 1..16 bf16 input rows [m][k] are quantised and multiplied in one call, and one of
 * the reference's four DecodeEpilogue forms (cuda/decode_mmv.hpp:45-51) is applied.  Outputs are [m][n],
 * token-major.  Validation follows cuda/decode_mmv.cu:440-540: a store epilogue must not supply a residual;
 * ResidualAddFp32 reads `residual` and writes `output`, or updates `residual` in place when `output` is NULL;
 * SwigluStoreBf16 needs the paired call, whose B side declares no output and shares A's input.
 * The reference's own Bf16 policy (weights reconstructed in fp32 and rounded to bf16, fp32 FMA with the bf16
 * activations, cuda/decode_mmv.cu:121-250) is accepted on the three decode entries as well. */
#define Q4K_EPILOGUE_STORE_BF16 1
#define Q4K_EPILOGUE_STORE_FP32 2
#define Q4K_EPILOGUE_RESIDUAL_ADD_FP32 3
#define Q4K_EPILOGUE_SWIGLU_STORE_BF16 4 /* paired gate/up only: y = bf16(SiLU(a.x) * b.x) */
#define Q4K_ACTIVATION_BF16 1            /* reference policy: bf16-rounded weights x bf16 activations */
#define Q4K_ACTIVATION_Q8_K32 2          /* Q8 activations, exact int32 K32 dots */

typedef struct q4k_decode_desc {
  q4k_weight weight;      /* DecodeMmvDesc layout/quantizer/n/k/padded_*, codes, scales */
  const uint16_t* input;  /* bf16 [m][k] */
  uint64_t input_len;     /* m * k */
  void* output;           /* bf16 or fp32 [m][n] by epilogue; NULL = in-place residual update */
  uint64_t output_len;    /* m * n elements, 0 when output is NULL */
  const float* residual;  /* fp32 [m][n] for RESIDUAL_ADD_FP32, else NULL */
  uint64_t residual_len;
  uint32_t m;             /* 1..16 (the reference's entry points take one row) */
  uint8_t epilogue;
  uint8_t activation_policy;
} q4k_decode_desc;

/* Scratch for one call: the Q8 pack of the input rows plus fp32 rows for the bf16/SwiGLU epilogues;
 * n_total = rows of all matrices in the call.  256-byte aligned device memory, caller-owned. */
uint64_t q4k_decode_workspace_bytes(uint32_t m, uint64_t n_total, uint32_t k);
int q4k_decode_mmv(const q4k_decode_desc* desc, void* workspace, uint64_t workspace_bytes, int* failure, void* stream);
int q4k_decode_mmv_paired(const q4k_decode_desc* a, const q4k_decode_desc* b, void* workspace,
                          uint64_t workspace_bytes, int* failure, void* stream);
/* Two or three output ranges that share K and input (launch_decode_mmv_ranges): quantised once. */
int q4k_decode_mmv_ranges(const q4k_decode_desc* ranges, uint32_t count, void* workspace,
                          uint64_t workspace_bytes, int* failure, void* stream);

/* PrefillEngine::project and ::paired_swiglu (cuda/prefill.hpp:88-96) for Q4_K weights with the quantise ->
 * MMQ dispatch (a new PrefillDispatch value on the reference side): the descriptor is PrefillProjection
 * (weight, bf16 input [valid_tokens][k], output, residual, valid_tokens = m, epilogue = PrefillEpilogue
 * 1..3, same numbering as DecodeEpilogue); first_position is not needed, the arithmetic is position free.
 * Up to Q4K_MAX_TOKENS rows; workspace as q4k_decode_workspace_bytes(valid_tokens, n, k).
 * PrefillEngine::mlp is q4k_q8_mlp. */
int q4k_prefill_project(const q4k_decode_desc* projection, void* workspace, uint64_t workspace_bytes, int* failure,
                        void* stream);
int q4k_prefill_paired_swiglu(const q4k_weight* gate, const q4k_weight* up, const uint16_t* normalized, uint16_t* swiglu,
                              uint32_t valid_tokens, void* workspace, uint64_t workspace_bytes, int* failure, void* stream);

/* Row-sharded decode with the gather fused into the projection (no counterpart in the reference, which is
 * single-GPU: output rows split over the GPUs of one node, output slices gathered on every GPU).
 * Every rank holds a full [m][total_rows] fp32 output buffer and a zeroed uint32[16] flag array (words 0-7:
 * deliveries per rank; 8-9: this rank's own bookkeeping), both mapped into
 * every other rank's address space (CUDA IPC, VMM or torch symmetric memory; plain peer stores, no
 * multicast).  q4k_q8_project_gather runs this rank's weight shard (rows row_offset ..
 * row_offset + shard->n) and stores each value into ALL ranks' buffers at
 * [token * total_rows + row_offset + row] with plain peer stores, and counts itself as finished.  Finished
 * projections are announced -- flags[g][rank] += count on every rank g -- by the next gather projection or
 * peer wait of the same stream, i.e. once the grid has completed and its stores are visible system-wide
 * (no system-scope fence inside the hot kernel).  `residual`, if given, is [m][total_rows] like the
 * outputs.  m <= 16, shards 16-byte aligned (a multiple of 8 rows always is).
 * q4k_peer_wait enqueues a one-warp kernel that announces what is still unannounced and then waits until
 * every peer's counter in this rank's own flag array has reached this rank's own -- every rank has
 * delivered as many projections as this rank has issued -- which is when the gathered outputs of the step
 * may be read.  `outputs` and `row_offset`/`total_rows` of the descriptor are not used by the wait.  The
 * wait gives up after limit_cycles SM clocks (0 = about two seconds) and then sets the status word of
 * q4k_kernel_status.  q4k_peer_announce does the announcement alone (a rank that has other work to enqueue
 * before it needs the peers' rows).  All ranks must enqueue the same sequence of gather projections.
 * m <= 16 runs the TMA-fed decode kernel, larger m (up to Q4K_MAX_TOKENS) the tcgen05 kernel; both store to the peers.
 *
 * Reuse of a gathered buffer: the protocol proves DELIVERY, not consumption.  When q4k_peer_wait returns on rank A
 * every peer has delivered step t, but a peer may still be reading its copy of the step-t outputs; A's next gather
 * projection into the same buffer would overwrite them.  A buffer may be written again only after every rank has
 * passed one more q4k_peer_wait since it last read the buffer.  In practice: alternate two sets of gathered outputs
 * by step parity (one wait per step then suffices, because a rank that stores step t+2 has passed the wait of
 * step t+1, and a peer's step t+1 projections run after its reads of step t when those are ordered before them
 * in the stream), as bench.py does.
 * A projection whose kernel gave up on a bounded wait (status word nonzero) is not counted as delivered. */
typedef struct q4k_gather_desc {
  float* outputs[8];    /* outputs[g]: rank g's buffer as addressable from this process */
  uint32_t* flags[8];   /* flags[g]: rank g's uint32[16] flag array as addressable from this process; start zeroed */
  uint32_t ranks, rank;
  uint32_t row_offset;  /* first output row of this rank's shard; a multiple of 8 */
  uint32_t total_rows;  /* N of the whole matrix */
  uint32_t options;     /* Q4K_FLAG_INPUT_SETTLED or 0 */
} q4k_gather_desc;
int q4k_q8_project_gather(const q4k_weight* shard, q4k_q8_input x, const q4k_gather_desc* desc,
                          const float* residual, uint64_t residual_len, void* stream);
int q4k_peer_wait(const q4k_gather_desc* desc, uint64_t limit_cycles, void* stream);
int q4k_peer_announce(const q4k_gather_desc* desc, void* stream);

/* Profiler ranges: when enabled for the calling thread (default off, as the reference's profiling::enabled,
 * src/runtime/profiling.hpp:9), q4k_pack_q8_*, q4k_q8_project* and the stages of q4k_q8_mlp run inside NVTX ranges
 * named like the reference's ("qw38:op name=q4k_project m=.. n=.. k=.. role=.. residual=.. compute=integer_dp4a|
 * integer_mma", "qw38:op name=q8_pack ..", "..hidden_rms_q8_pack..", "..swiglu_q8_pack..";
 * cuda/q4k_q8.cu:299-302,326,383, cuda/activation.cu:543), so that traces of the two engines can be compared. */
void q4k_set_profiling_ranges(int enabled);
int q4k_get_profiling_ranges(void);

/* Session: the scratch and the failure flag that the reference's entry points find in their engine or runtime
 * session (cuda/prefill.hpp:72-117 PrefillEngine owns its workspace; src/runtime/session owns the decode
 * workspace), for callers that want the reference's call signatures without a workspace argument.  Allocates
 * workspace_bytes (256-byte aligned) plus one zeroed failure flag on the current device; destroy frees them (after
 * the work that uses them has completed).  q4k_session_take_failure synchronises the stream, returns
 * Q4K_ERR_INVALID_ARGUMENT ("nonfinite producer ...") if a quantiser flagged non-finite data since the last call,
 * and clears the flag. */
typedef struct q4k_session q4k_session;
int q4k_session_create(uint64_t workspace_bytes, q4k_session** out);
void q4k_session_destroy(q4k_session* session);
void* q4k_session_workspace(const q4k_session* session);
uint64_t q4k_session_workspace_bytes(const q4k_session* session);
int* q4k_session_failure(const q4k_session* session);
int q4k_session_take_failure(q4k_session* session, void* stream);

/* Programmatic dependent launch for the decode path (no counterpart in the reference, which
 * replays its decode step as a CUDA graph of fully serialised kernels, src/runtime/language_model.cpp:324-356).
 * When enabled (process-wide, default off), q4k_pack_q8_*, and q4k_q8_project* for m <= 16 launch
 * their kernels so that they may begin while the preceding kernel of the stream is still draining:
 * blocks are placed as SMs free up, and the TMA kernel streams WEIGHT tiles into shared memory
 * before it waits for that kernel.  Activations, residual, output and scratch are touched only
 * after the preceding kernel has completed, so results are unchanged.  The caller's side of the
 * contract: no work still in flight earlier in the stream writes the weight operand (true for
 * decode, where weights are constant; leave it off around q4k_repack_blocks144 or uploads).
 * Works inside CUDA graph capture. */
void q4k_set_launch_overlap(int enabled);
int q4k_get_launch_overlap(void);

/* Synchronises the current device and reads the status word shared by the kernels that wait on
 * device-side barriers (tcgen05, TMA gemv, peer wait): 0 = every launch so far ran to completion;
 * nonzero = a bounded wait gave up at that site (0x5xx TMA gemv, 0x610 peer wait, 0x71x the int8
 * peak measurement, others tcgen05) and the affected block returned without writing its outputs.
 * The word is a static device variable of the library (one per device, no allocation), whatever
 * scratch the launches used.  A nonzero word is cleared by the read, and the arrival counters of the
 * library-owned split-K scratch are zeroed with it (a launch that gave up may have left some behind;
 * a caller that passes its own workspace has them cleared on every call anyway).
 * No counterpart in the reference, whose kernels have no device-side waits. */
int q4k_kernel_status(int* value);

/* Split-K scratch owned by the library (no counterpart in the reference, whose kernels have no split-K).
 * q4k_q8_project, _ex without a workspace, _ragged, _gather and the decode / prefill / MLP entries keep
 * their split-K partial tiles and arrival counters in ONE buffer per device, allocated on first need
 * (8 MiB) and replaced by a larger one when a call needs more.  What that means for the caller:
 *  - It is per device, not per stream.  Two streams that run split-K projections at the same time race
 *    on it; give such calls their own q4k_project_options.workspace, or serialise them.
 *  - A block that was handed out is never freed or moved (launches in flight and captured graphs keep
 *    its address); a replaced block stays allocated until the process ends.
 *  - A call that would have to grow the buffer while its stream is capturing is rejected with
 *    Q4K_ERR_INVALID_ARGUMENT.  q4k_reserve_scratch(bytes, stream) grows it ahead of time: call it once
 *    per device, before capturing, with the largest split_k * m * n * 4 the captured calls will need
 *    (q4k_project_workspace_bytes gives the figure for one call). */
int q4k_reserve_scratch(uint64_t partial_bytes, void* stream);

/* Dense int8 tensor throughput of the current device, measured with the prefill kernel's own
 * instruction (tcgen05.mma kind::i8, M128 x N256 x K32, operands resident in shared memory): every SM
 * issues mmas_per_sm MMAs back to back; *tops = 2*128*256*32 * MMAs / time, time by CUDA events around
 * the launch (returned in *milliseconds when given).  Synchronises the stream.  The reference records
 * its tensor peak as unknown (docs/architecture/cuda-hardware-model.md:57,299); this is the
 * denominator of the prefill roofline. */
int q4k_measure_int8_peak(uint32_t mmas_per_sm, double* tops, double* milliseconds, void* stream);

/* Padding rules (decode_pad_n / decode_pad_k / decode_code_bytes / decode_scale_bytes,
 * cuda/decode_mmv.hpp:148-205, Q4_K branch). */
uint64_t q4k_pad_n(uint32_t n);
uint32_t q4k_pad_k(uint32_t k);
uint64_t q4k_code_bytes(uint32_t padded_n, uint32_t padded_k);
uint64_t q4k_scale_bytes(uint32_t padded_n, uint32_t padded_k);

/* validate_prefill_device_span (cuda/prefill.hpp:28-31, cuda/prefill.cu:329-335):
 * device pointer on `device`, aligned, inside one allocation. */
int q4k_validate_device_span(const void* pointer, uint64_t bytes, uint32_t alignment, int device);

/* pack_q8 (cuda/q4k_q8.hpp:32-34, cuda/q4k_q8.cu:318-330): bf16 [m][k] -> Q8.
 * `failure` is one int in device memory, set to 1 by any K32 group that holds a
 * non-finite value; the owner clears it before and reads it after. */
int q4k_pack_q8_bf16(const uint16_t* input, uint64_t input_len, q4k_q8_input output,
                     int* failure, void* stream);
/* Same producer for fp32 rows (the single-GEMV benchmark configuration feeds fp32;
 * the device routine is the reference's q8_pack_warp, cuda/q8_device.cuh:5-25). */
int q4k_pack_q8_f32(const float* input, uint64_t input_len, q4k_q8_input output,
                    int* failure, void* stream);

/* 36-byte "Q8_1" records {fp16 d, fp16 s, int8 q[32]} from an exact pack:
 * d = fp16_rn(scale), s = fp16_rn(scale * sum).  No counterpart in the reference,
 * whose activations stay in the exact fp32/int32 form (cuda/q4k_q8.hpp:14-21). */
int q4k_export_q8_1(q4k_q8_input input, uint8_t* records, uint64_t records_bytes, void* stream);

/* q4k_q8_project (cuda/q4k_q8.hpp:35-37, cuda/q4k_q8.cu:332-345):
 * out[token*n + row] = sum_g a[token,g]*((d*sc_g)*dot_g - (dmin*m_g)*sum[token,g]) (+ residual).
 * residual may be NULL (residual_len 0).  The first call on a device may allocate the
 * library-owned split-K scratch (see q4k_reserve_scratch): it is shared by all streams of the device,
 * and must be large enough before a graph is captured. */
int q4k_q8_project(const q4k_weight* weight, q4k_q8_input input, float* output,
                   uint64_t output_len, const float* residual, uint64_t residual_len,
                   void* stream);
int q4k_q8_project_ex(const q4k_weight* weight, q4k_q8_input input, float* output,
                      uint64_t output_len, const float* residual, uint64_t residual_len,
                      const q4k_project_options* options, void* stream);
/* Scratch bytes q4k_q8_project_ex needs for (m, n, split_k); 0 when split_k <= 1. */
uint64_t q4k_project_workspace_bytes(uint32_t m, uint32_t n, uint32_t split_k);

/* The same projection for callers that must never allocate device memory -- a serving process
 * whose own arena owns the whole GPU, a latency-critical stream that cannot afford the implicit
 * synchronisation of an allocation, a host with allocator hooks that reject foreign requests.
 * It runs the split-K warp-MMA kernel (Q4K_KERNEL_MMA) with its scratch in a fixed array inside
 * the library image instead of a lazily allocated buffer: no cudaMalloc, no cudaFree, no
 * allocating library routine, on any call.  Limits: split_k * m * n * 4 <= Q4K_STATIC_SCRATCH_BYTES
 * and at most 4096 output tiles when split_k > 1; larger requests are rejected with
 * Q4K_ERR_INVALID_ARGUMENT and a message naming the limit.  The array costs that much device
 * memory (plus 16 KiB) on every GPU that loads the library, until the process exits.
 * The first call on a device looks up the array's device address; make that call before any
 * stream capture on that device.  All calls on a device share the one array, which keeps the
 * previous call's contents: the arrival counters are cleared at the start of each call, and
 * two calls whose kernels overlap on the GPU (different streams) race on it -- serialise them.
 * This entry point has no counterpart in the reference. */
#define Q4K_STATIC_SCRATCH_BYTES (8ull * 1024 * 1024)
int q4k_q8_project_static(const q4k_weight* weight, q4k_q8_input input, float* output,
                          uint64_t output_len, const float* residual, uint64_t residual_len,
                          uint32_t split_k, void* stream);

/* Ragged continuous batch: requests r = 0..n_requests-1 own the packed token rows
 * [row_offsets[r], row_offsets[r+1]) of one Q8 pack with m = row_offsets[n_requests].
 * The projection is row independent and position free (cuda/prefill.hpp:58-60), so
 * this is q4k_q8_project over the packed rows; row_offsets (host memory) is validated
 * (monotone, covering m) and each request's rows equal the same rows run alone.
 * The reference is single-sequence and has no such entry (its closest statement is
 * the token<m masking of cuda/q4k_q8.cu:137-141). */
int q4k_q8_project_ragged(const q4k_weight* weight, q4k_q8_input input,
                          const uint32_t* row_offsets, uint32_t n_requests, float* output,
                          uint64_t output_len, const q4k_project_options* options, void* stream);

/* 144-byte llama.cpp-native super-blocks [n][k/256] (k % 256 == 0, device memory)
 * -> split tiles, padded rows zeroed.  Resident prepare-once step; the reference
 * does the same permutation on the host (src/format/pack.cpp:175-222 fed by
 * third_party/llama.cpp-q4k/reference.hpp:244-248 element order). */
int q4k_repack_blocks144(const uint8_t* blocks, uint64_t blocks_bytes, uint32_t n, uint32_t k,
                         uint8_t* out_codes, uint64_t out_codes_bytes, uint8_t* out_scales,
                         uint64_t out_scales_bytes, void* stream);

/* format::validate_cuda_v0 for this layout (src/format/unpack.cpp:89-226) on a RESIDENT weight: rows
 * n..padded_n-1 hold zero codes and zero metadata, every live super-block's fp16 d and dmin are
 * non-negative and finite.  (Q4_K has no forbidden code value; k is a multiple of 256, so there are
 * no padded columns.)  verdict: two 64-bit words in device memory, written on `stream`:
 * verdict[0] = Q4K_VALID, or which rule the first offence in the reference's scan order breaks;
 * verdict[1] = its byte offset inside the codes span (Q4K_INVALID_CODES_PADDING) or the scales span
 * (the other two) -- the `offset` the reference's FormatError carries when the spans' file offsets
 * are given as zero. */
#define Q4K_VALID 0
#define Q4K_INVALID_CODES_PADDING 1  /* "Q4 padded coordinates must encode zero" */
#define Q4K_INVALID_SCALES_PADDING 2 /* "padded Q4_K metadata must be zero" */
#define Q4K_INVALID_SCALE 3          /* "Q4_K superblock scales must be nonnegative finite FP16" */
int q4k_validate_weight(const q4k_weight* weight, uint64_t* verdict, void* stream);

/* compiler::dequantize_to_bf16 (src/compiler/quantization/reference.cpp:141-166) from the resident
 * split-tile weight: output bf16 bits [n][k] row-major (k % 256 == 0, output_len = n*k), each value
 * bf16_rne((d*sc)*q - dmin*mn) with separately rounded fp32 operations -- the operand the reference's
 * BF16 unpack -> cuBLAS prefill path multiplies with (cuda/prefill.cu:329-335), and the weights its
 * reference GEMV sees. */
int q4k_dequantize_bf16(const q4k_weight* weight, uint16_t* output, uint64_t output_len, void* stream);

/* format::unpack_cuda_v0 (src/format/unpack.cpp:262-380) from the resident weight: levels int8 [n][k]
 * (0..15, codes_len = n*k) and the 16 metadata bytes of every super-block [n][k/256][16]
 * (metadata_len = n*(k/256)*16); k % 256 == 0.  The inverse of the pack inside q4k_fit_weight. */
int q4k_unpack_logical(const q4k_weight* weight, int8_t* codes, uint64_t codes_len, uint8_t* metadata,
                       uint64_t metadata_len, void* stream);

/* Q4_K fitter on the device: compiler::quantize_q4k_block (src/compiler/quantization/q4k.cpp:186-278)
 * over every 256 consecutive weights, bit for bit (codes and the 16 metadata bytes).  The reference
 * runs it on the host, one block after another (quantize_fp32, src/compiler/quantization/quantizer.cpp:173-182).
 * weights: device memory, fp32 (Q4K_FIT_FP32) or bf16 bits (Q4K_FIT_BF16; widened exactly, as the
 * reference's compiler does before fitting).  block_status (optional, device, one byte per block)
 * receives the reason a block was refused -- the reference's error for the first refused block in
 * index order is the status of the lowest such index; *failure (device int) is set to 1 if any
 * block was refused, and a refused block is written as zeros.  Asynchronous on `stream`. */
#define Q4K_FIT_FP32 0u
#define Q4K_FIT_BF16 1u
#define Q4K_FIT_OK 0          /* fitted */
#define Q4K_FIT_NONFINITE 1   /* "Q4_K input is nonfinite" */
#define Q4K_FIT_RANGE 2       /* "Q4_K fitting range exceeded" (|w| > 1e10) */
#define Q4K_FIT_RECIPROCAL 3  /* "Q4_K fitting reciprocal overflow" */
#define Q4K_FIT_COMPRESS 4    /* "Q4_K compression reciprocal overflow" */
#define Q4K_FIT_HALF 5        /* "Q4_K FP16 scale overflow" */
/* Logical form: codes int8 [blocks][256] (levels 0..15), metadata [blocks][16]. */
int q4k_fit_blocks(const void* weights, uint32_t weights_dtype, uint64_t blocks, int8_t* codes,
                   uint8_t* metadata, uint8_t* block_status, int* failure, void* stream);
/* Row-major weights [n][k] (k % 256 == 0) straight to the split-tile layout: the fitter and
 * format::pack_cuda_v0 (src/format/pack.cpp:175-222) in one pass; block b = row * (k/256) + kb. */
int q4k_fit_weight(const void* weights, uint32_t weights_dtype, uint32_t n, uint32_t k,
                   uint8_t* out_codes, uint64_t out_codes_bytes, uint8_t* out_scales,
                   uint64_t out_scales_bytes, uint8_t* block_status, int* failure, void* stream);

/* q8_mlp_workspace_bytes (cuda/q4k_q8.hpp:28-30), generalised from 17408/5120 to (ffn, hidden). */
uint64_t q4k_q8_mlp_workspace_bytes(uint32_t m, uint32_t hidden, uint32_t ffn);

/* q4k_q8_mlp (cuda/q4k_q8.hpp:44-49, cuda/q4k_q8.cu:347-398): RMS norm + Q8 pack ->
 * gate -> up -> SwiGLU + Q8 pack -> down + residual, one sticky failure flag.
 * With pending_failure == NULL the call clears, reads back and checks the flag
 * (synchronising the stream) and returns Q4K_ERR_INVALID_ARGUMENT for a non-finite
 * producer; otherwise it only enqueues.  *submitted is 0 for a pre-launch rejection
 * and 1 once device work was attempted. */
int q4k_q8_mlp(const q4k_weight* gate, const q4k_weight* up, const q4k_weight* down,
               const float* residual, const uint16_t* gamma, float eps, float* output,
               uint32_t m, void* workspace, uint64_t workspace_bytes, void* stream,
               int* submitted, int* pending_failure);

/* launch_hidden_rms_q8 (cuda/activation.cu:536-548, kernel :134-190). */
int q4k_hidden_rms_q8(const float* residual, const uint16_t* gamma, float eps, uint32_t m,
                      uint32_t hidden, q4k_q8_input output, int* failure, void* stream);
/* swiglu_pack_kernel (cuda/q4k_q8.cu:52-61). */
int q4k_swiglu_pack_q8(const float* gate, const float* up, uint32_t m, uint32_t ffn,
                       q4k_q8_input output, int* failure, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q4K_B200_H_ */
