/*
 * C ABI of the blockwise-int4 weight-only GEMM library, B200 (sm_100a) build.
 *
 * The first three entry points are the drop-in boundary: they keep the names,
 * argument order, argument meaning, return convention and data-layout contract
 * of the reference library's public header (reference include/ms_blkq4gemm.h:
 * blkq4_fp16_gemm_sm80 :41-50, blkq4_fp16_quant_sm80 :71-80,
 * blkq4_fp16_quant_size_sm80 :94-100), so a caller linked against the reference
 * links against this library unchanged.  The `_sm80` suffix is kept for that
 * reason only; the kernels behind it are written for sm_100a and there is no
 * other code path (no CPU fallback: without a usable device the calls fail).
 *
 * Like the reference header this file includes nothing: have <cstdint> and
 * <cstddef> included first.  The signatures use `bool` and a reference
 * parameter, so the header is C++.
 *
 * Conventions shared by all entry points
 *   - return 0 on success, -1 on error.  `error_message` is a `std::string*`
 *     passed as `void*` (may be null); it is written only on error.
 *   - every `*_ptr` is a device pointer owned by the caller, on the current
 *     device.  `stream` is a `cudaStream_t` passed as `void*` (null = default
 *     stream).  Work is enqueued on `stream`; the calls do not synchronise and
 *     allocate no device memory.
 *   - every `*_size` argument is a size in BYTES.
 *
 * Layout contract (identical to the reference)
 *   weights       fp16, K x N column-major with leading dimension >= K; this is
 *                 a PyTorch Linear.weight [out_features, in_features] as is.
 *   block         16, 32 or 64 (128 is accepted as an extension).  Column-wise
 *                 blocking: `block` consecutive k of one column share a scale.
 *                 Row-wise: `block` consecutive n of one row share a scale.
 *   quant weights K * N / 2 bytes, column-major [K, N/2].  Byte (kp, np) holds
 *                 q[k, n] in the low and q[k + 8, n] in the high nibble, with
 *                 n = 16*(np/8) + np%8 + 8*(kp%4 & 1) and
 *                 k = 16*(kp/16) + 2*((kp%16)/4) + (kp%4 >> 1).
 *   scales        fp16, (K/bk) * (N/bn) entries.  Column-wise: row-major
 *                 [K/block, N].  Row-wise: column-major [K, N/block] with every
 *                 16 rows permuted to 0 1 8 9 2 3 10 11 4 5 12 13 6 7 14 15.
 *   zero points   one 4-bit value per uint8_t, same shape as scales.  Row-wise:
 *                 every 16 rows permuted to 0 8 1 9 2 10 3 11 4 12 5 13 6 14 7 15.
 *                 A null pointer or zero size means symmetric quantization
 *                 (zero point 8; the scale may then be negative).
 *   activations   fp16 row-major [M, K];  output fp16 row-major [M, N].
 */

#pragma once

extern "C" {

/**
 * output[M,N] = act[M,K] x dequantize(weights[K,N]), fp32 accumulation, fp16 out.
 * Replaces reference include/ms_blkq4gemm.h:41-50 (src/blkq4_f16_gemm_sm80.cu:319-429).
 *
 * Sizes must match exactly: a_size = 2*M*K, weights_size = K*N/2,
 * scales_size = 2*meta, offsets_size = meta (or 0), output_size = 2*M*N, with
 * meta = (K/bk)*(N/bn).  Requires M, N, K > 0, K % 64 == 0, N % 16 == 0 and
 * whole quantization blocks.  M <= 16 takes the memory-bound skinny kernel,
 * larger M the tensor-core kernel.
 */
int blkq4_fp16_gemm_sm80(
  int block_size,
  bool column_wise_blocking,
  int m, int n, int k, void* stream,
  void const* act_ptr, size_t a_size,
  void const* weights_ptr, size_t weights_size,
  void const* scales_ptr, size_t scales_size,
  void const* offsets_ptr, size_t offsets_size,
  void* output_ptr, size_t output_size,
  void* error_message);

/**
 * Quantize an fp16 weight matrix blockwise to 4 bits and write it, its scales and
 * (optionally) its zero points in the prepacked layout the GEMM consumes.
 * Replaces reference include/ms_blkq4gemm.h:71-80 (src/blkq4_f16_gemm_sm80.cu:465-531).
 *
 * rows = K (input features), columns = N (output features).  Buffer sizes may
 * exceed what is needed (>=), as in the reference.  One fused kernel; unlike the
 * reference no temporary device buffers are allocated.
 */
extern int blkq4_fp16_quant_sm80(
    int block_size,
    bool column_wise_blocking,
    int rows, int columns, int leadingDimension,
    void* stream,
    void const* weights, size_t weights_size,
    void* quant_weights, size_t quant_weights_size,
    void* quant_scales, size_t quant_scales_size,
    void* offsets, size_t offsets_size,
    void* error_message);

/**
 * Element counts of the quantized tensors: quant_weights_size in uint8_t,
 * quant_meta_size in meta entries (fp16 scales, uint8_t zero points).
 * Replaces reference include/ms_blkq4gemm.h:94-100 (src/blkq4_f16_gemm_sm80.cu:431-463).
 * Host only.  Rejects rows % 64 != 0, columns % 32 != 0, empty shapes,
 * unsupported block sizes, and shapes whose last quantization block would be
 * partial (the reference lets some of those through and then writes out of
 * bounds; see the note in src of this library).
 */
int blkq4_fp16_quant_size_sm80(
    int block_size,
    bool column_wise_blocking,
    int rows, int columns,
    int64_t& quant_weights_size,
    int64_t& quant_meta_size,
    void* error_message);

/**
 * blkq4_fp16_gemm_sm80 with an optional bias and a `flags` word; without bias and with flags = 0
 * it is exactly that call.  No counterpart in the reference (the signature is reference
 * include/ms_blkq4gemm.h:41-50 plus the three arguments; the bias replaces the separate
 * `output += bias` of the reference module, python/ms_blkq4linear.py:26-27).
 *
 * bias_ptr: fp16 [N] (bias_size = 2*N bytes, 4-byte aligned), or null / size 0.  It is added in
 * fp16 to the result already rounded to fp16, so the output is bit-identical to running the GEMM
 * and then adding the bias to the fp16 output tensor, without the extra pass over [M, N].
 *
 * BLKQ4_GEMM_EARLY_WEIGHT_FETCH: the caller vouches that weights, scales and offsets are not
 * written by any work still pending on `stream` (inference weights, quantized once).  The
 * kernel is then launched with programmatic stream serialization: it may become resident and
 * fetch weights while the preceding kernel of the stream still runs, which keeps HBM busy
 * across the launches of a decode stack.  Activations are read, and the output written, only
 * after the preceding work has completed, so stream order holds for both (and for the split-K
 * workspace).  Both the skinny and the tensor-core kernel honour it.
 */
#define BLKQ4_GEMM_EARLY_WEIGHT_FETCH 1u
int blkq4_fp16_gemm_sm100(
  int block_size,
  bool column_wise_blocking,
  int m, int n, int k, void* stream,
  void const* act_ptr, size_t a_size,
  void const* weights_ptr, size_t weights_size,
  void const* scales_ptr, size_t scales_size,
  void const* offsets_ptr, size_t offsets_size,
  void* output_ptr, size_t output_size,
  void const* bias_ptr, size_t bias_size,
  unsigned flags,
  void* error_message);

/**
 * blkq4_fp16_gemm_sm100 with a caller-owned workspace: device memory of at least
 * blkq4_gemm_workspace_size(m, n, k) bytes, 256-byte aligned, ZERO-INITIALISED once (the kernel
 * leaves it zeroed), used by one call at a time (calls on one stream may share it).  With it the
 * tensor-core kernel splits K when the output has too few 128 x 256 tiles to fill the GPU's SMs
 * (e.g. M = 512, N = 4096: 64 tiles on 148 SMs): parts of a tile's K range run on different SMs,
 * leave fp32 partial tiles in the workspace and the last part adds them in a fixed order.  With
 * more tiles than SMs (or than pairs of SMs, for m >= 256) but far from a whole number of rounds
 * (e.g. 224 tiles on 148 SMs) it cuts the tiles' k steps in one balanced range per SM (or pair)
 * instead, and a tile that straddles two ranges is finished through an fp32 partial tile in the same
 * way.  Results are reproducible run to run with the same workspace size.  A null or too small
 * workspace, or a size query of 0, means the call runs exactly as blkq4_fp16_gemm_sm100.  No counterpart in the reference (its split-K template parameters
 * are unused, src/mickey/blk_q4/f16_gemm_sm80.h:86-90).
 */
size_t blkq4_gemm_workspace_size(int m, int n, int k);

/* No counterpart in the reference.  Host-only description of the work plan blkq4_fp16_gemm_ws_sm100 would
 * choose for the problem with a workspace of `workspace_size` bytes: nothing is launched and no device is
 * needed (the plan depends on the current device's SM count; 148 is assumed without a device).
 *   out6[0]  kernel: 0 = skinny kernels (m <= 16), 1 = tensor-core kernel with one CTA per tile,
 *            2 = tensor-core kernel with CTA pairs
 *   out6[1]  activation rows per tile        out6[2]  output tiles
 *   out6[3]  K split (1, 2 or 4)             out6[4]  1 when the tiles are cut in balanced k-step ranges
 *   out6[5]  units the balanced ranges are cut for (SMs or pairs of SMs), else 0
 * blkq4_gemm_plan_range_bound returns the first k step of unit b's range in the balanced plan's
 * (tile, k step) sequence of total_steps = tiles * (k / 64) steps (b == units: the end). */
int blkq4_gemm_plan(int m, int n, int k, size_t workspace_size, int* out6);
int blkq4_gemm_plan_range_bound(int total_steps, int k_steps, int units, int b);
int blkq4_fp16_gemm_ws_sm100(
  int block_size,
  bool column_wise_blocking,
  int m, int n, int k, void* stream,
  void const* act_ptr, size_t a_size,
  void const* weights_ptr, size_t weights_size,
  void const* scales_ptr, size_t scales_size,
  void const* offsets_ptr, size_t offsets_size,
  void* output_ptr, size_t output_size,
  void const* bias_ptr, size_t bias_size,
  unsigned flags,
  void* workspace, size_t workspace_size,
  void* error_message);

/**
 * blkq4_fp16_gemm_ws_sm100 with the workspace taken from a 12 MiB device array that is part of the
 * library (blkq4_static_scratch_size() bytes) instead of from the caller: nothing on this path
 * allocates, on the host or on the device.  A problem whose split-K workspace would not fit is
 * refused with an error (e.g. M = 256, N = K = 4096: 32 tiles split four ways need 12.6 MB); use
 * blkq4_fp16_gemm_sm100 for it.  A problem whose balanced-range workspace would not fit is not refused:
 * it runs in whole rounds, as it would without a workspace.  Every call on a
 * device shares the one array, so calls that can overlap on the GPU - on different streams, or
 * replays of captured graphs running side by side - race and corrupt each other's results: one
 * call at a time per device.  If a bounded in-kernel wait expires (blkq4_last_kernel_status != 0),
 * per-tile flag words may be left set in the array; blkq4_reset() clears them.  No counterpart in
 * the reference.
 */
size_t blkq4_static_scratch_size(void);
int blkq4_fp16_gemm_static_ws_sm100(
  int block_size,
  bool column_wise_blocking,
  int m, int n, int k, void* stream,
  void const* act_ptr, size_t a_size,
  void const* weights_ptr, size_t weights_size,
  void const* scales_ptr, size_t scales_size,
  void const* offsets_ptr, size_t offsets_size,
  void* output_ptr, size_t output_size,
  void const* bias_ptr, size_t bias_size,
  unsigned flags,
  void* error_message);

/*
 * N-sharded layers on one box, one process per GPU: skinny GEMM (M <= 16) fused with the
 * all-gather of the outputs.  No counterpart in the reference, which is single-GPU.
 *
 * Rank r holds the weight columns [r*n_shard, (r+1)*n_shard).  blkq4_gather_create allocates the
 * rank's exchange block (the one place this library allocates device memory: 1 KB of control
 * words plus six buffers of max_out_bytes) and returns its 64-byte CUDA IPC handle; the caller
 * exchanges the handles of all ranks by any means (e.g. its process group) and passes them,
 * ordered by rank, to blkq4_gather_connect.  blkq4_fp16_gemm_gather_sm100 then computes this
 * rank's [m, n_shard] slice and delivers the complete [m, world*n_shard] result into
 * output_ptr on EVERY rank.  Decode shapes (m <= 8, K a multiple of 256, K >= 2048) take ONE
 * launch: the kernel stores its results into all ranks' exchange buffers over NVLink as 8-byte
 * words that carry the call's number, then waits (bounded, ~1 s) for the words of all ranks and
 * copies the result out.  Other shapes on the skinny kernel's TMA path (m <= 16, 512 <= K <= 32768)
 * take two launches: the kernel stores fp16 results and raises a per-rank flag, a second small
 * kernel waits for all flags and copies out.  Prefill shapes on the CTA-pair tensor-core kernel
 * (m >= 256 with at least one round of 256 x 256 tiles per pair of SMs, at most 4 ranks) take three launches: the
 * GEMM kernel's epilogue stores every output tile into all ranks' exchange buffers, under the MMAs
 * of the next tile, and raises the per-rank flag; the small kernel waits; a full-width kernel
 * copies out.  All ranks must make the same sequence of calls;
 * work that reads output_ptr must be enqueued on `stream` before the next gather call.  A shape
 * outside these paths is refused with an error text starting "Kernel execution failed: unsupported":
 * compute with blkq4_fp16_gemm_sm80 and all-gather with the caller's collective instead;
 * blkq4_gather_supported_sm100 answers the question beforehand (1 / 0; a pure function of its
 * arguments and of the device's SM count; for m > 16 the context's world size must also be <= 4).  blkq4_gather_status synchronises `stream` and returns 0, or
 * (0x400 | rank) of the first rank whose data did not arrive in time; blkq4_gather_reset
 * (device drained on every rank, between the same two calls on every rank) clears that state.
 * blkq4_gather_destroy frees the rank's block: peers store into it from their own kernels, so
 * every rank must have drained its stream, and a cross-rank barrier must have passed, before ANY
 * rank destroys its context.
 */
int blkq4_gather_create(int world, int rank, size_t max_out_bytes, void** ctx, void* ipc_handle_64_bytes,
                        void* error_message);
int blkq4_gather_connect(void* ctx, void const* ipc_handles_world_x_64_bytes, void* error_message);
/* One process driving several GPUs (peer access enabled by the caller) connects its contexts
 * with plain pointers instead of IPC handles: blocks[r] = blkq4_gather_local_block(ctx of rank r). */
void* blkq4_gather_local_block(void* ctx);
int blkq4_gather_connect_pointers(void* ctx, void* const* blocks_by_rank, void* error_message);
int blkq4_fp16_gemm_gather_sm100(
  void* ctx,
  int block_size,
  bool column_wise_blocking,
  int m, int n_shard, int k, void* stream,
  void const* act_ptr, size_t a_size,
  void const* weights_ptr, size_t weights_size,
  void const* scales_ptr, size_t scales_size,
  void const* offsets_ptr, size_t offsets_size,
  void* output_ptr, size_t output_size,
  unsigned flags,
  void* error_message);
int blkq4_gather_status(void* ctx, void* stream);
int blkq4_gather_reset(void* ctx);
int blkq4_gather_supported_sm100(int block_size, bool column_wise_blocking, int m, int n_shard, int k);
int blkq4_gather_destroy(void* ctx);

/*
 * Additions with no counterpart in the reference.  The reference reports errors
 * through a std::string*, which only a C++ caller can supply.  These three let
 * a C, ctypes, cgo or JNI caller own such an object.
 */
void* blkq4_errmsg_create(void);              /* new std::string                 */
char const* blkq4_errmsg_cstr(void* errmsg);  /* its c_str(); valid until reused */
void blkq4_errmsg_destroy(void* errmsg);      /* delete                          */

/**
 * Synchronises `stream` and returns the device-side status word of the kernels: 0 when
 * every in-kernel wait completed.  Waits on mbarriers are bounded; one that expires makes
 * the CTA drain and records (role << 8 | barrier) here instead of hanging the GPU (the
 * skinny kernel's word is reported with bit 16 set).  -1 if the stream itself is in error.
 * No counterpart in the reference, whose kernels have no such waits.
 */
int blkq4_last_kernel_status(void* stream);

/**
 * Recovery after a non-zero blkq4_last_kernel_status: enqueues on `stream` the clearing of the
 * kernels' status words and of the flag words of the library's static scratch array
 * (blkq4_fp16_gemm_static_ws_sm100).  A caller-owned split-K workspace must be re-zeroed by its
 * owner.  Allocates nothing.  No counterpart in the reference.
 */
int blkq4_reset(void* stream);

/** Library identification: "gemmlib_b200 <version> sm_100a". */
char const* blkq4_version(void);

}  // extern "C"
