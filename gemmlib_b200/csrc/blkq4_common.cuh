// Shared definitions of the blockwise-int4 (W4A16) kernels for sm_100a.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace blkq4 {

// Quantization block extents along K and N for a (block, orientation) pair:
// column-wise blocks are (block x 1), row-wise blocks are (1 x block).
// Reference: src/mickey/blk_q4/f16_quant_sm80.cuh:159-162.
struct Blocking {
  int bk, bn;
  __host__ __device__ Blocking(int block, bool colwise)
      : bk(colwise ? block : 1), bn(colwise ? 1 : block) {}
};

inline bool supported_block(int b) { return b == 16 || b == 32 || b == 64 || b == 128; }

// Host-side launchers; each returns an empty string or an error text.
std::string launch_quant_prepack(int block, bool colwise, int K, int N, int ld,
                                 cudaStream_t stream, const __half* w, uint8_t* packed,
                                 __half* scales, uint8_t* zp);

std::string launch_gemv(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                        const __half* a, const uint8_t* packed, const __half* scales,
                        const uint8_t* zp, __half* out, const __half* bias, unsigned flags);

// The decode kernel (M <= 8, column-wise blocks >= 64, K a multiple of 256 and >= 2048): per-warp
// cp.async rings, two launches resident per SM.  Returns kStreamUnsupported for other shapes.
extern const char* const kStreamUnsupported;
struct GatherTable;
std::string launch_gemv_stream(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                               const __half* a, const uint8_t* packed, const __half* scales,
                               const uint8_t* zp, __half* out, const __half* bias, unsigned flags,
                               const GatherTable* gt = nullptr);

// The same weight stream for 9 <= M <= 16 (two row groups, two tiles per pass, activations from L2).
std::string launch_gemv_wide(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                             const __half* a, const uint8_t* packed, const __half* scales,
                             const uint8_t* zp, __half* out, const __half* bias, unsigned flags);

// Multiprocessor count of the CURRENT device (cached per device index).
int sm_count();

// ---- fused GEMV + all-gather over peer memory (one process per GPU, one box) ----------------
// Every rank owns one device block, mapped by all peers (CUDA IPC):
//   [0]   uint32 epoch      layer calls completed by this rank
//   [4]   uint32 done_ctr   CTAs of the running call that have finished storing
//   [8]   int    error      first wait that expired (0 = none)
//   [12]  uint32 tickets    CTAs of the wait kernel started so far (kGatherWaitCtas per call)
//   [64]  uint32 flags[2][kGatherMaxRanks]   flags[slot][src] = epoch whose slice from `src` landed (two-kernel protocol)
//   [kGatherCtrlBytes]                  gathered[2][buf_bytes]     fp16 [M, N_total] of even / odd epochs (two-kernel protocol)
//   [kGatherCtrlBytes + 2 buf_bytes]    flagged[2][2 * buf_bytes]  words {two fp16, epoch} of even / odd epochs (one-kernel protocol)
constexpr int kGatherMaxRanks = 8;
constexpr int kGatherCtrlBytes = 1024;
constexpr int kGatherEpochOff = 0, kGatherDoneOff = 4, kGatherErrorOff = 8, kGatherTicketOff = 12, kGatherFlagsOff = 64;
constexpr int kGatherMaxPrefillRanks = 4;  // the tensor-core path's fused exchange (see blkq4_fp16_gemm_gather_sm100)
constexpr int kGatherWaitCtas = 8;  // fixed grid of the wait kernel: its call number is tickets / 8

struct GatherTable {
  uint8_t* base[kGatherMaxRanks];  // every rank's block; base[rank] is the local one
  int world, rank;                 // world == 0: no gather (plain output)
  int n_total;                     // columns of the gathered output = world * N
  unsigned long long buf_bytes;    // bytes of one gathered buffer
};

// The skinny kernel with its epilogue storing this rank's [M, N] slice straight into every
// rank's gathered buffer.  *delivered = true: the launch also waited for the peers and copied the
// complete result to out_full (decode kernel); false: the caller launches the wait-and-copy kernel.
// Returns "unsupported" when the shape is on neither fast path.
std::string launch_gemv_gather(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                               const __half* a, const uint8_t* packed, const __half* scales,
                               const uint8_t* zp, __half* out_full, const GatherTable& gt, unsigned flags,
                               bool* delivered);

std::string launch_gemm_tc(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                           const __half* a, const uint8_t* packed, const __half* scales,
                           const uint8_t* zp, __half* out, const __half* bias, void* workspace,
                           size_t workspace_bytes, unsigned flags, const GatherTable* gt = nullptr);
// True when launch_gemm_tc takes the problem with a GatherTable (the CTA-pair kernel's fused all-gather).
bool gemm_tc_gather_supported(int M, int N, int K);
// Bytes of zero-initialised workspace with which launch_gemm_tc would split K for this problem
// (0: it would not).
size_t gemm_tc_workspace_bytes(int M, int N, int K);
// True when the preferred plan of the problem is the balanced one (more tiles than SMs): its workspace
// only buys balance; without it the same kernel runs in whole rounds.
bool gemm_tc_plan_balanced(int M, int N, int K);
// True when the one-CTA kernel's split-K plan of the problem needs more than `capacity` bytes (the
// static-scratch entry point refuses exactly those problems).
bool gemm_tc_split_plan_refusable(int M, int N, int K, size_t capacity);

// Synchronises `stream` and returns the tensor-core kernel's device error word
// (0 = every bounded wait completed; -1 = the stream itself reported an error).
int read_gemm_tc_error(cudaStream_t stream);
// The skinny kernel's device error word (call after the stream has been synchronised).
int read_gemv_error();
// Recovery after an expired wait: clear the kernels' error words / the static scratch's flag words.
int clear_gemm_tc_error(cudaStream_t stream);
int clear_gemv_error(cudaStream_t stream);
int reset_static_scratch(cudaStream_t stream);

#ifdef __CUDACC__

// One 32-bit word of the packed weight (4 bytes along kp at a fixed packed
// column np) holds 8 nibbles:  q[2r,n0] q[2r+8,n0] q[2r,n0+8] q[2r+8,n0+8]
// q[2r+1,n0] q[2r+9,n0] q[2r+1,n0+8] q[2r+9,n0+8]  (r = word index in its
// 16-byte group, n0 = 16*(np/8) + np%8).  This turns it into four half2 of
// fp16(16 + q), paired along k:
//   h[0] = (n0;   2r, 2r+1)    h[1] = (n0;   2r+8, 2r+9)
//   h[2] = (n0+8; 2r, 2r+1)    h[3] = (n0+8; 2r+8, 2r+9)
// 0x4c00 is fp16 16.0, whose mantissa step is 1/64, so a nibble placed at bits
// 6..9 adds its integer value.  Same numerics as the reference's weights2Half
// (src/mickey/cutlass_ext/q4gemm/warp/quantb_meta_mma_tensor_op_tile_iterator.h:69-104).
__device__ __forceinline__ void word_to_half16plus(uint32_t x, uint32_t h[4]) {
  constexpr uint32_t kMask = 0x03c003c0u, kSixteen = 0x4c004c00u;
  h[0] = ((x << 6) & kMask) | kSixteen;
  h[1] = ((x << 2) & kMask) | kSixteen;
  h[2] = ((x >> 2) & kMask) | kSixteen;
  h[3] = ((x >> 6) & kMask) | kSixteen;
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi) {
  return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

// Dequantization offset term rn_f16(scale * fp16(-16 - zp)); the dequantized
// weight is then fma_rn_f16(scale, fp16(16 + q), offset).  Two fp16 roundings,
// as in the reference kernel (same file as above, :436-543).
__device__ __forceinline__ __half dequant_offset(__half scale, int zp) {
  return __hmul_rn(scale, __int2half_rn(-16 - zp));
}

#endif  // __CUDACC__

}  // namespace blkq4
