// blkq4_fp16_gemm_static_ws_sm100: the split-K tensor-core GEMM with its workspace taken from a
// file-scope device array instead of from the caller.  Nothing on this path allocates: the array
// is part of the loaded module, its address is looked up once per device, and problems whose
// workspace would not fit are refused.  The reference has no counterpart.
#include <cstddef>
#include <cstdint>
#include <atomic>
#include <string>

#include <cuda_runtime.h>

#include "blkq4_common.cuh"
#include "ms_blkq4gemm.h"

namespace {

// 12 MiB.  Covers, e.g., M = 512 on 4096-wide layers (64 tiles, two-way split: 8.4 MB) and a 148-SM
// part's largest two-way split at BM = 256 (74 tiles x 128 KB = 9.7 MB).  A problem whose preferred
// plan needs more - e.g. M = 256, N = K = 4096: 32 tiles split four ways, 12.6 MB - is refused; call
// blkq4_fp16_gemm_sm100 (no split) or blkq4_fp16_gemm_ws_sm100 with memory of your own for those.
constexpr size_t kStaticScratchBytes = 12u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_ptr[kMaxDevices];

int fail(void* err, const std::string& msg) {
  if (err) *reinterpret_cast<std::string*>(err) = msg;
  return -1;
}

// Address of the scratch array on the current device; looked up once per device.
void* static_scratch(std::string& why) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    why = std::string("cudaGetDevice: ") + cudaGetErrorString(e);
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    why = "device index " + std::to_string(dev) + " out of range";
    return nullptr;
  }
  void* ptr = g_scratch_ptr[dev].load(std::memory_order_acquire);
  if (ptr) return ptr;
  e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
  if (e != cudaSuccess || !ptr) {
    why = std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e);
    return nullptr;
  }
  g_scratch_ptr[dev].store(ptr, std::memory_order_release);
  return ptr;
}

}  // namespace

extern "C" size_t blkq4_static_scratch_size(void) { return kStaticScratchBytes; }

namespace blkq4 {
// Zeroes the flag words at the head of the static scratch on the current device (the partial tiles
// behind them need no clearing).  Enqueued on `stream`; allocates nothing.
int reset_static_scratch(cudaStream_t stream) {
  std::string why;
  void* scratch = static_scratch(why);
  if (!scratch) return -1;
  // flags: one word per output tile, at most one tile per SM and split; 64 KB is far beyond any plan
  return cudaMemsetAsync(scratch, 0, 64 * 1024, stream) == cudaSuccess ? 0 : -1;
}
}  // namespace blkq4

extern "C" int blkq4_fp16_gemm_static_ws_sm100(int block_size, bool column_wise_blocking, int m, int n, int k,
                                               void* stream, void const* act_ptr, size_t a_size,
                                               void const* weights_ptr, size_t weights_size,
                                               void const* scales_ptr, size_t scales_size,
                                               void const* offsets_ptr, size_t offsets_size, void* output_ptr,
                                               size_t output_size, void const* bias_ptr, size_t bias_size,
                                               unsigned flags, void* err) {
  // A split-K plan of the one-CTA kernel that does not fit is refused.  Plans that only buy balance
  // (balanced ranges of either kernel) are not: when they do not fit, the launch picks what fits.
  if (blkq4::gemm_tc_split_plan_refusable(m, n, k, kStaticScratchBytes))
    return fail(err, "Split-K workspace of " + std::to_string(blkq4_gemm_workspace_size(m, n, k)) +
                         " bytes exceeds the static scratch of " + std::to_string(kStaticScratchBytes) + " bytes");
  std::string why;
  void* scratch = static_scratch(why);
  if (!scratch) return fail(err, "Static scratch unavailable: " + why);
  return blkq4_fp16_gemm_ws_sm100(block_size, column_wise_blocking, m, n, k, stream, act_ptr, a_size, weights_ptr,
                                  weights_size, scales_ptr, scales_size, offsets_ptr, offsets_size, output_ptr,
                                  output_size, bias_ptr, bias_size, flags, scratch, kStaticScratchBytes, err);
}
