// TMA / mbarrier helpers shared by the sm_100a kernels: host-side tensor-map encoding
// (driver entry point fetched through the runtime, so the library does not link libcuda)
// and the device-side PTX wrappers.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <memory>

namespace blkq4 {

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                       const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                       const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TensorMapEncodeFn tensor_map_encode_fn() {
  static TensorMapEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<TensorMapEncodeFn>(p);
  }();
  return fn;
}

// 2-D row-major tensor [rows][cols] of `elt` bytes per element; box = box_rows x box_cols.
// Requirements (checked by the driver): 16-byte aligned base, row pitch a multiple of 16
// bytes, box_cols * elt a multiple of 16 bytes, box extents <= 256.
// A descriptor is a pure function of the arguments below, and a decode loop asks for the same few
// hundred descriptors over and over: a small per-thread direct-mapped cache takes the driver call
// (~1 us each, three or four per launch) off the launch path.
inline bool encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elt, const void* ptr,
                                 uint64_t cols, uint64_t rows, uint32_t box_cols, uint32_t box_rows,
                                 CUtensorMapSwizzle swz) {
  struct Entry {
    const void* ptr;
    uint64_t cols, rows;
    uint32_t box_cols, box_rows;
    int dt, elt, swz;
    bool valid;
    CUtensorMap map;
  };
  constexpr int kEntries = 1024;
  thread_local std::unique_ptr<Entry[]> cache_mem;
  if (!cache_mem) cache_mem.reset(new Entry[kEntries]());
  Entry* cache = cache_mem.get();
  uint64_t h = reinterpret_cast<uintptr_t>(ptr) >> 4;
  h ^= (cols * 0x9e3779b97f4a7c15ull) ^ (rows * 0xc2b2ae3d27d4eb4full) ^ ((uint64_t)box_cols << 20) ^
       ((uint64_t)box_rows << 8) ^ (uint64_t)swz ^ ((uint64_t)dt << 4);
  h ^= h >> 29;
  Entry& e = cache[h % kEntries];
  if (e.valid && e.ptr == ptr && e.cols == cols && e.rows == rows && e.box_cols == box_cols &&
      e.box_rows == box_rows && e.dt == (int)dt && e.elt == elt && e.swz == (int)swz) {
    *map = e.map;
    return true;
  }
  TensorMapEncodeFn fn = tensor_map_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elt};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  e = Entry{ptr, cols, rows, box_cols, box_rows, (int)dt, elt, (int)swz, true, *map};
  return true;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is per device and sticky: raise it only when a launch
// needs more than an earlier one asked for.  `granted` is one table per kernel instance.
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kern, size_t bytes, std::atomic<int> (&granted)[64]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && granted[dev].load(std::memory_order_relaxed) >= (int)bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && dev >= 0 && dev < 64) granted[dev].store((int)bytes, std::memory_order_relaxed);
  return e;
}

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking poll (try_wait may suspend the thread for a hardware-defined time; this never does).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that may stay suspended for up to `ns` nanoseconds before it reports "not yet": a waiting
// role then polls once per microsecond instead of spinning, and leaves the issue slots and the ALU
// pipe to the warps that compute (measured on the tensor-core kernel at M = 64: ~40 % of all issued
// instructions were polls).
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `max_cycles`, or as soon as another thread of the CTA has
// given up (abort_flag, in shared memory).  On expiry records `who` in *error_word (global)
// and returns false; the caller drains instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* error_word, int who, long long max_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_hint(bar, parity, 1000u)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > max_cycles) {
      *abort_flag = 1;
      atomicCAS(error_word, 0, who);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace blkq4
