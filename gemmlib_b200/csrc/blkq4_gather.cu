// Fused GEMM + all-gather for N-sharded layers on one box (one process per GPU).
//
// Each rank owns one device block (control words, per-source flags, two gathered fp16 buffers, two
// buffers of flagged words) that all peers map through CUDA IPC.  Three shapes of a layer call, all
// on the caller's stream:
//   decode kernel (M <= 8), ONE launch: the kernel stores its results into every rank's block as
//      8-byte words {two fp16, epoch} (the data is its own flag), then polls its own block -
//      bounded - until every word carries the call's epoch and copies the result out;
//   TMA skinny kernel (M <= 16), TWO launches: the epilogue stores this rank's [M, N/g] columns
//      straight into EVERY rank's gathered buffer over NVLink (plain peer stores; no multicast, no
//      pulls) and the grid's last CTA raises this rank's flag in every rank's block; a small kernel,
//      resident alongside the first, waits - bounded - until the flags of all ranks carry the call's
//      epoch, then copies the complete [M, N] result into the caller's output tensor;
//   CTA-pair tensor-core kernel (prefill), THREE launches: the GEMM's epilogue stores every output
//      tile into every rank's gathered buffer under the MMAs of the next tile and publishes like
//      the skinny kernel; the small kernel only waits; a full-width kernel copies out.
// Everything a launch needs to know about "which call is this" lives in device memory (the
// epoch word), so the pair can be captured in a CUDA graph and replayed.
//
// Buffer reuse: epochs alternate between two gathered buffers.  A peer writes buffer b for
// epoch e + 2 only after its own wait for epoch e + 1 has passed, i.e. after this rank launched
// call e + 1, which is stream-ordered after this rank's copy-out of epoch e.
//
// The reference has no multi-GPU path; this file has no counterpart there.
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "blkq4_common.cuh"
#include "ms_blkq4gemm.h"

namespace blkq4 {
namespace {

constexpr long long kGatherWaitCycles = 2000000000ll;  // ~1 s

struct GatherCtx {
  int world = 0, rank = 0;
  size_t buf_bytes = 0;      // capacity of one gathered buffer
  size_t block_bytes = 0;
  uint8_t* base[kGatherMaxRanks] = {};
  bool opened[kGatherMaxRanks] = {};
};

inline int fail(void* err, const std::string& msg) {
  if (err) *reinterpret_cast<std::string*>(err) = msg;
  return -1;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until every rank's flag of this call's slot has reached the call's epoch, then copies
// the gathered result out.  Launched with programmatic stream serialization: its CTAs become
// resident while the skinny kernel of the same call still runs, so the flags are seen the moment
// they land and neither a launch gap nor a grid-completion round trip sits between the last
// store and the copy-out.  It therefore cannot read the call's epoch from the kernel it overlaps:
// it numbers itself, each CTA drawing a ticket (fixed grid of kGatherWaitCtas, tickets of
// consecutive calls cannot interleave because the next skinny kernel starts only after every
// CTA here has passed launch_dependents).
__global__ void __launch_bounds__(256)
gather_wait_copy_kernel(uint8_t* local, int world, unsigned long long buf_bytes, uint4* out, unsigned long long n16) {
  // out == nullptr: wait only (a large result is copied out by gather_copy_kernel afterwards)
  __shared__ unsigned s_epoch;
  if (threadIdx.x == 0)
    s_epoch = atomicAdd(reinterpret_cast<unsigned*>(local + kGatherTicketOff), 1u) / kGatherWaitCtas + 1u;
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;");
  const unsigned epoch = s_epoch;
  const unsigned slot = epoch & 1u;
  if ((int)threadIdx.x < world) {
    const unsigned* flag = reinterpret_cast<const unsigned*>(local + kGatherFlagsOff) + slot * kGatherMaxRanks + threadIdx.x;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(flag) - epoch) < 0) {
      if (clock64() - t0 > kGatherWaitCycles) {
        atomicCAS(reinterpret_cast<int*>(local + kGatherErrorOff), 0, 0x400 | (int)threadIdx.x);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  // Peers wrote these lines through NVLink into this GPU's memory: read around L1.
  if (!out) return;
  const uint4* src = reinterpret_cast<const uint4*>(local + kGatherCtrlBytes + (size_t)slot * buf_bytes);
  for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < n16;
       i += (unsigned long long)gridDim.x * blockDim.x)
    out[i] = __ldcg(src + i);
}

// Copy-out of a large gathered result (the tensor-core path): runs after the wait kernel has
// completed, when this rank's epoch word holds the call's epoch, so the buffer's parity is read
// from the device and the launch replays from a CUDA graph.
__global__ void __launch_bounds__(256)
gather_copy_kernel(const uint8_t* local, unsigned long long buf_bytes, uint4* out, unsigned long long n16) {
  const unsigned slot = *reinterpret_cast<const volatile unsigned*>(local + kGatherEpochOff) & 1u;
  const uint4* src = reinterpret_cast<const uint4*>(local + kGatherCtrlBytes + (size_t)slot * buf_bytes);
  for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < n16;
       i += (unsigned long long)gridDim.x * blockDim.x)
    out[i] = __ldcg(src + i);
}

}  // namespace
}  // namespace blkq4

using blkq4::GatherCtx;

extern "C" int blkq4_gather_create(int world, int rank, size_t max_out_bytes, void** ctx_out, void* ipc_handle,
                                   void* err) {
  if (world < 1 || world > blkq4::kGatherMaxRanks || rank < 0 || rank >= world)
    return blkq4::fail(err, "Unsupported world size / rank: " + std::to_string(world) + " / " + std::to_string(rank));
  if (!ctx_out || !ipc_handle || max_out_bytes == 0) return blkq4::fail(err, "Null argument");
  auto* c = new (std::nothrow) GatherCtx();
  if (!c) return blkq4::fail(err, "Out of host memory");
  c->world = world;
  c->rank = rank;
  c->buf_bytes = (max_out_bytes + 255) & ~(size_t)255;
  c->block_bytes = blkq4::kGatherCtrlBytes + 6 * c->buf_bytes;  // two fp16 buffers + two buffers of flagged words
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, c->block_bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, c->block_bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    delete c;
    return blkq4::fail(err, std::string("blkq4_gather_create: ") + cudaGetErrorString(e));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(ipc_handle, &h, sizeof(h));
  c->base[rank] = reinterpret_cast<uint8_t*>(p);
  *ctx_out = c;
  return 0;
}

extern "C" int blkq4_gather_connect(void* ctx, void const* handles, void* err) {
  auto* c = reinterpret_cast<GatherCtx*>(ctx);
  if (!c || !handles) return blkq4::fail(err, "Null argument");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank || c->opened[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, reinterpret_cast<const uint8_t*>(handles) + (size_t)r * sizeof(h), sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
      return blkq4::fail(err, "blkq4_gather_connect: rank " + std::to_string(r) + ": " + cudaGetErrorString(e));
    c->base[r] = reinterpret_cast<uint8_t*>(p);
    c->opened[r] = true;
  }
  return 0;
}

extern "C" void* blkq4_gather_local_block(void* ctx) {
  auto* c = reinterpret_cast<GatherCtx*>(ctx);
  return c ? c->base[c->rank] : nullptr;
}

extern "C" int blkq4_gather_connect_pointers(void* ctx, void* const* blocks, void* err) {
  auto* c = reinterpret_cast<GatherCtx*>(ctx);
  if (!c || !blocks) return blkq4::fail(err, "Null argument");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    if (!blocks[r]) return blkq4::fail(err, "Null block pointer for rank " + std::to_string(r));
    c->base[r] = reinterpret_cast<uint8_t*>(blocks[r]);  // not opened by this context: not closed by it
  }
  return 0;
}

extern "C" int blkq4_fp16_gemm_gather_sm100(void* ctx, int block_size, bool column_wise_blocking, int m,
                                            int n_shard, int k, void* stream_ptr, void const* act_ptr,
                                            size_t a_size, void const* weights_ptr, size_t weights_size,
                                            void const* scales_ptr, size_t scales_size,
                                            void const* offsets_ptr, size_t offsets_size, void* output_ptr,
                                            size_t output_size, unsigned flags, void* err) {
  auto* c = reinterpret_cast<GatherCtx*>(ctx);
  if (!c) return blkq4::fail(err, "Null gather context");
  for (int r = 0; r < c->world; ++r)
    if (!c->base[r]) return blkq4::fail(err, "Gather context is not connected to rank " + std::to_string(r));
  if (!blkq4::supported_block(block_size))
    return blkq4::fail(err, "Unsupported block size: " + std::to_string(block_size));
  if (m <= 0 || n_shard <= 0 || k <= 0)
    return blkq4::fail(err, "Empty problem size: " + std::to_string(m) + "x" + std::to_string(n_shard) + "x" +
                                std::to_string(k));
  const blkq4::Blocking b(block_size, column_wise_blocking);
  if ((k % 64) != 0 || (k % b.bk) != 0 || (n_shard % 16) != 0 || (n_shard % b.bn) != 0)
    return blkq4::fail(err, "Kernel execution failed: Error Misaligned Operand or Invalid Problem: " +
                                std::to_string(m) + "x" + std::to_string(n_shard) + "x" + std::to_string(k));
  const size_t meta = (size_t)(k / b.bk) * (size_t)(n_shard / b.bn);
  const size_t n_total = (size_t)n_shard * c->world;
  const bool has_offsets = offsets_ptr && offsets_size > 0;
  if (a_size != (size_t)m * k * 2 || weights_size != (size_t)(k / 2) * n_shard ||
      scales_size != meta * 2 || (has_offsets && offsets_size != meta) || output_size != (size_t)m * n_total * 2)
    return blkq4::fail(err, "Unexpected tensor size");
  if (output_size > c->buf_bytes)
    return blkq4::fail(err, "Gathered output of " + std::to_string(output_size) + " bytes exceeds the context's " +
                                std::to_string(c->buf_bytes));
  if (!act_ptr || !weights_ptr || !scales_ptr || !output_ptr) return blkq4::fail(err, "Null tensor pointer");
  if (reinterpret_cast<uintptr_t>(act_ptr) % 16 != 0 || reinterpret_cast<uintptr_t>(weights_ptr) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(output_ptr) % 16 != 0)
    return blkq4::fail(err, "Kernel execution failed: Error Misaligned Operand");

  blkq4::GatherTable gt{};
  for (int r = 0; r < c->world; ++r) gt.base[r] = c->base[r];
  gt.world = c->world;
  gt.rank = c->rank;
  gt.n_total = (int)n_total;
  gt.buf_bytes = c->buf_bytes;
  auto stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  if (m > 16) {
    // Tensor-core path: the CTA-pair kernel stores its tiles into every rank's gathered buffer and
    // publishes like the skinny kernels; the wait kernel only waits, a full-width kernel copies out.
    // Up to four ranks by default: measured on B200 (K = 8192, N = 28672, M = 4096) the fused call takes
    // 862-888 us against 1300-1404 us for kernel + NCCL all-gather at 2 ranks, 717 against 992 us at 4, and
    // 778 against 817 us at 8 - every GPU takes in ~300 GB/s from its peers whatever their number, about what
    // NCCL's all-gather reaches on the same box, so at 8 ranks the exchange, not the GEMM, sets the time.
    static const int max_prefill_ranks = getenv("BLKQ4_GATHER_PREFILL_MAX_RANKS") ? atoi(getenv("BLKQ4_GATHER_PREFILL_MAX_RANKS")) : blkq4::kGatherMaxPrefillRanks;
    if (c->world > max_prefill_ranks)
      return blkq4::fail(err, "Kernel execution failed: unsupported world size for the fused all-gather of m > 16");
    if (reinterpret_cast<uintptr_t>(scales_ptr) % 16 != 0 ||
        (has_offsets && reinterpret_cast<uintptr_t>(offsets_ptr) % 16 != 0))
      return blkq4::fail(err, "Kernel execution failed: Error Misaligned Operand (scales and offsets must be 16-byte aligned for m > 16)");
    const std::string e2 = blkq4::launch_gemm_tc(
        block_size, column_wise_blocking, m, n_shard, k, stream, reinterpret_cast<const __half*>(act_ptr),
        reinterpret_cast<const uint8_t*>(weights_ptr), reinterpret_cast<const __half*>(scales_ptr),
        has_offsets ? reinterpret_cast<const uint8_t*>(offsets_ptr) : nullptr, nullptr, nullptr, nullptr, 0, flags, &gt);
    if (!e2.empty()) return blkq4::fail(err, "Kernel execution failed: " + e2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blkq4::kGatherWaitCtas);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, blkq4::gather_wait_copy_kernel, c->base[c->rank], c->world,
                       (unsigned long long)c->buf_bytes, (uint4*)nullptr, 0ull);
    const int sms = blkq4::sm_count() > 0 ? blkq4::sm_count() : 148;
    blkq4::gather_copy_kernel<<<2 * sms, 256, 0, stream>>>(c->base[c->rank], (unsigned long long)c->buf_bytes,
                                                           reinterpret_cast<uint4*>(output_ptr), output_size / 16);
    const cudaError_t ce = cudaGetLastError();
    if (ce != cudaSuccess) return blkq4::fail(err, std::string("Kernel execution failed: ") + cudaGetErrorString(ce));
    return 0;
  }
  bool delivered = false;
  const std::string e = blkq4::launch_gemv_gather(
      block_size, column_wise_blocking, m, n_shard, k, stream, reinterpret_cast<const __half*>(act_ptr),
      reinterpret_cast<const uint8_t*>(weights_ptr), reinterpret_cast<const __half*>(scales_ptr),
      has_offsets ? reinterpret_cast<const uint8_t*>(offsets_ptr) : nullptr, reinterpret_cast<__half*>(output_ptr),
      gt, flags, &delivered);
  if (!e.empty()) return blkq4::fail(err, "Kernel execution failed: " + e);
  if (delivered) return 0;  // one launch did everything
  const unsigned long long n16 = output_size / 16;
  // The wait kernel's eight CTAs copy 32 KB per round trip to L2: fine for a few rows, ~1 us per 32 KB
  // beyond that (M = 16 of a 28672-wide layer: 0.9 MB, ~28 us).  Larger results are copied out by a
  // full-width kernel after the wait, like the tensor-core path's.
  const bool big = output_size > (size_t)128 * 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blkq4::kGatherWaitCtas);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, blkq4::gather_wait_copy_kernel, c->base[c->rank], c->world,
                     (unsigned long long)c->buf_bytes, big ? (uint4*)nullptr : reinterpret_cast<uint4*>(output_ptr),
                     big ? 0ull : n16);
  if (big) {
    const int sms = blkq4::sm_count() > 0 ? blkq4::sm_count() : 148;
    const unsigned long long want = (n16 + 255) / 256;
    const unsigned grid = (unsigned)(want < (unsigned long long)(2 * sms) ? want : (unsigned long long)(2 * sms));
    blkq4::gather_copy_kernel<<<grid, 256, 0, stream>>>(c->base[c->rank], (unsigned long long)c->buf_bytes,
                                                        reinterpret_cast<uint4*>(output_ptr), n16);
  }
  const cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return blkq4::fail(err, std::string("Kernel execution failed: ") + cudaGetErrorString(ce));
  return 0;
}

extern "C" int blkq4_gather_supported_sm100(int block_size, bool column_wise_blocking, int m, int n_shard, int k) {
  if (!blkq4::supported_block(block_size) || m <= 0 || n_shard <= 0 || k <= 0) return 0;
  const blkq4::Blocking b(block_size, column_wise_blocking);
  if ((k % 64) != 0 || (k % b.bk) != 0 || (n_shard % 16) != 0 || (n_shard % b.bn) != 0) return 0;
  if (m <= 16) return (column_wise_blocking && block_size >= 64 && k >= 512 && k <= 32768) ? 1 : 0;
  return blkq4::gemm_tc_gather_supported(m, n_shard, k) ? 1 : 0;
}

extern "C" int blkq4_gather_status(void* ctx, void* stream_ptr) {
  auto* c = reinterpret_cast<GatherCtx*>(ctx);
  if (!c) return -1;
  if (cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream_ptr)) != cudaSuccess) return -1;
  int v = 0;
  if (cudaMemcpy(&v, c->base[c->rank] + blkq4::kGatherErrorOff, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return -1;
  return v;
}

extern "C" int blkq4_gather_reset(void* ctx) {
  auto* c = reinterpret_cast<GatherCtx*>(ctx);
  if (!c) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  // control words only: the epoch restarts at zero on every rank, the buffers' stale flags (all
  // smaller than or equal to the old epoch) would be taken for fresh data, so they go too
  return cudaMemset(c->base[c->rank], 0, c->block_bytes) == cudaSuccess ? 0 : -1;
}

extern "C" int blkq4_gather_destroy(void* ctx) {
  auto* c = reinterpret_cast<GatherCtx*>(ctx);
  if (!c) return 0;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (r != c->rank && c->opened[r]) cudaIpcCloseMemHandle(c->base[r]);
  if (c->base[c->rank]) cudaFree(c->base[c->rank]);
  delete c;
  return 0;
}
