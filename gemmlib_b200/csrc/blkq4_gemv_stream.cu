// Decode kernel (M <= 8) for column-wise blocks of 64 or 128: out[M,N] = A[M,K] x dequant(W4[K,N]).
//
// The weight stream is the only large operand, so the kernel is organised around it.
//
//   * Every warp is its own producer and consumer.  A CTA has eight warps; warp w owns a fixed slice
//     of K (whole groups of four 64-k steps) of EVERY 16-column tile the CTA works on.  It copies its
//     slice of the packed weights, with the scales and zero points of those steps, into a private
//     ring of shared-memory slots with cp.async (16 bytes per lane, placed as [step][lane], so the
//     later 128-bit reads are conflict free) and waits with cp.async.wait_group, which, unlike a
//     plain load's scoreboard, lets older groups be consumed while younger ones are in flight.
//     D groups per warp are outstanding: 8 warps x 4 groups x 2 KB = 64 KB per CTA.
//   * Two CTAs fit on an SM and the grid has one CTA per SM (two when the tile count divides well),
//     so with programmatic stream serialization the NEXT launch's CTAs become resident beside this
//     one's, fill their rings, and only then wait for this launch to finish: HBM stays busy across
//     the launches of a decode stack.  Activations are read, and the output written, after that wait.
//   * Math as in the TMA skinny kernel (blkq4_gemv.cu): one packed word becomes four fp16 pairs
//     1024 + q / 64 + q with one shift and four lop3, mma.sync.m16n8k16 takes the weights as its
//     16-row operand and the activations as its 8-column operand, the accumulator of a 64-k step
//     starts at minus the activation-only term of that step, and the step's sum is scaled in fp32:
//         total += scale * (sum_k a_k (magic + q_k) - sum_k a_k (magic + 8)).
//     With zero points the term zp * scale * sum_k a_k is accumulated separately, one (step, column)
//     pair per lane, instead of inside the per-step code of every lane.
//   * At the end of a tile the warps leave their partial sums in shared memory, the CTA meets at one
//     barrier, and one warp (rotating) adds them in a fixed order, rounds to fp16 and stores.
//
// Instruction economy matters here: measured on B200 the kernel is bound by the integer / logic pipe
// (16 lop3 + 4 shifts per 64-k step and warp, at half rate), not by HBM, so everything else in the
// step is kept off that pipe: immediate-offset shared-memory loads, no predicates, no index math.
//
// Dequantization numerics: exact in fp32 up to the accumulation order (no fp16 rounding of scale * q);
// equal to the reference kernel's result where that is exact
// (src/mickey/cutlass_ext/q4gemm/warp/quantb_meta_mma_tensor_op_tile_iterator.h:69-104, :436-543).
#include <cstddef>
#include <cstdint>
#include <atomic>
#include <string>

#include "blkq4_common.cuh"
#include "blkq4_stream.cuh"
#include "blkq4_tma.cuh"
#include "ms_blkq4gemm.h"

namespace blkq4 {
namespace {

using namespace stream;
constexpr int kCorrStep = 4 * 16;    // bytes of mma-initialising terms per step: four row pairs, float4 each

struct StreamParams {
  const __half* a;
  __half* out;
  const __half* bias;
  const uint8_t* packed;
  const __half* scales;
  const uint8_t* zp;
  int M, N, K;
  int block_shift;  // 6 or 7
  int tiles;        // N / 16
  int steps;        // K / 64
  int a_pitch;      // halves per activation row in shared memory (K + 8: rows land on different banks)
  GatherTable gt;   // gather mode: the result goes to every rank's gathered buffer, then to `out` as [M, world * N]
};

constexpr long long kGatherWaitCycles = 2000000000ll;  // ~1 s

// Shared memory: rings [kWarps][D][kSlotBytes] | s_corr [steps][4] float4 | s_asum [steps][8] (zero points)
//                | s_part [2][PW][16][MS] | s_stage [8][16] fp16 (gather) | s_a [M][a_pitch]
// MZ: rows of the zero-point accumulators kept in registers (2 for M <= 2, else 8).
//
// GATHER (N-sharded layer, one process per GPU).  The exchange is latency-bound (a few tens of KB per
// rank), so it carries its own flags: the adding warp stores the tile's results into EVERY rank's
// exchange buffer as 8-byte words {two fp16 results, the call's epoch} - an aligned 8-byte store
// arrives whole, so a word whose flag equals the epoch holds that epoch's data and no fence, counter
// or second flag flight is needed.  When a CTA has finished its tiles it turns receiver: its threads
// poll - bounded - their share of the words of the complete [M, world * N] result in this rank's
// buffer and write the data halves to `out`.  The last CTA advances the rank's epoch.  One launch per
// layer.  Epochs alternate between two buffers: a peer writes epoch e + 2 only after it has received
// this rank's words of epoch e + 1, which this rank sends after its launch of epoch e has completed.
template <bool HAS_ZP, int D, int MZ, bool GATHER>
__global__ void __launch_bounds__(kWarps * 32, 2)
gemv_stream_kernel(const StreamParams p) {
  extern __shared__ __align__(16) uint8_t s_raw[];
  constexpr int W = kWarps, GS = kGroupSteps;
  constexpr int PW = HAS_ZP ? 2 * W : W;  // partial-sum entries per tile: the warps (+ their zero-point terms)
  const int MS = (p.M + 1) & ~1;
  uint8_t* s_ring = s_raw;
  float* s_corr = reinterpret_cast<float*>(s_ring + W * D * kSlotBytes);
  float* s_asum = s_corr + (size_t)p.steps * 16;
  float* s_part = s_asum + (HAS_ZP ? (size_t)p.steps * 8 : 0);
  __half* s_stage = reinterpret_cast<__half*>(s_part + (size_t)2 * PW * 16 * MS);
  __half* s_a = s_stage + 128;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = p.K, N = p.N, M = p.M;
  const int bs = p.block_shift - 6;
  const int kgroups = p.steps / GS;
  const int gb = (int)(((long long)kgroups * warp) / W);
  const int myg = (int)(((long long)kgroups * (warp + 1)) / W) - gb;  // >= 1: the launcher requires kgroups >= W
  const int my_tiles = (p.tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const uint32_t ring_addr = smem_u32(s_ring) + (uint32_t)warp * (D * kSlotBytes);
  const uint32_t ring_last = ring_addr + (D - 1) * kSlotBytes;

  // The next kernel of the stream may become resident now (a no-op unless it was launched with
  // programmatic stream serialization); it fills its rings and then waits for this grid to finish.
  asm volatile("griddepcontrol.launch_dependents;");

  // ---- loader: runs D groups ahead of the consumer; all addresses advance incrementally ----
  const uint8_t* wp = p.packed + (size_t)(blockIdx.x * 8 + g) * K + (size_t)gb * (GS * 64) + t * 16;
  const long long w_tile_adj = (long long)gridDim.x * 8 * K - (long long)myg * (GS * 64);
  // lanes 0-7 copy the scales of step lane / 2, column half lane % 2; lanes 8-11 the zero points of step lane - 8
  const uint32_t meta_lane = (lane < 2 * GS || (HAS_ZP && lane < 3 * GS)) ? 1u : 0u;
  const uint8_t* mp;
  uint32_t m_dst;
  long long m_step, m_tile_adj;
  {
    const int rows_per_group = GS >> bs;
    if (lane < 2 * GS) {
      const int u = lane >> 1, h = lane & 1;
      mp = reinterpret_cast<const uint8_t*>(p.scales) + ((size_t)((gb * GS + u) >> bs) * N + blockIdx.x * 16 + h * 8) * 2;
      m_dst = kSlotW + u * 32 + h * 16;
      m_step = (long long)rows_per_group * N * 2;
      m_tile_adj = (long long)gridDim.x * 32 - (long long)myg * m_step;
    } else {
      const int u = (lane - 2 * GS) % GS;
      mp = (HAS_ZP ? p.zp : p.packed) + (size_t)((gb * GS + u) >> bs) * N + blockIdx.x * 16;  // only used with zero points
      m_dst = kSlotW + kSlotS + u * 16;
      m_step = (long long)rows_per_group * N;
      m_tile_adj = (long long)gridDim.x * 16 - (long long)myg * m_step;
    }
  }
  int ld_left = my_tiles * myg, ld_j = 0;
  auto issue_group = [&](uint32_t dst) {
    const uint32_t go = ld_left > 0 ? 1u : 0u;
    const uint32_t dw = dst + lane * 16;
    cp_async16_if<0>(dw, wp, go);
    cp_async16_if<64>(dw, wp, go);
    cp_async16_if<128>(dw, wp, go);
    cp_async16_if<192>(dw, wp, go);
    cp_async16_if<0>(dst + m_dst, mp, go & meta_lane);
    cp_async_commit();  // always: the group count per iteration stays fixed
    --ld_left;
    const bool wrap = ++ld_j == myg;
    wp += (GS * 64) + (wrap ? w_tile_adj : 0);
    mp += m_step + (wrap ? m_tile_adj : 0);
    if (wrap) ld_j = 0;
  };
  // Weights, scales and zero points are read WITHOUT waiting for the preceding kernel of the stream
  // (the caller vouches for them when it asks for the early start).
  {
    uint32_t dst = ring_addr;
#pragma unroll
    for (int d = 0; d < D; ++d) {
      issue_group(dst);
      dst += kSlotBytes;
    }
  }

  // Activations and the output belong to stream order.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // Gather mode: this call's epoch is one past the calls this rank has completed (the word changes
  // only at the very end of a launch, and the preceding launch has completed: see the wait above).
  unsigned gather_epoch = 0;
  size_t gather_off = 0;
  if (GATHER) {
    gather_epoch = *reinterpret_cast<volatile unsigned*>(p.gt.base[p.gt.rank] + kGatherEpochOff) + 1u;
    gather_off = kGatherCtrlBytes + (size_t)(2 + 2 * (gather_epoch & 1u)) * p.gt.buf_bytes;  // flagged-word buffers follow the two fp16 ones
  }

  // ---- per warp: its own K slice of the activations into shared memory, and the activation-only
  //      terms of its steps.  Chunk c = 8 halves; even c is the "lo" half (k % 16 < 8) of a 16-k block.
  //      symmetric:   term = -(1024 lo + 64 hi + 8 (lo + hi));   zero points: -(1024 lo + 64 hi) and lo + hi
  {
    const int slice_k0 = gb * (GS * 64);
    const int chunks = myg * (GS * 8);  // a multiple of 32
    auto finish_row = [&](int m, int k0, const uint4& v) {
      *reinterpret_cast<uint4*>(s_a + (size_t)m * p.a_pitch + k0) = v;
      const __half2* h = reinterpret_cast<const __half2*>(&v);
      float s = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        s += f.x + f.y;
      }
      // the eight lanes of a step: sum the four chunks of equal parity, then pair lo with hi
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      const float other = __shfl_xor_sync(0xffffffffu, s, 1);
      if ((lane & 7) == 0) {
        const float lo = s, hi = other;
        const int step = k0 >> 6;
        // one float4 per row pair (m even, m odd, m even, m odd): the accumulator rows n and n + 8 start alike
        float* dst = s_corr + ((size_t)step * 4 + (m >> 1)) * 4 + (m & 1);
        const float nb = -(1024.0f * lo + 64.0f * hi);
        const float c = HAS_ZP ? nb : nb - 8.0f * (lo + hi);
        dst[0] = c;
        dst[2] = c;
        if (HAS_ZP) s_asum[(size_t)step * 8 + m] = lo + hi;
      }
    };
    if (MZ == 2) {
      for (int m = 0; m < M; ++m)
        for (int c0 = 0; c0 < chunks; c0 += 32) {
          const int k0 = slice_k0 + (c0 + lane) * 8;
          finish_row(m, k0, __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)m * K + k0)));
        }
    } else {
      // several rows: all rows' loads of a chunk first (one L2 round trip per chunk, not one per row)
      for (int c0 = 0; c0 < chunks; c0 += 32) {
        const int k0 = slice_k0 + (c0 + lane) * 8;
        uint4 v[8];
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (m < M) v[m] = __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)m * K + k0));
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (m < M) finish_row(m, k0, v[m]);
      }
    }
  }
  __syncwarp();

  constexpr uint32_t kLoMask = 0x000f000fu, kHiMask = 0x00f000f0u;
  constexpr uint32_t kLoMagic = 0x64006400u, kHiMagic = 0x54005400u;
  // rows >= M of the activation operand repeat row M - 1; their outputs are never stored
  const uint32_t a_base = smem_u32(s_a) + (uint32_t)(min(g, M - 1) * p.a_pitch + gb * (GS * 64) + t * 16) * 2u;
  const uint32_t c_base = smem_u32(s_corr) + (uint32_t)(gb * GS) * kCorrStep + (uint32_t)t * 16u;
  const uint32_t asum_base = smem_u32(s_asum) + (uint32_t)(gb * GS) * 32u;

  float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float ztot[MZ];  // zero-point terms of column (lane & 15), rows m, over the steps of half (lane >> 4)
#pragma unroll
  for (int m = 0; m < MZ; ++m) ztot[m] = 0.0f;

  uint32_t src = ring_addr;
  for (int tl = 0; tl < my_tiles; ++tl) {
    uint32_t a_addr = a_base, c_addr = c_base, as_addr = asum_base;
    for (int j2 = 0; j2 < myg; ++j2) {
      cp_async_wait<D - 1>();
      __syncwarp();  // the scales / zero points of the slot were copied by other lanes
      const uint32_t src_w = src + lane * 16;
      const uint32_t src_s = src + kSlotW + g * 2;
      if (HAS_ZP) {
        const uint32_t col = lane & 15, u0 = (lane >> 4) * (GS / 2);
#pragma unroll
        for (int uu = 0; uu < GS / 2; ++uu) {
          const uint32_t u = u0 + uu;
          const float s = lds_half_as_float<0>(src + kSlotW + u * 32 + col * 2);
          const float z = lds_u8_as_float(src + kSlotW + kSlotS + u * 16 + col);
          const float nsz = -s * z;
#pragma unroll
          for (int m = 0; m < MZ; m += 2) {
            if (m < M) {
              const float2 as = lds_f2(as_addr + u * 32 + m * 4);
              ztot[m] = fmaf(nsz, as.x, ztot[m]);
              ztot[m + 1] = fmaf(nsz, as.y, ztot[m + 1]);
            }
          }
        }
      }
#define BLKQ4_STREAM_STEP(U)                                                                    \
      {                                                                                         \
        const uint4 wv = lds_v4<(U) * 512>(src_w);                                              \
        const uint4 v0 = lds_v4<(U) * 128>(a_addr), v1 = lds_v4<(U) * 128 + 16>(a_addr);        \
        const float4 c = lds_f4<(U) * kCorrStep>(c_addr);                                       \
        const float sa = lds_half_as_float<(U) * 32>(src_s);                                    \
        const float sb = lds_half_as_float<(U) * 32 + 16>(src_s);                               \
        uint32_t lo_a[4], lo_b[4], hi_a[4], hi_b[4];                                            \
        const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};                                        \
        _Pragma("unroll") for (int r = 0; r < 4; ++r) {                                         \
          const uint32_t x = w4[r], y = x >> 8;                                                 \
          lo_a[r] = lop3_and_or(x, kLoMask, kLoMagic); /* (n;     k 2r, 2r+1)   1024 + q */     \
          hi_a[r] = lop3_and_or(x, kHiMask, kHiMagic); /* (n;     k 2r+8, 2r+9)   64 + q */     \
          lo_b[r] = lop3_and_or(y, kLoMask, kLoMagic); /* (n + 8; k 2r, 2r+1)            */     \
          hi_b[r] = lop3_and_or(y, kHiMask, kHiMagic); /* (n + 8; k 2r+8, 2r+9)          */     \
        }                                                                                       \
        float acc[4];                                                                           \
        mma_init(acc, lo_a[0], lo_b[0], lo_a[1], lo_b[1], v0.x, v0.y, c);                       \
        mma_acc(acc, lo_a[2], lo_b[2], lo_a[3], lo_b[3], v0.z, v0.w);                           \
        mma_acc(acc, hi_a[0], hi_b[0], hi_a[1], hi_b[1], v1.x, v1.y);                           \
        mma_acc(acc, hi_a[2], hi_b[2], hi_a[3], hi_b[3], v1.z, v1.w);                           \
        /* accumulator rows n (e = 0, 1) and n + 8 (e = 2, 3); columns m = 2 t + (e & 1) */     \
        total[0] = fmaf(sa, acc[0], total[0]);                                                  \
        total[1] = fmaf(sa, acc[1], total[1]);                                                  \
        total[2] = fmaf(sb, acc[2], total[2]);                                                  \
        total[3] = fmaf(sb, acc[3], total[3]);                                                  \
      }
      BLKQ4_STREAM_STEP(0)
      BLKQ4_STREAM_STEP(1)
      BLKQ4_STREAM_STEP(2)
      BLKQ4_STREAM_STEP(3)
#undef BLKQ4_STREAM_STEP
      issue_group(src);  // refill the slot just consumed
      src = (src == ring_last) ? ring_addr : src + kSlotBytes;
      a_addr += GS * 128;
      c_addr += GS * kCorrStep;
      as_addr += GS * 32;
    }
    // ---- tile end: double-buffered partial sums, one CTA barrier, one warp (rotating) adds them up.
    //      The adder of tile tl reaches the barrier of tile tl + 1 only after it has read the buffer,
    //      and nobody writes that buffer again before the barrier of tile tl + 1. ----
    float* buf = s_part + (size_t)(tl & 1) * (PW * 16 * MS);
    if (2 * t < M) {
      float* d0 = buf + ((size_t)warp * 16 + g) * MS + 2 * t;
      *reinterpret_cast<float2*>(d0) = make_float2(total[0], total[1]);
      *reinterpret_cast<float2*>(d0 + 8 * MS) = make_float2(total[2], total[3]);
    }
    total[0] = total[1] = total[2] = total[3] = 0.0f;
    if (HAS_ZP) {
#pragma unroll
      for (int m = 0; m < MZ; ++m) {
        if (m < MS) {
          const float z = ztot[m] + __shfl_xor_sync(0xffffffffu, ztot[m], 16);
          if (lane < 16) buf[((size_t)(W + warp) * 16 + lane) * MS + m] = z;
          ztot[m] = 0.0f;
        }
      }
    }
    __syncthreads();
    if (warp == tl % W) {
      const int tile = blockIdx.x + tl * gridDim.x;
      for (int idx = lane; idx < 16 * M; idx += 32) {
        const int row = idx & 15, m = idx >> 4;
        float sum = 0.0f;
#pragma unroll
        for (int w2 = 0; w2 < PW; ++w2) sum += buf[((size_t)w2 * 16 + row) * MS + m];
        const int n = tile * 16 + row;
        // bias joins the ROUNDED result in fp16, as a separate `output += bias` would
        const __half h = __float2half_rn(sum);
        if (GATHER) s_stage[idx] = h;  // [m][16]
        else p.out[(size_t)m * N + n] = p.bias ? __hadd(h, p.bias[n]) : h;
      }
      if (GATHER) {
        // this rank's 16 columns of row m as eight flagged words, into every rank's buffer
        __syncwarp();
        for (int w = lane; w < 8 * M; w += 32) {
          const int m = w >> 3, pair = w & 7;
          const uint32_t data = *reinterpret_cast<const uint32_t*>(s_stage + m * 16 + pair * 2);
          const size_t word = ((size_t)m * p.gt.n_total + (size_t)p.gt.rank * N + (size_t)tile * 16) / 2 + pair;
          for (int r = 0; r < p.gt.world; ++r) st_relaxed_sys_v2(p.gt.base[r] + gather_off + word * 8, data, gather_epoch);
        }
        __syncwarp();
      }
    }
  }
  cp_async_wait<0>();
  if (GATHER) {
    uint8_t* local = p.gt.base[p.gt.rank];
    // receiver: this CTA's share of the words of the complete result
    const unsigned long long nwords = (unsigned long long)M * p.gt.n_total / 2;
    const uint8_t* src = local + gather_off;
    uint32_t* dst = reinterpret_cast<uint32_t*>(p.out);
    bool expired = false;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < nwords;
         i += (unsigned long long)gridDim.x * blockDim.x) {
      uint2 w = ld_relaxed_sys_v2(src + i * 8);
      if (w.y != gather_epoch && !expired) {
        const long long t0 = clock64();
        while ((w = ld_relaxed_sys_v2(src + i * 8)).y != gather_epoch) {
          if (clock64() - t0 > kGatherWaitCycles) {
            // which rank's columns are missing: word i covers columns 2 (i % (n_total / 2)), + 1
            const int col = (int)(i % (unsigned long long)(p.gt.n_total / 2)) * 2;
            atomicCAS(reinterpret_cast<int*>(local + kGatherErrorOff), 0, 0x400 | (col / N));
            expired = true;  // this thread stops waiting for its other words too
            break;
          }
        }
      }
      if (w.y == gather_epoch) dst[i] = w.x;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned arrived = atomicAdd(reinterpret_cast<unsigned*>(local + kGatherDoneOff), 1u);
      if (arrived == gridDim.x - 1) {
        // last CTA of this rank: keep the two-kernel protocol's ticket numbering in step (its wait
        // kernel draws kGatherWaitCtas tickets per call) and advance the epoch
        *reinterpret_cast<volatile unsigned*>(local + kGatherDoneOff) = 0u;
        atomicAdd(reinterpret_cast<unsigned*>(local + kGatherTicketOff), (unsigned)kGatherWaitCtas);
        __threadfence();
        *reinterpret_cast<volatile unsigned*>(local + kGatherEpochOff) = gather_epoch;
      }
    }
  }
}

template <bool HAS_ZP, int D, int MZ, bool GATHER>
std::string launch_T(const StreamParams& p, size_t smem, int grid, cudaStream_t stream, bool early) {
  auto kern = gemv_stream_kernel<HAS_ZP, D, MZ, GATHER>;
  static std::atomic<int> granted[64];
  cudaError_t e = ensure_dynamic_smem(kern, smem, granted);
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  return std::string();
}

size_t stream_smem_bytes(int M, int K, bool has_zp, int D) {
  const int MS = (M + 1) & ~1, PW = has_zp ? 2 * kWarps : kWarps, steps = K / 64;
  return (size_t)kWarps * D * kSlotBytes + (size_t)steps * 64 + (has_zp ? (size_t)steps * 32 : 0) +
         (size_t)2 * PW * 16 * MS * 4 + 256 + (size_t)M * (K + 8) * 2;
}

}  // namespace

const char* const kStreamUnsupported = "unsupported by the stream kernel";

// Returns kStreamUnsupported when the shape is outside this kernel (the caller then takes another one).
std::string launch_gemv_stream(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                               const __half* a, const uint8_t* packed, const __half* scales,
                               const uint8_t* zp, __half* out, const __half* bias, unsigned flags,
                               const GatherTable* gt) {
  const int group_k = kGroupSteps * 64;
  if (!colwise || block < 64 || M < 1 || M > 8 || K % group_k != 0 || K / group_k < kWarps ||
      reinterpret_cast<uintptr_t>(scales) % 16 != 0 || (zp && reinterpret_cast<uintptr_t>(zp) % 16 != 0) ||
      (size_t)K * N / 2 >= ((size_t)1 << 40))
    return kStreamUnsupported;
  // Two CTAs per SM (this launch's and the next one's) share 227 KB; prefer four groups in flight per warp.
  constexpr size_t kHalfSm = (size_t)(227 * 1024) / 2 - 1024, kWholeSm = (size_t)227 * 1024;
  int D = 4;
  size_t smem = stream_smem_bytes(M, K, zp != nullptr, 4);
  if (smem > kHalfSm) {
    const size_t smem2 = stream_smem_bytes(M, K, zp != nullptr, 2);
    if (smem2 <= kHalfSm) { D = 2; smem = smem2; }
    else if (smem > kWholeSm) {
      if (smem2 > kWholeSm) return kStreamUnsupported;
      D = 2; smem = smem2;
    }
  }
  StreamParams p{};
  p.a = a; p.out = out; p.bias = bias; p.packed = packed; p.scales = scales; p.zp = zp;
  p.M = M; p.N = N; p.K = K;
  p.block_shift = block == 64 ? 6 : 7;
  p.tiles = N / 16;
  p.steps = K / 64;
  p.a_pitch = K + 8;
  if (gt) p.gt = *gt;
  const int sms = sm_count();
  // One CTA per SM leaves the second CTA slot of every SM to the next launch (its weights stream in
  // while this launch computes).  Two per SM double the warps that compute; worth it only when the
  // tiles then still divide evenly enough.
  int grid = p.tiles < sms ? p.tiles : sms;
  if (!gt && smem <= kHalfSm && p.tiles > sms) {  // gather mode: one CTA per SM, so that the whole grid is resident while it waits
    const int per2 = (p.tiles + 2 * sms - 1) / (2 * sms);
    const double eff2 = (double)p.tiles / (2.0 * sms) / per2;
    if (eff2 >= 0.85) grid = p.tiles < 2 * sms ? p.tiles : 2 * sms;
  }
  const bool early = (flags & BLKQ4_GEMM_EARLY_WEIGHT_FETCH) != 0;
  const bool small_m = M <= 2;
#define BLKQ4_STREAM_LAUNCH(G)                                                                                     \
  if (zp) {                                                                                                          \
    if (D == 4) return small_m ? launch_T<true, 4, 2, G>(p, smem, grid, stream, early) : launch_T<true, 4, 8, G>(p, smem, grid, stream, early); \
    return small_m ? launch_T<true, 2, 2, G>(p, smem, grid, stream, early) : launch_T<true, 2, 8, G>(p, smem, grid, stream, early); \
  }                                                                                                                  \
  if (D == 4) return small_m ? launch_T<false, 4, 2, G>(p, smem, grid, stream, early) : launch_T<false, 4, 8, G>(p, smem, grid, stream, early); \
  return small_m ? launch_T<false, 2, 2, G>(p, smem, grid, stream, early) : launch_T<false, 2, 8, G>(p, smem, grid, stream, early);
  if (gt) { BLKQ4_STREAM_LAUNCH(true) }
  BLKQ4_STREAM_LAUNCH(false)
#undef BLKQ4_STREAM_LAUNCH
}

}  // namespace blkq4
