// Skinny kernel for 9 <= M <= 16 rows, column-wise blocks of 64 or 128: the decode kernel's weight
// stream (blkq4_gemv_stream.cu: per-warp cp.async rings, fixed K slice per warp, mma.sync with the
// weights as the 16-row operand) with two 8-row groups of activations.
//
// What changes with more rows is where the activations live.  M x K activations no longer fit in
// shared memory next to the rings (16 x 8192 fp16 = 256 KB), so every warp reads the activation
// fragments of its K slice from global memory (they sit in L2), one 64-k step ahead of their use.
// Measured on B200 that traffic is not what bounds the kernel (pointing every fragment load at one
// address changes nothing); the warps' dependent instruction chains are, so the kernel keeps the
// decode kernel's shape of two resident CTAs per SM rather than fewer, fatter warps (a variant with
// two tiles per pass and 250 registers ran at half the speed).
// The arithmetic per weight is the decode kernel's (16 lop3 + 4 shifts per 64-k step and tile, bound
// by the logic pipe); the two extra mma.sync per step and row group ride on the idle tensor pipe, so
// M = 16 costs little more than M = 1 per weight byte.
//
// The activation-only terms of every step (and, with zero points, the plain sums) are computed once
// per CTA over all of K.  With zero points the accumulator of a step starts at
// -(1024 lo + 64 hi) - zp * (lo + hi) per (weight column, activation row): four fma per row group.
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

constexpr int MT = 2;   // 8-row groups of activations
constexpr int NT = 1;   // 16-column tiles per pass
constexpr int kPassSlot = NT * kSlotBytes;
constexpr int kCorrStepW = MT * 4 * 16;   // bytes of mma-initialising terms per step: 8 row pairs, float4 each
constexpr int kAsumStepW = MT * 8 * 4;    // bytes of plain activation sums per step (zero points)

struct WideParams {
  const __half* a;
  __half* out;
  const __half* bias;
  const uint8_t* packed;
  const __half* scales;
  const uint8_t* zp;
  int M, N, K;
  int block_shift;  // 6 or 7
  int pairs;        // N / 32: tile pairs
  int steps;        // K / 64
};

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Shared memory: rings [kWarps][D][NT][kSlotBytes] | s_corr [steps][8] float4 | s_asum [steps][16] (zero points)
//                | s_part [kWarps][NT][16][16]
template <bool HAS_ZP, int D>
__global__ void __launch_bounds__(kWarps * 32, 2)
gemv_wide_kernel(const WideParams p) {
  extern __shared__ __align__(16) uint8_t s_raw[];
  constexpr int W = kWarps, GS = kGroupSteps;
  uint8_t* s_ring = s_raw;
  float* s_corr = reinterpret_cast<float*>(s_ring + W * D * kPassSlot);
  float* s_asum = s_corr + (size_t)p.steps * (kCorrStepW / 4);
  float* s_part = s_asum + (HAS_ZP ? (size_t)p.steps * (kAsumStepW / 4) : 0);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = p.K, N = p.N, M = p.M;
  const int bs = p.block_shift - 6;
  const int kgroups = p.steps / GS;
  const int gb = (int)(((long long)kgroups * warp) / W);
  const int myg = (int)(((long long)kgroups * (warp + 1)) / W) - gb;  // >= 1
  const int my_passes = (p.pairs - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const uint32_t ring_addr = smem_u32(s_ring) + (uint32_t)warp * (D * kPassSlot);
  const uint32_t ring_last = ring_addr + (D - 1) * kPassSlot;

  asm volatile("griddepcontrol.launch_dependents;");

  // ---- loader: D groups ahead; a group carries the warp's four steps of BOTH tiles of the pass ----
  const uint8_t* wp = p.packed + (size_t)(blockIdx.x * (NT * 8) + g) * K + (size_t)gb * (GS * 64) + t * 16;
  const long long w_pass_adj = (long long)gridDim.x * (NT * 8) * K - (long long)myg * (GS * 64);
  const size_t w_tile = (size_t)8 * K;  // from a tile's packed columns to the next tile's
  // lanes 0 .. 8 NT - 1: scales of (tile lane / 8, step (lane % 8) / 2, column half lane % 2); the next 4 NT lanes:
  // zero points of (tile, step)
  const uint32_t meta_lane = (lane < 8 * NT || (HAS_ZP && lane < 12 * NT)) ? 1u : 0u;
  const uint8_t* mp;
  uint32_t m_dst;
  long long m_step, m_pass_adj;
  {
    const int rows_per_group = GS >> bs;
    if (lane < 8 * NT) {
      const int i = lane >> 3, u = (lane & 7) >> 1, h = lane & 1;
      mp = reinterpret_cast<const uint8_t*>(p.scales) +
           ((size_t)((gb * GS + u) >> bs) * N + (blockIdx.x * NT + i) * 16 + h * 8) * 2;
      m_dst = i * kSlotBytes + kSlotW + u * 32 + h * 16;
      m_step = (long long)rows_per_group * N * 2;
      m_pass_adj = (long long)gridDim.x * (NT * 32) - (long long)myg * m_step;
    } else {
      const int i = ((lane - 8 * NT) >> 2) % NT, u = (lane - 8 * NT) & 3;
      mp = (HAS_ZP ? p.zp : p.packed) + (size_t)((gb * GS + u) >> bs) * N + (blockIdx.x * NT + i) * 16;
      m_dst = i * kSlotBytes + kSlotW + kSlotS + u * 16;
      m_step = (long long)rows_per_group * N;
      m_pass_adj = (long long)gridDim.x * (NT * 16) - (long long)myg * m_step;
    }
  }
  int ld_left = my_passes * myg, ld_j = 0;
  auto issue_group = [&](uint32_t dst) {
    const uint32_t go = ld_left > 0 ? 1u : 0u;
    const uint32_t dw = dst + lane * 16;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const uint8_t* wt = wp + i * w_tile;
      cp_async16_if<0>(dw + i * kSlotBytes, wt, go);
      cp_async16_if<64>(dw + i * kSlotBytes, wt, go);
      cp_async16_if<128>(dw + i * kSlotBytes, wt, go);
      cp_async16_if<192>(dw + i * kSlotBytes, wt, go);
    }
    cp_async16_if<0>(dst + m_dst, mp, go & meta_lane);
    cp_async_commit();
    --ld_left;
    const bool wrap = ++ld_j == myg;
    wp += (GS * 64) + (wrap ? w_pass_adj : 0);
    mp += m_step + (wrap ? m_pass_adj : 0);
    if (wrap) ld_j = 0;
  };
  {
    uint32_t dst = ring_addr;
#pragma unroll
    for (int d = 0; d < D; ++d) {
      issue_group(dst);
      dst += kPassSlot;
    }
  }

  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- once per CTA: the activation-only terms of every (step, row); four threads per pair.  The
  //      loads of four rounds are issued before any is used: a round is one L2 round trip. ----
  {
    constexpr int UNR = 4;
    const int total = p.steps * M * 4;
    for (int base = 0; base < total; base += W * 32 * UNR) {
      uint4 x0[UNR], x1[UNR];
#pragma unroll
      for (int r = 0; r < UNR; ++r) {
        const int idx = base + r * (W * 32) + (int)threadIdx.x;
        x0[r] = x1[r] = make_uint4(0, 0, 0, 0);
        if (idx < total) {
          const int pair = idx >> 2, j = idx & 3;
          const int m = pair % M, step = pair / M;
          const uint4* ap = reinterpret_cast<const uint4*>(p.a + (size_t)m * K + step * 64 + j * 16);
          x0[r] = __ldg(ap);
          x1[r] = __ldg(ap + 1);
        }
      }
#pragma unroll
      for (int r = 0; r < UNR; ++r) {
        const int idx = base + r * (W * 32) + (int)threadIdx.x;
        const int pair = idx >> 2, j = idx & 3;
        const int m = pair % M, step = pair / M;
        float lo = 0.0f, hi = 0.0f;
        const __half2* h0 = reinterpret_cast<const __half2*>(&x0[r]);
        const __half2* h1 = reinterpret_cast<const __half2*>(&x1[r]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f0 = __half22float2(h0[e]), f1 = __half22float2(h1[e]);
          lo += f0.x + f0.y;
          hi += f1.x + f1.y;
        }
        lo += __shfl_xor_sync(0xffffffffu, lo, 1);
        hi += __shfl_xor_sync(0xffffffffu, hi, 1);
        lo += __shfl_xor_sync(0xffffffffu, lo, 2);
        hi += __shfl_xor_sync(0xffffffffu, hi, 2);
        if (idx < total && j == 0) {
          float* dst = s_corr + ((size_t)step * (MT * 4) + (m >> 1)) * 4 + (m & 1);
          const float nb = -(1024.0f * lo + 64.0f * hi);
          const float c = HAS_ZP ? nb : nb - 8.0f * (lo + hi);
          dst[0] = c;
          dst[2] = c;
          if (HAS_ZP) s_asum[(size_t)step * (MT * 8) + m] = lo + hi;
        }
      }
    }
  }
  __syncthreads();

  constexpr uint32_t kLoMask = 0x000f000fu, kHiMask = 0x00f000f0u;
  constexpr uint32_t kLoMagic = 0x64006400u, kHiMagic = 0x54005400u;
  // activation fragments of this lane: rows g and g + 8 (rows >= M repeat row M - 1), 32 bytes per step
  const __half* a_row[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) a_row[j] = p.a + (size_t)min(g + 8 * j, M - 1) * K + (size_t)gb * (GS * 64) + t * 16;
  const uint32_t c_base = smem_u32(s_corr) + (uint32_t)(gb * GS) * kCorrStepW + (uint32_t)t * 16u;
  const uint32_t as_base = smem_u32(s_asum) + (uint32_t)(gb * GS) * kAsumStepW + (uint32_t)t * 8u;

  float total[NT][MT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) total[i][j][e] = 0.0f;

  uint32_t src = ring_addr;
  for (int ps = 0; ps < my_passes; ++ps) {
    uint32_t c_addr = c_base, as_addr = as_base;
    const __half* ap[MT] = {a_row[0], a_row[1]};
    // activation fragments: one step ahead of their use
    uint4 nv0[MT], nv1[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      nv0[j] = ldg_nc_v4(ap[j]);
      nv1[j] = ldg_nc_v4(ap[j] + 8);
    }
    for (int j2 = 0; j2 < myg; ++j2) {
      cp_async_wait<D - 1>();
      __syncwarp();
      const uint32_t src_w = src + lane * 16;
      const uint32_t src_s = src + kSlotW + g * 2;
      const uint32_t src_z = src + kSlotW + kSlotS + g;
#define BLKQ4_WIDE_STEP(U)                                                                               \
      {                                                                                                  \
        uint4 v0[MT], v1[MT];                                                                            \
        _Pragma("unroll") for (int j = 0; j < MT; ++j) { v0[j] = nv0[j]; v1[j] = nv1[j]; }               \
        /* the next step's fragments (the last step of the pass re-reads its own: harmless) */           \
        {                                                                                                \
          const bool more = (U) < GS - 1 || j2 + 1 < myg;                                                \
          const int adv = more ? ((U) + 1) * 64 : (U) * 64;                                              \
          _Pragma("unroll") for (int j = 0; j < MT; ++j) {                                               \
            nv0[j] = ldg_nc_v4(ap[j] + adv);                                                             \
            nv1[j] = ldg_nc_v4(ap[j] + adv + 8);                                                         \
          }                                                                                              \
        }                                                                                                \
        float4 c[MT];                                                                                    \
        float2 as[MT];                                                                                   \
        _Pragma("unroll") for (int j = 0; j < MT; ++j) {                                                 \
          c[j] = lds_f4<(U) * kCorrStepW>(c_addr + j * 64);                                              \
          if (HAS_ZP) as[j] = lds_f2(as_addr + (U) * kAsumStepW + j * 32);                               \
        }                                                                                                \
        _Pragma("unroll") for (int i = 0; i < NT; ++i) {                                                 \
          const uint4 wv = lds_v4<(U) * 512>(src_w + i * kSlotBytes);                                    \
          const float sa = lds_half_as_float<(U) * 32>(src_s + i * kSlotBytes);                          \
          const float sb = lds_half_as_float<(U) * 32 + 16>(src_s + i * kSlotBytes);                     \
          float za = 0.0f, zb = 0.0f;                                                                    \
          if (HAS_ZP) {                                                                                  \
            za = lds_u8_as_float(src_z + i * kSlotBytes + (U) * 16);                                     \
            zb = lds_u8_as_float(src_z + i * kSlotBytes + (U) * 16 + 8);                                 \
          }                                                                                              \
          uint32_t lo_a[4], lo_b[4], hi_a[4], hi_b[4];                                                   \
          const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};                                               \
          _Pragma("unroll") for (int r = 0; r < 4; ++r) {                                                \
            const uint32_t x = w4[r], y = x >> 8;                                                        \
            lo_a[r] = lop3_and_or(x, kLoMask, kLoMagic);                                                 \
            hi_a[r] = lop3_and_or(x, kHiMask, kHiMagic);                                                 \
            lo_b[r] = lop3_and_or(y, kLoMask, kLoMagic);                                                 \
            hi_b[r] = lop3_and_or(y, kHiMask, kHiMagic);                                                 \
          }                                                                                              \
          _Pragma("unroll") for (int j = 0; j < MT; ++j) {                                               \
            float4 ci = c[j];                                                                            \
            if (HAS_ZP) {                                                                                \
              ci.x = fmaf(-za, as[j].x, ci.x);                                                           \
              ci.y = fmaf(-za, as[j].y, ci.y);                                                           \
              ci.z = fmaf(-zb, as[j].x, ci.z);                                                           \
              ci.w = fmaf(-zb, as[j].y, ci.w);                                                           \
            }                                                                                            \
            float acc[4];                                                                                \
            mma_init(acc, lo_a[0], lo_b[0], lo_a[1], lo_b[1], v0[j].x, v0[j].y, ci);                     \
            mma_acc(acc, lo_a[2], lo_b[2], lo_a[3], lo_b[3], v0[j].z, v0[j].w);                          \
            mma_acc(acc, hi_a[0], hi_b[0], hi_a[1], hi_b[1], v1[j].x, v1[j].y);                          \
            mma_acc(acc, hi_a[2], hi_b[2], hi_a[3], hi_b[3], v1[j].z, v1[j].w);                          \
            total[i][j][0] = fmaf(sa, acc[0], total[i][j][0]);                                           \
            total[i][j][1] = fmaf(sa, acc[1], total[i][j][1]);                                           \
            total[i][j][2] = fmaf(sb, acc[2], total[i][j][2]);                                           \
            total[i][j][3] = fmaf(sb, acc[3], total[i][j][3]);                                           \
          }                                                                                              \
        }                                                                                                \
      }
      BLKQ4_WIDE_STEP(0)
      BLKQ4_WIDE_STEP(1)
      BLKQ4_WIDE_STEP(2)
      BLKQ4_WIDE_STEP(3)
#undef BLKQ4_WIDE_STEP
      issue_group(src);
      src = (src == ring_last) ? ring_addr : src + kPassSlot;
      c_addr += GS * kCorrStepW;
      as_addr += GS * kAsumStepW;
#pragma unroll
      for (int j = 0; j < MT; ++j) ap[j] += GS * 64;
    }
    // ---- pass end: partial sums -> shared memory, barrier, every warp adds up a share, barrier ----
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        float* d0 = s_part + (((size_t)warp * NT + i) * 16 + g) * 16 + 8 * j + 2 * t;
        *reinterpret_cast<float2*>(d0) = make_float2(total[i][j][0], total[i][j][1]);
        *reinterpret_cast<float2*>(d0 + 8 * 16) = make_float2(total[i][j][2], total[i][j][3]);
#pragma unroll
        for (int e = 0; e < 4; ++e) total[i][j][e] = 0.0f;
      }
    __syncthreads();
    {
      const int pair = blockIdx.x + ps * gridDim.x;
      // NT * 16 columns x M rows of outputs, spread over the CTA's threads
      for (int idx = threadIdx.x; idx < NT * 16 * M; idx += W * 32) {
        const int col = idx % (NT * 16), m = idx / (NT * 16);
        const int i = col >> 4, row = col & 15;
        float sum = 0.0f;
#pragma unroll
        for (int w2 = 0; w2 < W; ++w2) sum += s_part[(((size_t)w2 * NT + i) * 16 + row) * 16 + m];
        const int n = pair * (NT * 16) + col;
        const __half h = __float2half_rn(sum);
        p.out[(size_t)m * N + n] = p.bias ? __hadd(h, p.bias[n]) : h;
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
}

template <bool HAS_ZP, int D>
std::string launch_T(const WideParams& p, size_t smem, int grid, cudaStream_t stream, bool early) {
  auto kern = gemv_wide_kernel<HAS_ZP, D>;
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

}  // namespace

// 9 <= M <= 16, column-wise blocks >= 64, K a multiple of 256 and >= 2048, N a multiple of 32.
// Returns kStreamUnsupported for other shapes.
std::string launch_gemv_wide(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                             const __half* a, const uint8_t* packed, const __half* scales,
                             const uint8_t* zp, __half* out, const __half* bias, unsigned flags) {
  const int group_k = kGroupSteps * 64;
  // Long K only: every CTA first reduces the whole activation matrix to its per-step correction
  // terms, and that prologue pays off over many tiles of long columns.  Measured on B200 against the
  // generic skinny kernel: K = 8192, N = 28672 symmetric, M = 16: 73 vs 79 us, M = 9: 60 vs 72 us;
  // K = 4096, N = 11008 with zero points, M = 16: 25 vs 21 us; K = 8192, N = 14336 (a half-width shard,
  // three tiles per CTA), M = 16: 56 vs 46 us.  So: long K and at least four tiles per resident CTA;
  // everything else stays on the TMA kernel.
  if (K < 8192 || N / (16 * NT) < 8 * sm_count()) return kStreamUnsupported;
  if (!colwise || block < 64 || M < 9 || M > 16 || K % group_k != 0 || K / group_k < kWarps || N % (16 * NT) != 0 ||
      reinterpret_cast<uintptr_t>(scales) % 16 != 0 || (zp && reinterpret_cast<uintptr_t>(zp) % 16 != 0))
    return kStreamUnsupported;
  const int steps = K / 64;
  auto smem_for = [&](int D) {
    return (size_t)kWarps * D * kPassSlot + (size_t)steps * kCorrStepW + (zp ? (size_t)steps * kAsumStepW : 0) +
           (size_t)kWarps * NT * 16 * 16 * 4;
  };
  // two CTAs per SM (both of this launch when the passes divide well, else this one's and the next one's)
  constexpr size_t kHalfSm = (size_t)(227 * 1024) / 2 - 1024;
  int D = 4;
  size_t smem = smem_for(4);
  if (smem > kHalfSm) {
    D = 2;
    smem = smem_for(2);
    if (smem > (size_t)227 * 1024) return kStreamUnsupported;
  }
  WideParams p{};
  p.a = a; p.out = out; p.bias = bias; p.packed = packed; p.scales = scales; p.zp = zp;
  p.M = M; p.N = N; p.K = K;
  p.block_shift = block == 64 ? 6 : 7;
  p.pairs = N / (16 * NT);
  p.steps = steps;
  const int sms = sm_count();
  int grid = p.pairs < sms ? p.pairs : sms;
  if (smem <= kHalfSm && p.pairs > sms) {
    const int per2 = (p.pairs + 2 * sms - 1) / (2 * sms);
    if ((double)p.pairs / (2.0 * sms) / per2 >= 0.85) grid = p.pairs < 2 * sms ? p.pairs : 2 * sms;
  }
  const bool early = (flags & BLKQ4_GEMM_EARLY_WEIGHT_FETCH) != 0;
  if (zp) return D == 4 ? launch_T<true, 4>(p, smem, grid, stream, early) : launch_T<true, 2>(p, smem, grid, stream, early);
  return D == 4 ? launch_T<false, 4>(p, smem, grid, stream, early) : launch_T<false, 2>(p, smem, grid, stream, early);
}

}  // namespace blkq4
