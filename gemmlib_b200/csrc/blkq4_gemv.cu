// Skinny W4A16 kernels (M <= 16) for sm_100a: out[M,N] = A[M,K] x dequant(W4[K,N]).
// This file holds the dispatch (launch_gemv: decode kernel -> wide kernel, both in files of their
// own, -> the TMA kernel and the generic kernel below) and the two kernels that take every shape
// the first two refuse.
//
// This regime is bound by HBM bandwidth: every packed weight byte is read once
// and used for at most 16 outputs, so the kernel is organised around the weight
// stream, not the tensor pipe.
//
//   * 128-bit loads.  A packed column np (weight columns n0 = 16*(np/8) + np%8
//     and n0 + 8) is K contiguous bytes; a lane loads 16 bytes = 16 k x 2 n.
//     The four lanes of a quad take four consecutive 16-byte chunks, the eight
//     quads of a warp take the eight packed columns of one 16-column tile.
//   * The 16 x 16 (n x k) product step uses mma.sync.m16n8k16 with the weights
//     as the 16-row operand and the activations as the 8-column operand.  One
//     32-bit word of the packed layout dequantizes (two shifts, four lop3, four
//     fp16 fma) into exactly one lane's A-fragment, so no data moves between
//     lanes.  Each mma reduces over the k held by the four lanes of a quad; the
//     k order inside an mma is permuted consistently for weights and activations.
//   * Split-K: the warps of a CTA take disjoint K ranges of the same columns and
//     combine their fp32 partial sums through shared memory.  No global scratch.
//
// Dequantization numerics are the reference kernel's: fp16(16 + q) by bit trick,
// then fma.rn.f16(scale, 16 + q, rn(scale * (-16 - zp))); reference
// src/mickey/cutlass_ext/q4gemm/warp/quantb_meta_mma_tensor_op_tile_iterator.h:69-104
// and :436-543.  Accumulation is fp32, output one rounding to fp16.
#include <cstddef>
#include <cstdint>
#include <cstdlib>

#include "blkq4_common.cuh"
#include "ms_blkq4gemm.h"
#include "blkq4_tma.cuh"

namespace blkq4 {
namespace {

__device__ __forceinline__ void mma_m16n8k16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Raw scales / zero points of one 16-k chunk of two weight columns (na, na + 8), fetched
// together with the chunk and expanded to half2 operands only when it is consumed.
template <bool COLWISE>
struct MetaRegs;

// Column-wise blocks: meta row-major [K/block, N]; the 16 k of a chunk share one block.
template <>
struct MetaRegs<true> {
  uint32_t s;  // scale(na) | scale(na + 8) << 16
  uint32_t z;  // zp(na) | zp(na + 8) << 8
  __device__ __forceinline__ void load(const __half* __restrict__ scales, const uint8_t* __restrict__ zps,
                                       int chunk, int na, int N, int K, int block) {
    const size_t mi = (size_t)((chunk * 16) / block) * N + na;
    const unsigned short* sp = reinterpret_cast<const unsigned short*>(scales) + mi;
    s = (uint32_t)__ldg(sp) | ((uint32_t)__ldg(sp + 8) << 16);
    z = zps ? ((uint32_t)__ldg(zps + mi) | ((uint32_t)__ldg(zps + mi + 8) << 8)) : 0x0808u;
  }
  __device__ __forceinline__ void expand(uint32_t (&s_lo_a)[4], uint32_t (&s_hi_a)[4], uint32_t (&o_lo_a)[4],
                                         uint32_t (&o_hi_a)[4], uint32_t (&s_lo_b)[4], uint32_t (&s_hi_b)[4],
                                         uint32_t (&o_lo_b)[4], uint32_t (&o_hi_b)[4]) const {
    const __half sa = __ushort_as_half((unsigned short)(s & 0xffffu));
    const __half sb = __ushort_as_half((unsigned short)(s >> 16));
    const __half oa = dequant_offset(sa, (int)(z & 0xffu)), ob = dequant_offset(sb, (int)(z >> 8));
    const uint32_t sa2 = pack_half2(sa, sa), sb2 = pack_half2(sb, sb);
    const uint32_t oa2 = pack_half2(oa, oa), ob2 = pack_half2(ob, ob);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      s_lo_a[r] = s_hi_a[r] = sa2;
      o_lo_a[r] = o_hi_a[r] = oa2;
      s_lo_b[r] = s_hi_b[r] = sb2;
      o_lo_b[r] = o_hi_b[r] = ob2;
    }
  }
};

// Row-wise blocks: meta column-major [K, N/block], 16-row groups permuted so that positions
// 4r..4r+3 hold k = 2r, 2r+1, 2r+8, 2r+9 (scales) and 2r, 2r+8, 2r+1, 2r+9 (zero points).
// Columns na and na + 8 share a block.
template <>
struct MetaRegs<false> {
  uint4 s0, s1, zv;
  __device__ __forceinline__ void load(const __half* __restrict__ scales, const uint8_t* __restrict__ zps,
                                       int chunk, int na, int N, int K, int block) {
    const size_t mi = (size_t)(na / block) * K + (size_t)chunk * 16;
    const uint4* sp = reinterpret_cast<const uint4*>(scales + mi);
    s0 = __ldg(sp);
    s1 = __ldg(sp + 1);
    zv = zps ? __ldg(reinterpret_cast<const uint4*>(zps + mi))
             : make_uint4(0x08080808u, 0x08080808u, 0x08080808u, 0x08080808u);
  }
  __device__ __forceinline__ void expand(uint32_t (&s_lo_a)[4], uint32_t (&s_hi_a)[4], uint32_t (&o_lo_a)[4],
                                         uint32_t (&o_hi_a)[4], uint32_t (&s_lo_b)[4], uint32_t (&s_hi_b)[4],
                                         uint32_t (&o_lo_b)[4], uint32_t (&o_hi_b)[4]) const {
    const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      s_lo_a[r] = s_lo_b[r] = sw[2 * r];
      s_hi_a[r] = s_hi_b[r] = sw[2 * r + 1];
      // fp16(-16 - z) by the same bit trick as the weights: 0xcc00 is -16.0
      const uint32_t nz_lo = ((zw[r] << 6) & 0x03c003c0u) | 0xcc00cc00u;
      const uint32_t nz_hi = ((zw[r] >> 2) & 0x03c003c0u) | 0xcc00cc00u;
      o_lo_a[r] = o_lo_b[r] = hmul2_u32(sw[2 * r], nz_lo);
      o_hi_a[r] = o_hi_b[r] = hmul2_u32(sw[2 * r + 1], nz_hi);
    }
  }
};

constexpr int kMaxWarps = 16;

// NT: 16-column tiles per warp.  MT: 8-row groups of activations (1: M <= 8, 2: M <= 16).
// U:  64-k steps loaded together; U * NT 16-byte weight loads are in flight per lane.
template <int NT, int MT, int U, bool COLWISE>
__global__ void __launch_bounds__(kMaxWarps * 32)
gemv_kernel(const __half* __restrict__ a, const uint8_t* __restrict__ packed,
            const __half* __restrict__ scales, const uint8_t* __restrict__ zps,
            __half* __restrict__ out, const __half* __restrict__ bias, int M, int N, int K, int block) {
  extern __shared__ float s_red[];  // [warps][NT*MT*4][32]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile0 = blockIdx.x * NT;
  const int ntiles = N >> 4;

  // This warp's K range, in steps of 64.
  const int total_steps = K >> 6;
  const int step_beg = (int)(((long long)total_steps * warp) / nwarps);
  const int step_end = (int)(((long long)total_steps * (warp + 1)) / nwarps);

  float acc[NT][MT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;

  const uint8_t* wcol[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int tile = min(tile0 + i, ntiles - 1);  // clamp: duplicates are discarded at the end
    wcol[i] = packed + (size_t)(tile * 8 + g) * K;
  }

  // Two register buffers of U * NT weight chunks with their scales / zero points; the
  // next group is requested before the current one is consumed, so that neither the
  // weight stream nor the (also HBM-resident) meta stream stalls the math.  (Two named
  // buffers, not one indexed by a runtime value, so that they stay in registers.)
  struct Group {
    uint4 w[U][NT];
    MetaRegs<COLWISE> m[U][NT];
  };
  Group grp_a, grp_b;
  auto load_group = [&](Group& gr, int step0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int step = min(step0 + u, step_end - 1);
      const int chunk = step * 4 + t;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        gr.w[u][i] = ldg_stream_v4(wcol[i] + (size_t)chunk * 16);
        const int tile = min(tile0 + i, ntiles - 1);
        gr.m[u][i].load(scales, zps, chunk, tile * 16 + g, N, K, block);
      }
    }
  };

  auto compute_group = [&](const Group& gr, int step0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int step = step0 + u;
      if (step >= step_end) break;
      const int chunk = step * 4 + t;  // this lane's 16 k: [16 chunk, 16 chunk + 16)

      // Activations: 16 halves of row g (and g + 8); rows >= M are zero.
      uint4 av[MT][2];
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        const int row = g + 8 * j;
        if (row < M) {
          const uint4* p = reinterpret_cast<const uint4*>(a + (size_t)row * K + chunk * 16);
          av[j][0] = __ldg(p);
          av[j][1] = __ldg(p + 1);
        } else {
          av[j][0] = make_uint4(0, 0, 0, 0);
          av[j][1] = make_uint4(0, 0, 0, 0);
        }
      }

#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int tile = min(tile0 + i, ntiles - 1);
        const int na = tile * 16 + g;
        const uint32_t w4[4] = {gr.w[u][i].x, gr.w[u][i].y, gr.w[u][i].z, gr.w[u][i].w};

        // Per word r: scale/offset half2 for the k pairs (2r, 2r+1) [lo] and
        // (2r+8, 2r+9) [hi], for column na (a) and na + 8 (b).
        uint32_t s_lo_a[4], s_hi_a[4], o_lo_a[4], o_hi_a[4];
        uint32_t s_lo_b[4], s_hi_b[4], o_lo_b[4], o_hi_b[4];
        gr.m[u][i].expand(s_lo_a, s_hi_a, o_lo_a, o_hi_a, s_lo_b, s_hi_b, o_lo_b, o_hi_b);

#pragma unroll
        for (int r = 0; r < 4; ++r) {
          uint32_t h[4];
          word_to_half16plus(w4[r], h);
          const uint32_t d0 = hfma2_u32(s_lo_a[r], h[0], o_lo_a[r]);  // (na;   2r, 2r+1)
          const uint32_t d1 = hfma2_u32(s_hi_a[r], h[1], o_hi_a[r]);  // (na;   2r+8, 2r+9)
          const uint32_t d2 = hfma2_u32(s_lo_b[r], h[2], o_lo_b[r]);  // (na+8; 2r, 2r+1)
          const uint32_t d3 = hfma2_u32(s_hi_b[r], h[3], o_hi_b[r]);  // (na+8; 2r+8, 2r+9)
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            const uint32_t b_lo[4] = {av[j][0].x, av[j][0].y, av[j][0].z, av[j][0].w};
            const uint32_t b_hi[4] = {av[j][1].x, av[j][1].y, av[j][1].z, av[j][1].w};
            mma_m16n8k16(acc[i][j], d0, d2, d1, d3, b_lo[r], b_hi[r]);
          }
        }
      }
    }
  };

  if (step_beg < step_end) load_group(grp_a, step_beg);
  for (int step0 = step_beg; step0 < step_end; step0 += 2 * U) {
    if (step0 + U < step_end) load_group(grp_b, step0 + U);
    compute_group(grp_a, step0);
    if (step0 + 2 * U < step_end) load_group(grp_a, step0 + 2 * U);
    if (step0 + U < step_end) compute_group(grp_b, step0 + U);
  }

  // ---- combine the warps' partial sums and write fp16 ----
  constexpr int VALS = NT * MT * 4;
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        s_red[(warp * VALS + (i * MT + j) * 4 + e) * 32 + lane] = acc[i][j][e];
  __syncthreads();
  for (int idx = threadIdx.x; idx < VALS * 32; idx += blockDim.x) {
    const int l = idx & 31, v = idx >> 5;
    const int e = v & 3, j = (v >> 2) % MT, i = (v >> 2) / MT;
    float sum = 0.0f;
    for (int w = 0; w < nwarps; ++w) sum += s_red[(w * VALS + v) * 32 + l];
    // accumulator element e of lane l: row (n) = l/4 + 8*(e>>1), column (m) = 2*(l%4) + (e&1)
    const int tile = tile0 + i;
    const int n = tile * 16 + (l >> 2) + 8 * (e >> 1);
    const int m = 8 * j + 2 * (l & 3) + (e & 1);
    if (tile < ntiles && m < M) {
      // bias joins the ROUNDED result in fp16, as a separate `output += bias` would
      const __half h = __float2half_rn(sum);
      out[(size_t)m * N + n] = bias ? __hadd(h, bias[n]) : h;
    }
  }
}


// ------------------------------------------------------------------------------------------
// Fast path: column-wise blocks of 64 or 128 (every 64-k step of a column has ONE scale).
//
// Memory side.  Persistent CTAs (one per SM) walk a static list of 16-column tiles.  A
// producer warp streams the packed weights through a ring of shared-memory slots with TMA
// (cp.async.bulk.tensor): one unit = 8 packed columns x 512 bytes (kUnitSteps = 8 steps of
// 64 k, 4 KB) plus the unit's scales / zero points, completing on the slot's "full" mbarrier.
// The ring (kRing = 32 slots) bounds the bytes in flight per SM (140 KB: enough to cover HBM
// latency) - measured on B200, asking for a whole launch's bytes up front makes every later
// small load (activations, scales) queue behind them for microseconds.  kCons = 16 consumer
// warps take units round-robin,
// release slots through "empty" mbarriers, and leave their partial sums of a tile in shared
// memory; the warp that completes a tile adds them in a fixed order, converts and stores.
//
// Math side.  Scaling is moved out of the per-weight work.  A packed word x gives, with one
// shift and four lop3, the half2 operands
//     (x      & 0x000f000f) | 0x64006400  =  1024 + q     (k pair 2r, 2r+1   of n0)
//     (x      & 0x00f000f0) | 0x54005400  =    64 + q     (k pair 2r+8, 2r+9 of n0)
//     (x >> 8 & ...)                         the same for n0 + 8
// (0x6400 = fp16 1024 with mantissa step 1; 0x5400 = fp16 64 with mantissa step 1/16, so a
// nibble at bits 4-7 also adds q).  Four mma per 64-k step accumulate, exactly as far as
// fp32 goes,  acc = sum_k a_k q_k + 1024 sum_lo a_k + 64 sum_hi a_k  ("lo": k % 16 < 8).
// The activation-only terms are computed once per CTA and step (shared memory) and removed,
// with the zero-point term zp * sum_k a_k, when the step's partial sum is scaled:
//     total += scale * (acc - bias - zp * asum).
// More accurate than dequantizing to fp16 first (no fp16 rounding of scale * q), equal to it
// where both are exact.  On B200 one mma.sync costs about 8 issue cycles of its scheduler, so
// the step is kept at four of them.
__device__ int g_gemv_error = 0;

constexpr int kUnitSteps = 8;                       // 64-k steps per unit
constexpr int kUnitKBytes = kUnitSteps * 64;        // 512 bytes of each packed column
constexpr int kUnitWBytes = 8 * kUnitKBytes;        // 4 KB of weights: one TMA box of 8 x 128 uint32
constexpr int kSlotScaleOff = kUnitWBytes;          // [rows <= 8][16] fp16
constexpr int kSlotZpOff = kUnitWBytes + 256;       // [rows <= 8][16] u8
constexpr int kSlotBytes = kUnitWBytes + 384;       // 4480, a multiple of 128
constexpr int kRing = 32;                           // slots: 140 KB in flight per SM
constexpr int kCons = 16;                           // consumer warps
// Parity waits on an mbarrier are only valid one phase at a time, so every slot must be
// produced by one thread (lane = slot) and consumed by one warp (slot % kCons).
static_assert(kRing <= 32 && kRing % kCons == 0, "slot ownership");
constexpr int kAccBufsMax = 4;                      // rotating per-tile sets of per-warp partial sums
constexpr int kPersistThreads = (kCons + 1) * 32;
constexpr int kCtrlBytes = 1024;                    // barriers + flags + counters
constexpr long long kGemvWaitCycles = 2000000000ll;

struct PersistParams {
  const __half* a;
  __half* out;
  const __half* bias;  // fp16 [N] added to the fp16 result, or null
  GatherTable gt;      // gt.world > 0: the result goes to every rank's gathered buffer instead of `out`
  int M, N, K;
  int block_shift;   // 6 or 7
  int tiles;         // N / 16
  int nsub;          // units per tile = K / 256
  int ring;          // slots actually used (<= kRing)
  int a_smem;        // activations staged in shared memory (M * K * 2 <= 32 KB, M <= 2)
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t bits) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(d) : "r"(x), "r"(mask), "r"(bits));  // (x & mask) | bits
  return d;
}
// D = A x B (+ 0): starts an accumulator without a separate clear.
__device__ __forceinline__ void mma_m16n8k16_init(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                  uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

template <int MT, bool HAS_ZP>
__global__ void __launch_bounds__(kPersistThreads, 1)
gemv_persistent_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_s,
                       const __grid_constant__ CUtensorMap tm_z, const PersistParams p) {
  extern __shared__ __align__(128) uint8_t s_raw[];
  constexpr int MR = 8 * MT;          // activation rows the mma sees (rows >= M repeat row M-1)
  constexpr int CW = HAS_ZP ? 2 : 1;  // correction floats per (step, row)
  constexpr int VALS = MT * 4;
  constexpr int kAccBufs = MT == 1 ? kAccBufsMax : 2;  // 8 KB (MT = 1) or 16 KB (MT = 2) each
  const int total_steps = p.K >> 6;

  // control block: full[kRing], empty[kRing] mbarriers, abort flag, tile counters / generations
  const uint32_t bar_full = smem_u32(s_raw), bar_empty = bar_full + 8 * kRing;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(s_raw + 16 * kRing);
  int* s_cnt = reinterpret_cast<int*>(s_raw + 16 * kRing + 16);        // [kAccBufs] arrivals
  volatile int* s_gen = reinterpret_cast<volatile int*>(s_cnt + kAccBufsMax);  // [kAccBufs] tiles finalized
  int* s_done = const_cast<int*>(s_gen) + kAccBufsMax;                          // consumer warps finished (gather)
  uint8_t* s_ring = s_raw + kCtrlBytes;
  float* s_acc = reinterpret_cast<float*>(s_ring + kRing * kSlotBytes);   // [kAccBufs][kCons][VALS][32]
  float* s_corr = s_acc + kAccBufs * kCons * VALS * 32;                            // [steps][MR][CW]
  __half* s_a = reinterpret_cast<__half*>(s_corr + total_steps * MR * CW); // [M][K] if a_smem

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int my_tiles = (p.tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int nunits = my_tiles * p.nsub;
  const int bs = p.block_shift - 6;          // meta row of a step = step >> bs
  const int meta_rows = kUnitSteps >> bs;    // rows of the scale / zero-point box of a unit

  // Lets the next kernel of the stream start as soon as every CTA of this one is resident (a
  // no-op unless that kernel was launched with programmatic stream serialization).
  asm volatile("griddepcontrol.launch_dependents;");
  // Set-up is on every launch's critical path (nothing streams before it): the producer warp
  // initialises its own barriers, one lane per slot, and fetches the tensor maps early.
  if (warp == kCons) {
    if (lane < kRing) {
      mbar_init(bar_full + 8 * lane, 1);
      mbar_init(bar_empty + 8 * lane, 1);
    }
    if (lane == 0) {
      prefetch_tensormap(&tm_w);
      prefetch_tensormap(&tm_s);
      if (HAS_ZP) prefetch_tensormap(&tm_z);
    }
    mbar_init_fence();
  } else if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kAccBufsMax; ++i) { s_cnt[i] = 0; s_gen[i] = 0; }
    *s_done = 0;
  }
  __syncthreads();

  if (warp == kCons) {
    // ================================ producer ================================
    // Weights, scales and zero points are read here WITHOUT waiting for the preceding kernel of
    // the stream (the caller vouches for them when it asks for the early start).
    // Issuing a TMA copy blocks the issuing thread for ~100 ns on B200, so up to 32 lanes issue
    // for different units at once.  Lane l owns ring slot l for the whole kernel (units
    // q = l, l + ring, ...): a slot's barriers are then waited on by one thread, one phase at
    // a time, which the parity form of mbarrier waits requires.
    const uint32_t tx = kUnitWBytes + (uint32_t)meta_rows * (HAS_ZP ? 48u : 32u);
    for (int q = lane; lane < p.ring && q < nunits; q += p.ring) {
      const int slot = lane;
      if (q >= p.ring &&
          !mbar_wait_bounded(bar_empty + 8 * slot, ((q / p.ring) - 1) & 1, abort_flag, &g_gemv_error,
                             0x100 | slot, kGemvWaitCycles))
        break;
      const int lt = q / p.nsub, sb = q - lt * p.nsub;
      const int tile = blockIdx.x + lt * gridDim.x;
      const uint32_t fb = bar_full + 8 * slot;
      const uint32_t dst = smem_u32(s_ring + slot * kSlotBytes);
      mbar_arrive_expect_tx(fb, tx);
      // Weights first: the lanes issue in lockstep and an SM starts one TMA copy every ~25-30 ns,
      // so whatever comes second is queued behind 32 copies; the 4 KB of weights are what the
      // consumers wait for, the few hundred bytes of scales catch up.
      tma_load_2d(dst, &tm_w, sb * (kUnitKBytes / 4), tile * 8, fb);  // x in uint32 elements
      const int mrow = (sb * kUnitSteps) >> bs;
      tma_load_2d(dst + kSlotScaleOff, &tm_s, tile * 16, mrow, fb);
      if (HAS_ZP) tma_load_2d(dst + kSlotZpOff, &tm_z, tile * 16, mrow, fb);
    }
  } else {
    // ================================ consumers ===============================
    const int g = lane >> 2, t = lane & 3;
    const int ctid = threadIdx.x;  // 0 .. kCons*32-1
    // Activations and the output belong to stream order: wait for the preceding kernel (returns
    // at once for a plain launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- once per CTA: activations into shared memory (small M) and the activation-only
    //      terms of every 64-k step:  lo = sum of a over k % 16 < 8, hi = sum over k % 16 >= 8
    //      symmetric:   corr = 1024 lo + 64 hi + 8 (lo + hi)
    //      zero points: (bias, asum) = (1024 lo + 64 hi, lo + hi)
    //      Four threads share a (row, step): each sums 8 "lo" and 8 "hi" values.
    {
      const int total = total_steps * p.M * 4;
      for (int base = 0; base < total; base += kCons * 32) {
        const int idx = base + ctid;
        const bool valid = idx < total;
        const int pair = idx >> 2, j = idx & 3;
        const int m = pair % p.M, step = pair / p.M;
        float lo = 0.0f, hi = 0.0f;
        if (valid) {
          const size_t off = (size_t)m * p.K + step * 64 + j * 16;
          const uint4 v0 = __ldg(reinterpret_cast<const uint4*>(p.a + off));
          const uint4 v1 = __ldg(reinterpret_cast<const uint4*>(p.a + off) + 1);
          if (p.a_smem) {
            *reinterpret_cast<uint4*>(s_a + off) = v0;
            *(reinterpret_cast<uint4*>(s_a + off) + 1) = v1;
          }
          const __half2* h0 = reinterpret_cast<const __half2*>(&v0);
          const __half2* h1 = reinterpret_cast<const __half2*>(&v1);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f0 = __half22float2(h0[e]), f1 = __half22float2(h1[e]);
            lo += f0.x + f0.y;
            hi += f1.x + f1.y;
          }
        }
        lo += __shfl_xor_sync(0xffffffffu, lo, 1);
        hi += __shfl_xor_sync(0xffffffffu, hi, 1);
        lo += __shfl_xor_sync(0xffffffffu, lo, 2);
        hi += __shfl_xor_sync(0xffffffffu, hi, 2);
        if (valid && j == 0) {
          const float bias = 1024.0f * lo + 64.0f * hi, asum = lo + hi;
          if (HAS_ZP) {
            s_corr[(step * MR + m) * 2] = bias;
            s_corr[(step * MR + m) * 2 + 1] = asum;
          } else {
            s_corr[step * MR + m] = bias + 8.0f * asum;
          }
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kCons * 32) : "memory");  // consumers only

    // rows >= M of the activation operand repeat row M-1; their outputs are never stored
    const __half* aptr[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j)
      aptr[j] = (p.a_smem ? s_a : p.a) + (size_t)min(g + 8 * j, p.M - 1) * p.K + t * 16;
    constexpr uint32_t kLoMask = 0x000f000fu, kHiMask = 0x00f000f0u;
    constexpr uint32_t kLoMagic = 0x64006400u, kHiMagic = 0x54005400u;
    const int expected = p.nsub < kCons ? p.nsub : kCons;  // warps contributing to a tile

    float total[MT][4];
    int cur_lt = -1;
    // Gather mode: the call's epoch is one past the calls completed so far (the word only changes
    // when every CTA of this call has finished); even / odd epochs alternate between two buffers.
    unsigned gather_epoch = 0;
    size_t gather_off = 0;
    if (p.gt.world > 0) {
      gather_epoch = *reinterpret_cast<volatile unsigned*>(p.gt.base[p.gt.rank] + kGatherEpochOff) + 1u;
      gather_off = kGatherCtrlBytes + (size_t)(gather_epoch & 1u) * p.gt.buf_bytes;
    }

    // Leaves this warp's partial sums of local tile `lt` in its own slot of the tile's buffer;
    // the warp that arrives last adds the slots up in a fixed order (the result does not depend
    // on which warp came last), rounds to fp16, stores, and recycles the buffer.
    auto flush = [&](int lt) {
      const int b = lt % kAccBufs;
      // the buffer's previous tile (lt - kAccBufs) must have been finalized
      if (lane == 0) {
        const long long t0 = clock64();
        while (s_gen[b] != lt / kAccBufs) {
          if (*abort_flag || clock64() - t0 > kGemvWaitCycles) {
            *abort_flag = 1;
            atomicCAS(&g_gemv_error, 0, 0x300 | b);
            break;
          }
        }
      }
      __syncwarp();
      float* buf = s_acc + b * (kCons * VALS * 32);
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) buf[(warp * VALS + j * 4 + e) * 32 + lane] = total[j][e];
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        __threadfence_block();
        last = (atomicAdd(&s_cnt[b], 1) == expected - 1);
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        __threadfence_block();
        const int tile = blockIdx.x + lt * gridDim.x;
        float sum[MT][4];
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) sum[j][e] = 0.0f;
        // contributors: the warps of the tile's first `expected` units, in unit order
        const int w0 = (lt * p.nsub) % kCons;
        for (int c = 0; c < expected; ++c) {
          const float* src = buf + ((w0 + c) % kCons) * (VALS * 32);
#pragma unroll
          for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sum[j][e] += src[(j * 4 + e) * 32 + lane];
        }
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // accumulator element e of a lane: row n = g + 8 (e >> 1), column m = 8 j + 2 t + (e & 1)
            const int n = tile * 16 + g + 8 * (e >> 1);
            const int m = 8 * j + 2 * t + (e & 1);
            if (m < p.M) {
              const __half h = __float2half_rn(sum[j][e]);
              if (p.gt.world > 0) {
                // this rank's columns of the gathered [M, n_total] result, in every rank's buffer
                const size_t off = gather_off + ((size_t)m * p.gt.n_total + (size_t)p.gt.rank * p.N + n) * sizeof(__half);
                for (int r = 0; r < p.gt.world; ++r) *reinterpret_cast<__half*>(p.gt.base[r] + off) = h;
              } else {
                p.out[(size_t)m * p.N + n] = p.bias ? __hadd(h, p.bias[n]) : h;
              }
            }
          }
        __syncwarp();
        if (lane == 0) {
          s_cnt[b] = 0;
          __threadfence_block();
          s_gen[b] = lt / kAccBufs + 1;
        }
      }
    };

    bool ok = true;
    for (int q = warp; ok && q < nunits; q += kCons) {
      const int lt = q / p.nsub, sb = q - lt * p.nsub;
      if (lt != cur_lt) {
        if (cur_lt >= 0) flush(cur_lt);
        cur_lt = lt;
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) total[j][e] = 0.0f;
      }
      const int slot = q % p.ring;
      ok = mbar_wait_bounded(bar_full + 8 * slot, (q / p.ring) & 1, abort_flag, &g_gemv_error, 0x200 | slot,
                             kGemvWaitCycles);
      if (!ok) break;
      const uint8_t* sw = s_ring + slot * kSlotBytes;
      const uint8_t* wlane = sw + g * kUnitKBytes + t * 16;  // [8 packed columns][512 bytes]
      const unsigned short* sc = reinterpret_cast<const unsigned short*>(sw + kSlotScaleOff);
      const uint8_t* zp = sw + kSlotZpOff;
#pragma unroll
      for (int u = 0; u < kUnitSteps; ++u) {
        const int step = sb * kUnitSteps + u;
        if (step >= total_steps) break;  // the last unit of a K that is not a multiple of 512 (TMA zero-filled the rest)
        const uint4 wv = *reinterpret_cast<const uint4*>(wlane + u * 64);
        const int mr = (u >> bs) * 16;
        const float sa = __half2float(__ushort_as_half(sc[mr + g]));
        const float sb_ = __half2float(__ushort_as_half(sc[mr + g + 8]));
        // Words 0,1 and 2,3 are paired into one mma each for their "lo" k pairs and one for
        // their "hi" k pairs, so that the activation operand of each mma is two ADJACENT
        // registers of the 16-byte loads (k pairs 0-1|2-3, 4-5|6-7, 8-9|10-11, 12-13|14-15).
        uint32_t lo_a[4], lo_b[4], hi_a[4], hi_b[4];
        const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t x = w4[r], y = x >> 8;
          lo_a[r] = lop3_and_or(x, kLoMask, kLoMagic);  // (na;   2r, 2r+1)    1024 + q
          hi_a[r] = lop3_and_or(x, kHiMask, kHiMagic);  // (na;   2r+8, 2r+9)    64 + q
          lo_b[r] = lop3_and_or(y, kLoMask, kLoMagic);  // (na+8; 2r, 2r+1)
          hi_b[r] = lop3_and_or(y, kHiMask, kHiMagic);  // (na+8; 2r+8, 2r+9)
        }
        float za = 0.0f, zb = 0.0f;
        if (HAS_ZP) {
          za = (float)zp[mr + g];
          zb = (float)zp[mr + g + 8];
        }
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          uint4 v0, v1;  // k 0-7 and 8-15 of this lane's chunk
          if (p.a_smem) {  // explicit shared-memory loads (a generic load would go through L1TEX)
            const uint32_t sa_addr = smem_u32(aptr[j] + step * 64);
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v0.x), "=r"(v0.y), "=r"(v0.z), "=r"(v0.w) : "r"(sa_addr));
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v1.x), "=r"(v1.y), "=r"(v1.z), "=r"(v1.w) : "r"(sa_addr + 16));
          } else {
            const uint4* ap = reinterpret_cast<const uint4*>(aptr[j] + step * 64);
            v0 = __ldg(ap);
            v1 = __ldg(ap + 1);
          }
          float acc[4];
          mma_m16n8k16_init(acc, lo_a[0], lo_b[0], lo_a[1], lo_b[1], v0.x, v0.y);
          mma_m16n8k16(acc, lo_a[2], lo_b[2], lo_a[3], lo_b[3], v0.z, v0.w);
          mma_m16n8k16(acc, hi_a[0], hi_b[0], hi_a[1], hi_b[1], v1.x, v1.y);
          mma_m16n8k16(acc, hi_a[2], hi_b[2], hi_a[3], hi_b[3], v1.z, v1.w);
          // accumulator rows na (e = 0, 1) and na + 8 (e = 2, 3); columns m = 8 j + 2 t + (e & 1)
          if (HAS_ZP) {
            const float4 c = *reinterpret_cast<const float4*>(&s_corr[(step * MR + 8 * j + 2 * t) * 2]);
            total[j][0] = fmaf(sa, acc[0] - fmaf(za, c.y, c.x), total[j][0]);
            total[j][1] = fmaf(sa, acc[1] - fmaf(za, c.w, c.z), total[j][1]);
            total[j][2] = fmaf(sb_, acc[2] - fmaf(zb, c.y, c.x), total[j][2]);
            total[j][3] = fmaf(sb_, acc[3] - fmaf(zb, c.w, c.z), total[j][3]);
          } else {
            const float2 c = *reinterpret_cast<const float2*>(&s_corr[step * MR + 8 * j + 2 * t]);
            total[j][0] = fmaf(sa, acc[0] - c.x, total[j][0]);
            total[j][1] = fmaf(sa, acc[1] - c.y, total[j][1]);
            total[j][2] = fmaf(sb_, acc[2] - c.x, total[j][2]);
            total[j][3] = fmaf(sb_, acc[3] - c.y, total[j][3]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
    }
    if (ok && cur_lt >= 0) flush(cur_lt);
    if (p.gt.world > 0 && ok) {
      // Publish.  A chain of release / acquire links, each at the narrowest scope that spans it:
      // storing lanes -> lane 0 of their warp (__syncwarp), warps -> the CTA's last warp (fence +
      // shared counter, CTA scope), CTAs -> the grid's last CTA (system fence + global counter),
      // which advances the local epoch and raises this rank's flag in every rank's block.  Only
      // one thread per CTA pays for a system-scope fence: 16 per CTA cost ~12 us per launch.
      __syncwarp();
      if (lane == 0) __threadfence_block();
      if (lane == 0 && atomicAdd(s_done, 1) == kCons - 1) {
        uint8_t* local = p.gt.base[p.gt.rank];
        __threadfence_system();
        const unsigned arrived = atomicAdd(reinterpret_cast<unsigned*>(local + kGatherDoneOff), 1u);
        if (arrived == gridDim.x - 1) {
          __threadfence_system();
          *reinterpret_cast<volatile unsigned*>(local + kGatherDoneOff) = 0u;
          *reinterpret_cast<volatile unsigned*>(local + kGatherEpochOff) = gather_epoch;
          __threadfence_system();
          const size_t foff = kGatherFlagsOff + ((gather_epoch & 1u) * kGatherMaxRanks + p.gt.rank) * sizeof(unsigned);
          for (int r = 0; r < p.gt.world; ++r)
            *reinterpret_cast<volatile unsigned*>(p.gt.base[r] + foff) = gather_epoch;
        }
      }
    }
  }
}

// Debugging knobs (environment, read once): BLKQ4_GEMV_WARPS = K splits per CTA,
// BLKQ4_GEMV_U = 64-k steps fetched together.  Unset means the built-in heuristic.
static int env_int(const char* name) {
  const char* v = getenv(name);
  return v ? atoi(v) : 0;
}

constexpr size_t kMaxDynamicSmem = 227 * 1024;
const char* const kTooMuchSmem = "shared memory";

template <int MT, bool HAS_ZP>
std::string launch_persistent_T(int M, int N, int K, int block, cudaStream_t stream, const __half* a,
                                const uint8_t* packed, const __half* scales, const uint8_t* zp,
                                __half* out, const __half* bias, bool early_fetch,
                                const GatherTable* gt = nullptr) {
  PersistParams p{};
  p.a = a; p.out = out; p.bias = bias;
  if (gt) p.gt = *gt; p.M = M; p.N = N; p.K = K;
  p.block_shift = block == 64 ? 6 : 7;
  p.tiles = N / 16;
  p.nsub = (K + kUnitKBytes - 1) / kUnitKBytes;  // the last unit may be partial
  p.ring = kRing;
  p.a_smem = (M <= 2 && (size_t)M * K * 2 <= 32 * 1024) ? 1 : 0;
  const int meta_rows = kUnitSteps >> (p.block_shift - 6);

  CUtensorMap tm_w, tm_s, tm_z;
  // the packed bytes viewed as uint32 [N/2][K/4]: a box row may then span 512 bytes
  bool ok = encode_tensor_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, packed, (uint64_t)(K / 4),
                                 (uint64_t)(N / 2), kUnitKBytes / 4, 8, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_tensor_map_2d(&tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scales, (uint64_t)N,
                                  (uint64_t)(K / block), 16, (uint32_t)meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
  ok = ok && encode_tensor_map_2d(&tm_z, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, zp ? zp : packed, (uint64_t)N,
                                  (uint64_t)(K / block), 16, (uint32_t)meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (!ok) return "cuTensorMapEncodeTiled failed";

  const int sms = sm_count();
  const int grid = p.tiles < sms ? p.tiles : sms;
  const size_t smem = kCtrlBytes + (size_t)kRing * kSlotBytes +
                      (size_t)(MT == 1 ? kAccBufsMax : 2) * kCons * MT * 4 * 32 * sizeof(float) +
                      (size_t)(K / 64) * 8 * MT * (HAS_ZP ? 2 : 1) * sizeof(float) +
                      (p.a_smem ? (size_t)M * K * 2 : 0);
  if (smem > kMaxDynamicSmem) return kTooMuchSmem;  // very long K with 9..16 rows: the generic kernel takes it
  auto kern = gemv_persistent_kernel<MT, HAS_ZP>;
  static std::atomic<int> granted[64];
  cudaError_t e = ensure_dynamic_smem(kern, smem, granted);
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kPersistThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // Programmatic stream serialization: this launch's CTAs may start, and its producer warp may
  // read weights, scales and zero points, while the preceding kernel of the stream drains.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early_fetch ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, tm_w, tm_s, tm_z, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  return std::string();
}

template <int NT, int MT, int U, bool COLWISE>
cudaError_t launch_T(int warps, int M, int N, int K, int block, cudaStream_t stream,
                     const __half* a, const uint8_t* packed, const __half* scales,
                     const uint8_t* zp, __half* out, const __half* bias) {
  const int ntiles = N / 16;
  const int grid = (ntiles + NT - 1) / NT;
  const size_t smem = (size_t)warps * NT * MT * 4 * 32 * sizeof(float);
  auto kern = gemv_kernel<NT, MT, U, COLWISE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, warps * 32, smem, stream>>>(a, packed, scales, zp, out, bias, M, N, K, block);
  return cudaGetLastError();
}

}  // namespace

int sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < 64) {
    const int c = cache[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
  if (dev >= 0 && dev < 64) cache[dev].store(sms, std::memory_order_relaxed);
  return sms;
}

int clear_gemv_error(cudaStream_t stream) {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_gemv_error) != cudaSuccess) return -1;
  return cudaMemsetAsync(p, 0, sizeof(int), stream) == cudaSuccess ? 0 : -1;
}

int read_gemv_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemv_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

std::string launch_gemv(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                        const __half* a, const uint8_t* packed, const __half* scales,
                        const uint8_t* zp, __half* out, const __half* bias, unsigned flags) {
  if (M < 1 || M > 16) return "skinny kernel needs 1 <= M <= 16";
  const bool early = (flags & BLKQ4_GEMM_EARLY_WEIGHT_FETCH) != 0;
  static const int env_warps = env_int("BLKQ4_GEMV_WARPS"), env_u = env_int("BLKQ4_GEMV_U");
  // Warps per CTA = K splits.  Each warp should see at least four 64-k steps.
  const int steps = K / 64;
  int warps = 8;
  while (warps > 1 && steps / warps < 4) warps >>= 1;
  if (env_warps >= 1 && env_warps <= kMaxWarps) warps = env_warps;
  const int u = env_u ? env_u : 4;
  cudaError_t e;
  static const int env_generic = env_int("BLKQ4_GEMV_GENERIC"), env_no_stream = env_int("BLKQ4_GEMV_NO_STREAM");
  // Decode shapes first: the cp.async stream kernel (blkq4_gemv_stream.cu).
  if (!env_generic && !env_no_stream) {
    const std::string r = M <= 8 ? launch_gemv_stream(block, colwise, M, N, K, stream, a, packed, scales, zp, out, bias, flags)
                                 : launch_gemv_wide(block, colwise, M, N, K, stream, a, packed, scales, zp, out, bias, flags);
    if (r != kStreamUnsupported) return r;
  }
  // Fast path: one scale per 64-k step; at least one 512-k unit (the last one may be partial), meta
  // rows and pointers 16-byte aligned (TMA), shared memory for the per-step terms within reach.
  if (colwise && block >= 64 && !env_generic && K >= kUnitKBytes && K <= 32768 &&
      reinterpret_cast<uintptr_t>(scales) % 16 == 0 && (!zp || reinterpret_cast<uintptr_t>(zp) % 16 == 0)) {
    const std::string r =
        (M <= 8) ? (zp ? launch_persistent_T<1, true>(M, N, K, block, stream, a, packed, scales, zp, out, bias, early)
                       : launch_persistent_T<1, false>(M, N, K, block, stream, a, packed, scales, zp, out, bias, early))
                 : (zp ? launch_persistent_T<2, true>(M, N, K, block, stream, a, packed, scales, zp, out, bias, early)
                       : launch_persistent_T<2, false>(M, N, K, block, stream, a, packed, scales, zp, out, bias, early));
    if (r != kTooMuchSmem) return r;
  }
  // Row-wise blocking carries 48 bytes of meta per chunk in registers, so it fetches
  // fewer steps at a time.
  if (M <= 8) {
    if (colwise)
      e = (u >= 8) ? launch_T<1, 1, 8, true>(warps, M, N, K, block, stream, a, packed, scales, zp, out, bias)
          : (u <= 2) ? launch_T<1, 1, 2, true>(warps, M, N, K, block, stream, a, packed, scales, zp, out, bias)
                     : launch_T<1, 1, 4, true>(warps, M, N, K, block, stream, a, packed, scales, zp, out, bias);
    else
      e = launch_T<1, 1, 2, false>(warps, M, N, K, block, stream, a, packed, scales, zp, out, bias);
  } else {
    e = colwise ? launch_T<2, 2, 2, true>(warps, M, N, K, block, stream, a, packed, scales, zp, out, bias)
                : launch_T<2, 2, 1, false>(warps, M, N, K, block, stream, a, packed, scales, zp, out, bias);
  }
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  return std::string();
}

std::string launch_gemv_gather(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                               const __half* a, const uint8_t* packed, const __half* scales,
                               const uint8_t* zp, __half* out_full, const GatherTable& gt, unsigned flags,
                               bool* delivered) {
  *delivered = false;
  if (M < 1 || M > 16) return "unsupported: the fused gather needs 1 <= M <= 16";
  // Decode shapes: the stream kernel computes, exchanges, waits and copies out in one launch.
  static const int env_no_stream = env_int("BLKQ4_GEMV_NO_STREAM");
  if (!env_no_stream) {
    const std::string r = launch_gemv_stream(block, colwise, M, N, K, stream, a, packed, scales, zp, out_full, nullptr,
                                             flags, &gt);
    if (r != kStreamUnsupported) {
      *delivered = r.empty();
      return r;
    }
  }
  if (!(colwise && block >= 64 && K >= kUnitKBytes && K <= 32768 &&
        reinterpret_cast<uintptr_t>(scales) % 16 == 0 && (!zp || reinterpret_cast<uintptr_t>(zp) % 16 == 0)))
    return "unsupported: the fused gather runs on the column-wise block >= 64 fast path only";
  const bool early = (flags & BLKQ4_GEMM_EARLY_WEIGHT_FETCH) != 0;
  const std::string r =
      (M <= 8) ? (zp ? launch_persistent_T<1, true>(M, N, K, block, stream, a, packed, scales, zp, nullptr, nullptr, early, &gt)
                     : launch_persistent_T<1, false>(M, N, K, block, stream, a, packed, scales, zp, nullptr, nullptr, early, &gt))
               : (zp ? launch_persistent_T<2, true>(M, N, K, block, stream, a, packed, scales, zp, nullptr, nullptr, early, &gt)
                     : launch_persistent_T<2, false>(M, N, K, block, stream, a, packed, scales, zp, nullptr, nullptr, early, &gt));
  return r == kTooMuchSmem ? std::string("unsupported: K too long for the fused gather at this M") : r;
}

}  // namespace blkq4
