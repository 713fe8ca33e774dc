// Tensor-core W4A16 GEMM for sm_100a (M > 16): out[M,N] = A[M,K] x dequant(W4[K,N]).
//
// Blackwell-native design: TMA-staged operands, in-kernel dequantization to fp16,
// tcgen05.mma with fp32 accumulators in tensor memory (TMEM).  The product is
// computed transposed ("swap-AB"): the 128 weight columns of a tile are the MMA's
// M side, up to 256 activation rows its N side, so one dequantized weight element
// feeds 256 multiply-adds and small M wastes no tensor work.
//
//   D^T[128 n x BM m] (TMEM, fp32)  +=  Wdq^T[128 n x 64 k] (smem)  x  A[BM m x 64 k]^T (smem)
//
// Persistent CTAs (one per SM) walk the tile list.  Warp roles:
//   warp 0      TMA producer: per 64-k step one activation tile (128-byte swizzle),
//               one 64 x 64-byte tile of packed int4 weights, its scales and zero points
//   warp 1      MMA issuer (one elected lane); owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld -> fp16 -> global, overlapped with the next tile
//               through a second TMEM accumulator buffer
//   warps 6-13  dequantizers, two groups of four warps on alternate steps: two 16-byte
//               chunks (16 k x 2 n each) per thread and step, written as fp16 in the
//               K-major 128-byte-swizzled operand layout
// Stages are handed over with mbarriers; every wait is bounded and, on expiry, sets
// an error word and drains the CTA instead of hanging the GPU.
//
// The packed weight layout was designed for mma.sync register fragments (reference
// src/mickey/blk_q4/f16_quant_sm80.cuh:362-417); a 16-byte run of a packed column
// still holds 16 consecutive k of two columns, which dequantizes into four
// 16-byte rows-segments of the UMMA operand.  Dequantization numerics are the
// reference kernel's (fp16(16+q) by bit trick, fma.rn.f16 with rn(scale*(-16-zp));
// src/mickey/cutlass_ext/q4gemm/warp/quantb_meta_mma_tensor_op_tile_iterator.h:69-104, :436-543).
#include "blkq4_common.cuh"
#include "blkq4_tma.cuh"

namespace blkq4 {

__device__ int g_gemm_tc_error = 0;  // 0 ok; otherwise (role << 8) | barrier id of the wait that gave up

namespace {

constexpr int TILE_N = 128;       // weight columns per tile (UMMA M)
constexpr int BLOCK_K = 64;       // k per pipeline step: one 128-byte swizzle row of fp16
constexpr int UMMA_K = 16;
constexpr int kStages = 4;        // TMA ring
constexpr int kDeqStages = 4;     // dequantized-weight ring
constexpr int kNumDeqWarps = 8;
constexpr int kDeqGroups = 2;     // warp groups taking alternate k steps
constexpr int kWarpsPerDeqGroup = kNumDeqWarps / kDeqGroups;
constexpr int kNumEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kNumEpiWarps + kNumDeqWarps);
constexpr int kDeqTileBytes = TILE_N * BLOCK_K * 2;  // 16 KB
constexpr int kPackTileBytes = (TILE_N / 2) * BLOCK_K;  // 4 KB: 64 packed columns x 64 bytes
constexpr int kScaleTileBytes = 1024;
constexpr int kZpTileBytes = 512;
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s: far beyond any legitimate wait

struct Params {
  int M, N, K, block;
  int BM;            // activation rows per tile = UMMA N (multiple of 16, <= 256)
  int m_tiles, n_tiles;
  int has_zp;
  int meta_rows;     // rows of the scale / zero-point box per step
  uint32_t meta_row_bytes_s, meta_row_bytes_z;  // bytes per box row
  __half* out;
};

// ---- PTX wrappers ---------------------------------------------------------------------------

// Bounded wait on an mbarrier; see mbar_wait_bounded.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int who) {
  return mbar_wait_bounded(bar, parity, abort_flag, &g_gemm_tc_error, who, kWaitCycles);
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes
// (64 fp16) with the 128-byte swizzle, rows contiguous, tile base 1024-byte aligned:
// start address >> 4 in bits 0-13, leading byte offset (unused for swizzled K-major) = 1
// in bits 16-29, stride byte offset 1024 >> 4 (one 8-row group) in bits 32-45, descriptor
// version 1 in bits 46-47, layout type 2 (SWIZZLE_128B) in bits 61-63.
__device__ __forceinline__ uint64_t make_sw128_kmajor_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulator (bits 4-5 = 1), fp16 A and B
// (formats 0), both K-major, N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ inline uint32_t make_idesc_f16(int umma_m, int umma_n) {
  return (1u << 4) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(umma_m >> 4) << 24);
}

// ---- shared-memory plan ---------------------------------------------------------------------

struct SmemPlan {
  uint32_t act, pack, scale, zp, deq, bars, total;
  uint32_t act_bytes;
};
__host__ __device__ inline SmemPlan make_plan(int BM) {
  SmemPlan p;
  p.act_bytes = (uint32_t)BM * 128u;
  uint32_t o = 0;
  p.deq = o;   o += kDeqStages * kDeqTileBytes;                     // 1024-aligned tiles
  p.act = o;   o += kStages * ((p.act_bytes + 1023u) & ~1023u);     // 1024-aligned tiles
  p.pack = o;  o += kStages * kPackTileBytes;
  p.scale = o; o += kStages * kScaleTileBytes;
  p.zp = o;    o += kStages * kZpTileBytes;
  p.bars = o;  o += 256;
  p.total = o + 1024;  // slack to align the dynamic base to 1024
  return p;
}

// Barrier slots (8 bytes each) inside the barrier block.
enum : int {
  BAR_FULL = 0,                           // [kStages]    TMA data landed
  BAR_EMPTY = BAR_FULL + kStages,         // [kStages]    stage consumed (MMA commit + dequant warps)
  BAR_DEQ_FULL = BAR_EMPTY + kStages,     // [kDeqStages] dequantized tile written
  BAR_DEQ_EMPTY = BAR_DEQ_FULL + kDeqStages,  // [kDeqStages] MMAs reading it retired
  BAR_ACC_FULL = BAR_DEQ_EMPTY + kDeqStages,  // [2] accumulator complete
  BAR_ACC_EMPTY = BAR_ACC_FULL + 2,       // [2] accumulator drained by the epilogue
  BAR_COUNT = BAR_ACC_EMPTY + 2
};
static_assert(BAR_COUNT * 8 + 16 <= 256, "barrier block too small");

template <bool COLWISE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_pack,
               const __grid_constant__ CUtensorMap tm_scale, const __grid_constant__ CUtensorMap tm_zp,
               const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const SmemPlan plan = make_plan(p.BM);
  const uint32_t act_stride = (plan.act_bytes + 1023u) & ~1023u;
  const uint32_t bars = base + plan.bars;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + plan.bars + BAR_COUNT * 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + plan.bars + BAR_COUNT * 8 + 8);
  auto bar = [&](int id) { return bars + 8u * (uint32_t)id; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.m_tiles * p.n_tiles;
  const int k_steps = p.K / BLOCK_K;
  const uint32_t tmem_cols = (2 * p.BM <= 32) ? 32u : (2 * p.BM <= 64) ? 64u : (2 * p.BM <= 128) ? 128u
                             : (2 * p.BM <= 256) ? 256u : 512u;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(BAR_FULL + i), 1);
      mbar_init(bar(BAR_EMPTY + i), 1 + kWarpsPerDeqGroup);
    }
    for (int i = 0; i < kDeqStages; ++i) {
      mbar_init(bar(BAR_DEQ_FULL + i), kWarpsPerDeqGroup);
      mbar_init(bar(BAR_DEQ_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_ACC_FULL + i), 1);
      mbar_init(bar(BAR_ACC_EMPTY + i), kNumEpiWarps);
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      const uint32_t tx = plan.act_bytes + kPackTileBytes + (uint32_t)p.meta_rows * p.meta_row_bytes_s +
                          (p.has_zp ? (uint32_t)p.meta_rows * p.meta_row_bytes_z : 0u);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int n_tile = tile / p.m_tiles, m_tile = tile % p.m_tiles;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kStages;
          if (it >= (uint32_t)kStages &&
              !mbar_wait(bar(BAR_EMPTY + s), ((it / kStages) - 1) & 1, abort_flag, 0x100 | s))
            goto producer_done;
          const uint32_t fb = bar(BAR_FULL + s);
          mbar_arrive_expect_tx(fb, tx);
          const int k0 = ks * BLOCK_K;
          tma_load_2d(base + plan.act + s * act_stride, &tm_act, k0, m_tile * p.BM, fb);
          tma_load_2d(base + plan.pack + s * kPackTileBytes, &tm_pack, k0, n_tile * (TILE_N / 2), fb);
          if (COLWISE) {
            // meta row-major [K/block, N]: box = meta_rows x 128 columns
            const int mrow = k0 / p.block;
            tma_load_2d(base + plan.scale + s * kScaleTileBytes, &tm_scale, n_tile * TILE_N, mrow, fb);
            if (p.has_zp)
              tma_load_2d(base + plan.zp + s * kZpTileBytes, &tm_zp, n_tile * TILE_N, mrow, fb);
          } else {
            // meta column-major [K, N/block]: box = meta_rows (n blocks) x 64 k
            const int mrow = n_tile * TILE_N / p.block;
            tma_load_2d(base + plan.scale + s * kScaleTileBytes, &tm_scale, k0, mrow, fb);
            if (p.has_zp) tma_load_2d(base + plan.zp + s * kZpTileBytes, &tm_zp, k0, mrow, fb);
          }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    // =============================== MMA issuer =================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(TILE_N, p.BM);
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
        const int ab = tcount & 1;
        if (tcount >= 2 &&
            !mbar_wait(bar(BAR_ACC_EMPTY + ab), ((tcount >> 1) - 1) & 1, abort_flag, 0x200 | ab))
          goto mma_done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(ab * p.BM);
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kStages, d = it % kDeqStages;
          if (!mbar_wait(bar(BAR_FULL + s), (it / kStages) & 1, abort_flag, 0x210 | s)) goto mma_done;
          if (!mbar_wait(bar(BAR_DEQ_FULL + d), (it / kDeqStages) & 1, abort_flag, 0x220 | d))
            goto mma_done;
          tc_fence_after();
          const uint32_t a_addr = base + plan.deq + d * kDeqTileBytes;
          const uint32_t b_addr = base + plan.act + s * act_stride;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            // 16 k = 32 bytes further along the swizzled row
            umma_f16(d_tmem, make_sw128_kmajor_desc(a_addr + k * 32), make_sw128_kmajor_desc(b_addr + k * 32),
                     idesc, (ks > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar(BAR_EMPTY + s));
          umma_commit(bar(BAR_DEQ_EMPTY + d));
        }
        umma_commit(bar(BAR_ACC_FULL + ab));
      }
    mma_done:;
    }
  } else if (warp < 2 + kNumEpiWarps) {
    // =============================== epilogue ===================================
    // A warp reads the TMEM lanes of its quarter (warp id % 4): lane = weight column n of
    // the tile, TMEM column = activation row m.  For one m the 32 lanes hold 32
    // consecutive n, i.e. 64 contiguous bytes of the row-major output.
    const int quarter = warp & 3;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const int n_tile = tile / p.m_tiles, m_tile = tile % p.m_tiles;
      const int ab = tcount & 1;
      if (!mbar_wait(bar(BAR_ACC_FULL + ab), (tcount >> 1) & 1, abort_flag, 0x300 | ab)) break;
      tc_fence_after();
      const int n = n_tile * TILE_N + quarter * 32 + lane;
      const int m0 = m_tile * p.BM;
      for (int c0 = 0; c0 < p.BM; c0 += 32) {
        if (m0 + c0 >= p.M) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * p.BM + c0), r);
        tmem_ld_wait();
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = m0 + c0 + j;
            if (m < p.M) p.out[(size_t)m * p.N + n] = __float2half_rn(__uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_ACC_EMPTY + ab));
    }
  } else {
    // =============================== dequantizers ===============================
    // Two groups of four warps take alternate 64-k steps, so that a group has two step times
    // for the dependent chain wait -> load -> convert -> store -> fence -> arrive of one step.
    // A step's packed tile is 256 chunks of 16 bytes; thread t of a group converts chunks
    // t and t + 128.  Chunk c: packed column np_l = c / 4 of the tile, 16-byte chunk
    // kc = c % 4 of its 64 bytes -> k in [16 kc, 16 kc + 16) of tile rows
    // na = 16 (np_l / 8) + np_l % 8 and na + 8.  Output: per row two 16-byte units (k 0-7
    // and 8-15 of the chunk) at unit index 2 kc and 2 kc + 1, XOR-swizzled with row % 8.
    const int dt = threadIdx.x - 32 * (2 + kNumEpiWarps);
    const int group = dt >> 7, t = dt & 127;
    int my_tiles = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) ++my_tiles;
    const uint32_t total_its = (uint32_t)my_tiles * (uint32_t)k_steps;
    for (uint32_t it = group; it < total_its; it += kDeqGroups) {
      const int s = it % kStages, d = it % kDeqStages;
      if (!mbar_wait(bar(BAR_FULL + s), (it / kStages) & 1, abort_flag, 0x400 | s)) break;
      if (it >= (uint32_t)kDeqStages &&
          !mbar_wait(bar(BAR_DEQ_EMPTY + d), ((it / kDeqStages) - 1) & 1, abort_flag, 0x410 | d))
        break;
      const uint8_t* pk = base_ptr + plan.pack + s * kPackTileBytes;
      const uint8_t* sc_tile = base_ptr + plan.scale + s * kScaleTileBytes;
      const uint8_t* zp_tile = base_ptr + plan.zp + s * kZpTileBytes;
      uint8_t* dq = base_ptr + plan.deq + d * kDeqTileBytes;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c = t + 128 * half;
        const int np_l = c >> 2, kc = c & 3;
        const int na = 16 * (np_l >> 3) + (np_l & 7), nb = na + 8;
        const uint4 wv = *reinterpret_cast<const uint4*>(pk + c * 16);
        const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};

        uint32_t s_lo_a[4], s_hi_a[4], o_lo_a[4], o_hi_a[4];
        uint32_t s_lo_b[4], s_hi_b[4], o_lo_b[4], o_hi_b[4];
        if (COLWISE) {
          // scale tile: meta_rows x 128 fp16; row of this chunk within the step
          const int mr = (p.block >= BLOCK_K) ? 0 : (kc * 16) / p.block;
          const __half* sp = reinterpret_cast<const __half*>(sc_tile) + mr * TILE_N;
          const __half sa = sp[na], sb = sp[nb];
          int za = 8, zb = 8;
          if (p.has_zp) {
            za = zp_tile[mr * TILE_N + na];
            zb = zp_tile[mr * TILE_N + nb];
          }
          const __half oa = dequant_offset(sa, za), ob = dequant_offset(sb, zb);
          const uint32_t sa2 = pack_half2(sa, sa), sb2 = pack_half2(sb, sb);
          const uint32_t oa2 = pack_half2(oa, oa), ob2 = pack_half2(ob, ob);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            s_lo_a[r] = s_hi_a[r] = sa2;
            o_lo_a[r] = o_hi_a[r] = oa2;
            s_lo_b[r] = s_hi_b[r] = sb2;
            o_lo_b[r] = o_hi_b[r] = ob2;
          }
        } else {
          // scale tile: (128 / block) rows x 64 k fp16, k permuted per 16 as
          // 0 1 8 9 2 3 10 11 ...; zero points 0 8 1 9 2 10 3 11 ...
          const int mr = na / p.block;
          const uint4* sp = reinterpret_cast<const uint4*>(sc_tile + mr * 128 + kc * 32);
          const uint4 s0 = sp[0], s1 = sp[1];
          const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          uint4 zv = make_uint4(0x08080808u, 0x08080808u, 0x08080808u, 0x08080808u);
          if (p.has_zp) zv = *reinterpret_cast<const uint4*>(zp_tile + mr * 64 + kc * 16);
          const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            s_lo_a[r] = s_lo_b[r] = sw[2 * r];
            s_hi_a[r] = s_hi_b[r] = sw[2 * r + 1];
            const uint32_t nz_lo = ((zw[r] << 6) & 0x03c003c0u) | 0xcc00cc00u;  // fp16(-16 - z)
            const uint32_t nz_hi = ((zw[r] >> 2) & 0x03c003c0u) | 0xcc00cc00u;
            o_lo_a[r] = o_lo_b[r] = hmul2_u32(sw[2 * r], nz_lo);
            o_hi_a[r] = o_hi_b[r] = hmul2_u32(sw[2 * r + 1], nz_hi);
          }
        }

        // word r -> k pairs (2r, 2r+1) and (2r+8, 2r+9) of both rows
        uint32_t a_lo[4], a_hi[4], b_lo[4], b_hi[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          uint32_t h[4];
          word_to_half16plus(w4[r], h);
          a_lo[r] = hfma2_u32(s_lo_a[r], h[0], o_lo_a[r]);
          a_hi[r] = hfma2_u32(s_hi_a[r], h[1], o_hi_a[r]);
          b_lo[r] = hfma2_u32(s_lo_b[r], h[2], o_lo_b[r]);
          b_hi[r] = hfma2_u32(s_hi_b[r], h[3], o_hi_b[r]);
        }
        const uint32_t row_a = (uint32_t)na * 128u, row_b = (uint32_t)nb * 128u;
        const uint32_t sw_a = (uint32_t)(na & 7), sw_b = (uint32_t)(nb & 7);
        *reinterpret_cast<uint4*>(dq + row_a + (((2 * kc) ^ sw_a) << 4)) = make_uint4(a_lo[0], a_lo[1], a_lo[2], a_lo[3]);
        *reinterpret_cast<uint4*>(dq + row_a + (((2 * kc + 1) ^ sw_a) << 4)) = make_uint4(a_hi[0], a_hi[1], a_hi[2], a_hi[3]);
        *reinterpret_cast<uint4*>(dq + row_b + (((2 * kc) ^ sw_b) << 4)) = make_uint4(b_lo[0], b_lo[1], b_lo[2], b_lo[3]);
        *reinterpret_cast<uint4*>(dq + row_b + (((2 * kc + 1) ^ sw_b) << 4)) = make_uint4(b_hi[0], b_hi[1], b_hi[2], b_hi[3]);
      }
      fence_proxy_async();  // generic-proxy writes -> visible to the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(BAR_DEQ_FULL + d));
        mbar_arrive(bar(BAR_EMPTY + s));
      }
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) __nanosleep(50000);  // let copies in flight land
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols)
                 : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------

}  // namespace

std::string launch_gemm_tc(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                           const __half* a, const uint8_t* packed, const __half* scales,
                           const uint8_t* zp, __half* out) {
  Params p{};
  p.M = M; p.N = N; p.K = K; p.block = block;
  p.BM = M >= 256 ? 256 : ((M + 15) / 16) * 16;
  p.m_tiles = (M + p.BM - 1) / p.BM;
  p.n_tiles = (N + TILE_N - 1) / TILE_N;
  p.has_zp = zp != nullptr;
  p.out = out;

  CUtensorMap tm_act, tm_pack, tm_scale, tm_zp;
  bool ok = encode_tensor_map_2d(&tm_act, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, (uint64_t)K, (uint64_t)M, BLOCK_K,
                      (uint32_t)p.BM, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && encode_tensor_map_2d(&tm_pack, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, packed, (uint64_t)K, (uint64_t)(N / 2),
                       BLOCK_K, TILE_N / 2, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (colwise) {
    p.meta_rows = block >= BLOCK_K ? 1 : BLOCK_K / block;
    p.meta_row_bytes_s = TILE_N * 2;
    p.meta_row_bytes_z = TILE_N;
    ok = ok && encode_tensor_map_2d(&tm_scale, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scales, (uint64_t)N,
                         (uint64_t)(K / block), TILE_N, (uint32_t)p.meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
    ok = ok && encode_tensor_map_2d(&tm_zp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, zp ? zp : packed, (uint64_t)N,
                         (uint64_t)(K / block), TILE_N, (uint32_t)p.meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
  } else {
    p.meta_rows = block >= TILE_N ? 1 : TILE_N / block;
    p.meta_row_bytes_s = BLOCK_K * 2;
    p.meta_row_bytes_z = BLOCK_K;
    ok = ok && encode_tensor_map_2d(&tm_scale, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scales, (uint64_t)K,
                         (uint64_t)(N / block), BLOCK_K, (uint32_t)p.meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
    ok = ok && encode_tensor_map_2d(&tm_zp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, zp ? zp : packed, (uint64_t)K,
                         (uint64_t)(N / block), BLOCK_K, (uint32_t)p.meta_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
  }
  if (!ok) return "cuTensorMapEncodeTiled failed";

  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int num_tiles = p.m_tiles * p.n_tiles;
  const int grid = num_tiles < sms ? num_tiles : sms;
  const SmemPlan plan = make_plan(p.BM);
  auto kern = colwise ? gemm_tc_kernel<true> : gemm_tc_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.total);
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  kern<<<grid, kThreads, plan.total, stream>>>(tm_act, tm_pack, tm_scale, tm_zp, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  return std::string();
}

int read_gemm_tc_error(cudaStream_t stream) {
  int v = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_gemm_tc_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace blkq4
