// Tensor-core W4A16 GEMM for sm_100a (M > 16): out[M,N] = A[M,K] x dequant(W4[K,N]).
//
// Blackwell-native design: TMA-staged operands, in-kernel dequantization to fp16,
// tcgen05.mma with fp32 accumulators in tensor memory (TMEM).  The product is
// computed transposed ("swap-AB"): the 128 weight columns of a tile are the MMA's
// M side, up to 256 activation rows its N side, so one dequantized weight element
// feeds 256 multiply-adds and small M wastes no tensor work.
//
//   D^T[128 n x BM m] (TMEM, fp32)  +=  Wdq^T[128 n x 64 k] (TMEM, fp16)  x  A[BM m x 64 k]^T (smem)
//
// The dequantized weights never touch shared memory: the dequantizer threads write them
// straight into tensor memory (tcgen05.st) and the MMA takes its first operand from there.
// Measured with the operand staged in shared memory instead, the 16 KB written plus 16 KB
// re-read per step, on top of the TMA traffic, cost a third of the step time.
//
// Two kernels share this design.  gemm_tc_kernel (this file; 16 < M < 256) gives every tile to one
// CTA; gemm_tc_pair_kernel (blkq4_gemm_tc_pair.cuh; M >= 256) gives a 256 x 256 tile to a CTA pair.
//
// Persistent CTAs (one per SM) walk the tile list.  Warp roles:
//   warp 0      TMA producer of the activation tiles (128-byte swizzle), kActStages stages
//   warp 14     TMA producer of the packed int4 weight tiles (64 x 64 bytes per 64-k step),
//               their scales and zero points, six stages
//   warp 1      MMA issuer (one elected lane); owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld -> fp16 -> global, overlapped with the next tile
//               through a second TMEM accumulator buffer
//   warps 6-13  dequantizers, two groups of four warps on alternate steps: thread = one
//               weight column n of the tile (TMEM lane n), 64 k per step = 32 TMEM columns
// Stages are handed over with mbarriers; every wait is bounded and, on expiry, sets
// an error word and drains the CTA instead of hanging the GPU.
//
// The packed weight layout was designed for mma.sync register fragments (reference
// src/mickey/blk_q4/f16_quant_sm80.cuh:362-417); a 16-byte run of a packed column
// still holds 16 consecutive k of two columns n0, n0 + 8, so the threads of columns n0 and
// n0 + 8 read the same 64 bytes per step and each keeps its own nibbles.  Dequantization numerics are the
// reference kernel's (fp16(16+q) by bit trick, fma.rn.f16 with rn(scale*(-16-zp));
// src/mickey/cutlass_ext/q4gemm/warp/quantb_meta_mma_tensor_op_tile_iterator.h:69-104, :436-543).
#include <cstddef>
#include <cstdint>
#include <cstdlib>

#include "blkq4_common.cuh"
#include "blkq4_tc.cuh"
#include "blkq4_tma.cuh"
#include "ms_blkq4gemm.h"

namespace blkq4 {

__device__ int g_gemm_tc_error = 0;  // 0 ok; otherwise (role << 8) | barrier id of the wait that gave up

namespace {

using namespace tc;
// Two rings.  The weight path (TMA -> shared memory -> dequantize -> tensor memory -> MMA) has a
// loop latency of several step times, so it is eight stages deep; its stages are small (5.5 KB of
// shared memory, 32 TMEM columns).  The activation path (TMA -> shared memory -> MMA) is short
// but its stages are 32 KB, so it gets six.
constexpr int kActStages = 6;
// The weight ring in shared memory (packed tile + scales + zero points per stage) is a template
// parameter of the kernels.
constexpr int kDeqStages = 8;     // dequantized weights in tensor memory
// tcgen05.commit costs about as much pipe time as one 128x256x16 MMA (measured: 128 cycles per MMA
// back to back, 241 with a commit after each), so completion is signalled once per kCommitSteps
// k steps and both rings are released at that granularity.
constexpr int kCommitSteps = 1;
constexpr int kDoneBars = kDeqStages / kCommitSteps;
static_assert(kActStages % kCommitSteps == 0 && kDeqStages % kCommitSteps == 0, "rings are released per commit group");
constexpr int kDeqGroups = 2;     // warp groups taking k steps in turn (three or four measured 3 % faster at most)
constexpr int kNumDeqWarps = 4 * kDeqGroups;
constexpr int kWarpsPerDeqGroup = kNumDeqWarps / kDeqGroups;
constexpr int kNumEpiWarps = 4;
constexpr int kWeightProducerWarp = 2 + kNumEpiWarps + kNumDeqWarps;  // last warp
constexpr int kSecondIssuerWarp = kWeightProducerWarp + 1;  // second MMA-issuing thread (DUAL kernels), else idle
constexpr int kMetaProducerWarp = kWeightProducerWarp + 2;  // TMA producer of the scales and zero points
constexpr int kThreads = 32 * (5 + kNumEpiWarps + kNumDeqWarps);
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s: far beyond any legitimate wait

struct Params {
  int M, N, K, block;
  int block_shift;   // log2(block)
  int BM;            // activation rows per tile = UMMA N (multiple of 16, <= 256)
  int m_tiles, n_tiles;
  int has_zp;
  int meta_rows;     // rows of the scale / zero-point box per step
  int acc_bufs;      // TMEM accumulator buffers: 2 when 2*BM + the dequantized stages fit in 512 columns
  int a_col0;        // first TMEM column of the dequantized stages
  uint32_t tmem_cols;  // allocation: power of two >= acc_bufs*BM + kDeqStages*kDeqCols
  uint32_t meta_row_bytes_s, meta_row_bytes_z;  // bytes per box row
  __half* out;
  const __half* bias;  // fp16 [N] added to the fp16 result, or null
  // Work items.  A tile's K range may be cut in parts that different CTAs compute: every part but
  // one leaves an fp32 partial tile in the workspace, the remaining one adds them to its own.
  //   balanced == 0: item = (tile, part), part < split covering k_per_item steps; CTA b takes items
  //     b, b + grid, ...; the last part of a tile adds the others.
  //   balanced == 1: the (tile, k step) sequence of the whole problem is cut in one contiguous range
  //     per CTA (range_bound), so that every SM gets the same number of steps whatever the tile
  //     count; a tile that straddles two ranges has its tail computed FIRST by the later CTA
  //     (partial tile, slot = that CTA) and its head LAST by the earlier CTA, which adds the partial.
  int split_shift;     // log2(split), split in {1, 2, 4}
  int k_per_item;      // 64-k steps per work item
  int num_items;       // tiles << split_shift
  int balanced;
  int k_steps;         // K / 64
  int total_steps;     // tiles * k_steps
  float* ws_partials;  // balanced: [cta][BM][128] fp32; otherwise [tile][split-1][BM][128]
  int gather_bulk;         // pair kernel, gather mode: peer copies as cp.async.bulk of whole rows
  int n_fastest, n_pairs;  // pair kernel: tile order (0: the m tiles of a pair of weight columns run together; 1: the column pairs of an m tile)
  GatherTable gt;      // pair kernel, gt.world > 0: the result goes to every rank's gathered buffer instead of `out`
  unsigned* ws_flags;  // balanced: [cta]; otherwise [tile]: arrivals (self-resetting)
};

// ---- PTX wrappers ---------------------------------------------------------------------------

// Bounded wait on an mbarrier; see mbar_wait_bounded.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int who) {
  return mbar_wait_bounded(bar, parity, abort_flag, &g_gemm_tc_error, who, kWaitCycles);
}
// ---- work items -----------------------------------------------------------------------------

constexpr int kMinPartSteps = 4;  // a range boundary closer than this to a tile boundary moves onto it

// First step of CTA b's range in balanced mode (b == grid: the end of the last range).
__host__ __device__ inline int range_bound(int total_steps, int k_steps, int grid, int b) {
  int x = (int)((long long)b * total_steps / grid);
  const int r = x % k_steps;
  if (r < kMinPartSteps) x -= r;
  else if (r > k_steps - kMinPartSteps) x += k_steps - r;
  return x;
}

struct Item {
  int tile, ks0, count;
  int role;    // 0: whole tile; 1: writes its partial tile to `slot`; 2: adds `nparts` partial tiles from `slot` on
  int slot, flag, nparts;
};
struct ItemCursor {
  int pos, end;  // balanced: steps of the range still to do; otherwise: next item index, item count
};
__device__ __forceinline__ ItemCursor first_item(const Params& p) {
  ItemCursor c;
  if (p.balanced) {
    c.pos = range_bound(p.total_steps, p.k_steps, (int)gridDim.x, (int)blockIdx.x);
    c.end = range_bound(p.total_steps, p.k_steps, (int)gridDim.x, (int)blockIdx.x + 1);
  } else {
    c.pos = (int)blockIdx.x;
    c.end = p.num_items;
  }
  return c;
}
__device__ __forceinline__ bool next_item(const Params& p, ItemCursor& c, Item& it) {
  if (c.pos >= c.end) return false;
  if (p.balanced) {
    it.tile = c.pos / p.k_steps;
    it.ks0 = c.pos - it.tile * p.k_steps;
    it.count = min(p.k_steps - it.ks0, c.end - c.pos);
    // a range is longer than a tile, so a cut tile has exactly two parts: its tail opens the later
    // CTA's range, its head closes the earlier one's
    it.role = it.ks0 > 0 ? 1 : (it.count < p.k_steps ? 2 : 0);
    it.slot = it.flag = (int)blockIdx.x + (it.role == 2 ? 1 : 0);
    it.nparts = 1;
    c.pos += it.count;
  } else {
    const int split = 1 << p.split_shift;
    it.tile = c.pos >> p.split_shift;
    const int part = c.pos - (it.tile << p.split_shift);
    it.ks0 = part * p.k_per_item;
    it.count = p.k_per_item;
    it.role = split == 1 ? 0 : (part < split - 1 ? 1 : 2);
    it.slot = it.tile * (split - 1) + (it.role == 1 ? part : 0);
    it.flag = it.tile;
    it.nparts = split - 1;
    c.pos += (int)gridDim.x;
  }
  return true;
}

// ---- shared-memory plan ---------------------------------------------------------------------

struct SmemPlan {
  uint32_t act, pack, scale, zp, out, bars, total;
  uint32_t act_bytes;
};
__host__ __device__ inline SmemPlan make_plan(int BM, int kStages, int act_stages, uint32_t out_bytes = 0) {
  SmemPlan p;
  p.act_bytes = (uint32_t)BM * 128u;
  uint32_t o = 0;
  p.act = o;   o += act_stages * ((p.act_bytes + 1023u) & ~1023u);  // 1024-aligned tiles
  p.pack = o;  o += kStages * kPackTileBytes;
  p.scale = o; o += kStages * kScaleTileBytes;
  p.zp = o;    o += kStages * kZpTileBytes;
  p.out = o;   o += out_bytes;  // output staging of the pair kernel's epilogue
  p.bars = o;  o += 512;
  p.total = o + 1024;  // slack to align the dynamic base to 1024
  return p;
}

// Barrier slots (8 bytes each) inside the barrier block.  Stage s of the TMA ring and stage s
// of the dequantized ring belong to the same k step, so one "MMA done" barrier frees both.
#define BLKQ4_TC_BARRIER_SLOTS(WS, ACT, DONE)                                                         \
  constexpr int kStages = (WS);                                                                                    \
  constexpr int BAR_ACT_FULL = 0;                        /* [kActStages] activation tile landed (-> MMA issuer) */  \
  constexpr int BAR_FULL = BAR_ACT_FULL + (ACT);         /* [kStages] packed weights + meta landed (-> dequantizers) */ \
  constexpr int BAR_PACK_FREE = BAR_FULL + kStages;      /* [kStages] packed weights / meta read (-> producer) */   \
  constexpr int BAR_DEQ_FULL = BAR_PACK_FREE + kStages;  /* [kDeqStages] dequantized stage in TMEM (-> MMA issuer) */ \
  constexpr int BAR_MMA_DONE = BAR_DEQ_FULL + kDeqStages;  /* [kDoneBars] commit group g = it / kCommitSteps retired, index g % kDoneBars */ \
  constexpr int BAR_ACC_FULL = BAR_MMA_DONE + (DONE);    /* [2] accumulator complete */                             \
  constexpr int BAR_ACC_EMPTY = BAR_ACC_FULL + 2;        /* [2] accumulator drained by the epilogue */              \
  constexpr int BAR_COUNT = BAR_ACC_EMPTY + 2;                                                                      \
  static_assert(BAR_COUNT * 8 + 16 <= 512, "barrier block too small");

// DUAL (BM <= 128): two threads issue the MMAs, the even k steps into one accumulator and the odd
// ones into a second, and the epilogue adds the two.  A thread gets one tcgen05.mma accepted per
// ~130 cycles whatever its N (measured: N = 32 .. 256, TMEM or shared-memory first operand), while
// the tensor pipe needs only N/2 cycles for it - two threads with accumulators of their own reach
// 65 cycles per MMA at N <= 64 and 71 at N = 128.  The sum order is fixed, so results stay reproducible.
template <bool COLWISE, int WS, bool DUAL>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_pack,
               const __grid_constant__ CUtensorMap tm_scale, const __grid_constant__ CUtensorMap tm_zp,
               const Params p) {
  BLKQ4_TC_BARRIER_SLOTS(WS, kActStages, kDoneBars)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const SmemPlan plan = make_plan(p.BM, kStages, kActStages);
  const uint32_t act_stride = (plan.act_bytes + 1023u) & ~1023u;
  const uint32_t bars = base + plan.bars;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + plan.bars + BAR_COUNT * 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + plan.bars + BAR_COUNT * 8 + 8);
  auto bar = [&](int id) { return bars + 8u * (uint32_t)id; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tmem_cols = p.tmem_cols;
  // Programmatic dependent launch: the next kernel of the stream may start its own set-up as soon
  // as every CTA of this one is resident.  In this kernel only the roles that touch activations,
  // the output or the split-K workspace wait for the preceding kernel (griddepcontrol.wait; it
  // returns at once for a plain launch); barrier set-up, TMEM allocation, the weight copies and the
  // dequantization of the first stages run ahead of it.
  asm volatile("griddepcontrol.launch_dependents;");

  if (threadIdx.x == 0) {
    for (int i = 0; i < kActStages; ++i) mbar_init(bar(BAR_ACT_FULL + i), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(BAR_FULL + i), 2);  // the packed-tile producer and the meta producer, each with its bytes
      mbar_init(bar(BAR_PACK_FREE + i), kWarpsPerDeqGroup);
    }
    for (int i = 0; i < kDeqStages; ++i) mbar_init(bar(BAR_DEQ_FULL + i), kWarpsPerDeqGroup);
    for (int i = 0; i < kDoneBars; ++i) mbar_init(bar(BAR_MMA_DONE + i), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_ACC_FULL + i), DUAL ? 2 : 1);
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
    // ========================= TMA producer: activations ========================
    // Stage sa = it % kActStages is free once the commit group of step it - kActStages retired.
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");  // activations belong to stream order
      uint32_t it = 0;
      ItemCursor cur = first_item(p);
      Item item;
      while (next_item(p, cur, item)) {
        const int m_tile = item.tile % p.m_tiles;
        for (int ks = item.ks0; ks < item.ks0 + item.count; ++ks, ++it) {
          const int sa = it % kActStages;
          if (it >= (uint32_t)kActStages) {
            const uint32_t g = (it - kActStages) / kCommitSteps;  // commit group of the stage's last user
            if (!mbar_wait(bar(BAR_MMA_DONE + g % kDoneBars), (g / kDoneBars) & 1, abort_flag, 0x100 | sa))
              goto act_producer_done;
          }
          const uint32_t fb = bar(BAR_ACT_FULL + sa);
          mbar_arrive_expect_tx(fb, plan.act_bytes);
          tma_load_2d(base + plan.act + sa * act_stride, &tm_act, ks * BLOCK_K, m_tile * p.BM, fb);
        }
      }
    act_producer_done:;
    }
  } else if (warp == kWeightProducerWarp || warp == kMetaProducerWarp) {
    // ============ TMA producers: packed weights (one warp), scales and zero points (another) ============
    // A thread gets one bulk-tensor copy accepted per ~110 cycles; with the stage wait and the byte-count
    // post, one thread issuing all three copies of a step is good for a step per ~600 cycles, which is
    // the whole kernel's pace once two threads issue the MMAs.  Hence two producer threads, each
    // arriving on the stage's barrier with its own byte count.
    if (lane == 0) {
      const bool meta = warp == kMetaProducerWarp;
      const uint32_t tx = meta ? (uint32_t)p.meta_rows * p.meta_row_bytes_s +
                                     (p.has_zp ? (uint32_t)p.meta_rows * p.meta_row_bytes_z : 0u)
                               : (uint32_t)kPackTileBytes;
      uint32_t it = 0;
      ItemCursor cur = first_item(p);
      Item item;
      while (next_item(p, cur, item)) {
        const int n_tile = item.tile / p.m_tiles;
        for (int ks = item.ks0; ks < item.ks0 + item.count; ++ks, ++it) {
          const int s = it % kStages;
          if (it >= (uint32_t)kStages &&
              !mbar_wait(bar(BAR_PACK_FREE + s), ((it / kStages) - 1) & 1, abort_flag, (meta ? 0x120 : 0x110) | s))
            goto w_producer_done;
          const uint32_t fb = bar(BAR_FULL + s);
          mbar_arrive_expect_tx(fb, tx);
          const int k0 = ks * BLOCK_K;
          if (!meta) {
            tma_load_2d(base + plan.pack + s * kPackTileBytes, &tm_pack, k0, n_tile * (TILE_N / 2), fb);
          } else if (COLWISE) {
            // meta row-major [K/block, N]: box = meta_rows x 128 columns
            const int mrow = k0 >> p.block_shift;
            tma_load_2d(base + plan.scale + s * kScaleTileBytes, &tm_scale, n_tile * TILE_N, mrow, fb);
            if (p.has_zp) tma_load_2d(base + plan.zp + s * kZpTileBytes, &tm_zp, n_tile * TILE_N, mrow, fb);
          } else {
            // meta column-major [K, N/block]: box = meta_rows (n blocks) x 64 k
            const int mrow = (n_tile * TILE_N) >> p.block_shift;
            tma_load_2d(base + plan.scale + s * kScaleTileBytes, &tm_scale, k0, mrow, fb);
            if (p.has_zp) tma_load_2d(base + plan.zp + s * kZpTileBytes, &tm_zp, k0, mrow, fb);
          }
        }
      }
    w_producer_done:;
    }
  } else if (DUAL && (warp == 1 || warp == kSecondIssuerWarp)) {
    // ========================= MMA issuers, DUAL: even steps / odd steps =========================
    if (lane == 0) {
      const uint32_t q = warp == 1 ? 0u : 1u;
      const uint32_t idesc = make_idesc_f16(TILE_N, p.BM);
      const uint32_t desc_hi = (uint32_t)(make_sw128_kmajor_desc(0) >> 32);
      const uint32_t desc_lo_flags = (uint32_t)(make_sw128_kmajor_desc(0) & 0xFFFFFFFFu);
      const uint32_t act_lo0 = desc_lo_flags | (((base + plan.act) >> 4) & 0x3FFFu);
      const uint32_t act_lo_step = act_stride >> 4;
      const uint32_t a_tmem0 = tmem_base + (uint32_t)p.a_col0;
      const uint32_t d_tmem = tmem_base + q * (uint32_t)p.BM;  // one accumulator per issuer, no double buffering
      uint32_t it = 0, tcount = 0;
      ItemCursor cur = first_item(p);
      Item item;
      for (; next_item(p, cur, item); ++tcount) {
        if (tcount >= 1u && !mbar_wait(bar(BAR_ACC_EMPTY), (tcount - 1u) & 1u, abort_flag, 0x200 | q)) goto mma2_done;
        tc_fence_after();
        uint32_t accumulate = 0u;
        for (uint32_t st = it + ((it ^ q) & 1u); st < it + (uint32_t)item.count; st += 2) {
          const uint32_t s = st % kDeqStages, sa = st % kActStages;
          const uint32_t bar_a = bar(BAR_ACT_FULL) + 8u * sa, bar_d = bar(BAR_DEQ_FULL) + 8u * s;
          const uint32_t par_sa = (st / kActStages) & 1u, par_s = (st / kDeqStages) & 1u;
          if (!mbar_try_wait(bar_a, par_sa) && !mbar_wait(bar_a, par_sa, abort_flag, 0x210 | sa)) goto mma2_done;
          if (!mbar_try_wait(bar_d, par_s) && !mbar_wait(bar_d, par_s, abort_flag, 0x220 | s)) goto mma2_done;
          tc_fence_after();
          umma_f16_ts_x4(d_tmem, a_tmem0 + s * kDeqCols, act_lo0 + sa * act_lo_step, desc_hi, idesc, accumulate);
          accumulate = 1u;
          umma_commit(bar(BAR_MMA_DONE) + 8u * (st % kDoneBars));
        }
        it += (uint32_t)item.count;
        umma_commit(bar(BAR_ACC_FULL));  // arrives at once for an issuer without a step in this item
      }
    mma2_done:;
    }
  } else if (warp == 1) {
    // =============================== MMA issuer =================================
    // One thread drives the tensor pipe, and its own instruction stream is the critical
    // path of the kernel: a 128x256x16 MMA takes 128 cycles, so the waits, address
    // arithmetic, four issues and the commit of a 64-k step must fit in 512 cycles of
    // dependent scalar code.  Hence: ring indices and parities are carried incrementally
    // (no division), the four MMAs of a step are one asm block, and the barrier polls take
    // the slow (bounded, instrumented) path only when the first poll fails.
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(TILE_N, p.BM);
      const uint32_t desc_hi = (uint32_t)(make_sw128_kmajor_desc(0) >> 32);
      const uint32_t desc_lo_flags = (uint32_t)(make_sw128_kmajor_desc(0) & 0xFFFFFFFFu);  // LBO field
      const uint32_t act_lo0 = desc_lo_flags | (((base + plan.act) >> 4) & 0x3FFFu);
      const uint32_t act_lo_step = act_stride >> 4;
      const uint32_t a_tmem0 = tmem_base + (uint32_t)p.a_col0;
      uint32_t s = 0, sa = 0, par_s = 0, par_sa = 0, gdone = 0, it = 0, tcount = 0;
      uint32_t ab = 0, par_acc = 0;
      // The barriers of step i + 1 are polled (without blocking) BEFORE the MMAs of step i are
      // issued, so that the poll's round trip to shared memory overlaps the issue instead of
      // extending the dependent chain of the next step.
      bool ready_a = false, ready_d = false;
#define BLKQ4_TC_MMA_ITEM(COUNT)                                                                                    \
  {                                                                                                                 \
    if (tcount >= (uint32_t)p.acc_bufs &&                                                                           \
        !mbar_wait(bar(BAR_ACC_EMPTY + ab), par_acc ^ 1u, abort_flag, 0x200 | ab))                                  \
      goto mma_done;                                                                                                \
    tc_fence_after();                                                                                               \
    const uint32_t d_tmem = tmem_base + ab * (uint32_t)p.BM;                                                        \
    for (int ks = 0; ks < (COUNT); ++ks, ++it) {                                                                    \
      const uint32_t bar_a = bar(BAR_ACT_FULL) + 8u * sa, bar_d = bar(BAR_DEQ_FULL) + 8u * s;                       \
      if (!ready_a && !mbar_try_wait(bar_a, par_sa) && !mbar_wait(bar_a, par_sa, abort_flag, 0x210 | sa))           \
        goto mma_done;                                                                                              \
      if (!ready_d && !mbar_try_wait(bar_d, par_s) && !mbar_wait(bar_d, par_s, abort_flag, 0x220 | s))              \
        goto mma_done;                                                                                              \
      tc_fence_after();                                                                                             \
      /* 16 k = 8 TMEM columns of the weights, 32 bytes (2 descriptor units) of the activation row */              \
      const uint32_t a_tmem = a_tmem0 + s * kDeqCols, b_lo = act_lo0 + sa * act_lo_step;                            \
      if (++s == kDeqStages) { s = 0; par_s ^= 1u; }                                                                \
      if (++sa == kActStages) { sa = 0; par_sa ^= 1u; }                                                             \
      ready_a = mbar_test_wait(bar(BAR_ACT_FULL) + 8u * sa, par_sa);                                                \
      ready_d = mbar_test_wait(bar(BAR_DEQ_FULL) + 8u * s, par_s);                                                  \
      umma_f16_ts_x4(d_tmem, a_tmem, b_lo, desc_hi, idesc, ks > 0 ? 1u : 0u);                                       \
      if (it % kCommitSteps == kCommitSteps - 1) {                                                                  \
        umma_commit(bar(BAR_MMA_DONE) + 8u * gdone);                                                                \
        if (++gdone == kDoneBars) gdone = 0;                                                                        \
      }                                                                                                             \
    }                                                                                                               \
    umma_commit(bar(BAR_ACC_FULL + ab));                                                                            \
    if (++ab == (uint32_t)p.acc_bufs) { ab = 0; par_acc ^= 1u; }                                                    \
  }
      if (!p.balanced) {
        for (int item = blockIdx.x; item < p.num_items; item += gridDim.x, ++tcount) BLKQ4_TC_MMA_ITEM(p.k_per_item)
      } else {
        int pos = range_bound(p.total_steps, p.k_steps, (int)gridDim.x, (int)blockIdx.x);
        const int end = range_bound(p.total_steps, p.k_steps, (int)gridDim.x, (int)blockIdx.x + 1);
        int to_tile_end = p.k_steps - pos % p.k_steps;
        for (; pos < end; ++tcount) {
          const int count = min(to_tile_end, end - pos);
          BLKQ4_TC_MMA_ITEM(count)
          pos += count;
          to_tile_end = p.k_steps;
        }
      }
#undef BLKQ4_TC_MMA_ITEM
    mma_done:;
    }
  } else if (warp < 2 + kNumEpiWarps) {
    // =============================== epilogue ===================================
    // A warp reads the TMEM lanes of its quarter (warp id % 4): lane = weight column n of
    // the tile, TMEM column = activation row m.  For one m the 32 lanes hold 32
    // consecutive n, i.e. 64 contiguous bytes of the row-major output.
    const int quarter = warp & 3;
    uint32_t tcount = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // output and workspace belong to stream order
    const size_t tile_floats = (size_t)p.BM * TILE_N;
    uint32_t it_base = 0;  // global index of the item's first k step
    ItemCursor cur = first_item(p);
    Item item;
    for (; next_item(p, cur, item); ++tcount) {
      const int n_tile = item.tile / p.m_tiles, m_tile = item.tile % p.m_tiles;
      const int ab = tcount % p.acc_bufs;
      if (!mbar_wait(bar(BAR_ACC_FULL + ab), (tcount / p.acc_bufs) & 1, abort_flag, 0x300 | ab)) break;
      tc_fence_after();
      // DUAL: the item's even steps were summed in accumulator 0 and its odd steps in accumulator 1 (an
      // item of a single step wrote only one of them); the result is accumulator 0 + accumulator 1.
      const bool have0 = !DUAL || item.count > 1 || (it_base & 1u) == 0u;
      const bool have1 = DUAL && (item.count > 1 || (it_base & 1u) == 1u);
      it_base += (uint32_t)item.count;
      auto load_acc = [&](int c0, uint32_t (&r)[32]) {
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        if (!DUAL) {
          tmem_ld_32x32b_x32(lane_base + (uint32_t)(ab * p.BM + c0), r);
          tmem_ld_wait();
        } else if (have0 && have1) {
          uint32_t r1[32];
          tmem_ld_32x32b_x32(lane_base + (uint32_t)c0, r);
          tmem_ld_32x32b_x32(lane_base + (uint32_t)(p.BM + c0), r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r1[j]));
        } else {
          tmem_ld_32x32b_x32(lane_base + (uint32_t)((have1 ? p.BM : 0) + c0), r);
          tmem_ld_wait();
        }
      };
      const int n_l = quarter * 32 + lane;
      if (item.role == 1) {
        // ---- a part that hands over: fp32 partial tile [m][n] to the workspace: for a row m
        //      the 32 lanes of a warp write 128 contiguous bytes.  (One line per lane, [n][m] with
        //      16-byte accesses, was measured slower: 32 lines touched per instruction.)
        float* dst_ws = p.ws_partials + (size_t)item.slot * tile_floats + n_l;
        const int rows = min(p.BM, p.M - m_tile * p.BM);
        for (int c0 = 0; c0 < rows; c0 += 32) {
          uint32_t r[32];
          load_acc(c0, r);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < rows) dst_ws[(size_t)(c0 + j) * TILE_N] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(BAR_ACC_EMPTY + ab));
          atomicAdd(p.ws_flags + item.flag, 1u);
        }
        continue;
      }
      if (item.role == 2) {
        // ---- the part that finishes the tile: wait (bounded) for the other parts' partial tiles ----
        if (lane == 0) {
          const unsigned want = (unsigned)(item.nparts * kNumEpiWarps);
          const long long t0 = clock64();
          while (*reinterpret_cast<volatile unsigned*>(p.ws_flags + item.flag) < want) {
            if (*abort_flag || clock64() - t0 > kWaitCycles) {
              *abort_flag = 1;
              atomicCAS(&g_gemm_tc_error, 0, 0x320 | quarter);
              break;
            }
          }
          __threadfence();
        }
        __syncwarp();
        if (*abort_flag) break;
      }
      const float* src_ws = p.ws_partials + (size_t)item.slot * tile_floats + n_l;
      const int n = n_tile * TILE_N + quarter * 32 + lane;
      const int m0 = m_tile * p.BM;
      // Lanes pair up (n even / odd) so that every store carries two adjacent n (4 bytes per
      // lane, 128 contiguous bytes per warp): the even lane writes the even rows m of a
      // 32-row chunk, the odd lane the odd rows, each with its partner's value alongside.
      const int odd = lane & 1;
      const bool n_ok = (n | 1) < p.N;  // N is a multiple of 16: the pair is in or out together
      for (int c0 = 0; c0 < p.BM; c0 += 32) {
        if (m0 + c0 >= p.M) break;  // warp-uniform
        uint32_t r[32];
        load_acc(c0, r);
        if (item.role == 2) {
          // add the other parts in part order (a fixed order: the result is reproducible)
          for (int q = 0; q < item.nparts; ++q) {
            const float* sq = src_ws + (size_t)q * tile_floats + (size_t)c0 * TILE_N;
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = (m0 + c0 + j < p.M) ? __ldcg(sq + (size_t)j * TILE_N) : 0.0f;
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + f[j]);
          }
        }
        int m = m0 + c0 + odd;
        __half* dst = p.out + (size_t)m * p.N + (n & ~1);
        // The bias is added to the ROUNDED result in fp16, which is what a separate
        // `output += bias` on the fp16 tensor computes.
        const bool add_bias = p.bias != nullptr && n_ok;
        const __half2 bias2 = add_bias ? *reinterpret_cast<const __half2*>(p.bias + (n & ~1)) : __half2();
        const size_t row_step = 2 * (size_t)p.N;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float mine = __uint_as_float(odd ? r[j + 1] : r[j]);       // my n, my row
          const float give = __uint_as_float(odd ? r[j] : r[j + 1]);       // my n, partner's row
          const float got = __shfl_xor_sync(0xffffffffu, give, 1);          // partner's n, my row
          __half2 v = odd ? __floats2half2_rn(got, mine) : __floats2half2_rn(mine, got);
          if (add_bias) v = __hadd2(v, bias2);
          if (n_ok && m < p.M) *reinterpret_cast<__half2*>(dst) = v;
          dst += row_step;
          m += 2;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(BAR_ACC_EMPTY + ab));
        // the warp that completes the tile's count puts the flag back to zero for the next launch
        if (item.role == 2 && atomicAdd(p.ws_flags + item.flag, 1u) == (unsigned)((item.nparts + 1) * kNumEpiWarps - 1))
          p.ws_flags[item.flag] = 0u;
      }
    }
  } else if (warp < kWeightProducerWarp) {
    // =============================== dequantizers ===============================
    // Two groups of four warps take alternate 64-k steps, so that a group has two step times
    // for the dependent chain wait -> load -> convert -> tcgen05.st -> arrive of one step.
    // A warp may only touch the TMEM lanes of its quarter (warp id % 4), and lane = row of the
    // MMA's first operand = weight column n of the tile: thread <-> n = 32 (warp % 4) + lane.
    // Column n lives in packed column np_l = 8 (n / 16) + n % 8 of the tile, in the "low"
    // nibble positions when n % 16 < 8 and 8 bits further up otherwise (the thread of n +- 8
    // reads the same bytes).  Per step it reads the column's 64 bytes and writes 32 TMEM
    // columns: column j = fp16 pair k = (2j, 2j + 1).
    const int dw = warp - (2 + kNumEpiWarps);
    const int group = dw / kWarpsPerDeqGroup;
    const int n_l = 32 * (warp & 3) + lane;
    const int np_l = 8 * (n_l >> 4) + (n_l & 7);
    const uint32_t nib_shift = (n_l & 8) ? 8u : 0u;
    const uint32_t tmem_row = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)p.a_col0;
    uint32_t total_its = 0;
    {
      ItemCursor cur = first_item(p);
      Item item;
      while (next_item(p, cur, item)) total_its += (uint32_t)item.count;
    }
    for (uint32_t it = group; it < total_its; it += kDeqGroups) {
      const int s = it % kStages, d = it % kDeqStages;
      if (it >= (uint32_t)kDeqStages) {
        const uint32_t g = (it - kDeqStages) / kCommitSteps;  // commit group of the TMEM stage's last user
        if (!mbar_wait(bar(BAR_MMA_DONE + g % kDoneBars), (g / kDoneBars) & 1, abort_flag, 0x410 | d)) break;
      }
      if (!mbar_wait(bar(BAR_FULL + s), (it / kStages) & 1, abort_flag, 0x400 | s)) break;
      tc_fence_after();
      const uint8_t* pk = base_ptr + plan.pack + s * kPackTileBytes + np_l * 64;
      const uint8_t* sc_tile = base_ptr + plan.scale + s * kScaleTileBytes;
      const uint8_t* zp_tile = base_ptr + plan.zp + s * kZpTileBytes;
      uint32_t out[32];
      dequant_step<COLWISE>(pk, sc_tile, zp_tile, n_l, nib_shift, p.block, p.block_shift, p.has_zp, out);
      tmem_st_32x32b_x32(tmem_row + (uint32_t)(d * kDeqCols), out);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(BAR_DEQ_FULL + d));
        mbar_arrive(bar(BAR_PACK_FREE + s));
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

#include "blkq4_gemm_tc_pair.cuh"

// ---- host side ---------------------------------------------------------------------------

}  // namespace

namespace {

// Work plan.  The kernel is persistent with one CTA per SM.  A problem with few output tiles
// (prefill of a 4096-wide layer at M = 512: 64 tiles on 148 SMs) leaves SMs idle: cutting every
// tile's K range in `split` work items fills them.  A problem with more tiles than SMs but not a
// whole number of rounds (256 tiles: the second round keeps 108 of 148 SMs busy) is cut in one
// contiguous range of k steps per CTA instead ("balanced", see Params).
struct SplitPlan {
  int split_shift;
  int balanced;
  size_t flags_bytes, total_bytes;  // workspace: [flags, 256-byte aligned][partials]
};

SplitPlan plan_split(int M, int N, int K, size_t ws_bytes_available) {
  const int BM = M >= 256 ? 256 : ((M + 15) / 16) * 16;
  const int tiles = ((M + BM - 1) / BM) * ((N + TILE_N - 1) / TILE_N);
  const int k_steps = K / BLOCK_K;
  const int sms = sm_count() > 0 ? sm_count() : 148;
  SplitPlan best{0, 0, 0, 0};
  if (tiles > sms) {
    // balanced ranges: every range longer than a tile (a cut tile then has exactly two parts), and
    // only when whole rounds would leave more than a fifth of the SM time idle.  Measured on B200:
    // 224 tiles of K = 8192 at M = 64: 98 -> 83 us; 172 tiles (M = 512, 4096 -> 11008): 55 -> 49 us;
    // 256 tiles (M = 2048, N = K = 4096; 86 % busy in whole rounds): 62 -> 66 us, the extra work item
    // and the fp32 exchange cost more than the balance gains, hence the threshold.
    const int rounds = (tiles + sms - 1) / sms;
    const long long total_steps = (long long)tiles * k_steps;
    static const bool off = getenv("BLKQ4_TC_NO_BALANCE") != nullptr;
    if (!off && total_steps < (1ll << 30) / sms && total_steps / sms >= k_steps + 2 * kMinPartSteps &&
        (double)tiles < 0.80 * rounds * sms) {
      const size_t flags = ((size_t)sms * sizeof(unsigned) + 255) & ~(size_t)255;
      const size_t total = flags + (size_t)sms * BM * TILE_N * sizeof(float);
      if (total <= ws_bytes_available) best = SplitPlan{0, 1, flags, total};
    }
    return best;
  }
  // Split only when every work item still gets an SM of its own (one round): measured on B200 a
  // second round of half-size items loses more to the fp32 exchange than it gains in balance.
  for (int shift = 1; shift <= 2; ++shift) {
    const int split = 1 << shift;
    if (k_steps % split != 0 || k_steps / split < 8 || tiles * split > sms) continue;
    const size_t flags = ((size_t)tiles * sizeof(unsigned) + 255) & ~(size_t)255;
    const size_t total = flags + (size_t)tiles * (split - 1) * BM * TILE_N * sizeof(float);
    if (total > ws_bytes_available) continue;
    best = SplitPlan{shift, 0, flags, total};
  }
  return best;
}

}  // namespace

namespace {

// Plan of the CTA-pair kernel (blkq4_gemm_tc_pair.cuh): two CTAs per 256 (weight columns) x BM tile, each
// staging half of the activation rows; the pair's UMMA N = BM must be a multiple of 32.  Used for
// M >= 256 when the pair tiles fill at least one round of the device's pairs (the pair kernel has no
// split-K: M = 512 on a 4096-wide layer, 32 pair tiles, runs faster split over single CTAs).  With a
// workspace, and when whole rounds would idle more than a fifth of the pairs' time, the work is cut in
// balanced ranges.  Measured on B200: 86 pair tiles on 74 pairs (M = 512, 4096 -> 11008) 52 -> 43 us;
// 112 tiles (M = 256, K = 8192, N = 28672) 103 -> 100 us; 128 tiles (c3, 86 % busy in whole rounds)
// 57 -> 61 us and 448 tiles (M = 1024) unchanged: one more accumulator hand-over per pair and the fp32
// exchange of a 128 KB partial tile per CTA cost what the balance gains there.
struct PairPlan {
  bool use;
  int BM, m_tiles, items, balanced;
  size_t flags_bytes, total_bytes;
};

PairPlan plan_pair(int M, int N, int K, size_t ws_bytes_available) {
  static const bool pair_off = getenv("BLKQ4_TC_NO_PAIR") != nullptr;
  static const int pair_min_m = getenv("BLKQ4_TC_PAIR_MIN_M") ? atoi(getenv("BLKQ4_TC_PAIR_MIN_M")) : 256;
  static const double balance_below =
      getenv("BLKQ4_TC_PAIR_BALANCE_BELOW") ? atof(getenv("BLKQ4_TC_PAIR_BALANCE_BELOW")) : 0.80;
  PairPlan pl{false, 0, 0, 0, 0, 0, 0};
  if (M < pair_min_m || pair_off) return pl;
  const int sms = sm_count() > 0 ? sm_count() : 148;
  const int pairs = sms / 2;
  pl.BM = M >= 256 ? 256 : ((M + 31) / 32) * 32;
  pl.m_tiles = (M + pl.BM - 1) / pl.BM;
  pl.items = pl.m_tiles * (((N + TILE_N - 1) / TILE_N + 1) / 2);
  const int k_steps = K / BLOCK_K;
  const long long total_steps = (long long)pl.items * k_steps;
  const int rounds = (pl.items + pairs - 1) / pairs;
  static const bool balance_off = getenv("BLKQ4_TC_NO_BALANCE") != nullptr;
  // Fewer tiles than pairs: the one-CTA kernel splits K.  (The pair kernel can do it too - ranges shorter
  // than a tile, a tile finished from several partial tiles - but measured slower: M = 512, K = N = 4096
  // 35.8 vs 28.7 us, K = 11008 54.0 vs 48.6 us; a 128 KB fp32 partial tile per CTA is a dear exchange.)
  if (pl.items < pairs) return pl;
  // Balanced ranges need a workspace (one flag word and one fp32 partial tile per CTA), ranges of at least
  // eight steps, and pay when whole rounds would idle more than a fifth of the pairs' time.
  const size_t flags = ((size_t)sms * sizeof(unsigned) + 255) & ~(size_t)255;
  const size_t total = flags + (size_t)sms * pl.BM * TILE_N * sizeof(float);
  const bool can_balance = !balance_off && total_steps < (1ll << 30) / pairs && total_steps / pairs >= 8 &&
                           (double)pl.items < balance_below * rounds * pairs && total <= ws_bytes_available;
  pl.use = true;
  if (can_balance) {
    pl.balanced = 1;
    pl.flags_bytes = flags;
    pl.total_bytes = total;
  }
  return pl;
}

}  // namespace

size_t gemm_tc_workspace_bytes(int M, int N, int K) {
  if (M <= 16) return 0;
  const PairPlan pp = plan_pair(M, N, K, ~(size_t)0);
  if (pp.use) return pp.total_bytes;
  return plan_split(M, N, K, ~(size_t)0).total_bytes;
}

bool gemm_tc_split_plan_refusable(int M, int N, int K, size_t capacity) {
  if (M <= 16) return false;
  const SplitPlan sp = plan_split(M, N, K, ~(size_t)0);
  return sp.total_bytes > capacity && sp.balanced == 0;
}

bool gemm_tc_gather_supported(int M, int N, int K) {
  return M > 16 && plan_pair(M, N, K, 0).use;
}

bool gemm_tc_plan_balanced(int M, int N, int K) {
  if (M <= 16) return false;
  const PairPlan pp = plan_pair(M, N, K, ~(size_t)0);
  if (pp.use) return pp.balanced != 0;
  return plan_split(M, N, K, ~(size_t)0).balanced != 0;
}

std::string launch_gemm_tc(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                           const __half* a, const uint8_t* packed, const __half* scales,
                           const uint8_t* zp, __half* out, const __half* bias, void* workspace,
                           size_t workspace_bytes, unsigned flags, const GatherTable* gt) {
  Params p{};
  if (gt) p.gt = *gt;
  p.M = M; p.N = N; p.K = K; p.block = block;
  p.block_shift = block == 16 ? 4 : block == 32 ? 5 : block == 64 ? 6 : 7;
  p.BM = M >= 256 ? 256 : ((M + 15) / 16) * 16;
  p.m_tiles = (M + p.BM - 1) / p.BM;
  p.n_tiles = (N + TILE_N - 1) / TILE_N;
  p.has_zp = zp != nullptr;
  p.out = out;
  p.bias = bias;
  // tensor memory: accumulators first, then the dequantized stages
  // BM <= 128: two accumulators, one per MMA-issuing thread (DUAL kernels); above, a single accumulator
  static const bool dual_off = getenv("BLKQ4_TC_NO_DUAL") != nullptr;
  const bool dual = p.BM <= 128 && !dual_off;
  p.acc_bufs = dual ? 1 : ((2 * p.BM + kDeqStages * kDeqCols <= 512) ? 2 : 1);
  p.a_col0 = dual ? 2 * p.BM : p.acc_bufs * p.BM;
  {
    const uint32_t need = (uint32_t)(p.a_col0 + kDeqStages * kDeqCols);
    p.tmem_cols = 32;
    while (p.tmem_cols < need) p.tmem_cols <<= 1;
  }

  const bool ws_ok = workspace && reinterpret_cast<uintptr_t>(workspace) % 256 == 0;
  // the fused exchange lives in the pair kernel's epilogue and runs in whole rounds
  const PairPlan pp = plan_pair(M, N, K, (ws_ok && !gt) ? workspace_bytes : 0);
  const bool pair = pp.use;
  if (gt && !pair) return "unsupported shape for the fused all-gather";
  if (pair) {
    p.BM = pp.BM;
    p.m_tiles = pp.m_tiles;
  }

  CUtensorMap tm_act, tm_pack, tm_scale, tm_zp;
  bool ok = encode_tensor_map_2d(&tm_act, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, (uint64_t)K, (uint64_t)M, BLOCK_K,
                      pair ? (uint32_t)(p.BM / 2) : (uint32_t)p.BM, CU_TENSOR_MAP_SWIZZLE_128B);
  // No swizzle on the packed tile: the dequantizers' 16-byte loads of eight neighbouring packed
  // columns (64 bytes apart) do conflict four ways, but a 64-byte TMA swizzle that removes the
  // conflicts measured 1-2 % SLOWER on the same GPU (c3 59.2 vs 58.2 us): those loads are not on
  // the critical path, the extra XOR per load is.
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

  const int sms = sm_count();
  if (pair) {
    p.k_steps = K / BLOCK_K;
    p.num_items = pp.items;
    p.n_pairs = (p.n_tiles + 1) / 2;
    // fused all-gather: walk the column pairs of one m tile together, so that at any moment the stores of all
    // ranks fall into a few hundred rows of every destination
    static const bool nf_off = getenv("BLKQ4_TC_GATHER_M_FASTEST") != nullptr;
    p.n_fastest = (gt && !nf_off) ? 1 : 0;
    static const bool bulk_off = getenv("BLKQ4_TC_GATHER_NO_BULK") != nullptr;
    p.gather_bulk = (gt && !bulk_off) ? 1 : 0;
    p.balanced = pp.balanced;
    p.total_steps = pp.balanced ? pp.items * p.k_steps : 0;
    p.ws_flags = reinterpret_cast<unsigned*>(workspace);
    p.ws_partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + pp.flags_bytes);
    auto kern = colwise ? gemm_tc_pair_kernel<true, kPairWeightStages> : gemm_tc_pair_kernel<false, kPairWeightStages>;
    const SmemPlan plan = make_plan(kPairRows, kPairWeightStages, kPairActStages, kPairOutBytes);
    static std::atomic<int> granted[2][64];
    cudaError_t e = ensure_dynamic_smem(kern, plan.total, granted[colwise ? 1 : 0]);
    if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = plan.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // pairs that can be resident at once (the cluster size is part of the kernel): one per two SMs at best
    static std::atomic<int> max_pairs[2][64];
    int dev = 0;
    cudaGetDevice(&dev);
    int pairs = (dev >= 0 && dev < 64) ? max_pairs[colwise ? 1 : 0][dev].load(std::memory_order_relaxed) : 0;
    if (pairs <= 0) {
      cfg.gridDim = dim3(sms & ~1);
      cfg.numAttrs = 0;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
      if (e != cudaSuccess || n <= 0) { cudaGetLastError(); n = sms / 2; }
      pairs = n < sms / 2 ? n : sms / 2;
      if (dev >= 0 && dev < 64) max_pairs[colwise ? 1 : 0][dev].store(pairs, std::memory_order_relaxed);
    }
    cfg.numAttrs = (flags & BLKQ4_GEMM_EARLY_WEIGHT_FETCH) ? 1 : 0;
    // balanced ranges use every resident pair, whole rounds at most one pair per tile
    cfg.gridDim = dim3(2 * ((p.balanced || p.num_items >= pairs) ? pairs : p.num_items));
    e = cudaLaunchKernelEx(&cfg, kern, tm_act, tm_pack, tm_scale, tm_zp, p);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
    return std::string();
  }
  const int num_tiles = p.m_tiles * p.n_tiles;
  const SplitPlan sp = ws_ok ? plan_split(M, N, K, workspace_bytes) : SplitPlan{0, 0, 0, 0};
  p.split_shift = sp.split_shift;
  p.k_per_item = (K / BLOCK_K) >> sp.split_shift;
  p.num_items = num_tiles << sp.split_shift;
  p.balanced = sp.balanced;
  p.k_steps = K / BLOCK_K;
  p.total_steps = sp.balanced ? num_tiles * p.k_steps : 0;
  p.ws_flags = reinterpret_cast<unsigned*>(workspace);
  p.ws_partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + sp.flags_bytes);
  const int grid = p.num_items < sms ? p.num_items : sms;
  // (a 16-stage weight ring measured no faster than 6 with either kernel)
  const SmemPlan plan = make_plan(p.BM, 6, kActStages);
  auto kern = dual ? (colwise ? gemm_tc_kernel<true, 6, true> : gemm_tc_kernel<false, 6, true>)
                   : (colwise ? gemm_tc_kernel<true, 6, false> : gemm_tc_kernel<false, 6, false>);
  static std::atomic<int> granted[4][64];
  cudaError_t e = ensure_dynamic_smem(kern, plan.total, granted[(colwise ? 1 : 0) + (dual ? 2 : 0)]);
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = plan.total;
  cfg.stream = stream;
  // BLKQ4_GEMM_EARLY_WEIGHT_FETCH: programmatic stream serialization, see the kernel's entry
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & BLKQ4_GEMM_EARLY_WEIGHT_FETCH) ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, tm_act, tm_pack, tm_scale, tm_zp, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  return std::string();
}

int clear_gemm_tc_error(cudaStream_t stream) {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_gemm_tc_error) != cudaSuccess) return -1;
  return cudaMemsetAsync(p, 0, sizeof(int), stream) == cudaSuccess ? 0 : -1;
}

int read_gemm_tc_error(cudaStream_t stream) {
  int v = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_gemm_tc_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace blkq4

extern "C" int blkq4_gemm_plan(int m, int n, int k, size_t workspace_size, int* out6) {
  if (!out6 || m <= 0 || n <= 0 || k <= 0 || (k % 64) != 0) return -1;
  for (int i = 0; i < 6; ++i) out6[i] = 0;
  if (m <= 16) return 0;
  const int sms = blkq4::sm_count() > 0 ? blkq4::sm_count() : 148;
  const blkq4::PairPlan pp = blkq4::plan_pair(m, n, k, workspace_size);
  if (pp.use) {
    out6[0] = 2; out6[1] = pp.BM; out6[2] = pp.items; out6[3] = 1; out6[4] = pp.balanced;
    out6[5] = pp.balanced ? sms / 2 : 0;
    return 0;
  }
  const blkq4::SplitPlan sp = blkq4::plan_split(m, n, k, workspace_size);
  const int bm = m >= 256 ? 256 : ((m + 15) / 16) * 16;
  out6[0] = 1; out6[1] = bm; out6[2] = ((m + bm - 1) / bm) * ((n + blkq4::tc::TILE_N - 1) / blkq4::tc::TILE_N);
  out6[3] = 1 << sp.split_shift; out6[4] = sp.balanced; out6[5] = sp.balanced ? sms : 0;
  return 0;
}

extern "C" int blkq4_gemm_plan_range_bound(int total_steps, int k_steps, int units, int b) {
  if (total_steps <= 0 || k_steps <= 0 || units <= 0 || b < 0 || b > units) return -1;
  return blkq4::range_bound(total_steps, k_steps, units, b);
}

