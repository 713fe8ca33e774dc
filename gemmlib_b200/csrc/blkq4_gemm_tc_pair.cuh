// CTA-pair variant of the tensor-core W4A16 GEMM (M >= 256).  Included by blkq4_gemm_tc.cu inside its
// anonymous namespace: it shares that file's Params, ring constants, barrier slots and error word.
//
// Why pairs.  With one CTA per tile a 64-k step stages 32 KB of activations (256 rows) in shared
// memory and the four MMAs read them back: 72 KB of shared-memory traffic per step against the
// 64 KB the SM can move in the 512 cycles the tensor pipe needs, so the step takes ~650 cycles.
// Two CTAs of a cluster (`cta_group::2`) compute one 256 (weight columns) x 256 (activation rows)
// tile together: each dequantizes ITS 128 weight columns into its own tensor memory and stages only
// ITS 128 activation rows; the pair's MMA (M = 256, N = 256, issued by the even CTA alone) reads
// every activation row once, from the CTA that holds it, for both halves of the weights.  Per SM and
// step: 16 KB of activations written, 16 KB read.
//
// Protocol (leader = cluster rank 0; every barrier the MMA thread waits on lives in the leader):
//   STEP_FULL[s]  (the slots named DEQ_FULL) count 9: the leader's activation producer arrives with
//                 expect_tx of BOTH halves of the step's activations, and the four dequantizer warps of
//                 each CTA arrive once their part of the step's weights is in tensor memory (the peer's
//                 remotely).  Both activation producers issue their TMA load with .cta_group::2, which
//                 lets the copy into the peer's own shared memory complete its bytes on the leader's
//                 barrier.
//   MMA_DONE[g]   tcgen05.commit with a two-CTA multicast: the copy in each CTA frees that CTA's
//                 activation stage and dequantized stage.
//   ACC_FULL      same multicast commit, to both epilogues; ACC_EMPTY count 8, like DEQ_FULL.
//   FULL / PACK_FREE (weight ring) stay local to each CTA.
// The loads here carry no cluster multicast: every CTA copies its own rows.  All waits are bounded;
// the two CTAs meet at a cluster barrier before either frees its tensor memory or exits.
//
// Work distribution: whole tiles in rounds over the resident pairs, or (with a workspace) one balanced
// range of k steps per pair with cut tiles finished through fp32 partial tiles (PairWalk).
// Epilogue: tensor memory -> fp16 staging in shared memory -> accumulator released -> global memory
// under the next tile's MMAs; with a GatherTable (N-sharded layers) the last hop goes to EVERY rank's
// exchange buffer as bulk copies of whole rows, and the grid's last CTA raises this rank's flag there.

constexpr int kPairRows = 128;  // most activation rows staged per CTA: half of the pair's UMMA N (p.BM / 2 are used)
// Rings of the pair kernel.  The activation ring is as deep as the ring of dequantized stages, so
// that ONE barrier per step ("step full") collects everything the MMAs of the step read - the bytes of
// both CTAs' activation copies and the arrivals of both CTAs' dequantizer warps - and the MMA thread
// polls one barrier per step instead of two: every instruction of that thread is on the critical path.
constexpr int kPairActStages = 8;     // 16 KB each
constexpr int kPairWeightStages = 6;  // 5.5 KB each; deeper rings measured no faster
constexpr int kPairCommitSteps = 1;   // a commit per two steps measured no faster
// fp16 staging of a CTA's 128 x 256 output tile: the epilogue empties the accumulator into it, hands
// the accumulator back, and only then writes global memory, under the next tile's MMAs
constexpr uint32_t kPairOutBytes = 128u * 256u * 2u;
// one "MMAs retired" barrier per commit group a waiter may look back to: the deeper of the two rings
constexpr int kPairDoneBars = (kPairActStages > kDeqStages ? kPairActStages : kDeqStages) / kPairCommitSteps + 1;
static_assert(kPairActStages == kDeqStages, "one barrier per step serves both rings");
static_assert(kDeqStages % kPairCommitSteps == 0, "rings are released per commit group");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// Arrival on a barrier of the peer CTA.  What it publishes lives in tensor memory and is ordered by
// tcgen05.wait::st / tcgen05.fence::before_thread_sync, so the arrive carries no cluster-scope release
// (measured: with .release.cluster the peer's dequantizer warps took 2.7x as long per step).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait with cluster-scope acquire (the arrivals may come from the peer CTA).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int who) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      atomicCAS(&g_gemm_tc_error, 0, who);
      return false;
    }
  }
}
// TMA load into THIS CTA's shared memory whose byte count completes on `bar_cluster_addr`, a barrier of
// either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
// The four pair MMAs of one 64-k step (see umma_f16_ts_x4).
__device__ __forceinline__ void umma_f16_ts_x4_pair(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                    uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 b0, b1, b2, b3;\n\t.reg .b32 l1, l2, l3, a1, a2, a3;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "add.u32 l1, %2, 2;\n\tadd.u32 l2, %2, 4;\n\tadd.u32 l3, %2, 6;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "mov.b64 b0, {%2, %3};\n\tmov.b64 b1, {l1, %3};\n\tmov.b64 b2, {l2, %3};\n\tmov.b64 b3, {l3, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], b0, %4, p;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a1], b1, %4, q;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a2], b2, %4, q;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a3], b3, %4, q;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives (once every earlier MMA of the pair has retired) on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(both)
      : "memory");
}

// warps 0 .. kWeightProducerWarp only: the one-CTA kernel's second issuer and meta producer have no part here
constexpr int kPairThreads = 32 * (kWeightProducerWarp + 1);

// Work items of one pair.  Whole rounds: pair tiles `pair`, `pair + num_pairs`, ... in full.  Balanced
// (p.balanced, needs a workspace): the (tile, k step) sequence of the whole problem is cut in one
// contiguous range per pair (range_bound); a tile that straddles two ranges has its tail computed FIRST
// by the later pair (role 1: each CTA leaves its fp32 partial tile in the workspace slot of its own
// CTA index) and its head LAST by the earlier pair (role 2: adds the partial of the CTA two indices up).
struct PairWalk {
  int pos, end, step, k_steps, balanced;
  __device__ __forceinline__ PairWalk(const Params& p, int pair, int num_pairs) {
    k_steps = p.k_steps;
    balanced = p.balanced;
    if (balanced) {
      pos = range_bound(p.total_steps, k_steps, num_pairs, pair);
      end = range_bound(p.total_steps, k_steps, num_pairs, pair + 1);
      step = 0;
    } else {
      pos = pair;
      end = p.num_items;
      step = num_pairs;
    }
  }
  // role: 0 whole tile, 1 hands a partial tile over, 2 finishes a tile with a partial from the next pair
  __device__ __forceinline__ bool next(int& tile, int& ks0, int& count, int& role) {
    if (pos >= end) return false;
    if (balanced) {
      tile = pos / k_steps;
      ks0 = pos - tile * k_steps;
      count = min(k_steps - ks0, end - pos);
      role = ks0 > 0 ? 1 : (count < k_steps ? 2 : 0);
      pos += count;
    } else {
      tile = pos;
      ks0 = 0;
      count = k_steps;
      role = 0;
      pos += step;
    }
    return true;
  }
};

template <bool COLWISE, int WS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_pack,
                    const __grid_constant__ CUtensorMap tm_scale, const __grid_constant__ CUtensorMap tm_zp,
                    const Params p) {
  constexpr int kActStages = kPairActStages, kDoneBars = kPairDoneBars, kCommitSteps = kPairCommitSteps;
  BLKQ4_TC_BARRIER_SLOTS(WS, kPairActStages, kPairDoneBars)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const SmemPlan plan = make_plan(kPairRows, kStages, kActStages, kPairOutBytes);
  const uint32_t act_stride = (plan.act_bytes + 1023u) & ~1023u;
  const uint32_t bars = base + plan.bars;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + plan.bars + BAR_COUNT * 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + plan.bars + BAR_COUNT * 8 + 8);
  unsigned* s_done = reinterpret_cast<unsigned*>(base_ptr + plan.bars + BAR_COUNT * 8 + 12);  // epilogue warps done storing
  unsigned* s_epi = reinterpret_cast<unsigned*>(base_ptr + plan.bars + BAR_COUNT * 8 + 16);   // epilogue warps' barrier count
  static_assert(BAR_COUNT * 8 + 20 <= 512, "barrier block too small");
  auto bar = [&](int id) { return bars + 8u * (uint32_t)id; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int half = p.BM >> 1;  // activation rows this CTA stages; p.BM (a multiple of 32, <= 256) is the pair's UMMA N
  const int pair = (int)(blockIdx.x >> 1), num_pairs = (int)(gridDim.x >> 1);
  constexpr uint32_t kTmemCols = 512;  // 256 accumulator columns + eight dequantized stages of 32
  constexpr uint32_t kAcol0 = 256;
  asm volatile("griddepcontrol.launch_dependents;");

  if (threadIdx.x == 0) {
    for (int i = 0; i < kActStages; ++i) mbar_init(bar(BAR_ACT_FULL + i), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(BAR_FULL + i), 1);
      mbar_init(bar(BAR_PACK_FREE + i), kWarpsPerDeqGroup);
    }
    for (int i = 0; i < kDeqStages; ++i) mbar_init(bar(BAR_DEQ_FULL + i), 1 + 2 * kWarpsPerDeqGroup);  // "step full"
    for (int i = 0; i < kDoneBars; ++i) mbar_init(bar(BAR_MMA_DONE + i), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_ACC_FULL + i), 1);
      mbar_init(bar(BAR_ACC_EMPTY + i), 2 * kNumEpiWarps);
    }
    *abort_flag = 0;
    *s_done = 0u;
    *s_epi = 0u;
    mbar_init_fence();
  }
  if (warp == 1) {
    // one warp of EACH CTA of the pair, same warp index, same destination offset
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything of this CTA signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int k_steps = p.k_steps;

  if (warp == 0) {
    // ========================= TMA producer: this CTA's 128 activation rows ========================
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");  // activations belong to stream order
      uint32_t it = 0;
      PairWalk walk(p, pair, num_pairs);
      int item, ks0, count, role;
      while (walk.next(item, ks0, count, role)) {
        const int m_tile = p.n_fastest ? item / p.n_pairs : item % p.m_tiles;
        for (int ks = ks0; ks < ks0 + count; ++ks, ++it) {
          const int sa = it % kActStages;
          if (it >= (uint32_t)kActStages) {
            const uint32_t g = (it - kActStages) / kCommitSteps;
            if (!mbar_wait(bar(BAR_MMA_DONE + g % kDoneBars), (g / kDoneBars) & 1, abort_flag, 0x100 | sa))
              goto act_producer_done;
          }
          const uint32_t fb = bar(BAR_DEQ_FULL + sa);  // the step's one barrier
          if (rank == 0) mbar_arrive_expect_tx(fb, 2u * (uint32_t)half * 128u);
          tma_load_2d_pair(base + plan.act + sa * act_stride, &tm_act, ks * BLOCK_K,
                           m_tile * p.BM + (int)rank * half, map_to_cta(fb, 0));
        }
      }
    act_producer_done:;
    }
  } else if (warp == kWeightProducerWarp) {
    // ==================== TMA producer: this CTA's packed weights and meta =================
    // (one thread: here the MMA thread sets the pace, and a second producer warp measured 3 % slower)
    if (lane == 0) {
      const uint32_t tx = kPackTileBytes + (uint32_t)p.meta_rows * p.meta_row_bytes_s +
                          (p.has_zp ? (uint32_t)p.meta_rows * p.meta_row_bytes_z : 0u);
      uint32_t it = 0;
      PairWalk walk(p, pair, num_pairs);
      int item, ks0, count, role;
      while (walk.next(item, ks0, count, role)) {
        const int n_tile = 2 * (p.n_fastest ? item % p.n_pairs : item / p.m_tiles) + (int)rank;
        for (int ks = ks0; ks < ks0 + count; ++ks, ++it) {
          const int s = it % kStages;
          if (it >= (uint32_t)kStages &&
              !mbar_wait(bar(BAR_PACK_FREE + s), ((it / kStages) - 1) & 1, abort_flag, 0x110 | s))
            goto w_producer_done;
          const uint32_t fb = bar(BAR_FULL + s);
          mbar_arrive_expect_tx(fb, tx);
          const int k0 = ks * BLOCK_K;
          tma_load_2d(base + plan.pack + s * kPackTileBytes, &tm_pack, k0, n_tile * (TILE_N / 2), fb);
          if (COLWISE) {
            const int mrow = k0 >> p.block_shift;
            tma_load_2d(base + plan.scale + s * kScaleTileBytes, &tm_scale, n_tile * TILE_N, mrow, fb);
            if (p.has_zp) tma_load_2d(base + plan.zp + s * kZpTileBytes, &tm_zp, n_tile * TILE_N, mrow, fb);
          } else {
            const int mrow = (n_tile * TILE_N) >> p.block_shift;
            tma_load_2d(base + plan.scale + s * kScaleTileBytes, &tm_scale, k0, mrow, fb);
            if (p.has_zp) tma_load_2d(base + plan.zp + s * kZpTileBytes, &tm_zp, k0, mrow, fb);
          }
        }
      }
    w_producer_done:;
    }
  } else if (warp == 1) {
    // =============================== MMA issuer: the leader's lane 0 =================================
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc_f16(2 * TILE_N, p.BM);
      const uint32_t desc_hi = (uint32_t)(make_sw128_kmajor_desc(0) >> 32);
      const uint32_t desc_lo_flags = (uint32_t)(make_sw128_kmajor_desc(0) & 0xFFFFFFFFu);
      const uint32_t act_lo0 = desc_lo_flags | (((base + plan.act) >> 4) & 0x3FFFu);
      const uint32_t act_lo_step = act_stride >> 4;
      const uint32_t a_tmem0 = tmem_base + kAcol0;
      uint32_t s = 0, par_s = 0, gdone = 0, it = 0, tcount = 0;
      // the barrier of step i + 1 is polled (without blocking) before the MMAs of step i are issued, so
      // that the poll's round trip overlaps the issue
      bool ready = false;
#define BLKQ4_TC_PAIR_MMA_ITEM(COUNT)                                                                              \
  {                                                                                                                 \
    if (tcount >= 1u && !mbar_wait_cluster(bar(BAR_ACC_EMPTY), (tcount - 1u) & 1u, abort_flag, 0x200)) goto mma_done; \
    tc_fence_after();                                                                                               \
    for (int ks = 0; ks < (COUNT); ++ks, ++it) {                                                                    \
      const uint32_t bar_d = bar(BAR_DEQ_FULL) + 8u * s;                                                            \
      if (!ready && !mbar_try_wait(bar_d, par_s) && !mbar_wait(bar_d, par_s, abort_flag, 0x220 | s)) goto mma_done; \
      tc_fence_after();                                                                                             \
      const uint32_t a_tmem = a_tmem0 + s * kDeqCols, b_lo = act_lo0 + s * act_lo_step;                             \
      if (++s == kDeqStages) { s = 0; par_s ^= 1u; }                                                                \
      ready = mbar_test_wait(bar(BAR_DEQ_FULL) + 8u * s, par_s);                                                    \
      umma_f16_ts_x4_pair(tmem_base, a_tmem, b_lo, desc_hi, idesc, ks > 0 ? 1u : 0u);                               \
      if (it % kCommitSteps == kCommitSteps - 1) {                                                                  \
        umma_commit_pair(bar(BAR_MMA_DONE) + 8u * gdone);                                                           \
        if (++gdone == kDoneBars) gdone = 0;                                                                        \
      }                                                                                                             \
    }                                                                                                               \
    umma_commit_pair(bar(BAR_ACC_FULL));                                                                            \
  }
      if (!p.balanced) {
        for (int item = pair; item < p.num_items; item += num_pairs, ++tcount) BLKQ4_TC_PAIR_MMA_ITEM(k_steps)
      } else {
        int pos = range_bound(p.total_steps, k_steps, num_pairs, pair);
        const int end = range_bound(p.total_steps, k_steps, num_pairs, pair + 1);
        int to_tile_end = k_steps - pos % k_steps;
        for (; pos < end; ++tcount) {
          const int count = min(to_tile_end, end - pos);
          BLKQ4_TC_PAIR_MMA_ITEM(count)
          pos += count;
          to_tile_end = k_steps;
        }
      }
#undef BLKQ4_TC_PAIR_MMA_ITEM
    mma_done:;
    }
  } else if (warp < 2 + kNumEpiWarps) {
    // =============================== epilogue: this CTA's 128 weight columns ===================================
    // A warp owns the 32 weight columns n of its TMEM quarter (lane = n) for all 256 activation rows m
    // (TMEM columns).  With the single 256-column accumulator the next tile's MMAs wait for this drain,
    // so it is kept short: tensor memory -> fp16 -> the warp's own staging block [256 m][32 n] in shared
    // memory, accumulator released, and only then staging -> global memory (64-byte row pieces, 8 bytes
    // per lane), which overlaps the next tile.  No other warp touches the block: only __syncwarp.
    const int quarter = warp & 3;
    uint32_t tcount = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the output belongs to stream order
    const uint32_t acc_empty_leader = map_to_cta(bar(BAR_ACC_EMPTY), 0);
    // Fused all-gather: the call's epoch is one past the calls completed so far (the word only changes
    // when every CTA of this call has finished); even / odd epochs alternate between two buffers.
    unsigned gather_epoch = 0;
    size_t gather_off = 0;
    if (p.gt.world > 0) {
      gather_epoch = *reinterpret_cast<volatile unsigned*>(p.gt.base[p.gt.rank] + kGatherEpochOff) + 1u;
      gather_off = kGatherCtrlBytes + (size_t)(gather_epoch & 1u) * p.gt.buf_bytes;
    }
    uint8_t* stage = base_ptr + plan.out + quarter * (256 * 64);
    // Barrier of the four epilogue warps (gather mode), bounded like every wait here: a counter in
    // shared memory that only grows; a warp that sees the CTA's abort flag leaves instead of waiting.
    unsigned epi_calls = 0;
    auto epi_barrier = [&]() -> bool {
      __syncwarp();
      ++epi_calls;
      if (lane == 0) {
        __threadfence_block();
        atomicAdd(s_epi, 1u);
        const long long t0 = clock64();
        while (*reinterpret_cast<volatile unsigned*>(s_epi) < epi_calls * (unsigned)kNumEpiWarps) {
          if (*abort_flag || clock64() - t0 > kWaitCycles) {
            *abort_flag = 1;
            atomicCAS(&g_gemm_tc_error, 0, 0x330 | quarter);
            break;
          }
        }
        __threadfence_block();
      }
      __syncwarp();
      return *abort_flag == 0;
    };
    const int odd = lane & 1;
    const bool bulk = p.gt.world > 0 && p.gather_bulk;
    const size_t tile_floats = (size_t)p.BM * TILE_N;
    PairWalk walk(p, pair, num_pairs);
    int item, ks0, count, role;
    for (; walk.next(item, ks0, count, role); ++tcount) {
      const int n_tile = 2 * (p.n_fastest ? item % p.n_pairs : item / p.m_tiles) + (int)rank;
      const int m_tile = p.n_fastest ? item / p.n_pairs : item % p.m_tiles;
      if (!mbar_wait_cluster(bar(BAR_ACC_FULL), tcount & 1u, abort_flag, 0x300)) break;
      tc_fence_after();
      const int m0 = m_tile * p.BM;
      const int rows = min(p.BM, p.M - m0);
      const int n_l = quarter * 32 + lane;
      if (role == 1) {
        // ---- the tail of a tile whose head another pair computes: fp32 partial tile [m][n] to this CTA's slot
        //      of the workspace (for a row m the 32 lanes of a warp write 128 contiguous bytes)
        float* dst_ws = p.ws_partials + (size_t)blockIdx.x * tile_floats + n_l;
        for (int c0 = 0; c0 < rows; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < rows) dst_ws[(size_t)(c0 + j) * TILE_N] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) mbar_arrive(bar(BAR_ACC_EMPTY));
          else mbar_arrive_remote(acc_empty_leader);
          atomicAdd(p.ws_flags + blockIdx.x, 1u);
        }
        continue;
      }
      // The other parts of a cut tile belong to the CTAs of the same rank in the following pairs: every
      // pair whose (non-empty) range starts before the tile ends.  Ranges shorter than a tile give a tile
      // several such parts (the split-K of problems with fewer tiles than pairs).
      const unsigned src_slot = blockIdx.x + 2u;
      int nparts = 0;
      if (role == 2) {
        const int tile_end = (item + 1) * k_steps;
        for (int q = pair + 1; q < num_pairs; ++q) {
          const int qs = range_bound(p.total_steps, k_steps, num_pairs, q);
          if (qs >= tile_end) break;
          if (range_bound(p.total_steps, k_steps, num_pairs, q + 1) > qs) ++nparts; else break;
        }
        if (lane == 0) {
          const long long t0 = clock64();
          for (int i = 0; i < nparts; ++i) {
            while (*reinterpret_cast<volatile unsigned*>(p.ws_flags + src_slot + 2u * i) < (unsigned)kNumEpiWarps) {
              if (*abort_flag || clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_tc_error, 0, 0x320 | quarter);
                break;
              }
            }
          }
          __threadfence();
        }
        __syncwarp();
        if (*abort_flag) break;
      }
      const float* src_ws = p.ws_partials + (size_t)src_slot * tile_floats + n_l;
      for (int c0 = 0; c0 < rows; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        for (int i = 0; i < nparts; ++i) {
          // own part + the following pairs' parts, always in this order: reproducible
          const float* sq = src_ws + (size_t)(2 * i) * tile_floats + (size_t)c0 * TILE_N;
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = (c0 + j < rows) ? __ldcg(sq + (size_t)j * TILE_N) : 0.0f;
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + f[j]);
        }
        // lanes pair up (n even / odd): the even lane writes the even rows of the chunk, the odd lane the
        // odd rows, each as half2 (n even, n odd) with its partner's value alongside
        // (bulk gather mode: one row-major [256 m][128 n] block of the whole CTA, so that a row is 256
        // contiguous bytes a bulk copy can take; otherwise the warp's own [256 m][32 n] block)
        uint8_t* dst = bulk ? base_ptr + plan.out + (c0 + odd) * 256 + quarter * 64 + (lane & ~1) * 2
                            : stage + (c0 + odd) * 64 + (lane & ~1) * 2;
        const int pitch = bulk ? 256 : 64;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float mine = __uint_as_float(odd ? r[j + 1] : r[j]);
          const float give = __uint_as_float(odd ? r[j] : r[j + 1]);
          const float got = __shfl_xor_sync(0xffffffffu, give, 1);
          *reinterpret_cast<__half2*>(dst + j * pitch) = odd ? __floats2half2_rn(got, mine) : __floats2half2_rn(mine, got);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(bar(BAR_ACC_EMPTY));
        else mbar_arrive_remote(acc_empty_leader);
        // the warp that completes a slot's count (4 writers + 4 readers) puts the flag back to zero
        for (int i = 0; i < nparts; ++i)
          if (atomicAdd(p.ws_flags + src_slot + 2u * i, 1u) == (unsigned)(2 * kNumEpiWarps - 1)) p.ws_flags[src_slot + 2u * i] = 0u;
      }
      // staging -> global: one instruction moves four rows' 64-byte pieces
      const int n4 = n_tile * TILE_N + quarter * 32 + (lane & 7) * 4;  // first of this lane's 4 columns
      const bool n_ok = n4 + 3 < p.N;                                    // N is a multiple of 16
      __half2 b01 = __half2(), b23 = __half2();
      const bool add_bias = p.bias != nullptr && n_ok;
      if (add_bias) {
        b01 = *reinterpret_cast<const __half2*>(p.bias + n4);
        b23 = *reinterpret_cast<const __half2*>(p.bias + n4 + 2);
      }
      if (p.gt.world == 0) {
        __half* gdst = p.out + (size_t)(m0 + (lane >> 3)) * p.N + n4;
        for (int r0 = 0; r0 < rows; r0 += 4) {
          uint2 v = *reinterpret_cast<const uint2*>(stage + r0 * 64 + lane * 8);
          if (add_bias) {
            // the bias is added to the ROUNDED result in fp16, as a separate `output += bias` would
            __half2 lo = __hadd2(*reinterpret_cast<__half2*>(&v.x), b01), hi = __hadd2(*reinterpret_cast<__half2*>(&v.y), b23);
            v.x = *reinterpret_cast<uint32_t*>(&lo);
            v.y = *reinterpret_cast<uint32_t*>(&hi);
          }
          if (n_ok && r0 + (lane >> 3) < rows) *reinterpret_cast<uint2*>(gdst) = v;
          gdst += 4 * (size_t)p.N;
        }
      } else if (bulk) {
        // Fused all-gather with bulk copies (the default): every row of the CTA's tile (256 contiguous
        // bytes in the row-major staging block) goes to every rank's gathered buffer as one
        // cp.async.bulk of the async proxy - 256 rows x world copies per tile, spread over the 128
        // epilogue threads - instead of 16-byte stores by the threads themselves (the branch below,
        // BLKQ4_TC_GATHER_NO_BULK=1).  Measured at 8 ranks, M = 4096: 778 vs 857 us; the same at 2 ranks.
        fence_proxy_async();  // the staging writes (generic proxy) before the bulk copies read them
        if (!epi_barrier()) break;
        const int cols = min(TILE_N, p.N - n_tile * TILE_N);
        if (cols > 0) {
          const uint32_t bytes = (uint32_t)cols * 2u;
          const size_t row_bytes = (size_t)p.gt.n_total * 2;
          const size_t off0 = gather_off + ((size_t)p.gt.rank * p.N + (size_t)n_tile * TILE_N) * 2;
          for (int row = quarter * 32 + lane; row < rows; row += 32 * kNumEpiWarps) {
            const uint32_t src = smem_u32(base_ptr + plan.out + row * 256);
            const size_t off = off0 + (size_t)(m0 + row) * row_bytes;
            int r = p.gt.rank;
            for (int i = 0; i < p.gt.world; ++i) {
              r = r + 1 == p.gt.world ? 0 : r + 1;
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(p.gt.base[r] + off), "r"(src),
                           "r"(bytes)
                           : "memory");
            }
          }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the staging block may be rewritten
        if (!epi_barrier()) break;
      } else {
        // Fused all-gather: this rank's columns go straight into EVERY rank's gathered buffer
        // [M, n_total] (plain stores over NVLink for the peers), under the next tile's MMAs.  Peer
        // stores want long contiguous runs, so here the four warps wait for one another and every warp
        // then writes whole 256-byte rows of the CTA's 128 columns (16 bytes per lane, two rows per
        // instruction) instead of its own 64-byte pieces (measured at 4 ranks: 64-byte pieces held the
        // kernel at twice its compute time).
        if (!epi_barrier()) break;
        const uint8_t* stage_all = base_ptr + plan.out;
        const int c8 = (lane & 15) * 8;                               // first of this lane's 8 columns in the tile
        const bool n_ok8 = n_tile * TILE_N + c8 + 7 < p.N;            // N is a multiple of 16
        const size_t row_bytes = (size_t)p.gt.n_total * 2;
        const size_t off0 = gather_off + ((size_t)p.gt.rank * p.N + (size_t)n_tile * TILE_N + c8) * 2;
        const uint8_t* src0 = stage_all + (c8 >> 5) * (256 * 64) + (c8 & 31) * 2;
        for (int r0 = 2 * quarter; r0 < rows; r0 += 2 * kNumEpiWarps) {
          const int row = r0 + (lane >> 4);
          if (n_ok8 && row < rows) {
            const uint4 v = *reinterpret_cast<const uint4*>(src0 + row * 64);
            const size_t off = off0 + (size_t)(m0 + row) * row_bytes;
            // destinations in rotated order, starting after this rank: at any moment the ranks of a job
            // aim at different peers instead of all at the same one
            int r = p.gt.rank;
            for (int i = 0; i < p.gt.world; ++i) {
              r = r + 1 == p.gt.world ? 0 : r + 1;
              *reinterpret_cast<uint4*>(p.gt.base[r] + off) = v;
            }
          }
        }
        if (!epi_barrier()) break;  // the staging blocks are rewritten by the next tile
      }
      __syncwarp();  // the block is rewritten by the next tile
    }
    if (bulk) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // this thread's bulk copies have landed
    if (p.gt.world > 0 && !*abort_flag) {
      // Publish (the chain of the skinny kernels' exchange): storing lanes -> lane 0 of their warp,
      // warps -> the CTA's last epilogue warp (fence + shared counter), CTAs -> the grid's last CTA
      // (system fence + counter in this rank's block), which advances the local epoch and raises this
      // rank's flag in every rank's block.  One system-scope fence per CTA.
      __syncwarp();
      if (lane == 0) __threadfence_block();
      if (lane == 0 && atomicAdd(s_done, 1u) == (unsigned)kNumEpiWarps - 1u) {
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
  } else if (warp < kWeightProducerWarp) {
    // =============================== dequantizers: this CTA's 128 weight columns ===============================
    const int dw = warp - (2 + kNumEpiWarps);
    const int group = dw / kWarpsPerDeqGroup;
    const int n_l = 32 * (warp & 3) + lane;
    const int np_l = 8 * (n_l >> 4) + (n_l & 7);
    const uint32_t nib_shift = (n_l & 8) ? 8u : 0u;
    const uint32_t tmem_row = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + kAcol0;
    const uint32_t deq_full_leader = map_to_cta(bar(BAR_DEQ_FULL), 0);
    uint32_t total_its = 0;
    {
      PairWalk walk(p, pair, num_pairs);
      int item, ks0, count, role;
      while (walk.next(item, ks0, count, role)) total_its += (uint32_t)count;
    }
    for (uint32_t it = group; it < total_its; it += kDeqGroups) {
      const int s = it % kStages, d = it % kDeqStages;
      if (it >= (uint32_t)kDeqStages) {
        const uint32_t g = (it - kDeqStages) / kCommitSteps;
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
        if (rank == 0) mbar_arrive(bar(BAR_DEQ_FULL + d));
        else mbar_arrive_remote(deq_full_leader + 8u * (uint32_t)d);
        mbar_arrive(bar(BAR_PACK_FREE + s));
      }
    }
  }

  // ---- teardown: neither CTA frees tensor memory or leaves while the other may still signal it ----
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) __nanosleep(50000);  // let copies in flight land
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}
