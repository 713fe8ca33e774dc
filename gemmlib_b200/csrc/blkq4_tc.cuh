// Pieces shared by the tensor-core W4A16 kernels (one CTA per tile, and CTA pairs): tile constants,
// tcgen05 / tensor-memory PTX wrappers, operand descriptors and the dequantization of one 64-k step of
// one weight column.
#pragma once

#include <cstdint>

#include "blkq4_common.cuh"
#include "blkq4_tma.cuh"

namespace blkq4 {
namespace tc {

constexpr int TILE_N = 128;       // weight columns per CTA tile (UMMA M of one CTA)
constexpr int BLOCK_K = 64;       // k per pipeline step: one 128-byte swizzle row of fp16
constexpr int kDeqCols = BLOCK_K / 2;  // TMEM columns of one dequantized stage: 2 fp16 per column
constexpr int kPackTileBytes = (TILE_N / 2) * BLOCK_K;  // 4 KB: 64 packed columns x 64 bytes
constexpr int kScaleTileBytes = 1024;
constexpr int kZpTileBytes = 512;

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// First operand from tensor memory: 128 lanes (rows) x 8 columns per 16 k, two fp16 per column.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The four MMAs of one 64-k step: operand A advances 8 TMEM columns, operand B two
// descriptor units (32 bytes) per 16 k.  Only the first may overwrite the accumulator.
__device__ __forceinline__ void umma_f16_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 b0, b1, b2, b3;\n\t.reg .b32 l1, l2, l3, a1, a2, a3;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "add.u32 l1, %2, 2;\n\tadd.u32 l2, %2, 4;\n\tadd.u32 l3, %2, 6;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "mov.b64 b0, {%2, %3};\n\tmov.b64 b1, {l1, %3};\n\tmov.b64 b2, {l2, %3};\n\tmov.b64 b3, {l3, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], b0, %4, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %4, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %4, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %4, q;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
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


// One 64-k step of weight column n_l of a tile: reads the column's 64 packed bytes (`pk`, already
// pointing at the packed column; `nib_shift` 0 or 8 selects which of the two columns sharing the bytes
// this thread owns), the step's scale / zero-point tile, and produces the 32 fp16 pairs of the
// dequantized stage: out[j] = k pair (2j, 2j + 1).  Numerics are the reference kernel's: fp16(16 + q)
// by bit placement, then fma.rn.f16 with rn(scale * (-16 - zp)).
template <bool COLWISE>
__device__ __forceinline__ void dequant_step(const uint8_t* pk, const uint8_t* sc_tile, const uint8_t* zp_tile,
                                             int n_l, uint32_t nib_shift, int block, int block_shift, int has_zp,
                                             uint32_t (&out)[32]) {
  const uint32_t rot_lo = nib_shift ? 30u : 6u, rot_hi = nib_shift ? 26u : 2u;
#pragma unroll
  for (int c = 0; c < 4; ++c) {  // 16-byte chunk: k in [16 c, 16 c + 16)
    const uint4 wv = *reinterpret_cast<const uint4*>(pk + c * 16);
    const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
    // scale / offset half2 for the k pairs (2r, 2r+1) [lo] and (2r+8, 2r+9) [hi] of word r
    uint32_t s_lo[4], s_hi[4], o_lo[4], o_hi[4];
    if (COLWISE) {
      // scale tile: meta_rows x 128 fp16; the 16 k of a chunk share one block
      const int mr = (block >= BLOCK_K) ? 0 : ((c * 16) >> block_shift);
      const uint32_t sc = reinterpret_cast<const unsigned short*>(sc_tile)[mr * TILE_N + n_l];
      const uint32_t z = has_zp ? (uint32_t)zp_tile[mr * TILE_N + n_l] : 8u;
      const uint32_t sc2 = sc | (sc << 16);
      // fp16(-16 - z) by bit placement (0xcc00 is -16.0, mantissa step 1/64), times the scale
      const uint32_t nz = 0xcc00u | (z << 6);
      const uint32_t of2 = hmul2_u32(sc2, nz | (nz << 16));
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        s_lo[r] = s_hi[r] = sc2;
        o_lo[r] = o_hi[r] = of2;
      }
    } else {
      // scale tile: (128 / block) rows x 64 k fp16, k permuted per 16 as
      // 0 1 8 9 2 3 10 11 ...; zero points 0 8 1 9 2 10 3 11 ...
      const int mr = n_l / block;
      const uint4* sp = reinterpret_cast<const uint4*>(sc_tile + mr * 128 + c * 32);
      const uint4 s0 = sp[0], s1 = sp[1];
      const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      uint4 zv = make_uint4(0x08080808u, 0x08080808u, 0x08080808u, 0x08080808u);
      if (has_zp) zv = *reinterpret_cast<const uint4*>(zp_tile + mr * 64 + c * 16);
      const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        s_lo[r] = sw[2 * r];
        s_hi[r] = sw[2 * r + 1];
        const uint32_t nz_lo = ((zw[r] << 6) & 0x03c003c0u) | 0xcc00cc00u;  // fp16(-16 - z)
        const uint32_t nz_hi = ((zw[r] >> 2) & 0x03c003c0u) | 0xcc00cc00u;
        o_lo[r] = hmul2_u32(sw[2 * r], nz_lo);
        o_hi[r] = hmul2_u32(sw[2 * r + 1], nz_hi);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      // Column n0's nibbles sit at bits 0-3 / 16-19 (k = 2r, 2r+1) and 4-7 / 20-23 (k = 2r+8, 2r+9), column
      // n0 + 8's eight bits further up; fp16(16 + q) by bit placement needs them at bits 6-9 / 22-25.  One
      // rotation per operand does it (instead of a shift to this thread's nibbles and a second one into
      // place): left by 6 / 2 for n0, by 30 / 26 (= right by 2 / 6) for n0 + 8; what wraps around falls
      // outside the mask.
      const uint32_t h_lo = (__funnelshift_l(w4[r], w4[r], rot_lo) & 0x03c003c0u) | 0x4c004c00u;
      const uint32_t h_hi = (__funnelshift_l(w4[r], w4[r], rot_hi) & 0x03c003c0u) | 0x4c004c00u;
      const uint32_t d_lo = hfma2_u32(s_lo[r], h_lo, o_lo[r]);
      const uint32_t d_hi = hfma2_u32(s_hi[r], h_hi, o_hi[r]);
      // chunk c, word r: k = 16 c + 2 r (+1) -> column 8 c + r; k + 8 -> column 8 c + 4 + r
      out[8 * c + r] = d_lo;
      out[8 * c + 4 + r] = d_hi;
    }
  }
}

}  // namespace tc
}  // namespace blkq4
