// Skinny W4A16 kernel (M <= 16) for sm_100a: out[M,N] = A[M,K] x dequant(W4[K,N]).
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
#include "blkq4_common.cuh"

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

constexpr int kMaxWarps = 16;

// NT: 16-column tiles per warp.  MT: 8-row groups of activations (1: M <= 8, 2: M <= 16).
// U:  64-k steps loaded together; U * NT 16-byte weight loads are in flight per lane.
template <int NT, int MT, int U, bool COLWISE>
__global__ void __launch_bounds__(kMaxWarps * 32)
gemv_kernel(const __half* __restrict__ a, const uint8_t* __restrict__ packed,
            const __half* __restrict__ scales, const uint8_t* __restrict__ zps,
            __half* __restrict__ out, int M, int N, int K, int block) {
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

  // Two register buffers of U * NT weight chunks; the next group is requested
  // before the current one is consumed.  (Two named arrays, not one indexed by a
  // runtime value, so that they stay in registers.)
  uint4 wv_a[U][NT], wv_b[U][NT];
  auto load_group = [&](uint4 (&wv)[U][NT], int step0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int step = min(step0 + u, step_end - 1);
      const int chunk = step * 4 + t;
#pragma unroll
      for (int i = 0; i < NT; ++i) wv[u][i] = ldg_stream_v4(wcol[i] + (size_t)chunk * 16);
    }
  };

  auto compute_group = [&](const uint4 (&wv)[U][NT], int step0) {
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
        const uint32_t w4[4] = {wv[u][i].x, wv[u][i].y, wv[u][i].z, wv[u][i].w};

        // Per word r: scale/offset half2 for the k pairs (2r, 2r+1) [lo] and
        // (2r+8, 2r+9) [hi], for column na (a) and na + 8 (b).
        uint32_t s_lo_a[4], s_hi_a[4], o_lo_a[4], o_hi_a[4];
        uint32_t s_lo_b[4], s_hi_b[4], o_lo_b[4], o_hi_b[4];
        if constexpr (COLWISE) {
          // meta row-major [K/block, N]; the 16 k of a chunk share one block
          const size_t mi = (size_t)((chunk * 16) / block) * N + na;
          const __half sa = scales[mi], sb = scales[mi + 8];
          const int za = zps ? zps[mi] : 8, zb = zps ? zps[mi + 8] : 8;
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
          // meta column-major [K, N/block], 16-row groups permuted so that
          // positions 4r..4r+3 hold k = 2r, 2r+1, 2r+8, 2r+9 (scales) and
          // 2r, 2r+8, 2r+1, 2r+9 (zero points).  na and na + 8 share a block.
          const size_t mi = (size_t)(na / block) * K + (size_t)chunk * 16;
          const uint4* sp = reinterpret_cast<const uint4*>(scales + mi);
          const uint4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
          const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          uint4 zv = make_uint4(0x08080808u, 0x08080808u, 0x08080808u, 0x08080808u);
          if (zps) zv = __ldg(reinterpret_cast<const uint4*>(zps + mi));
          const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            s_lo_a[r] = s_lo_b[r] = sw[2 * r];
            s_hi_a[r] = s_hi_b[r] = sw[2 * r + 1];
            // fp16(-16 - z) by the same bit trick: 0xcc00 is -16.0
            const uint32_t nz_lo = ((zw[r] << 6) & 0x03c003c0u) | 0xcc00cc00u;
            const uint32_t nz_hi = ((zw[r] >> 2) & 0x03c003c0u) | 0xcc00cc00u;
            o_lo_a[r] = o_lo_b[r] = hmul2_u32(sw[2 * r], nz_lo);
            o_hi_a[r] = o_hi_b[r] = hmul2_u32(sw[2 * r + 1], nz_hi);
          }
        }

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

  if (step_beg < step_end) load_group(wv_a, step_beg);
  for (int step0 = step_beg; step0 < step_end; step0 += 2 * U) {
    if (step0 + U < step_end) load_group(wv_b, step0 + U);
    compute_group(wv_a, step0);
    if (step0 + 2 * U < step_end) load_group(wv_a, step0 + 2 * U);
    if (step0 + U < step_end) compute_group(wv_b, step0 + U);
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
    if (tile < ntiles && m < M) out[(size_t)m * N + n] = __float2half_rn(sum);
  }
}

template <int NT, int MT, int U, bool COLWISE>
cudaError_t launch_T(int warps, int M, int N, int K, int block, cudaStream_t stream,
                     const __half* a, const uint8_t* packed, const __half* scales,
                     const uint8_t* zp, __half* out) {
  const int ntiles = N / 16;
  const int grid = (ntiles + NT - 1) / NT;
  const size_t smem = (size_t)warps * NT * MT * 4 * 32 * sizeof(float);
  auto kern = gemv_kernel<NT, MT, U, COLWISE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, warps * 32, smem, stream>>>(a, packed, scales, zp, out, M, N, K, block);
  return cudaGetLastError();
}

}  // namespace

std::string launch_gemv(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                        const __half* a, const uint8_t* packed, const __half* scales,
                        const uint8_t* zp, __half* out) {
  if (M < 1 || M > 16) return "skinny kernel needs 1 <= M <= 16";
  // Warps per CTA = K splits.  Each warp should see at least four 64-k steps.
  const int steps = K / 64;
  int warps = 8;
  while (warps > 1 && steps / warps < 4) warps >>= 1;
  cudaError_t e;
  if (M <= 8) {
    e = colwise ? launch_T<1, 1, 4, true>(warps, M, N, K, block, stream, a, packed, scales, zp, out)
                : launch_T<1, 1, 4, false>(warps, M, N, K, block, stream, a, packed, scales, zp, out);
  } else {
    e = colwise ? launch_T<2, 2, 2, true>(warps, M, N, K, block, stream, a, packed, scales, zp, out)
                : launch_T<2, 2, 2, false>(warps, M, N, K, block, stream, a, packed, scales, zp, out);
  }
  if (e != cudaSuccess) return std::string(cudaGetErrorString(e));
  return std::string();
}

}  // namespace blkq4
