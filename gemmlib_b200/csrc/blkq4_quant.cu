// Fused blockwise 4-bit quantization + prepack for sm_100a.
//
// One kernel per call replaces the reference's three (block_quantize_kernel,
// prepack_weights_kernel, prepack_scales_kernel; reference
// src/mickey/blk_q4/f16_quant_sm80.cuh:593-653) and its three temporary device
// buffers (src/blkq4_f16_gemm_sm80.cu:282-290).  It is memory bound: every fp16
// weight is read from HBM once (16-byte loads along K) and the packed bytes, scales
// and zero points are written once in their final order.  Output bytes are
// bit-identical to the reference's.  Two kernels:
//
// quant_prepack_colwise_kernel<BLOCK> - column-wise blocks with 16-byte aligned rows
// (the benchmark configurations): one thread per 16-byte packed chunk (16 k of the
// columns n0 and n0 + 8), everything in registers, the block's range by shuffles over
// the BLOCK / 16 neighbouring lanes, no shared memory.
//
// quant_prepack_kernel<BLOCK, COLWISE> - row-wise blocks and unaligned inputs: a CTA
// owns a TK x TN tile of the K x N weight.  Phases, separated by __syncthreads():
//   1. load the tile into shared memory
//   2. min/max of every 16-element segment of a quantization block
//   3. combine segments per block -> fp16 scale, zero point, fp32 reciprocal
//   4. quantize and emit one 16-byte packed chunk per thread (16 k x 2 n);
//      copy the tile's meta out in prepacked order
#include "blkq4_common.cuh"

namespace blkq4 {
namespace {

constexpr int kThreads = 256;
constexpr int kTileElems = 8192;  // TK * TN

template <int BLOCK, bool COLWISE>
struct QuantTile {
  // Column-wise blocks of 128 need 128 rows of K in the tile; everything else
  // uses 64 x 128 (row-wise blocks of 128 need 128 columns).
  static constexpr int TK = (COLWISE && BLOCK == 128) ? 128 : 64;
  static constexpr int TN = kTileElems / TK;
  static constexpr int PITCH = TK + 8;  // halves; keeps rows 16-byte aligned
  static constexpr int BK = COLWISE ? BLOCK : 1;
  static constexpr int BN = COLWISE ? 1 : BLOCK;
  static constexpr int SEGS = kTileElems / 16;            // 512
  static constexpr int SEGS_PER_BLOCK = BLOCK / 16;       // 1, 2, 4, 8
  static constexpr int BLOCKS = kTileElems / BLOCK;       // quant blocks per tile
  static constexpr int MR = TK / BK;                      // meta rows in tile
  static constexpr int MC = TN / BN;                      // meta columns in tile
};

// Scale and zero point from a block's range.  Same float operation sequence as
// the reference's range2scalezp (f16_quant_sm80.cuh:96-122): IEEE division,
// roundf (halves away from zero), clamp to [0, 15], fp32 -> fp16 round-to-nearest.
__device__ __forceinline__ void range_to_scale_zp(float mn, float mx, __half& scale, uint8_t& zp) {
  mn = fminf(mn, 0.0f);
  mx = fmaxf(mx, 0.0f);
  const float scale_f = __fdiv_rn(mx - mn, 15.0f);
  float zpf = mn;
  if (scale_f != 0.0f) zpf = 0.0f - __fdiv_rn(mn, scale_f);
  if (zpf < 0.0f) {
    zp = 0;
  } else if (zpf > 15.0f) {
    zp = 15;
  } else {
    zp = (uint8_t)roundf(zpf);
  }
  scale = __float2half_rn(scale_f);
}

// Symmetric case, reference range2scale (f16_quant_sm80.cuh:124-135): the
// extreme of larger magnitude, sign kept, over -8.  The reference scans a block
// sequentially with "v < min", so for an all-zero block its min is the first
// element it meets, sign of zero included; `first` reproduces that.
__device__ __forceinline__ __half range_to_scale(float mn, float mx, float first) {
  float m = fabsf(mx) > fabsf(mn) ? mx : mn;
  if (mn == 0.0f && mx == 0.0f) m = first;
  return __float2half_rn(__fdiv_rn(m, -8.0f));
}

// q = clamp(roundf(v * r + zp), 0, 15).  The reference's expression
// (f16_quant_sm80.cuh:295-296) is compiled by nvcc with its default fused
// multiply-add contraction; the fma is explicit here.  roundf (halves away from zero)
// commutes with the clamp because 0 and 15 are integers, and for x in [0, 15] it equals
// trunc(x + 0.5) when the addition rounds toward zero (the sum can then never be pushed
// up to the next integer), which is two instructions instead of a library call.
__device__ __forceinline__ uint32_t quantize_one(float v, float r, float zp) {
  float x = __fmaf_rn(v, r, zp);
  x = fmaxf(0.0f, fminf(15.0f, x));
  return (uint32_t)__float2int_rz(__fadd_rz(x, 0.5f));
}

// quantize_one for two values at once (sm_100a packed fp32 arithmetic).
__device__ __forceinline__ unsigned long long pack_f32x2(float x, float y) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
  return r;
}
__device__ __forceinline__ void quantize_two(float2 v, unsigned long long r2, unsigned long long zp2, uint32_t& q0,
                                             uint32_t& q1) {
  unsigned long long x;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(x) : "l"(pack_f32x2(v.x, v.y)), "l"(r2), "l"(zp2));
  asm("add.rz.f32x2 %0, %1, %2;" : "=l"(x) : "l"(x), "l"(pack_f32x2(0.5f, 0.5f)));
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(x));
  uint32_t ua, ub;
  asm("cvt.rzi.u32.f32 %0, %1;" : "=r"(ua) : "f"(a));  // negative -> 0
  asm("cvt.rzi.u32.f32 %0, %1;" : "=r"(ub) : "f"(b));
  q0 = min(ua, 15u);
  q1 = min(ub, 15u);
}

template <int BLOCK, bool COLWISE>
__global__ void __launch_bounds__(kThreads)
quant_prepack_kernel(const __half* __restrict__ w, int K, int N, int ld, bool vec_ok,
                     uint8_t* __restrict__ packed, __half* __restrict__ scales,
                     uint8_t* __restrict__ zps) {
  using T = QuantTile<BLOCK, COLWISE>;
  constexpr int TK = T::TK, TN = T::TN, PITCH = T::PITCH;

  __shared__ __align__(16) __half s_w[TN * PITCH];
  __shared__ float s_min[T::SEGS];
  __shared__ float s_max[T::SEGS];
  __shared__ float s_recip[T::BLOCKS];
  __shared__ __half s_scale[T::BLOCKS];
  __shared__ uint8_t s_zp[T::BLOCKS];

  const int tid = threadIdx.x;
  const int k0 = blockIdx.x * TK;
  const int n0 = blockIdx.y * TN;
  const bool has_zp = zps != nullptr;

  // ---- 1. tile -> shared memory (columns past N read as zero) ----
  constexpr int CHUNKS_PER_COL = TK / 8;
  for (int idx = tid; idx < TN * CHUNKS_PER_COL; idx += kThreads) {
    const int col = idx / CHUNKS_PER_COL, ch = idx % CHUNKS_PER_COL;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n0 + col < N) {
      const __half* src = w + (size_t)(n0 + col) * ld + k0 + ch * 8;
      if (vec_ok) {
        v = __ldg(reinterpret_cast<const uint4*>(src));
      } else {
        const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src);
        v.x = s16[0] | ((uint32_t)s16[1] << 16);
        v.y = s16[2] | ((uint32_t)s16[3] << 16);
        v.z = s16[4] | ((uint32_t)s16[5] << 16);
        v.w = s16[6] | ((uint32_t)s16[7] << 16);
      }
    }
    *reinterpret_cast<uint4*>(&s_w[col * PITCH + ch * 8]) = v;
  }
  __syncthreads();

  // ---- 2. min/max per 16-element segment ----
  // Column-wise: segment = 16 consecutive k of one column; segments of a block
  // are consecutive.  Row-wise: segment = 16 consecutive n at one k; index
  // seg = k * (TN/16) + n_group so that a block's segments are consecutive too.
  for (int seg = tid; seg < T::SEGS; seg += kThreads) {
    float mn = __FLT_MAX__, mx = -__FLT_MAX__;
    if constexpr (COLWISE) {
      const int col = seg / (TK / 16), sk = seg % (TK / 16);
      const uint4* p = reinterpret_cast<const uint4*>(&s_w[col * PITCH + sk * 16]);
      const uint4 v0 = p[0], v1 = p[1];
      const __half2* h0 = reinterpret_cast<const __half2*>(&v0);
      const __half2* h1 = reinterpret_cast<const __half2*>(&v1);
      // fp16 min/max are exact; NaNs are skipped as in the reference's "v < min" scan
      __half2 mn2 = __hmin2(h0[0], h1[0]), mx2 = __hmax2(h0[0], h1[0]);
#pragma unroll
      for (int i = 1; i < 4; ++i) {
        mn2 = __hmin2(mn2, __hmin2(h0[i], h1[i]));
        mx2 = __hmax2(mx2, __hmax2(h0[i], h1[i]));
      }
      const float2 fmn = __half22float2(mn2), fmx = __half22float2(mx2);
      mn = fminf(fmn.x, fmn.y);
      mx = fmaxf(fmx.x, fmx.y);
    } else {
      const int k = seg / (TN / 16), ng = seg % (TN / 16);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float v = __half2float(s_w[(ng * 16 + i) * PITCH + k]);
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
    }
    s_min[seg] = mn;
    s_max[seg] = mx;
  }
  __syncthreads();

  // ---- 3. one thread per quantization block ----
  // Block index b: column-wise b = col * MR + kb; row-wise b = k * MC + nb.
  for (int b = tid; b < T::BLOCKS; b += kThreads) {
    float mn = s_min[b * T::SEGS_PER_BLOCK], mx = s_max[b * T::SEGS_PER_BLOCK];
#pragma unroll
    for (int i = 1; i < T::SEGS_PER_BLOCK; ++i) {
      mn = fminf(mn, s_min[b * T::SEGS_PER_BLOCK + i]);
      mx = fmaxf(mx, s_max[b * T::SEGS_PER_BLOCK + i]);
    }
    __half sc;
    uint8_t zp = 8;
    if (has_zp) {
      range_to_scale_zp(mn, mx, sc, zp);
    } else {
      float first;
      if constexpr (COLWISE) {
        first = __half2float(s_w[(b / T::MR) * PITCH + (b % T::MR) * BLOCK]);
      } else {
        first = __half2float(s_w[((b % T::MC) * BLOCK) * PITCH + b / T::MC]);
      }
      sc = range_to_scale(mn, mx, first);
    }
    const float s = __half2float(sc);
    s_scale[b] = sc;
    s_zp[b] = zp;
    s_recip[b] = (s != 0.0f) ? __fdiv_rn(1.0f, s) : 0.0f;
  }
  __syncthreads();

  // ---- 4a. quantize + emit packed chunks ----
  // Chunk (np_l, kc): 16 bytes at packed[(np0 + np_l) * K + k0 + 16 kc], holding
  // k in [16 kc, 16 kc + 16) of columns na = 16 (np_l / 8) + np_l % 8 and na + 8.
  // Byte 4 row + sub = q[2 row + (sub >> 1), sub & 1 ? nb : na]
  //                  | q[the same k + 8, same n] << 4.
  // Reference: dev_prepack_weights, f16_quant_sm80.cuh:362-417.
  constexpr int KCH = TK / 16;
  for (int c = tid; c < (TN / 2) * KCH; c += kThreads) {
    const int np_l = c / KCH, kc = c % KCH;
    const int na = 16 * (np_l / 8) + (np_l % 8);
    if (n0 + na >= N) continue;  // N % 16 == 0: the whole 16-column group is out
    uint4 va[2], vb[2];
    va[0] = *reinterpret_cast<const uint4*>(&s_w[na * PITCH + kc * 16]);
    va[1] = *reinterpret_cast<const uint4*>(&s_w[na * PITCH + kc * 16 + 8]);
    vb[0] = *reinterpret_cast<const uint4*>(&s_w[(na + 8) * PITCH + kc * 16]);
    vb[1] = *reinterpret_cast<const uint4*>(&s_w[(na + 8) * PITCH + kc * 16 + 8]);
    const __half* ha = reinterpret_cast<const __half*>(va);
    const __half* hb = reinterpret_cast<const __half*>(vb);
    uint32_t qa[16], qb[16];
    if constexpr (COLWISE) {
      const int kb = (kc * 16) / BLOCK;
      const int ba = na * T::MR + kb, bb = (na + 8) * T::MR + kb;
      const float ra = s_recip[ba], rb = s_recip[bb];
      const float za = (float)s_zp[ba], zb = (float)s_zp[bb];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        qa[i] = quantize_one(__half2float(ha[i]), ra, za);
        qb[i] = quantize_one(__half2float(hb[i]), rb, zb);
      }
    } else {
      const int nb = na / BLOCK;  // na and na + 8 share a row-wise block
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int b = (kc * 16 + i) * T::MC + nb;
        const float r = s_recip[b], z = (float)s_zp[b];
        qa[i] = quantize_one(__half2float(ha[i]), r, z);
        qb[i] = quantize_one(__half2float(hb[i]), r, z);
      }
    }
    uint32_t out[4];
#pragma unroll
    for (int row = 0; row < 4; ++row) {
      out[row] = (qa[2 * row] | (qa[2 * row + 8] << 4)) |
                 ((qb[2 * row] | (qb[2 * row + 8] << 4)) << 8) |
                 ((qa[2 * row + 1] | (qa[2 * row + 9] << 4)) << 16) |
                 ((qb[2 * row + 1] | (qb[2 * row + 9] << 4)) << 24);
    }
    uint8_t* dst = packed + (size_t)(n0 / 2 + np_l) * K + k0 + kc * 16;
    *reinterpret_cast<uint4*>(dst) = make_uint4(out[0], out[1], out[2], out[3]);
  }

  // ---- 4b. meta in prepacked order (reference dev_prepack_scales, :457-547) ----
  if constexpr (COLWISE) {
    // row-major [K/BLOCK, N]
    for (int i = tid; i < T::MR * TN; i += kThreads) {
      const int kb = i / TN, col = i % TN;
      if (n0 + col >= N) continue;
      const size_t g = (size_t)(k0 / BLOCK + kb) * N + n0 + col;
      scales[g] = s_scale[col * T::MR + kb];
      if (has_zp) zps[g] = s_zp[col * T::MR + kb];
    }
  } else {
    // column-major [K, N/BLOCK]; inside every 16 rows destination position d
    // takes source row  scales: 2t + {0,1,8,9}[j],  zero points: 2t + {0,8,1,9}[j]
    // with t = d / 4, j = d % 4.
    for (int i = tid; i < TK * T::MC; i += kThreads) {
      const int nb = i / TK, d = i % TK;
      if (n0 + nb * BLOCK >= N) continue;
      const int g16 = d & ~15, t = (d & 15) >> 2, j = d & 3;
      const int src_s = g16 + 2 * t + (j & 1) + 8 * (j >> 1);
      const int src_z = g16 + 2 * t + (j >> 1) + 8 * (j & 1);
      const size_t g = (size_t)(n0 / BLOCK + nb) * K + k0 + d;
      scales[g] = s_scale[src_s * T::MC + nb];
      if (has_zp) zps[g] = s_zp[src_z * T::MC + nb];
    }
  }
}

// Column-wise blocks, 16-byte aligned rows: one thread per 16-byte packed chunk, everything in
// registers.  A chunk holds 16 consecutive k of columns na and na + 8, i.e. 32 contiguous bytes of
// each of two weight rows; the BLOCK / 16 lanes that share a quantization block are neighbours in
// the warp, so a block's range is a shuffle reduction.  No shared memory, no block-wide barrier:
// the kernel is a stream of independent 128-bit loads and stores.  Same arithmetic as the tiled
// kernel (range_to_scale_zp / range_to_scale / quantize_one), hence the same bits.
template <int BLOCK>
__global__ void __launch_bounds__(kThreads)
quant_prepack_colwise_kernel(const __half* __restrict__ w, int K, int N, int ld, uint8_t* __restrict__ packed,
                             __half* __restrict__ scales, uint8_t* __restrict__ zps) {
  constexpr int G = BLOCK / 16;  // lanes per quantization block: 1, 2, 4, 8
  const int kch = K / 16;        // chunks per packed column
  const long long total = (long long)(N / 2) * kch;
  const long long c_raw = (long long)blockIdx.x * kThreads + threadIdx.x;
  const bool valid = c_raw < total;
  const long long c = valid ? c_raw : total - 1;  // every lane stays for the shuffles
  const int np = (int)(c / kch), kc = (int)(c - (long long)np * kch);
  const int na = 16 * (np / 8) + (np % 8);
  const bool has_zp = zps != nullptr;
  const int lane = threadIdx.x & 31;

  const uint4* pa = reinterpret_cast<const uint4*>(w + (size_t)na * ld + kc * 16);
  const uint4* pb = reinterpret_cast<const uint4*>(w + (size_t)(na + 8) * ld + kc * 16);
  uint4 va[2], vb[2];
  va[0] = __ldg(pa);
  va[1] = __ldg(pa + 1);
  vb[0] = __ldg(pb);
  vb[1] = __ldg(pb + 1);
  const __half* ha = reinterpret_cast<const __half*>(va);
  const __half* hb = reinterpret_cast<const __half*>(vb);

  // range of the 16 values of each column (fp16 min/max are exact; NaNs are skipped as in the
  // reference's "v < min" scan), then of the whole block across its G lanes
  auto range16 = [](const uint4 (&v)[2], float& mn, float& mx) {
    const __half2* h0 = reinterpret_cast<const __half2*>(&v[0]);
    const __half2* h1 = reinterpret_cast<const __half2*>(&v[1]);
    __half2 mn2 = __hmin2(h0[0], h1[0]), mx2 = __hmax2(h0[0], h1[0]);
#pragma unroll
    for (int i = 1; i < 4; ++i) {
      mn2 = __hmin2(mn2, __hmin2(h0[i], h1[i]));
      mx2 = __hmax2(mx2, __hmax2(h0[i], h1[i]));
    }
    const float2 fmn = __half22float2(mn2), fmx = __half22float2(mx2);
    mn = fminf(fmn.x, fmn.y);
    mx = fmaxf(fmx.x, fmx.y);
  };
  float mna, mxa, mnb, mxb;
  range16(va, mna, mxa);
  range16(vb, mnb, mxb);
#pragma unroll
  for (int o = 1; o < G; o <<= 1) {
    mna = fminf(mna, __shfl_xor_sync(0xffffffffu, mna, o));
    mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, o));
    mnb = fminf(mnb, __shfl_xor_sync(0xffffffffu, mnb, o));
    mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, o));
  }
  // first element of the block (the symmetric all-zero case keeps its sign of zero)
  const int lead = lane & ~(G - 1);
  const float first_a = __shfl_sync(0xffffffffu, __half2float(ha[0]), lead);
  const float first_b = __shfl_sync(0xffffffffu, __half2float(hb[0]), lead);

  __half sca, scb;
  uint8_t zpa = 8, zpb = 8;
  if (has_zp) {
    range_to_scale_zp(mna, mxa, sca, zpa);
    range_to_scale_zp(mnb, mxb, scb, zpb);
  } else {
    sca = range_to_scale(mna, mxa, first_a);
    scb = range_to_scale(mnb, mxb, first_b);
  }
  const float sa = __half2float(sca), sb = __half2float(scb);
  const float ra = (sa != 0.0f) ? __fdiv_rn(1.0f, sa) : 0.0f;
  const float rb = (sb != 0.0f) ? __fdiv_rn(1.0f, sb) : 0.0f;
  const float za = (float)zpa, zb = (float)zpb;

  // Two values per instruction (fma.rn.f32x2 / add.rz.f32x2 are the same IEEE operations as the
  // scalar ones in quantize_one); the clamp moves behind the conversion: trunc(x + 0.5) saturated
  // at 0 by the conversion to unsigned, then min(., 15) - the same integer for every non-NaN x.
  uint32_t qa[16], qb[16];
  const unsigned long long ra2 = pack_f32x2(ra, ra), za2 = pack_f32x2(za, za);
  const unsigned long long rb2 = pack_f32x2(rb, rb), zb2 = pack_f32x2(zb, zb);
  const __half2* ha2 = reinterpret_cast<const __half2*>(va);
  const __half2* hb2 = reinterpret_cast<const __half2*>(vb);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    quantize_two(__half22float2(ha2[i]), ra2, za2, qa[2 * i], qa[2 * i + 1]);
    quantize_two(__half22float2(hb2[i]), rb2, zb2, qb[2 * i], qb[2 * i + 1]);
  }
  // Byte 4 row + sub = q[2 row + (sub >> 1), sub & 1 ? nb : na] | q[the same k + 8, same n] << 4
  // (reference dev_prepack_weights, f16_quant_sm80.cuh:362-417).
  uint32_t out[4];
#pragma unroll
  for (int row = 0; row < 4; ++row) {
    out[row] = (qa[2 * row] | (qa[2 * row + 8] << 4)) |
               ((qb[2 * row] | (qb[2 * row + 8] << 4)) << 8) |
               ((qa[2 * row + 1] | (qa[2 * row + 9] << 4)) << 16) |
               ((qb[2 * row + 1] | (qb[2 * row + 9] << 4)) << 24);
  }
  if (!valid) return;
  *reinterpret_cast<uint4*>(packed + (size_t)np * K + kc * 16) = make_uint4(out[0], out[1], out[2], out[3]);
  if (lane == lead) {
    // meta row-major [K / BLOCK, N] (reference dev_prepack_scales, column-wise branch)
    const size_t g = (size_t)((kc * 16) / BLOCK) * N + na;
    scales[g] = sca;
    scales[g + 8] = scb;
    if (has_zp) {
      zps[g] = zpa;
      zps[g + 8] = zpb;
    }
  }
}

template <int BLOCK, bool COLWISE>
void launch_T(int K, int N, int ld, cudaStream_t stream, const __half* w, uint8_t* packed,
              __half* scales, uint8_t* zp) {
  using T = QuantTile<BLOCK, COLWISE>;
  if constexpr (COLWISE) {
    if ((reinterpret_cast<uintptr_t>(w) % 16 == 0) && (ld % 8 == 0)) {
      const long long total = (long long)(N / 2) * (K / 16);
      quant_prepack_colwise_kernel<BLOCK><<<(unsigned)((total + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
          w, K, N, ld, packed, scales, zp);
      return;
    }
  }
  dim3 grid(K / T::TK, (N + T::TN - 1) / T::TN);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(w) % 16 == 0) && (ld % 8 == 0);
  quant_prepack_kernel<BLOCK, COLWISE>
      <<<grid, kThreads, 0, stream>>>(w, K, N, ld, vec_ok, packed, scales, zp);
}

}  // namespace

std::string launch_quant_prepack(int block, bool colwise, int K, int N, int ld,
                                 cudaStream_t stream, const __half* w, uint8_t* packed,
                                 __half* scales, uint8_t* zp) {
#define BLKQ4_CASE(B)                                                   \
  case B:                                                               \
    if (colwise)                                                        \
      launch_T<B, true>(K, N, ld, stream, w, packed, scales, zp);       \
    else                                                                \
      launch_T<B, false>(K, N, ld, stream, w, packed, scales, zp);      \
    break;
  switch (block) {
    BLKQ4_CASE(16)
    BLKQ4_CASE(32)
    BLKQ4_CASE(64)
    BLKQ4_CASE(128)
    default:
      return "Unsupported block size: " + std::to_string(block);
  }
#undef BLKQ4_CASE
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return std::string("Kernel launch failed: ") + cudaGetErrorString(e);
  return std::string();
}

}  // namespace blkq4
