/*
 * CPU oracle for the blockwise-int4 W4A16 path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm of the reference library
 * (chenfucn/gemmlib).  It is the checker the CUDA kernels are compared with; it
 * is never linked into, or called from, the shipped library.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may use it.
 *
 * Each function cites the reference file:line it follows.  The restatement is
 * pinned two ways: against the reference's own host prepack helpers compiled
 * from their sources (oracle/_ref/libblkq4_ref_host.so), and against the
 * reference tests' known-answer generator with its round-trip identity
 * quantize(dequantize(q, s, z)) == (q, s, z).
 *
 * Conventions (reference include/ms_blkq4gemm.h and
 * src/mickey/blk_q4/f16_quant_sm80.cuh:151-198):
 *   W          K x N weight, column-major, leading dimension ld >= K, fp16
 *              (a PyTorch Linear.weight [N, K] row-major is exactly this).
 *   bk, bn     quantization block extent along K and N: (block, 1) when
 *              column-wise, (1, block) when row-wise.
 *   meta       (K/bk) x (N/bn) scales (fp16) and zero points (one 4-bit value
 *              per uint8_t).
 *   "plain"    the quantizer's first-stage output: bytes column-major [K/2, N],
 *              low nibble = even k; meta column-major.
 *   "packed"   the layout the GEMM consumes: weight bytes column-major
 *              [K, N/2]; meta row-major [K/bk, N] when column-wise, permuted
 *              column-major [K, N/bn] when row-wise.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t h) {
  f16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f2h(float f) {
  f16 v = (f16)f; /* round to nearest even, as __float2half_rn */
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}

int blkq4_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a timed baseline sets its thread count itself. */
void blkq4_oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* Shape rules.  Reference: src/blkq4_f16_gemm_sm80.cu:155-203 (K % 64, N % 32,
 * empty problem) and f16_quant_sm80.cuh:190-198 (sizes).  Block 128 is accepted
 * here as an extension with the same rules (K % 128 when column-wise).  The
 * reference's divisibility test "columns % meta_shape[1]" lets through shapes
 * whose last quant block is partial (for example N = 96 with a row-wise block
 * of 64) and then writes meta out of bounds; this restatement rejects them. */
int blkq4_oracle_quant_size(int block, int colwise, int K, int N,
                            int64_t *w_bytes, int64_t *meta_elems) {
  if (block != 16 && block != 32 && block != 64 && block != 128) return -1;
  if (K <= 0 || N <= 0) return -1;
  int bk = colwise ? block : 1, bn = colwise ? 1 : block;
  if (K % 64 != 0 || K % bk != 0) return -1;
  if (N % 32 != 0 || N % bn != 0) return -1;
  *w_bytes = (int64_t)(K / 2) * N;
  *meta_elems = (int64_t)(K / bk) * (N / bn);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Scale / zero point from a block's range.
 * Reference: f16_quant_sm80.cuh:96-122 (range2scalezp). */
static void range2scalezp(float mn, float mx, uint16_t *scale, uint8_t *zp) {
  mn = mn < 0.0f ? mn : 0.0f;
  mx = mx > 0.0f ? mx : 0.0f;
  float scale_f = (mx - mn) / 15.0f;
  float zpf = mn;
  if (scale_f != 0.0f) zpf = 0.0f - mn / scale_f;
  if (zpf < 0.0f)
    *zp = 0;
  else if (zpf > 15.0f)
    *zp = 15;
  else
    *zp = (uint8_t)roundf(zpf);
  *scale = f2h(scale_f);
}

/* Reference: f16_quant_sm80.cuh:124-135 (range2scale).  The extreme of larger
 * magnitude, sign kept, divided by -8: the scale is negative when that extreme
 * is positive.  `first` is the block's first element in scan order: the
 * reference's sequential "v < min" scan keeps the first zero it meets, so an
 * all-zero block yields min == first (sign included) and scale = first / -8. */
static void range2scale(float mn, float mx, float first, uint16_t *scale) {
  float m = fabsf(mx) > fabsf(mn) ? mx : mn;
  if (mn == 0.0f && mx == 0.0f) m = first;
  *scale = f2h(m / -8.0f);
}

/* Reference: f16_quant_sm80.cuh:137-141 and :293-308.  nvcc contracts
 * v * r + zp into one fused multiply-add (its default -fmad=true); fmaf states
 * that explicitly.  roundf rounds halves away from zero on both sides. */
static inline uint8_t quant_one(float v, float r, uint8_t zp) {
  float x = roundf(fmaf(v, r, (float)zp));
  x = x < 15.0f ? x : 15.0f;
  x = x > 0.0f ? x : 0.0f;
  return (uint8_t)x;
}

/* Stage 1: blockwise quantization to the "plain" layout.
 * Reference: f16_quant_sm80.cuh:225-315 (dev_quantize_blk).
 *   q_plain     [K/2 * N] bytes, column-major [K/2, N]: q(k) | q(k+1) << 4
 *   scales_cm   [meta] fp16 bits, column-major: index n_blk * (K/bk) + k_blk
 *   zp_cm       same shape, or NULL for symmetric quantization (zp == 8) */
void blkq4_oracle_quantize_plain(int block, int colwise, int K, int N, int ld,
                                 const uint16_t *w, uint8_t *q_plain,
                                 uint16_t *scales_cm, uint8_t *zp_cm) {
  const int bk = colwise ? block : 1, bn = colwise ? 1 : block;
  const int mrows = K / bk, mcols = N / bn;
#pragma omp parallel for collapse(2) schedule(static)
  for (int mc = 0; mc < mcols; ++mc) {
    for (int mr = 0; mr < mrows; ++mr) {
      float mn = __FLT_MAX__, mx = -__FLT_MAX__;
      const float first = h2f(w[(size_t)(mc * bn) * ld + mr * bk]);
      for (int i = mr * bk; i < (mr + 1) * bk; ++i)
        for (int j = mc * bn; j < (mc + 1) * bn; ++j) {
          float v = h2f(w[(size_t)j * ld + i]);
          if (v < mn) mn = v;
          if (v > mx) mx = v;
        }
      size_t mi = (size_t)mc * mrows + mr;
      if (zp_cm)
        range2scalezp(mn, mx, &scales_cm[mi], &zp_cm[mi]);
      else
        range2scale(mn, mx, first, &scales_cm[mi]);
    }
  }
#pragma omp parallel for schedule(static)
  for (int j = 0; j < N; ++j) {
    for (int i = 0; i < K; i += 2) {
      uint8_t q[2];
      for (int e = 0; e < 2; ++e) {
        size_t mi = (size_t)(j / bn) * mrows + (i + e) / bk;
        float s = h2f(scales_cm[mi]);
        uint8_t zp = zp_cm ? zp_cm[mi] : 8;
        float r = s != 0.0f ? 1.0f / s : 0.0f;
        q[e] = quant_one(h2f(w[(size_t)j * ld + i + e]), r, zp);
      }
      q_plain[(size_t)j * (K / 2) + i / 2] = (uint8_t)((q[0] & 0xf) | (q[1] << 4));
    }
  }
}

/* Nibble k of column n in the plain layout. */
static inline uint8_t plain_at(const uint8_t *q_plain, int K, int k, int n) {
  uint8_t b = q_plain[(size_t)n * (K / 2) + k / 2];
  return (k & 1) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0xf);
}

/* Stage 2a: weight prepack, [K/2, N] bytes -> [K, N/2] bytes, both column-major.
 * Reference: f16_quant_sm80.cuh:362-417 (dev_prepack_weights), the same
 * permutation as test/blkq4_fp16_gemm_sm80.h:39-86.  Closed form used here: the
 * packed byte at row kp, column np (offset np * K + kp) holds
 *   low nibble  q[k, n],  high nibble q[k + 8, n]   with
 *   n = 16 * (np / 8) + np % 8 + 8 * (sub & 1),
 *   k = 16 * (kp / 16) + 2 * ((kp % 16) / 4) + (sub >> 1),   sub = kp % 4. */
void blkq4_oracle_prepack_weights(int K, int N, const uint8_t *q_plain,
                                  uint8_t *packed) {
#pragma omp parallel for schedule(static)
  for (int np = 0; np < N / 2; ++np) {
    for (int kp = 0; kp < K; ++kp) {
      int sub = kp % 4;
      int n = 16 * (np / 8) + np % 8 + 8 * (sub & 1);
      int k = 16 * (kp / 16) + 2 * ((kp % 16) / 4) + (sub >> 1);
      packed[(size_t)np * K + kp] =
          (uint8_t)(plain_at(q_plain, K, k, n) | (plain_at(q_plain, K, k + 8, n) << 4));
    }
  }
}

/* Position, inside a group of 16 meta rows, that source row r moves to when the
 * blocking is row-wise.  Reference: f16_quant_sm80.cuh:506-512 (scales:
 * dst[4t + {0,1,2,3}] = src[2t + {0,1,8,9}]) and :528-538 (zero points:
 * dst[4t + {0,1,2,3}] = src[2t + {0,8,1,9}]). */
static inline int perm16_scale_dst(int r) { /* r in [0,16) */
  int t = (r % 8) / 2, hi = r / 8, odd = r & 1;
  return 4 * t + 2 * hi + odd;
}
static inline int perm16_zp_dst(int r) {
  int t = (r % 8) / 2, hi = r / 8, odd = r & 1;
  return 4 * t + 2 * odd + hi;
}

/* Stage 2b: meta prepack.  Reference: f16_quant_sm80.cuh:457-547
 * (dev_prepack_scales).  Column-wise blocking: column-major -> row-major
 * [K/bk, N], no permutation.  Row-wise blocking: stays column-major [K, N/bn],
 * each group of 16 rows permuted as above. */
void blkq4_oracle_prepack_meta(int block, int colwise, int K, int N,
                               const uint16_t *scales_cm, const uint8_t *zp_cm,
                               uint16_t *scales_out, uint8_t *zp_out) {
  const int bk = colwise ? block : 1, bn = colwise ? 1 : block;
  const int mrows = K / bk, mcols = N / bn;
  for (int c = 0; c < mcols; ++c)
    for (int r = 0; r < mrows; ++r) {
      size_t src = (size_t)c * mrows + r;
      if (colwise) {
        size_t dst = (size_t)r * mcols + c;
        scales_out[dst] = scales_cm[src];
        if (zp_cm) zp_out[dst] = zp_cm[src];
      } else {
        int g = r / 16 * 16;
        scales_out[(size_t)c * mrows + g + perm16_scale_dst(r % 16)] = scales_cm[src];
        if (zp_cm) zp_out[(size_t)c * mrows + g + perm16_zp_dst(r % 16)] = zp_cm[src];
      }
    }
}

/* Quantize + prepack: what blkq4_fp16_quant_sm80 returns to its caller.
 * Reference: src/blkq4_f16_gemm_sm80.cu:205-314.  tmp_* are caller scratch of
 * the same sizes as the outputs. */
void blkq4_oracle_quant_prepack(int block, int colwise, int K, int N, int ld,
                                const uint16_t *w, uint8_t *packed, uint16_t *scales,
                                uint8_t *zp, uint8_t *tmp_q, uint16_t *tmp_s,
                                uint8_t *tmp_z) {
  blkq4_oracle_quantize_plain(block, colwise, K, N, ld, w, tmp_q, tmp_s, zp ? tmp_z : NULL);
  blkq4_oracle_prepack_weights(K, N, tmp_q, packed);
  blkq4_oracle_prepack_meta(block, colwise, K, N, tmp_s, zp ? tmp_z : NULL, scales, zp);
}

/* ------------------------------------------------------------------------- */
/* Locating one weight in the packed form (inverse of the two prepacks). */
static inline uint8_t packed_nibble(const uint8_t *packed, int K, int k, int n) {
  int kk = k % 16, nn = n % 16;
  int row = (kk % 8) / 2, odd = kk & 1, hi = kk / 8, nhi = nn / 8;
  int kp = 16 * (k / 16) + 4 * row + 2 * odd + nhi;
  int np = 8 * (n / 16) + nn % 8;
  uint8_t b = packed[(size_t)np * K + kp];
  return hi ? (uint8_t)(b >> 4) : (uint8_t)(b & 0xf);
}
static inline size_t packed_meta_index(int block, int colwise, int K, int N, int k,
                                       int n, int for_zp) {
  if (colwise) return (size_t)(k / block) * N + n;
  int g = k / 16 * 16, r = k % 16;
  return (size_t)(n / block) * K + g + (for_zp ? perm16_zp_dst(r) : perm16_scale_dst(r));
}

/* Dequantize the packed form back to a column-major K x N fp16 matrix (ld = K).
 *   mode 0: fp16(float(scale) * float(q - zp)), the reference tests' host
 *           dequantization (test/blkq4_fp16_gemm_sm80_test.cu:314-328,
 *           test/blkq4_fp16_quant_sm80_test.cu:165-186).
 *   mode 1: the GEMM kernel's in-register formula, two fp16 roundings:
 *           fma_rn_f16(scale, fp16(16 + q), rn_f16(scale * fp16(-16 - zp)))
 *           (src/mickey/cutlass_ext/q4gemm/warp/
 *           quantb_meta_mma_tensor_op_tile_iterator.h:69-104 and :436-543).
 * zp == NULL means symmetric quantization, zero point 8. */
void blkq4_oracle_dequant(int block, int colwise, int K, int N, const uint8_t *packed,
                          const uint16_t *scales, const uint8_t *zp, int mode,
                          uint16_t *w_out) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      int q = packed_nibble(packed, K, k, n);
      float s = h2f(scales[packed_meta_index(block, colwise, K, N, k, n, 0)]);
      int z = zp ? zp[packed_meta_index(block, colwise, K, N, k, n, 1)] : 8;
      uint16_t d;
      if (mode == 0) {
        d = f2h(s * (float)(q - z));
      } else {
        /* s * (-16 - z): an fp16 times a small integer is exact in fp32, so one
         * rounding to fp16 equals mul.rn.f16.  The fma result is likewise exact
         * in fp64 before its single rounding. */
        float off = h2f(f2h(s * (float)(-16 - z)));
        double exact = (double)s * (double)(16 + q) + (double)off;
        f16 r = (f16)exact;
        memcpy(&d, &r, 2);
      }
      w_out[(size_t)n * K + k] = d;
    }
}

/* C[M,N] (fp16, row-major) = A[M,K] (fp16, row-major) x Wdq[K,N] (fp16,
 * column-major, ld = K), fp32 accumulation in ascending k, one rounding to fp16.
 * Reference: the naive device GEMM the reference tests compare with,
 * test/blkq4_fp16_gemm_sm80_test.cu:54-107 and :446-459. */
void blkq4_oracle_gemm(int M, int N, int K, const uint16_t *a, const uint16_t *wdq,
                       uint16_t *c) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const f16 *wcol = (const f16 *)(wdq + (size_t)n * K);
    for (int m = 0; m < M; ++m) {
      const f16 *arow = (const f16 *)(a + (size_t)m * K);
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) acc = fmaf((float)arow[k], (float)wcol[k], acc);
      c[(size_t)m * N + n] = f2h(acc);
    }
  }
}

/* The reference's CPU-visible path in one call: dequantize the packed weight
 * (mode as above) and multiply.  wdq_tmp is caller scratch, K * N fp16. */
void blkq4_oracle_dequant_gemm(int block, int colwise, int M, int N, int K,
                               const uint16_t *a, const uint8_t *packed,
                               const uint16_t *scales, const uint8_t *zp, int mode,
                               uint16_t *wdq_tmp, uint16_t *c) {
  blkq4_oracle_dequant(block, colwise, K, N, packed, scales, zp, mode, wdq_tmp);
  blkq4_oracle_gemm(M, N, K, a, wdq_tmp, c);
}

/* ------------------------------------------------------------------------- */
/* The reference tests' deterministic known-answer generator (no RNG).
 * Reference: test/blkq4_fp16_quant_sm80_test.cu:72-112, the same sequence as
 * test/blkq4_fp16_gemm_sm80_test.cu:225-256 and python/blkq4linear_test.py:36-61.
 * Nibbles walk v -> (v + 5) % 16, skipping 3, 7, 11 (a 13-cycle), from v = 7,
 * down each column of the plain [K/2, N] byte matrix.  Then, continuing with
 * the same v, per meta entry (column outer, row inner):
 *   f = ((c*v + r + v/3) % 63) + 1;  v += 41;  m = c*v + r + v*3;
 *   scale = f / 2^(4 + m % 2);       zp = ((f + m + v) % 8) + 4.
 * Meta is produced here column-major (index c * mrows + r), i.e. the "plain"
 * order the quantizer's first stage would emit. */
static inline int kat_next(int v) {
  v = (v + 5) % 16;
  if (v == 11 || v == 7 || v == 3) v = (v + 5) % 16;
  return v;
}
void blkq4_oracle_kat_generate(int block, int colwise, int K, int N, uint8_t *q_plain,
                               uint16_t *scales_cm, uint8_t *zp_cm) {
  const int bk = colwise ? block : 1, bn = colwise ? 1 : block;
  const int mrows = K / bk, mcols = N / bn;
  int v = 7;
  for (int c = 0; c < N; ++c)
    for (int r = 0; r < K / 2; ++r) {
      int v0 = v;
      v = kat_next(v);
      int v1 = v;
      v = kat_next(v);
      q_plain[(size_t)c * (K / 2) + r] = (uint8_t)((v1 << 4) | v0);
    }
  for (int c = 0; c < mcols; ++c)
    for (int r = 0; r < mrows; ++r) {
      int f = ((c * v + r + v / 3) % 63) + 1;
      v += 41;
      int m = c * v + r + v * 3;
      scales_cm[(size_t)c * mrows + r] = f2h((float)f / (float)(1 << (4 + (m % 2))));
      if (zp_cm) zp_cm[(size_t)c * mrows + r] = (uint8_t)(((f + m + v) % 8) + 4);
    }
}

/* Host dequantization of the plain form into the column-major fp16 matrix the
 * tests then feed to the quantizer.  Reference:
 * test/blkq4_fp16_quant_sm80_test.cu:165-186. */
void blkq4_oracle_dequant_plain(int block, int colwise, int K, int N,
                                const uint8_t *q_plain, const uint16_t *scales_cm,
                                const uint8_t *zp_cm, uint16_t *w_out) {
  const int bk = colwise ? block : 1, bn = colwise ? 1 : block;
  const int mrows = K / bk;
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      size_t mi = (size_t)(n / bn) * mrows + k / bk;
      int z = zp_cm ? zp_cm[mi] : 8;
      int q = plain_at(q_plain, K, k, n);
      w_out[(size_t)n * K + k] = f2h(h2f(scales_cm[mi]) * (float)(q - z));
    }
}
