// extern "C" doorway onto the reference's own host-side prepack helpers
// (test/blkq4_fp16_gemm_sm80.h:39-226 of the reference), compiled from the
// reference sources where they lie.  TEST INFRASTRUCTURE ONLY: used to pin the
// CPU oracle and to generate the golden fixtures; never part of the library.
#include <cstdint>
#include <cstddef>
#include <string>
#include <stdexcept>
#include <vector>
#include <algorithm>

#include "blkq4_fp16_gemm_sm80.h"  // from <reference>/test

namespace rt = onnxruntime::cuda::test;
using cutlass::layout::ColumnMajor;
using cutlass::layout::RowMajor;

extern "C" int ref_prepack_weights(int K, int N, const uint8_t* q_plain, uint8_t* packed) {
  try {
    size_t sz = size_t(K / 2) * N;
    mickey::MatrixRef<uint8_t const, ColumnMajor, true> src(
        gsl::make_span(q_plain, sz), cutlass::make_Coord(K / 2, N));
    mickey::MatrixRef<uint8_t, ColumnMajor, true> dst(
        gsl::make_span(packed, sz), cutlass::make_Coord(K, N / 2));
    rt::prepack_weights_ref(K, N, src, dst);
  } catch (std::exception const&) { return -1; }
  return 0;
}

template <int block, bool colwise>
static int meta_T(int K, int N, const uint16_t* s_in, uint16_t* s_out,
                  const uint8_t* z_in, uint8_t* z_out) {
  using QB = std::conditional_t<colwise, cutlass::MatrixShape<block, 1>, cutlass::MatrixShape<1, block>>;
  using Layout = std::conditional_t<colwise, RowMajor, ColumnMajor>;  // LayoutQmeta
  auto shape = cutlass::make_Coord(K / QB::kRow, N / QB::kColumn);
  size_t sz = size_t(shape.product());
  using half_t = cutlass::half_t;
  mickey::MatrixRef<half_t const, Layout, true> ts(
      gsl::make_span(reinterpret_cast<half_t const*>(s_in), sz), shape);
  mickey::MatrixRef<half_t, Layout, true> td(
      gsl::make_span(reinterpret_cast<half_t*>(s_out), sz), shape);
  rt::prepack_quant_scales_ref<half_t, Layout, QB>(K, N, ts, td);
  if (z_in) {
    mickey::MatrixRef<uint8_t const, Layout, true> zs(gsl::make_span(z_in, sz), shape);
    mickey::MatrixRef<uint8_t, Layout, true> zd(gsl::make_span(z_out, sz), shape);
    rt::prepack_quant_offsets_ref<Layout, QB>(K, N, zs, zd);
  }
  return 0;
}

// Inputs are in the layout the reference's tests hold them in (LayoutQmeta:
// row-major [K/block, N] when column-wise, column-major [K, N/block] when
// row-wise); outputs are the prepacked meta in the same layout type.
extern "C" int ref_prepack_meta(int block, int colwise, int K, int N, const uint16_t* s_in,
                                uint16_t* s_out, const uint8_t* z_in, uint8_t* z_out) {
  try {
#define CASE(B)                                                                       \
  case B:                                                                             \
    return colwise ? meta_T<B, true>(K, N, s_in, s_out, z_in, z_out)                  \
                   : meta_T<B, false>(K, N, s_in, s_out, z_in, z_out);
    switch (block) { CASE(16) CASE(32) CASE(64) CASE(128) }
#undef CASE
  } catch (std::exception const&) { return -1; }
  return -2;
}
