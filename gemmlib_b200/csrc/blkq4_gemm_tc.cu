// placeholder: replaced by the tcgen05 kernel
#include "blkq4_common.cuh"
namespace blkq4 {
std::string launch_gemm_tc(int block, bool colwise, int M, int N, int K, cudaStream_t stream,
                           const __half* a, const uint8_t* packed, const __half* scales,
                           const uint8_t* zp, __half* out) {
  for (int m0 = 0; m0 < M; m0 += 16) {
    const int mm = M - m0 < 16 ? M - m0 : 16;
    std::string e = launch_gemv(block, colwise, mm, N, K, stream, a + (size_t)m0 * K, packed, scales, zp, out + (size_t)m0 * N);
    if (!e.empty()) return e;
  }
  return std::string();
}
}
