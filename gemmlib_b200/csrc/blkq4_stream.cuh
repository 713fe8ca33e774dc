// Device helpers shared by the cp.async stream kernels (blkq4_gemv_stream.cu, blkq4_gemv_wide.cu).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace blkq4 {
namespace stream {

constexpr int kWarps = 8;            // warps per CTA = K splits
constexpr int kGroupSteps = 4;       // 64-k steps per group (one ring slot)
constexpr int kSlotW = kGroupSteps * 512;   // [step][lane] 16 bytes
constexpr int kSlotS = kGroupSteps * 32;    // [step][16] fp16
constexpr int kSlotZ = kGroupSteps * 16;    // [step][16] u8
constexpr int kSlotBytes = kSlotW + kSlotS + kSlotZ;  // 2240

__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const void* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_v2(void* p, uint32_t x, uint32_t y) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t bits) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(d) : "r"(x), "r"(mask), "r"(bits));  // (x & mask) | bits
  return d;
}
// D = A x B + C with C in its own four registers (the negated activation-only terms).
__device__ __forceinline__ void mma_init(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const float4& c) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c.x), "f"(c.y), "f"(c.z), "f"(c.w));
}
__device__ __forceinline__ void mma_acc(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Shared-memory loads with the offset as an immediate: no address arithmetic per access.
template <int OFF>
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
template <int OFF>
__device__ __forceinline__ float lds_half_as_float(uint32_t addr) {
  float v;
  asm volatile("{\n\t.reg .b16 h;\n\tld.shared.b16 h, [%1+%2];\n\tcvt.f32.f16 %0, h;\n\t}" : "=f"(v) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ float lds_u8_as_float(uint32_t addr) {
  float v;
  asm volatile("{\n\t.reg .b32 r;\n\tld.shared.u8 r, [%1];\n\tcvt.rn.f32.u32 %0, r;\n\t}" : "=f"(v) : "r"(addr));
  return v;
}
// 16-byte global -> shared copy (L2 only), executed where pred != 0.  OFF bytes into the global row
// is 8 * OFF bytes into the slot (64 bytes of a packed column per step, 512 bytes of slot per step).
template <int OFF>
__device__ __forceinline__ void cp_async16_if(uint32_t dst, const void* src, uint32_t pred) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %2, 0;\n\t"
      "@p cp.async.cg.shared.global.L2::128B [%0+%3], [%1+%4], 16;\n\t}"
      ::"r"(dst), "l"(src), "r"(pred), "n"(OFF * 8), "n"(OFF)
      : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

}  // namespace stream
}  // namespace blkq4
