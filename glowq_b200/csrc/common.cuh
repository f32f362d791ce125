// Device helpers shared by the W4A16 kernels (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glowq {

// ---------------------------------------------------------------- bit tricks on packed half2
// (a & mask) | orv in one LOP3.
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// Zero-point constants for one (row, group): lo = half2(1024+z, 1024+z), hi = half2(-(64+z), -(64+z)).
// 1024+z = 0x6400|z and 64+z = 0x5400|(z<<4) exactly, because the fp16 ulp is 1 at 1024 and 1/16 at 64.
__device__ __forceinline__ void zero_consts(uint32_t z, uint32_t& zc_lo, uint32_t& zc_hi) {
  zc_lo = 0x64006400u | (z * 0x00010001u);
  zc_hi = 0xD400D400u | ((z << 4) * 0x00010001u);
}

// One packed word (codes n0..n7 of 8 consecutive input columns) -> four half2 holding the EXACT
// integers (n0-z, n4-z), (n1-z, n5-z), (n2-z, n6-z), (n3-z, n7-z).
// Low nibbles: (w & 0x000F000F) | 0x64006400 is half2(1024+n) and the subtraction is exact.
// High nibbles: (w & 0x00F000F0) | 0x64006400 is half2(1024+16n); fma(.., 1/16, -(64+z)) = n - z exactly.
__device__ __forceinline__ void unpack8_minus_zero(uint32_t w, uint32_t zc_lo, uint32_t zc_hi, uint32_t (&h)[4]) {
  constexpr uint32_t MLO = 0x000F000Fu, MHI = 0x00F000F0u, MAGIC = 0x64006400u, SIXTEENTH = 0x2C002C00u;
  const uint32_t w8 = w >> 8;
  h[0] = hsub2(lop3_and_or(w, MLO, MAGIC), zc_lo);
  h[1] = hfma2(lop3_and_or(w, MHI, MAGIC), SIXTEENTH, zc_hi);
  h[2] = hsub2(lop3_and_or(w8, MLO, MAGIC), zc_lo);
  h[3] = hfma2(lop3_and_or(w8, MHI, MAGIC), SIXTEENTH, zc_hi);
}

// Eight fp16 values in natural order (k0..k7 as 4 words) -> the pair order of unpack8_minus_zero:
// (k0,k4), (k1,k5), (k2,k6), (k3,k7).
__device__ __forceinline__ uint4 interleave_pairs(uint4 v) {
  uint4 o;
  o.x = prmt(v.x, v.z, 0x5410);
  o.y = prmt(v.x, v.z, 0x7632);
  o.z = prmt(v.y, v.w, 0x5410);
  o.w = prmt(v.y, v.w, 0x7632);
  return o;
}

// ---------------------------------------------------------------- memory
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cg_v4(const void* p) {  // L2-coherent (data written by other CTAs)
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float ldg_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {  // never from L1: polled words that another CTA writes
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---------------------------------------------------------------- warp MMA (fp16 x fp16 -> fp32)
// D[16x8] += A[16x16] * B[16x8]; fragments as in the PTX ISA for m16n8k16.
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t nibble(const int32_t* row, int idx) {
  return (static_cast<uint32_t>(row[idx >> 3]) >> ((idx & 7) * 4)) & 0xFu;
}

}  // namespace glowq
