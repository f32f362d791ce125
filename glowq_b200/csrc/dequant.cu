// Whole-weight dequantisation: out[OC, IC] fp16 = half_rn((code - zero) * scale), bit-exact with the
// reference definition.  The same unpack8_minus_zero + HMUL2 sequence produces the tensor-core
// kernel's shared-memory weight tiles, so this entry point is the bit-exactness check for both.
#include "common.cuh"
#include "params.h"

namespace glowq {
namespace {

__global__ void __launch_bounds__(256) dequant_kernel(const int32_t* __restrict__ qweight, const __half* __restrict__ scales,
                                                     const int32_t* __restrict__ qzeros, __half* __restrict__ out, int OC,
                                                     int IC, int group_size, int wstride, int zstride, int sstride,
                                                     int vec_ok) {
  const int row = blockIdx.x;
  const int wi = blockIdx.y * 256 + threadIdx.x;
  const int k0 = wi * 8;
  if (row >= OC || k0 >= IC) return;
  const int G = k0 / group_size;  // group_size % 8 == 0: a packed word never straddles two groups
  const uint32_t w = static_cast<uint32_t>(qweight[static_cast<size_t>(row) * wstride + wi]);
  const uint32_t z = nibble(qzeros + static_cast<size_t>(row) * zstride, G);
  const uint32_t s = __half_as_ushort(scales[static_cast<size_t>(row) * sstride + G]);
  uint32_t zlo, zhi, h[4];
  zero_consts(z, zlo, zhi);
  unpack8_minus_zero(w, zlo, zhi, h);
  const uint32_t s2 = s * 0x00010001u;
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = hmul2(h[i], s2);  // (n0,n4) (n1,n5) (n2,n6) (n3,n7)
  uint4 v;
  v.x = prmt(h[0], h[1], 0x5410);
  v.y = prmt(h[2], h[3], 0x5410);
  v.z = prmt(h[0], h[1], 0x7632);
  v.w = prmt(h[2], h[3], 0x7632);
  __half* dst = out + static_cast<size_t>(row) * IC + k0;
  if (vec_ok && k0 + 8 <= IC) {
    *reinterpret_cast<uint4*>(dst) = v;
  } else {
    const __half* e = reinterpret_cast<const __half*>(&v);
    for (int i = 0; i < 8 && k0 + i < IC; ++i) dst[i] = e[i];
  }
}

}  // namespace

cudaError_t launch_dequant(const int32_t* qweight, const __half* scales, const int32_t* qzeros, __half* out, int OC, int IC,
                           int group_size, int wstride, int zstride, int sstride, cudaStream_t stream) {
  const int words = (IC + 7) / 8;
  const int vec_ok = (IC % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  dim3 grid(OC, (words + 255) / 256);
  dequant_kernel<<<grid, 256, 0, stream>>>(qweight, scales, qzeros, out, OC, IC, group_size, wstride, zstride, sstride,
                                           vec_ok);
  return cudaGetLastError();
}

}  // namespace glowq
