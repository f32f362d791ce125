// r = x . R^T (the shared right factor applied to the activations) for 9 to 128 tokens, as ONE small launch in front
// of the tensor-core group GEMM.  The [M, rank] result is a handful of tiles, so the work is cut along K as well:
// CTA (unit, by) multiplies 16 rows of R with one 1024-column slice of K for 64 tokens (one 8-token block per warp,
// tokens on the N axis of m16n8k16 MMAs; the R tile is staged in shared memory once, before the wait for the previous
// kernel - R is static - and shared by the eight warps), parks its fp32 partial block in a slot, and the CTA that
// completes the count of an (R tile, token block) pair adds the K slices in slice order, rounds to fp16 and writes
// r_buf: deterministic, and no second launch.
#include <cstdlib>

#include "common.cuh"
#include "params.h"

namespace glowq {
namespace {

constexpr int kRpThreads = 256;
constexpr int kRpTok = 64;                            // tokens per CTA
constexpr int kRpCols = kChunkGroups * kGroup;        // K columns per CTA (1024)
constexpr int kRpPitch = kRpCols * 2 + 64;            // shared-memory row pitch of the R tile, bytes (64 mod 128: no bank conflicts)
constexpr int kRpBatch = 4;                           // quantisation groups whose activation loads are in flight together

struct RpParams {
  const __half* x;
  const __half* R;
  __half* r_buf;
  float* slots;        // [n_rt * SKr][n_by][kRpTok][16] fp32
  uint32_t* ctr;       // [n_rt][n_by] arrivals, zero between launches
  int M, IC, rank, x_stride, R_stride, n_rt, SKr, n_by;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds128_rp(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

__global__ void __launch_bounds__(kRpThreads) r_product_kernel(const __grid_constant__ RpParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint32_t s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int unit = blockIdx.x, rt = unit / p.SKr, ks = unit - rt * p.SKr, by = blockIdx.y;
  const int k0 = ks * kRpCols, kn = min(kRpCols, p.IC - k0);   // IC is a multiple of 8
  const uint32_t sR = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // R tile: rows [16 rt, 16 rt + 16) x columns [k0, k0 + kn); rows past the rank and columns past K read as zero
  for (int v = threadIdx.x; v < 16 * (kRpCols / 8); v += kRpThreads) {
    const int row = v / (kRpCols / 8), c8 = v - row * (kRpCols / 8);
    const uint32_t dst = sR + row * kRpPitch + c8 * 16;
    const int rrow = rt * 16 + row;
    if (rrow < p.rank && c8 * 8 < kn)
      cp_async16(dst, p.R + static_cast<size_t>(rrow) * p.R_stride + k0 + c8 * 8);
    else
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // x comes from the previous kernels of the stream

  // Lane (g, t) of warp w: token 64 by + 8 w + g on the B side, rows g and g + 8 of the R tile on the A side.  The
  // lane's 16-byte piece i of a group holds the columns 8 (4 i + t) .. + 7; A and B use the same assignment, so every
  // column meets its own activation, and the four lanes of a token read 64 contiguous bytes.
  const int tok = by * kRpTok + warp * 8 + g;
  const bool tok_ok = tok < p.M;
  const __half* xrow = p.x + static_cast<size_t>(tok_ok ? tok : 0) * p.x_stride + k0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  bool staged = false;
  for (int g0 = 0; g0 * kGroup < kn; g0 += kRpBatch) {
    uint4 xv[kRpBatch][4];
#pragma unroll
    for (int u = 0; u < kRpBatch; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = (g0 + u) * kGroup + 8 * (4 * i + t);
        xv[u][i] = (tok_ok && k + 8 <= kn) ? ldg_cg_v4(xrow + k) : make_uint4(0, 0, 0, 0);
      }
    if (!staged) {
      asm volatile("cp.async.wait_all;" ::: "memory");
      __syncthreads();
      staged = true;
    }
#pragma unroll
    for (int u = 0; u < kRpBatch; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = (g0 + u) * kGroup + 8 * (4 * i + t);
        if (k < kRpCols) {   // (columns past kn hold zeros in both operands)
          const uint4 a = lds128_rp(sR + g * kRpPitch + k * 2);
          const uint4 b = lds128_rp(sR + (g + 8) * kRpPitch + k * 2);
          mma16816(acc, a.x, b.x, a.y, b.y, xv[u][i].x, xv[u][i].y);
          mma16816(acc, a.z, b.z, a.w, b.w, xv[u][i].z, xv[u][i].w);
        }
      }
  }
  if (!staged) {
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
  }

  // park the partial block: acc = (row g, tokens 2t, 2t+1), (row g + 8, tokens 2t, 2t+1) of the warp's token block
  float* slot = p.slots + (static_cast<size_t>(unit) * p.n_by + by) * (kRpTok * 16);
  {
    const int tl = warp * 8 + 2 * t;
    slot[tl * 16 + g] = acc[0];
    slot[(tl + 1) * 16 + g] = acc[1];
    slot[tl * 16 + g + 8] = acc[2];
    slot[(tl + 1) * 16 + g + 8] = acc[3];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();   // (cumulative over the CTA's stores, which the barrier ordered before it)
    uint32_t* c = p.ctr + rt * p.n_by + by;
    const bool last = atomicAdd(c, 1u) == static_cast<uint32_t>(p.SKr - 1);
    if (last) {
      *c = 0u;         // every K slice has arrived: ready for the next launch
      __threadfence();
    }
    s_last = last ? 1u : 0u;
  }
  __syncthreads();
  if (s_last == 0u) return;

  // the K slices of this (R tile, token block), added in slice order
  const int tl = threadIdx.x >> 2, r4 = (threadIdx.x & 3) * 4;
  const int otok = by * kRpTok + tl, orow = rt * 16 + r4;
  if (otok < p.M && orow < p.rank) {   // the rank is a multiple of 8: four rows are valid together
    const float* base = p.slots + (static_cast<size_t>(rt) * p.SKr * p.n_by + by) * (kRpTok * 16) + tl * 16 + r4;
    const size_t stride = static_cast<size_t>(p.n_by) * (kRpTok * 16);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int z0 = 0; z0 < p.SKr; z0 += 4) {
      float4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        q[u] = (z0 + u < p.SKr) ? __ldcg(reinterpret_cast<const float4*>(base + (z0 + u) * stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        s.x += q[u].x;
        s.y += q[u].y;
        s.z += q[u].z;
        s.w += q[u].w;
      }
    }
    const __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p.r_buf + static_cast<size_t>(otok) * p.rank + orow) = pk;
  }
}

}  // namespace

// Slot bytes at the end of the workspace, and the launch.  `ctr` points at kRpCtrWords zeroed words.
size_t r_product_slot_bytes(int M, int IC, int rank) {
  const int n_rt = (rank + 15) / 16, SKr = (IC + kRpCols - 1) / kRpCols, n_by = (M + kRpTok - 1) / kRpTok;
  return static_cast<size_t>(n_rt) * SKr * n_by * kRpTok * 16 * 4;
}

cudaError_t launch_r_product(const __half* x, const __half* R, __half* r_buf, float* slots, uint32_t* ctr, int M, int IC,
                             int rank, int x_stride, int R_stride, cudaStream_t stream) {
  RpParams p{};
  p.x = x;
  p.R = R;
  p.r_buf = r_buf;
  p.slots = slots;
  p.ctr = ctr;
  p.M = M;
  p.IC = IC;
  p.rank = rank;
  p.x_stride = x_stride;
  p.R_stride = R_stride;
  p.n_rt = (rank + 15) / 16;
  p.SKr = (IC + kRpCols - 1) / kRpCols;
  p.n_by = (M + kRpTok - 1) / kRpTok;
  if (p.n_rt * p.n_by > kRpCtrWords) return cudaErrorInvalidValue;
  static const bool use_pdl = [] {
    const char* v = std::getenv("GLOWQ_PDL");
    return !(v && v[0] == '0');
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_rt * p.SKr, p.n_by);
  cfg.blockDim = dim3(kRpThreads);
  cfg.dynamicSmemBytes = 16 * kRpPitch;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, r_product_kernel, p);
}

}  // namespace glowq
