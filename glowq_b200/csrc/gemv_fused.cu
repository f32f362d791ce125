// Weight-streaming corrected W4A16 kernel for small token counts (decode): one launch computes, for
// every member i of a group,   y_i = x . dequant(Q_i)^T + alpha_i * (x . R^T) . L_i^T + bias_i.
//
// Work decomposition (grid = n_r_units + n_tiles * SK CTAs of 8 warps):
//   * a MAIN unit is one 16-row tile of one member x one K slice.  The 8 warps interleave over the
//     128-column quantisation groups of the slice.  In a warp, lane (g = lane/4, t = lane%4) streams
//     rows g and g+8 with 128-bit loads: the four lanes of a quad cover one whole group (64 B) of a
//     row, so one scale / zero-point applies to everything a lane holds in a step.  Codes become exact
//     fp16 integers (code - zero) with LOP3 + one HSUB2/HFMA2 per pair, feed m16n8k16 tensor-core MMAs
//     against the staged activations (tokens on the MMA N axis, so M <= 8 costs what M = 1 costs),
//     and the per-group fp32 result is scaled by the group's scale in fp32.
//   * an R unit is one 16-row tile of R_g x one K slice, same machinery with fp16 A operands; the
//     finished r tile is rounded to fp16 into r_buf and a counter is released.
//   * the L_i . r term is a few extra MMAs before the cross-warp reduction; CTAs wait for the counter
//     with a bounded spin.  R units are handed out through a ticket taken at CTA start, so every R
//     unit belongs to a CTA that is already running: the wait cannot depend on an unscheduled CTA.
//   * split-K partial tiles are summed, in slice order, by the last CTA to arrive at the tile.
#include "common.cuh"
#include "params.h"

namespace glowq {

namespace {

constexpr int kDepth = 4;  // groups of weight loads in flight per lane (2 x 16 B each)

// Stage x[0:M, g0*128 : (g0+ng)*128) into shared memory in MMA B-fragment order: for token m and
// group gl, 16-byte chunk (i*4 + t) holds the columns 32t+8i+{0,4,1,5,2,6,3,7} of that group.
__device__ __forceinline__ void stage_x(const GemvParams& p, int g0, int ng, unsigned char* xs) {
  const int per_tok = ng * 16;
  const int total = p.M * per_tok;
  for (int idx = threadIdx.x; idx < total; idx += kGemvThreads) {
    const int m = idx / per_tok;
    const int c = idx - m * per_tok;
    const int gl = c >> 4, s = c & 15;  // s = 8-column block of the group, in source order
    const int k = (g0 + gl) * kGroup + 8 * s;
    const __half* src = p.x + static_cast<size_t>(m) * p.x_stride + k;
    uint4 v;
    if (p.x_vec_ok && k + 8 <= p.IC) {
      v = *reinterpret_cast<const uint4*>(src);
    } else {
      __align__(16) __half tmp[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) tmp[e] = (k + e < p.IC) ? src[e] : __float2half(0.f);
      v = *reinterpret_cast<const uint4*>(tmp);
    }
    const int i = s & 3, t = s >> 2;
    *reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * p.xs_stride + (gl * 16 + i * 4 + t) * 16) =
        interleave_pairs(v);
  }
}

template <int NT>
__device__ __forceinline__ void load_xfrag(const GemvParams& p, const unsigned char* xs, int gl, int i, int g, int t,
                                           uint4 (&xb)[NT]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = nt * 8 + g;
    xb[nt] = (tok < p.M) ? *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(tok) * p.xs_stride +
                                                          (gl * 16 + i * 4 + t) * 16)
                         : make_uint4(0, 0, 0, 0);
  }
}

// Sum the per-warp accumulators; fin[tok][16] receives the CTA's [16 rows x 8*NT tokens] tile.
template <int NT>
__device__ __forceinline__ void cross_warp_reduce(float (&acc)[NT][4], float* red, float* fin) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
    reinterpret_cast<float4*>(red)[(warp * NT + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
  __syncthreads();
  for (int e = threadIdx.x; e < NT * 128; e += kGemvThreads) {
    const int nt = e >> 7, ln = (e & 127) >> 2, c = e & 3;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kGemvWarps; ++w) s += red[((w * NT + nt) * 32 + ln) * 4 + c];
    const int row = (ln >> 2) + ((c & 2) ? 8 : 0);
    const int tok = nt * 8 + (ln & 3) * 2 + (c & 1);
    fin[tok * 16 + row] = s;
  }
  __syncthreads();
}

// Combine K-slice partial tiles: every slice stores its tile; the last arrival sums all slices in
// slice order (deterministic) and returns true with the sum in fin.
template <int NT>
__device__ __forceinline__ bool splitk_combine(float* fin, float* partial_base, uint32_t* ctr, int slices, int ks,
                                               int* s_flag) {
  constexpr int kElems = NT * 128;
  float* mine = partial_base + static_cast<size_t>(ks) * kElems;
  for (int e = threadIdx.x; e < kElems; e += kGemvThreads) mine[e] = fin[e];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(ctr, 1u);
    *s_flag = (old == static_cast<uint32_t>(slices - 1));
  }
  __syncthreads();
  if (!*s_flag) return false;
  __threadfence();
  for (int e = threadIdx.x; e < kElems; e += kGemvThreads) {
    float s = 0.f;
    for (int k = 0; k < slices; ++k) s += ldg_cg_f32(partial_base + static_cast<size_t>(k) * kElems + e);
    fin[e] = s;
  }
  if (threadIdx.x == 0) *ctr = 0u;  // ready for the next launch that uses this workspace
  __syncthreads();
  return true;
}

template <int NT>
__device__ __forceinline__ void r_unit(const GemvParams& p, int unit, unsigned char* xs, float* red, float* fin,
                                       int* s_flag, bool x_staged) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int rt = unit / p.SKr, ks = unit - rt * p.SKr;
  const int j0 = rt * kTileRows;
  const int g0 = ks * p.gps_r, ng = min(p.G, g0 + p.gps_r) - g0;
  const __half* rowA = p.R + static_cast<size_t>(min(j0 + g, p.rank - 1)) * p.R_stride;
  const __half* rowB = p.R + static_cast<size_t>(min(j0 + g + 8, p.rank - 1)) * p.R_stride;
  if (!x_staged) {
    stage_x(p, g0, ng, xs);
    __syncthreads();
  }
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

  for (int gl = warp; gl < ng; gl += kGemvWarps) {
    const int kb = (g0 + gl) * kGroup + 32 * t;
    uint4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = kb + 8 * i;
      const bool ok = (k + 8 <= p.IC);
      a[i] = ok ? ldg_stream_v4(rowA + k) : make_uint4(0, 0, 0, 0);
      b[i] = ok ? ldg_stream_v4(rowB + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 pa = interleave_pairs(a[i]), pb = interleave_pairs(b[i]);
      uint4 xb[NT];
      load_xfrag<NT>(p, xs, gl, i, g, t, xb);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma16816(acc[nt], pa.x, pb.x, pa.y, pb.y, xb[nt].x, xb[nt].y);
        mma16816(acc[nt], pa.z, pb.z, pa.w, pb.w, xb[nt].z, xb[nt].w);
      }
    }
  }
  cross_warp_reduce<NT>(acc, red, fin);
  bool finalize = true;
  if (p.SKr > 1)
    finalize = splitk_combine<NT>(fin, p.r_partial + static_cast<size_t>(rt) * p.SKr * (NT * 128), p.r_tile_ctr + rt,
                                  p.SKr, ks, s_flag);
  if (finalize) {
    for (int e = threadIdx.x; e < p.M * 16; e += kGemvThreads) {
      const int tok = e >> 4, r = e & 15;
      if (j0 + r < p.rank) p.r_buf[static_cast<size_t>(tok) * p.rank + j0 + r] = __float2half_rn(fin[tok * 16 + r]);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(p.ws_head + WS_R_DONE, 1u);
  }
}

template <int NT>
__device__ __forceinline__ void main_unit(const GemvParams& p, int unit, unsigned char* xs, uint32_t* szs, float* red,
                                          float* fin, int* s_flag, bool x_staged) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int tile = unit / p.SK, ks = unit - tile * p.SK;
  int mi = 0;
#pragma unroll
  for (int i = 1; i < kMaxMembers; ++i)
    if (i < p.n_members && tile >= p.mem[i].tile_begin) mi = i;
  const MemberDev& mb = p.mem[mi];
  const int row0 = (tile - mb.tile_begin) * kTileRows;
  const int g0 = ks * p.gps, ng = min(p.G, g0 + p.gps) - g0;
  const int rA = min(row0 + g, mb.OC - 1), rB = min(row0 + g + 8, mb.OC - 1);
  const char* wA = reinterpret_cast<const char*>(mb.qweight + static_cast<size_t>(rA) * mb.wstride) + t * 16;
  const char* wB = reinterpret_cast<const char*>(mb.qweight + static_cast<size_t>(rB) * mb.wstride) + t * 16;
  const int n_my = (ng - warp + kGemvWarps - 1) / kGemvWarps;  // my groups: gl = warp + 8 j

  // Weight loads go out first; nothing they need depends on other CTAs.
  uint4 qa[kDepth], qb[kDepth];
#pragma unroll
  for (int d = 0; d < kDepth; ++d) {
    if (d < n_my) {
      const size_t off = static_cast<size_t>(g0 + warp + kGemvWarps * d) * 64;
      qa[d] = ldg_stream_v4(wA + off);
      qb[d] = ldg_stream_v4(wB + off);
    }
  }
  const bool corr = (ks == 0) && (p.r_mode != 0) && (mb.L != nullptr) && (mb.alpha != 0.f);
  const int n_chunks = (p.rank + 31) >> 5;
  uint4 la = make_uint4(0, 0, 0, 0), lb = la;
  if (corr && warp < n_chunks) {  // first L chunk of this warp, in flight during the main loop
    const int k = 32 * warp + 8 * t;
    if (k < p.rank) {
      la = ldg_stream_v4(mb.L + static_cast<size_t>(rA) * mb.Lstride + k);
      lb = ldg_stream_v4(mb.L + static_cast<size_t>(rB) * mb.Lstride + k);
    }
  }

  // scale (low 16 bits) and zero-point (high 16 bits) of every (row, group) of this unit
  for (int idx = threadIdx.x; idx < kTileRows * ng; idx += kGemvThreads) {
    const int r = idx / ng, gl = idx - r * ng;
    const int row = min(row0 + r, mb.OC - 1), G = g0 + gl;
    const uint32_t s = __half_as_ushort(mb.scales[static_cast<size_t>(row) * mb.sstride + G]);
    const uint32_t z = nibble(mb.qzeros + static_cast<size_t>(row) * mb.zstride, G);
    szs[r * p.gps + gl] = s | (z << 16);
  }
  if (!x_staged) stage_x(p, g0, ng, xs);
  __syncthreads();

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

  for (int it = 0; it < n_my; it += kDepth) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      const int j = it + d;
      if (j < n_my) {
        const int gl = warp + kGemvWarps * j;
        const uint4 A = qa[d], B = qb[d];
        if (j + kDepth < n_my) {
          const size_t off = static_cast<size_t>(g0 + gl + kGemvWarps * kDepth) * 64;
          qa[d] = ldg_stream_v4(wA + off);
          qb[d] = ldg_stream_v4(wB + off);
        }
        const uint32_t szA = szs[g * p.gps + gl], szB = szs[(g + 8) * p.gps + gl];
        uint32_t zloA, zhiA, zloB, zhiB;
        zero_consts(szA >> 16, zloA, zhiA);
        zero_consts(szB >> 16, zloB, zhiB);
        const float sA = __half2float(__ushort_as_half(static_cast<unsigned short>(szA & 0xFFFFu)));
        const float sB = __half2float(__ushort_as_half(static_cast<unsigned short>(szB & 0xFFFFu)));
        float ag[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) ag[nt][0] = ag[nt][1] = ag[nt][2] = ag[nt][3] = 0.f;
        const uint32_t wa[4] = {A.x, A.y, A.z, A.w}, wb[4] = {B.x, B.y, B.z, B.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t ha[4], hb[4];
          unpack8_minus_zero(wa[i], zloA, zhiA, ha);
          unpack8_minus_zero(wb[i], zloB, zhiB, hb);
          uint4 xb[NT];
          load_xfrag<NT>(p, xs, gl, i, g, t, xb);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma16816(ag[nt], ha[0], hb[0], ha[1], hb[1], xb[nt].x, xb[nt].y);
            mma16816(ag[nt], ha[2], hb[2], ha[3], hb[3], xb[nt].z, xb[nt].w);
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          acc[nt][0] = fmaf(sA, ag[nt][0], acc[nt][0]);
          acc[nt][1] = fmaf(sA, ag[nt][1], acc[nt][1]);
          acc[nt][2] = fmaf(sB, ag[nt][2], acc[nt][2]);
          acc[nt][3] = fmaf(sB, ag[nt][3], acc[nt][3]);
        }
      }
    }
  }

  if (corr) {
    if (p.r_mode == 1) {  // r is produced by R units of this launch: bounded wait on the release counter
      if (lane == 0) {
        unsigned spins = 0;
        while (ld_acquire_u32(p.ws_head + WS_R_DONE) < static_cast<uint32_t>(p.n_r_tiles)) {
          __nanosleep(200);
          if (++spins > kSpinLimit) {
            atomicExch(p.ws_head + WS_STATUS, 1u);
            break;
          }
        }
      }
      __syncwarp();
    }
    float al[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) al[nt][0] = al[nt][1] = al[nt][2] = al[nt][3] = 0.f;
    for (int c = warp; c < n_chunks; c += kGemvWarps) {
      const int k = 32 * c + 8 * t;
      if (c != warp) {
        la = lb = make_uint4(0, 0, 0, 0);
        if (k < p.rank) {
          la = ldg_stream_v4(mb.L + static_cast<size_t>(rA) * mb.Lstride + k);
          lb = ldg_stream_v4(mb.L + static_cast<size_t>(rB) * mb.Lstride + k);
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int tok = nt * 8 + g;
        uint4 rb = make_uint4(0, 0, 0, 0);
        if (tok < p.M && k < p.rank) rb = ldg_cg_v4(p.r_buf + static_cast<size_t>(tok) * p.rank + k);
        mma16816(al[nt], la.x, lb.x, la.y, lb.y, rb.x, rb.y);
        mma16816(al[nt], la.z, lb.z, la.w, lb.w, rb.z, rb.w);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nt][c] = fmaf(mb.alpha, al[nt][c], acc[nt][c]);
  }

  cross_warp_reduce<NT>(acc, red, fin);
  bool finalize = true;
  if (p.SK > 1)
    finalize = splitk_combine<NT>(fin, p.sk_partial + static_cast<size_t>(tile) * p.SK * (NT * 128), p.tile_ctr + tile,
                                  p.SK, ks, s_flag);
  if (!finalize) return;
  for (int e = threadIdx.x; e < p.M * 16; e += kGemvThreads) {
    const int tok = e >> 4, r = e & 15, row = row0 + r;
    if (row < mb.OC) {
      float v = fin[tok * 16 + r];
      if (mb.bias) v += __half2float(mb.bias[row]);
      const size_t o = static_cast<size_t>(tok) * mb.out_stride + row;
      if (p.out_fp32)
        static_cast<float*>(mb.out)[o] = v;
      else
        static_cast<__half*>(mb.out)[o] = __float2half_rn(v);
    }
  }
}

template <int NT>
__global__ void __launch_bounds__(kGemvThreads, (NT <= 2) ? 2 : 1)
gemv_fused_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_unit, s_flag;
  unsigned char* xs = smem;
  size_t off = (static_cast<size_t>(p.M) * p.xs_stride + 15) & ~static_cast<size_t>(15);
  uint32_t* szs = reinterpret_cast<uint32_t*>(smem + off);
  off += static_cast<size_t>(kTileRows) * p.gps * 4;
  off = (off + 15) & ~static_cast<size_t>(15);
  float* red = reinterpret_cast<float*>(smem + off);
  off += static_cast<size_t>(kGemvWarps) * NT * 512;
  float* fin = reinterpret_cast<float*>(smem + off);

  int unit = blockIdx.x;
  bool x_staged = false;
  if (p.r_mode == 1) {
    // Roles come from a ticket: the first n_r_units CTAs to START compute r, the rest stream weights.
    if (threadIdx.x == 0) s_unit = static_cast<int>(atomicAdd(p.ws_head + WS_TICKET, 1u));
    if (p.SK == 1 && p.SKr == 1) {  // every unit needs all of x: stage it while the ticket is in flight
      stage_x(p, 0, p.G, xs);
      x_staged = true;
    }
    __syncthreads();
    unit = s_unit;
  }
  if (unit < p.n_r_units)
    r_unit<NT>(p, unit, xs, red, fin, &s_flag, x_staged);
  else
    main_unit<NT>(p, unit - p.n_r_units, xs, szs, red, fin, &s_flag, x_staged);

  if (p.r_mode == 1) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(p.ws_head + WS_EXIT, 1u);
      if (old == gridDim.x - 1) {  // last CTA out re-arms the counters for the next launch
        p.ws_head[WS_TICKET] = 0u;
        p.ws_head[WS_R_DONE] = 0u;
        p.ws_head[WS_EXIT] = 0u;
        __threadfence();
      }
    }
  }
}

// Any-shape scalar kernel for layouts the streaming kernel does not take (group_size != 128, packed
// rows that are not 16-byte aligned).  One warp per output row; fp32 accumulation.
__global__ void __launch_bounds__(256) w4a16_generic_kernel(const __half* x, const int32_t* qweight, const __half* scales,
                                                           const int32_t* qzeros, const __half* bias, const __half* L,
                                                           const float* r32, float alpha, void* out, int out_fp32,
                                                           int M, int IC, int OC, int rank, int group_size, int x_stride,
                                                           int wstride, int zstride, int sstride, int Lstride,
                                                           int out_stride) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= OC) return;
  const int32_t* wrow = qweight + static_cast<size_t>(row) * wstride;
  const int32_t* zrow = qzeros + static_cast<size_t>(row) * zstride;
  for (int m = 0; m < M; ++m) {
    float acc = 0.f;
    for (int k = lane; k < IC; k += 32) {
      const int G = k / group_size;
      const float w = static_cast<float>(static_cast<int>(nibble(wrow, k)) - static_cast<int>(nibble(zrow, G))) *
                      __half2float(scales[static_cast<size_t>(row) * sstride + G]);
      acc = fmaf(w, __half2float(x[static_cast<size_t>(m) * x_stride + k]), acc);
    }
    float c = 0.f;
    if (L != nullptr && r32 != nullptr)
      for (int j = lane; j < rank; j += 32)
        c = fmaf(__half2float(L[static_cast<size_t>(row) * Lstride + j]), r32[static_cast<size_t>(m) * rank + j], c);
    acc = fmaf(alpha, c, acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      if (bias) acc += __half2float(bias[row]);
      const size_t oidx = static_cast<size_t>(m) * out_stride + row;
      if (out_fp32)
        static_cast<float*>(out)[oidx] = acc;
      else
        static_cast<__half*>(out)[oidx] = __float2half_rn(acc);
    }
  }
}

// r32[M, rank] = x . R^T for the generic path (one warp per (token, rank row)); also rounds to r_buf.
__global__ void __launch_bounds__(256) r_generic_kernel(const __half* x, const __half* R, float* r32, __half* r_buf, int M,
                                                       int IC, int rank, int x_stride, int R_stride) {
  const int w = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (w >= M * rank) return;
  const int m = w / rank, j = w - m * rank;
  float acc = 0.f;
  for (int k = lane; k < IC; k += 32)
    acc = fmaf(__half2float(R[static_cast<size_t>(j) * R_stride + k]), __half2float(x[static_cast<size_t>(m) * x_stride + k]), acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const __half h = __float2half_rn(acc);
    r_buf[static_cast<size_t>(m) * rank + j] = h;
    r32[static_cast<size_t>(m) * rank + j] = __half2float(h);
  }
}

__global__ void __launch_bounds__(256) r_widen_kernel(const __half* r_buf, float* r32, int n) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n) r32[i] = __half2float(r_buf[i]);
}

}  // namespace

// ---------------------------------------------------------------- host launchers (called from abi.cu)
size_t gemv_smem_bytes(const GemvParams& p, int NT) {
  size_t off = (static_cast<size_t>(p.M) * p.xs_stride + 15) & ~static_cast<size_t>(15);
  off += static_cast<size_t>(kTileRows) * p.gps * 4;
  off = (off + 15) & ~static_cast<size_t>(15);
  off += static_cast<size_t>(kGemvWarps) * NT * 512;
  off += static_cast<size_t>(NT) * 8 * 16 * 4;
  return off;
}

template <int NT>
static cudaError_t launch_nt(const GemvParams& p, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_fused_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  const int grid = p.n_r_units + p.n_tiles * p.SK;
  gemv_fused_kernel<NT><<<grid, kGemvThreads, gemv_smem_bytes(p, NT), stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_gemv_fused(const GemvParams& p, cudaStream_t stream) {
  const int nt = (p.M + 7) / 8;
  if (nt <= 1) return launch_nt<1>(p, stream);
  if (nt <= 2) return launch_nt<2>(p, stream);
  return launch_nt<4>(p, stream);
}

cudaError_t launch_generic_r(const __half* x, const __half* R, __half* r_buf, float* r32, int r_mode, int M, int IC,
                             int rank, int x_stride, int R_stride, cudaStream_t stream) {
  if (r_mode == 1)
    r_generic_kernel<<<(M * rank + 7) / 8, 256, 0, stream>>>(x, R, r32, r_buf, M, IC, rank, x_stride, R_stride);
  else
    r_widen_kernel<<<(M * rank + 255) / 256, 256, 0, stream>>>(r_buf, r32, M * rank);
  return cudaGetLastError();
}

cudaError_t launch_generic(const __half* x, const MemberDev& mb, const float* r32, int out_fp32, int M, int IC, int rank,
                           int group_size, int x_stride, cudaStream_t stream) {
  const bool corr = r32 != nullptr && mb.L != nullptr && mb.alpha != 0.f;
  w4a16_generic_kernel<<<(mb.OC + 7) / 8, 256, 0, stream>>>(x, mb.qweight, mb.scales, mb.qzeros, mb.bias,
                                                           corr ? mb.L : nullptr, corr ? r32 : nullptr, mb.alpha, mb.out,
                                                           out_fp32, M, IC, mb.OC, rank, group_size, x_stride, mb.wstride,
                                                           mb.zstride, mb.sstride, mb.Lstride, mb.out_stride);
  return cudaGetLastError();
}

}  // namespace glowq
