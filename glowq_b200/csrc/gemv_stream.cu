// Weight-streaming corrected W4A16 kernel for small token counts (decode).  One launch computes, for every
// member i of a group,   y_i = x . dequant(Q_i)^T + alpha_i * (x . R^T) . L_i^T + bias_i.
//
// Persistent CTAs (two per SM where shared memory allows), each with ten warps:
//   * warp 8 streams packed weights: for every 32-row tile of the CTA it issues one 2-D TMA copy per pipeline
//     stage (32 rows x 8 quantisation groups = 16 KB) into a shared-memory ring guarded by mbarriers, and after
//     a tile's weight stages the tile's rows of L_i.  It depends on no other warp's results.  The ring is shallow,
//     so it also asks L2 for the chunk that follows a few issues later, and - once all of its own copies are issued -
//     for its share of the head of the NEXT call's weights (a hint the caller may give).
//   * warp 9 fetches each tile's raw scales and zero-point words two tiles ahead (4-byte cp.async), converts them one
//     tile ahead of the consumers into fp32 pairs {scale * 2^24, -scale * zero} laid out [group][row], and finishes
//     tiles: it adds the consumer warps' partial sums in warp order, runs the split-K combine, adds the bias and
//     stores.  Only a CTA's last tile is summed by the consumer threads themselves.
//   * warps 0-7 consume: warp w owns group w of every stage.  Lane (g = lane/4, t = lane%4) reads rows g, g+8,
//     g+16, g+24 with one 128-bit shared load each - the four lanes of a quad cover the 64 B of one group - masks
//     the codes into fp16 subnormals (no conversion arithmetic) and feeds m16n8k16 tensor-core MMAs against the
//     activations it staged itself in B-fragment order (tokens on the MMA N axis, so up to 8 tokens stream the
//     weights once).  Each group's fp32 result takes two FMAs with the converted pair: the scale, and the zero-point
//     as -z * scale * sum(x over the group).
//   * Optionally the activations are transformed while they are staged: residual add and RMSNorm.
//   * r = R_g . x is produced inside the launch by "R units" (16 rows of R x a K slice) run by extra CTAs (the lowest
//     block indices, placed first; with K slices also by the CTAs of slices that apply no correction).  Each unit
//     stores an fp32 slot, a CTA publishes its units with one add to a release counter, and the CTA that completes
//     the count adds the slots in slot order, rounds to fp16 and writes r to r_buf and - as 8-byte words {two
//     elements, launch epoch} - to the workspace, where the row tiles poll the words they need (one L2 round trip, no
//     flag; identical bits everywhere).  The grid never exceeds what is resident at once, so the bounded poll before
//     the first L_i epilogue never depends on an unscheduled CTA.
//   * K can be sliced across CTAs; the last CTA to arrive at a tile sums the slices in slice order.
//   * Tensor-parallel row-split launches may perform their all-reduce themselves: tiles store their result to every
//     rank's word buffer as 8-byte words {fp16 value, call epoch}, and the launch's last CTAs poll all ranks' words in
//     the local buffer, add them in rank order and write the output.
//   * The weight stages land swizzled (128-byte pattern of the tensor map) so that the consumers' 128-bit loads are
//     free of bank conflicts, and the kernel is instantiated per feature set (correction, extras) so that launches
//     do not carry the code of features they do not use.
// Every wait (mbarrier, release counter) is bounded; on expiry the kernel records a status word and drains.
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "params.h"

namespace glowq {

namespace {

constexpr int kConsumerThreads = kConsumerWarps * 32;
// Polls of one mbarrier wait before the kernel gives up (status 2).  A failed try_wait is suspended for about 3 us in
// hardware, so this is seconds, not milliseconds: under programmatic dependent launch the copy and aux warps of a
// launch run ahead and then wait for ring / metadata slots that the consumers only free once the PREVIOUS kernel is
// complete - and with tensor parallelism that kernel may be an all-reduce waiting for a rank that is tens of
// milliseconds behind.  The drain loop after a failure uses the short limit below.
constexpr uint32_t kMbarSpinLimit = 1u << 20;
constexpr uint32_t kDrainSpinLimit = 1u << 12;
constexpr int kPushFinishers = 16;         // CTAs that complete a pushing launch's all-reduce
constexpr uint32_t kSuspendHintNs = 2000;  // a waiting thread sleeps in hardware instead of burning issue slots

// ---------------------------------------------------------------- mbarrier / bulk-copy primitives
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
// 2-D tiled TMA copy: the box of `tmap` at element coordinates (x, y) -> dense rows at dst (128-byte aligned).
// x * element size must be a multiple of 16 bytes.  No multicast: the box lands in this CTA only.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// 3-D form for the packed weights ([rows][group pairs][32 int32], swizzled image): coordinates (0, group / 2, row).
__device__ __forceinline__ void tma_load_w(void* dst, const CUtensorMap* tmap, int group, int row, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst)),
      "l"(tmap), "r"(0), "r"(group >> 1), "r"(row), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_w(const CUtensorMap* tmap, int group, int row) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];" ::"l"(tmap), "r"(0), "r"(group >> 1), "r"(row)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}
// L2 prefetch request (no shared memory involved) for a flat byte range (16-byte aligned address, size a multiple
// of 16).
__device__ __forceinline__ void l2_prefetch_bytes(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// 4-byte asynchronous copy global -> shared (LDGSTS) and its completion hook on an mbarrier: the arrive fires
// once all of this thread's earlier cp.async copies have landed; it counts as one of the barrier's arrivals.
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive(uint64_t* b) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

// Tuning switches (skip the MMAs, skip the copies, other wait flavours, timeline) exist only in builds with
// -DGLOWQ_GEMV_TRACE; otherwise this is the constant 0 and every branch on it is compiled out.
__device__ __forceinline__ int tuning_bits(const GemvParams& p) {
#ifdef GLOWQ_GEMV_TRACE
  return p.debug;
#else
  (void)p;
  return 0;
#endif
}

struct Ctx {
  volatile int* abort_flag;
  uint32_t* status;
  int mode;
};

// Tuning aid, compiled in with -DGLOWQ_GEMV_TRACE only (debug & 16, needs a workspace of at least 40 MB): event e of
// CTA b -> %globaltimer at workspace + 32 MB.
__device__ __forceinline__ void trace_event(const GemvParams& p, int e) {
#ifdef GLOWQ_GEMV_TRACE
  if (tuning_bits(p) & 16) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(p.ws_head) + (32u << 20))[blockIdx.x * 16 + e] = t;
  }
#else
  (void)p;
  (void)e;
#endif
}

// ---------------------------------------------------------------- activations
// Fused residual add + RMSNorm (HF LlamaRMSNorm / Qwen2RMSNorm semantics): h = fp16(x + residual),
// xn = w * fp16(h * rstd) with rstd = rsqrt(mean(h^2) + eps) in fp32.  Eight consecutive columns k .. k+7 of token m.
__device__ __forceinline__ uint4 residual_add8(const GemvParams& p, uint4 xv, int m, int k) {
  if (p.residual == nullptr) return xv;
  const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(m) * p.x_stride + k);
  const __half2* x2 = reinterpret_cast<const __half2*>(&xv);
  const __half2* r2 = reinterpret_cast<const __half2*>(&rv);
  uint4 out;
  __half2* o2 = reinterpret_cast<__half2*>(&out);
#pragma unroll
  for (int e = 0; e < 4; ++e) o2[e] = __hadd2(x2[e], r2[e]);
  return out;
}
__device__ __forceinline__ uint4 norm_x8(const GemvParams& p, uint4 xv, int m, int k, float rstd) {
  const uint4 hv = residual_add8(p, xv, m, k);
  const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + k);
  const __half2* h2 = reinterpret_cast<const __half2*>(&hv);
  const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
  uint4 out;
  __half2* o2 = reinterpret_cast<__half2*>(&out);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __half22float2(h2[e]);
    o2[e] = __hmul2(w2[e], __floats2half2_rn(f.x * rstd, f.y * rstd));
  }
  return out;
}
// rstd of every token row into s_rstd[0..M) (all consumer threads take part; `part` is scratch of 64 floats), and, on
// CTA 0, h -> hidden_out.  IC is a multiple of 8 and the rows are 16-byte aligned (checked on the host).
__device__ __forceinline__ void norm_stats(const GemvParams& p, float* part, float* s_rstd) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = p.IC >> 3;
  for (int m = 0; m < p.M; ++m) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nv; c += kConsumerThreads) {
      const uint4 xv = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.x_stride + 8 * c);
      const uint4 hv = residual_add8(p, xv, m, 8 * c);
      if (p.hidden_out != nullptr && blockIdx.x == 0)
        *reinterpret_cast<uint4*>(p.hidden_out + static_cast<size_t>(m) * p.x_stride + 8 * c) = hv;
      const __half2* h2 = reinterpret_cast<const __half2*>(&hv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h2[e]);
        ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) part[warp * 8 + m] = ss;
  }
  consumer_sync();
  if (threadIdx.x < p.M) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) tot += part[w * 8 + threadIdx.x];
    s_rstd[threadIdx.x] = rsqrtf(tot / static_cast<float>(p.IC) + p.norm_eps);
  }
  consumer_sync();
}

// Stage x[0:M, g0*128 : (g0+ng)*128) into shared memory in MMA B-fragment order: for token m and group gl,
// 16-byte chunk (i*4 + t) holds the columns 32t+8i+{0,4,1,5,2,6,3,7} of that group, the ones at odd positions of
// a packed word (1,5,3,7) multiplied by 1/16 (see the consumer loop), and xsum[gl][m] = sum of the group's x in
// fp32 (for the zero-point term).  Every consumer warp stages exactly the groups it consumes itself (gl = warp,
// warp + 8, ... of the slice; sixteen lanes per group, two groups per pass), so no warp waits for another one
// between "x is ready" and its first MMA: a __syncwarp() publishes the data.
__device__ __forceinline__ void stage_x(const GemvParams& p, int g0, int ng, unsigned char* xs, float* xsum, int mpad,
                                        const float* s_rstd, bool do_norm) {
  constexpr int kBatch = 4;  // global loads in flight per lane before any of them is consumed
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hsel = lane >> 4, s = lane & 15;   // s = 8-column block of the group, in source order
  const int n_mine = ng > warp ? (ng - warp + kConsumerWarps - 1) / kConsumerWarps : 0;
  const int passes = (n_mine + 1) >> 1;
  for (int m = 0; m < p.M; ++m) {
    for (int p0 = 0; p0 < passes; p0 += kBatch) {
      uint4 v[kBatch];
      int glv[kBatch];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int gl = warp + kConsumerWarps * (2 * (p0 + b) + hsel);
        const bool valid = (p0 + b) < passes && gl < ng;
        glv[b] = valid ? gl : -1;
        v[b] = make_uint4(0, 0, 0, 0);
        if (valid) {
          const int k = (g0 + gl) * kGroup + 8 * s;
          const __half* src = p.x + static_cast<size_t>(m) * p.x_stride + k;
          if (p.x_vec_ok && k + 8 <= p.IC) {
            v[b] = *reinterpret_cast<const uint4*>(src);
            if (do_norm) v[b] = norm_x8(p, v[b], m, k, s_rstd[m]);
          } else {
            __align__(16) __half tmp[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = (k + e < p.IC) ? src[e] : __float2half(0.f);
            v[b] = *reinterpret_cast<const uint4*>(tmp);
          }
        }
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const __half2* h2 = reinterpret_cast<const __half2*>(&v[b]);
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h2[e]);
          part += f.x + f.y;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);  // the 16 lanes of one (m, gl)
        if (glv[b] >= 0) {
          uint4 o4 = interleave_pairs(v[b]);
          o4.y = hmul2(o4.y, 0x2C002C00u);
          o4.w = hmul2(o4.w, 0x2C002C00u);
          const int i = s & 3, t = s >> 2;
          *reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * p.xs_stride + (glv[b] * 16 + i * 4 + t) * 16) = o4;
          if (s == 0) xsum[glv[b] * mpad + m] = part;
        }
      }
    }
  }
  __syncwarp();
}

// ---------------------------------------------------------------- shared-space (32-bit address) accessors
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
// The same loads with a compile-time byte offset folded into the instruction (an address register plus an immediate
// costs no integer add; a sum computed in C++ and passed to the asm statement does).
template <int OFF>
__device__ __forceinline__ uint4 lds128_at(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ float2 lds_f2_at(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(a), "n"(OFF));
  return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void mbar_arrive_u32(uint32_t a) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}
// Whole-warp bounded wait on one phase of an mbarrier (32-bit shared address).
__device__ __forceinline__ bool mbar_wait_u32(uint32_t a, uint32_t parity, const Ctx& cx) {
  uint32_t spins = 0;
  for (;;) {
    uint32_t ok;
    if (cx.mode & 4) {
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok)
                   : "r"(a), "r"(parity)
                   : "memory");
    } else {
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(a), "r"(parity), "r"((cx.mode & 8) ? 20u : kSuspendHintNs)
          : "memory");
    }
    if (ok) return true;
    if ((++spins & 15u) == 0 && *cx.abort_flag) return false;
    if (spins > kMbarSpinLimit) {
      *cx.abort_flag = 1;
      atomicExch(cx.status, 2u);
      return false;
    }
  }
}

// Sum the per-warp accumulators of NB fragment blocks; fin[b*128 + tok*16 + row] (tok < 8, row < 16) receives the
// CTA's sum of block b.
template <int NB>
__device__ __forceinline__ void cross_warp_reduce(float (&acc)[NB][4], float* red, float* fin) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int b = 0; b < NB; ++b)
    reinterpret_cast<float4*>(red)[(warp * NB + b) * 32 + lane] = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
  consumer_sync();
  for (int e = threadIdx.x; e < NB * 128; e += kConsumerThreads) {
    const int b = e >> 7, ln = (e & 127) >> 2, c = e & 3;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) s += red[((w * NB + b) * 32 + ln) * 4 + c];
    const int row = (ln >> 2) + ((c & 2) ? 8 : 0);
    const int tok = (ln & 3) * 2 + (c & 1);
    fin[b * 128 + tok * 16 + row] = s;
  }
  consumer_sync();
}

// The wait for the previous kernels of the stream, once per warp.
__device__ __forceinline__ void dep_wait(bool& pending) {
  if (!pending) return;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  pending = false;
}
// Epoch that stamps the words of r in this launch (never 0, the value of a word that was never written), from the
// epoch word as the CTA's registration found it: it carries the epoch of the PREVIOUS correcting launch.
__device__ __forceinline__ uint32_t launch_epoch(uint32_t eword) {
  const uint32_t e = ((eword >> kEpochShift) + 1u) & kEpochMask;
  return e == 0u ? 1u : e;
}

// R units u0, u0 + ustride, ... of this CTA.  One unit: rows [16 rt, 16 rt + 16) of R times the columns of K slice
// ks (gpr groups; warp w takes groups w, w + 8, ...), tokens 0..M-1.  The fp32 result goes to the unit's own slot of
// r_partial.  R is static: the first round's loads and L2 prefetch requests for every later round of the CTA go out
// before the wait for the previous kernel, and the CTA publishes all of its units with ONE fence and one add to the
// release counter.  The CTA whose add completes the count adds the SKr slots of every R tile in slot order, rounds
// to fp16 and writes r twice: plain into r_buf (for later launches that load it) and as 8-byte words {two elements,
// epoch of this launch} for the row tiles of this launch, which poll the words they need - one L2 round trip, no
// flag and no fence on the reading side, and every reader sees the same bits.
template <int NT>
__device__ __forceinline__ void r_units(const GemvParams& p, int u0, int ustride, float* red, float* fin,
                                        bool& dep_wait_pending, const volatile uint32_t* s_eword, uint32_t epoch_bar_u32,
                                        Ctx cx, const float* s_rstd, bool do_norm, bool& closes_epoch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  if (u0 >= p.n_r_units) return;
  uint4 a[4], b[4];
  // one round of a unit for this warp: 16 rows x 128 columns (group gl of the unit's K slice); `fetch` false only asks
  // L2 for the lines (no registers are held, the loads that follow later hit L2)
  auto load_round = [&](int unit, int gl, bool fetch) {
    const int rt = unit / p.SKr, ks = unit - rt * p.SKr;
    const int j0 = rt * kRTileRows;
    const int ng = min(p.gpr, p.G - ks * p.gpr);
    const __half* rowA = p.R + static_cast<size_t>(min(j0 + g, p.rank - 1)) * p.R_stride;
    const __half* rowB = p.R + static_cast<size_t>(min(j0 + g + 8, p.rank - 1)) * p.R_stride;
    const int kb = (ks * p.gpr + gl) * kGroup + 32 * t;
    if (!fetch) {
      if (gl < ng && kb + 32 <= p.IC) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(rowA + kb));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(rowB + kb));
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = kb + 8 * i;
      const bool ok = gl < ng && (k + 8 <= p.IC);
      a[i] = ok ? ldg_stream_v4(rowA + k) : make_uint4(0, 0, 0, 0);
      b[i] = ok ? ldg_stream_v4(rowB + k) : make_uint4(0, 0, 0, 0);
    }
  };
  // the lines of every later round of this CTA go to L2 right away; the first round is loaded for real
  for (int unit = u0; unit < p.n_r_units; unit += ustride)
    for (int gl = warp + (unit == u0 ? kConsumerWarps : 0); gl < p.gpr; gl += kConsumerWarps) load_round(unit, gl, false);
  load_round(u0, warp, true);
  int n_done = 0;
  for (int unit = u0; unit < p.n_r_units; unit += ustride) {
    const int rt = unit / p.SKr, ks = unit - rt * p.SKr;
    const int gbase = ks * p.gpr, ng = min(p.gpr, p.G - gbase);
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    for (int gl = warp; gl < ng || gl == warp; gl += kConsumerWarps) {
      const bool more_rounds = gl + kConsumerWarps < ng;
      if (gl != warp || unit != u0) load_round(unit, gl, true);
      dep_wait(dep_wait_pending);  // R is static, x is not: the earlier kernels must be complete before x is read
      if (gl < ng) {
        const int kb = (gbase + gl) * kGroup + 32 * t;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int tok = nt * 8 + g;
          // all four activation loads of the round go out before the first MMA needs one (they are L2 round trips)
          uint4 xv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int k = kb + 8 * i;
            xv[i] = make_uint4(0, 0, 0, 0);
            if (tok < p.M && k + 8 <= p.IC) {
              const __half* src = p.x + static_cast<size_t>(tok) * p.x_stride + k;
              if (p.x_vec_ok) {
                xv[i] = ldg_cg_v4(src);
              } else {
                __align__(16) __half tmp[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) tmp[e] = src[e];
                xv[i] = *reinterpret_cast<const uint4*>(tmp);
              }
            }
          }
          if (do_norm && p.x_vec_ok && tok < p.M) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (kb + 8 * i + 8 <= p.IC) xv[i] = norm_x8(p, xv[i], tok, kb + 8 * i, s_rstd[tok]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            mma16816(acc[nt], a[i].x, b[i].x, a[i].y, b[i].y, xv[i].x, xv[i].y);
            mma16816(acc[nt], a[i].z, b[i].z, a[i].w, b[i].w, xv[i].z, xv[i].w);
          }
        }
      }
      if (!more_rounds) break;
    }
    cross_warp_reduce<NT>(acc, red, fin);  // fin[nt*128 + tok8*16 + row16]
    float* slot = p.r_partial + static_cast<size_t>(unit) * (NT * 128);
    for (int e = threadIdx.x; e < NT * 128; e += kConsumerThreads) slot[e] = fin[e];
    ++n_done;
  }
  dep_wait(dep_wait_pending);
  consumer_sync();
  uint32_t* last_flag = reinterpret_cast<uint32_t*>(fin);   // fin is free again
  if (threadIdx.x == 0) {
    // Release / acquire by one thread on behalf of the CTA: the barrier above orders every thread's slot stores
    // before this thread's fence, and the barrier below orders its second fence before every thread's slot loads.
    __threadfence();
    const uint32_t before = atomicAdd(p.ws_head + WS_R_DONE, static_cast<uint32_t>(n_done));
    const bool last = before + static_cast<uint32_t>(n_done) == static_cast<uint32_t>(p.n_r_units);
    if (last) __threadfence();
    *last_flag = last ? 1u : 0u;
  }
  consumer_sync();
  if (*last_flag != 0u) {
    mbar_wait_u32(epoch_bar_u32, 0, cx);   // the CTA's registration (its aux warp) has returned
    const uint32_t epoch = launch_epoch(*s_eword);
    const int q4 = p.rank >> 2;  // rank is a multiple of 8
    for (int i = threadIdx.x; i < p.M * q4; i += kConsumerThreads) {
      const int tok = i / q4, j = (i - tok * q4) * 4;
      const float* base = p.r_partial + (static_cast<size_t>(j >> 4) * p.SKr * NT + (tok >> 3)) * 128 + (tok & 7) * 16 + (j & 15);
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int ks0 = 0; ks0 < p.SKr; ks0 += 4) {  // four slots in flight, added in slot order
        float4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          q[u] = (ks0 + u < p.SKr) ? __ldcg(reinterpret_cast<const float4*>(base + static_cast<size_t>(ks0 + u) * (NT * 128)))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s.x += q[u].x; s.y += q[u].y; s.z += q[u].z; s.w += q[u].w;
        }
      }
      const __half2 h01 = __floats2half2_rn(s.x, s.y), h23 = __floats2half2_rn(s.z, s.w);
      const uint32_t u01 = *reinterpret_cast<const uint32_t*>(&h01), u23 = *reinterpret_cast<const uint32_t*>(&h23);
      uint2* w = p.r_ll + static_cast<size_t>(tok) * (p.rank >> 1) + (j >> 1);
      w[0] = make_uint2(u01, epoch);
      w[1] = make_uint2(u23, epoch);
      if (p.r_buf != nullptr) *reinterpret_cast<uint2*>(p.r_buf + static_cast<size_t>(tok) * p.rank + j) = make_uint2(u01, u23);
    }
    if (threadIdx.x == 0) p.ws_head[WS_R_DONE] = 0u;   // nothing of this launch touches the unit counter any more
    closes_epoch = true;   // (the caller advances the epoch when the CTA retires: see advance_epoch)
  }
}

// The epoch of the workspace moves on once every CTA of the grid has registered on it.  All CTAs are resident and
// register right after the wait for the previous kernels; the CTA that completed r does this as its last action, long
// after, so the loop normally ends at once (bounded all the same).
__device__ __forceinline__ void advance_epoch(const GemvParams& p, uint32_t eword) {
  const uint32_t readers = gridDim.x;   // one registration per CTA
  uint32_t spins = 0;
  while ((ld_acquire_u32(p.ws_head + WS_EPOCH) & kEpochReaderMask) != readers) {
    __nanosleep(128);
    if (++spins > kSpinLimit) {
      atomicExch(p.ws_head + WS_STATUS, 1u);
      return;
    }
  }
  p.ws_head[WS_EPOCH] = launch_epoch(eword) << kEpochShift;
}

// Eight consecutive elements r[tok][j .. j+8) (j a multiple of 8) of THIS launch as four half2 registers: polls the
// four {two elements, epoch} words until all carry the launch's epoch (bounded).
__device__ __forceinline__ uint4 r_frag_poll(const GemvParams& p, int tok, int j, uint32_t epoch, volatile int* abort_flag) {
  const uint2* w = p.r_ll + static_cast<size_t>(tok) * (p.rank >> 1) + (j >> 1);   // 32-byte aligned
  uint32_t spins = 0;
  for (;;) {
    const uint4 a = ld_volatile_v4(w), b = ld_volatile_v4(w + 2);
    if (a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch) return make_uint4(a.x, a.z, b.x, b.z);
    if (*abort_flag || ++spins > kSpinLimit) {
      *abort_flag = 1;
      atomicExch(p.ws_head + WS_STATUS, 1u);
      return make_uint4(0, 0, 0, 0);
    }
  }
}

struct TileInfo {
  int mi, row0;
  bool corr;
};
__device__ __forceinline__ TileInfo tile_info(const GemvParams& p, int tile, int slice, int r_mode) {
  int mi = 0;
#pragma unroll
  for (int i = 1; i < kMaxMembers; ++i)
    if (i < p.n_members && tile >= p.mem[i].tile_begin) mi = i;
  TileInfo ti;
  ti.mi = mi;
  ti.row0 = (tile - p.mem[mi].tile_begin) * kTileRows;
  ti.corr = (slice == 0) && (r_mode != 0) && (p.mem[mi].L != nullptr) && (p.mem[mi].alpha != 0.f);
  return ti;
}

#ifndef GLOWQ_GEMV_MIN_CTAS
#define GLOWQ_GEMV_MIN_CTAS 2   // CTAs per SM the register allocation is bounded for
#endif
// FEAT selects what is compiled in: bit 0 the low-rank correction, bit 1 K slices, bits 2 and 3 the optional extras
// (tensor-parallel push, fused input transform).  A launch takes the smallest instantiation the host offers that covers
// it: the code of features that are switched off costs instruction-cache misses and predicated instructions on every
// launch (the everything-in instantiation is 1.6 times the size of the corrected one and measured 3 % slower on it).
enum : int { kFeatCorr = 1, kFeatSliced = 2, kFeatPush = 4, kFeatNorm = 8 };
template <int NT, int FEAT>
__global__ void __launch_bounds__(kGemvThreads, (NT <= 2) ? GLOWQ_GEMV_MIN_CTAS : 1)
gemv_stream_kernel(const __grid_constant__ GemvParams p, const __grid_constant__ TensorMaps tm) {
  const int r_mode = (FEAT & kFeatCorr) ? p.r_mode : 0;
  const int SK = (FEAT & kFeatSliced) ? p.SK : 1;
  const int push_world = (FEAT & kFeatPush) ? p.push_world : 0;
  const __half* const norm_w = (FEAT & kFeatNorm) ? p.norm_w : nullptr;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_abort;
  __shared__ uint32_t s_eword;   // the workspace's epoch word as this CTA's registration found it
  __shared__ float s_rstd[8];   // fused RMSNorm: 1 / rms of every token row
  constexpr int RT = kRowTiles;
  constexpr int NB = RT * NT;  // 16-row x 8-token fragment blocks per tile

  // shared-memory carve-up (must match gemv_smem_layout_bytes)
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* meta_full = empty_bar + kMaxStages;       // [kMetaDepth]: a tile's raw scales / zero words have landed
  uint64_t* cooked_full = meta_full + kMetaDepth;     // [kCookedDepth]: a tile's converted pairs are written
  uint64_t* cooked_empty = cooked_full + kCookedDepth;  // ... and the consumer warps are done with them
  uint64_t* red_empty = cooked_empty + kCookedDepth;  // the aux warp has drained the reduction buffer
  uint64_t* epoch_bar = red_empty + 1;                // the CTA's registration on the workspace's epoch word has returned
  // the swizzle of the weight stages works on shared-memory address bits: stages start on 1024-byte boundaries
  unsigned char* ring = smem + 256 + ((1024u - ((smem_u32(smem) + 256u) & 1023u)) & 1023u);
  const int meta_bytes = kTileRows * (p.meta_gp * 2 + p.meta_gw * 4);
  unsigned char* meta = ring + static_cast<size_t>(p.stages) * kStageBytes;
  const int cooked_bytes = p.gps * (kTileRows * 8);   // [group][row] float2 {scale * 2^24, -scale * zero}
  unsigned char* cooked = meta + static_cast<size_t>(kMetaDepth) * meta_bytes;
  float* red = reinterpret_cast<float*>(cooked + static_cast<size_t>(kCookedDepth) * cooked_bytes);
  float* fin = red + kConsumerWarps * NB * 128;      // one reduction buffer; fin serves the R units only
  float* xsum = fin + NT * 128;                      // [groups of the slice][8 NT]
  unsigned char* xs = reinterpret_cast<unsigned char*>(xsum + p.gps * (8 * NT));
  unsigned char* zero_row = xs + static_cast<size_t>(p.M) * p.xs_stride;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages;
  // Epoch stamped into the pushed words: this site's call counter + 1.  The counter only moves when the last CTA of a
  // pushing launch leaves; it is read AFTER the wait for the previous kernels (a launch may start long before its
  // predecessors are complete), by the roles that store outputs.
  uint32_t push_e = 0u;
  bool closes_epoch = false;   // consumer threads of the CTA that completed r: it advances the workspace's epoch at its end
  // The last n_r_ctas CTAs of the grid only compute r (their copy / aux warps have no tiles): a CTA that ran an R
  // unit AND a full share of row tiles would finish microseconds after the others and set the kernel's length.
  const int n_main = static_cast<int>(gridDim.x) - p.n_r_ctas;
  // Logical CTA index: main CTAs 0 .. n_main-1, then the R CTAs.  The R CTAs take the LOWEST block indices, which
  // the hardware places first: while the previous kernel still holds most CTA slots they are the ones that are
  // resident early, with their loads of R done before x is ready.
  const int bid = static_cast<int>(blockIdx.x) >= p.n_r_ctas ? static_cast<int>(blockIdx.x) - p.n_r_ctas
                                                             : n_main + static_cast<int>(blockIdx.x);
  const bool r_only = bid >= n_main;
  const int slice = bid % SK;
  const int first_tile = r_only ? p.n_tiles : bid / SK;
  const int tile_step = n_main / SK;
  // k-th row tile of this CTA (>= n_tiles: none left).  With K slices every CTA of a slice strides over the tiles.
  // Without, the first round of tiles goes to the main CTAs only and the rest is dealt over ALL CTAs, so that the
  // CTAs that computed r pick up row tiles afterwards instead of idling through a long launch.
  const bool deal_all = (SK == 1 && p.n_r_ctas > 0);
  // The leftover tiles are dealt in the order [R CTAs, main CTAs]: an R CTA is free again about two microseconds
  // into the launch, a main CTA only after its first tile.
  auto tile_at = [&](int k) -> int {
    if (!deal_all) return first_tile + k * tile_step;
    if (r_only) return bid + k * static_cast<int>(gridDim.x);
    return k == 0 ? bid : n_main + p.n_r_ctas + bid + (k - 1) * static_cast<int>(gridDim.x);
  };
  const int g0 = slice * p.gps;
  const int ng = min(p.G, g0 + p.gps) - g0;
  const int n_chunks = (ng + kChunkGroups - 1) / kChunkGroups;
  const int n_lstages = (p.rank + 255) >> 8;

  // Programmatic dependent launch: let the next kernel of the stream start its own prologue (barrier set-up, weight
  // and metadata copies - nothing that depends on this kernel) as soon as every CTA of this grid is resident.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) trace_event(p, 0);
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(full_bar + i, 1);
      mbar_init(empty_bar + i, kConsumerWarps);
    }
    for (int i = 0; i < kMetaDepth; ++i) mbar_init(meta_full + i, 32);
    for (int i = 0; i < kCookedDepth; ++i) {
      mbar_init(cooked_full + i, 1);
      mbar_init(cooked_empty + i, kConsumerWarps);
    }
    mbar_init(red_empty, 1);
    mbar_init(epoch_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x >= 32 && threadIdx.x < 32 + kZeroRowBytes / 4) reinterpret_cast<uint32_t*>(zero_row)[threadIdx.x - 32] = 0u;
  __syncthreads();
  if (threadIdx.x == 0) trace_event(p, 1);
  Ctx cx{&s_abort, p.ws_head + WS_STATUS, tuning_bits(p)};
  const uint32_t full_u32 = smem_u32(full_bar), empty_u32 = smem_u32(empty_bar);
  const uint32_t mfull_u32 = smem_u32(meta_full);
  const uint32_t cfull_u32 = smem_u32(cooked_full), cempty_u32 = smem_u32(cooked_empty);
  const uint32_t rempty_u32 = smem_u32(red_empty);
  const uint32_t epoch_bar_u32 = smem_u32(epoch_bar);

  if (warp == kConsumerWarps) {
    // ================================================================ weight / L copy warp
    // One 2-D TMA copy per pipeline stage: kTileRows rows x 512 B of packed weights (or x l_cols of L).  Per-row
    // bulk copies of 512 B cap the copy engine at a fraction of HBM rate; one 16 KB box per instruction does not.
    uint32_t st = 0, ph = 0, issued = 0;
    bool ok = true;
    for (int k = 0, tile; (tile = tile_at(k)) < p.n_tiles && ok; ++k) {
      const TileInfo ti = tile_info(p, tile, slice, r_mode);
      // L2 lookahead: with every weight chunk handed to the ring, the chunk that will follow S issues later (a later
      // chunk of this tile or one of the CTA's next tiles) is requested from L2.  The ring is only S stages deep, so
      // at the start of a launch - all slots filled, consumers still waiting for x - the chunks beyond it would
      // otherwise be fetched from HBM one by one as slots free up, each exposing a full DRAM round trip.
      for (int c = 0; c < n_chunks; ++c) {
        if (!(ok = mbar_wait_u32(empty_u32 + st * 8, ph ^ 1, cx))) break;
        if (lane == 0) {
          if (tuning_bits(p) & 2) {
            mbar_arrive(full_bar + st);
          } else {
            mbar_arrive_expect_tx(full_bar + st, kStageBytes);
            if (p.w_swizzled)
              tma_load_w(ring + static_cast<size_t>(st) * kStageBytes, &tm.w[ti.mi], g0 + c * kChunkGroups, ti.row0, full_bar + st);
            else
              tma_load_2d(ring + static_cast<size_t>(st) * kStageBytes, &tm.w[ti.mi], (g0 + c * kChunkGroups) * 16, ti.row0,
                          full_bar + st);
            if (p.deep_prefetch) {
              const int pi = k * n_chunks + c + S;              // weight chunk index (within this CTA) S issues ahead
              const int kp = pi / n_chunks, cp = pi - kp * n_chunks;
              const int tile_p = tile_at(kp);
              if (tile_p < p.n_tiles) {
                const TileInfo tp_ = tile_info(p, tile_p, slice, r_mode);
                if (p.w_swizzled)
                  tma_prefetch_w(&tm.w[tp_.mi], g0 + cp * kChunkGroups, tp_.row0);
                else
                  tma_prefetch_2d(&tm.w[tp_.mi], (g0 + cp * kChunkGroups) * 16, tp_.row0);
              }
            }
          }
        }
        ++issued;
        if (++st == static_cast<uint32_t>(S)) {
          st = 0;
          ph ^= 1;
        }
      }
      if (ok && ti.corr) {
        for (int l = 0; l < n_lstages; ++l) {
          if (!(ok = mbar_wait_u32(empty_u32 + st * 8, ph ^ 1, cx))) break;
          if (lane == 0) {
            mbar_arrive_expect_tx(full_bar + st, static_cast<uint32_t>(p.l_cols) * 2u * kTileRows);
            tma_load_2d(ring + static_cast<size_t>(st) * kStageBytes, &tm.l[ti.mi], 256 * l, ti.row0, full_bar + st);
          }
          ++issued;
          if (++st == static_cast<uint32_t>(S)) {
            st = 0;
            ph ^= 1;
          }
        }
      }
    }
    if (ok && p.n_pf > 0) {
      // This CTA's own copies are all issued: ask L2 for its share of what the NEXT call on the stream reads first
      // (slices of kPrefetchSlice bytes dealt round-robin over the grid's copy warps, one per lane and turn).
      for (int r = 0; r < p.n_pf; ++r) {
        const uint32_t bytes = p.pf_bytes[r];
        const uint32_t n_slices = (bytes + kPrefetchSlice - 1) / kPrefetchSlice;
        for (uint32_t sidx = blockIdx.x + lane * gridDim.x; sidx < n_slices; sidx += 32u * gridDim.x) {
          const uint32_t off = sidx * kPrefetchSlice;
          l2_prefetch_bytes(p.pf_ptr[r] + off, min(kPrefetchSlice, bytes - off));
        }
      }
    }
    if (!ok && !(tuning_bits(p) & 2)) {
      // Draining: copies already issued still land in this CTA's shared memory; wait (bounded) for them so that
      // the CTA does not retire under an in-flight copy.
      for (uint32_t j = (issued > static_cast<uint32_t>(S) ? issued - S : 0); j < issued; ++j) {
        uint32_t spins = 0;
        while (!mbar_try_wait(full_bar + (j % S), (j / S) & 1) && ++spins < kDrainSpinLimit) {
        }
      }
    }
  } else if (warp == kConsumerWarps + 1) {
    // ================================================================ aux warp: metadata + tile epilogues
    // Lane r fetches row r's scales / zero words three tiles ahead with asynchronous 4-byte copies (the warp never
    // waits for a load it has just issued), and one tile ahead of the consumers converts them ONCE per (row, group)
    // into the fp32 pair {scale * 2^24, -scale * zero} the consumers' group epilogue multiplies with, laid out
    // [group][row] (the consumer warps, four lanes per row, would otherwise each repeat the unpacking and the
    // conversions - on the integer pipe, which is the busiest unit of this kernel).  Between that it finishes tiles:
    // once the eight consumer warps have parked their partial sums in a reduction buffer (named barrier 2 + buf) it
    // adds them up, runs the split-K combine, bias and the store, and hands the buffer back.  Consumers therefore
    // never wait for one another; only a CTA's LAST tile is summed by the consumer warps themselves (when K is not
    // sliced), because they have nothing else left to do and 256 threads finish it sooner than one warp.
    uint32_t buf = 0;
    int k_m = 0;   // next tile (k-th of this CTA) whose raw metadata gets prefetched; raw slot k % kMetaDepth
    bool ok = true;
    auto prefetch_raw = [&]() {
      const int tile_m = tile_at(k_m);
      const TileInfo tm_i = tile_info(p, tile_m, slice, r_mode);
      const MemberDev& mbm = p.mem[tm_i.mi];
      const uint32_t slot = static_cast<uint32_t>(k_m % kMetaDepth);
      const int row = min(tm_i.row0 + lane, mbm.OC - 1);
      unsigned char* mbase = meta + static_cast<size_t>(slot) * meta_bytes;
      __half* ms = reinterpret_cast<__half*>(mbase) + lane * p.meta_gp;
      uint32_t* mz = reinterpret_cast<uint32_t*>(mbase + kTileRows * p.meta_gp * 2) + lane * p.meta_gw;
      const __half* srow = mbm.scales + static_cast<size_t>(row) * mbm.sstride + g0;
      if (((mbm.sstride | g0) & 1) == 0 && ((reinterpret_cast<uintptr_t>(mbm.scales) & 3) == 0)) {
        const int np_full = ng >> 1;
        for (int pi = 0; pi < np_full; ++pi) cp_async4(ms + 2 * pi, srow + 2 * pi);
        if (ng & 1) ms[ng - 1] = srow[ng - 1];  // odd tail: there may be no 4 readable bytes at the end of a row
      } else {
        for (int gl = 0; gl < ng; ++gl) ms[gl] = srow[gl];
      }
      const int32_t* zrow = mbm.qzeros + static_cast<size_t>(row) * mbm.zstride + (g0 >> 3);
      const int nw = (ng + 7) >> 3;
      for (int wi = 0; wi < nw; ++wi) cp_async4(mz + wi, zrow + wi);
      cp_async_mbar_arrive(meta_full + slot);
      ++k_m;
    };
    // convert the raw metadata of this CTA's kc-th tile (it was prefetched earlier) into cooked slot kc % kCookedDepth
    auto cook = [&](int kc) {
      const uint32_t rslot = static_cast<uint32_t>(kc % kMetaDepth), rph = static_cast<uint32_t>(kc / kMetaDepth) & 1u;
      const uint32_t cslot = static_cast<uint32_t>(kc % kCookedDepth), cph = static_cast<uint32_t>(kc / kCookedDepth) & 1u;
      ok = ok && mbar_wait_u32(mfull_u32 + rslot * 8, rph, cx);
      ok = ok && mbar_wait_u32(cempty_u32 + cslot * 8, cph ^ 1, cx);
      if (ok) {
        const unsigned char* mbase = meta + static_cast<size_t>(rslot) * meta_bytes;
        const __half* ms = reinterpret_cast<const __half*>(mbase) + lane * p.meta_gp;
        const uint32_t* mz = reinterpret_cast<const uint32_t*>(mbase + kTileRows * p.meta_gp * 2) + lane * p.meta_gw;
        float2* dst = reinterpret_cast<float2*>(cooked + static_cast<size_t>(cslot) * cooked_bytes) + lane;
        for (int wi = 0; wi * 8 < ng; ++wi) {
          const uint32_t zw = mz[wi];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const int gl = wi * 8 + j;
            if (gl < ng) {
              const __half2 sp = *reinterpret_cast<const __half2*>(ms + gl);   // groups gl, gl + 1 (pitch is even)
              const float2 sf = __half22float2(sp);
              const float z0 = static_cast<float>((zw >> (4 * j)) & 0xFu), z1 = static_cast<float>((zw >> (4 * j + 4)) & 0xFu);
              dst[gl * kTileRows] = make_float2(sf.x * 16777216.f, -sf.x * z0);
              if (gl + 1 < ng) dst[(gl + 1) * kTileRows] = make_float2(sf.y * 16777216.f, -sf.y * z1);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(cooked_full + cslot);
    };
    while (k_m < kMetaDepth && tile_at(k_m) < p.n_tiles) prefetch_raw();
    if (tile_at(0) < p.n_tiles) cook(0);
    // A correcting launch: ONE add per CTA registers it as a reader of the workspace's epoch word, once the previous
    // kernels are complete (eight adds per CTA - one per consumer warp - were 2400 operations on one address right
    // when every CTA comes out of its wait, and staggered the CTAs by a microsecond).  The consumers pick the value
    // up behind a barrier, at their first L epilogue.
    bool aux_dep_pending = true;
    if (r_mode == 1) {
      dep_wait(aux_dep_pending);
      if (lane == 0) {
        s_eword = atomicAdd(p.ws_head + WS_EPOCH, 1u);
        mbar_arrive(epoch_bar);
      }
    }
    for (int k = 0, tile; (tile = tile_at(k)) < p.n_tiles; ++k) {
      // raw slot k % kMetaDepth was cooked in the previous round: refill it with the tile three ahead
      if (k_m == k + kMetaDepth && tile_at(k_m) < p.n_tiles) prefetch_raw();
      const bool last = tile_at(k + 1) >= p.n_tiles;
      if (!last) cook(k + 1);
      if (last && SK == 1) break;   // the consumer warps finish this tile themselves

      // ---- epilogue of `tile` (outputs may still be read by the previous kernel until it has completed)
      if (k == 0) {
        dep_wait(aux_dep_pending);
        if (push_world > 0) push_e = *p.push_epoch + 1u;
      }
      const TileInfo ti = tile_info(p, tile, slice, r_mode);
      const MemberDev& mb = p.mem[ti.mi];
      if (buf == 0)
        asm volatile("bar.sync 2, %0;" ::"n"(kConsumerThreads + 32) : "memory");
      else
        asm volatile("bar.sync 3, %0;" ::"n"(kConsumerThreads + 32) : "memory");
      const float4* red4 = reinterpret_cast<const float4*>(red);
      float4 v[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        v[b] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          const float4 q = red4[(w * NB + b) * 32 + lane];
          v[b].x += q.x;
          v[b].y += q.y;
          v[b].z += q.z;
          v[b].w += q.w;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(red_empty);  // the consumers may refill the buffer
      buf ^= 1;                               // (the named barriers alternate)
      bool finalize = true;
      if (SK > 1) {
        // every K slice parks its tile; the last slice to arrive adds them up in slice order (deterministic)
        float4* part = reinterpret_cast<float4*>(p.sk_partial + static_cast<size_t>(tile) * SK * (NB * 128));
#pragma unroll
        for (int b = 0; b < NB; ++b) part[static_cast<size_t>(slice) * (NB * 32) + b * 32 + lane] = v[b];
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = (atomicAdd(p.tile_ctr + tile, 1u) == static_cast<uint32_t>(SK - 1));
        last = __shfl_sync(0xffffffffu, last, 0);
        finalize = (last != 0);
        if (finalize) {
          __threadfence();
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < SK; ++k) {
              const float4 q = __ldcg(part + static_cast<size_t>(k) * (NB * 32) + b * 32 + lane);
              s4.x += q.x;
              s4.y += q.y;
              s4.z += q.z;
              s4.w += q.w;
            }
            v[b] = s4;
          }
          if (lane == 0) p.tile_ctr[tile] = 0u;  // ready for the next launch that uses this workspace
        }
      }
      if (finalize) {
        // fragment block b = j * NT + nt; this lane holds rows (g, g+8) of row tile j for tokens 8 nt + 2t, +1
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int j = b / NT, nt = b - j * NT;
          const float vals[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int row = ti.row0 + j * 16 + g + ((c & 2) ? 8 : 0);
            const int tok = nt * 8 + 2 * t + (c & 1);
            if (row < mb.OC && tok < p.M) {
              float o = vals[c];
              if (mb.bias) o += __half2float(mb.bias[row]);
              const size_t idx = static_cast<size_t>(tok) * mb.out_stride + row;
              if (p.out_fp32) {
                static_cast<float*>(mb.out)[idx] = o;
              } else {
                const __half h = __float2half_rn(o);
                if (push_world == 0) static_cast<__half*>(mb.out)[idx] = h;
                // pushing: one 8-byte store per rank, {value, epoch} (out_stride == OC, so idx is the dense index);
                // the output itself is written by the CTAs that add up the ranks' words at the end of the launch
#pragma unroll 1
                for (int r = 0; r < push_world; ++r) p.push_slot[r][idx] = make_uint2(__half_as_ushort(h), push_e);
              }
            }
          }
        }
      }
    }
    if (lane == 0) trace_event(p, 9);
    asm volatile("cp.async.wait_all;" ::: "memory");  // nothing of this warp is in flight when the CTA retires
  } else {
    // ================================================================ consumer warps
    const int g = lane >> 2, t = lane & 3;
    bool dep_wait_pending = true;  // x (and a loaded r) come from earlier kernels of the stream
    uint32_t r_epoch = 0u;         // epoch of the words that carry r of this launch (set at the first L epilogue)
    {
      // Launch parameters live in constant memory, and the first touch of each of their cache lines is a miss of a few
      // hundred cycles: read what the staging and the first tile need NOW, while this CTA waits for the previous kernel
      // anyway, instead of one miss after another on the path from "x is ready" to the first MMA.
      const int t0 = tile_at(0);
      const TileInfo tf = tile_info(p, t0 < p.n_tiles ? t0 : 0, slice, r_mode);
      const MemberDev& m0 = p.mem[tf.mi];
      asm volatile("" ::"r"(m0.OC), "r"(m0.out_stride), "f"(m0.alpha), "l"(m0.bias), "l"(m0.out), "l"(m0.L), "r"(p.M),
                   "r"(p.xs_stride), "r"(p.rank), "r"(r_mode), "l"(p.x), "r"(p.x_stride), "r"(p.IC), "r"(p.x_vec_ok),
                   "r"(SK), "r"(p.out_fp32), "r"(push_world), "l"(norm_w));
    }
    if (norm_w != nullptr) {     // the row statistics come first: both the R units and the staging need them
      dep_wait(dep_wait_pending);
      norm_stats(p, red, s_rstd);
    }
    // R units of this CTA (first unit, stride; none if ru0 < 0).  The grid is persistent - never larger than what is
    // resident at once - so every unit's owner is running while the other CTAs wait (bounded) for r before their first
    // L epilogue.  R loads go out before the dependency wait; x is staged only afterwards, for the row tiles the CTA
    // picks up later.  With K slices and more units than R CTAs, an R CTA runs ONE unit and the CTAs of the slices
    // that do not apply the correction (all but slice 0) run the others before their tiles: every unit is then done
    // one round after x is ready, instead of several rounds on the few R CTAs while slice 0 waits for r.  Without
    // dedicated CTAs every CTA takes its share (dealt from the last CTA down) before its tiles.
    int ru0 = -1, rstride = 1;
    if (r_only) {
      ru0 = bid - n_main;
      rstride = (SK > 1 && p.n_r_units > p.n_r_ctas) ? (1 << 30) : p.n_r_ctas;
    } else if (r_mode == 1 && p.n_r_ctas > 0 && SK > 1 && slice != 0 && p.n_r_units > p.n_r_ctas) {
      ru0 = p.n_r_ctas + (bid / SK) * (SK - 1) + slice - 1;
      rstride = (n_main / SK) * (SK - 1);
    } else if (r_mode == 1 && p.n_r_ctas == 0) {
      ru0 = static_cast<int>(gridDim.x) - 1 - bid;
      rstride = static_cast<int>(gridDim.x);
    }
    if (r_mode == 1 && ru0 >= 0)
      r_units<NT>(p, ru0, rstride, red, fin, dep_wait_pending, &s_eword, epoch_bar_u32, cx, s_rstd, norm_w != nullptr, closes_epoch);
    if (threadIdx.x == 0 && r_only) trace_event(p, 6);
    dep_wait(dep_wait_pending);
    if (push_world > 0) push_e = *p.push_epoch + 1u;
    if (threadIdx.x == 0) trace_event(p, 2);
    // per warp: no CTA-wide barrier needed.  A CTA without row tiles (an R CTA of a launch with few tiles) stages
    // nothing and retires: the kernel is complete when its LAST CTA is.
    if (tile_at(0) < p.n_tiles) stage_x(p, g0, ng, xs, xsum, 8 * NT, s_rstd, norm_w != nullptr);
    if (threadIdx.x == 0) trace_event(p, 3);

    // per-lane constant shared addresses: weight quad (warp's group, lane's 16 B, lane's row), x chunk, x sums, the
    // converted scale / zero pairs.  A token slot of the MMA that holds no token reads an all-zero row instead (its
    // address does not advance), so that the loads below are unconditional.
    // Weight stage image: row r of the tile at r * 512 B, group w in its 64 B - with the 16-byte chunks of every
    // 128 B XORed by (128-byte line index mod 8) = (r & 1) * 4 + w / 2, as the tensor map's swizzle lays them down.
    // Rows g, g + 8, g + 16, g + 24 share their parity, so the XOR is a per-lane constant.
    const uint32_t ring_lane =
        smem_u32(ring) + g * kRowPitch +
        (p.w_swizzled ? (warp >> 1) * 128 + (((((warp & 1) << 2) | t) ^ (((g & 1) << 2) | (warp >> 1))) << 4)
                      : warp * 64 + t * 16);
    const uint32_t xsum_lane = smem_u32(xsum) + warp * (32 * NT) + t * 8;
    const uint32_t cooked_lane = smem_u32(cooked) + warp * (kTileRows * 8) + g * 8;
    uint32_t x_lane[NT], x_step[NT];
    bool tokv[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      tokv[nt] = (nt * 8 + g) < p.M;
      x_lane[nt] = tokv[nt] ? smem_u32(xs) + (nt * 8 + g) * p.xs_stride + t * 16 + warp * 256 : smem_u32(zero_row) + t * 16;
      x_step[nt] = tokv[nt] ? kChunkGroups * 256u : 0u;
    }

    uint32_t st = 0, ph = 0, rbuf = 0, rph = 0;
    bool ok = true, r_ready = (r_mode != 1), rb_cached = false;
    uint4 rb_keep[NT];  // r fragments of this lane (first L stage): the same for every row tile of the CTA
    for (int k = 0, tile; (tile = tile_at(k)) < p.n_tiles; ++k) {
      const TileInfo ti = tile_info(p, tile, slice, r_mode);
      const MemberDev& mb = p.mem[ti.mi];
      const uint32_t cslot = static_cast<uint32_t>(k % kCookedDepth), cph = static_cast<uint32_t>(k / kCookedDepth) & 1u;
      ok = ok && mbar_wait_u32(cfull_u32 + cslot * 8, cph, cx);

      float acc[NB][4];
#pragma unroll
      for (int b = 0; b < NB; ++b) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f;

      // Codes go to the tensor cores as fp16 SUBNORMALS: (w & 0x000F000F) is half2(n0, n4) * 2^-24 and
      // (w & 0x00F000F0) is half2(n1, n5) * 2^-20, exactly, with no conversion arithmetic at all; the matching
      // activations were staged divided by 16, so every product carries the factor 2^-24, which goes into the
      // group's scale.  The zero-point leaves the inner loop too:
      //   sum_k (n_k - z) x_k = sum_k n_k x_k - z * sum_k x_k,   with sum_k x_k staged per (group, token).
      uint32_t xa[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) xa[nt] = x_lane[nt];
      uint32_t ck = cooked_lane + cslot * cooked_bytes, xsu = xsum_lane;
      for (int c = 0; c < n_chunks; ++c) {
        ok = ok && mbar_wait_u32(full_u32 + st * 8, ph, cx);
        if (threadIdx.x == 0 && k == 0 && c == 0) trace_event(p, 4);
        if (ok && c * kChunkGroups + warp < ng && !(tuning_bits(p) & 1)) {
          const uint32_t wbase = ring_lane + st * kStageBytes;
          uint4 W[RT][2];
          static_assert(RT == 2, "row-tile offsets below are written out for two row tiles");
          W[0][0] = lds128_at<0>(wbase);
          W[0][1] = lds128_at<8 * kRowPitch>(wbase);
          W[1][0] = lds128_at<16 * kRowPitch>(wbase);
          W[1][1] = lds128_at<24 * kRowPitch>(wbase);
          float ag[RT][NT][4];
#pragma unroll
          for (int j = 0; j < RT; ++j)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) ag[j][nt][0] = ag[j][nt][1] = ag[j][nt][2] = ag[j][nt][3] = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            constexpr uint32_t MLO = 0x000F000Fu, MHI = 0x00F000F0u;
            uint4 xb[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
              xb[nt] = (i == 0) ? lds128_at<0>(xa[nt]) : (i == 1) ? lds128_at<64>(xa[nt]) : (i == 2) ? lds128_at<128>(xa[nt])
                                                                                                     : lds128_at<192>(xa[nt]);
#pragma unroll
            for (int j = 0; j < RT; ++j) {
              const uint32_t a = (i == 0) ? W[j][0].x : (i == 1) ? W[j][0].y : (i == 2) ? W[j][0].z : W[j][0].w;
              const uint32_t b = (i == 0) ? W[j][1].x : (i == 1) ? W[j][1].y : (i == 2) ? W[j][1].z : W[j][1].w;
              const uint32_t a8 = a >> 8, b8 = b >> 8;
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                mma16816(ag[j][nt], a & MLO, b & MLO, a & MHI, b & MHI, xb[nt].x, xb[nt].y);
                mma16816(ag[j][nt], a8 & MLO, b8 & MLO, a8 & MHI, b8 & MHI, xb[nt].z, xb[nt].w);
              }
            }
          }
          // group epilogue: rows g, g+8 (row tile 0), g+16, g+24 (row tile 1) of this warp's group
#pragma unroll
          for (int j = 0; j < RT; ++j) {
            // {s * 2^24, -s * z} of rows g, g + 8 of row tile j
            const float2 pA = (j == 0) ? lds_f2_at<0>(ck) : lds_f2_at<128>(ck);
            const float2 pB = (j == 0) ? lds_f2_at<64>(ck) : lds_f2_at<192>(ck);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const float2 xs2 = lds_f2(xsu + nt * 32);
              float* a4 = acc[j * NT + nt];
              a4[0] = fmaf(pA.x, ag[j][nt][0], fmaf(pA.y, xs2.x, a4[0]));
              a4[1] = fmaf(pA.x, ag[j][nt][1], fmaf(pA.y, xs2.y, a4[1]));
              a4[2] = fmaf(pB.x, ag[j][nt][2], fmaf(pB.y, xs2.x, a4[2]));
              a4[3] = fmaf(pB.x, ag[j][nt][3], fmaf(pB.y, xs2.y, a4[3]));
            }
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xa[nt] += x_step[nt];
        ck += kChunkGroups * (kTileRows * 8);
        xsu += kChunkGroups * (32 * NT);
        __syncwarp();
        if (lane == 0) mbar_arrive_u32(empty_u32 + st * 8);
        if (++st == static_cast<uint32_t>(S)) {
          st = 0;
          ph ^= 1;
        }
      }

      if (threadIdx.x == 0 && k == 0) trace_event(p, 5);
      if (ti.corr) {
        float al[NB][4];
#pragma unroll
        for (int b = 0; b < NB; ++b) al[b][0] = al[b][1] = al[b][2] = al[b][3] = 0.f;
        if (!r_ready && r_mode == 1) {   // the registration's round trip is long over
          ok = ok && mbar_wait_u32(epoch_bar_u32, 0, cx);
          r_epoch = launch_epoch(*static_cast<volatile uint32_t*>(&s_eword));
        }
        for (int l = 0; l < n_lstages; ++l) {
          ok = ok && mbar_wait_u32(full_u32 + st * 8, ph, cx);
          if (threadIdx.x == 0 && k == 0 && l == 0) trace_event(p, 11);
          const int cols = min(256, p.rank - 256 * l);
          const int k = 32 * warp + 8 * t;  // column inside this L stage
          if (ok && 32 * warp < cols) {  // warp-uniform: every lane of the warp takes part in the MMAs below
            const bool kin = k < cols;     // lanes past the last column of a narrow factor feed zeros
            const uint32_t lpitch = static_cast<uint32_t>(p.l_cols) * 2u;  // dense rows of the L box
            const uint32_t lbase = smem_u32(ring) + st * kStageBytes + g * lpitch + k * 2;
            uint4 rb[NT];
            if (l == 0 && rb_cached) {
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) rb[nt] = rb_keep[nt];
            } else {
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                if (!(kin && tokv[nt])) {
                  rb[nt] = make_uint4(0, 0, 0, 0);
                } else if (r_mode != 1) {
                  rb[nt] = ldg_cg_v4(p.r_buf + static_cast<size_t>(nt * 8 + g) * p.rank + 256 * l + k);
                } else {
                  rb[nt] = r_frag_poll(p, nt * 8 + g, 256 * l + k, r_epoch, &s_abort);
                }
              }
              __syncwarp();   // lanes may have polled different numbers of times
              if (threadIdx.x == 0 && !r_ready) trace_event(p, 7);
              r_ready = true;
              if (l == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) rb_keep[nt] = rb[nt];
                rb_cached = true;
              }
            }
#pragma unroll
            for (int j = 0; j < RT; ++j) {
              const uint4 la = kin ? lds128(lbase + (j * 16) * lpitch) : make_uint4(0, 0, 0, 0);
              const uint4 lb = kin ? lds128(lbase + (j * 16 + 8) * lpitch) : make_uint4(0, 0, 0, 0);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                mma16816(al[j * NT + nt], la.x, lb.x, la.y, lb.y, rb[nt].x, rb[nt].y);
                mma16816(al[j * NT + nt], la.z, lb.z, la.w, lb.w, rb[nt].z, rb[nt].w);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive_u32(empty_u32 + st * 8);
          if (++st == static_cast<uint32_t>(S)) {
            st = 0;
            ph ^= 1;
          }
        }
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[b][c] = fmaf(mb.alpha, al[b][c], acc[b][c]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_u32(cempty_u32 + cslot * 8);   // the aux warp may convert the tile after next into this slot

      // park the partial sums
      ok = ok && mbar_wait_u32(rempty_u32, rph ^ 1, cx);   // the aux warp has drained the previous tile's sums
      {
        float4* red4 = reinterpret_cast<float4*>(red);
#pragma unroll
        for (int b = 0; b < NB; ++b)
          red4[(warp * NB + b) * 32 + lane] = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
      }
      if (SK == 1 && tile_at(k + 1) >= p.n_tiles) {
        // This CTA's last tile (K not sliced): nothing is left to overlap with, so the 256 consumer threads add the
        // eight partial sums themselves - one output element each per fragment block - instead of handing the
        // tile to the single aux warp.
        consumer_sync();
        const float* redb = red;
        for (int e = threadIdx.x; e < NB * 128; e += kConsumerThreads) {
          const int b = e >> 7, ln = (e & 127) >> 2, cc = e & 3;
          const int j = b / NT, nt = b - j * NT;
          const int row = ti.row0 + j * 16 + (ln >> 2) + ((cc & 2) ? 8 : 0);
          const int tok = nt * 8 + (ln & 3) * 2 + (cc & 1);
          if (row < mb.OC && tok < p.M) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) o += redb[((w * NB + b) * 32 + ln) * 4 + cc];
            if (mb.bias) o += __half2float(mb.bias[row]);
            const size_t idx = static_cast<size_t>(tok) * mb.out_stride + row;
            if (p.out_fp32) {
              static_cast<float*>(mb.out)[idx] = o;
            } else {
              const __half h = __float2half_rn(o);
              if (push_world == 0) static_cast<__half*>(mb.out)[idx] = h;
#pragma unroll 1
              for (int r = 0; r < push_world; ++r) p.push_slot[r][idx] = make_uint2(__half_as_ushort(h), push_e);
            }
          }
        }
        break;
      }
      // ... and hand them to the aux warp, then move on to the next tile
      if (rbuf == 0)
        asm volatile("bar.arrive 2, %0;" ::"n"(kConsumerThreads + 32) : "memory");
      else
        asm volatile("bar.arrive 3, %0;" ::"n"(kConsumerThreads + 32) : "memory");
      rbuf ^= 1;
      rph ^= 1;
      if (threadIdx.x == 0 && k == 0) trace_event(p, 8);
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) trace_event(p, 10);
  if (r_mode == 1 && closes_epoch && threadIdx.x == 0) advance_epoch(p, s_eword);
  if (push_world > 0) {
    // The all-reduce completes inside the launch: CTAs take a ticket when their tiles are stored, and the last few
    // each poll a share of the output's words - every rank's, this one's included - in this rank's buffer until they
    // carry the call's epoch (bounded), add the ranks' values in rank order (fp32, the same order everywhere, so every
    // rank holds the same bits) and write the sum.  All words of an element are requested before the first is tested.
    __shared__ uint32_t s_ticket, s_epoch;
    if (threadIdx.x == 0) {
      s_ticket = atomicAdd(p.ws_head + WS_EXIT, 1u);
      s_epoch = push_e;
    }
    __syncthreads();
    const int ticket = static_cast<int>(s_ticket);
    const uint32_t e = s_epoch;
    const int nfin = min(kPushFinishers, static_cast<int>(gridDim.x)), first = static_cast<int>(gridDim.x) - nfin;
    if (ticket >= first) {
      const int n = p.M * p.mem[0].OC;
      __half* out = static_cast<__half*>(p.mem[0].out);
      for (int i = (ticket - first) * kGemvThreads + static_cast<int>(threadIdx.x); i < n; i += nfin * kGemvThreads) {
        uint2 w[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < push_world) w[r] = ld_volatile_v2(p.push_local + static_cast<size_t>(r) * p.push_max_n + i);
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < push_world) {
            unsigned spins = 0;
            while (w[r].y != e) {
              if (++spins > p.push_spin) {
                atomicExch(p.ws_head + WS_STATUS, 4u);
                break;
              }
              w[r] = ld_volatile_v2(p.push_local + static_cast<size_t>(r) * p.push_max_n + i);
            }
            acc += __half2float(__ushort_as_half(static_cast<unsigned short>(w[r].x)));
          }
        out[i] = __float2half_rn(acc);
      }
    }
    if (ticket == static_cast<int>(gridDim.x) - 1 && threadIdx.x == 0) {
      // every CTA has taken its ticket, so every CTA has read the site's call counter: advance it for the next call
      p.ws_head[WS_EXIT] = 0u;
      *p.push_epoch = e;
      __threadfence();
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
  return gemv_smem_layout_bytes(p.stages, p.meta_gp, p.meta_gw, p.gps, NT, p.M, p.xs_stride);
}

template <int FEAT>
static cudaError_t launch_feat(const GemvParams& p, const TensorMaps& tm, int grid, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<1, FEAT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  static const bool use_pdl = [] {
    const char* v = std::getenv("GLOWQ_PDL");
    return !(v && v[0] == '0');
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = gemv_smem_bytes(p, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<1, FEAT>, p, tm);
}

cudaError_t launch_gemv_stream(const GemvParams& p, const TensorMaps& tm, int NT, int grid, cudaStream_t stream) {
  // Launches carry at most 8 tokens (one token block): wider instantiations measured 3-13x slower per token than
  // repeated 8-token launches, so the host splits larger batches or takes the tensor-core GEMM.
  if (NT != 1) return cudaErrorInvalidValue;
  // K slices stay a run-time property of every instantiation: a decode step mixes sliced (down_proj) and unsliced
  // launches, and alternating between two kernels costs more than the slicing code does (the instruction cache stays
  // warm across back-to-back launches of ONE function: 2.44 against 2.53 ms per Llama-2-13B token step).
  // ... and once a process has used one of the extras (a tensor-parallel rank pushes from every other launch), all its
  // corrected launches take the instantiation with it, for the same reason.
  static std::atomic<int> extras_seen{0};
  static const bool sticky = [] {
    const char* v = std::getenv("GLOWQ_GEMV_STICKY_EXTRAS");
    return !(v && v[0] == '0');
  }();
  int extras = (p.push_world > 0 ? kFeatPush : 0) | (p.norm_w != nullptr ? kFeatNorm : 0);
  if (extras) extras_seen.fetch_or(extras, std::memory_order_relaxed);
  if (sticky && p.r_mode != 0) extras |= extras_seen.load(std::memory_order_relaxed);
  const int feat = (p.r_mode != 0 ? kFeatCorr : 0) | kFeatSliced | extras;
  switch (feat) {
    case kFeatSliced: return launch_feat<kFeatSliced>(p, tm, grid, stream);
    case kFeatSliced | kFeatCorr: return launch_feat<kFeatSliced | kFeatCorr>(p, tm, grid, stream);
    case kFeatSliced | kFeatPush: return launch_feat<kFeatSliced | kFeatPush>(p, tm, grid, stream);
    case kFeatSliced | kFeatPush | kFeatCorr: return launch_feat<kFeatSliced | kFeatPush | kFeatCorr>(p, tm, grid, stream);
    case kFeatSliced | kFeatNorm: return launch_feat<kFeatSliced | kFeatNorm>(p, tm, grid, stream);
    case kFeatSliced | kFeatNorm | kFeatCorr: return launch_feat<kFeatSliced | kFeatNorm | kFeatCorr>(p, tm, grid, stream);
    case kFeatSliced | kFeatPush | kFeatNorm: return launch_feat<kFeatSliced | kFeatPush | kFeatNorm>(p, tm, grid, stream);
    default: return launch_feat<kFeatSliced | kFeatPush | kFeatNorm | kFeatCorr>(p, tm, grid, stream);
  }
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
