// One-shot all-reduce (sum) of a small fp16 vector over NVLink peer memory, for the row-parallel linears of a
// tensor-parallel decode step ([M, hidden] fp16: 6 KB at M = 1).  Every rank
//   1. stores its partial vector into slot [site][rank] of EVERY rank's staging buffer (plain peer stores),
//   2. releases a per-(site, source) epoch flag on every rank (st.release.sys),
//   3. waits - bounded - until all sources' flags on its own memory carry this call's epoch (ld.acquire.sys),
//   4. adds the `world` slots of its own buffer in rank order (fp32), and writes the fp16 sum in place.
// Sums are bit-identical on all ranks (same order).  No NCCL call, so a whole token step including its collectives
// can be replayed from one CUDA graph; no peer LOADS, no multicast, no multimem.  The ranks' kernels run on
// different GPUs; a rank that never arrives makes the others record a status word and return.
#include <cstdlib>

#include "../../include/glowq_w4a16.h"
#include "common.cuh"
#include "params.h"

namespace glowq {
namespace {

constexpr int kArThreads = 512;
constexpr unsigned kArSpinLimit = 1u << 22;

// Polls a rank makes on a peer's flag before it gives up (status 4).  GLOWQ_AR_SPIN_LIMIT shortens it, for tests of
// the expiry path; read once.
unsigned ar_spin_limit() {
  static const unsigned v = [] {
    const char* e = std::getenv("GLOWQ_AR_SPIN_LIMIT");
    const long n = (e && *e) ? std::atol(e) : 0;
    return n > 0 ? static_cast<unsigned>(n) : kArSpinLimit;
  }();
  return v;
}

}  // namespace
unsigned allreduce_spin_limit() { return ar_spin_limit(); }
namespace {

struct ArParams {
  const uint2* ll_local;                 // finish only: this rank's word buffer [sites][world][max_n] {value, epoch}
  unsigned char* buf[GLOWQ_MAX_RANKS];   // staging buffer of every rank: [sites][world][max_n] fp16
  uint32_t* flag[GLOWQ_MAX_RANKS];       // epoch flags of every rank: [sites][world]
  uint32_t* epoch;                       // local: [sites] calls made so far per site
  uint32_t* status;                      // local status word
  __half* inout;                         // local vector, n halves (n % 8 == 0, 16-byte aligned)
  int world, rank, site, n, max_n;
  unsigned spin_limit;
  int finish_only;                       // the partial results were pushed by the producing launch: wait and sum only
};

__global__ void __launch_bounds__(kArThreads) allreduce_push_kernel(const __grid_constant__ ArParams p) {
  __shared__ uint32_t s_epoch;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // the partial sums come from the previous kernel
  if (threadIdx.x == 0) {
    // finish only: the pushing launch (complete by now) advanced the site's epoch and released the flags itself
    s_epoch = p.finish_only ? p.epoch[p.site] : p.epoch[p.site] + 1;
    if (!p.finish_only) p.epoch[p.site] = s_epoch;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  const int nv = p.n >> 3;  // 16-byte vectors
  if (!p.finish_only) {
    const size_t slot = (static_cast<size_t>(p.site) * p.world + p.rank) * p.max_n * sizeof(__half);
    const uint4* src = reinterpret_cast<const uint4*>(p.inout);
    for (int i = threadIdx.x; i < nv; i += kArThreads) {
      const uint4 v = src[i];
      for (int r = 0; r < p.world; ++r) reinterpret_cast<uint4*>(p.buf[r] + slot)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.world) {
      uint32_t* f = p.flag[threadIdx.x] + p.site * p.world + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
    }
  }
  if (p.finish_only) {
    // The producing launches stored every element as one 8-byte word {fp16 value, epoch}: poll each word until it
    // carries this call's epoch (bounded), add the ranks' values in rank order.
    const uint2* mine = p.ll_local + static_cast<size_t>(p.site) * p.world * p.max_n;
    __half* dst = p.inout;
    for (int i = threadIdx.x; i < p.n; i += kArThreads) {
      uint2 w[GLOWQ_MAX_RANKS];   // all ranks' words are requested before the first one is tested
#pragma unroll
      for (int r = 0; r < GLOWQ_MAX_RANKS; ++r)
        if (r < p.world) w[r] = ld_volatile_v2(mine + static_cast<size_t>(r) * p.max_n + i);
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < GLOWQ_MAX_RANKS; ++r)
        if (r < p.world) {
          unsigned spins = 0;
          while (w[r].y != e) {
            if (++spins > p.spin_limit) {
              atomicExch(p.status, 4u);
              break;
            }
            w[r] = ld_volatile_v2(mine + static_cast<size_t>(r) * p.max_n + i);
          }
          acc += __half2float(__ushort_as_half(static_cast<unsigned short>(w[r].x)));
        }
      dst[i] = __float2half_rn(acc);
    }
    return;
  }
  if (threadIdx.x < p.world) {
    const uint32_t* f = p.flag[p.rank] + p.site * p.world + threadIdx.x;
    unsigned spins = 0;
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int32_t>(v - e) >= 0) break;
      if (++spins > p.spin_limit) {
        atomicExch(p.status, 4u);
        break;
      }
    }
  }
  __syncthreads();
  const unsigned char* mine = p.buf[p.rank] + static_cast<size_t>(p.site) * p.world * p.max_n * sizeof(__half);
  uint4* dst = reinterpret_cast<uint4*>(p.inout);
  for (int i = threadIdx.x; i < nv; i += kArThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.world; ++r) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(mine + static_cast<size_t>(r) * p.max_n * sizeof(__half)) + i);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    __half2 t;
    t = __floats2half2_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2half2_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2half2_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2half2_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
    dst[i] = o;
  }
}

}  // namespace
}  // namespace glowq

namespace {
int launch_allreduce(const glowq_w4a16_peers_t* peers, void* inout, int n, int site, void* stream, int finish_only) {
  using namespace glowq;
  if (!peers || !inout || n <= 0 || site < 0) return GLOWQ_ERR_BAD_ARGUMENT;
  if (peers->world < 1 || peers->world > GLOWQ_MAX_RANKS || peers->rank < 0 || peers->rank >= peers->world)
    return GLOWQ_ERR_BAD_ARGUMENT;
  if ((n & 7) || (reinterpret_cast<uintptr_t>(inout) & 15) || n > peers->max_n || site >= peers->sites)
    return GLOWQ_ERR_UNSUPPORTED_SHAPE;
  ArParams p{};
  if (finish_only) {
    if (!peers->ll_buf[peers->rank]) return GLOWQ_ERR_BAD_ARGUMENT;
    p.ll_local = static_cast<const uint2*>(peers->ll_buf[peers->rank]);
  }
  for (int r = 0; r < peers->world; ++r) {
    if (!peers->buf[r] || !peers->flag[r]) return GLOWQ_ERR_BAD_ARGUMENT;
    p.buf[r] = static_cast<unsigned char*>(peers->buf[r]);
    p.flag[r] = static_cast<uint32_t*>(peers->flag[r]);
  }
  p.epoch = static_cast<uint32_t*>(peers->epoch);
  p.status = static_cast<uint32_t*>(peers->status);
  if (!p.epoch || !p.status) return GLOWQ_ERR_BAD_ARGUMENT;
  p.inout = static_cast<__half*>(inout);
  p.world = peers->world;
  p.rank = peers->rank;
  p.site = site;
  p.n = n;
  p.max_n = peers->max_n;
  p.spin_limit = ar_spin_limit();
  p.finish_only = finish_only;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, allreduce_push_kernel, p);
  return e == cudaSuccess ? GLOWQ_OK : GLOWQ_ERR_CUDA;
}
}  // namespace

extern "C" int glowq_w4a16_allreduce_f16(const glowq_w4a16_peers_t* peers, void* inout, int n, int site, void* stream) {
  return launch_allreduce(peers, inout, n, site, stream, 0);
}

extern "C" int glowq_w4a16_allreduce_finish_f16(const glowq_w4a16_peers_t* peers, void* out, int n, int site, void* stream) {
  return launch_allreduce(peers, out, n, site, stream, 1);
}
