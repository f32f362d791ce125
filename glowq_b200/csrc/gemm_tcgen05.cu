// Tensor-core corrected W4A16 GEMM for prefill token counts (sm_100a: tcgen05.mma, TMEM accumulators, TMA).
//
//   Y[M, OC] = X[M, IC] . dequant(Q)^T  +  alpha * r[M, rank] . L[OC, rank]^T  (+ bias),     r = X . R^T
//
// One CTA computes a block of Y (256 tokens x 256 columns as four 128 x 128 fp32 accumulators in tensor memory, or
// 128-token / 128-column variants; 256 x 128 with a separate correction accumulator when alpha != 1); a CTA PAIR
// (cluster of two, cta_group::2 MMAs) computes 256 tokens x 512 columns.  K runs in steps of 64 through two
// shared-memory rings: operand stages (activation tiles + fp16 weight tiles, 128-byte swizzle) and, many steps ahead
// of them, small packed stages (the int4 tiles as they lie in HBM).
//   warp 0      operand producer (one thread): TMA of the activation tiles; in the correction phase also the L tile
//               (fp16, swizzled, no dequantisation) - the correction is simply more K steps of the same pipeline.
//   warp 2      packed-weight producer (one thread): TMA of the 128 NN x 32 B int4 tile of each step.
//   warps 3..   dequantise, in kPassGroups teams that take alternate steps: a thread turns half-rows of the packed tile
//               into 32 fp16 values half_rn((code - zero) * scale) - the same exact-integer unpack + one HMUL2 as the
//               stand-alone dequant kernel, so the shared-memory tile is bit-identical to the reference's dequantised
//               weight - and stores them into the K-major, 128-byte-swizzled B tile of the operand stage; afterwards
//               these warps are the epilogue (TMEM -> registers -> bias / alpha -> global).
//   warp 1      allocates tensor memory and issues tcgen05.mma from one thread (N = 256 per instruction where two
//               weight tiles are stacked), then tcgen05.commit to release the stage.  In a pair only CTA 0 issues;
//               the peer's warp 1 relays "my operand copies have landed" to CTA 0's barrier.
// The dequantised weight never goes to HBM (the reference writes and re-reads a full fp16 copy per call).
// The same kernel with an fp16 B operand by TMA (no dequant work) computes r = X . R^T, K-sliced over gridDim.z
// into fp32 slots that slot_sum_kernel adds up in slice order.
// Every mbarrier wait is bounded; on expiry a status word is set and the CTA drains and frees its tensor memory.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../../include/glowq_w4a16.h"
#include "common.cuh"
#include "params.h"

namespace glowq {

// r = x . R^T for up to 128 tokens as one small launch (r_product.cu); above, the K-sliced GEMM of this file.  Measured
// group calls (microseconds, this path / GEMM + slot sum): Llama-2-13B q/k/v 40.2 / 45.1 at 32 tokens, 51.8 / 56.6 at
// 128, 68.4 / 70.8 at 256; Qwen3-14B down_proj (rank 256, K = 17408) 63.8 / 62.5 at 128 but 111.7 / 96.4 at 256, where
// every 64-token block stages the R tiles again.
constexpr int kRProductMaxM = 128;
size_t r_product_slot_bytes(int M, int IC, int rank);
cudaError_t launch_r_product(const __half* x, const __half* R, __half* r_buf, float* slots, uint32_t* ctr, int M, int IC,
                             int rank, int x_stride, int R_stride, cudaStream_t stream);
int tensor_map_2d_ex(CUtensorMap* out, CUtensorMapDataType dtype, const void* ptr, uint64_t dim0, uint64_t dim1,
                     uint64_t stride_bytes, uint32_t box0, uint32_t box1, int swizzle128);

namespace {

#ifndef GLOWQ_GEMM_PASS_GROUPS
#define GLOWQ_GEMM_PASS_GROUPS 2
#endif
#ifndef GLOWQ_GEMM_PAIR_PASS_GROUPS
#define GLOWQ_GEMM_PAIR_PASS_GROUPS 2
#endif
constexpr int BM = 128;   // tokens per accumulator (MMA M)
constexpr int MT = 2;     // accumulators per CTA
constexpr int BN = 128;   // output columns per CTA (MMA N)
constexpr int BK = 64;    // K per stage: 128 bytes of fp16 = one swizzle row
constexpr int kABytes = BM * BK * 2;        // 16 KB
constexpr int kBBytes = BN * BK * 2;        // 16 KB per 128 output columns
constexpr int kPBytes = BN * (BK / 8) * 4;  // 4 KB packed per 128 output columns
// NN = 128-column B tiles per CTA.  NN = 2 halves the activation traffic from L2 per flop (the x tile is read once
// per 256 output columns) and needs all 512 TMEM columns for its four accumulators, so the correction must
// accumulate in place (alpha == 1); NN = 1 keeps a separate correction accumulator for any alpha.
template <int NN> struct Cfg {
  static constexpr int kMaxStages = 8, kMaxPStages = 16;
  // dequant (then epilogue) warps: one thread per half-row (32 columns) of the step's 128 NN-row packed tile.
  static constexpr int kDequantWarps = 8 * NN;
  static constexpr int kCtrlWarps = 3;  // operand producer, MMA issuer, packed-weight producer
  static constexpr int kThreads = 32 * (kCtrlWarps + kDequantWarps);
  // The dequant warps work in kPassGroups teams; team g converts the packed tiles of steps g, g + kPassGroups, ...
  // (each thread then covers kPassGroups half-rows of a step), so that the fixed latency of a pass - barrier wake-up,
  // shared-memory round trip, proxy fence - overlaps between consecutive steps instead of adding up.
  static constexpr int kPassGroups = GLOWQ_GEMM_PASS_GROUPS;
  static constexpr int kPairPassGroups = GLOWQ_GEMM_PAIR_PASS_GROUPS;  // CTA pairs (4 operand and 4 packed stages)
  // An operand stage holds mt activation tiles and NN weight tiles (fp16, swizzled); a packed stage NN int4 tiles.
  // The operand ring is as deep as 227 KB allow after the packed ring: 3 stages for the 256 x 256 tile, 4 for
  // 128 x 256 and 256 x 128, 6 for 128 x 128.
  static constexpr int stage_bytes(int mt) { return mt * kABytes + NN * kBBytes; }
  static constexpr int kPStageBytes = NN * kPBytes;
  static constexpr int kPStages = NN == 2 ? 4 : 8;
  static constexpr int kSmemMax = 227 * 1024 - 256;  // the kernel also has a few bytes of static shared memory
  static int stages(int mt) { return std::min(kMaxStages, (kSmemMax - 2048 - kPStages * kPStageBytes) / stage_bytes(mt)); }
  // 1 KB alignment slack + 1 KB of barriers + the rings
  static int smem(int mt) { return 2048 + stages(mt) * stage_bytes(mt) + kPStages * kPStageBytes; }
};
constexpr uint32_t kGemmSpin = 1u << 18;
constexpr uint32_t kTmemCols = 512;

struct GemmMember {   // one linear of the group; its column tiles are blockIdx.x in [tile_begin, next tile_begin)
  const __half* scales;
  const int32_t* qzeros;
  const __half* bias;
  void* out;
  int OC, nk2, sstride, zstride, out_stride, lr_separate, out_vec_ok, tile_begin;
  float alpha;
};
struct GemmParams {
  uint32_t* status;
  int M, nk1, w4, out_fp32, n_members;
  int mt;  // 128-token accumulators per CTA actually used (1 or 2): 1 spreads a narrow product over more CTAs
  int stages, pstages;  // ring depths (operands, packed weights) for this mt
  // split-K (only the narrow r = X . R^T product uses it): gridDim.z CTAs share a tile's K steps, each writes its fp32
  // partial tile to its own slot; slot_sum_kernel then adds the slots in slice order
  int ksplit;
  // swap: up to 128 tokens.  The dequantised weight tile becomes the M side of the MMA (A operand, 128 output columns
  // per accumulator) and the activation tile its N side (nt = 32, 64 or 128 token rows, B operand): the activation
  // tile written and re-read per K step shrinks from 128 rows to nt, which is what bounds small token counts.
  int swap, nt;
  int debug;         // used by the clock trace of -DGLOWQ_GEMM_TRACE builds only (bit 2048, bit 4096 = trace CTA 1)
  // Work items (blockIdx.x, single-CTA kernels): tiles [0, full_tiles) are computed whole; each of the n_tail tiles
  // after them is cut into ksplit K slices (item = full_tiles + tail index * ksplit + slice).  Tiles are numbered
  // token tile major, column tile minor (n_x column tiles).  full_tiles = 0 slices every tile (few tokens);
  // full_tiles = whole waves slices only the last, partial wave of a large launch.
  int full_tiles, n_tail, n_x;
  float* slots;      // [ksplit][n_tail][NN * mt][slot_rows][128]
  int slot_rows;     // token rows kept per 128 x 128 accumulator in a slot (a multiple of 32, >= the tile's valid tokens)
  GemmMember mem[kMaxMembers];
};
struct alignas(64) GemmMaps {
  CUtensorMap a1, a2;                          // activations: x (phase 1), r (phase 2)
  CUtensorMap b1[kMaxMembers], b2[kMaxMembers];  // per member: packed weight (or fp16 B), L
};

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void g_mbar_init(uint32_t a, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void g_mbar_arrive(uint32_t a) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}
__device__ __forceinline__ void g_mbar_expect_tx(uint32_t a, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool g_mbar_wait(uint32_t a, uint32_t parity, volatile int* abort_flag, uint32_t* status) {
  uint32_t spins = 0;
  for (;;) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(a), "r"(parity)
                 : "memory");
    if (ok) return true;
    if ((++spins & 63u) == 0 && *abort_flag) return false;
    if (spins > kGemmSpin) {
      *abort_flag = 1;
      atomicExch(status, 3u);
      return false;
    }
  }
}
// the same with cluster-scope acquire: the arrivals come from the peer CTA as well
__device__ __forceinline__ bool g_mbar_wait_cluster(uint32_t a, uint32_t parity, volatile int* abort_flag, uint32_t* status) {
  uint32_t spins = 0;
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((++spins & 63u) == 0 && *abort_flag) return false;
    if (spins > kGemmSpin) {
      *abort_flag = 1;
      atomicExch(status, 3u);
      return false;
    }
  }
}
__device__ __forceinline__ void g_tma_2d(uint32_t dst, const CUtensorMap* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// K-major, 128-byte-swizzled operand tile: rows of 128 B, 8-row atoms 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}
template <int N>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  // instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, M = 128, N columns
  constexpr uint32_t kIdesc = (1u << 4) | ((static_cast<uint32_t>(N) >> 3) << 17) | ((BM >> 4) << 24);
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_f16_rt(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
template <int N>
__device__ __forceinline__ void umma_f16_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc) {  // D += A . B
  constexpr uint32_t kIdesc = (1u << 4) | ((static_cast<uint32_t>(N) >> 3) << 17) | ((BM >> 4) << 24);
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(kIdesc)
      : "memory");
}
__device__ __forceinline__ uint64_t mk64(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ bool g_mbar_try_once(uint32_t a, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(a), "r"(parity)
               : "memory");
  return ok != 0;
}
// ---- CTA-pair (cta_group::2) forms: one MMA spans two SMs (256 tokens), each CTA holding its 128 tokens of A and
// half of the B rows; barriers of the peer CTA are reached through shared::cluster addresses.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {  // shared::cta -> shared::cluster of `rank`
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void g_mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
template <int N>
__device__ __forceinline__ void umma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  // instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, M = 256 over the CTA pair, N columns
  constexpr uint32_t kIdesc = (1u << 4) | ((static_cast<uint32_t>(N) >> 3) << 17) | ((256u >> 4) << 24);
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma2_commit(uint32_t cluster_bar) {  // arrives once all MMAs issued so far are done
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// one poll of two barriers with both requests in flight together (a poll takes a few hundred clocks to answer)
__device__ __forceinline__ bool g_mbar_try_both(uint32_t a1, uint32_t parity1, uint32_t a2, uint32_t parity2) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 q, [%3], %4;\n\t"
      "and.pred p, p, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(a1), "r"(parity1), "r"(a2), "r"(parity2)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// PAIR: launched as clusters of two CTAs along x (NN = 2, mt = 1).  The pair computes 256 tokens x 512 columns: CTA r
// holds tokens [128 r, 128 r + 128) and dequantises weight rows [256 r, 256 r + 256) of the tile, i.e. half of the B
// rows of each of the two N = 256 MMAs per K slice - per flop, half the dequantisation and two thirds of the
// shared-memory traffic of the single-CTA 256 x 256 tile.  CTA 0 issues the MMAs; its `bready` barriers count the
// dequant warps of both CTAs, and its commits release the stages of both.
template <int NN, bool PAIR>
__global__ void __launch_bounds__(Cfg<NN>::kThreads, 1)
gemm_w4a16_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ GemmMaps tm) {
  static_assert(!PAIR || NN == 2, "the CTA pair works on two 128-row weight tiles per CTA");
  constexpr int kPG = PAIR ? Cfg<NN>::kPairPassGroups : Cfg<NN>::kPassGroups;
  // let the next kernel of the stream start its prologue and its weight prefetch as SMs free up
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int kStagesG = p.stages, kPStagesG = p.pstages;
  const uint32_t kBOff = p.mt * kABytes;              // B tiles inside an operand stage
  const uint32_t kStageG = kBOff + NN * kBBytes;      // operand stage: mt activation tiles + NN weight tiles
  constexpr uint32_t kPStage = NN * kPBytes;          // packed stage
  extern __shared__ unsigned char smem[];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem_base;
  const uint32_t smem0 = (sm_u32(smem) + 1023u) & ~1023u;  // swizzled operand tiles want 1024-byte alignment
  // barriers live in the first 1 KB: full[8], empty[8], bready[8], pfull[16], pempty[16], accum
  const uint32_t full_b = smem0, empty_b = smem0 + 64, bready_b = smem0 + 128, pfull_b = smem0 + 192,
                 pempty_b = smem0 + 320, accum_b = smem0 + 448;
  const uint32_t ring = smem0 + 1024;
  const uint32_t pring = ring + kStagesG * kStageG;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;   // 0: the CTA that issues the MMAs
  int tile_lin = 0, zslice = 0, ks = 1;   // (single CTA) tile, K slice and slice count of this work item
  if (!PAIR) {
    const int item = static_cast<int>(blockIdx.x);
    if (item < p.full_tiles) {
      tile_lin = item;
    } else {
      const int r = item - p.full_tiles, t = r / p.ksplit;
      tile_lin = p.full_tiles + t;
      zslice = r - t * p.ksplit;
      ks = p.ksplit;
    }
  }
  const int by = PAIR ? static_cast<int>(blockIdx.y) : tile_lin / p.n_x;                        // token tile index
  const int bx = PAIR ? static_cast<int>(blockIdx.x >> 1) : tile_lin - by * p.n_x;              // column tile index
  int mi = 0;
#pragma unroll
  for (int i = 1; i < kMaxMembers; ++i)
    if (i < p.n_members && bx >= p.mem[i].tile_begin) mi = i;
  const GemmMember& mb = p.mem[mi];
  // n0: first weight row this CTA dequantises; m0: its first token
  const int n0 = PAIR ? (bx - mb.tile_begin) * (2 * BN * NN) + static_cast<int>(crank) * (BN * NN) : (bx - mb.tile_begin) * (BN * NN);
  const int m0 = PAIR ? by * (2 * BM) + static_cast<int>(crank) * BM : (p.swap ? by * p.nt : by * (BM * p.mt));
  const int n_mt = (!PAIR && p.mt == 2 && m0 + BM < p.M) ? 2 : 1;
  const int n_nt = PAIR ? 2 : ((NN == 2 && n0 + BN < mb.OC) ? 2 : 1);
  const int nk_all = p.nk1 + mb.nk2;
  const int it0 = ks > 1 ? static_cast<int>(static_cast<long long>(nk_all) * zslice / ks) : 0;
  const int nk = ks > 1 ? static_cast<int>(static_cast<long long>(nk_all) * (zslice + 1) / ks) : nk_all;
  const int nk_packed = p.w4 ? min(nk, p.nk1) : it0;  // steps [it0, nk_packed) dequantise a packed tile

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kStagesG; ++i) {
      g_mbar_init(full_b + 8 * i, 1);
      g_mbar_init(empty_b + 8 * i, 1);
      // pair: the dequant warps of both CTAs, plus the peer's relay thread (its operand copies have landed)
      // single CTA: the dequant warps plus the operand producer, whose copies complete their bytes on this barrier too,
      // so that the MMA thread has ONE barrier to poll per step
      g_mbar_init(bready_b + 8 * i, 2 * Cfg<NN>::kDequantWarps / kPG + 1 - (PAIR ? 0 : Cfg<NN>::kDequantWarps / kPG));
    }
    for (int i = 0; i < kPStagesG; ++i) {
      g_mbar_init(pfull_b + 8 * i, 1);
      g_mbar_init(pempty_b + 8 * i, Cfg<NN>::kDequantWarps / kPG);
    }
    g_mbar_init(accum_b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {  // warp 1 of both CTAs
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_u32(&s_tmem_base)), "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_u32(&s_tmem_base)), "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  // Tuning aid, compiled in with -DGLOWQ_GEMM_TRACE only (debug & 2048): CTA (debug >> 12 & 1, 0, 0) records clock64()
  // per role / event / step at workspace + 4096.
#ifdef GLOWQ_GEMM_TRACE
  unsigned long long* trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(p.status) - WS_STATUS * 4 + 4096);
  const bool tracing = (p.debug & 2048) && blockIdx.x == ((p.debug >> 12) & 1) && blockIdx.y == 0 && lane == 0;
  auto tr = [&](int role, int ev, int step) {
    if (tracing && step < 256) trace[(role * 3 + ev) * 256 + step] = clock64();
  };
#else
  auto tr = [](int, int, int) {};
#endif
  // after a failed wait: give the copies of the last `depth` issues a bounded time to land
  auto drain = [&](uint32_t bars, int depth, int issued) {
    for (int j = (issued > depth ? issued - depth : 0); j < issued; ++j) {
      uint32_t spins = 0, done = 0;
      while (!done && ++spins < kGemmSpin)
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bars + 8 * (j % depth)), "r"((j / depth) & 1)
            : "memory");
    }
  };

  if (warp == 0) {
    // ================================================================ operand producer (one thread: a wait that
    // the whole warp executes costs 32 serialised barrier operations): activation tiles, and the B tile of the
    // steps that need no dequantisation
    if (lane == 0) {
      uint32_t st = 0, ph = 0;
      int issued = 0;
      bool ok = true;
      // activations, r and (for the r product) nothing else of this thread's copies may be read before the earlier
      // kernels of the stream are complete; the packed-weight producer and the dequant warps do not wait
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int it = it0; it < nk; ++it) {
        tr(0, 0, it - it0);
        if (!(ok = g_mbar_wait(empty_b + 8 * st, ph ^ 1, abort_flag, p.status))) break;
        tr(0, 1, it - it0);
        const uint32_t sbase = ring + st * kStageG, bar = (PAIR ? full_b : bready_b) + 8 * st;
        const bool phase1 = it < p.nk1;
        const int kk = phase1 ? it : it - p.nk1;
        const bool packed = it < nk_packed;
        g_mbar_expect_tx(bar, (p.swap ? p.nt * (BK * 2) : n_mt * kABytes) + (packed ? 0 : NN * kBBytes));
        const CUtensorMap* ta = phase1 ? &tm.a1 : &tm.a2;
        g_tma_2d(sbase, ta, kk * BK, m0, bar);
        if (n_mt == 2) g_tma_2d(sbase + kABytes, ta, kk * BK, m0 + BM, bar);
        if (!packed)  // one box of 128 NN rows x 128 B, swizzled: NN consecutive 16 KB operand tiles
          g_tma_2d(sbase + kBOff, phase1 ? &tm.b1[mi] : &tm.b2[mi], kk * BK, n0, bar);
        ++issued;
        if (++st == static_cast<uint32_t>(kStagesG)) {
          st = 0;
          ph ^= 1;
        }
      }
      if (!ok) drain(PAIR ? full_b : bready_b, kStagesG, issued);
    }
    __syncwarp();
  } else if (warp == 2) {
    // ================================================================ packed-weight producer (one thread).  The
    // packed tiles are small, so their ring runs many steps ahead of the operand ring: the DRAM latency of the
    // weight stream is then off the path stage-free -> tile-dequantised -> MMA.
    if (lane == 0) {
      uint32_t sp = 0, pph = 0;
      int issued = 0;
      bool ok = true;
      for (int it = it0; it < nk_packed; ++it) {
        if (!(ok = g_mbar_wait(pempty_b + 8 * sp, pph ^ 1, abort_flag, p.status))) break;
        const uint32_t bar = pfull_b + 8 * sp;
        g_mbar_expect_tx(bar, kPStage);
        g_tma_2d(pring + sp * kPStage, &tm.b1[mi], it * (BK / 8), n0, bar);  // one box of 128 NN rows x 32 B
        ++issued;
        if (++sp == static_cast<uint32_t>(kPStagesG)) {
          sp = 0;
          pph ^= 1;
        }
      }
      if (!ok) drain(pfull_b, kPStagesG, issued);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================================================ MMA issuer (one thread; in a pair, of CTA 0)
    if (lane == 0 && crank == 0) {
      // A single thread runs this loop, so every instruction in it is latency on the critical path: descriptors are
      // one 32-bit add each (the address field, in 16-byte units, never carries out of the low word).
      uint32_t st = 0, ph = 0;
      bool ok = true;
      const uint64_t desc0 = smem_desc_sw128(ring);
      const uint32_t desc_hi = static_cast<uint32_t>(desc0 >> 32);
      uint32_t desc_lo = static_cast<uint32_t>(desc0);
      const uint32_t desc_lo0 = desc_lo;
      const uint32_t stage16 = kStageG >> 4, boff16 = kBOff >> 4;
      const uint32_t peer_empty = PAIR ? map_to_cta(empty_b, 1) : 0u, peer_accum = PAIR ? map_to_cta(accum_b, 1) : 0u;
      for (int it = it0; it < nk; ++it) {
        if (PAIR) {  // `bready`: the dequant warps of both CTAs and the landing of the peer's operand copies
          ok = ok && g_mbar_wait_cluster(bready_b + 8 * st, ph, abort_flag, p.status);
          tr(1, 0, it - it0);
          if (ok && !g_mbar_try_once(full_b + 8 * st, ph)) ok = g_mbar_wait(full_b + 8 * st, ph, abort_flag, p.status);
          tr(1, 1, it - it0);
        } else {
          if (ok && !g_mbar_try_once(bready_b + 8 * st, ph)) ok = g_mbar_wait(bready_b + 8 * st, ph, abort_flag, p.status);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
          const bool phase2 = it >= p.nk1;
          const uint32_t lr_off = (phase2 && mb.lr_separate) ? BN : 0;
          // the first MMA into an accumulator overwrites it: the slice's first step (which may lie in the correction
          // phase when K is sliced), and the first correction step when the correction has an accumulator of its own
          const bool first = (it == it0) || (phase2 && mb.lr_separate && it == p.nk1);
          if (!PAIR && p.swap) {
            // accumulator nn: 128 output columns (TMEM lanes) x nt tokens (TMEM columns nn * nt ..)
            const uint32_t idesc = (1u << 4) | ((static_cast<uint32_t>(p.nt) >> 3) << 17) | ((BM >> 4) << 24);
            const uint32_t lr_cols = (phase2 && mb.lr_separate) ? p.nt : 0;
#pragma unroll
            for (int nn = 0; nn < NN; ++nn) {
              if (nn < n_nt) {
#pragma unroll
                for (int k16 = 0; k16 < BK / 16; ++k16) {
                  const uint64_t wd = mk64(desc_lo + boff16 + nn * (kBBytes >> 4) + k16 * 2, desc_hi);
                  const uint64_t xd = mk64(desc_lo + k16 * 2, desc_hi);
                  umma_f16_rt(tmem_base + nn * p.nt + lr_cols, wd, xd, idesc, (first && k16 == 0) ? 0u : 1u);
                }
              }
            }
          } else if constexpr (PAIR) {
            // accumulator n (TMEM columns 256 n ..): B rows 128 n .. of this CTA and of the peer, 256 columns in all
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
              for (int k16 = 0; k16 < BK / 16; ++k16) {
                const uint64_t ad = mk64(desc_lo + k16 * 2, desc_hi);
                const uint64_t bd = mk64(desc_lo + boff16 + n * (kBBytes >> 4) + k16 * 2, desc_hi);
                umma2_f16<2 * BN>(tmem_base + n * (2 * BN), ad, bd, (first && k16 == 0) ? 0u : 1u);
              }
            }
          } else {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            if (mt < n_mt) {
              // NN = 2: one N = 256 instruction covers both operand tiles (they are consecutive 8-row atoms)
              const uint32_t acc_col = (NN == 1) ? mt * (2 * BN) + lr_off : mt * (NN * BN);
#pragma unroll
              for (int k16 = 0; k16 < BK / 16; ++k16) {
                const uint64_t ad = mk64(desc_lo + (mt * (kABytes >> 4) + k16 * 2), desc_hi);
                const uint64_t bd = mk64(desc_lo + boff16 + k16 * 2, desc_hi);
                if (k16 == 0) umma_f16<NN * BN>(tmem_base + acc_col, ad, bd, first ? 0u : 1u);
                else umma_f16_acc<NN * BN>(tmem_base + acc_col, ad, bd);
              }
            }
          }
          }
        }
        if (PAIR) {  // the stage is free, in both CTAs, once the MMAs above have read it
          umma2_commit(empty_b + 8 * st);
          umma2_commit(peer_empty + 8 * st);
        } else {
          umma_commit(empty_b + 8 * st);  // the stage is free once the MMAs above have read it
        }
        tr(1, 2, it - it0);
        desc_lo += stage16;
        if (++st == static_cast<uint32_t>(kStagesG)) {
          st = 0;
          ph ^= 1;
          desc_lo = desc_lo0;
        }
      }
      if (PAIR) {
        umma2_commit(accum_b);
        umma2_commit(peer_accum);
      } else {
        umma_commit(accum_b);
      }
    }
    if (PAIR && lane == 0 && crank == 1) {
      // relay: tell the MMA thread (CTA 0) when this CTA's operand copies of a stage have landed
      const uint32_t bready0 = map_to_cta(bready_b, 0);
      uint32_t st = 0, ph = 0;
      bool ok = true;
      for (int it = it0; it < nk; ++it) {
        ok = ok && g_mbar_wait(full_b + 8 * st, ph, abort_flag, p.status);
        g_mbar_arrive_cluster(bready0 + 8 * st);
        tr(1, 1, it - it0);
        if (++st == static_cast<uint32_t>(kStagesG)) {
          st = 0;
          ph ^= 1;
        }
      }
    }
    __syncwarp();
  } else {
    // ================================================================ dequant warps, then epilogue
    // one thread per half-row (32 columns) of the step's 128 NN-row packed tile, kPassGroups such half-rows per pass
    constexpr int H = kPG;
    constexpr int kGroupThreads = Cfg<NN>::kDequantWarps * 32 / H;
    const int dt = threadIdx.x - 32 * Cfg<NN>::kCtrlWarps;
    const int pg = dt / kGroupThreads, lt = dt - pg * kGroupThreads;  // pass group, thread within it
    const bool tr_warp = warp == Cfg<NN>::kCtrlWarps;
    int rloc[H], half[H];
    bool rvalid[H];
    uint32_t b_row[H], sw[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const int item = lt + h * kGroupThreads;
      rloc[h] = item >> 1;
      half[h] = item & 1;
      rvalid[h] = (n0 + rloc[h]) < mb.OC;
      b_row[h] = (static_cast<uint32_t>(rloc[h]) >> 3) * 1024 + (static_cast<uint32_t>(rloc[h]) & 7) * 128;
      sw[h] = static_cast<uint32_t>(rloc[h]) & 7;
    }
    uint32_t st = pg, ph = 0, sp = pg, pph = 0;   // kPassGroups <= ring depths
    const uint32_t bready0 = PAIR ? map_to_cta(bready_b, 0) : bready_b;
    bool ok = true;
    // scale / zero-point of a row: quantisation group G covers steps 2G and 2G+1; the pair for the next step this pass
    // group will handle is fetched one pass ahead, so that the global-load latency never sits between a stage
    // becoming free and its tile being written
    const int n_groups = (p.nk1 + 1) >> 1;
    auto fetch_sz = [&](int h, int G, uint32_t& sbits, uint32_t& z) {
      sbits = 0;
      z = 0;
      if (rvalid[h] && G < n_groups && p.w4) {
        const size_t row = static_cast<size_t>(n0 + rloc[h]);
        sbits = __half_as_ushort(mb.scales[row * mb.sstride + G]);
        z = nibble(mb.qzeros + row * mb.zstride, G);
      }
    };
    uint32_t nx_s[H], nx_z[H], s2[H], zlo[H], zhi[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
      fetch_sz(h, (it0 + pg) >> 1, nx_s[h], nx_z[h]);
      s2[h] = zlo[h] = zhi[h] = 0;
    }
    int cur_g = -1;
    for (int it = it0 + pg; it < nk; it += H) {
      const bool packed = it < nk_packed;
      if (tr_warp) tr(2, 0, it - it0);
      if (lane == 0) {  // one lane polls: the packed tile has landed, and the MMAs that read this B slot are done
        if (!(packed && ok && g_mbar_try_both(pfull_b + 8 * sp, pph, empty_b + 8 * st, ph ^ 1))) {
          if (packed) ok = ok && g_mbar_wait(pfull_b + 8 * sp, pph, abort_flag, p.status);
          ok = ok && g_mbar_wait(empty_b + 8 * st, ph ^ 1, abort_flag, p.status);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (tr_warp) tr(2, 1, it - it0);
      if (packed) {
        if ((it >> 1) != cur_g) {  // first step of this pass group in quantisation group it/2
          cur_g = it >> 1;
#pragma unroll
          for (int h = 0; h < H; ++h) {
            s2[h] = nx_s[h] * 0x00010001u;
            zero_consts(nx_z[h], zlo[h], zhi[h]);
          }
        }
        if (((it + H) >> 1) != cur_g) {
#pragma unroll
          for (int h = 0; h < H; ++h) fetch_sz(h, (it + H) >> 1, nx_s[h], nx_z[h]);
        }
        if (ok) {
          const uint32_t sbase = ring + st * kStageG, psrc = pring + sp * kPStage;
#pragma unroll
          for (int h = 0; h < H; ++h) {
            const uint32_t pbase = psrc + rloc[h] * 32 + half[h] * 16;
            uint32_t w[4];
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(pbase));
            const uint32_t bbase = sbase + kBOff + b_row[h];  // row rloc of the NN stacked 128-row tiles
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 16-byte chunk c = columns 8c .. 8c+7 of the step
              const uint32_t c = static_cast<uint32_t>(half[h] * 4 + j);
              uint32_t hh[4];
              unpack8_minus_zero(w[j], zlo[h], zhi[h], hh);
#pragma unroll
              for (int i = 0; i < 4; ++i) hh[i] = hmul2(hh[i], s2[h]);  // (n0,n4) (n1,n5) (n2,n6) (n3,n7), rounded once
              const uint32_t v0 = prmt(hh[0], hh[1], 0x5410), v1 = prmt(hh[2], hh[3], 0x5410);
              const uint32_t v2 = prmt(hh[0], hh[1], 0x7632), v3 = prmt(hh[2], hh[3], 0x7632);
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(bbase + ((c ^ sw[h]) << 4)), "r"(v0), "r"(v1),
                           "r"(v2), "r"(v3)
                           : "memory");
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the MMA
        }
      }
      __syncwarp();
      if (lane == 0) {
        if (PAIR && crank != 0) {
          g_mbar_arrive_cluster(bready0 + 8 * st);
        } else {
          g_mbar_arrive(bready_b + 8 * st);
        }
        if (packed) g_mbar_arrive(pempty_b + 8 * sp);
      }
      if (tr_warp) tr(2, 2, it - it0);
      st += H;
      if (st >= static_cast<uint32_t>(kStagesG)) {
        st -= kStagesG;
        ph ^= 1;
      }
      if (packed) {
        sp += H;
        if (sp >= static_cast<uint32_t>(kPStagesG)) {
          sp -= kPStagesG;
          pph ^= 1;
        }
      }
    }

    // ---- epilogue: this warp owns TMEM lanes 32 (warp % 4) .. +31 = 32 tokens; one token per lane
    ok = ok && g_mbar_wait(accum_b, 0, abort_flag, p.status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // With a separate correction accumulator, a K slice that lies wholly in one phase never writes the other
    // phase's accumulator: that one counts as zero.
    const bool has_main = it0 < p.nk1, has_lr = nk > p.nk1;
    const int q = warp & 3;                          // TMEM lane quadrant this warp may read
    constexpr int kWays = Cfg<NN>::kDequantWarps / 4;  // warps that share a lane quadrant split the tile's columns
    constexpr int kCbPer = (BN / 32) / kWays;
    const int cb0 = ((warp - Cfg<NN>::kCtrlWarps) >> 2) * kCbPer;
    // bias, conversion and store of 32 consecutive columns c0.. of token tok
    auto emit = [&](float (&v)[32], int tok, int c0) {
      if (mb.bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < mb.OC) v[j] += __half2float(mb.bias[c0 + j]);
      }
      if (p.out_fp32) {
        float* o = static_cast<float*>(mb.out) + static_cast<size_t>(tok) * mb.out_stride + c0;
        if (mb.out_vec_ok && c0 + 32 <= mb.OC) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
          for (int j = 0; j < 32; ++j)
            if (c0 + j < mb.OC) o[j] = v[j];
        }
      } else {
        __half* o = static_cast<__half*>(mb.out) + static_cast<size_t>(tok) * mb.out_stride + c0;
        if (mb.out_vec_ok && c0 + 32 <= mb.OC) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk;
            __half2 h;
            h = __floats2half2_rn(v[j], v[j + 1]);
            pk.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(v[j + 2], v[j + 3]);
            pk.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(v[j + 4], v[j + 5]);
            pk.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(v[j + 6], v[j + 7]);
            pk.w = *reinterpret_cast<uint32_t*>(&h);
            *reinterpret_cast<uint4*>(o + j) = pk;
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (c0 + j < mb.OC) o[j] = __float2half_rn(v[j]);
        }
      }
    };
    const size_t kSlotFloats = static_cast<size_t>(NN) * p.mt * p.slot_rows * BN;
    if (!PAIR && p.swap) {
      // TMEM lane = output column, TMEM column = token: for a fixed token the 32 lanes of a warp store 32 consecutive
      // output columns (one 64-byte segment in fp16)
      const int units = NN * (p.nt >> 5);
      const int col_l = q * 32 + lane;
      for (int u = (warp - Cfg<NN>::kCtrlWarps) >> 2; u < units; u += kWays) {
        const int nn = u / (p.nt >> 5), cb = u - nn * (p.nt >> 5);
        if (nn >= n_nt) continue;
        uint32_t acc[32], lr[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + nn * p.nt + cb * 32;
        tmem_ld32(taddr, acc);
        if (NN == 1 && mb.lr_separate) tmem_ld32(taddr + p.nt, lr);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col = n0 + nn * BN + col_l;
        if (ok && col < mb.OC) {
          const float bias = mb.bias ? __half2float(mb.bias[col]) : 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = m0 + cb * 32 + j;
            if (tok < p.M) {
              float v = (has_main || !mb.lr_separate) ? __uint_as_float(acc[j]) : 0.f;
              if (NN == 1 && mb.lr_separate && has_lr) v = fmaf(mb.alpha, __uint_as_float(lr[j]), v);
              v += bias;
              const size_t idx = static_cast<size_t>(tok) * mb.out_stride + col;
              if (p.out_fp32)
                static_cast<float*>(mb.out)[idx] = v;
              else
                static_cast<__half*>(mb.out)[idx] = __float2half_rn(v);
            }
          }
        }
      }
    } else if constexpr (PAIR) {
      // two accumulators of 256 columns: column c of accumulator n is output column 128 n + c of this pair tile when
      // c < 128 (rows CTA 0 dequantised), 256 + 128 n + (c - 128) otherwise (CTA 1's rows); 16 blocks of 32 columns
      const int tile_n0 = (bx - mb.tile_begin) * (2 * BN * NN);
      const int tok = m0 + q * 32 + lane;
      constexpr int kUnits = 16 / kWays;
      const int u0 = ((warp - Cfg<NN>::kCtrlWarps) >> 2) * kUnits;
      for (int u = u0; u < u0 + kUnits; ++u) {
        const int n = u >> 3, cb = u & 7;
        uint32_t acc[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + n * (2 * BN) + cb * 32, acc);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int c = cb * 32;
        const int c0 = tile_n0 + (c < BN ? n * BN + c : 2 * BN + n * BN + (c - BN));
        if (ok && tok < p.M && c0 < mb.OC) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
          emit(v, tok, c0);
        }
      }
    } else {
    for (int at = 0; at < NN * MT; ++at) {
      const int nn = at / MT, mt = at - nn * MT;
      if (mt >= n_mt || nn >= n_nt) continue;
      const int tok = m0 + mt * BM + q * 32 + lane;
      const uint32_t acc_col = (NN == 1) ? mt * (2 * BN) : (mt * NN + nn) * BN;
      for (int cb = cb0; cb < cb0 + kCbPer; ++cb) {
        uint32_t acc[32], lr[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc_col + cb * 32;
        tmem_ld32(taddr, acc);
        if (NN == 1 && mb.lr_separate) tmem_ld32(taddr + BN, lr);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int c0 = n0 + nn * BN + cb * 32;
        if (ok && tok < p.M) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = (has_main || !mb.lr_separate) ? __uint_as_float(acc[j]) : 0.f;
            if (NN == 1 && mb.lr_separate && has_lr) v[j] = fmaf(mb.alpha, __uint_as_float(lr[j]), v[j]);
          }
          if (ks > 1) {
            float* sl = p.slots + (static_cast<size_t>(zslice) * p.n_tail + (tile_lin - p.full_tiles)) * kSlotFloats +
                        static_cast<size_t>(nn * p.mt + mt) * (p.slot_rows * BN) + (q * 32 + lane) * BN + cb * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 4) __stcg(reinterpret_cast<float4*>(sl + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
          } else {
            emit(v, tok, c0);
          }
        }
      }
    }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();  // neither CTA retires while the other's MMAs or arrivals may still touch it
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// out[tok, col..col+3] = half(sum over slices of the 128 x 128 fp32 slot tiles), slices added in order.
__global__ void slot_sum_kernel(const float* __restrict__ slots, __half* __restrict__ out, int M, int N, int out_stride,
                                int ksplit, int tiles_x, int tiles_all) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the slots come from the kernel before
  const int quads = N >> 2;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * quads) return;
  const int tok = idx / quads, col = (idx - tok * quads) << 2;
  const size_t tile = static_cast<size_t>(tok / BM) * tiles_x + col / BN;
  const size_t in_tile = static_cast<size_t>(tok % BM) * BN + (col % BN);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < ksplit; ++z) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(slots + (static_cast<size_t>(z) * tiles_all + tile) * (BM * BN) + in_tile));
    acc.x += t.x;
    acc.y += t.y;
    acc.z += t.z;
    acc.w += t.w;
  }
  __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
  uint2 pk;
  pk.x = *reinterpret_cast<uint32_t*>(&lo);
  pk.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(out + static_cast<size_t>(tok) * out_stride + col) = pk;
}

// K-sliced tiles of a group GEMM: out[tok, col .. col + 3] of the member that owns the tile's columns = sum over the K
// slices of the slot tiles (in slice order) + bias.  One thread per 4 columns of a sliced tile.
__global__ void slot_sum_members_kernel(const __grid_constant__ GemmParams p, int nn) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the slots come from the kernel before
  const int per_blk = p.slot_rows * (BN / 4), per_tile = nn * p.mt * per_blk;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.n_tail * per_tile) return;
  const int tail = idx / per_tile;
  int rem = idx - tail * per_tile;
  const int blk = rem / per_blk;                    // accumulator of the tile: column block major, token block minor
  rem -= blk * per_blk;
  const int row = rem / (BN / 4), c4 = (rem - row * (BN / 4)) * 4;
  const int tile_lin = p.full_tiles + tail, ty = tile_lin / p.n_x, tile = tile_lin - ty * p.n_x;
  const int nn_i = blk / p.mt, mt_i = blk - nn_i * p.mt;
  const int tok = ty * (BM * p.mt) + mt_i * BM + row;
  int mi = 0;
  for (int i = 1; i < kMaxMembers; ++i)
    if (i < p.n_members && tile >= p.mem[i].tile_begin) mi = i;
  const GemmMember& mb = p.mem[mi];
  const int col = (tile - mb.tile_begin) * (BN * nn) + nn_i * BN + c4;
  if (tok >= p.M || col >= mb.OC) return;
  const size_t slot_floats = static_cast<size_t>(nn) * p.mt * p.slot_rows * BN;
  const size_t in_slot = static_cast<size_t>(blk) * (p.slot_rows * BN) + static_cast<size_t>(row) * BN + c4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < p.ksplit; ++z) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(p.slots + (static_cast<size_t>(z) * p.n_tail + tail) * slot_floats + in_slot));
    acc.x += t.x;
    acc.y += t.y;
    acc.z += t.z;
    acc.w += t.w;
  }
  float v[4] = {acc.x, acc.y, acc.z, acc.w};
  const size_t o = static_cast<size_t>(tok) * mb.out_stride + col;
  for (int j = 0; j < 4; ++j) {
    if (col + j < mb.OC) {
      const float r = v[j] + (mb.bias ? __half2float(mb.bias[col + j]) : 0.f);
      if (p.out_fp32)
        static_cast<float*>(mb.out)[o + j] = r;
      else
        static_cast<__half*>(mb.out)[o + j] = __float2half_rn(r);
    }
  }
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch: a kernel of this file may start while its predecessor in the stream is still
// running; it touches nothing the predecessor may still write (activations, r, slots) before griddepcontrol.wait.
// GLOWQ_PDL=0 falls back to plain stream order.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("GLOWQ_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int NN, bool PAIR>
cudaError_t launch_gemm_nn(const GemmParams& p, const GemmMaps& tm, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_kernel<NN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         std::max(Cfg<NN>::smem(1), Cfg<NN>::smem(2)));
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  const int cols_per_tile = BN * NN * (PAIR ? 2 : 1);
  int n_tiles = 0;
  for (int i = 0; i < p.n_members; ++i) n_tiles = std::max(n_tiles, p.mem[i].tile_begin + cdiv(p.mem[i].OC, cols_per_tile));
  GemmParams q = p;
  q.stages = Cfg<NN>::stages(p.mt);
  q.pstages = Cfg<NN>::kPStages;
  if (q.ksplit < 1) q.ksplit = 1;
  if (!PAIR) {
    const int n_y = q.swap ? 1 : cdiv(p.M, BM * p.mt), total = n_tiles * n_y;
    q.n_x = n_tiles;
    if (q.ksplit == 1) {
      q.full_tiles = total;
      q.n_tail = 0;
    } else if (q.n_tail <= 0) {  // every tile sliced (the caller sets n_tail to slice the last wave only)
      q.full_tiles = 0;
      q.n_tail = total;
    }
    dim3 grid(q.full_tiles + q.n_tail * q.ksplit, 1, 1);
    return launch_pdl(gemm_w4a16_kernel<NN, false>, grid, dim3(Cfg<NN>::kThreads), Cfg<NN>::smem(p.mt), stream, q, tm);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * n_tiles, cdiv(p.M, 2 * BM), 1);  // clusters of two CTAs along x
  cfg.blockDim = dim3(Cfg<NN>::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg<NN>::smem(1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_w4a16_kernel<NN, PAIR>, q, tm);
}

// nn = 2 needs in-place accumulation of the correction (no separate accumulator columns left); pair implies nn = 2.
cudaError_t launch_gemm(const GemmParams& p, const GemmMaps& tm, int nn, bool pair, cudaStream_t stream) {
  if (pair) return launch_gemm_nn<2, true>(p, tm, stream);
  return nn == 2 ? launch_gemm_nn<2, false>(p, tm, stream) : launch_gemm_nn<1, false>(p, tm, stream);
}

}  // namespace

bool gemm_supported(const glowq_w4a16_group_t& g) {
  if (g.group_size != kGroup || g.M < 1) return false;
  if (!al16(g.x) || (g.x_stride & 7) || (g.IC & 7)) return false;
  const int G = (g.IC + kGroup - 1) / kGroup;
  for (int i = 0; i < g.n_members; ++i) {
    const auto& m = g.members[i];
    if (m.weight_stride_i32 < G * 16 || (m.weight_stride_i32 & 3) || !al16(m.qweight)) return false;
    if (g.r_mode != GLOWQ_R_NONE && m.L && (!al16(m.L) || (m.L_stride & 7))) return false;
  }
  if (g.r_mode != GLOWQ_R_NONE && ((g.rank & 7) || !al16(g.r_buf))) return false;
  if (g.r_mode == GLOWQ_R_COMPUTE && (!al16(g.R) || (g.R_stride & 7))) return false;
  return true;
}

// K slices of the r = X . R^T product (a [M, rank] output is a handful of tiles: without slicing a few CTAs would
// walk all of K while the rest of the GPU idles).  Device-independent so that the workspace size is, too.
constexpr size_t kRSlotBytes = static_cast<size_t>(BM) * BN * 4;   // slot of an NN = 1, mt = 1 tile
inline int r_ksplit(int M, int IC, int rank) {
  const int tiles = cdiv(rank, BN) * cdiv(M, BM), nk = cdiv(IC, BK);
  if (tiles > 64) return 1;
  return std::max(1, std::min({16, nk / 4, 128 / tiles}));
}

inline size_t r_slot_bytes(int M, int IC, int rank) {
  const int ks = r_ksplit(M, IC, rank);
  return ks > 1 ? static_cast<size_t>(ks) * cdiv(rank, BN) * cdiv(M, BM) * kRSlotBytes : 0;
}
// The slots sit at the END of the workspace, clear of the counters that the weight-streaming kernel keeps (zeroed)
// at its start: one workspace may serve launches of both kernels in turn.
inline size_t counters_end(int OC_total, int n_members) {
  const size_t n = kWsTileCtrOffset + (static_cast<size_t>(cdiv(OC_total, kTileRows)) + n_members) * 4;
  return (n + 255) & ~static_cast<size_t>(255);
}

// K slices of a group GEMM with few tiles (up to 128 tokens): planned for 148 SMs so that the workspace size does not
// depend on the device.
constexpr int kPlanSms = 148;
constexpr int kMaxTailSlots = 64;   // tiles x slices of a sliced last wave (256 KB of fp32 each for a 256 x 256 tile)
inline int main_ksplit(int tiles, int nk, int sms) {
  if (tiles * 2 > sms) return 1;
  return std::max(1, std::min({8, sms / tiles, nk / 8}));
}
inline int slot_rows_for(int M) { return std::min(BM, ((M + 31) / 32) * 32); }
inline size_t main_slot_bytes_bound(int M, int IC, int OC_total, int n_members) {
  // (up to 8 tokens the automatic choice never takes this kernel; a forced call then runs without slicing)
  const int m_tiles = cdiv(M, BM);
  if (M <= 8 || M > 2 * BM || cdiv(OC_total, 2 * BN) * m_tiles * 2 > kPlanSms) return 0;
  const int tiles_ub = (cdiv(OC_total, BN) + n_members) * m_tiles;  // 128 x 128 tiles
  // at most 8 slices, and slices x (256-column tiles) <= SMs, i.e. at most 2 SMs' worth of 128-column slot tiles
  const int slots_ub = std::min(8 * tiles_ub, 2 * kPlanSms + tiles_ub);
  return static_cast<size_t>(slots_ub) * slot_rows_for(M) * BN * 4;
}

size_t gemm_workspace_bytes(int M, int IC, int OC_total, int rank, int n_members) {
  size_t slots = std::max(rank > 0 ? r_slot_bytes(M, IC, rank) : 0, main_slot_bytes_bound(M, IC, OC_total, n_members));
  if (rank > 0 && M <= kRProductMaxM) slots = std::max(slots, r_product_slot_bytes(M, IC, rank));
  if (M > 2 * BM) slots = std::max(slots, static_cast<size_t>(kMaxTailSlots) * 2 * 2 * BM * BN * 4);  // sliced last wave
  if (slots == 0) return kWsHeaderBytes;
  return counters_end(OC_total, n_members) + slots + 256;
}

int gemm_group_forward(const glowq_w4a16_group_t& g, cudaStream_t stream, cudaError_t* cuda_err) {
  if (g.workspace_bytes < kWsHeaderBytes) return GLOWQ_ERR_WORKSPACE_TOO_SMALL;
  uint32_t* status = static_cast<uint32_t*>(g.workspace) + WS_STATUS;
  const int G = (g.IC + kGroup - 1) / kGroup;
  const bool any_corr = [&] {
    if (g.r_mode == GLOWQ_R_NONE) return false;
    for (int i = 0; i < g.n_members; ++i)
      if (g.members[i].L && g.members[i].alpha != 0.f) return true;
    return false;
  }();
  auto map = [&](CUtensorMap* out, CUtensorMapDataType dt, const void* ptr, uint64_t d0, uint64_t d1, uint64_t stride,
                 uint32_t b0, uint32_t b1, int sw) { return tensor_map_2d_ex(out, dt, ptr, d0, d1, stride, b0, b1, sw); };
  int rc;
  CUtensorMap tm_x;
  if ((rc = map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, g.x, g.IC, g.M, static_cast<uint64_t>(g.x_stride) * 2, BK, BM, 1)))
    return rc;

  // r = X . R^T, once per group, into r_buf.  Up to 128 tokens: one small launch (r_product.cu); the K-sliced GEMM
  // below plus its slot sum take about twenty microseconds.
  bool r_done = false;
  if (g.r_mode == GLOWQ_R_COMPUTE && g.M <= kRProductMaxM && cdiv(g.rank, 16) * cdiv(g.M, 64) <= kRpCtrWords) {
    int oc_total = 0;
    for (int i = 0; i < g.n_members; ++i) oc_total += g.members[i].OC;
    const size_t need = r_product_slot_bytes(g.M, g.IC, g.rank);
    const size_t off = g.workspace_bytes >= need ? ((g.workspace_bytes - need) & ~static_cast<size_t>(255)) : 0;
    if (off >= counters_end(oc_total, g.n_members)) {
      unsigned char* ws = static_cast<unsigned char*>(g.workspace);
      const cudaError_t e = launch_r_product(static_cast<const __half*>(g.x), static_cast<const __half*>(g.R),
                                             static_cast<__half*>(g.r_buf), reinterpret_cast<float*>(ws + off),
                                             reinterpret_cast<uint32_t*>(ws + kWsHeaderBytes), g.M, g.IC, g.rank, g.x_stride,
                                             g.R_stride, stream);
      if (e != cudaSuccess) {
        *cuda_err = e;
        return GLOWQ_ERR_CUDA;
      }
      r_done = true;
    }
  }
  if (g.r_mode == GLOWQ_R_COMPUTE && !r_done) {
    GemmParams p{};
    GemmMaps tm;
    std::memset(&tm, 0, sizeof(tm));
    tm.a1 = tm.a2 = tm_x;
    if ((rc = map(&tm.b1[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, g.R, g.IC, g.rank, static_cast<uint64_t>(g.R_stride) * 2, BK, BN, 1)))
      return rc;
    tm.b2[0] = tm.b1[0];
    p.status = status;
    p.M = g.M;
    p.nk1 = cdiv(g.IC, BK);
    p.w4 = 0;
    p.out_fp32 = 0;
    p.n_members = 1;
    p.mt = 1;  // narrow output (rank columns): small tiles, more CTAs
    p.ksplit = r_ksplit(g.M, g.IC, g.rank);
    int oc_total = 0;
    for (int i = 0; i < g.n_members; ++i) oc_total += g.members[i].OC;
    const size_t slot_bytes = r_slot_bytes(g.M, g.IC, g.rank);
    size_t slot_off = g.workspace_bytes >= slot_bytes ? ((g.workspace_bytes - slot_bytes) & ~static_cast<size_t>(255)) : 0;
    if (slot_off < counters_end(oc_total, g.n_members)) {  // workspace not sized for slicing: one CTA per tile walks all of K
      p.ksplit = 1;
      slot_off = kWsHeaderBytes;
    }
    p.slots = reinterpret_cast<float*>(static_cast<unsigned char*>(g.workspace) + slot_off);
    p.slot_rows = BM;
    p.mem[0].out = g.r_buf;
    p.mem[0].OC = g.rank;
    p.mem[0].out_stride = g.rank;
    p.mem[0].alpha = 1.f;
    p.mem[0].out_vec_ok = 1;  // rank % 8 == 0 and r_buf aligned
    cudaError_t e = launch_gemm(p, tm, 1, false, stream);
    if (e == cudaSuccess && p.ksplit > 1) {
      const int tiles_x = cdiv(g.rank, BN), tiles_all = tiles_x * cdiv(g.M, BM), n = g.M * (g.rank >> 2);
      e = launch_pdl(slot_sum_kernel, dim3(cdiv(n, 256)), dim3(256), 0, stream, static_cast<const float*>(p.slots),
                     static_cast<__half*>(g.r_buf), g.M, g.rank, g.rank, p.ksplit, tiles_x, tiles_all);
    }
    if (e != cudaSuccess) {
      *cuda_err = e;
      return GLOWQ_ERR_CUDA;
    }
  }
  CUtensorMap tm_r;
  std::memset(&tm_r, 0, sizeof(tm_r));
  if (any_corr &&
      (rc = map(&tm_r, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, g.r_buf, g.rank, g.M, static_cast<uint64_t>(g.rank) * 2, BK, BM, 1)))
    return rc;

  // All members in ONE launch: the grid's x index runs over the column tiles of member 0, then member 1, ...
  bool any_separate = false;
  for (int i = 0; i < g.n_members; ++i) {
    const auto& m = g.members[i];
    any_separate = any_separate || (g.r_mode != GLOWQ_R_NONE && m.L && m.alpha != 0.f && m.alpha != 1.f);
  }
  // Tile shape: the 256 x 256 CTA tile has the best operand reuse, but a problem that fills the SMs badly in whole
  // waves is faster with narrower (nn = 1) or shorter (mt = 1) tiles.  A separate correction accumulator needs nn = 1.
  int nn = 1, mt = 2;
  bool pair = false;
  static const int env_pair = [] { const char* e = std::getenv("GLOWQ_GEMM_PAIR"); return e ? std::atoi(e) : -1; }();
  static const int env_swap = [] { const char* e = std::getenv("GLOWQ_GEMM_SWAP"); return e ? std::atoi(e) : -1; }();
  // Up to 128 tokens: weights on the M side of the MMA, tokens on its N side (see GemmParams::swap).  Measured no
  // faster than tokens on the M side (31.5 vs 30.3 us for Llama-3.2-3B gate/up at 32 tokens): at these sizes the MMA
  // thread's issue rate sets the pace, and N = 256 instructions need half as many issues per weight row.  Opt-in.
  const bool swap = g.M <= BM && env_swap == 1;
  const int nt = g.M <= 32 ? 32 : (g.M <= 64 ? 64 : BM);
  {
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    double best = -1.0;
    static const int env_ks0 = [] { const char* e = std::getenv("GLOWQ_GEMM_KSPLIT"); return e ? std::atoi(e) : -1; }();
    const bool can_slice_tail = !any_separate && g.M > 2 * BM && env_ks0 != 0;
    auto consider = [&](int cnn, int cmt, bool cpair, long ctas, double reuse) {
      // waves this many tiles take; a last wave that fills at most half of the SMs is K-sliced (see the work partition
      // below) and then costs 1/slices of a wave plus the slot traffic
      double waves = static_cast<double>(cdiv(static_cast<int>(ctas), sms));
      const int rest = static_cast<int>(ctas % sms);
      if (can_slice_tail && !cpair && ctas > sms && rest > 0 && rest * 2 <= sms) {
        const int ks = std::min({8, kMaxTailSlots / rest, cdiv(g.IC, BK) / 8});
        if (ks >= 2) waves = static_cast<double>(ctas / sms) + 1.0 / ks + 0.3;
      }
      const double wave_eff = static_cast<double>(ctas) / (waves * sms);
      if (wave_eff * reuse > best) {
        best = wave_eff * reuse;
        nn = cnn;
        mt = cmt;
        pair = cpair;
      }
    };
    if (!any_separate && g.M > BM && env_pair == 1) {  // CTA pairs (measured no faster than one CTA per tile: opt-in): 256 tokens x 512 columns per pair
      long tiles = 0;
      for (int i = 0; i < g.n_members; ++i) tiles += cdiv(g.members[i].OC, 4 * BN);
      consider(2, 1, true, 2 * tiles * cdiv(g.M, 2 * BM), 1.3);
    }
    for (int cnn = any_separate ? 1 : 2; cnn >= 1; --cnn)
      for (int cmt = swap ? 1 : 2; cmt >= 1; --cmt) {
        long tiles = 0;
        for (int i = 0; i < g.n_members; ++i) tiles += cdiv(g.members[i].OC, BN * cnn);
        // mt = 1 doubles the dequant work per flop
        if (swap)
          consider(cnn, 1, false, tiles, cnn == 2 ? 1.0 : 0.9);
        else
          consider(cnn, cmt, false, tiles * cdiv(g.M, BM * cmt), (cnn == 2 ? 1.0 : 0.75) * (cmt == 2 ? 1.0 : 0.65));
      }
  }
  static const int env_ks = [] { const char* e = std::getenv("GLOWQ_GEMM_KSPLIT"); return e ? std::atoi(e) : -1; }();
  if (g.M <= 2 * BM && !any_separate && !swap && env_ks != 0) {
    // Up to 256 tokens a CTA's K-step rate bounds the launch, not the flops: pick the column-tile width together with
    // the K slicing, by steps per CTA x relative step time (a 256-column step takes about 4/3 of a 128-column one).
    int sms = kPlanSms, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int nk = cdiv(g.IC, BK);
    double best_cost = 1e30;
    for (int cnn = 2; cnn >= 1; --cnn)
      for (int cmt = 1; cmt <= (g.M > BM ? 2 : 1); ++cmt) {
        int tiles = 0;
        for (int i = 0; i < g.n_members; ++i) tiles += cdiv(g.members[i].OC, BN * cnn);
        tiles *= cdiv(g.M, BM * cmt);
        const int ks = cmt == 1 ? main_ksplit(tiles, nk, std::min(sms, kPlanSms)) : 1;  // slices are written per 128 tokens
        const double step = cmt == 2 ? (cnn == 2 ? 1.45 : 1.05) : (cnn == 2 ? 1.0 : 0.75);  // measured clocks per step, relative
        // + the fp32 slot traffic of a sliced launch, in step equivalents
        const double cost = static_cast<double>(cdiv(tiles * ks, sms)) * cdiv(nk, ks) * step +
                            (ks > 1 ? 14.0 * slot_rows_for(g.M) / BM : 0.0);
        if (cost < best_cost) {
          best_cost = cost;
          nn = cnn;
          mt = cmt;
          pair = false;
        }
      }
  }
  {  // tuning overrides (unset in production)
    static const int env_nn = [] { const char* e = std::getenv("GLOWQ_GEMM_NN"); return e ? std::atoi(e) : 0; }();
    static const int env_mt = [] { const char* e = std::getenv("GLOWQ_GEMM_MT"); return e ? std::atoi(e) : 0; }();
    if ((env_nn == 1 || env_nn == 2) && !(any_separate && env_nn == 2)) nn = env_nn, pair = false;
    if ((env_mt == 1 || env_mt == 2) && !swap) mt = env_mt, pair = false;
    if (env_pair == 1 && !any_separate && !swap) pair = true;
    if (pair) nn = 2, mt = 1;
  }
  GemmParams p{};
  GemmMaps tm;
  std::memset(&tm, 0, sizeof(tm));
  tm.a1 = tm_x;
  tm.a2 = any_corr ? tm_r : tm_x;
  if (swap) {  // activation boxes of nt token rows
    if ((rc = map(&tm.a1, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, g.x, g.IC, g.M, static_cast<uint64_t>(g.x_stride) * 2, BK, nt, 1)))
      return rc;
    tm.a2 = tm.a1;
    if (any_corr && (rc = map(&tm.a2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, g.r_buf, g.rank, g.M,
                              static_cast<uint64_t>(g.rank) * 2, BK, nt, 1)))
      return rc;
    p.swap = 1;
    p.nt = nt;
  }
  p.status = status;
  p.M = g.M;
  p.nk1 = cdiv(g.IC, BK);
  p.w4 = 1;
  p.out_fp32 = g.out_dtype == GLOWQ_OUT_F32;
  p.n_members = g.n_members;
  // Few tiles and few tokens: slice K over gridDim.z so that all SMs stream weights (a CTA's step rate, not the
  // amount of work, bounds small token counts), and add the slices up afterwards.
  int ksplit = 1;
  size_t main_slot_off = 0;
  if (!pair && !swap && !any_separate && g.M <= 2 * BM && mt == 1 && env_ks != 0) {
    int sms = kPlanSms, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long tiles = 0;
    for (int i = 0; i < g.n_members; ++i) tiles += cdiv(g.members[i].OC, BN * nn);
    tiles *= cdiv(g.M, BM);
    ksplit = main_ksplit(static_cast<int>(tiles), cdiv(g.IC, BK), std::min(sms, kPlanSms));
    if (env_ks > 0) ksplit = std::min(env_ks, std::max(1, cdiv(g.IC, BK) / 2));
    if (ksplit > 1) {
      int oc_total = 0;
      for (int i = 0; i < g.n_members; ++i) oc_total += g.members[i].OC;
      const size_t need = static_cast<size_t>(ksplit) * tiles * nn * slot_rows_for(g.M) * BN * 4;
      main_slot_off = g.workspace_bytes >= need ? ((g.workspace_bytes - need) & ~static_cast<size_t>(255)) : 0;
      if (main_slot_off < counters_end(oc_total, g.n_members)) ksplit = 1;  // workspace not sized for slicing
    }
    if (ksplit > 1) mt = 1;
  }
  p.mt = mt;
  p.ksplit = ksplit;
  p.slot_rows = slot_rows_for(g.M);
  p.slots = reinterpret_cast<float*>(static_cast<unsigned char*>(g.workspace) + main_slot_off);
  p.debug = g.reserved;
  int tile_begin = 0;
  for (int i = 0; i < g.n_members; ++i) {
    const auto& m = g.members[i];
    const bool corr = g.r_mode != GLOWQ_R_NONE && m.L && m.alpha != 0.f;
    if ((rc = map(&tm.b1[i], CU_TENSOR_MAP_DATA_TYPE_INT32, m.qweight, static_cast<uint64_t>(G) * 16, m.OC,
                  static_cast<uint64_t>(m.weight_stride_i32) * 4, BK / 8, BN * nn, 0)))
      return rc;
    tm.b2[i] = tm.b1[i];
    if (corr && (rc = map(&tm.b2[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, m.L, g.rank, m.OC,
                          static_cast<uint64_t>(m.L_stride) * 2, BK, BN * nn, 1)))
      return rc;
    GemmMember& d = p.mem[i];
    d.scales = static_cast<const __half*>(m.scales);
    d.qzeros = m.qzeros;
    d.bias = static_cast<const __half*>(m.bias);
    d.out = m.out;
    d.OC = m.OC;
    d.nk2 = corr ? cdiv(g.rank, BK) : 0;
    d.sstride = m.scale_stride;
    d.zstride = m.zero_stride_i32;
    d.out_stride = m.out_stride;
    d.alpha = m.alpha;
    d.lr_separate = corr && m.alpha != 1.f;
    const int esz = p.out_fp32 ? 4 : 2;
    d.out_vec_ok = al16(m.out) && ((static_cast<size_t>(m.out_stride) * esz) % 16 == 0);
    d.tile_begin = tile_begin;
    tile_begin += cdiv(m.OC, BN * nn * (pair ? 2 : 1));
  }
  // Work partition (see GemmParams): all tiles sliced for few tokens; for a large launch whose last wave would leave
  // more than half of the SMs idle, only that wave's tiles are sliced, so that it takes 1/ksplit of a tile's time.
  p.n_x = tile_begin;
  {
    const int total = tile_begin * cdiv(g.M, BM * mt);
    if (p.ksplit > 1) {
      p.full_tiles = 0;
      p.n_tail = total;
    } else if (!pair && !swap && !any_separate && g.M > 2 * BM && env_ks != 0) {
      int sms = kPlanSms, dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      const int waves = total / sms, rest = total % sms;
      if (waves >= 1 && rest > 0 && rest * 2 <= sms) {
        const int ks = std::min({8, kMaxTailSlots / rest, cdiv(g.IC, BK) / 8});
        int oc_total = 0;
        for (int i = 0; i < g.n_members; ++i) oc_total += g.members[i].OC;
        const size_t need = static_cast<size_t>(ks) * rest * nn * mt * BM * BN * 4;
        const size_t off = g.workspace_bytes >= need ? ((g.workspace_bytes - need) & ~static_cast<size_t>(255)) : 0;
        if (ks >= 2 && off >= counters_end(oc_total, g.n_members)) {
          p.ksplit = ks;
          p.full_tiles = waves * sms;
          p.n_tail = rest;
          p.slot_rows = BM;
          p.slots = reinterpret_cast<float*>(static_cast<unsigned char*>(g.workspace) + off);
        }
      }
    }
  }
  cudaError_t e = launch_gemm(p, tm, nn, pair, stream);
  if (e == cudaSuccess && p.ksplit > 1) {
    const int n = p.n_tail * nn * p.mt * p.slot_rows * (BN / 4);
    e = launch_pdl(slot_sum_members_kernel, dim3(cdiv(n, 256)), dim3(256), 0, stream, p, nn);
  }
  if (e != cudaSuccess) {
    *cuda_err = e;
    return GLOWQ_ERR_CUDA;
  }
  return GLOWQ_OK;
}

}  // namespace glowq
