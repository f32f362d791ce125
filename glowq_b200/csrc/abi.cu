// extern "C" entry points declared in include/glowq_w4a16.h: argument validation, launch planning
// (K slices, workspace layout) and dispatch.  No allocation and no synchronisation on the compute path.
#include "../../include/glowq_w4a16.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "params.h"

namespace glowq {
size_t gemv_smem_bytes(const GemvParams& p, int NT);
cudaError_t launch_gemv_stream(const GemvParams& p, const TensorMaps& tm, int NT, int grid, cudaStream_t stream);
cudaError_t launch_generic_r(const __half* x, const __half* R, __half* r_buf, float* r32, int r_mode, int M, int IC,
                             int rank, int x_stride, int R_stride, cudaStream_t stream);
cudaError_t launch_generic(const __half* x, const MemberDev& mb, const float* r32, int out_fp32, int M, int IC, int rank,
                           int group_size, int x_stride, cudaStream_t stream);
cudaError_t launch_dequant(const int32_t* qweight, const __half* scales, const int32_t* qzeros, __half* out, int OC, int IC,
                           int group_size, int wstride, int zstride, int sstride, cudaStream_t stream);
bool gemm_supported(const glowq_w4a16_group_t& g);
size_t gemm_workspace_bytes(int M, int IC, int OC_total, int rank, int n_members);
unsigned allreduce_spin_limit();
int gemm_group_forward(const glowq_w4a16_group_t& g, cudaStream_t stream, cudaError_t* cuda_err);
}  // namespace glowq

using namespace glowq;

namespace {
int tensor_map_2d(CUtensorMap* out, CUtensorMapDataType dtype, const void* ptr, uint64_t dim0, uint64_t dim1,
                  uint64_t stride_bytes, uint32_t box0, uint32_t box1, int swizzle128);
}
namespace glowq {
// Shared with the GEMM translation unit: cached encode of a row-major 2-D tensor map.
int tensor_map_2d_ex(CUtensorMap* out, CUtensorMapDataType dtype, const void* ptr, uint64_t dim0, uint64_t dim1,
                     uint64_t stride_bytes, uint32_t box0, uint32_t box1, int swizzle128) {
  return tensor_map_2d(out, dtype, ptr, dim0, dim1, stride_bytes, box0, box1, swizzle128);
}
}  // namespace glowq

namespace {

thread_local int t_last_cuda_error = 0;

int fail_cuda(cudaError_t e) {
  t_last_cuda_error = static_cast<int>(e);
  return GLOWQ_ERR_CUDA;
}

struct DeviceInfo {
  bool probed = false;
  int major = 0;
  int sms = 0;
};
DeviceInfo g_dev[64];
std::mutex g_dev_mutex;

int device_info(const DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e);
  if (dev < 0 || dev >= 64) return GLOWQ_ERR_UNSUPPORTED_DEVICE;
  DeviceInfo& d = g_dev[dev];
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!d.probed) {
    if ((e = cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return fail_cuda(e);
    if ((e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return fail_cuda(e);
    d.probed = true;
  }
  *out = &d;
  return d.major == 10 ? GLOWQ_OK : GLOWQ_ERR_UNSUPPORTED_DEVICE;
}

// ---------------------------------------------------------------- TMA descriptors
// cuTensorMapEncodeTiled is fetched from the driver at run time (no link-time dependency on libcuda), and encoded
// descriptors are kept in a small direct-mapped cache keyed by (address, shape, box): a decode loop that is not
// graph-captured re-uses them instead of re-encoding seven descriptors per layer per token.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t dim0, dim1, stride_bytes;
  uint32_t box0, box1, dtype, swizzle;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && dim0 == o.dim0 && dim1 == o.dim1 && stride_bytes == o.stride_bytes && box0 == o.box0 &&
           box1 == o.box1 && dtype == o.dtype && swizzle == o.swizzle;
  }
};
struct MapSlot {
  MapKey key{};
  bool valid = false;
  alignas(64) CUtensorMap map;
};
constexpr int kMapCacheSlots = 4096;
MapSlot g_map_cache[kMapCacheSlots];
std::mutex g_map_mutex;

// Row-major 2-D tensor [dim1 rows, dim0 elements], row pitch stride_bytes, box [box1 rows, box0 elements].
int tensor_map_2d(CUtensorMap* out, CUtensorMapDataType dtype, const void* ptr, uint64_t dim0, uint64_t dim1,
                  uint64_t stride_bytes, uint32_t box0, uint32_t box1, int swizzle128 = 0) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return GLOWQ_ERR_UNSUPPORTED_DEVICE;
  const MapKey key{ptr, dim0, dim1, stride_bytes, box0, box1, static_cast<uint32_t>(dtype), static_cast<uint32_t>(swizzle128)};
  size_t h = reinterpret_cast<uintptr_t>(ptr) >> 8;
  h = (h ^ (h >> 12) ^ (dim0 * 0x9E3779B97F4A7C15ull) ^ (dim1 << 7) ^ box0 ^ (box1 << 3) ^ swizzle128) % kMapCacheSlots;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  MapSlot& slot = g_map_cache[h];
  if (!(slot.valid && slot.key == key)) {
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {stride_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&slot.map, dtype, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      slot.valid = false;
      return GLOWQ_ERR_CUDA;
    }
    slot.key = key;
    slot.valid = true;
  }
  std::memcpy(out, &slot.map, sizeof(CUtensorMap));
  return GLOWQ_OK;
}

// Packed weights for the weight-streaming kernel when the group count is even: [OC rows][G / 2][32 int32], box
// 32 rows x 4 x 128 B, the shared-memory image swizzled (16-byte chunks XORed within 128 bytes by the 128-byte line
// index mod 8) so that the consumers' 128-bit loads - eight rows 512 B apart per quarter warp - spread over all
// banks.  (An odd group count keeps the plain 2-D image: a 128-byte inner box would reach past the last row.)
int tensor_map_w3d(CUtensorMap* out, const void* ptr, uint64_t group_pairs, uint64_t rows, uint64_t stride_bytes) {
  const uint64_t groups = group_pairs;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return GLOWQ_ERR_UNSUPPORTED_DEVICE;
  const MapKey key{ptr, groups, rows, stride_bytes, kChunkGroups, kTileRows,
                   static_cast<uint32_t>(CU_TENSOR_MAP_DATA_TYPE_INT32), 2u};
  size_t h = reinterpret_cast<uintptr_t>(ptr) >> 8;
  h = (h ^ (h >> 12) ^ (groups * 0x9E3779B97F4A7C15ull) ^ (rows << 7) ^ 0x5bd1e995u) % kMapCacheSlots;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  MapSlot& slot = g_map_cache[h];
  if (!(slot.valid && slot.key == key)) {
    const cuuint64_t dims[3] = {32, group_pairs, rows};
    const cuuint64_t strides[2] = {128, stride_bytes};
    const cuuint32_t box[3] = {32, kChunkGroups / 2, kTileRows};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(&slot.map, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      slot.valid = false;
      return GLOWQ_ERR_CUDA;
    }
    slot.key = key;
    slot.valid = true;
  }
  std::memcpy(out, &slot.map, sizeof(CUtensorMap));
  return GLOWQ_OK;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kGemvMaxM = 8;                  // tokens per launch of the weight-streaming kernel (one MMA N tile)
constexpr int kGemvAutoMaxM = 8;              // GLOWQ_KERNEL_AUTO: one such launch, the tensor-core GEMM above
constexpr size_t kSmemTwoPerSm = 112 * 1024;  // dynamic shared memory that still lets two CTAs share an SM
constexpr size_t kSmemOnePerSm = 224 * 1024;

int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  return (v && *v) ? std::atoi(v) : dflt;
}

// Launch plan of the weight-streaming kernel (K slices, pipeline depth, grid) and the workspace carve-up.
struct GemvPlan {
  int NT, G, n_tiles, SK, gps, n_r_tiles, SKr, gpr, stages, ctas_per_sm, meta_gp, meta_gw, xs_stride;
  size_t smem;
  size_t off_r_ctr, off_tile_ctr, off_r_partial, off_sk_partial, off_r32, total;
};

size_t plan_smem(const GemvPlan& pl, int Mc, int stages) {
  return gemv_smem_layout_bytes(stages, pl.meta_gp, pl.meta_gw, pl.gps, pl.NT, Mc, pl.xs_stride);
}

GemvPlan make_plan(int M, int IC, int n_tiles, int rank, int sms, int split_k) {
  static const int forced_stages = env_int("GLOWQ_GEMV_STAGES", 0);       // tuning overrides
  static const int forced_ctas = env_int("GLOWQ_GEMV_CTAS_PER_SM", 0);
  GemvPlan pl{};
  const int Mc = std::min(M, kGemvMaxM);
  pl.NT = Mc <= 8 ? 1 : (Mc <= 16 ? 2 : 4);
  pl.G = ceil_div(IC, kGroup);
  pl.n_tiles = n_tiles;
  const int chunks = ceil_div(pl.G, kChunkGroups);
  // K is sliced across CTAs on request, when an unsliced CTA does not fit shared memory (long rows with several
  // tokens: the staged activations and the converted scale pairs grow with the slice length), and for ONE token on
  // long rows with few tiles (down_proj of the 7B - 14B shapes, K >= 12288): there the slice length is also chosen so
  // that two CTAs per SM with four ring stages fit.  Measured, microseconds sliced / unsliced: Llama-2-13B down_proj
  // 19.7 / 20.0, Qwen3-14B 29.6 / 32.5, Qwen2.5-7B 20.0 / 27.2 - but Llama-3.2-3B down_proj (K = 8192) 11.2 / 9.0, and
  // at two tokens q/k/v of the 13B shape 28.4 / 16.3, its o_proj 15.8 / 9.7, its down_proj 25.3 / 22.2: the combine
  // of the partial tiles (fence, counter, re-read) costs more than a somewhat shorter K walk saves.
  const bool slice_long_rows = split_k <= 0 && Mc == 1 && n_tiles < 2 * sms && chunks >= 12;
  int sk = 1;
  if (split_k > 0) {
    sk = std::min(split_k, chunks);
  } else if (slice_long_rows) {
    sk = std::max(1, std::min(ceil_div(2 * sms, std::max(1, n_tiles)), chunks / 4));
  }
  for (;; ++sk) {
    pl.gps = ceil_div(chunks, sk) * kChunkGroups;   // whole pipeline stages per slice
    pl.SK = ceil_div(pl.G, pl.gps);
    pl.meta_gp = (std::min(pl.gps, pl.G) + 1) & ~1;
    pl.meta_gw = ceil_div(pl.gps, 8);
    pl.xs_stride = pl.gps * 256 + 64;
    // deepest ring that fits, preferring two CTAs per SM (16 consumer warps per SM) when that leaves >= 4 stages
    pl.ctas_per_sm = (pl.NT <= 2) ? 2 : 1;
    if (forced_ctas > 0) pl.ctas_per_sm = std::min(forced_ctas, pl.ctas_per_sm);
    pl.stages = 0;
    for (int cps = pl.ctas_per_sm; cps >= 1 && pl.stages == 0; --cps) {
      const size_t cap = cps == 2 ? kSmemTwoPerSm : kSmemOnePerSm;
      for (int st = kMaxStages; st >= (cps == 2 ? 3 : 2); --st)
        if (plan_smem(pl, Mc, st) <= cap) {
          pl.stages = st;
          pl.ctas_per_sm = cps;
          break;
        }
    }
    if (pl.gps == kChunkGroups) break;  // K cannot be sliced any finer
    const bool want_two = slice_long_rows && sk < 8 && n_tiles * (sk + 1) <= 8 * sms;
    if (pl.stages > 0 && ((pl.ctas_per_sm == 2 && pl.stages >= 4) || !want_two)) break;
  }
  if (forced_stages > 0 && pl.stages > 0) pl.stages = std::max(2, std::min(forced_stages, pl.stages));
  pl.smem = plan_smem(pl, Mc, pl.stages);
  pl.n_r_tiles = ceil_div(std::max(rank, 0), kRTileRows);
  pl.SKr = chunks;   // one quantisation group per warp and R unit: a single round of loads per unit
  const size_t tile_elems = static_cast<size_t>(kRowTiles) * pl.NT * 128;
  pl.off_r_ctr = kWsHeaderBytes;
  size_t off = kWsTileCtrOffset;
  pl.off_tile_ctr = off;
  off = align_up(off + static_cast<size_t>(n_tiles) * 4, 256);
  pl.off_r_partial = off;
  pl.gpr = ceil_div(pl.G, pl.SKr);
  pl.SKr = ceil_div(pl.G, pl.gpr);
  off = align_up(off + static_cast<size_t>(pl.n_r_tiles) * pl.SKr * pl.NT * 128 * 4, 256);
  pl.off_sk_partial = off;
  off = align_up(off + (pl.SK > 1 ? static_cast<size_t>(n_tiles) * pl.SK * tile_elems * 4 : 0), 256);
  pl.off_r32 = off;
  off = align_up(off + static_cast<size_t>(Mc) * std::max(rank, 0) * 4, 256);
  pl.total = off;
  return pl;
}

int validate_member(const glowq_w4a16_member_t& m, int IC, int group_size) {
  if (!m.qweight || !m.scales || !m.qzeros || !m.out || m.OC <= 0) return GLOWQ_ERR_BAD_ARGUMENT;
  const int G = ceil_div(IC, group_size);
  if (m.weight_stride_i32 < ceil_div(IC, 8) || m.scale_stride < G || m.zero_stride_i32 < ceil_div(G, 8))
    return GLOWQ_ERR_BAD_STRIDE;
  if (m.out_stride < m.OC) return GLOWQ_ERR_BAD_STRIDE;
  return GLOWQ_OK;
}

int validate_group(const glowq_w4a16_group_t& g) {
  if (g.M == 0 && g.IC > 0 && g.n_members >= 1 && g.n_members <= GLOWQ_MAX_MEMBERS) return GLOWQ_OK;  // empty batch
  if (!g.x || g.M < 0 || g.IC <= 0 || g.n_members < 1 || g.n_members > GLOWQ_MAX_MEMBERS) return GLOWQ_ERR_BAD_ARGUMENT;
  if (g.group_size <= 0 || g.group_size % 8 != 0) return GLOWQ_ERR_BAD_GROUP_SIZE;
  if (g.x_stride < g.IC) return GLOWQ_ERR_BAD_STRIDE;
  if (g.out_dtype != GLOWQ_OUT_F16 && g.out_dtype != GLOWQ_OUT_F32) return GLOWQ_ERR_BAD_ARGUMENT;
#if !defined(GLOWQ_GEMV_TRACE) && !defined(GLOWQ_GEMM_TRACE)
  // reserved fields must be zero: a struct that was not cleared is refused instead of steering anything
  if (g.reserved != 0 || g.reserved2 != 0 || g.reserved3 != 0) return GLOWQ_ERR_BAD_ARGUMENT;
  for (int i = 0; i < g.n_members; ++i)
    if (g.members[i].reserved != 0) return GLOWQ_ERR_BAD_ARGUMENT;
#endif
  if (g.r_mode != GLOWQ_R_NONE && g.r_mode != GLOWQ_R_COMPUTE && g.r_mode != GLOWQ_R_LOAD) return GLOWQ_ERR_BAD_ARGUMENT;
  if (g.r_mode != GLOWQ_R_NONE) {
    if (g.rank <= 0 || !g.r_buf) return GLOWQ_ERR_BAD_ARGUMENT;
    if (g.rank > kMaxRTiles * kRTileRows) return GLOWQ_ERR_TOO_LARGE;
    if (g.r_mode == GLOWQ_R_COMPUTE && (!g.R || g.R_stride < g.IC)) return GLOWQ_ERR_BAD_ARGUMENT;
  }
  for (int i = 0; i < g.n_members; ++i) {
    const int rc = validate_member(g.members[i], g.IC, g.group_size);
    if (rc != GLOWQ_OK) return rc;
    if (g.r_mode != GLOWQ_R_NONE && g.members[i].L && g.members[i].L_stride < g.rank) return GLOWQ_ERR_BAD_STRIDE;
  }
  if (!g.workspace) return GLOWQ_ERR_BAD_ARGUMENT;
  if (g.norm_weight != nullptr) {
    if (g.M > kGemvMaxM || g.kernel == GLOWQ_KERNEL_GEMM || (g.IC & 7) || (g.x_stride & 7) || !aligned16(g.x) ||
        !aligned16(g.norm_weight) || !aligned16(g.residual) || !aligned16(g.hidden_out) || !(g.norm_eps >= 0.f))
      return GLOWQ_ERR_UNSUPPORTED_SHAPE;
  } else if (g.residual != nullptr || g.hidden_out != nullptr) {
    return GLOWQ_ERR_BAD_ARGUMENT;   // these belong to the fused norm
  }
  if (g.push != nullptr) {
    const glowq_w4a16_peers_t& pp = *g.push;
    if (pp.world < 1 || pp.world > GLOWQ_MAX_RANKS || pp.rank < 0 || pp.rank >= pp.world || !pp.epoch)
      return GLOWQ_ERR_BAD_ARGUMENT;
    for (int r = 0; r < pp.world; ++r)
      if (!pp.ll_buf[r]) return GLOWQ_ERR_BAD_ARGUMENT;
    const long long n = static_cast<long long>(g.M) * g.members[0].OC;
    if (g.n_members != 1 || g.out_dtype != GLOWQ_OUT_F16 || g.members[0].out_stride != g.members[0].OC ||
        g.M > kGemvMaxM || n > pp.max_n || (n & 7) || g.push_site < 0 || g.push_site >= pp.sites ||
        g.kernel == GLOWQ_KERNEL_GEMM)
      return GLOWQ_ERR_UNSUPPORTED_SHAPE;
  }
  return GLOWQ_OK;
}

// Layouts the streaming kernel takes: group of 128, complete groups physically present in each packed
// row, 16-byte aligned packed rows / L rows / R rows / r rows.
bool gemv_fast_ok(const glowq_w4a16_group_t& g) {
  if (g.group_size != kGroup) return false;
  const int G = ceil_div(g.IC, kGroup);
  for (int i = 0; i < g.n_members; ++i) {
    const auto& m = g.members[i];
    if (m.weight_stride_i32 < G * 16 || (m.weight_stride_i32 & 3) || !aligned16(m.qweight)) return false;
    if (g.r_mode != GLOWQ_R_NONE && m.L && (!aligned16(m.L) || (m.L_stride & 7))) return false;
  }
  if (g.r_mode != GLOWQ_R_NONE && ((g.rank & 7) || !aligned16(g.r_buf))) return false;
  if (g.r_mode == GLOWQ_R_COMPUTE && (!aligned16(g.R) || (g.R_stride & 7) || (g.IC & 7))) return false;
  return true;
}

int n_tiles_of(const glowq_w4a16_group_t& g) {
  int n = 0;
  for (int i = 0; i < g.n_members; ++i) n += ceil_div(g.members[i].OC, kTileRows);
  return n;
}

int gemv_group_forward(const glowq_w4a16_group_t& g, const DeviceInfo& dev, cudaStream_t stream) {
  const bool fast = gemv_fast_ok(g);
  const int n_tiles = n_tiles_of(g);
  for (int m0 = 0; m0 < g.M; m0 += kGemvMaxM) {
    const int Mc = std::min(kGemvMaxM, g.M - m0);
    const GemvPlan pl = make_plan(Mc, g.IC, n_tiles, g.r_mode != GLOWQ_R_NONE ? g.rank : 0, dev.sms, g.split_k);
    if (pl.total > g.workspace_bytes) return GLOWQ_ERR_WORKSPACE_TOO_SMALL;
    unsigned char* ws = static_cast<unsigned char*>(g.workspace);
    const __half* x = static_cast<const __half*>(g.x) + static_cast<size_t>(m0) * g.x_stride;
    __half* r_buf = g.r_buf ? static_cast<__half*>(g.r_buf) + static_cast<size_t>(m0) * g.rank : nullptr;
    const int esz = g.out_dtype == GLOWQ_OUT_F32 ? 4 : 2;

    GemvParams p{};
    p.x = x;
    p.R = static_cast<const __half*>(g.R);
    p.r_buf = r_buf;
    p.ws_head = reinterpret_cast<uint32_t*>(ws);
    p.tile_ctr = reinterpret_cast<uint32_t*>(ws + pl.off_tile_ctr);
    p.r_partial = reinterpret_cast<float*>(ws + pl.off_r_partial);
    p.r_ll = reinterpret_cast<uint2*>(ws + kWsRllOffset);
    p.sk_partial = reinterpret_cast<float*>(ws + pl.off_sk_partial);
    p.M = Mc;
    p.IC = g.IC;
    p.x_stride = g.x_stride;
    p.R_stride = g.R_stride;
    p.G = pl.G;
    p.rank = g.r_mode != GLOWQ_R_NONE ? g.rank : 0;
    p.r_mode = g.r_mode;
    p.out_fp32 = g.out_dtype == GLOWQ_OUT_F32;
    p.n_members = g.n_members;
    p.n_tiles = n_tiles;
    p.SK = pl.SK;
    p.gps = pl.gps;
    p.n_r_tiles = pl.n_r_tiles;
    p.SKr = pl.SKr;
    p.gpr = pl.gpr;
    p.n_r_units = g.r_mode == GLOWQ_R_COMPUTE ? pl.n_r_tiles * pl.SKr : 0;
    p.x_vec_ok = aligned16(x) && (g.x_stride % 8 == 0);
    p.xs_stride = pl.xs_stride;
    p.stages = pl.stages;
#ifdef GLOWQ_GEMV_TRACE
    static const int env_debug = env_int("GLOWQ_GEMV_DEBUG", 0);   // tuning builds only
    p.debug = g.reserved | env_debug;
#else
    p.debug = 0;
#endif
    p.meta_gp = pl.meta_gp;
    p.meta_gw = pl.meta_gw;
    int tb = 0;
    bool any_corr = false;
    for (int i = 0; i < g.n_members; ++i) {
      const auto& m = g.members[i];
      MemberDev& d = p.mem[i];
      d.qweight = m.qweight;
      d.scales = static_cast<const __half*>(m.scales);
      d.qzeros = m.qzeros;
      d.bias = static_cast<const __half*>(m.bias);
      d.L = g.r_mode != GLOWQ_R_NONE ? static_cast<const __half*>(m.L) : nullptr;
      d.out = static_cast<unsigned char*>(m.out) + static_cast<size_t>(m0) * m.out_stride * esz;
      d.OC = m.OC;
      d.wstride = m.weight_stride_i32;
      d.zstride = m.zero_stride_i32;
      d.sstride = m.scale_stride;
      d.Lstride = m.L_stride;
      d.out_stride = m.out_stride;
      d.alpha = m.alpha;
      d.tile_begin = tb;
      tb += ceil_div(m.OC, kTileRows);
      any_corr = any_corr || (d.L != nullptr && d.alpha != 0.f);
    }
    if (p.r_mode != GLOWQ_R_NONE && !any_corr && p.r_mode == GLOWQ_R_LOAD) p.r_mode = GLOWQ_R_NONE;

    p.norm_w = static_cast<const __half*>(g.norm_weight);
    p.residual = static_cast<const __half*>(g.residual);
    p.hidden_out = static_cast<__half*>(g.hidden_out);
    p.norm_eps = g.norm_eps;
    if (p.norm_w != nullptr && !fast) return GLOWQ_ERR_UNSUPPORTED_SHAPE;
    p.push_world = 0;
    if (g.push != nullptr) {
      if (!fast) return GLOWQ_ERR_UNSUPPORTED_SHAPE;   // the any-layout kernels do not push
      const glowq_w4a16_peers_t& pp = *g.push;
      p.push_world = pp.world;
      const size_t slot = (static_cast<size_t>(g.push_site) * pp.world + pp.rank) * pp.max_n;
      for (int r = 0; r < pp.world; ++r) p.push_slot[r] = static_cast<uint2*>(pp.ll_buf[r]) + slot;
      p.push_epoch = static_cast<uint32_t*>(pp.epoch) + g.push_site;
      p.push_local = static_cast<const uint2*>(pp.ll_buf[pp.rank]) + static_cast<size_t>(g.push_site) * pp.world * pp.max_n;
      p.push_max_n = pp.max_n;
      p.push_spin = allreduce_spin_limit();
    }

    cudaError_t e;
    if (fast) {
      if (pl.stages < 2 || gemv_smem_bytes(p, pl.NT) > kSmemOnePerSm) return GLOWQ_ERR_UNSUPPORTED_SHAPE;
      // persistent grid: every CTA resident at once, a whole number of CTAs per K slice
      // R units run on dedicated CTAs (the lowest block indices; several units each when there are many), so that the
      // r chain (R loads, MMAs, slot, release counter) overlaps the other CTAs' x staging and weight streaming
      static const int max_r_ctas = env_int("GLOWQ_GEMV_R_CTAS", 96);
      // (the epoch word of the workspace counts the consumer warps of a grid in kEpochShift bits)
      const int cap = std::min(dev.sms * pl.ctas_per_sm, static_cast<int>(kEpochReaderMask) / kConsumerWarps);
      {
        int want = std::min(p.n_r_units, max_r_ctas);
        if (pl.SK > 1) {
          // K slices: the R CTAs take no row tiles afterwards, so give them the CTA slots that do not add a round
          // of tiles to the slices (at least a few, or r would arrive long after the first tiles are done)
          const int rounds = ceil_div(n_tiles * pl.SK, cap);
          const int spare = cap - pl.SK * ceil_div(n_tiles, rounds);
          want = std::min(p.n_r_units, std::max(std::min(spare, max_r_ctas), std::min(max_r_ctas, 16)));
        }
        p.n_r_ctas = std::max(0, std::min(want, cap / 3));
      }
      int grid = std::min(cap - p.n_r_ctas, n_tiles * pl.SK);
      grid = std::max(pl.SK, grid / pl.SK * pl.SK) + p.n_r_ctas;
      p.l_cols = std::min(std::max(p.rank, 8), 256);
      alignas(64) TensorMaps tm;
      std::memset(&tm, 0, sizeof(tm));
      p.w_swizzled = (pl.G % 2 == 0) ? 1 : 0;
      for (int i = 0; i < g.n_members; ++i) {
        const MemberDev& d = p.mem[i];
        int rc = p.w_swizzled
                     ? tensor_map_w3d(&tm.w[i], d.qweight, static_cast<uint64_t>(pl.G / 2), d.OC,
                                      static_cast<uint64_t>(d.wstride) * 4)
                     : tensor_map_2d(&tm.w[i], CU_TENSOR_MAP_DATA_TYPE_INT32, d.qweight, static_cast<uint64_t>(pl.G) * 16,
                                     d.OC, static_cast<uint64_t>(d.wstride) * 4, kChunkGroups * 16, kTileRows);
        if (rc == GLOWQ_OK && d.L != nullptr && p.r_mode != GLOWQ_R_NONE)
          rc = tensor_map_2d(&tm.l[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, d.L, p.rank, d.OC,
                             static_cast<uint64_t>(d.Lstride) * 2, p.l_cols, kTileRows);
        if (rc != GLOWQ_OK) return rc;
      }
      // L2 prefetch requests for the call that follows on this stream: its right factor, then a prefix of its packed
      // rows in tile order (what its CTAs read first)
      // Defaults from the Llama-2-13B token step (ms, next-call megabytes / in-launch lookahead): 16/off 2.365,
      // 8/off 2.357, 16/on 2.369, 32/on 2.440, 64/on 2.590, 0/off 2.407 - more than the head of the next call evicts
      // what this one still needs, and the lookahead no longer pays on top of it.
      static const int pf_mb = env_int("GLOWQ_GEMV_PREFETCH_MB", 16);
      static const int deep_pf = env_int("GLOWQ_GEMV_DEEP_PREFETCH", 0);
      p.deep_prefetch = deep_pf;
      p.n_pf = 0;
      if (g.next != nullptr && pf_mb > 0 && m0 + kGemvMaxM >= g.M) {
        const glowq_w4a16_group_t& nx = *g.next;
        size_t budget = static_cast<size_t>(pf_mb) << 20;
        auto add = [&](const void* ptr, size_t bytes) {
          bytes = std::min(bytes, budget) & ~static_cast<size_t>(15);
          if (ptr != nullptr && aligned16(ptr) && bytes >= 16 && p.n_pf < kMaxPrefetch) {
            p.pf_ptr[p.n_pf] = static_cast<const unsigned char*>(ptr);
            p.pf_bytes[p.n_pf] = static_cast<unsigned>(bytes);
            ++p.n_pf;
            budget -= bytes;
          }
        };
        if (nx.IC > 0 && nx.n_members >= 1 && nx.n_members <= GLOWQ_MAX_MEMBERS) {
          if (nx.r_mode == GLOWQ_R_COMPUTE && nx.R != nullptr && nx.rank > 0 && nx.R_stride >= nx.IC)
            add(nx.R, (static_cast<size_t>(nx.rank - 1) * nx.R_stride + nx.IC) * 2);
          for (int i = 0; i < nx.n_members; ++i) {
            const auto& m = nx.members[i];
            if (m.OC > 0 && m.weight_stride_i32 >= ceil_div(nx.IC, 8))
              add(m.qweight, (static_cast<size_t>(m.OC - 1) * m.weight_stride_i32 + ceil_div(nx.IC, 8)) * 4);
          }
        }
      }
      e = launch_gemv_stream(p, tm, pl.NT, grid, stream);
      if (e != cudaSuccess) return fail_cuda(e);
    } else {
      float* r32 = nullptr;
      if (p.r_mode != GLOWQ_R_NONE) {
        r32 = reinterpret_cast<float*>(ws + pl.off_r32);
        e = launch_generic_r(x, p.R, r_buf, r32, p.r_mode, Mc, g.IC, p.rank, g.x_stride, g.R_stride, stream);
        if (e != cudaSuccess) return fail_cuda(e);
      }
      for (int i = 0; i < g.n_members; ++i) {
        e = launch_generic(x, p.mem[i], r32, p.out_fp32, Mc, g.IC, p.rank, g.group_size, g.x_stride, stream);
        if (e != cudaSuccess) return fail_cuda(e);
      }
    }
  }
  return GLOWQ_OK;
}

}  // namespace

extern "C" {

int glowq_w4a16_version(void) { return GLOWQ_W4A16_ABI_VERSION; }

const char* glowq_w4a16_strerror(int status) {
  switch (status) {
    case GLOWQ_OK: return "ok";
    case GLOWQ_ERR_BAD_ARGUMENT: return "bad argument (null pointer, size, or rank/mode mismatch)";
    case GLOWQ_ERR_BAD_GROUP_SIZE: return "group_size must be > 0 and a multiple of 8";
    case GLOWQ_ERR_BAD_STRIDE: return "packed columns / scales / zero words / output stride too small";
    case GLOWQ_ERR_WORKSPACE_TOO_SMALL: return "workspace too small (see glowq_w4a16_workspace_bytes)";
    case GLOWQ_ERR_UNSUPPORTED_DEVICE: return "unsupported device: this library runs on sm_100 (B200) only; there is no fallback";
    case GLOWQ_ERR_CUDA: return "CUDA runtime error (see glowq_w4a16_last_cuda_error)";
    case GLOWQ_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case GLOWQ_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
    case GLOWQ_ERR_TOO_LARGE: return "size beyond the supported maximum";
    default: return "unknown status";
  }
}

int glowq_w4a16_last_cuda_error(void) { return t_last_cuda_error; }

int glowq_w4a16_dequant(const int32_t* qweight, const void* scales, const int32_t* qzeros, void* out_w, int OC, int IC,
                        int group_size, int weight_stride_i32, int zero_stride_i32, int scale_stride, void* stream) {
  if (!qweight || !scales || !qzeros || !out_w || OC <= 0 || IC <= 0) return GLOWQ_ERR_BAD_ARGUMENT;
  if (group_size <= 0 || group_size % 8 != 0) return GLOWQ_ERR_BAD_GROUP_SIZE;
  const int G = ceil_div(IC, group_size);
  if (weight_stride_i32 < ceil_div(IC, 8) || scale_stride < G || zero_stride_i32 < ceil_div(G, 8)) return GLOWQ_ERR_BAD_STRIDE;
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != GLOWQ_OK) return rc;
  cudaError_t e = launch_dequant(qweight, static_cast<const __half*>(scales), qzeros, static_cast<__half*>(out_w), OC, IC,
                                 group_size, weight_stride_i32, zero_stride_i32, scale_stride,
                                 static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? GLOWQ_OK : fail_cuda(e);
}

size_t glowq_w4a16_workspace_bytes(int M, int IC, int OC_total, int rank, int n_members) {
  if (M <= 0 || IC <= 0 || OC_total <= 0) return kWsHeaderBytes;
  n_members = std::max(1, std::min(n_members, GLOWQ_MAX_MEMBERS));
  const int n_tiles = ceil_div(OC_total, kTileRows) + n_members;
  // planned for more SMs than any device has, which bounds the split-K partial-sum area from above
  const GemvPlan pl = make_plan(M, IC, n_tiles, rank, 1024, 0);
  size_t need = pl.total;
  need = std::max(need, gemm_workspace_bytes(M, IC, OC_total, rank, n_members));
  return align_up(need, 256);
}

int glowq_w4a16_group_forward(const glowq_w4a16_group_t* group) {
  if (!group) return GLOWQ_ERR_BAD_ARGUMENT;
  const glowq_w4a16_group_t& g = *group;
  int rc = validate_group(g);
  if (rc != GLOWQ_OK) return rc;
  const DeviceInfo* dev = nullptr;
  rc = device_info(&dev);
  if (rc != GLOWQ_OK) return rc;
  if (g.M == 0) return GLOWQ_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(g.stream);
  // Measured on B200: up to 8 tokens fit one streaming launch (one MMA N tile); 9..16 tokens would take two, and at
  // 16 tokens the tcgen05 GEMM (K-sliced over all SMs when it has few tiles) is ahead on every Llama-2-13B shape
  // (q/k/v 44 vs 47 us, gate/up 65 vs 70, down_proj 43 vs 64, o_proj 26 vs 33, corrected), so it takes over from 9.
  bool use_gemm = g.kernel == GLOWQ_KERNEL_GEMM;
  if (g.kernel == GLOWQ_KERNEL_AUTO) use_gemm = g.M > kGemvAutoMaxM;
  if (use_gemm && gemm_supported(g)) {
    cudaError_t ce = cudaSuccess;
    rc = gemm_group_forward(g, stream, &ce);
    if (rc == GLOWQ_ERR_CUDA) return fail_cuda(ce);
    return rc;
  }
  return gemv_group_forward(g, *dev, stream);
}

int glowq_w4a16_group_forward_many(const glowq_w4a16_group_t* groups, int n) {
  if (!groups || n < 0) return GLOWQ_ERR_BAD_ARGUMENT;
  for (int i = 0; i < n; ++i) {
    int rc;
    if (groups[i].next == nullptr && i + 1 < n) {   // the array successor is what follows on the stream
      glowq_w4a16_group_t g = groups[i];
      g.next = groups + i + 1;
      rc = glowq_w4a16_group_forward(&g);
    } else {
      rc = glowq_w4a16_group_forward(groups + i);
    }
    if (rc != GLOWQ_OK) return rc;
  }
  return GLOWQ_OK;
}

static void fill_plain(glowq_w4a16_group_t& g, const void* x, const int32_t* qweight, const void* scales,
                       const int32_t* qzeros, void* out, int M, int IC, int OC, int group_size, int wstride, int zstride,
                       int sstride, void* workspace, size_t workspace_bytes, void* stream) {
  std::memset(&g, 0, sizeof(g));
  g.x = x;
  g.workspace = workspace;
  g.workspace_bytes = workspace_bytes;
  g.stream = stream;
  g.M = M;
  g.IC = IC;
  g.x_stride = IC;
  g.group_size = group_size;
  g.r_mode = GLOWQ_R_NONE;
  g.out_dtype = GLOWQ_OUT_F16;
  g.n_members = 1;
  g.members[0].qweight = qweight;
  g.members[0].scales = scales;
  g.members[0].qzeros = qzeros;
  g.members[0].out = out;
  g.members[0].OC = OC;
  g.members[0].weight_stride_i32 = wstride;
  g.members[0].zero_stride_i32 = zstride;
  g.members[0].scale_stride = sstride;
  g.members[0].out_stride = OC;
}

int glowq_w4a16_gemv_forward(const void* x, const int32_t* qweight, const void* scales, const int32_t* qzeros, void* out,
                             int M, int IC, int OC, int group_size, int weight_stride_i32, int zero_stride_i32,
                             int scale_stride, void* workspace, size_t workspace_bytes, void* stream) {
  glowq_w4a16_group_t g;
  fill_plain(g, x, qweight, scales, qzeros, out, M, IC, OC, group_size, weight_stride_i32, zero_stride_i32, scale_stride,
             workspace, workspace_bytes, stream);
  g.kernel = GLOWQ_KERNEL_GEMV;
  return glowq_w4a16_group_forward(&g);
}

int glowq_w4a16_gemm_forward(const void* x, const int32_t* qweight, const void* scales, const int32_t* qzeros, void* out,
                             int M, int IC, int OC, int group_size, int split_k_iters, int weight_stride_i32,
                             int zero_stride_i32, int scale_stride, void* workspace, size_t workspace_bytes, void* stream) {
  (void)split_k_iters;
  glowq_w4a16_group_t g;
  fill_plain(g, x, qweight, scales, qzeros, out, M, IC, OC, group_size, weight_stride_i32, zero_stride_i32, scale_stride,
             workspace, workspace_bytes, stream);
  g.kernel = GLOWQ_KERNEL_GEMM;
  return glowq_w4a16_group_forward(&g);
}

}  // extern "C"

// ---------------------------------------------------------------- scratch that is part of the library image
// One array per device context, zero at load time.  Host code must not pass `g_static_scratch` itself to a
// kernel - in host code the name is only a handle for cudaGetSymbolAddress - so the device address is looked
// up once per device (with that device current) and cached.
static __device__ __align__(256) unsigned char g_static_scratch[GLOWQ_W4A16_STATIC_SCRATCH_BYTES];

namespace {
void* g_static_scratch_addr[64] = {};
std::mutex g_static_scratch_mutex;

int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e);
  if (dev < 0 || dev >= 64) return GLOWQ_ERR_UNSUPPORTED_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return fail_cuda(e);
    if (!ptr) return GLOWQ_ERR_CUDA;
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return GLOWQ_OK;
}
}  // namespace

extern "C" {

int glowq_w4a16_gemv_forward_static(const void* x, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                                    void* out, int M, int IC, int OC, int group_size, int weight_stride_i32,
                                    int zero_stride_i32, int scale_stride, void* stream) {
  if (M < 0 || IC <= 0 || OC <= 0) return GLOWQ_ERR_BAD_ARGUMENT;
  if (group_size <= 0 || group_size % 8 != 0) return GLOWQ_ERR_BAD_GROUP_SIZE;
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != GLOWQ_OK) return rc;
  // The scratch this launch would use, from the same planner the launch itself runs.
  const int n_tiles = ceil_div(OC, kTileRows);
  const GemvPlan pl = make_plan(std::max(M, 1), IC, n_tiles, 0, dev->sms, 0);
  if (pl.total > GLOWQ_W4A16_STATIC_SCRATCH_BYTES) return GLOWQ_ERR_TOO_LARGE;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != GLOWQ_OK) return rc;
  if (M == 0) return GLOWQ_OK;
  // Counters must start at zero whatever an earlier (possibly failed) call left behind; partial sums are
  // always written before they are read and need no clearing.  The status word is left alone: it keeps a
  // timeout of an earlier call until glowq_w4a16_read_status(NULL, stream) collects it.
  unsigned char* sc = static_cast<unsigned char*>(scratch);
  cudaError_t e = cudaMemsetAsync(sc, 0, WS_STATUS * 4, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess)
    e = cudaMemsetAsync(sc + (WS_STATUS + 1) * 4, 0, pl.off_r_partial - (WS_STATUS + 1) * 4, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e);
  glowq_w4a16_group_t g;
  fill_plain(g, x, qweight, scales, qzeros, out, M, IC, OC, group_size, weight_stride_i32, zero_stride_i32, scale_stride,
             scratch, GLOWQ_W4A16_STATIC_SCRATCH_BYTES, stream);
  g.kernel = GLOWQ_KERNEL_GEMV;
  return glowq_w4a16_group_forward(&g);
}

int glowq_w4a16_group_forward_host(const glowq_w4a16_group_t* group, const void* x_host, void* const* out_host) {
  if (!group || !x_host || !out_host) return GLOWQ_ERR_BAD_ARGUMENT;
  const glowq_w4a16_group_t& g = *group;
  int rc = validate_group(g);
  if (rc != GLOWQ_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(g.stream);
  cudaError_t e;
  if (g.M > 0) {
    e = cudaMemcpy2DAsync(const_cast<void*>(g.x), static_cast<size_t>(g.x_stride) * 2, x_host, static_cast<size_t>(g.IC) * 2,
                          static_cast<size_t>(g.IC) * 2, g.M, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail_cuda(e);
  }
  rc = glowq_w4a16_group_forward(group);
  if (rc != GLOWQ_OK) return rc;
  const size_t esz = g.out_dtype == GLOWQ_OUT_F32 ? 4 : 2;
  for (int i = 0; i < g.n_members && g.M > 0; ++i) {
    const auto& m = g.members[i];
    if (!out_host[i]) return GLOWQ_ERR_BAD_ARGUMENT;
    e = cudaMemcpy2DAsync(out_host[i], m.OC * esz, m.out, m.out_stride * esz, m.OC * esz, g.M, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return fail_cuda(e);
  }
  e = cudaStreamSynchronize(stream);
  return e == cudaSuccess ? GLOWQ_OK : fail_cuda(e);
}

int glowq_w4a16_read_status(void* workspace, void* stream) {
  if (!workspace) {  // the library-resident scratch of glowq_w4a16_gemv_forward_static on the current device
    const int rc = static_scratch_address(&workspace);
    if (rc != GLOWQ_OK) return rc;
  }
  uint32_t host = 0;
  uint32_t* word = static_cast<uint32_t*>(workspace) + WS_STATUS;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&host, word, 4, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(e);
  if (host != 0) {
    e = cudaMemsetAsync(word, 0, 4, s);
    if (e != cudaSuccess) return fail_cuda(e);
    return GLOWQ_ERR_DEVICE_TIMEOUT;
  }
  return GLOWQ_OK;
}

}  // extern "C"
