// Launch descriptors passed by value to the kernels, and the workspace layout.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glowq {

constexpr int kMaxMembers = 4;
constexpr int kRowTiles = 2;        // MMA M tiles (16 rows) per work item of the weight-streaming kernel
constexpr int kTileRows = 16 * kRowTiles;  // output rows per work item
constexpr int kRTileRows = 16;      // rows of R per R unit
constexpr int kConsumerWarps = 8;   // warps that dequantise + MMA; warp w takes group w of every chunk
constexpr int kGemvThreads = (kConsumerWarps + 2) * 32;  // + weight-copy warp + metadata warp
constexpr int kGroup = 128;         // quantisation group of the fast paths
constexpr int kChunkGroups = 8;     // groups per pipeline stage: 1024 input columns = 512 packed bytes per row
constexpr int kRowPitch = kChunkGroups * 64;  // stage row pitch in shared memory: the dense box a 2-D TMA copy writes
constexpr int kStageBytes = kTileRows * kRowPitch;
constexpr int kMetaDepth = 2;       // tiles of raw scale / zero-point metadata in flight
constexpr int kMaxStages = 8;
constexpr unsigned kSpinLimit = 1u << 18;  // bound of every device-side wait loop

constexpr int kCookedDepth = 2;     // tiles of converted (fp32) scale / zero-point pairs ahead of the consumers
constexpr int kZeroRowBytes = 320;  // all-zero activation row for the token slots of an MMA that hold no token

// Dynamic shared memory of one CTA of the weight-streaming kernel (the kernel's carve-up follows this order):
// barriers | weight ring | raw metadata ring | converted metadata ring | reduction buffers | R-unit scratch |
// x sums | staged x | zero row.
inline size_t gemv_smem_layout_bytes(int stages, int meta_gp, int meta_gw, int gps, int NT, int M, int xs_stride) {
  size_t off = 256 + 1024;   // barriers, then up to 1 KB of padding: the weight ring starts on a 1024-byte boundary
  off += static_cast<size_t>(stages) * kStageBytes;
  off += static_cast<size_t>(kMetaDepth) * kTileRows * (meta_gp * 2 + meta_gw * 4);
  off += static_cast<size_t>(kCookedDepth) * gps * (kTileRows * 8);
  off += static_cast<size_t>(kConsumerWarps) * kRowTiles * NT * 512 + static_cast<size_t>(NT) * 512;
  off += static_cast<size_t>(gps) * NT * 32;
  off += static_cast<size_t>(M) * xs_stride;
  off += kZeroRowBytes;
  return off;
}

// Workspace header (uint32 words); the rest of the workspace follows at kWsHeaderBytes.
enum : int { WS_TICKET = 0, WS_R_DONE = 1, WS_EXIT = 2, WS_STATUS = 3, WS_EPOCH = 4, WS_HEADER_WORDS = 64 };
// WS_EPOCH packs {launch epoch : 20 bits, readers : 12 bits}: every consumer warp of a correcting launch adds 1 when it
// is past the wait for the previous kernels and takes the epoch from the value the add returns; the CTA that completes
// r advances the epoch (and clears the readers) once all warps of the grid have registered.
constexpr int kEpochShift = 12;
constexpr uint32_t kEpochReaderMask = (1u << kEpochShift) - 1u;
constexpr uint32_t kEpochMask = (1u << 20) - 1u;
constexpr size_t kWsHeaderBytes = WS_HEADER_WORDS * 4;
constexpr int kMaxRTiles = 64;      // rank <= 1024
// After the header: 1 KB of arrival counters for the stand-alone r product, then r of the running launch as the row tiles read it - 8-byte words
// {half2(r[tok][2j], r[tok][2j+1]), launch epoch}, up to 8 tokens x rank 1024 - then the tile counters.  Launches of
// the other kernels keep clear of everything up to the end of the tile counters.
constexpr int kRpCtrWords = 256;    // arrival counters of the stand-alone r product (rank / 16 x token blocks of 64)
constexpr size_t kWsRllOffset = kWsHeaderBytes + kRpCtrWords * 4;
constexpr size_t kWsRllBytes = 8 * 1024 * 4;
constexpr size_t kWsTileCtrOffset = kWsRllOffset + kWsRllBytes;
constexpr int kMaxPrefetch = kMaxMembers + 1;
constexpr int kMaxRanks = 8;        // GLOWQ_MAX_RANKS
constexpr unsigned kPrefetchSlice = 16u << 10;  // bytes per L2 prefetch request

struct MemberDev {
  const int32_t* qweight;
  const __half* scales;
  const int32_t* qzeros;
  const __half* bias;
  const __half* L;
  void* out;
  int OC, wstride, zstride, sstride, Lstride, out_stride;
  float alpha;
  int tile_begin;   // index of this member's first row tile (kTileRows rows) in the group's tile list
};

// TMA descriptors of every member's packed weight ([OC][G/2][32] int32, box kTileRows x kChunkGroups/2 x 32, shared-memory
// image swizzled within 128 bytes; or [OC][G*16] with box kTileRows x kChunkGroups*16 for an odd group count) and left factor ([OC, rank] fp16, box kTileRows x l_cols).  Rows, groups or columns
// of a box that fall outside the tensor read as zero.
struct alignas(64) TensorMaps {
  CUtensorMap w[kMaxMembers];
  CUtensorMap l[kMaxMembers];
};

struct GemvParams {
  const __half* x;
  const __half* R;
  __half* r_buf;
  uint32_t* ws_head;      // header words
  float* r_partial;       // [n_r_tiles][SKr][NT*128] fp32 partial products of r, one slot per R unit
  uint2* r_ll;            // [M][rank/2] words {two fp16 elements of r, launch epoch}: written by the CTA that completes r
  uint32_t* tile_ctr;     // [n_tiles] arrival counters of the split-K partial sums
  float* sk_partial;      // [n_tiles][SK][kRowTiles*NT*128]
  int M, IC, x_stride, R_stride, G, rank, r_mode, out_fp32, n_members;
  int n_tiles, SK, gps;          // main work: tiles x K slices, groups per slice (multiple of kChunkGroups)
  int n_r_tiles, SKr, gpr;       // r work: 16-row tiles of R x SKr K slices of gpr groups each
  int n_r_units;                 // n_r_tiles * SKr (0 unless r_mode == COMPUTE)
  int n_r_ctas;                  // CTAs (the lowest block indices) that run the R units before any row tile
  int x_vec_ok;                  // x rows are 16-byte aligned
  int xs_stride;                 // bytes between tokens of the staged x slice in shared memory
  int stages;                    // weight ring depth
  int debug;                     // tuning experiments only (0 in production)
  int l_cols;                    // columns of L per pipeline stage: min(rank, 256)
  int meta_gp, meta_gw;          // per-row metadata pitch: scale halves, zero words (of one K slice)
  int deep_prefetch;             // the copy warp also asks L2 for the chunk that follows S issues later
  int w_swizzled;                // weight stages arrive swizzled (3-D tensor map, even group count) or as plain rows
  // Byte ranges of the group call that follows on the stream (a prefix of its packed rows in tile order, its right
  // factor): every CTA's copy warp asks L2 for its share once its own copies are issued, so that HBM keeps streaming
  // through this launch's tail and the next launch's prologue.
  int n_pf;
  const unsigned char* pf_ptr[kMaxPrefetch];
  unsigned pf_bytes[kMaxPrefetch];
  // fused residual add + RMSNorm of the activations (norm_w == nullptr: none)
  const __half* norm_w;
  const __half* residual;
  __half* hidden_out;
  float norm_eps;
  // Tensor-parallel push (row-split linears): push_slot[r] = rank r's staging slot for THIS rank's partial result
  // ([M][OC] 8-byte words {fp16 value, epoch}), push_epoch = local call counter of the site.  The last CTAs to finish
  // their tiles poll the local word buffer and write the sum over the ranks to the output.  push_world == 0: none.
  int push_world;
  uint2* push_slot[kMaxRanks];
  uint32_t* push_epoch;
  const uint2* push_local;       // this rank's word buffer of the site: [world][push_max_n]
  int push_max_n;
  unsigned push_spin;            // polls of one word before the launch gives up (status 4)
  MemberDev mem[kMaxMembers];
};

}  // namespace glowq
