// Launch descriptors passed by value to the kernels, and the workspace layout.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glowq {

constexpr int kMaxMembers = 4;
constexpr int kTileRows = 16;      // output rows per CTA of the weight-streaming kernel (one MMA M tile)
constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kGroup = 128;        // quantisation group of the fast paths
constexpr unsigned kSpinLimit = 1u << 21;  // bounded device-side waits (x >= 200 ns each)

// Workspace header (uint32 words); the rest of the workspace follows at kWsHeaderBytes.
enum : int { WS_TICKET = 0, WS_R_DONE = 1, WS_EXIT = 2, WS_STATUS = 3, WS_HEADER_WORDS = 64 };
constexpr size_t kWsHeaderBytes = WS_HEADER_WORDS * 4;
constexpr int kMaxRTiles = 64;     // rank <= 1024

struct MemberDev {
  const int32_t* qweight;
  const __half* scales;
  const int32_t* qzeros;
  const __half* bias;
  const __half* L;
  void* out;
  int OC, wstride, zstride, sstride, Lstride, out_stride;
  float alpha;
  int tile_begin;   // index of this member's first 16-row tile in the group's tile list
};

struct GemvParams {
  const __half* x;
  const __half* R;
  __half* r_buf;
  uint32_t* ws_head;      // header words
  uint32_t* r_tile_ctr;   // [n_r_tiles] arrival counters of the r partial sums
  float* r_partial;       // [n_r_tiles][SKr][16][Mpad]
  uint32_t* tile_ctr;     // [n_tiles] arrival counters of the split-K partial sums
  float* sk_partial;      // [n_tiles][SK][16][Mpad]
  int M, IC, x_stride, R_stride, G, rank, r_mode, out_fp32, n_members;
  int n_tiles, SK, gps;          // main work: tiles x K slices, groups per slice
  int n_r_tiles, SKr, gps_r;     // r work
  int n_r_units;                 // n_r_tiles * SKr (0 unless r_mode == COMPUTE)
  int x_vec_ok;                  // x rows are 16-byte aligned
  int xs_stride;                 // bytes between tokens of the staged x slice in shared memory
  MemberDev mem[kMaxMembers];
};

}  // namespace glowq
