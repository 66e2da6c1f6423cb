// common.cuh -- shared definitions of the B200 MoE operator (tile geometry, device
// helpers, internal structs). Host and device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

// ---- repacked weight tiles --------------------------------------------------------
// Every quantised expert tensor is stored as tiles of 128 output rows x 64 K-elements:
//   [expert][m_tile][k_block][tile bytes]
// A tile starts with 4096 code bytes laid out [half h=0..1][row r=0..127][16 B]: the 16
// bytes hold the 32 four-bit codes of row r for K = 64*kb + 32*h .. +31, low nibble =
// even K (the nibble order of hgn q4cp, src/hgn.h:5-9 of the reference). The codes are
// followed by per-(row, 32-group) metadata whose size depends on the source format.
// A whole tile is one contiguous, 16-byte aligned object so that a single bulk async
// copy brings it into shared memory, and a warp reading "its" rows touches 512
// contiguous bytes.
constexpr int kTileM = 128;
constexpr int kTileK = 64;
constexpr int kCodeBytes = kTileM * kTileK / 2;  // 4096

enum Format : int {
  kQ4CP = 0,  // meta: [r][2] fp16 scale                                   -> 512 B
  kQ4K = 1,   // meta: [r]{fp16 d, fp16 dmin, u8 sc0, u8 m0, u8 sc1, u8 m1} -> 1024 B
  kQ51 = 2    // meta: [r][2]{fp16 d, fp16 m, u32 high bits}                -> 2048 B
};
// GGUF Q8_0 (int8 codes q, fp16 d per 32: w = d * q) has no tile layout of its own. With the
// biased code u = q + 128 = 16 * hi + lo the weight is d * (16 * hi - 128) + d * lo: two 4-bit
// tensors over the SAME activations. The image is kQ51 with twice the K blocks -- for every 64
// columns a block of the high nibbles (group constants d' = 16 d, m' = -128 d, no fifth bits)
// followed by a block of the low nibbles (d' = d, m' = 0) -- and act_shift = 1. 16 d and 128 d are
// exact in fp16, so every kernel reproduces d * q up to its usual single rounding.

__host__ __device__ constexpr int meta_bytes(int fmt) {
  return fmt == kQ4CP ? 512 : fmt == kQ4K ? 1024 : 2048;
}
__host__ __device__ constexpr int tile_bytes(int fmt) { return kCodeBytes + meta_bytes(fmt); }

// One repacked tensor set: n_experts x n_mtiles x n_kblocks tiles.
struct Image {
  uint8_t* data = nullptr;
  int fmt = kQ4CP;
  int n_experts = 0;
  int n_mtiles = 0;   // per expert
  int n_kblocks = 0;  // K / 64
  int paired = 0;     // 1: gate/up image (tile rows 0..63 gate, 64..127 the matching up rows)
  int dual_book = 0;  // 1: the two halves of a tile use different code books (separate gate / up tensors)
  int act_shift = 0;  // 1: two-plane image of 8-bit codes (GGUF Q8_0): K block kb of the image multiplies the
                      //    activations of K block kb >> 1 -- the high and the low nibble plane of the same 64 columns
  float* book = nullptr;  // device [32]: code book of tile rows 0..63, then of rows 64..127
  __host__ __device__ size_t tile_stride() const { return (size_t)tile_bytes(fmt); }
  __host__ __device__ size_t expert_stride() const {
    return (size_t)n_mtiles * n_kblocks * tile_bytes(fmt);
  }
  __host__ __device__ const uint8_t* tile(int e, int mt, int kb) const {
    return data + ((size_t)e * n_mtiles + mt) * n_kblocks * tile_bytes(fmt) +
           (size_t)kb * tile_bytes(fmt);
  }
};

// A run of permuted rows that belong to one expert (the unit the expert kernels work on).
struct Run {
  int expert;
  int first;
  int count;
};

// Work item of the grouped GEMM: at most 256 rows of one expert.
struct Tile {
  int expert;
  int first;
  int count;
};

constexpr int kMaxTopK = 16;
constexpr int kMaxExperts = 512;
constexpr int kIdStride = 16;  // internal top-k rows are 16 wide, like the engine's

// ---- device helpers ----------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
  return __uint_as_float((uint32_t)b << 16);
}
__device__ __forceinline__ float half_bits_to_f32(uint16_t h) {
  return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ float silu_f32(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f32(float v) { return 1.f / (1.f + expf(-v)); }

}  // namespace b200moe
