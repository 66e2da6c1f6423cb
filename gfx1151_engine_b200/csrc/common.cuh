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
  kQ4CP = 0,  // meta: [r]{fp16 scale of half 0, of half 1}                          -> 512 B
  kQ4K = 1,   // meta: [r]{fp16 d, fp16 dmin, u8 sc0, u8 m0, u8 sc1, u8 m1}           -> 1024 B
  kQ51 = 2    // meta: [r]{fp16 d0, fp16 m0, u32 fifth bits 0, fp16 d1, fp16 m1, u32 fifth bits 1} -> 2048 B
};
// kQ51, the fifth-bit word of a 32-group: bit i (i < 16) belongs to the LOW-nibble code of code
// byte i (element 2i of the group), bit 16 + i to its high-nibble code (element 2i + 1). With the
// two bits of a code byte 16 apart, one shift and one mask move them to bits 14 and 30 -- the
// fp16 pair (2.0 or 0, 2.0 or 0) -- and a single half2 multiply-add by 8 adds the 16s to the two
// looked-up codes.
__host__ __device__ inline uint32_t fifth_bits_split(uint32_t by_element) {  // bit j = element j  ->  the layout above
  uint32_t r = 0;
  for (int i = 0; i < 16; i++)
    r |= (((by_element >> (2 * i)) & 1u) << i) | (((by_element >> (2 * i + 1)) & 1u) << (16 + i));
  return r;
}
__host__ __device__ inline uint32_t fifth_bit_of(uint32_t split, int j) {  // fifth bit of element j of the group
  return (split >> ((j & 1) ? 16 + (j >> 1) : (j >> 1))) & 1u;
}
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
