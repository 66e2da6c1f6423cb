// repack.cu -- one-time conversion of the reference's expert tensor layouts (hgn q4cp, hgn v2 i4r,
// GGUF Q4_K, Q5_K, Q5_1, Q8_0, IQ4_NL, IQ4_XS) into the tiled image described in common.cuh, and the inverse
// check: dequantising rows of the image bit-identically to the reference's row
// dequantisers (q4cp_row, src/hgn.h:249-261; dequant_row, src/gguf.h:360-374, 408-441).
#include "kernels.h"

namespace b200moe {

namespace {

// Source row of tile row r of (expert e, m-tile mt).
__device__ __forceinline__ long long src_row(const Image& img, const SrcTensor& a,
                                             const SrcTensor& b, int e, int mt, int r,
                                             const SrcTensor** which) {
  if (img.paired) {
    const SrcTensor& s = r < 64 ? a : b;
    *which = r < 64 ? &a : &b;
    return (long long)e * s.rows_per_expert + s.row_off + 64ll * mt + (r & 63);
  }
  *which = &a;
  return (long long)e * a.rows_per_expert + a.row_off + 128ll * mt + r;
}

// q4cp: pure movement of 16-byte chunks and fp16 scale pairs.
__global__ void k_repack_q4cp(Image img, SrcTensor a, SrcTensor b, int K, int first_expert,
                              const int32_t* __restrict__ emap) {
  const long long per_tile = 256 + 128;  // 256 code chunks + 128 scale pairs
  const long long total = (long long)img.n_experts * img.n_mtiles * img.n_kblocks * per_tile;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i / per_tile;
    int j = (int)(i % per_tile);
    int kb = (int)(t % img.n_kblocks);
    long long t2 = t / img.n_kblocks;
    int mt = (int)(t2 % img.n_mtiles);
    int e = (int)(t2 / img.n_mtiles);
    uint8_t* dst = const_cast<uint8_t*>(img.tile(e, mt, kb));
    const SrcTensor* s;
    if (j < 256) {
      int h = j >> 7, r = j & 127;
      long long row = src_row(img, a, b, emap ? emap[e + first_expert] : e + first_expert, mt, r, &s);
      const uint4* src = (const uint4*)(s->codes + row * (K / 2) + kb * 32 + h * 16);
      *(uint4*)(dst + h * 2048 + r * 16) = *src;
    } else {
      int r = j - 256;
      long long row = src_row(img, a, b, emap ? emap[e + first_expert] : e + first_expert, mt, r, &s);
      if (s->scale_group == 128) {
        // hgn v2 i4r: one fp16 scale per 128 columns serves both 32-groups of two K blocks
        const uint32_t v = *(const uint16_t*)(s->scales + row * s->scale_stride + (kb >> 1) * 2);
        *(uint32_t*)(dst + kCodeBytes + r * 4) = v | (v << 16);
      } else {
        const uint32_t* src = (const uint32_t*)(s->scales + row * s->scale_stride + kb * 4);
        *(uint32_t*)(dst + kCodeBytes + r * 4) = *src;
      }
    }
  }
}

__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* p, uint8_t& sc, uint8_t& mn) {
  if (j < 4) {
    sc = p[j] & 63;
    mn = p[j + 4] & 63;
  } else {
    sc = (uint8_t)((p[j + 4] & 15) | ((p[j - 4] >> 6) << 4));
    mn = (uint8_t)((p[j + 4] >> 4) | ((p[j] >> 6) << 4));
  }
}

// Q4_K: one thread per (tile, row). A 64-wide K block is half of a 128-element pair of
// sub-blocks: low nibbles of 32 bytes are K 0..31, high nibbles K 32..63 (src/gguf.h:408-441).
__global__ void k_repack_q4k(Image img, SrcTensor a, SrcTensor b, int K, int first_expert,
                             const int32_t* __restrict__ emap) {
  const long long total = (long long)img.n_experts * img.n_mtiles * img.n_kblocks * 128;
  const long long row_bytes = (long long)K / 256 * 144;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int r = (int)(i & 127);
    long long t = i >> 7;
    int kb = (int)(t % img.n_kblocks);
    long long t2 = t / img.n_kblocks;
    int mt = (int)(t2 % img.n_mtiles);
    int e = (int)(t2 / img.n_mtiles);
    uint8_t* dst = const_cast<uint8_t*>(img.tile(e, mt, kb));
    const SrcTensor* s;
    long long row = src_row(img, a, b, emap ? emap[e + first_expert] : e + first_expert, mt, r, &s);
    const uint8_t* blk = s->codes + row * row_bytes + (long long)(kb >> 2) * 144;
    const int sub = kb & 3;
    const uint8_t* ql = blk + 16 + 32 * sub;
    uint8_t lo[16], hi[16];
#pragma unroll
    for (int q = 0; q < 16; q++) {
      uint8_t c0 = ql[2 * q], c1 = ql[2 * q + 1];
      lo[q] = (uint8_t)((c0 & 15) | ((c1 & 15) << 4));
      hi[q] = (uint8_t)((c0 >> 4) | ((c1 >> 4) << 4));
    }
    *(uint4*)(dst + r * 16) = *(uint4*)lo;
    *(uint4*)(dst + 2048 + r * 16) = *(uint4*)hi;
    uint8_t s0, m0, s1, m1;
    k4_scale_min(2 * sub, blk + 4, s0, m0);
    k4_scale_min(2 * sub + 1, blk + 4, s1, m1);
    uint8_t* meta = dst + kCodeBytes + r * 8;
    meta[0] = blk[0];
    meta[1] = blk[1];
    meta[2] = blk[2];
    meta[3] = blk[3];
    meta[4] = s0;
    meta[5] = m0;
    meta[6] = s1;
    meta[7] = m1;
  }
}

// Q5_1: one thread per (tile, row, half). Element j of a block is the low nibble of qs[j],
// element j+16 the high nibble (src/gguf.h:360-374); the fifth bits follow their codes into the
// image's order and then take the split layout of common.cuh.
__global__ void k_repack_q51(Image img, SrcTensor a, SrcTensor b, int K, int first_expert,
                             const int32_t* __restrict__ emap) {
  const long long total = (long long)img.n_experts * img.n_mtiles * img.n_kblocks * 256;
  const long long row_bytes = (long long)K / 32 * 24;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int r = (int)(i & 127);
    int h = (int)((i >> 7) & 1);
    long long t = i >> 8;
    int kb = (int)(t % img.n_kblocks);
    long long t2 = t / img.n_kblocks;
    int mt = (int)(t2 % img.n_mtiles);
    int e = (int)(t2 / img.n_mtiles);
    uint8_t* dst = const_cast<uint8_t*>(img.tile(e, mt, kb));
    const SrcTensor* s;
    long long row = src_row(img, a, b, emap ? emap[e + first_expert] : e + first_expert, mt, r, &s);
    const uint8_t* blk = s->codes + row * row_bytes + (long long)(kb * 2 + h) * 24;
    const uint8_t* qs = blk + 8;
    uint8_t out[16];
#pragma unroll
    for (int q = 0; q < 8; q++) {
      out[q] = (uint8_t)((qs[2 * q] & 15) | ((qs[2 * q + 1] & 15) << 4));
      out[q + 8] = (uint8_t)((qs[2 * q] >> 4) | ((qs[2 * q + 1] >> 4) << 4));
    }
    *(uint4*)(dst + h * 2048 + r * 16) = *(uint4*)out;
    uint8_t* meta = dst + kCodeBytes + r * 16 + h * 8;
#pragma unroll
    for (int q = 0; q < 4; q++) meta[q] = blk[q];
    // the image keeps the block's element order (code byte i = elements 2i, 2i+1), and bit j of the
    // source word belongs to element j
    const uint32_t qh = (uint32_t)blk[4] | ((uint32_t)blk[5] << 8) | ((uint32_t)blk[6] << 16) | ((uint32_t)blk[7] << 24);
    *(uint32_t*)(meta + 4) = fifth_bits_split(qh);
  }
}

// Q5_K (gate/up) -> the image format of Q5_1, "w = d' * (q + 16 * fifth bit) + m'" per 32
// elements: d' = fp16(d * sc), m' = fp16(-(dmin * mn)) -- the constants the tensor-core path
// forms for Q4_K as well -- and the group's 32 fifth bits gathered from bit 2*sub+h of the 32
// qh bytes (src/gguf.h:408-441). One thread per (tile, row, half).
__global__ void k_repack_q5k(Image img, SrcTensor a, SrcTensor b, int K, int first_expert,
                             const int32_t* __restrict__ emap) {
  const long long total = (long long)img.n_experts * img.n_mtiles * img.n_kblocks * 256;
  const long long row_bytes = (long long)K / 256 * 176;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int r = (int)(i & 127);
    int h = (int)((i >> 7) & 1);
    long long t = i >> 8;
    int kb = (int)(t % img.n_kblocks);
    long long t2 = t / img.n_kblocks;
    int mt = (int)(t2 % img.n_mtiles);
    int e = (int)(t2 / img.n_mtiles);
    uint8_t* dst = const_cast<uint8_t*>(img.tile(e, mt, kb));
    const SrcTensor* s;
    long long row = src_row(img, a, b, emap ? emap[e + first_expert] : e + first_expert, mt, r, &s);
    const uint8_t* blk = s->codes + row * row_bytes + (long long)(kb >> 2) * 176;
    const int sub = kb & 3;
    const uint8_t* ql = blk + 48 + 32 * sub;
    const uint8_t* qh = blk + 16;
    uint8_t out[16];
    uint32_t fifth = 0;
#pragma unroll
    for (int q = 0; q < 16; q++) {
      const uint8_t c0 = ql[2 * q], c1 = ql[2 * q + 1];
      out[q] = h ? (uint8_t)((c0 >> 4) | ((c1 >> 4) << 4)) : (uint8_t)((c0 & 15) | ((c1 & 15) << 4));
    }
#pragma unroll
    for (int l = 0; l < 32; l++) fifth |= (uint32_t)((qh[l] >> (2 * sub + h)) & 1) << l;
    *(uint4*)(dst + h * 2048 + r * 16) = *(uint4*)out;
    uint8_t sc, mn;
    k4_scale_min(2 * sub + h, blk + 4, sc, mn);
    const float d = half_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    const float dmin = half_bits_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
    uint8_t* meta = dst + kCodeBytes + r * 16 + h * 8;
    *(__half*)meta = __float2half_rn(__fmul_rn(d, (float)sc));
    *(__half*)(meta + 2) = __float2half_rn(-__fmul_rn(dmin, (float)mn));
    *(uint32_t*)(meta + 4) = fifth_bits_split(fifth);
  }
}

// GGUF IQ4_NL / IQ4_XS -> the q4cp image: one thread per (tile, row, half). Both formats are
// "grid value x one scale per 32 elements" (src/gguf.h:375-406), which is what a q4cp tile
// holds; element j of a block is the low nibble of qs[j], element j+16 the high nibble. The
// image carries fp16(d * 256 [* (ls - 32)]) as the group's scale and the handle's code book is
// grid / 256 -- the reference's GPU kernel makes the same exact rescale to keep the scales out
// of the fp16 subnormal range (src/gpu/parts/27_kernels_moe_lut.inc:312-326).
template <bool XS>
__global__ void k_repack_iq4(Image img, SrcTensor a, SrcTensor b, int K, int first_expert,
                             const int32_t* __restrict__ emap) {
  const long long total = (long long)img.n_experts * img.n_mtiles * img.n_kblocks * 256;
  const long long row_bytes = XS ? (long long)K / 256 * 136 : (long long)K / 32 * 18;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int r = (int)(i & 127);
    int h = (int)((i >> 7) & 1);
    long long t = i >> 8;
    int kb = (int)(t % img.n_kblocks);
    long long t2 = t / img.n_kblocks;
    int mt = (int)(t2 % img.n_mtiles);
    int e = (int)(t2 / img.n_mtiles);
    uint8_t* dst = const_cast<uint8_t*>(img.tile(e, mt, kb));
    const SrcTensor* s;
    long long row = src_row(img, a, b, emap ? emap[e + first_expert] : e + first_expert, mt, r, &s);
    const int blk32 = kb * 2 + h;  // 32-element block of the row
    const uint8_t* blk;
    const uint8_t* qs;
    float scale;
    if (XS) {
      blk = s->codes + row * row_bytes + (long long)(blk32 >> 3) * 136;
      const int ib = blk32 & 7;
      const uint32_t sh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8);
      const int ls = (int)((blk[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15) | (int)(((sh >> (2 * ib)) & 3u) << 4);
      scale = (float)(ls - 32);
      qs = blk + 8 + 16 * ib;
    } else {
      blk = s->codes + row * row_bytes + (long long)blk32 * 18;
      scale = 1.f;
      qs = blk + 2;
    }
    const float d = half_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    scale = __fmul_rn(__fmul_rn(d, 256.f), scale);
    uint8_t out[16];
#pragma unroll
    for (int q = 0; q < 8; q++) {
      out[q] = (uint8_t)((qs[2 * q] & 15) | ((qs[2 * q + 1] & 15) << 4));
      out[q + 8] = (uint8_t)((qs[2 * q] >> 4) | ((qs[2 * q + 1] >> 4) << 4));
    }
    *(uint4*)(dst + h * 2048 + r * 16) = *(uint4*)out;
    ((__half*)(dst + kCodeBytes))[r * 2 + h] = __float2half_rn(scale);
  }
}

// GGUF Q8_0 -> the two-plane kQ51 image (common.cuh): one thread per (image tile, row, half).
// Image K block 2*kb holds the high nibbles of the biased codes of columns 64*kb .. 64*kb+63,
// image K block 2*kb+1 the low nibbles (34 bytes per 32 elements: fp16 d, 32 int8; src/gguf.h:352-359).
__global__ void k_repack_q80(Image img, SrcTensor a, SrcTensor b, int K, int first_expert,
                             const int32_t* __restrict__ emap) {
  const long long total = (long long)img.n_experts * img.n_mtiles * img.n_kblocks * 256;
  const long long row_bytes = (long long)K / 32 * 34;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int r = (int)(i & 127);
    int h = (int)((i >> 7) & 1);
    long long t = i >> 8;
    int kbi = (int)(t % img.n_kblocks);   // image K block: 2 * (activation K block) + plane
    long long t2 = t / img.n_kblocks;
    int mt = (int)(t2 % img.n_mtiles);
    int e = (int)(t2 / img.n_mtiles);
    const int kb = kbi >> 1, plane = kbi & 1;  // plane 0: high nibbles, 1: low nibbles
    uint8_t* dst = const_cast<uint8_t*>(img.tile(e, mt, kbi));
    const SrcTensor* s;
    long long row = src_row(img, a, b, emap ? emap[e + first_expert] : e + first_expert, mt, r, &s);
    const uint8_t* blk = s->codes + row * row_bytes + (long long)(kb * 2 + h) * 34;
    const int8_t* qs = (const int8_t*)(blk + 2);
    uint8_t out[16];
#pragma unroll
    for (int q = 0; q < 16; q++) {
      const int u0 = (int)qs[2 * q] + 128, u1 = (int)qs[2 * q + 1] + 128;
      out[q] = plane ? (uint8_t)((u0 & 15) | ((u1 & 15) << 4)) : (uint8_t)((u0 >> 4) | ((u1 >> 4) << 4));
    }
    *(uint4*)(dst + h * 2048 + r * 16) = *(uint4*)out;
    const float d = half_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    uint8_t* meta = dst + kCodeBytes + r * 16 + h * 8;
    *(__half*)meta = __float2half_rn(plane ? d : __fmul_rn(d, 16.f));
    *(__half*)(meta + 2) = __float2half_rn(plane ? 0.f : __fmul_rn(d, -128.f));
    *(uint32_t*)(meta + 4) = 0u;
  }
}

// Rows of an expert, dequantised from the image with the reference's exact operation
// order (single fp32 multiply for q4cp; multiply then add/subtract, never fused, for GGUF).
__global__ void k_dequant_rows(Image img, int expert, int row0, int nrows, int mid_rows,
                               float* out) {
  const int K = (img.n_kblocks >> img.act_shift) * kTileK;
  const long long total = (long long)nrows * K;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int c = (int)(i % K);
    int row = row0 + (int)(i / K);
    int mt, r;
    if (img.paired) {
      if (row < mid_rows) {
        mt = row / 64;
        r = row % 64;
      } else {
        mt = (row - mid_rows) / 64;
        r = 64 + (row - mid_rows) % 64;
      }
    } else {
      mt = row / 128;
      r = row % 128;
    }
    int kb = c / 64, h = (c / 32) & 1, j = c & 31;
    if (img.act_shift) {
      // Q8_0 in two planes: put the code together again and multiply once, as the reference
      // does (y = d * q, src/gguf.h:352-359)
      const uint8_t* hi = img.tile(expert, mt, 2 * kb);
      const uint8_t* lo = img.tile(expert, mt, 2 * kb + 1);
      const uint8_t bh = hi[h * 2048 + r * 16 + j / 2], bl = lo[h * 2048 + r * 16 + j / 2];
      const int q = 16 * ((j & 1) ? (bh >> 4) : (bh & 15)) + ((j & 1) ? (bl >> 4) : (bl & 15)) - 128;
      const float d = half_bits_to_f32(*(const uint16_t*)(lo + kCodeBytes + r * 16 + h * 8));
      out[i] = __fmul_rn(d, (float)q);
      continue;
    }
    const uint8_t* tile = img.tile(expert, mt, kb);
    uint8_t byte = tile[h * 2048 + r * 16 + j / 2];
    int nib = (j & 1) ? (byte >> 4) : (byte & 15);
    const uint8_t* meta = tile + kCodeBytes;
    float v;
    if (img.fmt == kQ4CP) {
      float s = half_bits_to_f32(((const uint16_t*)meta)[r * 2 + h]);
      v = __fmul_rn(img.book[(r >= 64 ? 16 : 0) + nib], s);
    } else if (img.fmt == kQ4K) {
      const uint8_t* m = meta + r * 8;
      float d = half_bits_to_f32(*(const uint16_t*)m);
      float dmin = half_bits_to_f32(*(const uint16_t*)(m + 2));
      float d1 = __fmul_rn(d, (float)m[4 + 2 * h]);
      float dm1 = __fmul_rn(dmin, (float)m[5 + 2 * h]);
      v = __fsub_rn(__fmul_rn(d1, (float)nib), dm1);
    } else {
      const uint8_t* m = meta + r * 16 + h * 8;
      float d = half_bits_to_f32(*(const uint16_t*)m);
      float mn = half_bits_to_f32(*(const uint16_t*)(m + 2));
      uint32_t qh = *(const uint32_t*)(m + 4);
      int x = nib | (int)(fifth_bit_of(qh, j) << 4);
      v = __fadd_rn(__fmul_rn((float)x, d), mn);
    }
    out[i] = v;
  }
}

}  // namespace

cudaError_t launch_repack(const Image& img, const SrcTensor& a, const SrcTensor& b, int K,
                          int first_expert, cudaStream_t st, const int32_t* expert_map, int gguf_type) {
  const int threads = 256;
  const int blocks = 148 * 8;
  if (img.fmt == kQ4CP && gguf_type == 20) k_repack_iq4<false><<<blocks, threads, 0, st>>>(img, a, b, K, first_expert, expert_map);
  else if (img.fmt == kQ4CP && gguf_type == 23) k_repack_iq4<true><<<blocks, threads, 0, st>>>(img, a, b, K, first_expert, expert_map);
  else if (img.fmt == kQ4CP) k_repack_q4cp<<<blocks, threads, 0, st>>>(img, a, b, K, first_expert, expert_map);
  else if (img.fmt == kQ4K) k_repack_q4k<<<blocks, threads, 0, st>>>(img, a, b, K, first_expert, expert_map);
  else if (gguf_type == 13) k_repack_q5k<<<blocks, threads, 0, st>>>(img, a, b, K, first_expert, expert_map);
  else if (gguf_type == 8) k_repack_q80<<<blocks, threads, 0, st>>>(img, a, b, K, first_expert, expert_map);
  else k_repack_q51<<<blocks, threads, 0, st>>>(img, a, b, K, first_expert, expert_map);
  return cudaGetLastError();
}

cudaError_t launch_dequant_rows(const Image& img, int expert, int row0, int nrows, int mid_rows,
                                float* out, cudaStream_t st) {
  long long total = (long long)nrows * img.n_kblocks * kTileK;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  k_dequant_rows<<<blocks, 256, 0, st>>>(img, expert, row0, nrows, mid_rows, out);
  return cudaGetLastError();
}

}  // namespace b200moe
