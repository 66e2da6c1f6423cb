// expert_simt.cu -- expert FFN on the CUDA cores: fp32 weights dequantised exactly as the
// reference does, fp32 FMA accumulation. This is the decode / speculative-verify path
// (T <= 16; takes the place of k_q4cp_gemv_gg, k_silu_mul_g and k_q4cp_gemv_gd,
// src/gpu/parts/20_kernels_gemv.inc:1607-1764, and of the GGUF raw-block GEMV,
// src/gpu/parts/26_kernels_moe_gguf.inc:487-939) and, at any T, the slow exact path the
// tensor-core kernels are cross-checked against.
//
// Work decomposition: one block of 128 threads per (run of rows of one expert, m-tile);
// thread r owns output row r of the tile and streams that row's codes, 16 bytes per
// load, 512 contiguous bytes per warp. Rows of the run are processed NT at a time with
// their activations staged in shared memory (every thread reads the same activation
// address: a broadcast).
#include "kernels.h"

namespace b200moe {

namespace {

constexpr int kNT = 8;        // rows (tokens) per pass
constexpr int kPiece = 1024;  // K elements of activations staged at a time

template <int FMT>
struct RowMeta {};

// Per (row, 32-group) dequantisation constants, and the fp32 value of one code.
template <>
struct RowMeta<kQ4CP> {
  float s;
  const float* book;
  __device__ __forceinline__ void load(const uint8_t* meta, int r, int h, const float* bk) {
    s = half_bits_to_f32(((const uint16_t*)meta)[r * 2 + h]);
    book = bk;
  }
  __device__ __forceinline__ float value(int nib, int) const { return __fmul_rn(book[nib], s); }
};
template <>
struct RowMeta<kQ4K> {
  float d1, dm1;
  __device__ __forceinline__ void load(const uint8_t* meta, int r, int h, const float*) {
    const uint8_t* m = meta + r * 8;
    float d = half_bits_to_f32(*(const uint16_t*)m), dmin = half_bits_to_f32(*(const uint16_t*)(m + 2));
    d1 = __fmul_rn(d, (float)m[4 + 2 * h]);
    dm1 = __fmul_rn(dmin, (float)m[5 + 2 * h]);
  }
  __device__ __forceinline__ float value(int nib, int) const {
    return __fsub_rn(__fmul_rn(d1, (float)nib), dm1);
  }
};
template <>
struct RowMeta<kQ51> {
  float d, m;
  uint32_t qh;
  __device__ __forceinline__ void load(const uint8_t* meta, int r, int h, const float*) {
    const uint8_t* p = meta + r * 16 + h * 8;
    d = half_bits_to_f32(*(const uint16_t*)p);
    m = half_bits_to_f32(*(const uint16_t*)(p + 2));
    qh = *(const uint32_t*)(p + 4);
  }
  __device__ __forceinline__ float value(int nib, int j) const {
    int x = nib | (int)(fifth_bit_of(qh, j) << 4);
    return __fadd_rn(__fmul_rn((float)x, d), m);
  }
};

// acc[j] += sum over the K range [k0, k0+klen) of w[r][k] * xs[j][k - k0]
template <int FMT>
__device__ __forceinline__ void row_dot(const Image& img, int e, int mt, int r, int k0, int klen,
                                        const float* book, const float (*xs)[kPiece], int nt,
                                        float* acc) {
  // (a two-plane image of 8-bit codes has 1 << act_shift image K blocks per activation K block)
  for (int kbi = (k0 / kTileK) << img.act_shift; kbi < ((k0 + klen) / kTileK) << img.act_shift; kbi++) {
    const int kb = kbi >> img.act_shift;
    const uint8_t* tile = img.tile(e, mt, kbi);
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint4 c4 = *(const uint4*)(tile + h * 2048 + r * 16);
      RowMeta<FMT> rm;
      rm.load(tile + kCodeBytes, r, h, book);
      const uint32_t wds[4] = {c4.x, c4.y, c4.z, c4.w};
      const int xo = kb * kTileK - k0 + h * 32;
#pragma unroll
      for (int q = 0; q < 4; q++) {
#pragma unroll
        for (int n = 0; n < 8; n++) {
          const int j = q * 8 + n;
          const float w = rm.value((wds[q] >> (4 * n)) & 15, j);
#pragma unroll
          for (int t = 0; t < kNT; t++)
            if (t < nt) acc[t] = fmaf(w, xs[t][xo + j], acc[t]);
        }
      }
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__(128)
k_up_simt(Image img, const uint16_t* __restrict__ x, int d, int mid,
          const int32_t* __restrict__ tokidx, const Run* __restrict__ runs,
          const int32_t* __restrict__ n_runs, float* __restrict__ hid) {
  if ((int)blockIdx.y >= *n_runs) return;
  __shared__ float xs[kNT][kPiece];
  __shared__ float us[kNT][64];
  __shared__ float book_s[32];
  const Run run = runs[blockIdx.y];
  const int mt = blockIdx.x, r = threadIdx.x;
  if (r < 32) book_s[r] = img.book ? img.book[r] : 0.f;
  const float* book = book_s + (r >= 64 ? 16 : 0);
  for (int c0 = 0; c0 < run.count; c0 += kNT) {
    const int nt = min(kNT, run.count - c0);
    float acc[kNT];
#pragma unroll
    for (int t = 0; t < kNT; t++) acc[t] = 0.f;
    for (int k0 = 0; k0 < d; k0 += kPiece) {
      const int klen = min(kPiece, d - k0);
      __syncthreads();
      for (int t = 0; t < nt; t++) {
        const uint16_t* row = x + (size_t)tokidx[run.first + c0 + t] * d + k0;
        for (int i = r; i < klen; i += 128) xs[t][i] = bf16_bits_to_f32(row[i]);
      }
      __syncthreads();
      row_dot<FMT>(img, run.expert, mt, r, k0, klen, book, xs, nt, acc);
    }
    __syncthreads();
    if (r >= 64)
      for (int t = 0; t < nt; t++) us[t][r - 64] = acc[t];
    __syncthreads();
    if (r < 64)
      for (int t = 0; t < nt; t++)
        hid[(size_t)(run.first + c0 + t) * mid + mt * 64 + r] = silu_f32(acc[t]) * us[t][r];
  }
}

template <int FMT>
__global__ void __launch_bounds__(128)
k_down_simt(Image img, const float* __restrict__ hid, int d, int mid, const Run* __restrict__ runs,
            const int32_t* __restrict__ n_runs, float* __restrict__ pairs) {
  if ((int)blockIdx.y >= *n_runs) return;
  __shared__ float xs[kNT][kPiece];
  __shared__ float book_s[32];
  const Run run = runs[blockIdx.y];
  const int mt = blockIdx.x, r = threadIdx.x;
  if (r < 32) book_s[r] = img.book ? img.book[r] : 0.f;
  const float* book = book_s + (r >= 64 ? 16 : 0);
  for (int c0 = 0; c0 < run.count; c0 += kNT) {
    const int nt = min(kNT, run.count - c0);
    float acc[kNT];
#pragma unroll
    for (int t = 0; t < kNT; t++) acc[t] = 0.f;
    for (int k0 = 0; k0 < mid; k0 += kPiece) {
      const int klen = min(kPiece, mid - k0);
      __syncthreads();
      for (int t = 0; t < nt; t++) {
        const float* row = hid + (size_t)(run.first + c0 + t) * mid + k0;
        for (int i = r; i < klen; i += 128) xs[t][i] = row[i];
      }
      __syncthreads();
      row_dot<FMT>(img, run.expert, mt, r, k0, klen, book, xs, nt, acc);
    }
    for (int t = 0; t < nt; t++) pairs[(size_t)(run.first + c0 + t) * d + mt * 128 + r] = acc[t];
  }
}

}  // namespace

cudaError_t launch_up_simt(const Image& img, const void* x_bf16, int d, int mid,
                           const int32_t* tokidx, const Run* runs, const int32_t* n_runs,
                           int max_runs, float* hid_f32, cudaStream_t st) {
  dim3 grid(img.n_mtiles, max_runs);
  const uint16_t* x = (const uint16_t*)x_bf16;
  if (img.fmt == kQ4CP)
    k_up_simt<kQ4CP><<<grid, 128, 0, st>>>(img, x, d, mid, tokidx, runs, n_runs, hid_f32);
  else if (img.fmt == kQ4K)
    k_up_simt<kQ4K><<<grid, 128, 0, st>>>(img, x, d, mid, tokidx, runs, n_runs, hid_f32);
  else
    k_up_simt<kQ51><<<grid, 128, 0, st>>>(img, x, d, mid, tokidx, runs, n_runs, hid_f32);
  return cudaGetLastError();
}

cudaError_t launch_down_simt(const Image& img, const float* hid_f32, int d, int mid, const Run* runs,
                             const int32_t* n_runs, int max_runs, float* pairs_f32,
                             cudaStream_t st) {
  dim3 grid(img.n_mtiles, max_runs);
  if (img.fmt == kQ4CP)
    k_down_simt<kQ4CP><<<grid, 128, 0, st>>>(img, hid_f32, d, mid, runs, n_runs, pairs_f32);
  else if (img.fmt == kQ4K)
    k_down_simt<kQ4K><<<grid, 128, 0, st>>>(img, hid_f32, d, mid, runs, n_runs, pairs_f32);
  else
    k_down_simt<kQ51><<<grid, 128, 0, st>>>(img, hid_f32, d, mid, runs, n_runs, pairs_f32);
  return cudaGetLastError();
}

}  // namespace b200moe
