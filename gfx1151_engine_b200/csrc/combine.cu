// combine.cu -- the memory-bound ends of the path: the expert-sorted activation gather
// in front of the grouped GEMM and the weighted top-k combine behind it.
//
// Combine replaces k_moe_reduce_pw / k_moe_reduce_pw_sg
// (src/gpu/parts/24_kernels_moe_lt.inc:81-124 of the reference):
//   out[t][c] = sum_{s<k} pw[row_s] * pairs[row_s][c]   (+ gate[t] * pairs[shared row][c])
// with row_s = pairids[t*k + s], i.e. a fixed order (ascending expert id), fp32
// accumulation, every output element written exactly once -- deterministic, no atomics.
//
// With a state pointer the same kernels do the write-back of k_moe_reduce_pw_sg_hc
// (src/gpu/parts/24_kernels_moe_lt.inc:126-161) instead of storing `out`: the layer result is
// added into the four branches of the bf16 residual state,
//   R[t][b][c] = bf16(float(R[t][b][c]) + inj[t][b] * sum),  inj = 2 / (1 + exp(-w4[t][b] / 4)).
#include "kernels.h"

namespace b200moe {

namespace {

__device__ __forceinline__ void load8(const float* p, float* v) {
  float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __half* p, float* v) {
  uint4 u = *(const uint4*)p;
  const __half2* h = (const __half2*)&u;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

struct HcWriteBack {
  const float* w4;   // [T][4] inject gate pre-activations, or null: store `out`
  uint16_t* state;   // [T][4][d] bf16
};

__device__ __forceinline__ float hc_inject(float w) { return 2.f / (1.f + expf(-w * 0.25f)); }

__device__ __forceinline__ uint32_t hc_add2(uint32_t r, float inj, float a, float b) {
  const float lo = bf16_bits_to_f32((uint16_t)(r & 0xFFFFu)), hi = bf16_bits_to_f32((uint16_t)(r >> 16));
  const __nv_bfloat162 o = __floats2bfloat162_rn(fmaf(inj, a, lo), fmaf(inj, b, hi));
  return *(const uint32_t*)&o;
}

// One block per (token, 2048-column slice); each thread owns 8 consecutive columns.
// ROT (hgn v2 i4r experts, rotate.cu): the weighted sum is still in the rotated domain; 16
// neighbouring threads hold one 128-column block of it and turn it into rot_post * H128(sum) /
// sqrt(128) (natural-order Hadamard: three butterfly levels inside the thread, four by lane
// shuffles) before the result is stored or written back -- k_v2_reduce_rot of the reference
// (src/gpu/parts/28_kernels_hgn_v2.inc:145-152). d is a multiple of 128, so a half-warp is in
// range or out of range as a whole; the loop runs warp-uniformly so that the shuffles are legal.
template <typename TP, bool ROT = false>
__global__ void __launch_bounds__(256)
k_combine(const TP* __restrict__ pairs, const float* __restrict__ pw,
          const int32_t* __restrict__ pairids, int k, int d, int shared_row0,
          __nv_bfloat16* __restrict__ out, HcWriteBack hc, const float* __restrict__ rot_post = nullptr) {
  const int t = blockIdx.x;
  __shared__ int s_row[kMaxTopK + 1];
  __shared__ float s_w[kMaxTopK + 1];
  int n = k;
  if (threadIdx.x < k) {
    // a negative row marks a pair the bucketing dropped (expert id outside [0, E)): it adds nothing
    int row = pairids[(size_t)t * k + threadIdx.x];
    s_row[threadIdx.x] = row;
    s_w[threadIdx.x] = row >= 0 ? pw[row] : 0.f;
  }
  if (shared_row0 >= 0) {
    if (threadIdx.x == 0) {
      s_row[k] = shared_row0 + t;
      s_w[k] = pw[shared_row0 + t];
    }
    n = k + 1;
  }
  __syncthreads();
  const int lane8 = (threadIdx.x & 31) * 8;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c - (ROT ? lane8 : 0) < d; c += gridDim.y * blockDim.x * 8) {
    const bool live = !ROT || c < d;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < n; s++) {
      if (s_row[s] < 0 || !live) continue;
      float v[8];
      load8(pairs + (size_t)s_row[s] * d + c, v);
      const float w = s_w[s];
#pragma unroll
      for (int i = 0; i < 8; i++) acc[i] = fmaf(w, v[i], acc[i]);
    }
    if (ROT) {
#pragma unroll
      for (int b = 1; b < 8; b <<= 1)
#pragma unroll
        for (int i = 0; i < 8; i++)
          if (!(i & b)) {
            const float p = acc[i], q = acc[i | b];
            acc[i] = p + q;
            acc[i | b] = p - q;
          }
#pragma unroll
      for (int bit = 1; bit < 16; bit <<= 1) {
        const bool upper = (threadIdx.x & bit) != 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float o = __shfl_xor_sync(0xffffffffu, acc[i], bit);
          acc[i] = upper ? o - acc[i] : acc[i] + o;
        }
      }
      if (!live) continue;
      float post[8];
      load8(rot_post + c, post);
#pragma unroll
      for (int i = 0; i < 8; i++) acc[i] = acc[i] * 0.08838834764831845f * post[i];
    }
    if (hc.w4) {
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const float inj = hc_inject(hc.w4[(size_t)t * 4 + b]);
        uint4* rp = (uint4*)(hc.state + ((size_t)t * 4 + b) * d + c);
        uint4 r = *rp;
        r.x = hc_add2(r.x, inj, acc[0], acc[1]);
        r.y = hc_add2(r.y, inj, acc[2], acc[3]);
        r.z = hc_add2(r.z, inj, acc[4], acc[5]);
        r.w = hc_add2(r.w, inj, acc[6], acc[7]);
        *rp = r;
      }
      continue;
    }
    uint4 o;
    __nv_bfloat162* ob = (__nv_bfloat162*)&o;
#pragma unroll
    for (int i = 0; i < 4; i++) ob[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *(uint4*)(out + (size_t)t * d + c) = o;
  }
}

// Few tokens (decode): latency matters, not bandwidth. A thread owns 4 columns and issues the
// loads of all rows before it adds them (same order of additions as k_combine).
__global__ void __launch_bounds__(128)
k_combine_small(const float* __restrict__ pairs, const float* __restrict__ pw,
                const int32_t* __restrict__ pairids, int k, int d, int shared_row0,
                __nv_bfloat16* __restrict__ out, HcWriteBack hc) {
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  pdl_trigger();
  pdl_wait();
  if (c >= d) return;
  const int n = k + (shared_row0 >= 0 ? 1 : 0);
  float4 v[kMaxTopK + 1];
  float w[kMaxTopK + 1];
#pragma unroll
  for (int s = 0; s < kMaxTopK + 1; s++) {
    if (s < n) {
      const int row = s < k ? pairids[(size_t)t * k + s] : shared_row0 + t;
      const bool live = row >= 0;  // negative: a pair the bucketing dropped (expert id outside [0, E))
      w[s] = live ? pw[row] : 0.f;
      v[s] = live ? *(const float4*)(pairs + (size_t)row * d + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int s = 0; s < kMaxTopK + 1; s++) {
    if (s < n) {
      acc.x = fmaf(w[s], v[s].x, acc.x);
      acc.y = fmaf(w[s], v[s].y, acc.y);
      acc.z = fmaf(w[s], v[s].z, acc.z);
      acc.w = fmaf(w[s], v[s].w, acc.w);
    }
  }
  if (hc.w4) {
#pragma unroll
    for (int b = 0; b < 4; b++) {
      const float inj = hc_inject(hc.w4[(size_t)t * 4 + b]);
      uint2* rp = (uint2*)(hc.state + ((size_t)t * 4 + b) * d + c);
      uint2 r = *rp;
      r.x = hc_add2(r.x, inj, acc.x, acc.y);
      r.y = hc_add2(r.y, inj, acc.z, acc.w);
      *rp = r;
    }
    return;
  }
  uint2 o;
  *(__nv_bfloat162*)&o.x = __floats2bfloat162_rn(acc.x, acc.y);
  *(__nv_bfloat162*)&o.y = __floats2bfloat162_rn(acc.z, acc.w);
  *(uint2*)(out + (size_t)t * d + c) = o;
}

// Finite values saturate to the fp16 range; NaN stays NaN (fminf/fmaxf alone would turn it into
// a finite number and hide a broken activation from the caller).
__device__ __forceinline__ float clamp_f16_range(float v) {
  return v != v ? v : fminf(fmaxf(v, -65504.f), 65504.f);
}

// plain row gather of fp16 rows (the source is already fp16: rotated activations of hgn v2 i4r layers)
__global__ void __launch_bounds__(256)
k_gather_rows16(const uint4* __restrict__ x, const int32_t* __restrict__ tokidx, int rows, int per_row,
                uint4* __restrict__ xs) {
  const int lane = threadIdx.x & 31;
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += n_warps) {
    const uint4* src = x + (size_t)tokidx[row] * per_row;
    uint4* dst = xs + (size_t)row * per_row;
    for (int v = lane; v < per_row; v += 32) dst[v] = src[v];
  }
}

// x_sorted[row][:] = fp16(x[tokidx[row]][:]); bf16 -> fp16 is exact for 2^-14 <= |v| < 65520,
// larger magnitudes (infinities included) saturate to the largest finite half, NaN stays NaN.
// One warp per row: the token index is read once, a lane keeps four 16-byte loads in flight.
__global__ void __launch_bounds__(256)
k_gather_f16(const uint16_t* __restrict__ x, const int32_t* __restrict__ tokidx, int rows, int d,
             __half* __restrict__ xs) {
  const int lane = threadIdx.x & 31;
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  const int per_row = d / 8;  // 16-byte pieces
  for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += n_warps) {
    const uint4* src = (const uint4*)(x + (size_t)tokidx[row] * d);
    uint4* dst = (uint4*)(xs + (size_t)row * d);
    for (int v0 = lane; v0 < per_row; v0 += 128) {
      uint4 u[4];
#pragma unroll
      for (int i = 0; i < 4; i++)
        if (v0 + 32 * i < per_row) u[i] = src[v0 + 32 * i];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        if (v0 + 32 * i < per_row) {
          const uint16_t* b = (const uint16_t*)&u[i];
          uint4 o;
          __half2* oh = (__half2*)&o;
#pragma unroll
          for (int j = 0; j < 4; j++) {
            oh[j] = __floats2half2_rn(clamp_f16_range(bf16_bits_to_f32(b[2 * j])), clamp_f16_range(bf16_bits_to_f32(b[2 * j + 1])));
          }
          dst[v0 + 32 * i] = o;
        }
      }
    }
  }
}

}  // namespace

cudaError_t launch_combine_f32(const float* pairs, const float* pw, const int32_t* pairids, int T,
                               int k, int d, int shared_row0, void* out_bf16, cudaStream_t st,
                               const float* hc_w4, void* hc_state) {
  const HcWriteBack hc{hc_w4, (uint16_t*)hc_state};
  if (T <= 64 && d % 4 == 0)
    return launch_pdl(k_combine_small, dim3(T, (d / 4 + 127) / 128), dim3(128), 0, st, pairs, pw, pairids, k, d, shared_row0,
                      (__nv_bfloat16*)out_bf16, hc);
  else
    k_combine<float><<<dim3(T, (d + 2047) / 2048), 256, 0, st>>>(pairs, pw, pairids, k, d, shared_row0, (__nv_bfloat16*)out_bf16, hc);
  return cudaGetLastError();
}

cudaError_t launch_combine_f16(const __half* pairs, const float* pw, const int32_t* pairids, int T,
                               int k, int d, int shared_row0, void* out_bf16, cudaStream_t st,
                               const float* hc_w4, void* hc_state) {
  k_combine<__half><<<dim3(T, (d + 2047) / 2048), 256, 0, st>>>(pairs, pw, pairids, k, d, shared_row0,
                                       (__nv_bfloat16*)out_bf16, HcWriteBack{hc_w4, (uint16_t*)hc_state});
  return cudaGetLastError();
}

cudaError_t launch_combine_f16_rot(const __half* pairs, const float* pw, const int32_t* pairids, int T,
                                   int k, int d, const float* rot_post, void* out_bf16, cudaStream_t st,
                                   const float* hc_w4, void* hc_state) {
  if (d % 128 != 0 || !rot_post) return cudaErrorInvalidValue;
  k_combine<__half, true><<<dim3(T, (d + 2047) / 2048), 256, 0, st>>>(pairs, pw, pairids, k, d, -1, (__nv_bfloat16*)out_bf16,
                                                                      HcWriteBack{hc_w4, (uint16_t*)hc_state}, rot_post);
  return cudaGetLastError();
}

cudaError_t launch_gather_f16(const void* x_bf16, const int32_t* tokidx, int rows, int d,
                              __half* x_sorted, cudaStream_t st, bool src_f16) {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  int blocks = (rows + 7) / 8;
  if (blocks > sms * 8) blocks = sms * 8;
  if (blocks < 1) blocks = 1;
  if (src_f16) k_gather_rows16<<<blocks, 256, 0, st>>>((const uint4*)x_bf16, tokidx, rows, d / 8, (uint4*)x_sorted);
  else k_gather_f16<<<blocks, 256, 0, st>>>((const uint16_t*)x_bf16, tokidx, rows, d, x_sorted);
  return cudaGetLastError();
}

}  // namespace b200moe
