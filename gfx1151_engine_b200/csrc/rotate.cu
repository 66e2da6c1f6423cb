// rotate.cu -- the Hadamard steps of hgn v2 "i4r" experts (dtype 23: 4-bit codes nib - 8, one fp16
// scale per 128 columns, stored in a rotated domain). The reference keeps the weights rotated and
// moves the rotation onto the activations (src/gpu/parts/28_kernels_hgn_v2.inc:1-15):
//   W = diag(svh) . Hn . G . Hn . diag(suh),  Hn = H128 / sqrt(128) block-diagonal, H128 the
//   Sylvester Hadamard matrix in natural order,
// so   y = W x = svh * Hn( G . Hn(suh * x) ).
// One MoE layer therefore is (src/gpu/parts/40_model.inc:4559-4680):
//   xr  = Hn(suh_gu * x)                         k_rot_in     (k_v2_rot of the reference)
//   z   = G_gate_up . xr                         grouped GEMM, no activation function
//   g|u = svh_gu * Hn(z);  h = silu(g) * u;  hr = Hn(suh_dn * h)      k_i4r_mid
//   p   = G_down . hr                            grouped GEMM
//   out = svh_dn * Hn(sum_k w_k p_k)             the combine kernel with its rotation step
// A warp owns one 128-vector: lane l holds elements 4l .. 4l+3, so loads and stores are
// contiguous; index bits 0-1 are butterflies inside the lane, bits 2-6 are lane shuffles. The
// transform in natural order does not depend on the order in which the seven bits are taken.
#include "kernels.h"

namespace b200moe {

namespace {

constexpr float kRs128 = 0.08838834764831845f;  // 1 / sqrt(128)

// in-place 128-point Walsh-Hadamard transform (natural order, unnormalised) of the warp's vector
__device__ __forceinline__ void fwht128(float (&v)[4], int lane) {
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c;
  v[1] = b + d;
  v[2] = a - c;
  v[3] = b - d;
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1) {
    const bool upper = (lane & bit) != 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], bit);
      v[j] = upper ? o - v[j] : v[j] + o;
    }
  }
}

__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi) {
  uint32_t r;  // finite values saturate to the fp16 range, NaN stays NaN
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// xr[t][b*128 ..] = fp16( Hn(pre * x[t][b*128 ..]) ), one warp per (token, block)
__global__ void __launch_bounds__(256)
k_rot_in(const uint16_t* __restrict__ x, const float* __restrict__ pre, int T, int d, __half* __restrict__ xr) {
  const int lane = threadIdx.x & 31;
  const int nb = d >> 7;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)T * nb) return;
  const int t = (int)(w / nb), b = (int)(w % nb);
  const size_t off = (size_t)t * d + b * 128 + lane * 4;
  const uint2 u = *(const uint2*)(x + off);
  const float4 p = *(const float4*)(pre + b * 128 + lane * 4);
  float v[4] = {bf16_bits_to_f32((uint16_t)(u.x & 0xFFFFu)) * p.x, bf16_bits_to_f32((uint16_t)(u.x >> 16)) * p.y,
                bf16_bits_to_f32((uint16_t)(u.y & 0xFFFFu)) * p.z, bf16_bits_to_f32((uint16_t)(u.y >> 16)) * p.w};
  fwht128(v, lane);
  uint2 o;
  o.x = pack_f16x2_sat(v[0] * kRs128, v[1] * kRs128);
  o.y = pack_f16x2_sat(v[2] * kRs128, v[3] * kRs128);
  *(uint2*)(xr + off) = o;
}

__device__ __forceinline__ void load4(const __half* p, float (&v)[4]) {
  const uint2 u = *(const uint2*)p;
  const float2 a = __half22float2(*(const __half2*)&u.x), b = __half22float2(*(const __half2*)&u.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// hr[row][b*128 ..] = fp16( Hn( suh_dn * silu(g) * u ) ) with g = svh_gu * Hn(z[row][b*128 ..]),
// u = svh_gu[mid + ..] * Hn(z[row][mid + b*128 ..]); one warp per (row, block of mid)
// (k_i4r_mid of the reference, src/gpu/parts/28_kernels_hgn_v2.inc:98-143).
__global__ void __launch_bounds__(256)
k_i4r_mid(const __half* __restrict__ z, const float* __restrict__ svh_gu, const float* __restrict__ suh_dn,
          long long rows, int mid, __half* __restrict__ hr) {
  const int lane = threadIdx.x & 31;
  const int nb = mid >> 7;
  const long long total = rows * nb;
  for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total;
       w += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long row = w / nb;
    const int c = (int)(w % nb) * 128 + lane * 4;
    float g[4], u[4];
    load4(z + row * 2 * mid + c, g);
    load4(z + row * 2 * mid + mid + c, u);
    fwht128(g, lane);
    fwht128(u, lane);
    const float4 sg = *(const float4*)(svh_gu + c), su = *(const float4*)(svh_gu + mid + c), sd = *(const float4*)(suh_dn + c);
    const float sgv[4] = {sg.x, sg.y, sg.z, sg.w}, suv[4] = {su.x, su.y, su.z, su.w}, sdv[4] = {sd.x, sd.y, sd.z, sd.w};
    float h[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float gv = g[j] * kRs128 * sgv[j], uv = u[j] * kRs128 * suv[j];
      h[j] = silu_f32(gv) * uv * sdv[j];
    }
    fwht128(h, lane);
    uint2 o;
    o.x = pack_f16x2_sat(h[0] * kRs128, h[1] * kRs128);
    o.y = pack_f16x2_sat(h[2] * kRs128, h[3] * kRs128);
    *(uint2*)(hr + row * mid + c) = o;
  }
}

__global__ void k_f16_to_f32(const uint16_t* __restrict__ src, float* __restrict__ dst, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = half_bits_to_f32(src[i]);
}

}  // namespace

cudaError_t launch_rot_in(const void* x_bf16, const float* pre, int T, int d, __half* xr, cudaStream_t st) {
  const long long warps = (long long)T * (d >> 7);
  if (warps == 0) return cudaSuccess;
  k_rot_in<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>((const uint16_t*)x_bf16, pre, T, d, xr);
  return cudaGetLastError();
}

cudaError_t launch_i4r_mid(const __half* z, const float* svh_gu, const float* suh_dn, int rows, int mid, __half* hr,
                           cudaStream_t st) {
  long long warps = (long long)rows * (mid >> 7);
  long long blocks = (warps + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  k_i4r_mid<<<(unsigned)blocks, 256, 0, st>>>(z, svh_gu, suh_dn, (long long)rows, mid, hr);
  return cudaGetLastError();
}

cudaError_t launch_f16_to_f32(const void* src_f16_dev, float* dst, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  k_f16_to_f32<<<(n + 255) / 256, 256, 0, st>>>((const uint16_t*)src_f16_dev, dst, n);
  return cudaGetLastError();
}

}  // namespace b200moe
