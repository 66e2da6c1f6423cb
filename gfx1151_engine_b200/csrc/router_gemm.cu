// router_gemm.cu -- router logits from hidden states: logits[t][e] = sum_c W[e][c] * x[t][c],
// W = layers.L.mlp.gate.weight, bf16 [E][d]. It takes the place of the engine's router GEMM
// (gemm(gate_weight(l), d_xb, d_routerb, P), src/gpu/parts/40_model.inc:4022-4025) and follows
// the reference's CPU arithmetic (matvec, src/ref.cpp:68-77: products in double, summed in
// index order, rounded to float once) wherever the difference could change the routing:
//   * k_router_gemm: bf16 x bf16 -> fp32 on the tensor cores (tcgen05.mma, both operands from
//     shared memory by TMA, accumulators in tensor memory). A CTA owns 256 tokens x 256
//     experts: two M=128 halves share every expert tile, so the weight matrix is read from L2
//     once per 256 tokens. Products are exact; the fp32 accumulation differs from the
//     reference's double sum by ~1e-6.
//   * k_router_dots: few tokens (T <= 16): every logit as a double tree sum of the exact
//     products, rounded to float (within 1e-9 of the reference's index-order sum, i.e. the same
//     float except when the sum sits on a rounding boundary).
//   * k_router_flag: the experts that decide a token's top-k -- its k largest logits and
//     everything within two margins below the k-th -- are put on a list when two of them are
//     closer than the margin (1e-4 x magnitude after the tensor-core GEMM, whose accumulation
//     error is ~1e-5; 5e-7 after the double sums).
//   * k_router_pairs: the listed (token, expert) logits in the reference's arithmetic. Any
//     order of adding n exact terms in double is within n * 2^-53 * sum |term| of the true sum;
//     when that whole interval rounds to one float it is the reference's logit, otherwise the
//     index order is replayed.
//   With exact values for every expert that can be in or next to the top-k, the ids and their
//   order are the reference's; the other logits only enter the softmax denominator, which
//   cancels in the renormalised weights up to the last bit.
// Every wait on an mbarrier is bounded; a timeout sets the status word and the CTA leaves
// after releasing its tensor memory.
#include "kernels.h"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace b200moe {

struct RouterPlan {
  PFN_cuTensorMapEncodeTiled_v12000 enc = nullptr;
};

namespace {

constexpr int kRgThreads = 192;   // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int kRgStages = 3;
constexpr int kRgTileM = 256, kRgTileN = 256;
constexpr int kRgStageBytes = (kRgTileM + kRgTileN) * 128;  // 64 K-elements of bf16 per row
constexpr int kRgSmem = kRgStages * kRgStageBytes + 1024 + 1024;  // + alignment slack + barriers
constexpr long long kRgWaitNs = 2000000000ll;

__device__ __forceinline__ uint32_t rg_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void rg_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void rg_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool rg_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false after 2 s (status {4, where}) or when another wait of the CTA gave up.
__device__ __forceinline__ bool rg_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                        int where) {
  if (rg_try(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t spin = 1;; spin++) {
    if (rg_try(bar, parity)) return true;
    if ((spin & 255u) == 0) {
      if (*abort_flag) return false;
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > (unsigned long long)kRgWaitNs) {
        *abort_flag = 1;
        if (atomicCAS(status, 0, 4) == 0) status[1] = where;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void rg_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// K-major tile of 128-byte rows with the 128-byte swizzle (what the TMA copy writes)
__device__ __forceinline__ uint64_t rg_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void rg_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void rg_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool rg_elect() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__global__ void __launch_bounds__(kRgThreads, 1)
k_router_gemm(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, int T, int E,
              int d, float* __restrict__ logits, int32_t* status) {
  extern __shared__ __align__(1024) uint8_t rg_raw[];
  const uint32_t raw0 = rg_smem_u32(rg_raw);
  const uint32_t base = (raw0 + 1023u) & ~1023u;            // stage buffers need 1 KB alignment
  uint8_t* const sm = rg_raw + (base - raw0);
  const uint32_t bars = base + kRgStages * kRgStageBytes;   // full[3], empty[3], acc_full
  volatile int* abort_flag = (volatile int*)(sm + kRgStages * kRgStageBytes + 64);
  uint32_t* tmem_slot = (uint32_t*)(sm + kRgStages * kRgStageBytes + 72);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kRgTileM, n0 = blockIdx.y * kRgTileN;
  const int KB = d / 64;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kRgStages; i++) {
      rg_mbar_init(bars + 8 * i, 1);
      rg_mbar_init(bars + 8 * (kRgStages + i), 1);
    }
    rg_mbar_init(bars + 8 * (2 * kRgStages), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(rg_smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < KB && ok; kb++) {
        const int s = kb % kRgStages, ph = (kb / kRgStages) & 1;
        ok = rg_wait(bars + 8 * (kRgStages + s), ph ^ 1, abort_flag, status, 1);
        if (!ok) break;
        rg_expect_tx(bars + 8 * s, kRgStageBytes);
        rg_tma_2d(base + s * kRgStageBytes, &map_x, kb * 64, m0, bars + 8 * s);
        rg_tma_2d(base + s * kRgStageBytes + kRgTileM * 128, &map_w, kb * 64, n0, bars + 8 * s);
      }
    }
  } else if (warp == 1) {
    // D fp32, A and B bf16, both K-major, M = 128, N = 256
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kRgTileN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    bool ok = true;
    for (int kb = 0; kb < KB && ok; kb++) {
      const int s = kb % kRgStages, ph = (kb / kRgStages) & 1;
      ok = __all_sync(0xffffffffu, rg_wait(bars + 8 * s, ph, abort_flag, status, 2));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a0 = base + s * kRgStageBytes, b0 = a0 + kRgTileM * 128;
      if (rg_elect()) {
#pragma unroll
        for (int mh = 0; mh < 2; mh++) {
#pragma unroll
          for (int ks = 0; ks < 4; ks++)
            rg_mma_ss(tmem + mh * kRgTileN, rg_desc(a0 + mh * 128 * 128) + (uint64_t)(ks * 2),
                      rg_desc(b0) + (uint64_t)(ks * 2), idesc, (kb | ks) != 0 ? 1u : 0u);
        }
        rg_commit(bars + 8 * (kRgStages + s));                     // the stage may be refilled
        if (kb == KB - 1) rg_commit(bars + 8 * (2 * kRgStages));  // the accumulators are complete
      }
      __syncwarp();
    }
  } else {
    // epilogue: warp w reads tensor-memory lanes (w & 3) * 32 .. +31 = token rows of both halves
    const int q = warp & 3;
    const bool ok = __all_sync(0xffffffffu, rg_wait(bars + 8 * (2 * kRgStages), 0, abort_flag, status, 3));
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int mh = 0; mh < 2; mh++) {
        const int row = m0 + mh * 128 + q * 32 + lane;
        for (int c0 = 0; c0 < kRgTileN; c0 += 32) {
          uint32_t v[32];
          const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + mh * kRgTileN + c0;
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
              "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
              "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
              : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
                "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                "=r"(v[30]), "=r"(v[31])
              : "r"(taddr)
              : "memory");
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (row < T) {
            float* dst = logits + (size_t)row * E + n0 + c0;
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (n0 + c0 + j < E) dst[j] = __uint_as_float(v[j]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// ---- logits in double --------------------------------------------------------------------
// A block takes 8 tokens x 8 experts: the tokens' activations are staged in shared memory,
// warp w owns expert 8*chunk + w and adds the eight dot products side by side in double (one
// fused multiply-add per term: the product of two bf16 values is exact in double, so the
// fused form rounds exactly like multiply-then-add). Tokens 0 .. n-1.
constexpr int kExTok = 8, kExExp = 8;

__global__ void __launch_bounds__(256)
k_router_dots(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, int n, int E, int d,
              float* __restrict__ logits) {
  extern __shared__ __align__(16) uint16_t ex_x[];  // [kExTok][d] bf16 bits
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_groups = (n + kExTok - 1) / kExTok, n_chunks = (E + kExExp - 1) / kExExp;
  for (long long job = blockIdx.x; job < (long long)n_groups * n_chunks; job += gridDim.x) {
    const int grp = (int)(job / n_chunks), chunk = (int)(job % n_chunks);
    __syncthreads();  // the previous job's reads of the staged rows are over
    for (int g = 0; g < kExTok; g++) {
      const int t = grp * kExTok + g;
      for (int c = threadIdx.x * 8; c < d; c += 256 * 8) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < n) v = *(const uint4*)(x + (size_t)t * d + c);
        *(uint4*)(ex_x + (size_t)g * d + c) = v;
      }
    }
    __syncthreads();
    const int e = chunk * kExExp + warp;
    if (e < E) {
      const uint16_t* wr = w + (size_t)e * d;
      double acc[kExTok];
#pragma unroll
      for (int g = 0; g < kExTok; g++) acc[g] = 0;
      for (int c = lane * 8; c < d; c += 256) {
        const uint4 wv = __ldg((const uint4*)(wr + c));
        const uint16_t* wb = (const uint16_t*)&wv;
        double wd[8];
#pragma unroll
        for (int j = 0; j < 8; j++) wd[j] = (double)bf16_bits_to_f32(wb[j]);
#pragma unroll
        for (int g = 0; g < kExTok; g++) {
          const uint4 xv = *(const uint4*)(ex_x + (size_t)g * d + c);
          const uint16_t* xb = (const uint16_t*)&xv;
#pragma unroll
          for (int j = 0; j < 8; j++) acc[g] = fma(wd[j], (double)bf16_bits_to_f32(xb[j]), acc[g]);
        }
      }
#pragma unroll
      for (int g = 0; g < kExTok; g++) {
#pragma unroll
        for (int o = 16; o; o >>= 1)
          acc[g] += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(acc[g]), o),
                                     __shfl_xor_sync(0xffffffffu, __double2loint(acc[g]), o));
      }
      if (lane < kExTok && grp * kExTok + lane < n) {
        double a = acc[0];
#pragma unroll
        for (int g = 1; g < kExTok; g++)
          if (lane == g) a = acc[g];
        logits[(size_t)(grp * kExTok + lane) * E + e] = (float)a;
      }
    }
  }
}

// ---- listed logits in the reference's arithmetic: one warp per (token, expert) pair ----------
__global__ void __launch_bounds__(256)
k_router_pairs(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, const int32_t* __restrict__ pairs,
               const int32_t* __restrict__ count, int cap, int E, int d, float* __restrict__ logits) {
  __shared__ double s_prod[8][256];  // per warp: the products of 256 elements, for the index-order replay
  const int lane = threadIdx.x & 31;
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  const int n = min(*count, cap);
  for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += n_warps) {
    const int t = pairs[i] / E, e = pairs[i] % E;
    const uint16_t* xr = x + (size_t)t * d;
    const uint16_t* wr = w + (size_t)e * d;
    double acc = 0, mag = 0;
    for (int c = lane * 8; c < d; c += 256) {
      const uint4 xv = *(const uint4*)(xr + c), wv = __ldg((const uint4*)(wr + c));
      const uint16_t* xb = (const uint16_t*)&xv;
      const uint16_t* wb = (const uint16_t*)&wv;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const double pd = (double)bf16_bits_to_f32(wb[j]) * (double)bf16_bits_to_f32(xb[j]);  // exact
        acc += pd;
        mag += fabs(pd);
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      acc += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(acc), o),
                              __shfl_xor_sync(0xffffffffu, __double2loint(acc), o));
      mag += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(mag), o),
                              __shfl_xor_sync(0xffffffffu, __double2loint(mag), o));
    }
    acc = __hiloint2double(__shfl_sync(0xffffffffu, __double2hiint(acc), 0), __shfl_sync(0xffffffffu, __double2loint(acc), 0));
    mag = __hiloint2double(__shfl_sync(0xffffffffu, __double2hiint(mag), 0), __shfl_sync(0xffffffffu, __double2loint(mag), 0));
    // |index-order sum - true sum| <= gamma(d-1) * sum|p|, |this tree sum - true sum| <=
    // gamma(d/32 + 5) * sum|p| (d/32 additions per lane, five shuffle levels), gamma(n) ~ n * 2^-53;
    // `mag` is within the same tiny factor of sum|p|: 1 % of slack covers both second-order terms
    const double delta = 1.01 * (double)(d + d / 32 + 8) * 1.1102230246251565e-16 * mag;
    if ((float)(acc - delta) != (float)(acc + delta)) {  // warp-uniform
      // replay of the reference's order: the lanes form the (exact) products of 256 elements at a
      // time, lane 0 adds them in index order -- the chain of dependent additions is all that is
      // left on one thread
      acc = 0;
      double* sp = s_prod[threadIdx.x >> 5];
      for (int c0 = 0; c0 < d; c0 += 256) {
        const int c = c0 + lane * 8;
        if (c < d) {
          const uint4 xv = *(const uint4*)(xr + c), wv = __ldg((const uint4*)(wr + c));
          const uint16_t* xb = (const uint16_t*)&xv;
          const uint16_t* wb = (const uint16_t*)&wv;
#pragma unroll
          for (int j = 0; j < 8; j++) sp[lane * 8 + j] = (double)bf16_bits_to_f32(wb[j]) * (double)bf16_bits_to_f32(xb[j]);
        }
        __syncwarp();
        if (lane == 0) {
          const int n = min(256, d - c0);
          for (int j = 0; j < n; j++) acc += sp[j];
        }
        __syncwarp();
      }
    }
    if (lane == 0) logits[(size_t)t * E + e] = (float)acc;
  }
}

// One warp per token, E <= 512. The experts that decide the token's top-k are its k largest
// logits and every other one within two margins of the k-th. If any two of them are closer
// than the margin (relative to the magnitude of the largest logit), all of them go on the
// pair list (token * E + expert) for recomputation in the reference's arithmetic.
__global__ void __launch_bounds__(256)
k_router_flag(const float* __restrict__ logits, int T, int E, int k, float rel_margin, int32_t* __restrict__ pairs,
              int32_t* __restrict__ count, int cap, int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  float v[16], v0[16];
#pragma unroll
  for (int j = 0; j < 16; j++) v0[j] = v[j] = j * 32 + lane < E ? logits[(size_t)t * E + j * 32 + lane] : -INFINITY;
  float prev = 0.f, margin = 0.f;
  bool close = false;
  const int rounds = min(k, E);
  for (int r = 0; r < rounds; r++) {
    float bv = -INFINITY;
    int bj = 0;
#pragma unroll
    for (int j = 0; j < 16; j++)
      if (v[j] > bv) {
        bv = v[j];
        bj = j;
      }
    float m = bv;
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // remove ONE instance of the maximum (equal values are a tie, which the margin catches)
    const unsigned who = __ballot_sync(0xffffffffu, bv == m);
    if (lane == __ffs(who) - 1) {
#pragma unroll
      for (int j = 0; j < 16; j++)
        if (j == bj) v[j] = -INFINITY;
    }
    if (r == 0) margin = rel_margin * fmaxf(1.f, fabsf(m));
    else if (prev - m < margin) close = true;
    prev = m;
  }
  // prev = the k-th largest; challengers from below
  float rest = -INFINITY;
#pragma unroll
  for (int j = 0; j < 16; j++) rest = fmaxf(rest, v[j]);
#pragma unroll
  for (int o = 16; o; o >>= 1) rest = fmaxf(rest, __shfl_xor_sync(0xffffffffu, rest, o));
  if (prev - rest < margin) close = true;
  if (!close) return;
  const float floor_v = prev - 2.f * margin;
#pragma unroll
  for (int j = 0; j < 16; j++)
    if (v0[j] >= floor_v) {
      const int i = atomicAdd(count, 1);
      if (i < cap) pairs[i] = t * E + j * 32 + lane;
      // more near-ties than the list holds: those logits keep their GEMM values, the order of
      // the top-k is then not guaranteed to be the reference's -- say so instead of hiding it
      else if (status && atomicCAS(status, 0, 7) == 0) status[1] = t;
    }
}

}  // namespace

cudaError_t router_plan_create(RouterPlan** out) {
  *out = nullptr;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
  RouterPlan* p = new RouterPlan();
  p->enc = (PFN_cuTensorMapEncodeTiled_v12000)fn;
  e = cudaFuncSetAttribute(k_router_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, kRgSmem);
  if (e != cudaSuccess) {
    delete p;
    return e;
  }
  *out = p;
  return cudaSuccess;
}

void router_plan_destroy(RouterPlan* p) { delete p; }

static cudaError_t rg_encode(RouterPlan* p, CUtensorMap* map, const void* base, long long rows, long long cols) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, 256};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = p->enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t launch_router_gemm(RouterPlan* p, const void* x_bf16, const void* w_bf16, int T, int E, int d,
                               float* logits, int32_t* status, cudaStream_t st) {
  CUtensorMap mx, mw;
  cudaError_t e = rg_encode(p, &mx, x_bf16, T, d);
  if (e == cudaSuccess) e = rg_encode(p, &mw, w_bf16, E, d);
  if (e != cudaSuccess) return e;
  dim3 grid((T + kRgTileM - 1) / kRgTileM, (E + kRgTileN - 1) / kRgTileN);
  k_router_gemm<<<grid, kRgThreads, kRgSmem, st>>>(mx, mw, T, E, d, logits, status);
  return cudaGetLastError();
}

cudaError_t launch_router_flag(const float* logits, int T, int E, int k, float rel_margin, int32_t* pairs,
                               int32_t* count, int cap, cudaStream_t st, int32_t* status) {
  cudaError_t e = cudaMemsetAsync(count, 0, sizeof(int32_t), st);
  if (e != cudaSuccess) return e;
  k_router_flag<<<(T + 7) / 8, 256, 0, st>>>(logits, T, E, k, rel_margin, pairs, count, cap, status);
  return cudaGetLastError();
}

cudaError_t launch_router_dots(const void* x_bf16, const void* w_bf16, int T, int E, int d, float* logits,
                               cudaStream_t st) {
  const size_t smem = (size_t)kExTok * d * 2;
  static size_t smem_set = 0;
  if (smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(k_router_dots, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    smem_set = smem;
  }
  long long jobs = (long long)((T + kExTok - 1) / kExTok) * ((E + kExExp - 1) / kExExp);
  int blocks = (int)(jobs < 148 * 3 ? jobs : 148 * 3);
  if (blocks < 1) blocks = 1;
  k_router_dots<<<blocks, 256, smem, st>>>((const uint16_t*)x_bf16, (const uint16_t*)w_bf16, T, E, d, logits);
  return cudaGetLastError();
}

cudaError_t launch_router_pairs(const void* x_bf16, const void* w_bf16, const int32_t* pairs, const int32_t* count,
                                int cap, int E, int d, float* logits, cudaStream_t st) {
  int blocks = (cap + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  k_router_pairs<<<blocks, 256, 0, st>>>((const uint16_t*)x_bf16, (const uint16_t*)w_bf16, pairs, count, cap, E, d, logits);
  return cudaGetLastError();
}

}  // namespace b200moe
