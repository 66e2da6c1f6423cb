// expert_gemv.cu -- decode / speculative-verify path (T <= 16) for q4cp experts: a
// bandwidth-oriented dequant GEMV. It takes the place of k_q4cp_gemv_gg, k_silu_mul_g and
// k_q4cp_gemv_gd (src/gpu/parts/20_kernels_gemv.inc:1607-1764 of the reference): per
// (token, expert) the 2*mid gate/up dot products, SwiGLU, then the d down dot products.
//
// At one token the whole layer is ~78 MB of 4-bit weights and 138 M multiply-adds; what
// decides the speed is how few instructions it takes to turn a code into a multiply-add.
//   * Like the reference's kernel, the lanes of a warp split K: lane l owns the 32-groups
//     l, l+32, ... of a row and keeps the matching activations in registers as half2, so the
//     inner loop reads nothing but weights.
//   * A code BYTE (two codes) is decoded by one lookup in a 256-entry half2 table that is
//     replicated per lane in shared memory (no bank conflicts); the eight products of one
//     32-bit code word are chained in half2 (one HFMA2 per byte), then widened and added in
//     fp32; the fp16 group scale multiplies the fp32 sum of a group once.
//   * Rows are reduced across the warp by shuffles; gate row r and up row r are handled by
//     the same warp, so SwiGLU needs no second pass and no partial sums exist anywhere.
//   * The kernel is persistent: the (run, token, row block) space is cut into one contiguous
//     chunk per warp, token-major, so a warp reloads its activations only when the token
//     changes and the tables are built once per CTA.
// (mma.sync was tried here first: on this GPU it retires an m16n8k16 only every ~50 cycles
// per SM, which made the kernel several times slower than the multiply-add form.)
#include "kernels.h"

namespace b200moe {

namespace {

constexpr int kGemvThreads = 512;     // 16 warps, in teams of 1, 2 or 4
constexpr int kGemvRows = 4;          // weight rows per task (gate/up: 4 gate + 4 up rows)
constexpr int kGemvMaxChunks = 4;     // warps per team: K <= 4096
constexpr int kGemvMaxRuns = 192;

struct GemvParams {
  Image img;             // routed experts
  Image img_sh;          // shared expert (data == nullptr: none)
  const Run* runs;       // routed runs [n_runs[0]]; the shared run sits at runs[kMaxExperts]
  const int32_t* n_runs;
  int K;                 // d (gate/up) or mid (down)
  int mid;
  const uint16_t* x;     // gate/up: bf16 [T][d]
  const int32_t* tokidx;
  const float* hid;      // down: fp32 [rows][mid]
  float* out;            // gate/up: hid fp32 [rows][mid]; down: pairs fp32 [rows][d]
};

__device__ __forceinline__ __half2 lds_half2(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return *(__half2*)&v;
}

// sum over one 16-byte chunk (32 codes of one group) of w[k] * x[k], as float.
// lut: shared-window address of this lane's column of the pair table (entry stride 128 B).
__device__ __forceinline__ float chunk_dot(const uint4 c, uint32_t lut, const uint32_t* xh) {
  const uint32_t w4[4] = {c.x, c.y, c.z, c.w};
  float sum = 0.f;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    // two code bytes (four products) per half2 chain, then widened: keeps the fp16 rounding
    // of the sums at the level of the operand rounding
    __half2 a = __hmul2(lds_half2(lut + ((w4[q] & 0xFFu) << 7)), *(const __half2*)&xh[q * 4 + 0]);
    a = __hfma2(lds_half2(lut + (((w4[q] >> 8) & 0xFFu) << 7)), *(const __half2*)&xh[q * 4 + 1], a);
    __half2 b = __hmul2(lds_half2(lut + (((w4[q] >> 16) & 0xFFu) << 7)), *(const __half2*)&xh[q * 4 + 2]);
    b = __hfma2(lds_half2(lut + ((w4[q] >> 24) << 7)), *(const __half2*)&xh[q * 4 + 3], b);
    const float2 f = __half22float2(a), e = __half22float2(b);
    sum += (f.x + f.y) + (e.x + e.y);
  }
  return sum;
}

__device__ __forceinline__ uint32_t pack_half2_sat(float a, float b) {
  __half2 h = __floats2half2_rn(fminf(fmaxf(a, -65504.f), 65504.f), fminf(fmaxf(b, -65504.f), 65504.f));
  return *(uint32_t*)&h;
}

template <bool UP>
__global__ void __launch_bounds__(kGemvThreads, 1)
k_gemv(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t gsm[];
  const bool has_sh = p.img_sh.data != nullptr;
  uint32_t* lut_r = (uint32_t*)gsm;                  // routed book          [256][32] half2
  uint32_t* lut_s0 = lut_r + 256 * 32;               // shared, tile rows 0..63
  uint32_t* lut_s1 = lut_s0 + (p.img_sh.dual_book ? 256 * 32 : 0);
  __shared__ __half2 s_book[3][256];
  __shared__ int s_first[kGemvMaxRuns + 2];          // unit prefix: rows before run i
  __shared__ int s_units;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t a_lut_r = (uint32_t)__cvta_generic_to_shared(lut_r) + lane * 4,
                 a_lut_s0 = (uint32_t)__cvta_generic_to_shared(lut_s0) + lane * 4,
                 a_lut_s1 = (uint32_t)__cvta_generic_to_shared(lut_s1) + lane * 4;
  const int n_routed = p.n_runs[0];
  const int n_runs_all = min(n_routed + (has_sh ? 1 : 0), kGemvMaxRuns);
  auto run_of = [&](int i) { return i < n_routed ? p.runs[i] : p.runs[kMaxExperts]; };

  // ---- pair tables (entry b = f16(book[b & 15]), f16(book[b >> 4])) and the unit prefix ----
  for (int i = threadIdx.x; i < 3 * 256; i += kGemvThreads) {
    const int b = i >> 8, e = i & 255;
    const float* bk = b == 0 ? p.img.book : (has_sh ? p.img_sh.book + (b - 1) * 16 : nullptr);
    if (bk) s_book[b][e] = __floats2half2_rn(bk[e & 15], bk[e >> 4]);
  }
  for (int i = threadIdx.x; i < n_runs_all; i += kGemvThreads) s_first[i] = run_of(i).count;
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < n_runs_all; i++) {
      const int c = s_first[i];
      s_first[i] = acc;
      acc += c;
    }
    s_first[n_runs_all] = acc;
    s_units = acc;
  }
  __syncthreads();
  {
    const int nl = has_sh ? (p.img_sh.dual_book ? 3 : 2) : 1;
    for (int i = threadIdx.x; i < nl * 256 * 32; i += kGemvThreads)
      lut_r[i] = *(const uint32_t*)&s_book[i >> 13][(i >> 5) & 255];
  }
  __syncthreads();

  // tasks: (unit = one row of the permuted activations, block of kGemvRows outputs), handled
  // by a TEAM of ts warps: warp wq of a team owns the 32-groups wq*32 + lane of every row, so
  // a lane keeps only 32 activations (16 registers) and many warps fit on an SM; the ts
  // partial sums of a row meet in shared memory and are added in a fixed order.
  const int n_groups = p.K / 32;
  const int n_chunks = (n_groups + 31) / 32;
  const int ts = n_chunks <= 1 ? 1 : n_chunks <= 2 ? 2 : 4;
  const int teams_per_cta = (kGemvThreads / 32) / ts;
  const int team_local = warp / ts, wq = warp % ts;
  const int out_rows = UP ? p.mid : p.img.n_mtiles * kTileM;
  const int per_unit = out_rows / kGemvRows;
  const long long total = (long long)s_units * per_unit;
  const int n_teams = gridDim.x * teams_per_cta, team = blockIdx.x * teams_per_cta + team_local;
  const int chunk = (int)((total + n_teams - 1) / n_teams);
  const int t0 = (int)min((long long)team * chunk, total), t1 = (int)min((long long)t0 + chunk, total);
  const int grp = lane + 32 * wq;
  const bool live = grp < n_groups;
  constexpr int kR = UP ? 2 * kGemvRows : kGemvRows;
  __shared__ float s_part[2][kGemvThreads / 32][kR];

  uint32_t xh[16];  // activations of this lane's group, half2
  int cur_unit = -1, ri = 0;
  Run run = Run{0, 0, 0};
  for (int task = t0; task < t1; task++) {
    const int unit = task / per_unit, j = task % per_unit;
    if (unit != cur_unit) {
      // ---- new token row: find its run, reload this lane's activations ----
      int lo = 0, hi = n_runs_all - 1;
      while (lo < hi) {
        const int m = (lo + hi + 1) >> 1;
        if (s_first[m] <= unit) lo = m; else hi = m - 1;
      }
      ri = lo;
      run = run_of(ri);
      const int row = run.first + (unit - s_first[ri]);
#pragma unroll
      for (int q = 0; q < 16; q++) xh[q] = 0u;
      if (live) {
        if (UP) {
          const uint4* src = (const uint4*)(p.x + (size_t)p.tokidx[row] * p.K + grp * 32);
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const uint4 u = __ldg(src + q);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; e++)
              xh[q * 4 + e] = pack_half2_sat(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xFFFF0000u));
          }
        } else {
          const float4* src = (const float4*)(p.hid + (size_t)row * p.mid + grp * 32);
#pragma unroll
          for (int q = 0; q < 8; q++) {
            const float4 u = src[q];
            xh[q * 2] = pack_half2_sat(u.x, u.y);
            xh[q * 2 + 1] = pack_half2_sat(u.z, u.w);
          }
        }
      }
      cur_unit = unit;
    }
    const bool routed = ri < n_routed;
    const Image& im = routed ? p.img : p.img_sh;
    const int row_out = run.first + (unit - s_first[ri]);
    const int o0 = j * kGemvRows;  // first output of the task
    const int mt = UP ? o0 / 64 : o0 / kTileM, rr = UP ? o0 % 64 : o0 % kTileM;
    float acc[kR];
#pragma unroll
    for (int i = 0; i < kR; i++) acc[i] = 0.f;
    if (live) {
      const uint8_t* tile = im.tile(run.expert, mt, grp >> 1);
      const uint8_t* tp = tile + (grp & 1) * 2048;
      const uint8_t* sp = tile + kCodeBytes + (grp & 1) * 2;
      uint4 cw[kR];
      uint32_t sw[kR];
#pragma unroll
      for (int i = 0; i < kR; i++) {
        const int r = UP ? (i < kGemvRows ? rr + i : 64 + rr + (i - kGemvRows)) : rr + i;
        cw[i] = __ldg((const uint4*)(tp + r * 16));
        sw[i] = __ldg((const unsigned short*)(sp + r * 4));
      }
#pragma unroll
      for (int i = 0; i < kR; i++) {
        const int r = UP ? (i < kGemvRows ? rr + i : 64 + rr + (i - kGemvRows)) : rr + i;
        const uint32_t lut = (routed ? a_lut_r : (r >= 64 ? a_lut_s1 : a_lut_s0));
        acc[i] = half_bits_to_f32((uint16_t)sw[i]) * chunk_dot(cw[i], lut, xh);
      }
    }
    // ---- reduce every row over the 32 lanes, then over the team's warps ----
#pragma unroll
    for (int i = 0; i < kR; i++) {
#pragma unroll
      for (int o = 16; o; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    }
    float mine = acc[0];
#pragma unroll
    for (int i = 1; i < kR; i++)
      if (lane == i) mine = acc[i];  // lane i < kR now holds row i
    const int buf = task & 1;
    if (ts > 1) {
      if (lane < kR) s_part[buf][warp][lane] = mine;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + team_local), "r"(ts * 32) : "memory");
      if (wq == 0 && lane < kR) {
        mine = 0.f;
        for (int w2 = 0; w2 < ts; w2++) mine += s_part[buf][team_local * ts + w2][lane];
      }
    }
    if (wq == 0) {
      if (UP) {
        const float up = __shfl_down_sync(0xffffffffu, mine, kGemvRows);  // lane i gets row kGemvRows+i
        if (lane < kGemvRows) p.out[(size_t)row_out * p.mid + o0 + lane] = silu_f32(mine) * up;
      } else {
        if (lane < kGemvRows) p.out[(size_t)row_out * out_rows + o0 + lane] = mine;
      }
    }
  }
}

template <bool UP>
cudaError_t launch_gemv(const GemvParams& p, cudaStream_t st) {
  constexpr int kMaxSmem = 3 * 256 * 32 * 4;
  const int smem = (p.img_sh.data ? 3 : 1) * 256 * 32 * 4;
  static bool attr_done = false;
  static int sms = 0;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k_gemv<UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return e;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    attr_done = true;
  }
  k_gemv<UP><<<sms, kGemvThreads, smem, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

int gemv_max_runs() { return kGemvMaxRuns; }
int gemv_max_k() { return kGemvMaxChunks * 32 * 32; }

cudaError_t launch_up_gemv(const Image& img, const Image* img_sh, const void* x_bf16, int d, int mid,
                           const int32_t* tokidx, const Run* runs, const int32_t* n_runs,
                           float* hid_f32, cudaStream_t st) {
  GemvParams p{};
  p.img = img;
  if (img_sh) p.img_sh = *img_sh;
  p.runs = runs; p.n_runs = n_runs; p.K = d; p.mid = mid;
  p.x = (const uint16_t*)x_bf16; p.tokidx = tokidx; p.out = hid_f32;
  return launch_gemv<true>(p, st);
}

cudaError_t launch_down_gemv(const Image& img, const Image* img_sh, const float* hid_f32, int d, int mid,
                             const Run* runs, const int32_t* n_runs, float* pairs_f32, cudaStream_t st) {
  GemvParams p{};
  p.img = img;
  if (img_sh) p.img_sh = *img_sh;
  p.runs = runs; p.n_runs = n_runs; p.K = mid; p.mid = mid;
  p.hid = hid_f32; p.out = pairs_f32;
  return launch_gemv<false>(p, st);
}

}  // namespace b200moe
