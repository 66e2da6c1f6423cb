// expert_gemv.cu -- decode / speculative-verify path (T <= 16) for q4cp experts: a
// bandwidth-oriented dequant GEMV. It takes the place of k_q4cp_gemv_gg, k_silu_mul_g and
// k_q4cp_gemv_gd (src/gpu/parts/20_kernels_gemv.inc:1607-1764 of the reference): per
// (token, expert) the 2*mid gate/up dot products, SwiGLU, then the d down dot products.
//
// At one token the whole layer is ~78 MB of 4-bit weights and 138 M multiply-adds; what
// decides the speed is (1) that DRAM sees long contiguous reads, (2) how many bytes each SM
// keeps in flight, (3) how few instructions and shared-memory wavefronts turn a code into a
// multiply-add.
//   * A lane owns a weight ROW: in the tiled image the 32 rows of a warp are 512 contiguous
//     bytes per half K block, so every load instruction of a warp is one long burst. (Lanes
//     that split K instead -- the reference's mapping -- read 16-byte pieces 2 KB apart from
//     this layout and reached 1 TB/s.) A lane's dot product needs no cross-lane reduction.
//   * The 16 warps of a CTA split K of the same rows; their partial sums meet in shared
//     memory and are added in a fixed order. The activations of the current token are staged
//     in shared memory as fp16 and read by broadcast (one 16-byte load per 4 code bytes).
//   * A code BYTE (two codes) is decoded by one lookup in a 256-entry half2 table that is
//     replicated per lane in shared memory (no bank conflicts); a table line is 256 bytes, on
//     a 64 KB boundary, so the lookup address is a single byte permute. The two products go
//     into an fp32 accumulator with the mixed-precision multiply-add (f32 += f16 * f16):
//     exact products, fp32 sums. The fp16 group scale multiplies the fp32 sum of a group once.
//   * A warp's share of a task is at most four K blocks = eight 16-byte loads per lane; as
//     soon as one K block has been consumed, the same registers receive the matching block
//     of the CTA's NEXT task, so every SM keeps ~64 KB in flight while it computes.
//   * Gate row r and up row r sit in lanes l and l+16 of the same warp: SwiGLU is a shuffle.
//   * The kernels are persistent: (row of the permuted activations, row block) tasks are cut
//     into one contiguous range per CTA; the tables are built once per CTA.
// (mma.sync was tried here first: on this GPU it retires an m16n8k16 only every ~50 cycles
// per SM, which made the kernel several times slower than the multiply-add form.)
#include "kernels.h"

namespace b200moe {

namespace {

constexpr int kGemvThreads = 512;     // 16 warps
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kKpw = 4;               // K blocks per warp and task, at most
constexpr int kGemvMaxRuns = 192;
constexpr int kGemvMaxK = 4096;       // staged activations: 8 KB of fp16
constexpr uint32_t kTab0 = 65536;     // absolute shared addresses of the two table blocks
constexpr uint32_t kTab1 = 131072;

struct GemvParams {
  Image img;             // routed experts
  Image img_sh;          // shared expert (data == nullptr: none)
  const Run* runs;       // routed runs [n_runs[0]]; the shared run sits at runs[kMaxExperts]
  const int32_t* n_runs;
  int K;                 // d (gate/up) or mid (down)
  int mid;
  const uint16_t* x;     // gate/up: bf16 [T][d]
  const int32_t* tokidx;
  __half* hid;           // gate/up writes, down reads: fp16 [rows][mid] = silu(gate) * up
  float* out;            // down: pairs fp32 [rows][d]
};

__device__ __forceinline__ uint32_t lds_b32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// acc += w.lo * x.lo + w.hi * x.hi with exact products and fp32 sums
__device__ __forceinline__ void fma_pair(float& acc, uint32_t w, uint32_t x) {
  asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
      "mov.b32 {wl, wh}, %1;\n\t"
      "mov.b32 {xl, xh}, %2;\n\t"
      "fma.rn.f32.f16 %0, wl, xl, %0;\n\t"
      "fma.rn.f32.f16 %0, wh, xh, %0;\n\t}"
      : "+f"(acc)
      : "r"(w), "r"(x));
}

// sum over one 16-byte chunk (32 codes of one group) of w[k] * x[k], as float.
// lut: constant half of the lookup address { lane*4 (+128), -, table >> 16, 0 };
// xs: shared address of the 32 fp16 activations of the group (same for all lanes: broadcast).
__device__ __forceinline__ float chunk_dot(const uint4 c, uint32_t lut, uint32_t xs) {
  const uint32_t w4[4] = {c.x, c.y, c.z, c.w};
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    uint32_t x0, x1, x2, x3;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(xs + q * 16));
    fma_pair(s0, lds_b32(__byte_perm(w4[q], lut, 0x7604)), x0);
    fma_pair(s1, lds_b32(__byte_perm(w4[q], lut, 0x7614)), x1);
    fma_pair(s0, lds_b32(__byte_perm(w4[q], lut, 0x7624)), x2);
    fma_pair(s1, lds_b32(__byte_perm(w4[q], lut, 0x7634)), x3);
  }
  return s0 + s1;
}

// Q5_1: the same with the fifth bits (bits i, 16 + i of qh belong to code byte i; shifted to bits
// 14 and 30 they are the fp16 pair 2.0 / 0) added to the looked-up pair as 8 * 2.0 by one half2
// multiply-add before the products: q + 16*bit <= 31 is exact in fp16.
__device__ __forceinline__ float chunk_dot5(const uint4 c, uint32_t qh, uint32_t lut, uint32_t xs) {
  const uint32_t w4[4] = {c.x, c.y, c.z, c.w};
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    uint32_t x[4];
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]) : "r"(xs + q * 16));
#pragma unroll
    for (int b = 0; b < 4; b++) {
      const int i = q * 4 + b;
      const uint32_t u = (i <= 14 ? (qh << (14 - i)) : (qh >> 1)) & 0x40004000u;
      const uint32_t pair = lds_b32(__byte_perm(w4[q], lut, 0x7604 | (b << 4)));
      const __half2 w2 = __hfma2(*(const __half2*)&u, __float2half2_rn(8.f), *(const __half2*)&pair);
      fma_pair((b & 1) ? s1 : s0, *(const uint32_t*)&w2, x[b]);
    }
  }
  return s0 + s1;
}

// finite values saturate to the fp16 range, NaN stays NaN
__device__ __forceinline__ float sat_f16(float v) { return v != v ? v : fminf(fmaxf(v, -65504.f), 65504.f); }
__device__ __forceinline__ uint32_t pack_half2_sat(float a, float b) {
  __half2 h = __floats2half2_rn(sat_f16(a), sat_f16(b));
  return *(uint32_t*)&h;
}



struct GemvShared {
  int first[kGemvMaxRuns + 2];  // unit prefix: rows before run i ("unit" = one row of the permuted activations)
  float book[3][16];
};

// FMT: format of the image this kernel reads (gate/up: q4cp or Q4_K; down: q4cp or Q5_1). The
// GGUF formats use the identity code book (table entry = the two code values) and fold their
// affine constants into the group sums: Q4_K  sum w x = (d*sc) * sum q x - (dmin*m) * sum x,
// Q5_1  sum w x = d * sum (q + 16 bit) x + m * sum x, with sum x per 32-group staged next to
// the activations.
template <bool UP, int FMT>
__global__ void __launch_bounds__(kGemvThreads, 1)
k_gemv(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t gsm[];
  __shared__ GemvShared sh;
  __shared__ __align__(16) __half xs[kGemvMaxK];   // activations of the current unit
  __shared__ float xsum[kGemvMaxK / 32];            // their sums per 32-group (GGUF formats)
  __shared__ float red[2][kGemvWarps][32];          // partial sums of the K slices, double-buffered by task
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t dyn0 = (uint32_t)__cvta_generic_to_shared(gsm);
  uint8_t* const smem = gsm - dyn0;  // smem + A is the generic pointer of absolute shared address A
  const bool has_sh = p.img_sh.data != nullptr;
  const bool two = UP && has_sh && p.img_sh.dual_book;
  pdl_trigger();
  {
    // The table blocks live at fixed absolute shared addresses: a launch whose dynamic
    // allocation does not cover them is refused (uniform for the grid; the host sizes it).
    uint32_t dyn_size;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (dyn0 > kTab0 || dyn0 + dyn_size < (two ? kTab1 + 65536 : kTab0 + 65536)) return;
  }
  // ---- code books and pair tables: weights only, nothing an earlier kernel of the stream
  // writes, so this part may overlap that kernel's tail ----
  if (threadIdx.x < 48) {
    const int b = threadIdx.x >> 4, e = threadIdx.x & 15;
    if (b == 0) sh.book[0][e] = p.img.book[e];
    else if (has_sh && (b == 1 || two)) sh.book[b][e] = p.img_sh.book[(b - 1) * 16 + e];
  }
  __syncthreads();
  {
    // entry e = (f16(book[e & 15]), f16(book[e >> 4])), one 256-byte line per code byte:
    // [32 lanes x 4 B of book A][32 lanes x 4 B of book B]. Block 0 holds the routed book (A)
    // and the shared expert's first book (B); block 1 the shared expert's second book (rows
    // 64..127 of its gate/up tiles, when that image has two books).
    // Warp w writes the 16 lines whose high code is w; lane l writes copy l of each line.
    const int nb = has_sh ? (two ? 3 : 2) : 1;
    for (int b = 0; b < nb; b++) {
      const uint32_t hi16 = (uint32_t)__half_as_ushort(__float2half_rn(sh.book[b][warp])) << 16;
      uint8_t* dst = smem + (b == 2 ? kTab1 : kTab0) + (b == 1 ? 128 : 0) + (warp * 16) * 256 + lane * 4;
#pragma unroll
      for (int c = 0; c < 16; c++)
        *(uint32_t*)(dst + c * 256) = hi16 | (uint32_t)__half_as_ushort(__float2half_rn(sh.book[b][c]));
    }
  }
  pdl_wait();
  // ---- unit prefix ----
  const int n_routed = p.n_runs[0];
  const int n_runs_all = min(n_routed + (has_sh ? 1 : 0), kGemvMaxRuns);
  for (int i = threadIdx.x; i < n_runs_all; i += kGemvThreads)
    sh.first[i] = (i < n_routed ? p.runs[i] : p.runs[kMaxExperts]).count;
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < n_runs_all; i++) {
      const int c = sh.first[i];
      sh.first[i] = acc;
      acc += c;
    }
    sh.first[n_runs_all] = acc;
  }
  __syncthreads();

  // ---- geometry. gate/up: a task = 16 hidden outputs (lanes 0..15 the gate rows, lanes 16..31
  // the matching up rows), every warp a K slice. down: a task = 64 output rows, warps = 2 row
  // groups x 8 K slices. A warp's share of a task is kpw <= 4 K blocks ("items"). ----
  const int KB = p.img.n_kblocks;        // image K blocks (twice p.K / 64 for a two-plane image of 8-bit codes)
  const int ash = p.img.act_shift;       // an image K block multiplies the activations of K block (index >> ash)
  constexpr int kSlices = UP ? kGemvWarps : kGemvWarps / 2;
  const int slice = UP ? warp : warp >> 1;
  const int kpw = (KB + kSlices - 1) / kSlices;  // <= kKpw (the host checks K)
  const int kb0 = slice * kpw;
  const int out_rows = UP ? p.mid : p.img.n_mtiles * kTileM;
  const int tpu = UP ? out_rows / 16 : out_rows / 64;  // tasks per unit
  const long long total = (long long)sh.first[n_runs_all] * tpu;
  const long long base = total / gridDim.x, rem = total % gridDim.x;
  const long long c0 = blockIdx.x * base + min((long long)blockIdx.x, rem), c1 = c0 + base + ((long long)blockIdx.x < rem ? 1 : 0);
  constexpr size_t tile_b = tile_bytes(FMT);     // the routed and the shared image have the same format
  constexpr int kMetaRow = FMT == kQ4CP ? 4 : FMT == kQ4K ? 8 : 16;  // bytes of metadata per tile row
  const uint32_t xs_addr = (uint32_t)__cvta_generic_to_shared(xs);

  uint4 cw[2 * kKpw];  // four item slots: codes of both halves of a K block ...
  uint4 sw[kKpw];      // ... and the row's metadata of the K block (q4cp: .x = two fp16 scales)
  int cur_tok = -1, buf = 0;
  for (long long seg = c0; seg < c1;) {
    // ---- a segment: the CTA's tasks j0 .. j1-1 of one unit ----
    const int unit = (int)(seg / tpu), j0 = (int)(seg % tpu);
    const int j1 = (int)min((long long)tpu, (long long)j0 + (c1 - seg));
    seg += j1 - j0;
    int lo = 0, hi = n_runs_all - 1;
    while (lo < hi) {
      const int m = (lo + hi + 1) >> 1;
      if (sh.first[m] <= unit) lo = m; else hi = m - 1;
    }
    const bool routed = lo < n_routed;
    Run run = routed ? p.runs[lo] : p.runs[kMaxExperts];
    run.first += unit - sh.first[lo];
    const Image& im = routed ? p.img : p.img_sh;
    const size_t mt_b = (size_t)im.n_kblocks * tile_b;
    const uint8_t* const ebase = im.data + (size_t)run.expert * im.n_mtiles * mt_b + (size_t)kb0 * tile_b;
    const uint32_t lut = (routed ? kTab0 : (UP && lane >= 16 && im.dual_book ? kTab1 : kTab0 + 128)) + lane * 4;
    // this lane's row of task j: offset of its codes in the first K block of the warp's slice
    auto row_off = [&](int j) -> size_t {
      if (UP) return (size_t)(j >> 2) * mt_b + ((lane < 16 ? 0 : 48) + (j & 3) * 16 + lane) * 16;  // gate rows 0..63, up rows 64..127
      return (size_t)(j >> 1) * mt_b + ((j & 1) * 64 + (warp & 1) * 32 + lane) * 16;
    };
    auto fetch = [&](int s, int j, int i) {  // item (task j, K block i of the slice) into slot s
      if (kb0 + i < KB) {
        const uint8_t* pc = ebase + row_off(j) + (size_t)i * tile_b;
        const size_t r16 = row_off(j) - (size_t)(UP ? j >> 2 : j >> 1) * mt_b;  // row * 16
        cw[2 * s] = __ldg((const uint4*)pc);
        cw[2 * s + 1] = __ldg((const uint4*)(pc + 2048));
        const uint8_t* pm = pc - r16 + kCodeBytes + (r16 >> 4) * kMetaRow;
        if (FMT == kQ4CP) {
          sw[s].x = __ldg((const uint32_t*)pm);
        } else if (FMT == kQ4K) {
          const uint2 u = __ldg((const uint2*)pm);
          sw[s].x = u.x;
          sw[s].y = u.y;
        } else {
          sw[s] = __ldg((const uint4*)pm);
        }
      }
    };
    const int nseg = (j1 - j0) * kpw;
    // the first four items go out before anything else: they are in flight while the tables
    // are built and the activations staged
    int pj = j0, pi = 0;  // the fetch stream's position
#pragma unroll
    for (int s = 0; s < kKpw; s++) {
      if (s < nseg) fetch(s, pj, pi);
      if (++pi == kpw) { pi = 0; pj++; }
    }
    // activations of the unit (the previous segment's reads of xs ended before its last barrier)
    bool staged = false;
    if (UP) {
      const int tok = p.tokidx[run.first];
      if (tok != cur_tok) {
        for (int c = threadIdx.x; c < p.K / 8; c += kGemvThreads) {
          const uint4 u = __ldg((const uint4*)(p.x + (size_t)tok * p.K) + c);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
          uint4 o;
          o.x = pack_half2_sat(__uint_as_float(w[0] << 16), __uint_as_float(w[0] & 0xFFFF0000u));
          o.y = pack_half2_sat(__uint_as_float(w[1] << 16), __uint_as_float(w[1] & 0xFFFF0000u));
          o.z = pack_half2_sat(__uint_as_float(w[2] << 16), __uint_as_float(w[2] & 0xFFFF0000u));
          o.w = pack_half2_sat(__uint_as_float(w[3] << 16), __uint_as_float(w[3] & 0xFFFF0000u));
          ((uint4*)xs)[c] = o;
        }
        cur_tok = tok;
        staged = true;
      }
    } else {
      for (int c = threadIdx.x; c < p.K / 8; c += kGemvThreads)
        ((uint4*)xs)[c] = ((const uint4*)(p.hid + (size_t)run.first * p.mid))[c];  // written by the previous kernel: plain loads
      staged = true;
    }
    if (staged) {
      __syncthreads();
      if (FMT != kQ4CP) {
        for (int g = threadIdx.x; g < p.K / 32; g += kGemvThreads) {
          float t = 0.f;
          for (int i = 0; i < 32; i++) t += __half2float(xs[g * 32 + i]);
          xsum[g] = t;
        }
        __syncthreads();
      }
    }

    int cj = j0, ci = 0;  // the compute stream's position
    float acc = 0.f;
    for (int n0 = 0; n0 < nseg; n0 += kKpw) {
#pragma unroll
      for (int s = 0; s < kKpw; s++) {
        if (n0 + s < nseg) {
          if (kb0 + ci < KB) {
            const uint32_t xa = xs_addr + (uint32_t)((kb0 + ci) >> ash) * (kTileK * 2);
            if (FMT == kQ4CP) {
              const float d0 = chunk_dot(cw[2 * s], lut, xa), d1 = chunk_dot(cw[2 * s + 1], lut, xa + 64);
              acc += half_bits_to_f32((uint16_t)(sw[s].x & 0xFFFFu)) * d0 + half_bits_to_f32((uint16_t)(sw[s].x >> 16)) * d1;
            } else if (FMT == kQ4K) {
              // metadata {fp16 d, fp16 dmin, u8 sc0, u8 m0, u8 sc1, u8 m1}
              const float d0 = chunk_dot(cw[2 * s], lut, xa), d1 = chunk_dot(cw[2 * s + 1], lut, xa + 64);
              const float dd = half_bits_to_f32((uint16_t)(sw[s].x & 0xFFFFu)), dm = half_bits_to_f32((uint16_t)(sw[s].x >> 16));
              const float x0 = xsum[2 * ((kb0 + ci) >> ash)], x1 = xsum[2 * ((kb0 + ci) >> ash) + 1];
              acc += (dd * (float)(sw[s].y & 0xFFu)) * d0 - (dm * (float)((sw[s].y >> 8) & 0xFFu)) * x0;
              acc += (dd * (float)((sw[s].y >> 16) & 0xFFu)) * d1 - (dm * (float)(sw[s].y >> 24)) * x1;
            } else {
              // metadata [2]{fp16 d, fp16 m, u32 fifth bits}
              const float d0 = chunk_dot5(cw[2 * s], sw[s].y, lut, xa), d1 = chunk_dot5(cw[2 * s + 1], sw[s].w, lut, xa + 64);
              const float x0 = xsum[2 * ((kb0 + ci) >> ash)], x1 = xsum[2 * ((kb0 + ci) >> ash) + 1];
              acc += half_bits_to_f32((uint16_t)(sw[s].x & 0xFFFFu)) * d0 + half_bits_to_f32((uint16_t)(sw[s].x >> 16)) * x0;
              acc += half_bits_to_f32((uint16_t)(sw[s].z & 0xFFFFu)) * d1 + half_bits_to_f32((uint16_t)(sw[s].z >> 16)) * x1;
            }
          }
          // the slot just consumed receives the item four further down the stream
          if (n0 + s + kKpw < nseg) fetch(s, pj, pi);
          if (++pi == kpw) { pi = 0; pj++; }
          if (++ci == kpw) {
            // ---- end of a task: the K slices meet in shared memory; one warp per row group
            // adds them in slice order ----
            red[buf][warp][lane] = acc;
            __syncthreads();
            if (UP) {
              if (warp == 0) {
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kGemvWarps; w++) tot += red[buf][w][lane];
                const float up = __shfl_down_sync(0xffffffffu, tot, 16);
                if (lane < 16)
                  p.hid[(size_t)run.first * p.mid + cj * 16 + lane] =
                      __float2half_rn(sat_f16(silu_f32(tot) * up));
              }
            } else {
              if (warp < 2) {
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kGemvWarps / 2; w++) tot += red[buf][2 * w + warp][lane];
                p.out[(size_t)run.first * out_rows + cj * 64 + warp * 32 + lane] = tot;
              }
            }
            buf ^= 1;
            acc = 0.f;
            ci = 0;
            cj++;
          }
        }
      }
    }
  }
}

template <bool UP, int FMT>
cudaError_t launch_gemv(const GemvParams& p, cudaStream_t st) {
  // the dynamic allocation must reach the end of the last table, wherever it starts
  constexpr int kMaxSmem = UP ? kTab1 + 65536 : kTab0 + 65536;
  const bool two = UP && p.img_sh.data && p.img_sh.dual_book;
  const int smem = two ? kTab1 + 65536 : kTab0 + 65536;
  static bool attr_done = false;
  static int sms = 0;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k_gemv<UP, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return e;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    attr_done = true;
  }
  return launch_pdl(k_gemv<UP, FMT>, dim3(sms), dim3(kGemvThreads), (size_t)smem, st, p);
}

}  // namespace

int gemv_max_runs() { return kGemvMaxRuns; }
int gemv_max_k() { return kGemvMaxK; }                       // 16 K slices x 4 K blocks
int gemv_max_mid() { return (kGemvWarps / 2) * kKpw * kTileK; }  // 8 K slices x 4 K blocks = 2048

cudaError_t launch_up_gemv(const Image& img, const Image* img_sh, const void* x_bf16, int d, int mid,
                           const int32_t* tokidx, const Run* runs, const int32_t* n_runs,
                           __half* hid16, cudaStream_t st) {
  GemvParams p{};
  p.img = img;
  if (img_sh) p.img_sh = *img_sh;
  p.runs = runs; p.n_runs = n_runs; p.K = d; p.mid = mid;
  p.x = (const uint16_t*)x_bf16; p.tokidx = tokidx; p.hid = hid16;
  if (img.fmt == kQ4K) return launch_gemv<true, kQ4K>(p, st);
  if (img.fmt == kQ51) return launch_gemv<true, kQ51>(p, st);
  return launch_gemv<true, kQ4CP>(p, st);
}

cudaError_t launch_down_gemv(const Image& img, const Image* img_sh, const __half* hid16, int d, int mid,
                             const Run* runs, const int32_t* n_runs, float* pairs_f32, cudaStream_t st) {
  GemvParams p{};
  p.img = img;
  if (img_sh) p.img_sh = *img_sh;
  p.runs = runs; p.n_runs = n_runs; p.K = mid; p.mid = mid;
  p.hid = const_cast<__half*>(hid16);
  p.out = pairs_f32;
  if (img.fmt == kQ4K) return launch_gemv<false, kQ4K>(p, st);
  if (img.fmt == kQ51) return launch_gemv<false, kQ51>(p, st);
  return launch_gemv<false, kQ4CP>(p, st);
}

}  // namespace b200moe
