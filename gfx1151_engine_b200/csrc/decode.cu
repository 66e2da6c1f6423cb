// decode.cu -- decode / speculative verify (T <= 8 tokens) of a q4cp layer as ONE kernel:
// routing, gate/up GEMV + SwiGLU, down GEMV and the weighted combine.
//
// It stands where the reference launches k_router_topk, k_q4cp_gemv_gg, k_silu_mul_g,
// k_q4cp_gemv_gd(_topk_h16) and the shared expert's GEMVs one after the other
// (GpuModel::moe, src/gpu/parts/40_model.inc:1806-1861; kernels
// src/gpu/parts/20_kernels_gemv.inc:1433-1835), and it reads every expert once for all the
// rows of a call that use it -- the reference's expert dedup for 2 <= P <= 8
// (src/gpu/parts/26_kernels_moe_gguf.inc:749-793, 893-939) -- with, as there, results that are
// bit-identical to processing the rows one by one.
//
// A decode call moves ~78 MB of 4-bit weights once and does almost no arithmetic, so what
// counts is how little of the call is NOT spent streaming weights:
//   * one launch instead of four: no launch gaps, no re-reading of routing tables from global
//     memory, the code-book tables are built once per phase;
//   * every block repeats the routing of the few tokens for itself in shared memory (512
//     threads, route_small.cuh), so no block waits for another one before it knows its experts;
//   * weights travel global -> shared memory by cp.async into a ring of three slots per warp
//     (a lane copies and later reads its own 16-byte pieces: no barrier, no registers held by
//     bytes in flight), two slots in flight while the third is consumed;
//   * a lane owns a weight row (a warp's read is 512 contiguous bytes of the tiled image), the
//     32 warps of a block split K; code byte -> half2 pair by one lookup in a lane-replicated
//     table whose address is one byte permute; exact products, fp32 sums (as expert_gemv.cu);
//   * between the phases the blocks meet at one grid-wide barrier (bounded wait); the first
//     down-phase weights are already in flight when it is reached;
//   * the down phase gives each block a 32-row slice of the output for ALL tokens and experts:
//     the weighted top-k sum (ascending expert id, then the shared expert -- the order of
//     k_moe_reduce_pw_sg, src/gpu/parts/24_kernels_moe_lt.inc:103-124) happens inside the block
//     and the bf16 result is written once. No pairs buffer, no combine kernel.
#include "kernels.h"
#include "route_small.cuh"

namespace b200moe {

namespace {

constexpr int kDecThreads = 1024;
constexpr int kDecWarps = 32;
constexpr int kDecMaxT = 8;
constexpr int kDecMaxPairs = 128;  // T * k
constexpr int kDecRows = 2;        // rows of one expert that share one pass over its weights
constexpr int kDepth = 3;          // ring slots per warp

// ---- shared-memory map, absolute addresses of the block's shared window ----
// The lookup table has one 256-byte line per code byte of which the first 128 bytes hold the
// 32 lane copies of the entry; it sits on a 64 KB boundary so that a lookup address is one
// byte permute {lane*4, code byte, 1, 0}. The second halves of the lines ("holes", 32 KB in
// 128-byte pieces) hold the code bytes of ring slot 0 of every warp.
constexpr uint32_t kOffLow = 2048;     // the dynamic allocation must start at or below this
constexpr uint32_t kOffRes = 2048;     // DecShared
constexpr uint32_t kOffWork = 10240;   // routing scratch, then partial sums (32 KB)
constexpr uint32_t kOffS0 = 43008;     // slot 0 of every warp: metadata + activation slices (32 x 384 B)
constexpr uint32_t kOffTab = 65536;    // 256 lines x 256 B
constexpr uint32_t kOffRing = 131072;  // slots 1, 2 of every warp (32 x 2 x 1408 B)
constexpr uint32_t kSlotBytes = 1408;  // 1024 code bytes + 128 metadata + 256 activation slices
constexpr uint32_t kDecSmemEnd = kOffRing + kDecWarps * (kDepth - 1) * kSlotBytes;  // 221184
static_assert(kOffS0 + kDecWarps * 384 <= kOffTab, "slot 0 overlaps the table");
static_assert(kDecSmemEnd <= 232448, "shared memory map exceeds the SM");

struct DecShared {
  int32_t tokidx[kDecMaxPairs + kDecMaxT];
  float pw[kDecMaxPairs + kDecMaxT];
  Run runs[kDecMaxPairs + 1];          // routed runs in ascending expert id; the shared expert's run last
  int32_t n_runs[2];
  int32_t uf[kDecMaxPairs + 2];        // exclusive prefix over the routed runs of their sub-units (<= kDecRows rows each)
  float book[5][16];                   // gate/up routed, shared gate, shared up, down routed, shared down
  int32_t abort;
};
static_assert(sizeof(DecShared) <= kOffWork - kOffRes, "DecShared too large");
static_assert(sizeof(RouteSmallScratch<kDecMaxT>) <= 32768, "routing scratch too large");

struct DecParams {
  Image gu, dn, sh_gu, sh_dn;   // sh_*.data == nullptr: no shared expert
  const float* logits;          // [T][E], or null: ids / w given
  const int32_t* ids;
  const float* w;
  int stride;
  const uint16_t* x;            // bf16 [T][d]
  const uint16_t* gate_w;       // bf16 [d] (shared expert's gate) or null
  int T, E, k, d, mid;
  __half* hid;                  // workspace fp16 [T*k + T][mid]
  uint16_t* out;                // bf16 [T][d], or null with hc_state
  const float* hc_w4;
  uint16_t* hc_state;
  RouteBuffers rb;              // global routing results (written by block 0)
  unsigned* bar;                // [2]: arrival count, generation
  int32_t* status;
};

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32_tab(uint32_t a) {  // table lookups: not volatile, may be scheduled freely
  uint32_t v;
  asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
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

// finite values saturate to the fp16 range, NaN stays NaN
__device__ __forceinline__ float sat_f16(float v) { return v != v ? v : fminf(fmaxf(v, -65504.f), 65504.f); }

// Dot products of one 16-byte chunk (32 codes of one 32-group of the lane's weight row) with the
// matching 32 fp16 activations of NR rows. xa: shared address of row 0's activations, rows
// `row_stride` bytes apart (the same for every lane: broadcast reads). The order of the
// operations of a row does not depend on NR: a row's result is the same alone or in company.
template <int NR>
__device__ __forceinline__ void chunk_dots(const uint4 c, uint32_t lut, uint32_t xa, uint32_t row_stride, float* out) {
  const uint32_t w4[4] = {c.x, c.y, c.z, c.w};
  float s0[NR], s1[NR];
#pragma unroll
  for (int r = 0; r < NR; r++) s0[r] = s1[r] = 0.f;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    uint4 x[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) x[r] = lds128(xa + r * row_stride + q * 16);
    const uint32_t p0 = lds32_tab(__byte_perm(w4[q], lut, 0x7604)), p1 = lds32_tab(__byte_perm(w4[q], lut, 0x7614));
    const uint32_t p2 = lds32_tab(__byte_perm(w4[q], lut, 0x7624)), p3 = lds32_tab(__byte_perm(w4[q], lut, 0x7634));
#pragma unroll
    for (int r = 0; r < NR; r++) {
      fma_pair(s0[r], p0, x[r].x);
      fma_pair(s1[r], p1, x[r].y);
      fma_pair(s0[r], p2, x[r].z);
      fma_pair(s1[r], p3, x[r].w);
    }
  }
#pragma unroll
  for (int r = 0; r < NR; r++) out[r] = s0[r] + s1[r];
}

// ---- ring slot addresses (slot 0: codes in the table's holes, the rest below the table) ----
struct Ring {
  uint32_t hole;   // lane part of a slot-0 code address
  uint32_t s0;     // slot 0 metadata / activation block of this warp
  uint32_t hi;     // slots 1.. of this warp
  int warp, lane;
  __device__ __forceinline__ void init(int w, int l) {
    warp = w;
    lane = l;
    hole = kOffTab + 128 + (uint32_t)(l >> 3) * 256 + (uint32_t)(l & 7) * 16;
    s0 = kOffS0 + (uint32_t)w * 384;
    hi = kOffRing + (uint32_t)w * (kDepth - 1) * kSlotBytes;
  }
  __device__ __forceinline__ uint32_t codes(int s, int h) const {  // this lane's 16 bytes of half h
    return s == 0 ? hole + (uint32_t)(warp * 2 + h) * 1024 : hi + (uint32_t)(s - 1) * kSlotBytes + (uint32_t)h * 512 + (uint32_t)lane * 16;
  }
  __device__ __forceinline__ uint32_t meta(int s) const {  // this lane's 4 bytes
    return (s == 0 ? s0 : hi + (uint32_t)(s - 1) * kSlotBytes + 1024) + (uint32_t)lane * 4;
  }
  __device__ __forceinline__ uint32_t act(int s) const {  // 256 bytes shared by the warp
    return s == 0 ? s0 + 128 : hi + (uint32_t)(s - 1) * kSlotBytes + 1152;
  }
};

// One unit of work of the expert phases: up to kDecRows rows of one expert.
struct Unit {
  const Image* img;
  int expert, first, count;
  bool shared;
};

// Bounded grid-wide barrier. bar[0] counts arrivals, bar[1] is the generation; the last block
// resets the count and bumps the generation. Every block reads the generation before it
// arrives, so the barrier cannot complete (and the generation cannot move) before that read.
// Returns false when the wait gave up after 2 s (status {5, block}); the caller stops working.
__device__ __forceinline__ bool grid_barrier(unsigned* bar, DecShared* res, int32_t* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned gen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(bar + 1) : "memory");
    __threadfence();
    const unsigned old = atomicAdd(bar, 1u);
    if (old == gridDim.x - 1) {
      bar[0] = 0;
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + 1), "r"(gen + 1) : "memory");
    } else {
      unsigned long long t0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      for (uint32_t spin = 0;; spin++) {
        unsigned g;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(g) : "l"(bar + 1) : "memory");
        if (g != gen) break;
        if ((spin & 63u) == 63u) {
          unsigned long long t1;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
          if (t1 - t0 > 2000000000ull) {
            if (atomicCAS(status, 0, 5) == 0) status[1] = (int)blockIdx.x;
            res->abort = 1;
            break;
          }
          __nanosleep(100);
        }
      }
    }
  }
  __syncthreads();
  return res->abort == 0;
}

__global__ void __launch_bounds__(kDecThreads, 1)
k_decode(const DecParams p) {
  extern __shared__ __align__(16) uint8_t dsm[];
  const uint32_t dyn0 = (uint32_t)__cvta_generic_to_shared(dsm);
  uint8_t* const smem = dsm - dyn0;  // smem + A is the generic pointer of absolute shared address A
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  {
    uint32_t dyn_size;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (dyn0 > kOffLow || dyn0 + dyn_size < kDecSmemEnd) {
      // the fixed map does not fit this launch: refuse (uniform for the grid; nobody reaches the barrier)
      if (tid == 0 && atomicCAS(p.status, 0, 2) == 0) p.status[1] = (int)dyn0;
      return;
    }
  }
  DecShared* const res = (DecShared*)(smem + kOffRes);
  const bool has_sh = p.sh_gu.data != nullptr;
  const int T = p.T, P = p.T * p.k, mid = p.mid, d = p.d;
  pdl_trigger();

  // ---- code books (weights: nothing an earlier kernel of the stream writes) ----
  if (tid < 80) {
    const int b = tid >> 4, e = tid & 15;
    float v = 0.f;
    if (b == 0) v = p.gu.book[e];
    else if (b == 3) v = p.dn.book[e];
    else if (has_sh) v = b == 1 ? p.sh_gu.book[e] : b == 2 ? p.sh_gu.book[(p.sh_gu.dual_book ? 16 : 0) + e] : p.sh_dn.book[e];
    res->book[b][e] = v;
  }
  if (tid == 0) res->abort = 0;
  __syncthreads();
  // table entry of code byte b for lane l: (f16(book[b & 15]), f16(book[b >> 4])), lanes 0..15
  // from book `lo`, lanes 16..31 from book `hi` (gate rows and up rows of the shared expert
  // come from different tensors). Warp w writes the 8 lines whose high code is w >> 1 ...
  auto build_table = [&](int lo, int hi) {
    const float* bk = res->book[lane < 16 ? lo : hi];
    const int hc = warp >> 1;
    const uint32_t hi16 = (uint32_t)__half_as_ushort(__float2half_rn(bk[hc])) << 16;
#pragma unroll
    for (int c = 0; c < 8; c++) {
      const int lc = (warp & 1) * 8 + c;
      sts32(kOffTab + (uint32_t)(hc * 16 + lc) * 256 + (uint32_t)lane * 4, hi16 | (uint32_t)__half_as_ushort(__float2half_rn(bk[lc])));
    }
  };
  enum { kTabNone = 0, kTabUpRouted, kTabUpShared, kTabDnRouted, kTabDnShared };
  int cur_tab = kTabUpRouted;
  build_table(0, 0);
  pdl_wait();  // from here on: inputs an earlier kernel may have written, buffers it may still read

  // ---- routing, repeated by every block for itself (threads 0..511) ----
  if (warp < 16) {
    RouteSmallScratch<kDecMaxT>& sc = *(RouteSmallScratch<kDecMaxT>*)(smem + kOffWork);
    RouteSmallOut loc, glob;
    loc.tokidx = res->tokidx;
    loc.pw = res->pw;
    loc.runs = res->runs;
    loc.shared_slot = kDecMaxPairs;
    loc.n_runs = res->n_runs;
    if (blockIdx.x == 0) {
      glob.topids = p.rb.topids; glob.topw = p.rb.topw; glob.tokidx = p.rb.tokidx; glob.pw = p.rb.pw;
      glob.pairids = p.rb.pairids; glob.eoff = p.rb.eoff; glob.runs = p.rb.runs; glob.shared_slot = kMaxExperts;
      glob.n_runs = p.rb.n_runs; glob.tiles = p.rb.tiles; glob.tiles_sh = p.rb.tiles_sh; glob.n_tiles = p.rb.n_tiles;
      glob.sgate = p.rb.sgate;
    }
    route_small_body<kDecMaxT>(p.logits, p.ids, p.w, p.stride, T, p.E, p.k, p.x, has_sh ? p.gate_w : nullptr, d, sc, loc,
                               glob, blockIdx.x == 0 ? p.status : nullptr);
  }
  __syncthreads();
  const int n_routed = min(res->n_runs[0], kDecMaxPairs);
  if (warp == 0) {
    // exclusive prefix of the runs' sub-unit counts
    int carry = 0;
    for (int i0 = 0; i0 < n_routed; i0 += 32) {
      const int i = i0 + lane;
      const int n = i < n_routed ? (res->runs[i].count + kDecRows - 1) / kDecRows : 0;
      int incl = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (i < n_routed) res->uf[i] = carry + incl - n;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) res->uf[n_routed] = carry;
  }
  __syncthreads();
  const int nu_routed = res->uf[n_routed];
  const int nu_shared = has_sh ? (T + kDecRows - 1) / kDecRows : 0;
  // sub-unit v of the routed runs
  auto routed_unit = [&](int v) -> Unit {
    int lo = v, hi = n_routed - 1;
    if (nu_routed != n_routed) {  // some run has more than kDecRows rows: search the prefix
      lo = 0;
      while (lo < hi) {
        const int m = (lo + hi + 1) >> 1;
        if (res->uf[m] <= v) lo = m; else hi = m - 1;
      }
    }
    const Run r = res->runs[lo];
    const int sub = v - res->uf[lo];
    return Unit{nullptr, r.expert, r.first + sub * kDecRows, min(kDecRows, r.count - sub * kDecRows), false};
  };
  auto shared_unit = [&](int v) -> Unit {
    return Unit{nullptr, 0, P + v * kDecRows, min(kDecRows, T - v * kDecRows), true};
  };

  Ring ring;
  ring.init(warp, lane);
  const uint32_t lut = (kOffTab & 0xFFFF0000u) | 0x00010000u | (uint32_t)(lane * 4);  // bytes {lane*4, -, 1, 0}: table at 64 KB
  constexpr size_t tile_b = tile_bytes(kQ4CP);

  // =========================== gate/up + SwiGLU ===========================
  // Units: the shared expert's sub-units first, then the routed ones. A task = 16 hidden outputs
  // of a unit (lanes 0..15 the gate rows, lanes 16..31 the matching up rows); the 32 warps split
  // K (kpw K blocks each). The tasks are cut into one contiguous range per block.
  {
    const int KB = d / kTileK;
    const int kpw = (KB + kDecWarps - 1) / kDecWarps;
    const int kb0 = warp * kpw;
    const int tpu = mid / 16;
    const long long total = (long long)(nu_shared + nu_routed) * tpu;
    const long long base = total / gridDim.x, rem = total % gridDim.x;
    const long long c0 = blockIdx.x * base + min((long long)blockIdx.x, rem);
    const int n_tasks = (int)(base + ((long long)blockIdx.x < rem ? 1 : 0));
    const int n_items = n_tasks * kpw;
    auto unit_of = [&](int task) -> Unit {
      const int u = (int)((c0 + task) / tpu);
      Unit un = u < nu_shared ? shared_unit(u) : routed_unit(u - nu_shared);
      un.img = un.shared ? &p.sh_gu : &p.gu;
      return un;
    };
    // item i of this warp = (task i / kpw, K block kb0 + i % kpw)
    int iss_task = -1;
    Unit iss_u{};
    auto issue = [&](int i) {
      if (i < n_items) {
        const int task = i / kpw, kb = kb0 + i % kpw;
        if (kb < KB) {
          if (task != iss_task) {
            iss_u = unit_of(task);
            iss_task = task;
          }
          const Unit& un = iss_u;
          const int j = (int)((c0 + task) % tpu);
          const int s = i % kDepth;
          const int row = (lane < 16 ? 0 : 48) + (j & 3) * 16 + lane;  // gate rows 0..63, up rows 64..127 of the tile
          const uint8_t* tp = un.img->data + (((size_t)un.expert * un.img->n_mtiles + (j >> 2)) * un.img->n_kblocks + kb) * tile_b;
          cp16(ring.codes(s, 0), tp + row * 16);
          cp16(ring.codes(s, 1), tp + 2048 + row * 16);
          cp4(ring.meta(s), tp + kCodeBytes + row * 4);
          if (lane < un.count * 8) {
            const int r = lane >> 3, piece = lane & 7;
            cp16(ring.act(s) + r * 128 + piece * 16, p.x + (size_t)res->tokidx[un.first + r] * d + kb * kTileK + piece * 8);
          }
        }
      }
      cp_commit();
    };
#pragma unroll
    for (int i = 0; i < kDepth; i++) issue(i);
    float acc[kDecRows] = {0.f, 0.f};
    int buf = 0;
    Unit un{};
    for (int i = 0; i < n_items; i++) {
      const int task = i / kpw, ik = i % kpw, kb = kb0 + ik, s = i % kDepth;
      if (ik == 0) un = unit_of(task);  // (block-uniform)
      if (ik == 0) {
        const int need = un.shared ? kTabUpShared : kTabUpRouted;
        if (need != cur_tab) {  // every warp has passed the previous task's barrier: nobody reads the old table
          if (un.shared) build_table(1, 2); else build_table(0, 0);
          cur_tab = need;
          __syncthreads();
        }
      }
      cp_wait<kDepth - 1>();
      __syncwarp();
      if (kb < KB) {
        // activations bf16 -> fp16 in place (finite values saturate; exact for |v| in [2^-14, 65504])
        const uint32_t xa = ring.act(s);
        for (int r = 0; r < un.count; r++) {
          const uint32_t u = lds32(xa + r * 128 + lane * 4);
          const __half2 h = __floats2half2_rn(sat_f16(__uint_as_float(u << 16)), sat_f16(__uint_as_float(u & 0xFFFF0000u)));
          sts32(xa + r * 128 + lane * 4, *(const uint32_t*)&h);
        }
        __syncwarp();
        const uint4 ca = lds128(ring.codes(s, 0)), cb = lds128(ring.codes(s, 1));
        const uint32_t m = lds32(ring.meta(s));
        const float sc0 = half_bits_to_f32((uint16_t)(m & 0xFFFFu)), sc1 = half_bits_to_f32((uint16_t)(m >> 16));
        float d0[kDecRows], d1[kDecRows];
        if (un.count == 1) {
          chunk_dots<1>(ca, lut, xa, 128, d0);
          chunk_dots<1>(cb, lut, xa + 64, 128, d1);
          acc[0] += sc0 * d0[0] + sc1 * d1[0];
        } else {
          chunk_dots<2>(ca, lut, xa, 128, d0);
          chunk_dots<2>(cb, lut, xa + 64, 128, d1);
          acc[0] += sc0 * d0[0] + sc1 * d1[0];
          acc[1] += sc0 * d0[1] + sc1 * d1[1];
        }
      }
      __syncwarp();  // the slot is free for the copy that follows
      issue(i + kDepth);
      if (ik == kpw - 1) {
        // ---- end of a task: the K slices meet in shared memory; warp r adds row r in slice order ----
        float* red = (float*)(smem + kOffWork) + buf * (kDecRows * kDecWarps * 32);
#pragma unroll
        for (int r = 0; r < kDecRows; r++) red[(r * kDecWarps + warp) * 32 + lane] = acc[r];
        __syncthreads();
        if (warp < un.count) {
          float tot = 0.f;
#pragma unroll
          for (int w = 0; w < kDecWarps; w++) tot += red[(warp * kDecWarps + w) * 32 + lane];
          const float up = __shfl_down_sync(0xffffffffu, tot, 16);
          const int j = (int)((c0 + task) % tpu);
          if (lane < 16) p.hid[(size_t)(un.first + warp) * mid + j * 16 + lane] = __float2half_rn(sat_f16(silu_f32(tot) * up));
        }
        buf ^= 1;
        acc[0] = acc[1] = 0.f;
      }
    }
    cp_wait<0>();
  }

  // =========================== down + weighted combine ===========================
  // A block owns 32 rows of the output (one warp-row of a weight tile) for every token: units in
  // ascending expert order, the shared expert last; the 32 warps split K in 32-wide groups; a
  // warp keeps its partial sums per token in shared memory, the block adds them at the end.
  const int n_rb = d / 32;
  const int GH = mid / 32;                                   // 32-groups along K
  const int hpw = (GH + kDecWarps - 1) / kDecWarps;           // groups per warp (1 for mid <= 1024)
  const int nu_all = nu_routed + nu_shared;
  auto unit_dn = [&](int u) -> Unit {
    Unit un = u < nu_routed ? routed_unit(u) : shared_unit(u - nu_routed);
    un.img = un.shared ? &p.sh_dn : &p.dn;
    return un;
  };
  const int my_first_rb = blockIdx.x;
  // item i of this warp for row block rb = (unit i / hpw, group warp + 32 * (i % hpw))
  auto issue_dn = [&](int rb, int i, int n_items, bool with_act) {
    if (i < n_items) {
      const int u = i / hpw, hb = warp + kDecWarps * (i % hpw);
      if (hb < GH) {
        const Unit un = unit_dn(u);
        const int s = i % kDepth;
        const int row = (rb & 3) * 32 + lane;
        const uint8_t* tp = un.img->data + (((size_t)un.expert * un.img->n_mtiles + (rb >> 2)) * un.img->n_kblocks + (hb >> 1)) * tile_b;
        cp16(ring.codes(s, 0), tp + (hb & 1) * 2048 + row * 16);
        cp4(ring.meta(s), tp + kCodeBytes + row * 4);
        if (with_act && lane < un.count * 4) {
          const int r = lane >> 2, piece = lane & 3;
          cp16(ring.act(s) + r * 64 + piece * 16, p.hid + (size_t)(un.first + r) * mid + hb * 32 + piece * 8);
        }
      }
    }
    cp_commit();
  };
  auto issue_act_only = [&](int i, int n_items) {
    if (i < n_items) {
      const int u = i / hpw, hb = warp + kDecWarps * (i % hpw);
      if (hb < GH) {
        const Unit un = unit_dn(u);
        const int s = i % kDepth;
        if (lane < un.count * 4) {
          const int r = lane >> 2, piece = lane & 3;
          cp16(ring.act(s) + r * 64 + piece * 16, p.hid + (size_t)(un.first + r) * mid + hb * 32 + piece * 8);
        }
      }
    }
  };
  const int n_items_dn = nu_all * hpw;
  // the first weights of the down phase travel while the blocks meet at the barrier
  if (my_first_rb < n_rb)
    for (int i = 0; i < kDepth; i++) issue_dn(my_first_rb, i, n_items_dn, false);
  if (!grid_barrier(p.bar, res, p.status)) {
    cp_wait<0>();
    return;
  }
  for (int rb = my_first_rb; rb < n_rb; rb += gridDim.x) {
    float* sacc = (float*)(smem + kOffWork) + (size_t)warp * kDecMaxT * 32;
    for (int t = 0; t < T; t++) sacc[t * 32 + lane] = 0.f;
    if (rb == my_first_rb) {
      for (int i = 0; i < kDepth; i++) issue_act_only(i, n_items_dn);  // the hidden rows exist only now
      cp_commit();
      cp_wait<0>();
    } else {
      for (int i = 0; i < kDepth; i++) issue_dn(rb, i, n_items_dn, true);
    }
    __syncwarp();
    for (int i = 0; i < n_items_dn; i++) {
      const int u = i / hpw, hb = warp + kDecWarps * (i % hpw), s = i % kDepth;
      const Unit un = unit_dn(u);  // (block-uniform)
      if (i % hpw == 0) {
        const int need = un.shared ? kTabDnShared : kTabDnRouted;
        if (need != cur_tab) {
          __syncthreads();  // every warp is done with the table that is replaced
          if (un.shared) build_table(4, 4); else build_table(3, 3);
          cur_tab = need;
          __syncthreads();
        }
      }
      cp_wait<kDepth - 1>();
      __syncwarp();
      if (hb < GH) {
        const uint4 c = lds128(ring.codes(s, 0));
        const uint32_t m = lds32(ring.meta(s));
        const float scale = half_bits_to_f32((uint16_t)((hb & 1) ? (m >> 16) : (m & 0xFFFFu)));
        float dots[kDecRows];
        if (un.count == 1) chunk_dots<1>(c, lut, ring.act(s), 64, dots);
        else chunk_dots<2>(c, lut, ring.act(s), 64, dots);
#pragma unroll
        for (int r = 0; r < kDecRows; r++)
          if (r < un.count) {
            const int t = res->tokidx[un.first + r];
            sacc[t * 32 + lane] += res->pw[un.first + r] * (scale * dots[r]);
          }
      }
      __syncwarp();
      issue_dn(rb, i + kDepth, n_items_dn, true);
    }
    cp_wait<0>();
    __syncthreads();
    if (warp < T) {
      const float* all = (const float*)(smem + kOffWork);
      float y = 0.f;
#pragma unroll 8
      for (int w = 0; w < kDecWarps; w++) y += all[((size_t)w * kDecMaxT + warp) * 32 + lane];
      const int col = rb * 32 + lane;
      if (p.hc_w4) {
        // write-back into the four branches of the bf16 residual state (k_moe_reduce_pw_sg_hc)
#pragma unroll
        for (int b = 0; b < 4; b++) {
          const float inj = 2.f / (1.f + expf(-p.hc_w4[(size_t)warp * 4 + b] * 0.25f));
          uint16_t* q = p.hc_state + ((size_t)warp * 4 + b) * d + col;
          const __nv_bfloat16 o = __float2bfloat16_rn(fmaf(inj, y, bf16_bits_to_f32(*q)));
          *q = *(const uint16_t*)&o;
        }
      } else {
        const __nv_bfloat16 o = __float2bfloat16_rn(y);
        p.out[(size_t)warp * d + col] = *(const uint16_t*)&o;
      }
    }
    __syncthreads();  // the partial sums are cleared by the next row block
  }
}

}  // namespace

int decode_max_tokens() { return kDecMaxT; }

bool decode_supported(const Image& gu, const Image& dn, const Image* sh_gu, const Image* sh_dn, int T, int k, int E, int d, int mid) {
  if (T < 1 || T > kDecMaxT || T * k > kDecMaxPairs || T * k > route_small_max_pairs() || E > kMaxExperts) return false;
  if (gu.fmt != kQ4CP || dn.fmt != kQ4CP || gu.dual_book) return false;
  if (sh_gu && (sh_gu->fmt != kQ4CP || !sh_dn || sh_dn->fmt != kQ4CP)) return false;
  return d % 128 == 0 && mid % 64 == 0;
}

cudaError_t launch_decode(const Image& gu, const Image& dn, const Image* sh_gu, const Image* sh_dn, const float* logits,
                          const int32_t* ids, const float* w, int stride, const void* x_bf16, const uint16_t* gate_w, int T,
                          int E, int k, int d, int mid, __half* hid16, void* out_bf16, const float* hc_w4, void* hc_state,
                          const RouteBuffers& rb, unsigned* bar, int32_t* status, cudaStream_t st) {
  static bool attr_done = false;
  static int sms = 0;
  const int smem = (int)(kDecSmemEnd - 1024);
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k_decode, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    int dev = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // the grid-wide barrier needs every block resident at once: one block per SM must fit
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode, kDecThreads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1 || sms < 1) return cudaErrorLaunchOutOfResources;
    attr_done = true;
  }
  DecParams p{};
  p.gu = gu;
  p.dn = dn;
  if (sh_gu) p.sh_gu = *sh_gu;
  if (sh_dn) p.sh_dn = *sh_dn;
  p.logits = logits; p.ids = ids; p.w = w; p.stride = stride;
  p.x = (const uint16_t*)x_bf16; p.gate_w = gate_w;
  p.T = T; p.E = E; p.k = k; p.d = d; p.mid = mid;
  p.hid = hid16; p.out = (uint16_t*)out_bf16; p.hc_w4 = hc_w4; p.hc_state = (uint16_t*)hc_state;
  p.rb = rb; p.bar = bar; p.status = status;
  return launch_pdl(k_decode, dim3(sms), dim3(kDecThreads), (size_t)smem, st, p);
}

}  // namespace b200moe
