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
//   * the warps of a block never meet at a block-wide barrier inside a phase: at the end of a
//     task a warp leaves its partial sums in shared memory, bumps a counter and goes on; one
//     warp per task (they take turns) waits for the 32 arrivals and adds the sums in a fixed order;
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
constexpr int kMaxRecs = kDecMaxPairs + kDecMaxT;  // task / unit records held at a time
constexpr int kRedBufs = 4;        // partial-sum buffers of the gate/up phase (tasks in flight per block)

// ---- shared-memory map, absolute addresses of the block's shared window ----
// The lookup table has one 256-byte line per code byte of which the first 128 bytes hold the
// 32 lane copies of the entry; it sits on a 64 KB boundary so that a lookup address is one
// byte permute {lane*4, code byte, 1, 0}. The second halves of the lines (256 "work rows" of
// 32 floats) hold the partial sums the warps of a block exchange.
constexpr uint32_t kOffLow = 2048;     // the dynamic allocation must start at or below this
constexpr uint32_t kOffRes = 2048;     // DecShared
constexpr uint32_t kOffRec = 6144;     // task / unit records (kMaxRecs x 32 B)
constexpr uint32_t kOffS0 = 12288;     // ring slot 0 of every warp
constexpr uint32_t kOffTab = 65536;    // 256 lines x 256 B
constexpr uint32_t kOffRing = 131072;  // ring slots 1, 2 of every warp; the routing scratch before that
constexpr uint32_t kSlotBytes = 1536;  // 1024 code bytes + 256 metadata + 256 activation slices
constexpr uint32_t kDecSmemEnd = kOffRing + kDecWarps * (kDepth - 1) * kSlotBytes;  // 229376
static_assert(kOffRec + kMaxRecs * 32 <= kOffS0, "records overlap the ring");
static_assert(kOffS0 + kDecWarps * kSlotBytes <= kOffTab, "slot 0 overlaps the table");
static_assert(kDecSmemEnd <= 232448, "shared memory map exceeds the SM");
static_assert(kRedBufs * kDecRows * kDecWarps == 256 && kDecWarps * kDecMaxT == 256, "work rows");

struct DecShared {
  int32_t tokidx[kDecMaxPairs + kDecMaxT];
  float pw[kDecMaxPairs + kDecMaxT];
  Run runs[kDecMaxPairs + 1];          // routed runs in ascending expert id; the shared expert's run last
  int32_t n_runs[2];
  int32_t uf[kDecMaxPairs + 2];        // exclusive prefix over the routed runs of their sub-units (<= kDecRows rows each)
  int32_t uw[kMaxRecs + 2];            // exclusive prefix over the gate/up units of their cost per task
  float book[5][16];                   // gate/up routed, shared gate, shared up, down routed, shared down
  int32_t cnt[kRedBufs];               // arrivals at each partial-sum buffer (never reset)
  int32_t done[kRedBufs];              // uses of each buffer that have been added up
  int32_t abort;
};
static_assert(sizeof(DecShared) <= kOffRec - kOffRes, "DecShared too large");
static_assert(sizeof(RouteSmallScratch<kDecMaxT>) <= kDecSmemEnd - kOffRing, "routing scratch too large");

// One gate/up task (16 hidden outputs of up to kDecRows rows of one expert) or one down unit.
struct __align__(16) Rec {
  const uint8_t* base;  // the expert's weight tile of K block 0 (gate/up: m-tile of the task; down: m-tile of the row block)
  int first;            // first permuted row
  int info;             // rows | shared expert << 8 | task index within the unit << 16
  int tok0, tok1;       // tokens of the rows
  float pw0, pw1;       // their combine weights
};
static_assert(sizeof(Rec) == 32, "Rec is two 16-byte loads");

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
  unsigned long long* bar;      // arrival counter of the grid-wide barrier (never reset)
  int32_t* status;
  unsigned long long* trace;    // debug: [blocks][8] nanosecond stamps of the phase boundaries, or null
};

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds32_tab(uint32_t a) {  // table lookups: may be scheduled freely
  uint32_t v;
  asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
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
// two bf16 values -> two fp16 values (round to nearest, magnitudes beyond the fp16 range saturate)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t u) {
  uint32_t h;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(__uint_as_float(u & 0xFFFF0000u)), "f"(__uint_as_float(u << 16)));
  return h;
}

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

// Bounded spin on a counter in shared memory that other warps of the block advance. Gives up
// after ~2 s (status {6, site}) and lets the block run on: the result is then flagged, not hung.
__device__ __forceinline__ void wait_shared_ge(const int32_t* ctr, int target, DecShared* res, int32_t* status, int site) {
  const volatile int32_t* v = ctr;
  if (*v >= target) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t spin = 1;; spin++) {
    if (*v >= target) return;
    __nanosleep(32);  // a waiting warp must not take issue slots from the warps it waits for
    if ((spin & 1023u) == 0) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (res->abort || t1 - t0 > 2000000000ull) {
        if (atomicCAS(status, 0, 6) == 0) status[1] = site;
        res->abort = 1;
        return;
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Routing inside the decode kernel. The general body (route_small.cuh) follows the reference's
// arithmetic to the letter -- double exp, double index-order sum, double divisions -- and is
// ~5000 instructions of mostly straight-line code that each launch runs once with a cold
// instruction cache: ~12 us, a quarter of a one-token call. This version decides the SAME
// top-k ids and order from the logits themselves (exp and the division by the sum are
// monotone, so "largest probability, ties to the lowest id" is "largest logit, ties to the
// lowest id" unless two different logits round to one float probability) and is a few hundred
// instructions. Where two logits of a token's k+1 largest are closer than 1e-6 -- the only case in
// which their probabilities could round to the same float -- or a logit is not finite, the block
// runs the general body instead, so the ids are the reference's in every case. The weights
// p_i / sum of the selected p come from float exponentials: within ~2e-7 of the reference's
// (its own rounding of p to float is 6e-8); the sum over all experts cancels and is not formed.
struct FastScratch {
  double gpart[kDecMaxT][16];     // shared expert's gate: partial sums of the 16 gate warps
  float wmax[kDecMaxT][16];       // per token: maxima of the 16 groups of 32 experts
  float mx[kDecMaxT], bound[kDecMaxT];
  int32_t ccount[kDecMaxT];
  int32_t fallback;
  int32_t wcnt[16];
  float sel_v[kDecMaxT][17];
  int32_t sel_id[kDecMaxT][17];
  int32_t key[kDecMaxPairs];      // selected expert of pair t*k + s
  float w[kDecMaxPairs];
  float cand_v[kDecMaxT][kMaxExperts];
  int32_t cand_id[kDecMaxT][kMaxExperts];
};
static_assert(sizeof(FastScratch) + sizeof(RouteSmallScratch<kDecMaxT>) <= kDecSmemEnd - kOffRing, "routing scratch too large");

struct RouteOuts {
  RouteSmallOut loc, glob;
};

// The general body, kept out of line: the fast path's instruction footprint stays small.
__device__ __noinline__ void route_exact(const DecParams& p, RouteSmallScratch<kDecMaxT>* sc, const RouteOuts* o, int32_t* status) {
  route_small_body<kDecMaxT, 2>(p.logits, p.ids, p.w, p.stride, p.T, p.E, p.k, p.x, nullptr, p.d, *sc, o->loc, o->glob, status);
}

// Threads 0..511. Fills fs.key / fs.w (pair order) from the logits; returns false when the
// general body has to run instead.
__device__ __forceinline__ bool route_fast_select(const DecParams& p, FastScratch& fs, const RouteSmallOut& glob) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.T, E = p.E, k = p.k;
  // (the few logits of a thread are re-read from the cache in each step instead of being kept in
  // registers: the loops over the tokens stay rolled and the code small)
  bool odd = false;  // a logit that is NaN or infinite
  if (tid < kDecMaxT) fs.ccount[tid] = 0;
  if (tid == 0) fs.fallback = 0;
#pragma unroll 1
  for (int t = 0; t < T; t++) {
    float m = tid < E ? p.logits[(size_t)t * E + tid] : -INFINITY;
    if (tid < E && !(fabsf(m) <= 3.0e38f)) odd = true;
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) fs.wmax[t][warp] = m;
  }
  if (__any_sync(0xffffffffu, odd) && lane == 0) fs.fallback = 1;
  rs_sync();
  if (warp < T) {
    // the k-th largest of the 16 group maxima is a lower bound of the k-th largest logit
    const float m = lane < 16 ? fs.wmax[warp][lane] : -INFINITY;
    int rank = 0;
    float mxv = m;
#pragma unroll 4
    for (int i = 0; i < 16; i++) {
      const float o = __shfl_sync(0xffffffffu, m, i);
      rank += (o > m) || (o == m && i < lane);
      mxv = fmaxf(mxv, o);
    }
    const unsigned hit = __ballot_sync(0xffffffffu, lane < 16 && rank == min(k, 16) - 1);
    const float bound = hit ? __shfl_sync(0xffffffffu, m, __ffs(hit) - 1) : -INFINITY;
    if (lane == 0) {
      fs.bound[warp] = bound;
      fs.mx[warp] = mxv;
    }
  }
  rs_sync();
#pragma unroll 1
  for (int t = 0; t < T; t++) {
    const float vt = tid < E ? p.logits[(size_t)t * E + tid] : -INFINITY;
    const bool c = tid < E && vt >= fs.bound[t];
    const unsigned bal = __ballot_sync(0xffffffffu, c);
    int base = 0;
    if (lane == 0 && bal) base = atomicAdd(&fs.ccount[t], __popc(bal));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (c) {
      const int pos = base + __popc(bal & ((1u << lane) - 1u));
      fs.cand_v[t][pos] = vt;
      fs.cand_id[t][pos] = tid;
    }
  }
  rs_sync();
  // rank of every candidate among its token's candidates: (logit descending, id ascending)
#pragma unroll 1
  for (int t = 0; t < T; t++) {
    const int C = fs.ccount[t];
    if (tid < C) {
      const float mv = fs.cand_v[t][tid];
      const int mi = fs.cand_id[t][tid];
      int rank = 0;
#pragma unroll 4
      for (int i = 0; i < C; i++) {
        const float o = fs.cand_v[t][i];
        rank += (o > mv) || (o == mv && fs.cand_id[t][i] < mi);
      }
      if (rank <= k) {
        fs.sel_v[t][rank] = mv;
        fs.sel_id[t][rank] = mi;
      }
    }
  }
  rs_sync();
  if (warp < T) {
    const int t = warp, C = fs.ccount[t];
    const float vr = (lane <= k && lane < C) ? fs.sel_v[t][lane] : -INFINITY;
    const int id = (lane < k && lane < C) ? fs.sel_id[t][lane] : 0;
    const float vn = __shfl_down_sync(0xffffffffu, vr, 1);
    // neighbours in the order closer than 1e-6: their probabilities might round to one float
    const bool close = lane < k && lane + 1 < C && !(vr - vn > 1e-6f * fmaxf(1.f, fabsf(vr)));
    if (__any_sync(0xffffffffu, close) || C < k) {
      if (lane == 0) fs.fallback = 1;
    }
    const float ef = lane < k ? expf(vr - fs.mx[t]) : 0.f;
    double kept = 0;
#pragma unroll 1
    for (int r = 0; r < k; r++) kept += (double)__shfl_sync(0xffffffffu, ef, r);  // rank order, as the reference adds
    const float wv = lane < k ? (float)((double)ef / kept) : 0.f;
    if (lane < kIdStride) {
      if (glob.topids) {
        glob.topids[(size_t)t * kIdStride + lane] = id;
        glob.topw[(size_t)t * kIdStride + lane] = wv;
      }
      if (lane < k) {
        fs.key[t * k + lane] = id;
        fs.w[t * k + lane] = wv;
      }
    }
  }
  rs_sync();
  return fs.fallback == 0;
}

// Threads 0..511: stable bucketing of the P = T*k pairs in fs.key / fs.w by expert (rank counting),
// expert offsets, runs. Same definitions as the general body's.
__device__ __forceinline__ void route_fast_place(const DecParams& p, FastScratch& fs, const RouteSmallOut& loc,
                                                 const RouteSmallOut& glob) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.T, E = p.E, k = p.k, P = T * k;
  int n_bad = 0;
  if (tid < P) {
    const int key = fs.key[tid], t = tid / k;
    int row = 0, rank = 0;
#pragma unroll 4
    for (int q = 0; q < P; q++) {
      const int kq = fs.key[q];
      row += (kq < key) || (kq == key && q < tid);
      n_bad += kq == kBadKey;
    }
#pragma unroll 1
    for (int q = t * k; q < t * k + k; q++) rank += (fs.key[q] < key) || (fs.key[q] == key && q < tid);
    loc.tokidx[row] = t;
    loc.pw[row] = fs.w[tid];
    if (glob.tokidx) {
      glob.tokidx[row] = t;
      glob.pw[row] = fs.w[tid];
      glob.pairids[(size_t)t * k + rank] = key == kBadKey ? -1 : row;
    }
  }
  int cnt = 0, lt = 0;
  if (tid < E) {
#pragma unroll 4
    for (int q = 0; q < P; q++) {
      const int kq = fs.key[q];
      cnt += kq == tid;
      lt += kq < tid;
    }
  }
  const unsigned active = __ballot_sync(0xffffffffu, cnt > 0);
  if (lane == 0) fs.wcnt[warp] = __popc(active);
  rs_sync();
  int before = __popc(active & ((1u << lane) - 1u)), n_active = 0;
#pragma unroll 1
  for (int w2 = 0; w2 < 16; w2++) {
    if (w2 < warp) before += fs.wcnt[w2];
    n_active += fs.wcnt[w2];
  }
  if (tid < E && glob.eoff) glob.eoff[tid] = lt;
  if (cnt > 0) {
    loc.runs[before] = Run{tid, lt, cnt};
    if (glob.runs) {
      glob.runs[before] = Run{tid, lt, cnt};
      glob.tiles[before] = Tile{tid, lt, cnt};
    }
  }
  if (tid == 0) {
    loc.n_runs[0] = n_active;
    if (glob.runs) {
      glob.eoff[E] = P - n_bad;
      glob.n_runs[0] = n_active;
      glob.n_runs[1] = 1;
      glob.runs[kMaxExperts] = Run{0, P, T};
      glob.n_tiles[0] = n_active;
      glob.n_tiles[1] = 1;
      glob.tiles_sh[0] = Tile{0, P, T};
    }
  }
}

// Bounded grid-wide barrier on ONE 64-bit arrival counter that is never reset: every launch
// adds gridDim.x to it, so a block that read the counter at any time before its own arrival
// (target_of) knows the value that means "all blocks of this launch have arrived" -- the next
// multiple of the grid size. One release-add and acquire polls; no reset, no second word.
// Returns false when the wait gave up after 2 s (status {5, block}); the caller stops working.
__device__ __forceinline__ unsigned long long barrier_target(const unsigned long long* ctr) {
  unsigned long long c;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(ctr) : "memory");
  return (c / gridDim.x + 1) * gridDim.x;
}
__device__ __forceinline__ bool grid_barrier(unsigned long long* ctr, unsigned long long target, DecShared* res, int32_t* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long old;
    asm volatile("atom.add.release.gpu.global.u64 %0, [%1], 1;" : "=l"(old) : "l"(ctr) : "memory");
    if (old + 1 < target) {
      unsigned long long t0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      for (uint32_t spin = 0;; spin++) {
        unsigned long long c;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(ctr) : "memory");
        if (c >= target) break;
        if ((spin & 63u) == 63u) {
          unsigned long long t1;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
          if (t1 - t0 > 2000000000ull) {
            if (atomicCAS(status, 0, 5) == 0) status[1] = (int)blockIdx.x;
            res->abort = 1;
            break;
          }
        }
      }
    } else {
      __threadfence();  // (acquire side of the last arrival)
    }
  }
  __syncthreads();
  return res->abort == 0;
}

#define DEC_TRACE(slot)                                                        \
  do {                                                                         \
    if (p.trace && threadIdx.x == 0) {                                         \
      unsigned long long t_;                                                   \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                   \
      p.trace[(size_t)blockIdx.x * 8 + (slot)] = t_;                           \
    }                                                                          \
  } while (0)

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
  DEC_TRACE(0);
  unsigned long long bar_target = 0;
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
  if (tid < kRedBufs) res->cnt[tid] = res->done[tid] = 0;
  if (tid == 0) res->abort = 0;
  __syncthreads();
  // table entry of code byte b for lane l: (f16(book[b & 15]), f16(book[b >> 4])), lanes 0..15
  // from book `lo`, lanes 16..31 from book `hi` (gate rows and up rows of the shared expert
  // come from different tensors). Warp w writes the lines whose high code is w >> 1.
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
  DEC_TRACE(1);
  if (tid == 0) bar_target = barrier_target(p.bar);  // (long before this block's own arrival; only thread 0 uses it)

  // ---- routing, repeated by every block for itself: warps 0..15 the router and the bucketing,
  // warps 16..31 the shared expert's scalar gate (src/ref.cpp:623-626: a d-long dot product in double) ----
  FastScratch& fs = *(FastScratch*)(smem + kOffRing);
  if (warp < 16) {
    auto fill_outs = [&](RouteSmallOut& loc, RouteSmallOut& glob) {
      loc.tokidx = res->tokidx;
      loc.pw = res->pw;
      loc.runs = res->runs;
      loc.shared_slot = kDecMaxPairs;
      loc.n_runs = res->n_runs;
      if (blockIdx.x == 0) {
        glob.topids = p.rb.topids; glob.topw = p.rb.topw; glob.tokidx = p.rb.tokidx; glob.pw = p.rb.pw;
        glob.pairids = p.rb.pairids; glob.eoff = p.rb.eoff; glob.runs = p.rb.runs; glob.shared_slot = kMaxExperts;
        glob.n_runs = p.rb.n_runs; glob.tiles = p.rb.tiles; glob.tiles_sh = p.rb.tiles_sh; glob.n_tiles = p.rb.n_tiles;
      }
    };
    RouteSmallOut loc, glob;
    fill_outs(loc, glob);
    bool placed = false;
    if (p.logits) {
      if (route_fast_select(p, fs, glob)) {
        route_fast_place(p, fs, loc, glob);
        placed = true;
      }
    } else {
      // the caller's ids: an id outside [0, E) must never index anything -- the pair is dropped
      // (its key sorts behind every expert) and the status word records it
      for (int q = tid; q < P; q += 512) {
        const int id = p.ids[(size_t)(q / p.k) * p.stride + q % p.k];
        const bool bad = (unsigned)id >= (unsigned)p.E;
        if (bad && blockIdx.x == 0 && atomicCAS(p.status, 0, kStatusBadId) == 0) p.status[1] = id;
        fs.key[q] = bad ? kBadKey : id;
        fs.w[q] = p.w[(size_t)(q / p.k) * p.stride + q % p.k];
      }
      rs_sync();
      route_fast_place(p, fs, loc, glob);
      placed = true;
    }
    if (!placed) {
      // a near-tie or a non-finite logit: the reference's arithmetic decides (block-uniform, rare;
      // its argument block is only built here so that the common path keeps everything in registers)
      RouteOuts ro;
      fill_outs(ro.loc, ro.glob);
      route_exact(p, (RouteSmallScratch<kDecMaxT>*)(smem + kOffRing + sizeof(FastScratch)), &ro, blockIdx.x == 0 ? p.status : nullptr);
    }
  } else if (has_sh) {
    const int gtid = tid - 512, gw = warp - 16;
#pragma unroll 1
    for (int t = 0; t < T; t++) {
      double a = 0;
      const uint4* xv = (const uint4*)(p.x + (size_t)t * d);
      const uint4* gv = (const uint4*)p.gate_w;
#pragma unroll 1
      for (int c = gtid; c < d / 8; c += 512) {
        const uint4 xa = xv[c], ga = __ldg(gv + c);
        const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w}, gq[4] = {ga.x, ga.y, ga.z, ga.w};
#pragma unroll
        for (int q = 0; q < 4; q++) {
          a += (double)__uint_as_float(gq[q] << 16) * (double)__uint_as_float(xw[q] << 16);
          a += (double)__uint_as_float(gq[q] & 0xFFFF0000u) * (double)__uint_as_float(xw[q] & 0xFFFF0000u);
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1)
        a += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(a), o),
                              __shfl_xor_sync(0xffffffffu, __double2loint(a), o));
      if (lane == 0) fs.gpart[t][gw] = a;
    }
  }
  __syncthreads();
  if (has_sh && tid < T) {
    // the shared expert's rows sit behind the routed ones, in token order, weighted by the gate
    double tot = 0;
#pragma unroll 1
    for (int w2 = 0; w2 < 16; w2++) tot += fs.gpart[tid][w2];
    const float gate = sigmoid_f32((float)tot);
    res->tokidx[P + tid] = tid;
    res->pw[P + tid] = gate;
    if (blockIdx.x == 0) {
      p.rb.sgate[tid] = gate;
      p.rb.tokidx[P + tid] = tid;
      p.rb.pw[P + tid] = gate;
    }
  }
  __syncthreads();
  DEC_TRACE(2);
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
  // Record of a unit: v-th sub-unit of the routed runs, or of the shared expert's T rows.
  auto unit_rec = [&](int v, bool shared_unit, Rec& r) {
    if (shared_unit) {
      r.first = P + v * kDecRows;
      r.info = min(kDecRows, T - v * kDecRows) | 256;
      r.base = nullptr;  // (the caller adds the image; expert 0)
      r.tok0 = 0;        // filled below
    } else {
      int lo = v, hi = n_routed - 1;
      if (nu_routed != n_routed) {  // some run has more than kDecRows rows: search the prefix
        lo = 0;
        while (lo < hi) {
          const int m = (lo + hi + 1) >> 1;
          if (res->uf[m] <= v) lo = m; else hi = m - 1;
        }
      }
      const Run run = res->runs[lo];
      const int sub = v - res->uf[lo];
      r.first = run.first + sub * kDecRows;
      r.info = min(kDecRows, run.count - sub * kDecRows);
      r.tok0 = run.expert;  // (expert id, replaced by the token below)
    }
  };
  auto finish_rec = [&](Rec& r, const Image& img, int expert, int mtile) {
    r.base = img.data + ((size_t)expert * img.n_mtiles + mtile) * img.n_kblocks * tile_bytes(kQ4CP);
    const int cnt = r.info & 255;
    r.tok0 = res->tokidx[r.first];
    r.pw0 = res->pw[r.first];
    r.tok1 = cnt > 1 ? res->tokidx[r.first + 1] : 0;
    r.pw1 = cnt > 1 ? res->pw[r.first + 1] : 0.f;
  };

  // ring slots of this warp and the constant half of a lookup address
  const uint32_t slot_lo = kOffS0 + (uint32_t)warp * kSlotBytes;
  const uint32_t slot_hi = kOffRing + (uint32_t)warp * (kDepth - 1) * kSlotBytes;
  auto slot_base = [&](int s) -> uint32_t { return s == 0 ? slot_lo : slot_hi + (uint32_t)(s - 1) * kSlotBytes; };
  const uint32_t lut = 0x00010000u | (uint32_t)(lane * 4);  // address bytes {lane*4, code byte, 1, 0}: the table sits at 64 KB
  const uint32_t work = kOffTab + 128 + (uint32_t)lane * 4;  // work row R of this lane: work + R * 256
  constexpr int tile_b = tile_bytes(kQ4CP);

  // =========================== gate/up + SwiGLU ===========================
  // Units: the shared expert's sub-units first, then the routed ones. A task = 16 hidden outputs
  // of a unit (lanes 0..15 the gate rows, lanes 16..31 the matching up rows); the 32 warps split
  // K (my_k K blocks each). The tasks are cut into one contiguous range per block.
  {
    const int KB = d / kTileK;
    const int kpw = (KB + kDecWarps - 1) / kDecWarps;
    const int kb0 = warp * kpw;
    const int my_k = max(0, min(kpw, KB - kb0));
    const int tpu = mid / 16;
    // The tasks are cut into one contiguous range per block by COST, not by count: a task over two
    // rows does almost twice the arithmetic of a task over one (the kernel is bound by instruction
    // issue, not by bytes). Cost 5 per single-row task, 8 per two-row task; res->uw = exclusive
    // prefix of the units' costs per task (shared sub-units first).
    const int n_units = nu_shared + nu_routed;
    if (warp == 0) {
      int carry = 0;
      for (int i0 = 0; i0 < n_units; i0 += 32) {
        const int u = i0 + lane;
        int cst = 0;
        if (u < n_units) {
          Rec r;
          unit_rec(u < nu_shared ? u : u - nu_shared, u < nu_shared, r);
          cst = (r.info & 255) > 1 ? 8 : 5;
        }
        int incl = cst;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        if (u < n_units) res->uw[u] = carry + incl - cst;
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) res->uw[n_units] = carry;
    }
    __syncthreads();
    // global task index at which the cost prefix reaches `target` (cost units x tasks per unit)
    auto task_at = [&](long long target) -> int {
      int lo = 0, hi = n_units;  // first unit u with uw[u + 1] * tpu > target
      while (lo < hi) {
        const int m = (lo + hi) >> 1;
        if ((long long)res->uw[m + 1] * tpu > target) hi = m; else lo = m + 1;
      }
      if (lo >= n_units) return n_units * tpu;
      const int per = res->uw[lo + 1] - res->uw[lo];
      return lo * tpu + (int)((target - (long long)res->uw[lo] * tpu + per - 1) / per);
    };
    const long long total_cost = (long long)res->uw[n_units] * tpu;
    const int c0 = task_at(total_cost * blockIdx.x / gridDim.x);
    const int n_tasks = task_at(total_cost * (blockIdx.x + 1) / gridDim.x) - c0;
    int gt = 0;  // tasks of this block done so far
    for (int b0 = 0; b0 < n_tasks; b0 += kMaxRecs) {
      const int nb = min(kMaxRecs, n_tasks - b0);
      __syncthreads();  // the records of the previous batch are no longer read
      if (tid < nb) {
        const int g = c0 + b0 + tid, u = g / tpu, j = g - u * tpu;
        Rec r;
        const bool sh = u < nu_shared;
        unit_rec(sh ? u : u - nu_shared, sh, r);
        const int expert = sh ? 0 : r.tok0;
        finish_rec(r, sh ? p.sh_gu : p.gu, expert, j >> 2);
        r.info |= j << 16;
        *(Rec*)(smem + kOffRec + tid * 32) = r;
      }
      __syncthreads();

      // ---- the warp's copy stream: item = (task, K block of the warp's slice), kDepth items ahead ----
      int q_task = 0, q_ik = 0, q_s = 0;
      const uint8_t* q_ptr = nullptr;   // this lane's 16 code bytes of the next item (first half of the K block)
      const uint8_t* q_mptr = nullptr;  // this lane's scale pair
      const uint16_t* q_xp = nullptr;   // this lane's 16 bytes of the rows' activations (lanes < 8 * rows), else null
      auto q_load = [&]() {
        const uint4 a = lds128(kOffRec + q_task * 32), b = lds128(kOffRec + q_task * 32 + 16);
        const uint8_t* base = (const uint8_t*)(((unsigned long long)a.y << 32) | a.x);
        const int info = (int)a.w, j = info >> 16, cnt = info & 255;
        const int row = (lane < 16 ? 0 : 48) + (j & 3) * 16 + lane;  // gate rows 0..63, up rows 64..127 of the tile
        q_ptr = base + (size_t)kb0 * tile_b + row * 16;
        q_mptr = base + (size_t)kb0 * tile_b + kCodeBytes + row * 4;
        const int tok = lane < 8 ? (int)b.x : (int)b.y;
        q_xp = lane < cnt * 8 ? p.x + (size_t)tok * d + kb0 * kTileK + (lane & 7) * 8 : nullptr;
      };
      auto issue = [&]() {
        if (q_task < nb && my_k > 0) {
          const uint32_t sb = slot_base(q_s);
          cp16(sb + lane * 16, q_ptr);
          cp16(sb + 512 + lane * 16, q_ptr + 2048);
          cp4(sb + 1024 + lane * 4, q_mptr);
          if (q_xp) cp16(sb + 1280 + lane * 16, q_xp);
          q_ptr += tile_b;
          q_mptr += tile_b;
          if (q_xp) q_xp += kTileK;
          if (++q_ik == my_k) {
            q_ik = 0;
            if (++q_task < nb) q_load();
          }
        }
        cp_commit();
        q_s = q_s == kDepth - 1 ? 0 : q_s + 1;
      };
      if (my_k > 0) q_load();
#pragma unroll
      for (int i = 0; i < kDepth; i++) issue();

      int c_s = 0;
      for (int task = 0; task < nb; task++, gt++) {
        const uint4 ra = lds128(kOffRec + task * 32);
        const int info = (int)ra.w, cnt = info & 255, j = info >> 16, first = (int)ra.z;
        const int need = (info & 256) ? kTabUpShared : kTabUpRouted;
        if (need != cur_tab) {  // block-uniform; at most once per phase (shared units come first)
          __syncthreads();
          if (info & 256) build_table(1, 2); else build_table(0, 0);
          cur_tab = need;
          __syncthreads();
        }
        float acc0 = 0.f, acc1 = 0.f;
        for (int ik = 0; ik < my_k; ik++) {
          cp_wait<kDepth - 1>();
          __syncwarp();
          const uint32_t sb = slot_base(c_s);
          // activations bf16 -> fp16 in place (finite values saturate; exact for |v| in [2^-14, 65504])
          const uint32_t xa = sb + 1280;
          sts32(xa + lane * 4, bf16x2_to_f16x2(lds32(xa + lane * 4)));
          if (cnt > 1) sts32(xa + 128 + lane * 4, bf16x2_to_f16x2(lds32(xa + 128 + lane * 4)));
          __syncwarp();
          const uint4 ca = lds128(sb + lane * 16), cb = lds128(sb + 512 + lane * 16);
          const uint32_t m = lds32(sb + 1024 + lane * 4);
          const float sc0 = half_bits_to_f32((uint16_t)(m & 0xFFFFu)), sc1 = half_bits_to_f32((uint16_t)(m >> 16));
          float d0[kDecRows], d1[kDecRows];
          if (cnt == 1) {
            chunk_dots<1>(ca, lut, xa, 128, d0);
            chunk_dots<1>(cb, lut, xa + 64, 128, d1);
            acc0 += sc0 * d0[0] + sc1 * d1[0];
          } else {
            chunk_dots<2>(ca, lut, xa, 128, d0);
            chunk_dots<2>(cb, lut, xa + 64, 128, d1);
            acc0 += sc0 * d0[0] + sc1 * d1[0];
            acc1 += sc0 * d0[1] + sc1 * d1[1];
          }
          __syncwarp();  // the slot is free for the copy that follows
          issue();
          c_s = c_s == kDepth - 1 ? 0 : c_s + 1;
        }
        // ---- end of the warp's share of the task: leave the partial sums, count the arrival ----
        const int rb = gt & (kRedBufs - 1), use = (gt >> 2) + 1;  // kRedBufs == 4
        if (use > 1) wait_shared_ge(&res->done[rb], use - 1, res, p.status, 1);  // the buffer's previous sums have been taken
        sts32(work + (uint32_t)((rb * kDecRows + 0) * kDecWarps + warp) * 256, __float_as_uint(acc0));
        sts32(work + (uint32_t)((rb * kDecRows + 1) * kDecWarps + warp) * 256, __float_as_uint(acc1));
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          atomicAdd(&res->cnt[rb], 1);
        }
        if (warp == (gt & (kDecWarps - 1))) {
          // this warp's turn to add the task's 32 slices, in slice order, and finish the outputs
          wait_shared_ge(&res->cnt[rb], use * kDecWarps, res, p.status, 2);
          __threadfence_block();
          __syncwarp();
#pragma unroll
          for (int r = 0; r < kDecRows; r++) {
            if (r < cnt) {
              float tot = 0.f;
#pragma unroll 8
              for (int w = 0; w < kDecWarps; w++) tot += __uint_as_float(lds32(work + (uint32_t)((rb * kDecRows + r) * kDecWarps + w) * 256));
              const float up = __shfl_down_sync(0xffffffffu, tot, 16);
              if (lane < 16) p.hid[(size_t)(first + r) * mid + j * 16 + lane] = __float2half_rn(sat_f16(silu_f32(tot) * up));
            }
          }
          __syncwarp();
          if (lane == 0) {
            __threadfence_block();
            *(volatile int32_t*)&res->done[rb] = use;
          }
        }
      }
      cp_wait<0>();
    }
  }

  // =========================== down + weighted combine ===========================
  // A block owns 32 rows of the output (one warp-row of a weight tile) for every token: units in
  // ascending expert order, the shared expert last; the 32 warps split K in 32-wide groups; an
  // item = one group of up to two units. A warp keeps its partial sums per token in shared
  // memory (a work row per token), the block adds them in warp order at the end.
  const int n_rb = d / 32;
  const int GH = mid / 32;                                    // 32-groups along K
  const int hpw = (GH + kDecWarps - 1) / kDecWarps;            // groups per warp (1 for mid <= 1024)
  const int nu_all = min(nu_routed + nu_shared, kMaxRecs);
  const int ni_routed = (nu_routed + 1) >> 1, ni_all = ni_routed + ((nu_shared + 1) >> 1);
  // units of item it: a, and b (or -1)
  auto item_units = [&](int it, int& a, int& b) {
    if (it < ni_routed) {
      a = 2 * it;
      b = a + 1 < nu_routed ? a + 1 : -1;
    } else {
      a = nu_routed + 2 * (it - ni_routed);
      b = a + 1 < nu_all ? a + 1 : -1;
    }
  };
  auto build_dn_recs = [&](int rb) {
    if (tid < nu_all) {
      Rec r;
      const bool sh = tid >= nu_routed;
      unit_rec(sh ? tid - nu_routed : tid, sh, r);
      const int expert = sh ? 0 : r.tok0;
      finish_rec(r, sh ? p.sh_dn : p.dn, expert, rb >> 2);
      *(Rec*)(smem + kOffRec + tid * 32) = r;
    }
  };
  const int my_first_rb = blockIdx.x;
  int q_it = 0, q_hbi = 0, q_s = 0;
  int q_rb = my_first_rb;
  // one copy item; with_act = false leaves out the hidden rows (they do not exist before the grid barrier)
  auto issue_dn = [&](bool with_w, bool with_act) {
    const int hb = warp + kDecWarps * q_hbi;
    if (q_it < ni_all && q_hbi < hpw && hb < GH) {
      int ua, ub;
      item_units(q_it, ua, ub);
      const uint32_t sb = slot_base(q_s);
      const int row = (q_rb & 3) * 32 + lane;
      const size_t koff = (size_t)(hb >> 1) * tile_b + (hb & 1) * 2048 + row * 16;
      const size_t moff = (size_t)(hb >> 1) * tile_b + kCodeBytes + row * 4;
      const uint4 a0 = lds128(kOffRec + ua * 32);
      const uint8_t* base_a = (const uint8_t*)(((unsigned long long)a0.y << 32) | a0.x);
      if (with_w) {
        cp16(sb + lane * 16, base_a + koff);
        cp4(sb + 1024 + lane * 4, base_a + moff);
      }
      if (with_act && lane < ((int)a0.w & 255) * 4)
        cp16(sb + 1280 + lane * 16, p.hid + (size_t)((int)a0.z + (lane >> 2)) * mid + hb * 32 + (lane & 3) * 8);
      if (ub >= 0) {
        const uint4 b0 = lds128(kOffRec + ub * 32);
        const uint8_t* base_b = (const uint8_t*)(((unsigned long long)b0.y << 32) | b0.x);
        if (with_w) {
          cp16(sb + 512 + lane * 16, base_b + koff);
          cp4(sb + 1152 + lane * 4, base_b + moff);
        }
        if (with_act && lane >= 8 && lane < 8 + ((int)b0.w & 255) * 4)
          cp16(sb + 1280 + lane * 16, p.hid + (size_t)((int)b0.z + ((lane - 8) >> 2)) * mid + hb * 32 + (lane & 3) * 8);
      }
    }
  };
  auto advance_q = [&]() {
    if (++q_it >= ni_all) {
      q_it = 0;
      q_hbi++;
    }
    q_s = q_s == kDepth - 1 ? 0 : q_s + 1;
  };
  // the first weights of the down phase travel while the blocks meet at the barrier
  __syncthreads();  // (every warp is done with the gate/up records)
  DEC_TRACE(3);
  if (my_first_rb < n_rb) {
    build_dn_recs(my_first_rb);
    __syncthreads();
    for (int i = 0; i < kDepth; i++) {
      issue_dn(true, false);
      cp_commit();
      advance_q();
    }
  }
  if (!grid_barrier(p.bar, bar_target, res, p.status)) {
    cp_wait<0>();
    return;
  }
  DEC_TRACE(4);
  for (int rb = my_first_rb; rb < n_rb; rb += gridDim.x) {
    for (int t = 0; t < T; t++) sts32(work + (uint32_t)(warp * kDecMaxT + t) * 256, 0u);
    if (rb == my_first_rb) {
      // the hidden rows exist only now: fetch them for the items already under way
      q_it = 0; q_hbi = 0; q_s = 0;
      for (int i = 0; i < kDepth; i++) {
        issue_dn(false, true);
        advance_q();
      }
      cp_commit();
      cp_wait<0>();
    } else {
      __syncthreads();
      build_dn_recs(rb);
      __syncthreads();
      q_it = 0; q_hbi = 0; q_s = 0; q_rb = rb;
      for (int i = 0; i < kDepth; i++) {
        issue_dn(true, true);
        cp_commit();
        advance_q();
      }
    }
    __syncwarp();
    int c_s = 0;
    for (int hbi = 0; hbi < hpw; hbi++) {
      const int hb = warp + kDecWarps * hbi;
      for (int it = 0; it < ni_all; it++) {
        const int need = it >= ni_routed ? kTabDnShared : kTabDnRouted;
        if (need != cur_tab) {  // block-uniform
          __syncthreads();      // every warp is done with the table that is replaced
          if (it >= ni_routed) build_table(4, 4); else build_table(3, 3);
          cur_tab = need;
          __syncthreads();
        }
        cp_wait<kDepth - 1>();
        __syncwarp();
        if (hb < GH) {
          int ua, ub;
          item_units(it, ua, ub);
          const uint32_t sb = slot_base(c_s);
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const int u = h ? ub : ua;
            if (u >= 0) {
              const uint4 r0 = lds128(kOffRec + u * 32), r1 = lds128(kOffRec + u * 32 + 16);
              const int cnt = (int)r0.w & 255;
              const uint4 c = lds128(sb + h * 512 + lane * 16);
              const uint32_t m = lds32(sb + 1024 + h * 128 + lane * 4);
              const float scale = half_bits_to_f32((uint16_t)((hb & 1) ? (m >> 16) : (m & 0xFFFFu)));
              float dots[kDecRows];
              if (cnt == 1) chunk_dots<1>(c, lut, sb + 1280 + h * 128, 64, dots);
              else chunk_dots<2>(c, lut, sb + 1280 + h * 128, 64, dots);
              {
                const uint32_t a = work + (uint32_t)(warp * kDecMaxT + (int)r1.x) * 256;
                sts32(a, __float_as_uint(__uint_as_float(lds32(a)) + __uint_as_float(r1.z) * (scale * dots[0])));
              }
              if (cnt > 1) {
                const uint32_t a = work + (uint32_t)(warp * kDecMaxT + (int)r1.y) * 256;
                sts32(a, __float_as_uint(__uint_as_float(lds32(a)) + __uint_as_float(r1.w) * (scale * dots[1])));
              }
            }
          }
        }
        __syncwarp();
        issue_dn(true, true);
        cp_commit();
        advance_q();
        c_s = c_s == kDepth - 1 ? 0 : c_s + 1;
      }
    }
    cp_wait<0>();
    __syncthreads();
    if (warp < T) {
      float y = 0.f;
#pragma unroll 8
      for (int w = 0; w < kDecWarps; w++) y += __uint_as_float(lds32(work + (uint32_t)(w * kDecMaxT + warp) * 256));
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
  DEC_TRACE(5);
}


// The same routing as a kernel of its own, for the decode path that keeps the GEMVs and the
// combine as separate kernels: 512 threads select and bucket, 512 threads form the shared
// expert's gate. Writes what k_route_small writes.
struct RouteFastParams {
  const float* logits;
  const uint16_t* x;
  const uint16_t* gate_w;  // null: no shared expert
  int T, E, k, d;
  RouteBuffers rb;
};

__global__ void __launch_bounds__(kDecThreads, 1)
k_route_fast(const RouteFastParams q) {
  extern __shared__ __align__(16) uint8_t rsm[];
  FastScratch& fs = *(FastScratch*)rsm;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = q.T, P = q.T * q.k, d = q.d;
  DecParams p{};  // the fields the routing pieces read
  p.logits = q.logits; p.x = q.x; p.gate_w = q.gate_w; p.T = q.T; p.E = q.E; p.k = q.k; p.d = q.d;
  p.status = q.rb.status;
  pdl_trigger();
  pdl_wait();  // inputs may come from the previous kernel; the buffers written here may still be read by it
  if (warp < 16) {
    RouteSmallOut out, none;
    out.topids = q.rb.topids; out.topw = q.rb.topw; out.tokidx = q.rb.tokidx; out.pw = q.rb.pw;
    out.pairids = q.rb.pairids; out.eoff = q.rb.eoff; out.runs = q.rb.runs; out.shared_slot = kMaxExperts;
    out.n_runs = q.rb.n_runs; out.tiles = q.rb.tiles; out.tiles_sh = q.rb.tiles_sh; out.n_tiles = q.rb.n_tiles;
    if (route_fast_select(p, fs, out)) {
      // (loc and glob are the same arrays here: the placement writes each result twice, harmlessly)
      route_fast_place(p, fs, out, out);
    } else {
      RouteOuts ro;
      ro.loc = out;
      ro.glob = none;
      route_exact(p, (RouteSmallScratch<kDecMaxT>*)(rsm + sizeof(FastScratch)), &ro, q.rb.status);
    }
  } else if (q.gate_w) {
    const int gtid = tid - 512, gw = warp - 16;
#pragma unroll 1
    for (int t = 0; t < T; t++) {
      double a = 0;
      const uint4* xv = (const uint4*)(q.x + (size_t)t * d);
      const uint4* gv = (const uint4*)q.gate_w;
#pragma unroll 1
      for (int c = gtid; c < d / 8; c += 512) {
        const uint4 xa = xv[c], ga = __ldg(gv + c);
        const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w}, gq[4] = {ga.x, ga.y, ga.z, ga.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          a += (double)__uint_as_float(gq[i] << 16) * (double)__uint_as_float(xw[i] << 16);
          a += (double)__uint_as_float(gq[i] & 0xFFFF0000u) * (double)__uint_as_float(xw[i] & 0xFFFF0000u);
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1)
        a += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(a), o),
                              __shfl_xor_sync(0xffffffffu, __double2loint(a), o));
      if (lane == 0) fs.gpart[t][gw] = a;
    }
  }
  __syncthreads();
  if (q.gate_w && tid < T) {
    double tot = 0;
#pragma unroll 1
    for (int w2 = 0; w2 < 16; w2++) tot += fs.gpart[tid][w2];
    const float gate = sigmoid_f32((float)tot);
    q.rb.sgate[tid] = gate;
    q.rb.tokidx[P + tid] = tid;
    q.rb.pw[P + tid] = gate;
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
                          const RouteBuffers& rb, unsigned long long* bar, int32_t* status, cudaStream_t st, unsigned long long* trace) {
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
  p.rb = rb; p.bar = bar; p.status = status; p.trace = trace;
  return launch_pdl(k_decode, dim3(sms), dim3(kDecThreads), (size_t)smem, st, p);
}


// Routing stage of a decode call (logits given, T <= decode_max_tokens(), T*k <= 128) in one launch;
// same outputs as launch_route_small.
cudaError_t launch_route_fast(const RouteBuffers& rb, const float* logits, int T, int k, int E, const void* x_bf16,
                              const uint16_t* gate_w_bf16, int d, cudaStream_t st) {
  static bool attr_done = false;
  const int smem = (int)(sizeof(FastScratch) + sizeof(RouteSmallScratch<kDecMaxT>));
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k_route_fast, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  RouteFastParams q{};
  q.logits = logits; q.x = (const uint16_t*)x_bf16; q.gate_w = gate_w_bf16; q.T = T; q.E = E; q.k = k; q.d = d; q.rb = rb;
  return launch_pdl(k_route_fast, dim3(1), dim3(kDecThreads), (size_t)smem, st, q);
}

}  // namespace b200moe
