// expert_tc.cu -- prefill path: persistent grouped dequant-GEMM on the 5th-generation
// tensor cores (tcgen05, accumulators in tensor memory), sm_100a only.
//
// It takes the place of the reference's LUT-decoded 4-bit expert GEMM (k_moe_lut,
// src/gpu/parts/27_kernels_moe_lut.inc:110-640) and keeps its numerics: operands are
// fp16 -- weights w = f16(f16(codebook[code]) * f16(scale)), activations f16 -- and the
// accumulation is fp32; like the reference, weight rows sit on the fixed M side (128
// rows per tile) and the rows of one expert on the variable N side (16..192), so that a
// nearly empty expert costs a narrow instruction instead of a padded token tile.
//
// One CTA per SM, 16 warps with fixed roles:
//   warp 0      producer of activation tiles: one TMA tensor copy (128-byte swizzle, box of
//               16/64/128/192 rows) per K block into a shared-memory ring
//   warp 2      producer of packed 4-bit weight tiles: one bulk-async copy of a contiguous
//               4.5 KB object per tile and K block (a single thread can only start a copy
//               every ~170 cycles, hence two producer threads and one copy each per K block)
//   warp 1      issues tcgen05.mma (A from tensor memory, B from shared memory), owns the
//               tensor-memory allocation
//   warps 4-11  dequantise: two groups of four warps alternate K blocks; thread = one
//               weight row; 256-entry half2 pair table replicated per lane in shared
//               memory (bank-conflict free), one half2 multiply by the group scale, result
//               written straight into tensor memory (tcgen05.st) as the MMA's A operand
//   warps 12-15 epilogue: tcgen05.ld the fp32 accumulator, SwiGLU (gate/up rows live in
//               different lanes, exchanged through shared memory) or plain convert,
//               fp16 stores; overlaps the next tile's main loop (two accumulators)
// Every wait on an mbarrier is bounded; when one gives up the CTA records a status
// word, stops issuing work, and leaves after releasing its tensor memory.
#include "tc.h"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdio>
#include <cstdlib>

namespace b200moe {

struct TcPlan {
  CUtensorMap x[4], h[4];  // activation / hidden maps with boxes of 16, 64, 128, 192 rows
  int sms = 148;
  long long* trace = nullptr;  // debug timeline of CTA 0 (environment B200MOE_TC_TRACE=<file>)
};

namespace {

constexpr int kNB = 4;    // activation stages
constexpr int kNW = 6;    // packed weight stages
constexpr int kNA = 4;    // tensor-memory A stages (32 columns each)
constexpr int kBStage = kTcTileN * 128;  // bytes: rows x 64 halfs
constexpr int kWStage = 6144;
constexpr int kLutBytes = 256 * 32 * 4;
constexpr int kThreads = 512;
constexpr int kAccCols = kTcTileN;       // columns per accumulator
constexpr int kTmemA = 2 * kAccCols;     // first column of the A stages (384)

// Shared-memory map in ABSOLUTE addresses of the CTA's shared window (the dynamic
// allocation starts at 1 KB when the kernel has no static shared memory). The pair table
// sits exactly at 64 KB so that the address of a lookup is a single byte permute:
//   address = 0x00010000 | code byte << 8 | table half << 7 | lane << 2
// i.e. entry stride 256 B = [table of tile rows 0..63: 32 lanes x 4 B][rows 64..127: 32 x 4 B].
constexpr int kOffW = 2048;                          // packed weight stages
constexpr int kOffU = kOffW + kNW * kWStage;         // SwiGLU exchange buffer (8 KB)
constexpr int kOffBar = kOffU + 2 * 32 * 32 * 4;     // barriers and flags (512 B)
constexpr int kOffLut = 65536;                       // pair tables (64 KB)
constexpr int kOffB = 131072;                        // activation stages, 1 KB aligned
constexpr int kSmemEnd = kOffB + kNB * kBStage;      // 229376
constexpr int kSmemBytes = kSmemEnd - 1024;          // dynamic bytes requested
static_assert(kOffBar + 512 <= kOffLut, "low region overflows into the pair tables");
static_assert(kSmemEnd <= 233472, "shared memory map exceeds the SM");

// barrier slots (8 bytes each) inside the barrier block
constexpr int kBarWFull = 0, kBarWEmpty = kBarWFull + kNW, kBarBFull = kBarWEmpty + kNW,
              kBarBEmpty = kBarBFull + kNB, kBarAFull = kBarBEmpty + kNB,
              kBarAEmpty = kBarAFull + kNA, kBarAccFull = kBarAEmpty + kNA,
              kBarAccEmpty = kBarAccFull + 2, kNumBars = kBarAccEmpty + 2;
static_assert(kNumBars * 8 + 16 + 32 <= 512, "barrier block too small");

constexpr long long kWaitLimitNs = 2000000000ll;  // 2 s: far beyond any legitimate wait

// ---- PTX wrappers ------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait. Returns false when the CTA is aborting (this wait or another one gave up).
// `nap_ns` > 0 makes the waiting warp sleep between polls: warps that poll in a tight loop
// take issue slots from the warp that shares their scheduler, and the thread that issues
// the MMAs must not be slowed down by waiters.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status, int where, unsigned nap_ns = 0) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  for (uint32_t spin = 1;; spin++) {
    if (nap_ns) __nanosleep(nap_ns);
    if (mbar_try(bar, parity)) return true;
    if ((spin & 255u) == 0) {
      if (*abort_flag) return false;
      if (now_ns() - t0 > (unsigned long long)kWaitLimitNs) {
        *abort_flag = 1;
        if (atomicCAS(status, 0, 1) == 0) status[1] = where;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]; fp16 operands, fp32 accumulate.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
      "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
      "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major fp16 tile stored as rows of 128 bytes with
// the 128-byte swizzle (what the TMA tensor copy writes): 8-row groups are 1024 bytes
// apart, descriptor version 1 (Blackwell), layout type 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t b_descriptor(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading-dimension offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride between 8-row groups
  d |= (uint64_t)1 << 46;            // descriptor version
  d |= (uint64_t)2 << 61;            // 128-byte swizzle
  return d;
}

// Instruction descriptor: D fp32, A/B fp16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

struct KParams {
  Image img;
  const Tile* tiles;
  const int32_t* n_tiles;
  __half* out;
  int out_ld;   // mid (gate/up) or d (down)
  int32_t* status;
  long long* trace;  // null, or [8 roles][kTraceSlots][4] clock samples written by CTA 0
};
constexpr int kTraceSlots = 512;
#define TR(role, slot, ev)                                                            \
  do {                                                                                \
    if (p.trace && blockIdx.x == 0 && (slot) < (uint32_t)kTraceSlots)                 \
      p.trace[((role) * kTraceSlots + (slot)) * 4 + (ev)] = clock64();                \
  } while (0)

template <bool UP>
__global__ void __launch_bounds__(kThreads, 1)
k_expert_tc(const __grid_constant__ CUtensorMap map16, const __grid_constant__ CUtensorMap map64,
            const __grid_constant__ CUtensorMap map128, const __grid_constant__ CUtensorMap map192,
            const KParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // smem + A is the generic pointer of absolute shared address A
  const uint32_t dyn0 = smem_u32(smem_raw);
  uint8_t* const smem = smem_raw - dyn0;
  constexpr uint32_t sbase = 0;
  {
    uint32_t dyn_size;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (dyn0 > (uint32_t)kOffW || dyn0 + dyn_size < (uint32_t)kSmemEnd) {
      // the fixed map does not fit this launch: refuse (uniform for the whole CTA)
      if (threadIdx.x == 0 && atomicCAS(p.status, 0, 2) == 0) p.status[1] = (int)dyn0;
      return;
    }
  }
  const uint32_t bars = sbase + kOffBar;
  volatile int* abort_flag = (volatile int*)(smem + kOffBar + kNumBars * 8);
  uint32_t* tmem_slot = (uint32_t*)(smem + kOffBar + kNumBars * 8 + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Image img = p.img;
  const int KB = img.n_kblocks;
  const int wbytes = tile_bytes(img.fmt);
  const int n_items = p.n_tiles[0] * img.n_mtiles;

  // ---- set-up ----
  if (threadIdx.x == 0) {
    for (int i = 0; i < kNW; i++) {
      mbar_init(bars + 8 * (kBarWFull + i), 1);
      mbar_init(bars + 8 * (kBarWEmpty + i), 4);
    }
    for (int i = 0; i < kNB; i++) {
      mbar_init(bars + 8 * (kBarBFull + i), 1);
      mbar_init(bars + 8 * (kBarBEmpty + i), 1);
    }
    for (int i = 0; i < kNA; i++) {
      mbar_init(bars + 8 * (kBarAFull + i), 4);
      mbar_init(bars + 8 * (kBarAEmpty + i), 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(bars + 8 * (kBarAccFull + i), 1);
      mbar_init(bars + 8 * (kBarAccEmpty + i), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  // pair table: entry b = (f16(book[b & 15]), f16(book[b >> 4])), one private copy per lane
  for (int i = threadIdx.x; i < 2 * 256 * 32; i += kThreads) {
    const int half_id = i >> 13, entry = (i >> 5) & 255;
    const float lo = img.book[half_id * 16 + (entry & 15)], hi = img.book[half_id * 16 + (entry >> 4)];
    *(__half2*)(smem + kOffLut + entry * 256 + half_id * 128 + (i & 31) * 4) = __floats2half2_rn(lo, hi);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ================= producer of activation tiles (one tensor copy per K block) =========
    if (lane == 0) {
      uint32_t kbi = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
        const Tile t = p.tiles[it / img.n_mtiles];
        const int n_pad = (t.count + 15) & ~15;
        // smallest box that covers the tile's rows: 16, 64, 128 or 192 rows of 64 halfs
        const CUtensorMap* map = n_pad <= 16 ? &map16 : n_pad <= 64 ? &map64 : n_pad <= 128 ? &map128 : &map192;
        const uint32_t bytes = (n_pad <= 16 ? 16 : n_pad <= 64 ? 64 : n_pad <= 128 ? 128 : 192) * 128;
        for (int kb = 0; kb < KB && ok; kb++, kbi++) {
          const uint32_t bs = kbi % kNB, bph = (kbi / kNB) & 1;
          ok = mbar_wait(bars + 8 * (kBarBEmpty + bs), bph ^ 1, abort_flag, p.status, 2, 64);
          if (!ok) break;
          TR(0, kbi, 1);
          const uint32_t bbar = bars + 8 * (kBarBFull + bs);
          mbar_expect_tx(bbar, bytes);
          tma_load_2d(sbase + kOffB + bs * kBStage, map, kb * kTileK, t.first, bbar);
        }
      }
    }
  } else if (warp == 2) {
    // ================= producer of packed weight tiles (one bulk copy per K block) ========
    if (lane == 0) {
      uint32_t kbi = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
        const Tile t = p.tiles[it / img.n_mtiles];
        const int mt = it % img.n_mtiles;
        const uint8_t* src = img.tile(t.expert, mt, 0);
        for (int kb = 0; kb < KB && ok; kb++, kbi++, src += wbytes) {
          const uint32_t ws = kbi % kNW, wph = (kbi / kNW) & 1;
          ok = mbar_wait(bars + 8 * (kBarWEmpty + ws), wph ^ 1, abort_flag, p.status, 1, 64);
          if (!ok) break;
          TR(0, kbi, 0);
          mbar_expect_tx(bars + 8 * (kBarWFull + ws), wbytes);
          bulk_copy_g2s(sbase + kOffW + ws * kWStage, src, wbytes, bars + 8 * (kBarWFull + ws));
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issue =================
    if (lane == 0) {
      uint32_t kbi = 0, li = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, li++) {
        const Tile t = p.tiles[it / img.n_mtiles];
        const int n_pad = (t.count + 15) & ~15;
        const uint32_t idesc = instr_desc(n_pad);
        const uint32_t acc = li & 1, accph = (li >> 1) & 1;
        ok = mbar_wait(bars + 8 * (kBarAccEmpty + acc), accph ^ 1, abort_flag, p.status, 3);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * kAccCols;
        for (int kb = 0; kb < KB && ok; kb++, kbi++) {
          const uint32_t bs = kbi % kNB, bph = (kbi / kNB) & 1;
          const uint32_t as = kbi % kNA, aph = (kbi / kNA) & 1;
          ok = mbar_wait(bars + 8 * (kBarBFull + bs), bph, abort_flag, p.status, 4);
          if (!ok) break;
          TR(1, kbi, 0);
          ok = mbar_wait(bars + 8 * (kBarAFull + as), aph, abort_flag, p.status, 5);
          if (!ok) break;
          TR(1, kbi, 1);
          tc_fence_after();
          const uint64_t bdesc = b_descriptor(sbase + kOffB + bs * kBStage);
          const uint32_t a_tmem = tmem + kTmemA + as * 32;
#pragma unroll
          for (int ks = 0; ks < 4; ks++)
            tc_mma_ts(d_tmem, a_tmem + ks * 8, bdesc + (uint64_t)(ks * 2), idesc,
                      (kb | ks) != 0 ? 1u : 0u);
          TR(1, kbi, 3);
          tc_commit(bars + 8 * (kBarAEmpty + as));
          tc_commit(bars + 8 * (kBarBEmpty + bs));
          TR(1, kbi, 2);
        }
        if (ok) tc_commit(bars + 8 * (kBarAccFull + acc));
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ================= dequantise into tensor memory =================
    const int grp = (warp - 4) >> 2, quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lut = (uint32_t)kOffLut | (uint32_t)((r >= 64 ? 128 : 0) + lane * 4);
    uint32_t kbi = 0;
    bool ok = true;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
      for (int kb = 0; kb < KB && ok; kb++, kbi++) {
        if ((int)(kbi & 1) != grp) continue;
        const uint32_t ws = kbi % kNW, wph = (kbi / kNW) & 1;
        ok = mbar_wait(bars + 8 * (kBarWFull + ws), wph, abort_flag, p.status, 6, 32);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0 && quarter == 0) TR(2 + grp, kbi, 0);
        const uint8_t* wt = smem + kOffW + ws * kWStage;
        uint32_t v[32];
        const uint32_t sc = *(const uint32_t*)(wt + kCodeBytes + r * 4);
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const uint4 c4 = *(const uint4*)(wt + h * 2048 + r * 16);
          const uint32_t w4[4] = {c4.x, c4.y, c4.z, c4.w};
          const uint32_t s16 = h ? (sc >> 16) : (sc & 0xFFFFu);
          const uint32_t s2 = s16 | (s16 << 16);
#pragma unroll
          for (int q = 0; q < 4; q++) {
#pragma unroll
            for (int b = 0; b < 4; b++) {
              // bytes (3,2,1,0) of the address = (table.3, table.2, code byte b, table.0)
              const uint32_t addr = __byte_perm(w4[q], lut, 0x7604 | (b << 4));
              uint32_t pair;
              asm("ld.shared.b32 %0, [%1];" : "=r"(pair) : "r"(addr));
              __half2 w2 = __hmul2(*(__half2*)&pair, *(const __half2*)&s2);
              v[h * 16 + q * 4 + b] = *(uint32_t*)&w2;
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + 8 * (kBarWEmpty + ws));
        const uint32_t as = kbi % kNA, aph = (kbi / kNA) & 1;
        if (lane == 0 && quarter == 0) TR(2 + grp, kbi, 1);
        ok = mbar_wait(bars + 8 * (kBarAEmpty + as), aph ^ 1, abort_flag, p.status, 7, 32);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0 && quarter == 0) TR(2 + grp, kbi, 2);
        tc_fence_after();
        tc_st32(tmem + ((uint32_t)(quarter * 32) << 16) + kTmemA + as * 32, v);
        tc_wait_st();
        if (lane == 0 && quarter == 0) TR(2 + grp, kbi, 3);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + 8 * (kBarAFull + as));
      }
    }
  } else if (warp >= 12) {
    // ================= epilogue =================
    const int quarter = warp & 3;
    float* ubuf = (float*)(smem + kOffU);
    volatile int* ep_ok = (volatile int*)(smem + kOffBar + kNumBars * 8 + 16);
    uint32_t li = 0;
    bool ok = true;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, li++) {
      const Tile t = p.tiles[it / img.n_mtiles];
      const int mt = it % img.n_mtiles;
      const uint32_t acc = li & 1, accph = (li >> 1) & 1;
      ok = mbar_wait(bars + 8 * (kBarAccFull + acc), accph, abort_flag, p.status, 8, 256);
      // The four epilogue warps must take the same decision (they meet at named barriers
      // below): publish each warp's result, meet once, and combine.
      ok = __all_sync(0xffffffffu, ok);
      if (lane == 0) ep_ok[(li & 1) * 4 + quarter] = ok ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      ok = (ep_ok[(li & 1) * 4] & ep_ok[(li & 1) * 4 + 1] & ep_ok[(li & 1) * 4 + 2] &
            ep_ok[(li & 1) * 4 + 3]) != 0;
      if (!ok) break;
      if (lane == 0 && quarter == 0) TR(4, li, 0);
      tc_fence_after();
      const uint32_t src = tmem + ((uint32_t)(quarter * 32) << 16) + acc * kAccCols;
      for (int c0 = 0; c0 < t.count; c0 += 32) {
        uint32_t v[32];
        tc_ld32(src + c0, v);
        tc_wait_ld();
        if (UP) {
          if (quarter >= 2) {
#pragma unroll
            for (int j = 0; j < 32; j++) ubuf[((quarter - 2) * 32 + j) * 32 + lane] = __uint_as_float(v[j]);
          }
          asm volatile("bar.sync 2, 128;" ::: "memory");
          if (quarter < 2) {
            __half* dst = p.out + (size_t)(t.first + c0) * p.out_ld + mt * 64 + quarter * 32 + lane;
#pragma unroll
            for (int j = 0; j < 32; j++) {
              if (c0 + j < t.count) {
                const float g = __uint_as_float(v[j]);
                const float u = ubuf[(quarter * 32 + j) * 32 + lane];
                dst[(size_t)j * p.out_ld] = __float2half_rn(silu_f32(g) * u);
              }
            }
          }
          asm volatile("bar.sync 3, 128;" ::: "memory");
        } else {
          __half* dst = p.out + (size_t)(t.first + c0) * p.out_ld + mt * 128 + quarter * 32 + lane;
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (c0 + j < t.count) dst[(size_t)j * p.out_ld] = __float2half_rn(__uint_as_float(v[j]));
        }
      }
      if (lane == 0 && quarter == 0) TR(4, li, 1);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kBarAccEmpty + acc));
    }
  }

  // ---- teardown ----
  __syncthreads();
  if (*abort_flag) {
    // give copies still in flight time to land before the CTA's shared memory goes away
    const unsigned long long t0 = now_ns();
    while (now_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512)
                 : "memory");
  }
}

cudaError_t encode_2d(PFN_cuTensorMapEncodeTiled_v12000 enc, CUtensorMap* map, const void* base,
                      long long rows, long long cols, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <bool UP>
cudaError_t launch(TcPlan* plan, const CUtensorMap* m, const Image& img,
                   const Tile* tiles, const int32_t* n_tiles, int max_tiles, __half* out, int out_ld,
                   int32_t* status, cudaStream_t st) {
  if (img.fmt != kQ4CP) return cudaErrorNotSupported;
  static bool attr_set[2] = {false, false};
  if (!attr_set[UP]) {
    cudaError_t e = cudaFuncSetAttribute(k_expert_tc<UP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[UP] = true;
  }
  KParams p{img, tiles, n_tiles, out, out_ld, status, UP ? plan->trace : nullptr};
  long long max_items = (long long)max_tiles * img.n_mtiles;
  int grid = (int)(max_items < plan->sms ? max_items : plan->sms);
  if (grid < 1) grid = 1;
  k_expert_tc<UP><<<grid, kThreads, kSmemBytes, st>>>(m[0], m[1], m[2], m[3], p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_create(TcPlan** out, const __half* x_sorted, const __half* hid16, long long rows_cap,
                      int d, int mid) {
  *out = nullptr;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
  auto enc = (PFN_cuTensorMapEncodeTiled_v12000)fn;
  TcPlan* plan = new TcPlan();
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&plan->sms, cudaDevAttrMultiProcessorCount, dev);
  const int boxes[4] = {16, 64, 128, kTcTileN};
  e = cudaSuccess;
  for (int i = 0; i < 4 && e == cudaSuccess; i++) e = encode_2d(enc, &plan->x[i], x_sorted, rows_cap, d, boxes[i]);
  for (int i = 0; i < 4 && e == cudaSuccess; i++) e = encode_2d(enc, &plan->h[i], hid16, rows_cap, mid, boxes[i]);
  if (e != cudaSuccess) {
    delete plan;
    return e;
  }
  if (getenv("B200MOE_TC_TRACE")) {
    const size_t bytes = (size_t)8 * kTraceSlots * 4 * sizeof(long long);
    if (cudaMalloc((void**)&plan->trace, bytes) == cudaSuccess) cudaMemset(plan->trace, 0, bytes);
    else plan->trace = nullptr;
  }
  *out = plan;
  return cudaSuccess;
}

void tc_destroy(TcPlan* plan) {
  if (plan && plan->trace) {
    // debug aid: dump CTA 0's timeline of the last gate/up launch as raw int64
    const size_t n = (size_t)8 * kTraceSlots * 4;
    long long* host = new long long[n];
    if (cudaMemcpy(host, plan->trace, n * sizeof(long long), cudaMemcpyDeviceToHost) == cudaSuccess) {
      if (FILE* f = fopen(getenv("B200MOE_TC_TRACE") ? getenv("B200MOE_TC_TRACE") : "tc_trace.bin", "wb")) {
        fwrite(host, sizeof(long long), n, f);
        fclose(f);
      }
    }
    delete[] host;
    cudaFree(plan->trace);
  }
  delete plan;
}

cudaError_t launch_up_tc(TcPlan* plan, const Image& img, const Tile* tiles, const int32_t* n_tiles,
                         int max_tiles, __half* hid16, int32_t* status, cudaStream_t st) {
  return launch<true>(plan, plan->x, img, tiles, n_tiles, max_tiles, hid16,
                      img.n_mtiles * 64, status, st);
}

cudaError_t launch_down_tc(TcPlan* plan, const Image& img, const Tile* tiles, const int32_t* n_tiles,
                           int max_tiles, __half* pairs16, int32_t* status, cudaStream_t st) {
  return launch<false>(plan, plan->h, img, tiles, n_tiles, max_tiles, pairs16,
                       img.n_mtiles * 128, status, st);
}

}  // namespace b200moe
