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
// One CTA per SM, 24 warps with fixed roles. K blocks (64 wide) are handled in pairs:
//   warp 0      producer of activation tiles: TMA tensor copies (128-byte swizzle, box of
//               16/64/128/192 rows), one per K block, into a ring of 3 pair-slots in shared
//               memory; the same thread asks for the packed weight tiles of a later pair to be
//               brought into L2 (one bulk prefetch per pair)
//   warp 1      issues tcgen05.mma (A from tensor memory, B from shared memory): eight per
//               pair behind ONE barrier wait and ONE commit; owns the tensor-memory allocation
//   warp 3      relay: folds "activations of the pair have landed" into the barrier the MMA
//               warp waits on, so that warp polls a single barrier
//   warps 4-19  dequantise: two sets of eight warps alternate pairs (set s owns tensor-memory
//               slot s); thread = one weight row of one K block. Packed codes come straight
//               from global memory (a warp's 32 rows are 512 contiguous bytes) into ONE set of
//               registers, refilled for the next own pair as soon as the decode has used them
//               up, through a pointer that walks with the stream (the tile list is read one item
//               ahead, never on the critical path); each code byte indexes a 256-entry half2
//               pair table replicated per lane in shared memory (bank-conflict free, the
//               address is one byte permute); one half2 multiply by the group scale; the
//               result goes straight into tensor memory (tcgen05.st) as the MMA's A operand
//   warps 20-23 epilogue: tcgen05.ld the fp32 accumulator, SwiGLU (gate/up rows live in
//               different lanes, exchanged through shared memory, work split over all four
//               warps) or plain convert, transposed through shared memory into 16-byte
//               global stores; overlaps the next tile's main loop (two accumulators)
// Measured limits that shaped this: a single thread starts a TMA copy only every ~170
// cycles; a barrier check costs 150-250 cycles under load; an M=128 MMA from tensor memory
// takes N/2 + 9.5 cycles and the MMA queue holds about four of them; the table lookups are
// bound by shared-memory wavefronts at ~25 code bytes per cycle per SM; and every instruction
// in the per-pair loops of the dequantising and MMA warps costs measurable time (a warp there
// issues only every 5-6 cycles), so these loops carry counters instead of divisions and no
// debugging code unless it is compiled in.
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
  int margin = 0;
  long long* trace = nullptr;  // debug timeline of CTA 0 (environment B200MOE_TC_TRACE=<file>)
};

namespace {

constexpr int kNS = 2;    // tensor-memory A slots; a slot holds a pair of K blocks (64 columns)
constexpr int kNBSMax = 3;
constexpr int kBStage = kTcTileN * 128;  // bytes of one K block of activations: rows x 64 halfs
constexpr int kThreads = 768;           // 24 warps: 4 service, 16 dequantising, 4 epilogue
constexpr int kAccCols = kTcTileN;       // columns per accumulator
constexpr int kTmemA = 2 * kAccCols;     // first column of the A slots
static_assert(kTmemA + kNS * 64 <= 512, "tensor memory: two accumulators and the A slots");

// Shared-memory map in ABSOLUTE addresses of the CTA's shared window (the dynamic
// allocation starts at 1 KB when the kernel has no static shared memory). The pair table
// has one 256-byte line per code byte: 32 lanes x 4 B of code book 0 (tile rows 0..63, or all
// rows), then 32 lanes x 4 B of code book 1 (tile rows 64..127 when the halves of a tile use
// different books: the shared expert's separate gate and up tensors). It sits on a 64 KB
// boundary, so that a lookup address is ONE byte permute:
//   bytes { lane*4 (+128), code byte, table >> 16, 0 }.
// The first activation slot fits below the table, the other two above it.
struct Map {
  static constexpr int kNBS = 3;                       // activation ring depth, in pairs of K blocks
  static constexpr int kOffLow = 2048;                 // the dynamic allocation must start at or below this
  static constexpr int kOffBar = 2048;                 // barriers and flags (1 KB)
  static constexpr int kOffU = 3072;                   // epilogue exchange + output tile (12 KB)
  static constexpr int kOffB0 = 15360;                 // activation slot 0 (1 KB aligned)
  static constexpr int kOffLut = 65536;                // 256 lines of 256 B
  static constexpr int kOffB1 = 131072;                // activation slots 1, 2
  static constexpr int kSmemEnd = kOffB1 + 2 * 2 * kBStage;
  static constexpr int kSmemBytes = kSmemEnd - 1024;   // dynamic bytes requested
  static_assert(kOffB0 + 2 * kBStage <= kOffLut, "slot 0 overlaps the table");
  static_assert(kSmemEnd <= 233472, "shared memory map exceeds the SM");
  __host__ __device__ static constexpr uint32_t slot(uint32_t s) {
    return s == 0 ? (uint32_t)kOffB0 : (uint32_t)(kOffB1 + (s - 1) * 2 * kBStage);
  }
};

// barrier slots (8 bytes each) inside the barrier block
constexpr int kBarAFull = 0,                   // [tensor-memory slot]: A of a pair stored, activations landed
              kBarBFull = kBarAFull + kNS,     // [activation slot]
              kBarDone = kBarBFull + kNBSMax,  // [activation slot]: all MMAs of a pair have completed
              kBarAccFull = kBarDone + kNBSMax,
              kBarAccEmpty = kBarAccFull + 2, kNumBars = kBarAccEmpty + 2;
static_assert(kNumBars * 8 + 16 + 32 <= 1024, "barrier block too small");

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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(20000u)  // suspend-time hint (ns): sleep in hardware, not in a poll loop
      : "memory");
  return ok != 0;
}
// One lane of a converged warp. Code around it stays warp-uniform, which lets the compiler
// keep descriptors and addresses in uniform registers instead of converting per instruction.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
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

// finite values saturate to the fp16 range (as on the GEMV path), NaN stays NaN
// fp32 -> fp16, finite values saturating to the fp16 range, NaN staying NaN: one conversion
__device__ __forceinline__ __half f16_sat(float v) {
  unsigned short h;
  asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
  return __ushort_as_half(h);
}

struct KParams {
  Image img;
  const Tile* tiles;
  const int32_t* n_tiles;
  __half* out;
  int out_ld;   // mid (gate/up) or d (down)
  int32_t* status;
  long long* trace;  // null, or [8 roles][kTraceSlots][4] clock samples written by CTA 0
  int l2_ahead;      // weight tiles are asked into L2 this many own pairs ahead of their register fetch (0: off)
  const int32_t* rowmap;    // down kernel, may be null: tile-list row r >= map_base[0] is written to output row
  const int32_t* map_base;  // rowmap[r - map_base[0]] (rows below map_base[0], and all rows without a map: to row r)
};
constexpr int kTraceSlots = 512;
// Timeline stamps of CTA 0 (a debugging aid: build with -DB200MOE_TRACE and set
// B200MOE_TC_TRACE=<file>). Compiled out otherwise: with the stamps merely present but switched
// off the benchmark call took 7 % longer -- the loops below are that sensitive to extra
// instructions.
#ifndef B200MOE_TRACE
#define TR(role, slot, ev) do {} while (0)
#else
#define TR(role, slot, ev)                                                            \
  do {                                                                                \
    if (p.trace && blockIdx.x == 0 && (slot) < (uint32_t)kTraceSlots)                 \
      p.trace[((role) * kTraceSlots + (slot)) * 4 + (ev)] = clock64();                \
  } while (0)
#endif

// Per (row, K block) metadata of the source format, as loaded by a dequantising thread.
struct RowMetaTc {
  uint32_t a, b, c, d;
};

// Two fp16 weights from one code byte's table entry `pair` (the two codes as fp16 numbers
// for the GGUF formats, the two code-book values for q4cp) and the group's constants.
template <int FMT>
struct GroupDecode {};
template <>
struct GroupDecode<kQ4CP> {  // w = f16(book) * f16(scale)
  __half2 s2;
  __device__ __forceinline__ void init(const RowMetaTc& m, int h) {
    const uint32_t v = __byte_perm(m.a, 0u, h ? 0x3232u : 0x1010u);  // the half's fp16 scale in both lanes
    s2 = *(const __half2*)&v;
  }
  __device__ __forceinline__ __half2 weight(uint32_t pair, int) const { return __hmul2(*(__half2*)&pair, s2); }
};
template <>
struct GroupDecode<kQ4K> {  // w = (d*sc)*q - (dmin*m), the packed form of src/gguf.h:423-432
  __half2 a2, nb2;
  __device__ __forceinline__ void init(const RowMetaTc& m, int h) {
    const float d = half_bits_to_f32((uint16_t)(m.a & 0xFFFFu)), dmin = half_bits_to_f32((uint16_t)(m.a >> 16));
    const float sc = (float)((m.b >> (16 * h)) & 0xFFu), mn = (float)((m.b >> (16 * h + 8)) & 0xFFu);
    a2 = __float2half2_rn(d * sc);
    nb2 = __float2half2_rn(-(dmin * mn));
  }
  __device__ __forceinline__ __half2 weight(uint32_t pair, int) const { return __hfma2(*(__half2*)&pair, a2, nb2); }
};
template <>
struct GroupDecode<kQ51> {  // w = d*(q + 16*fifth bit) + m, src/gguf.h:360-374
  __half2 d2, m2;
  uint32_t qh;
  __device__ __forceinline__ void init(const RowMetaTc& m, int h) {
    const uint32_t dm = h ? m.c : m.a;
    qh = h ? m.d : m.b;
    d2 = __half2half2(__ushort_as_half((unsigned short)(dm & 0xFFFFu)));
    m2 = __half2half2(__ushort_as_half((unsigned short)(dm >> 16)));
  }
  // byte i of the group holds elements 2i, 2i+1; their fifth bits are bits i, 16 + i of qh:
  // shifted to bits 14 and 30 they read as the fp16 pair (2.0 or 0, 2.0 or 0)
  __device__ __forceinline__ __half2 weight(uint32_t pair, int i) const {
    const uint32_t u = (i <= 14 ? (qh << (14 - i)) : (qh >> 1)) & 0x40004000u;
    const __half2 q5 = __hfma2(*(const __half2*)&u, __float2half2_rn(8.f), *(const __half2*)&pair);
    return __hfma2(q5, d2, m2);
  }
};

template <bool UP, bool DUAL, int FMT>
__global__ void __launch_bounds__(kThreads, 1)
k_expert_tc(const __grid_constant__ CUtensorMap map16, const __grid_constant__ CUtensorMap map64,
            const __grid_constant__ CUtensorMap map128, const __grid_constant__ CUtensorMap map192,
            const KParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // smem + A is the generic pointer of absolute shared address A
  const uint32_t dyn0 = smem_u32(smem_raw);
  uint8_t* const smem = smem_raw - dyn0;
  constexpr uint32_t sbase = 0;
  using M = Map;
  constexpr int kNBS = M::kNBS, kOffLow = M::kOffLow, kOffU = M::kOffU, kOffBar = M::kOffBar,
                kSmemEnd = M::kSmemEnd;
  {
    uint32_t dyn_size;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (dyn0 > (uint32_t)kOffLow || dyn0 + dyn_size < (uint32_t)kSmemEnd) {
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
  const int n_items = p.n_tiles[0] * img.n_mtiles;

  // ---- set-up ----
  if (threadIdx.x == 0) {
    for (int i = 0; i < kNS; i++) mbar_init(bars + 8 * (kBarAFull + i), 9);  // 8 dequantising warps + relay
    for (int i = 0; i < kNBS; i++) {
      mbar_init(bars + 8 * (kBarBFull + i), 1);    // activation producer (with byte count)
      mbar_init(bars + 8 * (kBarDone + i), 1);     // one tcgen05.commit per pair
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
    if (half_id == 0 || DUAL)
      *(__half2*)(smem + M::kOffLut + entry * 256 + half_id * 128 + (i & 31) * 4) = __floats2half2_rn(lo, hi);
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

  // K blocks are handled two at a time ("pair"): one barrier wait and one commit of the MMA
  // thread then cover eight MMAs, which keeps that thread's bookkeeping below the tensor
  // pipe's time for the pair. A pair owns one slot of the A (tensor memory) and B (shared
  // memory) rings and one stage of the packed-weight ring; the two dequantising groups work
  // on the two K blocks of a pair side by side. An odd tail is a pair with one K block.
  const int NP = (KB + 1) >> 1;
  if (warp == 0) {
    // ================= producer of activation tiles (one tensor copy per K block) =========
    if (lane == 0) {
      uint32_t pi = 0, slot = 0, sph = 0;
      bool ok = true;
      Tile t_ahead = (int)blockIdx.x < n_items ? p.tiles[blockIdx.x / img.n_mtiles] : Tile{0, 0, 0};
      for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
        const Tile t = t_ahead;  // read one item ahead: its latency is off this loop's critical path
        if (it + (int)gridDim.x < n_items) t_ahead = p.tiles[(it + gridDim.x) / img.n_mtiles];
        const int n_pad = (t.count + 15) & ~15;
        // smallest box that covers the tile's rows: 16, 64, 128 or 192 rows of 64 halfs
        const CUtensorMap* map = n_pad <= 16 ? &map16 : n_pad <= 64 ? &map64 : n_pad <= 128 ? &map128 : &map192;
        const uint32_t bytes = (n_pad <= 16 ? 16 : n_pad <= 64 ? 64 : n_pad <= 128 ? 128 : kTcTileN) * 128;
        // The dequantising warps fetch their packed weights into registers only one own pair ahead
        // of their use (~18 KB in flight per SM). This thread, which has time to spare, also asks for
        // both tiles of a later pair -- of this item or of the next one -- to be brought into L2
        // with one bulk prefetch, so that the fetch finds them there. Measured: 6 % on a launch
        // whose tiles all have ~10 rows (short MMAs: the fetch latency shows), nothing on the
        // benchmark's mix; with every weight read served from L2 (a diagnostic run on one expert's
        // tiles) such a launch gains 23 %.
        constexpr size_t w_tile_b = tile_bytes(FMT);
        const uint8_t* w_this = img.tile(t.expert, it % img.n_mtiles, 0);
        const uint8_t* w_next =
            it + (int)gridDim.x < n_items ? img.tile(t_ahead.expert, (it + (int)gridDim.x) % img.n_mtiles, 0) : nullptr;
        for (int pp = 0; pp < NP && ok; pp++, pi++) {
          if (p.l2_ahead > 0) {
            int q = pp + 2 * p.l2_ahead;
            const uint8_t* b2 = w_this;
            if (q >= NP) {
              q -= NP;
              b2 = w_next;
            }
            if (b2 != nullptr && q < NP)
              asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(b2 + (size_t)(2 * q) * w_tile_b),
                           "r"((uint32_t)(min(2, KB - 2 * q) * (int)w_tile_b))
                           : "memory");
          }
          // slot = pi % kNBS, sph = (pi / kNBS) & 1, kept as counters (no division in the loop)
          const int nk = min(2, KB - 2 * pp);
          ok = mbar_wait(bars + 8 * (kBarDone + slot), sph ^ 1, abort_flag, p.status, 2, 64);
          if (!ok) break;
          TR(0, pi, 1);
          const uint32_t bar = bars + 8 * (kBarBFull + slot);
          mbar_expect_tx(bar, nk * bytes);
          for (int j = 0; j < nk; j++)
            tma_load_2d(sbase + M::slot(slot) + j * kBStage, map, ((2 * pp + j) >> img.act_shift) * kTileK, t.first, bar);
          if (++slot == (uint32_t)kNBS) {
            slot = 0;
            sph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issue =================
    // The whole warp runs the loop (converged); one elected lane issues.
    // (Measured: checking a barrier costs this warp 150-250 cycles under load even when its
    // phase is long complete, and the MMA queue holds about four instructions.)
    uint32_t pi = 0, li = 0;
    uint32_t aslot = 0, aph = 0, bslot = 0;  // pi % kNS, (pi / kNS) & 1, pi % kNBS as counters
    bool ok = true;
    Tile t_ahead = (int)blockIdx.x < n_items ? p.tiles[blockIdx.x / img.n_mtiles] : Tile{0, 0, 0};
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, li++) {
      const Tile t = t_ahead;  // read one item ahead: its latency is off this loop's critical path
      if (it + (int)gridDim.x < n_items) t_ahead = p.tiles[(it + gridDim.x) / img.n_mtiles];
      const int n_pad = (t.count + 15) & ~15;
      const uint32_t idesc = instr_desc(n_pad);
      const uint32_t acc = li & 1, accph = (li >> 1) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (kBarAccEmpty + acc), accph ^ 1, abort_flag, p.status, 3));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem + acc * kAccCols;
      for (int pp = 0; pp < NP && ok; pp++, pi++) {
        const int nk = min(2, KB - 2 * pp);
        // one wait covers both operands: the relay thread arrives only after the
        // activation tiles of this pair have landed
        if (lane == 0) TR(1, pi, 1);
        ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (kBarAFull + aslot), aph, abort_flag, p.status, 4));
        if (!ok) break;
        if (lane == 0) TR(1, pi, 0);
        tc_fence_after();
        const uint64_t bdesc = b_descriptor(sbase + M::slot(bslot));
        const uint32_t a_tmem = tmem + kTmemA + aslot * 64;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 4; ks++)
            tc_mma_ts(d_tmem, a_tmem + ks * 8, bdesc + (uint64_t)(ks * 2), idesc, (pp | ks) != 0 ? 1u : 0u);
          if (nk == 2) {
#pragma unroll
            for (int ks = 0; ks < 4; ks++)
              tc_mma_ts(d_tmem, a_tmem + 32 + ks * 8, bdesc + (uint64_t)((kBStage >> 4) + ks * 2), idesc, 1u);
          }
          // one commit per pair: frees the activation slot for the producer and, kNS pairs
          // later, the tensor-memory slot for the dequantising warps
          tc_commit(bars + 8 * (kBarDone + bslot));
          if (pp == NP - 1) tc_commit(bars + 8 * (kBarAccFull + acc));
        }
        __syncwarp();
        if (lane == 0) TR(1, pi, 2);
        if (++aslot == (uint32_t)kNS) {
          aslot = 0;
          aph ^= 1;
        }
        if (++bslot == (uint32_t)kNBS) bslot = 0;
      }
    }
  } else if (warp >= 4 && warp < 20) {
    // ================= dequantise into tensor memory =================
    // Sixteen warps = two sets of eight. Set s serves the pairs with index == s (mod 2) and
    // therefore always fills tensor-memory slot s: while one set waits for its slot and
    // stores, the other decodes. Inside a set, a group of four warps (one per 32-lane quarter
    // of tensor memory) owns one K block of the pair; a thread decodes the 64 codes of its
    // weight row for that K block and stores 32 columns.
    // Packed codes come straight from global memory (the tile layout makes a warp's 32 rows
    // one contiguous 512-byte read per half), one own pair ahead of their use.
    const int set = (warp - 4) >> 3, kblk = ((warp - 4) >> 2) & 1, quarter = warp & 3;
    const int r = quarter * 32 + lane;
    // constant half of the lookup address: table base, code book, lane
    const uint32_t lut = (uint32_t)M::kOffLut | (uint32_t)(DUAL && r >= 64 ? 128 : 0) | (uint32_t)(lane * 4);
    const int my_items = (int)blockIdx.x < n_items ? (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const uint32_t total = (uint32_t)my_items * (uint32_t)NP;
    uint4 ca = make_uint4(0, 0, 0, 0), cb = ca;
    RowMetaTc sc = RowMetaTc{0, 0, 0, 0};
    // The fetch stream runs one own pair ahead of the decode. It walks (item, pair) with
    // counters, and the first tile of the NEXT item is looked up when an item is entered,
    // so that no fetch waits for the dependent read of the tile list.
    constexpr size_t tile_b = tile_bytes(FMT);  // the launcher picks FMT from img.fmt
    // byte offsets of this thread's reads inside a tile: its 16 code bytes of half 0 and its metadata
    constexpr int kMetaRow = FMT == kQ4CP ? 4 : FMT == kQ4K ? 8 : 16;
    const uint32_t off_c = (uint32_t)r * 16u, off_m = (uint32_t)kCodeBytes + (uint32_t)r * kMetaRow;
    auto item_base = [&](int io) -> const uint8_t* {
      const int item = blockIdx.x + io * (int)gridDim.x;
      if (io >= my_items) return nullptr;
      return img.tile(p.tiles[item / img.n_mtiles].expert, item % img.n_mtiles, 0);
    };
    const int io_step = NP == 1 ? 2 : 1;  // a set visits every item, or every other one when an item is one pair
    int f_io = set / NP, f_pp = set % NP;
    const uint8_t* f_base = item_base(f_io);
    const uint8_t* f_next = item_base(f_io + io_step);
    // f_tile walks with the stream: the tile of K block 2 * f_pp + kblk of the current item
    const uint8_t* f_tile = f_base ? f_base + (size_t)(2 * f_pp + kblk) * tile_b : nullptr;
    const size_t step_b = 4 * tile_b;  // the set's next pair is two pairs = four K blocks further
    bool f_valid = false;              // the last fetch had a K block to read (false only beyond an odd tail or the last item)
    auto fetch = [&](uint4& a, uint4& b, RowMetaTc& s2x) {
      f_valid = f_tile != nullptr && 2 * f_pp + kblk < KB;
      if (f_valid) {
        const uint8_t* pc = f_tile + off_c;  // the metadata sits off_m - off_c bytes further
        a = __ldg((const uint4*)pc);
        b = __ldg((const uint4*)(pc + 2048));
        if (FMT == kQ4CP) {
          s2x.a = __ldg((const uint32_t*)(pc + (off_m - off_c)));
        } else if (FMT == kQ4K) {
          const uint2 u = __ldg((const uint2*)(pc + (off_m - off_c)));
          s2x.a = u.x;
          s2x.b = u.y;
        } else {
          const uint4 u = __ldg((const uint4*)(pc + (off_m - off_c)));
          s2x = RowMetaTc{u.x, u.y, u.z, u.w};
        }
      }
      f_pp += 2;
      if (f_pp < NP) {
        if (f_tile != nullptr) f_tile += step_b;
      } else {
        f_pp -= NP * io_step;  // NP == 1: two items further, same pair
        f_io += io_step;
        f_base = f_next;
        f_next = item_base(f_io + io_step);
        f_tile = f_base ? f_base + (size_t)(2 * f_pp + kblk) * tile_b : nullptr;
      }
    };
    fetch(ca, cb, sc);
    bool mine = f_valid;  // the codes in (ca, cb, sc) are a K block of this thread's
    bool ok = true;
    static_assert(kNS == 2, "a set always fills the tensor-memory slot of its own index");
    const uint32_t aslot = (uint32_t)set;
    uint32_t qslot = (uint32_t)set % kNBS, qph = 0;  // (pi - kNS) % kNBS and ((pi - kNS) / kNBS) & 1, from pi == set + kNS on
    for (uint32_t pi = set; pi < total && ok; pi += 2) {
      if (lane == 0 && quarter == 0) TR(2 + kblk, pi, 0);
      uint32_t v[32];
      const bool mine_now = mine;
      if (mine_now) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
          GroupDecode<FMT> gd;
          gd.init(sc, h);
          const uint4 c4 = h ? cb : ca;
          const uint32_t w4[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
          for (int q = 0; q < 4; q++) {
#pragma unroll
            for (int b = 0; b < 4; b++) {
              const uint32_t addr = __byte_perm(w4[q], lut, 0x7604u | (uint32_t)(b << 4));
              uint32_t pair;
              asm("ld.shared.b32 %0, [%1];" : "=r"(pair) : "r"(addr));
              __half2 w2 = gd.weight(pair, q * 4 + b);
              v[h * 16 + q * 4 + b] = *(uint32_t*)&w2;
            }
          }
        }
      }
      // The codes are used up: the next own pair's go into the same registers (no second set, no
      // copies). They have the rest of this iteration and the wait of the next one to arrive, and
      // the producer thread's L2 prefetch has put them close.
      fetch(ca, cb, sc);
      mine = f_valid;
      if (lane == 0 && quarter == 0) TR(2 + kblk, pi, 1);
      if (pi >= (uint32_t)kNS) {
        // the slot is free once the MMAs of the pair that used it before (pi - kNS) have completed
        ok = mbar_wait(bars + 8 * (kBarDone + qslot), qph, abort_flag, p.status, 7);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        qslot += 2;  // the set's next pair is two further
        if (qslot >= (uint32_t)kNBS) {
          qslot -= kNBS;
          qph ^= 1;
        }
      }
      if (lane == 0 && quarter == 0) TR(2 + kblk, pi, 2);
      if (mine_now) {
        tc_fence_after();
        tc_st32(tmem + ((uint32_t)(quarter * 32) << 16) + kTmemA + aslot * 64 + kblk * 32, v);
        tc_wait_st();
      }
      if (lane == 0 && quarter == 0) TR(2 + kblk, pi, 3);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kBarAFull + aslot));
    }
  } else if (warp == 3) {
    // ================= relay: "activations landed" folded into the A-slot barrier ==========
    if (lane == 0) {
      uint32_t pi = 0;
      uint32_t bslot = 0, bph = 0;  // pi % kNBS, (pi / kNBS) & 1
      uint32_t qslot = 0, qph = 0;  // the same for q = pi - kNS (valid from pi == kNS on)
      uint32_t aslot = 0;           // pi % kNS
      bool ok = true;
      for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
        for (int pp = 0; pp < NP && ok; pp++, pi++) {
          ok = mbar_wait(bars + 8 * (kBarBFull + bslot), bph, abort_flag, p.status, 9);
          if (!ok) break;
          // an arrival must fall into the barrier's current phase: the slot's previous use is
          // over once the MMAs of pair pi - kNS have completed
          if (pi >= (uint32_t)kNS) {
            ok = mbar_wait(bars + 8 * (kBarDone + qslot), qph, abort_flag, p.status, 10);
            if (!ok) break;
            if (++qslot == (uint32_t)kNBS) {
              qslot = 0;
              qph ^= 1;
            }
          }
          mbar_arrive(bars + 8 * (kBarAFull + aslot));
          if (++bslot == (uint32_t)kNBS) {
            bslot = 0;
            bph ^= 1;
          }
          if (++aslot == (uint32_t)kNS) aslot = 0;
        }
      }
    }
  } else if (warp >= 20) {
    // ================= epilogue =================
    const int quarter = warp & 3;
    float* ubuf = (float*)(smem + kOffU);
    volatile int* ep_ok = (volatile int*)(smem + kOffBar + kNumBars * 8 + 16);
    uint32_t li = 0;
    bool ok = true;
    Tile t_ahead = (int)blockIdx.x < n_items ? p.tiles[blockIdx.x / img.n_mtiles] : Tile{0, 0, 0};
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, li++) {
      const Tile t = t_ahead;
      if (it + (int)gridDim.x < n_items) t_ahead = p.tiles[(it + gridDim.x) / img.n_mtiles];
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
      // Results leave through a shared-memory tile [column = row of the expert][weight row]
      // so that every global store is a full 16-byte piece of one output row.
      const int e128 = quarter * 32 + lane;
      // (down kernel) rows from map_base on are written where the row map says
      const int map_base = !UP && p.rowmap != nullptr ? p.map_base[0] : 0x7fffffff;
      for (int c0 = 0; c0 < t.count; c0 += 32) {
        uint32_t v[32];
        tc_ld32(src + c0, v);
        tc_wait_ld();
        if (UP) {
          // gate rows live in lanes 0..63 (warps 0,1), the matching up rows in lanes 64..127
          // (warps 2,3). Each side hands half of its columns to its partner so that all four
          // warps share the SwiGLU arithmetic: gate warps finish columns 0..15, up warps 16..31.
          float* xg = ubuf;                 // [2][16][32] gate values of columns 16..31
          float* xu = ubuf + 2 * 16 * 32;   // [2][16][32] up values of columns 0..15
          __half* outs = (__half*)(ubuf + 4 * 16 * 32);  // [32][64]
          const int pq = quarter & 1;
          if (quarter < 2) {
#pragma unroll
            for (int j = 0; j < 16; j++) xg[(pq * 16 + j) * 32 + lane] = __uint_as_float(v[16 + j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; j++) xu[(pq * 16 + j) * 32 + lane] = __uint_as_float(v[j]);
          }
          asm volatile("bar.sync 2, 128;" ::: "memory");
          if (quarter < 2) {
#pragma unroll
            for (int j = 0; j < 16; j++) {
              const float g = __uint_as_float(v[j]), u = xu[(pq * 16 + j) * 32 + lane];
              outs[j * 64 + pq * 32 + lane] = f16_sat(__fdividef(g, 1.f + __expf(-g)) * u);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; j++) {
              const float u = __uint_as_float(v[16 + j]), g = xg[(pq * 16 + j) * 32 + lane];
              outs[(16 + j) * 64 + pq * 32 + lane] = f16_sat(__fdividef(g, 1.f + __expf(-g)) * u);
            }
          }
          asm volatile("bar.sync 3, 128;" ::: "memory");
#pragma unroll
          for (int k = 0; k < 2; k++) {
            const int piece = e128 + 128 * k, col = piece >> 3, seg = piece & 7;
            if (c0 + col < t.count)
              *(uint4*)(p.out + (size_t)(t.first + c0 + col) * p.out_ld + mt * 64 + seg * 8) =
                  *(const uint4*)(outs + col * 64 + seg * 8);
          }
        } else {
          // (writing the values straight to global memory -- 2-byte stores, 64 contiguous bytes per
          // warp and row, no shared-memory transposition and no barrier -- was measured slower:
          // 1.87 ms against 1.54 ms for the down launch of the benchmark layer)
          __half* outs = (__half*)ubuf;  // [32][128]
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            // two values per conversion; finite values saturate to the fp16 range, NaN stays NaN
            uint32_t h2;
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(h2) : "f"(__uint_as_float(v[j + 1])), "f"(__uint_as_float(v[j])));
            outs[j * 128 + e128] = __ushort_as_half((unsigned short)(h2 & 0xFFFFu));
            outs[(j + 1) * 128 + e128] = __ushort_as_half((unsigned short)(h2 >> 16));
          }
          asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
          for (int k = 0; k < 4; k++) {
            const int piece = e128 + 128 * k, col = piece >> 4, seg = piece & 15;
            if (c0 + col < t.count) {
              const int row = t.first + c0 + col;
              const size_t orow = row >= map_base ? (size_t)p.rowmap[row - map_base] : (size_t)row;
              *(uint4*)(p.out + orow * p.out_ld + mt * 128 + seg * 8) = *(const uint4*)(outs + col * 128 + seg * 8);
            }
          }
          asm volatile("bar.sync 3, 128;" ::: "memory");
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

template <bool UP, bool DUAL, int FMT>
cudaError_t launch(TcPlan* plan, const CUtensorMap* m, const Image& img,
                   const Tile* tiles, const int32_t* n_tiles, int max_tiles, __half* out, int out_ld,
                   int32_t* status, cudaStream_t st, const int32_t* rowmap = nullptr, const int32_t* map_base = nullptr) {
  constexpr int kSmemBytes = Map::kSmemBytes;
  static bool attr_set = false;  // one flag per template instance
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(k_expert_tc<UP, DUAL, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  static const int l2_ahead = getenv("B200MOE_TC_L2_AHEAD") ? atoi(getenv("B200MOE_TC_L2_AHEAD")) : 3;
  KParams p{img, tiles, n_tiles, out, out_ld, status, (UP != (getenv("B200MOE_TC_TRACE_DOWN") != nullptr)) ? plan->trace : nullptr,
            l2_ahead, rowmap, map_base};
  long long max_items = (long long)max_tiles * img.n_mtiles;
  const int usable = plan->sms - plan->margin > 1 ? plan->sms - plan->margin : 1;
  int grid = (int)(max_items < usable ? max_items : usable);
  if (grid < 1) grid = 1;
  k_expert_tc<UP, DUAL, FMT><<<grid, kThreads, kSmemBytes, st>>>(m[0], m[1], m[2], m[3], p);
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

void tc_set_sm_margin(TcPlan* plan, int sms) {
  if (plan) plan->margin = sms < 0 ? 0 : sms;
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
  if (img.fmt == kQ4K)
    return launch<true, false, kQ4K>(plan, plan->x, img, tiles, n_tiles, max_tiles, hid16, img.n_mtiles * 64, status, st);
  if (img.fmt == kQ51)  // Q5_K gate/up in the Q5_1 image form
    return launch<true, false, kQ51>(plan, plan->x, img, tiles, n_tiles, max_tiles, hid16, img.n_mtiles * 64, status, st);
  if (img.fmt != kQ4CP) return cudaErrorNotSupported;
  if (img.dual_book)
    return launch<true, true, kQ4CP>(plan, plan->x, img, tiles, n_tiles, max_tiles, hid16, img.n_mtiles * 64, status, st);
  return launch<true, false, kQ4CP>(plan, plan->x, img, tiles, n_tiles, max_tiles, hid16,
                      img.n_mtiles * 64, status, st);
}

cudaError_t launch_down_tc(TcPlan* plan, const Image& img, const Tile* tiles, const int32_t* n_tiles,
                           int max_tiles, __half* pairs16, int32_t* status, cudaStream_t st, const int32_t* rowmap,
                           const int32_t* map_base) {
  if ((rowmap == nullptr) != (map_base == nullptr)) return cudaErrorInvalidValue;
  if (img.fmt == kQ51)
    return launch<false, false, kQ51>(plan, plan->h, img, tiles, n_tiles, max_tiles, pairs16, img.n_mtiles * 128, status, st,
                                      rowmap, map_base);
  if (img.fmt != kQ4CP) return cudaErrorNotSupported;
  return launch<false, false, kQ4CP>(plan, plan->h, img, tiles, n_tiles, max_tiles, pairs16,
                       img.n_mtiles * 128, status, st, rowmap, map_base);
}

cudaError_t launch_raw_tc(TcPlan* plan, const Image& img, const Tile* tiles, const int32_t* n_tiles,
                          int max_tiles, __half* z16, int32_t* status, cudaStream_t st) {
  if (img.fmt != kQ4CP || img.paired) return cudaErrorNotSupported;
  return launch<false, false, kQ4CP>(plan, plan->x, img, tiles, n_tiles, max_tiles, z16, img.n_mtiles * 128, status, st);
}

}  // namespace b200moe
