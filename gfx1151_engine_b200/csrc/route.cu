// route.cu -- router top-k and the expert bucketing of (token, slot) pairs.
//
// Semantics follow the reference:
//   * probabilities as its CPU path forms them (src/ref.cpp:574-582): exp in double of
//     (logit - max), rounded to float, summed in double in index order, divided in
//     double, rounded to float; selection of the k largest, descending, ties to the lowest
//     expert id (the rule of its GPU router, src/gpu/parts/20_kernels_gemv.inc:1488-1494);
//     weights p / sum(selected p) with the sum taken in rank order (src/ref.cpp:587-588, 606).
//   * bucketing = stable sort of pair index p = t*k + s by expert
//     (src/gpu/parts/10_ple_io.inc:844-853; CPU twin src/gpu/parts/40_model.inc:4171-4183),
//     eoff filled for empty experts too, pairids[t*k + rank] with rank = number of the
//     token's experts with a smaller id (src/gpu/parts/10_ple_io.inc:802-806).
// Everything here is integer/bookkeeping work and deterministic: no atomics on global
// memory, no dependence on block scheduling order.
#include "kernels.h"
#include "route_small.cuh"

namespace b200moe {

namespace {

constexpr int kRouterWarps = 8;

constexpr int kChunk = 512;  // pairs handled by one single-warp block of the bucketing kernels

__device__ __forceinline__ double shfl_double(double v, int src) {
  int lo = __double2loint(v), hi = __double2hiint(v);
  lo = __shfl_sync(0xffffffffu, lo, src);
  hi = __shfl_sync(0xffffffffu, hi, src);
  return __hiloint2double(hi, lo);
}

// Router for one token by one warp, E <= 512: lane holds experts lane, lane+32, ...
// sp: this warp's scratch row of kMaxExperts floats in shared memory.
__device__ __forceinline__ void router_one_token(const float* __restrict__ lg, int E, int k, int lane,
                                                 float* sp, int32_t* __restrict__ ids_row,
                                                 float* __restrict__ w_row, int stride) {
  float v[16];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 16; j++) {
    int e = j * 32 + lane;
    v[j] = e < E ? lg[e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const double dmx = (double)mx;
#pragma unroll
  for (int j = 0; j < 16; j++) {
    int e = j * 32 + lane;
    float p = e < E ? (float)exp((double)v[j] - dmx) : 0.f;
    if (e < E) sp[e] = p;
    v[j] = p;
  }
  __syncwarp();
  // Sum of the exponentials, as the reference takes it: in double, in index order. All terms
  // are floats in (0, 1]: when the smallest non-zero one's last mantissa bit still fits a
  // double that holds the total, every partial sum of ANY order is exact, so the tree sum has
  // the very same bits and the E dependent additions are only needed otherwise.
  double se = 0;
  float mn = 2.f;
#pragma unroll
  for (int j = 0; j < 16; j++)
    if (j * 32 + lane < E) {
      se += (double)v[j];
      if (v[j] > 0.f) mn = fminf(mn, v[j]);
    }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    se += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(se), o),
                           __shfl_xor_sync(0xffffffffu, __double2loint(se), o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  se = shfl_double(se, 0);  // (inexact sums may differ between lanes in the last bit: take one)
  {
    const int e_min = (int)((__float_as_uint(mn) >> 23) & 0xFF) - 127;
    const int bits_total = (int)((__double2hiint(se) >> 20) & 0x7FF) - 1023 + 2;  // generous by one bit
    const bool exact = mn >= 1.17549435e-38f && bits_total - (e_min - 23) <= 53;
    if (!exact) {  // warp-uniform: mn and se are the same in every lane
      se = 0;
      if (lane == 0)
        for (int i = 0; i < E; i++) se += (double)sp[i];  // index order, as the reference sums
      se = shfl_double(se, 0);
    }
  }
#pragma unroll
  for (int j = 0; j < 16; j++) {
    int e = j * 32 + lane;
    v[j] = e < E ? (float)((double)v[j] / se) : -1.f;
  }
  int my_id = 0;
  float my_p = 0.f;
  double kept = 0;
  for (int r = 0; r < k; r++) {
    // The search starts from an id inside [0, E) (the reference's GPU router starts at `lane`,
    // src/gpu/parts/20_kernels_gemv.inc:1517): with a non-finite logit every probability is NaN, no
    // comparison below is ever true, and the ids written are then still valid expert numbers
    // (with NaN weights, so the token's output is NaN) instead of an out-of-range value.
    float bv = -1.f;
    int bi = min(lane, E - 1);
#pragma unroll
    for (int j = 0; j < 16; j++)
      if (v[j] > bv) {
        bv = v[j];
        bi = j * 32 + lane;
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    bi = __shfl_sync(0xffffffffu, bi, 0);  // (NaN probabilities: the lanes may disagree; take lane 0's)
    bv = __shfl_sync(0xffffffffu, bv, 0);
    if (bv < 0.f) bv = __int_as_float(0x7fc00000);  // nothing was selectable: the weight is NaN, as in the reference
#pragma unroll
    for (int j = 0; j < 16; j++)
      if (j == (bi >> 5) && lane == (bi & 31)) v[j] = -1.f;
    if (lane == r) {
      my_id = bi;
      my_p = bv;
    }
    kept += (double)bv;
  }
  for (int i = lane; i < stride; i += 32) {
    // lanes >= k hold zeros; stride > 32 is padded with zeros as well
    bool valid = i < k && i < 32;
    ids_row[i] = valid ? my_id : 0;
    w_row[i] = valid ? (float)((double)my_p / kept) : 0.f;
  }
}

__global__ void __launch_bounds__(kRouterWarps * 32)
k_router_topk(const float* __restrict__ logits, int T, int E, int k, int32_t* __restrict__ ids,
              float* __restrict__ w, int stride) {
  __shared__ float s_p[kRouterWarps][kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouterWarps + warp;
  if (t >= T) return;
  router_one_token(logits + (size_t)t * E, E, k, lane, s_p[warp], ids + (size_t)t * stride,
                   w + (size_t)t * stride, stride);
}

// Decode / verify (T*k <= 256): the whole routing stage in ONE block (route_small.cuh).
__global__ void __launch_bounds__(kMaxExperts, 1)
k_route_small(const float* __restrict__ logits, const int32_t* __restrict__ ids_in,
              const float* __restrict__ w_in, int stride_in, int T, int E, int k, RouteBuffers rb,
              const uint16_t* __restrict__ x, const uint16_t* __restrict__ gw, int d) {
  __shared__ RouteSmallScratch<16> sc;
  pdl_trigger();
  pdl_wait();  // inputs may come from the previous kernel; the buffers written here may still be read by it
  RouteSmallOut o;
  o.topids = rb.topids; o.topw = rb.topw; o.tokidx = rb.tokidx; o.pw = rb.pw; o.pairids = rb.pairids;
  o.eoff = rb.eoff; o.runs = rb.runs; o.shared_slot = kMaxExperts; o.n_runs = rb.n_runs; o.tiles = rb.tiles;
  o.tiles_sh = rb.tiles_sh; o.n_tiles = rb.n_tiles; o.sgate = rb.sgate;
  route_small_body<16>(logits, ids_in, w_in, stride_in, T, E, k, x, gw, d, sc, o, RouteSmallOut{}, rb.status);
}

__global__ void __launch_bounds__(32)
k_route_count(const int32_t* __restrict__ ids, int stride, int pairs, int k, int E,
              int32_t* __restrict__ blockcnt, int32_t* __restrict__ status) {
  __shared__ int hist[kMaxExperts];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) hist[e] = 0;
  __syncwarp();
  const int base = blockIdx.x * kChunk;
  for (int it = 0; it < kChunk / 32; it++) {
    int p = base + it * 32 + lane;
    if (p < pairs) {
      const int e = ids[(size_t)(p / k) * stride + p % k];
      if ((unsigned)e < (unsigned)E) atomicAdd(&hist[e], 1);  // ids outside [0, E) are dropped, never used as an index
      else if (status && atomicCAS(status, 0, kStatusBadId) == 0) status[1] = e;
    }
  }
  __syncwarp();
  for (int e = lane; e < E; e += 32) blockcnt[(size_t)blockIdx.x * E + e] = hist[e];
}

// One block of 512 threads: per-expert exclusive prefix over the chunk counts, expert
// offsets, the list of non-empty experts and the grouped-GEMM tile list (full tiles first,
// then the ragged ones in descending size so that a static round-robin stays balanced).
__global__ void __launch_bounds__(kMaxExperts)
k_route_scan(int32_t* __restrict__ blockcnt, int nblk, int E, int pairs, int T, int tile_cap,
             int32_t* __restrict__ eoff, Run* __restrict__ runs, int32_t* __restrict__ n_runs,
             Tile* __restrict__ tiles, Tile* __restrict__ tiles_sh, int32_t* __restrict__ n_tiles) {
  __shared__ int s_a[kMaxExperts], s_b[kMaxExperts], s_c[kMaxExperts];
  const int e = threadIdx.x;
  int cnt = 0;
  if (e < E) {
    // exclusive prefix down this expert's column of the chunk counts; the loads of eight
    // rows are issued together so that the walk does not pay one memory latency per chunk
    int b = 0;
    for (; b + 8 <= nblk; b += 8) {
      int c[8];
#pragma unroll
      for (int i = 0; i < 8; i++) c[i] = blockcnt[(size_t)(b + i) * E + e];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        blockcnt[(size_t)(b + i) * E + e] = cnt;
        cnt += c[i];
      }
    }
    for (; b < nblk; b++) {
      const int c = blockcnt[(size_t)b * E + e];
      blockcnt[(size_t)b * E + e] = cnt;
      cnt += c;
    }
  }
  // three inclusive scans side by side: counts, non-empty flags, full tiles
  const int nfull = cnt / tile_cap, part = cnt % tile_cap;
  s_a[e] = cnt;
  s_b[e] = cnt > 0;
  s_c[e] = nfull;
  __syncthreads();
  for (int o = 1; o < kMaxExperts; o <<= 1) {
    int a = e >= o ? s_a[e - o] : 0, b = e >= o ? s_b[e - o] : 0, c = e >= o ? s_c[e - o] : 0;
    __syncthreads();
    s_a[e] += a;
    s_b[e] += b;
    s_c[e] += c;
    __syncthreads();
  }
  const int first = s_a[e] - cnt;
  const int total_full = s_c[kMaxExperts - 1];
  if (e < E) eoff[e] = first;
  if (e == 0) {
    eoff[E] = s_a[kMaxExperts - 1];  // pairs placed (= T*k unless ids outside [0, E) were dropped)
    n_runs[0] = s_b[kMaxExperts - 1];
    n_runs[1] = 1;  // the shared expert's run, kept at runs[kMaxExperts]
    runs[kMaxExperts] = Run{0, pairs, T};
  }
  if (cnt > 0) runs[s_b[e] - 1] = Run{e, first, cnt};
  const int full0 = s_c[e] - nfull;
  for (int j = 0; j < nfull; j++) tiles[full0 + j] = Tile{e, first + j * tile_cap, tile_cap};
  __syncthreads();
  // rank of the ragged tile among all ragged tiles: larger first, ties to the lower id
  s_a[e] = part;
  __syncthreads();
  int rank = 0, nparts = 0;
  for (int o = 0; o < kMaxExperts; o++) {
    int p = s_a[o];
    nparts += p > 0;
    rank += (p > part) || (p == part && o < e);
  }
  if (part > 0) tiles[total_full + rank] = Tile{e, first + nfull * tile_cap, part};
  // tiles of the shared expert: all T tokens in token order, rows behind the routed ones
  const int nsh = (T + tile_cap - 1) / tile_cap;
  for (int j = e; j < nsh; j += kMaxExperts)
    tiles_sh[j] = Tile{0, pairs + j * tile_cap, min(tile_cap, T - j * tile_cap)};
  if (e == 0) {
    n_tiles[0] = total_full + nparts;
    n_tiles[1] = nsh;
  }
}

__global__ void __launch_bounds__(32)
k_route_place(const int32_t* __restrict__ ids, const float* __restrict__ w, int stride, int pairs,
              int k, int E, const int32_t* __restrict__ blockcnt, const int32_t* __restrict__ eoff,
              int32_t* __restrict__ tokidx, float* __restrict__ pw, int32_t* __restrict__ pairids) {
  __shared__ int cursor[kMaxExperts];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) cursor[e] = eoff[e] + blockcnt[(size_t)blockIdx.x * E + e];
  __syncwarp();
  const int base = blockIdx.x * kChunk;
  for (int it = 0; it < kChunk / 32; it++) {
    const int p = base + it * 32 + lane;
    const bool live = p < pairs;
    const unsigned act = __ballot_sync(0xffffffffu, live);
    if (live) {
      const int t = p / k, s = p % k;
      const int e = ids[(size_t)t * stride + s];
      const bool good = (unsigned)e < (unsigned)E;
      const unsigned same = __match_any_sync(act, good ? e : -1);
      const int leader = __ffs(same) - 1;
      int start = 0;
      if (good && lane == leader) {
        start = cursor[e];
        cursor[e] = start + __popc(same);
      }
      start = __shfl_sync(same, start, leader);
      const int row = start + __popc(same & ((1u << lane) - 1u));
      if (good) {
        tokidx[row] = t;
        pw[row] = w[(size_t)t * stride + s];
      }
      // slot in the token's reduce order: ascending expert id; equal ids keep their slot order,
      // so every slot is written; a dropped pair's slot holds -1 (the combine skips it)
      int rank = 0;
      const int key = good ? e : kBadKey;
      for (int q = 0; q < k; q++) {
        const int eq = ids[(size_t)t * stride + q];
        const int kq = (unsigned)eq < (unsigned)E ? eq : kBadKey;  // dropped pairs sort behind every expert
        rank += (kq < key) || (kq == key && q < s);
      }
      pairids[(size_t)t * k + rank] = good ? row : -1;
    }
    __syncwarp();
  }
}

// Scalar sigmoid gate of the shared expert (src/ref.cpp:623-626, 635): one warp per token.
// Also appends the shared expert's rows (token order) behind the routed rows.
__global__ void __launch_bounds__(256)
k_shared_gate(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gw, int T, int d, int k,
              int32_t* __restrict__ tokidx, float* __restrict__ pw, float* __restrict__ sgate) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= T) return;
  double a = 0;
  for (int c = lane; c < d; c += 32)
    a += (double)bf16_bits_to_f32(gw[c]) * (double)bf16_bits_to_f32(x[(size_t)t * d + c]);
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    int lo = __shfl_xor_sync(0xffffffffu, __double2loint(a), o);
    int hi = __shfl_xor_sync(0xffffffffu, __double2hiint(a), o);
    a += __hiloint2double(hi, lo);
  }
  if (lane == 0) {
    float g = sigmoid_f32((float)a);
    sgate[t] = g;
    tokidx[(size_t)T * k + t] = t;
    pw[(size_t)T * k + t] = g;
  }
}

}  // namespace

cudaError_t launch_router_topk(const float* logits, int T, int E, int k, int32_t* ids, float* w,
                               int stride, cudaStream_t st) {
  k_router_topk<<<(T + kRouterWarps - 1) / kRouterWarps, kRouterWarps * 32, 0, st>>>(
      logits, T, E, k, ids, w, stride);
  return cudaGetLastError();
}

cudaError_t launch_route(const RouteBuffers& rb, const int32_t* ids, const float* w, int stride,
                         int T, int k, int E, int tile_cap, cudaStream_t st, int* launches) {
  const int pairs = T * k;
  const int nblk = (pairs + kChunk - 1) / kChunk;
  k_route_count<<<nblk, 32, 0, st>>>(ids, stride, pairs, k, E, rb.blockcnt, rb.status);
  k_route_scan<<<1, kMaxExperts, 0, st>>>(rb.blockcnt, nblk, E, pairs, T, tile_cap, rb.eoff, rb.runs,
                                           rb.n_runs, rb.tiles, rb.tiles_sh, rb.n_tiles);
  k_route_place<<<nblk, 32, 0, st>>>(ids, w, stride, pairs, k, E, rb.blockcnt, rb.eoff, rb.tokidx,
                                     rb.pw, rb.pairids);
  if (launches) *launches += 3;
  return cudaGetLastError();
}

cudaError_t launch_shared_gate(const void* x_bf16, const uint16_t* gate_w_bf16, int T, int d, int k,
                               const RouteBuffers& rb, cudaStream_t st) {
  k_shared_gate<<<(T + 7) / 8, 256, 0, st>>>((const uint16_t*)x_bf16, gate_w_bf16, T, d, k,
                                             rb.tokidx, rb.pw, rb.sgate);
  return cudaGetLastError();
}

// ---- expert parallelism ---------------------------------------------------------------
// ids <- place[ids]: experts renumbered so that rank r owns the ids [r*E/G, (r+1)*E/G).
__global__ void k_apply_placement(int32_t* __restrict__ ids, int stride, int T, int k, int E,
                                  const int32_t* __restrict__ place) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p < T * k) {
    int32_t* q = ids + (size_t)(p / k) * stride + p % k;
    if ((unsigned)*q < (unsigned)E) *q = place[*q];
  }
}

// Work list of the receiving rank. The receive buffer holds, source rank after source rank,
// that source's rows for this rank's experts in ascending expert order; eoff_all[s] is source
// s's expert offset table (E+1 entries). One thread per (source, local expert) segment:
// its position in the buffer, then tiles of at most tile_cap rows (full tiles first, ragged
// ones by descending size), exactly as the single-GPU tile list is built.
//
// part 4 (the other ranks' rows with their TAILS MERGED by expert): the receive buffer is
// source-major, so an expert that got rows from seven ranks has seven segments there and up to
// seven ragged tiles. Full tiles of a segment stay where they are; the rows behind a segment's
// last full tile (its tail) are copied behind the received rows, expert after expert, and tiled
// there: one ragged tile per expert instead of one per (source, expert). segs[] lists the tails in
// the order of their destination, {first row in the receive buffer, first row in the merged area,
// rows}; counts[1] = received rows R (the merged area starts there), counts[2] = merged rows (0
// when the buffer has no room for them behind R: the list is then part 2's).
__global__ void __launch_bounds__(kMaxExperts)
k_ep_tiles(const int32_t* __restrict__ eoff_all, int G, int E, int e0, int El, int tile_cap, int own, int part,
           Tile* __restrict__ tiles, int32_t* __restrict__ n_tiles, int32_t* __restrict__ counts,
           int32_t* __restrict__ segs, int cap_rows) {
  __shared__ int s_a[kMaxExperts], s_c[kMaxExperts];
  const int tid = threadIdx.x;
  const int src = tid / El, e = tid % El;
  const bool live = tid < G * El;
  int cnt = 0, first = 0;
  if (live) {
    const int32_t* eo = eoff_all + (size_t)src * (E + 1);
    cnt = eo[e0 + e + 1] - eo[e0 + e];
    first = eo[e0 + e] - eo[e0];                      // offset inside the source's segment
    for (int s2 = 0; s2 < src; s2++) {                // segments of the sources before it
      const int32_t* e2 = eoff_all + (size_t)s2 * (E + 1);
      first += e2[e0 + El] - e2[e0];
    }
    // part 1: only the rows this rank sent to itself; part 2 and 4: only the other ranks' rows;
    // part 3: this rank's own rows where they lie in its SEND buffer (row = its own expert offset)
    if ((part == 1 && src != own) || ((part == 2 || part == 4) && src == own) || (part == 3 && src != own)) cnt = 0;
    if (part == 3) first = eo[e0 + e];
  }
  int R = 0;  // rows of the source-major layout
  for (int s2 = 0; s2 < G; s2++) {
    const int32_t* e2 = eoff_all + (size_t)s2 * (E + 1);
    R += e2[e0 + El] - e2[e0];
  }
  // tiles of this thread: nf_a full tiles from first, nf_b full tiles from first_b, one ragged tile
  int nf_a = cnt / tile_cap, nf_b = 0, first_b = 0, rag = cnt % tile_cap, rag_first = first + nf_a * tile_cap;
  int merged_rows = 0;
  if (part == 4) {
    const int tail = rag;
    s_c[tid] = tail;
    __syncthreads();
    int before = 0, ttot = 0;  // tail rows of expert e from the sources before this one, from all
    if (live)
      for (int s2 = 0; s2 < G; s2++) {
        const int c2 = s_c[s2 * El + e];
        ttot += c2;
        before += s2 < src ? c2 : 0;
      }
    __syncthreads();
    if (tid < El) s_a[tid] = ttot;
    __syncthreads();
    int tbase = 0, all_tails = 0;  // tail rows of the experts before e, of all experts
    for (int e2 = 0; e2 < El; e2++) {
      all_tails += s_a[e2];
      tbase += e2 < e ? s_a[e2] : 0;
    }
    __syncthreads();
    if (R + all_tails <= cap_rows) {
      merged_rows = all_tails;
      if (live) {
        int32_t* sg = segs + 3 * (e * G + src);   // destination order: expert-major
        sg[0] = rag_first;
        sg[1] = R + tbase + before;
        sg[2] = tail;
      }
      // the tail leaves this thread; the thread of source 0 tiles the expert's merged tails
      rag = 0;
      if (live && src == 0) {
        nf_b = ttot / tile_cap;
        first_b = R + tbase;
        rag = ttot % tile_cap;
        rag_first = first_b + nf_b * tile_cap;
      }
    }
  }
  const int nfull = nf_a + nf_b;
  s_c[tid] = nfull;
  __syncthreads();
  for (int o = 1; o < kMaxExperts; o <<= 1) {
    const int c = tid >= o ? s_c[tid - o] : 0;
    __syncthreads();
    s_c[tid] += c;
    __syncthreads();
  }
  const int total_full = s_c[kMaxExperts - 1], full0 = s_c[tid] - nfull;
  for (int j = 0; j < nf_a; j++) tiles[full0 + j] = Tile{e, first + j * tile_cap, tile_cap};
  for (int j = 0; j < nf_b; j++) tiles[full0 + nf_a + j] = Tile{e, first_b + j * tile_cap, tile_cap};
  s_a[tid] = rag;
  __syncthreads();
  int rank = 0, nparts = 0;
  for (int o = 0; o < kMaxExperts; o++) {
    const int pp = s_a[o];
    nparts += pp > 0;
    rank += (pp > rag) || (pp == rag && o < tid);
  }
  if (rag > 0) tiles[total_full + rank] = Tile{e, rag_first, rag};
  if (tid == 0) {
    n_tiles[0] = total_full + nparts;
    counts[0] = R;
    counts[1] = merged_rows;
  }
}

cudaError_t launch_apply_placement(int32_t* ids, int stride, int T, int k, int E, const int32_t* place,
                                   cudaStream_t st) {
  k_apply_placement<<<(T * k + 255) / 256, 256, 0, st>>>(ids, stride, T, k, E, place);
  return cudaGetLastError();
}

cudaError_t launch_ep_tiles(const int32_t* eoff_all, int G, int E, int e0, int El, int tile_cap,
                            Tile* tiles, int32_t* n_tiles, int32_t* counts, cudaStream_t st, int own, int part,
                            int32_t* segs, int cap_rows) {
  if (part == 4 && !segs) return cudaErrorInvalidValue;
  k_ep_tiles<<<1, kMaxExperts, 0, st>>>(eoff_all, G, E, e0, El, tile_cap, own, part, tiles, n_tiles, counts, segs, cap_rows);
  return cudaGetLastError();
}

// The tails of part 4 copied into the merged area behind the received rows: one warp per merged
// row; its segment is found by bisection in segs[] (in destination order; empty segments share
// their first row with the next one, so the LAST segment starting at or before the row holds it).
// rowmap[merged row - R] = the row's place in the source-major layout: the down GEMM writes the
// result there, so that results leave in the senders' order without another pass.
__global__ void __launch_bounds__(256)
k_ep_merge_tails(uint4* __restrict__ x_recv, const int32_t* __restrict__ segs, int n_seg,
                 const int32_t* __restrict__ counts, int per_row, int32_t* __restrict__ rowmap) {
  __shared__ int s_src[kMaxExperts], s_dst[kMaxExperts];
  for (int i = threadIdx.x; i < n_seg; i += blockDim.x) {
    s_src[i] = segs[3 * i];
    s_dst[i] = segs[3 * i + 1];
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int R = counts[0], rows = counts[1];
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < rows; i += n_warps) {
    const int dst = R + i;
    int lo = 0, hi = n_seg - 1;
    while (lo < hi) {
      const int m = (lo + hi + 1) >> 1;
      if (s_dst[m] <= dst) lo = m; else hi = m - 1;
    }
    const int j = s_src[lo] + (dst - s_dst[lo]);
    const uint4* src = x_recv + (size_t)j * per_row;
    uint4* out = x_recv + (size_t)dst * per_row;
    for (int v = lane; v < per_row; v += 32) out[v] = src[v];
    if (lane == 0) rowmap[i] = j;
  }
}

cudaError_t launch_ep_merge_tails(__half* x_recv, const int32_t* segs, int n_seg, const int32_t* counts, int d,
                                  int32_t* rowmap, int sms, cudaStream_t st) {
  k_ep_merge_tails<<<sms * 4, 256, 0, st>>>((uint4*)x_recv, segs, n_seg, counts, d / 8, rowmap);
  return cudaGetLastError();
}

cudaError_t launch_route_small(const RouteBuffers& rb, const float* logits, const int32_t* ids,
                               const float* w, int stride, int T, int k, int E, const void* x_bf16,
                               const uint16_t* gate_w_bf16, int d, cudaStream_t st) {
  return launch_pdl(k_route_small, dim3(1), dim3(kMaxExperts), 0, st, logits, ids, w, stride, T, E, k, rb, (const uint16_t*)x_bf16,
                                           gate_w_bf16, d);
}

// Waits until every one of n flags (written by peer GPUs' copy engines behind their data)
// has reached `expected`. Bounded: after 2 s the kernel records status {3, index of the
// missing flag} and returns, so that the context stays usable and the host sees the timeout.
__global__ void k_wait_flags(const int32_t* flags, int n, int32_t expected, int32_t* status) {
  const int i = threadIdx.x;
  if (i >= n) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t spin = 0;; spin++) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
    if (v - expected >= 0) return;
    if ((spin & 63u) == 63u) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > 2000000000ull) {
        if (atomicCAS(status, 0, 3) == 0) status[1] = i;
        return;
      }
      __nanosleep(200);
    }
  }
}

cudaError_t launch_wait_flags(const int32_t* flags, int n, int32_t expected, int32_t* status, cudaStream_t st) {
  k_wait_flags<<<1, 32, 0, st>>>(flags, n, expected, status);
  return cudaGetLastError();
}

int route_small_max_pairs() { return kSmallPairs; }
int route_chunk() { return kChunk; }

}  // namespace b200moe
