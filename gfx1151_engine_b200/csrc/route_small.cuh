// route_small.cuh -- the whole routing stage for a few tokens (T*k <= 256) as a device function
// run by 512 threads of one block: shared expert's sigmoid gate, router top-k, stable bucketing
// by rank counting, expert offsets, run and tile lists. Used by k_route_small (route.cu) and by
// the fused decode kernel (decode.cu), where every block repeats it for itself.
// Arithmetic and tie rule: see route.cu.
#pragma once
#include "kernels.h"

namespace b200moe {

constexpr int kBadKey = 0x7fffffff;   // sort key of a dropped pair (expert id outside [0, E))
constexpr int kStatusBadId = 4;       // status word {4, offending id}: reported as B200MOE_ERR_BAD_ARG

// Decode / verify (T*k <= 256): the whole routing stage in ONE block -- router top-k (when
// logits are given), stable bucketing by rank counting, expert offsets, run and tile lists,
// and the shared expert's sigmoid gate. Same results as the general kernels below.
constexpr int kSmallPairs = 256;

// Shared-memory scratch of the routing body; NROW = most tokens it is used for (at least 3:
// the single-token selection keeps its candidate list in rows 1 and 2).
template <int NROW>
struct RouteSmallScratch {
  double se[16], part[16];
  float p[NROW][kMaxExperts];  // router scratch, one row per token
  int key[kSmallPairs];
  float w[kSmallPairs];
  int wcnt[17];
  float bv[2][16];
  int bi[2][16];
};

// Where the body leaves its results. Every pointer may be null (that result is then not
// stored); the body takes two of these so that a fused kernel can keep what it needs in shared
// memory and still leave the complete set in the handle's global workspace.
struct RouteSmallOut {
  int32_t* topids = nullptr;   // [T][16]
  float* topw = nullptr;       // [T][16]
  int32_t* tokidx = nullptr;   // [T*k (+T)]
  float* pw = nullptr;         // [T*k (+T)]
  int32_t* pairids = nullptr;  // [T*k]
  int32_t* eoff = nullptr;     // [E+1]
  Run* runs = nullptr;         // non-empty experts in ascending id; the shared expert's run at [shared_slot]
  int shared_slot = kMaxExperts;
  int32_t* n_runs = nullptr;   // [2]
  Tile* tiles = nullptr;
  Tile* tiles_sh = nullptr;
  int32_t* n_tiles = nullptr;  // [2]
  float* sgate = nullptr;      // [T]
};
#define RS_PUT(field, idx, val)                 \
  do {                                          \
    if (o1.field) o1.field[idx] = (val);        \
    if (o2.field) o2.field[idx] = (val);        \
  } while (0)

// barrier of the 512 threads that run the body (named barrier 1: the kernel around it may have
// more warps, which do not take part)
__device__ __forceinline__ void rs_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// Run by threads 0..511 of a block (tid = threadIdx.x < 512). Inputs as k_route_small's.
// GU: 16-byte pieces of the shared expert's gate product a lane loads before it uses any (a
// register-hungry prefetch: 8 where the body has the whole SM's registers, 2 inside a larger kernel).
template <int NROW, int GU = 8>
__device__ __forceinline__ void route_small_body(
    const float* __restrict__ logits, const int32_t* __restrict__ ids_in, const float* __restrict__ w_in,
    int stride_in, int T, int E, int k, const uint16_t* __restrict__ x, const uint16_t* __restrict__ gw, int d,
    RouteSmallScratch<NROW>& sc, const RouteSmallOut& o1, const RouteSmallOut& o2, int32_t* status,
    unsigned long long* dbg = nullptr) {
#define RS_STAMP(i)                                                     \
  do {                                                                  \
    if (dbg && threadIdx.x == 0) {                                      \
      unsigned long long t_;                                            \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));            \
      dbg[i] = t_;                                                      \
    }                                                                   \
  } while (0)
  float (*s_p)[kMaxExperts] = sc.p;
  int* s_key = sc.key;
  float* s_w = sc.w;
  int* s_wcnt = sc.wcnt;
  float (*s_bv)[16] = sc.bv;
  int (*s_bi)[16] = sc.bi;
  double* s_se = sc.se;
  double* s_part = sc.part;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int P = T * k;
  // W = 16 / T' warps share a token (T' = T rounded up to a power of two)
  const int Tp = T <= 1 ? 1 : T <= 2 ? 2 : T <= 4 ? 4 : T <= 8 ? 8 : 16;
  const int W = 16 / Tp, ts = warp / W, wq = warp % W;  // token slot, warp in the token's group
  const bool tok = ts < T;
  if (gw) {
    // scalar sigmoid gate of the shared expert: a d-long dot product in double, 16-byte
    // loads spread over the token's warps, partial sums added in a fixed order
    double a = 0;
    if (tok) {
      const uint4* xv = (const uint4*)(x + (size_t)ts * d);
      const uint4* gv = (const uint4*)gw;
      // eight pieces per lane are loaded before any is used (with one warp per token the loop
      // would otherwise pay a global-load latency per piece); the additions keep their order
      for (int c0 = wq * 32 + lane; c0 < d / 8; c0 += W * 32 * GU) {
        uint4 xa[GU], ga[GU];
#pragma unroll
        for (int u = 0; u < GU; u++) {
          const int c = c0 + u * W * 32;
          if (c < d / 8) {
            xa[u] = xv[c];
            ga[u] = __ldg(gv + c);
          }
        }
#pragma unroll
        for (int u = 0; u < GU; u++) {
          if (c0 + u * W * 32 < d / 8) {
            const uint32_t xw[4] = {xa[u].x, xa[u].y, xa[u].z, xa[u].w}, gq[4] = {ga[u].x, ga[u].y, ga[u].z, ga[u].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
              a += (double)__uint_as_float(gq[q] << 16) * (double)__uint_as_float(xw[q] << 16);
              a += (double)__uint_as_float(gq[q] & 0xFFFF0000u) * (double)__uint_as_float(xw[q] & 0xFFFF0000u);
            }
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1)
      a += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(a), o),
                            __shfl_xor_sync(0xffffffffu, __double2loint(a), o));
    if (lane == 0) s_part[warp] = a;
    rs_sync();
    if (tok && wq == 0 && lane == 0) {
      double tot = 0;
      for (int w2 = 0; w2 < W; w2++) tot += s_part[ts * W + w2];
      const float gate = sigmoid_f32((float)tot);
      RS_PUT(sgate, ts, gate);
      RS_PUT(tokidx, P + ts, ts);
      RS_PUT(pw, P + ts, gate);
    }
    rs_sync();  // s_part is reused by the router
  RS_STAMP(0);
  }
  if (logits) {
    // Router: the token's W warps share its exponentials, divisions and the selection, so
    // that a single token is spread over the whole block instead of one warp. Same arithmetic
    // and tie rule as router_one_token.
    const int NV = 16 / W;  // values per lane
    const float* lg = logits + (size_t)(tok ? ts : 0) * E;
    float v[16];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int e = (j * W + wq) * 32 + lane;
      v[j] = (j < NV && tok && e < E) ? lg[e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_bv[0][warp] = mx;
    rs_sync();
  RS_STAMP(1);
    for (int w2 = 0; w2 < W; w2++) mx = fmaxf(mx, s_bv[0][ts * W + w2]);
    const double dmx = (double)mx;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int e = (j * W + wq) * 32 + lane;
      if (j < NV && tok && e < E) {
        v[j] = (float)exp((double)v[j] - dmx);
        s_p[ts][e] = v[j];
      }
    }
    rs_sync();
  RS_STAMP(2);
    // Sum of the exponentials, as the reference takes it: in double, in index order. All terms
    // are floats in (0, 1]: when the smallest non-zero one is at least 2^(B - 30), B = bits of
    // the total's integer part, every partial sum of ANY order is a multiple of one grid that
    // a double holds exactly, so a tree sum gives the very same bits and the 512 dependent
    // additions are only needed otherwise.
    {
      double part = 0;
      float mn = 2.f;
#pragma unroll
      for (int j = 0; j < 16; j++)
        if (j < NV && tok && (j * W + wq) * 32 + lane < E) {
          part += (double)v[j];
          if (v[j] > 0.f) mn = fminf(mn, v[j]);
        }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        part += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(part), o),
                                 __shfl_xor_sync(0xffffffffu, __double2loint(part), o));
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      }
      if (lane == 0) {
        s_part[warp] = part;
        s_bv[1][warp] = mn;
      }
    }
    rs_sync();
  RS_STAMP(3);
    if (tok && wq == 0 && lane == 0) {
      double se = 0;
      float mn = 2.f;
      for (int w2 = 0; w2 < W; w2++) {
        se += s_part[ts * W + w2];
        mn = fminf(mn, s_bv[1][ts * W + w2]);
      }
      // last mantissa bit of the smallest term against the bits the total needs
      const int e_min = (int)((__float_as_uint(mn) >> 23) & 0xFF) - 127;
      const int bits_total = (int)((__double2hiint(se) >> 20) & 0x7FF) - 1023 + 2;  // generous by one bit
      const bool exact = mn >= 1.17549435e-38f && bits_total - (e_min - 23) <= 53;
      if (!exact) {
        se = 0;
        for (int i = 0; i < E; i++) se += (double)s_p[ts][i];  // index order, as the reference sums
      }
      s_se[ts] = se;
    }
    rs_sync();
  RS_STAMP(4);
    const double se = tok ? s_se[ts] : 1.0;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int e = (j * W + wq) * 32 + lane;
      v[j] = (j < NV && tok && e < E) ? (float)((double)v[j] / se) : -1.f;
    }
    int my_id = 0;
    float my_p = 0.f;
    double kept = 0;
    if (W == 16) {
      // One token, one probability per thread (expert = tid). The k-th largest of the 16 warp
      // maxima is a lower bound of the k-th largest probability (k <= 16), so every selected
      // expert is among the values >= that bound: usually a few dozen candidates, which are
      // then ranked against each other in (probability descending, id ascending) order.
      const float mine = v[0];
      float wm = mine;
#pragma unroll
      for (int o = 16; o; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
      if (lane == 0) s_bv[0][warp] = wm;
      if (tid == 0) s_wcnt[16] = 0;
      if (tid < k) {
        // non-finite logits make every probability NaN and no candidate is ever ranked: the
        // selection then stays at these in-range ids with NaN weights
        s_key[tid] = tid;
        s_w[tid] = __int_as_float(0x7fc00000);
      }
      rs_sync();
      if (warp == 0) {
        const float m = lane < 16 ? s_bv[0][lane] : -1.f;
        int rank = 0;
#pragma unroll
        for (int i = 0; i < 16; i++) {
          const float o = __shfl_sync(0xffffffffu, m, i);
          rank += (o > m) || (o == m && i < lane);
        }
        const unsigned hit = __ballot_sync(0xffffffffu, lane < 16 && rank == min(k, 16) - 1);
        const float bound = hit ? __shfl_sync(0xffffffffu, m, __ffs(hit) - 1) : __int_as_float(0x7fc00000);
        if (lane == 0) s_bv[1][0] = bound;
      }
      rs_sync();
      const bool cand = tid < E && mine >= s_bv[1][0];
      const unsigned cm = __ballot_sync(0xffffffffu, cand);
      int cbase = 0;
      if (lane == 0 && cm) cbase = atomicAdd(&s_wcnt[16], __popc(cm));
      cbase = __shfl_sync(0xffffffffu, cbase, 0);
      if (cand) {
        const int pos = cbase + __popc(cm & ((1u << lane) - 1u));
        s_p[1][pos] = mine;           // rows 1 and 2 of the scratch are free with one token
        ((int*)s_p[2])[pos] = tid;
      }
      rs_sync();
      const int C = s_wcnt[16];
      if (cand) {
        int rank = 0;
        for (int i = 0; i < C; i++) {
          const float o = s_p[1][i];
          const int oi = ((const int*)s_p[2])[i];
          rank += (o > mine) || (o == mine && oi < tid);
        }
        if (rank < k) {
          s_key[rank] = tid;
          s_w[rank] = mine;
        }
      }
      rs_sync();
      for (int r = 0; r < k; r++) kept += (double)s_w[r];  // in selection order
      if (lane < k) {
        my_id = s_key[lane];
        my_p = s_w[lane];
      }
      rs_sync();  // s_key / s_w are reused below
    } else {
      // k rounds of arg-max over the group's values: lanes, then the group's warps
      for (int r = 0; r < k; r++) {
        float bv = -1.f;
        int bi = min(wq * 32 + lane, E - 1);  // an id inside [0, E) even when nothing compares greater (NaN)
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (v[j] > bv) {  // ascending expert id within a lane: the first maximum is the lowest id
            bv = v[j];
            bi = (j * W + wq) * 32 + lane;
          }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
          }
        }
        if (W > 1) {
          if (lane == 0) {
            s_bv[r & 1][warp] = bv;
            s_bi[r & 1][warp] = bi;
          }
          rs_sync();
          // lane l < W takes the candidate of the group's warp l; W <= 8 lanes are merged
          bv = lane < W ? s_bv[r & 1][ts * W + lane] : -1.f;
          bi = lane < W ? s_bi[r & 1][ts * W + lane] : s_bi[r & 1][ts * W];
#pragma unroll
          for (int o = 4; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
              bv = ov;
              bi = oi;
            }
          }
        }
        bv = __shfl_sync(0xffffffffu, bv, 0);  // (with NaN probabilities the lanes may disagree: take lane 0's)
        bi = __shfl_sync(0xffffffffu, bi, 0);
        if (bv < 0.f) bv = __int_as_float(0x7fc00000);  // nothing was selectable: the weight is NaN
#pragma unroll
        for (int j = 0; j < 16; j++)
          if ((j * W + wq) * 32 + lane == bi) v[j] = -1.f;
        if (lane == r) {
          my_id = bi;
          my_p = bv;
        }
        kept += (double)bv;
      }
    }
    if (tok && wq == 0) {
      for (int i = lane; i < kIdStride; i += 32) {
        const bool valid = i < k && i < 32;
        RS_PUT(topids, (size_t)ts * kIdStride + i, valid ? my_id : 0);
        const float wv = valid ? (float)((double)my_p / kept) : 0.f;
        RS_PUT(topw, (size_t)ts * kIdStride + i, wv);
        if (valid) {  // the bucketing below takes the selection from shared memory, not back from global
          s_key[ts * k + i] = my_id;
          s_w[ts * k + i] = wv;
        }
      }
    }
  } else {
    for (int p = tid; p < P; p += blockDim.x) {
      // a caller-supplied id outside [0, E) must never index anything: the pair is dropped
      // (key kBadKey sorts behind every expert) and the status word records it
      const int id = ids_in[(size_t)(p / k) * stride_in + p % k];
      const bool bad = (unsigned)id >= (unsigned)E;
      if (bad && status && atomicCAS(status, 0, kStatusBadId) == 0) status[1] = id;
      s_key[p] = bad ? kBadKey : id;
      s_w[p] = w_in[(size_t)(p / k) * stride_in + p % k];
    }
  }
  rs_sync();
  RS_STAMP(5);
  // pair p -> row = number of pairs ordered before it by (expert, p)
  int n_bad = 0;
  if (tid < P) {
    const int key = s_key[tid], t = tid / k;
    int row = 0, rank = 0;
    for (int q = 0; q < P; q++) {
      const int kq = s_key[q];
      row += (kq < key) || (kq == key && q < tid);
      n_bad += kq == kBadKey;
    }
    // slot of the pair in the token's reduce order: ascending expert id; equal ids (a caller's
    // duplicate, or two dropped pairs) keep their slot order, so every slot is written
    for (int q = t * k; q < t * k + k; q++) rank += (s_key[q] < key) || (s_key[q] == key && q < tid);
    RS_PUT(tokidx, row, t);
    RS_PUT(pw, row, s_w[tid]);
    RS_PUT(pairids, (size_t)t * k + rank, key == kBadKey ? -1 : row);  // the combine skips negative rows
  }
  // expert e: offset, count, position among the non-empty experts
  int cnt = 0, lt = 0;
  if (tid < E)
    for (int q = 0; q < P; q++) {
      const int kq = s_key[q];
      cnt += kq == tid;
      lt += kq < tid;
    }
  const unsigned active = __ballot_sync(0xffffffffu, cnt > 0);
  if (lane == 0) s_wcnt[warp] = __popc(active);
  rs_sync();
  RS_STAMP(6);
  int before = __popc(active & ((1u << lane) - 1u)), n_active = 0;
  for (int w2 = 0; w2 < 16; w2++) {
    if (w2 < warp) before += s_wcnt[w2];
    n_active += s_wcnt[w2];
  }
  if (tid < E) RS_PUT(eoff, tid, lt);
  if (cnt > 0) {
    RS_PUT(runs, before, (Run{tid, lt, cnt}));
    RS_PUT(tiles, before, (Tile{tid, lt, cnt}));
  }
  if (tid == 0) {
    RS_PUT(eoff, E, P - n_bad);  // pairs actually placed (thread 0 counted the dropped ones above)
    RS_PUT(n_runs, 0, n_active);
    RS_PUT(n_runs, 1, 1);
    if (o1.runs) o1.runs[o1.shared_slot] = Run{0, P, T};
    if (o2.runs) o2.runs[o2.shared_slot] = Run{0, P, T};
    RS_PUT(n_tiles, 0, n_active);
    RS_PUT(n_tiles, 1, 1);
    RS_PUT(tiles_sh, 0, (Tile{0, P, T}));
  }
}
#undef RS_PUT
#undef RS_STAMP


}  // namespace b200moe
