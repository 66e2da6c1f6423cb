// moe_oracle.cpp -- TEST INFRASTRUCTURE ONLY. Not part of the product library.
//
// A CPU restatement of the routed-expert MoE FFN of gfx1151-engine, written to be
// the checker for the CUDA path: tests, the smoke check and the CPU-baseline leg of
// the benchmark call it; the product library never does.
//
// Parity status: PINNED. Every function here is compared, bit for bit, against the
// reference's own code compiled from its sources (oracle/ref_adapter.cpp ->
// oracle/_ref/libref.so) and against golden vectors produced by that build
// (tests/golden/).
//
// What each function follows in the reference (paths relative to the reference
// project root):
//   orc_q4cp_rows        src/hgn.h:219-261   (q4cp_parse / q4cp_row)
//   orc_gguf_rows        src/gguf.h:328-336, 352-359, 360-374, 375-406, 408-441 (scale_min_k4, Q8_0,
//                        Q5_1, IQ4_NL, IQ4_XS, Q4_K, Q5_K)
//   orc_router_topk      src/ref.cpp:574-588 (softmax in double, partial_sort on probs)
//   orc_route            src/gpu/parts/40_model.inc:4171-4193 (host bucketing) and
//                        src/gpu/parts/10_ple_io.inc:790-811 (pairids rank rule)
//   orc_tiles            src/gpu/parts/10_ple_io.inc:813-825 (k_moe_tiles)
//   orc_moe_forward      src/ref.cpp:563-637 (Model::moe), with the row dequantiser
//                        swapped for gguf rows when the layer is GGUF
//                        (precedent: tools/moe_gguf_gemv_test.cu:145-195)
//
// Build: g++ -O3 -fopenmp -ffp-contract=off -shared -fPIC (no -march=native): the
// reference dequantisers are "multiply then add", never fused.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float half_bits_to_float(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u, ex = (h >> 10) & 31u, man = h & 1023u;
  float v;
  if (ex == 0) v = (float)man * 0x1p-24f;
  else if (ex == 31) v = man ? NAN : INFINITY;
  else v = ldexpf((float)(1024u + man), (int)ex - 25);
  return sign ? -v : v;
}

inline float bf16_bits_to_float(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// View of one q4cp tensor blob: [16 x f32 codebook][rows*cols/2 code bytes][rows x stride scale bytes]
struct Q4View {
  const float* book;
  const uint8_t* codes;
  const uint8_t* scales;
  uint64_t rows, cols, stride;
};

inline Q4View q4_view(const uint8_t* blob, uint64_t rows, uint64_t cols) {
  Q4View v;
  v.rows = rows;
  v.cols = cols;
  v.stride = ((cols / 32 * 2) + 15) & ~15ull;
  v.book = (const float*)blob;
  v.codes = blob + 64;
  v.scales = blob + 64 + rows * cols / 2;
  return v;
}

inline void q4_row(const Q4View& v, uint64_t row, float* out) {
  const uint8_t* c = v.codes + row * (v.cols / 2);
  const uint16_t* s = (const uint16_t*)(v.scales + row * v.stride);
  for (uint64_t g = 0; g < v.cols / 32; g++) {
    float sc = half_bits_to_float(s[g]);
    for (uint64_t j = 0; j < 32; j += 2) {
      uint8_t b = c[(g * 32 + j) / 2];
      out[g * 32 + j] = v.book[b & 15] * sc;
      out[g * 32 + j + 1] = v.book[b >> 4] * sc;
    }
  }
}

enum { GG_Q5_1 = 7, GG_Q8_0 = 8, GG_Q4_K = 12, GG_Q5_K = 13, GG_IQ4_NL = 20, GG_IQ4_XS = 23 };

inline bool gg_known(uint32_t t) { return t == GG_Q5_1 || t == GG_Q8_0 || t == GG_Q4_K || t == GG_Q5_K || t == GG_IQ4_NL || t == GG_IQ4_XS; }

inline uint64_t gg_row_bytes(uint32_t type, uint64_t k) {
  if (type == GG_Q4_K) return k / 256 * 144;
  if (type == GG_Q5_K) return k / 256 * 176;
  if (type == GG_Q5_1) return k / 32 * 24;
  if (type == GG_Q8_0) return k / 32 * 34;
  if (type == GG_IQ4_NL) return k / 32 * 18;
  if (type == GG_IQ4_XS) return k / 256 * 136;
  return 0;
}

inline void k4_scale_min(int j, const uint8_t* p, uint8_t& sc, uint8_t& mn) {
  if (j < 4) {
    sc = p[j] & 63;
    mn = p[j + 4] & 63;
  } else {
    sc = (uint8_t)((p[j + 4] & 15) | ((p[j - 4] >> 6) << 4));
    mn = (uint8_t)((p[j + 4] >> 4) | ((p[j] >> 6) << 4));
  }
}

inline void gg_row(uint32_t type, const uint8_t* src, float* y, uint64_t k) {
  if (type == GG_Q8_0) {  // 34 bytes per 32: fp16 d, 32 int8 codes, y = d * q (src/gguf.h:352-359)
    for (uint64_t b = 0; b < k / 32; b++, src += 34) {
      uint16_t dh;
      memcpy(&dh, src, 2);
      const float d = half_bits_to_float(dh);
      for (int j = 0; j < 32; j++) y[b * 32 + j] = d * (float)(int8_t)src[2 + j];
    }
    return;
  }
  if (type == GG_Q5_1) {
    for (uint64_t b = 0; b < k / 32; b++, src += 24) {
      uint16_t dh, mh;
      uint32_t hi;
      memcpy(&dh, src, 2);
      memcpy(&mh, src + 2, 2);
      memcpy(&hi, src + 4, 4);
      const float d = half_bits_to_float(dh), m = half_bits_to_float(mh);
      const uint8_t* q = src + 8;
      for (int j = 0; j < 16; j++) {
        int a = (q[j] & 15) | (int)(((hi >> j) & 1u) << 4);
        int c = (q[j] >> 4) | (int)(((hi >> (j + 16)) & 1u) << 4);
        y[b * 32 + j] = a * d + m;
        y[b * 32 + j + 16] = c * d + m;
      }
    }
    return;
  }
  if (type == GG_IQ4_NL || type == GG_IQ4_XS) {
    // the non-linear 4-bit grid shared by both formats (src/gguf.h:376-377, 389-390)
    static const int8_t grid[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
    if (type == GG_IQ4_NL) {  // 18 bytes per 32: fp16 d, 16 code bytes (src/gguf.h:375-387)
      for (uint64_t b = 0; b < k / 32; b++, src += 18) {
        uint16_t dh;
        memcpy(&dh, src, 2);
        const float d = half_bits_to_float(dh);
        for (int j = 0; j < 16; j++) {
          y[b * 32 + j] = d * grid[src[2 + j] & 15];
          y[b * 32 + j + 16] = d * grid[src[2 + j] >> 4];
        }
      }
      return;
    }
    // IQ4_XS, 136 bytes per 256: fp16 d, u16 high scale bits, 4 bytes of low scale nibbles,
    // 128 code bytes; sub-block scale = d * (6-bit value - 32) (src/gguf.h:388-406)
    for (uint64_t b = 0; b < k / 256; b++, src += 136) {
      uint16_t dh, sh;
      memcpy(&dh, src, 2);
      memcpy(&sh, src + 2, 2);
      const float d = half_bits_to_float(dh);
      for (int ib = 0; ib < 8; ib++) {
        const int ls = ((src[4 + ib / 2] >> (4 * (ib % 2))) & 15) | (((sh >> (2 * ib)) & 3) << 4);
        const float dl = d * (float)(ls - 32);
        const uint8_t* q = src + 8 + 16 * ib;
        for (int j = 0; j < 16; j++) {
          y[b * 256 + ib * 32 + j] = dl * grid[q[j] & 15];
          y[b * 256 + ib * 32 + j + 16] = dl * grid[q[j] >> 4];
        }
      }
    }
    return;
  }
  // Q4_K (144 bytes per 256) and Q5_K (176 bytes: 32 bytes of fifth bits between the packed
  // scales and the nibbles; bit 2*sub / 2*sub+1 of qh[l] belongs to element l of the low / high
  // group of the sub-th 64 elements), src/gguf.h:408-441
  const bool five = type == GG_Q5_K;
  for (uint64_t b = 0; b < k / 256; b++, src += five ? 176 : 144) {
    uint16_t dh, mh;
    memcpy(&dh, src, 2);
    memcpy(&mh, src + 2, 2);
    const float d = half_bits_to_float(dh), dmin = half_bits_to_float(mh);
    const uint8_t* packed = src + 4;
    const uint8_t* hb = src + 16;
    const uint8_t* q = src + (five ? 48 : 16);
    float* o = y + b * 256;
    for (int sub = 0; sub < 4; sub++) {
      uint8_t s0, m0, s1, m1;
      k4_scale_min(2 * sub, packed, s0, m0);
      k4_scale_min(2 * sub + 1, packed, s1, m1);
      const float a0 = d * s0, b0 = dmin * m0, a1 = d * s1, b1 = dmin * m1;
      for (int l = 0; l < 32; l++) {
        const int lo = (q[32 * sub + l] & 15) + (five && ((hb[l] >> (2 * sub)) & 1) ? 16 : 0);
        o[64 * sub + l] = a0 * lo - b0;
      }
      for (int l = 0; l < 32; l++) {
        const int hi = (q[32 * sub + l] >> 4) + (five && ((hb[l] >> (2 * sub + 1)) & 1) ? 16 : 0);
        o[64 * sub + 32 + l] = a1 * hi - b1;
      }
    }
  }
}

inline float silu_f(float v) { return v / (1.f + expf(-v)); }
inline float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

inline double dot_d(const float* w, const float* x, int n) {
  double a = 0;
  for (int i = 0; i < n; i++) a += (double)w[i] * x[i];
  return a;
}

}  // namespace

extern "C" {

// Layer description handed over from Python (ctypes mirrors this struct field by field).
struct OrcLayer {
  int32_t experts, topk, d, mid;
  int32_t format;              // 0 = hgn q4cp, 1 = GGUF (block types in gg_type_gu / gg_type_dn)
  int32_t gg_type_gu, gg_type_dn;
  int32_t has_shared;
  const uint8_t* gate_up;      // q4cp: fused [E*2*mid, d] blob; GGUF: unused
  const uint8_t* down;         // q4cp: [E*d, mid] blob; GGUF: raw blocks [E][d rows of mid]
  const uint8_t* gg_gate;      // GGUF raw blocks [E][mid rows of d]
  const uint8_t* gg_up;
  const uint16_t* router_w;    // bf16 [E][d] or null when logits are supplied
  const uint8_t* sh_gate;      // shared expert q4cp blobs [mid,d], [mid,d], [d,mid]
  const uint8_t* sh_up;
  const uint8_t* sh_down;
  const uint16_t* sh_gate_w;   // bf16 [d], scalar sigmoid gate of the shared expert
};

void orc_q4cp_rows(const uint8_t* blob, uint64_t rows, uint64_t cols, uint64_t row0,
                   uint64_t n, float* out) {
  Q4View v = q4_view(blob, rows, cols);
  for (uint64_t r = 0; r < n; r++) q4_row(v, row0 + r, out + r * cols);
}

int orc_gguf_rows(uint32_t type, const uint8_t* src, uint64_t k, uint64_t n, float* out) {
  if (!gg_known(type) || gg_row_bytes(type, k) == 0) return -1;
  uint64_t rb = gg_row_bytes(type, k);
  for (uint64_t r = 0; r < n; r++) gg_row(type, src + r * rb, out + r * k, k);
  return 0;
}

// Router: probabilities exactly as the reference's CPU path forms them, then the k
// largest by std::partial_sort with the same comparator (so ties fall the same way
// under the same libstdc++). ids/w rows have `stride` entries, first k valid.
void orc_router_topk(const float* logits, int T, int E, int k, int stride, int32_t* ids,
                     float* w, float* probs_or_null) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++) {
    const float* lg = logits + (size_t)t * E;
    std::vector<float> p(E);
    double top = -1e300;
    for (int i = 0; i < E; i++) top = std::max(top, (double)lg[i]);
    double total = 0;
    for (int i = 0; i < E; i++) {
      p[i] = (float)exp((double)lg[i] - top);
      total += p[i];
    }
    for (int i = 0; i < E; i++) p[i] = (float)(p[i] / total);
    std::vector<int> order(E);
    for (int i = 0; i < E; i++) order[i] = i;
    std::partial_sort(order.begin(), order.begin() + k, order.end(),
                      [&](int a, int b) { return p[a] > p[b]; });
    double kept = 0;
    for (int i = 0; i < k; i++) kept += p[order[i]];
    for (int i = 0; i < stride; i++) {
      ids[(size_t)t * stride + i] = i < k ? order[i] : 0;
      w[(size_t)t * stride + i] = i < k ? (float)(p[order[i]] / kept) : 0.f;
    }
    if (probs_or_null) memcpy(probs_or_null + (size_t)t * E, p.data(), sizeof(float) * E);
  }
}

// Number of tokens whose selection depends on an exact tie of float probabilities at
// ranks <= k+1 (such tokens have no unique expected answer across sort implementations).
int orc_count_topk_ties(const float* probs, int T, int E, int k) {
  int bad = 0;
  for (int t = 0; t < T; t++) {
    std::vector<float> p(probs + (size_t)t * E, probs + (size_t)(t + 1) * E);
    std::sort(p.begin(), p.end(), [](float a, float b) { return a > b; });
    bool tie = false;
    for (int i = 0; i < k && i + 1 < E; i++) tie |= p[i] == p[i + 1];
    bad += tie;
  }
  return bad;
}

// Bucketing of (token, slot) pairs by expert: stable in (t, s) order.
void orc_route(const int32_t* ids, const float* w, int T, int k, int E, int stride,
               int32_t* tokidx, float* pw, int32_t* eoff, int32_t* pairids) {
  std::vector<int> cursor(E + 1, 0);
  for (int i = 0; i <= E; i++) eoff[i] = 0;
  for (int t = 0; t < T; t++)
    for (int s = 0; s < k; s++) eoff[ids[(size_t)t * stride + s] + 1]++;
  for (int e = 0; e < E; e++) eoff[e + 1] += eoff[e];
  for (int e = 0; e < E; e++) cursor[e] = eoff[e];
  for (int t = 0; t < T; t++)
    for (int s = 0; s < k; s++) {
      int e = ids[(size_t)t * stride + s];
      int row = cursor[e]++;
      tokidx[row] = t;
      pw[row] = w[(size_t)t * stride + s];
    }
  // reduce order of a token = its experts in ascending id (rows are already sorted by expert)
  std::vector<int> seen(T, 0);
  for (int row = 0; row < T * k; row++) {
    int t = tokidx[row];
    pairids[(size_t)t * k + seen[t]++] = row;
  }
}

// Tile list: each expert's row range cut into pieces of at most `cap` rows.
int orc_tiles(const int32_t* eoff, int E, int cap, int32_t* tiles /* [n][3] */) {
  int n = 0;
  for (int e = 0; e < E; e++) {
    int first = eoff[e], cnt = eoff[e + 1] - first;
    for (int j = 0; j * cap < cnt; j++) {
      tiles[3 * n + 0] = e;
      tiles[3 * n + 1] = first + j * cap;
      tiles[3 * n + 2] = std::min(cap, cnt - j * cap);
      n++;
    }
  }
  return n;
}

// Whole layer, token by token. x is fp32 [T][d] (callers pass bf16-valued floats).
// Router logits from hidden states: y = W x with W bf16 [E][d], products and sum in double in
// index order, rounded to float once (matvec, src/ref.cpp:68-77; called at src/ref.cpp:565-567).
extern "C" void orc_router_logits(const uint16_t* router_w, const float* x, int T, int E, int d, float* logits) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++) {
    const float* xt = x + (size_t)t * d;
    for (int e = 0; e < E; e++) {
      const uint16_t* wr = router_w + (size_t)e * d;
      double a = 0;
      for (int c = 0; c < d; c++) a += (double)bf16_bits_to_float(wr[c]) * xt[c];
      logits[(size_t)t * E + e] = (float)a;
    }
  }
}

// logits: fp32 [T][E] or null (then router_w must be set and logits = float(sum_double)).
// ids_out / w_out (optional) receive the selection, rows of 16 entries.
int orc_moe_forward(const OrcLayer* L, const float* x, const float* logits, int T, float* y,
                    int32_t* ids_out, float* w_out, int threads) {
  const int E = L->experts, k = L->topk, d = L->d, mid = L->mid;
  if (!logits && !L->router_w) return -1;
  if (L->format == 1 && (!gg_known((uint32_t)L->gg_type_gu) || !gg_known((uint32_t)L->gg_type_dn))) return -2;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
  int fail = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int t = 0; t < T; t++) {
    const float* xt = x + (size_t)t * d;
    std::vector<float> lg(E);
    if (logits) {
      memcpy(lg.data(), logits + (size_t)t * E, sizeof(float) * E);
    } else {
      for (int e = 0; e < E; e++) {
        const uint16_t* wr = L->router_w + (size_t)e * d;
        double a = 0;
        for (int c = 0; c < d; c++) a += (double)bf16_bits_to_float(wr[c]) * xt[c];
        lg[e] = (float)a;
      }
    }
    int32_t sel[16];
    float selw[16];
    {
      // single-token router (same arithmetic as orc_router_topk)
      std::vector<float> p(E);
      double top = -1e300;
      for (int i = 0; i < E; i++) top = std::max(top, (double)lg[i]);
      double total = 0;
      for (int i = 0; i < E; i++) {
        p[i] = (float)exp((double)lg[i] - top);
        total += p[i];
      }
      for (int i = 0; i < E; i++) p[i] = (float)(p[i] / total);
      std::vector<int> order(E);
      for (int i = 0; i < E; i++) order[i] = i;
      std::partial_sort(order.begin(), order.begin() + k, order.end(),
                        [&](int a, int b) { return p[a] > p[b]; });
      double kept = 0;
      for (int i = 0; i < k; i++) kept += p[order[i]];
      for (int i = 0; i < 16; i++) {
        sel[i] = i < k ? order[i] : 0;
        selw[i] = i < k ? (float)(p[order[i]] / kept) : 0.f;
      }
    }
    if (ids_out) memcpy(ids_out + (size_t)t * 16, sel, sizeof sel);
    if (w_out) memcpy(w_out + (size_t)t * 16, selw, sizeof selw);

    std::vector<float> acc(d, 0.f), gu(2 * (size_t)mid), hid(mid), row(std::max(d, mid));
    Q4View vgu{}, vdn{};
    if (L->format == 0) {
      vgu = q4_view(L->gate_up, (uint64_t)E * 2 * mid, d);
      vdn = q4_view(L->down, (uint64_t)E * d, mid);
    }
    const uint64_t rb_gu = gg_row_bytes(L->gg_type_gu, d), rb_dn = gg_row_bytes(L->gg_type_dn, mid);
    for (int i = 0; i < k; i++) {
      const int e = sel[i];
      const float wt = selw[i];
      for (int r = 0; r < 2 * mid; r++) {
        if (L->format == 0) {
          q4_row(vgu, (uint64_t)e * 2 * mid + r, row.data());
        } else {
          const uint8_t* base = r < mid ? L->gg_gate : L->gg_up;
          gg_row(L->gg_type_gu, base + ((uint64_t)e * mid + (r % mid)) * rb_gu, row.data(), d);
        }
        gu[r] = (float)dot_d(row.data(), xt, d);
      }
      for (int r = 0; r < mid; r++) hid[r] = silu_f(gu[r]) * gu[mid + r];
      for (int r = 0; r < d; r++) {
        if (L->format == 0) q4_row(vdn, (uint64_t)e * d + r, row.data());
        else gg_row(L->gg_type_dn, L->down + ((uint64_t)e * d + r) * rb_dn, row.data(), mid);
        acc[r] += wt * (float)dot_d(row.data(), hid.data(), mid);
      }
    }
    float* yt = y + (size_t)t * d;
    if (L->has_shared) {
      double sg = 0;
      for (int c = 0; c < d; c++) sg += (double)bf16_bits_to_float(L->sh_gate_w[c]) * xt[c];
      Q4View g = q4_view(L->sh_gate, mid, d), u = q4_view(L->sh_up, mid, d),
             dn = q4_view(L->sh_down, d, mid);
      std::vector<float> g1(mid), u1(mid);
      for (int r = 0; r < mid; r++) {
        q4_row(g, r, row.data());
        g1[r] = (float)dot_d(row.data(), xt, d);
      }
      for (int r = 0; r < mid; r++) {
        q4_row(u, r, row.data());
        u1[r] = (float)dot_d(row.data(), xt, d);
      }
      for (int r = 0; r < mid; r++) g1[r] = silu_f(g1[r]) * u1[r];
      const float gate = sigmoid_f((float)sg);
      for (int r = 0; r < d; r++) {
        q4_row(dn, r, row.data());
        float ey = (float)dot_d(row.data(), g1.data(), mid);
        yt[r] = acc[r] + gate * ey;
      }
    } else {
      for (int r = 0; r < d; r++) yt[r] = acc[r];
    }
  }
  return fail;
}

int orc_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
