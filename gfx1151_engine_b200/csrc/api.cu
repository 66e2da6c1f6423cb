// api.cu -- the C ABI declared in include/b200moe.h: handle, workspaces, weight loading
// (one-time repack into HBM) and the forward sequences. Host-side mirror of the
// reference's GpuModel::moe / moe_b / moe_q4w_run / moe_gguf dispatch
// (src/gpu/parts/40_model.inc:1664-1861, 4018-4157): same thresholds (T <= 16 takes the
// GEMV path), same order of stages, status codes instead of exit().
#include "../../include/b200moe.h"
#include "kernels.h"
#include "tc.h"

#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

using namespace b200moe;

namespace {

constexpr int kProfRing = 64, kProfEvents = 6;

struct LayerWeights {
  Image gu, dn, sh_gu, sh_dn;
  uint16_t* sh_gate_w = nullptr;
  uint16_t* router_w = nullptr;  // bf16 [E][d], null until b200moe_load_router
  bool loaded = false, shared_loaded = false;
  bool borrowed = false;  // images belong to another handle
  // hgn v2 i4r: the images hold rotated weights (gu is a plain, unpaired image of 2*mid rows);
  // rot = one allocation [d + 2*mid + mid + d] f32: gu_suh, gu_svh, dn_suh, dn_svh
  bool i4r = false;
  float* rot = nullptr;
};

}  // namespace

struct b200moe_ctx {
  b200moe_config cfg{};
  int decode_max = 16;
  int tile_cap = kTcTileN;
  std::vector<LayerWeights> layers;
  std::vector<void*> allocs;  // everything cudaMalloc'ed for workspaces
  RouteBuffers rb{};
  void* hid = nullptr;      // [rows][mid] fp32 (GEMV path) or fp16 (tensor-core path)
  void* pairs = nullptr;    // [rows][d]   fp32 or fp16
  __half* x_sorted = nullptr;
  __half* x_rot = nullptr;  // [max_tokens][d] fp16: rotated activations of hgn v2 i4r layers (allocated by the first such load)
  int dec_rows = 0;
  RouterPlan* rplan = nullptr;     // router logits from hidden states
  const float* hc_w4 = nullptr;    // set for the duration of b200moe_forward_hc: the combine
  void* hc_state = nullptr;        // adds into the residual state instead of storing `out`
  float* router_logits = nullptr;  // [max_tokens][E]
  int32_t* flag_list = nullptr;    // (token * E + expert) pairs whose logits are recomputed exactly
  int32_t* flag_count = nullptr;
  void *x_stage = nullptr, *out_stage = nullptr;
  float* logits_stage = nullptr;
  int32_t* status_dev = nullptr;
  int32_t* status_host = nullptr;  // pinned
  unsigned long long* grid_bar = nullptr;  // arrival counter of the fused decode kernel's grid-wide barrier
  unsigned long long* dec_trace = nullptr;  // debug timeline of the fused decode kernel (environment B200MOE_DECODE_TRACE=<file>)
  // forward_host: copy streams and per-chunk events of the pipelined host path
  static constexpr int kHostChunks = 4;
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[kHostChunks] = {}, ev_done[kHostChunks] = {}, ev_out[kHostChunks] = {}, ev_start = nullptr;
  TcPlan* tc = nullptr;
  // expert parallelism
  int32_t *place_dev = nullptr, *source_of_placed_dev = nullptr;
  bool place_borrowed = false;
  __half *ep_x_send = nullptr, *ep_x_recv = nullptr, *ep_pairs_recv = nullptr, *ep_pairs_back = nullptr;
  __half* ep_hid = nullptr;
  Tile* ep_tiles = nullptr;
  int32_t* ep_counts = nullptr;  // [0] tiles, [1] received rows
  long long ep_cap_rows = 0;
  int ep_max_tiles = 0;
  TcPlan* tc_ep = nullptr;
  TcPlan* tc_own = nullptr;        // own-rows pass in place: activations from x_send, results into pairs_back
  // part 4 (the other ranks' rows with the tails of their segments merged by expert): the place of
  // every merged row in the source-major layout, the table of the tails
  int32_t *ep_rowmap = nullptr, *ep_segs = nullptr;
  int sms = 148;
  int64_t launches = 0;
  // stage timer: ring of event sets, one set (7 events) per forward call
  bool prof = false;
  std::vector<cudaEvent_t> prof_ev;
  int prof_head = 0, prof_pending = 0;
  int max_rows = 0, max_tiles = 0, max_tiles_sh = 0;
  std::string err;
};

namespace {

int fail(b200moe_handle h, int code, const std::string& msg) {
  if (h) h->err = msg;
  return code;
}

#define CU_TRY(h, expr)                                                                  \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return fail(h, B200MOE_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

template <typename T>
cudaError_t dev_alloc(b200moe_handle h, T** p, size_t count) {
  void* q = nullptr;
  cudaError_t e = cudaMalloc(&q, count * sizeof(T) + 256);
  if (e == cudaSuccess) {
    h->allocs.push_back(q);
    *p = (T*)q;
  }
  return e;
}

size_t q4cp_bytes(size_t rows, size_t cols) {
  return 64 + rows * cols / 2 + rows * (((cols / 32 * 2) + 15) & ~(size_t)15);
}

bool is_device_ptr(const void* p) {
  cudaPointerAttributes a{};
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Device-visible copy of a source blob: the pointer itself when it already is device
// memory, else a temporary upload (freed by the caller through `tmp`).
cudaError_t stage(const void* src, size_t bytes, const uint8_t** dev, std::vector<void*>& tmp) {
  if (is_device_ptr(src)) {
    *dev = (const uint8_t*)src;
    return cudaSuccess;
  }
  void* q = nullptr;
  cudaError_t e = cudaMalloc(&q, bytes + 16);
  if (e != cudaSuccess) return e;
  tmp.push_back(q);
  e = cudaMemcpy(q, src, bytes, cudaMemcpyHostToDevice);
  *dev = (const uint8_t*)q;
  return e;
}

void free_all(std::vector<void*>& v) {
  for (void* p : v) cudaFree(p);
  v.clear();
}

cudaError_t alloc_image(Image& img, int fmt, int n_experts, int rows, int K, int paired) {
  img.fmt = fmt;
  img.n_experts = n_experts;
  img.paired = paired;
  img.n_mtiles = paired ? rows / 64 : rows / 128;  // paired: rows = mid (gate rows)
  img.n_kblocks = K / kTileK;
  cudaError_t e = cudaMalloc((void**)&img.data, img.expert_stride() * n_experts + 256);
  if (e != cudaSuccess) return e;
  return cudaMalloc((void**)&img.book, 32 * sizeof(float));
}

void free_image(Image& img) {
  if (img.data) cudaFree(img.data);
  if (img.book) cudaFree(img.book);
  img = Image{};
}

SrcTensor q4cp_src(const uint8_t* blob, long long rows_total, long long cols,
                   long long rows_per_expert, long long row_off) {
  SrcTensor s;
  s.codes = blob + 64;
  s.scales = blob + 64 + rows_total * cols / 2;
  s.rows_per_expert = rows_per_expert;
  s.row_off = row_off;
  s.scale_stride = ((cols / 32 * 2) + 15) & ~15ll;
  return s;
}

// Turns the device status word (copied to status_host) into a return code and clears it on the
// device. {1|2|3|5|6, site}: a bounded device-side wait gave up; {4, id}: a caller-supplied expert
// id outside [0, experts) was dropped by the bucketing; {7, token}: the router's near-tie list overflowed.
int report_status(b200moe_handle h, cudaStream_t st) {
  const int code = h->status_host[0], detail = h->status_host[1];
  if (code == 0) return B200MOE_OK;
  cudaError_t e = cudaMemsetAsync(h->status_dev, 0, 16, st);
  // a grid-wide barrier that gave up leaves its arrival count behind: start it afresh
  if (e == cudaSuccess && code == 5) e = cudaMemsetAsync(h->grid_bar, 0, 16, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(h, B200MOE_ERR_CUDA, std::string("clearing the status word: ") + cudaGetErrorString(e));
  char buf[256];
  if (code == 4) {
    snprintf(buf, sizeof buf, "expert id %d outside [0, %d) in the caller's top-k ids: the pair was dropped", detail,
             h->cfg.experts);
    return fail(h, B200MOE_ERR_BAD_ARG, buf);
  }
  if (code == 7) {
    snprintf(buf, sizeof buf, "router logits: more near-ties than the exact-recomputation list holds (first dropped at token %d); "
             "the top-k order of this call is not guaranteed to be the reference's", detail);
    return fail(h, B200MOE_ERR_TOO_LARGE, buf);
  }
  snprintf(buf, sizeof buf, "device-side wait timed out (code %d, wait site %d)", code, detail);
  return fail(h, B200MOE_ERR_DEVICE_TIMEOUT, buf);
}

int check_layer(b200moe_handle h, int layer) {
  if (!h) return B200MOE_ERR_BAD_ARG;
  if (layer < 0 || layer >= (int)h->layers.size())
    return fail(h, B200MOE_ERR_BAD_ARG, "layer index out of range");
  return B200MOE_OK;
}

int local_experts(const b200moe_config& c) { return c.experts / c.ep_size; }
int first_expert(const b200moe_config& c) { return c.ep_rank * (c.experts / c.ep_size); }

}  // namespace

extern "C" {

const char* b200moe_version(void) { return "b200moe 0.1 sm_100a"; }

const char* b200moe_status_string(int s) {
  switch (s) {
    case B200MOE_OK: return "ok";
    case B200MOE_ERR_BAD_ARG: return "bad argument";
    case B200MOE_ERR_UNSUPPORTED: return "unsupported shape or format";
    case B200MOE_ERR_CUDA: return "CUDA error";
    case B200MOE_ERR_NOT_LOADED: return "layer weights not loaded";
    case B200MOE_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case B200MOE_ERR_NCCL: return "NCCL error";
    case B200MOE_ERR_ALLOC: return "out of memory";
    case B200MOE_ERR_TOO_LARGE: return "request exceeds the fixed scratch capacity of the allocation-free entry point";
    default: return "unknown status";
  }
}

const char* b200moe_last_error(b200moe_handle h) { return h ? h->err.c_str() : "null handle"; }

int64_t b200moe_launch_count(b200moe_handle h) { return h ? h->launches : 0; }

int b200moe_create(const b200moe_config* cfg, b200moe_handle* out) {
  if (!cfg || !out) return B200MOE_ERR_BAD_ARG;
  *out = nullptr;
  b200moe_config c = *cfg;
  if (c.ep_size <= 0) c.ep_size = 1;
  if (c.n_layers <= 0) c.n_layers = 1;
  if (c.experts < 1 || c.topk < 1 || c.d_model < 1 || c.d_mid < 1 || c.max_tokens < 1 ||
      c.ep_rank < 0 || c.ep_rank >= c.ep_size)
    return B200MOE_ERR_BAD_ARG;
  if (c.experts > kMaxExperts || c.topk > kMaxTopK || c.topk > c.experts ||
      c.d_model % 128 != 0 || c.d_mid % 64 != 0 || c.experts % c.ep_size != 0)
    return B200MOE_ERR_UNSUPPORTED;
  if (cudaSetDevice(c.device) != cudaSuccess) {
    cudaGetLastError();
    return B200MOE_ERR_CUDA;
  }
  b200moe_handle h = new (std::nothrow) b200moe_ctx();
  if (!h) return B200MOE_ERR_ALLOC;
  h->cfg = c;
  h->decode_max = c.decode_max_tokens > 0 ? c.decode_max_tokens : 16;
  h->layers.resize(c.n_layers);
  const int Tm = c.max_tokens, k = c.topk, E = c.experts, d = c.d_model, mid = c.d_mid;
  const size_t pairs = (size_t)Tm * k;
  const size_t rows = pairs + (c.has_shared ? Tm : 0);
  h->max_rows = (int)rows;
  h->max_tiles = (int)(pairs / h->tile_cap) + E + 1;
  h->max_tiles_sh = Tm / h->tile_cap + 1;
  const size_t dec_rows = (size_t)std::min(Tm, h->decode_max) * (k + (c.has_shared ? 1 : 0));
  const bool simt_all = c.gemm_impl == B200MOE_GEMM_SIMT;
  const size_t hid_bytes = std::max(rows * mid * (simt_all ? 4 : 2), dec_rows * mid * 4);
  const size_t pair_bytes = std::max(rows * d * (simt_all ? 4 : 2), dec_rows * d * 4);
  cudaError_t e = cudaSuccess;
  auto A = [&](auto** p, size_t n) {
    if (e == cudaSuccess) e = dev_alloc(h, p, n);
  };
  A(&h->rb.topids, (size_t)Tm * kIdStride);
  A(&h->rb.topw, (size_t)Tm * kIdStride);
  A(&h->rb.tokidx, rows);
  A(&h->rb.pw, rows);
  A(&h->rb.eoff, (size_t)E + 1);
  A(&h->rb.pairids, pairs);
  A(&h->rb.blockcnt, ((pairs + 511) / 512) * E);
  A(&h->rb.runs, (size_t)kMaxExperts + 1);
  A(&h->rb.n_runs, 2);
  A(&h->rb.tiles, (size_t)h->max_tiles);
  A(&h->rb.tiles_sh, (size_t)h->max_tiles_sh);
  A(&h->rb.n_tiles, 2);
  A(&h->rb.sgate, (size_t)Tm);
  A((uint8_t**)&h->hid, hid_bytes);
  A((uint8_t**)&h->pairs, pair_bytes);
  if (!simt_all) A(&h->x_sorted, rows * d);
  h->dec_rows = (int)dec_rows;
  A(&h->router_logits, (size_t)Tm * E);
  A(&h->flag_list, (size_t)Tm * 16);
  A(&h->flag_count, 1);
  A((uint8_t**)&h->x_stage, (size_t)Tm * d * 2);
  A((uint8_t**)&h->out_stage, (size_t)Tm * d * 2);
  A(&h->logits_stage, (size_t)Tm * E);
  A(&h->status_dev, 4);
  h->rb.status = h->status_dev;
  if (e == cudaSuccess) e = cudaMemset(h->status_dev, 0, 16);
  A(&h->grid_bar, 2);
  if (e == cudaSuccess) e = cudaMemset(h->grid_bar, 0, 16);
  if (getenv("B200MOE_DECODE_TRACE")) {
    A(&h->dec_trace, (size_t)1024 * 8);
    if (e == cudaSuccess) e = cudaMemset(h->dec_trace, 0, 1024 * 8 * sizeof(unsigned long long));
  }
  if (e == cudaSuccess) e = cudaMallocHost((void**)&h->status_host, 16);
  if (e == cudaSuccess && !simt_all)
    e = tc_create(&h->tc, h->x_sorted, (__half*)h->hid, (long long)rows, d, mid);
  if (e == cudaSuccess && !simt_all) e = router_plan_create(&h->rplan);
  if (e != cudaSuccess) {
    std::string msg = std::string("b200moe_create: ") + cudaGetErrorString(e);
    cudaGetLastError();
    b200moe_destroy(h);
    fprintf(stderr, "%s\n", msg.c_str());
    return e == cudaErrorMemoryAllocation ? B200MOE_ERR_ALLOC : B200MOE_ERR_CUDA;
  }
  *out = h;
  return B200MOE_OK;
}

int b200moe_destroy(b200moe_handle h) {
  if (!h) return B200MOE_ERR_BAD_ARG;
  cudaSetDevice(h->cfg.device);
  cudaDeviceSynchronize();
  b200moe_ep_shutdown(h);  // the library-side expert-parallel host, if one was set up on this handle
  if (h->dec_trace) {
    // debug aid: per-block phase time stamps (ns) of the last fused decode launch, raw uint64 [1024][8]
    std::vector<unsigned long long> host((size_t)1024 * 8);
    if (cudaMemcpy(host.data(), h->dec_trace, host.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess)
      if (FILE* f = fopen(getenv("B200MOE_DECODE_TRACE") ? getenv("B200MOE_DECODE_TRACE") : "decode_trace.bin", "wb")) {
        fwrite(host.data(), 8, host.size(), f);
        fclose(f);
      }
  }
  for (auto& L : h->layers) {
    if (L.borrowed) continue;
    free_image(L.gu);
    free_image(L.dn);
    free_image(L.sh_gu);
    free_image(L.sh_dn);
    if (L.sh_gate_w) cudaFree(L.sh_gate_w);
    if (L.router_w) cudaFree(L.router_w);
    if (L.rot) cudaFree(L.rot);
  }
  free_all(h->allocs);
  if (h->place_dev && !h->place_borrowed) cudaFree(h->place_dev);
  if (h->source_of_placed_dev && !h->place_borrowed) cudaFree(h->source_of_placed_dev);
  if (h->ep_hid) cudaFree(h->ep_hid);
  if (h->ep_tiles) cudaFree(h->ep_tiles);
  if (h->ep_counts) cudaFree(h->ep_counts);
  if (h->tc_ep) tc_destroy(h->tc_ep);
  if (h->tc_own) tc_destroy(h->tc_own);
  if (h->ep_rowmap) cudaFree(h->ep_rowmap);
  if (h->ep_segs) cudaFree(h->ep_segs);
  for (auto& e : h->prof_ev) cudaEventDestroy(e);
  if (h->s_in) cudaStreamDestroy(h->s_in);
  if (h->s_out) cudaStreamDestroy(h->s_out);
  for (int i = 0; i < b200moe_ctx::kHostChunks; i++) {
    if (h->ev_in[i]) cudaEventDestroy(h->ev_in[i]);
    if (h->ev_done[i]) cudaEventDestroy(h->ev_done[i]);
    if (h->ev_out[i]) cudaEventDestroy(h->ev_out[i]);
  }
  if (h->ev_start) cudaEventDestroy(h->ev_start);
  if (h->status_host) cudaFreeHost(h->status_host);
  if (h->tc) tc_destroy(h->tc);
  if (h->rplan) router_plan_destroy(h->rplan);
  cudaGetLastError();
  delete h;
  return B200MOE_OK;
}

int b200moe_load_q4cp(b200moe_handle h, int layer, const void* gate_up_src, size_t gate_up_bytes,
                      const void* down_src, size_t down_bytes) {
  if (int s = check_layer(h, layer)) return s;
  if (!gate_up_src || !down_src) return fail(h, B200MOE_ERR_BAD_ARG, "null weight pointer");
  const b200moe_config& c = h->cfg;
  const size_t E = c.experts, d = c.d_model, mid = c.d_mid;
  if (gate_up_bytes != q4cp_bytes(E * 2 * mid, d) || down_bytes != q4cp_bytes(E * d, mid))
    return fail(h, B200MOE_ERR_BAD_ARG, "q4cp blob size does not match [E*2*mid,d] / [E*d,mid]");
  if (((uintptr_t)gate_up_src | (uintptr_t)down_src) & 15)
    return fail(h, B200MOE_ERR_BAD_ARG, "q4cp blobs must be 16-byte aligned");
  CU_TRY(h, cudaSetDevice(c.device));
  LayerWeights& L = h->layers[layer];
  free_image(L.gu);
  free_image(L.dn);
  L.loaded = false;
  L.i4r = false;
  std::vector<void*> tmp;
  const uint8_t *gu = nullptr, *dn = nullptr;
  const int nl = local_experts(c), e0 = first_expert(c);
  cudaError_t e = stage(gate_up_src, gate_up_bytes, &gu, tmp);
  if (e == cudaSuccess) e = alloc_image(L.gu, kQ4CP, nl, (int)mid, (int)d, 1);
  if (e == cudaSuccess) {
    SrcTensor g = q4cp_src(gu, E * 2 * mid, d, 2 * mid, 0), u = q4cp_src(gu, E * 2 * mid, d, 2 * mid, mid);
    e = launch_repack(L.gu, g, u, (int)d, e0, 0, h->source_of_placed_dev);
    h->launches++;
  }
  if (e == cudaSuccess) e = cudaMemcpy(L.gu.book, gu, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(L.gu.book + 16, gu, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  if (e == cudaSuccess) e = stage(down_src, down_bytes, &dn, tmp);
  if (e == cudaSuccess) e = alloc_image(L.dn, kQ4CP, nl, (int)d, (int)mid, 0);
  if (e == cudaSuccess) {
    SrcTensor a = q4cp_src(dn, E * d, mid, d, 0);
    e = launch_repack(L.dn, a, a, (int)mid, e0, 0, h->source_of_placed_dev);
    h->launches++;
  }
  if (e == cudaSuccess) e = cudaMemcpy(L.dn.book, dn, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(L.dn.book + 16, dn, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(h, e == cudaErrorMemoryAllocation ? B200MOE_ERR_ALLOC : B200MOE_ERR_CUDA,
                std::string("load_q4cp: ") + cudaGetErrorString(e));
  }
  L.loaded = true;
  return B200MOE_OK;
}

int b200moe_load_i4r(b200moe_handle h, int layer, const void* gate_up_src, size_t gate_up_bytes,
                     const void* down_src, size_t down_bytes, const void* gu_suh_f16, const void* gu_svh_f16,
                     const void* dn_suh_f16, const void* dn_svh_f16) {
  if (int s = check_layer(h, layer)) return s;
  if (!gate_up_src || !down_src || !gu_suh_f16 || !gu_svh_f16 || !dn_suh_f16 || !dn_svh_f16)
    return fail(h, B200MOE_ERR_BAD_ARG, "load_i4r: null pointer");
  const b200moe_config& c = h->cfg;
  const size_t E = c.experts, d = c.d_model, mid = c.d_mid;
  if (d % 128 || mid % 128 || 2 * mid > d)
    return fail(h, B200MOE_ERR_UNSUPPORTED, "load_i4r: needs d % 128 == 0, mid % 128 == 0 and 2*mid <= d");
  if (c.has_shared || c.ep_size > 1 || c.gemm_impl == B200MOE_GEMM_SIMT || !h->tc)
    return fail(h, B200MOE_ERR_UNSUPPORTED,
                "load_i4r: not with a shared expert, expert parallelism or the fp32 kernels");
  auto i4r_bytes = [](size_t rows, size_t cols) { return rows * cols / 2 + rows * (cols / 128) * 2; };
  if (gate_up_bytes != i4r_bytes(E * 2 * mid, d) || down_bytes != i4r_bytes(E * d, mid))
    return fail(h, B200MOE_ERR_BAD_ARG, "i4r blob size does not match [E*2*mid,d] / [E*d,mid]");
  if (((uintptr_t)gate_up_src | (uintptr_t)down_src) & 15)
    return fail(h, B200MOE_ERR_BAD_ARG, "i4r blobs must be 16-byte aligned");
  CU_TRY(h, cudaSetDevice(c.device));
  LayerWeights& L = h->layers[layer];
  free_image(L.gu);
  free_image(L.dn);
  if (L.rot) cudaFree(L.rot);
  L.rot = nullptr;
  L.loaded = false;
  L.i4r = false;
  std::vector<void*> tmp;
  cudaError_t e = cudaSuccess;
  if (!h->x_rot) e = dev_alloc(h, &h->x_rot, (size_t)c.max_tokens * d);
  static const float kBook[32] = {-8, -7, -6, -5, -4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 6, 7,
                                  -8, -7, -6, -5, -4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 6, 7};
  const uint8_t* src = nullptr;
  // gate_up: a plain image of 2*mid rows per expert (the rotation mixes 128 consecutive output
  // rows, so gate row r and up row r cannot share a tile the way the q4cp image pairs them)
  if (e == cudaSuccess) e = stage(gate_up_src, gate_up_bytes, &src, tmp);
  if (e == cudaSuccess) e = alloc_image(L.gu, kQ4CP, (int)E, (int)(2 * mid), (int)d, 0);
  if (e == cudaSuccess) {
    SrcTensor a;
    a.codes = src;
    a.scales = src + E * 2 * mid * d / 2;
    a.rows_per_expert = (long long)(2 * mid);
    a.scale_stride = (long long)(d / 128 * 2);
    a.scale_group = 128;
    e = launch_repack(L.gu, a, a, (int)d, 0, 0, nullptr);
    h->launches++;
  }
  if (e == cudaSuccess) e = cudaMemcpy(L.gu.book, kBook, sizeof kBook, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  if (e == cudaSuccess) e = stage(down_src, down_bytes, &src, tmp);
  if (e == cudaSuccess) e = alloc_image(L.dn, kQ4CP, (int)E, (int)d, (int)mid, 0);
  if (e == cudaSuccess) {
    SrcTensor a;
    a.codes = src;
    a.scales = src + E * d * mid / 2;
    a.rows_per_expert = (long long)d;
    a.scale_stride = (long long)(mid / 128 * 2);
    a.scale_group = 128;
    e = launch_repack(L.dn, a, a, (int)mid, 0, 0, nullptr);
    h->launches++;
  }
  if (e == cudaSuccess) e = cudaMemcpy(L.dn.book, kBook, sizeof kBook, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  // the four sign-scale planes, fp16 -> f32 as the reference uploads them (30_host_util.inc:824-838)
  if (e == cudaSuccess) e = cudaMalloc((void**)&L.rot, (2 * d + 3 * mid) * sizeof(float));
  const void* planes[4] = {gu_suh_f16, gu_svh_f16, dn_suh_f16, dn_svh_f16};
  const size_t lens[4] = {d, 2 * mid, mid, d};
  size_t off = 0;
  for (int i = 0; i < 4 && e == cudaSuccess; i++) {
    e = stage(planes[i], lens[i] * 2, &src, tmp);
    if (e == cudaSuccess) e = launch_f16_to_f32(src, L.rot + off, (int)lens[i], 0);
    h->launches++;
    off += lens[i];
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(h, e == cudaErrorMemoryAllocation ? B200MOE_ERR_ALLOC : B200MOE_ERR_CUDA,
                std::string("load_i4r: ") + cudaGetErrorString(e));
  }
  L.i4r = true;
  L.loaded = true;
  return B200MOE_OK;
}

// Image format, bytes per row of K elements and K granule of a GGUF block type; fmt < 0: not read.
static void gguf_type_info(int type, bool down, size_t K, int* fmt, size_t* row_bytes, size_t* granule, int* act_shift) {
  *fmt = -1;
  *row_bytes = 0;
  *granule = 256;
  *act_shift = 0;
  if (type == B200MOE_GGML_Q8_0) {  // two nibble planes in the Q5_1 image form (common.cuh)
    *fmt = kQ51, *row_bytes = K / 32 * 34, *granule = 32, *act_shift = 1;
    return;
  }
  if (type == B200MOE_GGML_Q4_K && !down) *fmt = kQ4K, *row_bytes = K / 256 * 144;
  else if (type == B200MOE_GGML_Q5_K && !down) *fmt = kQ51, *row_bytes = K / 256 * 176;
  else if (type == B200MOE_GGML_Q5_1 && down) *fmt = kQ51, *row_bytes = K / 32 * 24, *granule = 32;
  else if (type == B200MOE_GGML_IQ4_NL) *fmt = kQ4CP, *row_bytes = K / 32 * 18, *granule = 32;
  else if (type == B200MOE_GGML_IQ4_XS) *fmt = kQ4CP, *row_bytes = K / 256 * 136;
}

// Code book of an image made from GGUF blocks: IQ4 = the non-linear grid / 256 (the image's
// scales carry the factor 256), Q4_K / Q5_1 = the code itself (scale and offset applied after).
static void gguf_book(int type, float* book32) {
  static const int8_t grid[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
  const bool iq = type == B200MOE_GGML_IQ4_NL || type == B200MOE_GGML_IQ4_XS;
  for (int i = 0; i < 32; i++) book32[i] = iq ? (float)grid[i & 15] * (1.f / 256.f) : (float)(i & 15);
}

int b200moe_load_gguf(b200moe_handle h, int layer, const void* gate_src, const void* up_src,
                      const void* down_src, int type_gu, int type_dn) {
  if (int s = check_layer(h, layer)) return s;
  if (!gate_src || !up_src || !down_src) return fail(h, B200MOE_ERR_BAD_ARG, "null weight pointer");
  const b200moe_config& c = h->cfg;
  const size_t E = c.experts, d = c.d_model, mid = c.d_mid;
  int fmt_gu, fmt_dn, ash_gu, ash_dn;
  size_t rb_gu, rb_dn, gr_gu, gr_dn;
  gguf_type_info(type_gu, false, d, &fmt_gu, &rb_gu, &gr_gu, &ash_gu);
  gguf_type_info(type_dn, true, mid, &fmt_dn, &rb_dn, &gr_dn, &ash_dn);
  if (fmt_gu < 0 || fmt_dn < 0)
    return fail(h, B200MOE_ERR_UNSUPPORTED,
                "GGUF experts: gate/up must be Q4_K, Q5_K, Q8_0, IQ4_NL or IQ4_XS and down Q5_1, Q8_0, IQ4_NL or IQ4_XS");
  if (d % gr_gu != 0 || mid % gr_dn != 0)
    return fail(h, B200MOE_ERR_UNSUPPORTED, "GGUF experts: row length is not a whole number of blocks");
  CU_TRY(h, cudaSetDevice(c.device));
  LayerWeights& L = h->layers[layer];
  free_image(L.gu);
  free_image(L.dn);
  L.loaded = false;
  L.i4r = false;
  const size_t gu_bytes = E * mid * rb_gu, dn_bytes = E * d * rb_dn;
  std::vector<void*> tmp;
  const uint8_t *g = nullptr, *u = nullptr, *dn = nullptr;
  const int nl = local_experts(c), e0 = first_expert(c);
  cudaError_t e = stage(gate_src, gu_bytes, &g, tmp);
  if (e == cudaSuccess) e = stage(up_src, gu_bytes, &u, tmp);
  if (e == cudaSuccess) e = alloc_image(L.gu, fmt_gu, nl, (int)mid, (int)d << ash_gu, 1);
  L.gu.act_shift = ash_gu;
  if (e == cudaSuccess) {
    SrcTensor sg, su;
    sg.codes = g;
    sg.rows_per_expert = mid;
    su.codes = u;
    su.rows_per_expert = mid;
    e = launch_repack(L.gu, sg, su, (int)d, e0, 0, h->source_of_placed_dev, type_gu);
    h->launches++;
  }
  float book[32];
  gguf_book(type_gu, book);
  if (e == cudaSuccess) e = cudaMemcpy(L.gu.book, book, sizeof book, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  if (e == cudaSuccess) e = stage(down_src, dn_bytes, &dn, tmp);
  if (e == cudaSuccess) e = alloc_image(L.dn, fmt_dn, nl, (int)d, (int)mid << ash_dn, 0);
  L.dn.act_shift = ash_dn;
  if (e == cudaSuccess) {
    SrcTensor a;
    a.codes = dn;
    a.rows_per_expert = d;
    e = launch_repack(L.dn, a, a, (int)mid, e0, 0, h->source_of_placed_dev, type_dn);
    h->launches++;
  }
  gguf_book(type_dn, book);
  if (e == cudaSuccess) e = cudaMemcpy(L.dn.book, book, sizeof book, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(h, e == cudaErrorMemoryAllocation ? B200MOE_ERR_ALLOC : B200MOE_ERR_CUDA,
                std::string("load_gguf: ") + cudaGetErrorString(e));
  }
  L.loaded = true;
  return B200MOE_OK;
}

int b200moe_load_shared_q4cp(b200moe_handle h, int layer, const void* gate_src, const void* up_src,
                             const void* down_src, const void* gate_w_bf16_src) {
  if (int s = check_layer(h, layer)) return s;
  if (!h->cfg.has_shared) return fail(h, B200MOE_ERR_BAD_ARG, "handle was created without a shared expert");
  if (!gate_src || !up_src || !down_src || !gate_w_bf16_src)
    return fail(h, B200MOE_ERR_BAD_ARG, "null weight pointer");
  if (((uintptr_t)gate_src | (uintptr_t)up_src | (uintptr_t)down_src) & 15)
    return fail(h, B200MOE_ERR_BAD_ARG, "q4cp blobs must be 16-byte aligned");
  const b200moe_config& c = h->cfg;
  const size_t d = c.d_model, mid = c.d_mid;
  CU_TRY(h, cudaSetDevice(c.device));
  LayerWeights& L = h->layers[layer];
  free_image(L.sh_gu);
  free_image(L.sh_dn);
  if (L.sh_gate_w) cudaFree(L.sh_gate_w), L.sh_gate_w = nullptr;
  L.shared_loaded = false;
  std::vector<void*> tmp;
  const uint8_t *g = nullptr, *u = nullptr, *dn = nullptr;
  cudaError_t e = stage(gate_src, q4cp_bytes(mid, d), &g, tmp);
  if (e == cudaSuccess) e = stage(up_src, q4cp_bytes(mid, d), &u, tmp);
  if (e == cudaSuccess) e = stage(down_src, q4cp_bytes(d, mid), &dn, tmp);
  if (e == cudaSuccess) e = alloc_image(L.sh_gu, kQ4CP, 1, (int)mid, (int)d, 1);
  if (e == cudaSuccess) e = alloc_image(L.sh_dn, kQ4CP, 1, (int)d, (int)mid, 0);
  if (e == cudaSuccess) {
    e = launch_repack(L.sh_gu, q4cp_src(g, mid, d, mid, 0), q4cp_src(u, mid, d, mid, 0), (int)d, 0, 0);
    h->launches++;
  }
  if (e == cudaSuccess) {
    SrcTensor a = q4cp_src(dn, d, mid, d, 0);
    e = launch_repack(L.sh_dn, a, a, (int)mid, 0, 0);
    h->launches++;
  }
  L.sh_gu.dual_book = 1;
  if (e == cudaSuccess) e = cudaMemcpy(L.sh_gu.book, g, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(L.sh_gu.book + 16, u, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(L.sh_dn.book, dn, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(L.sh_dn.book + 16, dn, 64, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMalloc((void**)&L.sh_gate_w, d * 2);
  if (e == cudaSuccess) e = cudaMemcpy(L.sh_gate_w, gate_w_bf16_src, d * 2, cudaMemcpyDefault);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  free_all(tmp);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(h, e == cudaErrorMemoryAllocation ? B200MOE_ERR_ALLOC : B200MOE_ERR_CUDA,
                std::string("load_shared_q4cp: ") + cudaGetErrorString(e));
  }
  L.shared_loaded = true;
  return B200MOE_OK;
}

int b200moe_router_topk(b200moe_handle h, const float* logits_dev, int T, int32_t* topids_dev,
                        float* topw_dev, int stride, void* stream) {
  if (!h) return B200MOE_ERR_BAD_ARG;
  if (!logits_dev || !topids_dev || !topw_dev || T < 0 || stride < h->cfg.topk)
    return fail(h, B200MOE_ERR_BAD_ARG, "router_topk: bad argument");
  if (T == 0) return B200MOE_OK;
  CU_TRY(h, launch_router_topk(logits_dev, T, h->cfg.experts, h->cfg.topk, topids_dev, topw_dev,
                               stride, (cudaStream_t)stream));
  h->launches++;
  return B200MOE_OK;
}

int b200moe_route(b200moe_handle h, const int32_t* topids_dev, const float* topw_dev, int stride,
                  int T, void* stream) {
  if (!h) return B200MOE_ERR_BAD_ARG;
  if (!topids_dev || !topw_dev || T < 0 || T > h->cfg.max_tokens || stride < h->cfg.topk)
    return fail(h, B200MOE_ERR_BAD_ARG, "route: bad argument");
  if (T == 0) return B200MOE_OK;
  int n = 0;
  CU_TRY(h, launch_route(h->rb, topids_dev, topw_dev, stride, T, h->cfg.topk, h->cfg.experts,
                         h->tile_cap, (cudaStream_t)stream, &n));
  h->launches += n;
  return B200MOE_OK;
}

// logits != nullptr: the router has not run yet (the fused small-T routing kernel runs it).
static int forward_impl(b200moe_handle h, int layer, const void* x, int T, const int32_t* ids,
                        const float* w, int stride, void* out, cudaStream_t st,
                        bool router_timed = false, const float* logits = nullptr) {
  const b200moe_config& c = h->cfg;
  LayerWeights& L = h->layers[layer];
  const int k = c.topk, E = c.experts, d = c.d_model, mid = c.d_mid;
  const bool shared = c.has_shared != 0;
  if (!L.loaded || (shared && !L.shared_loaded))
    return fail(h, B200MOE_ERR_NOT_LOADED, "forward: layer weights not loaded");
  int n = 0;
  cudaEvent_t* ev = nullptr;
  if (h->prof) {
    ev = &h->prof_ev[(size_t)h->prof_head * kProfEvents];
    // ev[0] was recorded by the caller of forward_impl (before the router) when it ran one
    if (!router_timed) CU_TRY(h, cudaEventRecord(ev[0], st));
  }
  // decode / verify of q4cp layers as ONE kernel (routing, both GEMVs, combine, every expert read
  // once for all its rows): opt-in with decode_impl = B200MOE_DECODE_FUSED in the configuration or B200MOE_FUSED_DECODE=1. Measured slower than the
  // separate kernels (whose launches overlap through programmatic dependent launch), so they
  // stay the default.
  static const bool fused_env = getenv("B200MOE_FUSED_DECODE") != nullptr && atoi(getenv("B200MOE_FUSED_DECODE")) != 0;
  const bool fused = fused_env || c.decode_impl == B200MOE_DECODE_FUSED;
  if (L.i4r && (c.gemm_impl == B200MOE_GEMM_SIMT || !h->tc || !h->x_rot))
    return fail(h, B200MOE_ERR_UNSUPPORTED, "forward: hgn v2 i4r layers run on the tensor-core path only");
  if (fused && !L.i4r && c.gemm_impl == B200MOE_GEMM_AUTO && T <= h->decode_max && T <= decode_max_tokens() &&
      ((uintptr_t)x & 15) == 0 && (size_t)T * (k + (shared ? 1 : 0)) <= (size_t)h->dec_rows &&
      decode_supported(L.gu, L.dn, shared ? &L.sh_gu : nullptr, shared ? &L.sh_dn : nullptr, T, k, E, d, mid)) {
    CU_TRY(h, launch_decode(L.gu, L.dn, shared ? &L.sh_gu : nullptr, shared ? &L.sh_dn : nullptr, logits, ids, w, stride, x,
                            shared ? L.sh_gate_w : nullptr, T, E, k, d, mid, (__half*)h->hid, out, h->hc_w4, h->hc_state,
                            h->rb, h->grid_bar, h->status_dev, st, h->dec_trace));
    if (ev) {
      for (int i = 1; i <= 5; i++) CU_TRY(h, cudaEventRecord(ev[i], st));  // one kernel: no stage boundaries
      h->prof_head = (h->prof_head + 1) % kProfRing;
      if (h->prof_pending < kProfRing) h->prof_pending++;
    }
    h->launches += 1;
    return B200MOE_OK;
  }
  static const bool slow_router = getenv("B200MOE_EXACT_ROUTER") != nullptr;  // A/B: the general routing body for every call
  if (logits && !slow_router && T <= decode_max_tokens() && T * k <= 128 && d % 8 == 0 && (!shared || ((uintptr_t)x & 15) == 0)) {
    // decode / verify: the compact router (ids from the logits' order, general body only on a near-tie)
    CU_TRY(h, launch_route_fast(h->rb, logits, T, k, E, x, shared ? L.sh_gate_w : nullptr, d, st));
    n++;
  } else if (T * k <= route_small_max_pairs() && T <= 16) {
    CU_TRY(h, launch_route_small(h->rb, logits, ids, w, stride, T, k, E, x, shared ? L.sh_gate_w : nullptr,
                                 d, st));
    n++;
  } else {
    if (logits) {
      CU_TRY(h, launch_router_topk(logits, T, E, k, h->rb.topids, h->rb.topw, kIdStride, st));
      n++;
      ids = h->rb.topids;
      w = h->rb.topw;
      stride = kIdStride;
    }
    CU_TRY(h, launch_route(h->rb, ids, w, stride, T, k, E, h->tile_cap, st, &n));
    if (shared) {
      CU_TRY(h, launch_shared_gate(x, L.sh_gate_w, T, d, k, h->rb, st));
      n++;
    }
  }
  if (ev) CU_TRY(h, cudaEventRecord(ev[1], st));
  const int pairs = T * k;
  const bool simt = !L.i4r && (c.gemm_impl == B200MOE_GEMM_SIMT ||
                                (c.gemm_impl == B200MOE_GEMM_AUTO && T <= h->decode_max));
  if (simt && c.gemm_impl != B200MOE_GEMM_SIMT && T > h->decode_max)
    return fail(h, B200MOE_ERR_BAD_ARG, "forward: T exceeds the GEMV path's workspace");
  // (the shared expert's images are q4cp: it can ride along only with q4cp routed experts)
  const bool gemv = simt && c.gemm_impl == B200MOE_GEMM_AUTO &&
                    (!shared || (L.gu.fmt == kQ4CP && L.dn.fmt == kQ4CP)) &&
                    pairs + (shared ? T : 0) <= h->dec_rows && std::min(E, pairs) + 1 <= gemv_max_runs() &&
                    (d << L.gu.act_shift) <= gemv_max_k() && (mid << L.dn.act_shift) <= gemv_max_mid() && d % 32 == 0 &&
                    mid % 32 == 0;
  if (gemv) {
    // decode / verify: persistent dequant GEMV, routed and shared expert in one launch each
    if (ev) CU_TRY(h, cudaEventRecord(ev[2], st));
    CU_TRY(h, launch_up_gemv(L.gu, shared ? &L.sh_gu : nullptr, x, d, mid, h->rb.tokidx, h->rb.runs,
                             h->rb.n_runs, (__half*)h->hid, st));
    if (ev) CU_TRY(h, cudaEventRecord(ev[3], st));
    CU_TRY(h, launch_down_gemv(L.dn, shared ? &L.sh_dn : nullptr, (const __half*)h->hid, d, mid,
                               h->rb.runs, h->rb.n_runs, (float*)h->pairs, st));
    if (ev) CU_TRY(h, cudaEventRecord(ev[4], st));
    CU_TRY(h, launch_combine_f32((const float*)h->pairs, h->rb.pw, h->rb.pairids, T, k, d,
                                 shared ? pairs : -1, out, st, h->hc_w4, h->hc_state));
    n += 3;
  } else if (simt) {
    const int max_runs = std::min(E, pairs);
    if (ev) CU_TRY(h, cudaEventRecord(ev[2], st));
    CU_TRY(h, launch_up_simt(L.gu, x, d, mid, h->rb.tokidx, h->rb.runs, h->rb.n_runs, max_runs,
                             (float*)h->hid, st));
    n++;
    if (shared) {
      CU_TRY(h, launch_up_simt(L.sh_gu, x, d, mid, h->rb.tokidx, h->rb.runs + kMaxExperts,
                               h->rb.n_runs + 1, 1, (float*)h->hid, st));
      n++;
    }
    if (ev) CU_TRY(h, cudaEventRecord(ev[3], st));
    CU_TRY(h, launch_down_simt(L.dn, (const float*)h->hid, d, mid, h->rb.runs, h->rb.n_runs,
                               max_runs, (float*)h->pairs, st));
    n++;
    if (shared) {
      CU_TRY(h, launch_down_simt(L.sh_dn, (const float*)h->hid, d, mid, h->rb.runs + kMaxExperts,
                                 h->rb.n_runs + 1, 1, (float*)h->pairs, st));
      n++;
    }
    if (ev) CU_TRY(h, cudaEventRecord(ev[4], st));
    CU_TRY(h, launch_combine_f32((const float*)h->pairs, h->rb.pw, h->rb.pairids, T, k, d,
                                 shared ? pairs : -1, out, st, h->hc_w4, h->hc_state));
    n++;
  } else {
    if (!h->tc) return fail(h, B200MOE_ERR_UNSUPPORTED, "tensor-core path not available on this handle");
    const int rows = pairs + (shared ? T : 0);
    if (L.i4r) {
      // hgn v2 i4r (rotate.cu): rotate the tokens once, gather the rotated rows, plain GEMM into
      // the pair buffer (2*mid <= d columns of it), then the Hadamard / SwiGLU / Hadamard step
      CU_TRY(h, launch_rot_in(x, L.rot, T, d, h->x_rot, st));
      CU_TRY(h, launch_gather_f16(h->x_rot, h->rb.tokidx, rows, d, h->x_sorted, st, true));
      n += 2;
      if (ev) CU_TRY(h, cudaEventRecord(ev[2], st));
      CU_TRY(h, launch_raw_tc(h->tc, L.gu, h->rb.tiles, h->rb.n_tiles, h->max_tiles, (__half*)h->pairs, h->status_dev, st));
      CU_TRY(h, launch_i4r_mid((const __half*)h->pairs, L.rot + d, L.rot + d + 2 * mid, rows, mid, (__half*)h->hid, st));
      n += 2;
      if (ev) CU_TRY(h, cudaEventRecord(ev[3], st));
      CU_TRY(h, launch_down_tc(h->tc, L.dn, h->rb.tiles, h->rb.n_tiles, h->max_tiles, (__half*)h->pairs, h->status_dev, st));
      if (ev) CU_TRY(h, cudaEventRecord(ev[4], st));
      CU_TRY(h, launch_combine_f16_rot((const __half*)h->pairs, h->rb.pw, h->rb.pairids, T, k, d, L.rot + d + 3 * mid, out, st,
                                       h->hc_w4, h->hc_state));
      n += 2;
      if (ev) {
        CU_TRY(h, cudaEventRecord(ev[5], st));
        h->prof_head = (h->prof_head + 1) % kProfRing;
        if (h->prof_pending < kProfRing) h->prof_pending++;
      }
      h->launches += n;
      return B200MOE_OK;
    }
    CU_TRY(h, launch_gather_f16(x, h->rb.tokidx, rows, d, h->x_sorted, st));
    n++;
    if (ev) CU_TRY(h, cudaEventRecord(ev[2], st));
    CU_TRY(h, launch_up_tc(h->tc, L.gu, h->rb.tiles, h->rb.n_tiles, h->max_tiles, (__half*)h->hid,
                           h->status_dev, st));
    n++;
    if (shared) {
      CU_TRY(h, launch_up_tc(h->tc, L.sh_gu, h->rb.tiles_sh, h->rb.n_tiles + 1, h->max_tiles_sh,
                             (__half*)h->hid, h->status_dev, st));
      n++;
    }
    if (ev) CU_TRY(h, cudaEventRecord(ev[3], st));
    CU_TRY(h, launch_down_tc(h->tc, L.dn, h->rb.tiles, h->rb.n_tiles, h->max_tiles,
                             (__half*)h->pairs, h->status_dev, st));
    n++;
    if (shared) {
      CU_TRY(h, launch_down_tc(h->tc, L.sh_dn, h->rb.tiles_sh, h->rb.n_tiles + 1, h->max_tiles_sh,
                               (__half*)h->pairs, h->status_dev, st));
      n++;
    }
    if (ev) CU_TRY(h, cudaEventRecord(ev[4], st));
    CU_TRY(h, launch_combine_f16((const __half*)h->pairs, h->rb.pw, h->rb.pairids, T, k, d,
                                 shared ? pairs : -1, out, st, h->hc_w4, h->hc_state));
    n++;
  }
  if (ev) {
    CU_TRY(h, cudaEventRecord(ev[5], st));
    h->prof_head = (h->prof_head + 1) % kProfRing;
    if (h->prof_pending < kProfRing) h->prof_pending++;
  }
  h->launches += n;
  return B200MOE_OK;
}

int b200moe_forward(b200moe_handle h, int layer, const void* x_bf16_dev, int T,
                    const float* logits_dev, void* out_bf16_dev, void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!x_bf16_dev || !logits_dev || !out_bf16_dev || T < 0 || T > h->cfg.max_tokens)
    return fail(h, B200MOE_ERR_BAD_ARG, "forward: bad argument (null pointer or T out of range)");
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (h->prof) CU_TRY(h, cudaEventRecord(h->prof_ev[(size_t)h->prof_head * kProfEvents], st));
  return forward_impl(h, layer, x_bf16_dev, T, h->rb.topids, h->rb.topw, kIdStride, out_bf16_dev, st,
                      h->prof, logits_dev);
}

int b200moe_forward_hc(b200moe_handle h, int layer, const void* x_bf16_dev, int T, const float* logits_dev,
                       const float* inject_w4_dev, void* state_bf16_dev, void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!x_bf16_dev || !logits_dev || !inject_w4_dev || !state_bf16_dev || T < 0 || T > h->cfg.max_tokens)
    return fail(h, B200MOE_ERR_BAD_ARG, "forward_hc: bad argument (null pointer or T out of range)");
  if (h->cfg.d_model % 8 != 0 || ((uintptr_t)state_bf16_dev & 15))
    return fail(h, B200MOE_ERR_BAD_ARG, "forward_hc: the state needs d_model % 8 == 0 and 16-byte alignment");
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (h->prof) CU_TRY(h, cudaEventRecord(h->prof_ev[(size_t)h->prof_head * kProfEvents], st));
  h->hc_w4 = inject_w4_dev;
  h->hc_state = state_bf16_dev;
  const int rc = forward_impl(h, layer, x_bf16_dev, T, h->rb.topids, h->rb.topw, kIdStride, nullptr, st, h->prof,
                              logits_dev);
  h->hc_w4 = nullptr;
  h->hc_state = nullptr;
  return rc;
}

int b200moe_get_config(b200moe_handle h, b200moe_config* out) {
  if (!h || !out) return B200MOE_ERR_BAD_ARG;
  *out = h->cfg;
  return B200MOE_OK;
}

int b200moe_load_router(b200moe_handle h, int layer, const void* gate_weight_bf16) {
  if (int s = check_layer(h, layer)) return s;
  if (!gate_weight_bf16) return fail(h, B200MOE_ERR_BAD_ARG, "load_router: null pointer");
  if (h->cfg.experts > 512 || h->cfg.d_model % 64 != 0)
    return fail(h, B200MOE_ERR_UNSUPPORTED, "load_router: needs experts <= 512 and d_model % 64 == 0");
  LayerWeights& L = h->layers[layer];
  if (L.borrowed) return fail(h, B200MOE_ERR_BAD_ARG, "load_router: this handle borrows its weights");
  const size_t bytes = (size_t)h->cfg.experts * h->cfg.d_model * 2;
  if (!L.router_w) CU_TRY(h, cudaMalloc((void**)&L.router_w, bytes));
  CU_TRY(h, cudaMemcpy(L.router_w, gate_weight_bf16, bytes, cudaMemcpyDefault));
  return B200MOE_OK;
}

int b200moe_router_logits(b200moe_handle h, int layer, const void* x_bf16_dev, int T, float* logits_dev,
                          void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!x_bf16_dev || !logits_dev || T < 0 || T > h->cfg.max_tokens)
    return fail(h, B200MOE_ERR_BAD_ARG, "router_logits: bad argument");
  LayerWeights& L = h->layers[layer];
  if (!L.router_w) return fail(h, B200MOE_ERR_NOT_LOADED, "router_logits: router weight not loaded");
  if (T == 0) return B200MOE_OK;
  const int E = h->cfg.experts, d = h->cfg.d_model;
  cudaStream_t st = (cudaStream_t)stream;
  const int cap = h->cfg.max_tokens * 16;
  if (T <= 16 || !h->rplan) {
    // few tokens: double sums (1e-9 from the reference), then the reference's arithmetic for
    // the experts that decide the top-k where two of them are within a few float ulps
    CU_TRY(h, launch_router_dots(x_bf16_dev, L.router_w, T, E, d, logits_dev, st));
    CU_TRY(h, launch_router_flag(logits_dev, T, E, h->cfg.topk, 5e-7f, h->flag_list, h->flag_count, cap, st, h->status_dev));
  } else {
    CU_TRY(h, launch_router_gemm(h->rplan, x_bf16_dev, L.router_w, T, E, d, logits_dev, h->status_dev, st));
    CU_TRY(h, launch_router_flag(logits_dev, T, E, h->cfg.topk, 1e-4f, h->flag_list, h->flag_count, cap, st, h->status_dev));
  }
  CU_TRY(h, launch_router_pairs(x_bf16_dev, L.router_w, h->flag_list, h->flag_count, cap, E, d, logits_dev, st));
  h->launches += 3;
  return B200MOE_OK;
}

int b200moe_forward_hidden(b200moe_handle h, int layer, const void* x_bf16_dev, int T, void* out_bf16_dev,
                           void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!x_bf16_dev || !out_bf16_dev || T < 0 || T > h->cfg.max_tokens)
    return fail(h, B200MOE_ERR_BAD_ARG, "forward_hidden: bad argument (null pointer or T out of range)");
  if (T == 0) return B200MOE_OK;
  if (int s = b200moe_router_logits(h, layer, x_bf16_dev, T, h->router_logits, stream)) return s;
  return b200moe_forward(h, layer, x_bf16_dev, T, h->router_logits, out_bf16_dev, stream);
}

int b200moe_forward_routed(b200moe_handle h, int layer, const void* x_bf16_dev, int T,
                           const int32_t* topids_dev, const float* topw_dev, int stride,
                           void* out_bf16_dev, void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!x_bf16_dev || !topids_dev || !topw_dev || !out_bf16_dev || T < 0 ||
      T > h->cfg.max_tokens || stride < h->cfg.topk)
    return fail(h, B200MOE_ERR_BAD_ARG, "forward_routed: bad argument");
  if (T == 0) return B200MOE_OK;
  return forward_impl(h, layer, x_bf16_dev, T, topids_dev, topw_dev, stride, out_bf16_dev,
                      (cudaStream_t)stream);
}

int b200moe_forward_host(b200moe_handle h, int layer, const void* x_bf16_host, int T,
                         const float* logits_host, void* out_bf16_host, void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!x_bf16_host || !logits_host || !out_bf16_host || T < 0 || T > h->cfg.max_tokens)
    return fail(h, B200MOE_ERR_BAD_ARG, "forward_host: bad argument");
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int d = h->cfg.d_model, E = h->cfg.experts;
  // Large chunks are cut into up to four token ranges (of unequal size, see below): the copy of range c+1 to the device
  // and the copy of range c-1 back run on their own streams while range c computes. A
  // token's result does not depend on which other tokens share its call, so the output is
  // the same as for one call. B200MOE_HOST_CHUNKS overrides the number of ranges.
  static const int forced = getenv("B200MOE_HOST_CHUNKS") ? atoi(getenv("B200MOE_HOST_CHUNKS")) : 0;
  int C = forced > 0 ? forced : (T >= 8192 ? 4 : T >= 2048 ? 2 : 1);
  C = std::min(C, (int)b200moe_ctx::kHostChunks);
  if (C > 1 && !h->s_in) {
    CU_TRY(h, cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking));
    CU_TRY(h, cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking));
    CU_TRY(h, cudaEventCreateWithFlags(&h->ev_start, cudaEventDisableTiming));
    for (int i = 0; i < b200moe_ctx::kHostChunks; i++) {
      CU_TRY(h, cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming));
      CU_TRY(h, cudaEventCreateWithFlags(&h->ev_done[i], cudaEventDisableTiming));
      CU_TRY(h, cudaEventCreateWithFlags(&h->ev_out[i], cudaEventDisableTiming));
    }
  }
  if (C == 1) {
    const size_t xb = (size_t)T * d * 2;
    CU_TRY(h, cudaMemcpyAsync(h->x_stage, x_bf16_host, xb, cudaMemcpyHostToDevice, st));
    CU_TRY(h, cudaMemcpyAsync(h->logits_stage, logits_host, (size_t)T * E * 4, cudaMemcpyHostToDevice, st));
    if (int s = b200moe_forward(h, layer, h->x_stage, T, h->logits_stage, h->out_stage, stream)) return s;
    CU_TRY(h, cudaMemcpyAsync(out_bf16_host, h->out_stage, xb, cudaMemcpyDeviceToHost, st));
  } else {
    // range boundaries. Four ranges are cut 1/8, 2/8, 4/8, 1/8: a short first range puts the first
    // GEMMs behind a short copy, every later copy in is about as long as the compute it hides
    // behind (copying a token in takes about half as long as computing it), and the last range
    // -- whose copy out nothing hides -- is short again. Otherwise equal ranges.
    int off[b200moe_ctx::kHostChunks + 1];
    for (int c = 0; c <= C; c++) off[c] = (int)((long long)T * c / C);
    if (C == 4 && forced <= 0) {
      int w[4] = {1, 2, 4, 1};
      if (const char* sp = getenv("B200MOE_HOST_SPLIT")) {  // tuning aid: four weights that add up to 8
        int v[4];
        if (sscanf(sp, "%d,%d,%d,%d", &v[0], &v[1], &v[2], &v[3]) == 4 && v[0] > 0 && v[1] > 0 && v[2] > 0 && v[3] > 0 &&
            v[0] + v[1] + v[2] + v[3] == 8)
          for (int i = 0; i < 4; i++) w[i] = v[i];
      }
      const int eighth = T / 8;
      off[1] = w[0] * eighth;
      off[2] = off[1] + w[1] * eighth;
      off[3] = off[2] + w[2] * eighth;
    }
    // the copy streams start after whatever the caller's stream has queued (the staging
    // buffers may still be in use by an earlier call)
    CU_TRY(h, cudaEventRecord(h->ev_start, st));
    CU_TRY(h, cudaStreamWaitEvent(h->s_in, h->ev_start, 0));
    CU_TRY(h, cudaStreamWaitEvent(h->s_out, h->ev_start, 0));
    for (int c = 0; c < C; c++) {
      const int a = off[c], n = off[c + 1] - a;
      if (n <= 0) continue;
      CU_TRY(h, cudaMemcpyAsync((uint8_t*)h->x_stage + (size_t)a * d * 2, (const uint8_t*)x_bf16_host + (size_t)a * d * 2,
                                (size_t)n * d * 2, cudaMemcpyHostToDevice, h->s_in));
      CU_TRY(h, cudaMemcpyAsync(h->logits_stage + (size_t)a * E, logits_host + (size_t)a * E, (size_t)n * E * 4,
                                cudaMemcpyHostToDevice, h->s_in));
      CU_TRY(h, cudaEventRecord(h->ev_in[c], h->s_in));
    }
    for (int c = 0; c < C; c++) {
      const int a = off[c], n = off[c + 1] - a;
      if (n <= 0) continue;
      CU_TRY(h, cudaStreamWaitEvent(st, h->ev_in[c], 0));
      if (int s = b200moe_forward(h, layer, (uint8_t*)h->x_stage + (size_t)a * d * 2, n, h->logits_stage + (size_t)a * E,
                                  (uint8_t*)h->out_stage + (size_t)a * d * 2, stream))
        return s;
      CU_TRY(h, cudaEventRecord(h->ev_done[c], st));
      CU_TRY(h, cudaStreamWaitEvent(h->s_out, h->ev_done[c], 0));
      CU_TRY(h, cudaMemcpyAsync((uint8_t*)out_bf16_host + (size_t)a * d * 2, (uint8_t*)h->out_stage + (size_t)a * d * 2,
                                (size_t)n * d * 2, cudaMemcpyDeviceToHost, h->s_out));
      CU_TRY(h, cudaEventRecord(h->ev_out[c], h->s_out));
    }
    // the caller's stream ends after the last copy back (the copies of one stream are ordered)
    for (int c = C - 1; c >= 0; c--)
      if (off[c + 1] > off[c]) {
        CU_TRY(h, cudaStreamWaitEvent(st, h->ev_out[c], 0));
        break;
      }
  }
  CU_TRY(h, cudaMemcpyAsync(h->status_host, h->status_dev, 16, cudaMemcpyDeviceToHost, st));
  CU_TRY(h, cudaStreamSynchronize(st));
  return report_status(h, st);  // also clears the condition, as b200moe_synchronize does
}

int b200moe_debug_get_routing(b200moe_handle h, int T, int32_t* topids_host, float* topw_host,
                              int32_t* tokidx_host, float* pw_host, int32_t* eoff_host,
                              int32_t* pairids_host) {
  if (!h || T < 0 || T > h->cfg.max_tokens) return B200MOE_ERR_BAD_ARG;
  CU_TRY(h, cudaDeviceSynchronize());
  const size_t pairs = (size_t)T * h->cfg.topk;
  if (topids_host) CU_TRY(h, cudaMemcpy(topids_host, h->rb.topids, (size_t)T * kIdStride * 4, cudaMemcpyDeviceToHost));
  if (topw_host) CU_TRY(h, cudaMemcpy(topw_host, h->rb.topw, (size_t)T * kIdStride * 4, cudaMemcpyDeviceToHost));
  if (tokidx_host) CU_TRY(h, cudaMemcpy(tokidx_host, h->rb.tokidx, pairs * 4, cudaMemcpyDeviceToHost));
  if (pw_host) CU_TRY(h, cudaMemcpy(pw_host, h->rb.pw, pairs * 4, cudaMemcpyDeviceToHost));
  if (eoff_host) CU_TRY(h, cudaMemcpy(eoff_host, h->rb.eoff, ((size_t)h->cfg.experts + 1) * 4, cudaMemcpyDeviceToHost));
  if (pairids_host) CU_TRY(h, cudaMemcpy(pairids_host, h->rb.pairids, pairs * 4, cudaMemcpyDeviceToHost));
  CU_TRY(h, cudaMemcpy(h->status_host, h->status_dev, 16, cudaMemcpyDeviceToHost));
  return report_status(h, nullptr);
}

int b200moe_profile_enable(b200moe_handle h, int on) {
  if (!h) return B200MOE_ERR_BAD_ARG;
  if (on && h->prof_ev.empty()) {
    h->prof_ev.resize((size_t)kProfRing * kProfEvents);
    for (auto& e : h->prof_ev) CU_TRY(h, cudaEventCreate(&e));
  }
  h->prof = on != 0;
  h->prof_pending = 0;
  return B200MOE_OK;
}

int b200moe_profile_read(b200moe_handle h, float* stage_ms6, int* n_calls) {
  if (!h || !stage_ms6 || !n_calls) return B200MOE_ERR_BAD_ARG;
  for (int i = 0; i < 6; i++) stage_ms6[i] = 0.f;
  *n_calls = h->prof_pending;
  if (h->prof_pending == 0) return B200MOE_OK;
  const int last = (h->prof_head + kProfRing - 1) % kProfRing;
  CU_TRY(h, cudaEventSynchronize(h->prof_ev[(size_t)last * kProfEvents + 5]));
  for (int c = 0; c < h->prof_pending; c++) {
    const int slot = (h->prof_head + kProfRing - 1 - c) % kProfRing;
    cudaEvent_t* ev = &h->prof_ev[(size_t)slot * kProfEvents];
    float ms;
    for (int s = 0; s < 5; s++) {
      CU_TRY(h, cudaEventElapsedTime(&ms, ev[s], ev[s + 1]));
      stage_ms6[s] += ms;
    }
    CU_TRY(h, cudaEventElapsedTime(&ms, ev[0], ev[5]));
    stage_ms6[5] += ms;
  }
  for (int i = 0; i < 6; i++) stage_ms6[i] /= (float)h->prof_pending;
  h->prof_pending = 0;
  return B200MOE_OK;
}

// ---------------------------------------------------------------- expert parallelism ----
int b200moe_ep_set_placement(b200moe_handle h, const int32_t* place_host) {
  if (!h || !place_host) return B200MOE_ERR_BAD_ARG;
  const int E = h->cfg.experts;
  std::vector<int32_t> inv(E, -1);
  for (int e = 0; e < E; e++) {
    const int p = place_host[e];
    if (p < 0 || p >= E || inv[p] >= 0) return fail(h, B200MOE_ERR_BAD_ARG, "placement is not a permutation");
    inv[p] = e;
  }
  CU_TRY(h, cudaSetDevice(h->cfg.device));
  if (!h->place_dev) CU_TRY(h, cudaMalloc((void**)&h->place_dev, E * sizeof(int32_t)));
  if (!h->source_of_placed_dev) CU_TRY(h, cudaMalloc((void**)&h->source_of_placed_dev, E * sizeof(int32_t)));
  CU_TRY(h, cudaMemcpy(h->place_dev, place_host, E * sizeof(int32_t), cudaMemcpyHostToDevice));
  CU_TRY(h, cudaMemcpy(h->source_of_placed_dev, inv.data(), E * sizeof(int32_t), cudaMemcpyHostToDevice));
  for (auto& L : h->layers) L.loaded = false;  // weights must be (re)loaded under the new numbering
  return B200MOE_OK;
}

int b200moe_share_weights(b200moe_handle h, b200moe_handle owner) {
  if (!h || !owner || h == owner) return B200MOE_ERR_BAD_ARG;
  const b200moe_config &a = h->cfg, &b = owner->cfg;
  if (a.experts != b.experts || a.topk != b.topk || a.d_model != b.d_model || a.d_mid != b.d_mid ||
      a.n_layers != b.n_layers || a.device != b.device || a.ep_rank != b.ep_rank || a.ep_size != b.ep_size ||
      a.has_shared != b.has_shared)
    return fail(h, B200MOE_ERR_BAD_ARG, "share_weights: the two handles differ in shape or placement");
  for (size_t i = 0; i < h->layers.size(); i++) {
    LayerWeights& L = h->layers[i];
    if (!L.borrowed) {
      free_image(L.gu);
      free_image(L.dn);
      free_image(L.sh_gu);
      free_image(L.sh_dn);
      if (L.sh_gate_w) cudaFree(L.sh_gate_w);
      if (L.router_w) cudaFree(L.router_w);
      if (L.rot) cudaFree(L.rot);
    }
    L = owner->layers[i];
    L.borrowed = true;
    if (L.i4r && !h->x_rot)
      CU_TRY(h, dev_alloc(h, &h->x_rot, (size_t)h->cfg.max_tokens * h->cfg.d_model));
  }
  if (h->place_dev && !h->place_borrowed) cudaFree(h->place_dev);
  if (h->source_of_placed_dev && !h->place_borrowed) cudaFree(h->source_of_placed_dev);
  h->place_dev = owner->place_dev;
  h->source_of_placed_dev = owner->source_of_placed_dev;
  h->place_borrowed = true;
  return B200MOE_OK;
}

int b200moe_ep_attach(b200moe_handle h, void* x_send, void* x_recv, void* pairs_recv, void* pairs_back,
                      int64_t cap_rows) {
  if (!h || !x_send || !x_recv || !pairs_recv || !pairs_back || cap_rows < 1) return B200MOE_ERR_BAD_ARG;
  if (h->cfg.gemm_impl == B200MOE_GEMM_SIMT) return fail(h, B200MOE_ERR_UNSUPPORTED, "expert parallelism needs the tensor-core path");
  CU_TRY(h, cudaSetDevice(h->cfg.device));
  h->ep_x_send = (__half*)x_send;
  h->ep_x_recv = (__half*)x_recv;
  h->ep_pairs_recv = (__half*)pairs_recv;
  h->ep_pairs_back = (__half*)pairs_back;
  h->ep_cap_rows = cap_rows;
  h->ep_max_tiles = (int)(cap_rows / h->tile_cap) + kMaxExperts + 1;
  if (h->ep_hid) cudaFree(h->ep_hid), h->ep_hid = nullptr;
  if (h->ep_tiles) cudaFree(h->ep_tiles), h->ep_tiles = nullptr;
  if (h->tc_ep) tc_destroy(h->tc_ep), h->tc_ep = nullptr;
  if (h->tc_own) tc_destroy(h->tc_own), h->tc_own = nullptr;
  if (h->ep_rowmap) cudaFree(h->ep_rowmap), h->ep_rowmap = nullptr;
  if (h->ep_segs) cudaFree(h->ep_segs), h->ep_segs = nullptr;
  // the hidden rows of the received rows (indexed like x_recv) and of the own-rows pass in place
  // (indexed like x_send, the shared expert's rows behind the routed ones)
  const long long hid_rows = std::max<long long>(cap_rows, h->max_rows);
  CU_TRY(h, cudaMalloc((void**)&h->ep_hid, (size_t)hid_rows * h->cfg.d_mid * 2 + 256));
  CU_TRY(h, cudaMalloc((void**)&h->ep_tiles, (size_t)h->ep_max_tiles * sizeof(Tile)));
  if (!h->ep_counts) CU_TRY(h, cudaMalloc((void**)&h->ep_counts, 16));
  CU_TRY(h, tc_create(&h->tc_ep, h->ep_x_recv, h->ep_hid, cap_rows, h->cfg.d_model, h->cfg.d_mid));
  CU_TRY(h, tc_create(&h->tc_own, h->ep_x_send, h->ep_hid, h->max_rows, h->cfg.d_model, h->cfg.d_mid));
  tc_set_sm_margin(h->tc_ep, h->cfg.ep_sm_margin);
  tc_set_sm_margin(h->tc_own, h->cfg.ep_sm_margin);
  // part 4: row map of the merged area (at most one tail per source and expert), table of the tails
  CU_TRY(h, cudaMalloc((void**)&h->ep_rowmap, (size_t)kMaxExperts * h->tile_cap * sizeof(int32_t) + 256));
  CU_TRY(h, cudaMalloc((void**)&h->ep_segs, (size_t)kMaxExperts * 3 * sizeof(int32_t)));
  CU_TRY(h, cudaMemset(h->ep_segs, 0, (size_t)kMaxExperts * 3 * sizeof(int32_t)));
  {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&h->sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || h->sms < 1) h->sms = 148;
  }
  return B200MOE_OK;
}

int b200moe_ep_route(b200moe_handle h, int layer, const void* x, int T, const float* logits,
                     int32_t* eoff_out, void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!x || !logits || T < 1 || T > h->cfg.max_tokens || !h->ep_x_send)
    return fail(h, B200MOE_ERR_BAD_ARG, "ep_route: bad argument or buffers not attached");
  const b200moe_config& c = h->cfg;
  LayerWeights& L = h->layers[layer];
  const bool shared = c.has_shared != 0;
  if (shared && !L.shared_loaded) return fail(h, B200MOE_ERR_NOT_LOADED, "ep_route: shared expert not loaded");
  cudaStream_t st = (cudaStream_t)stream;
  int n = 0;
  CU_TRY(h, launch_router_topk(logits, T, c.experts, c.topk, h->rb.topids, h->rb.topw, kIdStride, st));
  if (h->place_dev) {
    CU_TRY(h, launch_apply_placement(h->rb.topids, kIdStride, T, c.topk, c.experts, h->place_dev, st));
    n++;
  }
  CU_TRY(h, launch_route(h->rb, h->rb.topids, h->rb.topw, kIdStride, T, c.topk, c.experts, h->tile_cap, st, &n));
  if (shared) {
    // the shared expert stays on the token's own rank: its rows (token order) follow the routed ones
    CU_TRY(h, launch_shared_gate(x, L.sh_gate_w, T, c.d_model, c.topk, h->rb, st));
    n++;
  }
  CU_TRY(h, launch_gather_f16(x, h->rb.tokidx, T * c.topk + (shared ? T : 0), c.d_model, h->ep_x_send, st));
  if (eoff_out)
    CU_TRY(h, cudaMemcpyAsync(eoff_out, h->rb.eoff, ((size_t)c.experts + 1) * 4, cudaMemcpyDeviceToDevice, st));
  h->launches += n + 2;
  return B200MOE_OK;
}

int b200moe_ep_offsets(b200moe_handle h, const int32_t** eoff_dev) {
  if (!h || !eoff_dev) return B200MOE_ERR_BAD_ARG;
  *eoff_dev = h->rb.eoff;
  return B200MOE_OK;
}

int b200moe_ep_experts(b200moe_handle h, int layer, const int32_t* eoff_all_dev, void* stream) {
  return b200moe_ep_experts_part(h, layer, eoff_all_dev, 0, stream);
}

int b200moe_ep_experts_part(b200moe_handle h, int layer, const int32_t* eoff_all_dev, int part, void* stream) {
  if (int s = check_layer(h, layer)) return s;
  if (!eoff_all_dev || !h->tc_ep || part < 0 || part > 4)
    return fail(h, B200MOE_ERR_BAD_ARG, "ep_experts: bad argument or buffers not attached");
  LayerWeights& L = h->layers[layer];
  const b200moe_config& c = h->cfg;
  const bool shared = c.has_shared != 0;
  if (!L.loaded || (shared && !L.shared_loaded)) return fail(h, B200MOE_ERR_NOT_LOADED, "ep_experts: layer weights not loaded");
  cudaStream_t st = (cudaStream_t)stream;
  const int El = local_experts(c);
  CU_TRY(h, launch_ep_tiles(eoff_all_dev, c.ep_size, c.experts, first_expert(c), El, h->tile_cap, h->ep_tiles,
                            h->ep_counts, h->ep_counts + 1, st, c.ep_rank, part, h->ep_segs, (int)h->ep_cap_rows));
  if (part == 4) {
    // the other ranks' rows with the tails of their (source, expert) segments merged by expert:
    // full tiles are multiplied where they were received; the rows behind a segment's last full
    // tile are copied behind the received rows, expert after expert (a small memory pass: at most
    // one tile's worth of rows per segment), and tiled there -- one ragged tile per expert instead
    // of one per source and expert --; the down GEMM writes their results back to their places in
    // the source-major result buffer, so that the return needs no pass of its own
    CU_TRY(h, launch_ep_merge_tails(h->ep_x_recv, h->ep_segs, c.ep_size * El, h->ep_counts + 1, c.d_model, h->ep_rowmap,
                                    h->sms, st));
    CU_TRY(h, launch_up_tc(h->tc_ep, L.gu, h->ep_tiles, h->ep_counts, h->ep_max_tiles, h->ep_hid, h->status_dev, st));
    CU_TRY(h, launch_down_tc(h->tc_ep, L.dn, h->ep_tiles, h->ep_counts, h->ep_max_tiles, h->ep_pairs_recv, h->status_dev, st,
                             h->ep_rowmap, h->ep_counts + 1));
    h->launches += 4;
    return B200MOE_OK;
  }
  if (part == 3) {
    // own rows in place: activations straight from the send buffer, results straight into the
    // result buffer (same row order) -- no copy in either direction; the shared expert, which
    // never leaves the token's rank, rides along
    CU_TRY(h, launch_up_tc(h->tc_own, L.gu, h->ep_tiles, h->ep_counts, h->ep_max_tiles, h->ep_hid, h->status_dev, st));
    if (shared)
      CU_TRY(h, launch_up_tc(h->tc_own, L.sh_gu, h->rb.tiles_sh, h->rb.n_tiles + 1, h->max_tiles_sh, h->ep_hid, h->status_dev, st));
    CU_TRY(h, launch_down_tc(h->tc_own, L.dn, h->ep_tiles, h->ep_counts, h->ep_max_tiles, h->ep_pairs_back, h->status_dev, st));
    if (shared)
      CU_TRY(h, launch_down_tc(h->tc_own, L.sh_dn, h->rb.tiles_sh, h->rb.n_tiles + 1, h->max_tiles_sh, h->ep_pairs_back,
                               h->status_dev, st));
    h->launches += shared ? 5 : 3;
    return B200MOE_OK;
  }
  if (shared && part != 2)
    return fail(h, B200MOE_ERR_UNSUPPORTED, "ep_experts: with a shared expert the own rows must run in place (part 3 + part 2 or 4)");
  CU_TRY(h, launch_up_tc(h->tc_ep, L.gu, h->ep_tiles, h->ep_counts, h->ep_max_tiles, h->ep_hid, h->status_dev, st));
  CU_TRY(h, launch_down_tc(h->tc_ep, L.dn, h->ep_tiles, h->ep_counts, h->ep_max_tiles, h->ep_pairs_recv,
                           h->status_dev, st));
  h->launches += 3;
  return B200MOE_OK;
}

int b200moe_ep_combine(b200moe_handle h, int T, void* out, void* stream) {
  if (!h || !out || T < 1 || T > h->cfg.max_tokens || !h->ep_pairs_back) return B200MOE_ERR_BAD_ARG;
  CU_TRY(h, launch_combine_f16(h->ep_pairs_back, h->rb.pw, h->rb.pairids, T, h->cfg.topk, h->cfg.d_model,
                               h->cfg.has_shared ? T * h->cfg.topk : -1, out, (cudaStream_t)stream));
  h->launches++;
  return B200MOE_OK;
}

int b200moe_ep_wait_flags(b200moe_handle h, const int32_t* flags_dev, int n, int32_t expected, void* stream) {
  if (!h || !flags_dev || n < 1 || n > 32) return B200MOE_ERR_BAD_ARG;
  CU_TRY(h, launch_wait_flags(flags_dev, n, expected, h->status_dev, (cudaStream_t)stream));
  h->launches++;
  return B200MOE_OK;
}

int b200moe_synchronize(b200moe_handle h, void* stream) {
  if (!h) return B200MOE_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  CU_TRY(h, cudaMemcpyAsync(h->status_host, h->status_dev, 16, cudaMemcpyDeviceToHost, st));
  CU_TRY(h, cudaStreamSynchronize(st));
  return report_status(h, st);
}

int b200moe_dequant_rows(b200moe_handle h, int layer, int which, int expert, int row0, int nrows,
                         float* out_dev, void* stream) {
  if (int s = check_layer(h, layer)) return s;
  LayerWeights& L = h->layers[layer];
  if (which < 0 || which > 3 || !out_dev || nrows < 0 || row0 < 0)
    return fail(h, B200MOE_ERR_BAD_ARG, "dequant_rows: bad argument");
  const bool sh = which >= 2;
  if (sh ? !L.shared_loaded : !L.loaded) return fail(h, B200MOE_ERR_NOT_LOADED, "dequant_rows: not loaded");
  const Image& img = which == 0 ? L.gu : which == 1 ? L.dn : which == 2 ? L.sh_gu : L.sh_dn;
  const int e_local = sh ? expert : expert - first_expert(h->cfg);
  const int rows_per = img.paired ? 2 * h->cfg.d_mid : img.n_mtiles * kTileM;
  if (e_local < 0 || e_local >= img.n_experts || row0 + nrows > rows_per)
    return fail(h, B200MOE_ERR_BAD_ARG, "dequant_rows: expert or rows out of range");
  if (nrows == 0) return B200MOE_OK;
  CU_TRY(h, launch_dequant_rows(img, e_local, row0, nrows, h->cfg.d_mid, out_dev, (cudaStream_t)stream));
  h->launches++;
  return B200MOE_OK;
}

}  // extern "C"
