// kernels.h -- internal launch interface between the C-ABI layer (api.cu) and the kernel
// translation units. Every launcher enqueues on `st` and returns the CUDA launch status;
// none synchronises or allocates.
#pragma once
#include "common.cuh"

#include <cstdlib>
#include <utility>

namespace b200moe {

// Programmatic dependent launch for the decode chain (route -> gate/up -> down -> combine):
// the next kernel of the stream may start its prologue (code-book tables, index setup) while
// this one drains. A kernel launched this way must call pdl_wait() before it touches anything
// an earlier kernel of the stream wrote (or still reads); pdl_trigger() lets its own successor
// start early. B200MOE_NO_PDL=1 in the environment turns the attribute off (plain launches).
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  static const bool off = std::getenv("B200MOE_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = off ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}
#endif


// Source of one half (tile rows 0..63 or 64..127) of a repacked image, in the layout of
// the reference's files.
struct SrcTensor {
  const uint8_t* codes = nullptr;   // q4cp: code bytes; GGUF: raw blocks
  const uint8_t* scales = nullptr;  // q4cp only
  long long rows_per_expert = 0;
  long long row_off = 0;            // first row of this half inside an expert
  long long scale_stride = 0;       // q4cp: bytes per scale record
  int scale_group = 32;             // columns per fp16 scale: 32 (q4cp) or 128 (hgn v2 i4r)
};

// ---- repack.cu ----
// expert_map (device, may be null): source expert of image expert i is expert_map[first_expert + i]
// (placement for expert parallelism), else first_expert + i. gguf_type 20 / 23: the source is
// GGUF IQ4_NL / IQ4_XS blocks and the image is q4cp (scale = fp16(256 * block scale)); 13: the
// source is Q5_K and the image has the Q5_1 form.
cudaError_t launch_repack(const Image& img, const SrcTensor& a, const SrcTensor& b, int K,
                          int first_expert, cudaStream_t st, const int32_t* expert_map = nullptr,
                          int gguf_type = 0);
cudaError_t launch_dequant_rows(const Image& img, int expert, int row0, int nrows, int mid_rows,
                                float* out, cudaStream_t st);

// ---- route.cu ----
struct RouteBuffers {
  int32_t* topids;   // [T][16]
  float* topw;       // [T][16]
  int32_t* tokidx;   // [rows]  rows = T*k (+T with a shared expert)
  float* pw;         // [rows]
  int32_t* eoff;     // [E+1]
  int32_t* pairids;  // [T*k]
  int32_t* blockcnt; // [nblocks][E] scratch
  Run* runs;         // [E+1] active experts in ascending id (+ the shared expert last)
  int32_t* n_runs;   // [2]: routed runs, 1 (the shared run sits at runs[kMaxExperts])
  Tile* tiles;       // grouped GEMM work list, large tiles first
  Tile* tiles_sh;    // work list of the shared expert (all T tokens)
  int32_t* n_tiles;  // [2]: routed, shared
  float* sgate;      // [T] sigmoid gate of the shared expert
  int32_t* status;   // the handle's status word (may be null): {4, id} when an expert id outside [0, E) was dropped
};
cudaError_t launch_router_topk(const float* logits, int T, int E, int k, int32_t* ids, float* w,
                               int stride, cudaStream_t st);
cudaError_t launch_route(const RouteBuffers& rb, const int32_t* ids, const float* w, int stride,
                         int T, int k, int E, int tile_cap, cudaStream_t st, int* launches);
// Whole routing stage in one launch for T*k <= route_small_max_pairs(): logits != nullptr runs
// the router too (ids/w ignored), gate_w_bf16 != nullptr adds the shared expert's gate.
int route_small_max_pairs();
cudaError_t launch_route_small(const RouteBuffers& rb, const float* logits, const int32_t* ids,
                               const float* w, int stride, int T, int k, int E, const void* x_bf16,
                               const uint16_t* gate_w_bf16, int d, cudaStream_t st);
cudaError_t launch_shared_gate(const void* x_bf16, const uint16_t* gate_w_bf16, int T, int d,
                               int k, const RouteBuffers& rb, cudaStream_t st);

cudaError_t launch_apply_placement(int32_t* ids, int stride, int T, int k, int E, const int32_t* place,
                                   cudaStream_t st);
cudaError_t launch_ep_merge_tails(__half* x_recv, const int32_t* segs, int n_seg, const int32_t* counts, int d,
                                  int32_t* rowmap, int sms, cudaStream_t st);
// counts (device): [0] = rows of the source-major layout, [1] = rows of part 4's merged area behind them
cudaError_t launch_ep_tiles(const int32_t* eoff_all, int G, int E, int e0, int El, int tile_cap,
                            Tile* tiles, int32_t* n_tiles, int32_t* counts, cudaStream_t st,
                            int own_rank = 0, int part = 0,   // part 1: rows from own_rank only, 2: all others, 3: own rows at their place in the send buffer,
                            int32_t* segs = nullptr,          // 4: all others, the tails of their segments merged by expert (segs: [G * El][3])
                            int cap_rows = 0);                //    behind the received rows, as far as the buffer (cap_rows) has room

// ---- expert_simt.cu ----
cudaError_t launch_up_simt(const Image& img, const void* x_bf16, int d, int mid,
                           const int32_t* tokidx, const Run* runs, const int32_t* n_runs,
                           int max_runs, float* hid_f32, cudaStream_t st);
cudaError_t launch_down_simt(const Image& img, const float* hid_f32, int d, int mid, const Run* runs,
                             const int32_t* n_runs, int max_runs, float* pairs_f32,
                             cudaStream_t st);

// ---- expert_gemv.cu (q4cp decode / verify path) ----
int gemv_max_runs();
int gemv_max_k();     // largest d
int gemv_max_mid();   // largest mid
// img_sh: the shared expert's image (nullptr: none); its run is runs[kMaxExperts].
// hid16: fp16 [rows][mid] hidden activations silu(gate) * up, written by the gate/up kernel and
// read by the down kernel.
cudaError_t launch_up_gemv(const Image& img, const Image* img_sh, const void* x_bf16, int d, int mid,
                           const int32_t* tokidx, const Run* runs, const int32_t* n_runs,
                           __half* hid16, cudaStream_t st);
cudaError_t launch_down_gemv(const Image& img, const Image* img_sh, const __half* hid16, int d, int mid,
                             const Run* runs, const int32_t* n_runs, float* pairs_f32, cudaStream_t st);

// ---- decode.cu (q4cp decode / verify, T <= decode_max_tokens(), as one kernel) ----
// Routing (from logits, or from the caller's ids / w when logits is null), gate/up GEMV + SwiGLU,
// down GEMV and the weighted combine in one launch; every expert is read once for all the rows
// that use it. sh_gu / sh_dn: the shared expert's images or null. hid16: workspace
// [T*k + T][mid]. bar: one zero-initialised 64-bit word in device memory (grid-wide barrier).
// out_bf16, or hc_w4 + hc_state for the residual write-back. x_bf16 must be 16-byte aligned.
int decode_max_tokens();
bool decode_supported(const Image& gu, const Image& dn, const Image* sh_gu, const Image* sh_dn, int T, int k, int E, int d,
                      int mid);
cudaError_t launch_decode(const Image& gu, const Image& dn, const Image* sh_gu, const Image* sh_dn, const float* logits,
                          const int32_t* ids, const float* w, int stride, const void* x_bf16, const uint16_t* gate_w, int T,
                          int E, int k, int d, int mid, __half* hid16, void* out_bf16, const float* hc_w4, void* hc_state,
                          const RouteBuffers& rb, unsigned long long* bar, int32_t* status, cudaStream_t st,
                          unsigned long long* trace = nullptr);  // trace: debug, [SMs][8] phase time stamps of the last launch

// The routing stage alone with the decode kernel's compact router (logits given, T <= decode_max_tokens(),
// T*k <= 128, x 16-byte aligned when gate_w_bf16 is given); same outputs as launch_route_small.
cudaError_t launch_route_fast(const RouteBuffers& rb, const float* logits, int T, int k, int E, const void* x_bf16,
                              const uint16_t* gate_w_bf16, int d, cudaStream_t st);

// Bounded wait (2 s) until n <= 32 flags written by other GPUs have reached `expected`; a
// timeout sets status {3, flag index}.
cudaError_t launch_wait_flags(const int32_t* flags, int n, int32_t expected, int32_t* status, cudaStream_t st);

// ---- router_gemm.cu (router logits from hidden states) ----
struct RouterPlan;
cudaError_t router_plan_create(RouterPlan** out);
void router_plan_destroy(RouterPlan* p);
// logits[T][E] fp32 = x[T][d] (bf16) . w[E][d]^T (bf16) on the tensor cores (T > 16)
cudaError_t launch_router_gemm(RouterPlan* p, const void* x_bf16, const void* w_bf16, int T, int E, int d,
                               float* logits, int32_t* status, cudaStream_t st);
// few tokens: every logit as a double tree sum of the exact products, rounded to float
cudaError_t launch_router_dots(const void* x_bf16, const void* w_bf16, int T, int E, int d, float* logits,
                               cudaStream_t st);
// pairs/count <- (token * E + expert) of the experts that decide a token's top-k, for tokens
// where two of them are closer than rel_margin x magnitude (at most cap pairs are stored)
cudaError_t launch_router_flag(const float* logits, int T, int E, int k, float rel_margin, int32_t* pairs,
                               int32_t* count, int cap, cudaStream_t st, int32_t* status = nullptr);  // status {7, token}: list overflow
// the listed logits in the reference's arithmetic
cudaError_t launch_router_pairs(const void* x_bf16, const void* w_bf16, const int32_t* pairs, const int32_t* count,
                                int cap, int E, int d, float* logits, cudaStream_t st);

// ---- combine.cu ----
// hc_w4 / hc_state non-null: add the result into the four branches of the bf16 state
// [T][4][d] with gates 2*sigmoid(w4[t][b]/4) instead of storing out_bf16.
cudaError_t launch_combine_f32(const float* pairs, const float* pw, const int32_t* pairids, int T,
                               int k, int d, int shared_row0, void* out_bf16, cudaStream_t st,
                               const float* hc_w4 = nullptr, void* hc_state = nullptr);
cudaError_t launch_combine_f16(const __half* pairs, const float* pw, const int32_t* pairids, int T,
                               int k, int d, int shared_row0, void* out_bf16, cudaStream_t st,
                               const float* hc_w4 = nullptr, void* hc_state = nullptr);
// rot_post non-null (fp16 pairs only): out[t] = rot_post * Hn(sum), the output rotation of hgn v2 i4r
// experts (rotate.cu), applied per 128-column block before the result is stored or written back.
cudaError_t launch_combine_f16_rot(const __half* pairs, const float* pw, const int32_t* pairids, int T,
                                   int k, int d, const float* rot_post, void* out_bf16, cudaStream_t st,
                                   const float* hc_w4 = nullptr, void* hc_state = nullptr);
// src_f16: the source rows are fp16 already (rotated activations) instead of bf16
cudaError_t launch_gather_f16(const void* x_bf16, const int32_t* tokidx, int rows, int d,
                              __half* x_sorted, cudaStream_t st, bool src_f16 = false);

// ---- rotate.cu (hgn v2 i4r: Hadamard steps around the two GEMMs) ----
cudaError_t launch_rot_in(const void* x_bf16, const float* pre, int T, int d, __half* xr, cudaStream_t st);
cudaError_t launch_i4r_mid(const __half* z, const float* svh_gu, const float* suh_dn, int rows, int mid, __half* hr,
                           cudaStream_t st);
cudaError_t launch_f16_to_f32(const void* src_f16_dev, float* dst, int n, cudaStream_t st);

}  // namespace b200moe
