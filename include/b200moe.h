/* b200moe.h -- C ABI of the B200 (sm_100a) routed-expert MoE FFN operator.
 *
 * This library stands behind the MoE call sites of gfx1151-engine's layer loop. The
 * engine has no plugin interface: its operator surface is a set of GpuModel member
 * functions in one translation unit. Each entry point below names the reference
 * function (path within the reference project, file:line) whose job it takes over.
 *
 * Conventions
 *   - Every function returns an int status (B200MOE_OK == 0). Nothing aborts, throws
 *     across the boundary or falls back to the CPU; an unsupported request is an error.
 *   - Pointers named *_dev are device pointers on the handle's GPU; *_host are host
 *     pointers; `src` pointers of the loaders may be either.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 *   - A handle belongs to one GPU and one host thread at a time.
 *   - Hidden states are bf16 row-major [T][d_model]; router logits fp32 [T][experts];
 *     top-k id / weight rows carry `stride` entries of which the first topk are valid
 *     (the engine uses stride 16, src/gpu/parts/40_model.inc:4116-4136).
 */
#ifndef B200MOE_H
#define B200MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200moe_ctx* b200moe_handle;

enum {
  B200MOE_OK = 0,
  B200MOE_ERR_BAD_ARG = 1,      /* null pointer, negative size, T > max_tokens ... */
  B200MOE_ERR_UNSUPPORTED = 2,  /* shape / format outside what the kernels implement */
  B200MOE_ERR_CUDA = 3,         /* a CUDA runtime or driver call failed */
  B200MOE_ERR_NOT_LOADED = 4,   /* forward before the layer's weights were loaded */
  B200MOE_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait gave up */
  B200MOE_ERR_NCCL = 6,         /* libnccl missing, or an NCCL call of b200moe_ep_init / b200moe_ep_forward failed */
  B200MOE_ERR_ALLOC = 7,
  B200MOE_ERR_TOO_LARGE = 8     /* request exceeds a fixed capacity: b200moe_route_static's scratch, or the router's near-tie list */
};

/* GGUF tensor type ids accepted by b200moe_load_gguf (values of ggml / src/gguf.h:36-41). */
enum { B200MOE_GGML_Q5_1 = 7, B200MOE_GGML_Q8_0 = 8, B200MOE_GGML_Q4_K = 12, B200MOE_GGML_Q5_K = 13, B200MOE_GGML_IQ4_NL = 20, B200MOE_GGML_IQ4_XS = 23 };

/* Which expert GEMM implementation forward uses for T > decode_max_tokens. */
enum {
  B200MOE_GEMM_AUTO = 0,   /* tcgen05 grouped GEMM */
  B200MOE_GEMM_SIMT = 1,   /* fp32 CUDA-core kernels (the decode path, at any T); for A/B checks */
  B200MOE_GEMM_TC = 2      /* tcgen05 grouped GEMM even for T <= decode_max_tokens */
};

/* How decode / verify calls (T <= decode_max_tokens) of q4cp layers run. */
enum {
  B200MOE_DECODE_AUTO = 0,   /* routing, gate/up GEMV, down GEMV, combine as four kernels chained by programmatic dependent launch */
  B200MOE_DECODE_FUSED = 1   /* T <= 8: ONE kernel for the whole call; every expert is read once for all the rows that use it
                                (the reference's expert dedup, src/gpu/parts/26_kernels_moe_gguf.inc:749-793), bit-identical to T = 1 */
};

typedef struct {
  int32_t experts;        /* routed experts E (<= 512, as in k_router_topk, src/gpu/parts/20_kernels_gemv.inc:1443) */
  int32_t topk;           /* experts per token k (<= 16) */
  int32_t d_model;        /* multiple of 128 */
  int32_t d_mid;          /* expert intermediate size, multiple of 64 */
  int32_t n_layers;       /* layers sharing this handle's workspaces */
  int32_t max_tokens;     /* largest T of any forward call (the engine's maxbatch_cap, src/gpu/parts/40_model.inc:611-655) */
  int32_t has_shared;     /* 1: an always-on shared expert with a sigmoid scalar gate exists */
  int32_t device;         /* CUDA device ordinal */
  int32_t gemm_impl;      /* B200MOE_GEMM_* */
  int32_t decode_max_tokens; /* T up to which the GEMV path runs; 0 = default 16 (moe_naive_max, src/gpu/parts/40_model.inc:1963-1966) */
  int32_t ep_rank;        /* expert-parallel rank and size; size 1 = single GPU */
  int32_t ep_size;
  int32_t ep_sm_margin;   /* expert parallelism: SMs the grouped GEMM leaves free for the all-to-all kernels */
  int32_t decode_impl;    /* B200MOE_DECODE_*: how calls of T <= decode_max_tokens run */
  int32_t reserved[2];
} b200moe_config;

/* Replaces: GpuModel construction of the MoE workspaces (src/gpu/parts/40_model.inc:611-655)
 * and GpuMoeRouting::init (src/gpu/parts/10_ple_io.inc:833-843). Allocates every buffer a
 * later forward needs; forward itself never allocates. */
int b200moe_create(const b200moe_config* cfg, b200moe_handle* out);
int b200moe_destroy(b200moe_handle h);

/* Human-readable text for a status code / the last failure recorded on the handle
 * (replaces the message printed by CK(), src/gpu/parts/00_platform.inc:59-67). */
const char* b200moe_status_string(int status);
const char* b200moe_last_error(b200moe_handle h);

/* Replaces: wview() over the hgn q4cp expert tensors (src/gpu/parts/30_host_util.inc:875-899;
 * blob layout src/hgn.h:5-9, 219-238): gate_up is the fused [E*2*mid, d] tensor, down is
 * [E*d, mid]; each blob = [16 x f32 codebook][codes][per-row fp16 scale records].
 * One-time repack into library-owned HBM tiles; the source may be freed on return.
 * With expert parallelism every rank passes the full tensors and keeps its own experts. */
int b200moe_load_q4cp(b200moe_handle h, int layer, const void* gate_up_src, size_t gate_up_bytes,
                      const void* down_src, size_t down_bytes);

/* Replaces: gguf_experts_open / GgExperts (src/gpu/parts/30_host_util.inc:348-452): raw GGUF
 * blocks of blk.L.ffn_{gate,up,down}_exps.weight, expert e's rows at e*rows*row_bytes
 * (src/gguf.h:3-11). type_gu: Q4_K, Q5_K, Q8_0, IQ4_NL or IQ4_XS; type_dn: Q5_1, Q8_0, IQ4_NL or IQ4_XS
 * (the types of moe_gg_up / moe_gg_down, src/gpu/parts/26_kernels_moe_gguf.inc:9-20, 93-96, and of the
 * table-decoded kernels, src/gpu/parts/27_kernels_moe_lut.inc:4-19, 659-671). Q8_0 (the experts of the
 * MTP sidecar) is stored as two 4-bit planes, high and low nibble of the biased code, with exact
 * group constants: w = (16 d) * hi - 128 d + d * lo = d * q. The IQ4 types become the q4cp tile image:
 * code book = grid / 256, group scale = fp16(256 * d [* (ls - 32)]), the exact rescale of
 * 27_kernels_moe_lut.inc:312-326; Q5_K becomes the Q5_1 image form (d' = fp16(d*sc),
 * m' = fp16(-dmin*mn) per 32 elements, fifth bits regrouped). */
int b200moe_load_gguf(b200moe_handle h, int layer, const void* gate_src, const void* up_src,
                      const void* down_src, int type_gu, int type_dn);

/* Replaces: the shared-expert weight views used by moe_b_shared(_ey)
 * (src/gpu/parts/40_model.inc:4689-4711) and ref.cpp:623-636: three q4cp tensors
 * [mid,d], [mid,d], [d,mid] and the bf16 [d] weight of the scalar sigmoid gate. */
int b200moe_load_shared_q4cp(b200moe_handle h, int layer, const void* gate_src, const void* up_src,
                             const void* down_src, const void* gate_w_bf16_src);

/* Replaces: moe_b_v2 (src/gpu/parts/40_model.inc:4559-4680), the routed experts of hgn v2
 * checkpoints: dtype 23 "i4r" tensors ([E*2*mid, d] and [E*d, mid]: rows*cols/2 code bytes, low
 * nibble = even column, then one fp16 scale per 128 columns, w = (nib - 8) * scale) that live in
 * a Hadamard-rotated domain, with their four fp16 sign-scale planes (the .suh / .svh sidecars of
 * src/gpu/parts/30_host_util.inc:818-858, one per tensor, shared by all experts):
 *   gu_suh [d], gu_svh [2*mid], dn_suh [mid], dn_svh [d].
 * The layer then computes, per token and chosen expert,
 *   out = dn_svh * Hn( sum_k w_k G_down . Hn( dn_suh * silu(g) * u ) ),  g|u = gu_svh * Hn( G_gate_up . Hn(gu_suh * x) )
 * with Hn the block-diagonal 128-point Hadamard transform / sqrt(128) (28_kernels_hgn_v2.inc:1-15,
 * 98-152). Every pointer may be host or device memory. Needs d % 128 == 0, mid % 128 == 0 and
 * 2*mid <= d; runs on the tensor-core path for every T; not combined with a shared expert, with
 * expert parallelism or with B200MOE_GEMM_SIMT (B200MOE_ERR_UNSUPPORTED). */
int b200moe_load_i4r(b200moe_handle h, int layer, const void* gate_up_src, size_t gate_up_bytes,
                     const void* down_src, size_t down_bytes, const void* gu_suh_f16, const void* gu_svh_f16,
                     const void* dn_suh_f16, const void* dn_svh_f16);

/* Replaces: GpuModel::moe_b from the router top-k on (src/gpu/parts/40_model.inc:4018-4157) and
 * GpuModel::moe (:1806-1861); oracle Model::moe, src/ref.cpp:574-637. Asynchronous on
 * `stream`; no allocation, no host synchronisation. out is fully overwritten. */
int b200moe_forward(b200moe_handle h, int layer, const void* x_bf16_dev, int T,
                    const float* logits_dev, void* out_bf16_dev, void* stream);

/* Replaces: the seam below the router, moe_q4w_run (src/gpu/parts/40_model.inc:1736-1804) and
 * moe_gguf (:1664-1714): the caller supplies top-k ids and weights (descending probability). */
int b200moe_forward_routed(b200moe_handle h, int layer, const void* x_bf16_dev, int T,
                           const int32_t* topids_dev, const float* topw_dev, int stride,
                           void* out_bf16_dev, void* stream);

/* The same call for callers whose buffers live in host memory (pinned or pageable):
 * copies x and logits to the GPU, runs b200moe_forward, copies out back and waits.
 * This is the end-to-end path the benchmark times against the CPU reference. */
int b200moe_forward_host(b200moe_handle h, int layer, const void* x_bf16_host, int T,
                         const float* logits_host, void* out_bf16_host, void* stream);

/* The configuration the handle was created with. */
/* Replaces: the layer call followed by k_moe_reduce_pw_sg_hc
 * (src/gpu/parts/24_kernels_moe_lt.inc:126-161): as b200moe_forward, but the result is not
 * stored; it is added into the four branches of the bf16 residual state [T][4][d_model],
 *   state[t][b][c] = bf16(float(state[t][b][c]) + 2*sigmoid(inject_w4[t][b] / 4) * y[t][c]),
 * with y in fp32 (no bf16 rounding of the layer output in between). inject_w4 is fp32 [T][4]. */
int b200moe_forward_hc(b200moe_handle h, int layer, const void* x_bf16_dev, int T, const float* logits_dev,
                       const float* inject_w4_dev, void* state_bf16_dev, void* stream);

int b200moe_get_config(b200moe_handle h, b200moe_config* out);

/* Expert tensors of one layer straight from a model file (mapped read-only for the duration of
 * the call). `model_layer` is the layer number inside the file; `layer` the handle's slot.
 *   load_hgn_file:  the engine's own container (Checkpoint::map_file, src/hgn.h:48-62, 295-363):
 *                   layers.L.mlp.experts.{gate_up_proj,down_proj}.weight (dtype 5, q4cp), with
 *                   has_shared also layers.L.mlp.shared_expert.* and shared_expert_gate.weight,
 *                   and the router weight layers.L.mlp.gate.weight when present (src/ref.cpp:566-633).
 *   load_gguf_file: GGUF v2/v3 (src/gguf.h:1-11, 136-314), sharded or not (pass any shard of
 *                   NAME-0000i-of-0000n.gguf): blk.L.ffn_{gate,up,down}_exps.weight, ne = [K, N, E]
 *                   (src/gpu/parts/30_host_util.inc:384-412), any of the block types b200moe_load_gguf reads.
 * B200MOE_ERR_BAD_ARG: file missing, malformed or without the tensors; B200MOE_ERR_UNSUPPORTED:
 * shapes or types that do not match the handle. */
int b200moe_load_hgn_file(b200moe_handle h, int layer, const char* path, int model_layer);
int b200moe_load_gguf_file(b200moe_handle h, int layer, const char* path, int model_layer);

/* Router logits from hidden states. Replaces the engine's router GEMM in front of moe_b
 * (gemm(gate_weight(l), d_xb, d_routerb, P), src/gpu/parts/40_model.inc:4022-4025) and follows the
 * CPU reference (matvec over layers.L.mlp.gate.weight, src/ref.cpp:68-77, 565-567: double
 * products summed in index order, rounded to float once).
 *   load_router:    bf16 [experts][d_model], host or device pointer, copied into library memory.
 *   router_logits:  logits_dev[T][experts] fp32. T <= 16: double sums of the exact products
 *                   (1e-9 from the reference's sum). T > 16: tensor-core GEMM (exact bf16
 *                   products, fp32 sums, ~1e-5 from the reference). In both cases the experts
 *                   that decide a token's top-k (its k largest logits and everything within two
 *                   margins of the k-th) are recomputed in the reference's arithmetic whenever
 *                   two of them are closer than the margin, so that the top-k ids and their
 *                   order are the reference's; the remaining logits only enter the softmax
 *                   denominator, which cancels in the renormalised weights.
 *   forward_hidden: router_logits into a workspace, then b200moe_forward. */
int b200moe_load_router(b200moe_handle h, int layer, const void* gate_weight_bf16);
int b200moe_router_logits(b200moe_handle h, int layer, const void* x_bf16_dev, int T, float* logits_dev,
                          void* stream);
int b200moe_forward_hidden(b200moe_handle h, int layer, const void* x_bf16_dev, int T, void* out_bf16_dev,
                           void* stream);

/* Replaces: router_topk_b / k_router_topk_w32 (src/gpu/parts/40_model.inc:4011-4017,
 * src/gpu/parts/20_kernels_gemv.inc:1495-1562); arithmetic of src/ref.cpp:574-588.
 * Order: descending probability, ties to the lowest expert id. */
int b200moe_router_topk(b200moe_handle h, const float* logits_dev, int T, int32_t* topids_dev,
                        float* topw_dev, int stride, void* stream);

/* Replaces: GpuMoeRouting::run + k_moe_tiles (src/gpu/parts/10_ple_io.inc:784-861). Builds, in
 * the handle's workspace, the stable (expert, pair) permutation, expert offsets, reduce
 * order and tile list for the given selection. Ids are checked on the device: a pair whose expert
 * id is outside [0, experts) is dropped (it contributes nothing to the layer output) and the next
 * b200moe_synchronize returns B200MOE_ERR_BAD_ARG; the same holds for b200moe_forward_routed. */
int b200moe_route(b200moe_handle h, const int32_t* topids_dev, const float* topw_dev, int stride,
                  int T, void* stream);

/* The bucketing of b200moe_route for hosts that cannot allocate device memory at this point
 * (all HBM already given to their own arena or KV pool, a fixed memory budget, or a section
 * where cudaMalloc's implicit synchronisation is not acceptable) and therefore have no handle.
 * It has no counterpart in the reference. Needs no handle and calls no allocator: its scratch
 * (per-chunk expert counts) is a 256 KiB __device__ array inside the library, present on every
 * GPU that loads it. Limits: T*topk <= 65536, experts <= 512, topk <= 16; beyond them the call
 * returns B200MOE_ERR_TOO_LARGE and launches nothing. Outputs are caller buffers on the current
 * device: tokidx[T*topk], pw[T*topk], eoff[experts+1], pairids[T*topk], same definitions and
 * same bytes as b200moe_route produces. All calls on a GPU share the scratch: calls whose
 * kernels overlap (unordered streams, several threads) race; keep them on one stream. The
 * first call on a device looks up the scratch's device address and caches it for the life of
 * the process -- make that call before any stream capture, and do not use this entry point on a
 * device after the host has called cudaDeviceReset() on it (the cached address would be stale).
 * Expert ids outside [0, experts) are never used as an index: such a pair is dropped (no row, its
 * pairids slot is -1) and eoff[experts], the number of rows placed, is then below T*topk. */
int b200moe_route_static(const int32_t* topids_dev, const float* topw_dev, int stride, int T,
                         int topk, int experts, int32_t* tokidx_dev, float* pw_dev,
                         int32_t* eoff_dev, int32_t* pairids_dev, void* stream);

/* ---- Expert parallelism (no counterpart in the reference, which runs on one device) -------
 * With ep_size > 1 in the config, rank r owns experts [r*E/G, (r+1)*E/G) of the PLACED
 * numbering (b200moe_ep_set_placement; identity by default). A forward is three library
 * phases with the two all-to-all exchanges in between done by the caller (NCCL):
 *   ep_route:    router top-k, bucketing, gather of this rank's rows into x_send, sorted by
 *                placed expert id and therefore by destination rank;
 *   (all-gather of every rank's expert offsets, all-to-all of the rows into x_recv)
 *   ep_experts:  grouped GEMMs over the received rows -> pairs_recv (same row order);
 *   (all-to-all of pairs_recv back into pairs_back, which then has x_send's row order)
 *   ep_combine:  weighted top-k combine of this rank's tokens.
 * ep_attach hands the library the four fp16 row buffers [rows][d_model] (caller-owned device
 * memory: x_send and pairs_back hold max_tokens*topk rows -- plus max_tokens rows behind them when
 * the layer has a shared expert -- x_recv and pairs_recv cap_rows). A shared expert is not
 * sharded: every rank holds it and runs it for its own tokens (rows max_tokens*topk.. of x_send /
 * pairs_back, in token order), as part of the in-place own-rows pass (part 3 below). */
int b200moe_ep_set_placement(b200moe_handle h, const int32_t* placed_id_of_expert_host);
/* Makes `h` use the repacked weights (and placement) of `owner` instead of holding its own:
 * several handles with separate workspaces can then work on different token chunks of the same
 * layer at once (the chunked, overlapped expert-parallel forward). `owner` must outlive `h` and
 * have the same shape configuration. */
int b200moe_share_weights(b200moe_handle h, b200moe_handle owner);
int b200moe_ep_attach(b200moe_handle h, void* x_send_dev, void* x_recv_dev, void* pairs_recv_dev,
                      void* pairs_back_dev, int64_t cap_rows);
int b200moe_ep_route(b200moe_handle h, int layer, const void* x_bf16_dev, int T,
                     const float* logits_dev, int32_t* eoff_out_dev /* [experts+1], may be NULL */,
                     void* stream);
int b200moe_ep_offsets(b200moe_handle h, const int32_t** eoff_dev);
int b200moe_ep_experts(b200moe_handle h, int layer, const int32_t* eoff_all_dev, void* stream);
/* The same over a part of the received rows: part 1 = the rows this rank sent to itself (they need
 * no exchange, so their GEMMs can run while the other ranks' rows are still arriving), part 2 = the
 * other ranks' rows, 0 = all. Parts 1 and 2 together write what part 0 writes. Part 3 = the own
 * rows IN PLACE: read from x_send where ep_route left them and written to pairs_back where
 * ep_combine expects them -- neither direction is copied -- together with the shared expert's rows
 * when the layer has one. A forward is then part 3 + part 2; the own segment of x_recv / pairs_recv
 * stays unused. Part 4 = part 2 with the TAILS of the other ranks' rows merged by expert: x_recv is
 * source-major, so an expert that received rows from seven ranks has seven runs there and up to
 * seven ragged GEMM tiles. Part 4 multiplies the full tiles of every run where they lie, copies
 * the rows behind each run's last full tile to the free end of x_recv (behind the received rows;
 * as far as cap_rows leaves room, else it is part 2), expert after expert, tiles them there -- one
 * ragged tile per expert -- and has the down GEMM write their results to their source-major places
 * in pairs_recv: the same bytes as part 2 with far fewer small tiles (at 8 ranks and three
 * chunks: 820 full + 197 ragged tile columns against 755 + 606). */
int b200moe_ep_experts_part(b200moe_handle h, int layer, const int32_t* eoff_all_dev, int part, void* stream);
int b200moe_ep_combine(b200moe_handle h, int T, void* out_bf16_dev, void* stream);
/* For hosts that move the rows with peer copies (copy engines) instead of a collective: every
 * sender writes its sequence number into the receiver's flag array behind its data (same
 * stream, so the copy engine orders them); this enqueues a wait until all n <= 32 flags have
 * reached `expected`. The wait is bounded (2 s): a timeout is reported by b200moe_synchronize as
 * B200MOE_ERR_DEVICE_TIMEOUT and the stream continues. */
int b200moe_ep_wait_flags(b200moe_handle h, const int32_t* flags_dev, int n, int32_t expected, void* stream);

/* The host side of expert parallelism inside the library, for hosts written in C / C++ (no
 * counterpart in the reference): the exchanges are NCCL point-to-point groups, NCCL is loaded at run
 * time (libnccl.so.2; B200MOE_ERR_NCCL when it is missing or a call fails).
 *   ep_unique_id: rank 0 makes the 128-byte NCCL id; the host carries it to the other ranks.
 *   ep_init:      collective over the ep_size ranks (handles created with ep_rank / ep_size): builds
 *                 the communicator, allocates the four row buffers (receive side cap_factor x
 *                 max_tokens*topk rows, >= 1.0; 2.0 is ample with a balanced placement) and attaches them.
 *   ep_forward:   one layer call of this rank's T tokens: route, all-gather of the offset tables,
 *                 own rows in place, dispatch, other ranks' rows, return, combine -- all on `stream`,
 *                 with one host wait for the tables. Every rank must call it (with its own T).
 *                 B200MOE_ERR_TOO_LARGE on EVERY rank when some rank's receive buffer would overflow
 *                 (nothing has been exchanged then); B200MOE_ERR_NCCL with b200moe_ep_last_error.
 *   ep_shutdown:  frees the communicator and the buffers (b200moe_destroy does it too). */
int b200moe_ep_unique_id(void* id128);
int b200moe_ep_init(b200moe_handle h, const void* id128, double cap_factor);
int b200moe_ep_forward(b200moe_handle h, int layer, const void* x_bf16_dev, int T, const float* logits_dev,
                       void* out_bf16_dev, void* stream);
int b200moe_ep_shutdown(b200moe_handle h);
const char* b200moe_ep_last_error(b200moe_handle h);

/* Reads back what the last forward / route call left in the workspace (host buffers; any may
 * be NULL): tokidx[T*k], pw[T*k], eoff[E+1], pairids[T*k] as defined by
 * src/gpu/parts/10_ple_io.inc:790-811, and topids/topw rows of 16. Synchronises the device. */
int b200moe_debug_get_routing(b200moe_handle h, int T, int32_t* topids_host, float* topw_host,
                              int32_t* tokidx_host, float* pw_host, int32_t* eoff_host,
                              int32_t* pairids_host);

/* Dequantises rows of a loaded tensor from the repacked image into fp32 (device buffer
 * [nrows][cols]); bit-identical to q4cp_row (src/hgn.h:249-261) / gguf::dequant_row
 * (src/gguf.h:339-443). which: 0 gate_up (rows 0..2*mid-1 of an expert: gate then up),
 * 1 down (rows 0..d-1), 2 shared gate_up, 3 shared down. */
int b200moe_dequant_rows(b200moe_handle h, int layer, int which, int expert, int row0, int nrows,
                         float* out_dev, void* stream);

/* Waits for `stream` and reports B200MOE_ERR_DEVICE_TIMEOUT if a kernel of an earlier
 * forward gave up a bounded wait, or B200MOE_ERR_BAD_ARG if a caller-supplied expert id was out
 * of range (replaces the implicit check of CK() after hipStreamSynchronize in the reference's
 * layer loop). Clears the recorded condition. */
int b200moe_synchronize(b200moe_handle h, void* stream);

/* Stage timer (replaces the reference's event-ring kernel profiler KP()/kprof,
 * src/gpu/parts/07_kprof.inc:1-134, tags moe:route/up/down/reduce). When enabled, forward
 * records CUDA events between its stages on the caller's stream; profile_read waits for the
 * last recorded call and returns, per stage, the mean milliseconds over the calls since the
 * previous read (at most the last 64): [0] router top-k + bucketing, [1] activation gather,
 * [2] gate/up GEMM + SwiGLU, [3] down GEMM, [4] combine, [5] whole call. */
int b200moe_profile_enable(b200moe_handle h, int on);
int b200moe_profile_read(b200moe_handle h, float* stage_ms6, int* n_calls);

/* Number of kernels this library launched since the handle was created (the benchmark
 * reports the difference across its timed region). */
int64_t b200moe_launch_count(b200moe_handle h);

/* Library build information: "b200moe <version> sm_100a". */
const char* b200moe_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H */
