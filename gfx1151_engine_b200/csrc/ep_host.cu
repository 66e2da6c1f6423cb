// ep_host.cu -- expert parallelism with the HOST side inside the library: b200moe_ep_init /
// b200moe_ep_forward. A C++ engine (the reference is one, src/gpu/parts/40_model.inc:4018) calls
// one function per layer and rank; no Python, no PyTorch.
//
// The reference runs on one device and has no counterpart of this file. The exchange uses
// NCCL (point-to-point sends and receives grouped into one all-to-all per direction, plus one
// all-gather of the ranks' expert offset tables). NCCL is loaded at run time (dlopen of
// libnccl.so.2) so that single-GPU users need no NCCL and a process that already carries an
// NCCL (a PyTorch host) keeps using its own copy.
//
// One forward of rank r:
//   1. ep_route          router top-k, bucketing by placed expert (= by destination rank), gather
//                        of this rank's rows into the send buffer
//   2. all-gather        every rank's expert offset table; its copy on the host gives the row
//                        counts of both exchanges (every rank sees every count: a receive buffer
//                        that is too small stops ALL ranks with B200MOE_ERR_TOO_LARGE, before any
//                        row moves)
//   3. own rows          GEMMs over the rows that stay on this rank, in place (no copy), enqueued
//                        before the host waits for the table: they run while it travels
//   4. dispatch          rows to the owners of their experts (ncclSend / ncclRecv group)
//   5. other ranks' rows GEMMs over what arrived
//   6. return            results back to the rows' owners
//   7. ep_combine        weighted top-k sum of this rank's tokens
// Everything is enqueued on the caller's stream; the one host wait is the read of the offset
// tables in step 2.
#include "../../include/b200moe.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace {

struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;
std::mutex g_nccl_lock;

// Loads libnccl.so.2 once. A copy the process already holds is found first (RTLD_NOLOAD).
bool load_nccl(std::string* why) {
  std::lock_guard<std::mutex> guard(g_nccl_lock);
  if (g_nccl.lib) return true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* lib = nullptr;
  for (const char* n : names)
    if ((lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL))) break;
  if (!lib)
    for (const char* n : names)
      if ((lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
  if (!lib) {
    *why = std::string("libnccl.so.2 not found: ") + (dlerror() ? dlerror() : "");
    return false;
  }
  NcclApi a;
  a.lib = lib;
#define B200MOE_SYM(field, name)                                             \
  a.field = (decltype(a.field))dlsym(lib, name);                             \
  if (!a.field) {                                                            \
    *why = std::string("libnccl.so.2 lacks ") + name;                        \
    return false;                                                            \
  }
  B200MOE_SYM(GetUniqueId, "ncclGetUniqueId")
  B200MOE_SYM(CommInitRank, "ncclCommInitRank")
  B200MOE_SYM(CommDestroy, "ncclCommDestroy")
  B200MOE_SYM(AllGather, "ncclAllGather")
  B200MOE_SYM(Send, "ncclSend")
  B200MOE_SYM(Recv, "ncclRecv")
  B200MOE_SYM(GroupStart, "ncclGroupStart")
  B200MOE_SYM(GroupEnd, "ncclGroupEnd")
  B200MOE_SYM(GetErrorString, "ncclGetErrorString")
#undef B200MOE_SYM
  g_nccl = a;
  return true;
}

}  // namespace

// The state b200moe_ep_init hangs on a handle (kept apart from b200moe_ctx: api.cu stays free of NCCL).
struct b200moe_ep_state {
  ncclComm_t comm = nullptr;
  int rank = 0, size = 1, experts = 0, topk = 0, d = 0, max_tokens = 0, has_shared = 0;
  long long cap_rows = 0;
  void *x_send = nullptr, *x_recv = nullptr, *pairs_recv = nullptr, *pairs_back = nullptr;
  int32_t *eoff = nullptr, *eoff_all = nullptr;
  int32_t* eoff_host = nullptr;  // pinned
  cudaEvent_t table_ready = nullptr;
  std::string err;
};

namespace {

std::mutex g_states_lock;
std::vector<std::pair<b200moe_handle, b200moe_ep_state*>> g_states;

b200moe_ep_state* state_of(b200moe_handle h) {
  std::lock_guard<std::mutex> guard(g_states_lock);
  for (auto& p : g_states)
    if (p.first == h) return p.second;
  return nullptr;
}

void free_state(b200moe_ep_state* s) {
  if (!s) return;
  if (s->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(s->comm);
  for (void* p : {s->x_send, s->x_recv, s->pairs_recv, s->pairs_back, (void*)s->eoff, (void*)s->eoff_all})
    if (p) cudaFree(p);
  if (s->eoff_host) cudaFreeHost(s->eoff_host);
  if (s->table_ready) cudaEventDestroy(s->table_ready);
  delete s;
}

}  // namespace

extern "C" {

int b200moe_ep_unique_id(void* id128) {
  if (!id128) return B200MOE_ERR_BAD_ARG;
  std::string why;
  if (!load_nccl(&why)) {
    fprintf(stderr, "b200moe_ep_unique_id: %s\n", why.c_str());
    return B200MOE_ERR_NCCL;
  }
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  if (g_nccl.GetUniqueId(&id) != ncclSuccess) return B200MOE_ERR_NCCL;
  memcpy(id128, &id, sizeof id);
  return B200MOE_OK;
}

int b200moe_ep_init(b200moe_handle h, const void* id128, double cap_factor) {
  if (!h || !id128) return B200MOE_ERR_BAD_ARG;
  b200moe_config c;
  if (int s = b200moe_get_config(h, &c)) return s;
  if (c.ep_size < 2 || cap_factor < 1.0) return B200MOE_ERR_BAD_ARG;
  if (state_of(h)) return B200MOE_ERR_BAD_ARG;  // once per handle
  std::string why;
  if (!load_nccl(&why)) {
    fprintf(stderr, "b200moe_ep_init: %s\n", why.c_str());
    return B200MOE_ERR_NCCL;
  }
  if (cudaSetDevice(c.device) != cudaSuccess) return B200MOE_ERR_CUDA;
  b200moe_ep_state* s = new b200moe_ep_state();
  s->rank = c.ep_rank; s->size = c.ep_size; s->experts = c.experts; s->topk = c.topk; s->d = c.d_model;
  s->max_tokens = c.max_tokens; s->has_shared = c.has_shared;
  const long long pairs = (long long)c.max_tokens * c.topk;
  const long long own_rows = pairs + (c.has_shared ? c.max_tokens : 0);
  s->cap_rows = (long long)(cap_factor * (double)pairs);
  const size_t row = (size_t)c.d_model * 2;
  cudaError_t e = cudaMalloc(&s->x_send, own_rows * row);
  if (e == cudaSuccess) e = cudaMalloc(&s->x_recv, s->cap_rows * row);
  if (e == cudaSuccess) e = cudaMalloc(&s->pairs_recv, s->cap_rows * row);
  if (e == cudaSuccess) e = cudaMalloc(&s->pairs_back, own_rows * row);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->eoff, ((size_t)c.experts + 1) * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->eoff_all, (size_t)c.ep_size * (c.experts + 1) * 4);
  if (e == cudaSuccess) e = cudaMallocHost((void**)&s->eoff_host, (size_t)c.ep_size * (c.experts + 1) * 4);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->table_ready, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    cudaGetLastError();
    free_state(s);
    return e == cudaErrorMemoryAllocation ? B200MOE_ERR_ALLOC : B200MOE_ERR_CUDA;
  }
  ncclUniqueId id;
  memcpy(&id, id128, sizeof id);
  const ncclResult_t r = g_nccl.CommInitRank(&s->comm, c.ep_size, id, c.ep_rank);
  if (r != ncclSuccess) {
    fprintf(stderr, "b200moe_ep_init: ncclCommInitRank: %s\n", g_nccl.GetErrorString(r));
    s->comm = nullptr;
    free_state(s);
    return B200MOE_ERR_NCCL;
  }
  if (int st = b200moe_ep_attach(h, s->x_send, s->x_recv, s->pairs_recv, s->pairs_back, s->cap_rows)) {
    free_state(s);
    return st;
  }
  std::lock_guard<std::mutex> guard(g_states_lock);
  g_states.emplace_back(h, s);
  return B200MOE_OK;
}

int b200moe_ep_shutdown(b200moe_handle h) {
  b200moe_ep_state* s = nullptr;
  {
    std::lock_guard<std::mutex> guard(g_states_lock);
    for (size_t i = 0; i < g_states.size(); i++)
      if (g_states[i].first == h) {
        s = g_states[i].second;
        g_states.erase(g_states.begin() + i);
        break;
      }
  }
  if (!s) return B200MOE_ERR_BAD_ARG;
  cudaDeviceSynchronize();
  free_state(s);
  return B200MOE_OK;
}

const char* b200moe_ep_last_error(b200moe_handle h) {
  b200moe_ep_state* s = state_of(h);
  return s ? s->err.c_str() : "expert parallelism not initialised on this handle";
}

int b200moe_ep_forward(b200moe_handle h, int layer, const void* x_bf16_dev, int T, const float* logits_dev,
                       void* out_bf16_dev, void* stream) {
  b200moe_ep_state* s = state_of(h);
  if (!s || !x_bf16_dev || !logits_dev || !out_bf16_dev || T < 1 || T > s->max_tokens) return B200MOE_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int G = s->size, E = s->experts, per = E / G;
  auto nccl_fail = [&](const char* what, ncclResult_t r) {
    s->err = std::string(what) + ": " + g_nccl.GetErrorString(r);
    return (int)B200MOE_ERR_NCCL;
  };
  auto cuda_fail = [&](const char* what, cudaError_t e) {
    s->err = std::string(what) + ": " + cudaGetErrorString(e);
    return (int)B200MOE_ERR_CUDA;
  };
  // 1, 2: routing, offset tables of all ranks, their copy on the host
  if (int rc = b200moe_ep_route(h, layer, x_bf16_dev, T, logits_dev, s->eoff, stream)) return rc;
  ncclResult_t r = g_nccl.AllGather(s->eoff, s->eoff_all, (size_t)E + 1, ncclInt32, s->comm, st);
  if (r != ncclSuccess) return nccl_fail("ncclAllGather", r);
  cudaError_t e = cudaMemcpyAsync(s->eoff_host, s->eoff_all, (size_t)G * (E + 1) * 4, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaEventRecord(s->table_ready, st);
  if (e != cudaSuccess) return cuda_fail("offset tables to the host", e);
  // 3: the rows that stay here (and the shared expert's), in place; they run while the host waits
  if (int rc = b200moe_ep_experts_part(h, layer, s->eoff_all, 3, stream)) return rc;
  e = cudaEventSynchronize(s->table_ready);
  if (e != cudaSuccess) return cuda_fail("waiting for the offset tables", e);
  // rows source q sends to destination p: cnt[q][p]; offsets in q's send buffer: bd[q][p]
  auto bd = [&](int q, int p) { return (long long)s->eoff_host[(size_t)q * (E + 1) + (size_t)p * per]; };
  auto cnt = [&](int q, int p) { return bd(q, p + 1) - bd(q, p); };
  for (int p = 0; p < G; p++) {
    long long need = 0;
    for (int q = 0; q < G; q++) need += cnt(q, p);
    if (need > s->cap_rows) {  // the same table on every rank: all of them return here
      char buf[160];
      snprintf(buf, sizeof buf, "receive buffer too small: rank %d would receive %lld rows, capacity %lld", p, need, s->cap_rows);
      s->err = buf;
      return B200MOE_ERR_TOO_LARGE;
    }
  }
  const size_t row = (size_t)s->d;  // halves per row
  std::vector<long long> recv_off(G + 1, 0);
  for (int q = 0; q < G; q++) recv_off[q + 1] = recv_off[q] + cnt(q, s->rank);
  // 4: dispatch (own rows stay where they are)
  if ((r = g_nccl.GroupStart()) != ncclSuccess) return nccl_fail("ncclGroupStart", r);
  for (int p = 0; p < G; p++) {
    if (p == s->rank) continue;
    if (cnt(s->rank, p) && (r = g_nccl.Send((const __half*)s->x_send + (size_t)bd(s->rank, p) * row, (size_t)cnt(s->rank, p) * row,
                                            ncclHalf, p, s->comm, st)) != ncclSuccess)
      break;
    if (cnt(p, s->rank) && (r = g_nccl.Recv((__half*)s->x_recv + (size_t)recv_off[p] * row, (size_t)cnt(p, s->rank) * row, ncclHalf,
                                            p, s->comm, st)) != ncclSuccess)
      break;
  }
  const ncclResult_t r_end = g_nccl.GroupEnd();
  if (r != ncclSuccess) return nccl_fail("dispatch", r);
  if (r_end != ncclSuccess) return nccl_fail("ncclGroupEnd", r_end);
  // 5: the other ranks' rows (from four ranks on with the tails of their runs merged by expert)
  if (int rc = b200moe_ep_experts_part(h, layer, s->eoff_all, G >= 4 ? 4 : 2, stream)) return rc;
  // 6: results back to their owners (into the owner's send order)
  if ((r = g_nccl.GroupStart()) != ncclSuccess) return nccl_fail("ncclGroupStart", r);
  for (int p = 0; p < G; p++) {
    if (p == s->rank) continue;
    if (cnt(p, s->rank) && (r = g_nccl.Send((const __half*)s->pairs_recv + (size_t)recv_off[p] * row, (size_t)cnt(p, s->rank) * row,
                                            ncclHalf, p, s->comm, st)) != ncclSuccess)
      break;
    if (cnt(s->rank, p) && (r = g_nccl.Recv((__half*)s->pairs_back + (size_t)bd(s->rank, p) * row, (size_t)cnt(s->rank, p) * row,
                                            ncclHalf, p, s->comm, st)) != ncclSuccess)
      break;
  }
  const ncclResult_t r_end2 = g_nccl.GroupEnd();
  if (r != ncclSuccess) return nccl_fail("return exchange", r);
  if (r_end2 != ncclSuccess) return nccl_fail("ncclGroupEnd", r_end2);
  // 7
  return b200moe_ep_combine(h, T, out_bf16_dev, stream);
}

}  // extern "C"
