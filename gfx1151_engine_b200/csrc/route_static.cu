// route_static.cu -- b200moe_route_static: the expert bucketing as a call that allocates
// nothing.
//
// Who needs it: hosts that must not (or cannot) call cudaMalloc when they reach the MoE
// layer -- an engine that has already handed all device memory to its own arena or KV-cache
// pool, a plugin loaded into a process whose memory budget is fixed at start-up, code that
// runs in a latency-critical section where the allocator's implicit device synchronisation
// is not acceptable. Such a host cannot create a b200moe handle (b200moe_create allocates
// the workspaces), yet it may still want the routing tables for its own expert kernels.
//
// How: the only scratch the bucketing needs -- the per-chunk expert counts -- lives in a
// file-scope __device__ array of fixed size below. Every GPU that loads this library
// carries that array (256 KiB) until the process exits; that is the price of never
// allocating. The limit that follows: T*topk <= 65536 pairs and experts <= 512 per call;
// anything larger is refused with B200MOE_ERR_TOO_LARGE before any launch.
//
// Sharing: all calls on one GPU use the same array, and it keeps whatever the previous
// call left. Nothing in it has to start at zero -- the first kernel overwrites every entry
// the later kernels read -- but two calls whose kernels overlap on the GPU (different
// streams without an ordering between them, or two host threads) race on it. Keep the
// calls of one GPU on one stream, or order them with events.
//
// First call on a device: resolves the array's device address (cudaGetSymbolAddress) for
// the device that is current, and caches it per device ordinal for the life of the process.
// Make that first call outside any stream capture; later calls only launch kernels. A host
// that calls cudaDeviceReset() destroys the context the cached address belongs to: this entry
// point must not be used on that device afterwards (the library has no way to notice).
//
// Ids the caller passes are checked on the device: a pair whose expert id is outside
// [0, experts) is dropped -- it is not counted, gets no row, and its slot of pairids holds -1 --
// and eoff[experts] (the number of rows placed) is then smaller than T*topk, which is how the
// caller detects it.
//
// The kernels repeat the arithmetic of route.cu (stable bucketing by expert, offsets for
// empty experts, pairids = rank among the token's experts) on caller-provided outputs.
#include "../../include/b200moe.h"
#include "common.cuh"

#include <mutex>

namespace b200moe {
namespace {

constexpr int kStaticChunk = 512;           // pairs per single-warp block
constexpr int kStaticMaxPairs = 65536;      // T * topk
constexpr int kStaticMaxExperts = 512;
constexpr int kStaticMaxChunks = kStaticMaxPairs / kStaticChunk;  // 128

// The scratch itself. In host code this name is only a handle for the symbol, never an
// address a kernel may be given: the launcher below asks the runtime for the device address.
static __device__ __align__(256) int32_t g_route_scratch[kStaticMaxChunks * kStaticMaxExperts];

constexpr int kMaxDevices = 64;
int32_t* g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_lock;

__global__ void __launch_bounds__(32)
k_static_count(const int32_t* __restrict__ ids, int stride, int pairs, int k, int E,
               int32_t* __restrict__ chunkcnt) {
  __shared__ int hist[kStaticMaxExperts];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) hist[e] = 0;
  __syncwarp();
  const int base = blockIdx.x * kStaticChunk;
  for (int it = 0; it < kStaticChunk / 32; it++) {
    const int p = base + it * 32 + lane;
    if (p < pairs) {
      // an id outside [0, E) never becomes an index: the pair is dropped (see the header)
      const int e = ids[(size_t)(p / k) * stride + p % k];
      if ((unsigned)e < (unsigned)E) atomicAdd(&hist[e], 1);
    }
  }
  __syncwarp();
  // every entry of this chunk's row is written, so stale contents never survive
  for (int e = lane; e < E; e += 32) chunkcnt[(size_t)blockIdx.x * E + e] = hist[e];
}

__global__ void __launch_bounds__(kStaticMaxExperts)
k_static_scan(int32_t* __restrict__ chunkcnt, int nchunks, int E, int32_t* __restrict__ eoff) {
  __shared__ int s[kStaticMaxExperts];
  const int e = threadIdx.x;
  int cnt = 0;
  if (e < E)
    for (int b = 0; b < nchunks; b++) {
      const int c = chunkcnt[(size_t)b * E + e];
      chunkcnt[(size_t)b * E + e] = cnt;  // exclusive prefix of this expert over the chunks
      cnt += c;
    }
  s[e] = cnt;
  __syncthreads();
  for (int o = 1; o < kStaticMaxExperts; o <<= 1) {
    const int a = e >= o ? s[e - o] : 0;
    __syncthreads();
    s[e] += a;
    __syncthreads();
  }
  if (e < E) eoff[e] = s[e] - cnt;
  if (e == 0) eoff[E] = s[kStaticMaxExperts - 1];  // pairs placed: T*topk unless ids outside [0, E) were dropped
}

__global__ void __launch_bounds__(32)
k_static_place(const int32_t* __restrict__ ids, const float* __restrict__ w, int stride, int pairs,
               int k, int E, const int32_t* __restrict__ chunkcnt, const int32_t* __restrict__ eoff,
               int32_t* __restrict__ tokidx, float* __restrict__ pw, int32_t* __restrict__ pairids) {
  __shared__ int cursor[kStaticMaxExperts];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) cursor[e] = eoff[e] + chunkcnt[(size_t)blockIdx.x * E + e];
  __syncwarp();
  const int base = blockIdx.x * kStaticChunk;
  for (int it = 0; it < kStaticChunk / 32; it++) {
    const int p = base + it * 32 + lane;
    const bool live = p < pairs;
    const unsigned act = __ballot_sync(0xffffffffu, live);
    if (live) {
      const int t = p / k, slot = p % k;
      const int e = ids[(size_t)t * stride + slot];
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
        pw[row] = w[(size_t)t * stride + slot];
      }
      // slot in the token's reduce order: ascending expert id, equal ids in slot order (every
      // slot is written); a dropped pair's slot holds -1
      int rank = 0;
      const int key = good ? e : 0x7fffffff;  // dropped pairs sort behind every expert
      for (int q = 0; q < k; q++) {
        const int eq = ids[(size_t)t * stride + q];
        const int kq = (unsigned)eq < (unsigned)E ? eq : 0x7fffffff;
        rank += (kq < key) || (kq == key && q < slot);
      }
      pairids[(size_t)t * k + rank] = good ? row : -1;
    }
    __syncwarp();
  }
}

// Device address of the scratch array on the current device; resolved once per device.
int scratch_for_current_device(int32_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return B200MOE_ERR_CUDA;
  }
  std::lock_guard<std::mutex> guard(g_setup_lock);
  if (!g_scratch_addr[dev]) {
    int32_t* addr = nullptr;
    if (cudaGetSymbolAddress((void**)&addr, g_route_scratch) != cudaSuccess || !addr) {
      cudaGetLastError();
      return B200MOE_ERR_CUDA;
    }
    g_scratch_addr[dev] = addr;
  }
  *out = g_scratch_addr[dev];
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_route_static(const int32_t* topids_dev, const float* topw_dev, int stride,
                                    int T, int topk, int experts, int32_t* tokidx_dev,
                                    float* pw_dev, int32_t* eoff_dev, int32_t* pairids_dev,
                                    void* stream) {
  using namespace b200moe;
  if (!topids_dev || !topw_dev || !tokidx_dev || !pw_dev || !eoff_dev || !pairids_dev || T < 0 ||
      topk < 1 || experts < 1 || stride < topk)
    return B200MOE_ERR_BAD_ARG;
  if (experts > kStaticMaxExperts || topk > kMaxTopK || (long long)T * topk > kStaticMaxPairs)
    return B200MOE_ERR_TOO_LARGE;
  int32_t* scratch = nullptr;
  if (int s = scratch_for_current_device(&scratch)) return s;
  cudaStream_t st = (cudaStream_t)stream;
  const int pairs = T * topk;
  const int nchunks = (pairs + kStaticChunk - 1) / kStaticChunk;
  if (nchunks > 0) k_static_count<<<nchunks, 32, 0, st>>>(topids_dev, stride, pairs, topk, experts, scratch);
  k_static_scan<<<1, kStaticMaxExperts, 0, st>>>(scratch, nchunks, experts, eoff_dev);
  if (nchunks > 0)
    k_static_place<<<nchunks, 32, 0, st>>>(topids_dev, topw_dev, stride, pairs, topk, experts, scratch,
                                           eoff_dev, tokidx_dev, pw_dev, pairids_dev);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}
