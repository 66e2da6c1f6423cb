// tc.h -- interface of the tcgen05 grouped dequant-GEMM (expert_tc.cu).
#pragma once
#include "common.cuh"

namespace b200moe {

struct TcPlan;  // tensor maps over the activation buffers + device properties

// x_sorted: [rows_cap][d] fp16 (expert-sorted activations); hid16: [rows_cap][mid] fp16.
cudaError_t tc_create(TcPlan** plan, const __half* x_sorted, const __half* hid16,
                      long long rows_cap, int d, int mid);
void tc_destroy(TcPlan* plan);
// Leave `sms` SMs free of the persistent GEMM CTAs (for communication kernels that must run
// at the same time).
void tc_set_sm_margin(TcPlan* plan, int sms);

// Largest number of rows in one grouped-GEMM tile (the MMA N extent).
constexpr int kTcTileN = 192;

// gate/up GEMM + SwiGLU: hid16[row][mid] = silu(W_gate x) * (W_up x) for every row of every tile.
cudaError_t launch_up_tc(TcPlan* plan, const Image& img, const Tile* tiles, const int32_t* n_tiles,
                         int max_tiles, __half* hid16, int32_t* status, cudaStream_t st);
// down GEMM: pairs16[row][d] = W_down hid16[row].
// rowmap + map_base (device, both or neither): result row r >= map_base[0] of the tile list goes to
// pairs16[rowmap[r - map_base[0]]] instead of pairs16[r].
cudaError_t launch_down_tc(TcPlan* plan, const Image& img, const Tile* tiles, const int32_t* n_tiles,
                           int max_tiles, __half* pairs16, int32_t* status, cudaStream_t st,
                           const int32_t* rowmap = nullptr, const int32_t* map_base = nullptr);

// plain GEMM over the expert-sorted activations (no activation function): z16[row][n_mtiles*128] =
// W x_sorted[row], for images whose rows are not gate/up pairs (hgn v2 i4r gate_up).
cudaError_t launch_raw_tc(TcPlan* plan, const Image& img, const Tile* tiles, const int32_t* n_tiles,
                          int max_tiles, __half* z16, int32_t* status, cudaStream_t st);

}  // namespace b200moe
