// Argument block shared by the grouped-GEMM kernels (both stages, both implementations).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace flymoe {

struct GemmArgs {
  // A operand: e4m3 rows of k_dim bytes; layout says how a sorted row finds its A row.
  const uint8_t* a;
  const float* scale_a;        // element (kb, row) at kb * sa_stride + row * sa_row_stride
  long long sa_stride;
  long long sa_row_stride;     // 1 for the transposed [k_dim/128, rows] layout, k_dim/128 for row-major
  int a_layout;                // FLYMOE_ROWS_*
  int a_scale_layout;          // FLYMOE_ROWS_*
  long long a_rows;            // rows addressable in `a` (bounds for the TMA descriptor)
  // B operand: e4m3 [experts, wrows, k_dim], wrows = 2*n_dim (stage 1) or n_dim (stage 2)
  const uint8_t* w;
  const float* scale_w;        // [experts, wrows/128, k_dim/128]
  // routing
  const int* sorted_ids;
  const int* sorted_expert_ids;
  const float* sorted_weights;
  const int* num_valid_ids;
  // output
  void* out;
  float* out_scale;            // stage 1, e4m3 output: [n_dim/128, out_scale_stride]
  long long out_scale_stride;
  int out_dtype;               // FLYMOE_F16 / BF16 / F32 / E4M3
  int out_layout;              // stage 1: BY_PAIR or SORTED
  int accumulate;              // stage 2: atomic add into [T, n_dim] vs store into [T*k, n_dim]
  const unsigned long long* row_dst;   // stage 2, accumulate == 0, optional: byte address of output row t*k+s
                                       // (0 = drop the row); may point into a peer GPU's memory
  int doweight;
  // FLYMOE_SCALE_BLOCK128: scale_a [k_dim/128, rows] (strided as above), scale_w [experts, wrows/128, k_dim/128];
  // FLYMOE_SCALE_PER_TOKEN: scale_a [rows] (one per activation row), scale_w [experts, wrows] (one per weight row)
  int scaling;
  int in_dtype;                // FLYMOE_E4M3, or (per-token scaling only) FLYMOE_I8 / F16 / BF16
  // sizes
  int num_tokens, topk, experts;
  int n_dim;                   // stage 1: inter_dim; stage 2: model_dim
  int k_dim;                   // stage 1: model_dim; stage 2: inter_dim
  int size_expert_ids, tile_m;
  int* status;                 // device status word (bounded waits report here)
};

int launch_gemm_simt(int stage, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_sm100(int stage, const GemmArgs& args, cudaStream_t stream);

}  // namespace flymoe
