// Top-k softmax gating: one warp per token, logits held in registers, warp-shuffle
// reductions for max / sum / argmax.  Selection is made on the raw fp32 logits
// (order-equivalent to exact softmax) with ties resolved to the lower expert id, so
// the chosen indices do not depend on the exp() implementation.
#include <math_constants.h>

#include "common.cuh"

namespace flymoe {

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(__ldg(p)); }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(__ldg(p));
}

constexpr int kGatingWarpsPerBlock = 4;

// VPL = logits per lane; expert e lives in lane (e % 32), register (e / 32).
template <int VPL, typename T>
__global__ void __launch_bounds__(kGatingWarpsPerBlock * 32)
topk_gating_softmax_kernel(const T* __restrict__ gating, float* __restrict__ topk_weights,
                           int* __restrict__ topk_indices, int* __restrict__ token_expert_indices,
                           int num_tokens, int num_experts, int topk, int renormalize) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kGatingWarpsPerBlock + (threadIdx.x >> 5);
  if (token >= num_tokens) return;
  const T* row = gating + size_t(token) * num_experts;

  float v[VPL];
  float vmax = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = i * 32 + lane;
    v[i] = (e < num_experts) ? load_as_float<T>(row + e) : -CUDART_INF_F;
    vmax = fmaxf(vmax, v[i]);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));

  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = i * 32 + lane;
    if (e < num_experts) sum += expf(v[i] - vmax);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);

  // k rounds of arg-max; lane j keeps the j-th pick.
  uint32_t taken = 0;
  float my_val = 0.f;
  int my_idx = 0;
  for (int round = 0; round < topk; ++round) {
    float bv = -CUDART_INF_F;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int e = i * 32 + lane;
      const bool ok = (e < num_experts) && !((taken >> i) & 1u);
      if (ok && (bi == 0x7fffffff || v[i] > bv)) { bv = v[i]; bi = e; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      const bool other_valid = oi != 0x7fffffff;
      const bool mine_valid = bi != 0x7fffffff;
      if (other_valid && (!mine_valid || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (bi != 0x7fffffff && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (lane == round) { my_val = bv; my_idx = bi; }
  }

  float p = (lane < topk) ? expf(my_val - vmax) / sum : 0.f;
  float psum = p;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
  if (renormalize) p = p / fmaxf(psum, 1e-20f);

  if (lane < topk) {
    const size_t o = size_t(token) * topk + lane;
    topk_weights[o] = p;
    topk_indices[o] = my_idx;
    token_expert_indices[o] = lane * num_tokens + token;
  }
}

template <typename T>
static int launch_gating(const void* gating, float* w, int* idx, int* tei, int T_, int E, int k,
                         int renorm, cudaStream_t stream) {
  const int vpl = ceil_div(E, 32);
  dim3 grid(ceil_div(T_, kGatingWarpsPerBlock)), block(kGatingWarpsPerBlock * 32);
  const T* g = static_cast<const T*>(gating);
#define FLYMOE_GATING_CASE(V)                                                                    \
  topk_gating_softmax_kernel<V, T><<<grid, block, 0, stream>>>(g, w, idx, tei, T_, E, k, renorm)
  if (vpl <= 1) FLYMOE_GATING_CASE(1);
  else if (vpl <= 2) FLYMOE_GATING_CASE(2);
  else if (vpl <= 4) FLYMOE_GATING_CASE(4);
  else if (vpl <= 8) FLYMOE_GATING_CASE(8);
  else if (vpl <= 16) FLYMOE_GATING_CASE(16);
  else FLYMOE_GATING_CASE(32);
#undef FLYMOE_GATING_CASE
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

}  // namespace flymoe

extern "C" int flymoe_topk_gating_softmax(const void* gating, int gating_dtype, float* topk_weights,
                                          int32_t* topk_indices, int32_t* token_expert_indices,
                                          int num_tokens, int num_experts, int topk, int renormalize,
                                          void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(num_tokens >= 0, "gating: num_tokens < 0");
  FLYMOE_REQUIRE(num_experts >= 1 && num_experts <= 1024, "gating: num_experts must be in [1, 1024]");
  FLYMOE_REQUIRE(topk >= 1 && topk <= 32 && topk <= num_experts, "gating: topk must be in [1, min(32, E)]");
  if (num_tokens == 0) return FLYMOE_OK;
  FLYMOE_REQUIRE(gating && topk_weights && topk_indices && token_expert_indices, "gating: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (gating_dtype) {
    case FLYMOE_F32:
      return launch_gating<float>(gating, topk_weights, topk_indices, token_expert_indices, num_tokens,
                                  num_experts, topk, renormalize, s);
    case FLYMOE_F16:
      return launch_gating<__half>(gating, topk_weights, topk_indices, token_expert_indices, num_tokens,
                                   num_experts, topk, renormalize, s);
    case FLYMOE_BF16:
      return launch_gating<__nv_bfloat16>(gating, topk_weights, topk_indices, token_expert_indices,
                                          num_tokens, num_experts, topk, renormalize, s);
    default:
      set_last_error_msg("gating: dtype must be F32, F16 or BF16");
      return FLYMOE_ERR_INVALID_ARGUMENT;
  }
}
