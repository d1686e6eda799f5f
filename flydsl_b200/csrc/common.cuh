// Shared device/host helpers for the flymoe sm_100a library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/flymoe.h"

namespace flymoe {

// ---- host-side error plumbing -------------------------------------------------------
// Last CUDA runtime/driver error text seen by this thread (returned by flymoe_last_error).
void set_last_error(const char* where, cudaError_t err);
void set_last_error_msg(const char* msg);

#define FLYMOE_CUDA_CHECK(expr)                                   \
  do {                                                            \
    cudaError_t _e = (expr);                                      \
    if (_e != cudaSuccess) {                                      \
      ::flymoe::set_last_error(#expr, _e);                        \
      return FLYMOE_ERR_CUDA;                                     \
    }                                                             \
  } while (0)

#define FLYMOE_REQUIRE(cond, msg)                                 \
  do {                                                            \
    if (!(cond)) {                                                \
      ::flymoe::set_last_error_msg(msg);                          \
      return FLYMOE_ERR_INVALID_ARGUMENT;                         \
    }                                                             \
  } while (0)

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int* device_status_ptr();  // device address of the per-device status word (nullptr on failure)
int sm_count();  // multiprocessor count of the current device (cached per device)

// ---- packed sorted-id format ----------------------------------------------------------
// id = (slot << 24) | token ; padding rows carry token == num_tokens.
__host__ __device__ __forceinline__ int id_token(int id) { return id & 0x00FFFFFF; }
__host__ __device__ __forceinline__ int id_slot(int id) { return (id >> 24) & 0xFF; }

// ---- small device utilities -----------------------------------------------------------
__device__ __forceinline__ float fp8_e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Two floats -> two e4m3 codes (round-to-nearest-even, saturating), low byte = a.
__device__ __forceinline__ uint16_t float2_to_e4m3x2(float a, float b) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(a), "f"(b));
  return r;
}

__device__ __forceinline__ uint32_t float4_to_e4m3x4(float a, float b, float c, float d) {
  return uint32_t(float2_to_e4m3x2(a, b)) | (uint32_t(float2_to_e4m3x2(c, d)) << 16);
}

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace flymoe
