// Error plumbing, device status word and small host utilities shared by every entry point.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace flymoe {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* where, cudaError_t err) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorString(err),
           cudaGetErrorName(err));
}
void set_last_error_msg(const char* msg) { snprintf(g_last_error, sizeof(g_last_error), "%s", msg); }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Set by kernels whose bounded waits gave up; read and cleared by flymoe_device_status().
__device__ int g_device_status = 0;

// Device address of the status word for the current device (kernels in other
// translation units receive it as a parameter).
int* device_status_ptr() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

}  // namespace flymoe

extern "C" {

int flymoe_abi_version(void) { return FLYMOE_ABI_VERSION; }

const char* flymoe_error_string(int code) {
  switch (code) {
    case FLYMOE_OK: return "ok";
    case FLYMOE_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FLYMOE_ERR_CUDA: return "CUDA error";
    case FLYMOE_ERR_UNSUPPORTED: return "unsupported configuration";
    case FLYMOE_ERR_WORKSPACE: return "workspace too small";
    case FLYMOE_ERR_DEVICE_TIMEOUT: return "a device-side bounded wait gave up";
    default: return "unknown error";
  }
}

const char* flymoe_last_error(void) { return flymoe::g_last_error; }

int flymoe_device_status(int* status_out) {
  int* p = flymoe::device_status_ptr();
  if (p == nullptr) {
    flymoe::set_last_error_msg("flymoe_device_status: no CUDA device");
    return FLYMOE_ERR_CUDA;
  }
  int v = 0;
  FLYMOE_CUDA_CHECK(cudaDeviceSynchronize());
  FLYMOE_CUDA_CHECK(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) FLYMOE_CUDA_CHECK(cudaMemset(p, 0, sizeof(int)));
  if (status_out) *status_out = v;
  return FLYMOE_OK;
}

}  // extern "C"
