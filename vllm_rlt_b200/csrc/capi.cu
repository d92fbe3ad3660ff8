// Library identification, error text and per-device property cache.
#include <mutex>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace rlt {

namespace {
thread_local char g_last_error[512] = "";
constexpr int kMaxDevices = 64;
std::mutex g_info_mutex;
DeviceInfo g_info[kMaxDevices];
bool g_info_ready[kMaxDevices] = {};
}  // namespace

void set_last_error(const char* what, cudaError_t err) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorString(err),
           cudaGetErrorName(err));
}

void set_last_error_text(const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s", what);
}

int current_device_info(DeviceInfo* out) {
  int device = 0;
  RLT_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) {
    set_last_error_text("device index out of range");
    return RLT_ERR_INVALID;
  }
  std::lock_guard<std::mutex> lock(g_info_mutex);
  if (!g_info_ready[device]) {
    DeviceInfo info;
    info.device = device;
    int value = 0;
    RLT_CUDA_TRY(cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device));
    RLT_CUDA_TRY(cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, device));
    RLT_CUDA_TRY(cudaDeviceGetAttribute(&info.cc_minor, cudaDevAttrComputeCapabilityMinor, device));
    RLT_CUDA_TRY(cudaDeviceGetAttribute(&value, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    info.smem_optin = static_cast<size_t>(value);
    g_info[device] = info;
    g_info_ready[device] = true;
  }
  *out = g_info[device];
  return RLT_OK;
}

}  // namespace rlt

extern "C" RLT_API const char* rlt_version(void) { return "rlt_verify 0.1.0 sm_100a"; }

extern "C" RLT_API const char* rlt_last_error(void) { return rlt::g_last_error; }
