// Library state shared by all kernels: per-device status word, device properties.
#include <cuda_runtime.h>

#include "host_api.h"

namespace {
constexpr int kMaxDevices = 16;
unsigned long long* g_status[kMaxDevices] = {nullptr};
int g_sms[kMaxDevices] = {0};
}  // namespace

extern "C" int atlas_init(int device) {
  if (device < 0 || device >= kMaxDevices) return -1;
  if (g_status[device]) return 0;
  int prev = 0;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) return -2;
  unsigned long long* p = nullptr;
  if (cudaMalloc(&p, sizeof(unsigned long long)) != cudaSuccess) return -3;
  cudaMemset(p, 0, sizeof(unsigned long long));
  g_status[device] = p;
  cudaDeviceGetAttribute(&g_sms[device], cudaDevAttrMultiProcessorCount, device);
  cudaSetDevice(prev);
  return 0;
}

extern "C" unsigned long long* atlas_status_ptr(int device) {
  return (device >= 0 && device < kMaxDevices) ? g_status[device] : nullptr;
}

extern "C" unsigned long long atlas_read_status(int device, int clear) {
  if (device < 0 || device >= kMaxDevices || !g_status[device]) return 0;
  unsigned long long v = 0;
  cudaMemcpy(&v, g_status[device], sizeof(v), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(g_status[device], 0, sizeof(v));
  return v;
}

extern "C" int atlas_num_sms(int device) {
  return (device >= 0 && device < kMaxDevices) ? g_sms[device] : 0;
}
