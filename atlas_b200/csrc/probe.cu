// Measurement probe: raw tcgen05.mma throughput.  One CTA per SM issues `iters` groups of four back-to-back MMAs
// (M = 128, one 128-byte K slice per group) on a fixed, zero-filled shared-memory tile and waits for the last one; the
// host times the launch with CUDA events.  Used by `python -m atlas_b200.bench.microbench --only mma_rate` to tell an
// instruction-rate bound from an operand-feed bound in the GEMM kernels.
#include "common.cuh"
#include "host_api.h"

namespace atlas {

template <int N, bool FP8>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int iters, status_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (128 * 128 + 256 * 128) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = make_idesc(128, N, FP8 ? 0u : 1u);
    const uint32_t sa = smem_u32(smem);
    const uint64_t adesc = make_smem_desc_sw128(sa), bdesc = make_smem_desc_sw128(sa + 128 * 128);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (FP8) umma_f8(tmem_base + (it & 1) * 256, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
        else     umma_f16(tmem_base + (it & 1) * 256, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
      }
    }
    umma_commit(&bar);
    mbar_wait(&bar, 0, &abort_flag, status, 0x900);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int N, bool FP8>
static float run_rate(int iters, int grid, status_t* status, cudaStream_t st) {
  auto k = mma_rate_kernel<N, FP8>;
  constexpr int kSmem = 50 * 1024;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  k<<<grid, 128, kSmem, st>>>(iters, status);        // warm-up
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  cudaEventRecord(a, st);
  k<<<grid, 128, kSmem, st>>>(iters, status);
  cudaEventRecord(b, st);
  cudaEventSynchronize(b);
  float ms = -1.f;
  cudaEventElapsedTime(&ms, a, b);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return cudaGetLastError() == cudaSuccess ? ms : -1.f;
}

}  // namespace atlas

using namespace atlas;

// Milliseconds for `iters` x 4 MMAs per CTA (kind 0 = bf16, 1 = e4m3; n in {64, 128, 256}); negative on error.
extern "C" float atlas_probe_mma_rate(int kind, int n, int iters, int grid, unsigned long long* status, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 0) {
    if (n == 64) return run_rate<64, false>(iters, grid, status, st);
    if (n == 128) return run_rate<128, false>(iters, grid, status, st);
    if (n == 256) return run_rate<256, false>(iters, grid, status, st);
  } else {
    if (n == 64) return run_rate<64, true>(iters, grid, status, st);
    if (n == 128) return run_rate<128, true>(iters, grid, status, st);
    if (n == 256) return run_rate<256, true>(iters, grid, status, st);
  }
  return -2.f;
}
