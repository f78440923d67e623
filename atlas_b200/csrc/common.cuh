// Shared device-side helpers for the sm_100a kernel library: mbarrier (bounded waits), TMA bulk-tensor
// loads, tcgen05 / TMEM wrappers, descriptor builders, small numeric utilities.
//
// Every wait in this library is bounded: a poll loop gives up after a fixed number of iterations, records
// where it gave up in a global status word and lets the CTA finish (TMEM is still released), so a
// logic error shows up as an error code on the host instead of a GPU that stops answering.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdlib>
#include <map>
#include <mutex>
#include <stdint.h>
#include <utility>

#define ATLAS_DEVICE __device__ __forceinline__

namespace atlas {

// ----------------------------------------------------------------------------- status word
// One 64-bit word per process: bits [0,8) error class, [8,32) site id, [32,64) detail (block index).
enum StatusCode : uint32_t {
  kOk = 0,
  kMbarTimeout = 1,     // an mbarrier wait ran out of polls
  kFlagTimeout = 2,     // a wait on a peer / semaphore flag ran out of polls
  kBoundsError = 3,     // an index check failed; the access was skipped
};

// The word lives in device global memory owned by the host library (one per device) and is passed to every
// kernel that can wait.
typedef unsigned long long status_t;

ATLAS_DEVICE void report_status(status_t* status, uint32_t code, uint32_t site) {
  unsigned long long v = (unsigned long long)code | ((unsigned long long)(site & 0xFFFFFFu) << 8) |
                         ((unsigned long long)blockIdx.x << 32);
  if (status) atomicCAS(status, 0ull, v);   // keep the first failure
}

// ----------------------------------------------------------------------------- misc
ATLAS_DEVICE uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

ATLAS_DEVICE uint32_t lane_id() { return threadIdx.x & 31; }

ATLAS_DEVICE bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

ATLAS_DEVICE void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ----------------------------------------------------------------------------- mbarrier
ATLAS_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
ATLAS_DEVICE void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }

ATLAS_DEVICE void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
ATLAS_DEVICE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
ATLAS_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait budget in SM clock cycles (about a second at ~2 GHz): far beyond any healthy wait, still finite.
constexpr long long kMbarMaxCycles = 2000ll * 1000ll * 1000ll;

// Bounded wait. `abort_flag` lives in shared memory; once any role sets it every waiter returns false.
ATLAS_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, status_t* status,
                            uint32_t site) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15u) == 15u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kMbarMaxCycles) break;
    }
  }
  *abort_flag = 1u;
  report_status(status, kMbarTimeout, site);
  return false;
}

// ----------------------------------------------------------------------------- TMA (no multicast anywhere)
ATLAS_DEVICE void tma_prefetch_desc(const CUtensorMap* d) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(d)) : "memory");
}

// 2-D tiled load global -> shared, completion on `bar` (tx bytes). c0 = innermost coordinate.
ATLAS_DEVICE void tma_load_2d(void* smem_dst, const CUtensorMap* desc, uint64_t* bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
ATLAS_DEVICE void tma_load_3d(void* smem_dst, const CUtensorMap* desc, uint64_t* bar, int32_t c0, int32_t c1,
                              int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2)
      : "memory");
}
// L2 prefetch of a tile (no shared memory, no completion tracking): pulls HBM data towards L2 ahead of the load.
ATLAS_DEVICE void tma_prefetch_l2_2d(const CUtensorMap* desc, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n" ::"l"(reinterpret_cast<uint64_t>(desc)),
               "r"(c0), "r"(c1)
               : "memory");
}
ATLAS_DEVICE void bulk_prefetch_l2(const void* gptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(reinterpret_cast<uint64_t>(gptr)), "r"(bytes) : "memory");
}
// 2-D tiled store shared -> global (bulk async group).
ATLAS_DEVICE void tma_store_2d(const CUtensorMap* desc, const void* smem_src, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(
                   reinterpret_cast<uint64_t>(desc)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
ATLAS_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
template <int N>
ATLAS_DEVICE void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
template <int N>
ATLAS_DEVICE void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;\n" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------- tcgen05 / TMEM
ATLAS_DEVICE void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
ATLAS_DEVICE void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
ATLAS_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {        // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
ATLAS_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
ATLAS_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.  kind::f16 covers bf16/fp16, kind::f8f6f4 covers e4m3.
ATLAS_DEVICE void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
ATLAS_DEVICE void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` when all MMAs issued so far by this thread have completed.
ATLAS_DEVICE void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
               : "memory");
}

// TMEM -> registers: 32 lanes x 32 consecutive fp32 columns (one row per thread of the warp).
ATLAS_DEVICE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
ATLAS_DEVICE void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
ATLAS_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// ----------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of exactly 128 bytes with the
// 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B and a 128-byte inner box produces).
// Rows are grouped by 8 (1024-byte swizzle atoms): stride-byte-offset = 1024; the leading-byte-offset is
// unused for swizzled K-major layouts.  Bits [46,48) = 1 marks the sm_100 descriptor version; bits
// [61,64) = 2 selects SWIZZLE_128B.  The tile base must be 1024-byte aligned; advancing along K inside
// the 128-byte row is done by adding the byte offset (>>4) to the start-address field.
ATLAS_DEVICE uint64_t make_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address, 14 bits
  d |= (uint64_t)1 << 16;                               // LBO (ignored)
  d |= (uint64_t)(1024 >> 4) << 32;                     // SBO = 1024 B
  d |= (uint64_t)1 << 46;                               // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 / kind::f8f6f4, fp32 accumulate, both operands K-major.
// a/b format: kind::f16 -> 0 = f16, 1 = bf16; kind::f8f6f4 -> 0 = e4m3, 1 = e5m2.
ATLAS_DEVICE constexpr uint32_t make_idesc(uint32_t m, uint32_t n, uint32_t ab_format) {
  return (1u << 4)                 // c_format = f32
         | (ab_format << 7)        // a_format
         | (ab_format << 10)       // b_format
         | (0u << 15) | (0u << 16) // a_major, b_major = K
         | ((n >> 3) << 17)        // n_dim
         | ((m >> 4) << 24);       // m_dim
}

// ----------------------------------------------------------------------------- numerics
ATLAS_DEVICE float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
ATLAS_DEVICE uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
ATLAS_DEVICE float fp8_e4m3_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
ATLAS_DEVICE uint8_t f32_to_fp8_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
ATLAS_DEVICE float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
ATLAS_DEVICE float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}


// ----------------------------------------------------------------------------- programmatic dependent launch
// A kernel launched with launch_chain() may start while its predecessor in the stream is still running: its on-chip
// prologue (barrier init, TMEM allocation, descriptor prefetch) and the launch latency overlap the predecessor's tail.
// chain_wait() blocks until the predecessor grid has completed and its memory operations are visible, so every global
// memory access of such a kernel comes after it; chain_trigger() lets the next kernel in the stream start launching.
// A kernel launched the ordinary way is unaffected by either instruction.
// Thread-block cluster barrier (every thread of every CTA of the cluster takes part, like __syncthreads for the
// cluster) and a store into the shared memory of another CTA of the cluster.  The arrive has release, the wait acquire
// semantics at cluster scope, so distributed-shared-memory stores before the arrive are visible after the wait.
ATLAS_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
ATLAS_DEVICE uint32_t cluster_map_shared(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank));
  return r;
}
ATLAS_DEVICE void st_cluster_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

ATLAS_DEVICE void chain_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
ATLAS_DEVICE void chain_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// The dynamic shared-memory limit of a kernel is a per-device attribute: remember what was set for every
// (kernel, device) pair so that a process driving several GPUs raises it on each of them.
inline cudaError_t ensure_dynamic_smem(const void* kern, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  int& have = done[std::make_pair(kern, dev)];
  if (have >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) have = bytes;
  return e;
}

inline bool chain_enabled() {
  static const bool on = [] {
    const char* e = getenv("ATLAS_PDL");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

// `early` false launches the ordinary way (prefill-size work gains nothing from an early start and measured ~0.5 % slower).
template <typename... P, typename... A>
inline cudaError_t launch_chain_if(bool early, void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                   A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (early && chain_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}
// The same for a grid of thread-block clusters of `cluster_x` CTAs along x (grid.x a multiple of it).
template <typename... P, typename... A>
inline cudaError_t launch_chain_cluster(bool early, unsigned cluster_x, void (*kern)(P...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t st, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (early && chain_enabled()) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}
template <typename... P, typename... A>
inline cudaError_t launch_chain(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... args) {
  return launch_chain_if(true, kern, grid, block, smem, st, args...);
}

}  // namespace atlas
