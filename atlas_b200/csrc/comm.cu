// Collectives over NVLink peer memory, written as plain peer loads / stores from inside kernels (no NCCL, no
// multimem, no cluster-multicast loads): every rank owns one "symmetric" allocation, exported with CUDA IPC and
// mapped by all peers, holding data slots and per-CTA signal flags.
//
//   allreduce_oneshot   each CTA publishes its slice into the local slot, raises a flag in every peer, waits for the
//                       peers' flags (bounded), then reduces the same slice straight out of all peers' slots.
//                       One barrier; every rank reads all data (best below a few MB: decode-size messages).
//   allreduce_twoshot   reduce-scatter (rank r reduces slice r out of all peers' slots and stores the result into every
//                       peer's result slot) + all-gather by those stores; two barriers, 2x less traffic per rank.
//   alltoall_rows       expert-parallel dispatch / combine: every rank stores rows into per-source regions of the
//                       destination ranks' slots (row counts first), then raises flags.
//
// Waits are bounded (about a second of SM clock): on expiry the kernel records a status word and returns, so a dead
// or late peer surfaces as an error code on the host and the CUDA context stays usable.
// Reference ops replaced: the 2-rank ncclSend/ncclRecv + bf16_add_inplace fast path
// (crates/spark-comm/src/nccl_backend.rs:381-467, kernels/gb10/common/bf16_add.cu) and ncclAllReduce itself.
#include <cstring>

#include "common.cuh"
#include "host_api.h"

namespace atlas {

constexpr int kMaxRanks = 8;
constexpr int kMaxCommBlocks = 256;
constexpr long long kFlagMaxCycles = 2000ll * 1000ll * 1000ll;

struct SymmCtx {
  uint8_t* data[kMaxRanks];        // peers' data areas (index = rank; own entry is the local pointer)
  uint32_t* flags[kMaxRanks];      // peers' flag areas: [phase(2)][block][src rank]
  int rank, world;
};

ATLAS_DEVICE void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
ATLAS_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *p has reached epoch `want`. Bounded.
ATLAS_DEVICE bool wait_flag(const uint32_t* p, uint32_t want, status_t* status, uint32_t site, long long max_cycles) {
  const long long t0 = clock64();
  while ((int32_t)(ld_acquire_sys(p) - want) < 0) {      // epochs only grow; a peer one call ahead also ends the wait
    if (clock64() - t0 > max_cycles) {
      report_status(status, kFlagTimeout, site);
      return false;
    }
    __nanosleep(20);
  }
  return true;
}

// Block-level barrier with all peers for `phase` (0/1) of this call: data stores of the whole block are made visible
// system-wide first.  Returns false when a peer did not arrive in time.
// Ordering: the block's data stores happen-before the bar.sync, and the flag stores are system-scope releases issued
// after it, so they are cumulative over the whole block's stores; one fence per signalling lane instead of one per
// thread (a system fence by all 512 threads cost ~10 us per barrier).
ATLAS_DEVICE bool peer_barrier(const SymmCtx& c, int phase, uint32_t epoch, status_t* status, long long max_cycles,
                               volatile int* ok_slot) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < c.world) st_release_sys(c.flags[t] + ((size_t)phase * kMaxCommBlocks + blockIdx.x) * kMaxRanks + c.rank, epoch);
  if (t == 0) *ok_slot = 1;
  __syncthreads();
  if (t < c.world) {
    if (!wait_flag(c.flags[c.rank] + ((size_t)phase * kMaxCommBlocks + blockIdx.x) * kMaxRanks + t, epoch, status,
                   0x500 + phase, max_cycles))
      *ok_slot = 0;
  }
  __syncthreads();
  return *ok_slot != 0;
}

ATLAS_DEVICE void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}
// Sum of vector i over all ranks' slots, in rank order (identical bits on every rank).  All peer loads are issued before
// the first add: issued one by one behind their adds they cost one NVLink round trip each (8 ranks: 35 us for 64 KiB).
ATLAS_DEVICE void sum_over_ranks(const SymmCtx& c, size_t byte_off, size_t i, float (&acc)[8]) {
  uint4 v[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < c.world) v[r] = reinterpret_cast<const uint4*>(c.data[r] + byte_off)[i];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < c.world) add_bf16x8(acc, v[r]);
}
ATLAS_DEVICE uint4 pack_bf16x8(const float (&acc)[8]) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return o;
}

// state[0] = epoch of the last finished call, state[1] = blocks finished in the current call
ATLAS_DEVICE void finish_call(unsigned int* state, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(&state[1], 1u);
    if (done == gridDim.x - 1) {
      state[1] = 0;
      __threadfence();
      state[0] = epoch;
    }
  }
}

// n8 = number of 16-byte vectors.  Slot (epoch & 1) of the data area is used so that a rank may start call e+1 while
// a slower peer still reads call e's slot; call e+2 cannot start before every peer entered call e+1.
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(const SymmCtx c, const uint4* __restrict__ in, uint4* __restrict__ out, size_t n8,
                         size_t slot_bytes, unsigned int* state, status_t* status, long long max_cycles) {
  __shared__ int ok_slot;
  const uint32_t epoch = state[0] + 1;
  const size_t per = (n8 + gridDim.x - 1) / gridDim.x;
  const size_t lo = per * blockIdx.x, hi = min(n8, lo + per);
  const size_t slot_off = (size_t)(epoch & 1u) * slot_bytes;
  uint4* mine = reinterpret_cast<uint4*>(c.data[c.rank] + slot_off);
  for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) mine[i] = in[i];
  const bool ok = peer_barrier(c, 0, epoch, status, max_cycles, &ok_slot);
  if (ok) {
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      sum_over_ranks(c, slot_off, i, acc);
      out[i] = pack_bf16x8(acc);
    }
  }
  finish_call(state, epoch);
}

// Two-shot.  Data area layout per slot: [input copy: n8 vectors][result: n8 vectors].
//   copy-in   every block stages its sub-range of the PEERS' slices into the local slot (the own slice is read from `in`)
//   reduce    rank r pulls its slice from every peer with UNROLL independent 16-byte loads per peer in flight per thread,
//             adds in rank order, writes the sum into `out` locally and pushes it into every peer's result area
//   gather    after the second barrier the other owners' slices are copied from the local result area to `out`
// Block b of every rank covers the same sub-range of every slice, so a block only needs block b of each peer (one flag
// per (phase, block, source)), and the grid covers all SMs.
template <int UNROLL>
__global__ void __launch_bounds__(512)
allreduce_twoshot_kernel(const SymmCtx c, const uint4* in, uint4* out, size_t n8,       // `in` may alias `out`
                         size_t slot_bytes, unsigned int* state, status_t* status, long long max_cycles) {
  __shared__ int ok_slot;
  const uint32_t epoch = state[0] + 1;
  const size_t slot_off = (size_t)(epoch & 1u) * slot_bytes;
  const size_t res_off = slot_off + n8 * sizeof(uint4);
  const size_t per_rank = (n8 + c.world - 1) / c.world;
  const size_t per_blk = (per_rank + gridDim.x - 1) / gridDim.x;
  const size_t step = (size_t)blockDim.x * 4;
  uint4* mine = reinterpret_cast<uint4*>(c.data[c.rank] + slot_off);
  for (int r = 0; r < c.world; ++r) {
    if (r == c.rank) continue;
    const size_t lo = r * per_rank + per_blk * blockIdx.x;
    const size_t hi = min(min(n8, (r + 1) * per_rank), lo + per_blk);
    for (size_t i0 = lo + threadIdx.x; i0 < hi; i0 += step) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { const size_t i = i0 + (size_t)u * blockDim.x; if (i < hi) v[u] = in[i]; }
#pragma unroll
      for (int u = 0; u < 4; ++u) { const size_t i = i0 + (size_t)u * blockDim.x; if (i < hi) mine[i] = v[u]; }
    }
  }
  bool ok = peer_barrier(c, 0, epoch, status, max_cycles, &ok_slot);
  if (ok) {
    const size_t lo = c.rank * per_rank + per_blk * blockIdx.x;
    const size_t hi = min(min(n8, (size_t)(c.rank + 1) * per_rank), lo + per_blk);
    for (size_t i0 = lo + threadIdx.x; i0 < hi; i0 += (size_t)blockDim.x * UNROLL) {
      uint4 v[kMaxRanks][UNROLL];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r >= c.world) break;
        const uint4* src = r == c.rank ? in : reinterpret_cast<const uint4*>(c.data[r] + slot_off);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const size_t i = i0 + (size_t)u * blockDim.x;
          if (i < hi) v[r][u] = src[i];
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const size_t i = i0 + (size_t)u * blockDim.x;
        if (i >= hi) break;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < c.world) add_bf16x8(acc, v[r][u]);              // rank order: identical bits on every rank
        const uint4 o = pack_bf16x8(acc);
        out[i] = o;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < c.world && r != c.rank) reinterpret_cast<uint4*>(c.data[r] + res_off)[i] = o;
      }
    }
  }
  ok = peer_barrier(c, 1, epoch, status, max_cycles, &ok_slot) && ok;
  if (ok) {
    const uint4* res = reinterpret_cast<const uint4*>(c.data[c.rank] + res_off);
    for (int r = 0; r < c.world; ++r) {
      if (r == c.rank) continue;
      const size_t lo = r * per_rank + per_blk * blockIdx.x;
      const size_t hi = min(min(n8, (r + 1) * per_rank), lo + per_blk);
      for (size_t i0 = lo + threadIdx.x; i0 < hi; i0 += step) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { const size_t i = i0 + (size_t)u * blockDim.x; if (i < hi) v[u] = __ldcs(res + i); }
#pragma unroll
        for (int u = 0; u < 4; ++u) { const size_t i = i0 + (size_t)u * blockDim.x; if (i < hi) out[i] = v[u]; }
      }
    }
  }
  finish_call(state, epoch);
}

// Expert-parallel combine fused with its reduction (activations replicated across the group, every rank runs its own
// experts): the weighted top-k sum of this rank's expert outputs is formed straight into the local slot (it never
// exists as a separate tensor), one flag exchange follows, and every rank then sums all ranks' partials out of their
// slots in rank order and adds the residual / shared-expert term.  One launch replaces combine + all-reduce.
//   y [rows, H] expert outputs of the expert-sorted rows, slot_of [T*k] row of each (token, choice) pair or -1 when the
//   expert lives on another rank, topk_w [T*k] router weights.
__global__ void __launch_bounds__(512)
moe_combine_allreduce_kernel(const SymmCtx c, const __nv_bfloat16* __restrict__ y, long long ldy,
                             const int* __restrict__ slot_of, const float* __restrict__ topk_w, int T, int k, int H,
                             const __nv_bfloat16* addend, long long ld_add, __nv_bfloat16* out, long long ldo,
                             size_t slot_bytes, unsigned int* state, status_t* status, long long max_cycles) {
  __shared__ int ok_slot;
  const uint32_t epoch = state[0] + 1;
  const int hv = H >> 3;                                   // 16-byte vectors per row
  const size_t n8 = (size_t)T * hv;
  const size_t per = (n8 + gridDim.x - 1) / gridDim.x;
  const size_t lo = per * blockIdx.x, hi = min(n8, lo + per);
  const size_t slot_off = (size_t)(epoch & 1u) * slot_bytes;
  uint4* mine = reinterpret_cast<uint4*>(c.data[c.rank] + slot_off);
  for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const int t = (int)(i / hv), e = (int)(i % hv) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int slot = slot_of[t * k + j];
      if (slot < 0) continue;
      const float w = topk_w[t * k + j];
      const uint4 raw = *reinterpret_cast<const uint4*>(y + (long long)slot * ldy + e);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(h[q]); acc[2 * q] += w * f.x; acc[2 * q + 1] += w * f.y; }
    }
    mine[i] = pack_bf16x8(acc);
  }
  const bool ok = peer_barrier(c, 0, epoch, status, max_cycles, &ok_slot);
  if (ok) {
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const int t = (int)(i / hv), e = (int)(i % hv) * 8;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      sum_over_ranks(c, slot_off, i, acc);
      if (addend) add_bf16x8(acc, *reinterpret_cast<const uint4*>(addend + (long long)t * ld_add + e));
      *reinterpret_cast<uint4*>(out + (long long)t * ldo + e) = pack_bf16x8(acc);
    }
  }
  finish_call(state, epoch);
}

// All-to-all of variable row counts (expert-parallel dispatch / combine).  Rank s sends rows
// [send_off[d], send_off[d+1]) of `in` to rank d; they land in d's slot at region s (capacity `region_rows`), with the
// count in the region header.  After the barrier every rank compacts its regions into `out` and writes recv_off.
__global__ void __launch_bounds__(512)
alltoall_rows_kernel(const SymmCtx c, const uint4* __restrict__ in, const int* __restrict__ send_off, uint4* __restrict__ out,
                     int* __restrict__ recv_off, int row_vecs, int region_rows, size_t slot_bytes, unsigned int* state,
                     status_t* status, long long max_cycles) {
  __shared__ int ok_slot;
  __shared__ int s_off[kMaxRanks + 1];
  const uint32_t epoch = state[0] + 1;
  const size_t slot_off = (size_t)(epoch & 1u) * slot_bytes;
  const size_t region_bytes = 16 + (size_t)region_rows * row_vecs * sizeof(uint4);
  for (int d = 0; d < c.world; ++d) {
    const int r0 = send_off[d], r1 = send_off[d + 1];
    // more rows than the destination region holds: recorded as a bounds error (the host raises), the excess is not sent
    if (r1 - r0 > region_rows && blockIdx.x == 0 && threadIdx.x == 0) report_status(status, kBoundsError, 0x511);
    const int nrows = min(r1 - r0, region_rows);
    uint8_t* region = c.data[d] + slot_off + (size_t)c.rank * region_bytes;
    if (blockIdx.x == 0 && threadIdx.x == 0) *reinterpret_cast<int*>(region) = nrows;
    uint4* dst = reinterpret_cast<uint4*>(region + 16);
    const size_t total = (size_t)nrows * row_vecs;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
      dst[i] = in[(size_t)r0 * row_vecs + i];
  }
  // every block must see every other block's stores of every peer: all blocks signal, block b waits for block b
  // of each peer, and rows were strided over blocks, so wait for ALL blocks' flags of each peer instead
  __syncthreads();
  if (threadIdx.x < c.world)
    st_release_sys(c.flags[threadIdx.x] + ((size_t)0 * kMaxCommBlocks + blockIdx.x) * kMaxRanks + c.rank, epoch);
  if (threadIdx.x == 0) ok_slot = 1;
  __syncthreads();
  for (int i = threadIdx.x; i < c.world * (int)gridDim.x; i += blockDim.x) {
    const int src = i % c.world, blk = i / c.world;
    if (!wait_flag(c.flags[c.rank] + ((size_t)0 * kMaxCommBlocks + blk) * kMaxRanks + src, epoch, status, 0x510, max_cycles))
      ok_slot = 0;
  }
  __syncthreads();
  if (ok_slot) {
    if (threadIdx.x == 0) {
      int off = 0;
      for (int s = 0; s < c.world; ++s) {
        s_off[s] = off;
        off += *reinterpret_cast<const int*>(c.data[c.rank] + slot_off + (size_t)s * region_bytes);
      }
      s_off[c.world] = off;
      if (blockIdx.x == 0)
        for (int s = 0; s <= c.world; ++s) recv_off[s] = s_off[s];
    }
    __syncthreads();
    for (int s = 0; s < c.world; ++s) {
      const uint4* src = reinterpret_cast<const uint4*>(c.data[c.rank] + slot_off + (size_t)s * region_bytes + 16);
      const size_t total = (size_t)(s_off[s + 1] - s_off[s]) * row_vecs;
      uint4* dst = out + (size_t)s_off[s] * row_vecs;
      for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = src[i];
    }
  }
  finish_call(state, epoch);
}

}  // namespace atlas

using namespace atlas;

// ---- symmetric allocation over CUDA IPC (one process per GPU)
extern "C" int atlas_symm_alloc(size_t bytes, void** ptr) {
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return -1;
  return cudaMemset(*ptr, 0, bytes) == cudaSuccess ? 0 : -2;
}
extern "C" int atlas_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int atlas_ipc_export(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return -1;
  memcpy(handle64, &h, sizeof(h));
  return (int)sizeof(h);
}
extern "C" int atlas_ipc_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}
extern "C" int atlas_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }

static SymmCtx make_ctx(void* const* data, void* const* flags, int rank, int world) {
  SymmCtx c;
  for (int i = 0; i < kMaxRanks; ++i) {
    c.data[i] = i < world ? reinterpret_cast<uint8_t*>(data[i]) : nullptr;
    c.flags[i] = i < world ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
  }
  c.rank = rank; c.world = world;
  return c;
}

// kind: 0 = one-shot, 1 = two-shot.  `n_bytes` multiple of 16; slot_bytes >= n_bytes (one-shot) / 2*n_bytes (two-shot).
extern "C" int atlas_allreduce_bf16(int kind, void* const* data, void* const* flags, int rank, int world, const void* in,
                                    void* out, size_t n_bytes, size_t slot_bytes, unsigned int* state, int blocks,
                                    unsigned long long* status, long long max_cycles, void* stream) {
  if (n_bytes == 0) return 0;
  if (n_bytes % 16 || world > kMaxRanks || blocks > kMaxCommBlocks || blocks < 1) return -1;
  if ((kind == 0 && slot_bytes < n_bytes) || (kind == 1 && slot_bytes < 2 * n_bytes)) return -2;
  SymmCtx c = make_ctx(data, flags, rank, world);
  const size_t n8 = n_bytes / 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long mc = max_cycles > 0 ? max_cycles : kFlagMaxCycles;
  if (kind == 0)
    allreduce_oneshot_kernel<<<blocks, 512, 0, st>>>(c, reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out), n8,
                                                      slot_bytes, state, status, mc);
  else if (world <= 4)
    allreduce_twoshot_kernel<4><<<blocks, 512, 0, st>>>(c, reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out),
                                                         n8, slot_bytes, state, status, mc);
  else
    allreduce_twoshot_kernel<2><<<blocks, 512, 0, st>>>(c, reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out),
                                                         n8, slot_bytes, state, status, mc);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_alltoall_rows(void* const* data, void* const* flags, int rank, int world, const void* in,
                                   const int* send_off, void* out, int* recv_off, int row_bytes, int region_rows,
                                   size_t slot_bytes, unsigned int* state, int blocks, unsigned long long* status,
                                   long long max_cycles, void* stream) {
  if (row_bytes % 16 || world > kMaxRanks || blocks > kMaxCommBlocks || blocks < 1) return -1;
  const size_t region_bytes = 16 + (size_t)region_rows * row_bytes;
  if (slot_bytes < region_bytes * world) return -2;
  SymmCtx c = make_ctx(data, flags, rank, world);
  const long long mc = max_cycles > 0 ? max_cycles : kFlagMaxCycles;
  alltoall_rows_kernel<<<blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      c, reinterpret_cast<const uint4*>(in), send_off, reinterpret_cast<uint4*>(out), recv_off, row_bytes / 16, region_rows,
      slot_bytes, state, status, mc);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

// Expert outputs -> weighted top-k sum -> sum over the expert-parallel group (+ addend) in one kernel; see
// moe_combine_allreduce_kernel.  T * H * 2 bytes must fit one slot; meant for decode-size steps.
extern "C" int atlas_moe_combine_allreduce(void* const* data, void* const* flags, int rank, int world, const void* y,
                                           long long ldy, const int* slot_of, const float* topk_w, int T, int k, int H,
                                           const void* addend, long long ld_add, void* out, long long ldo, size_t slot_bytes,
                                           unsigned int* state, int blocks, unsigned long long* status, long long max_cycles,
                                           void* stream) {
  if (T <= 0) return 0;
  if (H % 8 || world > kMaxRanks || blocks > kMaxCommBlocks || blocks < 1 || (ldy % 8) || (ldo % 8) || (addend && (ld_add % 8)))
    return -1;
  if ((size_t)T * H * 2 > slot_bytes) return -2;
  SymmCtx c = make_ctx(data, flags, rank, world);
  moe_combine_allreduce_kernel<<<blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      c, reinterpret_cast<const __nv_bfloat16*>(y), ldy, slot_of, topk_w, T, k, H, reinterpret_cast<const __nv_bfloat16*>(addend),
      ld_add, reinterpret_cast<__nv_bfloat16*>(out), ldo, slot_bytes, state, status, max_cycles > 0 ? max_cycles : kFlagMaxCycles);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
