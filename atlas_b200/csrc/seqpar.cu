// Sequence-parallel glue between a row-parallel GEMM and the next column-parallel GEMM under tensor parallelism.
//
// The row-parallel GEMM (o_proj, down_proj) runs with the reduce-scatter epilogue of gemm.cu: every rank stores its bf16
// partial tiles straight into the memory of the rank that owns the row block.  The kernel here runs on the owner:
//
//   reduce   sum the partials of all ranks in rank order (they are all in local memory by now), add the residual
//            shard, store the new residual shard
//   norm     RMSNorm weight and FP8 quantisation per 128-wide group; the row's 1/rms factor is folded into the group
//            scales, so nothing has to wait for the end of the row
//   gather   FP8 rows and scales are stored into EVERY rank's gathered-activation buffer with peer stores, then one
//            flag per group of eight rows is raised at every rank
//
// The next GEMM (qkv, gate_up) reads its A operand from the gathered buffer and polls those flags in its TMA producer
// warp (gemm.cu, `a_ready`), so the all-gather overlaps that GEMM tile by tile.  Per layer half this moves
// (W-1)/W * T * H * 3 bytes per rank over NVLink (bf16 partials out, FP8 rows in) against 4 bytes for a bf16
// all-reduce, and the norm / quantisation work is done once per row instead of once per rank.
//
// All waits are bounded and report through the status word.  Data moves with ordinary peer stores only.
//
// Reference counterpart: the all-reduce after o_proj / down_proj of the tensor-parallel decoder
// (crates/spark-model/src/layers/qwen3_attention/trait_impl/prefill_inner.rs:194) followed by residual_add_rms_norm
// (kernels/gb10/common/rms_norm.cu) and per_token_group_quant_fp8.
#include "common.cuh"
#include "host_api.h"

namespace atlas {

constexpr int kSpMaxRanks = 8;
constexpr int kSpRowsPerCta = 8;          // one warp per row; also the granularity of the arrival flags
constexpr float kSpFp8Max = 448.f;

struct SpParams {
  const uint8_t* part;                  // local partial area [world][rows_cap][H] bf16
  size_t part_src_stride;               // bytes between two source ranks' regions
  const uint32_t* rs_flags;             // local [local m-tile][n_tiles][8]: epoch of the GEMM whose tile has landed
  const unsigned int* rs_state;         // [0] = epoch of the GEMM that produced the partials
  int n_tiles;                          // column tiles of that GEMM
  __nv_bfloat16* residual;              // this rank's residual shard [rows_own][H], updated in place (may be null)
  const __nv_bfloat16* norm_w;
  uint8_t* ag_q[kSpMaxRanks];           // gathered FP8 rows [T][H] on every rank
  float* ag_s[kSpMaxRanks];             // gathered scales, k-group major: scale(row, g) = ag_s[g * sa_k + row]
  __nv_bfloat16* ag_h[kSpMaxRanks];     // mode 1: gathered bf16 rows [T][H] on every rank
  uint32_t* ag_flags[kSpMaxRanks];      // one flag per 8 global rows on every rank
  unsigned int* ag_state;               // [0] epoch of the last finished gather, [1] CTAs done in this call
  status_t* status;
  long long sa_k;
  long long max_cycles;
  float eps;
  int plus_one, rank, world, H, row0, rows_own, mode;
  unsigned int* row_counters;           // per-row form: rows finished per group of eight local rows (local memory, zero between calls)
};

ATLAS_DEVICE void sp_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
ATLAS_DEVICE uint32_t sp_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
ATLAS_DEVICE bool sp_wait(const uint32_t* p, uint32_t want, status_t* status, uint32_t site, long long max_cycles) {
  const long long t0 = clock64();
  while ((int32_t)(sp_ld_acquire(p) - want) < 0) {
    if (clock64() - t0 > max_cycles) { report_status(status, kFlagTimeout, site); return false; }
    __nanosleep(20);
  }
  return true;
}

ATLAS_DEVICE void sp_unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
ATLAS_DEVICE uint4 sp_pack8(const float (&f)[8]) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return o;
}
ATLAS_DEVICE uint2 sp_quant8(const float (&f)[8], float scale) {
  const float inv = __frcp_rn(scale);
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[h * 4 + 0] * inv, f[h * 4 + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[h * 4 + 2] * inv, f[h * 4 + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    w[h] = lo | (hi << 16);
  }
  return make_uint2(w[0], w[1]);
}

// grid = ceil(rows_own / 8), 256 threads.  H % 256 == 0, H <= 16384.
__global__ void __launch_bounds__(256)
sp_reduce_norm_gather_kernel(const SpParams p) {
  __shared__ float sc_buf[kSpRowsPerCta][128];
  __shared__ float rstd_s[kSpRowsPerCta];
  __shared__ int ok_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lrow0 = blockIdx.x * kSpRowsPerCta;
  const uint32_t rs_epoch = p.rs_state[0];
  const uint32_t ag_epoch = p.ag_state[0] + 1u;
  if (tid == 0) ok_slot = 1;
  __syncthreads();
  // ---- every (column tile, source rank) partial of this row block has landed?  (a rank that owns no rows skips this)
  if (lrow0 < p.rows_own) {
    const int local_tile = lrow0 >> 7;
    const uint32_t* f = p.rs_flags + (size_t)local_tile * p.n_tiles * 8;
    for (int i = tid; i < p.n_tiles * p.world; i += blockDim.x) {
      const int src = i % p.world, nt = i / p.world;
      if (!sp_wait(f + (size_t)nt * 8 + src, rs_epoch, p.status, 0x800, p.max_cycles)) ok_slot = 0;
    }
  }
  __syncthreads();
  const bool ok = ok_slot != 0;
  const int lrow = lrow0 + warp;
  const bool live = ok && lrow < p.rows_own;
  const long long grow = (long long)p.row0 + lrow;
  float ss = 0.f;
  if (live) {
    for (int j = 0; j < p.H / 256; ++j) {
      const int e = j * 256 + lane * 8;
      uint4 raw[kSpMaxRanks];
#pragma unroll
      for (int s = 0; s < kSpMaxRanks; ++s)
        if (s < p.world)
          raw[s] = *reinterpret_cast<const uint4*>(p.part + (size_t)s * p.part_src_stride + ((size_t)lrow * p.H + e) * 2);
      float h[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < kSpMaxRanks; ++s) {            // rank order: the same bits whoever owns the row
        if (s >= p.world) break;
        float f[8];
        sp_unpack8(raw[s], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] += f[i];
      }
      if (p.residual) {
        float r[8];
        sp_unpack8(*reinterpret_cast<const uint4*>(p.residual + (size_t)lrow * p.H + e), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] += r[i];
      }
      const uint4 hb = sp_pack8(h);
      if (p.residual) *reinterpret_cast<uint4*>(p.residual + (size_t)lrow * p.H + e) = hb;
      if (p.mode == 1) {
#pragma unroll
        for (int d = 0; d < kSpMaxRanks; ++d)
          if (d < p.world) *reinterpret_cast<uint4*>(p.ag_h[d] + grow * p.H + e) = hb;
        continue;
      }
      sp_unpack8(hb, h);                                 // normalise what was stored (the rounded residual stream)
      float wv[8], hw[8];
      sp_unpack8(*reinterpret_cast<const uint4*>(p.norm_w + e), wv);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss += h[i] * h[i];
        hw[i] = h[i] * (p.plus_one ? wv[i] + 1.f : wv[i]);
        amax = fmaxf(amax, fabsf(hw[i]));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // 16 lanes = one group
      const float sc = fmaxf(amax, 1e-20f) / kSpFp8Max;
      const uint2 q = sp_quant8(hw, sc);
#pragma unroll
      for (int d = 0; d < kSpMaxRanks; ++d)
        if (d < p.world) *reinterpret_cast<uint2*>(p.ag_q[d] + grow * p.H + e) = q;
      if ((lane & 15) == 0) sc_buf[warp][j * 2 + (lane >> 4)] = sc;
    }
    if (p.mode == 0) {
      ss = warp_sum(ss);
      if (lane == 0) rstd_s[warp] = rsqrtf(ss / (float)p.H + p.eps);
    }
  }
  __syncthreads();
  if (ok && p.mode == 0) {
    // scales with the row's 1/rms folded in; eight consecutive rows of one group are 32 contiguous bytes
    const int groups = p.H >> 7;
    for (int idx = tid; idx < groups * kSpRowsPerCta; idx += blockDim.x) {
      const int g = idx / kSpRowsPerCta, r = idx % kSpRowsPerCta;
      if (lrow0 + r >= p.rows_own) continue;
      const float v = sc_buf[r][g] * rstd_s[r];
#pragma unroll
      for (int d = 0; d < kSpMaxRanks; ++d)
        if (d < p.world) p.ag_s[d][(long long)g * p.sa_k + p.row0 + lrow0 + r] = v;
    }
  }
  __syncthreads();
  // one release store per destination, after the barrier: cumulative over the whole block's stores
  if (ok && tid < p.world && lrow0 < p.rows_own) sp_st_release(p.ag_flags[tid] + ((p.row0 + lrow0) >> 3), ag_epoch);
  if (tid == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(&p.ag_state[1], 1u);
    if (done == gridDim.x - 1) {
      p.ag_state[1] = 0;
      __threadfence();
      p.ag_state[0] = ag_epoch;
    }
  }
}

// The same work with ONE ROW PER CTA (eight warps share the row's columns), for decode-size steps where a rank owns a
// few dozen rows at most and eight rows per CTA would leave the GPU to two or four CTAs.  The arrival flag of a group of
// eight rows is raised by whichever of its rows finishes last (a counter in local memory; every CTA fences its peer stores
// before it counts itself, so the last one's release covers them all).
__global__ void __launch_bounds__(256)
sp_reduce_norm_gather_row_kernel(const SpParams p) {
  __shared__ float sc_buf[128];
  __shared__ float ss_part[8];
  __shared__ int ok_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lrow = blockIdx.x;
  const uint32_t rs_epoch = p.rs_state[0];
  const uint32_t ag_epoch = p.ag_state[0] + 1u;
  if (tid == 0) ok_slot = 1;
  __syncthreads();
  const bool mine = lrow < p.rows_own;
  if (mine) {
    const uint32_t* f = p.rs_flags;                       // row-level ownership: the single m-tile's flags
    for (int i = tid; i < p.n_tiles * p.world; i += blockDim.x) {
      const int src = i % p.world, nt = i / p.world;
      if (!sp_wait(f + (size_t)nt * 8 + src, rs_epoch, p.status, 0x801, p.max_cycles)) ok_slot = 0;
    }
  }
  __syncthreads();
  const bool ok = ok_slot != 0;
  const bool live = ok && mine;
  const long long grow = (long long)p.row0 + lrow;
  float ss = 0.f;
  if (live) {
    for (int j = warp; j < p.H / 256; j += 8) {
      const int e = j * 256 + lane * 8;
      uint4 raw[kSpMaxRanks];
#pragma unroll
      for (int s = 0; s < kSpMaxRanks; ++s)
        if (s < p.world)
          raw[s] = *reinterpret_cast<const uint4*>(p.part + (size_t)s * p.part_src_stride + ((size_t)lrow * p.H + e) * 2);
      float h[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < kSpMaxRanks; ++s) {            // rank order: the same bits whoever owns the row
        if (s >= p.world) break;
        float f[8];
        sp_unpack8(raw[s], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] += f[i];
      }
      if (p.residual) {
        float r[8];
        sp_unpack8(*reinterpret_cast<const uint4*>(p.residual + (size_t)lrow * p.H + e), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] += r[i];
      }
      const uint4 hb = sp_pack8(h);
      if (p.residual) *reinterpret_cast<uint4*>(p.residual + (size_t)lrow * p.H + e) = hb;
      if (p.mode == 1) {
#pragma unroll
        for (int d = 0; d < kSpMaxRanks; ++d)
          if (d < p.world) *reinterpret_cast<uint4*>(p.ag_h[d] + grow * p.H + e) = hb;
        continue;
      }
      sp_unpack8(hb, h);                                 // normalise what was stored (the rounded residual stream)
      float wv[8], hw[8];
      sp_unpack8(*reinterpret_cast<const uint4*>(p.norm_w + e), wv);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss += h[i] * h[i];
        hw[i] = h[i] * (p.plus_one ? wv[i] + 1.f : wv[i]);
        amax = fmaxf(amax, fabsf(hw[i]));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // 16 lanes = one group
      const float sc = fmaxf(amax, 1e-20f) / kSpFp8Max;
      const uint2 q = sp_quant8(hw, sc);
#pragma unroll
      for (int d = 0; d < kSpMaxRanks; ++d)
        if (d < p.world) *reinterpret_cast<uint2*>(p.ag_q[d] + grow * p.H + e) = q;
      if ((lane & 15) == 0) sc_buf[j * 2 + (lane >> 4)] = sc;
    }
    if (p.mode == 0) {
      ss = warp_sum(ss);
      if (lane == 0) ss_part[warp] = ss;
    }
  }
  __syncthreads();
  if (live && p.mode == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += ss_part[w];          // fixed order
    const float rstd = rsqrtf(t / (float)p.H + p.eps);
    const int groups = p.H >> 7;
    for (int idx = tid; idx < groups * p.world; idx += blockDim.x) {
      const int g = idx % groups, d = idx / groups;
      p.ag_s[d][(long long)g * p.sa_k + grow] = sc_buf[g] * rstd;
    }
  }
  __syncthreads();
  if (tid == 0) {
    if (live) {
      __threadfence_system();                              // this row's peer stores, before it is counted
      const int grp = lrow >> 3;
      const unsigned int want = (unsigned int)min(kSpRowsPerCta, p.rows_own - grp * kSpRowsPerCta);
      const unsigned int seen = atomicAdd(&p.row_counters[grp], 1u);
      if (seen == want - 1u) {
        p.row_counters[grp] = 0;
        __threadfence_system();
        for (int d = 0; d < p.world; ++d) sp_st_release(p.ag_flags[d] + ((p.row0 + grp * kSpRowsPerCta) >> 3), ag_epoch);
      }
    }
    __threadfence();
    const unsigned int done = atomicAdd(&p.ag_state[1], 1u);
    if (done == gridDim.x - 1) {
      p.ag_state[1] = 0;
      __threadfence();
      p.ag_state[0] = ag_epoch;
    }
  }
}

// Blocks until every 8-row group of rows [0, T) carries the epoch in state[0] (the gather that ran last on this stream).
__global__ void __launch_bounds__(256)
sp_wait_rows_kernel(const uint32_t* flags, const unsigned int* state, int groups, status_t* status, long long max_cycles) {
  const uint32_t want = state[0];
  for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += gridDim.x * blockDim.x)
    if (!sp_wait(flags + g, want, status, 0x810, max_cycles)) return;
}

}  // namespace atlas

using namespace atlas;

// mode 0: reduce + residual + RMSNorm + FP8 quantisation, gathered to every rank (ag_q / ag_s).
// mode 1: reduce + residual, bf16 rows gathered to every rank (ag_h); norm_w unused.
// `part`, `rs_flags`, `rs_state`, `residual` are local; the ag_* arrays hold one pointer per rank (own entry = local).
// rows_own rows starting at global row `row0` belong to this rank; row0 is a multiple of 128, or, with row-level ownership
// inside a single 128-row block (decode-size steps), of 8.
extern "C" int atlas_sp_reduce_norm_gather(int mode, const void* part, size_t part_src_stride, const void* rs_flags,
                                           const unsigned int* rs_state, int n_tiles, void* residual, const void* norm_w,
                                           int plus_one, float eps, void* const* ag_q, void* const* ag_s, long long sa_k,
                                           void* const* ag_h, void* const* ag_flags, unsigned int* ag_state, int rank,
                                           int world, int H, int row0, int rows_own, long long max_cycles,
                                           unsigned long long* status, void* stream, unsigned int* row_counters) {
  if (world < 1 || world > kSpMaxRanks || H % 256 || H > 16384 || (row0 & 7)) return -1;
  if (mode != 0 && mode != 1) return -2;
  if (mode == 0 && !norm_w) return -3;
  SpParams p;
  p.part = reinterpret_cast<const uint8_t*>(part); p.part_src_stride = part_src_stride;
  p.rs_flags = reinterpret_cast<const uint32_t*>(rs_flags); p.rs_state = rs_state; p.n_tiles = n_tiles;
  p.residual = reinterpret_cast<__nv_bfloat16*>(residual); p.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  for (int i = 0; i < kSpMaxRanks; ++i) {
    p.ag_q[i] = (i < world && ag_q) ? reinterpret_cast<uint8_t*>(ag_q[i]) : nullptr;
    p.ag_s[i] = (i < world && ag_s) ? reinterpret_cast<float*>(ag_s[i]) : nullptr;
    p.ag_h[i] = (i < world && ag_h) ? reinterpret_cast<__nv_bfloat16*>(ag_h[i]) : nullptr;
    p.ag_flags[i] = i < world ? reinterpret_cast<uint32_t*>(ag_flags[i]) : nullptr;
  }
  if (mode == 0 && (!ag_q || !ag_s)) return -4;
  if (mode == 1 && !ag_h) return -4;
  p.ag_state = ag_state; p.status = status; p.sa_k = sa_k;
  p.max_cycles = max_cycles > 0 ? max_cycles : kMbarMaxCycles;
  p.eps = eps; p.plus_one = plus_one; p.rank = rank; p.world = world; p.H = H; p.row0 = row0; p.rows_own = rows_own;
  p.mode = mode;
  p.row_counters = row_counters;
  // decode-size steps (row-level ownership, row0 not on a 128-row boundary or few rows): one CTA per row
  if (row_counters != nullptr && rows_own <= 64 && H <= 128 * 128) {
    sp_reduce_norm_gather_row_kernel<<<rows_own > 0 ? rows_own : 1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -20;
  }
  // a rank that owns no rows still takes part: the epoch of its gather state must advance with everyone else's
  const int grid = rows_own > 0 ? (rows_own + kSpRowsPerCta - 1) / kSpRowsPerCta : 1;
  sp_reduce_norm_gather_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_sp_wait_rows(const void* flags, const unsigned int* state, int T, long long max_cycles,
                                  unsigned long long* status, void* stream) {
  const int groups = (T + kSpRowsPerCta - 1) / kSpRowsPerCta;
  if (groups <= 0) return 0;
  const int grid = (groups + 255) / 256;
  sp_wait_rows_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(flags), state, groups, status, max_cycles > 0 ? max_cycles : kMbarMaxCycles);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
