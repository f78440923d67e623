// Mixture-of-experts support kernels around the grouped tcgen05 GEMM (gemm.cu, grouped mode):
//   moe_route_kernel    router logits -> softmax / sigmoid scores -> top-k ids + (re)normalised weights
//   moe_align_kernel    per-expert histogram, 128-row padded segment offsets, row slot of every (token, k) pair,
//                       m-tile -> expert worklist and the live tile count (all on device: graph-capturable)
//   moe_gather_kernel   expert-sorted activation rows (bf16 copy, or FP8 + k-group-major scales)
//   moe_combine_kernel  out[t] = sum_j w[t,j] * y[slot(t,j)]  (+ optional addend, e.g. shared expert / residual)
// Reference ops replaced: kernels/gb10/common/{moe_topk,moe_topk_sigmoid,moe_permute}.cu
// (moe_count_experts, moe_sort_by_expert, moe_permute_tokens, moe_build_tile_worklist, moe_unpermute_reduce).
#include "common.cuh"
#include "host_api.h"

namespace atlas {

// Router options beyond plain top-k of softmax / sigmoid scores (all optional):
//   score_mode 2   sqrt(softplus(logit)) scores
//   sel_bias       per-expert correction added for SELECTION only; weights come from the unbiased scores
//   n_group / topk_group   group-limited routing: experts split into n_group equal groups, a group scores the sum of
//                  its two best (score + bias), only the topk_group best groups stay eligible
//   hash_table     static selection: expert ids of token id `tok` are hash_table[tok * k ...]; scores still weight them
//   out_scale      factor on the final weights (routed_scaling_factor)
// Reference ops replaced: kernels/gb10/common/{moe_topk_sqrtsoftplus,moe_topk_softmax_bias,moe_hash_route,moe_gate_topk}.cu
struct RouteOpts {
  int score_mode;            // 0 softmax, 1 sigmoid, 2 sqrt-softplus
  const float* sel_bias;     // [E] or null
  int n_group, topk_group;   // 0 / 0 = off
  const int* hash_table;     // [vocab, k] or null
  const int* token_ids;      // [T] (with hash_table)
  float out_scale;
};

__device__ __forceinline__ float route_score(float x, float mx, int mode) {
  if (mode == 1) return 1.f / (1.f + __expf(-x));
  if (mode == 2) return sqrtf(x > 20.f ? x : log1pf(__expf(x)));
  return __expf(x - mx);
}

// one warp per token; E <= 1024
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ logits, long long ld, int T_, int E, int k, int norm, RouteOpts o,
                 float* __restrict__ w_out, int* __restrict__ id_out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= T_) return;
  constexpr int kMaxPer = 32;
  float v[kMaxPer];            // unbiased scores (weights)
  float sel[kMaxPer];          // selection keys
  const int per = (E + 31) / 32;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int e = i * 32 + lane;
    v[i] = (i < per && e < E) ? (float)logits[t * ld + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    if (i < per && v[i] > -INFINITY) {
      v[i] = route_score(v[i], mx, o.score_mode);
      sum += o.score_mode == 0 ? v[i] : 0.f;
    }
  }
  sum = warp_sum(sum);
  const float inv = o.score_mode == 0 ? 1.f / sum : 1.f;
  // selection keys: the normalised score plus the selection-only correction
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int e = i * 32 + lane;
    sel[i] = (i < per && e < E && v[i] > -INFINITY) ? v[i] * inv + (o.sel_bias ? o.sel_bias[e] : 0.f) : -INFINITY;
  }

  if (o.hash_table != nullptr) {
    // static selection: lane j < k owns pick j and scores its expert straight from the logits row
    const int tok = o.token_ids[t];
    int my_e = lane < k ? o.hash_table[(long long)tok * k + lane] : 0;
    my_e = min(max(my_e, 0), E - 1);
    const float my_w = lane < k ? route_score((float)logits[t * ld + my_e], mx, o.score_mode) * inv : 0.f;
    float wsum = warp_sum(lane < k ? my_w : 0.f);
    if (lane < k) {
      w_out[(long long)t * k + lane] = (norm ? my_w / (wsum + 1e-20f) : my_w) * o.out_scale;
      id_out[(long long)t * k + lane] = my_e;
    }
    return;
  }

  if (o.n_group > 1 && o.topk_group > 0 && o.topk_group < o.n_group) {
    const int gsz = E / o.n_group;
    float my_g = -INFINITY;                    // lane g holds the score of group g
#pragma unroll 1
    for (int g = 0; g < o.n_group; ++g) {
      float a = -INFINITY, b = -INFINITY;      // two best of the group seen by this lane
#pragma unroll
      for (int i = 0; i < kMaxPer; ++i) {
        const int e = i * 32 + lane;
        if (i < per && e < E && e / gsz == g) {
          const float x = sel[i];
          if (x > a) { b = a; a = x; } else if (x > b) { b = x; }
        }
      }
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, sft), ob = __shfl_xor_sync(0xffffffffu, b, sft);
        const float hi = fmaxf(a, oa), lo = fmaxf(fminf(a, oa), fmaxf(b, ob));
        a = hi; b = lo;
      }
      if (lane == g) my_g = a + (gsz > 1 ? b : 0.f);
    }
    unsigned keep = 0;
    for (int j = 0; j < o.topk_group; ++j) {
      float best = my_g;
      int bg = lane;
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, sft);
        const int og = __shfl_xor_sync(0xffffffffu, bg, sft);
        if (ob > best || (ob == best && og < bg)) { best = ob; bg = og; }
      }
      keep |= 1u << bg;
      if (lane == bg) my_g = -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      const int e = i * 32 + lane;
      if (i < per && e < E && !((keep >> (e / gsz)) & 1u)) sel[i] = -INFINITY;
    }
  }

  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY, bw = 0.f;
    int bi = 0x7FFFFFFF;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      const int e = i * 32 + lane;
      if (i < per && e < E && (sel[i] > best)) { best = sel[i]; bi = e; bw = v[i]; }
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, sft);
      const float ow = __shfl_xor_sync(0xffffffffu, bw, sft);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, sft);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; bw = ow; }
    }
    // remove the winner (ties resolve to the lowest expert id)
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kMaxPer; ++i)
        if (i == (bi >> 5)) sel[i] = -INFINITY;
    }
    const float pw = bw * inv;
    wsum += pw;
    if (lane == j) { my_w = pw; my_id = bi; }
  }
  if (lane < k) {
    w_out[(long long)t * k + lane] = (norm ? my_w / fmaxf(wsum, 1e-20f) : my_w) * o.out_scale;
    id_out[(long long)t * k + lane] = my_id;
  }
}

// Single CTA (1024 threads).  counts/offsets live in shared memory (E <= 1024).
// slot_of[t*k+j] = row in the expert-sorted buffer, or -1 for experts outside [e_lo, e_lo + E_local).
// The per-expert tile counts are prefix-summed by the whole block (one expert per thread, log-step scan).  A pair whose
// row would fall beyond max_rows is dropped and recorded as a bounds error in the status word.
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ topk_ids, int n_pairs, int e_lo, int E_local, int* __restrict__ slot_of,
                 int* __restrict__ row_token, int* __restrict__ tile_expert, int* __restrict__ num_tiles,
                 int max_rows, int k, status_t* status) {
  __shared__ int counts[1024];
  __shared__ int scan[2][1024];
  __shared__ int cursor[1024];
  const int tid = threadIdx.x;
  counts[tid] = 0;
  cursor[tid] = 0;
  __syncthreads();
  for (int i = tid; i < n_pairs; i += blockDim.x) {
    const int e = topk_ids[i] - e_lo;
    if (e >= 0 && e < E_local) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  const int my_tiles = tid < E_local ? (counts[tid] + 127) >> 7 : 0;
  int cur = 0;
  scan[0][tid] = my_tiles;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {               // inclusive scan of the tile counts
    const int v = scan[cur][tid] + (tid >= d ? scan[cur][tid - d] : 0);
    scan[cur ^ 1][tid] = v;
    cur ^= 1;
    __syncthreads();
  }
  const int tile0 = scan[cur][tid] - my_tiles;        // exclusive prefix = first tile of this expert
  const int max_tiles = max_rows >> 7;
  for (int i = 0; i < my_tiles; ++i)
    if (tile0 + i < max_tiles) tile_expert[tile0 + i] = tid;
  if (tid == 1023) {
    const int tiles = scan[cur][1023];
    if (tiles > max_tiles) report_status(status, kBoundsError, 0x700);
    *num_tiles = min(tiles, max_tiles);
  }
  for (int r = tid; r < max_rows; r += blockDim.x) row_token[r] = -1;
  __syncthreads();
  // Rank inside an expert: pairs are visited in index order by a fixed thread, but threads race on the cursor;
  // the row order inside an expert does not change any row's result, and the combine sums in fixed k order.
  for (int i = tid; i < n_pairs; i += blockDim.x) {
    const int e = topk_ids[i] - e_lo;
    int slot = -1;
    if (e >= 0 && e < E_local) {
      slot = ((scan[cur][e] - ((counts[e] + 127) >> 7)) << 7) + atomicAdd(&cursor[e], 1);
      if (slot < max_rows) row_token[slot] = i / k;
      else { slot = -1; report_status(status, kBoundsError, 0x701); }
    }
    slot_of[i] = slot;
  }
}

// xs[row] = x[row_token[row]] ; optional FP8 group quantisation (scales k-group major over sorted rows)
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ row_token,
                  const int* __restrict__ num_tiles, int H, __nv_bfloat16* y, uint8_t* q, float* scale, long long scale_ld) {
  const int row = blockIdx.x;         // rows on grid.x: row counts can exceed the 65535 limit of grid.y
  if (row >= (*num_tiles) * 128) return;
  const int t = row_token[row];
  const int e = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const bool live = e < H;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live && t >= 0) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + t * ldx + e);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  if (q) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (live) {
      const float sc = fmaxf(amax, 1e-10f) / 448.f;
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t acc = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc |= (uint32_t)f32_to_fp8_e4m3(__fdiv_rn(v[h * 4 + i], sc)) << (8 * i);
        w[h] = acc;
      }
      *reinterpret_cast<uint2*>(q + (long long)row * H + e) = make_uint2(w[0], w[1]);
      if ((threadIdx.x & 15) == 0) scale[(long long)(e >> 7) * scale_ld + row] = sc;
    }
  } else if (live) {
    uint4 out;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(y + (long long)row * H + e) = out;
  }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const int* __restrict__ slot_of,
                   const float* __restrict__ topk_w, int k, int H, const __nv_bfloat16* addend, long long ld_add,
                   __nv_bfloat16* out, long long ldo) {
  const int t = blockIdx.x;
  const int e = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (e >= H) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < k; ++j) {
    const int slot = slot_of[t * k + j];
    if (slot < 0) continue;
    const float w = topk_w[t * k + j];
    const uint4 raw = *reinterpret_cast<const uint4*>(y + (long long)slot * ldy + e);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); acc[2 * i] += w * f.x; acc[2 * i + 1] += w * f.y; }
  }
  if (addend) {
    const uint4 raw = *reinterpret_cast<const uint4*>(addend + (long long)t * ld_add + e);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
  }
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  *reinterpret_cast<uint4*>(out + (long long)t * ldo + e) = o;
}

// ---------------------------------------------------------------------------- expert-parallel dispatch
// Rank r owns experts [r * experts_per_rank, (r + 1) * experts_per_rank).  One block: histogram of destination ranks
// over all (token, k) pairs, prefix sums -> send_off[world + 1], and the position of every pair inside its
// destination's segment (pos[pair]).  Positions come from shared-memory cursors, so the order inside a segment is
// arbitrary; nothing downstream depends on it (results are summed per token in k order).
__global__ void __launch_bounds__(1024)
moe_dispatch_prep_kernel(const int* __restrict__ topk_ids, int pairs, int experts_per_rank, int world,
                         int* __restrict__ send_off, int* __restrict__ pos) {
  __shared__ int cnt[8], cursor[8];
  if (threadIdx.x < 8) cnt[threadIdx.x] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int d = min(max(topk_ids[p] / experts_per_rank, 0), world - 1);
    atomicAdd(&cnt[d], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int d = 0; d < world; ++d) { send_off[d] = off; cursor[d] = off; off += cnt[d]; }
    send_off[world] = off;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int d = min(max(topk_ids[p] / experts_per_rank, 0), world - 1);
    pos[p] = atomicAdd(&cursor[d], 1);
  }
}

// send row layout: H bf16 activations followed by a 16-byte trailer {expert id, 0, 0, 0}
__global__ void __launch_bounds__(256)
moe_dispatch_pack_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ topk_ids,
                         const int* __restrict__ pos, int k, int H, uint8_t* __restrict__ send, int row_bytes) {
  const int pair = blockIdx.x;
  const int t = pair / k;
  uint8_t* dst = send + (size_t)pos[pair] * row_bytes;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * ldx);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = src[i];
  if (threadIdx.x == 0) *reinterpret_cast<int4*>(dst + (size_t)H * 2) = make_int4(topk_ids[pair], 0, 0, 0);
}

// expert ids of the received rows; rows past the live count (recv_off[world]) get -1 so that they take no work
__global__ void __launch_bounds__(256)
moe_recv_ids_kernel(const uint8_t* __restrict__ recv, int row_bytes, int H, const int* __restrict__ recv_off, int world,
                    int cap_rows, int* __restrict__ ids) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= cap_rows) return;
  ids[r] = r < recv_off[world] ? *reinterpret_cast<const int*>(recv + (size_t)r * row_bytes + (size_t)H * 2) : -1;
}

}  // namespace atlas

using namespace atlas;

static int route_launch(const void* logits, long long ld, int is_bf16, int T, int E, int k, int norm, RouteOpts o,
                        float* w_out, int* id_out, void* stream) {
  if (T <= 0) return 0;
  if (E > 1024 || k > 32 || k > E) return -1;
  if (o.n_group > 1 && (o.n_group > 32 || E % o.n_group)) return -1;
  if (o.hash_table && !o.token_ids) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = (T + 3) / 4;
  if (is_bf16) moe_route_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, T, E, k, norm, o, w_out, id_out);
  else moe_route_kernel<float><<<grid, 128, 0, st>>>(reinterpret_cast<const float*>(logits), ld, T, E, k, norm, o, w_out, id_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_moe_route(const void* logits, long long ld, int is_bf16, int T, int E, int k, int norm, int sigmoid,
                               float* w_out, int* id_out, void* stream) {
  RouteOpts o = {};
  o.score_mode = sigmoid ? 1 : 0;
  o.out_scale = 1.f;
  return route_launch(logits, ld, is_bf16, T, E, k, norm, o, w_out, id_out, stream);
}

extern "C" int atlas_moe_route_ex(const void* logits, long long ld, int is_bf16, int T, int E, int k, int norm, int score_mode,
                                  const float* sel_bias, int n_group, int topk_group, const int* hash_table,
                                  const int* token_ids, float out_scale, float* w_out, int* id_out, void* stream) {
  RouteOpts o = {};
  o.score_mode = score_mode; o.sel_bias = sel_bias; o.n_group = n_group; o.topk_group = topk_group;
  o.hash_table = hash_table; o.token_ids = token_ids; o.out_scale = out_scale;
  return route_launch(logits, ld, is_bf16, T, E, k, norm, o, w_out, id_out, stream);
}

extern "C" int atlas_moe_align(const int* topk_ids, int T, int k, int e_lo, int E_local, int* slot_of, int* row_token,
                               int* tile_expert, int* num_tiles, int max_rows, unsigned long long* status, void* stream) {
  if (E_local > 1024 || max_rows % 128) return -1;
  moe_align_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(topk_ids, T * k, e_lo, E_local, slot_of, row_token,
                                                                          tile_expert, num_tiles, max_rows, k, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_moe_gather(const void* x, long long ldx, const int* row_token, const int* num_tiles, int max_rows,
                                int H, void* y, void* q, float* scale, long long scale_ld, void* stream) {
  if (max_rows <= 0) return 0;
  if (H % 8 || (q && H % 128)) return -1;
  dim3 grid(max_rows, (H / 8 + 255) / 256);
  moe_gather_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, row_token, num_tiles, H, reinterpret_cast<__nv_bfloat16*>(y),
      reinterpret_cast<uint8_t*>(q), scale, scale_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_moe_combine(const void* y, long long ldy, const int* slot_of, const float* topk_w, int T, int k, int H,
                                 const void* addend, long long ld_add, void* out, long long ldo, void* stream) {
  if (T <= 0) return 0;
  if (H % 8) return -1;
  dim3 grid(T, (H / 8 + 255) / 256);
  moe_combine_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(y), ldy, slot_of, topk_w, k, H, reinterpret_cast<const __nv_bfloat16*>(addend),
      ld_add, reinterpret_cast<__nv_bfloat16*>(out), ldo);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

// Expert-parallel dispatch helpers (see the kernels above).  `pairs` = T * k.
extern "C" int atlas_moe_dispatch_prep(const int* topk_ids, int pairs, int experts_per_rank, int world, int* send_off,
                                       int* pos, void* stream) {
  if (world < 1 || world > 8 || experts_per_rank < 1) return -1;
  moe_dispatch_prep_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(topk_ids, pairs, experts_per_rank, world,
                                                                                   send_off, pos);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_moe_dispatch_pack(const void* x, long long ldx, const int* topk_ids, const int* pos, int T, int k, int H,
                                       void* send, int row_bytes, void* stream) {
  if (H % 8 || row_bytes < H * 2 + 16 || row_bytes % 16) return -1;
  if (T * k == 0) return 0;
  moe_dispatch_pack_kernel<<<T * k, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, topk_ids, pos, k, H, reinterpret_cast<uint8_t*>(send), row_bytes);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_moe_recv_ids(const void* recv, int row_bytes, int H, const int* recv_off, int world, int cap_rows, int* ids,
                                  void* stream) {
  if (cap_rows <= 0) return 0;
  moe_recv_ids_kernel<<<(cap_rows + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(recv), row_bytes, H, recv_off, world, cap_rows, ids);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
