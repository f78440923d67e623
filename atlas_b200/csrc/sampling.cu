// Token selection kernels.
//   * argmax over bf16 / fp32 logits, ties resolve to the lowest index (greedy decoding contract)
//   * temperature / top-k / top-p / min-p sampling with a caller-supplied uniform per row, exact (no sort):
//     a radix descent over the float bit patterns finds the probability threshold that realises the
//     top-k / top-p / min-p cut, ties at the threshold are kept in index order, then the token is drawn by
//     inverse CDF over the kept set in index order
//   * speculative verify/accept: longest prefix of draft tokens that equals the target's choices
// Reference ops replaced: kernels/gb10/common/argmax_bf16.cu; the host sampler of
// crates/spark-runtime/src/sampler.rs; kernels/ada/common/spec_accept_sample_ada.cu.
#include "common.cuh"
#include "host_api.h"

namespace atlas {

template <typename T> ATLAS_DEVICE float to_f32(T v);
template <> ATLAS_DEVICE float to_f32<float>(float v) { return v; }
template <> ATLAS_DEVICE float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One CTA per row.  bf16 rows whose base and leading dimension allow it are read as 16-byte vectors, four in flight per
// thread (a 128256-entry row is 256 KB: with scalar loads the kernel ran at 0.07 of the copy roofline).  Ties resolve to
// the lowest index.  `out_val` (optional) receives the row maximum, which a vocab-parallel head needs to pick the
// winning shard.
template <typename T>
__global__ void __launch_bounds__(1024)
argmax_kernel(const T* __restrict__ logits, long long ld, int V, long long* out, float* out_val) {
  const T* row = logits + (long long)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7FFFFFFF;
  int done = 0;
  if (sizeof(T) == 2 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    const uint4* row4 = reinterpret_cast<const uint4*>(row);
    const int nvec = V / 8;
    constexpr int kUnroll = 4;
    for (int i0 = threadIdx.x; i0 < nvec; i0 += blockDim.x * kUnroll) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < nvec) v[u] = __ldg(row4 + i);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i >= nvec) break;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          if (f.x > best || bi == 0x7FFFFFFF) { best = f.x; bi = i * 8 + 2 * k; }
          if (f.y > best) { best = f.y; bi = i * 8 + 2 * k + 1; }
        }
      }
    }
    done = nvec * 8;
  }
  for (int i = done + threadIdx.x; i < V; i += blockDim.x) {
    const float v = to_f32(row[i]);
    if (v > best || bi == 0x7FFFFFFF) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7FFFFFFF;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      out[blockIdx.x] = bi == 0x7FFFFFFF ? 0 : bi;
      if (out_val) out_val[blockIdx.x] = best;
    }
  }
}

// ----------------------------------------------------------------------------- sampling
ATLAS_DEVICE float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;      // every thread of every warp holds the total
}
ATLAS_DEVICE float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// One CTA per row.  probs are recomputed from logits on every pass (V floats do not fit in shared memory for
// 150k vocabularies; the row stays in L2).
template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, long long ld, int V, const float* temperature, const int* top_k,
              const float* top_p, const float* min_p, const float* uniform, long long* out) {
  __shared__ float red[32];
  __shared__ unsigned int hist_cnt[256];
  __shared__ float hist_mass[256];
  __shared__ unsigned int sh_prefix, sh_need_cnt;
  __shared__ float sh_need_mass;
  __shared__ int sh_pick;
  const int b = blockIdx.x;
  const T* row = logits + (long long)b * ld;
  const float temp = temperature[b];
  const int tid = threadIdx.x;

  // greedy rows
  if (temp <= 0.f) {
    float best = -INFINITY; int bi = 0x7FFFFFFF;
    for (int i = tid; i < V; i += blockDim.x) {
      const float v = to_f32(row[i]);
      if (v > best || bi == 0x7FFFFFFF) { best = v; bi = i; }
    }
    const float gmax = block_max(best, red);
    int cand = (best == gmax) ? bi : 0x7FFFFFFF;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int smin[32];
    __syncthreads();
    if ((tid & 31) == 0) smin[tid >> 5] = cand;
    __syncthreads();
    if (tid == 0) {
      int m = 0x7FFFFFFF;
      for (int w = 0; w < (blockDim.x >> 5); ++w) m = min(m, smin[w]);
      out[b] = m == 0x7FFFFFFF ? 0 : m;
    }
    return;
  }
  const float inv_t = 1.f / fmaxf(temp, 1e-6f);
  float lmax = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) lmax = fmaxf(lmax, to_f32(row[i]) * inv_t);
  lmax = block_max(lmax, red);
  float z = 0.f;
  for (int i = tid; i < V; i += blockDim.x) z += __expf(to_f32(row[i]) * inv_t - lmax);
  z = block_sum(z, red);
  const float inv_z = 1.f / z;
  // p_i = exp(l_i/T - lmax) / z ; p_max = 1/z
  const float pmax = inv_z;
  int k = top_k[b];
  if (k <= 0 || k > V) k = V;
  const float tp = top_p[b];
  const float minp_thr = min_p[b] * pmax;

  // Radix descent over the (non-negative) float bit pattern of p, most significant byte first.  Invariant:
  // all kept candidates strictly above the current prefix bucket are accounted for in (cnt_above, mass_above).
  // We look for the smallest threshold bucket such that tokens with p above it do not yet satisfy either
  // stopping rule: count >= k  or  mass >= top_p.
  unsigned int prefix = 0;
  unsigned int cnt_above = 0;
  float mass_above = 0.f;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += blockDim.x) { hist_cnt[i] = 0; hist_mass[i] = 0.f; }
    __syncthreads();
    const unsigned int hi_mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += blockDim.x) {
      const float pr = __expf(to_f32(row[i]) * inv_t - lmax) * inv_z;
      const unsigned int bits = __float_as_uint(pr);
      if ((bits & hi_mask) == (prefix & hi_mask)) {
        const unsigned int bucket = (bits >> shift) & 0xFFu;
        atomicAdd(&hist_cnt[bucket], 1u);
        atomicAdd(&hist_mass[bucket], pr);
      }
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int cnt = cnt_above;
      float mass = mass_above;
      int chosen = 0;
      for (int bkt = 255; bkt >= 0; --bkt) {
        const unsigned int c2 = cnt + hist_cnt[bkt];
        const float m2 = mass + hist_mass[bkt];
        // does the cut fall inside this bucket?  (taking the whole bucket reaches k tokens or top_p mass)
        if (c2 >= (unsigned int)k || m2 >= tp || bkt == 0) { chosen = bkt; break; }
        cnt = c2; mass = m2;
      }
      sh_prefix = prefix | ((unsigned int)chosen << shift);
      sh_need_cnt = cnt;
      sh_need_mass = mass;
    }
    __syncthreads();
    prefix = sh_prefix;
    cnt_above = sh_need_cnt;
    mass_above = sh_need_mass;
    __syncthreads();
  }
  // `prefix` is now the exact bit pattern of the threshold probability t*.  Tokens with p > t* are all kept
  // (cnt_above of them, mass mass_above); of the tokens with p == t*, keep in index order while
  // count < k and mass-before < top_p.
  const float thr = __uint_as_float(prefix);
  int ties_keep;
  {
    const int room_k = k - (int)cnt_above;
    int room_p = 0;
    if (thr > 0.f) {
      const float need = tp - mass_above;
      room_p = need > 0.f ? (int)ceilf(need / thr) : 0;
    } else {
      room_p = 0x7FFFFFFF;
    }
    ties_keep = max(1 - (int)cnt_above, min(room_k, room_p));
    if (cnt_above == 0 && ties_keep < 1) ties_keep = 1;
  }
  // min-p: drop anything below min_p * p_max (the top token always survives)
  // Kept mass for renormalisation, then inverse CDF in index order.  Two sweeps in fixed chunk order keep the
  // result independent of thread scheduling.
  float kept = 0.f;
  {
    // count ties before each index requires an ordered scan; do it chunk by chunk (blockDim tokens per chunk)
    __shared__ unsigned int tie_base;
    __shared__ float mass_base;
    __shared__ unsigned int warp_ties[32];
    __shared__ float warp_mass[32];
    if (tid == 0) { tie_base = 0; mass_base = 0.f; sh_pick = -1; }
    __syncthreads();
    const float u = uniform[b];
    // first sweep: total kept mass
    unsigned int my_tie_total = 0;
    for (int base = 0; base < V; base += blockDim.x) {
      const int i = base + tid;
      float pr = 0.f; bool tie = false, above = false;
      if (i < V) {
        pr = __expf(to_f32(row[i]) * inv_t - lmax) * inv_z;
        above = pr > thr; tie = pr == thr;
      }
      // exclusive count of ties before me inside the chunk
      const unsigned int bal = __ballot_sync(0xffffffffu, tie);
      const unsigned int before_w = __popc(bal & ((1u << (tid & 31)) - 1u));
      if ((tid & 31) == 0) warp_ties[tid >> 5] = __popc(bal);
      __syncthreads();
      unsigned int before = tie_base + before_w;
      for (int w = 0; w < (tid >> 5); ++w) before += warp_ties[w];
      const bool keep = (above || (tie && (int)before < ties_keep)) && (pr >= minp_thr || pr >= pmax);
      kept += keep ? pr : 0.f;
      __syncthreads();
      if (tid == 0) { unsigned int t = 0; for (int w = 0; w < (blockDim.x >> 5); ++w) t += warp_ties[w]; tie_base += t; }
      __syncthreads();
      (void)my_tie_total;
    }
    kept = block_sum(kept, red);
    const float target = u * kept * (1.f - 1e-7f);
    if (tid == 0) { tie_base = 0; mass_base = 0.f; }
    __syncthreads();
    // second sweep: find the first index whose inclusive kept-CDF exceeds target
    for (int base = 0; base < V; base += blockDim.x) {
      const int i = base + tid;
      float pr = 0.f; bool tie = false, above = false;
      if (i < V) {
        pr = __expf(to_f32(row[i]) * inv_t - lmax) * inv_z;
        above = pr > thr; tie = pr == thr;
      }
      const unsigned int bal = __ballot_sync(0xffffffffu, tie);
      const unsigned int before_w = __popc(bal & ((1u << (tid & 31)) - 1u));
      if ((tid & 31) == 0) warp_ties[tid >> 5] = __popc(bal);
      __syncthreads();
      unsigned int before = tie_base + before_w;
      for (int w = 0; w < (tid >> 5); ++w) before += warp_ties[w];
      const bool keep = (above || (tie && (int)before < ties_keep)) && (pr >= minp_thr || pr >= pmax);
      const float mine = keep ? pr : 0.f;
      // inclusive scan of `mine` across the block (warp scan + warp totals)
      float sc = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, sc, o);
        if ((tid & 31) >= o) sc += n;
      }
      if ((tid & 31) == 31) warp_mass[tid >> 5] = sc;
      __syncthreads();
      float pre = mass_base;
      for (int w = 0; w < (tid >> 5); ++w) pre += warp_mass[w];
      const float incl = pre + sc;
      if (keep && incl > target && (incl - mine) <= target) atomicCAS(&sh_pick, -1, i);
      __syncthreads();
      if (tid == 0) {
        unsigned int t = 0; float mm = 0.f;
        for (int w = 0; w < (blockDim.x >> 5); ++w) { t += warp_ties[w]; mm += warp_mass[w]; }
        tie_base += t; mass_base += mm;
      }
      __syncthreads();
      if (sh_pick >= 0) break;
    }
    if (tid == 0) {
      int pick = sh_pick;
      if (pick < 0) pick = 0;     // numerical corner: fall back below
      out[b] = pick;
    }
  }
}

// Greedy speculative acceptance: draft [B,K] (-1 = no draft at that depth), target [B,K+1] -> n_accepted [B]
__global__ void spec_accept_kernel(const long long* draft, const long long* target, int K, int* n_acc, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int n = 0;
  while (n < K && draft[(long long)b * K + n] >= 0 && draft[(long long)b * K + n] == target[(long long)b * (K + 1) + n]) ++n;
  n_acc[b] = n;
}

// Sparse logit edits of one sampling step, one thread per (row, token) pair; a pair appears at most once in the list,
// so no two threads touch the same element.  The edit is the composition, in the pipeline's order, of
//   x += add          (logit bias)
//   x = x > 0 ? x / rep : x * rep      (repetition penalty, rep != 1)
//   x -= sub          (presence + frequency + DRY penalties)
//   x = -inf          (flag bit 0: token banned at this step, e.g. EOS before min_tokens)
struct LogitEdit {
  int row, token;
  float add, rep, sub;
  int flags;
};
__global__ void __launch_bounds__(256)
logit_edit_kernel(float* logits, long long ld, const LogitEdit* __restrict__ edits, int n, int V, int B) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const LogitEdit e = edits[i];
  if (e.row < 0 || e.row >= B || e.token < 0 || e.token >= V) return;
  float* p = logits + (long long)e.row * ld + e.token;
  float x = *p + e.add;
  if (e.rep != 1.f) x = x > 0.f ? x / e.rep : x * e.rep;
  x -= e.sub;
  if (e.flags & 1) x = -INFINITY;
  *p = x;
}

}  // namespace atlas

using namespace atlas;

extern "C" int atlas_argmax(const void* logits, long long ld, int B, int V, int is_bf16, long long* out, float* out_val,
                            void* stream) {
  if (B <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16)
    argmax_kernel<__nv_bfloat16><<<B, 1024, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, out, out_val);
  else
    argmax_kernel<float><<<B, 1024, 0, st>>>(reinterpret_cast<const float*>(logits), ld, V, out, out_val);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_sample(const void* logits, long long ld, int B, int V, int is_bf16, const float* temperature,
                            const int* top_k, const float* top_p, const float* min_p, const float* uniform,
                            long long* out, void* stream) {
  if (B <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<B, 1024, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, temperature,
                                                     top_k, top_p, min_p, uniform, out);
  else
    sample_kernel<float><<<B, 1024, 0, st>>>(reinterpret_cast<const float*>(logits), ld, V, temperature, top_k, top_p,
                                             min_p, uniform, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_spec_accept(const long long* draft, const long long* target, int B, int K, int* n_acc, void* stream) {
  if (B <= 0) return 0;
  spec_accept_kernel<<<(B + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(draft, target, K, n_acc, B);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

// `edits`: n records of {int row, int token, float add, float rep, float sub, int flags} (24 bytes each) on the device;
// `logits` fp32 [B, V] with row stride ld, edited in place.
extern "C" int atlas_logit_edits(float* logits, long long ld, int B, int V, const void* edits, int n, void* stream) {
  if (n <= 0) return 0;
  logit_edit_kernel<<<(n + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, ld, reinterpret_cast<const LogitEdit*>(edits), n, V, B);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
