// Mamba-2 (SSD) recurrence, gated group RMSNorm and relu^2 for the Nemotron-H blocks.
//
//   mamba2_scan_kernel      one CTA per (head, sequence), one thread per channel p of the head; the thread keeps its row
//                           h[p][0..N) of the fp32 state in registers and walks the sequence's rows:
//                             dt = max(softplus(dt_raw + dt_bias), dt_min),  a = exp(-exp(A_log) * dt)
//                             h[p][n] = a * h[p][n] + dt * x[p] * B[n];   y[p] = sum_n h[p][n] * C[n] + D * x[p]
//                           B / C of the row's group are staged in shared memory.  Varlen batches, state slots, snapshot
//                           rows and the accepted-prefix limit follow the Gated-DeltaNet kernels (gdn.cu).
//   mamba2_gated_norm_kernel  out = rmsnorm_per_group(y * silu(z)) * w, one warp per (row, group)
//   relu2_kernel            y = relu(x)^2
//
// Reference ops replaced: kernels/gb10/common/mamba2_ssm_decode.cu, mamba2_ssd_chunk.cu (sequential form here),
// gated_rms_norm, relu_squared.cu.
#include "common.cuh"
#include "host_api.h"

namespace atlas {

struct Mamba2Params {
  const __nv_bfloat16* y; long long ldy;            // conv output rows [x | B | C]
  const __nv_bfloat16* dt; long long lddt;           // raw dt [T, H]
  const float* A_log; const float* D; const float* dt_bias;
  float* h;                                          // [slots, H, P, N]
  __nv_bfloat16* out; long long ldo;                 // [T, H * P]
  const int* query_start_loc; const int* state_slots; const unsigned char* has_state; const int* limit;
  const int* snap_rows; const int* snap_slots; int num_snaps_per_seq;
  int H, P, G, commit;
  float dt_min;
};

template <int N>
__global__ void __launch_bounds__(128)
mamba2_scan_kernel(const Mamba2Params p) {
  const int head = blockIdx.x, bseq = blockIdx.y;
  const int ch = threadIdx.x;
  const bool live_ch = ch < p.P;
  const int q0 = p.query_start_loc[bseq];
  const int qlen = p.query_start_loc[bseq + 1] - q0;
  const int n_rows = p.limit ? min(p.limit[bseq], qlen) : qlen;
  if (n_rows <= 0) return;
  const long long slot = p.state_slots[bseq];
  float* hs = p.h + (((long long)slot * p.H + head) * p.P + ch) * N;
  float h[N];
  const bool had = p.has_state[bseq] != 0 && live_ch;
#pragma unroll
  for (int n = 0; n < N; ++n) h[n] = had ? hs[n] : 0.f;
  __shared__ float sB[N], sC[N];
  const int group = head / (p.H / p.G);
  const int d_inner = p.H * p.P;
  const float neg_a = -__expf(p.A_log[head]);
  const float dskip = p.D[head], dtb = p.dt_bias[head];
  for (int r = 0; r < n_rows; ++r) {
    const long long t = q0 + r;
    const __nv_bfloat16* row = p.y + t * p.ldy;
    __syncthreads();                               // the previous row's readers are done with sB / sC
    for (int n = ch; n < N; n += blockDim.x) {
      sB[n] = __bfloat162float(row[d_inner + group * N + n]);
      sC[n] = __bfloat162float(row[d_inner + p.G * N + group * N + n]);
    }
    __syncthreads();
    const float raw = __bfloat162float(p.dt[t * p.lddt + head]) + dtb;
    const float dtv = fmaxf(raw > 20.f ? raw : log1pf(__expf(raw)), p.dt_min);
    const float decay = __expf(neg_a * dtv);
    const float x = live_ch ? __bfloat162float(row[head * p.P + ch]) : 0.f;
    const float dx = dtv * x;
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      h[n] = fmaf(h[n], decay, dx * sB[n]);
      acc = fmaf(h[n], sC[n], acc);
    }
    if (live_ch) p.out[t * p.ldo + head * p.P + ch] = __float2bfloat16_rn(acc + dskip * x);
    for (int s = 0; s < p.num_snaps_per_seq; ++s) {
      if (p.snap_rows[bseq * p.num_snaps_per_seq + s] == r + 1 && live_ch) {
        float* dst = p.h + (((long long)p.snap_slots[bseq * p.num_snaps_per_seq + s] * p.H + head) * p.P + ch) * N;
#pragma unroll
        for (int n = 0; n < N; ++n) dst[n] = h[n];
      }
    }
  }
  if (p.commit && live_ch) {
#pragma unroll
    for (int n = 0; n < N; ++n) hs[n] = h[n];
  }
}

// one warp per (row, group): v = y * silu(z); out = v * rsqrt(mean(v^2) + eps) * w
__global__ void __launch_bounds__(256)
mamba2_gated_norm_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const __nv_bfloat16* __restrict__ z, long long ldz,
                         const __nv_bfloat16* __restrict__ w, __nv_bfloat16* out, long long ldo, int T, int groups, int gsize,
                         float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T * groups) return;
  const int t = warp / groups, g = warp % groups;
  const __nv_bfloat16* yr = y + (long long)t * ldy + g * gsize;
  const __nv_bfloat16* zr = z + (long long)t * ldz + g * gsize;
  float ss = 0.f;
  for (int i = lane; i < gsize; i += 32) {
    const float zv = __bfloat162float(zr[i]);
    const float v = __bfloat162float(yr[i]) * (zv / (1.f + __expf(-zv)));
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)gsize + eps);
  for (int i = lane; i < gsize; i += 32) {
    const float zv = __bfloat162float(zr[i]);
    const float v = __bfloat162float(yr[i]) * (zv / (1.f + __expf(-zv)));
    out[(long long)t * ldo + g * gsize + i] = __float2bfloat16_rn(v * rstd * __bfloat162float(w[g * gsize + i]));
  }
}

__global__ void __launch_bounds__(256)
relu2_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* y, long long ldy, int cols) {
  const long long t = blockIdx.x;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < cols; c += gridDim.y * blockDim.x * 8) {
    if (c + 8 <= cols) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + t * ldx + c);
      const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v);
      uint4 o;
      __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(hv[i]);
        f.x = f.x > 0.f ? f.x * f.x : 0.f;
        f.y = f.y > 0.f ? f.y * f.y : 0.f;
        ho[i] = __floats2bfloat162_rn(f.x, f.y);
      }
      *reinterpret_cast<uint4*>(y + t * ldy + c) = o;
    } else {
      for (int i = c; i < cols; ++i) {
        const float f = __bfloat162float(x[t * ldx + i]);
        y[t * ldy + i] = __float2bfloat16_rn(f > 0.f ? f * f : 0.f);
      }
    }
  }
}

}  // namespace atlas

using namespace atlas;

extern "C" int atlas_mamba2_scan(const void* y, long long ldy, const void* dt, long long lddt, const float* A_log, const float* D,
                                 const float* dt_bias, float dt_min, float* h, void* out, long long ldo, const int* qsl,
                                 const int* slots, const unsigned char* has, const int* limit, const int* snap_rows,
                                 const int* snap_slots, int snaps, int B, int H, int P, int N, int G, int commit, void* stream) {
  if (B <= 0) return 0;
  if (P > 128 || P < 1 || H % G) return -1;
  Mamba2Params p;
  p.y = reinterpret_cast<const __nv_bfloat16*>(y); p.ldy = ldy; p.dt = reinterpret_cast<const __nv_bfloat16*>(dt); p.lddt = lddt;
  p.A_log = A_log; p.D = D; p.dt_bias = dt_bias; p.h = h; p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.query_start_loc = qsl; p.state_slots = slots; p.has_state = has; p.limit = limit; p.snap_rows = snap_rows;
  p.snap_slots = snap_slots; p.num_snaps_per_seq = snaps; p.H = H; p.P = P; p.G = G; p.commit = commit; p.dt_min = dt_min;
  dim3 grid(H, B);
  const int threads = (P + 31) / 32 * 32;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (N) {
    case 16: mamba2_scan_kernel<16><<<grid, threads, 0, st>>>(p); break;
    case 32: mamba2_scan_kernel<32><<<grid, threads, 0, st>>>(p); break;
    case 64: mamba2_scan_kernel<64><<<grid, threads, 0, st>>>(p); break;
    case 128: mamba2_scan_kernel<128><<<grid, threads, 0, st>>>(p); break;
    default: return -2;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_mamba2_gated_norm(const void* y, long long ldy, const void* z, long long ldz, const void* w, void* out,
                                       long long ldo, int T, int groups, int gsize, float eps, void* stream) {
  if (T <= 0) return 0;
  const long long warps = (long long)T * groups;
  const int blocks = (int)((warps * 32 + 255) / 256);
  mamba2_gated_norm_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(y), ldy, reinterpret_cast<const __nv_bfloat16*>(z), ldz,
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(out), ldo, T, groups, gsize, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_relu2(const void* x, long long ldx, void* y, long long ldy, int T, int cols, void* stream) {
  if (T <= 0 || cols <= 0) return 0;
  if ((ldx % 8) || (ldy % 8) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15)) return -1;
  dim3 grid(T, min(8, (cols / 8 + 255) / 256 > 0 ? (cols / 8 + 255) / 256 : 1));
  relu2_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                                                          reinterpret_cast<__nv_bfloat16*>(y), ldy, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
