// Gated DeltaNet kernels (Qwen3-Next linear attention), varlen over the step's sequences:
//   gdn_conv_kernel        depthwise causal conv1d (width W <= 8) + SiLU over the mixed q|k|v channels, reading the
//                          per-sequence conv window from the state slot
//   gdn_conv_state_kernel  rolls the conv window forward (optionally only the first `limit` rows: write-on-accept)
//   gdn_recurrent_kernel   h_t = exp(g_t) h_{t-1} + k_t (x) ((v_t - h_{t-1}^T k_t) beta_t),  o_t = h_t^T q_t / sqrt(Dk)
//                          one CTA per (value head, sequence); thread j keeps column j of the fp32 state in registers;
//                          q/k L2-normalisation and the gates (g from A_log / dt_bias, beta = sigmoid(b)) are fused in.
//                          The same kernel serves decode (1 row), speculative verify (K rows, no commit), the
//                          write-on-accept fold (commit with a row limit) and prefill chunks, and can store
//                          mid-chunk snapshots of the state for the prefix cache.
// State layout: h [slots, Hv, Dk, Dv] fp32, conv window [slots, C, W-1] bf16.
// Reference ops replaced: kernels/gb10/common/{causal_conv1d,ssm_preprocess,gated_delta_rule*}.cu.
#include "common.cuh"
#include "host_api.h"

namespace atlas {

__global__ void __launch_bounds__(256)
gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w, int C, int W,
                const __nv_bfloat16* __restrict__ conv_state, const int* __restrict__ seq_of_token,
                const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                const unsigned char* __restrict__ has_state, __nv_bfloat16* y, long long ldy, int T) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C || t >= T) return;
  const int b = seq_of_token[t];
  const int q0 = query_start_loc[b];
  const int rel = t - q0;                      // row inside this sequence's chunk
  const long long slot = state_slots[b];
  const bool live = has_state[b] != 0;
  float acc = 0.f;
  // tap i multiplies the input i - (W-1) rows back... weight[c][W-1] is the current row
  for (int i = 0; i < W; ++i) {
    const int back = W - 1 - i;                // rows back from t
    float xv;
    if (back <= rel) {
      xv = __bfloat162float(x[(long long)(t - back) * ldx + c]);
    } else {
      const int sidx = (W - 1) - (back - rel);  // position in the stored window (oldest first)
      xv = live ? __bfloat162float(conv_state[(slot * C + c) * (W - 1) + sidx]) : 0.f;
    }
    acc += xv * __bfloat162float(w[c * W + i]);
  }
  y[(long long)t * ldy + c] = __float2bfloat16_rn(acc / (1.f + __expf(-acc)));
}

// new window = last W-1 entries of (old window ++ first n rows of the chunk), n = limit ? limit[b] : q_len
__global__ void __launch_bounds__(256)
gdn_conv_state_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int C, int W, __nv_bfloat16* conv_state,
                      const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                      const unsigned char* __restrict__ has_state, const int* __restrict__ limit,
                      const int* __restrict__ snap_rows, const int* __restrict__ snap_slots, int num_snaps_per_seq) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int q0 = query_start_loc[b];
  const int qlen = query_start_loc[b + 1] - q0;
  const long long slot = state_slots[b];
  const bool live = has_state[b] != 0;
  float old[8];
  for (int i = 0; i < W - 1; ++i) old[i] = live ? __bfloat162float(conv_state[(slot * C + c) * (W - 1) + i]) : 0.f;
  auto window_after = [&](int n, long long dst_slot) {
    for (int i = 0; i < W - 1; ++i) {
      const int src = n - (W - 1) + i;          // index into the chunk rows; negative -> old window
      float v;
      if (src >= 0) v = __bfloat162float(x[(long long)(q0 + src) * ldx + c]);
      else v = old[(W - 1) + src];
      conv_state[(dst_slot * C + c) * (W - 1) + i] = __float2bfloat16_rn(v);
    }
  };
  for (int s = 0; s < num_snaps_per_seq; ++s) {
    const int rows = snap_rows[b * num_snaps_per_seq + s];
    if (rows > 0 && rows <= qlen) window_after(rows, snap_slots[b * num_snaps_per_seq + s]);
  }
  const int n = limit ? limit[b] : qlen;
  if (n >= 0 && !(limit && n == 0)) window_after(n, slot);
}

struct GdnParams {
  const __nv_bfloat16* y; long long ldy;      // conv output: [T, 2*Hk*Dk + Hv*Dv] = q | k | v
  const __nv_bfloat16* a; long long lda;      // [T, Hv]
  const __nv_bfloat16* b; long long ldb;      // [T, Hv]
  const float* A_log; const float* dt_bias;    // [Hv]
  float* h;                                    // [slots, Hv, Dk, Dv]
  __nv_bfloat16* out; long long ldo;           // [T, Hv*Dv]
  const int* query_start_loc; const int* state_slots; const unsigned char* has_state;
  const int* limit;                            // rows to process per sequence (nullptr = all)
  const int* snap_rows; const int* snap_slots; int num_snaps_per_seq;
  int Hk, Hv, Dv, commit;
  float scale;
};

template <int DK>
__global__ void __launch_bounds__(256)
gdn_recurrent_kernel(const GdnParams p) {
  const int hv = blockIdx.x, bseq = blockIdx.y;
  const int j = threadIdx.x;                   // column of the state (value dim)
  const int DV = p.Dv;
  const int hk = hv / (p.Hv / p.Hk);
  const int q0 = p.query_start_loc[bseq];
  const int qlen = p.query_start_loc[bseq + 1] - q0;
  const int n = p.limit ? min(p.limit[bseq], qlen) : qlen;
  if (n <= 0) return;
  const long long slot = p.state_slots[bseq];
  float* hs = p.h + ((slot * p.Hv + hv) * (long long)DK) * DV;
  float h[DK];
  const bool live = p.has_state[bseq] != 0 && j < DV;
#pragma unroll
  for (int k = 0; k < DK; ++k) h[k] = live ? hs[(long long)k * DV + j] : 0.f;
  __shared__ float sq[DK], sk[DK];
  __shared__ float s_scal[4];                  // q norm scale, k norm scale, exp(g), beta
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const int kd = p.Hk * DK;
  const int snaps = p.num_snaps_per_seq;
  for (int r = 0; r < n; ++r) {
    const long long t = q0 + r;
    const __nv_bfloat16* row = p.y + t * p.ldy;
    if (j < DK) {
      sq[j] = __bfloat162float(row[hk * DK + j]);
      sk[j] = __bfloat162float(row[kd + hk * DK + j]);
    }
    __syncthreads();
    if (j < 64) {
      // warp 0 -> q, warp 1 -> k : L2 norms
      const float* src = (j < 32) ? sq : sk;
      const int l = j & 31;
      float ss = 0.f;
      for (int k = l; k < DK; k += 32) ss += src[k] * src[k];
      ss = warp_sum(ss);
      if (l == 0) s_scal[j >> 5] = rsqrtf(ss + 1e-6f);
    } else if (j == 64) {
      const float av = __bfloat162float(p.a[t * p.lda + hv]) + dtb;
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      s_scal[2] = __expf(neg_a * sp);
      s_scal[3] = 1.f / (1.f + __expf(-__bfloat162float(p.b[t * p.ldb + hv])));
    }
    __syncthreads();
    if (j < DV) {
      const float qn = s_scal[0] * p.scale, kn = s_scal[1], decay = s_scal[2], beta = s_scal[3];
      const float vt = __bfloat162float(row[2 * kd + hv * DV + j]);
      float mem = 0.f;
#pragma unroll
      for (int k = 0; k < DK; ++k) { h[k] *= decay; mem = fmaf(h[k], sk[k] * kn, mem); }
      const float delta = (vt - mem) * beta;
      float o = 0.f;
#pragma unroll
      for (int k = 0; k < DK; ++k) { h[k] = fmaf(sk[k] * kn, delta, h[k]); o = fmaf(h[k], sq[k] * qn, o); }
      p.out[t * p.ldo + hv * DV + j] = __float2bfloat16_rn(o);
      for (int s = 0; s < snaps; ++s) {
        if (p.snap_rows[bseq * snaps + s] == r + 1) {
          float* dst = p.h + (((long long)p.snap_slots[bseq * snaps + s] * p.Hv + hv) * (long long)DK) * DV;
#pragma unroll
          for (int k = 0; k < DK; ++k) dst[(long long)k * DV + j] = h[k];
        }
      }
    }
    __syncthreads();
  }
  if (p.commit && j < DV) {
#pragma unroll
    for (int k = 0; k < DK; ++k) hs[(long long)k * DV + j] = h[k];
  }
}

}  // namespace atlas

using namespace atlas;

extern "C" int atlas_gdn_conv(const void* x, long long ldx, const void* w, int C, int W, const void* conv_state,
                              const int* seq_of_token, const int* query_start_loc, const int* state_slots,
                              const unsigned char* has_state, void* y, long long ldy, int T, void* stream) {
  if (T <= 0) return 0;
  if (W < 2 || W > 8) return -1;
  dim3 grid((C + 255) / 256, T);
  gdn_conv_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(w), C, W,
      reinterpret_cast<const __nv_bfloat16*>(conv_state), seq_of_token, query_start_loc, state_slots, has_state,
      reinterpret_cast<__nv_bfloat16*>(y), ldy, T);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_gdn_conv_state(const void* x, long long ldx, int C, int W, void* conv_state,
                                    const int* query_start_loc, const int* state_slots, const unsigned char* has_state,
                                    const int* limit, const int* snap_rows, const int* snap_slots, int num_snaps_per_seq,
                                    int B, void* stream) {
  if (B <= 0) return 0;
  dim3 grid((C + 255) / 256, B);
  gdn_conv_state_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, C, W, reinterpret_cast<__nv_bfloat16*>(conv_state), query_start_loc,
      state_slots, has_state, limit, snap_rows, snap_slots, num_snaps_per_seq);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_gdn_recurrent(const void* y, long long ldy, const void* a, long long lda, const void* b, long long ldb,
                                   const float* A_log, const float* dt_bias, float* h, void* out, long long ldo,
                                   const int* query_start_loc, const int* state_slots, const unsigned char* has_state,
                                   const int* limit, const int* snap_rows, const int* snap_slots, int num_snaps_per_seq,
                                   int B, int Hk, int Hv, int Dk, int Dv, int commit, void* stream) {
  if (B <= 0) return 0;
  if (Dv > 256 || Hv % Hk) return -1;
  GdnParams p;
  p.y = reinterpret_cast<const __nv_bfloat16*>(y); p.ldy = ldy;
  p.a = reinterpret_cast<const __nv_bfloat16*>(a); p.lda = lda;
  p.b = reinterpret_cast<const __nv_bfloat16*>(b); p.ldb = ldb;
  p.A_log = A_log; p.dt_bias = dt_bias; p.h = h;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.query_start_loc = query_start_loc; p.state_slots = state_slots; p.has_state = has_state; p.limit = limit;
  p.snap_rows = snap_rows; p.snap_slots = snap_slots; p.num_snaps_per_seq = num_snaps_per_seq;
  p.Hk = Hk; p.Hv = Hv; p.Dv = Dv; p.commit = commit; p.scale = 1.f / sqrtf((float)Dk);
  dim3 grid(Hv, B);
  int threads = ((max(Dv, max(Dk, 65)) + 31) / 32) * 32;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (Dk == 128) gdn_recurrent_kernel<128><<<grid, threads, 0, st>>>(p);
  else if (Dk == 64) gdn_recurrent_kernel<64><<<grid, threads, 0, st>>>(p);
  else if (Dk == 32) gdn_recurrent_kernel<32><<<grid, threads, 0, st>>>(p);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
