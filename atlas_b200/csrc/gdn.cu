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
                const unsigned char* __restrict__ has_state, __nv_bfloat16* y, long long ldy, int T,
                const __nv_bfloat16* __restrict__ bias) {
  const int t = blockIdx.x;           // rows on grid.x (no 65535 limit)
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C || t >= T) return;
  const int b = seq_of_token[t];
  const int q0 = query_start_loc[b];
  const int rel = t - q0;                      // row inside this sequence's chunk
  const long long slot = state_slots[b];
  const bool live = has_state[b] != 0;
  float acc = bias ? __bfloat162float(bias[c]) : 0.f;
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


// ---------------------------------------------------------------------------- chunked form (prefill)
// The same recurrence evaluated 64 tokens at a time on the tensor cores (TF32 mma.sync, fp32 state and accumulation).
// With G_i the running sum of the log-decays inside the chunk and h0 the state at its start:
//   (I + A) D = B,   A_ij = beta_i e^{G_i - G_j} (k_i . k_j)  (j < i),   B_i = beta_i (v_i - e^{G_i} h0^T k_i)
//   o_i = e^{G_i} h0^T q_i + sum_{j <= i} e^{G_i - G_j} (q_i . k_j) D_j
//   h   = e^{G_C} h0 + sum_j e^{G_C - G_j} k_j (x) D_j
// so one chunk is six small matrix products plus a 64-step forward substitution in which every thread owns one value
// column (no synchronisation inside the solve).  One CTA per (value head, sequence) walks its chunks in order; the
// state stays in shared memory between chunks.  Decays are differences of non-positive running sums, so every
// exponential is <= 1.  Reference ops replaced: gated_delta_rule_fla.cu / gated_delta_rule_chunk*.cu (WY chunk form).
constexpr int kGC = 64;          // chunk length
constexpr int kGLd = 132;        // leading dimension of the [.][128] fp32 tiles (padding spreads banks)
constexpr int kGLdS = 68;        // leading dimension of the [64][64] tiles

ATLAS_DEVICE uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
  return r;
}
ATLAS_DEVICE void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// c (16 x 8 tile at m0, n0) += A[m0.., 0..K) * B[0..K, n0..); a_at(m, k) and b_at(k, n) read fp32 from shared memory
template <typename FA, typename FB>
ATLAS_DEVICE void warp_tile_tf32(float (&c)[4], int m0, int n0, int K, FA a_at, FB b_at, int lane) {
  const int g = lane >> 2, t = lane & 3;
  for (int k0 = 0; k0 < K; k0 += 8) {
    uint32_t a[4] = {to_tf32(a_at(m0 + g, k0 + t)), to_tf32(a_at(m0 + g + 8, k0 + t)), to_tf32(a_at(m0 + g, k0 + t + 4)),
                     to_tf32(a_at(m0 + g + 8, k0 + t + 4))};
    uint32_t b[2] = {to_tf32(b_at(k0 + t, n0 + g)), to_tf32(b_at(k0 + t + 4, n0 + g))};
    mma_tf32(c, a, b);
  }
}

// DVC = value columns per CTA.  The columns of the state evolve independently (the solve and every product below are
// column-wise in v), so a head can be cut into 128 / DVC CTAs (grid.z) when sequences x heads alone would leave SMs idle;
// each CTA then repeats the K K^T / Q K^T products, which do not depend on v.
template <int DVC>
__global__ void __launch_bounds__(256, 1)
gdn_chunk_kernel(const GdnParams p) {
  constexpr int DK = 128, DV = 128;
  constexpr int LDV = DVC + 4;              // leading dimension of the [.][DVC] tiles
  constexpr int NT = DVC / 8;               // 8-wide column tiles of a slice
  extern __shared__ float gsm[];
  float* sh = gsm;                          // state slice [DK][LDV]
  float* sK = sh + DK * LDV;                // [64][kGLd]
  float* sQ = sK + kGC * kGLd;
  float* sV = sQ + kGC * kGLd;              // [64][LDV]: v, then B, then D (in place)
  float* sA = sV + kGC * LDV;               // [64][kGLdS]
  float* sP = sA + kGC * kGLdS;
  float* sG = sP + kGC * kGLdS;             // running log-decay [64]
  float* sBeta = sG + kGC;                  // [64]
  float* sE = sBeta + kGC;                  // e^{G_i}
  float* sW = sE + kGC;                     // e^{G_C - G_i}
  const int hv = blockIdx.x, bseq = blockIdx.y;
  const int v0 = blockIdx.z * DVC;          // first value column of this CTA
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int hk = hv / (p.Hv / p.Hk);
  const int q0 = p.query_start_loc[bseq];
  const int n = p.query_start_loc[bseq + 1] - q0;
  if (n <= 0) return;
  const long long slot = p.state_slots[bseq];
  float* hs = p.h + ((slot * p.Hv + hv) * (long long)DK) * DV;
  const bool live = p.has_state[bseq] != 0;
  for (int i = tid; i < DK * DVC; i += 256) sh[(i / DVC) * LDV + (i % DVC)] = live ? hs[(i / DVC) * DV + v0 + (i % DVC)] : 0.f;
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const int kd = p.Hk * DK;
  const int snaps = p.num_snaps_per_seq;
  __syncthreads();

  for (int c0 = 0; c0 < n;) {
    int rows = min(kGC, n - c0);
    for (int s = 0; s < snaps; ++s) {          // a snapshot inside the chunk ends it there (any row may be a snapshot row)
      const int r = p.snap_rows[bseq * snaps + s];
      if (r > c0 && r < c0 + rows) rows = r - c0;
    }
    // ---- 1. rows of the chunk: q, k L2-normalised (q also scaled), v; gates
    for (int i = warp; i < kGC; i += 8) {
      float q[4] = {0.f, 0.f, 0.f, 0.f}, k[4] = {0.f, 0.f, 0.f, 0.f}, v[4] = {0.f, 0.f, 0.f, 0.f};
      if (i < rows) {
        const __nv_bfloat16* row = p.y + (long long)(q0 + c0 + i) * p.ldy;
        const uint2 rq = *reinterpret_cast<const uint2*>(row + hk * DK + lane * 4);
        const uint2 rk = *reinterpret_cast<const uint2*>(row + kd + hk * DK + lane * 4);
        const uint2 rv = lane * 4 < DVC ? *reinterpret_cast<const uint2*>(row + 2 * kd + hv * DV + v0 + lane * 4) : make_uint2(0u, 0u);
        const __nv_bfloat162* hq = reinterpret_cast<const __nv_bfloat162*>(&rq);
        const __nv_bfloat162* hkk = reinterpret_cast<const __nv_bfloat162*>(&rk);
        const __nv_bfloat162* hvv = reinterpret_cast<const __nv_bfloat162*>(&rv);
        for (int e = 0; e < 2; ++e) {
          float2 f = __bfloat1622float2(hq[e]); q[2 * e] = f.x; q[2 * e + 1] = f.y;
          f = __bfloat1622float2(hkk[e]); k[2 * e] = f.x; k[2 * e + 1] = f.y;
          f = __bfloat1622float2(hvv[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y;
        }
      }
      const float qs = warp_sum(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
      const float ks = warp_sum(k[0] * k[0] + k[1] * k[1] + k[2] * k[2] + k[3] * k[3]);
      const float qn = rsqrtf(qs + 1e-6f) * p.scale, kn = rsqrtf(ks + 1e-6f);
      for (int e = 0; e < 4; ++e) {
        sQ[i * kGLd + lane * 4 + e] = q[e] * qn;
        sK[i * kGLd + lane * 4 + e] = k[e] * kn;
        if (lane * 4 < DVC) sV[i * LDV + lane * 4 + e] = v[e];
      }
      if (lane == 0) {
        float gi = 0.f, bi = 0.f;
        if (i < rows) {
          const long long tt = q0 + c0 + i;
          const float av = __bfloat162float(p.a[tt * p.lda + hv]) + dtb;
          const float sp = av > 20.f ? av : log1pf(__expf(av));
          gi = neg_a * sp;
          bi = 1.f / (1.f + __expf(-__bfloat162float(p.b[tt * p.ldb + hv])));
        }
        sG[i] = gi;
        sBeta[i] = bi;
      }
    }
    __syncthreads();
    if (warp == 0) {            // inclusive running sum of the 64 log-decays (two per lane)
      float a0 = sG[lane], a1 = sG[lane + 32];
      for (int o = 1; o < 32; o <<= 1) {
        const float u0 = __shfl_up_sync(0xffffffffu, a0, o), u1 = __shfl_up_sync(0xffffffffu, a1, o);
        if (lane >= o) { a0 += u0; a1 += u1; }
      }
      const float tot0 = __shfl_sync(0xffffffffu, a0, 31);
      sG[lane] = a0;
      sG[lane + 32] = a1 + tot0;
      const float gl = __shfl_sync(0xffffffffu, a1 + tot0, 31);
      sE[lane] = __expf(a0); sE[lane + 32] = __expf(a1 + tot0);
      sW[lane] = __expf(gl - a0); sW[lane + 32] = __expf(gl - a1 - tot0);
    }
    __syncthreads();
    // ---- 2. B = beta (v - e^G (K h0)); A and P from K K^T and Q K^T
    for (int tile = warp; tile < 4 * NT; tile += 8) {
      const int m0 = (tile / NT) * 16, n0 = (tile % NT) * 8;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      warp_tile_tf32(c, m0, n0, DK, [&](int m, int k) { return sK[m * kGLd + k]; }, [&](int k, int nn) { return sh[k * LDV + nn]; }, lane);
      for (int e = 0; e < 4; ++e) {
        const int i = m0 + g + (e >> 1) * 8, j = n0 + 2 * t4 + (e & 1);
        sV[i * LDV + j] = sBeta[i] * (sV[i * LDV + j] - sE[i] * c[e]);
      }
    }
    for (int tile = warp; tile < 64; tile += 8) {
      const bool is_q = tile >= 32;
      const int tl = tile & 31;
      const int m0 = (tl >> 3) * 16, n0 = (tl & 7) * 8;
      const float* src = is_q ? sQ : sK;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      warp_tile_tf32(c, m0, n0, DK, [&](int m, int k) { return src[m * kGLd + k]; }, [&](int k, int nn) { return sK[nn * kGLd + k]; }, lane);
      for (int e = 0; e < 4; ++e) {
        const int i = m0 + g + (e >> 1) * 8, j = n0 + 2 * t4 + (e & 1);
        const float dec = __expf(sG[i] - sG[j]);
        if (is_q) sP[i * kGLdS + j] = (j <= i) ? dec * c[e] : 0.f;
        else      sA[i * kGLdS + j] = (j < i) ? sBeta[i] * dec * c[e] : 0.f;
      }
    }
    __syncthreads();
    // ---- 3. forward substitution (I + A) D = B, one value column per thread
    if (tid < DVC) {
      float d[kGC];
#pragma unroll
      for (int i = 0; i < kGC; ++i) {
        float acc = sV[i * LDV + tid];
#pragma unroll
        for (int j = 0; j < i; ++j) acc = fmaf(-sA[i * kGLdS + j], d[j], acc);
        d[i] = acc;
      }
#pragma unroll
      for (int i = 0; i < kGC; ++i) sV[i * LDV + tid] = d[i];
    }
    __syncthreads();
    // ---- 4. o = e^G (Q h0) + P D
    for (int tile = warp; tile < 4 * NT; tile += 8) {
      const int m0 = (tile / NT) * 16, n0 = (tile % NT) * 8;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      warp_tile_tf32(c, m0, n0, DK, [&](int m, int k) { return sQ[m * kGLd + k]; }, [&](int k, int nn) { return sh[k * LDV + nn]; }, lane);
      const float e0 = sE[m0 + g], e1 = sE[m0 + g + 8];
      c[0] *= e0; c[1] *= e0; c[2] *= e1; c[3] *= e1;
      warp_tile_tf32(c, m0, n0, kGC, [&](int m, int k) { return sP[m * kGLdS + k]; }, [&](int k, int nn) { return sV[k * LDV + nn]; }, lane);
      for (int hlf = 0; hlf < 2; ++hlf) {
        const int i = m0 + g + hlf * 8;
        if (i < rows) {
          __nv_bfloat162 o2 = __floats2bfloat162_rn(c[2 * hlf], c[2 * hlf + 1]);
          *reinterpret_cast<__nv_bfloat162*>(p.out + (long long)(q0 + c0 + i) * p.ldo + hv * DV + v0 + n0 + 2 * t4) = o2;
        }
      }
    }
    __syncthreads();
    // ---- 5. h = e^{G_C} h0 + sum_j e^{G_C - G_j} k_j (x) D_j
    {
      const float gC = sE[kGC - 1];
      for (int tile = warp; tile < 8 * NT; tile += 8) {
        const int m0 = (tile / NT) * 16, n0 = (tile % NT) * 8;
        float c[4];
        for (int e = 0; e < 4; ++e) c[e] = sh[(m0 + g + (e >> 1) * 8) * LDV + n0 + 2 * t4 + (e & 1)] * gC;
        warp_tile_tf32(c, m0, n0, kGC, [&](int m, int k) { return sK[k * kGLd + m] * sW[k]; },
                       [&](int k, int nn) { return sV[k * LDV + nn]; }, lane);
        for (int e = 0; e < 4; ++e) sh[(m0 + g + (e >> 1) * 8) * LDV + n0 + 2 * t4 + (e & 1)] = c[e];
      }
    }
    __syncthreads();
    for (int s = 0; s < snaps; ++s) {
      if (p.snap_rows[bseq * snaps + s] == c0 + rows) {
        float* dst = p.h + (((long long)p.snap_slots[bseq * snaps + s] * p.Hv + hv) * (long long)DK) * DV;
        for (int i = tid; i < DK * DVC; i += 256) dst[(i / DVC) * DV + v0 + (i % DVC)] = sh[(i / DVC) * LDV + (i % DVC)];
      }
    }
    c0 += rows;
  }
  if (p.commit)
    for (int i = tid; i < DK * DVC; i += 256) hs[(i / DVC) * DV + v0 + (i % DVC)] = sh[(i / DVC) * LDV + (i % DVC)];
}

}  // namespace atlas

using namespace atlas;

extern "C" int atlas_gdn_conv(const void* x, long long ldx, const void* w, int C, int W, const void* conv_state,
                              const int* seq_of_token, const int* query_start_loc, const int* state_slots,
                              const unsigned char* has_state, void* y, long long ldy, int T, void* stream) {
  if (T <= 0) return 0;
  if (W < 2 || W > 8) return -1;
  dim3 grid(T, (C + 255) / 256);
  gdn_conv_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(w), C, W,
      reinterpret_cast<const __nv_bfloat16*>(conv_state), seq_of_token, query_start_loc, state_slots, has_state,
      reinterpret_cast<__nv_bfloat16*>(y), ldy, T, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

// Same depth-wise causal convolution + SiLU with a per-channel bias (Mamba-2 blocks).
extern "C" int atlas_conv1d_bias_silu(const void* x, long long ldx, const void* w, const void* bias, int C, int W,
                                      const void* conv_state, const int* seq_of_token, const int* query_start_loc,
                                      const int* state_slots, const unsigned char* has_state, void* y, long long ldy, int T,
                                      void* stream) {
  if (T <= 0) return 0;
  if (W < 2 || W > 8) return -1;
  dim3 grid(T, (C + 255) / 256);
  gdn_conv_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(w), C, W,
      reinterpret_cast<const __nv_bfloat16*>(conv_state), seq_of_token, query_start_loc, state_slots, has_state,
      reinterpret_cast<__nv_bfloat16*>(y), ldy, T, reinterpret_cast<const __nv_bfloat16*>(bias));
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

// Chunked (64-token) evaluation of the same recurrence for prefill-sized chunks: Dk = Dv = 128, whole sequences (no row
// limit); a snapshot row inside a chunk simply ends that chunk early.  Same state layout and arguments as
// atlas_gdn_recurrent.
extern "C" int atlas_gdn_chunked(const void* y, long long ldy, const void* a, long long lda, const void* b, long long ldb,
                                 const float* A_log, const float* dt_bias, float* h, void* out, long long ldo,
                                 const int* query_start_loc, const int* state_slots, const unsigned char* has_state,
                                 const int* snap_rows, const int* snap_slots, int num_snaps_per_seq, int B, int Hk, int Hv,
                                 int Dk, int Dv, int commit, void* stream) {
  if (B <= 0) return 0;
  if (Dk != 128 || Dv != 128 || Hv % Hk || (ldy % 4) || (ldo % 2)) return 1;       // caller falls back to the recurrence
  GdnParams p;
  p.y = reinterpret_cast<const __nv_bfloat16*>(y); p.ldy = ldy;
  p.a = reinterpret_cast<const __nv_bfloat16*>(a); p.lda = lda;
  p.b = reinterpret_cast<const __nv_bfloat16*>(b); p.ldb = ldb;
  p.A_log = A_log; p.dt_bias = dt_bias; p.h = h;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.query_start_loc = query_start_loc; p.state_slots = state_slots; p.has_state = has_state; p.limit = nullptr;
  p.snap_rows = snap_rows; p.snap_slots = snap_slots; p.num_snaps_per_seq = num_snaps_per_seq;
  p.Hk = Hk; p.Hv = Hv; p.Dv = Dv; p.commit = commit; p.scale = 1.f / sqrtf((float)Dk);
  // value-column slices per head: as many as keep the grid within the SM count (few long sequences), else one
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      num_sms = 1;
  }
  int split = 1;
  if (const char* e = getenv("ATLAS_GDN_SPLIT")) split = atoi(e);
  else if ((long long)Hv * B * 4 <= num_sms) split = 4;
  else if ((long long)Hv * B * 2 <= num_sms) split = 2;
  if (split != 1 && split != 2 && split != 4) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(Hv, B, split);
  auto smem_of = [](int dvc) { return (128 * (dvc + 4) + 2 * kGC * kGLd + kGC * (dvc + 4) + 2 * kGC * kGLdS + 4 * kGC) * 4; };
  if (split == 1) {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gdn_chunk_kernel<128>), smem_of(128)) != cudaSuccess) return -20;
    gdn_chunk_kernel<128><<<grid, 256, smem_of(128), st>>>(p);
  } else if (split == 2) {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gdn_chunk_kernel<64>), smem_of(64)) != cudaSuccess) return -20;
    gdn_chunk_kernel<64><<<grid, 256, smem_of(64), st>>>(p);
  } else {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gdn_chunk_kernel<32>), smem_of(32)) != cudaSuccess) return -20;
    gdn_chunk_kernel<32><<<grid, 256, smem_of(32), st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
