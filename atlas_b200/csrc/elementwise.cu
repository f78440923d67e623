// Bandwidth-bound fused ops around the GEMMs (all 16-byte vectorised, one pass over the data):
//   * residual add + RMSNorm (+ per-token 128-group FP8 quantisation feeding the block-scaled GEMM)
//   * SiLU(gate) * up (+ FP8 group quantisation)
//   * stand-alone per-token-group FP8 quantisation
//   * per-head q/k RMSNorm + rotary embedding + FP8 quantisation + paged KV-cache write
//   * gated RMSNorm of the Gated-DeltaNet output
//
// FP8 activation scales are written "k-group major": scale[(k/128) * scale_ld + token], so that the GEMM
// epilogue's per-row scale reads are coalesced.
//
// Paged KV layout written here (and read by attention.cu):
//   K: [num_blocks, Hkv, block_size, D]      one page of one head is a contiguous [block_size, D] tile
//   V: [num_blocks, Hkv, D, block_size]      transposed inside the page: tokens are the contiguous axis, which is
//                                            the K-major operand layout for P*V on the tensor cores
// Reference ops replaced: kernels/gb10/common/{rms_norm,moe_silu_mul,per_token_group_quant_fp8,rope,
// reshape_and_cache,fused_k_norm_rope_cache}.cu.
#include "common.cuh"
#include "host_api.h"

namespace atlas {

constexpr float kFp8Max = 448.f;

struct __align__(16) bf16x8 {
  __nv_bfloat162 v[4];
};

ATLAS_DEVICE void load8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 r = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
ATLAS_DEVICE void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = r;
}
// 8 floats -> 8 e4m3 bytes with a common scale, packed.  The scale's reciprocal is formed once (IEEE) and multiplied in;
// against x / scale this moves a value by at most one fp32 ulp before the e4m3 rounding, i.e. an occasional code on a
// rounding boundary differs by one step.  Conversions go two at a time (cvt.rn.satfinite.e4m3x2.f32).
ATLAS_DEVICE uint2 quant8(const float (&f)[8], float scale) {
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
// max |x| over the 16 consecutive lanes that hold one 128-element group
ATLAS_DEVICE float group16_absmax(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int kMaxIters>
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* residual, long long ldr,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* res_out, long long ldro, __nv_bfloat16* y,
               long long ldy, uint8_t* q, long long ldq, float* scale, long long scale_ld, int H, float eps,
               int plus_one) {
  chain_trigger();
  chain_wait();
  const int t = blockIdx.x;
  const int tid = threadIdx.x;
  float vals[kMaxIters][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxIters; ++it) {
    const int e = (it * blockDim.x + tid) * 8;
    if (e < H) {
      load8(x + t * ldx + e, vals[it]);
      if (residual) {
        float r[8];
        load8(residual + t * ldr + e, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) vals[it][i] += r[i];
        if (res_out) {
          store8(res_out + t * ldro + e, vals[it]);
          // normalise what was stored (the rounded residual stream), like the unfused sequence would
#pragma unroll
          for (int i = 0; i < 8; ++i) vals[it][i] = __bfloat162float(__float2bfloat16_rn(vals[it][i]));
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += vals[it][i] * vals[it][i];
    }
  }
  __shared__ float red[32];
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  if (tid < 32) {
    float v = tid < (blockDim.x >> 5) ? red[tid] : 0.f;
    v = warp_sum(v);
    if (tid == 0) red[0] = v;
  }
  __syncthreads();
  const float rstd = rsqrtf(red[0] / (float)H + eps);
#pragma unroll
  for (int it = 0; it < kMaxIters; ++it) {
    const int e = (it * blockDim.x + tid) * 8;
    const bool live = e < H;
    float o[8];
    float amax = 0.f;
    if (live) {
      float wv[8];
      load8(w + e, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float ww = plus_one ? wv[i] + 1.f : wv[i];
        o[i] = __bfloat162float(__float2bfloat16_rn(vals[it][i] * rstd * ww));   // same rounding as the bf16 output
        amax = fmaxf(amax, fabsf(o[i]));
      }
    }
    if (q) {
      amax = group16_absmax(amax);
      if (live) {
        const float sc = fmaxf(amax, 1e-10f) / kFp8Max;
        *reinterpret_cast<uint2*>(q + t * ldq + e) = quant8(o, sc);
        if ((tid & 15) == 0) scale[(long long)(e >> 7) * scale_ld + t] = sc;
      }
    } else if (live) {
      store8(y + t * ldy + e, o);
    }
  }
}

// gate_up [T, 2I] -> act(gate) * up, bf16 or fp8+scale.  ACT 0: SiLU, 1: tanh-approximated GELU (Gemma).
template <int ACT>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, long long ld, int I, __nv_bfloat16* y, long long ldy, uint8_t* q,
                long long ldq, float* scale, long long scale_ld, const int* live_tiles) {
  chain_trigger();
  chain_wait();
  const int t = blockIdx.x;           // rows on grid.x: row counts can exceed the 65535 limit of grid.y
  if (live_tiles && t >= (*live_tiles) * 128) return;      // expert-sorted buffers: rows past the live tiles are unused
  const int e = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const bool live = e < I;
  float o[8];
  float amax = 0.f;
  if (live) {
    float g[8], u[8];
    load8(gu + t * ld + e, g);
    load8(gu + t * ld + I + e, u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s;
      if (ACT == 0) {
        s = __fdividef(g[i], 1.f + __expf(-g[i]));
      } else {
        const float x = g[i];
        s = 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
      }
      o[i] = __bfloat162float(__float2bfloat16_rn(s * u[i]));
      amax = fmaxf(amax, fabsf(o[i]));
    }
  }
  if (q) {
    amax = group16_absmax(amax);
    if (live) {
      const float sc = fmaxf(amax, 1e-10f) / kFp8Max;
      *reinterpret_cast<uint2*>(q + t * ldq + e) = quant8(o, sc);
      if ((threadIdx.x & 15) == 0) scale[(long long)(e >> 7) * scale_ld + t] = sc;
    }
  } else if (live) {
    store8(y + t * ldy + e, o);
  }
}

__global__ void __launch_bounds__(256)
quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int K, uint8_t* q, long long ldq, float* scale,
                 long long scale_ld) {
  chain_trigger();
  chain_wait();
  const int t = blockIdx.x;           // rows on grid.x: row counts can exceed the 65535 limit of grid.y
  const int e = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const bool live = e < K;
  float o[8];
  float amax = 0.f;
  if (live) {
    load8(x + t * ld + e, o);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(o[i]));
  }
  amax = group16_absmax(amax);
  if (live) {
    const float sc = fmaxf(amax, 1e-10f) / kFp8Max;
    *reinterpret_cast<uint2*>(q + t * ldq + e) = quant8(o, sc);
    if ((threadIdx.x & 15) == 0) scale[(long long)(e >> 7) * scale_ld + t] = sc;
  }
}

// One warp per (token, head): heads [0,Hq) are q (norm + rope, in place), [Hq,Hq+Hkv) are k (norm + rope + cache
// write), [Hq+Hkv, Hq+2Hkv) are v (cache write).  D <= 512, D % 64 == 0.
struct RopeKvParams {
  __nv_bfloat16* q; long long ldq;
  const __nv_bfloat16* k; long long ldk;
  const __nv_bfloat16* v; long long ldv;
  const int* positions;
  const float* rope;      // [max_pos, rotary_dim]: cos half then sin half
  const __nv_bfloat16* q_norm_w;
  const __nv_bfloat16* k_norm_w;
  void* k_cache; void* v_cache;
  const int* slot_mapping;
  int T, Hq, Hkv, D, rotary_dim, block_size, kv_fp8, plus_one;
  int v_separate;          // V rows are written by v_write_pages_kernel (prefill-size batches), not here
  int rotate;              // Walsh-Hadamard rotation of every q / k / v head before the write (head_dim-128 kernel only)
  float eps, inv_k_scale, inv_v_scale;
};

__global__ void __launch_bounds__(128)
rope_kv_write_kernel(const RopeKvParams p) {
  extern __shared__ float sm_rope[];          // [4 warps][D]
  chain_trigger();
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  const int heads = p.Hq + (p.v_separate ? 1 : 2) * p.Hkv;
  if (unit >= (long long)p.T * heads) return;
  const int t = (int)(unit / heads);
  const int h = (int)(unit % heads);
  float* buf = sm_rope + warp * p.D;
  const int D = p.D;
  const bool is_q = h < p.Hq;
  const bool is_k = !is_q && h < p.Hq + p.Hkv;
  const int hh = is_q ? h : (is_k ? h - p.Hq : h - p.Hq - p.Hkv);
  const __nv_bfloat16* src = is_q ? p.q + t * p.ldq + hh * D : (is_k ? p.k + t * p.ldk + hh * D : p.v + t * p.ldv + hh * D);
  const int slot = p.slot_mapping[t];
  if (!is_q && slot < 0) return;
  float ss = 0.f;
  for (int e = lane * 2; e < D; e += 64) {
    float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + e));
    buf[e] = f.x;
    buf[e + 1] = f.y;
    ss += f.x * f.x + f.y * f.y;
  }
  const __nv_bfloat16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
  if (nw) {
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + p.eps);
    for (int e = lane * 2; e < D; e += 64) {
      float2 wv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(nw + e));
      if (p.plus_one) { wv.x += 1.f; wv.y += 1.f; }
      // round like the unfused op chain would (norm output is bf16)
      buf[e] = __bfloat162float(__float2bfloat16_rn(buf[e] * rstd * wv.x));
      buf[e + 1] = __bfloat162float(__float2bfloat16_rn(buf[e + 1] * rstd * wv.y));
    }
  }
  __syncwarp();
  const int half = p.rotary_dim >> 1;
  const float* cs = p.rope + (long long)p.positions[t] * p.rotary_dim;
  long long kbase = 0, vbase = 0;
  int tok_in_blk = 0;
  if (!is_q) {
    const int blk = slot / p.block_size;
    tok_in_blk = slot % p.block_size;
    kbase = (((long long)blk * p.Hkv + hh) * p.block_size + tok_in_blk) * D;          // K: [blk][head][tok][d]
    vbase = ((long long)blk * p.Hkv + hh) * (long long)D * p.block_size + tok_in_blk;  // V: [blk][head][d][tok]
  }
  for (int e = lane * 2; e < D; e += 64) {
    float o[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int d = e + i;
      float val = buf[d];
      if (!(!is_q && !is_k) && d < p.rotary_dim) {
        if (d < half) val = buf[d] * cs[d] - buf[d + half] * cs[half + d];
        else          val = buf[d] * cs[d - half] + buf[d - half] * cs[d];
      }
      o[i] = val;
    }
    if (is_q) {
      *reinterpret_cast<__nv_bfloat162*>(p.q + t * p.ldq + hh * D + e) = __floats2bfloat162_rn(o[0], o[1]);
    } else if (is_k) {
      if (p.kv_fp8) {
        uint16_t pk = (uint16_t)f32_to_fp8_e4m3(o[0] * p.inv_k_scale) | ((uint16_t)f32_to_fp8_e4m3(o[1] * p.inv_k_scale) << 8);
        *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(p.k_cache) + kbase + e) = pk;
      } else {
        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.k_cache) + kbase + e) =
            __floats2bfloat162_rn(o[0], o[1]);
      }
    } else {
      if (p.kv_fp8) {
        uint8_t* vc = reinterpret_cast<uint8_t*>(p.v_cache) + vbase;
        vc[(long long)e * p.block_size] = f32_to_fp8_e4m3(o[0] * p.inv_v_scale);
        vc[(long long)(e + 1) * p.block_size] = f32_to_fp8_e4m3(o[1] * p.inv_v_scale);
      } else {
        __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(p.v_cache) + vbase;
        vc[(long long)e * p.block_size] = __float2bfloat16_rn(o[0]);
        vc[(long long)(e + 1) * p.block_size] = __float2bfloat16_rn(o[1]);
      }
    }
  }
}

// Same contract as rope_kv_write_kernel for head_dim = rotary_dim = 128: a lane owns four consecutive dims, the rotation
// partner (d +- 64) sits in lane ^ 16, so the whole unit stays in registers (one 8-byte load and store per lane, no
// shared memory).
// Orthonormal 128-point Walsh-Hadamard transform of one head held four consecutive dims per lane (natural order,
// H[i][j] = (-1)^popcount(i & j) / sqrt(128)): two butterfly stages inside the lane, five across lanes.  The transform is
// its own inverse and keeps dot products, so attention over rotated q / k / v gives the rotated output; what it buys is
// a near-Gaussian coordinate distribution without the outlier channels that cost an FP8 cache its range.
__device__ __forceinline__ void wht128_lane4(float (&o)[4], int lane) {
  const float a = o[0] + o[1], b = o[0] - o[1], c = o[2] + o[3], d = o[2] - o[3];
  o[0] = a + c; o[1] = b + d; o[2] = a - c; o[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pv = __shfl_xor_sync(0xffffffffu, o[i], m);
      o[i] = (lane & m) ? pv - o[i] : o[i] + pv;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] *= 0.08838834764831845f;
}

// In-place rotation of bf16 rows [T, H, 128] (the attention output of a rotated cache back to model coordinates).
__global__ void __launch_bounds__(128)
wht_d128_kernel(__nv_bfloat16* x, long long ld, long long units, int H) {
  chain_trigger();
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  if (unit >= units) return;
  __nv_bfloat16* row = x + (unit / H) * ld + (unit % H) * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(row);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  float o[4] = {a.x, a.y, b.x, b.y};
  wht128_lane4(o, lane);
  uint2 pk;
  pk.x = pack_bf16x2(o[0], o[1]);
  pk.y = pack_bf16x2(o[2], o[3]);
  *reinterpret_cast<uint2*>(row) = pk;
}

__global__ void __launch_bounds__(128)
rope_kv_write_d128_kernel(const RopeKvParams p) {
  chain_trigger();
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  const int heads = p.Hq + (p.v_separate ? 1 : 2) * p.Hkv;
  if (unit >= (long long)p.T * heads) return;
  const int t = (int)(unit / heads);
  const int h = (int)(unit % heads);
  constexpr int D = 128;
  const bool is_q = h < p.Hq;
  const bool is_k = !is_q && h < p.Hq + p.Hkv;
  const int hh = is_q ? h : (is_k ? h - p.Hq : h - p.Hq - p.Hkv);
  const __nv_bfloat16* src = is_q ? p.q + t * p.ldq + hh * D : (is_k ? p.k + t * p.ldk + hh * D : p.v + t * p.ldv + hh * D);
  const int slot = p.slot_mapping[t];
  if (!is_q && slot < 0) return;
  const int d0 = lane * 4;
  float v[4];
  {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + d0);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  const __nv_bfloat16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
  if (nw) {
    const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
    const float rstd = rsqrtf(ss / (float)D + p.eps);
    const uint2 wr = *reinterpret_cast<const uint2*>(nw + d0);
    const float2 wa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.x));
    const float2 wb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.y));
    const float w4[4] = {wa.x, wa.y, wb.x, wb.y};
#pragma unroll
    for (int i = 0; i < 4; ++i)      // round like the unfused op chain would (norm output is bf16)
      v[i] = __bfloat162float(__float2bfloat16_rn(v[i] * rstd * (w4[i] + (p.plus_one ? 1.f : 0.f))));
  }
  float o[4] = {v[0], v[1], v[2], v[3]};
  if (is_q || is_k) {
    const float* cs = p.rope + (long long)p.positions[t] * D;
    const int dd = d0 & 63;
    const float4 c4 = *reinterpret_cast<const float4*>(cs + dd);
    const float4 s4 = *reinterpret_cast<const float4*>(cs + 64 + dd);
    const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pv = __shfl_xor_sync(0xffffffffu, v[i], 16);
      o[i] = lane < 16 ? v[i] * cc[i] - pv * sn[i] : v[i] * cc[i] + pv * sn[i];
    }
  }
  if (p.rotate) wht128_lane4(o, lane);
  if (is_q) {
    uint2 pk;
    pk.x = pack_bf16x2(o[0], o[1]);
    pk.y = pack_bf16x2(o[2], o[3]);
    *reinterpret_cast<uint2*>(p.q + t * p.ldq + hh * D + d0) = pk;
    return;
  }
  const int blk = slot / p.block_size, tok_in_blk = slot % p.block_size;
  if (p.kv_fp8 == 2) {
    // ---- NVFP4 cache (page layout: see paged_attn_kernel): one e4m3 scale per token and 16 dims = four lanes
    const float inv_g = is_k ? p.inv_k_scale : p.inv_v_scale;
    float x[4];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { x[i] = o[i] * inv_g; amax = fmaxf(amax, fabsf(x[i])); }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint8_t s8 = f32_to_fp8_e4m3(amax * (1.f / 6.f));
    const float sdq = fp8_e4m3_to_f32(s8);
    const float inv = sdq > 0.f ? __frcp_rn(sdq) : 0.f;
    uint16_t lo8, hi8;                                           // (x0, x1) and (x2, x3): the first value in the low nibble
    asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\tcvt.u16.u8 %0, b;\n\t}\n" : "=h"(lo8) : "f"(x[0] * inv), "f"(x[1] * inv));
    asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\tcvt.u16.u8 %0, b;\n\t}\n" : "=h"(hi8) : "f"(x[2] * inv), "f"(x[3] * inv));
    const long long page = ((long long)blk * p.Hkv + hh) * ((long long)p.block_size * D * 9 / 16);
    if (is_k) {
      uint8_t* base = reinterpret_cast<uint8_t*>(p.k_cache) + page;
      *reinterpret_cast<uint16_t*>(base + (long long)tok_in_blk * (D / 2) + d0 / 2) = (uint16_t)(lo8 | (hi8 << 8));
      if ((lane & 3) == 0) base[(long long)p.block_size * (D / 2) + (long long)tok_in_blk * (D / 16) + (d0 >> 4)] = s8;
    } else {
      // V^T: dim-major, two TOKENS per byte -> the neighbouring token's nibble shares the byte: word-wide atomics
      uint8_t* base = reinterpret_cast<uint8_t*>(p.v_cache) + page;
      const uint32_t nib[4] = {lo8 & 0xFu, (lo8 >> 4) & 0xFu, hi8 & 0xFu, (hi8 >> 4) & 0xFu};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const long long byte = (long long)(d0 + i) * (p.block_size / 2) + (tok_in_blk >> 1);
        unsigned int* word = reinterpret_cast<unsigned int*>(base + (byte & ~3ll));
        const int shift = (int)(byte & 3) * 8 + (tok_in_blk & 1) * 4;
        atomicAnd(word, ~(0xFu << shift));
        atomicOr(word, nib[i] << shift);
      }
      if ((lane & 3) == 0) base[(long long)D * (p.block_size / 2) + (long long)(d0 >> 4) * p.block_size + tok_in_blk] = s8;
    }
    return;
  }
  if (is_k) {
    const long long kbase = (((long long)blk * p.Hkv + hh) * p.block_size + tok_in_blk) * D + d0;
    if (p.kv_fp8) {
      uint32_t w = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) w |= (uint32_t)f32_to_fp8_e4m3(o[i] * p.inv_k_scale) << (8 * i);
      *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(p.k_cache) + kbase) = w;
    } else {
      uint2 pk;
      pk.x = pack_bf16x2(o[0], o[1]);
      pk.y = pack_bf16x2(o[2], o[3]);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.k_cache) + kbase) = pk;
    }
    return;
  }
  const long long vbase = ((long long)blk * p.Hkv + hh) * (long long)D * p.block_size + tok_in_blk;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (p.kv_fp8) reinterpret_cast<uint8_t*>(p.v_cache)[vbase + (long long)(d0 + i) * p.block_size] = f32_to_fp8_e4m3(o[i] * p.inv_v_scale);
    else reinterpret_cast<__nv_bfloat16*>(p.v_cache)[vbase + (long long)(d0 + i) * p.block_size] = __float2bfloat16_rn(o[i]);
  }
}

// V rows of a prefill-size batch -> the transposed FP8 page layout [blk][head][d][tok16].  One warp per (16 consecutive
// batch rows, kv head).  When the 16 rows fill one page in order (the common case inside a prompt chunk) every lane
// gathers 16 tokens for its dims and writes whole 16-byte page rows; otherwise each row falls back to byte stores.
__global__ void __launch_bounds__(128)
v_write_pages_kernel(const RopeKvParams p) {
  chain_trigger();
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  const int groups = (p.T + 15) / 16;
  if (unit >= (long long)groups * p.Hkv) return;
  const int g = (int)(unit / p.Hkv), hh = (int)(unit % p.Hkv);
  const int t0 = g * 16, D = p.D;
  const int my_slot = (lane < 16 && t0 + lane < p.T) ? p.slot_mapping[t0 + lane] : -2;
  const int slot0 = __shfl_sync(0xffffffffu, my_slot, 0);
  const bool in_order = lane >= 16 || (slot0 >= 0 && my_slot == slot0 + lane);
  const bool fast = __all_sync(0xffffffffu, in_order) && (slot0 % 16) == 0 && t0 + 16 <= p.T;
  uint8_t* vc_all = reinterpret_cast<uint8_t*>(p.v_cache);
  if (fast) {
    uint8_t* page = vc_all + ((long long)(slot0 / 16) * p.Hkv + hh) * (long long)D * 16;
    for (int d0 = lane * 4; d0 < D; d0 += 128) {
      uint32_t col[4][4];                       // [dim][token quad] packed fp8
#pragma unroll
      for (int tq = 0; tq < 4; ++tq) {
        float vals[4][4];                       // [token in quad][dim]
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint2 raw = *reinterpret_cast<const uint2*>(p.v + (long long)(t0 + tq * 4 + i) * p.ldv + hh * D + d0);
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
          vals[i][0] = a.x; vals[i][1] = a.y; vals[i][2] = b.x; vals[i][3] = b.y;
        }
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          uint32_t w = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) w |= (uint32_t)f32_to_fp8_e4m3(vals[i][d] * p.inv_v_scale) << (8 * i);
          col[d][tq] = w;
        }
      }
#pragma unroll
      for (int d = 0; d < 4; ++d)
        *reinterpret_cast<uint4*>(page + (long long)(d0 + d) * 16) = make_uint4(col[d][0], col[d][1], col[d][2], col[d][3]);
    }
    return;
  }
  for (int i = 0; i < 16 && t0 + i < p.T; ++i) {
    const int slot = __shfl_sync(0xffffffffu, my_slot, i);
    if (slot < 0) continue;
    uint8_t* vc = vc_all + ((long long)(slot / 16) * p.Hkv + hh) * (long long)D * 16 + (slot % 16);
    const __nv_bfloat16* src = p.v + (long long)(t0 + i) * p.ldv + hh * D;
    for (int e = lane; e < D; e += 32) vc[(long long)e * 16] = f32_to_fp8_e4m3(__bfloat162float(src[e]) * p.inv_v_scale);
  }
}

// y = rmsnorm(x) * w * silu(z), one warp per (token, head); x,z [T, H, D] with token strides
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ z,
                     long long ldz, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* y, long long ldy, int T, int H,
                     int D, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  if (unit >= (long long)T * H) return;
  const int t = (int)(unit / H), h = (int)(unit % H);
  const __nv_bfloat16* xr = x + t * ldx + h * D;
  const __nv_bfloat16* zr = z + t * ldz + h * D;
  float ss = 0.f;
  for (int e = lane * 2; e < D; e += 64) {
    float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + e));
    ss += f.x * f.x + f.y * f.y;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)D + eps);
  for (int e = lane * 2; e < D; e += 64) {
    float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + e));
    float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(zr + e));
    float2 wv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + e));
    const float a = f.x * rstd * wv.x * (g.x / (1.f + __expf(-g.x)));
    const float b = f.y * rstd * wv.y * (g.y / (1.f + __expf(-g.y)));
    *reinterpret_cast<__nv_bfloat162*>(y + t * ldy + h * D + e) = __floats2bfloat162_rn(a, b);
  }
}


// Per-row LoRA update ("batched gather matrix-vector"): y[t, col0 + n] += scaling_s * sum_r B_s[n, r] * (A_s[r, :] . x[t, :])
// with s = slot[t] (0 = no adapter: the row is left alone).  One CTA per row: warps take the r dot products of the
// shrink step round-robin, then every thread expands a strided set of output columns.
// Reference op replaced: kernels/gb10/common/lora_bgmv.cu (shrink / expand pair).
struct LoraParams {
  const __nv_bfloat16* A[8];     // [rank, K] per slot (index 0 unused)
  const __nv_bfloat16* B[8];     // [N, rank] per slot
  int rank[8];
  float scaling[8];
};

__global__ void __launch_bounds__(256)
lora_bgmv_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const long long* __restrict__ slot, const LoraParams lp,
                 __nv_bfloat16* y, long long ldy, int col0, int K, int N) {
  __shared__ float tvec[64];
  const int t = blockIdx.x;
  const int s = (int)slot[t];
  if (s <= 0 || s >= 8 || lp.A[s] == nullptr) return;
  const int rank = lp.rank[s];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + t * ldx;
  for (int r = warp; r < rank; r += 8) {
    const __nv_bfloat16* ar = lp.A[s] + (long long)r * K;
    float acc = 0.f;
    for (int k = lane * 2; k < K; k += 64) {
      const float2 xv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + k));
      const float2 av = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(ar + k));
      acc += xv.x * av.x + xv.y * av.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) tvec[r] = acc * lp.scaling[s];
  }
  __syncthreads();
  for (int n = threadIdx.x; n < N; n += 256) {
    const __nv_bfloat16* br = lp.B[s] + (long long)n * rank;
    float acc = 0.f;
    for (int r = 0; r < rank; ++r) acc += __bfloat162float(br[r]) * tvec[r];
    __nv_bfloat16* dst = y + t * ldy + col0 + n;
    *dst = __float2bfloat16_rn(__bfloat162float(*dst) + acc);
  }
}

// x[t, :] *= sigmoid(gate[t, :]) in place (the output gate of gated attention); n % 8 == 0
__global__ void __launch_bounds__(256)
sigmoid_gate_mul_kernel(__nv_bfloat16* x, long long ldx, const __nv_bfloat16* __restrict__ gate, long long ldg, int n) {
  const long long t = blockIdx.x;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < n; c += gridDim.y * blockDim.x * 8) {
    float xv[8], gv[8];
    load8(x + t * ldx + c, xv);
    load8(gate + t * ldg + c, gv);
#pragma unroll
    for (int i = 0; i < 8; ++i) xv[i] *= 1.f / (1.f + __expf(-gv[i]));
    store8(x + t * ldx + c, xv);
  }
}

// y[t, :] += s[t, :] * sigmoid(<x[t, :], wg>)   (shared expert behind a scalar gate); one CTA per row
__global__ void __launch_bounds__(256)
shared_expert_blend_kernel(__nv_bfloat16* y, long long ldy, const __nv_bfloat16* __restrict__ s, long long lds,
                           const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ wg, int H) {
  const long long t = blockIdx.x;
  __shared__ float red[8];
  float dot = 0.f;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float xv[8], wv[8];
    load8(x + t * ldx + c, xv);
    load8(wg + c, wv);
#pragma unroll
    for (int i = 0; i < 8; ++i) dot += xv[i] * wv[i];
  }
  dot = warp_sum(dot);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float g = 1.f / (1.f + __expf(-tot));
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float yv[8], sv[8];
    load8(y + t * ldy + c, yv);
    load8(s + t * lds + c, sv);
#pragma unroll
    for (int i = 0; i < 8; ++i) yv[i] += sv[i] * g;
    store8(y + t * ldy + c, yv);
  }
}

}  // namespace atlas

using namespace atlas;

extern "C" int atlas_rmsnorm(const void* x, long long ldx, const void* residual, long long ldr, const void* w,
                             void* res_out, long long ldro, void* y, long long ldy, void* q, long long ldq,
                             float* scale, long long scale_ld, int T, int H, float eps, int plus_one, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 || (q && H % 128)) return -1;
  int threads = ((H / 8 + 31) / 32) * 32;
  int iters = 1;
  while (threads > 1024) { iters *= 2; threads = (((H / 8 + iters - 1) / iters + 31) / 32) * 32; }
  if (q && threads % 16) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<const __nv_bfloat16*>(residual);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto RO = reinterpret_cast<__nv_bfloat16*>(res_out);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  auto Qp = reinterpret_cast<uint8_t*>(q);
  if (iters == 1) launch_chain_if(T <= 256, rmsnorm_kernel<1>, dim3(T), dim3(threads), 0, st, X, ldx, R, ldr, W, RO, ldro, Y, ldy, Qp, ldq, scale, scale_ld, H, eps, plus_one);
  else if (iters == 2) launch_chain_if(T <= 256, rmsnorm_kernel<2>, dim3(T), dim3(threads), 0, st, X, ldx, R, ldr, W, RO, ldro, Y, ldy, Qp, ldq, scale, scale_ld, H, eps, plus_one);
  else if (iters == 4) launch_chain_if(T <= 256, rmsnorm_kernel<4>, dim3(T), dim3(threads), 0, st, X, ldx, R, ldr, W, RO, ldro, Y, ldy, Qp, ldq, scale, scale_ld, H, eps, plus_one);
  else return -3;
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_silu_mul(const void* gu, long long ld, int T, int I, void* y, long long ldy, void* q,
                              long long ldq, float* scale, long long scale_ld, const int* live_tiles, void* stream) {
  if (T <= 0) return 0;
  if (I % 8 || (q && I % 128)) return -1;
  dim3 grid(T, (I / 8 + 255) / 256);
  launch_chain_if(T <= 256, silu_mul_kernel<0>, grid, dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(gu), ld, I, reinterpret_cast<__nv_bfloat16*>(y), ldy,
      reinterpret_cast<uint8_t*>(q), ldq, scale, scale_ld, live_tiles);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_gelu_tanh_mul(const void* gu, long long ld, int T, int I, void* y, long long ldy, void* q,
                                   long long ldq, float* scale, long long scale_ld, void* stream) {
  if (T <= 0) return 0;
  if (I % 8 || (q && I % 128)) return -1;
  dim3 grid(T, (I / 8 + 255) / 256);
  launch_chain_if(T <= 256, silu_mul_kernel<1>, grid, dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(gu), ld, I, reinterpret_cast<__nv_bfloat16*>(y), ldy,
      reinterpret_cast<uint8_t*>(q), ldq, scale, scale_ld, static_cast<const int*>(nullptr));
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_quant_fp8(const void* x, long long ld, int T, int K, void* q, long long ldq, float* scale,
                               long long scale_ld, void* stream) {
  if (T <= 0) return 0;
  if (K % 128) return -1;
  dim3 grid(T, (K / 8 + 255) / 256);
  launch_chain_if(T <= 256, quant_fp8_kernel, grid, dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(x), ld, K, reinterpret_cast<uint8_t*>(q), ldq, scale, scale_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_rope_kv_write(void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                                   const int* positions, const float* rope, const void* q_norm_w,
                                   const void* k_norm_w, void* k_cache, void* v_cache, const int* slot_mapping, int T,
                                   int Hq, int Hkv, int D, int rotary_dim, int block_size, int kv_fp8, int plus_one,
                                   float eps, float k_scale, float v_scale, void* stream) {
  if (T <= 0) return 0;
  if (D % 64 || D > 512 || rotary_dim > D || rotary_dim % 2) return -1;
  RopeKvParams p;
  p.q = reinterpret_cast<__nv_bfloat16*>(q); p.ldq = ldq;
  p.k = reinterpret_cast<const __nv_bfloat16*>(k); p.ldk = ldk;
  p.v = reinterpret_cast<const __nv_bfloat16*>(v); p.ldv = ldv;
  p.positions = positions; p.rope = rope;
  p.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(q_norm_w);
  p.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(k_norm_w);
  p.k_cache = k_cache; p.v_cache = v_cache; p.slot_mapping = slot_mapping;
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.rotary_dim = rotary_dim; p.block_size = block_size;
  p.rotate = (kv_fp8 & 8) ? 1 : 0;           // bit 3 of the cache mode asks for the Hadamard rotation
  kv_fp8 &= 7;
  p.kv_fp8 = kv_fp8; p.plus_one = plus_one; p.eps = eps; p.inv_k_scale = 1.f / k_scale; p.inv_v_scale = 1.f / v_scale;
  // prefill-size batches with 16-token FP8 pages: V goes through the page-row writer (16-byte stores)
  p.v_separate = (T >= 256 && kv_fp8 == 1 && !p.rotate && block_size == 16 && D % 4 == 0 && (ldv % 4) == 0 &&
                  (reinterpret_cast<uintptr_t>(v) & 7) == 0) ? 1 : 0;
  const long long units = (long long)T * (Hq + (p.v_separate ? 1 : 2) * Hkv);
  const int grid = (int)((units + 3) / 4);
  const bool d128 = D == 128 && rotary_dim == 128 && (ldq % 4) == 0 && (ldk % 4) == 0 && (ldv % 4) == 0 &&
                    ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(rope) & 15) == 0;
  if (p.rotate && !d128) return -2;                                   // so is the rotation
  if (kv_fp8 == 2 && (!d128 || block_size % 16)) return -2;          // the NVFP4 cache is written by the head_dim-128 kernel only
  if (d128)
    launch_chain_if(T <= 256, rope_kv_write_d128_kernel, dim3(grid), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), p);
  else
    launch_chain_if(T <= 256, rope_kv_write_kernel, dim3(grid), dim3(128), 4 * D * sizeof(float), reinterpret_cast<cudaStream_t>(stream), p);
  if (cudaGetLastError() != cudaSuccess) return -20;
  if (p.v_separate) {
    const long long vunits = (long long)((T + 15) / 16) * Hkv;
    launch_chain_if(false, v_write_pages_kernel, dim3((unsigned)((vunits + 3) / 4)), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_wht_d128(void* x, long long ld, int T, int H, void* stream) {
  if (T <= 0 || H <= 0) return 0;
  if ((ld % 4) || (reinterpret_cast<uintptr_t>(x) & 7)) return -1;
  const long long units = (long long)T * H;
  launch_chain_if(T <= 256, wht_d128_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream),
                  reinterpret_cast<__nv_bfloat16*>(x), ld, units, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_gated_rmsnorm(const void* x, long long ldx, const void* z, long long ldz, const void* w, void* y,
                                   long long ldy, int T, int H, int D, float eps, void* stream) {
  if (T <= 0) return 0;
  if (D % 2) return -1;
  const long long units = (long long)T * H;
  gated_rmsnorm_kernel<<<(int)((units + 3) / 4), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(z), ldz,
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(y), ldy, T, H, D, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

// LoRA update of y[:, col0 : col0 + N] in place; slot [T] int64 per row, per-slot A [rank,K] / B [N,rank] bf16 device
// pointers (arrays of 8, index 0 ignored), ranks <= 64, K even.
extern "C" int atlas_lora_bgmv(const void* x, long long ldx, const long long* slot, const void* const* A, const void* const* B,
                               const int* rank, const float* scaling, void* y, long long ldy, int col0, int T, int K, int N,
                               void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K % 2) return -1;
  LoraParams lp;
  for (int i = 0; i < 8; ++i) {
    lp.A[i] = reinterpret_cast<const __nv_bfloat16*>(A[i]);
    lp.B[i] = reinterpret_cast<const __nv_bfloat16*>(B[i]);
    lp.rank[i] = rank[i];
    lp.scaling[i] = scaling[i];
    if (rank[i] > 64) return -2;
  }
  lora_bgmv_kernel<<<T, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, slot, lp, reinterpret_cast<__nv_bfloat16*>(y), ldy, col0, K, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_sigmoid_gate_mul(void* x, long long ldx, const void* gate, long long ldg, int T, int n, void* stream) {
  if (T <= 0 || n <= 0) return 0;
  if (n % 8 || ldx % 8 || ldg % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(gate) & 15)) return -1;
  dim3 grid(T, (n / 8 + 255) / 256);
  sigmoid_gate_mul_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(gate), ldg, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

extern "C" int atlas_shared_expert_blend(void* y, long long ldy, const void* s, long long lds, const void* x, long long ldx,
                                         const void* wg, int T, int H, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 || ldy % 8 || lds % 8 || ldx % 8) return -1;
  shared_expert_blend_kernel<<<T, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(y), ldy, reinterpret_cast<const __nv_bfloat16*>(s), lds,
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(wg), H);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
