// Decode-size MoE expert GEMMs on NVFP4 weights: a few rows per expert (batch x top-k spread over all experts), so the
// work is streaming every touched expert's packed weights once.  The 128-row tcgen05 tile of the grouped kernel is ~6 %
// full there and pays a shared-memory round trip per converted weight; here the weights are the MMA's M operand
// (16 rows per warp), the expert's tokens the N operand (8 per `mma.sync.m16n8k16`), and FP4 -> f16 happens in
// registers on the way from global memory to the tensor core.
//
//   mode 1  a[row, j]  = silu(x[token(row)] . Wg[j]) * (x[token(row)] . Wu[j])      W13 = [E][2I][K/2], rows gathered by token
//   mode 0  y[row, n]  = a[row] . W2[n]                                              W2  = [E][H][K/2]
//
// Rows live in the expert-sorted, 128-row padded buffer built by moe_align (tile i belongs to expert tile_expert[i],
// its live rows are the leading ones with row_token >= 0), so align and combine are shared with the grouped path.
// One CTA = one tile x 64 weight rows (mode 1: 32 gate rows + the matching 32 up rows).  Per 128-wide K span a thread
// loads 16 bytes (32 weights) of each of its two rows; k is assigned to MMA slots so that those bytes are used in place:
// step s of the span takes the thread's weights 4s..4s+3, and the activation tile is staged in shared memory in the
// same order.  Block scales multiply the f16 weights (exact), the per-row global scale the fp32 result.
// Reference ops replaced: moe_w4a16_grouped_gemv*.cu / w4a16_gemv*.cu (kernels/gb10/common).
#include <cuda_fp4.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "host_api.h"

namespace atlas {

constexpr int kSmThreads = 128;
constexpr int kSmTokens = 32;          // tokens per pass (four n8 tiles)
constexpr int kSmKc = 256;             // K elements staged per step (two 128-wide spans)
constexpr int kSmRow = kSmKc + 16;     // f16 per staged token row: 136 words, so 8 tokens x 4 lanes hit distinct banks

struct SmallMoeParams {
  const __nv_bfloat16* x; long long ldx;
  const int* row_token;
  const int* tile_expert;
  const int* num_tiles;
  const uint8_t* w;        // [E][N][K/2]
  const uint8_t* sc;       // [E*N][K/16] e4m3
  const float* gs;         // [E*N]
  __nv_bfloat16* out; long long ldo;
  int K, N, I;
};

ATLAS_DEVICE uint32_t fp4x2_scaled(uint32_t byte, __half2 sc) {
  __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xFFu), __NV_E2M1);
  __half2 h = __hmul2(*reinterpret_cast<__half2*>(&hr), sc);
  return *reinterpret_cast<uint32_t*>(&h);
}
ATLAS_DEVICE __half2 e4m3_half2(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(byte & 0xFFu), __NV_E4M3);
  return __half2half2(*reinterpret_cast<__half*>(&h));
}
ATLAS_DEVICE void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MODE>
__global__ void __launch_bounds__(kSmThreads)
moe_small_w4_kernel(const SmallMoeParams p) {
  __shared__ __align__(16) __half xs[kSmTokens * kSmRow];
  __shared__ float ex[MODE == 1 ? 2 * 32 * (kSmTokens + 1) : 1];
  __shared__ int tok_sm[128];
  __shared__ int n_live_sm;
  const int tile = blockIdx.y;
  if (tile >= *p.num_tiles) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int e = p.tile_expert[tile];
  // live rows of the tile: the leading ones
  {
    const int tok = p.row_token[tile * 128 + threadIdx.x];
    tok_sm[threadIdx.x] = tok;
    const int cnt = __syncthreads_count(tok >= 0);
    if (threadIdx.x == 0) n_live_sm = cnt;
  }
  __syncthreads();
  const int n_live = n_live_sm;
  if (n_live == 0) return;
  // the two weight rows of this thread (g and g + 8 of the warp's 16)
  int row0;
  if (MODE == 1) row0 = (warp < 2 ? 0 : p.I) + blockIdx.x * 32 + (warp & 1) * 16;
  else           row0 = blockIdx.x * 64 + warp * 16;
  const long long wrow = (long long)e * p.N + row0 + g;
  const uint8_t* w_lo = p.w + wrow * (p.K >> 1) + 16 * t;
  const uint8_t* w_hi = w_lo + 8ll * (p.K >> 1);
  const uint8_t* s_lo = p.sc + wrow * (p.K >> 4) + 2 * t;
  const uint8_t* s_hi = s_lo + 8ll * (p.K >> 4);
  const float gs_lo = p.gs[wrow], gs_hi = p.gs[wrow + 8];

  for (int pass0 = 0; pass0 < n_live; pass0 += kSmTokens) {
    const int n_tok = min(kSmTokens, n_live - pass0);
    const int n_nt = (n_tok + 7) >> 3;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    for (int k0 = 0; k0 < p.K; k0 += kSmKc) {
      // weights of this step first: their latency overlaps the activation staging below
      uint4 wl[2], wh[2];
      uint32_t sl[2], sh[2];
#pragma unroll
      for (int sp = 0; sp < 2; ++sp) {
        const int kb = (k0 >> 1) + sp * 64;
        wl[sp] = __ldg(reinterpret_cast<const uint4*>(w_lo + kb));
        wh[sp] = __ldg(reinterpret_cast<const uint4*>(w_hi + kb));
        sl[sp] = __ldg(reinterpret_cast<const unsigned short*>(s_lo + (k0 >> 4) + sp * 8));
        sh[sp] = __ldg(reinterpret_cast<const unsigned short*>(s_hi + (k0 >> 4) + sp * 8));
      }
      __syncthreads();                       // previous step's readers are done with xs
      // stage activations: token r, k = k0 + 4q .. 4q+3 -> position (span, step s, lane t) order
      for (int i = threadIdx.x; i < n_nt * 8 * (kSmKc / 4); i += kSmThreads) {
        const int r = i / (kSmKc / 4), q = i % (kSmKc / 4);
        uint2 packed = make_uint2(0u, 0u);
        if (r < n_tok) {
          const int row = tile * 128 + pass0 + r;
          const __nv_bfloat16* src = MODE == 1 ? p.x + (long long)tok_sm[pass0 + r] * p.ldx : p.x + (long long)row * p.ldx;
          const uint2 raw = *reinterpret_cast<const uint2*>(src + k0 + 4 * q);
          const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
          const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
          const __half2 h0 = __floats2half2_rn(fminf(fmaxf(f0.x, -65504.f), 65504.f), fminf(fmaxf(f0.y, -65504.f), 65504.f));
          const __half2 h1 = __floats2half2_rn(fminf(fmaxf(f1.x, -65504.f), 65504.f), fminf(fmaxf(f1.y, -65504.f), 65504.f));
          packed.x = *reinterpret_cast<const uint32_t*>(&h0);
          packed.y = *reinterpret_cast<const uint32_t*>(&h1);
        }
        const int kl = 4 * q;                                  // k inside the step
        const int span = kl >> 7, in_span = kl & 127;
        const int tt = in_span >> 5, ss = (in_span & 31) >> 2;
        *reinterpret_cast<uint2*>(&xs[r * kSmRow + span * 128 + ss * 16 + tt * 4]) = packed;
      }
      __syncthreads();
#pragma unroll
      for (int sp = 0; sp < 2; ++sp) {
        const uint32_t wl_[4] = {wl[sp].x, wl[sp].y, wl[sp].z, wl[sp].w};
        const uint32_t wh_[4] = {wh[sp].x, wh[sp].y, wh[sp].z, wh[sp].w};
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const __half2 scl = e4m3_half2(sl[sp] >> (8 * (s >> 2)));
          const __half2 sch = e4m3_half2(sh[sp] >> (8 * (s >> 2)));
          const uint32_t lo16 = wl_[s >> 1] >> (16 * (s & 1));
          const uint32_t hi16 = wh_[s >> 1] >> (16 * (s & 1));
          const uint32_t a0 = fp4x2_scaled(lo16, scl), a2 = fp4x2_scaled(lo16 >> 8, scl);
          const uint32_t a1 = fp4x2_scaled(hi16, sch), a3 = fp4x2_scaled(hi16 >> 8, sch);
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            if (nt < n_nt) {
              const uint2 b = *reinterpret_cast<const uint2*>(&xs[(nt * 8 + g) * kSmRow + sp * 128 + s * 16 + t * 4]);
              mma_f16(acc[nt], a0, a1, a2, a3, b.x, b.y);
            }
          }
        }
      }
    }
    // ---- epilogue: c0,c1 = (row g, tokens 2t, 2t+1), c2,c3 = (row g+8, same tokens)
    if (MODE == 0) {
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int tok = nt * 8 + 2 * t + j;
          if (tok < n_tok) {
            __nv_bfloat16* o = p.out + (long long)(tile * 128 + pass0 + tok) * p.ldo + row0 + g;
            o[0] = __float2bfloat16_rn(acc[nt][j] * gs_lo);
            o[8] = __float2bfloat16_rn(acc[nt][2 + j] * gs_hi);
          }
        }
      }
    } else {
      __syncthreads();
      const int which = warp >> 1;                 // 0 = gate, 1 = up
      const int col = (warp & 1) * 16 + g;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int tok = nt * 8 + 2 * t + j;
          ex[(which * 32 + col) * (kSmTokens + 1) + tok] = acc[nt][j] * gs_lo;
          ex[(which * 32 + col + 8) * (kSmTokens + 1) + tok] = acc[nt][2 + j] * gs_hi;
        }
      }
      __syncthreads();
      for (int i = threadIdx.x; i < n_tok * 32; i += kSmThreads) {
        const int tok = i >> 5, c = i & 31;
        // round gate and up to bf16 first, like the unfused GEMM -> SiLU chain does
        const float gv = __bfloat162float(__float2bfloat16_rn(ex[c * (kSmTokens + 1) + tok]));
        const float uv = __bfloat162float(__float2bfloat16_rn(ex[(32 + c) * (kSmTokens + 1) + tok]));
        const float sv = gv / (1.f + __expf(-gv)) * uv;
        p.out[(long long)(tile * 128 + pass0 + tok) * p.ldo + blockIdx.x * 32 + c] = __float2bfloat16_rn(sv);
      }
    }
  }
}

}  // namespace atlas

using namespace atlas;

// mode 1: x [T, K] token rows (gathered through row_token), out [max_rows, I] = silu(gate) * up, N = 2 I rows per expert
// mode 0: x [max_rows, K] sorted rows, out [max_rows, N]
// K % 256 == 0; mode 1: I % 32 == 0; mode 0: N % 64 == 0.  max_tiles bounds the grid; CTAs past *num_tiles return.
extern "C" int atlas_moe_small_w4(int mode, const void* x, long long ldx, const int* row_token, const int* tile_expert,
                                  const int* num_tiles, int max_tiles, const void* w, const void* sc, const float* gs,
                                  void* out, long long ldo, int K, int N, void* stream) {
  if (max_tiles <= 0) return 0;
  if (K % kSmKc || (ldx % 4)) return -1;
  SmallMoeParams p;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x); p.ldx = ldx;
  p.row_token = row_token; p.tile_expert = tile_expert; p.num_tiles = num_tiles;
  p.w = reinterpret_cast<const uint8_t*>(w); p.sc = reinterpret_cast<const uint8_t*>(sc); p.gs = gs;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.K = K; p.N = N; p.I = N / 2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mode == 1) {
    if (N % 64) return -2;
    moe_small_w4_kernel<1><<<dim3(p.I / 32, max_tiles), kSmThreads, 0, st>>>(p);
  } else {
    if (N % 64) return -2;
    moe_small_w4_kernel<0><<<dim3(N / 64, max_tiles), kSmThreads, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
