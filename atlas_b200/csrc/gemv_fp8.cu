// FP8 block-scaled GEMM for one to eight activation rows (single-stream and low-concurrency decode): the work is streaming
// the weight matrix once, and a 128-row tcgen05 tile spends its fixed cost (pipeline fill, TMEM round trip per K slice,
// split-K reduction) on a tile that is at most 6 % full.  Here the weights are the M operand of `mma.sync.m16n8k16`
// (16 rows per warp, converted e4m3 -> f16 in registers, exact), the activation rows the N operand, and K is split over
// CTAs so that several CTAs per SM keep loads in flight.
//
//   C[m, n] = sum_kb a_scale[kb, m] * b_scale[n / 128, kb] * sum_{k in kb} Aq[m, k] * Bq[n, k]
//
// Same two-level accumulation as the tcgen05 kernel: products inside a 128-wide K block are exact in fp32, the block is
// folded with its two scales.  Split-K partials go to a workspace; the CTA that takes the last ticket of a 64-row block
// adds them in split order (deterministic) and writes bf16.
// Reference ops replaced: kernels/gb10/common/fp8_gemv*.cu (single-token decode projections).
#include <cuda_fp8.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "host_api.h"

namespace atlas {

constexpr int kGvThreads = 128;
constexpr int kGvKc = 512;               // K elements staged per step (four scale blocks)
constexpr int kGvRow = kGvKc + 16;       // f16 per staged row: 264 words = 8 mod 32 -> conflict-free 8-byte reads

struct GemvParams {
  const uint8_t* a; long long lda;       // [M, K] e4m3
  const float* a_scale; long long sa_k;  // scale(m, kb) = a_scale[kb * sa_k + m]
  const uint8_t* b; long long ldb;       // [N, K] e4m3
  const float* b_scale; int b_scale_ld;  // [ceil(N/128), K/128]
  __nv_bfloat16* c; long long ldc;
  float* workspace;                      // [splits][8][N] fp32 (splits > 1)
  int* counters;                         // [N / 64], zero between launches
  int M, N, K, kb_per_split, splits;
};

ATLAS_DEVICE uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two_bytes & 0xFFFFu), __NV_E4M3);
  return *reinterpret_cast<uint32_t*>(&hr);
}
ATLAS_DEVICE void mma_f16_k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kGvThreads)
gemv_fp8_block_kernel(const GemvParams p) {
  __shared__ __align__(16) __half xs[8 * kGvRow];
  __shared__ int ticket_sm;
  chain_trigger();
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 64 + warp * 16;           // this warp's 16 weight rows
  const int split = blockIdx.y;
  const int k_blocks = p.K >> 7;
  const int kb_lo = split * p.kb_per_split, kb_hi = min(k_blocks, kb_lo + p.kb_per_split);
  const bool rows_live = row0 < p.N;                        // N % 16 == 0: a warp is all in or all out
  const uint8_t* w_lo = p.b + (long long)(row0 + g) * p.ldb + 16 * t;
  const uint8_t* w_hi = w_lo + 8 * p.ldb;
  const float* bs = p.b_scale + (long long)(row0 >> 7) * p.b_scale_ld;
  const int tok0 = 2 * t, tok1 = 2 * t + 1;                 // the two activation rows of this thread's accumulators
  float total[4] = {0.f, 0.f, 0.f, 0.f};

  for (int kc = kb_lo * 128; kc < kb_hi * 128; kc += kGvKc) {
    const int k_len = min(kGvKc, kb_hi * 128 - kc);
    __syncthreads();                                        // previous step's readers are done with xs
    // stage activations as f16 in (64-wide span, step s, lane t) order: the order the MMA steps consume a thread's bytes
    for (int i = threadIdx.x; i < 8 * (k_len >> 2); i += kGvThreads) {
      const int r = i / (k_len >> 2), q = i % (k_len >> 2);
      uint2 packed = make_uint2(0u, 0u);
      if (r < p.M) {
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(p.a + (long long)r * p.lda + kc + 4 * q);
        packed.x = e4m3x2_to_f16x2(raw);
        packed.y = e4m3x2_to_f16x2(raw >> 16);
      }
      const int kl = 4 * q;
      const int span = kl >> 6, in_span = kl & 63;
      const int tt = in_span >> 4, ss = (in_span & 15) >> 2;
      *reinterpret_cast<uint2*>(&xs[r * kGvRow + span * 64 + ss * 16 + tt * 4]) = packed;
    }
    __syncthreads();
    if (!rows_live) continue;
    // two scale blocks per iteration: all eight 16-byte weight loads are issued before the first conversion, so a warp
    // has 256 K elements of both of its row groups in flight
    for (int kb0 = 0; kb0 < (k_len >> 7); kb0 += 2) {
      const int nkb = min(2, (k_len >> 7) - kb0);
      uint4 wl[2][2], wh[2][2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u < nkb) {
#pragma unroll
          for (int sp = 0; sp < 2; ++sp) {
            wl[u][sp] = __ldg(reinterpret_cast<const uint4*>(w_lo + kc + (kb0 + u) * 128 + sp * 64));
            wh[u][sp] = __ldg(reinterpret_cast<const uint4*>(w_hi + kc + (kb0 + u) * 128 + sp * 64));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u >= nkb) break;
        const int kb = kb0 + u;
        const int kbg = (kc >> 7) + kb;
        float blk[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int sp = 0; sp < 2; ++sp) {
          const uint32_t lo[4] = {wl[u][sp].x, wl[u][sp].y, wl[u][sp].z, wl[u][sp].w};
          const uint32_t hi[4] = {wh[u][sp].x, wh[u][sp].y, wh[u][sp].z, wh[u][sp].w};
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const uint2 b = *reinterpret_cast<const uint2*>(&xs[g * kGvRow + (kb * 2 + sp) * 64 + s * 16 + t * 4]);
            mma_f16_k16(blk, e4m3x2_to_f16x2(lo[s]), e4m3x2_to_f16x2(hi[s]), e4m3x2_to_f16x2(lo[s] >> 16),
                        e4m3x2_to_f16x2(hi[s] >> 16), b.x, b.y);
          }
        }
        const float sb = __ldg(bs + kbg);
        const float s0 = tok0 < p.M ? __ldg(p.a_scale + (long long)kbg * p.sa_k + tok0) * sb : 0.f;
        const float s1 = tok1 < p.M ? __ldg(p.a_scale + (long long)kbg * p.sa_k + tok1) * sb : 0.f;
        total[0] = fmaf(blk[0], s0, total[0]);
        total[1] = fmaf(blk[1], s1, total[1]);
        total[2] = fmaf(blk[2], s0, total[2]);
        total[3] = fmaf(blk[3], s1, total[3]);
      }
    }
  }

  // ---- write out: total[0], total[1] = (row g, tokens 2t, 2t+1); total[2], total[3] = (row g + 8, same tokens)
  if (p.splits == 1) {
    if (rows_live) {
      if (tok0 < p.M) {
        p.c[(long long)tok0 * p.ldc + row0 + g] = __float2bfloat16_rn(total[0]);
        p.c[(long long)tok0 * p.ldc + row0 + g + 8] = __float2bfloat16_rn(total[2]);
      }
      if (tok1 < p.M) {
        p.c[(long long)tok1 * p.ldc + row0 + g] = __float2bfloat16_rn(total[1]);
        p.c[(long long)tok1 * p.ldc + row0 + g + 8] = __float2bfloat16_rn(total[3]);
      }
    }
    return;
  }
  float* ws = p.workspace + (long long)split * 8 * p.N;
  if (rows_live) {
    ws[(long long)tok0 * p.N + row0 + g] = total[0];
    ws[(long long)tok0 * p.N + row0 + g + 8] = total[2];
    ws[(long long)tok1 * p.N + row0 + g] = total[1];
    ws[(long long)tok1 * p.N + row0 + g + 8] = total[3];
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) ticket_sm = atomicAdd(&p.counters[blockIdx.x], 1);
  __syncthreads();
  if (ticket_sm != p.splits - 1) return;
  __threadfence();
  // last CTA of this 64-row block: add the partials in split order
  for (int i = threadIdx.x; i < p.M * 64; i += kGvThreads) {
    const int m = i >> 6, n = blockIdx.x * 64 + (i & 63);
    if (n >= p.N) continue;
    float sum = 0.f;
    for (int sp = 0; sp < p.splits; ++sp) sum += __ldcg(p.workspace + ((long long)sp * 8 + m) * p.N + n);
    p.c[(long long)m * p.ldc + n] = __float2bfloat16_rn(sum);
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;          // ready for the next launch
}

}  // namespace atlas

using namespace atlas;

// M <= 8, K % 128 == 0, N % 16 == 0, rows of A and B 16-byte aligned.  `workspace` needs splits * 8 * N floats and
// `counters` ceil(N / 64) zero-initialised ints when splits > 1.
extern "C" int atlas_gemv_fp8_block(const void* A, const void* B, void* C, const float* a_scale, long long sa_k,
                                    const float* b_scale, int b_scale_ld, int M, int N, int K, long long lda, long long ldb,
                                    long long ldc, int splits, float* workspace, int* counters, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 8 || (K % 128) || (N % 16)) return -1;
  if ((lda % 4) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) & 3) || (reinterpret_cast<uintptr_t>(B) & 15)) return -2;
  GemvParams p;
  p.a = reinterpret_cast<const uint8_t*>(A); p.lda = lda;
  p.a_scale = a_scale; p.sa_k = sa_k;
  p.b = reinterpret_cast<const uint8_t*>(B); p.ldb = ldb;
  p.b_scale = b_scale; p.b_scale_ld = b_scale_ld;
  p.c = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.workspace = workspace; p.counters = counters;
  p.M = M; p.N = N; p.K = K;
  const int k_blocks = K / 128;
  if (splits < 1) splits = 1;
  if (splits > k_blocks) splits = k_blocks;
  p.kb_per_split = (k_blocks + splits - 1) / splits;
  // whole staging steps per split keep every split's K range a multiple of the staged chunk, except the last one
  p.kb_per_split = (p.kb_per_split + 3) / 4 * 4;
  p.splits = (k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  if (p.splits > 1 && (!workspace || !counters)) return -5;
  dim3 grid((N + 63) / 64, p.splits);
  launch_chain(gemv_fp8_block_kernel, grid, dim3(kGvThreads), 0, reinterpret_cast<cudaStream_t>(stream), p);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
