// Paged attention over the FP8 KV cache.
//
//   decode  : one CTA per (kv head, k-split, sequence).  The G = Hq/Hkv query heads that share the kv head are
//             packed into the M rows of the tensor-core tile (GQA packing), the CTA's four warps take alternating
//             16-token pages of the split's range, keep online-softmax state in registers and are merged through
//             shared memory; splits are merged by a second tiny kernel (flash-decoding).
//   prefill : one warp per 16 query rows of one head; loops causally over the sequence's pages.
//
// K pages are [block_size, D] row-major per head, V pages are stored transposed [D, block_size] (see
// elementwise.cu).  FP8 bytes are widened to f16 in registers (cvt.f16x2.e4m3x2) and fed to
// mma.sync.m16n8k16; the head-dim (for QK^T) and token (for PV) indices are permuted so that every thread reads
// contiguous 16/4-byte pieces and the C fragment of QK^T is directly the A fragment of PV:
//   * QK^T k-index: thread c = lane%4 owns dims [c*D/4, (c+1)*D/4); k-step ks uses its bytes ks*4..ks*4+3.
//   * token <-> n-column inside a 16-token page: tile i (0/1), column j  <->  token (j/2)*4 + 2*i + j%2,
//     so a thread's four P values of a row are tokens c*4 .. c*4+3, exactly one 32-bit word of a V^T row.
// The FP8 K scale is folded into the query scaling, the V scale into the final normalisation (hoisted out of the
// loop like the reference's paged_decode_attn_fp8.cu:42-48).
//
// Reference ops replaced: kernels/gb10/common/paged_decode_attn*.cu (SIMT), inferspark_prefill_paged_fp8.cu.
#include "common.cuh"
#include "host_api.h"
#include "no_alloc_api.h"

namespace atlas {

struct AttnParams {
  const __nv_bfloat16* q; long long ldq;       // [T, Hq, D], token stride ldq
  __nv_bfloat16* out; long long ldo;           // [T, Hq, D]
  const uint8_t* k_cache; const uint8_t* v_cache;
  const int* block_tables; int bt_ld;
  const int* seq_lens; const int* query_start_loc;
  int seq_base;                                 // index of the first sequence this launch covers
  float qk_scale_log2;                          // softmax scale * k_scale * log2(e)
  float v_scale;
  int Hq, Hkv, block_size, window;
  // decode
  int num_splits;
  float* part_o;                                // [B, Hq, splits, D]
  float* part_ml;                               // [B, Hq, splits, 2]
  // prefill
  const int* tile_seq; const int* tile_q0; int num_tiles;
  // decode, D == 128 only: write the output as FP8 with one scale per (row, head) -- a head is one 128-wide quantisation
  // group of the output projection's A operand -- instead of bf16 `out`.  Scale of (row, head) at s_out[head * s_ld + row].
  uint8_t* q_out; long long ldqo;
  float* s_out; long long s_ld;
};

ATLAS_DEVICE void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
ATLAS_DEVICE uint32_t fp8x2_to_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(r) : "h"(v));
  return r;
}
ATLAS_DEVICE uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
ATLAS_DEVICE void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// KV16: the cache holds bf16 (two bytes per element, same page layouts); queries, probabilities and the cache then meet
// in bf16 MMAs and no scale applies.  Otherwise FP8 e4m3 bytes widened to f16.
// KV4: NVFP4 cache.  A (block, kv head) page of K is [bs][D/2] packed e2m1 bytes (even dim in the low nibble) followed by
// [bs][D/16] e4m3 scales (one per token and 16 dims); a page of V is [D][bs/2] packed bytes (even TOKEN in the low nibble)
// followed by [D/16][bs] scales (one per token and 16 dims, token-contiguous).  Both pages are bs * D * 9 / 16 bytes.  K is
// widened to f16 and multiplied by its scale element by element (a k-step spans four scale groups); V's scales depend on
// the token only inside a 16-dim group, so they are folded into the P operand, once per two n-tiles.
ATLAS_DEVICE uint32_t e2m1x2_to_f16x2(uint32_t byte) {
  uint32_t r;
  asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}\n" : "=r"(r) : "r"(byte));
  return r;
}
ATLAS_DEVICE uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <int D, bool PREFILL, bool KV16 = false, bool KV4 = false>
__global__ void __launch_bounds__(128)
paged_attn_kernel(const AttnParams p) {
  constexpr int ES = KV16 ? 2 : 1;      // bytes per cache element (KV4 computes its own offsets)
  constexpr int KS = D / 16;            // k-steps of QK^T
  constexpr int NT = D / 8;             // n-tiles of PV
  constexpr int DQ = D / 4;             // dims owned by one thread of a quad
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = lane & 3, rq = lane >> 2;
  const int G = p.Hq / p.Hkv;

  int b, kvh, q_row0, q_len, L, qhead = 0, tile_q0 = 0, split = 0;
  if (PREFILL) {
    const int tile = blockIdx.x * 4 + warp;
    if (tile >= p.num_tiles) return;
    b = p.tile_seq[tile];
    tile_q0 = p.tile_q0[tile];
    qhead = blockIdx.y;
    kvh = qhead / G;
  } else {
    b = p.seq_base + blockIdx.z;
    kvh = blockIdx.x;
    split = blockIdx.y;
  }
  L = p.seq_lens[b];
  q_row0 = p.query_start_loc[b];
  q_len = p.query_start_loc[b + 1] - q_row0;

  // ---- query fragments (scaled, f16)
  uint32_t qf[KS][4];
  {
    const __nv_bfloat16* qrow[2] = {nullptr, nullptr};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rq + 8 * h;
      if (PREFILL) {
        if (tile_q0 + r < q_len) qrow[h] = p.q + (long long)(q_row0 + tile_q0 + r) * p.ldq + qhead * D;
      } else {
        if (r < G) qrow[h] = p.q + (long long)q_row0 * p.ldq + (kvh * G + r) * D;
      }
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (qrow[h]) {
          const uint2 raw = *reinterpret_cast<const uint2*>(qrow[h] + c * DQ + ks * 4);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          v[0] = __low2float(lo) * p.qk_scale_log2; v[1] = __high2float(lo) * p.qk_scale_log2;
          v[2] = __low2float(hi) * p.qk_scale_log2; v[3] = __high2float(hi) * p.qk_scale_log2;
        }
        qf[ks][h] = KV16 ? pack_bf16x2(v[0], v[1]) : pack_f16x2(v[0], v[1]);         // a0 / a1 : k = c*2 + {0,1}
        qf[ks][2 + h] = KV16 ? pack_bf16x2(v[2], v[3]) : pack_f16x2(v[2], v[3]);     // a2 / a3 : k = c*2 + 8 + {0,1}
      }
    }
  }

  // ---- page range
  const int n_pages = (L + 15) >> 4;
  int pg_begin, pg_end, pg_step;
  int qpos[2];                                       // absolute position of this thread's two rows (causal bound)
  if (PREFILL) {
    const int first_pos = L - q_len + tile_q0;
    qpos[0] = first_pos + rq;
    qpos[1] = first_pos + rq + 8;
    const int last_pos = min(L - 1, first_pos + 15);
    pg_begin = 0;
    if (p.window > 0) pg_begin = max(0, first_pos - p.window + 1) >> 4;
    pg_end = (last_pos >> 4) + 1;
    pg_step = 1;
  } else {
    qpos[0] = qpos[1] = L - 1;
    const int per_split = (n_pages + p.num_splits - 1) / p.num_splits;
    int lo = split * per_split;
    if (p.window > 0) lo = max(lo, max(0, L - p.window) >> 4);
    pg_begin = lo + warp;
    pg_end = min(n_pages, (split + 1) * per_split);
    pg_step = 4;
  }

  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int* bt = p.block_tables + (long long)b * p.bt_ld;
  const int bs = p.block_size;

  for (int pg = pg_begin; pg < pg_end; pg += pg_step) {
    const int tok0 = pg << 4;
    const int blk = bt[tok0 / bs];
    const int off = tok0 % bs;
    const uint8_t* kpage = p.k_cache + ((((long long)blk * p.Hkv + kvh) * bs + off) * D) * ES;
    const uint8_t* vpage = p.v_cache + (((long long)blk * p.Hkv + kvh) * (long long)D * bs + off) * ES;
    // NVFP4: start of this (block, kv head)'s K and V pages
    const long long page4 = ((long long)blk * p.Hkv + kvh) * ((long long)bs * D * 9 / 16);

    // ---- S = Q K^T for the 16 tokens of this page
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      const int tok_in_page = (rq >> 1) * 4 + 2 * i + (rq & 1);
      const uint4* krow = reinterpret_cast<const uint4*>(kpage + (tok_in_page * D + c * DQ) * ES);
      if constexpr (KV4) {
        // this thread's DQ dims of the token: DQ / 2 packed bytes and DQ / 16 scales (k-step ks uses bytes 2 ks, 2 ks + 1)
        const uint8_t* kd = p.k_cache + page4 + (long long)(off + tok_in_page) * (D / 2) + c * (DQ / 2);
        const uint8_t* ksc = p.k_cache + page4 + (long long)bs * (D / 2) + (long long)(off + tok_in_page) * (D / 16) + c * (DQ / 16);
#pragma unroll
        for (int g = 0; g < DQ / 16; ++g) {
          const uint32_t s2 = fp8x2_to_f16x2((uint16_t)(ksc[g] * 0x0101u));          // the scale in both halves
          const uint2 raw = __ldg(reinterpret_cast<const uint2*>(kd) + g);               // 16 dims = four k-steps
          const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
          for (int wi = 0; wi < 4; ++wi) {
            const uint32_t two = (w[wi >> 1] >> (16 * (wi & 1))) & 0xFFFFu;
            const uint32_t b0 = hmul2_u32(e2m1x2_to_f16x2(two & 0xFFu), s2);
            const uint32_t b1 = hmul2_u32(e2m1x2_to_f16x2(two >> 8), s2);
            mma_f16(s[i], qf[g * 4 + wi], b0, b1);
          }
        }
      } else if constexpr (KV16) {
#pragma unroll
        for (int v4 = 0; v4 < DQ / 8; ++v4) {          // eight bf16 = two k-steps
          const uint4 raw = __ldg(krow + v4);
          mma_bf16(s[i], qf[v4 * 2], raw.x, raw.y);
          mma_bf16(s[i], qf[v4 * 2 + 1], raw.z, raw.w);
        }
      } else {
#pragma unroll
      for (int v4 = 0; v4 < DQ / 16; ++v4) {
        const uint4 raw = __ldg(krow + v4);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint32_t b0 = fp8x2_to_f16x2((uint16_t)(w[wi] & 0xFFFFu));
          const uint32_t b1 = fp8x2_to_f16x2((uint16_t)(w[wi] >> 16));
          mma_f16(s[i], qf[v4 * 4 + wi], b0, b1);
        }
      }
      }
    }
    // ---- mask + online softmax.  s[i][j] (row rq) and s[i][2+j] (row rq+8) belong to token tok0 + c*4 + 2i + j.
    float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int tok = tok0 + c * 4 + 2 * i + j;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          bool ok = tok <= qpos[h] && tok < L;
          if (p.window > 0) ok = ok && tok > qpos[h] - p.window;
          float& sv = s[i][2 * h + j];
          sv = ok ? sv : -INFINITY;
          mx[h] = fmaxf(mx[h], sv);
        }
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      alpha[h] = (mx[h] == -INFINITY) ? 1.f : exp2f(m_run[h] - mx[h]);
      m_run[h] = mx[h];
      l_run[h] *= alpha[h];
    }
    uint32_t pf[4];
    {
      float pv[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const float x = (mx[h] == -INFINITY) ? 0.f : exp2f(s[i][e] - mx[h]);
          pv[i][e] = x;
          l_run[h] += x;
        }
      if (KV16) {
        pf[0] = pack_bf16x2(pv[0][0], pv[0][1]); pf[1] = pack_bf16x2(pv[0][2], pv[0][3]);
        pf[2] = pack_bf16x2(pv[1][0], pv[1][1]); pf[3] = pack_bf16x2(pv[1][2], pv[1][3]);
      } else {
        pf[0] = pack_f16x2(pv[0][0], pv[0][1]);
        pf[1] = pack_f16x2(pv[0][2], pv[0][3]);
        pf[2] = pack_f16x2(pv[1][0], pv[1][1]);
        pf[3] = pack_f16x2(pv[1][2], pv[1][3]);
      }
    }
    // tokens past the sequence end may hold stale bytes: zero them so 0 * garbage cannot produce NaN
    uint32_t vmask = 0xFFFFFFFFu;
    {
      const int first = tok0 + c * 4;
      if (first + 3 >= L) {
        vmask = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (first + j < L) vmask |= 0xFFu << (8 * j);
      }
    }
    // ---- O = alpha * O + P V
    uint32_t pfs[4] = {pf[0], pf[1], pf[2], pf[3]};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      uint32_t b0, b1;
      if constexpr (KV4) {
        const uint32_t m0 = ((vmask & 0xFFu) ? 0xFFFFu : 0u) | ((vmask & 0xFF00u) ? 0xFFFF0000u : 0u);
        const uint32_t m1 = ((vmask & 0xFF0000u) ? 0xFFFFu : 0u) | ((vmask & 0xFF000000u) ? 0xFFFF0000u : 0u);
        if ((j & 1) == 0) {
          // scales of this thread's four tokens for dims [8 j, 8 j + 16): folded into P (stale scale bytes of tokens past
          // the end are masked like the data)
          const uint32_t sw = __ldg(reinterpret_cast<const uint32_t*>(p.v_cache + page4 + (long long)D * (bs / 2) +
                                                                       (long long)(j >> 1) * bs + off + c * 4)) & vmask;
          const uint32_t s01 = fp8x2_to_f16x2((uint16_t)(sw & 0xFFFFu)), s23 = fp8x2_to_f16x2((uint16_t)(sw >> 16));
          pfs[0] = hmul2_u32(pf[0], s01); pfs[1] = hmul2_u32(pf[1], s01);
          pfs[2] = hmul2_u32(pf[2], s23); pfs[3] = hmul2_u32(pf[3], s23);
        }
        const uint32_t two = __ldg(reinterpret_cast<const uint16_t*>(p.v_cache + page4 + (long long)(j * 8 + rq) * (bs / 2) +
                                                                      ((off + c * 4) >> 1)));
        b0 = e2m1x2_to_f16x2(two & 0xFFu) & m0;
        b1 = e2m1x2_to_f16x2(two >> 8) & m1;
      } else if constexpr (KV16) {
        // four bf16 of one V^T row; vmask carries one byte flag per token, widened here to 16-bit lanes
        const uint2 w2 = __ldg(reinterpret_cast<const uint2*>(vpage + ((long long)(j * 8 + rq) * bs + c * 4) * 2));
        const uint32_t m0 = ((vmask & 0xFFu) ? 0xFFFFu : 0u) | ((vmask & 0xFF00u) ? 0xFFFF0000u : 0u);
        const uint32_t m1 = ((vmask & 0xFF0000u) ? 0xFFFFu : 0u) | ((vmask & 0xFF000000u) ? 0xFFFF0000u : 0u);
        b0 = w2.x & m0;
        b1 = w2.y & m1;
      } else {
      const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(vpage + (long long)(j * 8 + rq) * bs + c * 4)) & vmask;
      b0 = fp8x2_to_f16x2((uint16_t)(word & 0xFFFFu));
      b1 = fp8x2_to_f16x2((uint16_t)(word >> 16));
      }
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
      o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
      if (KV16) mma_bf16(o[j], pf, b0, b1); else if (KV4) mma_f16(o[j], pfs, b0, b1); else mma_f16(o[j], pf, b0, b1);
    }
  }
  // quad-reduce the row sums
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  if (PREFILL) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rq + 8 * h;
      if (tile_q0 + r >= q_len) continue;
      const float inv = l_run[h] > 0.f ? p.v_scale / l_run[h] : 0.f;
      __nv_bfloat16* orow = p.out + (long long)(q_row0 + tile_q0 + r) * p.ldo + qhead * D;
#pragma unroll
      for (int j = 0; j < NT; ++j)
        *reinterpret_cast<__nv_bfloat162*>(orow + j * 8 + c * 2) =
            __floats2bfloat162_rn(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
    }
    return;
  } else {
    // ---- merge the four warps through shared memory
    extern __shared__ float sm[];
    float* sm_m = sm;                    // [4][16]
    float* sm_l = sm + 64;               // [4][16]
    float* sm_o = sm + 128;              // [4][16][D]
    if (c == 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sm_m[warp * 16 + rq + 8 * h] = m_run[h];
        sm_l[warp * 16 + rq + 8 * h] = l_run[h];
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rq + 8 * h;
      if (r < G) {
        float* dst = sm_o + ((warp * 16 + r) * D);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          dst[j * 8 + c * 2] = o[j][2 * h];
          dst[j * 8 + c * 2 + 1] = o[j][2 * h + 1];
        }
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += 128) {
      const int r = idx / D, d = idx % D;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) m = fmaxf(m, sm_m[w * 16 + r]);
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = sm_m[w * 16 + r];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
        acc += f * sm_o[(w * 16 + r) * D + d];
        l += f * sm_l[w * 16 + r];
      }
      const int head = kvh * G + r;
      if (p.num_splits == 1) {
        const float inv = l > 0.f ? p.v_scale / l : 0.f;
        p.out[(long long)q_row0 * p.ldo + head * D + d] = __float2bfloat16_rn(acc * inv);
      } else {
        const long long pi = ((long long)(b - p.seq_base) * p.Hq + head) * p.num_splits + split;
        p.part_o[pi * D + d] = acc;
        if (d == 0) {
          p.part_ml[pi * 2] = m;
          p.part_ml[pi * 2 + 1] = l;
        }
      }
    }
  }
}

// ----------------------------------------------------------------------------- decode (bulk-copy pipeline)
// One CTA per (kv head, k-split, sequence): warp 4 streams whole KV blocks of that head (K block and V^T block are
// each one contiguous region) into a shared-memory ring with cp.async.bulk + mbarriers; warps 0..3 take the
// blocks round-robin and keep online-softmax state in registers.
//
// The tensor-core tiles are oriented with TOKENS on the M dimension and the (up to 8) query heads that share the
// kv head on N:   S^T[16 tok x 8 heads] = K[16 x D] * Q^T[D x 8],   O^T[D x 8 heads] += V^T[D x 16 tok] * P^T[16 x 8].
// K and V^T are the A operands (FP8 bytes widened pairwise to f16), Q^T lives in registers as B fragments, and
// P^T is obtained from the S^T accumulator with two movmatrix transposes.  Token <-> row mapping inside a
// 16-token page: row r <-> token (r%8/2)*4 + 2*(r/8) + r%2, which makes every thread's fragment bytes contiguous.
constexpr int kDecodeThreads = 160;
constexpr int kBtSmemEntries = 1024;

ATLAS_DEVICE void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// four e4m3 bytes -> two f16x2 registers (bytes 0,1 and bytes 2,3)
ATLAS_DEVICE void fp8x4_to_f16x2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}
ATLAS_DEVICE uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
  return r;
}

// Tail of the decode kernels: merge the four consumer warps' online-softmax states through shared memory (the KV ring is
// dead by then) and write the rows out: bf16, FP8 + per-head scale, or split-K partials.  `o` holds O^T fragments (rows =
// dims mt*16 + rq (+8), columns = heads 2c, 2c+1); `acc_scale` undoes a fixed scaling of the P operand.
template <int D>
ATLAS_DEVICE void decode_merge_store(const AttnParams& p, uint8_t* ring, const float (&o)[D / 16][4], const float (&m_run)[2],
                                     const float (&l_run)[2], int warp, int lane, int G, int kvh, int split, int b, int q_row0,
                                     float acc_scale) {
  constexpr int MT = D / 16;
  const int c = lane & 3, rq = lane >> 2;
  // ---- merge the four consumer warps (the ring is dead now; reuse it)
  __syncthreads();
  float* sm_m = reinterpret_cast<float*>(ring);          // [4][8]
  float* sm_l = sm_m + 32;                               // [4][8]
  float* sm_o = sm_m + 64;                               // [4][8][D]
  if (warp < 4) {
    if (rq == 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sm_m[warp * 8 + c * 2 + h] = m_run[h];
        sm_l[warp * 8 + c * 2 + h] = l_run[h];
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int head = c * 2 + (e & 1);
        const int dim = mt * 16 + rq + 8 * (e >> 1);
        if (head < G) sm_o[(warp * 8 + head) * D + dim] = o[mt][e];
      }
  }
  const bool q8 = p.q_out != nullptr && p.num_splits == 1;
  int* sm_amax = reinterpret_cast<int*>(sm_o + 4 * 8 * D);            // [8] per-head max |output| (float bits, >= 0)
  if (q8 && threadIdx.x < 8) sm_amax[threadIdx.x] = 0;
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += (int)blockDim.x) {
    const int r = idx / D, d = idx % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, sm_m[w * 8 + r]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm_m[w * 8 + r];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      acc += f * sm_o[(w * 8 + r) * D + d] * acc_scale;
      l += f * sm_l[w * 8 + r];
    }
    const int head = kvh * G + r;
    if (q8) {
      // a warp's 32 consecutive idx lie inside one head (D and the thread count are multiples of 32): the value is
      // parked in the first warp's slot, which only this thread reads, and the head's maximum is gathered per warp
      const float inv = l > 0.f ? p.v_scale / l : 0.f;
      const float v = __bfloat162float(__float2bfloat16_rn(acc * inv));
      sm_o[r * D + d] = v;
      float a = fabsf(v);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
      if (lane == 0) atomicMax(&sm_amax[r], __float_as_int(a));
    } else if (p.num_splits == 1) {
      const float inv = l > 0.f ? p.v_scale / l : 0.f;
      p.out[(long long)q_row0 * p.ldo + head * D + d] = __float2bfloat16_rn(acc * inv);
    } else {
      const long long pi = ((long long)(b - p.seq_base) * p.Hq + head) * p.num_splits + split;
      p.part_o[pi * D + d] = acc;
      if (d == 0) {
        p.part_ml[pi * 2] = m;
        p.part_ml[pi * 2 + 1] = l;
      }
    }
  }
  if (q8) {
    __syncthreads();
    for (int idx = threadIdx.x * 4; idx < G * D; idx += (int)blockDim.x * 4) {
      const int r = idx / D, d = idx % D;
      const int head = kvh * G + r;
      const float sc = fmaxf(__int_as_float(sm_amax[r]), 1e-10f) / 448.f;
      const float inv = __frcp_rn(sc);
      const float4 v = *reinterpret_cast<const float4*>(sm_o + r * D + d);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x * inv, v.y * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z * inv, v.w * inv), __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<uint32_t*>(p.q_out + (long long)q_row0 * p.ldqo + head * D + d) = lo | (hi << 16);
      if (d == 0) p.s_out[(long long)head * p.s_ld + q_row0] = sc;
    }
  }
}

template <int D, int BS>       // BS: block size known at compile time (0 = runtime)
__global__ void __launch_bounds__(kDecodeThreads)
attn_decode_kernel(const AttnParams p, int stages, status_t* status) {
  constexpr int KS = D / 16, MT = D / 16, DQ = D / 4;
  extern __shared__ __align__(128) uint8_t dsm[];
  const int bs = BS ? BS : p.block_size;
  const int stage_bytes = 2 * bs * D;
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm);
  uint64_t* empty = full + stages;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty + stages);
  int* bt_sm = reinterpret_cast<int*>(dsm + 512);
  uint8_t* ring = dsm + 512 + kBtSmemEntries * 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = lane & 3, rq = lane >> 2;
  const int G = p.Hq / p.Hkv;
  const int b = p.seq_base + blockIdx.z, kvh = blockIdx.x, split = blockIdx.y;
  chain_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  chain_wait();                       // everything above is on-chip; global memory is only touched from here on
  const int L = p.seq_lens[b];
  const int q_row0 = p.query_start_loc[b];
  const int n_blocks = (L + bs - 1) / bs;
  const int per_split = (n_blocks + p.num_splits - 1) / p.num_splits;
  int blk_lo = split * per_split;
  const int blk_hi = min(n_blocks, (split + 1) * per_split);
  if (p.window > 0) blk_lo = max(blk_lo, max(0, L - p.window) / bs);
  const int n_mine = max(0, blk_hi - blk_lo);
  const int* bt = p.block_tables + (long long)b * p.bt_ld + blk_lo;
  for (int i = threadIdx.x; i < min(n_mine, kBtSmemEntries); i += kDecodeThreads) bt_sm[i] = bt[i];
  __syncthreads();

  // per-thread state: heads c*2, c*2+1 (n columns), dims mt*16 + rq (+8)
  float o[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  if (warp == 4) {
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < n_mine && ok; ++i) {
        const int st = i % stages;
        if (!mbar_wait(&empty[st], ((i / stages) & 1) ^ 1u, abort_flag, status, 0x400)) { ok = false; break; }
        const int blk = i < kBtSmemEntries ? bt_sm[i] : bt[i];
        const long long off = ((long long)blk * p.Hkv + kvh) * (long long)bs * D;
        uint8_t* dst = ring + (size_t)st * stage_bytes;
        mbar_expect_tx(&full[st], stage_bytes);
        bulk_g2s(dst, p.k_cache + off, bs * D, &full[st]);
        bulk_g2s(dst + bs * D, p.v_cache + off, bs * D, &full[st]);
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else {
    // ---- Q^T as B fragments: b0 = (k = c*2+{0,1}, n = rq) , b1 = (k = c*2+8+{0,1}, n = rq); n = head in group.
    // dim permutation: MMA k index kk of k-step ks <-> dim c'*DQ + ks*4 + ..., matching the K bytes a thread reads.
    uint32_t qb[KS][2];
    {
      const __nv_bfloat16* qrow = rq < G ? p.q + (long long)q_row0 * p.ldq + (kvh * G + rq) * D : nullptr;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (qrow) {
          const uint2 raw = *reinterpret_cast<const uint2*>(qrow + c * DQ + ks * 4);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          v[0] = __low2float(lo) * p.qk_scale_log2; v[1] = __high2float(lo) * p.qk_scale_log2;
          v[2] = __low2float(hi) * p.qk_scale_log2; v[3] = __high2float(hi) * p.qk_scale_log2;
        }
        qb[ks][0] = pack_f16x2(v[0], v[1]);
        qb[ks][1] = pack_f16x2(v[2], v[3]);
      }
    }
    const int win_lo = p.window > 0 ? L - 1 - p.window : -1;  // tokens <= win_lo are outside the window
    // this thread's two token rows inside a page
    const int tok_r0 = (rq >> 1) * 4 + (rq & 1);
    const int tok_r1 = tok_r0 + 2;
    bool ok = true;
    for (int i = warp; i < n_mine && ok; i += 4) {
      const int st = i % stages;
      if (!mbar_wait(&full[st], (i / stages) & 1u, abort_flag, status, 0x401)) { ok = false; break; }
      const uint8_t* kblk = ring + (size_t)st * stage_bytes;
      const uint8_t* vblk = kblk + bs * D;
      const int blk_tok0 = (blk_lo + i) * bs;
#pragma unroll 1
      for (int sub = 0; sub * 16 < bs; ++sub) {
        const int tok0 = blk_tok0 + sub * 16;
        if (tok0 >= L) break;
        // ---- S^T = K Q^T : rows = tokens (tok_r0 -> row rq, tok_r1 -> row rq+8), cols = heads
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        const uint4* k0 = reinterpret_cast<const uint4*>(kblk + (sub * 16 + tok_r0) * D + c * DQ);
        const uint4* k1 = reinterpret_cast<const uint4*>(kblk + (sub * 16 + tok_r1) * D + c * DQ);
#pragma unroll
        for (int v4 = 0; v4 < DQ / 16; ++v4) {
          const uint4 ra = k0[v4], rb = k1[v4];
          const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w};
          const uint32_t wb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
          for (int wi = 0; wi < 4; ++wi) {
            uint32_t a[4];
            fp8x4_to_f16x2x2(wa[wi], a[0], a[2]);      // row rq   : k lo / k hi
            fp8x4_to_f16x2x2(wb[wi], a[1], a[3]);      // row rq+8
            mma_f16(s, a, qb[v4 * 4 + wi][0], qb[v4 * 4 + wi][1]);
          }
        }
        // ---- mask (token validity is per row), online softmax per head column
        const bool in0 = (tok0 + tok_r0) < L && (tok0 + tok_r0) > win_lo;
        const bool in1 = (tok0 + tok_r1) < L && (tok0 + tok_r1) > win_lo;
        s[0] = in0 ? s[0] : -INFINITY; s[1] = in0 ? s[1] : -INFINITY;
        s[2] = in1 ? s[2] : -INFINITY; s[3] = in1 ? s[3] : -INFINITY;
        float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
          mx[h] = fmaxf(mx[h], m_run[h]);
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          alpha[h] = (mx[h] == -INFINITY) ? 1.f : exp2f(m_run[h] - mx[h]);
          m_run[h] = mx[h];
        }
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e & 1;
          pv[e] = (mx[h] == -INFINITY) ? 0.f : exp2f(s[e] - mx[h]);
        }
        l_run[0] = l_run[0] * alpha[0] + pv[0] + pv[2];
        l_run[1] = l_run[1] * alpha[1] + pv[1] + pv[3];
        // P^T as the B operand of the PV product: transpose the two 8x8 (token x head) blocks
        const uint32_t pb0 = movmatrix_trans(pack_f16x2(pv[0], pv[1]));
        const uint32_t pb1 = movmatrix_trans(pack_f16x2(pv[2], pv[3]));
        // after the transpose this thread holds head rq, tokens c*4+{0,1} (pb0) and c*4+{2,3} (pb1)
        uint32_t vmask = 0xFFFFFFFFu;
        {
          const int first = tok0 + c * 4;
          if (first + 3 >= L) {
            vmask = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (first + j < L) vmask |= 0xFFu << (8 * j);
          }
        }
        // rescale only when some head's running max moved (the accumulator's columns are heads c*2, c*2+1)
        const bool rescale = __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f);
        // ---- O^T += V^T P^T : rows = dims, k = tokens
        const uint8_t* vsub = vblk + sub * 16 + c * 4;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(vsub + (mt * 16 + rq) * bs) & vmask;
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(vsub + (mt * 16 + rq + 8) * bs) & vmask;
          uint32_t a[4];
          fp8x4_to_f16x2x2(w0, a[0], a[2]);
          fp8x4_to_f16x2x2(w1, a[1], a[3]);
          if (rescale) {
            o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1];
            o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
          }
          mma_f16(o[mt], a, pb0, pb1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
    }
    // column (head) sums live split across the 8 row-lanes
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
    }
  }

  decode_merge_store<D>(p, ring, o, m_run, l_run, warp, lane, G, kvh, split, b, q_row0, 1.f);
}

// ---- e4m3 tensor-core tiles (used by the e4m3 decode variants below)
ATLAS_DEVICE void mma_e4m3(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two floats -> two e4m3 bytes (`lo` in bits 7..0, `hi` in bits 15..8) and back
ATLAS_DEVICE uint32_t pack_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
ATLAS_DEVICE float2 unpack_e4m3x2(uint32_t v) {
  const uint32_t h = fp8x2_to_f16x2(static_cast<uint16_t>(v));
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
// (x0, x1) as a leading e4m3 pair and the e4m3 pair of what the first one missed
ATLAS_DEVICE void split_e4m3x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = pack_e4m3x2(x0, x1);
  const float2 back = unpack_e4m3x2(hi);
  lo = pack_e4m3x2(x0 - back.x, x1 - back.y);
}

// The same tiles fed by per-thread 16-byte asynchronous copies instead of the bulk-copy engine: every warp streams its own
// pages (page i of the CTA's range goes to warp i % 4) through a private ring of kCpDepth slots (2 or 3) and waits for them with
// cp.async.wait_group, so there is no producer warp, no mbarrier and no wait that could run out.  The copy engine moves
// the 2 KB K and V blocks of a page at ~26 KB/us per SM whatever the ring depth; 16-byte copies issued by all 128 threads
// stream the same bytes at ~32 KB/us per SM (`microbench --only stream`).
constexpr int kCpThreads = 128;
// KV4: NVFP4 pages (layout above paged_attn_kernel): 9/16 of the bytes per page; K is widened and scaled element by
// element, V's per-token scales are folded into the P operand once per 16-dim tile.
// F8: FP8 pages go to e4m3 tensor-core tiles as they are (mma.m16n8k32, no widening); Q and P, which are not cached bytes,
// are fed as two e4m3 terms each (see attn_decode_f8_kernel).  One page per step: the upper half of the 32-wide k
// dimension of the PV product stays zero, which costs tensor-pipe slots this kernel has to spare.
template <int D, int BS, int kCpDepth, bool KV4 = false, bool F8 = false>       // BS: block size known at compile time (0 = runtime)
__global__ void __launch_bounds__(kCpThreads)
attn_decode_cp_kernel(const AttnParams p) {
  constexpr int KS = D / 16, MT = D / 16, DQ = D / 4;
  constexpr float kPScale = 256.f;
  extern __shared__ __align__(128) uint8_t dsm[];
  const int bs = BS ? BS : p.block_size;
  const int stage_bytes = KV4 ? 2 * (bs * D * 9 / 16) : 2 * bs * D;
  int* bt_sm = reinterpret_cast<int*>(dsm);
  uint8_t* ring = dsm + kBtSmemEntries * 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = lane & 3, rq = lane >> 2;
  const int G = p.Hq / p.Hkv;
  const int b = p.seq_base + blockIdx.z, kvh = blockIdx.x, split = blockIdx.y;
  chain_trigger();
  chain_wait();                       // global memory is only touched from here on
  const int L = p.seq_lens[b];
  const int q_row0 = p.query_start_loc[b];
  const int n_blocks = (L + bs - 1) / bs;
  const int per_split = (n_blocks + p.num_splits - 1) / p.num_splits;
  int blk_lo = split * per_split;
  const int blk_hi = min(n_blocks, (split + 1) * per_split);
  if (p.window > 0) blk_lo = max(blk_lo, max(0, L - p.window) / bs);
  const int n_mine = max(0, blk_hi - blk_lo);
  const int* bt = p.block_tables + (long long)b * p.bt_ld + blk_lo;
  for (int i = threadIdx.x; i < min(n_mine, kBtSmemEntries); i += kCpThreads) bt_sm[i] = bt[i];
  __syncthreads();

  // per-thread state: heads c*2, c*2+1 (n columns), dims mt*16 + rq (+8)
  float o[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  {
    // ---- Q^T as B fragments: b0 = (k = c*2+{0,1}, n = rq) , b1 = (k = c*2+8+{0,1}, n = rq); n = head in group.
    // dim permutation: MMA k index kk of k-step ks <-> dim c'*DQ + ks*4 + ..., matching the K bytes a thread reads.
    uint32_t qb[KS][2];
    {
      const __nv_bfloat16* qrow = rq < G ? p.q + (long long)q_row0 * p.ldq + (kvh * G + rq) * D : nullptr;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (qrow) {
          const uint2 raw = *reinterpret_cast<const uint2*>(qrow + c * DQ + ks * 4);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          v[0] = __low2float(lo) * p.qk_scale_log2; v[1] = __high2float(lo) * p.qk_scale_log2;
          v[2] = __low2float(hi) * p.qk_scale_log2; v[3] = __high2float(hi) * p.qk_scale_log2;
        }
        qb[ks][0] = pack_f16x2(v[0], v[1]);
        qb[ks][1] = pack_f16x2(v[2], v[3]);
      }
    }
    // e4m3 form of Q^T: k index 4c+j of k-step ks8 is dim c*DQ + ks8*8 + j, k index 16+4c+j is dim c*DQ + ks8*8 + 4 + j
    uint32_t qh[F8 ? D / 32 : 1][2], ql[F8 ? D / 32 : 1][2];
    float sq[2] = {1.f, 1.f};
    if constexpr (F8) {
      float qv[DQ];
      float amax = 0.f;
      if (rq < G) {
        const __nv_bfloat16* qrow = p.q + (long long)q_row0 * p.ldq + (kvh * G + rq) * D + c * DQ;
#pragma unroll
        for (int j = 0; j < DQ; j += 4) {
          const uint2 raw = *reinterpret_cast<const uint2*>(qrow + j);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          qv[j] = __low2float(lo) * p.qk_scale_log2; qv[j + 1] = __high2float(lo) * p.qk_scale_log2;
          qv[j + 2] = __low2float(hi) * p.qk_scale_log2; qv[j + 3] = __high2float(hi) * p.qk_scale_log2;
        }
#pragma unroll
        for (int j = 0; j < DQ; ++j) amax = fmaxf(amax, fabsf(qv[j]));
      } else {
#pragma unroll
        for (int j = 0; j < DQ; ++j) qv[j] = 0.f;
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const float qs = fmaxf(amax, 1e-30f) * (1.f / 448.f);
      const float qinv = __frcp_rn(qs);
#pragma unroll
      for (int k8 = 0; k8 < D / 32; ++k8)
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          uint32_t h0, l0, h1, l1;
          split_e4m3x2(qv[k8 * 8 + w * 4 + 0] * qinv, qv[k8 * 8 + w * 4 + 1] * qinv, h0, l0);
          split_e4m3x2(qv[k8 * 8 + w * 4 + 2] * qinv, qv[k8 * 8 + w * 4 + 3] * qinv, h1, l1);
          qh[k8][w] = h0 | (h1 << 16);
          ql[k8][w] = l0 | (l1 << 16);
        }
      sq[0] = __shfl_sync(0xffffffffu, qs, (2 * c) * 4);
      sq[1] = __shfl_sync(0xffffffffu, qs, (2 * c + 1) * 4);
    }
    const int win_lo = p.window > 0 ? L - 1 - p.window : -1;  // tokens <= win_lo are outside the window
    // this thread's two token rows inside a page
    const int tok_r0 = (rq >> 1) * 4 + (rq & 1);
    const int tok_r1 = tok_r0 + 2;
    // this warp's pages: i = warp + 4 k, slot k % kCpDepth of its private ring
    uint8_t* myring = ring + (size_t)warp * kCpDepth * stage_bytes;
    const int n_w = n_mine > warp ? (n_mine - warp + 3) / 4 : 0;
    const int half_bytes = KV4 ? bs * D * 9 / 16 : bs * D;          // one page of K or of V
    auto issue = [&](int k) {
      const int i = warp + 4 * k;
      const int blk = i < kBtSmemEntries ? bt_sm[i] : bt[i];
      const long long off = ((long long)blk * p.Hkv + kvh) * (long long)half_bytes;
      const uint32_t dst = smem_u32(myring + (size_t)(k % kCpDepth) * stage_bytes);
      const uint8_t* ks = p.k_cache + off;
      const uint8_t* vs = p.v_cache + off;
      for (int o16 = lane * 16; o16 < half_bytes; o16 += 512) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + o16), "l"(ks + o16) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + half_bytes + o16), "l"(vs + o16) : "memory");
      }
    };
#pragma unroll
    for (int k = 0; k < kCpDepth - 1; ++k) {
      if (k < n_w) issue(k);
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    for (int k = 0; k < n_w; ++k) {
      if (k + kCpDepth - 1 < n_w) issue(k + kCpDepth - 1);
      asm volatile("cp.async.commit_group;\n" ::: "memory");
      asm volatile("cp.async.wait_group %0;\n" ::"n"(kCpDepth - 1) : "memory");      // page k has landed
      __syncwarp();
      const int i = warp + 4 * k;
      const uint8_t* kblk = myring + (size_t)(k % kCpDepth) * stage_bytes;
      const uint8_t* vblk = kblk + half_bytes;
      const int blk_tok0 = (blk_lo + i) * bs;
#pragma unroll 1
      for (int sub = 0; sub * 16 < bs; ++sub) {
        const int tok0 = blk_tok0 + sub * 16;
        if (tok0 >= L) break;
        // ---- S^T = K Q^T : rows = tokens (tok_r0 -> row rq, tok_r1 -> row rq+8), cols = heads
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        const uint4* k0 = reinterpret_cast<const uint4*>(kblk + (sub * 16 + tok_r0) * D + c * DQ);
        const uint4* k1 = reinterpret_cast<const uint4*>(kblk + (sub * 16 + tok_r1) * D + c * DQ);
        if constexpr (F8) {
#pragma unroll
          for (int v4 = 0; v4 < DQ / 16; ++v4) {
            const uint4 ra = k0[v4], rb = k1[v4];
            const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w};
            const uint32_t wb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
            for (int hk = 0; hk < 2; ++hk) {
              const uint32_t a[4] = {wa[2 * hk], wb[2 * hk], wa[2 * hk + 1], wb[2 * hk + 1]};
              mma_e4m3(s, a, qh[v4 * 2 + hk][0], qh[v4 * 2 + hk][1]);
              mma_e4m3(s, a, ql[v4 * 2 + hk][0], ql[v4 * 2 + hk][1]);
            }
          }
          s[0] *= sq[0]; s[1] *= sq[1]; s[2] *= sq[0]; s[3] *= sq[1];
        } else if constexpr (KV4) {
          const int ta = sub * 16 + tok_r0, tb = sub * 16 + tok_r1;
          const uint8_t* ka = kblk + ta * (D / 2) + c * (DQ / 2);
          const uint8_t* kb = kblk + tb * (D / 2) + c * (DQ / 2);
          const uint8_t* sa = kblk + bs * (D / 2) + ta * (D / 16) + c * (DQ / 16);
          const uint8_t* sb = kblk + bs * (D / 2) + tb * (D / 16) + c * (DQ / 16);
#pragma unroll
          for (int g = 0; g < DQ / 16; ++g) {
            const uint32_t s2a = fp8x2_to_f16x2((uint16_t)(sa[g] * 0x0101u)), s2b = fp8x2_to_f16x2((uint16_t)(sb[g] * 0x0101u));
            const uint2 ra = reinterpret_cast<const uint2*>(ka)[g], rb = reinterpret_cast<const uint2*>(kb)[g];
            const uint32_t wa[2] = {ra.x, ra.y}, wb[2] = {rb.x, rb.y};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              const uint32_t ta2 = (wa[wi >> 1] >> (16 * (wi & 1))) & 0xFFFFu, tb2 = (wb[wi >> 1] >> (16 * (wi & 1))) & 0xFFFFu;
              uint32_t a[4];
              a[0] = hmul2_u32(e2m1x2_to_f16x2(ta2 & 0xFFu), s2a); a[2] = hmul2_u32(e2m1x2_to_f16x2(ta2 >> 8), s2a);
              a[1] = hmul2_u32(e2m1x2_to_f16x2(tb2 & 0xFFu), s2b); a[3] = hmul2_u32(e2m1x2_to_f16x2(tb2 >> 8), s2b);
              mma_f16(s, a, qb[g * 4 + wi][0], qb[g * 4 + wi][1]);
            }
          }
        } else
#pragma unroll
        for (int v4 = 0; v4 < DQ / 16; ++v4) {
          const uint4 ra = k0[v4], rb = k1[v4];
          const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w};
          const uint32_t wb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
          for (int wi = 0; wi < 4; ++wi) {
            uint32_t a[4];
            fp8x4_to_f16x2x2(wa[wi], a[0], a[2]);      // row rq   : k lo / k hi
            fp8x4_to_f16x2x2(wb[wi], a[1], a[3]);      // row rq+8
            mma_f16(s, a, qb[v4 * 4 + wi][0], qb[v4 * 4 + wi][1]);
          }
        }
        // ---- mask (token validity is per row), online softmax per head column
        const bool in0 = (tok0 + tok_r0) < L && (tok0 + tok_r0) > win_lo;
        const bool in1 = (tok0 + tok_r1) < L && (tok0 + tok_r1) > win_lo;
        s[0] = in0 ? s[0] : -INFINITY; s[1] = in0 ? s[1] : -INFINITY;
        s[2] = in1 ? s[2] : -INFINITY; s[3] = in1 ? s[3] : -INFINITY;
        float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
          mx[h] = fmaxf(mx[h], m_run[h]);
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          alpha[h] = (mx[h] == -INFINITY) ? 1.f : exp2f(m_run[h] - mx[h]);
          m_run[h] = mx[h];
        }
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e & 1;
          pv[e] = (mx[h] == -INFINITY) ? 0.f : exp2f(s[e] - mx[h]);
        }
        l_run[0] = l_run[0] * alpha[0] + pv[0] + pv[2];
        l_run[1] = l_run[1] * alpha[1] + pv[1] + pv[3];
        // P^T as the B operand of the PV product: transpose the two 8x8 (token x head) blocks
        const uint32_t pb0 = movmatrix_trans(pack_f16x2(pv[0], pv[1]));
        const uint32_t pb1 = movmatrix_trans(pack_f16x2(pv[2], pv[3]));
        // after the transpose this thread holds head rq, tokens c*4+{0,1} (pb0) and c*4+{2,3} (pb1)
        uint32_t vmask = 0xFFFFFFFFu;
        {
          const int first = tok0 + c * 4;
          if (first + 3 >= L) {
            vmask = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (first + j < L) vmask |= 0xFFu << (8 * j);
          }
        }
        // rescale only when some head's running max moved (the accumulator's columns are heads c*2, c*2+1)
        const bool rescale = __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f);
        // ---- O^T += V^T P^T : rows = dims, k = tokens
        const uint8_t* vsub = vblk + sub * 16 + c * 4;
        if constexpr (F8) {
          // P^T as two e4m3 terms: a b16 unit carries one head's values of this thread's two token rows; the 8x8 transpose
          // leaves head rq's tokens 4c, 4c+2, 4c+1, 4c+3 in a register, a byte permute puts them in order
          uint32_t h0, l0, h1, l1;
          split_e4m3x2(pv[0] * kPScale, pv[2] * kPScale, h0, l0);
          split_e4m3x2(pv[1] * kPScale, pv[3] * kPScale, h1, l1);
          const uint32_t pbh = __byte_perm(movmatrix_trans(h0 | (h1 << 16)), 0u, 0x3120);
          const uint32_t pbl = __byte_perm(movmatrix_trans(l0 | (l1 << 16)), 0u, 0x3120);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t a[4] = {*reinterpret_cast<const uint32_t*>(vsub + (mt * 16 + rq) * bs) & vmask,
                                   *reinterpret_cast<const uint32_t*>(vsub + (mt * 16 + rq + 8) * bs) & vmask, 0u, 0u};
            if (rescale) {
              o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1];
              o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
            }
            mma_e4m3(o[mt], a, pbh, 0u);
            mma_e4m3(o[mt], a, pbl, 0u);
          }
        } else if constexpr (KV4) {
          const uint32_t m0 = ((vmask & 0xFFu) ? 0xFFFFu : 0u) | ((vmask & 0xFF00u) ? 0xFFFF0000u : 0u);
          const uint32_t m1 = ((vmask & 0xFF0000u) ? 0xFFFFu : 0u) | ((vmask & 0xFF000000u) ? 0xFFFF0000u : 0u);
          const uint8_t* vd = vblk + ((sub * 16 + c * 4) >> 1);                       // two tokens per byte
          const uint8_t* vsc = vblk + D * (bs / 2) + sub * 16 + c * 4;                // [D/16][bs] scales
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t sw = *reinterpret_cast<const uint32_t*>(vsc + mt * bs) & vmask;
            const uint32_t pbs0 = hmul2_u32(pb0, fp8x2_to_f16x2((uint16_t)(sw & 0xFFFFu)));
            const uint32_t pbs1 = hmul2_u32(pb1, fp8x2_to_f16x2((uint16_t)(sw >> 16)));
            const uint32_t w0 = *reinterpret_cast<const uint16_t*>(vd + (mt * 16 + rq) * (bs / 2));
            const uint32_t w1 = *reinterpret_cast<const uint16_t*>(vd + (mt * 16 + rq + 8) * (bs / 2));
            uint32_t a[4];
            a[0] = e2m1x2_to_f16x2(w0 & 0xFFu) & m0; a[2] = e2m1x2_to_f16x2(w0 >> 8) & m1;
            a[1] = e2m1x2_to_f16x2(w1 & 0xFFu) & m0; a[3] = e2m1x2_to_f16x2(w1 >> 8) & m1;
            if (rescale) {
              o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1];
              o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
            }
            mma_f16(o[mt], a, pbs0, pbs1);
          }
        } else
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(vsub + (mt * 16 + rq) * bs) & vmask;
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(vsub + (mt * 16 + rq + 8) * bs) & vmask;
          uint32_t a[4];
          fp8x4_to_f16x2x2(w0, a[0], a[2]);
          fp8x4_to_f16x2x2(w1, a[1], a[3]);
          if (rescale) {
            o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1];
            o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
          }
          mma_f16(o[mt], a, pb0, pb1);
        }
      }
      __syncwarp();                  // the slot is refilled two iterations from now
    }
    asm volatile("cp.async.wait_all;\n" ::: "memory");
    // column (head) sums live split across the 8 row-lanes
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
    }
  }

  decode_merge_store<D>(p, ring, o, m_run, l_run, warp, lane, G, kvh, split, b, q_row0, F8 ? 1.f / kPScale : 1.f);
}

// ----------------------------------------------------------------------------- decode on FP8 tensor-core tiles
// The same pipeline (16-token pages only), but the cached bytes go into the tensor cores as they are:
// mma.m16n8k32 with e4m3 operands.  Nothing is widened to f16, which is what the f16 form spends most of its issue
// slots on.  The two operands that are not cached bytes keep 16-bit-class precision by being fed as TWO e4m3 terms each,
// x = e4m3(x) + e4m3(x - e4m3(x)), accumulated into the same fp32 accumulator:
//   S^T[16 tok x 8 heads] = K[16 x 32 dims] (Qhi^T + Qlo^T)      Q scaled per head to the e4m3 range, scale applied to S
//   O^T[16 dims x 8 heads] += V^T[16 x 32 tok] (Phi^T + Plo^T)    P scaled by 256 (undone at the end)
// A warp takes two pages per step so that the PV product's 32-token k dimension is full.
template <int D>
__global__ void __launch_bounds__(kDecodeThreads)
attn_decode_f8_kernel(const AttnParams p, int stages, status_t* status) {
  constexpr int KS = D / 32, MT = D / 16, DQ = D / 4, bs = 16;
  constexpr float kPScale = 256.f;
  extern __shared__ __align__(128) uint8_t dsm[];
  constexpr int stage_bytes = 2 * bs * D;
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm);
  uint64_t* empty = full + stages;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty + stages);
  int* bt_sm = reinterpret_cast<int*>(dsm + 512);
  uint8_t* ring = dsm + 512 + kBtSmemEntries * 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = lane & 3, rq = lane >> 2;
  const int G = p.Hq / p.Hkv;
  const int b = p.seq_base + blockIdx.z, kvh = blockIdx.x, split = blockIdx.y;
  chain_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  chain_wait();                       // everything above is on-chip; global memory is only touched from here on
  const int L = p.seq_lens[b];
  const int q_row0 = p.query_start_loc[b];
  const int n_blocks = (L + bs - 1) / bs;
  const int per_split = (n_blocks + p.num_splits - 1) / p.num_splits;
  int blk_lo = split * per_split;
  const int blk_hi = min(n_blocks, (split + 1) * per_split);
  if (p.window > 0) blk_lo = max(blk_lo, max(0, L - p.window) / bs);
  const int n_mine = max(0, blk_hi - blk_lo);
  const int* bt = p.block_tables + (long long)b * p.bt_ld + blk_lo;
  for (int i = threadIdx.x; i < min(n_mine, kBtSmemEntries); i += kDecodeThreads) bt_sm[i] = bt[i];
  __syncthreads();

  float o[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  if (warp == 4) {
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < n_mine && ok; ++i) {
        const int st = i % stages;
        if (!mbar_wait(&empty[st], ((i / stages) & 1) ^ 1u, abort_flag, status, 0x410)) { ok = false; break; }
        const int blk = i < kBtSmemEntries ? bt_sm[i] : bt[i];
        const long long off = ((long long)blk * p.Hkv + kvh) * (long long)bs * D;
        uint8_t* dst = ring + (size_t)st * stage_bytes;
        mbar_expect_tx(&full[st], stage_bytes);
        bulk_g2s(dst, p.k_cache + off, bs * D, &full[st]);
        bulk_g2s(dst + bs * D, p.v_cache + off, bs * D, &full[st]);
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else {
    // ---- Q^T as e4m3 B fragments, two terms.  Thread (rq, c) holds head rq, dims [c*DQ, c*DQ + DQ): k index 4c+j of
    // k-step ks is dim c*DQ + ks*8 + j, k index 16+4c+j is dim c*DQ + ks*8 + 4 + j -- the bytes of K a thread reads.
    uint32_t qh[KS][2], ql[KS][2];
    float sq[2];                       // S = accumulator * sq[h] for this thread's two head columns
    {
      float qv[DQ];
      float amax = 0.f;
      if (rq < G) {
        const __nv_bfloat16* qrow = p.q + (long long)q_row0 * p.ldq + (kvh * G + rq) * D + c * DQ;
#pragma unroll
        for (int j = 0; j < DQ; j += 4) {
          const uint2 raw = *reinterpret_cast<const uint2*>(qrow + j);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          qv[j] = __low2float(lo) * p.qk_scale_log2; qv[j + 1] = __high2float(lo) * p.qk_scale_log2;
          qv[j + 2] = __low2float(hi) * p.qk_scale_log2; qv[j + 3] = __high2float(hi) * p.qk_scale_log2;
        }
#pragma unroll
        for (int j = 0; j < DQ; ++j) amax = fmaxf(amax, fabsf(qv[j]));
      } else {
#pragma unroll
        for (int j = 0; j < DQ; ++j) qv[j] = 0.f;
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const float qs = fmaxf(amax, 1e-30f) * (1.f / 448.f);
      const float qinv = __frcp_rn(qs);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          uint32_t h0, l0, h1, l1;
          split_e4m3x2(qv[ks * 8 + w * 4 + 0] * qinv, qv[ks * 8 + w * 4 + 1] * qinv, h0, l0);
          split_e4m3x2(qv[ks * 8 + w * 4 + 2] * qinv, qv[ks * 8 + w * 4 + 3] * qinv, h1, l1);
          qh[ks][w] = h0 | (h1 << 16);
          ql[ks][w] = l0 | (l1 << 16);
        }
      sq[0] = __shfl_sync(0xffffffffu, qs, (2 * c) * 4);
      sq[1] = __shfl_sync(0xffffffffu, qs, (2 * c + 1) * 4);
    }
    const int win_lo = p.window > 0 ? L - 1 - p.window : -1;  // tokens <= win_lo are outside the window
    const int tok_r0 = (rq >> 1) * 4 + (rq & 1);               // this thread's two token rows inside a page
    const int tok_r1 = tok_r0 + 2;
    bool ok = true;
    for (int u = warp; 2 * u < n_mine && ok; u += 4) {
      const int i0 = 2 * u, i1 = i0 + 1;
      const int st0 = i0 % stages, st1 = i1 % stages;
      const int tokA = (blk_lo + i0) * bs;
      const bool two = i1 < n_mine && tokA + bs < L;
      if (!mbar_wait(&full[st0], (i0 / stages) & 1u, abort_flag, status, 0x411)) { ok = false; break; }
      if (i1 < n_mine && !mbar_wait(&full[st1], (i1 / stages) & 1u, abort_flag, status, 0x412)) { ok = false; break; }
      const uint8_t* kblk[2] = {ring + (size_t)st0 * stage_bytes, ring + (size_t)st1 * stage_bytes};
      // ---- S^T = K Q^T for both pages: rows = tokens (tok_r0 -> row rq, tok_r1 -> row rq+8), cols = heads
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        if (j == 1 && !two) continue;
        const uint4* k0 = reinterpret_cast<const uint4*>(kblk[j] + tok_r0 * D + c * DQ);
        const uint4* k1 = reinterpret_cast<const uint4*>(kblk[j] + tok_r1 * D + c * DQ);
#pragma unroll
        for (int v4 = 0; v4 < DQ / 16; ++v4) {
          const uint4 ra = k0[v4], rb = k1[v4];
          const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w};
          const uint32_t wb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
          for (int hk = 0; hk < 2; ++hk) {
            const uint32_t a[4] = {wa[2 * hk], wb[2 * hk], wa[2 * hk + 1], wb[2 * hk + 1]};
            mma_e4m3(s[j], a, qh[v4 * 2 + hk][0], qh[v4 * 2 + hk][1]);
            mma_e4m3(s[j], a, ql[v4 * 2 + hk][0], ql[v4 * 2 + hk][1]);
          }
        }
      }
      // ---- scale, mask (token validity is per row), online softmax per head column over the 32 tokens
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int t0 = tokA + j * bs;
        const bool live = j == 0 || two;
        const bool in0 = live && (t0 + tok_r0) < L && (t0 + tok_r0) > win_lo;
        const bool in1 = live && (t0 + tok_r1) < L && (t0 + tok_r1) > win_lo;
        s[j][0] = in0 ? s[j][0] * sq[0] : -INFINITY; s[j][1] = in0 ? s[j][1] * sq[1] : -INFINITY;
        s[j][2] = in1 ? s[j][2] * sq[0] : -INFINITY; s[j][3] = in1 ? s[j][3] * sq[1] : -INFINITY;
      }
      float mx[2] = {fmaxf(fmaxf(s[0][0], s[0][2]), fmaxf(s[1][0], s[1][2])), fmaxf(fmaxf(s[0][1], s[0][3]), fmaxf(s[1][1], s[1][3]))};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
        mx[h] = fmaxf(mx[h], m_run[h]);
      }
      float alpha[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        alpha[h] = (mx[h] == -INFINITY) ? 1.f : exp2f(m_run[h] - mx[h]);
        m_run[h] = mx[h];
      }
      // P^T as the B operand of the PV product, two e4m3 terms.  A b16 unit carries one head's values of this thread's two
      // token rows; the 8x8 transpose then leaves head rq's tokens 4c, 4c+2, 4c+1, 4c+3 in a register (put in order by a
      // byte permute), i.e. the k indices 4c .. 4c+3 of the page.
      uint32_t pbh[2], pbl[2];
      float lsum[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e & 1;
          pv[e] = (mx[h] == -INFINITY) ? 0.f : exp2f(s[j][e] - mx[h]);
        }
        lsum[0] += pv[0] + pv[2];
        lsum[1] += pv[1] + pv[3];
        uint32_t h0, l0, h1, l1;
        split_e4m3x2(pv[0] * kPScale, pv[2] * kPScale, h0, l0);      // head 2c:   (tok_r0, tok_r1)
        split_e4m3x2(pv[1] * kPScale, pv[3] * kPScale, h1, l1);      // head 2c+1
        pbh[j] = __byte_perm(movmatrix_trans(h0 | (h1 << 16)), 0u, 0x3120);
        pbl[j] = __byte_perm(movmatrix_trans(l0 | (l1 << 16)), 0u, 0x3120);
      }
      l_run[0] = l_run[0] * alpha[0] + lsum[0];
      l_run[1] = l_run[1] * alpha[1] + lsum[1];
      // bytes of V^T past the sequence's end may hold anything (0 x NaN): mask them
      uint32_t vmask[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int first = tokA + j * bs + c * 4;
        vmask[j] = (j == 1 && !two) ? 0u : 0xFFFFFFFFu;
        if (first + 3 >= L) {
          uint32_t mk = 0;
#pragma unroll
          for (int t = 0; t < 4; ++t)
            if (first + t < L) mk |= 0xFFu << (8 * t);
          vmask[j] &= mk;
        }
      }
      const bool rescale = __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f);
      // ---- O^T += V^T P^T : rows = dims, k = the 32 tokens of the two pages
      const uint8_t* v0 = kblk[0] + bs * D + c * 4;
      const uint8_t* v1 = kblk[1] + bs * D + c * 4;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(v0 + (mt * 16 + rq) * bs) & vmask[0];
        a[1] = *reinterpret_cast<const uint32_t*>(v0 + (mt * 16 + rq + 8) * bs) & vmask[0];
        a[2] = two ? (*reinterpret_cast<const uint32_t*>(v1 + (mt * 16 + rq) * bs) & vmask[1]) : 0u;
        a[3] = two ? (*reinterpret_cast<const uint32_t*>(v1 + (mt * 16 + rq + 8) * bs) & vmask[1]) : 0u;
        if (rescale) {
          o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1];
          o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
        }
        mma_e4m3(o[mt], a, pbh[0], pbh[1]);
        mma_e4m3(o[mt], a, pbl[0], pbl[1]);
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&empty[st0]);
        if (i1 < n_mine) mbar_arrive(&empty[st1]);
      }
    }
    // column (head) sums live split across the 8 row-lanes
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
    }
  }
  decode_merge_store<D>(p, ring, o, m_run, l_run, warp, lane, G, kvh, split, b, q_row0, 1.f / kPScale);
}

// Merge split partials: grid (Hq, B), D threads.
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  __nv_bfloat16* out, long long ldo, const int* query_start_loc, int seq_base, int Hq,
                                  int D, int splits, float v_scale, uint8_t* q_out, long long ldqo, float* s_out,
                                  long long s_ld) {
  __shared__ float wmax[8];
  const int head = blockIdx.x, bi = blockIdx.y, d = threadIdx.x;
  const long long base = ((long long)bi * Hq + head) * splits;
  chain_trigger();
  chain_wait();
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    acc += f * part_o[(base + s) * D + d];
    l += f * part_ml[(base + s) * 2 + 1];
  }
  const float inv = l > 0.f ? v_scale / l : 0.f;
  const int row = query_start_loc[seq_base + bi];
  if (q_out == nullptr) {
    out[(long long)row * ldo + head * D + d] = __float2bfloat16_rn(acc * inv);
    return;
  }
  // FP8 output, one scale per (row, head); D == 128 (the block is the quantisation group)
  const float v = __bfloat162float(__float2bfloat16_rn(acc * inv));
  float a = fabsf(v);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
  if ((d & 31) == 0) wmax[d >> 5] = a;
  __syncthreads();
  a = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
  const float sc = fmaxf(a, 1e-10f) / 448.f;
  const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v * __frcp_rn(sc), __NV_SATFINITE, __NV_E4M3);
  q_out[(long long)row * ldqo + head * D + d] = q;
  if (d == 0) s_out[(long long)head * s_ld + row] = sc;
}

// Which decode kernel serves 16-token pages: the f16 tensor-core form (default) or the e4m3 form (ATLAS_ATTN_F8MMA=1 or
// atlas_attn_set_decode_f8).  Both are bound by how many bytes of KV a CTA keeps in flight, not by instruction issue: the
// e4m3 form issues half the instructions per page but holds more registers (3 instead of 4 CTAs per SM) and measured
// 102 us against 78 us on 128 sequences x 1152 tokens.
static int g_decode_f8 = -1;
static bool decode_f8_enabled() {
  if (g_decode_f8 < 0) {
    const char* e = getenv("ATLAS_ATTN_F8MMA");
    g_decode_f8 = (e && e[0] == '1') ? 1 : 0;
  }
  return g_decode_f8 == 1;
}
// Bytes of KV ring per decode CTA (ATLAS_ATTN_RING_KB, default 32)
static int decode_ring_bytes() {
  static const int v = [] {
    const char* e = getenv("ATLAS_ATTN_RING_KB");
    const int kb = e ? atoi(e) : 32;
    return (kb < 16 ? 16 : (kb > 96 ? 96 : kb)) * 1024;
  }();
  return v;
}

template <int D, int BS>
static int launch_decode_bs(const AttnParams& p, int B, status_t* status, cudaStream_t st) {
  const int stage_bytes = 2 * p.block_size * D;
  int stages = decode_ring_bytes() / stage_bytes;
  stages = stages > 24 ? 24 : (stages < 4 ? 4 : stages);
  stages = (stages / 4) * 4;                       // block i -> stage i % stages -> warp i % 4
  const int merge_bytes = (64 + 4 * 8 * D + 8) * (int)sizeof(float);
  const int ring_bytes = stages * stage_bytes > merge_bytes ? stages * stage_bytes : merge_bytes;
  const int smem = 512 + kBtSmemEntries * 4 + ring_bytes;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_decode_kernel<D, BS>), smem) != cudaSuccess) return -20;
  dim3 grid(p.Hkv, p.num_splits, B);
  if (launch_chain(attn_decode_kernel<D, BS>, grid, dim3(kDecodeThreads), (size_t)smem, st, p, stages, status) != cudaSuccess) return -21;
  if (p.num_splits > 1) {
    dim3 g2(p.Hq, B);
    if (launch_chain(attn_merge_kernel, g2, dim3(D), 0, st, p.part_o, p.part_ml, p.out, p.ldo, p.query_start_loc, p.seq_base,
                     p.Hq, D, p.num_splits, p.v_scale, p.q_out, p.ldqo, p.s_out, p.s_ld) != cudaSuccess)
      return -22;
  }
  return 0;
}
template <int D>
static int launch_decode_f8(const AttnParams& p, int B, status_t* status, cudaStream_t st) {
  constexpr int stage_bytes = 2 * 16 * D;
  int stages = decode_ring_bytes() / stage_bytes;
  stages = stages > 24 ? 24 : (stages < 8 ? 8 : stages);       // every consumer warp may hold two pages
  stages = (stages / 8) * 8;
  const int merge_bytes = (64 + 4 * 8 * D + 8) * (int)sizeof(float);
  const int ring_bytes = stages * stage_bytes > merge_bytes ? stages * stage_bytes : merge_bytes;
  const int smem = 512 + kBtSmemEntries * 4 + ring_bytes;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_decode_f8_kernel<D>), smem) != cudaSuccess) return -20;
  dim3 grid(p.Hkv, p.num_splits, B);
  if (launch_chain(attn_decode_f8_kernel<D>, grid, dim3(kDecodeThreads), (size_t)smem, st, p, stages, status) != cudaSuccess) return -21;
  if (p.num_splits > 1) {
    dim3 g2(p.Hq, B);
    if (launch_chain(attn_merge_kernel, g2, dim3(D), 0, st, p.part_o, p.part_ml, p.out, p.ldo, p.query_start_loc, p.seq_base,
                     p.Hq, D, p.num_splits, p.v_scale, p.q_out, p.ldqo, p.s_out, p.s_ld) != cudaSuccess)
      return -22;
  }
  return 0;
}

// ATLAS_ATTN_CPASYNC=0 keeps the bulk-copy pipeline (producer warp + mbarriers)
static bool decode_cpasync_enabled() {
  static const bool on = [] { const char* e = getenv("ATLAS_ATTN_CPASYNC"); return !(e && e[0] == '0'); }();
  return on;
}

// Slots of a warp's private page ring (ATLAS_ATTN_CP_DEPTH = 2 or 3)
static int decode_cp_depth() {
  static const int v = [] { const char* e = getenv("ATLAS_ATTN_CP_DEPTH"); return (e && atoi(e) == 2) ? 2 : 3; }();
  return v;
}

template <int D, int BS, int kCpDepth, bool KV4 = false, bool F8 = false>
static int launch_decode_cp(const AttnParams& p, int B, cudaStream_t st) {
  const int stage_bytes = KV4 ? 2 * (p.block_size * D * 9 / 16) : 2 * p.block_size * D;
  const int merge_bytes = (64 + 4 * 8 * D + 8) * (int)sizeof(float);
  const int ring_bytes = 4 * kCpDepth * stage_bytes > merge_bytes ? 4 * kCpDepth * stage_bytes : merge_bytes;
  const int smem = kBtSmemEntries * 4 + ring_bytes;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_decode_cp_kernel<D, BS, kCpDepth, KV4, F8>), smem) != cudaSuccess) return -20;
  dim3 grid(p.Hkv, p.num_splits, B);
  if (launch_chain(attn_decode_cp_kernel<D, BS, kCpDepth, KV4, F8>, grid, dim3(kCpThreads), (size_t)smem, st, p) != cudaSuccess) return -21;
  if (p.num_splits > 1) {
    dim3 g2(p.Hq, B);
    if (launch_chain(attn_merge_kernel, g2, dim3(D), 0, st, p.part_o, p.part_ml, p.out, p.ldo, p.query_start_loc, p.seq_base,
                     p.Hq, D, p.num_splits, p.v_scale, p.q_out, p.ldqo, p.s_out, p.s_ld) != cudaSuccess)
      return -22;
  }
  return 0;
}

template <int D>
static int launch_decode(const AttnParams& p, int B, status_t* status, cudaStream_t st) {
  if (decode_cpasync_enabled() && decode_f8_enabled() && 4 * 3 * 2 * p.block_size * D <= 96 * 1024) {
    if (p.block_size == 16) return launch_decode_cp<D, 16, 3, false, true>(p, B, st);
    return launch_decode_cp<D, 0, 3, false, true>(p, B, st);
  }
  if (p.block_size == 16 && decode_f8_enabled()) return launch_decode_f8<D>(p, B, status, st);
  if (decode_cpasync_enabled() && 4 * 3 * 2 * p.block_size * D <= 96 * 1024) {
    if (decode_cp_depth() == 2) {
      if (p.block_size == 16) return launch_decode_cp<D, 16, 2>(p, B, st);
      return launch_decode_cp<D, 0, 2>(p, B, st);
    }
    if (p.block_size == 16) return launch_decode_cp<D, 16, 3>(p, B, st);
    return launch_decode_cp<D, 0, 3>(p, B, st);
  }
  if (p.block_size == 16) return launch_decode_bs<D, 16>(p, B, status, st);
  return launch_decode_bs<D, 0>(p, B, status, st);
}

template <int D>
static int launch_prefill(const AttnParams& p, cudaStream_t st) {
  dim3 grid((p.num_tiles + 3) / 4, p.Hq);
  paged_attn_kernel<D, true><<<grid, 128, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace atlas

using namespace atlas;

static int fill_common(AttnParams& p, const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                       const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                       const int* query_start_loc, int seq_base, float scale, float k_scale, float v_scale, int Hq,
                       int Hkv, int D, int block_size, int window) {
  if (Hq % Hkv || block_size % 16 || (D != 64 && D != 128 && D != 256)) return -1;
  if (ldq % 4 || ldo % 2) return -2;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q); p.ldq = ldq;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.k_cache = reinterpret_cast<const uint8_t*>(k_cache); p.v_cache = reinterpret_cast<const uint8_t*>(v_cache);
  p.block_tables = block_tables; p.bt_ld = bt_ld; p.seq_lens = seq_lens; p.query_start_loc = query_start_loc;
  p.seq_base = seq_base;
  p.qk_scale_log2 = scale * k_scale * 1.4426950408889634f;
  p.v_scale = v_scale;
  p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size; p.window = window;
  p.num_splits = 1; p.part_o = nullptr; p.part_ml = nullptr; p.tile_seq = nullptr; p.tile_q0 = nullptr; p.num_tiles = 0;
  p.q_out = nullptr; p.ldqo = 0; p.s_out = nullptr; p.s_ld = 0;
  return 0;
}

// Decode attention for sequences [seq_base, seq_base+B), one query row each.  With num_splits > 1 the caller
// provides scratch: part_o [B*Hq*splits*D] floats and part_ml [B*Hq*splits*2] floats.
extern "C" int atlas_attn_decode(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                 const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                 const int* query_start_loc, int seq_base, int B, float scale, float k_scale,
                                 float v_scale, int Hq, int Hkv, int D, int block_size, int window, int num_splits,
                                 float* part_o, float* part_ml, unsigned long long* status, void* stream) {
  if (B <= 0) return 0;
  AttnParams p;
  int rc = fill_common(p, q, ldq, out, ldo, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, seq_base,
                       scale, k_scale, v_scale, Hq, Hkv, D, block_size, window);
  if (rc) return rc;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  if (p.num_splits > 1 && (!part_o || !part_ml)) return -3;
  p.part_o = part_o; p.part_ml = part_ml;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (p.block_size * D * 2 > 96 * 1024) return -4;
  if (Hq / Hkv > 8) return -5;        // one n-tile of heads per kv head
  if (D == 64) return launch_decode<64>(p, B, status, st);
  if (D == 128) return launch_decode<128>(p, B, status, st);
  return launch_decode<256>(p, B, status, st);
}

// The same with the output written as FP8 [row, Hq * 128] plus one scale per (row, head) in the k-group-major layout the
// FP8 GEMMs read (scale of (row, head) at s_out[head * s_ld + row]): the activation quantisation in front of the output
// projection happens where the rows are produced.  head_dim 128 only.  The values are rounded to bf16 before they are
// quantised, so the result equals quantising the bf16 output of atlas_attn_decode.
extern "C" int atlas_attn_decode_q8(const void* q, long long ldq, void* q_out, long long ldqo, float* s_out, long long s_ld,
                                    const void* k_cache, const void* v_cache, const int* block_tables, int bt_ld,
                                    const int* seq_lens, const int* query_start_loc, int seq_base, int B, float scale,
                                    float k_scale, float v_scale, int Hq, int Hkv, int block_size, int window,
                                    int num_splits, float* part_o, float* part_ml, unsigned long long* status, void* stream) {
  if (B <= 0) return 0;
  if (!q_out || !s_out || (ldqo % 4) || (reinterpret_cast<uintptr_t>(q_out) & 3)) return -6;
  AttnParams p;
  int rc = fill_common(p, q, ldq, nullptr, 0, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, seq_base,
                       scale, k_scale, v_scale, Hq, Hkv, 128, block_size, window);
  if (rc) return rc;
  p.q_out = reinterpret_cast<uint8_t*>(q_out); p.ldqo = ldqo; p.s_out = s_out; p.s_ld = s_ld;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  if (p.num_splits > 1 && (!part_o || !part_ml)) return -3;
  p.part_o = part_o; p.part_ml = part_ml;
  if (p.block_size * 128 * 2 > 96 * 1024) return -4;
  if (Hq / Hkv > 8) return -5;
  return launch_decode<128>(p, B, status, reinterpret_cast<cudaStream_t>(stream));
}

// Selects the decode kernel for 16-token pages at run time (1 = e4m3 tensor-core tiles, 0 = f16 tiles).
extern "C" void atlas_attn_set_decode_f8(int on) { g_decode_f8 = on ? 1 : 0; }

// Prefill / verify attention: `num_tiles` 16-row query tiles described by (sequence index, first query row of the
// tile inside the sequence's chunk).
extern "C" int atlas_attn_prefill(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                  const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                  const int* query_start_loc, const int* tile_seq, const int* tile_q0, int num_tiles,
                                  float scale, float k_scale, float v_scale, int Hq, int Hkv, int D, int block_size,
                                  int window, void* stream) {
  if (num_tiles <= 0) return 0;
  AttnParams p;
  int rc = fill_common(p, q, ldq, out, ldo, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, 0, scale,
                       k_scale, v_scale, Hq, Hkv, D, block_size, window);
  if (rc) return rc;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.num_tiles = num_tiles;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 64) return launch_prefill<64>(p, st);
  if (D == 128) return launch_prefill<128>(p, st);
  return launch_prefill<256>(p, st);
}

// ---- bf16 KV cache (high-precision layers, accuracy checks): the general mma.sync kernel in both roles.
template <int D>
static int launch_kv16(const AttnParams& p, int B, bool prefill, cudaStream_t st) {
  if (prefill) {
    dim3 grid((p.num_tiles + 3) / 4, p.Hq);
    paged_attn_kernel<D, true, true><<<grid, 128, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  const int smem = (128 + 4 * 16 * D) * (int)sizeof(float);
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(paged_attn_kernel<D, false, true>), smem) != cudaSuccess) return -20;
  dim3 grid(p.Hkv, p.num_splits, B);
  paged_attn_kernel<D, false, true><<<grid, 128, smem, st>>>(p);
  if (cudaGetLastError() != cudaSuccess) return -21;
  if (p.num_splits > 1) {
    dim3 g2(p.Hq, B);
    attn_merge_kernel<<<g2, D, 0, st>>>(p.part_o, p.part_ml, p.out, p.ldo, p.query_start_loc, p.seq_base, p.Hq, D, p.num_splits,
                                       p.v_scale, nullptr, 0, nullptr, 0);
    if (cudaGetLastError() != cudaSuccess) return -22;
  }
  return 0;
}

// ---- NVFP4 KV cache: the general kernel in both roles (page layout in the comment above paged_attn_kernel).
template <int D>
static int launch_kv4(const AttnParams& p, int B, bool prefill, cudaStream_t st) {
  if (prefill) {
    dim3 grid((p.num_tiles + 3) / 4, p.Hq);
    paged_attn_kernel<D, true, false, true><<<grid, 128, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  // decode rows: the cp.async pipeline with NVFP4 pages when the warp rings fit, the general kernel otherwise
  if (4 * 3 * 2 * (p.block_size * D * 9 / 16) <= 96 * 1024 && p.Hq / p.Hkv <= 8) {
    if (p.block_size == 16) return launch_decode_cp<D, 16, 3, true>(p, B, st);
    return launch_decode_cp<D, 0, 3, true>(p, B, st);
  }
  const int smem = (128 + 4 * 16 * D) * (int)sizeof(float);
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(paged_attn_kernel<D, false, false, true>), smem) != cudaSuccess) return -20;
  dim3 grid(p.Hkv, p.num_splits, B);
  paged_attn_kernel<D, false, false, true><<<grid, 128, smem, st>>>(p);
  if (cudaGetLastError() != cudaSuccess) return -21;
  if (p.num_splits > 1) {
    dim3 g2(p.Hq, B);
    attn_merge_kernel<<<g2, D, 0, st>>>(p.part_o, p.part_ml, p.out, p.ldo, p.query_start_loc, p.seq_base, p.Hq, D, p.num_splits,
                                       p.v_scale, nullptr, 0, nullptr, 0);
    if (cudaGetLastError() != cudaSuccess) return -22;
  }
  return 0;
}

// Same contracts as atlas_attn_decode / atlas_attn_prefill with an NVFP4 cache; k_scale / v_scale are the tensors' second
// level (global) scales.  head_dim 128 or 256, block_size a multiple of 16.
extern "C" int atlas_attn_decode_kv4(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                     const int* query_start_loc, int seq_base, int B, float scale, float k_scale, float v_scale,
                                     int Hq, int Hkv, int D, int block_size, int window, int num_splits, float* part_o,
                                     float* part_ml, void* stream) {
  if (B <= 0) return 0;
  if (D != 128 && D != 256) return -1;
  AttnParams p;
  int rc = fill_common(p, q, ldq, out, ldo, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, seq_base, scale,
                       k_scale, v_scale, Hq, Hkv, D, block_size, window);
  if (rc) return rc;
  if (Hq / Hkv > 16) return -5;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  if (p.num_splits > 1 && (!part_o || !part_ml)) return -3;
  p.part_o = part_o; p.part_ml = part_ml;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_kv4<128>(p, B, false, st);
  return launch_kv4<256>(p, B, false, st);
}

extern "C" int atlas_attn_prefill_kv4(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                      const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                      const int* query_start_loc, const int* tile_seq, const int* tile_q0, int num_tiles,
                                      float scale, float k_scale, float v_scale, int Hq, int Hkv, int D, int block_size,
                                      int window, void* stream) {
  if (num_tiles <= 0) return 0;
  if (D != 128 && D != 256) return -1;
  AttnParams p;
  int rc = fill_common(p, q, ldq, out, ldo, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, 0, scale, k_scale,
                       v_scale, Hq, Hkv, D, block_size, window);
  if (rc) return rc;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.num_tiles = num_tiles;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_kv4<128>(p, 0, true, st);
  return launch_kv4<256>(p, 0, true, st);
}

// Same contracts as atlas_attn_decode / atlas_attn_prefill with a bf16 cache (K [nb, Hkv, bs, D], V [nb, Hkv, D, bs]).
extern "C" int atlas_attn_decode_kv16(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                      const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                      const int* query_start_loc, int seq_base, int B, float scale, int Hq, int Hkv, int D,
                                      int block_size, int window, int num_splits, float* part_o, float* part_ml, void* stream) {
  if (B <= 0) return 0;
  AttnParams p;
  int rc = fill_common(p, q, ldq, out, ldo, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, seq_base, scale,
                       1.f, 1.f, Hq, Hkv, D, block_size, window);
  if (rc) return rc;
  if (Hq / Hkv > 16) return -5;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  if (p.num_splits > 1 && (!part_o || !part_ml)) return -3;
  p.part_o = part_o; p.part_ml = part_ml;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 64) return launch_kv16<64>(p, B, false, st);
  if (D == 128) return launch_kv16<128>(p, B, false, st);
  return launch_kv16<256>(p, B, false, st);
}

extern "C" int atlas_attn_prefill_kv16(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                       const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                       const int* query_start_loc, const int* tile_seq, const int* tile_q0, int num_tiles,
                                       float scale, int Hq, int Hkv, int D, int block_size, int window, void* stream) {
  if (num_tiles <= 0) return 0;
  AttnParams p;
  int rc = fill_common(p, q, ldq, out, ldo, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, 0, scale, 1.f,
                       1.f, Hq, Hkv, D, block_size, window);
  if (rc) return rc;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.num_tiles = num_tiles;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 64) return launch_kv16<64>(p, 0, true, st);
  if (D == 128) return launch_kv16<128>(p, 0, true, st);
  return launch_kv16<256>(p, 0, true, st);
}

// ================================================================================ allocation-free decode attention
// Split-K scratch (per-split partial outputs and softmax statistics) for callers that may not allocate device
// memory.  The array is part of the library image: every GPU that loads the library carries these 16 MiB until the
// process exits.
static __device__ __align__(256) float g_noalloc_decode_scratch[ATLAS_NOALLOC_DECODE_SCRATCH_FLOATS];

// Device address of the array above for each device, resolved the first time that device is used.  (In host code the
// array's name only stands for the symbol; the address a kernel can dereference comes from cudaGetSymbolAddress.)
static float* g_noalloc_scratch_ptr[16] = {nullptr};

extern "C" int atlas_attn_decode_noalloc(const void* q, long long ldq, void* out, long long ldo, const void* k_cache,
                                         const void* v_cache, const int* block_tables, int bt_ld, const int* seq_lens,
                                         const int* query_start_loc, int B, float scale, float k_scale, float v_scale,
                                         int Hq, int Hkv, int D, int block_size, int window, int num_splits,
                                         unsigned long long* status, void* stream) {
  if (B <= 0) return 0;
  if (num_splits < 1) num_splits = 1;
  // shape checks first: the size test below is only meaningful for positive, supported Hq / Hkv / D
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || block_size <= 0 || block_size % 16 || (D != 64 && D != 128 && D != 256)) return -1;
  const long long need = (long long)B * Hq * num_splits * (D + 2);
  if (need > (long long)ATLAS_NOALLOC_DECODE_SCRATCH_FLOATS) return ATLAS_NOALLOC_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return ATLAS_NOALLOC_ERR_DEVICE;
  if (!g_noalloc_scratch_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_decode_scratch) != cudaSuccess || !p) return ATLAS_NOALLOC_ERR_SYMBOL;
    g_noalloc_scratch_ptr[dev] = reinterpret_cast<float*>(p);
  }
  float* part_o = g_noalloc_scratch_ptr[dev];
  float* part_ml = part_o + (long long)B * Hq * num_splits * D;
  AttnParams p;
  int rc = fill_common(p, q, ldq, out, ldo, k_cache, v_cache, block_tables, bt_ld, seq_lens, query_start_loc, 0, scale,
                       k_scale, v_scale, Hq, Hkv, D, block_size, window);
  if (rc) return rc;
  if (p.block_size * D * 2 > 96 * 1024) return -4;
  if (Hq / Hkv > 8) return -5;
  p.num_splits = num_splits;
  p.part_o = part_o; p.part_ml = part_ml;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 64) return launch_decode<64>(p, B, status, st);
  if (D == 128) return launch_decode<128>(p, B, status, st);
  return launch_decode<256>(p, B, status, st);
}
