// NVFP4 x NVFP4 GEMM on the block-scaled tensor-core path: tcgen05.mma kind::mxf4nvf4 (block16, UE4M3 scale factors
// read from TMEM), TMA 128B-swizzled operand tiles, accumulation of the WHOLE K extent in TMEM.
//
//   C[M,N] (bf16) = row_scale[m] * col_scale[n] * sum_k (A4[m,k] * SFA[m,k/16]) * (B4[n,k] * SFB[n,k/16])
//
// A4 / B4 are e2m1 values packed two per byte, K-major.  SFA / SFB are e4m3 scale factors, one per 16 values, stored in
// the 128 x 4 "atom" order the tensor core reads: for row block rb = row / 128 and scale group kg = (k / 16) / 4, the
// 512-byte atom at ((rb * ceil(K/64) + kg) * 512) holds byte (row % 32) * 16 + ((row % 128) / 32) * 4 + (k / 16) % 4.
// One tcgen05.cp (32x128b, replicated to the four lane quarters) moves an atom into four TMEM columns, where an
// MMA of K = 64 finds the four scale factors of every row.  row_scale carries the per-token second-level scale of
// the activation quantiser, col_scale the per-output-row global scale of the weight (both fp32).
//
// CTA = 128 x 128 or 128 x 256 output tile, K step 256 values (one 128-byte swizzled row), persistent over tiles.
//   warp 0      TMA producer: A tile, B tile, their scale-factor atoms (plain bulk copies), one mbarrier per stage
//   warp 1      TMEM owner and MMA issuer: per stage 8 or 12 tcgen05.cp + 4 tcgen05.mma, commit frees the stage
//   warps 2-9   epilogue: tcgen05.ld of the finished accumulator (released right after the reads), scales, bf16 stores
// 128-wide: two accumulators alternate so the epilogue of tile i overlaps the MMAs of tile i + 1.  256-wide (chosen
// when such tiles still fill every SM): a third fewer operand bytes per FLOP, one accumulator.  The scale-factor
// columns in TMEM alternate with the stage parity.  Every wait is bounded and reports through the status word.
//
// The activation quantiser (bf16 -> e2m1 + UE4M3 atoms + per-row scale) is in this file too.
// Reference ops replaced: kernels/gb10/qwen3.6-27b/nvfp4/w4a4_gemm.cu (mma.sync m16n8k64 e2m1 with software scales),
// kernels/gb10/common/quantize_nvfp4.cu.
#include "common.cuh"
#include "host_api.h"
#include "tmap.h"

namespace atlas {

constexpr int kF4BlockM = 128;
constexpr int kF4BlockK = 256;                         // values per stage = 128 bytes per row
constexpr int kF4Threads = 320;                        // producer, MMA issuer, eight epilogue warps
constexpr int kF4TmemCols = 512;

// BLOCK_N = 128: six stages, two accumulators (the epilogue of a tile overlaps the next tile's MMAs).
// BLOCK_N = 256: four stages, ONE accumulator of 256 columns (two would leave no TMEM for the scale factors); the
// operand ring keeps filling while the epilogue drains it, and the fill is what bounds these tiles.
template <int BLOCK_N>
struct F4Cfg {
  static constexpr int kNBlocks = BLOCK_N / 128;                   // 128-row scale-factor blocks of the B tile
  static constexpr int kStages = BLOCK_N == 128 ? 6 : 4;
  static constexpr int kATile = kF4BlockM * 128;                   // bytes
  static constexpr int kBTile = BLOCK_N * 128;
  static constexpr int kSfA = 4 * 512;                             // four atoms: K 256 = 16 scale factors per row
  static constexpr int kSfB = kNBlocks * 4 * 512;
  static constexpr int kStageBytes = kATile + kBTile + kSfA + kSfB;
  static constexpr int kAccStages = BLOCK_N == 128 ? 2 : 1;
  static constexpr int kSfColBase = kAccStages * BLOCK_N;
  static constexpr int kSfColsPerBuf = 16 + 16 * kNBlocks;         // SFA then SFB, per stage parity
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(kSfColBase + 2 * kSfColsPerBuf <= kF4TmemCols, "TMEM budget");
};

struct Fp4Params {
  int M, N, K;
  const uint8_t* sfa;           // [ceil(M/128)][ceil(K/64)][512]
  const uint8_t* sfb;           // [ceil(N/128)][ceil(K/64)][512]
  const float* row_scale;       // [M] or null
  const float* col_scale;       // [N] or null
  float alpha;
  __nv_bfloat16* C;
  long long ldc;
  status_t* status;
};

// no-swizzle K-major descriptor of one 512-byte scale-factor atom: 8-row x 16-byte core matrices, 128 bytes apart
ATLAS_DEVICE uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;                     // SBO = 128 B between 8-row groups
  d |= (uint64_t)1 << 46;                              // descriptor version
  return d;
}
ATLAS_DEVICE void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(taddr), "l"(desc) : "memory");
}
// block-scaled instruction descriptor: e2m1 x e2m1, UE4M3 scales, K = 64, both operands K-major
ATLAS_DEVICE constexpr uint32_t make_idesc_f4(uint32_t m, uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (0u << 23) | ((m >> 4) << 24);
}
ATLAS_DEVICE void umma_f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
ATLAS_DEVICE void bulk_g2s_f4(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int BLOCK_N>
__global__ void __launch_bounds__(kF4Threads, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap ta, const __grid_constant__ CUtensorMap tb, Fp4Params p) {
  extern __shared__ uint8_t smem_raw[];
  using Cfg = F4Cfg<BLOCK_N>;
  constexpr int kF4Stages = Cfg::kStages, kF4StageBytes = Cfg::kStageBytes, kF4BlockN = BLOCK_N;
  constexpr int kAcc = Cfg::kAccStages;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kF4Stages * kF4StageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kF4Stages;
  uint64_t* acc_full = bars + 2 * kF4Stages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kF4BlockM - 1) / kF4BlockM, n_tiles = (p.N + kF4BlockN - 1) / kF4BlockN;
  const int k_steps = (p.K + kF4BlockK - 1) / kF4BlockK;
  const int k_groups = (p.K + 63) / 64;                 // scale-factor atoms per row block
  const int tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF4Stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < kAcc; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 8); }
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&ta);
    tma_prefetch_desc(&tb);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kF4TmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int mt = tile % m_tiles, nt = tile / m_tiles;          // consecutive CTAs share the B tile
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kF4Stages;
          const uint32_t ph = (it / kF4Stages) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.status, 0x900)) goto producer_done;
          uint8_t* st = smem + (size_t)s * kF4StageBytes;
          const int groups = min(4, k_groups - ks * 4);             // atoms that exist at the K tail
          mbar_expect_tx(&full[s], Cfg::kATile + Cfg::kBTile + (1 + Cfg::kNBlocks) * groups * 512);
          tma_load_2d(st, &ta, &full[s], ks * 128, mt * kF4BlockM);
          tma_load_2d(st + Cfg::kATile, &tb, &full[s], ks * 128, nt * kF4BlockN);
          uint8_t* sf_s = st + Cfg::kATile + Cfg::kBTile;
          bulk_g2s_f4(sf_s, p.sfa + ((size_t)mt * k_groups + ks * 4) * 512, groups * 512, &full[s]);
#pragma unroll
          for (int nb = 0; nb < Cfg::kNBlocks; ++nb)
            bulk_g2s_f4(sf_s + Cfg::kSfA + nb * 2048,
                        p.sfb + ((size_t)(nt * Cfg::kNBlocks + nb) * k_groups + ks * 4) * 512, groups * 512, &full[s]);
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f4(kF4BlockM, kF4BlockN);
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++tcount) {
        const int a = tcount % kAcc;
        if (!mbar_wait(&acc_empty[a], ((tcount / kAcc) & 1u) ^ 1u, abort_flag, p.status, 0x901)) break;
        tc_fence_after();
        const uint32_t acc = tmem + a * BLOCK_N;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kF4Stages;
          if (!mbar_wait(&full[s], (it / kF4Stages) & 1u, abort_flag, p.status, 0x902)) goto mma_done;
          tc_fence_after();
          uint8_t* st = smem + (size_t)s * kF4StageBytes;
          // scale-factor columns of this stage parity: [0,16) SFA (4 per MMA), then SFB (4 per 128 rows per MMA)
          const uint32_t sf_cols = tmem + Cfg::kSfColBase + (it & 1u) * Cfg::kSfColsPerBuf;
          const uint32_t sfa_s = smem_u32(st + Cfg::kATile + Cfg::kBTile), sfb_s = sfa_s + Cfg::kSfA;
          const int groups = min(4, k_groups - ks * 4);
          for (int g = 0; g < groups; ++g) {
            tmem_cp_sf(sf_cols + g * 4, make_sf_desc(sfa_s + g * 512));
#pragma unroll
            for (int nb = 0; nb < Cfg::kNBlocks; ++nb)
              tmem_cp_sf(sf_cols + 16 + g * 4 * Cfg::kNBlocks + nb * 4, make_sf_desc(sfb_s + nb * 2048 + g * 512));
          }
          const uint64_t da = make_smem_desc_sw128(smem_u32(st)), db = make_smem_desc_sw128(smem_u32(st + Cfg::kATile));
          for (int g = 0; g < groups; ++g)                                     // 64 values = 32 bytes along the row
            umma_f4(acc, da + (uint64_t)(g * 32 >> 4), db + (uint64_t)(g * 32 >> 4), idesc, sf_cols + g * 4,
                    sf_cols + 16 + g * 4 * Cfg::kNBlocks, (ks | g) ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        umma_commit(&acc_full[a]);
      }
    mma_done:;
    }
  } else {
    // eight epilogue warps: warp w reads the TMEM lane quarter (w % 4) and the column half (w - 2) / 4.  All of a
    // warp's columns are pulled into registers first and the accumulator is handed back to the MMA warp BEFORE the
    // conversion and the stores, so a single accumulator is only held for the duration of the TMEM reads.
    const int q = warp & 3, half = (warp - 2) >> 2;
    constexpr int kCols = BLOCK_N / 2;                   // columns per warp
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++tcount) {
      const int mt = tile % m_tiles, nt = tile / m_tiles;
      const int a = tcount % kAcc;
      if (!mbar_wait(&acc_full[a], (tcount / kAcc) & 1u, abort_flag, p.status, 0x903)) break;
      tc_fence_after();
      uint32_t r[kCols / 32][32];
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c)
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + a * BLOCK_N + half * kCols + c * 32, r[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
      const int row = mt * kF4BlockM + q * 32 + lane;
      const float rs = (row < p.M && p.row_scale ? p.row_scale[row] : 1.f) * p.alpha;
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c) {
        const int col0 = nt * BLOCK_N + half * kCols + c * 32;
        if (row < p.M && col0 < p.N) {
          __nv_bfloat16* dst = p.C + (long long)row * p.ldc + col0;
          if (col0 + 32 <= p.N && (p.ldc % 8) == 0) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int cc = v * 8 + j * 2;
                const float s0 = p.col_scale ? p.col_scale[col0 + cc] : 1.f, s1 = p.col_scale ? p.col_scale[col0 + cc + 1] : 1.f;
                ow[j] = pack_bf16x2(__uint_as_float(r[c][cc]) * rs * s0, __uint_as_float(r[c][cc + 1]) * rs * s1);
              }
              *reinterpret_cast<uint4*>(dst + v * 8) = o;
            }
          } else {
#pragma unroll
            for (int cc = 0; cc < 32; ++cc)
              if (col0 + cc < p.N)
                dst[cc] = __float2bfloat16_rn(__uint_as_float(r[c][cc]) * rs * (p.col_scale ? p.col_scale[col0 + cc] : 1.f));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, kF4TmemCols);
  }
}

// ----------------------------------------------------------------------------- activation quantiser
// One warp per row: row amax -> second-level scale g = amax / (6 * 448); per 16 values the e4m3 scale factor
// s = amax16 / (6 g) and the e2m1 codes of x / (s g).  Packed bytes go to q[M, K/2], scale factors to the atom layout,
// g to row_scale[M].  Rows beyond M inside the last 128-row block keep whatever the buffer holds (their products land
// in output rows that are never stored).
ATLAS_DEVICE uint32_t f32x8_to_e2m1x8(const float (&v)[8]) {
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint16_t b;
    asm volatile("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}\n"
                 : "=h"(b)
                 : "f"(v[2 * i + 1]), "f"(v[2 * i]));
    out |= (uint32_t)(b & 0xFF) << (8 * i);
  }
  return out;
}

__global__ void __launch_bounds__(256)
quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M, int K, uint8_t* __restrict__ q,
                   uint8_t* __restrict__ sf, float* __restrict__ row_scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= M) return;
  const __nv_bfloat16* xr = x + (long long)row * ldx;
  float amax = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + k);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = warp_max(amax);
  const float g = amax > 0.f ? amax * (1.f / (6.f * 448.f)) : 1.f;
  if (lane == 0) row_scale[row] = g;
  const float inv_g6 = 1.f / (6.f * g);
  const int k_groups = (K + 63) / 64;
  uint8_t* sf_row = sf + (size_t)(row / 128) * k_groups * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4;
  // two lanes share one group of 16 values
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + k);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float v[8];
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      v[2 * j] = f.x; v[2 * j + 1] = f.y;
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    const uint8_t s8 = f32_to_fp8_e4m3(m * inv_g6);
    const float s = fp8_e4m3_to_f32(s8) * g;
    const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= inv;
    *reinterpret_cast<uint32_t*>(q + (size_t)row * (K / 2) + k / 2) = f32x8_to_e2m1x8(v);
    if ((lane & 1) == 0) {
      const int grp = k / 16;
      sf_row[(size_t)(grp / 4) * 512 + (grp % 4)] = s8;
    }
  }
}

}  // namespace atlas

using namespace atlas;

extern "C" int atlas_quant_nvfp4(const void* x, long long ldx, int M, int K, void* q, void* sf, float* row_scale, void* stream) {
  if (M <= 0) return 0;
  if (K % 16 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  quant_nvfp4_kernel<<<(M + 7) / 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, M, K, reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(sf),
      row_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}

// A4 [M, K/2] and B4 [N, K/2] packed e2m1 (row pitch K/2 bytes), scale factors in the atom layout (see the header).
extern "C" int atlas_gemm_nvfp4_w4a4(const void* A4, const void* sfa, const float* row_scale, const void* B4, const void* sfb,
                                     const float* col_scale, float alpha, void* C, long long ldc, int M, int N, int K,
                                     int num_sms, unsigned long long* status, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 32 || K < 64) return -1;                      // TMA inner extent: K/2 bytes, a multiple of 16
  const int m_tiles = (M + kF4BlockM - 1) / kF4BlockM;
  const bool wide = (N % 256 == 0) && m_tiles * (N / 256) >= num_sms;       // enough 256-wide tiles for every SM
  const int block_n = wide ? 256 : 128;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A4, M, K / 2, K / 2, kF4BlockM, 1, 128, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B4, N, K / 2, K / 2, block_n, 1, 128, true);
  if (rc) return rc;
  Fp4Params p = {};
  p.M = M; p.N = N; p.K = K;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.row_scale = row_scale; p.col_scale = col_scale; p.alpha = alpha;
  p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc; p.status = status;
  const int tiles = m_tiles * ((N + block_n - 1) / block_n);
  const int grid = tiles < num_sms ? tiles : num_sms;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (wide) {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_nvfp4_kernel<256>), (int)F4Cfg<256>::kSmemBytes) != cudaSuccess) return -12;
    gemm_nvfp4_kernel<256><<<grid, kF4Threads, F4Cfg<256>::kSmemBytes, st>>>(ta, tb, p);
  } else {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_nvfp4_kernel<128>), (int)F4Cfg<128>::kSmemBytes) != cudaSuccess) return -12;
    gemm_nvfp4_kernel<128><<<grid, kF4Threads, F4Cfg<128>::kSmemBytes, st>>>(ta, tb, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -20;
}
