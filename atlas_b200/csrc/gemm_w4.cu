// NVFP4 weight-only GEMM for sm_100a:  C[M,N] = A[M,K] (bf16) * dequant(B)[N,K]^T, fp32 accumulation in TMEM.
//
// B is stored as the checkpoint ships it: E2M1 nibbles packed two per byte ([N, K/2], even k in the low nibble), one
// e4m3 scale per 16 consecutive k ([N, K/16]) and an fp32 global scale per output row.  HBM traffic is therefore
// 4.5 bits per weight; the tensor cores still see bf16:
//
//   warp 0        TMA producer of the packed B slices (BLOCK_N x 32 bytes each) into a deep ring: this is the HBM
//                 stream, so it runs many slices ahead of everything else (bytes in flight, not operand tiles, bound it)
//   warp 14       TMA producer of the A tiles (128 x 64 bf16, 128-byte swizzle; activations, L2 resident)
//   warps 2..9    converters: nibbles -> f16 (cvt.rn.f16x2.e2m1x2) x block scale -> bf16 (exact: the product has at
//                 most six significant bits), written straight into the 128-byte-swizzled K-major operand layout
//   warp 1        tcgen05.mma kind::f16 issuer (bf16 x bf16), two TMEM accumulator buffers
//   warps 10..13  epilogue: tcgen05.ld, multiply column n by its global scale, bf16 stores
//
// The global scale is applied once per output element instead of once per weight.  Plain and grouped (MoE: rows sorted
// by expert, every expert padded to whole 128-row tiles, B the stack of all experts) forms share the kernel.
// Reference ops replaced: w4a16_gemm*.cu / w4a16_gemv*.cu / moe_w4a16_grouped_gemm*.cu (kernels/gb10/common), which
// dequantise in registers for mma.sync.
#include <cuda_fp4.h>

#include "common.cuh"
#include "host_api.h"
#include "tmap.h"

namespace atlas {

constexpr int kW4BlockM = 128;
constexpr int kW4ConvWarps = 8;          // two per scheduler: the conversion is ALU work, the second warp hides its latency
constexpr int kW4EpiWarps = 4;
constexpr int kW4Threads = 32 * (2 + kW4ConvWarps + kW4EpiWarps + 1);
constexpr int kW4AWarp = 2 + kW4ConvWarps + kW4EpiWarps;      // index of the A-tile producer warp

template <int BLOCK_N>
struct W4Cfg {
  static constexpr int kABytes = kW4BlockM * 128;       // 128 rows x 64 bf16
  static constexpr int kBBytes = BLOCK_N * 128;         // converted operand, same layout as a TMA-swizzled tile
  static constexpr int kPBytes = BLOCK_N * 32;          // packed nibbles of one 64-wide K slice
  static constexpr int kStageBytes = kABytes + kBBytes;   // operand stage: A + converted B
  static constexpr int kStages = BLOCK_N == 128 ? 4 : 5;
  static constexpr int kPStages = 16;                     // packed-slice ring (the HBM stream)
  static constexpr int kAccStages = 2;
  static constexpr int kTmemCols = kAccStages * BLOCK_N;
  static constexpr int kGsBytes = 2 * BLOCK_N * 4;      // global scales of the tile's columns, double buffered
  static constexpr int kOperandBytes = kStages * kStageBytes;
  static constexpr int kSmemBytes = kOperandBytes + kPStages * kPBytes + kGsBytes + 1024 /*align*/ + 512 /*barriers*/;
};

struct W4Params {
  void* C;
  const uint8_t* bscale;      // e4m3 [rows(B), K/16]
  const float* gscale;        // fp32 [rows(B)]
  status_t* status;
  long long ldc;
  int M, N, K, k_blocks, m_tiles, n_tiles;
  int scale_ld;               // K / 16
  int b_rows;                 // rows of B (N, or E * N for the grouped form)
  int vec_ok;
  const int* tile_expert;     // nullptr = plain GEMM
  const int* num_m_tiles_ptr;
  int expert_n;
};

// two packed E2M1 values (low nibble first) times a block scale -> two bf16
ATLAS_DEVICE uint32_t w4_pair(uint32_t byte, __half2 sc) {
  __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xFFu), __NV_E2M1);
  __half2 h = __hmul2(*reinterpret_cast<__half2*>(&hr), sc);
  const float2 f = __half22float2(h);
  return pack_bf16x2(f.x, f.y);
}
ATLAS_DEVICE uint4 w4_word(uint32_t w, __half2 sc) {      // eight weights -> one 16-byte chunk
  uint4 o;
  o.x = w4_pair(w, sc);
  o.y = w4_pair(w >> 8, sc);
  o.z = w4_pair(w >> 16, sc);
  o.w = w4_pair(w >> 24, sc);
  return o;
}
ATLAS_DEVICE __half2 e4m3_to_half2(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(byte & 0xFFu), __NV_E4M3);
  return __half2half2(*reinterpret_cast<__half*>(&h));
}

template <int BLOCK_N>
__global__ void __launch_bounds__(kW4Threads, 1)
gemm_w4a16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_p,
                          const W4Params p) {
  using Cfg = W4Cfg<BLOCK_N>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kAcc = Cfg::kAccStages;
  constexpr uint32_t kIdesc = make_idesc(kW4BlockM, BLOCK_N, 1u);      // bf16 x bf16

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kPStages = Cfg::kPStages;
  uint8_t* pring = smem + Cfg::kOperandBytes;                           // [kPStages][BLOCK_N][32]
  float* gs_smem = reinterpret_cast<float*>(pring + kPStages * Cfg::kPBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(gs_smem) + Cfg::kGsBytes);
  uint64_t* full = bars;                       // A tile landed
  uint64_t* conv = bars + kStages;             // converters finished the stage's B operand
  uint64_t* empty = bars + 2 * kStages;        // MMAs of the stage retired (frees A and B)
  uint64_t* acc_full = bars + 3 * kStages;
  uint64_t* acc_empty = acc_full + kAcc;
  uint64_t* p_full = acc_empty + kAcc;         // packed slice landed
  uint64_t* p_empty = p_full + kPStages;       // converters are done with the packed slice
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_empty + kPStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&conv[s], kW4ConvWarps);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < kAcc; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kW4EpiWarps);
    }
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(&p_full[s], 1);
      mbar_init(&p_empty[s], kW4ConvWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_p);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = p.tile_expert ? *p.num_m_tiles_ptr : p.m_tiles;
  const int total_items = m_tiles * p.n_tiles;
  const int M_rows = p.tile_expert ? m_tiles * kW4BlockM : p.M;

  if (warp == 0) {
    // ------------------------------------------------------------------ packed-B producer (HBM stream)
    if (lane == 0) {
      uint32_t ps = 0, pphase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int m_tile = item % m_tiles, n_tile = item / m_tiles;
        const int brow0 = (p.tile_expert ? p.tile_expert[m_tile] * p.expert_n : 0) + n_tile * BLOCK_N;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&p_empty[ps], pphase ^ 1u, abort_flag, p.status, 0x700)) { ok = false; break; }
          mbar_expect_tx(&p_full[ps], Cfg::kPBytes);
          tma_load_2d(pring + ps * Cfg::kPBytes, &tmap_p, &p_full[ps], kb * 32, brow0);
          if (++ps == kPStages) { ps = 0; pphase ^= 1u; }
        }
      }
      if (!ok)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);       // let copies in flight land before shared memory goes away
    }
  } else if (warp == kW4AWarp) {
    // ------------------------------------------------------------------ A-tile producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int m_tile = item % m_tiles;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 0x701)) { ok = false; break; }
          mbar_expect_tx(&full[stage], Cfg::kABytes);
          tma_load_2d(smem + stage * Cfg::kStageBytes, &tmap_a, &full[stage], kb * 64, m_tile * kW4BlockM);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc_iter = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const uint32_t buf = acc_iter % kAcc, aph = (acc_iter / kAcc) & 1u;
        if (!mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag, p.status, 0x710)) break;
        tc_fence_after();
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 0x711)) { ok = false; break; }
          if (!mbar_wait(&conv[stage], phase, abort_flag, p.status, 0x712)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + Cfg::kABytes);
          const uint32_t d = tmem_base + buf * BLOCK_N;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);
        ++acc_iter;
      }
    }
  } else if (warp < 2 + kW4ConvWarps) {
    // ------------------------------------------------------------------ converters
    const int ct = threadIdx.x - 64;                               // 0..255
    constexpr int kThreadsPerRow = 32 * kW4ConvWarps / BLOCK_N;    // 2 (BLOCK_N 128) or 4 (BLOCK_N 64)
    constexpr int kWords = 8 / kThreadsPerRow;                     // 32-bit words (8 weights each) per thread and slice
    constexpr int kScaleBytes = 4 / kThreadsPerRow;                // block scales per thread and slice (2 or 1)
    const int row = ct / kThreadsPerRow;
    const int part = ct % kThreadsPerRow;
    const int sw = row & 7;
    uint32_t stage = 0, phase = 0, ps = 0, pphase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int m_tile = item % m_tiles, n_tile = item / m_tiles;
      const int brow = (p.tile_expert ? p.tile_expert[m_tile] * p.expert_n : 0) + n_tile * BLOCK_N + row;
      const bool live = brow < p.b_rows && (n_tile * BLOCK_N + row) < p.N;
      // block scales of this row: 4 bytes per 64-wide slice (2 per thread when two threads share a row)
      const uint8_t* srow = p.bscale + (size_t)(live ? brow : 0) * p.scale_ld + part * kScaleBytes;
      auto load_scales = [&](int kb) -> uint32_t {
        const uint8_t* a = srow + (size_t)kb * 4;
        return kScaleBytes == 2 ? (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(a)) : (uint32_t)__ldg(a);
      };
      uint32_t sc_next = live ? load_scales(0) : 0u;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        const uint32_t sc = sc_next;
        if (live && kb + 1 < p.k_blocks) sc_next = load_scales(kb + 1);
        if (!mbar_wait(&p_full[ps], pphase, abort_flag, p.status, 0x720)) { ok = false; break; }
        const uint32_t* pk = reinterpret_cast<const uint32_t*>(pring + ps * Cfg::kPBytes + row * 32 + part * (kWords * 4));
        uint32_t w[kWords];
        if (kWords == 4) {
          const uint4 v = *reinterpret_cast<const uint4*>(pk);
          w[0] = v.x; w[1] = v.y; w[2 % kWords] = v.z; w[3 % kWords] = v.w;
        } else {
          const uint2 v = *reinterpret_cast<const uint2*>(pk);
          w[0] = v.x; w[1] = v.y;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_empty[ps]);          // the slice is in registers: its slot can be refilled
        if (++ps == kPStages) { ps = 0; pphase ^= 1u; }
        // the operand stage is free once the MMAs that read it last time have retired
        if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, 0x721)) { ok = false; break; }
        uint8_t* brow_smem = smem + stage * Cfg::kStageBytes + Cfg::kABytes + (row >> 3) * 1024 + sw * 128;
#pragma unroll
        for (int j = 0; j < kWords; ++j) {
          const __half2 s2 = e4m3_to_half2(sc >> (8 * (j >> 1)));          // one scale per 16 weights = two words
          const int chunk = part * kWords + j;                             // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(brow_smem + ((chunk ^ sw) << 4)) = w4_word(w[j], s2);
        }
        fence_proxy_async();                 // generic-proxy stores -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&conv[stage]);
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp < 2 + kW4ConvWarps + kW4EpiWarps) {
    // ------------------------------------------------------------------ epilogue
    const int lane_group = warp & 3;
    const int row_in_tile = lane_group * 32 + lane;
    const uint32_t t_lane = (uint32_t)(lane_group * 32) << 16;
    const int epi_tid = threadIdx.x - 32 * (2 + kW4ConvWarps);
    uint32_t acc_iter = 0, tile_iter = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const int m_tile = item % m_tiles, n_tile = item / m_tiles;
      const int m = m_tile * kW4BlockM + row_in_tile;
      const int brow0 = (p.tile_expert ? p.tile_expert[m_tile] * p.expert_n : 0) + n_tile * BLOCK_N;
      float* gs = gs_smem + (tile_iter & 1u) * BLOCK_N;
      ++tile_iter;
      for (int i = epi_tid; i < BLOCK_N; i += 32 * kW4EpiWarps)
        gs[i] = (brow0 + i < p.b_rows && n_tile * BLOCK_N + i < p.N) ? __ldg(p.gscale + brow0 + i) : 0.f;
      asm volatile("bar.sync 1, %0;\n" ::"n"(32 * kW4EpiWarps));
      if (!ok) continue;
      const uint32_t buf = acc_iter % kAcc, aph = (acc_iter / kAcc) & 1u;
      if (!mbar_wait(&acc_full[buf], aph, abort_flag, p.status, 0x730)) { ok = false; continue; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + t_lane + buf * BLOCK_N;
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc;
#pragma unroll
      for (int c0 = 0; c0 < BLOCK_N; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c0, r);
        tmem_ld_wait();
        if (c0 + 32 >= BLOCK_N) {          // the last chunk is in registers: hand the buffer back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (m < M_rows) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const int n = n_tile * BLOCK_N + c0 + j;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[j + i]) * gs[c0 + j + i];
            if (p.vec_ok && n + 8 <= p.N) {
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(crow + n) = o;
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (n + i < p.N) crow[n + i] = __float2bfloat16_rn(v[i]);
            }
          }
        }
      }
      ++acc_iter;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BLOCK_N>
static int launch_w4(const CUtensorMap& ta, const CUtensorMap& tp, const W4Params& p, int grid, cudaStream_t st) {
  using Cfg = W4Cfg<BLOCK_N>;
  auto kern = gemm_w4a16_tcgen05_kernel<BLOCK_N>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::kSmemBytes) != cudaSuccess) return -20;
  kern<<<grid, kW4Threads, Cfg::kSmemBytes, st>>>(ta, tp, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

static int w4_common(const void* A, const void* packed, const void* bscale, const float* gscale, void* C, int M, int N,
                     int K, long long lda, long long ldc, int block_n, int b_rows, const int* tile_expert,
                     const int* num_m_tiles, int num_sms, unsigned long long* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 64) return -3;                                  // one slice = 64 weights = 4 block scales
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(packed) & 15)) return -1;
  if ((lda * 2) % 16 || (K / 2) % 16) return -2;
  if ((reinterpret_cast<uintptr_t>(bscale) & 3)) return -7;
  if (block_n != 64 && block_n != 128) return -4;
  if (tile_expert && (N % block_n)) return -10;           // a tile must not straddle two experts
  CUtensorMap ta, tp;
  int rc = make_tmap_2d(&ta, A, M, K, lda, kW4BlockM, 2, 128, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tp, packed, b_rows, K / 2, K / 2, block_n, 1, 32, false);
  if (rc) return rc;
  W4Params p;
  p.C = C; p.bscale = reinterpret_cast<const uint8_t*>(bscale); p.gscale = gscale; p.status = status; p.ldc = ldc;
  p.M = M; p.N = N; p.K = K; p.k_blocks = K / 64;
  p.m_tiles = (M + kW4BlockM - 1) / kW4BlockM;
  p.n_tiles = (N + block_n - 1) / block_n;
  p.scale_ld = K / 16; p.b_rows = b_rows;
  p.vec_ok = ((ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
  p.tile_expert = tile_expert; p.num_m_tiles_ptr = num_m_tiles; p.expert_n = tile_expert ? N : 0;
  const long long items = (long long)p.m_tiles * p.n_tiles;
  const int grid = (int)(items < num_sms ? items : num_sms);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return block_n == 64 ? launch_w4<64>(ta, tp, p, grid, st) : launch_w4<128>(ta, tp, p, grid, st);
}

}  // namespace atlas

using namespace atlas;

// C[M,N] (bf16) = A[M,K] (bf16, row stride lda) * dequant(packed [N,K/2], bscale e4m3 [N,K/16], gscale fp32 [N])^T.
// K must be a multiple of 64.  Returns 0 or a negative error code.
extern "C" int atlas_gemm_w4a16(const void* A, const void* packed, const void* bscale, const float* gscale, void* C,
                                int M, int N, int K, long long lda, long long ldc, int block_n, int num_sms,
                                unsigned long long* status, void* stream) {
  return w4_common(A, packed, bscale, gscale, C, M, N, K, lda, ldc, block_n, N, nullptr, nullptr, num_sms, status, stream);
}

// Grouped (MoE) form: rows of A are expert-sorted, every expert's segment padded to whole 128-row tiles; m-tile i uses
// expert tile_expert[i]; *num_m_tiles (device memory) tiles are live.  packed / bscale / gscale are the stacks over
// E experts ([E*N, K/2], [E*N, K/16], [E*N]).
extern "C" int atlas_gemm_w4a16_grouped(const void* A, const void* packed, const void* bscale, const float* gscale,
                                        void* C, int max_rows, int N, int K, int E, long long lda, long long ldc,
                                        int block_n, const int* tile_expert, const int* num_m_tiles, int num_sms,
                                        unsigned long long* status, void* stream) {
  if (max_rows % kW4BlockM) return -9;
  return w4_common(A, packed, bscale, gscale, C, max_rows, N, K, lda, ldc, block_n, E * N, tile_expert, num_m_tiles,
                   num_sms, status, stream);
}
